"""A per-layer token input: after a layer's sublayers, a row of a table that belongs to the token is gated by a projection of
the stream, projected back to the stream's width, normed and added.

    e = table[token][first : first + dim];   g = gelu_tanh(W_gate x) * e;   y = W_proj g;   x += y / rms(y) * w

``table`` [vocab, columns] is one tensor that all layers share (each reads its own ``dim`` columns from ``first`` on); the
part whose ``declares_table`` is true names it among its tensors.  The norm is an RMS norm with a plain weight; the sum and
the norm are float32.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorDecl, WeightSource, register_part
from .linear import Linear


@register_part("side_input", "gated_token_row")
class GatedTokenRow(Part):
    def __init__(self, prefix: str, hidden_size: int, vocab_size: int, dim: int, first: int, columns: int, eps: float,
                 table: str = "side.embed", declares_table: bool = False, names: dict | None = None):
        if hidden_size <= 0 or vocab_size <= 0 or dim <= 0 or first < 0 or first + dim > columns or eps <= 0:
            raise ValueError("gated_token_row: sizes must be positive and the columns must lie in the table")
        self.hidden_size, self.vocab_size, self.dim, self.first, self.columns = hidden_size, vocab_size, dim, first, columns
        self.eps, self.table_name, self.declares_table = float(eps), table, bool(declares_table)
        names = names or {"gate": "side.gate", "proj": "side.proj", "norm": "side.norm"}
        self.names = {key: prefix + value for key, value in names.items()}
        self.runtime = None

    def tensor_decls(self):
        decls = [TensorDecl(self.table_name, (self.vocab_size, self.columns))] if self.declares_table else []
        return decls + [TensorDecl(self.names["gate"], (self.dim, self.hidden_size)),
                        TensorDecl(self.names["proj"], (self.hidden_size, self.dim)),
                        TensorDecl(self.names["norm"], (self.hidden_size,), "gain")]

    def load(self, source: WeightSource):
        self.runtime = source.runtime
        status = source.runtime.status
        self.table = source.matrix(self.table_name)                      # loaded once, whichever layer asks first
        self.gate = Linear(source.matrix(self.names["gate"]), None, status, any_inner_size=True)
        self.proj = Linear(source.matrix(self.names["proj"]), None, status, any_inner_size=True)
        self.gain = source.vector(self.names["norm"])

    def forward(self, x, ctx):
        dtype = self.runtime.dtype
        if dtype != torch.float32 and x.shape[0] <= kernels.SIDE_FEW_TOKENS and self.dim <= kernels.SIDE_FEW_MAX_DIM \
                and self.hidden_size <= 10240:
            # a handful of tokens: two light launches (the gated row; the projection with the norm and the sum).  The 32-bit
            # path keeps the products whose order of additions does not depend on the number of tokens
            kernels.side_input_few(x, self.gate.weight, self.proj.weight, self.gain, self.table, self.first, ctx.token_ids, self.eps,
                                   self.runtime.status)
            return
        stream = x if dtype == torch.float32 else kernels.narrow_rows(x)      # the projection reads the stream in the compute dtype
        z = self.gate.forward(stream)
        g = torch.empty((x.shape[0], self.dim), dtype=dtype, device=x.device)
        kernels.side_gate(z, self.table, self.first, ctx.token_ids, g, self.runtime.status)
        y = self.proj.forward(g, out_dtype=torch.float32)
        kernels.rms_add(y, self.gain, x, self.eps)

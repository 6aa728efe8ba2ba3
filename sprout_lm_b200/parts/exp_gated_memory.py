"""A matrix memory with exponential gates (the mLSTM recurrence): a float32 state per request and head, no keys or values
per token.

q = W_q h * dim^(-1/2), k = W_k h (heads x dim), v = W_v h (heads x value_dim).  Per head a log input gate
i = cap tanh((W_i h + b_i) / cap) and a log forget gate f = logsigmoid(cap tanh((W_f h + b_f) / cap)) (``gate_cap``; None: the
projections as they are), and with a running maximum m that starts at 0:

    m_t = max(f_t + m_(t-1), i_t)
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

Each head's o is divided by its root mean square over value_dim (``eps``); the heads side by side are multiplied by a weight
[heads * value_dim] and by sigmoid(W_g h), then projected by W_o.  ``out_scale`` multiplies the mixer's output.

The state has two tensors per request: [heads, dim, value_dim + up to 4] float32, whose column ``value_dim`` is n (the scan
feeds that column the constant 1 as a value; the columns after it are padding that keeps rows on 16-byte boundaries), and the
running maxima [heads].  Both start at zero.  The scan is the one of ``csrc/gated_recurrence.cu`` with ready-made decays per
head; the gates and the maxima are made first, in the tokens' order (``csrc/exp_gated_memory.cu``).  Everything but the matrix
products is float32 in both compute dtypes, and the projections leave their product in float32 as well, so nothing that
enters the recurrence is rounded to 16 bits.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, StateSpec, StateView, TensorDecl, WeightSource, register_part
from .linear import Linear


@register_part("mixer", "exp_gated_matrix_memory")
class ExpGatedMatrixMemory(Part):
    DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "f": "f", "i_bias": "i.b",
                     "f_bias": "f.b"}

    def __init__(self, prefix: str, hidden_size: int, heads: int, dim: int, value_dim: int, eps: float, gate_cap: float | None = None,
                 out_scale: float = 1.0, names: dict | None = None):
        if hidden_size <= 0 or heads <= 0 or dim <= 0 or value_dim <= 0 or eps <= 0:
            raise ValueError("exp_gated_matrix_memory: sizes and eps must be positive")
        if gate_cap is not None and gate_cap <= 0:
            raise ValueError("exp_gated_matrix_memory: the gates' cap must be positive")
        self.hidden_size, self.heads, self.dim, self.value_dim = hidden_size, heads, dim, value_dim
        self.eps, self.gate_cap, self.out_scale = float(eps), None if gate_cap is None else float(gate_cap), float(out_scale)
        self.state_cols = (value_dim + 1 + 3) // 4 * 4          # the values' columns, the normaliser's, padding to a multiple of 4
        self.names = {key: prefix + value for key, value in {**self.DEFAULT_NAMES, **(names or {})}.items()}
        self.runtime = None

    def cache_spec(self):
        return None

    def state_spec(self):
        return (StateSpec(shape=(self.heads, self.dim, self.state_cols), dtype=torch.float32),
                StateSpec(shape=(self.heads,), dtype=torch.float32))

    def tensor_decls(self):
        n, qk, vw = self.names, self.heads * self.dim, self.heads * self.value_dim
        return [TensorDecl(n["q"], (qk, self.hidden_size)), TensorDecl(n["k"], (qk, self.hidden_size)),
                TensorDecl(n["v"], (vw, self.hidden_size)), TensorDecl(n["g"], (vw, self.hidden_size)),
                TensorDecl(n["o"], (self.hidden_size, vw)), TensorDecl(n["norm"], (vw,), "gain"),
                TensorDecl(n["i"], (self.heads, self.hidden_size)), TensorDecl(n["i_bias"], (self.heads,), "bias"),
                TensorDecl(n["f"], (self.heads, self.hidden_size)), TensorDecl(n["f_bias"], (self.heads,), "bias")]

    def load(self, source: WeightSource):
        n, status = self.names, source.runtime.status
        self.runtime = source.runtime
        # one product for everything that reads h: [q | k | v | g | i | f], padded to rows of a multiple of 4 floats
        fused = torch.cat([source.raw(n[key]) for key in ("q", "k", "v", "g", "i", "f")], dim=0)
        if fused.shape[0] % 8:
            fused = torch.cat([fused, fused.new_zeros((8 - fused.shape[0] % 8, fused.shape[1]))], dim=0)
        self.proj = Linear(source.to_device_matrix(fused), None, status, any_inner_size=True)
        self.bias_i, self.bias_f = source.vector(n["i_bias"]), source.vector(n["f_bias"])
        self.gain = source.vector(n["norm"])
        self.out = Linear(source.matrix(n["o"]), None, status, any_inner_size=True)

    def forward(self, h, x, ctx, cache, state: StateView):
        """x (float32) += out_scale * W_o (per-head rmsnorm(o) * w * sigmoid(W_g h)); the requests' states advance."""
        if state is None:
            raise RuntimeError("exp_gated_matrix_memory: the layer needs a state slot per request")
        status = self.runtime.status
        rows = self.proj.forward_float32(h)                     # float32 whatever the compute dtype
        qk, vw, heads = self.heads * self.dim, self.heads * self.value_dim, self.heads
        q, k, v = rows[:, :qk], rows[:, qk:2 * qk], rows[:, 2 * qk:2 * qk + vw]
        gate = rows[:, 2 * qk + vw:2 * qk + 2 * vw]
        at = 2 * qk + 2 * vw
        memory, tops = state.part(0), state.part(1)
        a, c, m = kernels.exp_gates(rows[:, at:at + heads], rows[:, at + heads:at + 2 * heads], self.bias_i, self.bias_f,
                                    self.gate_cap or 0.0, ctx, tops.buffer, tops.slots, status)
        o = torch.empty((rows.shape[0], heads * self.state_cols), dtype=torch.float32, device=rows.device)
        kernels.gated_scan(q, k, v, None, None, ctx, memory, o, heads, heads, self.dim, self.state_cols, status,
                           q_scale=self.dim ** -0.5, given=(a, c), ones_col=True)
        gated = torch.empty((rows.shape[0], vw), dtype=h.dtype, device=rows.device)
        kernels.exp_memory_out(o, m, gate, self.gain, gated, heads, self.value_dim, self.eps, self.out_scale)
        self.out.forward(gated, residual=x)

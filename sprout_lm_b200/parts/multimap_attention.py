"""Grouped-query attention whose heads hold one or two softmax maps over shared values (two: differential
attention), on the paged cache.

With ``maps`` = 2 a query head has two query vectors and a key/value head two key vectors of ``dim`` elements, laid
out head by head as [map 0, map 1], and one value vector of ``value_dim`` elements.  Each map is a causal softmax
attention of its own (score = scale * q . k) over the head's values; the head's output is
a_0 - lambda * a_1 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (one number per layer, learned vectors of
``dim`` elements), divided by its root mean square over the head's values (``norm_eps``; no weight) and multiplied by
``out_scale``.  The first ``2 * table width`` elements of every query and key vector are rotated by the position.
The cache keeps a key/value head's maps side by side in one key row (rotated) and its value row.

Options, each a constructor parameter: ``mask`` = ("window", n) lets a query see itself and the n - 1 positions before
it (the cache slot is then of kind ``window``: pages no later query can see are given back), ("window", n, first) also the
first ``first`` positions of the sequence, which keep their own positions (their pages stay), ("chunk", n) the positions
of its own chunk of n, counted from position 0; ``softcap`` > 0: every scaled score s becomes softcap * tanh(s / softcap);
``bias``: the query, key and value projections have biases (the matrix's name + ".b"); ``qk_norm_eps`` > 0: before the
rotation every query and key vector is divided by its root mean square over ``dim`` and multiplied by a weight of ``dim``
elements (``q_norm`` for queries, ``k_norm`` for keys, each shared by the heads); ``sink``: a learned number per head whose exponential joins every softmax
denominator (no key, no value, not scaled); ``gate``: head h's output is multiplied by sigmoid(W_g h)_h, W_g [heads,
hidden], read from the same input as the projections; ``unit_norm_eps`` > 0: after the rotation every query and key
vector is divided by its root mean square over ``dim``; ``value_from_key``: there is no value projection, the value row
is the key row as projected, before rotation and norm (``value_dim`` = ``maps * dim``).

A layer may read the keys and values another layer cached (its run-order entry has ``writes_cache=False``): it then
has no key and value projections, only queries, lambda vectors and the output projection of its own.
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..config.specs import PartSpec
from .base import CacheSpec, CacheView, Part, TensorDecl, WeightSource, build_part, register_part
from .linear import Linear

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2", "sink": "sink",
                 "g": "g", "q_norm": "q.norm", "k_norm": "k.norm"}
BIAS_SUFFIX = ".b"


@register_part("mixer", "multimap_attention")
class MultiMapAttention(Part):
    def __init__(self, prefix: str, hidden_size: int, heads: int, kv_heads: int, dim: int, value_dim: int, scale: float,
                 position: PartSpec, maps: int = 2, diff: float = 0.0, norm_eps: float = 0.0, out_scale: float = 1.0,
                 own_kv: bool = True, names: dict | None = None, mask=None, sink: bool = False, gate: bool = False,
                 unit_norm_eps: float = 0.0, value_from_key: bool = False, softcap: float = 0.0, bias: bool = False,
                 qk_norm_eps: float = 0.0):
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ValueError(f"multimap_attention: heads ({heads}) must be a positive multiple of kv_heads ({kv_heads})")
        if maps not in (1, 2):
            raise ValueError("multimap_attention: one or two maps per head")
        if dim <= 0 or value_dim <= 0 or value_dim > 512:
            raise ValueError("multimap_attention: dim must be positive and value_dim at most 512")
        mask = None if mask is None or mask[0] == "causal" else tuple([str(mask[0])] + [int(n) for n in mask[1:]])
        if mask is not None and (mask[0] not in ("window", "chunk") or mask[1] <= 0 or len(mask) > 3
                                 or (len(mask) == 3 and (mask[0] != "window" or mask[2] < 0))):
            raise ValueError("multimap_attention: mask must be ('window', n[, kept first positions]) or ('chunk', n) with n > 0")
        if mask is not None and len(mask) == 3 and mask[2] == 0:
            mask = mask[:2]
        if softcap < 0 or qk_norm_eps < 0:
            raise ValueError("multimap_attention: softcap and qk_norm_eps must not be negative")
        if bias and not own_kv:
            raise ValueError("multimap_attention: biases are for layers with projections of their own")
        self.softcap, self.has_bias, self.qk_norm_eps = float(softcap), bool(bias), float(qk_norm_eps)
        self.q_norm = self.k_norm = None
        if value_from_key and value_dim != maps * dim:
            raise ValueError("multimap_attention: values that are the keys have the keys' width")
        if unit_norm_eps < 0:
            raise ValueError("multimap_attention: unit_norm_eps must not be negative")
        self.mask, self.has_sink, self.has_gate = mask, bool(sink), bool(gate)
        self.unit_norm_eps, self.value_from_key = float(unit_norm_eps), bool(value_from_key)
        self.hidden_size, self.heads, self.kv_heads, self.dim, self.value_dim = hidden_size, heads, kv_heads, dim, value_dim
        self.maps, self.scale, self.diff = maps, float(scale), float(diff)
        self.norm_eps, self.out_scale, self.own_kv = float(norm_eps), float(out_scale), bool(own_kv)
        self.names = {key: prefix + value for key, value in {**DEFAULT_NAMES, **(names or {})}.items()}
        self.position = build_part("position", position)
        self.q_width = heads * maps * dim
        self.k_width = kv_heads * maps * dim
        self.v_width = 0 if self.value_from_key else kv_heads * value_dim
        self.lam = 0.0
        self.sink = None
        self.runtime = None

    def cache_spec(self):
        if self.mask is not None and self.mask[0] == "window":
            return CacheSpec(kv_heads=self.kv_heads, head_dim=self.maps * self.dim, kind="window", window=self.mask[1],
                             value_dim=self.value_dim, keep_first=self.mask[2] if len(self.mask) > 2 else 0)
        return CacheSpec(kv_heads=self.kv_heads, head_dim=self.maps * self.dim, kind="full", value_dim=self.value_dim)

    def state_spec(self):
        return None

    def decode_plan(self, requests: int, max_keys: int, planned_context: int, page_tokens: int):
        """Into how many CTAs a step of one token per request divides a request's keys: it follows the contexts' length."""
        return kernels.multimap_key_split(requests, self.kv_heads, self.heads // self.kv_heads, 1,
                                          kernels.visible_keys(self.mask, planned_context))

    def tensor_decls(self):
        n = self.names
        decls = [TensorDecl(n["q"], (self.q_width, self.hidden_size))]
        if self.own_kv:
            decls.append(TensorDecl(n["k"], (self.k_width, self.hidden_size)))
            if not self.value_from_key:
                decls.append(TensorDecl(n["v"], (self.v_width, self.hidden_size)))
        if self.has_sink:
            decls.append(TensorDecl(n["sink"], (self.heads,), "bias"))
        if self.has_gate:
            decls.append(TensorDecl(n["g"], (self.heads, self.hidden_size)))
        if self.has_bias:
            decls.append(TensorDecl(n["q"] + BIAS_SUFFIX, (self.q_width,), "bias"))
            decls.append(TensorDecl(n["k"] + BIAS_SUFFIX, (self.k_width,), "bias"))
            if not self.value_from_key:
                decls.append(TensorDecl(n["v"] + BIAS_SUFFIX, (self.v_width,), "bias"))
        if self.qk_norm_eps > 0:
            decls += [TensorDecl(n["q_norm"], (self.dim,), "gain"), TensorDecl(n["k_norm"], (self.dim,), "gain")]
        if self.maps == 2:
            decls += [TensorDecl(n[key], (self.dim,), "wide") for key in ("lq1", "lk1", "lq2", "lk2")]
        decls.append(TensorDecl(n["o"], (self.hidden_size, self.heads * self.value_dim)))
        return decls

    def load(self, source: WeightSource):
        n, status = self.names, source.runtime.status
        self.runtime = source.runtime
        keys = (("q", "k") if self.value_from_key else ("q", "k", "v")) if self.own_kv else ("q",)
        if self.has_gate:
            keys += ("g",)                 # the gates' columns follow the projections' in the fused product
        fused = torch.cat([source.raw(n[key]) for key in keys], dim=0)
        self.gate_at = fused.shape[0] - self.heads
        if fused.shape[0] % 8:
            # rows of the product that start on 16-byte boundaries: the tensor-core attention fetches queries 16 bytes at a time
            fused = torch.cat([fused, fused.new_zeros((8 - fused.shape[0] % 8, fused.shape[1]))], dim=0)
        if self.has_sink:
            self.sink = source.vector(n["sink"])
        bias = None
        if self.has_bias:
            # the projections' biases, zeros for the gates' and the padding's columns
            bias = torch.zeros(fused.shape[0], dtype=torch.float32)
            at = 0
            for key in keys:
                rows = source.raw(n[key]).shape[0]
                if key != "g":
                    bias[at:at + rows] = source.raw(n[key] + BIAS_SUFFIX).to(torch.float32)
                at += rows
            bias = bias.to(source.runtime.device)
        if self.qk_norm_eps > 0:
            self.q_norm, self.k_norm = source.vector(n["q_norm"]), source.vector(n["k_norm"])
        self.qkv = Linear(source.to_device_matrix(fused), bias, status, any_inner_size=True)
        self.out = Linear(source.matrix(n["o"]), None, status, any_inner_size=True)
        if self.maps == 2:
            lq1, lk1, lq2, lk2 = (source.raw(n[key]).to(torch.float32) for key in ("lq1", "lk1", "lq2", "lk2"))
            # one number per layer, in float32 as the other 32-bit quantities
            self.lam = float(torch.exp(torch.sum(lq1 * lk1)) - torch.exp(torch.sum(lq2 * lk2)) + torch.tensor(self.diff, dtype=torch.float32))
        self.tables = self.position.rotary_tables(source.runtime)
        if self.tables is not None and 2 * self.tables[0].shape[1] > self.dim:
            raise ValueError("multimap_attention: the rotation is wider than a query vector")

    def forward(self, h, x, ctx, cache: CacheView, state=None):
        """x (float32) += W_o attention(h); appends this step's keys and values when the cache slot is this layer's."""
        if cache.write != self.own_kv:
            raise RuntimeError("multimap_attention: a layer with key and value projections of its own writes its cache slot, "
                               "a layer without them reads another layer's")
        status = self.runtime.status
        cos, sin = self.tables if self.tables is not None else (None, None)
        rows = self.qkv.forward(h)
        kernels.rope_maps_append(rows, ctx.positions, ctx.seq_of_token, cache.block_table, cos, sin, cache.k, cache.v,
                                 self.heads * self.maps, self.kv_heads, self.maps, self.dim, self.value_dim, cache.page_tokens,
                                 cache.write, status, unit_eps=self.unit_norm_eps, value_from_key=self.value_from_key,
                                 q_weight=self.q_norm, k_weight=self.k_norm, weight_eps=self.qk_norm_eps)
        attended = torch.empty((rows.shape[0], self.heads * self.value_dim), dtype=rows.dtype, device=rows.device)
        kernels.multimap_attention(rows[:, :self.q_width], cache, ctx, attended, self.heads, self.kv_heads, self.maps, self.dim,
                                   self.value_dim, self.scale, self.lam, self.norm_eps, self.out_scale, status, mask=self.mask,
                                   sink=self.sink, gate=rows[:, self.gate_at:self.gate_at + self.heads] if self.has_gate else None,
                                   softcap=self.softcap)
        self.out.forward(attended, residual=x)

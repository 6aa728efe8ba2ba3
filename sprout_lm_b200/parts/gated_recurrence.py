"""Recurrent mixers whose decay is made from the input: a float32 state per request and head, no keys or values per token.

Both run S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T, o_t = S_t^T q_t per head on the same scan kernel
(``csrc/gated_recurrence.cu``); the state [heads, dim, value_dim] starts at zero, is float32 and lives in the request's
state slot.  Everything that enters the recurrence beside the projections (decays and their logarithms, softplus,
exponentials, step sizes, norms) is float32 in both compute dtypes.

``gated_linear_attention``: q = W_q h * dim^(-1/2), k = W_k h (heads x dim), v = W_v h (heads x value_dim); a decay per key
channel a = sigmoid(z)^(1 / tau) with z = W_a2 (W_a1 h) + b_a2 (heads x dim), c = 1.  Each head's o is divided by its root
mean square over value_dim and multiplied by a weight [value_dim] that the heads share; the heads side by side are
multiplied by silu(W_g h) and projected by W_o.

``selective_state_space``: W_in h = [z: inner | x: inner | B: groups x state | C: groups x state | dt: heads] with
inner = heads x value_dim; x, B and C pass a causal convolution per channel (``taps`` taps, a bias, zeros before the
start of the sequence) and silu; dt = softplus(dt + dt_bias); per head (head h reads group h // (heads / groups)):
a = exp(-exp(A_log_h) dt) for all of the head's rows, c = dt, k = B, q = C, v = x, and o gets D_h x added.  The heads side
by side are multiplied by silu(z), then divided in ``norm_groups`` equal parts by each part's root mean square and
multiplied by a weight [inner], then projected by W_o.  The convolution's last taps - 1 inputs are a second state tensor.

``out_scale`` multiplies the mixer's output (it is folded into the norm's weight), so that a block that runs several
mixers side by side can weigh them without a kernel of its own.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, StateSpec, StateView, TensorDecl, WeightSource, register_part
from .linear import Linear


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Part):
    DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"}

    def __init__(self, prefix: str, hidden_size: int, heads: int, dim: int, value_dim: int, tau: float, eps: float,
                 decay_rank: int | None = None, out_scale: float = 1.0, names: dict | None = None):
        if hidden_size <= 0 or heads <= 0 or dim <= 0 or value_dim <= 0 or tau <= 0 or eps <= 0:
            raise ValueError("gated_linear_attention: sizes, tau and eps must be positive")
        if decay_rank is not None and decay_rank <= 0:
            raise ValueError("gated_linear_attention: the decay's inner size must be positive")
        self.hidden_size, self.heads, self.dim, self.value_dim = hidden_size, heads, dim, value_dim
        self.tau, self.eps, self.out_scale, self.decay_rank = float(tau), float(eps), float(out_scale), decay_rank
        self.names = {key: prefix + value for key, value in {**self.DEFAULT_NAMES, **(names or {})}.items()}
        self.runtime = None

    def cache_spec(self):
        return None

    def state_spec(self):
        return StateSpec(shape=(self.heads, self.dim, self.value_dim), dtype=torch.float32)

    def tensor_decls(self):
        n, qk, vw, rank = self.names, self.heads * self.dim, self.heads * self.value_dim, self.decay_rank
        # rank None: the decay's inner size is whatever the checkpoint's tensors have
        return [TensorDecl(n["q"], (qk, self.hidden_size)), TensorDecl(n["k"], (qk, self.hidden_size)),
                TensorDecl(n["v"], (vw, self.hidden_size)), TensorDecl(n["g"], (vw, self.hidden_size)),
                TensorDecl(n["a1"], (rank, self.hidden_size)), TensorDecl(n["a2"], (qk, rank)),
                TensorDecl(n["a2_bias"], (qk,), "bias"), TensorDecl(n["norm"], (self.value_dim,), "gain"),
                TensorDecl(n["o"], (self.hidden_size, vw))]

    def load(self, source: WeightSource):
        n, status = self.names, source.runtime.status
        self.runtime = source.runtime
        # one product for everything that reads h; the decay's inner vector stands first, so that its view starts where
        # the rows start
        fused = torch.cat([source.raw(n[key]) for key in ("a1", "q", "k", "v", "g")], dim=0)
        self.rank = source.raw(n["a1"]).shape[0]
        if source.raw(n["a2"]).shape[1] != self.rank:
            raise ValueError("gated_linear_attention: the decay's two matrices do not fit each other")
        self.proj = Linear(source.to_device_matrix(fused), None, status, any_inner_size=True)
        self.decay_out = Linear(source.matrix(n["a2"]), None, status, any_inner_size=True)
        self.decay_bias = source.vector(n["a2_bias"])
        self.gain = (source.vector(n["norm"]) * self.out_scale).contiguous()
        self.out = Linear(source.matrix(n["o"]), None, status, any_inner_size=True)

    def forward(self, h, x, ctx, cache, state: StateView):
        """x (float32) += out_scale * W_o (rmsnorm_per_head(o) * w * silu(W_g h)); the requests' states advance."""
        if state is None:
            raise RuntimeError("gated_linear_attention: the layer needs a state slot per request")
        rows = self.proj.forward(h)
        qk, vw = self.heads * self.dim, self.heads * self.value_dim
        at = self.rank
        z = self.decay_out.forward(rows[:, :at], out_dtype=torch.float32)
        q, k, v = rows[:, at:at + qk], rows[:, at + qk:at + 2 * qk], rows[:, at + 2 * qk:at + 2 * qk + vw]
        gate = rows[:, at + 2 * qk + vw:]
        o = torch.empty((rows.shape[0], vw), dtype=torch.float32, device=rows.device)
        kernels.gated_scan(q, k, v, z, self.decay_bias, ctx, state, o, self.heads, self.heads, self.dim, self.value_dim,
                           self.runtime.status, tau=self.tau, q_scale=self.dim ** -0.5)
        gated = torch.empty((rows.shape[0], vw), dtype=rows.dtype, device=rows.device)
        kernels.gated_group_norm(o, gate, self.gain, gated, self.eps, groups=self.heads, gate_first=False, silu=True)
        self.out.forward(gated, residual=x)


@register_part("mixer", "selective_state_space")
class SelectiveStateSpace(Part):
    DEFAULT_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D",
                     "norm": "norm", "o": "o"}

    def __init__(self, prefix: str, hidden_size: int, heads: int, value_dim: int, state: int, groups: int, taps: int,
                 norm_groups: int, eps: float, out_scale: float = 1.0, names: dict | None = None):
        if hidden_size <= 0 or heads <= 0 or value_dim <= 0 or state <= 0 or groups <= 0 or heads % groups or eps <= 0:
            raise ValueError("selective_state_space: sizes and eps must be positive, heads a multiple of groups")
        if taps < 2:
            raise ValueError("selective_state_space: the convolution has at least two taps")
        if norm_groups <= 0 or (heads * value_dim) % norm_groups:
            raise ValueError("selective_state_space: the norm's parts must divide heads * value_dim")
        self.hidden_size, self.heads, self.value_dim, self.state, self.groups = hidden_size, heads, value_dim, state, groups
        self.taps, self.norm_groups, self.eps, self.out_scale = taps, norm_groups, float(eps), float(out_scale)
        self.inner = heads * value_dim
        self.channels = self.inner + 2 * groups * state           # what the convolution sees: x, B, C
        self.names = {key: prefix + value for key, value in {**self.DEFAULT_NAMES, **(names or {})}.items()}
        self.runtime = None

    def cache_spec(self):
        return None

    def state_spec(self):
        return (StateSpec(shape=(self.taps - 1, self.channels), dtype=torch.float32),
                StateSpec(shape=(self.heads, self.state, self.value_dim), dtype=torch.float32))

    def tensor_decls(self):
        n = self.names
        return [TensorDecl(n["in"], (self.inner + self.channels + self.heads, self.hidden_size)),
                TensorDecl(n["conv"], (self.channels, self.taps), "conv"), TensorDecl(n["conv_bias"], (self.channels,), "bias"),
                TensorDecl(n["dt_bias"], (self.heads,), "bias"), TensorDecl(n["a_log"], (self.heads,), "bias"),
                TensorDecl(n["skip"], (self.heads,), "gain"), TensorDecl(n["norm"], (self.inner,), "gain"),
                TensorDecl(n["o"], (self.hidden_size, self.inner))]

    def load(self, source: WeightSource):
        n, status = self.names, source.runtime.status
        self.runtime = source.runtime
        self.proj = Linear(source.matrix(n["in"]), None, status, any_inner_size=True)
        self.conv = source.vector(n["conv"])
        self.conv_bias = source.vector(n["conv_bias"])
        self.dt_bias, self.a_log, self.skip = source.vector(n["dt_bias"]), source.vector(n["a_log"]), source.vector(n["skip"])
        self.gain = (source.vector(n["norm"]) * self.out_scale).contiguous()
        self.out = Linear(source.matrix(n["o"]), None, status, any_inner_size=True)

    def forward(self, h, x, ctx, cache, state: StateView):
        if state is None:
            raise RuntimeError("selective_state_space: the layer needs a state slot per request")
        status = self.runtime.status
        rows = self.proj.forward(h)
        inner, gn = self.inner, self.groups * self.state
        conv = torch.empty((rows.shape[0], self.channels), dtype=rows.dtype, device=rows.device)
        kernels.causal_conv(rows[:, inner:inner + self.channels], self.conv, self.conv_bias, conv, ctx, state.part(0), status,
                            silu=True)
        y = torch.empty((rows.shape[0], inner), dtype=torch.float32, device=rows.device)
        kernels.gated_scan(conv[:, inner + gn:], conv[:, inner:inner + gn], conv[:, :inner], rows[:, inner + self.channels:],
                           self.dt_bias, ctx, state.part(1), y, self.heads, self.groups, self.state, self.value_dim, status,
                           per_head=True, a_log=self.a_log, skip=self.skip)
        gated = torch.empty((rows.shape[0], inner), dtype=rows.dtype, device=rows.device)
        kernels.gated_group_norm(y, rows[:, :inner], self.gain, gated, self.eps, groups=self.norm_groups, gate_first=True,
                                 silu=True)
        self.out.forward(gated, residual=x)

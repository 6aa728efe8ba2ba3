"""SwiGLU feed-forward: x += W_down (silu(W_gate h) * W_up h), no biases (src/qwen.ts:196-200).

Gate and up are one fused product.  On the tensor-core path its weight rows interleave the two
in blocks of 8 (rows 16b..16b+7 are gate rows 8b..8b+7, rows 16b+8..16b+15 the matching up
rows), so that the product's epilogue sees a gate value and its up value side by side; that needs
an intermediate size that is a multiple of 8.  The 32-bit path has no such epilogue: it keeps the
gate rows first and the up rows after them, and takes any intermediate size.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorDecl, WeightSource, register_part
from .linear import Linear, small_batch_enabled

INTERLEAVE = 8
FUSED_TOKENS = 16         # the one-kernel decode form takes up to this many tokens (two tiles of the MMA's 8 columns)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = INTERLEAVE) -> torch.Tensor:
    inter, hidden = gate.shape
    blocks = inter // block
    return torch.stack([gate.reshape(blocks, block, hidden), up.reshape(blocks, block, hidden)],
                       dim=1).reshape(2 * inter, hidden).contiguous()


@register_part("feed_forward", "swiglu_mlp")
class SwiGLUMLP(Part):
    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, names: dict | None = None):
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("swiglu_mlp: sizes must be positive")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.block = INTERLEAVE            # rows of gate, then as many of up, and so on (set at load)
        names = names or {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}
        self.names = {key: prefix + value for key, value in names.items()}
        self.gate_up = self.down = None
        self._fused_tokens = 0            # up to this many tokens the one-kernel decode form runs

    def tensor_decls(self):
        return [TensorDecl(self.names["gate"] + ".weight", (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["up"] + ".weight", (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["down"] + ".weight", (self.hidden_size, self.intermediate_size))]

    def load(self, source: WeightSource):
        if source.runtime.dtype == torch.bfloat16:
            if self.intermediate_size % INTERLEAVE:
                raise ValueError(f"swiglu_mlp: on the bfloat16 path intermediate_size must be a multiple of {INTERLEAVE} "
                                 f"(got {self.intermediate_size}): the tensor-core epilogue pairs gate and up rows in "
                                 f"blocks of {INTERLEAVE}; the float32 path takes any size")
            self.block = INTERLEAVE
        else:
            self.block = self.intermediate_size
        fused = interleave_gate_up(source.raw(self.names["gate"] + ".weight"), source.raw(self.names["up"] + ".weight"),
                                   self.block)
        self.gate_up = Linear(source.to_device_matrix(fused), None, source.runtime.status)
        self.down = Linear(source.matrix(self.names["down"] + ".weight"), None, source.runtime.status)
        # Small layers decode in one kernel that also takes the norm before the feed-forward
        # (csrc/ffn_decode.cu).
        if self.gate_up.weight.dtype == torch.bfloat16 and small_batch_enabled():
            for tokens in (FUSED_TOKENS, 8):             # two tiles of 8 tokens where the layer's shares leave room, else one
                if kernels.ffn_decode_supported(tokens, self.hidden_size, self.intermediate_size):
                    self._fused_tokens = tokens
                    break

    def forward(self, h, x, ctx=None):
        self.down.forward(self.gate_up.forward_swiglu(h, self.block), residual=x)

    def forward_with_norm(self, norm, x, ctx=None) -> bool:
        """x += feed_forward(norm(x)) in one kernel, if this layer and this batch allow it: an
        RMSNorm before it, a few tokens, a layer that fits.  False means nothing was done and the
        caller runs the norm and ``forward``."""
        tokens = x.shape[0]
        if getattr(norm, "fused_kind", None) != "rmsnorm" or tokens > self._fused_tokens:
            return False
        kernels.ffn_decode(x, norm.gain, norm.eps, self.gate_up.weight, self.down.weight, self.gate_up.status)
        return True


@register_part("feed_forward", "polynorm_mlp")
class PolyNormMLP(Part):
    """x += W_down act(W_up h) with act(z) = a N(z) + b N(z^2) + c N(z^3) + e: powers element by element,
    N divides a token's vector by its root mean square (eps inside the root), and (a, b, c, e) is a
    learned tensor of four numbers.  The up product's output and the three means are float32."""

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, eps: float, names: dict | None = None):
        if hidden_size <= 0 or intermediate_size <= 0 or eps <= 0:
            raise ValueError("polynorm_mlp: sizes and eps must be positive")
        self.hidden_size, self.intermediate_size, self.eps = hidden_size, intermediate_size, float(eps)
        names = names or {"up": "up.weight", "down": "down.weight", "act": "act"}
        self.names = {key: prefix + value for key, value in names.items()}
        self.up = self.down = self.coefficients = None

    def tensor_decls(self):
        return [TensorDecl(self.names["up"], (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["down"], (self.hidden_size, self.intermediate_size)),
                TensorDecl(self.names["act"], (4,), "polynomial")]

    def load(self, source: WeightSource):
        self.up = Linear(source.matrix(self.names["up"]), None, source.runtime.status, any_inner_size=True)
        self.down = Linear(source.matrix(self.names["down"]), None, source.runtime.status, any_inner_size=True)
        self.coefficients = source.vector(self.names["act"])

    def forward(self, h, x, ctx=None):
        z = self.up.forward_float32(h)
        act = torch.empty(z.shape, dtype=h.dtype, device=h.device)
        kernels.polynorm(z, act, self.coefficients, self.eps)
        self.down.forward(act, residual=x)


@register_part("feed_forward", "relu2_mlp")
class SquaredReLUMLP(Part):
    """x += W_down relu(W_up h)^2, no biases."""

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, names: dict | None = None):
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("relu2_mlp: sizes must be positive")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        names = names or {"up": "up", "down": "down"}
        self.names = {key: prefix + value for key, value in names.items()}
        self.up = self.down = None

    def tensor_decls(self):
        return [TensorDecl(self.names["up"], (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["down"], (self.hidden_size, self.intermediate_size))]

    def load(self, source: WeightSource):
        self.up = Linear(source.matrix(self.names["up"]), None, source.runtime.status, any_inner_size=True)
        self.down = Linear(source.matrix(self.names["down"]), None, source.runtime.status, any_inner_size=True)

    def forward(self, h, x, ctx=None):
        z = self.up.forward(h)
        kernels.relu2(z, z)
        self.down.forward(z, residual=x)


class ClampedGLU:
    """W_down f(W_gate h, W_up h) with f(g, u) = g' sigmoid(alpha g') (u' + 1), g' = min(g, limit),
    u' = clamp(u, -limit, limit): one dense expert.  Gate rows first, then up rows, in one fused matrix."""

    def __init__(self, gate, up, down, limit: float, alpha: float, source: WeightSource):
        status = source.runtime.status
        self.limit, self.alpha = float(limit), float(alpha)
        self.ff = gate.shape[0]
        self.gate_up = Linear(source.to_device_matrix(torch.cat([gate, up], dim=0)), None, status, any_inner_size=True)
        self.down = Linear(source.to_device_matrix(down), None, status, any_inner_size=True)

    def forward(self, h, x):
        gate_up = self.gate_up.forward(h)
        act = torch.empty((h.shape[0], self.ff), dtype=h.dtype, device=h.device)
        kernels.glu_clamped(gate_up, act, self.limit, self.alpha)
        self.down.forward(act, residual=x)


@register_part("feed_forward", "clamped_glu_mlp")
class ClampedGLUMLP(Part):
    """x += W_down (g' sigmoid(alpha g') (u' + 1)) with g' = min(W_gate h, limit), u' = clamp(W_up h, -limit, limit): the
    dense form of the layer the routed experts are made of (``ClampedGLU``)."""

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702,
                 names: dict | None = None):
        if hidden_size <= 0 or intermediate_size <= 0 or limit <= 0:
            raise ValueError("clamped_glu_mlp: sizes and limit must be positive")
        self.hidden_size, self.intermediate_size, self.limit, self.alpha = hidden_size, intermediate_size, float(limit), float(alpha)
        names = names or {"gate": "gate", "up": "up", "down": "down"}
        self.names = {key: prefix + value for key, value in names.items()}
        self.layer = None

    def tensor_decls(self):
        return [TensorDecl(self.names["gate"], (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["up"], (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["down"], (self.hidden_size, self.intermediate_size))]

    def load(self, source: WeightSource):
        gate, up, down = (source.raw(self.names[key]) for key in ("gate", "up", "down"))
        self.layer = ClampedGLU(gate, up, down, self.limit, self.alpha, source)

    def forward(self, h, x, ctx=None):
        self.layer.forward(h, x)


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """A mixture of small feed-forward layers of which each token uses ``top``.

    Router: z = W_router h in float32, s = softmax(z) over all ``experts + identity`` outputs; the ``top`` largest of
    s + correction are taken (the correction only steers the choice); their weights are s / (sum of the taken s + 1e-20)
    * ``scale``.  The last ``identity`` router outputs are identity experts: they have no tensors and return h itself.
    Experts and the optional shared expert (run for every token and added) are ``ClampedGLU`` layers with sizes and
    limits of their own.  x += weighted sum of the taken experts' outputs (+ shared expert).

    Tensors: ``router`` [experts + identity, hidden], ``correction`` [experts + identity], ``e<i>.gate|up|down``,
    ``shared.gate|up|down``."""

    def __init__(self, prefix: str, hidden_size: int, experts: int, identity: int, top: int, scale: float, expert_ff: int,
                 expert_limit: float, alpha: float = 1.702, shared_ff: int | None = None, shared_limit: float | None = None,
                 names: dict | None = None):
        if hidden_size <= 0 or experts < 0 or identity < 0 or experts + identity <= 0 or not 0 < top <= experts + identity:
            raise ValueError("routed_experts: bad sizes")
        if experts and (expert_ff <= 0 or expert_limit <= 0):
            raise ValueError("routed_experts: experts need a positive size and limit")
        if shared_ff is not None and (shared_ff <= 0 or shared_limit is None or shared_limit <= 0):
            raise ValueError("routed_experts: a shared expert needs a positive size and limit")
        self.hidden_size, self.experts, self.identity, self.top = hidden_size, experts, identity, top
        self.scale, self.expert_ff, self.expert_limit, self.alpha = float(scale), expert_ff, float(expert_limit), float(alpha)
        self.shared_ff, self.shared_limit = shared_ff, shared_limit
        self.prefix = prefix
        base = {"router": "router", "correction": "correction", "expert": "e{}.", "shared": "shared.",
                "gate": "gate", "up": "up", "down": "down"}
        self.names = {**base, **(names or {})}
        self.shared = None
        self.runtime = None

    def _expert_names(self, index):
        stem = self.prefix + (self.names["shared"] if index is None else self.names["expert"].format(index))
        return stem + self.names["gate"], stem + self.names["up"], stem + self.names["down"]

    def tensor_decls(self):
        outputs = self.experts + self.identity
        decls = [TensorDecl(self.prefix + self.names["router"], (outputs, self.hidden_size), "bias"),
                 TensorDecl(self.prefix + self.names["correction"], (outputs,), "bias")]
        for index in [*range(self.experts), *([None] if self.shared_ff else [])]:
            ff = self.shared_ff if index is None else self.expert_ff
            gate, up, down = self._expert_names(index)
            decls += [TensorDecl(gate, (ff, self.hidden_size)), TensorDecl(up, (ff, self.hidden_size)),
                      TensorDecl(down, (self.hidden_size, ff))]
        return decls

    def load(self, source: WeightSource):
        self.runtime = source.runtime
        device = source.runtime.device
        self.router = source.vector(self.prefix + self.names["router"])            # float32: the router's product is 32-bit
        self.correction = source.vector(self.prefix + self.names["correction"])
        if self.experts:
            stacks = [[], []]
            for index in range(self.experts):
                gate, up, down = (source.raw(name) for name in self._expert_names(index))
                stacks[0].append(torch.cat([gate, up], dim=0))
                stacks[1].append(down)
            self.w_gate_up = source.to_device_matrix(torch.stack(stacks[0]))        # [experts, 2 ff, hidden]
            self.w_down = source.to_device_matrix(torch.stack(stacks[1]))          # [experts, hidden, ff]
        if self.shared_ff:
            gate, up, down = (source.raw(name) for name in self._expert_names(None))
            self.shared = ClampedGLU(gate, up, down, self.shared_limit, self.alpha, source)
        self.counts = torch.zeros(max(self.experts, 1), dtype=torch.int32, device=device)   # left zeroed by every step
        self.offsets = torch.zeros(self.experts + 1, dtype=torch.int32, device=device)

    def forward(self, h, x, ctx=None):
        tokens, device = h.shape[0], h.device
        entries = tokens * self.top
        ids = torch.empty((tokens, self.top), dtype=torch.int32, device=device)
        weights = torch.empty((tokens, self.top), dtype=torch.float32, device=device)
        kernels.moe_route(h, self.router, self.correction, ids, weights, self.counts, self.experts, self.top, self.scale)
        place_of = torch.empty(entries, dtype=torch.int32, device=device)
        rows = None
        if self.experts:
            order = torch.empty(entries, dtype=torch.int32, device=device)
            kernels.moe_arrange(ids, self.counts, self.offsets, order, place_of, self.experts)
            act = torch.empty((entries, self.expert_ff), dtype=h.dtype, device=device)
            rows = torch.empty((entries, self.hidden_size), dtype=torch.float32, device=device)
            kernels.moe_experts(h, order, self.offsets, self.w_gate_up, self.w_down, act, rows, self.experts, self.top,
                                self.expert_limit, self.alpha)
        else:
            place_of.fill_(-1)
        if self.shared is not None:
            self.shared.forward(h, x)
        kernels.moe_combine(x, h, ids, weights, place_of, rows, self.top)

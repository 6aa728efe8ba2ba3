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


@register_part("feed_forward", "gated_mlp")
class GatedMLP(Part):
    """x += W_down (act(W_gate h) * (W_up h)), no biases; ``activation`` is "silu", "gelu_tanh" (the tanh form of gelu) or
    "gelu_erf" (the exact form).  One fused product for gate and up.  On the tensor-core path, for silu and the tanh form
    of gelu and sizes in multiples of 8, the rows interleave gate and up in blocks of 8 and the activation runs in the
    product's epilogue on the float32 accumulators; otherwise gate rows first, then up rows, and the activation is a
    kernel of its own (float32 arithmetic on the product's results)."""

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "gelu_tanh", names: dict | None = None):
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("gated_mlp: sizes must be positive")
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"gated_mlp: unknown activation {activation!r}")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        names = names or {"gate": "gate", "up": "up", "down": "down"}
        self.names = {key: prefix + value for key, value in names.items()}
        self.gate_up = self.down = None

    def tensor_decls(self):
        return [TensorDecl(self.names["gate"], (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["up"], (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["down"], (self.hidden_size, self.intermediate_size))]

    def load(self, source: WeightSource):
        status = source.runtime.status
        gate, up = source.raw(self.names["gate"]), source.raw(self.names["up"])
        self.in_epilogue = source.runtime.dtype == torch.bfloat16 and self.activation in ("silu", "gelu_tanh") \
            and self.intermediate_size % INTERLEAVE == 0 and self.hidden_size % 8 == 0
        fused = interleave_gate_up(gate, up, INTERLEAVE) if self.in_epilogue else torch.cat([gate, up], dim=0)
        self.gate_up = Linear(source.to_device_matrix(fused), None, status, any_inner_size=True)
        self.down = Linear(source.matrix(self.names["down"]), None, status, any_inner_size=True)

    def forward(self, h, x, ctx=None):
        if self.in_epilogue and h.stride(0) % 8 == 0:
            self.down.forward(self.gate_up.forward_gated(h, self.activation), residual=x)
            return
        if self.in_epilogue:
            raise RuntimeError("gated_mlp: the tensor-core path needs rows that start on 16-byte boundaries")
        gate_up = self.gate_up.forward(h)
        act = torch.empty((h.shape[0], self.intermediate_size), dtype=h.dtype, device=h.device)
        kernels.unit_act(gate_up, act, self.activation, gated=True)
        self.down.forward(act, residual=x)


class PlainUnit:
    """W_down act(W_up h): one expert without a gate."""

    def __init__(self, up, down, activation: str, source: WeightSource):
        status = source.runtime.status
        self.activation, self.ff = activation, up.shape[0]
        self.up = Linear(source.to_device_matrix(up), None, status, any_inner_size=True)
        self.down = Linear(source.to_device_matrix(down), None, status, any_inner_size=True)

    def forward(self, h, x, row_logits=None):
        """x += the unit's output, row t times sigmoid(row_logits[t]) when given (the factor goes onto the activation's rows:
        the product after it is linear)."""
        z = self.up.forward(h)
        kernels.unit_act(z, z, self.activation, gated=False, row_logits=row_logits)
        self.down.forward(z, residual=x)


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """A mixture of small feed-forward layers of which each token uses ``top``.

    Router: z = W_router h in float32, s = softmax(z) over all ``experts + identity`` outputs; the ``top`` largest of
    s + correction are taken (the correction only steers the choice); their weights are s / (sum of the taken s + 1e-20)
    * ``scale``.  The last ``identity`` router outputs are identity experts: they have no tensors and return h itself.
    Experts and the optional shared expert (run for every token and added) are ``ClampedGLU`` layers with sizes and
    limits of their own.  x += weighted sum of the taken experts' outputs (+ shared expert).

    Options: ``expert_kind`` = "plain": experts (and the shared one) are W_down gelu(W_up h) with the exact gelu, no gate
    and no limit; ``correction`` False: the scores alone decide; ``renormalize`` False: the weights are the taken scores
    times ``scale``; ``groups`` = (count, keep): the experts form ``count`` equal groups of neighbours, a group's score is
    its largest score, and only experts of the ``keep`` best groups can be taken; ``shared_gate``: the shared expert's
    output is multiplied by sigmoid(w_sg . h), one number per token, its row ``shared.sg`` [1, hidden] multiplied in the
    router's 32-bit product.

    Tensors: ``router`` [experts + identity, hidden], ``correction`` [experts + identity], ``e<i>.gate|up|down``,
    ``shared.gate|up|down`` (no ``gate`` matrices for plain experts), ``shared.sg``."""

    def __init__(self, prefix: str, hidden_size: int, experts: int, identity: int, top: int, scale: float, expert_ff: int,
                 expert_limit: float = 0.0, alpha: float = 1.702, shared_ff: int | None = None, shared_limit: float | None = None,
                 names: dict | None = None, expert_kind: str = "clamped_glu", correction: bool = True, renormalize: bool = True,
                 groups=None, shared_gate: bool = False):
        if hidden_size <= 0 or experts < 0 or identity < 0 or experts + identity <= 0 or not 0 < top <= experts + identity:
            raise ValueError("routed_experts: bad sizes")
        if expert_kind not in ("clamped_glu", "plain"):
            raise ValueError("routed_experts: experts are 'clamped_glu' or 'plain'")
        self.plain = expert_kind == "plain"
        if experts and (expert_ff <= 0 or (not self.plain and expert_limit <= 0)):
            raise ValueError("routed_experts: experts need a positive size and limit")
        if shared_ff is not None and (shared_ff <= 0 or (not self.plain and (shared_limit is None or shared_limit <= 0))):
            raise ValueError("routed_experts: a shared expert needs a positive size and limit")
        if groups is not None:
            count, keep = int(groups[0]), int(groups[1])
            if count <= 0 or not 0 < keep <= count or (experts + identity) % count or top > keep * ((experts + identity) // count):
                raise ValueError("routed_experts: the groups must be equal and the kept ones must hold at least `top` experts")
            groups = (count, keep)
        if shared_gate and shared_ff is None:
            raise ValueError("routed_experts: a gate without a shared expert")
        self.has_correction, self.renormalize, self.groups, self.shared_gate = bool(correction), bool(renormalize), groups, bool(shared_gate)
        if self.plain:
            expert_limit = 0.0           # what tells the experts' kernels that there is no gate
        self.hidden_size, self.experts, self.identity, self.top = hidden_size, experts, identity, top
        self.scale, self.expert_ff, self.expert_limit, self.alpha = float(scale), expert_ff, float(expert_limit), float(alpha)
        self.shared_ff, self.shared_limit = shared_ff, shared_limit
        self.prefix = prefix
        base = {"router": "router", "correction": "correction", "expert": "e{}.", "shared": "shared.",
                "gate": "gate", "up": "up", "down": "down", "shared_gate": "shared.sg"}
        self.names = {**base, **(names or {})}
        self.shared = None
        self.runtime = None

    def _expert_names(self, index):
        stem = self.prefix + (self.names["shared"] if index is None else self.names["expert"].format(index))
        return stem + self.names["gate"], stem + self.names["up"], stem + self.names["down"]

    def tensor_decls(self):
        outputs = self.experts + self.identity
        decls = [TensorDecl(self.prefix + self.names["router"], (outputs, self.hidden_size), "bias")]
        if self.has_correction:
            decls.append(TensorDecl(self.prefix + self.names["correction"], (outputs,), "bias"))
        for index in [*range(self.experts), *([None] if self.shared_ff else [])]:
            ff = self.shared_ff if index is None else self.expert_ff
            gate, up, down = self._expert_names(index)
            if not self.plain:
                decls.append(TensorDecl(gate, (ff, self.hidden_size)))
            decls += [TensorDecl(up, (ff, self.hidden_size)), TensorDecl(down, (self.hidden_size, ff))]
        if self.shared_gate:
            decls.append(TensorDecl(self.prefix + self.names["shared_gate"], (1, self.hidden_size), "bias"))
        return decls

    def load(self, source: WeightSource):
        self.runtime = source.runtime
        device = source.runtime.device
        self.router = source.vector(self.prefix + self.names["router"])            # float32: the router's product is 32-bit
        if self.shared_gate:
            # the shared expert's gate is one more row of the router's matrix: the same 32-bit product gives it
            gate_row = source.vector(self.prefix + self.names["shared_gate"]).reshape(1, self.hidden_size)
            self.router = torch.cat([self.router, gate_row], dim=0).contiguous()
        self.correction = source.vector(self.prefix + self.names["correction"]) if self.has_correction else None
        if self.experts:
            stacks = [[], []]
            for index in range(self.experts):
                gate, up, down = self._expert_names(index)
                stacks[0].append(source.raw(up) if self.plain else torch.cat([source.raw(gate), source.raw(up)], dim=0))
                stacks[1].append(source.raw(down))
            self.w_gate_up = source.to_device_matrix(torch.stack(stacks[0]))        # [experts, 2 ff (plain: ff), hidden]
            self.w_down = source.to_device_matrix(torch.stack(stacks[1]))          # [experts, hidden, ff]
        if self.shared_ff:
            gate, up, down = self._expert_names(None)
            if self.plain:
                self.shared = PlainUnit(source.raw(up), source.raw(down), "gelu_erf", source)
            else:
                self.shared = ClampedGLU(source.raw(gate), source.raw(up), source.raw(down), self.shared_limit, self.alpha, source)
        self.counts = torch.zeros(max(self.experts, 1), dtype=torch.int32, device=device)   # left zeroed by every step
        self.offsets = torch.zeros(self.experts + 1, dtype=torch.int32, device=device)

    def forward(self, h, x, ctx=None):
        tokens, device = h.shape[0], h.device
        entries = tokens * self.top
        ids = torch.empty((tokens, self.top), dtype=torch.int32, device=device)
        weights = torch.empty((tokens, self.top), dtype=torch.float32, device=device)
        gate_logits = torch.empty((tokens, 1), dtype=torch.float32, device=device) if self.shared_gate else None
        kernels.moe_route(h, self.router, self.correction, ids, weights, self.counts, self.experts, self.top, self.scale,
                          groups=self.groups, renormalize=self.renormalize, extra_out=gate_logits)
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
        if self.shared is not None and self.shared_gate and self.plain:
            self.shared.forward(h, x, row_logits=gate_logits)
        elif self.shared is not None and self.shared_gate:
            y = torch.zeros((tokens, self.hidden_size), dtype=torch.float32, device=device)
            self.shared.forward(h, y)
            kernels.gated_rows_add(x, y, gate_logits)
        elif self.shared is not None:
            self.shared.forward(h, x)
        kernels.moe_combine(x, h, ids, weights, place_of, rows, self.top)

"""Arrangements of a layer's parts.  ``pre_norm``: x += mixer(norm_0(x)); x += ffn(norm_1(x))
(src/qwen.ts:164-200); a layer without a feed-forward (``feed_forward.kind == "none"``) is the first half alone."""
from __future__ import annotations

from ..config.specs import LayerSpec
from .base import Part, build_part, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Part):
    def __init__(self, prefix: str, layer: LayerSpec):
        self.has_ffn = layer.feed_forward.kind != "none"
        if len(layer.norms) != (2 if self.has_ffn else 1):
            raise ValueError("a pre_norm block has one norm per sublayer")
        self.norms = [build_part("norm", spec, prefix) for spec in layer.norms]
        self.mixer = build_part("mixer", layer.mixer, prefix)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, prefix) if self.has_ffn else None

    def parts(self):
        return [*self.norms, self.mixer, *([self.feed_forward] if self.has_ffn else [])]

    def tensor_decls(self):
        return [decl for part in self.parts() for decl in part.tensor_decls()]

    def load(self, source):
        for part in self.parts():
            part.load(source)

    def forward(self, x, ctx, cache, state):
        # a mixer or a feed-forward may offer to take the norm before it into its own kernel
        fused = getattr(self.mixer, "forward_with_norm", None)
        if fused is None or not fused(self.norms[0], x, ctx, cache, state):
            self.mixer.forward(self.norms[0].forward(x), x, ctx, cache, state)
        if not self.has_ffn:
            return
        fused = getattr(self.feed_forward, "forward_with_norm", None)
        if fused is None or not fused(self.norms[1], x, ctx):
            self.feed_forward.forward(self.norms[1].forward(x), x, ctx)


def build_block(layer: LayerSpec):
    from .base import _REGISTRY
    from ..config.specs import ConfigError
    try:
        cls = _REGISTRY["block"][layer.block]
    except KeyError:
        raise ConfigError(f"no block arrangement {layer.block!r} is registered") from None
    return cls(prefix=layer.prefix, layer=layer)


@register_part("block", "post_norm")
class PostNormBlock(Part):
    """The norm comes after the sum: x <- norm_0(alpha x + mixer(x)), then x <- norm_1(alpha x + ffn(x));
    the sublayers read x itself.  The sums and the stream are float32; a sublayer reads x in the compute
    dtype.  A layer without a feed-forward (``feed_forward.kind == "none"``) is the first half alone.

    A sublayer gets ``h`` = x in the compute dtype and ``y`` = alpha x (float32) and adds its output to
    y; the norm kernel that follows writes x and, for the second sublayer, the next h and y as well.
    """

    def __init__(self, prefix: str, layer: LayerSpec):
        self.alpha = float(layer.options.get("alpha", 1.0))
        self.has_ffn = layer.feed_forward.kind != "none"
        if len(layer.norms) != (2 if self.has_ffn else 1):
            raise ValueError("a post_norm block has one norm per sublayer")
        self.norms = [build_part("norm", spec, prefix) for spec in layer.norms]
        for norm in self.norms:
            if getattr(norm, "fused_kind", None) != "rmsnorm":
                raise ValueError("a post_norm block takes RMS norms")
        self.mixer = build_part("mixer", layer.mixer, prefix)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, prefix) if self.has_ffn else None

    def parts(self):
        return [*self.norms, self.mixer, *([self.feed_forward] if self.has_ffn else [])]

    def tensor_decls(self):
        return [decl for part in self.parts() for decl in part.tensor_decls()]

    def load(self, source):
        for part in self.parts():
            part.load(source)
        self.dtype = source.runtime.dtype

    def readers(self, x):
        """Buffers for what this block's first sublayer reads: (y, h) with y = alpha x and h = x in the compute dtype
        (None in float32, where the sublayer reads x itself).  Whoever makes x may fill them (``primed``)."""
        import torch
        y = torch.empty_like(x)
        h = torch.empty(x.shape, dtype=self.dtype, device=x.device) if self.dtype != torch.float32 else None
        return y, h

    def forward(self, x, ctx, cache, state, primed=None, finish=None):
        """``primed``: (y, h) already filled for this x.  ``finish(y, gain, eps)``: instead of the block's last norm, the
        caller's continuation, which must leave the layer's result (or what follows from it) in x."""
        import torch
        from .. import kernels
        narrow = self.dtype != torch.float32
        if primed is None:
            y, h = self.readers(x)
            kernels.scale_cast(x, y, h, self.alpha)
        else:
            y, h = primed
        self.mixer.forward(h if narrow else x, y, ctx, cache, state)
        norm = self.norms[0]
        if self.has_ffn:
            kernels.sum_norm(y, norm.gain, x, norm.eps, y2=y, h=h, alpha=self.alpha)
            self.feed_forward.forward(h if narrow else x, y, ctx)
            norm = self.norms[1]
        if finish is not None:
            finish(y, norm.gain, norm.eps)
        else:
            kernels.sum_norm(y, norm.gain, x, norm.eps)


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Part):
    """A norm before and after each sublayer: x += norm_1(mixer(norm_0(x))), then x += norm_3(ffn(norm_2(x))).
    The stream and the sums are float32.  A layer without a feed-forward (``feed_forward.kind == "none"``) has the
    first two norms only.  A sublayer adds its output into a zeroed float32 buffer; one kernel then norms that
    buffer, adds it to the stream and, after the mixer, also makes what the feed-forward reads."""

    def __init__(self, prefix: str, layer: LayerSpec):
        self.has_ffn = layer.feed_forward.kind != "none"
        if len(layer.norms) != (4 if self.has_ffn else 2):
            raise ValueError("a sandwich_norm block has two norms per sublayer")
        self.norms = [build_part("norm", spec, prefix) for spec in layer.norms]
        for norm in self.norms:
            if getattr(norm, "fused_kind", None) != "layernorm":
                raise ValueError("a sandwich_norm block takes layer norms")
        self.mixer = build_part("mixer", layer.mixer, prefix)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, prefix) if self.has_ffn else None

    def parts(self):
        return [*self.norms, self.mixer, *([self.feed_forward] if self.has_ffn else [])]

    def tensor_decls(self):
        return [decl for part in self.parts() for decl in part.tensor_decls()]

    def load(self, source):
        for part in self.parts():
            part.load(source)
        self.dtype = source.runtime.dtype

    def forward(self, x, ctx, cache, state):
        import torch
        from .. import kernels
        before, after = self.norms[0], self.norms[1]
        y = torch.zeros_like(x)
        self.mixer.forward(before.forward(x), y, ctx, cache, state)
        if not self.has_ffn:
            kernels.norm_add(y, after.gain, x, after.eps)
            return
        if self.norms[2].eps == after.eps:
            h = torch.empty(x.shape, dtype=self.dtype, device=x.device)
            kernels.norm_add(y, after.gain, x, after.eps, next_gain=self.norms[2].gain, h=h)
        else:
            kernels.norm_add(y, after.gain, x, after.eps)
            h = self.norms[2].forward(x)
        y.zero_()
        self.feed_forward.forward(h, y, ctx)
        kernels.norm_add(y, self.norms[3].gain, x, self.norms[3].eps)


@register_part("block", "parallel_residual")
class ParallelResidualBlock(Part):
    """One norm whose output both sublayers read: h = norm_0(x), x += mixer(h) + ffn(h).  A layer without a feed-forward
    (``feed_forward.kind == "none"``) adds the mixer alone.  ``options["side"]`` (a ``side_input`` PartSpec) runs after the
    sublayers and adds to the stream what it makes from the step's token ids.  The stream and the sum are float32."""

    def __init__(self, prefix: str, layer: LayerSpec):
        self.has_ffn = layer.feed_forward.kind != "none"
        if len(layer.norms) != 1:
            raise ValueError("a parallel_residual block has one norm")
        self.norms = [build_part("norm", layer.norms[0], prefix)]
        self.mixer = build_part("mixer", layer.mixer, prefix)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, prefix) if self.has_ffn else None
        side = layer.options.get("side")
        self.side = build_part("side_input", side, prefix) if side is not None else None

    def parts(self):
        return [*self.norms, self.mixer, *([self.feed_forward] if self.has_ffn else []), *([self.side] if self.side else [])]

    def tensor_decls(self):
        return [decl for part in self.parts() for decl in part.tensor_decls()]

    def load(self, source):
        for part in self.parts():
            part.load(source)

    def forward(self, x, ctx, cache, state):
        h = self.norms[0].forward(x)
        self.mixer.forward(h, x, ctx, cache, state)
        if self.has_ffn:
            self.feed_forward.forward(h, x, ctx)
        if self.side is not None:
            self.side.forward(x, ctx)

"""Learned RMSNorm: out = fround(x / sqrt(mean(x^2) + eps)) * gain (src/qwen.ts:72-77).

``offset`` is added to the stored weight to give the gain: 0 for a weight stored around one, 1 for a
weight stored around zero (gain = 1 + w).  ``suffix`` is what follows the part's name in the
checkpoint's tensor name."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorDecl, WeightSource, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    fused_kind = "rmsnorm"       # a consumer that has this norm's arithmetic in its own kernel may take gain and eps

    def __init__(self, prefix: str, size: int, eps: float, name: str = "norm", offset: float = 0.0, suffix: str = ".weight"):
        if eps <= 0:
            raise ValueError("rmsnorm: eps must be positive")
        self.size, self.eps, self.offset = int(size), float(eps), float(offset)
        self.tensor_name = f"{prefix}{name}{suffix}"
        self.gain = None
        self.out_dtype = None

    def tensor_decls(self):
        return [TensorDecl(self.tensor_name, (self.size,), "gain" if self.offset == 0.0 else "bias")]

    def load(self, source: WeightSource):
        self.gain = source.vector(self.tensor_name)
        if self.offset:
            self.gain = (self.gain + self.offset).contiguous()
        self.out_dtype = source.runtime.dtype

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        count = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((count, self.size), dtype=self.out_dtype, device=x.device)
        kernels.rmsnorm(x, self.gain, out, self.eps, rows)
        return out


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """out = (x - mean) / sqrt(var + eps) * w (+ b), var the mean of the squared deviations.  ``bias_suffix`` names the
    bias tensor (the weight's name plus the suffix); None: a weight and no bias.  float32 arithmetic; the output has the
    compute dtype."""
    fused_kind = "layernorm"     # a block that sums and norms in one kernel may take gain and eps

    def __init__(self, prefix: str, size: int, eps: float, name: str = "norm", suffix: str = "", bias_suffix: str | None = None):
        if eps <= 0:
            raise ValueError("layernorm: eps must be positive")
        self.size, self.eps = int(size), float(eps)
        self.tensor_name = f"{prefix}{name}{suffix}"
        self.bias_name = None if bias_suffix is None else self.tensor_name + bias_suffix
        self.gain = self.bias = None
        self.out_dtype = None

    def tensor_decls(self):
        decls = [TensorDecl(self.tensor_name, (self.size,), "gain")]
        if self.bias_name is not None:
            decls.append(TensorDecl(self.bias_name, (self.size,), "bias"))
        return decls

    def load(self, source: WeightSource):
        self.gain = source.vector(self.tensor_name)
        if self.bias_name is not None:
            self.bias = source.vector(self.bias_name)
        self.out_dtype = source.runtime.dtype

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        count = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((count, self.size), dtype=self.out_dtype, device=x.device)
        kernels.layernorm(x, self.gain, out, self.eps, rows, bias=self.bias)
        return out

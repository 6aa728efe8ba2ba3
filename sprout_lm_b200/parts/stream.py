"""What travels from one layer call to the next when that is not simply the layer's result.

``depth_weighted_average``: every layer call's result X_(n+1) is kept (X_0 is the embedding's
output), and what the next call (or the final norm) reads is sum_{j <= n+1} w_n[j] X_j with a learned
weight vector per call.  The history lives for one step: float32 [calls + 1, tokens, hidden].

``loop_restart``: a span of the run order runs several times with the same weights.  Before every pass of the span, right
before its first layer call, a learned vector of that pass (``steps`` [passes, hidden]) is added to the stream, and before
every pass but the first also the embedding's output as it was before the first layer.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorDecl, WeightSource, register_part


@register_part("stream", "depth_weighted_average")
class DepthWeightedAverage(Part):
    def __init__(self, prefix: str, names: tuple):
        """``names[n]`` is the tensor of call n's weights; it has n + 2 entries."""
        self.names = tuple(prefix + name for name in names)
        self.weights: list = []

    def tensor_decls(self):
        # a fresh model passes the latest result on (the last entry is 1 + noise, the others noise)
        return [TensorDecl(name, (n + 2,), "pass_last") for n, name in enumerate(self.names)]

    def load(self, source: WeightSource):
        self.weights = [source.vector(name) for name in self.names]

    def begin(self, x: torch.Tensor, calls: int):
        if calls != len(self.names):
            raise ValueError(f"depth_weighted_average: {len(self.names)} weight vectors for {calls} layer calls")
        history = torch.empty((calls + 1, *x.shape), dtype=torch.float32, device=x.device)
        history[0].copy_(x)
        return history

    def after(self, history, n: int, x: torch.Tensor) -> None:
        kernels.depth_average(history, x, self.weights[n], n)

    def norm_after(self, history, n: int, y, gain, eps: float, x, y2=None, h=None, alpha: float = 1.0) -> None:
        """``after`` for a layer that ends in an RMS norm of ``y``: the norm, the average into ``x`` and, when given, the
        next layer's readers ``y2 = alpha x`` and ``h`` (x in h's dtype) in one launch."""
        kernels.sum_norm(y, gain, x, eps, y2=y2, h=h, alpha=alpha, history=history, weights=self.weights[n], n=n)


@register_part("stream", "loop_restart")
class LoopRestart(Part):
    def __init__(self, prefix: str, hidden_size: int, starts: tuple, name: str = "loop.step"):
        """``starts[t]`` is the index in the run order of the first layer call of pass t."""
        self.hidden_size, self.starts, self.tensor_name = int(hidden_size), tuple(int(n) for n in starts), prefix + name
        if not self.starts or list(self.starts) != sorted(set(self.starts)) or self.starts[0] < 0:
            raise ValueError("loop_restart: the passes' first calls must be distinct and in order")
        self.steps = None

    def tensor_decls(self):
        return [TensorDecl(self.tensor_name, (len(self.starts), self.hidden_size), "bias")]

    def load(self, source: WeightSource):
        self.steps = source.vector(self.tensor_name)

    def _enter(self, first, x, call: int) -> None:
        if call in self.starts:
            t = self.starts.index(call)
            kernels.add_rows(x, self.steps[t], other=first if t > 0 else None)

    def begin(self, x: torch.Tensor, calls: int):
        if self.starts[-1] >= calls:
            raise ValueError("loop_restart: a pass starts beyond the run order")
        first = x.clone() if len(self.starts) > 1 else None          # the embedding's output, for the later passes
        self._enter(first, x, 0)
        return first

    def after(self, first, n: int, x: torch.Tensor) -> None:
        self._enter(first, x, n + 1)

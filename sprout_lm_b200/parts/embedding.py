"""Token embedding (a row copy, src/qwen.ts:162-163; ``scale`` multiplies the rows when a model asks for it) and the output head
(logits = W h, no bias; W is the embedding matrix itself when tied: src/qwen.ts:152,203).
With ``softcap`` the head's logits become softcap * tanh(logits / softcap)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorDecl, WeightSource, register_part
from .linear import Linear


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, name: str = "embed_tokens", suffix: str = ".weight",
                 scale: float = 1.0):
        self.vocab_size, self.hidden_size, self.scale = vocab_size, hidden_size, float(scale)
        self.tensor_name = f"{prefix}{name}{suffix}"
        self.table = None
        self.runtime = None

    def tensor_decls(self):
        return [TensorDecl(self.tensor_name, (self.vocab_size, self.hidden_size))]

    def load(self, source: WeightSource):
        self.table = source.matrix(self.tensor_name)
        self.runtime = source.runtime

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        x = torch.empty((token_ids.numel(), self.hidden_size), dtype=torch.float32, device=token_ids.device)
        kernels.embed(self.table, token_ids, x, self.runtime.status, scale=self.scale)
        return x


@register_part("head", "lm_head")
class LMHead(Part):
    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, tied_to: str | None = None,
                 name: str = "lm_head", suffix: str = ".weight", softcap: float | None = None,
                 any_inner_size: bool = False):
        if softcap is not None and not softcap > 0:
            raise ValueError("lm_head: softcap must be positive")
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.softcap = None if softcap is None else float(softcap)
        self.any_inner_size = any_inner_size
        self.tensor_name = f"{prefix}{tied_to or name}{suffix}"
        self.tied = tied_to is not None
        self.linear = None

    def tensor_decls(self):
        return [] if self.tied else [TensorDecl(self.tensor_name, (self.vocab_size, self.hidden_size))]

    def load(self, source: WeightSource):
        self.linear = Linear(source.matrix(self.tensor_name), None, source.runtime.status, any_inner_size=self.any_inner_size)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.linear.forward(h, out_dtype=torch.float32)
        if self.softcap is not None:
            kernels.softcap(logits, self.softcap)
        return logits

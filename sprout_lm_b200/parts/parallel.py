"""Several mixers side by side: all read the same normed input h, and the layer's mixer output is the weighted sum
``sum_i scales[i] * mixer_i(h)``.

Each sub-mixer is a registered mixer of its own, built from its ``PartSpec`` with the prefix ``prefix + names[i]`` and with
its weight as the constructor parameter ``out_scale`` (every mixer that can stand here folds that factor into its own last
step before the output projection, so the sum costs no kernel).  At most one sub-mixer may keep keys and values per token
(the layer has one cache slot) and at most one a per-request state (the layer has one state entry); they get the layer's
cache and state views, the others get None.
"""
from __future__ import annotations

from ..config.specs import PartSpec
from .base import Part, build_part, register_part


@register_part("mixer", "parallel_mixers")
class ParallelMixers(Part):
    def __init__(self, prefix: str, mixers, scales, names):
        mixers, scales, names = tuple(mixers), tuple(float(s) for s in scales), tuple(names)
        if not mixers or len(mixers) != len(scales) or len(mixers) != len(names):
            raise ValueError("parallel_mixers: one scale and one name per mixer, at least one mixer")
        self.scales = scales
        self.mixers = [build_part("mixer", PartSpec(spec.kind, {**spec.params, "out_scale": scale * spec.params.get("out_scale", 1.0)}),
                                  prefix + name)
                       for spec, scale, name in zip(mixers, scales, names)]
        self.cached = [i for i, m in enumerate(self.mixers) if m.cache_spec() is not None]
        self.stateful = [i for i, m in enumerate(self.mixers) if m.state_spec() is not None]
        if len(self.cached) > 1 or len(self.stateful) > 1:
            raise ValueError("parallel_mixers: at most one mixer with keys and values per token and one with a state")

    def cache_spec(self):
        return self.mixers[self.cached[0]].cache_spec() if self.cached else None

    def state_spec(self):
        return self.mixers[self.stateful[0]].state_spec() if self.stateful else None

    def decode_plan(self, requests: int, max_keys: int, planned_context: int, page_tokens: int):
        return tuple(m.decode_plan(requests, max_keys, planned_context, page_tokens) for m in self.mixers)

    def tensor_decls(self):
        return [decl for m in self.mixers for decl in m.tensor_decls()]

    def load(self, source):
        for m in self.mixers:
            m.load(source)

    def forward(self, h, x, ctx, cache, state):
        for i, m in enumerate(self.mixers):
            m.forward(h, x, ctx, cache if i in self.cached else None, state if i in self.stateful else None)

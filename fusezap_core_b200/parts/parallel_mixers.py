"""Several mixers side by side: all read the same input, the result is the weighted sum of theirs.

`mixers`: (tensor-name prefix, PartSpec of a registered mixer, weight) each. At most one of them may use the paged
cache (a schedule entry has one cache slot); per-request state of any of them is kept under its prefix. The sum
`sum_i weight_i * mixer_i(h)` is 32-bit, added in the order given.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import MIXERS, LayerCache, Mixer, build, register_mixer


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, hidden_size: int, mixers):
        self.D = hidden_size
        self.parts = [(prefix, build(MIXERS, "mixer", spec), float(weight)) for prefix, spec, weight in mixers]
        if not self.parts:
            raise ValueError("parallel mixers need at least one mixer")
        if sum(m.cache_need() is not None for _, m, _ in self.parts) > 1:
            raise ValueError("at most one of several parallel mixers may use the paged cache")
        self.graph_safe = all(getattr(m, "graph_safe", True) for _, m, _ in self.parts)

    def children(self):
        return tuple((prefix, m) for prefix, m, _ in self.parts)

    def tensors(self) -> dict[str, ParamSpec]:
        return {f"{prefix}.{k}": v for prefix, m, _ in self.parts for k, v in m.tensors().items()}

    def bind(self, tensors, ops) -> None:
        for prefix, m, _ in self.parts:
            m.bind({k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}, ops)

    def cache_need(self):
        return next((m.cache_need() for _, m, _ in self.parts if m.cache_need() is not None), None)

    def state_need(self) -> dict:
        return {f"{prefix}.{k}": v for prefix, m, _ in self.parts for k, v in m.state_need().items()}

    def position_name(self) -> str | None:
        return next((m.position_name() for _, m, _ in self.parts if m.position_name() is not None), None)

    def step_needs(self) -> tuple[str, ...]:
        return tuple(k for _, m, _ in self.parts for k in m.step_needs())

    def weight_tensors(self) -> list:
        return []          # the children are parts of their own

    def forward(self, ctx, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        terms, weights = [], []
        for prefix, m, weight in self.parts:
            own = LayerCache(cache.keys, cache.values, cache.group, cache.page_size, cache.write,
                             {k[len(prefix) + 1:]: v for k, v in cache.state.items() if k.startswith(prefix + ".")})
            terms.append(m.forward(ctx, h, own))
            weights.append(weight)
        out = ctx.ws.get("mixers_sum", (h.shape[0], self.D), torch.float32)
        ctx.ops.weighted_sum(terms, weights, out)
        return out

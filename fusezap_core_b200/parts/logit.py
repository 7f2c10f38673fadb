"""Logit transforms: what a model does to the float32 logits of the wanted rows after the output product."""
from __future__ import annotations

from .base import LogitTransform, register_logit_transform


@register_logit_transform("scale")
class ScaleLogits(LogitTransform):
    """logits *= factor, in 32-bit."""
    def __init__(self, factor: float):
        self.factor = float(factor)

    def forward(self, ctx, logits) -> None:
        ctx.ops.scale_(logits, self.factor)

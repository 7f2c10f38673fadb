"""Logit transforms: what a model does to the float32 logits of the wanted rows after the output product."""
from __future__ import annotations

from .base import LogitTransform, register_logit_transform


@register_logit_transform("scale")
class ScaleLogits(LogitTransform):
    """logits *= factor, in 32-bit. A positive factor keeps the order of a row's logits (`keeps_order`), so a step that
    only wants the largest logit's index may skip the transform."""
    def __init__(self, factor: float):
        self.factor = float(factor)
        self.keeps_order = self.factor > 0

    def forward(self, ctx, logits) -> None:
        ctx.ops.scale_(logits, self.factor)

"""Mixture of small gated feed-forwards whose experts are chosen by a table, not by a router.

`table[token id]` (integers, `top` distinct experts per row) names the experts of a token; each has weight 1 / top.
Expert e: `g = min(W_gate,e h, limit)`, `u = clamp(W_up,e h, -limit, limit)`, `y = g * sigmoid(alpha * g) * (u + 1)`,
output `W_down,e y`; no biases. The step sorts its (row, choice) pairs by expert on the device and runs each expert's
products over its own rows only (`Ops.route_by_table`, `Ops.grouped_linear*`); a row's result does not depend on which
other rows share its expert. The products accumulate in 32-bit; the activation is computed from the unrounded sums.
The sum over a row's experts is left to the block (returned as `(terms, top, 1 / top)`), which adds it in 32-bit
together with its own terms.
"""
from __future__ import annotations
import math

import torch

from ..weights import ParamSpec
from .base import FeedForward, register_feed_forward

_NAMES = {"table": "table", "expert": "experts.{}", "gate": "gate_proj", "up": "up_proj", "down": "down_proj"}


@register_feed_forward("table_moe")
class TableMoE(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, vocab_size: int,
                 limit: float, alpha: float = 1.702, names: dict | None = None):
        if not 0 < top <= num_experts:
            raise ValueError(f"top {top} must lie in 1..{num_experts}")
        self.D, self.I, self.E, self.top, self.V = hidden_size, intermediate_size, num_experts, top, vocab_size
        self.limit, self.alpha = float(limit), float(alpha)
        self.names = {**_NAMES, **(names or {})}
        self.table = self.w_gate_up = self.w_down = None

    def _expert(self, e: int, which: str) -> str:
        return f"{self.names['expert'].format(e)}.{self.names[which]}"

    def tensors(self) -> dict[str, ParamSpec]:
        out = {}
        for e in range(self.E):
            out[self._expert(e, "gate")] = ParamSpec((self.I, self.D))
            out[self._expert(e, "up")] = ParamSpec((self.I, self.D))
            out[self._expert(e, "down")] = ParamSpec((self.D, self.I))
        out[self.names["table"]] = ParamSpec((self.V, self.top), role="int_table", high=self.E)
        return out

    def bind(self, tensors, ops) -> None:
        E = self.E
        # (E, 2 I, D): an expert's gate rows, then its up rows; (E, D, I)
        self.w_gate_up = torch.stack([torch.cat([tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")]], 0)
                                      for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")] for e in range(E)]).contiguous()
        self.table = tensors[self.names["table"]].contiguous()

    def step_needs(self) -> tuple[str, ...]:
        return ("token_ids",)

    def forward(self, ctx, h: torch.Tensor):
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        route = ops.route_by_table(ctx.token_ids, ctx.meta, self.table, self.E, math.gcd(self.D, self.I))
        y = ws.get("moe_act", (n * self.top, self.I), ops.dtype)             # rows in the sorted order of the pairs
        ops.grouped_linear_glu(h, self.w_gate_up, route, y, self.alpha, self.limit)
        terms = ws.get("moe_terms", (n * self.top, self.D), torch.float32)   # row n * top + k: the k-th expert of row n
        ops.grouped_linear_scatter(y, self.w_down, route, terms)
        return terms, self.top, 1.0 / self.top

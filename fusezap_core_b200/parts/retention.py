"""Retention: linear attention with a fixed decay per head and no softmax or denominator.

Per head h with state S (key_dim x value_dim, float32, zero at a request's start, one per request and layer):

    S_t = decay_h * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t

q and k are rotated by the token's position on their first `rotated` dimensions (`pairing`: "halves" pairs dimension i
with i + rotated/2, "neighbours" pairs 2i with 2i+1), k is multiplied by `key_scale` after the rotation. Each head's o
is divided by its root mean square (`eps` inside the root, no weight), the heads are concatenated and multiplied by
`gate`(W_g h) ("silu", "sigmoid" or None for no gate), then the output product. The rotation, the recurrence, the
state and the norm are 32-bit in both dtypes; the projections accumulate in 32-bit and leave q, k, v unrounded.

A step may bring any portion of a sequence: the kernel walks a portion's tokens in order from the state its request's
slot holds and leaves the state there afterwards (`Ops.retention_scan`).
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import LayerCache, Mixer, register_mixer

_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "gate": "g_proj", "out": "o_proj"}
PAIRINGS = {"halves": 0, "neighbours": 1}


@register_mixer("retention")
class Retention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay, key_scale: float = 1.0,
                 rotated: int = 0, pairing: str = "halves", position: str | None = None, eps: float = 1e-6,
                 gate: str | None = "silu", names: dict | None = None):
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        if pairing not in PAIRINGS:
            raise ValueError(f"pairing {pairing!r} is not one of {sorted(PAIRINGS)}")
        if rotated % 2 or not 0 <= rotated <= key_dim:
            raise ValueError(f"{rotated} rotated dimensions must be even and at most key_dim {key_dim}")
        self.D, self.H, self.dk, self.dv = hidden_size, num_heads, key_dim, value_dim
        self.decay_values, self.key_scale, self.rotated, self.pairing = tuple(float(x) for x in decay), float(key_scale), int(rotated), pairing
        self.position, self.eps, self.gate = (position if rotated else None), float(eps), gate
        self.names = {**_NAMES, **(names or {})}
        self.w_in = self.wo = self.decay = None

    def tensors(self) -> dict[str, ParamSpec]:
        n, H = self.names, self.H
        out = {n["q"]: ParamSpec((H * self.dk, self.D)), n["k"]: ParamSpec((H * self.dk, self.D)),
               n["v"]: ParamSpec((H * self.dv, self.D)), n["out"]: ParamSpec((self.D, H * self.dv))}
        if self.gate:
            out[n["gate"]] = ParamSpec((H * self.dv, self.D))
        return out

    def bind(self, tensors, ops) -> None:
        n = self.names
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]] + ([tensors[n["gate"]]] if self.gate else [])
        self.w_in = torch.cat(rows, 0).contiguous()                # one product: [q | k | v | gate]
        self.wo = tensors[n["out"]]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.wo.device)
        self.state_shape = ops.recurrent_state_shape(self.H, self.dk, self.dv)

    def state_need(self) -> dict:
        return {"S": self.state_shape}

    def position_name(self) -> str | None:
        return self.position

    def forward(self, ctx, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        H, dk, dv = self.H, self.dk, self.dv
        width = H * (2 * dk + dv) + (H * dv if self.gate else 0)
        proj = ws.get("retention_in", (n, width), torch.float32)
        ops.linear(h, self.w_in, None, proj)
        pos = ctx.positions[self.position] if self.position is not None else None
        o = ws.get("retention_o", (n, H * dv), torch.float32)
        ops.retention_scan(proj, H, dk, dv, self.decay, self.key_scale, pos.cos if pos else None, pos.sin if pos else None,
                           self.rotated, PAIRINGS[self.pairing], cache.state["S"], ctx.meta, o)
        y = ws.get("attn_out", (n, H * dv), ops.dtype)
        ops.head_norm_gate(o, H, dv, None, self.eps, proj if self.gate else None, H * (2 * dk + dv), self.gate, y)
        delta = ws.get("delta", (n, self.D), torch.float32)
        ops.linear(y, self.wo, None, delta)
        return delta

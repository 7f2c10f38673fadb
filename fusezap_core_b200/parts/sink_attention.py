"""Grouped-query attention over a sliding window that keeps the first tokens, with a sink in the softmax.

Row i (position p_i of its request) sees key j if `j <= i and (i - j < window or j < keep_first)` (window 0: every
earlier key). Kept tokens keep their true positions. Query head h reads kv head `h // (heads / kv_heads)`; keys have
`key_dim` and values `value_dim` dimensions. The score is `(q . k) * scale`; with `sink` the softmax's denominator
also holds `exp(sink_h)`, a learned number per head that has no key and no value and is not scaled:

    o = sum_j exp(s_j - m) v_j / (sum_j exp(s_j - m) + exp(sink_h - m)),      m = max(max_j s_j, sink_h)

q and k are rotated by position on their first `rotated` dimensions (`pairing` "neighbours": 2i with 2i+1; "halves":
i with i + rotated/2), v is not. One product with the rows [q; k; v] leaves float32; the rotation, scores, softmax and
the value sum are 32-bit in both dtypes; keys and values are rounded once into the paged cache. The cache group of this
mixer gives back pages that lie wholly between the kept first tokens and the window.
"""
from __future__ import annotations
import torch

from ..cache import KVNeed
from ..weights import ParamSpec
from .base import LayerCache, Mixer, register_mixer
from .retention import PAIRINGS

_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "sink": "sinks", "out": "o_proj"}


@register_mixer("sink_attention")
class SinkAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 window: int = 0, keep_first: int = 0, sink: bool = True, rotated: int = 0, pairing: str = "neighbours",
                 position: str | None = None, names: dict | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        if pairing not in PAIRINGS:
            raise ValueError(f"pairing {pairing!r} is not one of {sorted(PAIRINGS)}")
        if rotated % 2 or not 0 <= rotated <= key_dim:
            raise ValueError(f"{rotated} rotated dimensions must be even and at most key_dim {key_dim}")
        self.D, self.Hq, self.Hkv, self.dk, self.dv = hidden_size, num_heads, num_kv_heads, key_dim, value_dim
        self.scale, self.window, self.keep_first, self.has_sink = float(scale), int(window), int(keep_first), bool(sink)
        self.rotated, self.pairing, self.position = int(rotated), pairing, (position if rotated else None)
        self.names = {**_NAMES, **(names or {})}
        self.wqkv = self.wo = self.sink = None

    def tensors(self) -> dict[str, ParamSpec]:
        n = self.names
        out = {n["q"]: ParamSpec((self.Hq * self.dk, self.D)), n["k"]: ParamSpec((self.Hkv * self.dk, self.D)),
               n["v"]: ParamSpec((self.Hkv * self.dv, self.D)), n["out"]: ParamSpec((self.D, self.Hq * self.dv))}
        if self.has_sink:
            out[n["sink"]] = ParamSpec((self.Hq,), role="vector")
        return out

    def bind(self, tensors, ops) -> None:
        n = self.names
        self.wqkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], 0).contiguous()
        self.wo = tensors[n["out"]]
        self.sink = tensors[n["sink"]].float().contiguous() if self.has_sink else None
        ops.check_sink_attention(self.Hq, self.Hkv, self.dk, self.dv)

    def cache_need(self) -> KVNeed:
        return KVNeed(self.Hkv, self.dk, self.window, value_dim=self.dv, keep_first=self.keep_first if self.window else 0)

    def position_name(self) -> str | None:
        return self.position

    def step_needs(self) -> tuple[str, ...]:
        return ("portions",)      # its kernels tile the rows of portions: the longest portion is part of a step's shape

    def forward(self, ctx, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        Hq, Hkv, dk, dv = self.Hq, self.Hkv, self.dk, self.dv
        qkv = ws.get("sink_qkv", (n, (Hq + Hkv) * dk + Hkv * dv), torch.float32)
        ops.linear(h, self.wqkv, None, qkv)
        q = ws.get("sink_q", (n, Hq * dk), ops.dtype)
        pos = ctx.positions[self.position] if self.position is not None else None
        ops.rotate_kv_write(qkv, pos.cos if pos else None, pos.sin if pos else None, self.rotated, PAIRINGS[self.pairing],
                            ctx.meta, cache, q, Hq, Hkv, dk, dv)
        o = ws.get("sink_out", (n, Hq * dv), ops.dtype)
        ops.sink_attention(q, cache, ctx.meta, o, Hq, Hkv, dk, dv, self.scale, self.window, self.keep_first, self.sink)
        delta = ws.get("sink_delta", (n, self.D), torch.float32)
        ops.linear(o, self.wo, None, delta)
        return delta

"""Gated delta rule: a recurrent mixer whose state is corrected towards each token's value and decays per key channel.

`q = W_q h`, `k = W_k h` (num_key_heads x key_dim), `v = W_v h` (num_heads x value_dim); each passes a short causal
convolution over time per channel (`taps` wide, the last column is the token's own, no bias, zeros before the start)
and then silu. q and k become unit vectors per head, `x / sqrt(sum(x^2) + unit_eps)`, q is also multiplied by
`query_scale`. Value head h uses q/k head `h // (num_heads / num_key_heads)`. Per head, with S (key_dim x value_dim):

    beta = sigmoid(W_b h)                                            one per head
    g    = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) + dt_bias))    one per head and key channel (rows of S)
    S <- g * S;   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q        (the read-out sees the token's write)

Each head's o is divided by its root mean square over value_dim (`eps` inside the root), times the weight `norm`
(value_dim, shared by the heads), times `sigmoid(W_g2 (W_g1 h))`, then the output product. S (float32, zero at a
request's start) and the convolution's last `taps - 1` inputs are request state. Unit norms, beta, the decay with its
softplus and exponentials, the recurrence and the output norm are 32-bit in both dtypes; the projections and the
convolution with its silu run in the activation dtype with 32-bit sums.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import LayerCache, Mixer, register_mixer
from .short_conv import ShortConv

_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "conv": "conv", "beta": "b_proj", "decay_log": "A_log",
          "decay_in": "a_down", "decay_out": "a_up", "decay_bias": "dt_bias", "gate_in": "g_down", "gate_out": "g_up",
          "norm": "norm", "out": "o_proj"}


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_key_heads: int, key_dim: int, value_dim: int, taps: int,
                 unit_eps: float = 1e-6, query_scale: float = 1.0, eps: float = 1e-6, names: dict | None = None,
                 low_rank: int = 0):
        """low_rank: the inner size of the two-step decay and gate projections for writers of random weights (0: an
        eighth of the hidden size, at least 8); a checkpoint's own sizes are read from its tensors."""
        if num_heads % num_key_heads:
            raise ValueError(f"{num_heads} value heads are not a multiple of {num_key_heads} key heads")
        self.D, self.H, self.Hk, self.dk, self.dv = hidden_size, num_heads, num_key_heads, key_dim, value_dim
        self.unit_eps, self.query_scale, self.eps = float(unit_eps), float(query_scale), float(eps)
        self.names = {**_NAMES, **(names or {})}
        self.C = 2 * self.Hk * key_dim + num_heads * value_dim            # channels of [q | k | v]
        self.conv = ShortConv(self.C, taps, name="", residual=False, activation="silu")
        self.ra = self.rg = 0
        self.low_rank = int(low_rank) or max(8, hidden_size // 8)
        self.w_qkv = self.w_low = self.w_high = self.w_beta = self.wo = None
        self.a_log = self.dt_bias = self.norm_w = None

    def tensors(self) -> dict[str, ParamSpec]:
        n, H, Hk, dk, dv, D = self.names, self.H, self.Hk, self.dk, self.dv, self.D
        taps = self.conv.taps
        r = self.low_rank      # the inner sizes of the two-step projections are whatever the checkpoint has
        return {n["q"]: ParamSpec((Hk * dk, D)), n["k"]: ParamSpec((Hk * dk, D)), n["v"]: ParamSpec((H * dv, D)),
                f"{n['q']}.{n['conv']}": ParamSpec((Hk * dk, taps)), f"{n['k']}.{n['conv']}": ParamSpec((Hk * dk, taps)),
                f"{n['v']}.{n['conv']}": ParamSpec((H * dv, taps)),
                n["beta"]: ParamSpec((H, D)), n["decay_log"]: ParamSpec((H,), role="vector"),
                n["decay_in"]: ParamSpec((-1, D), open=r), n["decay_out"]: ParamSpec((H * dk, -1), open=r),
                n["decay_bias"]: ParamSpec((H * dk,), role="vector"),
                n["gate_in"]: ParamSpec((-1, D), open=r), n["gate_out"]: ParamSpec((H * dv, -1), open=r),
                n["norm"]: ParamSpec((dv,), role="vector", init="ones"), n["out"]: ParamSpec((D, H * dv))}

    def bind(self, tensors, ops) -> None:
        n, H, dk, dv = self.names, self.H, self.dk, self.dv
        self.w_qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], 0).contiguous()
        self.conv.bind({"": torch.cat([tensors[f"{n[x]}.{n['conv']}"] for x in ("q", "k", "v")], 0).contiguous()}, ops)
        a1, a2, g1, g2 = (tensors[n[x]] for x in ("decay_in", "decay_out", "gate_in", "gate_out"))
        self.ra, self.rg = a1.shape[0], g1.shape[0]
        if a2.shape[1] != self.ra or g2.shape[1] != self.rg:
            raise ValueError(f"the two steps of the decay or gate projection do not fit: {tuple(a1.shape)} -> {tuple(a2.shape)}, "
                             f"{tuple(g1.shape)} -> {tuple(g2.shape)}")
        # both first steps as one product [a1; g1], both second steps as one product with the matrix [a2 0; 0 g2]
        # (the zero blocks add exact zeros), whose float32 result is [decay input | gate input]
        self.w_low = torch.cat([a1, g1], 0).contiguous()
        high = torch.zeros((H * dk + H * dv, self.ra + self.rg), dtype=a2.dtype, device=a2.device)
        high[:H * dk, :self.ra] = a2
        high[H * dk:, self.ra:] = g2
        self.w_high = high
        self.w_beta = tensors[n["beta"]]
        self.a_log = tensors[n["decay_log"]].float().contiguous()
        self.dt_bias = tensors[n["decay_bias"]].float().contiguous()
        self.norm_w = tensors[n["norm"]].float().contiguous()
        self.wo = tensors[n["out"]]
        self.state_shape = ops.recurrent_state_shape(H, dk, dv)

    def children(self):
        return (("conv", self.conv),)

    def state_need(self) -> dict:
        return {"S": self.state_shape, **self.conv.state_need()}

    def forward(self, ctx, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        H, Hk, dk, dv = self.H, self.Hk, self.dk, self.dv
        qkv = ws.get("delta_qkv", (n, self.C), ops.dtype)
        ops.linear(h, self.w_qkv, None, qkv)
        qkv = self.conv.forward(ctx, qkv, cache.state.get("conv"), tag="delta_conv")
        low = ws.get("delta_low", (n, self.ra + self.rg), ops.dtype)
        ops.linear(h, self.w_low, None, low)
        high = ws.get("delta_high", (n, H * dk + H * dv), torch.float32)        # [decay input | gate input]
        ops.linear(low, self.w_high, None, high)
        beta = ws.get("delta_beta", (n, H), torch.float32)
        ops.linear(h, self.w_beta, None, beta)
        o = ws.get("delta_o", (n, H * dv), torch.float32)
        ops.gated_delta_scan(qkv, H, Hk, dk, dv, high, beta, self.a_log, self.dt_bias, self.unit_eps, self.query_scale,
                             cache.state["S"], ctx.meta, o)
        y = ws.get("delta_y", (n, H * dv), ops.dtype)
        ops.head_norm_gate(o, H, dv, self.norm_w, self.eps, high, H * dk, "sigmoid", y)
        delta = ws.get("delta_delta", (n, self.D), torch.float32)
        ops.linear(y, self.wo, None, delta)
        return delta

"""A plain, slow Pepilix on whole sequences: one function per mechanism, written from the design's equations, sharing no
code with the package. Everything is computed in float64 on the CPU from the checkpoint's tensors by name; `rounded`
optionally rounds what the engine keeps in bfloat16 (matrix operands and the cache), to judge bfloat16 runs.

Unlike the engine, the attention here builds every head's keys and values from the latent explicitly.
"""
from __future__ import annotations
import math

import torch

F = torch.float64


def grouped_rms_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """x (..., D) split into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps); times w."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(x.shape) * w


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h (T, C), w (C, taps): out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v (T, ..., R): dimension i < dims/2 is paired with i + dims/2 and turned by the angle p * base^(-2i/dims); the
    dimensions from `dims` on pass unchanged."""
    half = dims // 2
    out = v.clone()
    for i in range(half):
        ang = positions.to(F) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang), torch.sin(ang)
        while c.dim() < v.dim() - 1:
            c, s = c.unsqueeze(-1), s.unsqueeze(-1)
        a, b = v[..., i], v[..., i + half]
        out[..., i] = a * c - b * s
        out[..., i + half] = b * c + a * s
    return out


def latent_entries(hm: torch.Tensor, w_dkv: torch.Tensor, w_norm: torch.Tensor, rank: int, eps: float, base: float,
                   dims: int, rnd) -> tuple[torch.Tensor, torch.Tensor]:
    """What a layer with a down projection caches per token: the normed latent c (T, rank) and the rotated shared key
    part (T, rot_dim)."""
    T = hm.shape[0]
    d = hm @ w_dkv.T
    c = d[:, :rank]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * w_norm
    kr = rotate(d[:, rank:], torch.arange(T), base, dims)
    return rnd(c), rnd(kr)


def latent_attention(hm: torch.Tensor, c: torch.Tensor, kr: torch.Tensor, w_q, w_uk, w_uv, w_o, heads: int, dim: int,
                     rot_dim: int, vdim: int, scale: float, base: float, dims: int, rnd) -> torch.Tensor:
    """Causal softmax attention with per-head keys [W_uk c | k_r] and values W_uv c built explicitly."""
    T = hm.shape[0]
    q = rnd(hm @ w_q.T).view(T, heads, dim + rot_dim)
    q_n, q_r = q[..., :dim], rotate(q[..., dim:], torch.arange(T), base, dims)
    k = (c @ w_uk.T).view(T, heads, dim)
    v = (c @ w_uv.T).view(T, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=F)
    for h in range(heads):
        s = (q_n[:, h] @ k[:, h].T + q_r[:, h] @ kr.T) * scale
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, h]
    return rnd(out.reshape(T, heads * vdim)) @ w_o.T


def expert(h: torch.Tensor, w_gate, w_up, w_down, limit: float, rnd) -> torch.Tensor:
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, -limit, limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1)
    return rnd(y) @ w_down.T


def table_moe(h: torch.Tensor, tokens, W: dict, prefix: str, top: int, limit: float, rnd) -> torch.Tensor:
    out = torch.zeros(h.shape[0], W[prefix + "e0.down"].shape[0], dtype=F)
    table = W[prefix + "table"]
    for t, tok in enumerate(tokens):
        for e in table[tok].tolist():
            p = f"{prefix}e{e}."
            out[t] += expert(h[t], W[p + "gate"], W[p + "up"], W[p + "down"], limit, rnd) / top
    return out


def forward(cfg: dict, weights: dict, tokens, rounded: bool = False, layers_out: list | None = None) -> torch.Tensor:
    """Logits (T, vocab) of one whole sequence. rounded: matrices, matrix inputs and cache entries pass through bfloat16."""
    rnd = (lambda t: t.to(torch.bfloat16).to(F)) if rounded else (lambda t: t)
    W = {k: (v.long() if not v.dtype.is_floating_point else (rnd(v.to(F)) if v.dim() >= 2 else v.to(F))) for k, v in weights.items()}
    eps, groups, taps = cfg["norm"]["eps"], cfg["norm"]["groups"], (cfg.get("canon") or {}).get("taps", 0)
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    cached: dict[int, tuple] = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h1 = rnd(grouped_rms_norm(x, W[p + "norm1"], groups, eps))
        hm = rnd(h1 + causal_conv(h1, W[p + "canon1"])) if taps >= 1 else h1
        base, dims = m["rot"]["base"], m["rot"]["dims"]
        if m.get("kv_from") is None:
            cached[i] = latent_entries(hm, W[p + "mix.dkv"], W[p + "mix.dkv.norm"], m["kv_rank"], eps, base, dims, rnd)
            c, kr = cached[i]
        else:
            c, kr = cached[m["kv_from"]]
        a = latent_attention(hm, c, kr, W[p + "mix.q"], W[p + "mix.uk"], W[p + "mix.uv"], W[p + "mix.o"], m["heads"], m["dim"],
                             m["rot_dim"], m["vdim"], m["scale"], base, dims, rnd)
        delta = a * torch.sigmoid(h1 @ W[p + "rg1"].T + W[p + "rg1.b"])
        if L["mlp"] is not None:
            h2 = rnd(grouped_rms_norm(x, W[p + "norm2"], groups, eps))
            f = table_moe(h2, tokens, W, p + "mlp.", L["mlp"]["router"]["top"], L["mlp"]["expert"]["limit"], rnd)
            delta = delta + f * torch.sigmoid(h2 @ W[p + "rg2"].T + W[p + "rg2.b"])
        x = x + delta
        if layers_out is not None:
            layers_out.append(x.clone())
    h = rnd(grouped_rms_norm(x, W["final.norm"], groups, eps))
    return (h @ W["embed"].T) * cfg["logit_scale"]


def greedy(cfg: dict, weights: dict, prompt, n: int) -> list[int]:
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(forward(cfg, weights, ids)[-1])))
    return ids[len(prompt):]

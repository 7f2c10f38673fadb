"""A plain, slow Gizulorn: one function per mechanism, written from the design's equations in 64-bit, whole sequences,
token by token where the design is a recurrence. It shares no code with the package and is the oracle of its tests.

`forward(config, tensors, tokens)` takes the config.json dict, a dict name -> torch tensor and a list of token ids, and
returns (logits (T, vocab), residual stream after every layer (L, T, width)), both float64.
"""
from __future__ import annotations
import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def frequencies(rot):
    """f_i = base^(-2i/dims), then the wavelength-dependent scaling if the rotation has one."""
    dims = int(rot["dims"])
    f = [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f:
            wl = 2 * math.pi / fi
            if wl < orig / high:
                out.append(fi)
            elif wl > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wl - low) / (high - low)
                out.append((1 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F)


def rotate(x, rot, layout, pos0=0):
    """x: (T, heads, dim). The first rot.dims dimensions of every head are turned by the token's position; `layout`
    'interleaved' pairs (2i, 2i+1), 'half' pairs (i, i + dims/2)."""
    dims = int(rot["dims"])
    T = x.shape[0]
    a = (torch.arange(pos0, pos0 + T, dtype=F)[:, None] * frequencies(rot)[None, :])[:, None, :]      # (T, 1, dims/2)
    c, s = torch.cos(a), torch.sin(a)
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    return out


def sink_window_attention(q, k, v, scale, window, keep_first, sink):
    """q: (T, H, d), k: (T, G, d), v: (T, G, dv), sink: (H,). Row i sees j <= i with i - j < window or j < keep_first;
    the softmax's denominator also holds exp(sink_h)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if i - j < window or j < keep_first]
            s = torch.stack([(q[i, h] * k[j, g]).sum() * scale for j in js])
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + torch.exp(sink[h] - m)
            out[i, h] = sum(e[n] * v[j, g] for n, j in enumerate(js)) / den
    return out


def causal_conv(x, w):
    """x: (T, C), w: (C, taps), the last column multiplies the token's own input; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], 0)
    return sum(pad[j: j + T] * w[:, j][None, :] for j in range(taps))


def gated_delta(q, k, v, beta, g):
    """q, k: (T, Hk, d) (unit vectors, q scaled), v: (T, H, dv), beta: (T, H), g: (T, H, d) decays. Returns (T, H, dv)."""
    T, H, dv = v.shape
    Hk, d = q.shape[1], q.shape[2]
    out = torch.zeros(T, H, dv, dtype=F)
    for h in range(H):
        kh = h // (H // Hk)
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, h] = S.T @ q[t, kh]
    return out


def retention(q, k, v, decay):
    """q, k: (T, H, d), v: (T, H, dv), decay: (H,). S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, dv = v.shape
    out = torch.zeros(T, H, dv, dtype=F)
    for h in range(H):
        S = torch.zeros(q.shape[2], dv, dtype=F)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def gated_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def routed_choice(z, top, groups, keep):
    """z: (E,) router logits of one token. Returns (chosen expert ids, their softmax scores)."""
    s = torch.softmax(z, -1)
    E = s.shape[0]
    per = E // groups
    best = sorted(range(groups), key=lambda gi: (-float(s[gi * per:(gi + 1) * per].max()), gi))[:keep]
    allowed = [e for e in range(E) if e // per in best]
    chosen = sorted(allowed, key=lambda e: (-float(s[e]), e))[:top]
    return chosen, [s[e] for e in chosen]


class Weights:
    def __init__(self, tensors):
        self.t = tensors

    def __call__(self, name):
        return self.t[name].to(F)


def mixer_retention(W, p, m, h, eps):
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W(p + "q").T).view(T, H, d)
    k = (h @ W(p + "k").T).view(T, H, d)
    v = (h @ W(p + "v").T).view(T, H, dv)
    q, k = rotate(q, m["rot"], "half"), rotate(k, m["rot"], "half") * d ** -0.5
    o = retention(q, k, v, torch.tensor([float(x) for x in m["decay"]], dtype=F))
    o = rms(o, eps).reshape(T, H * dv) * silu(h @ W(p + "g").T)
    return o @ W(p + "o").T


def mixer_left(W, p, m, h):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rotate((h @ W(p + "q").T).view(T, H, d), m["rot"], "interleaved")
    k = rotate((h @ W(p + "k").T).view(T, G, d), m["rot"], "interleaved")
    v = (h @ W(p + "v").T).view(T, G, dv)
    o = sink_window_attention(q, k, v, float(m["scale"]), int(m["mask"]["size"]), int(m["mask"]["keep_first"]), W(p + "sink"))
    return o.reshape(T, H * dv) @ W(p + "o").T


def mixer_right(W, p, m, h, eps):
    T = h.shape[0]
    H, Hk, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_conv(h @ W(p + "q").T, W(p + "q.conv"))).view(T, Hk, d)
    k = silu(causal_conv(h @ W(p + "k").T, W(p + "k.conv"))).view(T, Hk, d)
    v = silu(causal_conv(h @ W(p + "v").T, W(p + "v.conv"))).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W(p + "b").T)
    a = (h @ W(p + "a1").T) @ W(p + "a2").T + W(p + "dt_bias")
    g = torch.exp(-torch.exp(W(p + "A_log"))[None, :, None] * softplus(a).view(T, H, d))
    o = gated_delta(q, k, v, beta, g)
    gate = torch.sigmoid((h @ W(p + "g1").T) @ W(p + "g2").T).view(T, H, dv)
    o = rms(o, eps) * W(p + "norm")[None, None, :] * gate
    return o.reshape(T, H * dv) @ W(p + "o").T


def feed_forward(W, p, mlp, h):
    if mlp["kind"] == "dense":
        return gated_ff(h, W(p + "gate"), W(p + "up"), W(p + "down"))
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = h @ W(p + "router").T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, weights = routed_choice(z[t], top, int(groups["count"]), int(groups["keep"]))
        for e, w in zip(chosen, weights):
            out[t] += w * gated_ff(h[t], W(f"{p}e{e}.gate"), W(f"{p}e{e}.up"), W(f"{p}e{e}.down"))
    if mlp.get("shared"):
        sp = p + "shared."
        out = out + torch.sigmoid(h @ W(sp + "sg").T) * gated_ff(h, W(sp + "gate"), W(sp + "up"), W(sp + "down"))
    return out


def forward(config, tensors, tokens):
    W = Weights(tensors)
    eps = float(config["norm"]["eps"])
    x = W("embed")[torch.tensor(list(tokens), dtype=torch.long)]
    after = []
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms(x, eps) * W(p + "norm1")
        m = L["mixer"]
        if L["type"] == "retention":
            x = x + mixer_retention(W, p + "mix.", m, h, eps)
        elif L["type"] == "parallel":
            x = x + float(m["left_scale"]) * mixer_left(W, p + "mix.left.", m["left"], h) \
                  + float(m["right_scale"]) * mixer_right(W, p + "mix.right.", m["right"], h, eps)
        else:
            raise NotImplementedError(L["type"])
        if L.get("mlp") is not None:
            x = x + feed_forward(W, p + "mlp.", L["mlp"], rms(x, eps) * W(p + "norm2"))
        after.append(x.clone())
    logits = (rms(x, eps) * W("final.norm")) @ W("head").T
    return logits, torch.stack(after)

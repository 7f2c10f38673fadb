"""Small Pepilix configurations and drivers shared by the CPU and GPU tests of that design.

The configurations differ from one another in every size and constant, and use values that make different sizes
distinct (query, rotated and value sizes all unequal; a latent size that is no multiple of 32; one expert per token and
several; one norm group and several; two taps and many; a layer without feed-forward; cache sharing between layers that
are not neighbours; no embedding or logit scale)."""
from __future__ import annotations
import copy
import os

import numpy as np
import torch


def _mixer(heads, dim, rot_dim, vdim, rank, scale, base, kv_from=None, dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


PEP_SMALL = {      # three norm groups, three taps, one expert per token, a layer without feed-forward, sharing 0 -> 2
    "architecture": "Pepilix", "vocab": 211, "width": 96, "embedding": {"scale": 3.5}, "logit_scale": 0.25,
    "norm": {"eps": 1e-5, "groups": 3}, "canon": {"taps": 3},
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(3, 16, 8, 24, 40, 0.2, 10000.0), "mlp": _moe(5, 1, 24, 0.75)},
        {"type": "latent_attention", "mixer": _mixer(2, 8, 4, 16, 24, 0.3, 300.0), "mlp": None},
        {"type": "latent_attention", "mixer": _mixer(3, 16, 8, 24, 40, 0.2, 10000.0, kv_from=0), "mlp": _moe(4, 3, 40, 2.0)},
    ]}
PEP_WIDE = {       # one norm group, two taps, no scales, 40 heads (more than one block's slice), partly rotated keys
    "architecture": "Pepilix", "vocab": 97, "width": 64, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
    "norm": {"eps": 1e-6, "groups": 1}, "canon": {"taps": 2},
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(40, 4, 6, 2, 16, 0.5, 50.0, dims=4), "mlp": _moe(3, 2, 16, 1.5)},
        {"type": "latent_attention", "mixer": _mixer(40, 4, 6, 2, 16, 0.5, 50.0, kv_from=0, dims=4), "mlp": _moe(7, 7, 8, 0.5)},
    ]}
PEP_TAPS = {       # five taps (longer than the shortest portions), four norm groups, a single layer
    "architecture": "Pepilix", "vocab": 61, "width": 128, "embedding": {"scale": 0.5}, "logit_scale": 2.0,
    "norm": {"eps": 1e-4, "groups": 4}, "canon": {"taps": 5},
    "layers": [{"type": "latent_attention", "mixer": _mixer(1, 64, 32, 48, 72, 0.1, 1e6), "mlp": _moe(2, 2, 72, 1.0)}]}
CONFIGS = {"small": (PEP_SMALL, 3), "wide": (PEP_WIDE, 5), "taps": (PEP_TAPS, 9)}
STD_SCALE = 4.0


def make_dir(name: str, tmp) -> tuple[str, dict, dict]:
    """Writes configuration `name` with seeded random weights (float32); returns (folder, config, weights by name)."""
    from fusezap_core_b200.weights import write_random_model
    from safetensors.torch import load_file
    cfg, seed = CONFIGS[name]
    cfg = copy.deepcopy(cfg)
    d = os.path.join(str(tmp), f"pepilix-{name}")
    write_random_model(cfg, d, seed, "float32", norm_noise=True, std_scale=STD_SCALE)
    return d, cfg, load_file(os.path.join(d, "model.safetensors"))


def tokens_for(cfg: dict, lengths, seed: int) -> list[list[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], n).tolist() for n in lengths]


def run_cut(runner, cache, req: str, toks, cuts, free: bool = True) -> np.ndarray:
    """One request alone, in portions of the sizes `cuts` (cycled); logits of every position."""
    from fusezap_core_b200.engine import Portion
    out, at, k = [], 0, 0
    while at < len(toks):
        n = min(cuts[k % len(cuts)], len(toks) - at)
        out.append(runner.run([Portion(req, toks[at: at + n], list(range(n)))]).detach().cpu().numpy().copy())
        at, k = at + n, k + 1
    if free:
        cache.free(req)
    return np.concatenate(out)


def run_mixed(runner, cache, reqs: dict, plan) -> dict:
    """plan: a list of steps, each a list of (request, tokens to take). Requests that reach their end are freed after
    the step. Returns every request's logits at all positions."""
    from fusezap_core_b200.engine import Portion
    at = {r: 0 for r in reqs}
    got = {r: [] for r in reqs}
    for step in plan:
        portions = []
        for r, n in step:
            n = min(n, len(reqs[r]) - at[r])
            if n > 0:
                portions.append(Portion(r, reqs[r][at[r]: at[r] + n], list(range(n))))
        if not portions:
            continue
        lg = runner.run(portions).detach().cpu().numpy()
        k = 0
        for p in portions:
            got[p.req].append(lg[k: k + len(p.tokens)].copy())
            k += len(p.tokens)
            at[p.req] += len(p.tokens)
            if at[p.req] == len(reqs[p.req]):
                cache.free(p.req)
    return {r: np.concatenate(v) for r, v in got.items() if v}


def rel_rms(got: np.ndarray, ref: np.ndarray) -> float:
    """The largest per-row root-mean-square difference (row mean removed), relative to the rms of the reference."""
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    scale = float(np.sqrt(((ref - ref.mean(-1, keepdims=True)) ** 2).mean()))
    return float(np.sqrt((d ** 2).mean(-1)).max() / scale)


LIMIT = {"float32": 2e-5, "bfloat16": 3e-2}

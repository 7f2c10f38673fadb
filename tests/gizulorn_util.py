"""Small Gizulorn configurations shared by the CPU and GPU tests of that design.

The configurations differ from one another in every size and constant and use values that keep different sizes
distinct: key and value sizes unequal, partly rotated heads, key sizes that are no multiple of 16, grouped and ungrouped
heads, windows shorter and longer than a page, kept first tokens that span no page, one page and several, one to four
taps, one expert per token and all of them, one group and several, with and without a shared expert, a layer without
feed-forward, every order of the two layer types."""
from __future__ import annotations
import copy
import os

import numpy as np
import torch


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def _ret(heads, dim, vdim, decay, base, dims):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": _rot(base, dims)}


def _par(left, right, ls, rs):
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


def _left(heads, kv, dim, vdim, scale, size, keep, rot):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size, "keep_first": keep}, "rot": rot}


def _right(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(experts, top, ff, count=1, keep=1, shared=0):
    m = {"kind": "moe", "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


GIZ_MIX = {        # retention / parallel / retention without feed-forward; partly rotated heads; grouped experts, shared expert
    "architecture": "Gizulorn", "vocab": 173, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "retention", "mixer": _ret(2, 16, 24, [0.9, 0.97], 10000.0, 8), "mlp": {"kind": "dense", "ff": 48}},
        {"type": "parallel", "mixer": _par(_left(4, 2, 16, 8, 0.3, 9, 3, _rot(5000.0, 8, (4.0, 1.0, 4.0, 16))),
                                          _right(4, 2, 8, 16, 3), 0.7, 1.3), "mlp": _moe(6, 2, 16, 3, 2, 24)},
        {"type": "retention", "mixer": _ret(2, 16, 24, [0.5, 0.999], 10000.0, 8), "mlp": None},
    ]}
GIZ_ODD = {        # parallel first; sizes that are no multiples of 16; ungrouped heads; window shorter than a page, nothing kept;
                   # every expert chosen and none shared; one expert of five groups; five lanes' worth of key rows (40 -> 64)
    "architecture": "Gizulorn", "vocab": 89, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "parallel", "mixer": _par(_left(3, 3, 24, 40, 0.2, 5, 0, _rot(300.0, 24)), _right(2, 1, 20, 12, 2), 1.0, 0.25),
         "mlp": _moe(4, 4, 24)},
        {"type": "retention", "mixer": _ret(3, 40, 8, [0.75, 0.96875, 1.0], 1e6, 40), "mlp": _moe(5, 1, 8, 5, 1, 16)},
    ]}
GIZ_KEEP = {       # a single head; one tap (no convolution state); kept first tokens spanning several pages; a long window
    "architecture": "Gizulorn", "vocab": 61, "width": 32, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "parallel", "mixer": _par(_left(1, 1, 32, 16, 0.25, 33, 11, _rot(20.0, 32, (8.0, 1.0, 2.0, 64))),
                                          _right(1, 1, 16, 32, 1), 0.5, 2.0), "mlp": {"kind": "dense", "ff": 40}},
        {"type": "parallel", "mixer": _par(_left(6, 1, 8, 8, 0.35, 17, 2, _rot(10000.0, 2)), _right(3, 3, 12, 8, 4), 1.5, 0.5),
         "mlp": _moe(8, 3, 8, 4, 3, 0)},
    ]}
CONFIGS = {"mix": (GIZ_MIX, 3), "odd": (GIZ_ODD, 5), "keep": (GIZ_KEEP, 9)}
STD_SCALE = 5.0


def make_dir(name: str, tmp, cfg: dict | None = None, seed: int | None = None, change=None) -> tuple[str, dict, dict]:
    """Writes configuration `name` with seeded random weights (float32); `change(tensors)` may edit them before they
    are written. Returns (folder, config, weights by name)."""
    from fusezap_core_b200.weights import write_random_model
    from fusezap_core_b200.weights.safetensors_io import read_model_dir, write_file
    base, s = CONFIGS.get(name, (cfg, seed))
    cfg = copy.deepcopy(cfg if cfg is not None else base)
    d = os.path.join(str(tmp), f"gizulorn-{name}")
    write_random_model(cfg, d, seed if seed is not None else s, "float32", norm_noise=True, std_scale=STD_SCALE)
    w = read_model_dir(d)
    if change is not None:
        w = {k: v.clone() for k, v in w.items()}
        change(w)
        write_file(os.path.join(d, "model.safetensors"), w)
    return d, cfg, w


def tokens_for(cfg: dict, lengths, seed: int) -> list[list[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], n).tolist() for n in lengths]


def rounded(w: dict) -> dict:
    """The weights as a bfloat16 engine holds them: matrices rounded once, vectors stored in 32-bit as they are."""
    return {k: v.to(torch.bfloat16).to(torch.float32) if v.dim() >= 2 else v for k, v in w.items()}

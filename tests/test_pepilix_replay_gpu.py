"""Pepilix through the trace replay program on the GPU: a `bin/trace_run` process replays the same requests whole, with
their last 32 tokens one by one, in portions down to two tokens, and four at a time in a pool so small that pages and
state slots are used again; every position is compared with the plain model's logits of the whole request, and in
float32 the cuttings must agree with each other bit for bit (every sum's order is a function of the row alone).

The small configurations are those of `pepilix_util`; the two larger ones have layer sizes of a few hundred, a
bfloat16 checkpoint, requests of up to 1,300 tokens (key ranges cut and merged, keys far back) and sizes that reach
every tensor-core kernel (cached vectors of 112 and 192 values) or none (a width of 200, cached vectors of 80).
"""
import copy
import os

import numpy as np
import pytest
import torch

import plain_pepilix
from pepilix_util import CONFIGS, LIMIT, _mixer, _moe, rel_rms, tokens_for
from test_replay_gpu import LENGTHS, POOL_TOKENS, build_trace
from util import TraceBuilder, run_trace

pytestmark = pytest.mark.gpu


def _write(cfg: dict, path: str, seed: int, dtype: str) -> dict:
    from fusezap_core_b200.weights import write_random_model
    from safetensors.torch import load_file
    write_random_model(copy.deepcopy(cfg), path, seed, dtype, norm_noise=True, std_scale=4.0)
    return load_file(os.path.join(path, "model.safetensors"))


def _compare(got: dict, tb_prefix_of, refs, dtype: str, what: str) -> None:
    for rid, rows in sorted(got.items()):
        ref = refs[tb_prefix_of(rid)]
        assert sorted(rows) == list(range(len(ref))), f"{what} {rid}: positions {sorted(rows)[:5]}..."
        g = np.stack([rows[p] for p in range(len(ref))])
        assert rel_rms(g, ref) < LIMIT[dtype], f"{what} {dtype} request {rid}: {rel_rms(g, ref):.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_replay_all_cuttings(name, dtype, tmp_path):
    cfg, seed = CONFIGS[name]
    w = _write(cfg, str(tmp_path / "m"), seed, "float32")
    P = tokens_for(cfg, LENGTHS, seed=3)
    refs = [plain_pepilix.forward(cfg, w, ids, rounded=dtype == "bfloat16").numpy() for ids in P]
    tb = build_trace(P)
    assert tb.most_live == 4 and max(len(s["entries"]) for s in tb.steps) == 4
    outs = run_trace(str(tmp_path / "m"), dtype, str(tmp_path / "out"), max_tokens=POOL_TOKENS, steps=tb.steps)
    got = tb.collect(outs, cfg["vocab"])
    _compare(got, lambda rid: int(rid[1:]), refs, dtype, name)
    assert {r[0] for r in got} == {"w", "d", "p", "m"}
    if dtype == "float32":
        for rid, rows in sorted(got.items()):
            if rid[0] == "w":
                continue
            whole = got["w" + rid[1:]]
            for p, row in rows.items():
                assert np.array_equal(row, whole[p]), (f"{name}: request {rid} position {p} differs from the whole "
                                                       f"request's row by {np.abs(row - whole[p]).max():.3e}")


def _larger(which: str) -> dict:
    if which == "tensor_cores":      # every size a multiple of 16; cached vectors of 112 and 192; a layer without feed-forward
        a = lambda kf=None: _mixer(4, 48, 16, 40, 96, 0.11, 10000.0, kf)
        b = lambda kf=None: _mixer(7, 40, 32, 56, 160, 0.1, 500000.0, kf)
        layers = [(a(), _moe(8, 1, 128, 2.0)), (b(), _moe(10, 3, 112, 1.0)), (a(0), None), (b(1), _moe(10, 3, 112, 1.0)),
                  (a(), _moe(8, 8, 64, 0.5)), (a(4), _moe(8, 1, 128, 2.0))]
        head = {"vocab": 512, "width": 384, "embedding": {"scale": 19.6}, "logit_scale": 0.4,
                "norm": {"eps": 1e-5, "groups": 3}, "canon": {"taps": 3}}
    else:                            # a width of 200 in five norm groups, cached vectors of 80, six taps
        d = lambda kf=None: _mixer(3, 24, 8, 24, 72, 0.2, 300.0, kf)
        layers = [(d(), _moe(6, 2, 56, 1.5)), (d(), _moe(6, 2, 56, 1.5)), (d(0), _moe(24, 5, 16, 0.25))]
        head = {"vocab": 333, "width": 200, "embedding": {"scale": 7.0}, "logit_scale": 2.0,
                "norm": {"eps": 1e-4, "groups": 5}, "canon": {"taps": 6}}
    return {"architecture": "Pepilix", **head,
            "layers": [{"type": "latent_attention", "mixer": m, "mlp": f} for m, f in layers]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["tensor_cores", "general"])
def test_replay_larger_models_long_requests_in_a_small_pool(which, dtype, tmp_path):
    cfg = _larger(which)
    w = _write(cfg, str(tmp_path / "m"), 11, "bfloat16")
    assert w["embed"].dtype == torch.bfloat16 and w["l0.mlp.table"].dtype == torch.int32
    lengths = (1300, 260, 1, 23, 333, 97)
    P = dict(zip("abcdef", tokens_for(cfg, lengths, seed=5)))
    refs = {r: plain_pepilix.forward(cfg, w, ids, rounded=dtype == "bfloat16").numpy() for r, ids in P.items()}
    # a little scheduler: up to four live; portions of changing size, then each request's last tokens one by one
    rng = np.random.default_rng(8)
    tb, waiting, live, peak = TraceBuilder(), list(P), {}, 0
    single = {r: max(0, len(P[r]) - int(rng.integers(8, 40))) for r in P}
    while waiting or live:
        while waiting and len(live) < 4 and (not live or rng.random() < 0.7):
            live[waiting.pop(0)] = 0
        peak = max(peak, sum(-(-len(P[r]) // 64) * 64 for r in live))
        entries, ends = [], []
        for r in list(live):
            if rng.random() < 0.2 and len(live) > 1:
                continue
            at = live[r]
            n = 1 if at >= single[r] else min(int(rng.choice([2, 3, 5, 16, 17, 64, 100, 200])), single[r] - at)
            entries.append((r, P[r][at: at + n], "all"))
            live[r] = at + n
            if live[r] == len(P[r]):
                ends.append(r)
                del live[r]
        if entries:
            tb.step(entries, end=ends)
    assert max(len(s["entries"]) for s in tb.steps) == 4 and peak < sum(-(-n // 64) * 64 for n in lengths)
    outs = run_trace(str(tmp_path / "m"), dtype, str(tmp_path / "out"), max_tokens=peak, steps=tb.steps)
    _compare(tb.collect(outs, cfg["vocab"]), lambda rid: rid, refs, dtype, which)

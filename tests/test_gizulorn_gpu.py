"""Gizulorn on the GPU: the whole model through the engine's step function, cache manager and kernels against the plain
implementation (`plain_gizulorn.py`, 64-bit, whole sequences), in float32 and bfloat16."""
import numpy as np
import pytest
import torch

import plain_gizulorn
from gizulorn_util import CONFIGS, make_dir, rounded, tokens_for
from pepilix_util import rel_rms, run_cut, run_mixed
from fusezap_core_b200.cache import CacheManager
from fusezap_core_b200.engine import StepRunner, load_model

pytestmark = pytest.mark.gpu
LIMIT = {"float32": 2e-5, "bfloat16": 4e-2}


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gizulorn")
    return {name: make_dir(name, tmp) for name in CONFIGS}


def engine_parts(d, dtype, page=4, pages=48, slots=3, max_len=192):
    model = load_model(d, dtype, "cuda:0", max_len=max_len)
    cache = CacheManager(model.cache_needs(), model.state_needs(), page, pages, slots, max_len, model.ops.dtype, "cuda:0")
    return model, cache, StepRunner(model, cache, max_rows=max_len, max_wanted=max_len, max_segments=slots)


def oracle(cfg, w, toks, dtype):
    return plain_gizulorn.forward(cfg, w if dtype == "float32" else rounded(w), toks)[0].numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_every_size_against_the_whole_sequence(dirs, name, dtype):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, dtype)
    toks = tokens_for(cfg, (75,), seed=11)[0]
    ref = oracle(cfg, w, toks, dtype)
    for cuts in ((75,), (1,), (2,), (5, 3, 1, 7, 2, 19), (40, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1)):
        got = run_cut(runner, cache, "r", toks, cuts)
        model.ops.check_errors()
        assert rel_rms(got, ref) < LIMIT[dtype], (name, dtype, cuts, rel_rms(got, ref))
        cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(dirs, name, dtype):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, dtype, page=4, pages=40, slots=3, max_len=96)
    reqs = dict(zip("abcde", tokens_for(cfg, (61, 9, 33, 2, 47), seed=5)))
    plan = [[("a", 17), ("b", 2)], [("a", 1), ("b", 7), ("c", 30)], [("a", 20), ("c", 1)], [("a", 1), ("c", 1), ("d", 2)],
            [("a", 22), ("c", 1), ("e", 5)], [("e", 1)], [("e", 40)], [("e", 1)]]
    got = run_mixed(runner, cache, reqs, plan)
    model.ops.check_errors()
    cache.check()
    assert cache.live_requests() == []
    for r, toks in reqs.items():
        assert rel_rms(got[r], oracle(cfg, w, toks, dtype)) < LIMIT[dtype], (name, dtype, r)

"""Gizulorn on the CPU: the package's host side (configuration, model description, weights, cache pages with kept first
tokens, state slots, step packing, scheduler, entry point) with the plain operation table, against the plain
implementation on whole sequences."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_gizulorn
from gizulorn_util import CONFIGS, GIZ_MIX, GIZ_ODD, make_dir, tokens_for
from pepilix_util import rel_rms, run_cut, run_mixed
from plain_ops import PlainOpsSeq
from fusezap_core_b200 import LLMEngine, SamplingParams
from fusezap_core_b200.cache import CacheManager, KVNeed
from fusezap_core_b200.config import describe
from fusezap_core_b200.config.gizulorn import GizulornConfig
from fusezap_core_b200.engine import StepRunner, load_model
from fusezap_core_b200.engine.model import DecoderModel


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gizulorn")
    return {name: make_dir(name, tmp) for name in CONFIGS}


def engine_parts(d, page=4, pages=48, slots=3, max_len=160):
    model = load_model(d, "float32", "cpu", max_len=max_len, ops=PlainOpsSeq(torch.float32))
    cache = CacheManager(model.cache_needs(), model.state_needs(), page, pages, slots, max_len, torch.float32, "cpu")
    return model, cache, StepRunner(model, cache, max_rows=max_len, max_wanted=max_len, max_segments=slots)


def test_config_reads_every_size_and_round_trips():
    typed, spec = describe(copy.deepcopy(GIZ_MIX))
    assert isinstance(typed, GizulornConfig) and typed.to_json() == json.loads(json.dumps(GIZ_MIX))
    kinds = [L.mixer.kind for L in spec.layers]
    assert kinds == ["retention", "parallel_mixers", "retention"] and spec.layers[2].ffn is None
    left, right = (m for _, m, _ in spec.layers[1].mixer.params["mixers"])
    assert (left.params["window"], left.params["keep_first"], left.params["value_dim"]) == (9, 3, 8)
    assert right.params["taps"] == 3 and right.params["query_scale"] == 8 ** -0.5
    moe = spec.layers[1].ffn.params
    assert (moe["num_experts"], moe["top"], moe["groups"], moe["keep_groups"], moe["shared_size"]) == (6, 2, 3, 2, 24)
    assert spec.layers[0].ffn.kind == "swiglu" and spec.lm_head_name == "head" and not spec.tie_embeddings
    assert len(spec.positions) == 2      # the two retention layers share one rotation, the attention has another


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="other"), "not supported"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["left"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(conv=0), "tap"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="other"), "not supported"),
    (lambda c: c.pop("norm"), "lacks"),
])
def test_config_refusals(change, message):
    c = copy.deepcopy(GIZ_MIX)
    change(c)
    with pytest.raises((ValueError, NotImplementedError), match=message):
        describe(c)


def test_random_weights_name_every_tensor(dirs):
    d, cfg, w = dirs["mix"]
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.g", "l0.mix.o", "l0.mlp.gate", "l0.mlp.down",
            "l1.mix.left.q", "l1.mix.left.sink", "l1.mix.right.q.conv", "l1.mix.right.v.conv", "l1.mix.right.b", "l1.mix.right.A_log",
            "l1.mix.right.a1", "l1.mix.right.a2", "l1.mix.right.dt_bias", "l1.mix.right.g1", "l1.mix.right.g2", "l1.mix.right.norm",
            "l1.mlp.router", "l1.mlp.e5.up", "l1.mlp.shared.gate", "l1.mlp.shared.sg", "l2.norm1", "l2.mix.v"} <= set(w)
    assert "l2.norm2" not in w and not any(k.startswith("l2.mlp") for k in w)
    assert tuple(w["l1.mix.left.k"].shape) == (2 * 16, 64) and tuple(w["l1.mix.left.v"].shape) == (2 * 8, 64)
    assert tuple(w["l1.mix.right.v.conv"].shape) == (4 * 16, 3) and tuple(w["l1.mlp.shared.sg"].shape) == (1, 64)
    assert w["l1.mix.right.a2"].shape[1] == w["l1.mix.right.a1"].shape[0]


def test_inner_sizes_of_the_two_step_projections_come_from_the_checkpoint(tmp_path):
    def other_ranks(w):
        g = torch.Generator().manual_seed(0)
        w["l1.mix.right.a1"], w["l1.mix.right.a2"] = torch.randn(5, 64, generator=g) * 0.1, torch.randn(4 * 8, 5, generator=g) * 0.1
        w["l1.mix.right.g1"], w["l1.mix.right.g2"] = torch.randn(3, 64, generator=g) * 0.1, torch.randn(4 * 16, 3, generator=g) * 0.1
    d, cfg, w = make_dir("ranks", tmp_path, GIZ_MIX, 4, change=other_ranks)
    model, cache, runner = engine_parts(d)
    toks = tokens_for(cfg, (20,), seed=1)[0]
    assert rel_rms(run_cut(runner, cache, "r", toks, (20,)), plain_gizulorn.forward(cfg, w, toks)[0].numpy()) < 2e-5


def test_pages_between_the_kept_first_tokens_and_the_window_are_given_back():
    need = KVNeed(2, 16, window=9, value_dim=8, keep_first=6)
    cache = CacheManager({0: need}, {}, 4, 12, 2, 200, torch.float32, "cpu")
    assert cache.groups[0].pool.shape == (1, 12, 2, 4, 24)
    k, v = cache.groups[0].view(0)
    assert k.shape == (12, 2, 4, 16) and v.shape == (12, 2, 4, 8)
    for n in range(1, 41):
        cache.ensure("a", n)
        cache.commit("a", n)
        cache.check()
        row = cache.table(0, "a")
        # the next query is at position n: it sees n - 8 .. n and 0 .. 5; pages of tokens 0 .. 5 are pages 0 and 1
        live = {p // 4 for p in range(max(0, n - 8), n)} | {0, 1}
        assert {i for i, p in enumerate(row) if p >= 0} == {i for i in live if i < len(row)}, (n, row)
    assert cache.num_free_pages == 12 - len([p for p in cache.table(0, "a") if p >= 0])
    cache.free("a")
    assert cache.num_free_pages == 12


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_every_size_against_the_whole_sequence(dirs, name):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d)
    toks = tokens_for(cfg, (50,), seed=11)[0]
    ref = plain_gizulorn.forward(cfg, w, toks)[0].numpy()
    for cuts in ((50,), (1,), (2,), (5, 3, 1, 7, 2, 19)):
        assert rel_rms(run_cut(runner, cache, "r", toks, cuts), ref) < 2e-5, (name, cuts)
        cache.check()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(dirs, name):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, page=4, pages=30, slots=3, max_len=64)
    reqs = dict(zip("abcde", tokens_for(cfg, (41, 9, 23, 2, 30), seed=5)))
    plan = [[("a", 17), ("b", 2)], [("a", 1), ("b", 7), ("c", 20)], [("a", 20), ("c", 1)], [("a", 1), ("c", 1), ("d", 2)],
            [("a", 2), ("c", 1), ("e", 5)], [("e", 1)], [("e", 24)]]
    got = run_mixed(runner, cache, reqs, plan)
    cache.check()
    assert cache.live_requests() == [] and cache.states.num_free == 3
    for r, toks in reqs.items():
        assert rel_rms(got[r], plain_gizulorn.forward(cfg, w, toks)[0].numpy()) < 2e-5, (name, r)


def test_state_is_declared_per_layer_and_kept_in_slots(dirs):
    d, cfg, w = dirs["mix"]
    model, cache, runner = engine_parts(d, slots=2)
    names = sorted(model.state_needs())
    assert names == [(0, "S"), (1, "right.S"), (1, "right.conv"), (2, "S")]
    assert model.state_needs()[(1, "right.conv")] == (2, 2 * 2 * 8 + 4 * 16)
    assert isinstance(model.cache_needs()[1], KVNeed) and list(model.cache_needs()) == [1]
    assert model.graph_safe()


def test_greedy_generation_through_the_entry_point(dirs):
    """Through `LLMEngine` and its scheduler: portions of prompts beside decoding requests, more requests than state
    slots, a pool that does not hold all of them at once."""
    d, cfg, w = dirs["odd"]
    eng = LLMEngine.from_pretrained(d, dtype="float32", device="cpu", ops=PlainOpsSeq(torch.float32), max_model_len=64,
                                    num_blocks=14, block_size=8, max_num_seqs=2, max_prefill_tokens=8, cuda_graphs=False)
    P = tokens_for(cfg, (7, 19, 2, 30), seed=2)
    out = eng.generate(P, SamplingParams(max_tokens=5, ignore_eos=True))
    for prompt, new in zip(P, out):
        lg = plain_gizulorn.forward(cfg, w, list(prompt) + new)[0].numpy()
        for i, t in enumerate(new):
            row = lg[len(prompt) - 1 + i]
            assert int(row.argmax()) == t or row.max() - row[t] < 1e-3


def test_command_line_writes_a_preset_and_the_engine_loads_it(tmp_path):
    import os
    from fusezap_core_b200.cli import main, presets
    from fusezap_core_b200.weights.safetensors_io import read_model_dir
    assert "tiny-gizulorn" in presets()
    out = str(tmp_path / "m")
    assert main(["random-weights", "--preset", "tiny-gizulorn", "--out", out, "--seed", "4", "--dtype", "float32", "--num-layers", "2"]) == 0
    with open(os.path.join(out, "config.json")) as f:
        cfg = json.load(f)
    assert [L["type"] for L in cfg["layers"]] == ["retention", "parallel"]
    w = read_model_dir(out)
    model, cache, runner = engine_parts(out)
    toks = tokens_for(cfg, (19,), seed=6)[0]
    got = run_cut(runner, cache, "r", toks, [6, 1, 12])
    assert np.isfinite(got).all() and got.shape == (19, 512)
    # weights of N(0, 0.02) make small logits: the difference is judged against the residual's size, not theirs
    ref = plain_gizulorn.forward(cfg, w, toks)[0].numpy()
    assert np.abs(got - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())

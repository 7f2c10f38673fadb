"""Pepilix on the CPU: the package's host side (configuration, model description, weights, cache and state slots, step
packing, scheduler, entry point) with the plain operation table, against the plain implementation on whole sequences."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_pepilix
from pepilix_util import CONFIGS, LIMIT, PEP_SMALL, make_dir, rel_rms, run_cut, run_mixed, tokens_for
from plain_ops import PlainOpsWide
from fusezap_core_b200 import LLMEngine, SamplingParams
from fusezap_core_b200.cache import CacheManager, LatentNeed
from fusezap_core_b200.config import describe
from fusezap_core_b200.config.pepilix import PepilixConfig
from fusezap_core_b200.engine import StepRunner, load_model


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("pepilix")
    return {name: make_dir(name, tmp) for name in CONFIGS}


def engine_parts(d, page=4, pages=40, slots=3, max_len=160):
    model = load_model(d, "float32", "cpu", max_len=max_len, ops=PlainOpsWide(torch.float32))
    cache = CacheManager(model.cache_needs(), model.state_needs(), page, pages, slots, max_len, torch.float32, "cpu")
    return model, cache, StepRunner(model, cache, max_rows=max_len, max_wanted=max_len, max_segments=slots)


def test_config_reads_every_size_and_round_trips():
    typed, spec = describe(copy.deepcopy(PEP_SMALL))
    assert isinstance(typed, PepilixConfig) and typed.to_json() == json.loads(json.dumps(PEP_SMALL))
    assert [e.cache for e in spec.schedule] == [0, 1, 0] and [e.write_cache for e in spec.schedule] == [True, True, False]
    assert spec.layers[1].ffn is None and spec.layers[0].ffn.params["top"] == 1 and spec.layers[2].ffn.params["num_experts"] == 4
    assert spec.embed_scale == 3.5 and spec.logit_transform.params["factor"] == 0.25
    assert spec.final_norm.params["groups"] == 3 and spec.layers[0].block.params["taps"] == 3
    assert len(spec.positions) == 2      # two distinct rotations among the three layers


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "differ"),
    (lambda c: c["norm"].update(groups=5), "norm groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0].update(type="other_mixer"), "not supported"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "even"),
])
def test_config_refusals(change, message):
    c = copy.deepcopy(PEP_SMALL)
    change(c)
    with pytest.raises((ValueError, NotImplementedError), match=message):
        describe(c)


def test_random_weights_name_every_tensor_and_tables_hold_distinct_experts(dirs):
    d, cfg, w = dirs["small"]
    assert {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.canon1", "l0.rg1", "l0.rg1.b", "l0.rg2.b", "l0.mix.dkv",
            "l0.mix.dkv.norm", "l0.mix.uk", "l0.mlp.e4.down", "l0.mlp.table", "l2.mlp.e3.gate"} <= set(w)
    assert "l2.mix.dkv" not in w and "l1.norm2" not in w and "l1.rg2" not in w and "l1.mlp.table" not in w
    t = w["l2.mlp.table"]
    assert t.dtype == torch.int32 and tuple(t.shape) == (211, 3) and int(t.min()) >= 0 and int(t.max()) < 4
    assert all(len(set(r)) == 3 for r in t.tolist())
    model, cache, _ = engine_parts(d)
    assert model.cache_needs() == {0: LatentNeed(48), 1: LatentNeed(28)}
    assert {k: v for k, v in model.state_needs().items()} == {(i, "conv"): (2, 96) for i in range(3)}
    assert [tuple(g.pool.shape) for g in cache.groups] == [(1, 40, 4, 48), (1, 40, 4, 28)]


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_single_tokens_equal_whole_sequences(dirs, name):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d)
    for toks in tokens_for(cfg, (1, 2, 37, 90), seed=4):
        ref = plain_pepilix.forward(cfg, w, toks).numpy()
        for cuts in ([len(toks)], [1], [2], [len(toks) - 1, 1] if len(toks) > 1 else [1], [5, 1, 3, 2, 11, 1, 1, 4]):
            got = run_cut(runner, cache, "r", toks, cuts)
            assert rel_rms(got, ref) < LIMIT["float32"], f"{name}, {len(toks)} tokens in portions {cuts}"
    cache.check()
    assert cache.states.num_free == 3 and cache.num_free_pages == 40


@pytest.mark.parametrize("name", ["small", "wide"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(dirs, name):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, page=4, pages=36, slots=3)
    toks = dict(zip("abcde", tokens_for(cfg, (41, 9, 66, 23, 50), seed=8)))
    ref = {r: plain_pepilix.forward(cfg, w, t).numpy() for r, t in toks.items()}
    plan = [[("a", 7), ("b", 2)], [("a", 1), ("b", 1), ("c", 30)], [("b", 6), ("c", 2), ("a", 20)], [("a", 1), ("c", 1)],
            [("c", 33), ("a", 12)],          # a and c end here: their pages and slots go back
            [("d", 5), ("e", 17)], [("d", 1), ("e", 1)], [("e", 32), ("d", 17)]]
    got = run_mixed(runner, cache, toks, plan)
    for r in toks:
        assert got[r].shape == ref[r].shape
        assert rel_rms(got[r], ref[r]) < LIMIT["float32"], f"{name}, request {r}"
    cache.check()
    assert cache.states.num_free == 3 and cache.num_free_pages == 36


def test_greedy_generation_through_the_entry_point_and_scheduler(dirs):
    d, cfg, w = dirs["small"]
    eng = LLMEngine.from_pretrained(d, dtype="float32", device="cpu", max_model_len=96, ops=PlainOpsWide(torch.float32),
                                    num_blocks=14, block_size=8, max_num_seqs=2, max_prefill_tokens=16, cuda_graphs=False)
    prompts = tokens_for(cfg, (3, 29, 12, 1), seed=2)
    out = eng.generate(prompts, SamplingParams(max_tokens=7, ignore_eos=True))
    for prompt, new in zip(prompts, out):
        lg = plain_pepilix.forward(cfg, w, list(prompt) + new).numpy()
        for i, t in enumerate(new):          # every pick is the plain model's best logit (ties within rounding)
            row = lg[len(prompt) - 1 + i]
            assert row.max() - row[t] <= 1e-4 * np.abs(row).max()
    assert eng.cache.states.num_free == 2 and eng.cache.num_free_pages == 14


@pytest.mark.parametrize("taps", [0, 1])
def test_one_tap_and_no_convolution(tmp_path, taps):
    """One tap is a per-channel scale of the mixer's input without state; a configuration without the key has no
    convolution and no such tensor."""
    from fusezap_core_b200.weights import write_random_model
    from safetensors.torch import load_file
    cfg = copy.deepcopy(PEP_SMALL)
    if taps:
        cfg["canon"] = {"taps": taps}
    else:
        del cfg["canon"]
    d = write_random_model(cfg, str(tmp_path / "m"), 31, "float32", norm_noise=True, std_scale=4.0)
    w = load_file(os.path.join(d, "model.safetensors"))
    assert ("l0.canon1" in w) == bool(taps)
    model, cache, runner = engine_parts(d)
    assert model.state_needs() == {}
    toks = tokens_for(cfg, (33,), seed=1)[0]
    got = run_cut(runner, cache, "r", toks, [4, 1, 9])
    assert rel_rms(got, plain_pepilix.forward(cfg, w, toks).numpy()) < LIMIT["float32"]


def test_tensors_of_an_absent_feed_forward_are_passed_over(dirs, tmp_path):
    """A checkpoint that carries a second norm and gate for a layer without feed-forward loads, and they change nothing."""
    from fusezap_core_b200.weights.safetensors_io import write_file
    d, cfg, w = dirs["small"]
    more = dict(w)
    more["l1.norm2"], more["l1.rg2"], more["l1.rg2.b"] = torch.ones(96), torch.ones(96, 96), torch.ones(96)
    d2 = str(tmp_path / "m")
    os.makedirs(d2)
    with open(os.path.join(d2, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(d2, "model.safetensors"), more.items())
    toks = tokens_for(cfg, (20,), seed=3)[0]
    out = []
    for folder in (d, d2):
        model, cache, runner = engine_parts(folder)
        out.append(run_cut(runner, cache, "r", toks, [20]))
    assert np.array_equal(out[0], out[1])


def test_command_line_writes_a_preset_and_the_engine_loads_it(tmp_path):
    from fusezap_core_b200.cli import main, presets
    assert "tiny-pepilix" in presets()
    out = str(tmp_path / "m")
    assert main(["random-weights", "--preset", "tiny-pepilix", "--out", out, "--seed", "4", "--dtype", "float32", "--num-layers", "2"]) == 0
    with open(os.path.join(out, "config.json")) as f:
        cfg = json.load(f)
    assert len(cfg["layers"]) == 2 and cfg["layers"][1]["mixer"]["kv_from"] == 0
    from safetensors.torch import load_file
    w = load_file(os.path.join(out, "model.safetensors"))
    model, cache, runner = engine_parts(out)
    toks = tokens_for(cfg, (19,), seed=6)[0]
    got = run_cut(runner, cache, "r", toks, [6, 1, 12])
    assert np.isfinite(got).all() and got.shape == (19, 512)
    # weights of N(0, 0.02) make small logits: the difference is judged against the residual's size, not theirs
    ref = plain_pepilix.forward(cfg, w, toks).numpy()
    assert np.abs(got - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())

"""Gizulorn on the GPU: the whole model through the engine's step function, cache manager and kernels against the plain
implementation (`plain_gizulorn.py`, 64-bit, whole sequences), in float32 and bfloat16."""
import numpy as np
import pytest
import torch

import plain_gizulorn
from gizulorn_util import CONFIGS, _left, _moe, _par, _ret, _right, _rot, make_dir, rounded, tokens_for
from pepilix_util import rel_rms, run_cut, run_mixed
from fusezap_core_b200.cache import CacheManager
from fusezap_core_b200.engine import StepRunner, load_model

pytestmark = pytest.mark.gpu
# float32: sequential 32-bit sums against a 64-bit oracle: 1e-5 of the logits' scale and less. The head norms divide
# small recurrent outputs by their root mean square, which carries the rounding of a state that is still nearly empty
# into the logits of a sequence's first tokens (measured: up to 7e-5 at single positions, the first above all), so the
# bound is asked of 19 rows in 20 and no row may be off by more than ten times the bound.
LIMIT = {"float32": 2e-5, "bfloat16": 4e-2}


def row_errors(got, ref):
    """Per row: the root-mean-square difference (row mean removed), relative to the rms of the reference's logits."""
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    scale = float(np.sqrt(((ref - ref.mean(-1, keepdims=True)) ** 2).mean()))
    return np.sqrt((d ** 2).mean(-1)) / scale


def agrees(got, ref, dtype, what=None):
    """float32: see LIMIT. bfloat16: rounding moves a row's logits by a per cent or two of their
    scale, but where two experts' router scores nearly tie, rounding picks the other one and that row differs by much
    more (the oracle has no such rounding); so the bound is asked of the median row and of nine rows in ten, and no row
    may be off by more than the scale of the logits itself."""
    e = row_errors(got, ref)
    if dtype == "float32":
        assert np.quantile(e, 0.95) < LIMIT[dtype] and e.max() < 10 * LIMIT[dtype], (what, float(np.quantile(e, 0.95)), float(e.max()))
    else:
        assert np.median(e) < LIMIT[dtype] and np.quantile(e, 0.9) < 2 * LIMIT[dtype] and e.max() < 1.0, \
            (what, float(np.median(e)), float(np.quantile(e, 0.9)), float(e.max()))


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
        agrees(got, ref, dtype, (name, cuts))
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
        agrees(got[r], oracle(cfg, w, toks, dtype), dtype, (name, r))


# ------------------------------------------------------------------------------------------------ every mechanism alone
import plain_gizulorn as plain
from fusezap_core_b200 import LLMEngine, SamplingParams
from fusezap_core_b200.cache import KVNeed
from fusezap_core_b200.engine.step import StepContext, Workspace
from fusezap_core_b200.kernels import cuda_ops
from fusezap_core_b200.parts import LayerCache
from fusezap_core_b200.parts.routed_moe import RoutedMoE

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64


class Meta:
    """The step metadata a kernel reads, for portions laid out by the test itself: (rows, first position, state slot)
    each; `tables`: int32 (portions, pages per request); `pad` rows of padding at the end."""
    def __init__(self, portions, tables=None, pad=0, max_segments=None):
        row, pos, seg, at = [], [], [], 0
        for s, (n, p0, slot) in enumerate(portions):
            row += [s] * n
            pos += list(range(p0, p0 + n))
            seg.append((at, n, p0, slot))
            at += n
        self.max_segments = max_segments or len(portions) + 2
        seg_all = seg + [(0, 0, 0, 0)] * (self.max_segments - len(seg))
        self.seq_row = torch.tensor(row + [-1] * pad, dtype=torch.int32, device=DEV)
        self.pos = torch.tensor(pos + [0] * pad, dtype=torch.int32, device=DEV)
        self.seg = torch.tensor(seg_all, dtype=torch.int32, device=DEV)
        self.n_segments, self.n_rows = len(portions), at + pad
        self.max_context = max(p0 + n for n, p0, _ in portions)
        self._table = tables.to(DEV) if tables is not None else None

        class Sg:
            def __init__(s, a): s.row0, s.n, s.pos0, s.state_slot = a
        self.segments = [Sg(a) for a in seg]

    def table(self, group):
        return self._table


def close(got, ref, dtype, what=""):
    """float32: a few units in the last place of the largest value around (sums of up to a few hundred terms of that
    size); bfloat16: one rounding of the result."""
    got, ref = got.detach().cpu().to(F), ref.to(F)
    if dtype == "float32":
        bad = (got - ref).abs() > 3e-6 * (ref.abs() + ref.abs().max() + 1e-3)
    else:
        bad = (got - ref).abs() > 2.0 ** -7 * (ref.abs() + ref.abs().mean() + 1e-3)
    assert not bad.any(), (what, float((got - ref).abs().max()), float(ref.abs().max()))


def cos_sin(rot, max_len):
    a = torch.arange(max_len, dtype=F)[:, None] * plain.frequencies(rot)[None, :]
    return torch.cos(a).float().to(DEV), torch.sin(a).float().to(DEV)


def paged(need, page, pages, dtype):
    pool = torch.zeros(need.pool_shape(1, pages, page), dtype=DT[dtype], device=DEV)
    keys, values = need.views(pool[0])
    return LayerCache(keys, values, 0, page, True, {})


def shuffled_tables(requests, per, pages, seed):
    """A block table per request with `per` pages each, drawn without repetition from `pages`."""
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(seed))[: requests * per]
    return order.to(torch.int32).view(requests, per)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,dk,dv,rotated,pairing", [(4, 2, 16, 8, 8, "neighbours"), (3, 3, 24, 40, 24, "halves"),
                                                          (6, 1, 8, 8, 2, "neighbours"), (2, 1, 32, 16, 0, "halves"),
                                                          (2, 2, 40, 72, 40, "neighbours")])
def test_rotation_and_cache_write(dtype, Hq, Hkv, dk, dv, rotated, pairing):
    """Two portions and a padding row on shuffled pages: q leaves rotated, k rotated and v as it is lie at each token's
    place, nothing else is written."""
    ops, g, page = cuda_ops(dtype), torch.Generator().manual_seed(dk + dv), 4
    rot = {"base": 300.0, "dims": rotated, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}}
    portions = [(5, 9, 0), (1, 2, 1)]
    tables = shuffled_tables(2, 4, 11, seed=dk)
    meta = Meta(portions, tables, pad=1)
    n = meta.n_rows
    qkv = torch.randn(n, (Hq + Hkv) * dk + Hkv * dv, generator=g)
    cache = paged(KVNeed(Hkv, dk, 0, value_dim=dv), page, 11, dtype)
    cache.keys.fill_(7.0), cache.values.fill_(7.0)
    cos, sin = cos_sin(rot, 32) if rotated else (None, None)
    q_out = torch.empty(n, Hq * dk, dtype=DT[dtype], device=DEV)
    ops.rotate_kv_write(qkv.to(DEV), cos, sin, rotated, {"halves": 0, "neighbours": 1}[pairing], meta, cache, q_out, Hq, Hkv, dk, dv)
    ops.check_errors()
    layout = "interleaved" if pairing == "neighbours" else "half"
    written = torch.zeros_like(cache.keys[..., 0], dtype=torch.bool)
    at = 0
    for s, (cnt, p0, _) in enumerate(portions):
        x = qkv[at: at + cnt].to(F)
        q = x[:, :Hq * dk].view(cnt, Hq, dk)
        k = x[:, Hq * dk:(Hq + Hkv) * dk].view(cnt, Hkv, dk)
        if rotated:
            q, k = plain.rotate(q, rot, layout, p0), plain.rotate(k, rot, layout, p0)
        close(q_out[at: at + cnt].view(cnt, Hq, dk), q, dtype, "q")
        for i in range(cnt):
            pg, off = int(tables[s, (p0 + i) // page]), (p0 + i) % page
            close(cache.keys[pg, :, off], k[i], dtype, "k")
            close(cache.values[pg, :, off], x[i, (Hq + Hkv) * dk:].view(Hkv, dv), dtype, "v")
            written[pg, :, off] = True
        at += cnt
    assert float(q_out[at:].abs().max()) == 0.0
    assert (cache.keys[~written] == 7.0).all() and (cache.values[~written] == 7.0).all()


def attention_case(dtype, Hq, Hkv, dk, dv, window, keep, sink, T, portions, page, seed, loud=None):
    """Keys and values of one sequence of T tokens go into shuffled pages through `rotate_kv_write` (no rotation), then
    `portions` ((rows, first position) each, all of that sequence) are asked for in one step, each with a block table
    of its own that names the same pages. loud: (key position, factor): that key and every query point one way, so its
    score stands out by the factor. Returns (rows' outputs, the plain result for the same rows)."""
    ops, g = cuda_ops(dtype), torch.Generator().manual_seed(seed)
    dt = DT[dtype]
    q = torch.randn(T, Hq, dk, generator=g).to(dt)
    k = torch.randn(T, Hkv, dk, generator=g).to(dt)
    v = torch.randn(T, Hkv, dv, generator=g).to(dt)
    if loud is not None:
        j, factor = loud
        way = torch.nn.functional.normalize(torch.randn(dk, generator=g), dim=0)
        k[j] = (way * factor).to(dt)
        q = (q.float() * 0.1 + way * factor).to(dt)
    sk = (torch.randn(Hq, generator=g) * 2).float() if sink else None
    scale = 0.3
    pages = -(-T // page)
    table = shuffled_tables(1, pages, pages + 5, seed)
    cache = paged(KVNeed(Hkv, dk, window, value_dim=dv, keep_first=keep), page, pages + 5, dtype)
    qkv = torch.cat([q.view(T, -1), k.view(T, -1), v.view(T, -1)], 1).float()
    ops.rotate_kv_write(qkv.to(DEV), None, None, 0, 0, Meta([(T, 0, 0)], table), cache, torch.empty(T, Hq * dk, dtype=dt, device=DEV), Hq, Hkv, dk, dv)
    meta = Meta([(n, p0, 0) for n, p0 in portions], table.repeat(len(portions), 1), pad=1)
    rows = [p for n, p0 in portions for p in range(p0, p0 + n)]
    qs = torch.cat([q[rows].view(len(rows), -1), torch.zeros(1, Hq * dk, dtype=dt)]).to(DEV)
    out = torch.empty(len(rows) + 1, Hq * dv, dtype=dt, device=DEV)
    ops.sink_attention(qs, cache, meta, out, Hq, Hkv, dk, dv, scale, window, keep, sk.to(DEV) if sink else None)
    ops.check_errors()
    assert float(out[-1].abs().max()) == 0.0
    ref = plain.sink_window_attention(q.to(F), k.to(F), v.to(F), scale, window or T + 1, keep,
                                      sk.to(F) if sink else torch.full((Hq,), -1e30, dtype=F))
    return out[:-1].view(len(rows), Hq, dv), ref[rows], (q, k, v)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,dk,dv,window,keep,sink", [(4, 2, 16, 8, 9, 3, True), (3, 3, 24, 40, 5, 0, True), (6, 1, 8, 8, 17, 2, False),
                                                           (1, 1, 32, 16, 33, 11, True), (2, 1, 64, 64, 0, 0, True), (40, 1, 16, 16, 6, 6, True),
                                                           (8, 2, 64, 64, 40, 6, True), (4, 4, 128, 128, 33, 0, False), (6, 3, 64, 64, 70, 65, True)])
def test_attention_rows_of_portions_and_single_tokens(dtype, Hq, Hkv, dk, dv, window, keep, sink):
    """Rows of a long portion, of a two-token portion and single tokens, at the start of the sequence and far into it."""
    got, ref, _ = attention_case(dtype, Hq, Hkv, dk, dv, window, keep, sink, T=90, page=4, seed=Hq * dk + window,
                                 portions=[(30, 0), (2, 40), (1, 57), (1, 89), (1, 5), (20, 64)])
    close(got, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("as_portion", [True, False])
@pytest.mark.parametrize("dk,dv", [(16, 8), (64, 64)])      # (in bfloat16 the second pair runs portions on tensor cores)
def test_a_key_that_stands_out_is_seen_exactly_where_the_mask_says(dtype, as_portion, dk, dv):
    """One key's score exceeds all others by far, so a row's output is that key's value if the row sees the key and
    something else if not: the key far back, at a page border, just inside and just outside the window, the last kept
    first token and the first one not kept, for rows of a portion and for single tokens."""
    window, keep, page, T = 12, 5, 8, 700
    for j in (0, keep - 1, keep, 7, 8, 300, T - 1 - window, T - window, T - 2):
        rows = sorted({p for p in (j, j + 1, j + window - 1, j + window, j + window + 1, T - 1) if j <= p < T})
        # (a portion of at least 20 rows: long enough for the kernel that takes tiles of rows)
        portions = [(min(max(rows[-1] - rows[0] + 1, 20), T - rows[0]), rows[0])] if as_portion and rows[-1] - rows[0] < 40 else [(1, p) for p in rows]
        got, ref, (q, k, v) = attention_case(dtype, 2, 1, dk, dv, window, keep, False, T, portions, page, seed=j, loud=(j, 12.0))
        close(got, ref, dtype, f"key {j}")
        at = 0
        for n, p0 in portions:
            for p in range(p0, p0 + n):
                sees = p - j < window or j < keep
                same = (got[at].float().cpu() - v[j].float()).abs().max() < 0.05
                assert bool(same) == sees, (j, p, sees)
                at += 1


def scan_portions(total, seed):
    """Two sequences of `total` tokens cut into portions (down to one token), interleaved in the steps."""
    rng = np.random.default_rng(seed)
    steps, at = [], [0, 0]
    while min(at) < total:
        step = []
        for r in (0, 1):
            if at[r] < total and (rng.random() < 0.8 or at[1 - r] >= total):
                n = int(min(total - at[r], rng.choice([1, 1, 2, 3, 8, 9, 17, 30])))
                step.append((r, at[r], n))
                at[r] += n
        if step:
            steps.append(step)
    return steps


@pytest.mark.parametrize("H,dk,dv,rotated,pairing", [(2, 16, 24, 8, 0), (3, 40, 8, 40, 1), (1, 128, 64, 64, 0), (2, 24, 100, 0, 0), (5, 8, 300, 8, 1),
                                                     (2, 9, 7, 4, 1), (1, 200, 6, 100, 0)])
def test_retention_scan_carries_its_state_across_portions(H, dk, dv, rotated, pairing):
    ops, g, T = cuda_ops("float32"), torch.Generator().manual_seed(dk), 70
    rot = {"base": 50.0, "dims": rotated}
    decay = torch.tensor([0.5, 0.96875, 1.0, 0.9, 0.999][:H])
    cos, sin = cos_sin(rot, 128) if rotated else (None, None)
    proj = [torch.randn(T, H * (2 * dk + dv) + 5, generator=g) for _ in range(2)]      # (some columns follow that the scan leaves alone)
    state = torch.zeros(4, *ops.recurrent_state_shape(H, dk, dv), device=DEV)
    state[2] = 3.0        # a slot nobody uses must stay as it is
    slots, got = (3, 1), [torch.zeros(T, H * dv), torch.zeros(T, H * dv)]
    for step in scan_portions(T, seed=dv):
        meta = Meta([(n, p0, slots[r]) for r, p0, n in step], pad=1)
        x = torch.cat([proj[r][p0: p0 + n] for r, p0, n in step] + [torch.zeros(1, proj[0].shape[1])]).to(DEV)
        out = torch.full((meta.n_rows, H * dv), 9.0, device=DEV)
        ops.retention_scan(x, H, dk, dv, decay.to(DEV), dk ** -0.5, cos, sin, rotated, pairing, state, meta, out)
        at = 0
        for r, p0, n in step:
            got[r][p0: p0 + n] = out[at: at + n].cpu()
            at += n
    ops.check_errors()
    layout = "interleaved" if pairing else "half"
    for r in (0, 1):
        x = proj[r].to(F)
        q, k = x[:, :H * dk].view(T, H, dk), x[:, H * dk: 2 * H * dk].view(T, H, dk)
        v = x[:, 2 * H * dk: 2 * H * dk + H * dv].view(T, H, dv)
        if rotated:
            q, k = plain.rotate(q, rot, layout), plain.rotate(k, rot, layout)
        ref = plain.retention(q, k * dk ** -0.5, v, decay.to(F))
        close(got[r].view(T, H, dv), ref, "float32", f"request {r}")
    assert (state[2] == 3.0).all() and float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,Hk,dk,dv", [(4, 2, 8, 16), (2, 1, 20, 12), (1, 1, 16, 32), (3, 3, 12, 8), (2, 2, 128, 40), (6, 3, 48, 260),
                                        (2, 1, 9, 7), (1, 1, 136, 10)])
def test_gated_delta_scan_carries_its_state_across_portions(dtype, H, Hk, dk, dv):
    ops, g, T, dt = cuda_ops(dtype), torch.Generator().manual_seed(dk + dv), 60, DT[dtype]
    C = 2 * Hk * dk + H * dv
    qkv = [torch.randn(T, C, generator=g).to(dt) for _ in range(2)]
    high = [torch.randn(T, H * dk + 7, generator=g) for _ in range(2)]
    beta = [torch.randn(T, H, generator=g) * 2 for _ in range(2)]
    a_log, dt_bias = torch.randn(H, generator=g) * 0.5, torch.randn(H * dk, generator=g)
    state = torch.zeros(3, *ops.recurrent_state_shape(H, dk, dv), device=DEV)
    slots, got = (2, 0), [torch.zeros(T, H * dv), torch.zeros(T, H * dv)]
    for step in scan_portions(T, seed=dk):
        meta = Meta([(n, p0, slots[r]) for r, p0, n in step], pad=2)
        cat = lambda xs, w, d: torch.cat([xs[r][p0: p0 + n] for r, p0, n in step] + [torch.zeros(2, w, dtype=d)]).to(DEV)
        out = torch.full((meta.n_rows, H * dv), 9.0, device=DEV)
        ops.gated_delta_scan(cat(qkv, C, dt), H, Hk, dk, dv, cat(high, H * dk + 7, torch.float32), cat(beta, H, torch.float32),
                             a_log.to(DEV), dt_bias.to(DEV), 1e-6, dk ** -0.5, state, meta, out)
        at = 0
        for r, p0, n in step:
            got[r][p0: p0 + n] = out[at: at + n].cpu()
            at += n
    for r in (0, 1):
        x = qkv[r].to(F)
        q, k, v = x[:, :Hk * dk].view(T, Hk, dk), x[:, Hk * dk: 2 * Hk * dk].view(T, Hk, dk), x[:, 2 * Hk * dk:].view(T, H, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        gd = torch.exp(-torch.exp(a_log.to(F))[None, :, None] * plain.softplus(high[r][:, :H * dk].to(F) + dt_bias.to(F)).view(T, H, dk))
        ref = plain.gated_delta(q, k, v, torch.sigmoid(beta[r].to(F)), gd)
        close(got[r].view(T, H, dv), ref, "float32", f"request {r}")
    assert float(state[1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dv,weight,act", [(2, 24, False, "silu"), (4, 16, True, "sigmoid"), (3, 100, True, None), (9, 8, False, "sigmoid")])
def test_head_norm_and_gate(dtype, H, dv, weight, act):
    ops, g, n = cuda_ops(dtype), torch.Generator().manual_seed(dv), 6
    o, gate = torch.randn(n, H * dv, generator=g) * 3, torch.randn(n, H * dv + 11, generator=g)
    w = torch.rand(dv, generator=g) + 0.5 if weight else None
    meta = Meta([(n - 1, 0, 0)], pad=1)
    ops._meta_rows = meta.seq_row
    out = torch.empty(n, H * dv, dtype=DT[dtype], device=DEV)
    ops.head_norm_gate(o.to(DEV), H, dv, w.to(DEV) if weight else None, 1e-5, gate.to(DEV) if act else None, 11, act, out)
    ref = plain.rms(o.to(F).view(n, H, dv), 1e-5)
    if weight:
        ref = ref * w.to(F)
    if act:
        z = gate[:, 11:].to(F).view(n, H, dv)
        ref = ref * (torch.sigmoid(z) if act == "sigmoid" else plain.silu(z))
    close(out[:-1].view(n - 1, H, dv), ref[:-1], dtype)
    assert float(out[-1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,C", [(4, 48), (1, 24), (3, 30), (2, 64)])
def test_convolution_with_silu_across_portions(dtype, taps, C):
    ops, g, dt, T = cuda_ops(dtype), torch.Generator().manual_seed(taps), DT[dtype], 23
    h, w = torch.randn(T, C, generator=g).to(dt), (torch.randn(C, taps, generator=g) * 0.5).to(dt)
    state = torch.zeros(2, taps - 1, C, device=DEV) if taps > 1 else None
    got, at = [], 0
    for n in (1, 1, 2, 1, 7, 11):
        meta = Meta([(n, at, 1)])
        out = torch.empty(n, C, dtype=dt, device=DEV)
        ops.short_conv(h[at: at + n].to(DEV), w.to(DEV), state, meta, out, False, "silu")
        got.append(out.cpu())
        at += n
    close(torch.cat(got), plain.silu(plain.causal_conv(h.to(F), w.to(F))), dtype)


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 2, 1), (6, 2, 3, 2), (5, 1, 5, 1), (4, 4, 1, 1), (12, 3, 4, 3), (64, 6, 8, 4), (7, 3, 1, 1)])
@pytest.mark.parametrize("renorm", [False, True])
def test_router_takes_the_best_experts_of_the_best_groups(E, top, groups, keep, renorm):
    ops, g, n = cuda_ops("float32"), torch.Generator().manual_seed(E * top), 37
    z = torch.randn(n, E + 1, generator=g) * 2
    meta = Meta([(n - 1, 0, 0)], pad=1)
    w = torch.empty(n, top, device=DEV)
    route = ops.route_by_scores(z.to(DEV), E, top, groups, keep, renorm, meta, w)
    choice = ops._scratch_bufs["router choices"][: n * top].view(n, top).cpu()
    for i in range(n - 1):
        chosen, weights = plain.routed_choice(z[i, :E].to(F), top, groups, keep)
        assert choice[i].tolist() == chosen, (i, choice[i].tolist(), chosen)
        ref = torch.stack(weights)
        close(w[i], ref / ref.sum() if renorm else ref, "float32")
    # the sorted pairs: every (row, choice) of a live row once, under its expert
    a_idx, c_idx, tiles, max_tiles, _, _, _, tile = route
    pairs = set()
    for e, first, count in tiles.view(-1, 3).cpu().tolist():
        for s in range(first, first + count):
            row, c = int(a_idx[s]), int(c_idx[s])
            assert c // top == row and int(choice[row, c % top]) == e
            pairs.add(c)
    assert pairs == set(range((n - 1) * top))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,I,E,top,groups,keep,shared,n", [(64, 16, 6, 2, 3, 2, 24, 19), (96, 24, 4, 4, 1, 1, 0, 5), (32, 8, 8, 3, 4, 3, 16, 1),
                                                            (128, 64, 8, 2, 2, 1, 64, 300)])
def test_routed_experts_with_a_shared_expert(dtype, D, I, E, top, groups, keep, shared, n):
    ops, g, dt = cuda_ops(dtype), torch.Generator().manual_seed(D + n), DT[dtype]
    part = RoutedMoE(D, I, E, top, groups, keep, shared, names={"expert": "e{}", "gate": "gate", "up": "up", "down": "down",
                                                                    "shared": "shared", "shared_gate": "sg"})
    w = {k: (torch.randn(p.shape, generator=g) * (1.0 if k == "router" else 0.15)).to(dt) for k, p in part.tensors().items()}
    part.bind({k: v.to(DEV) for k, v in w.items()}, ops)
    meta = Meta([(n, 0, 0)], pad=1)
    h = torch.cat([torch.randn(n, D, generator=g), torch.zeros(1, D)]).to(dt)
    ctx = StepContext(ops, Workspace(torch.device(DEV), n + 1), meta, {}, None)
    out = part.forward(ctx, h.to(DEV))
    ops.check_errors()
    mlp = {"kind": "moe", "router": {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}, "shared": {"ff": shared} if shared else None}
    ref = plain.feed_forward(plain.Weights({"m." + k: v for k, v in w.items()}), "m.", mlp, h[:n].to(F))
    got = out.cpu().to(F)
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert float((got[:n] - ref).abs().max()) <= tol * float(ref.abs().max()), float((got[:n] - ref).abs().max())
    assert float(got[n].abs().max()) == 0.0


def test_weighted_sum():
    ops, g = cuda_ops("float32"), torch.Generator().manual_seed(1)
    ts = [torch.randn(9, 40, generator=g) for _ in range(3)]
    out = torch.empty(9, 40, device=DEV)
    ops.weighted_sum([t.to(DEV) for t in ts], [0.8, 0.5, -2.0], out)
    close(out, 0.8 * ts[0].to(F) + 0.5 * ts[1].to(F) - 2.0 * ts[2].to(F), "float32")


# ------------------------------------------------------------------------------------------------ the model, further
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_token_by_token(dirs, dtype):
    """A short prompt, then hundreds of single tokens: the window passes over decoded tokens and gives pages back, the
    states are carried by every step."""
    d, cfg, w = dirs["mix"]
    model, cache, runner = engine_parts(d, dtype, page=4, pages=24, slots=2, max_len=400)
    toks = tokens_for(cfg, (330,), seed=3)[0]
    got = run_cut(runner, cache, "r", toks, (6,) + (1,) * 400)
    model.ops.check_errors()
    agrees(got, oracle(cfg, w, toks, dtype), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dirs, dtype):
    """Through `LLMEngine` and its scheduler (portions of prompts beside decoding requests, a pool that does not hold
    all requests at once): every generated token is the plain model's choice, or within rounding of it."""
    d, cfg, w = dirs["odd"]
    eng = LLMEngine.from_pretrained(d, dtype=dtype, device=DEV, max_model_len=96, num_blocks=20, block_size=8,
                                    max_num_seqs=3, max_prefill_tokens=16)
    P = tokens_for(cfg, (7, 23, 2, 41, 12), seed=2)
    out = eng.generate(P, SamplingParams(max_tokens=9, ignore_eos=True))
    margin = 1e-3 if dtype == "float32" else 0.15
    for prompt, new in zip(P, out):
        lg = oracle(cfg, w, list(prompt) + new, dtype)
        for i, t in enumerate(new):
            row = lg[len(prompt) - 1 + i]
            assert int(row.argmax()) == t or row.max() - row[t] < margin, (dtype, i, t)


def test_command_line_generates_from_a_preset_with_random_weights(capsys):
    import json
    from fusezap_core_b200.cli import main
    assert main(["generate", "--random", "tiny-gizulorn", "--prompt-lens", "5,40,1", "--max-tokens", "6", "--ignore-eos",
                 "--max-model-len", "128", "--num-blocks", "32", "--max-num-seqs", "2"]) == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.splitlines() if x.startswith("{")]
    assert [o["num_prompt_tokens"] for o in lines] == [5, 40, 1]
    assert all(len(o["token_ids"]) == 6 and o["finish_reason"] == "length" for o in lines)


def _random_config(seed: int) -> dict:
    """A configuration drawn from a seed: odd and even sizes, either layer type in any order, grouped and ungrouped heads,
    partly rotated heads with and without scaled frequencies, windows from a few tokens to longer than the sequence,
    dense feed-forwards, routed ones and none."""
    rng = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    width = int(pick(24, 40, 56, 72, 100))

    def rot(dim):
        dims = int(pick(0, 2, dim // 2 * 2, max(2, dim // 4 * 2)))
        scaling = pick(None, (4.0, 1.0, 4.0, 32), (8.0, 1.0, 2.0, 16))
        return _rot(float(pick(50.0, 10000.0, 1e6)), dims, scaling if dims else None)

    def mlp():
        kind = pick("dense", "moe", "moe", None)
        if kind is None:
            return None
        if kind == "dense":
            return {"kind": "dense", "ff": int(pick(16, 36, 64))}
        groups = int(pick(1, 2, 3))
        per = int(pick(1, 2, 3))
        keep = int(rng.integers(1, groups + 1))
        top = int(rng.integers(1, keep * per + 1))
        return _moe(groups * per, top, int(pick(8, 20, 32)), groups, keep, int(pick(0, 16, 24)))

    layers = []
    for _ in range(int(rng.integers(1, 4))):
        if rng.random() < 0.5:
            H, dk, dv = int(pick(1, 2, 3)), int(pick(6, 8, 16, 20, 36)), int(pick(4, 7, 16, 24))
            m = _ret(H, dk, dv, [float(pick(0.5, 0.9, 0.99, 1.0)) for _ in range(H)], 1.0, 0)
            m["rot"] = rot(dk)
            layers.append({"type": "retention", "mixer": m, "mlp": mlp()})
        else:
            kv = int(pick(1, 2))
            dk, dv = int(pick(8, 12, 16, 40)), int(pick(4, 8, 12, 40))
            left = _left(kv * int(pick(1, 2, 3)), kv, dk, dv, float(pick(0.2, 0.35)), int(pick(3, 7, 16, 200)), int(pick(0, 1, 5, 9)), rot(dk))
            kh = int(pick(1, 2))
            right = _right(kh * int(pick(1, 2)), kh, int(pick(4, 9, 16, 24)), int(pick(3, 8, 20)), int(pick(1, 2, 4, 5)))
            layers.append({"type": "parallel", "mixer": _par(left, right, float(pick(0.5, 1.0)), float(pick(0.25, 1.5))), "mlp": mlp()})
    return {"architecture": "Gizulorn", "vocab": int(pick(37, 64, 150)), "width": width, "norm": {"eps": float(pick(1e-6, 1e-5))},
            "layers": layers}


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Every size and constant comes from the configuration: eight drawn ones, in float32 against the plain model (whole,
    in portions, token by token), and in bfloat16."""
    cfg = _random_config(seed)
    d, cfg, w = make_dir(f"drawn{seed}", tmp_path, cfg, seed)
    toks = tokens_for(cfg, (45,), seed=seed)[0]
    for dtype in ("float32", "bfloat16"):
        model, cache, runner = engine_parts(d, dtype, page=4, pages=30, slots=2, max_len=64)
        ref = oracle(cfg, w, toks, dtype)
        for cuts in ((45,), (1,), (6, 2, 1, 17)):
            got = run_cut(runner, cache, "r", toks, cuts)
            model.ops.check_errors()
            agrees(got, ref, dtype, (seed, dtype, cuts, json_of(cfg)))


def json_of(cfg):
    import json
    return json.dumps(cfg)[:400]

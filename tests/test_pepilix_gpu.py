"""Pepilix on the GPU: every mechanism's kernel alone against the plain function of the same mechanism, then the model
through the step function (portions, single tokens, unequal batches, pages and slots used again) and through the entry
point, in both dtypes, against the plain implementation on whole sequences."""
import numpy as np
import pytest
import torch

import plain_pepilix
from pepilix_util import CONFIGS, LIMIT, make_dir, rel_rms, run_cut, run_mixed, tokens_for
from fusezap_core_b200 import LLMEngine, SamplingParams
from fusezap_core_b200.cache import CacheManager
from fusezap_core_b200.engine import Portion, StepRunner, load_model
from fusezap_core_b200.kernels import cuda_ops
from fusezap_core_b200.parts import LayerCache

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64


class Meta:
    """The step metadata a kernel reads, for one or several portions laid out by the test itself."""
    def __init__(self, portions, tables, pad=0):
        """portions: (rows, first position, state slot) each; tables: int32 (portions, pages per request)."""
        row, pos, seg, at = [], [], [], 0
        for s, (n, p0, slot) in enumerate(portions):
            row += [s] * n
            pos += list(range(p0, p0 + n))
            seg.append((at, n, p0, slot))
            at += n
        row += [-1] * pad
        pos += [0] * pad
        self.seq_row = torch.tensor(row, dtype=torch.int32, device=DEV)
        self.pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
        self.seg = torch.tensor(seg, dtype=torch.int32, device=DEV)
        self.n_segments, self.n_rows = len(portions), at + pad
        self.max_context = max(p0 + n for n, p0, _ in portions)
        self._table = tables.to(DEV)

        class Sg:
            def __init__(s, a): s.row0, s.n, s.pos0, s.state_slot = a
        self.segments = [Sg(a) for a in seg]

    def table(self, group):
        return self._table


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,G", [(96, 3), (320, 2), (64, 8), (1024, 16), (40, 5), (30, 3), (2100, 2), (2048, 2), (4104, 1)])
def test_grouped_norm(dtype, D, G):
    ops, g = cuda_ops(dtype), torch.Generator().manual_seed(D + G)
    x, dl, w = torch.randn(7, D, generator=g) * 3, torch.randn(7, D, generator=g), torch.rand(D, generator=g) + 0.5
    ref = plain_pepilix.grouped_rms_norm((x + dl).to(F), w.to(F), G, 1e-5)
    xd, h = x.to(DEV), torch.empty(7, D, dtype=DT[dtype], device=DEV)
    ops.add_rmsnorm(xd, dl.to(DEV), w.to(DEV), 1e-5, h, groups=G)
    assert torch.equal(xd.cpu(), x + dl)
    tol = 2e-6 if dtype == "float32" else 2.0 ** -8
    assert ((h.cpu().to(F) - ref).abs() <= tol * ref.abs() + 1e-6).all()
    rows = torch.tensor([5, -1, 0], dtype=torch.int32, device=DEV)
    h2 = torch.empty(3, D, dtype=DT[dtype], device=DEV)
    ops.add_rmsnorm(xd, None, w.to(DEV), 1e-5, h2, rows, groups=G)
    assert torch.equal(h2[0], h[5]) and torch.equal(h2[2], h[0]) and float(h2[1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,C", [(2, 64), (4, 320), (5, 96), (16, 40), (3, 30), (1, 24)])
def test_short_conv_carries_its_state_across_portions(dtype, taps, C):
    """A sequence cut into portions (some shorter than taps - 1, down to one token), two requests interleaved and one
    padding row: equal to the convolution of the whole sequence; the state ends as the last taps - 1 inputs."""
    ops, g, dt = cuda_ops(dtype), torch.Generator().manual_seed(taps), DT[dtype]
    T = 50
    h = [(torch.randn(T, C, generator=g)).to(dt) for _ in range(2)]
    w = (torch.randn(C, taps, generator=g) * 0.5).to(dt)
    ref = [h[i].to(F) + plain_pepilix.causal_conv(h[i].to(F), w.to(F)) for i in range(2)]
    state = torch.zeros(3, taps - 1, C, device=DEV) if taps > 1 else None
    if taps > 1:
        state[1] = 7.0      # a slot nobody uses must stay as it is
    got, at = [[], []], [0, 0]
    cuts = [(1, 3), (2, 1), (1, 1), (7, max(1, taps - 1)), (taps, 20), (30, 1), (40, 40)]
    for ca, cb in cuts:
        na, nb = min(ca, T - at[0]), min(cb, T - at[1])
        parts = [(n, at[i], slot) for i, (n, slot) in enumerate(((na, 2), (nb, 0))) if n > 0]
        who = [i for i, n in enumerate((na, nb)) if n > 0]
        if not parts:
            break
        meta = Meta(parts, torch.zeros(len(parts), 1, dtype=torch.int32), pad=1)
        hin = torch.cat([h[i][at[i]: at[i] + n] for i, (n, _, _) in zip(who, parts)] + [torch.ones(1, C, dtype=dt)]).to(DEV)
        out = torch.empty_like(hin)
        ops.short_conv(hin, w.to(DEV), state, meta, out, True)
        k = 0
        for i, (n, _, _) in zip(who, parts):
            got[i].append(out[k: k + n].cpu())
            k, at[i] = k + n, at[i] + n
        assert float(out[k].abs().max()) == 0.0
    for i, slot in ((0, 2), (1, 0)):
        o = torch.cat(got[i]).to(F)
        tol = 1e-5 if dtype == "float32" else 2.0 ** -7
        assert ((o - ref[i]).abs() <= tol * (1 + ref[i].abs())).all()
        if taps > 1:
            assert torch.equal(state[slot].cpu(), h[i][T - (taps - 1):].float())
    if taps > 1:
        assert float((state[1] - 7.0).abs().max()) == 0.0
    ops.check_errors()


def test_gated_sum_and_scale():
    ops, g = cuda_ops("float32"), torch.Generator().manual_seed(1)
    N, D, K = 9, 50, 3
    a, ga, gf = (torch.randn(N, D, generator=g) for _ in range(3))
    f = torch.randn(N * K, D, generator=g)
    out = torch.empty(N, D, device=DEV)
    ops.gated_sum(a.to(DEV), ga.to(DEV), f.to(DEV), gf.to(DEV), out, K, 1.0 / K)
    ref = a.to(F) * torch.sigmoid(ga.to(F)) + f.to(F).view(N, K, D).sum(1) / K * torch.sigmoid(gf.to(F))
    assert (out.cpu().to(F) - ref).abs().max() < 1e-5
    ops.gated_sum(a.to(DEV), ga.to(DEV), None, None, out)
    assert (out.cpu().to(F) - a.to(F) * torch.sigmoid(ga.to(F))).abs().max() < 1e-5
    ops.gated_sum(a.to(DEV), None, f[:N].to(DEV).contiguous(), None, out)
    assert (out.cpu().to(F) - (a + f[:N]).to(F)).abs().max() < 1e-5
    ops.scale_(out, 0.25)
    assert (out.cpu().to(F) - (a + f[:N]).to(F) * 0.25).abs().max() < 1e-5


def _pool(pages, page, width, dtype):
    return torch.zeros(pages, page, width, dtype=DT[dtype], device=DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("L,R,dims", [(40, 8, 8), (128, 32, 32), (16, 6, 4), (72, 32, 0)])
def test_latent_cache_write_norms_rotates_and_lands_on_the_right_page(dtype, L, R, dims):
    from fusezap_core_b200.parts.rope import RotaryEncoding
    ops, g, page = cuda_ops(dtype), torch.Generator().manual_seed(L), 4
    base = 300.0
    pos = RotaryEncoding(max(dims, 2), base, precise=True)
    pos.prepare(64, torch.device(DEV))
    cos, sin = (pos.cos, pos.sin) if dims else (pos.cos[:, :0].contiguous(), pos.sin[:, :0].contiguous())
    tables = torch.tensor([[5, 2, 7, 0, -1, -1], [1, 6, 3, -1, -1, -1]], dtype=torch.int32)
    meta = Meta([(9, 3, -1), (2, 7, -1)], tables, pad=2)       # positions 3..11 of one request, 7..8 of another
    down = torch.randn(13, L + R, generator=g)
    w = torch.rand(L, generator=g) + 0.5
    pool = _pool(8, page, L + R, dtype)
    ops.latent_cache_write(down.to(DEV), w.to(DEV), 1e-5, cos, sin, dims, meta, LayerCache(keys=pool, group=0, page_size=page))
    ops.check_errors()
    seen = torch.zeros(8, page, dtype=torch.bool)
    tol = 3e-6 if dtype == "float32" else 2.0 ** -8
    for i in range(11):
        s, p = int(meta.seq_row[i]), int(meta.pos[i])
        c = down[i, :L].to(F)
        c = c / torch.sqrt((c * c).mean() + 1e-5) * w.to(F)
        kr = plain_pepilix.rotate(down[i: i + 1, L:].to(F), torch.tensor([p]), base, dims)[0] if dims else down[i, L:].to(F)
        ref = torch.cat([c, kr])
        pg = int(tables[s, p // page])
        assert ((pool[pg, p % page].cpu().to(F) - ref).abs() <= tol * (1 + ref.abs())).all(), f"row {i}"
        seen[pg, p % page] = True
    assert float(pool.float().abs().sum(-1).cpu()[~seen].max()) == 0.0      # nothing else was written


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("N,H,dn,dr,r,dims", [(70, 5, 12, 10, 24, 6), (300, 16, 64, 32, 128, 32), (5, 6, 32, 32, 128, 32),
                                              (70, 3, 16, 8, 40, 8)])
def test_rotate_heads_and_products_per_head(dtype, N, H, dn, dr, r, dims):
    from fusezap_core_b200.parts.rope import RotaryEncoding
    ops, g, dt = cuda_ops(dtype), torch.Generator().manual_seed(3), DT[dtype]
    pos = RotaryEncoding(dims, 77.0, precise=True)
    pos.prepare(512, torch.device(DEV))
    meta = Meta([(N - 1, 130, -1)], torch.zeros(1, 1, dtype=torch.int32), pad=1)
    q = torch.randn(N, H, dn + dr, generator=g).to(dt)
    wt = torch.randn(H, r, dn, generator=g).to(dt)
    qa = torch.zeros(N, H, r + dr, dtype=dt, device=DEV)
    ops.rotate_heads(q.to(DEV), dn, pos.cos, pos.sin, dims, meta, qa, r)
    ops.linear_heads(q.to(DEV), 0, dn, wt.to(DEV), qa, 0)
    ref_r = plain_pepilix.rotate(q[:N - 1, :, dn:].to(F), torch.arange(130, 129 + N), 77.0, dims)
    ref_n = torch.einsum("nhk,hmk->nhm", q[:, :, :dn].to(F), wt.to(F))
    tol = 1e-5 if dtype == "float32" else 2.0 ** -7
    got = qa.cpu().to(F)
    assert ((got[:N - 1, :, r:] - ref_r).abs() <= tol * (1 + ref_r.abs())).all()
    assert float(got[N - 1, :, r:].abs().max()) == 0.0
    assert ((got[..., :r] - ref_n).abs() <= tol * (1 + ref_n.abs()) * max(1.0, dn ** 0.5 / 4)).all()
    if dtype == "bfloat16":       # the plain kernel where the tensor-core one had taken the sizes
        ops.grouped_tensor_cores = False
        try:
            qa2 = torch.zeros_like(qa)
            ops.linear_heads(q.to(DEV), 0, dn, wt.to(DEV), qa2, 0)
        finally:
            ops.grouped_tensor_cores = True
        assert ((qa2[..., :r].cpu().to(F) - ref_n).abs() <= tol * (1 + ref_n.abs()) * max(1.0, dn ** 0.5 / 4)).all()


def _attention_reference(q, entries, Wv, scale, lo, p):
    e = entries[lo: p + 1].to(F)
    w = torch.softmax((q.to(F) @ e.T) * scale, -1)
    return w @ e[:, :Wv]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,W,Wv,page", [(6, 160, 128, 16), (40, 22, 16, 4), (1, 104, 72, 8), (3, 48, 40, 64),
                                         (16, 576, 512, 16), (5, 64, 32, 8), (20, 96, 80, 4), (70, 32, 32, 16),
                                         (33, 1000, 500, 16)])
def test_latent_attention_rows_of_any_portion(dtype, H, W, Wv, page):
    """Two requests on shuffled pages: a long portion behind a prefix, single tokens, and a padding row, against the
    plain softmax over each row's own keys."""
    ops, g, dt = cuda_ops(dtype), torch.Generator().manual_seed(H * W), DT[dtype]
    T = [300, 75]
    ent = [(torch.randn(t, W, generator=g)).to(dt) for t in T]
    n_pages = sum(-(-t // page) for t in T) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    pool = _pool(n_pages, page, W, dtype)
    tables = torch.full((2, 80), -1, dtype=torch.int32)
    for i, t in enumerate(T):
        for k in range(-(-t // page)):
            tables[i, k] = pg = perm.pop()
            chunk = ent[i][k * page: (k + 1) * page]
            pool[pg, : chunk.shape[0]] = chunk.to(DEV)
    meta = Meta([(45, 255, -1), (1, 74, -1)], tables, pad=1)
    q = (torch.randn(47, H, W, generator=g) * 0.5).to(dt)
    out = torch.empty(47, H, Wv, dtype=dt, device=DEV)
    ops.latent_attention(q.to(DEV), LayerCache(keys=pool, group=0, page_size=page), meta, out, Wv, 0.3, 0)
    ops.check_errors()
    tol = 2e-5 if dtype == "float32" else 2.0 ** -6
    for i in list(range(0, 45, 7)) + [44, 45]:
        s, p = int(meta.seq_row[i]), int(meta.pos[i])
        ref = _attention_reference(q[i], ent[s], Wv, 0.3, 0, p)
        assert ((out[i].cpu().to(F) - ref).abs() <= tol * (1 + ref.abs())).all(), f"row {i}"
    assert float(out[46].float().abs().max()) == 0.0
    if dtype == "bfloat16":       # the tensor-core kernel without its cut along the keys, and the general kernel: the same
        for knob in ("latent_key_cuts", "latent_tensor_cores"):      # within rounding
            setattr(ops, knob, False)
            try:
                out2 = torch.empty_like(out)
                ops.latent_attention(q.to(DEV), LayerCache(keys=pool, group=0, page_size=page), meta, out2, Wv, 0.3, 0)
            finally:
                setattr(ops, knob, True)
            assert (out2.float() - out.float()).abs().max() <= 2.0 ** -5, knob


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 31, 32, 63, 64, 511, 512, 900])
def test_one_key_that_stands_out_is_found_wherever_it_lies(dtype, far):
    """Among 1,000 random keys one is made to match the query: the output must be that key's values, whether it is the
    first token, lies at a page's border or hundreds of tokens back; in a prompt's portion and for a single token."""
    ops, g, dt = cuda_ops(dtype), torch.Generator().manual_seed(far), DT[dtype]
    H, W, Wv, page, T = 2, 48, 32, 16, 1000
    ent = (torch.randn(T, W, generator=g) * 0.3).to(dt)
    q = (torch.randn(20, H, W, generator=g) * 0.3).to(dt)
    probe = torch.zeros(W)
    probe[Wv + 3] = 6.0                       # a direction outside the value part: the output shows the key's values
    ent[far] += probe.to(dt) * 4
    q += probe.to(dt)
    pool = _pool(64, page, W, dtype)
    pool.view(-1, W)[:T] = ent.to(DEV)
    tables = torch.arange(64, dtype=torch.int32).view(1, 64)
    cache = LayerCache(keys=pool, group=0, page_size=page)
    for meta in (Meta([(20, T - 20, -1)], tables), Meta([(1, T - 1, -1)], tables)):
        n = meta.n_rows
        out = torch.empty(n, H, Wv, dtype=dt, device=DEV)
        ops.latent_attention(q[:n].to(DEV).contiguous(), cache, meta, out, Wv, 1.0, 0)
        assert (out.cpu().float() - ent[far, :Wv].float()).abs().max() < (1e-3 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 5, 16, 33])
def test_window_edges(dtype, window):
    """With a window the key at p - window + 1 counts and the one at p - window does not, for portion rows and single
    tokens alike (shown by a key that would dominate if it were seen)."""
    ops, g, dt = cuda_ops(dtype), torch.Generator().manual_seed(window), DT[dtype]
    H, W, Wv, page, T = 3, 48, 24, 8, 120
    ent = (torch.randn(T, W, generator=g) * 0.3).to(dt)
    probe = torch.zeros(W)
    probe[Wv + 1] = 6.0
    pool = _pool(16, page, W, dtype)
    tables = torch.arange(16, dtype=torch.int32).view(1, 16)
    for inside in (True, False):
        for rows, p0 in ((9, T - 9), (1, T - 1)):
            target = p0 - window + (1 if inside else 0)     # just inside / just outside the window of the first row
            e = ent.clone()
            e[target] += probe.to(dt) * 4
            pool.view(-1, W)[:T] = e.to(DEV)
            q = (torch.randn(rows, H, W, generator=g) * 0.3 + probe).to(dt)
            out = torch.empty(rows, H, Wv, dtype=dt, device=DEV)
            ops.latent_attention(q.to(DEV), LayerCache(keys=pool, group=0, page_size=page), Meta([(rows, p0, -1)], tables), out,
                                 Wv, 1.0, window)
            ref = _attention_reference(q[0], e, Wv, 1.0, max(0, p0 - window + 1), p0)
            assert (out[0].cpu().to(F) - ref).abs().max() < (1e-4 if dtype == "float32" else 3e-2)
            hit = (out[0].cpu().float() - e[target, :Wv].float()).abs().max() < 3e-2
            assert bool(hit) == inside, f"window {window}, inside {inside}, {rows} rows"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tensor_cores", [True, False])
@pytest.mark.parametrize("E,top,K,I,D,N", [(5, 1, 96, 24, 96, 150), (4, 3, 64, 40, 72, 150), (7, 7, 32, 8, 32, 150),
                                           (12, 2, 320, 96, 320, 150), (12, 2, 320, 96, 320, 7), (32, 4, 256, 128, 264, 40),
                                           (3, 2, 20, 6, 10, 33), (2, 2, 64, 32, 64, 400), (3, 1, 128, 64, 128, 900)])
def test_table_routed_experts(dtype, E, top, K, I, D, N, tensor_cores):
    """Rows sorted by expert on the device, each expert over its own rows, summed per row: against the plain loop. The
    inputs are scaled so that both clamps and the unclamped range occur."""
    ops, g, dt = cuda_ops(dtype), torch.Generator().manual_seed(E * top), DT[dtype]
    if dtype == "float32" and not tensor_cores:
        pytest.skip("the float32 path has the plain kernels only")
    ops.grouped_tensor_cores = tensor_cores
    ops.grouped_tiles_128 = N >= 400        # the large row tiles are an option of the table: exercised here
    V, limit = 31, 0.8
    h = torch.randn(N, K, generator=g).to(dt)
    wgu = (torch.randn(E, 2 * I, K, generator=g) * 0.12).to(dt)
    wd = (torch.randn(E, D, I, generator=g) * 0.2).to(dt)
    table = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32)
    tok = torch.randint(0, V, (N,), generator=g).to(torch.int32)
    k2 = (N - 1) // 3
    meta = Meta([(N - 1 - k2, 0, -1), (k2, 5, -1)], torch.zeros(2, 1, dtype=torch.int32), pad=1)
    import math
    route = ops.route_by_table(tok.to(DEV), meta, table.to(DEV), E, math.gcd(D, I))
    y = torch.empty(N * top, I, dtype=dt, device=DEV)
    ops.grouped_linear_glu(h.to(DEV), wgu.to(DEV), route, y, 1.702, limit)
    terms = torch.full((N * top, D), float("nan"), device=DEV)
    ops.grouped_linear_scatter(y, wd.to(DEV), route, terms)
    ops.grouped_tensor_cores, ops.grouped_tiles_128 = True, False
    ops.check_errors()
    rnd = (lambda t: t) if dtype == "float32" else (lambda t: t.to(torch.bfloat16).to(F))
    tol = 2e-5 if dtype == "float32" else 2.0 ** -6
    tol *= max(1.0, (max(K, I) / 64) ** 0.5)
    for n in range(N - 1):
        for k in range(top):
            e = int(table[tok[n], k])
            ref = plain_pepilix.expert(h[n].to(F), wgu[e, :I].to(F), wgu[e, I:].to(F), wd[e].to(F), limit, rnd)
            assert ((terms[n * top + k].cpu().to(F) - ref).abs() <= tol * (1 + ref.abs())).all(), f"row {n}, choice {k}"
    assert float(terms[(N - 1) * top:].abs().max()) == 0.0       # the padding row's terms


# ------------------------------------------------------------------------------------------------ the model
@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("pepilix")
    return {name: make_dir(name, tmp) for name in CONFIGS}


def engine_parts(d, dtype, page=16, pages=24, slots=3, max_len=384):
    model = load_model(d, dtype, DEV, max_len=max_len)
    cache = CacheManager(model.cache_needs(), model.state_needs(), page, pages, slots, max_len, model.ops.dtype, model.device)
    return model, cache, StepRunner(model, cache, max_rows=max_len, max_wanted=max_len, max_segments=slots)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_single_tokens_equal_whole_sequences(dirs, name, dtype):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, dtype)
    for toks in tokens_for(cfg, (1, 2, 45, 200), seed=5):
        ref = plain_pepilix.forward(cfg, w, toks, rounded=dtype == "bfloat16").numpy()
        for cuts in ([len(toks)], [1], [2], [max(1, len(toks) - 40), 1], [5, 1, 3, 2, 64, 1, 1, 17]):
            if len(toks) > 100 and cuts in ([1], [2]):
                continue
            got = run_cut(runner, cache, "r", toks, cuts)
            assert rel_rms(got, ref) < LIMIT[dtype], f"{name}, {len(toks)} tokens in portions {cuts}"
    model.ops.check_errors()
    cache.check()
    assert cache.states.num_free == 3 and cache.num_free_pages == 24


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "wide"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(dirs, name, dtype):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, dtype, page=8, pages=26, slots=3)
    toks = dict(zip("abcde", tokens_for(cfg, (70, 9, 120, 23, 150), seed=8)))
    ref = {r: plain_pepilix.forward(cfg, w, t, rounded=dtype == "bfloat16").numpy() for r, t in toks.items()}
    plan = [[("a", 7), ("b", 2)], [("a", 1), ("b", 1), ("c", 64)], [("b", 6), ("c", 2), ("a", 40)], [("a", 1), ("c", 1)],
            [("c", 53), ("a", 21)],          # a and c end here: their pages and slots go back
            [("d", 5), ("e", 100)], [("d", 1), ("e", 1)], [("e", 49), ("d", 17)]]
    got = run_mixed(runner, cache, toks, plan)
    for r in toks:
        assert got[r].shape == ref[r].shape
        assert rel_rms(got[r], ref[r]) < LIMIT[dtype], f"{name}, request {r}"
    model.ops.check_errors()
    cache.check()
    assert cache.states.num_free == 3 and cache.num_free_pages == 26


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_one_token_at_a_time(dirs, dtype):
    d, cfg, w = dirs["taps"]
    model, cache, runner = engine_parts(d, dtype, page=16, pages=24, slots=2)
    toks = tokens_for(cfg, (330,), seed=12)[0]
    ref = plain_pepilix.forward(cfg, w, toks, rounded=dtype == "bfloat16").numpy()
    got = run_cut(runner, cache, "r", toks, [10] + [1] * 320)
    assert rel_rms(got, ref) < LIMIT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point_and_scheduler(dirs, dtype):
    d, cfg, w = dirs["small"]
    eng = LLMEngine.from_pretrained(d, dtype=dtype, device=DEV, max_model_len=128, num_blocks=20, block_size=8,
                                    max_num_seqs=3, max_prefill_tokens=16)
    prompts = tokens_for(cfg, (3, 29, 12, 1, 40), seed=2)
    out = eng.generate(prompts, SamplingParams(max_tokens=9, ignore_eos=True))
    for prompt, new in zip(prompts, out):
        lg = plain_pepilix.forward(cfg, w, list(prompt) + new, rounded=dtype == "bfloat16").numpy()
        scale = np.abs(lg).max()
        for i, t in enumerate(new):
            row = lg[len(prompt) - 1 + i]
            assert row.max() - row[t] <= (1e-4 if dtype == "float32" else 4e-2) * scale
    model_ops = eng.model.ops
    model_ops.check_errors()
    assert eng.cache.states.num_free == 3 and eng.cache.num_free_pages == 20


def test_command_line_generates_from_a_preset_with_random_weights(capsys):
    import json
    from fusezap_core_b200.cli import main
    assert main(["generate", "--random", "tiny-pepilix", "--prompt-lens", "5,40,1", "--max-tokens", "6", "--ignore-eos",
                 "--max-model-len", "128", "--num-blocks", "32", "--max-num-seqs", "2"]) == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.splitlines() if x.startswith("{")]
    assert [o["num_prompt_tokens"] for o in lines] == [5, 40, 1]
    assert all(len(o["token_ids"]) == 6 and o["finish_reason"] == "length" for o in lines)


def _random_config(seed: int) -> dict:
    """A configuration drawn from a seed: odd and even sizes, any order of layers that own or borrow a cache, layers
    without feed-forward, one to several norm groups and taps."""
    rng = np.random.default_rng(seed)
    groups = int(rng.choice([1, 2, 3, 5]))
    width = groups * int(rng.integers(5, 40))
    taps = int(rng.integers(1, 7))
    vocab = int(rng.integers(20, 300))
    kinds = []
    for _ in range(int(rng.integers(1, 3))):      # one or two kinds of mixer sizes; layers borrow only from their own kind
        rot = 2 * int(rng.integers(1, 9))
        kinds.append(dict(heads=int(rng.integers(1, 10)), dim=int(rng.integers(1, 40)), rot_dim=rot + int(rng.choice([0, 0, 3])),
                          vdim=int(rng.integers(1, 40)), kv_rank=int(rng.integers(3, 70)), scale=float(rng.uniform(0.05, 0.4)),
                          rot={"base": float(rng.choice([100.0, 10000.0, 500000.0])), "dims": rot}))
    layers, owners = [], {}
    for i in range(int(rng.integers(1, 6))):
        k = int(rng.integers(0, len(kinds)))
        m = dict(kinds[k])
        m["heads"], m["dim"], m["vdim"] = int(rng.integers(1, 10)), int(rng.integers(1, 40)), int(rng.integers(1, 40))
        if k in owners and rng.random() < 0.5:
            m["kv_from"] = int(rng.choice(owners[k]))
        else:
            owners.setdefault(k, []).append(i)
        mlp = None
        if rng.random() < 0.8:
            experts = int(rng.integers(1, 9))
            mlp = {"kind": "moe", "router": {"experts": experts, "top": int(rng.integers(1, experts + 1))},
                   "expert": {"ff": int(rng.integers(1, 50)), "limit": float(rng.uniform(0.3, 3.0))}}
        layers.append({"type": "latent_attention", "mixer": m, "mlp": mlp})
    return {"architecture": "Pepilix", "vocab": vocab, "width": width, "embedding": {"scale": float(rng.uniform(0.5, 20))},
            "logit_scale": float(rng.uniform(0.2, 2.0)), "norm": {"eps": float(rng.choice([1e-6, 1e-5, 1e-3])), "groups": groups},
            "canon": {"taps": taps}, "layers": layers}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    """Whatever sizes a configuration gives (odd ones included, which take the general kernels), portions and single
    tokens through the engine equal the plain model on the whole sequence."""
    from fusezap_core_b200.weights import write_random_model
    from safetensors.torch import load_file
    import os
    cfg = _random_config(seed)
    d = write_random_model(cfg, str(tmp_path / "m"), 100 + seed, "float32", norm_noise=True, std_scale=4.0)
    w = load_file(os.path.join(d, "model.safetensors"))
    model, cache, runner = engine_parts(d, dtype, page=16, pages=12, slots=2, max_len=192)
    toks = tokens_for(cfg, (150,), seed=seed)[0]
    ref = plain_pepilix.forward(cfg, w, toks, rounded=dtype == "bfloat16").numpy()
    for cuts in ([150], [9, 1, 2, 33, 1, 1, 64]):
        got = run_cut(runner, cache, "r", toks, cuts)
        assert rel_rms(got, ref) < LIMIT[dtype], f"seed {seed}: {cfg}"
    model.ops.check_errors()

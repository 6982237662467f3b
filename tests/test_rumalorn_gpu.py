"""Rumalorn on the GPU: each new kernel against its plain statement, and the engine (32-bit and
bfloat16) against the plain model under every way of cutting and batching the work."""

import math

import pytest
import torch

import kernel_refs as ref
from freetoken_b200.engine.engine import StepEntry
from helpers import make_engine, mixed_schedule, model_folder, replay_cuts, replay_mixed, replay_whole, tokens_for
from plain.rumalorn_plain import PlainRumalorn, dynamic_tanh
from tiny_rumalorn import ALL, RUMA_1

from freetoken_b200.engine.attention_plan import build_plan
from freetoken_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
PAGE = {"R1": 4, "R2": 8, "R3": 4, "R4": 16, "R5": 16, "R6": 8, "R7": 4}


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def row_error(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: root mean square over the vocabulary of the difference (its mean taken off, a shift of
    all logits changes nothing), in units of the spread of the wanted logits."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.double().std()


F32_ROW, BF16_ROW = 1e-4, 5e-2


def assert_rows(got, want, dtype, what=""):
    e = row_error(got.cpu(), want)
    bound = F32_ROW if dtype == "float32" else BF16_ROW
    assert torch.isfinite(got).all() and float(e.max()) < bound, f"{what}: worst row {float(e.max()):.3g} at {int(e.argmax())}"


# --------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,T,k", [(64, 9, 2), (100, 5, 3), (7, 3, 1), (3072, 4, 4)])
def test_stream_add_norm(dtype, H, T, k):
    res = rnd(T, H, seed=1)
    x1, x2 = rnd(T, H, dtype=dtype, seed=2), rnd(T, H, dtype=dtype, seed=3)
    y = rnd(T * k, H, dtype=dtype, seed=4)
    pos = torch.randperm(T * k, generator=torch.Generator().manual_seed(5)).to(torch.int32).to(DEV)
    table, ids = rnd(11, H, dtype=dtype, seed=6), torch.randint(0, 11, (T,), generator=torch.Generator().manual_seed(7)).to(torch.int32).to(DEV)
    vec = rnd(H, seed=8)
    w, b, alpha = rnd(H, seed=9) + 1, rnd(H, seed=10), torch.tensor([0.6], device=DEV)
    norm = ("dynamic_tanh", w, b, alpha)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    for kw in (dict(x1=x1), dict(x1=x1, x2=x2), dict(routed=(y, pos, k)), dict(table=table, ids=ids, vec=vec),
               dict(x1=x1, x2=x2, routed=(y, pos, k), table=table, ids=ids, vec=vec), dict()):
        r_got, r_want = res.clone(), res.clone()
        out, want = torch.empty(T, H, dtype=dtype, device=DEV), torch.empty(T, H, dtype=dtype, device=DEV)
        ops.stream_add_norm(r_got, out, norm=norm, **kw)
        ref.stream_add_norm(r_want, want, norm=norm, **kw)
        torch.testing.assert_close(r_got, r_want, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(out.float(), want.float(), **tol)
        # the plain model's own statement of the norm, on the kernel's own sum
        torch.testing.assert_close(out.float(), dynamic_tanh(r_got, w, b, alpha).float(), **tol)
    # chosen rows only: the stream stays as it is
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    r_got = res.clone()
    out = torch.empty(2, H, dtype=dtype, device=DEV)
    ops.stream_add_norm(r_got, out, x1=x1, x2=x2, table=table, ids=ids, norm=norm, rows=rows)
    assert torch.equal(r_got, res)
    z = (res + x1.float() + x2.float() + table[ids.long()].float())[rows.long()]
    torch.testing.assert_close(out.float(), dynamic_tanh(z, w, b, alpha), **tol)
    # no norm, no out: the addends are folded into the stream
    r_got = res.clone()
    ops.stream_add_norm(r_got, None, x1=x1, vec=vec)
    torch.testing.assert_close(r_got, res + x1.float() + vec, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,Dp,P,extra", [(4, 2, 16, 16, 4, 4), (6, 6, 24, 32, 8, 6), (8, 1, 40, 48, 4, 0), (8, 2, 64, 64, 16, 8),
                                                 (3, 1, 128, 128, 16, 3)])
def test_head_store_with_bias_position_factor_and_padding(dtype, Hq, Hkv, D, Dp, P, extra):
    T = 37
    x = rnd(T, (Hq + Hkv) * D + extra, dtype=dtype, seed=1)
    qb, kb = rnd(Hq * D, seed=2), rnd(Hkv * D, seed=3)
    factors = 1 + torch.rand(50, generator=torch.Generator().manual_seed(4)).to(DEV)
    positions = torch.randint(0, 60, (T,), generator=torch.Generator().manual_seed(5)).to(torch.int32).to(DEV)  # some beyond the table
    n_pages = 12
    slots = torch.randperm(n_pages * P, generator=torch.Generator().manual_seed(6))[:T].to(torch.int32).to(DEV)
    slots[3] = -1
    outs = []
    for fn in (ops.norm_rope_store, ref.norm_rope_store):
        q = torch.zeros(T, Hq, Dp, dtype=dtype, device=DEV)
        slab = torch.full((n_pages, Hkv, P, Dp), 7.0, dtype=dtype, device=DEV)
        fn(x, D, 0, positions, None, 0.0, False, [
            dict(first_head=0, n_heads=Hq, norm_weight=None, rotate=False, dense_out=q, dst_head_dim=Dp, bias=qb, pos_scale=factors),
            dict(first_head=Hq, n_heads=Hkv, norm_weight=None, rotate=False, slab=slab, slot_map=slots, dst_head_dim=Dp, bias=kb)])
        outs.append((q, slab))
    tol = dict(rtol=1e-6, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(outs[0][0].float(), outs[1][0].float(), **tol)
    torch.testing.assert_close(outs[0][1].float(), outs[1][1].float(), **tol)
    assert float(outs[0][0][..., D:].abs().sum()) == 0  # the padding is zeros
    want_q = (x[:, : Hq * D].float() + qb).view(T, Hq, D) * factors[positions.long().clamp(max=49)][:, None, None]
    torch.testing.assert_close(outs[0][0][..., :D].float(), want_q, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_gate_table_route_and_scale(dtype):
    T, H, D = 13, 6, 24
    wide = rnd(T, 50 + H, dtype=dtype, seed=1)
    o = rnd(T, H, D, dtype=dtype, seed=2)
    want = o.float() * torch.sigmoid(wide[:, 50:].float())[:, :, None]
    ops.head_gate(o, wide[:, 50:])
    torch.testing.assert_close(o.float(), want, **(dict(rtol=1e-6, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)))
    table = torch.tensor([[2, 0], [1, 3], [4, 1], [0, 4]], dtype=torch.int32, device=DEV)
    toks = torch.tensor([3, 0, 0, 2, 1], dtype=torch.int32, device=DEV)
    ids = torch.empty(5, 2, dtype=torch.int32, device=DEV)
    wts = torch.empty(5, 2, dtype=torch.float32, device=DEV)
    ops.table_route(toks, table, 5, ids, wts)
    assert ids.tolist() == [[0, 4], [2, 0], [2, 0], [4, 1], [1, 3]] and wts.unique().tolist() == [0.5]
    x = rnd(5, 77, seed=3)
    want = x * 0.3
    ops.scale_(x, 0.3)
    torch.testing.assert_close(x, want)


def attention_problem(dtype, Hq, Hkv, D, P, segs, seed=0, scale_k=1.0):
    """A shuffled page layout with NaN in every unwritten slot; the values are the keys."""
    width = max(-(-kv // P) for _, kv in segs) + 1
    n_pages = sum(-(-kv // P) for _, kv in segs) + 3
    g = torch.Generator().manual_seed(seed)
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    bt = torch.zeros(len(segs) + 1, width, dtype=torch.int32)
    ks = torch.full((n_pages, Hkv, P, D), float("nan"), dtype=dtype)
    seg_info, q_start = [], 0
    for (q_len, kv_len), row in zip(segs, range(len(segs), 0, -1)):
        for b in range(-(-kv_len // P)):
            page = perm.pop()
            bt[row, b] = page
            n = min(P, kv_len - b * P)
            ks[page, :, :n] = (torch.randn(Hkv, n, D, generator=g) * scale_k).to(dtype)
        seg_info.append([q_start, q_len, kv_len, row])
        q_start += q_len
    q = torch.randn(q_start, Hq, D, generator=g).to(dtype).to(DEV)
    return q, ks.to(DEV), bt.to(DEV), torch.tensor(seg_info, dtype=torch.int32, device=DEV)


def run_biased(dtype, Hq, Hkv, D, P, segs, dist_bias, tile, fixed_splits=None, force_split=False, q=None, problem=None,
               few_rows=False, kv_split=1):
    qq, ks, bt, seg = problem or attention_problem(dtype, Hq, Hkv, D, P, segs)
    q = qq if q is None else q
    kw = dict(sm_count=4096, min_split_keys=32) if force_split else dict(sm_count=148)
    if tile == 128 or few_rows:
        kw["key_tile"] = 128  # as the engine plans the tcgen05 kernels' work
    Hv = Hkv * kv_split  # the kernel takes every KV head as kv_split heads of the same keys
    plan = build_plan(segs, Hq // Hv, tile, None, Hv, fixed_splits=fixed_splits, **kw)
    items = torch.from_numpy(plan.items).to(DEV)
    part_o = part_ml = None
    if plan.n_slots:
        part_o = torch.full((plan.n_slots, Hv, tile, D), float("nan"), dtype=torch.float32, device=DEV)
        part_ml = torch.full((plan.n_slots, Hv, tile, 2), float("nan"), dtype=torch.float32, device=DEV)
    out = torch.full(q.shape, float("nan"), dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    scale = 0.8 * D ** -0.5
    ops.paged_attention(q, ks, ks, bt, seg, len(segs), items, plan.n_items, part_o, part_ml, out, tile, scale, None,
                        dist_bias=dist_bias, few_rows=few_rows, kv_split=kv_split)
    ref.paged_attention(q, ks, ks, bt, seg, len(segs), items, plan.n_items, None, None, want, tile, scale, None,
                        dist_bias=dist_bias)
    return out, want, plan


def attn_tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,P,L", [(4, 2, 16, 4, 13), (6, 6, 32, 8, 40), (8, 1, 48, 4, 5), (12, 2, 128, 16, 200), (10, 2, 96, 16, 1)])
def test_attention_with_distance_bias_and_keys_as_values(dtype, Hq, Hkv, D, P, L):
    bias = rnd(Hq, L, seed=3, scale=1.5)
    segs = [(1, 1), (5, 5), (70, 70), (2, 131), (1, 64), (33, 97), (1, 300)]
    tile = 64 if dtype == torch.bfloat16 else 16
    out, want, _ = run_biased(dtype, Hq, Hkv, D, P, segs, bias, tile)
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    # steps of single tokens (tiles of 16 rows in bfloat16), whole and cut along the keys
    dec = [(1, 1), (1, 17), (1, 64), (1, 65), (1, 333), (1, 128)]
    for fixed in (None, 1, 5):
        out, want, plan = run_biased(dtype, Hq, Hkv, D, P, dec, bias, 16, fixed_splits=fixed)
        torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    out, want, plan = run_biased(dtype, Hq, Hkv, D, P, segs, bias, tile, force_split=True)
    assert plan.n_slots > 0
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,split", [(40, 1, 16, 4), (48, 2, 32, 2), (160, 2, 16, 5)])
def test_more_query_heads_per_kv_head_than_a_tile_has_rows(dtype, Hq, Hkv, D, split):
    bias = rnd(Hq, 9, seed=3)
    tile = 64 if dtype == torch.bfloat16 else 16
    for segs, t, fixed, force in (([(1, 1), (30, 30), (2, 131), (33, 97)], tile, None, False), ([(1, 300), (1, 17)], 16, 3, False),
                                  ([(20, 400)], tile, None, True)):
        if t == 16 and dtype == torch.bfloat16 and Hq // Hkv // split > 16:
            t = 64
        out, want, plan = run_biased(dtype, Hq, Hkv, D, 8, segs, bias, t, fixed_splits=fixed, force_split=force, kv_split=split)
        torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))


@pytest.mark.parametrize("Hq,Hkv,P,L", [(12, 2, 16, 200), (4, 4, 32, 7), (16, 1, 16, 130), (6, 2, 64, 1)])
def test_attention_with_distance_bias_on_the_tensor_core_kernel(Hq, Hkv, P, L):
    bias = rnd(Hq, L, seed=3, scale=1.5)
    for segs, force in (([(300, 300)], False), ([(128, 128), (1, 40), (200, 517), (3, 3)], False), ([(256, 900)], True)):
        out, want, plan = run_biased(torch.bfloat16, Hq, Hkv, 128, P, segs, bias, 128, force_split=force)
        assert ops.variant_counts().get("attention: tcgen05, 128-row query tiles, bias by distance", 0) > 0
        assert not force or plan.n_slots > 0
        torch.testing.assert_close(out.float(), want.float(), **attn_tol(torch.bfloat16))
    assert ops.read_status() == 0
    if Hq // Hkv <= 16:  # steps of single tokens on the same kernel in its form for tiles of at most 16 rows
        dec = [(1, 1), (1, 130), (1, 128), (1, 129), (1, 1000), (1, 257), (1, L + 127), (1, L + 128), (1, L + 129)]
        for fixed in (None, 1, 4, 16):
            out, want, plan = run_biased(torch.bfloat16, Hq, Hkv, 128, P, dec, bias, 16, fixed_splits=fixed, few_rows=True)
            assert ops.variant_counts().get("attention: tcgen05, tiles of at most 16 rows, bias by distance", 0) > 0
            torch.testing.assert_close(out.float(), want.float(), **attn_tol(torch.bfloat16))
        assert ops.read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tile", [16, 64, 128, "few"])
def test_a_bias_that_singles_out_one_distance_picks_that_key(dtype, tile):
    """With queries of zero the scores are the bias alone: +60 at one distance makes the output that key
    (the values are the keys), so a table read one entry off, or clamped one entry early, shows at once."""
    if dtype == torch.float32 and tile != 16:
        pytest.skip("the 32-bit kernel has 16-row tiles")
    few = tile == "few"  # the tcgen05 kernel's form for tiles of at most 16 rows
    tile = 16 if few else tile
    Hq, Hkv, D, P, L = (4, 2, 32, 8, 24) if tile != 128 and not few else (4, 2, 128, 16, 24)
    segs = [(40, 100), (1, 90)] if tile == 64 else [(1, 100), (1, 90)] if tile == 16 else [(150, 400), (130, 390)]
    problem = attention_problem(dtype, Hq, Hkv, D, P, segs, seed=2)
    q, ks, bt, seg = problem
    for d_star in (0, 1, 7, 8, L - 2):
        bias = torch.zeros(Hq, L, device=DEV)
        bias[:, d_star] = 60.0
        out, want, _ = run_biased(dtype, Hq, Hkv, D, P, segs, bias, tile, q=torch.zeros_like(q), problem=problem, few_rows=few)
        torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
        for q_start, q_len, kv_len, row in seg.tolist():
            i = kv_len - 1  # the segment's last query
            j = i - d_star
            key = ks[int(bt[row, j // P]), :, j % P].float()  # [Hkv, D]
            got = out[q_start + q_len - 1].float().view(Hkv, Hq // Hkv, D)
            torch.testing.assert_close(got, key[:, None, :].expand_as(got), **attn_tol(dtype))
    # the last entry stands for every distance from L - 1 on: the output is the mean of all those keys
    bias = torch.zeros(Hq, L, device=DEV)
    bias[:, L - 1] = 60.0
    out, want, _ = run_biased(dtype, Hq, Hkv, D, P, segs, bias, tile, q=torch.zeros_like(q), problem=problem, few_rows=few)
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    q_start, q_len, kv_len, row = seg.tolist()[1]
    far = torch.stack([ks[int(bt[row, j // P]), :, j % P].float() for j in range(0, kv_len - 1 - (L - 1) + 1)]).mean(0)
    got = out[q_start + q_len - 1].float().view(Hkv, Hq // Hkv, D)
    torch.testing.assert_close(got, far[:, None, :].expand_as(got), **attn_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_that_matches_the_query_stands_out(dtype):
    Hq, Hkv, D, P = 4, 2, 32, 16
    segs = [(1, 700), (50, 650)]
    tile_list = [16] if dtype == torch.float32 else [16, 64]
    for tile in tile_list:
        use = segs if tile == 64 else [(1, 700), (1, 650)]
        problem = attention_problem(dtype, Hq, Hkv, D, P, use, seed=4, scale_k=0.3)
        q, ks, bt, seg = problem
        bias = rnd(Hq, 30, seed=1, scale=0.5)
        # key 5 of every request points where its last query points, twenty times as long
        for q_start, q_len, kv_len, row in seg.tolist():
            last = q[q_start + q_len - 1].float().view(Hkv, Hq // Hkv, D)[:, 0]
            ks[int(bt[row, 5 // P]), :, 5 % P] = (20.0 * last / last.norm(dim=-1, keepdim=True)).to(dtype)
        q = q.clone()
        for q_start, q_len, kv_len, row in seg.tolist():  # all heads of a group ask the same
            v = q[q_start + q_len - 1].view(Hkv, Hq // Hkv, D)
            v[:] = v[:, :1] * 3
        for force in (False, True):
            out, want, _ = run_biased(dtype, Hq, Hkv, D, P, use, bias, tile, force_split=force, q=q, problem=problem)
            torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
            for q_start, q_len, kv_len, row in seg.tolist():
                got = out[q_start + q_len - 1].float().view(Hkv, Hq // Hkv, D)
                key = ks[int(bt[row, 0]), :, 5].float()
                assert float((got - key[:, None, :]).abs().max()) < 0.2 * float(key.abs().max())


# --------------------------------------------------------------------------- the engine against the plain model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["R1", "R2", "R3", "R4", "R5", "R6", "R7"])
def test_cuts_and_batches_agree_with_the_plain_model(name, dtype, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainRumalorn(folder)
    eng = make_engine(folder, dtype, DEV, PAGE[name], pages=60)
    toks = tokens_for(plain.vocab, 90, 11)
    want = plain.logits(toks)
    assert_rows(replay_whole(eng, "w", toks), want, dtype, "whole")
    assert_rows(replay_cuts(eng, "d", toks, [58]), want, dtype, "last 32 one by one")
    assert_rows(replay_cuts(eng, "c", toks, [7, 2, 13, 2, 5, 3, 2, 11, 2, 17, 2]), want, dtype, "portions")
    assert_rows(replay_cuts(eng, "t", toks[:40], []), want[:40], dtype, "token by token from the first")
    eng.cache.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["R1", "R4"])
def test_mixed_steps_with_few_pages(name, dtype, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainRumalorn(folder)
    lengths = {"r0": 45, "r1": 60, "r2": 38, "r3": 52, "r4": 41, "r5": 47, "r6": 1, "r7": 2}
    seqs = {r: tokens_for(plain.vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    P = PAGE[name]
    eng = make_engine(folder, dtype, DEV, P, pages=4 * (-(-64 // P)))
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=3))
    alone = make_engine(folder, dtype, DEV, P, pages=40)
    for r, toks in seqs.items():
        assert_rows(got[r], plain.logits(toks), dtype, f"{r} in a batch")
        # beside others or alone: the same up to rounding
        e = row_error(got[r], replay_whole(alone, r, toks).double())
        assert float(e.max()) < (2e-5 if dtype == "float32" else BF16_ROW), r
    pool = eng.cache.paged[0].pool
    assert pool.handed_out > pool.num_pages, "the trace was meant to use pages again"
    assert pool.free_count == pool.num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_and_long_decoding(dtype, tmp_path_factory):
    """Keys far beyond the bias table's last distance, across many pages; then a hundred tokens one by one."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "R1", RUMA_1)
    plain = PlainRumalorn(folder)
    toks = tokens_for(plain.vocab, 420, 3)
    want = plain.logits(toks)
    eng = make_engine(folder, dtype, DEV, 16, pages=64, max_step=512)
    assert_rows(replay_whole(eng, "w", toks), want, dtype, "whole")
    assert_rows(replay_cuts(eng, "d", toks, [320]), want, dtype, "a hundred tokens one by one")
    assert_rows(replay_cuts(eng, "c", toks, [63, 2, 64, 65, 127, 2, 33] + [1] * 20 + [30, 2]), want, dtype, "portions")


def test_long_steps_of_heads_of_128_run_the_tensor_core_attention(tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), "R5", ALL["R5"])
    plain = PlainRumalorn(folder)
    toks = tokens_for(plain.vocab, 450, 9)
    want = plain.logits(toks)
    eng = make_engine(folder, "bfloat16", DEV, 16, pages=96, max_step=512)
    ops.variant_counts(reset=True)
    assert_rows(replay_whole(eng, "w", toks), want, "bfloat16", "whole")
    assert ops.variant_counts().get("attention: tcgen05, 128-row query tiles, bias by distance", 0) == 3
    assert_rows(replay_cuts(eng, "c", toks, [200, 130, 2, 100]), want, "bfloat16", "portions, the rest one by one")
    assert ops.variant_counts().get("attention: tcgen05, tiles of at most 16 rows, bias by distance", 0) > 0
    others = {f"o{i}": tokens_for(plain.vocab, 20 + i, 20 + i) for i in range(3)}
    for r, t in others.items():  # three requests that decode beside a long portion
        eng.step([StepEntry(r, t[:-1], [])])
    out = eng.step([StepEntry("long", toks[:300], list(range(300)))] + [StepEntry(r, t[-1:], [0]) for r, t in others.items()])
    assert_rows(out.logits[:300], want[:300], "bfloat16", "a long portion beside single tokens")
    for i, (r, t) in enumerate(others.items()):
        assert_rows(out.logits[300 + i:301 + i], plain.logits(t)[-1:], "bfloat16", r)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_step_after_recorded_decode_steps_of_layers_that_differ_in_size(dtype, tmp_path_factory):
    """Decode steps are replayed from CUDA graphs that hold the addresses of the work buffers; a later step that
    is long enough to need the larger of two layers' buffers must not move what the graphs point to."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "R4", ALL["R4"])
    plain = PlainRumalorn(folder)
    a, b = tokens_for(plain.vocab, 40, 1), tokens_for(plain.vocab, 230, 2)
    eng = make_engine(folder, dtype, DEV, 16, pages=40, max_step=256)
    got = [eng.step([StepEntry("a", a[:3], [0, 1, 2])]).logits.float().cpu().clone()]
    for i in range(3, 12):  # recorded at the first of these, replayed afterwards
        got.append(eng.step([StepEntry("a", a[i:i + 1], [0])]).logits.float().cpu().clone())
    long = eng.step([StepEntry("b", b, list(range(len(b))))]).logits.float().cpu().clone()
    for i in range(12, 40):
        got.append(eng.step([StepEntry("a", a[i:i + 1], [0])]).logits.float().cpu().clone())
    assert_rows(long, plain.logits(b), dtype, "the long step")
    assert_rows(torch.cat(got), plain.logits(a), dtype, "decode steps before and after it")
    assert eng.graphs, "the decode steps were meant to be replayed from graphs"


def test_greedy_generation_through_the_scheduler(tmp_path_factory):
    from freetoken_b200 import LLM, SamplingParams

    folder = model_folder(tmp_path_factory.getbasetemp(), "R1", RUMA_1)
    plain = PlainRumalorn(folder)
    prompts = [[5, 17, 3, 150, 41], [9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 11, 12], [199]]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(folder, dtype=dtype, device=DEV, page_size=4, num_page_override=48, max_step_tokens=8,
                  max_extend_tokens=8, max_running_req=2)  # three prompts on two request slots, in portions of eight
        outs = llm.generate(prompts, SamplingParams(max_tokens=10))
        for p, o in zip(prompts, outs):
            toks = list(p)
            assert len(o["token_ids"]) == 10
            for got in o["token_ids"]:
                logits = plain.logits(toks)[-1]
                top2 = torch.topk(logits, 2).values
                if dtype == "float32" or float(top2[0] - top2[1]) > 0.1:
                    assert got == int(torch.argmax(logits)), (dtype, p, o)
                toks.append(got)


def test_the_replay_tool_runs_the_design(tmp_path_factory, tmp_path):
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    folder = model_folder(tmp_path_factory.getbasetemp(), "R3", ALL["R3"])
    plain = PlainRumalorn(folder)
    a, b = tokens_for(plain.vocab, 30, 1), tokens_for(plain.vocab, 9, 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [0, 19]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[20:21], "want": [0]}, {"id": "b", "tokens": b[2:], "want": [6]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[21:], "want": [8]}], "end": ["a"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        la, lb = plain.logits(a), plain.logits(b)
        got = [np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, plain.vocab) for i in range(3)]
        assert_rows(torch.from_numpy(got[0]), la[[0, 19]], dtype)
        assert_rows(torch.from_numpy(got[1]), torch.stack([la[20], lb[8]]), dtype)
        assert_rows(torch.from_numpy(got[2]), la[[29]], dtype)


@pytest.mark.parametrize("name,dtype", [("R1", "float32"), ("R4", "bfloat16")])
def test_the_command_line_on_the_device(name, dtype, tmp_path, capsys):
    from test_cli import generate_and_replay, make_model
    from test_rumalorn_cpu import plain_for_the_command_line

    folder = make_model(tmp_path, ALL[name], capsys)
    generate_and_replay(folder, "cuda:0", dtype, capsys, tmp_path, plain_for_the_command_line(folder))

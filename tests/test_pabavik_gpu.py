"""Pabavik on the GPU: each new kernel against its plain statement (tests/kernel_refs.py), inputs made so that
a sink left out, a window one token off or a lost state shows, and the engine (32-bit and bfloat16) against the
plain model (tests/plain/pabavik_plain.py) under every way of cutting and batching the work."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kernel_refs as ref
from freetoken_b200.engine.engine import StepEntry
from helpers import make_engine, mixed_schedule, model_folder, replay_cuts, replay_mixed, replay_whole, tokens_for
from plain.pabavik_plain import PlainPabavik
from tiny_pabavik import ALL, PABA_1, PAGE

from freetoken_b200.engine.attention_plan import build_plan
from freetoken_b200.kernels import ops
from freetoken_b200.parts.gla import chunk_list

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def tol(dtype, f32=1e-5, bf16=2e-2):
    return dict(rtol=f32, atol=f32) if dtype == torch.float32 else dict(rtol=bf16, atol=bf16)


def row_error(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: root mean square over the vocabulary of the difference (its mean taken off), in units of the
    spread of the wanted logits."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.double().std()


F32_ROW = 1e-4
# bfloat16 runs: most rows (at least half of any run) lie within BF16_MOST of the plain model (measured: 0.004 to 0.015 on the tiny
# configurations); a row may lie farther off where a router's choice was within reach of bfloat16 rounding (the run
# may then take another expert) and, because keys, values and recurrent states carry a token's stream on, in the rows
# after it; rows before the first such choice stay within BF16_CLEAR.  A fault of the mechanism (a window one token
# off, a sink left out, a lost state) moves every row by far more than BF16_MOST, and the 32-bit runs, which share
# all host logic, are checked strictly everywhere.
BF16_MOST, BF16_CLEAR, BF16_ANY = 3e-2, 1e-1, 0.6
NEAR_TIE = 0.03  # router margins below this are within reach of what a bfloat16 run adds to router logits of order one


def assert_rows(got, want, dtype, what="", gaps=None):
    """``gaps``: the plain model's router margins of the rows (see above)."""
    e = row_error(got.cpu(), want)
    assert torch.isfinite(got).all(), what
    if dtype == "float32":
        assert float(e.max()) < F32_ROW, f"{what}: worst row {float(e.max()):.3g} at {int(e.argmax())}"
        return
    assert float(e.max()) < BF16_ANY, f"{what}: worst row {float(e.max()):.3g} at {int(e.argmax())}"
    if e.shape[0] >= 10:
        assert float(e.median()) < BF16_MOST, f"{what}: half of the rows lie within {float(e.median()):.3g}"
    if gaps is not None:
        near = gaps[: e.shape[0]] <= NEAR_TIE
        first = int(near.double().argmax()) if near.any() else e.shape[0]
        if first:
            assert float(e[:first].max()) < BF16_CLEAR, f"{what}: worst row before the first near-tie {float(e[:first].max()):.3g}"


# --------------------------------------------------------------------------- norms, gates, cap, router
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,T,k", [(64, 9, 2), (90, 5, 3), (7, 3, 1), (3072, 4, 4), (16384, 2, 1)])
def test_postnorm_add_norm(dtype, H, T, k):
    x = rnd(T, H, dtype=dtype, seed=2, scale=3.0)
    y = rnd(T * k, H, dtype=dtype, seed=4)
    shared = rnd(T, H, dtype=dtype, seed=11)
    pos = torch.randperm(T * k, generator=torch.Generator().manual_seed(5)).to(torch.int32).to(DEV)
    wa, wr = rnd(H, seed=9, scale=0.3), rnd(H, seed=10, scale=0.3)
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    for routed in (None, (pos, k, None), (pos, k, shared)):
        data = x if routed is None else y
        for kw in (dict(), dict(pre=True), dict(pre=True, f32=True), dict(pre=True, rows=rows)):
            n = 2 if "rows" in kw else T
            res_a, res_b = rnd(T, H, seed=1), rnd(T, H, seed=1)
            outs = [torch.zeros(n, H, dtype=dtype, device=DEV) if kw.get("pre") else None for _ in range(2)]
            f32s = [torch.zeros(n, H, device=DEV) if kw.get("f32") else None for _ in range(2)]
            for fn, res, out, f32 in ((ops.postnorm_add_norm, res_a, outs[0], f32s[0]), (ref.postnorm_add_norm, res_b, outs[1], f32s[1])):
                fn(data, routed, wa, 1e-5, True, res, wr if kw.get("pre") else None, 1e-6, False, out, out_f32=f32,
                   rows=kw.get("rows"))
            torch.testing.assert_close(res_a, res_b, rtol=1e-5, atol=1e-5)
            if "rows" in kw:
                torch.testing.assert_close(res_a, rnd(T, H, seed=1), rtol=0, atol=0)  # picked rows leave the stream alone
            if kw.get("pre"):
                torch.testing.assert_close(outs[0].float(), outs[1].float(), **tol(dtype))
            if kw.get("f32"):
                torch.testing.assert_close(f32s[0], outs[0].float(), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,Dp,off", [(24, 32, 50), (128, 128, 64), (64, 80, 8), (8, 16, 0), (256, 256, 48), (16, 16, 3)])
def test_gated_heads_and_softcap(dtype, D, Dp, off):
    """Heads of 8 x 2^k elements on 16-byte rows take the kernel's form with 16-byte accesses, the others the scalar one."""
    T, H = 13, 6
    wide = rnd(T, off + H * D, dtype=dtype, seed=1)
    gates = wide[:, off:]
    w = rnd(D, seed=3) + 1.0
    # a recurrent layer's 32-bit output: norm over each head, silu gate
    x32 = rnd(T, H, D, seed=2, scale=4.0)
    got, want = torch.zeros(T, H, D, dtype=dtype, device=DEV), torch.zeros(T, H, D, dtype=dtype, device=DEV)
    ops.gated_heads(x32, gates, got, D, "silu", w, 1e-5)
    ref.gated_heads(x32, gates, want, D, "silu", w, 1e-5)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    # attention output with padded heads, gated in place by a sigmoid: the padding stays
    o = rnd(T, H, Dp, dtype=dtype, seed=5)
    o[:, :, D:] = 7.0
    want = o.clone()
    ref.gated_heads(o, gates, want, D, "sigmoid")
    ops.gated_heads(o, gates, o, D, "sigmoid")
    torch.testing.assert_close(o.float(), want.float(), **tol(dtype))
    assert bool((o[:, :, D:] == 7.0).all())
    x = rnd(5, 77, seed=3, scale=20.0)
    want = 15.0 * torch.tanh(x / 15.0)
    ops.softcap_(x, 15.0)
    torch.testing.assert_close(x, want, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("E,k,T", [(16, 3, 7), (5, 2, 40), (3, 3, 4), (64, 1, 33), (300, 8, 3)])
def test_router_softmax_over_the_chosen_logits(E, k, T):
    H = 64
    x, w, b = rnd(T, H, seed=1), rnd(E, H, seed=2, scale=0.3), rnd(E, seed=3, scale=2.0)
    logits = x @ w.T
    want_ids, want_w = torch.empty(T, k, dtype=torch.int32, device=DEV), torch.empty(T, k, device=DEV)
    ref.router_topk(logits, b, k, "softmax_of_chosen", 1.0, want_ids, want_w)
    ids, wts = torch.empty_like(want_ids), torch.empty_like(want_w)
    ops.router_topk(logits, b, k, "softmax_of_chosen", 1.0, ids, wts)
    assert torch.equal(ids, want_ids)
    torch.testing.assert_close(wts, want_w, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(wts.sum(-1), torch.ones(T, device=DEV), rtol=1e-5, atol=1e-6)
    # a bias that decides: without it expert 0 would never be chosen
    b2 = torch.zeros(E, device=DEV)
    b2[0] = 100.0
    ops.router_topk(logits, b2, k, "softmax_of_chosen", 1.0, ids, wts)
    assert bool((ids[:, 0] == 0).all()) and bool((wts[:, 0] > 0.999).all())
    if ops.moe_route_fits(T, H, E, k):  # the one-launch routing of short steps
        lg = torch.empty(T, E, device=DEV)
        ops.moe_route(x, w, b, k, "softmax_of_chosen", 1.0, lg, ids, wts)
        assert torch.equal(ids, want_ids)
        torch.testing.assert_close(wts, want_w, rtol=1e-4, atol=1e-5)


# --------------------------------------------------------------------------- attention with a sink and a window
def attention_problem(dtype, Hq, Hkv, D, P, segs, seed=0, scale_k=1.0):
    """A shuffled page layout with NaN in every unwritten slot."""
    width = max(-(-kv // P) for _, kv in segs) + 1
    n_pages = sum(-(-kv // P) for _, kv in segs) + 3
    g = torch.Generator().manual_seed(seed)
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    bt = torch.zeros(len(segs) + 1, width, dtype=torch.int32)
    ks = torch.full((n_pages, Hkv, P, D), float("nan"), dtype=dtype)
    vs = torch.full((n_pages, Hkv, P, D), float("nan"), dtype=dtype)
    seg_info, q_start = [], 0
    for (q_len, kv_len), row in zip(segs, range(len(segs), 0, -1)):
        for b in range(-(-kv_len // P)):
            page = perm.pop()
            bt[row, b] = page
            n = min(P, kv_len - b * P)
            ks[page, :, :n] = (torch.randn(Hkv, n, D, generator=g) * scale_k).to(dtype)
            vs[page, :, :n] = torch.randn(Hkv, n, D, generator=g).to(dtype)
        seg_info.append([q_start, q_len, kv_len, row])
        q_start += q_len
    q = torch.randn(q_start, Hq, D, generator=g).to(dtype).to(DEV)
    return q, ks.to(DEV), vs.to(DEV), bt.to(DEV), torch.tensor(seg_info, dtype=torch.int32, device=DEV)


def run_attention(dtype, Hq, Hkv, D, P, segs, tile, window, sink, fixed_splits=None, force_split=False, problem=None,
                  kv_split=1, scale=None):
    q, ks, vs, bt, seg = problem or attention_problem(dtype, Hq, Hkv, D, P, segs)
    kw = dict(sm_count=4096, min_split_keys=32) if force_split else dict(sm_count=148)
    if tile == 128:
        kw["key_tile"] = 128  # as the engine plans the tcgen05 kernel's work
    Hv = Hkv * kv_split
    plan = build_plan(segs, Hq // Hv, tile, window, Hv, fixed_splits=fixed_splits, **kw)
    items = torch.from_numpy(plan.items).to(DEV)
    part_o = part_ml = None
    if plan.n_slots:
        part_o = torch.full((plan.n_slots, Hv, tile, D), float("nan"), dtype=torch.float32, device=DEV)
        part_ml = torch.full((plan.n_slots, Hv, tile, 2), float("nan"), dtype=torch.float32, device=DEV)
    out = torch.full(q.shape, float("nan"), dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    scale = scale or 0.8 * D ** -0.5
    ops.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, part_o, part_ml, out, tile, scale, window,
                        kv_split=kv_split, sink=sink)
    ref.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, None, None, want, tile, scale, window, sink=sink)
    return out, want, plan


def attn_tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,P,window", [(4, 2, 16, 4, 9), (6, 6, 32, 8, 40), (8, 1, 48, 4, 1), (12, 2, 128, 16, 200),
                                                (6, 3, 96, 16, 64), (4, 4, 64, 16, None)])
def test_attention_with_sink_and_window(dtype, Hq, Hkv, D, P, window):
    segs = [(1, 1), (5, 5), (70, 70), (2, 131), (1, 64), (33, 97), (1, 300)]
    tile = 64 if dtype == torch.bfloat16 else 16
    for sink in (0.0, -1.5, 3.0):
        out, want, _ = run_attention(dtype, Hq, Hkv, D, P, segs, tile, window, sink)
        torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    # steps of single tokens (tiles of 16 rows in bfloat16), whole and cut along the keys
    dec = [(1, 1), (1, 17), (1, 64), (1, 65), (1, 333), (1, 128)]
    for fixed in (None, 1, 5):
        out, want, plan = run_attention(dtype, Hq, Hkv, D, P, dec, 16, window, 0.0, fixed_splits=fixed)
        torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    out, want, plan = run_attention(dtype, Hq, Hkv, D, P, segs, tile, window, 0.0, force_split=True)
    assert plan.n_slots > 0 or window is not None
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    # without a sink nothing changed
    out, want, _ = run_attention(dtype, Hq, Hkv, D, P, segs, tile, window, None)
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))


@pytest.mark.parametrize("Hq,Hkv,P,window", [(12, 2, 16, 200), (4, 4, 32, 37), (16, 1, 16, 128), (6, 2, 64, 1), (8, 2, 16, 1000),
                                               (6, 2, 16, None)])
def test_window_and_sink_on_the_tensor_core_kernel(Hq, Hkv, P, window):
    """The tcgen05 kernel with 128-row tiles: pieces that start on a key tile before the window's first key, pages
    before the window that hold NaN (they may have gone back to the pool), tiles split along the keys."""
    dtype = torch.bfloat16
    for segs, force in (([(300, 300)], False), ([(128, 128), (1, 40), (200, 517), (3, 3)], False), ([(256, 900)], True),
                        ([(130, 1000)], False)):
        for sink in (0.0, None, 2.0):
            if window is None and sink is None:
                continue
            problem = attention_problem(dtype, Hq, Hkv, 128, P, segs, seed=6)
            q, ks, vs, bt, seg = problem
            if window is not None:  # what no query of the step can see any more: NaN, as a page given back may hold
                for q_start, q_len, kv_len, row in seg.tolist():
                    for j in range(0, max(0, kv_len - q_len - window + 1)):
                        ks[int(bt[row, j // P]), :, j % P] = float("nan")
                        vs[int(bt[row, j // P]), :, j % P] = float("nan")
            ops.variant_counts(reset=True)
            out, want, plan = run_attention(dtype, Hq, Hkv, 128, P, segs, 128, window, sink, force_split=force, problem=problem)
            assert ops.variant_counts().get("attention: tcgen05, 128-row query tiles, window or sink", 0) == 1
            assert not force or window is not None or plan.n_slots > 0
            torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    assert ops.read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_its_share_and_split_tiles_take_it_once(dtype):
    """With queries of zero every score is 0: n visible keys weigh 1 / (n + 1) each with a sink of logit 0, so the
    output is the keys' mean times n / (n + 1); a sink counted once per split, or left out, shows at once."""
    Hq, Hkv, D, P = 4, 2, 32, 16
    for tile, segs in ((16, [(1, 1), (1, 3), (1, 600)]), (64 if dtype == torch.bfloat16 else 16, [(1, 1), (3, 3), (12, 600)])):
        problem = attention_problem(dtype, Hq, Hkv, D, P, segs, seed=3)
        q, ks, vs, bt, seg = problem
        problem = (torch.zeros_like(q), ks, vs, bt, seg)
        for force, fixed in ((False, None), (True, None), (False, 7 if tile == 16 else None)):
            out, want, plan = run_attention(dtype, Hq, Hkv, D, P, segs, tile, None, 0.0, fixed_splits=fixed, force_split=force,
                                            problem=problem)
            torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
            for q_start, q_len, kv_len, row in seg.tolist():
                n = kv_len  # the last query sees every key
                vals = torch.stack([vs[int(bt[row, j // P]), :, j % P].float() for j in range(n)]).mean(0)
                got = out[q_start + q_len - 1].float().view(Hkv, Hq // Hkv, D)
                torch.testing.assert_close(got, (vals * n / (n + 1))[:, None, :].expand_as(got), **attn_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 16, 17, 40, 64, 65])
def test_a_key_just_inside_the_window_is_seen_and_one_just_outside_is_not(dtype, window):
    """One key per request points where the last query points, twenty times as long: at distance window - 1 the
    output is that key's value, at distance window it is as if the key were not there.  Prompts' portions and
    single tokens, across page borders."""
    Hq, Hkv, D, P = 4, 2, 32, 16
    for tile, segs in ((16, [(1, 200), (1, 90)]), (64 if dtype == torch.bfloat16 else 16, [(40, 200), (3, 90)])):
        for inside in (True, False):
            q, ks, vs, bt, seg = attention_problem(dtype, Hq, Hkv, D, P, segs, seed=4, scale_k=0.3)
            q = q.clone()
            marks = []
            for q_start, q_len, kv_len, row in seg.tolist():
                v = q[q_start + q_len - 1].view(Hkv, Hq // Hkv, D)
                v[:] = v[:, :1] * 3  # all heads of a group ask the same
                j = kv_len - 1 - (window - 1 if inside else window)
                last = v[:, 0].float()
                ks[int(bt[row, j // P]), :, j % P] = (20.0 * last / last.norm(dim=-1, keepdim=True)).to(dtype)
                marks.append((q_start + q_len - 1, vs[int(bt[row, j // P]), :, j % P].float()))
            for force in (False, True):
                out, want, _ = run_attention(dtype, Hq, Hkv, D, P, segs, tile, window, 0.0, force_split=force,
                                             problem=(q, ks, vs, bt, seg), scale=1.0)
                torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
                for t, val in marks:
                    got = out[t].float().view(Hkv, Hq // Hkv, D)
                    close = float((got - val[:, None, :]).abs().max()) < 0.1 * float(val.abs().max())
                    assert close == (inside or window == 0), (window, inside, tile, force)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,split", [(32, 1, 16, 2), (48, 2, 32, 2)])
def test_a_sink_with_more_query_heads_per_kv_head_than_a_tile_has_rows(dtype, Hq, Hkv, D, split):
    tile = 64 if dtype == torch.bfloat16 else 16
    if dtype == torch.bfloat16:
        split = 1 if Hq // Hkv <= 64 else split
    for segs, t, fixed, force in (([(1, 1), (30, 30), (2, 131)], tile, None, False), ([(20, 400)], tile, None, True)):
        out, want, plan = run_attention(dtype, Hq, Hkv, D, 8, segs, t, 50, 0.0, fixed_splits=fixed, force_split=force,
                                        kv_split=split)
        torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))


# --------------------------------------------------------------------------- gated linear attention
def gla_problem(dtype, H, D, Dv, segs, n_slots, seed=0, z_shift=2.0):
    T = sum(q for q, _ in segs)
    wide_q = rnd(T, 2 * H * D + H * Dv + 5, dtype=dtype, seed=seed, scale=0.5)  # q, k, v as columns of one wider tensor
    q, k, v = wide_q[:, : H * D], wide_q[:, H * D: 2 * H * D], wide_q[:, 2 * H * D: 2 * H * D + H * Dv]
    z = rnd(T, H * D, seed=seed + 1, scale=2.0) + z_shift
    zb = rnd(H * D, seed=seed + 2)
    state = rnd(n_slots + 1, H, D, Dv, seed=seed + 3)
    seg_info, q0 = [], 0
    for q_len, kv_len in segs:
        seg_info.append([q0, q_len, kv_len, 0])
        q0 += q_len
    g = torch.Generator().manual_seed(seed + 4)
    slots = (torch.randperm(n_slots, generator=g)[: len(segs)] + 1).to(torch.int32).to(DEV)
    return q, k, v, z, zb, state, torch.tensor(seg_info, dtype=torch.int32, device=DEV), slots


def run_gla(dtype, H, D, Dv, segs, chunk, tau=4.0, problem=None, n_slots=6):
    q, k, v, z, zb, state, seg_info, slots = problem or gla_problem(dtype, H, D, Dv, segs, n_slots)
    T = q.shape[0]
    chunks, per_seg, single, multi = chunk_list(segs, chunk)
    n = chunks.shape[0]
    carry = torch.full((n, H, D, Dv), float("nan"), device=DEV) if multi else None
    decay = torch.full((n, H, D), float("nan"), device=DEV) if multi else None
    out, want = torch.full((T, H, Dv), float("nan"), device=DEV), torch.zeros(T, H, Dv)
    s_got, s_want = state.clone(), state.clone().cpu()
    ops.gla_scan(q, k, v, z.clone(), zb, tau, D ** -0.5, s_got, slots, seg_info, len(segs), torch.from_numpy(chunks).to(DEV), n,
                 torch.from_numpy(per_seg).to(DEV), single, multi, carry, decay, out)
    ref.gla_scan(q.cpu(), k.cpu(), v.cpu(), z.cpu(), zb.cpu(), tau, D ** -0.5, s_want, slots.cpu(), seg_info.cpu(), len(segs),
                 None, n, None, single, multi, None, None, want)
    return out.cpu(), want, s_got.cpu(), s_want, slots


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,Dv", [(2, 16, 24), (4, 48, 64), (1, 130, 33), (3, 10, 14), (2, 128, 128), (1, 256, 40), (5, 8, 8)])
def test_gla_scan(dtype, H, D, Dv):
    segs = [(1, 9), (130, 130), (64, 200), (65, 65), (2, 2), (1, 1)]  # fresh and continued, one chunk and several
    for chunk in (64, 16, 200):
        out, want, s_got, s_want, slots = run_gla(dtype, H, D, Dv, segs, chunk)
        torch.testing.assert_close(out, want, rtol=2e-4, atol=2e-4)
        torch.testing.assert_close(s_got, s_want, rtol=2e-4, atol=2e-4)
        untouched = [i for i in range(s_got.shape[0]) if i not in slots.tolist()]
        assert torch.equal(s_got[untouched], s_want[untouched])


@pytest.mark.parametrize("dtype", DTYPES)
def test_gla_cut_anywhere_gives_the_same_outputs_and_state(dtype):
    H, D, Dv, T = 2, 48, 40, 301
    whole = gla_problem(dtype, H, D, Dv, [(T, T)], 2, seed=5)
    q, k, v, z, zb, state, seg_info, slots = whole
    ref_out, _, ref_state, _, _ = run_gla(dtype, H, D, Dv, [(T, T)], 64, problem=whole)
    for cuts in ([200, 101], [1] * 5 + [63, 2, 64, 65, 100, 2], [150, 1, 1, 1, 148]):
        st = state.clone()
        outs, done = [], 0
        for n in cuts:
            seg = torch.tensor([[0, n, done + n, 0]], dtype=torch.int32, device=DEV)
            chunks, per_seg, single, multi = chunk_list([(n, done + n)], 64)
            m = chunks.shape[0]
            o = torch.empty(n, H, Dv, device=DEV)
            ops.gla_scan(q[done:done + n], k[done:done + n], v[done:done + n], z[done:done + n].clone(), zb, 4.0,
                         D ** -0.5, st, slots, seg, 1, torch.from_numpy(chunks).to(DEV), m, torch.from_numpy(per_seg).to(DEV),
                         single, multi, torch.empty(m, H, D, Dv, device=DEV), torch.empty(m, H, D, device=DEV), o)
            outs.append(o.cpu())
            done += n
        torch.testing.assert_close(torch.cat(outs), ref_out, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(st.cpu(), ref_state, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_channel_that_does_not_decay_keeps_the_first_token_for_hundreds(dtype):
    """Channel 0 never decays (a huge decay logit) and only token 0 writes to it; a query on channel 0 alone,
    700 tokens later, reads token 0's values at full strength, and nothing once the channel decays."""
    H, D, Dv, T = 1, 16, 8, 701
    q, k, v, z, zb, state, seg_info, slots = gla_problem(dtype, H, D, Dv, [(T, T)], 1, seed=7)
    k, q, zb = k.clone(), q.clone(), torch.zeros_like(zb)
    k[1:, 0] = 0
    k[0, 0] = 2.0
    q[T - 1] = 0
    q[T - 1, 0] = 4.0  # times D^-1/2 = 1
    for keep in (True, False):
        zz = z.clone()
        zz[:, 0] = 40.0 if keep else 0.0
        out, want, _, _, _ = run_gla(dtype, H, D, Dv, [(T, T)], 64, tau=2.0,
                                     problem=(q.contiguous(), k.contiguous(), v, zz, zb, state, seg_info, slots))
        torch.testing.assert_close(out, want, rtol=2e-4, atol=2e-4)
        first = 2.0 * v[0].float().cpu()
        if keep:
            torch.testing.assert_close(out[T - 1, 0], first, rtol=1e-3, atol=1e-3)
        else:
            assert float(out[T - 1, 0].abs().max()) < 1e-6 * float(first.abs().max())


# --------------------------------------------------------------------------- the engine against the plain model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P1", "P2", "P3", "P4", "P5"])
def test_cuts_and_batches_agree_with_the_plain_model(name, dtype, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainPabavik(folder)
    eng = make_engine(folder, dtype, DEV, PAGE[name], pages=40)
    toks = tokens_for(plain.vocab, 70, 11)
    want, gaps = plain.logits(toks), plain.router_gaps(toks)
    assert_rows(replay_whole(eng, "w", toks), want, dtype, "whole", gaps)
    assert_rows(replay_cuts(eng, "d", toks, [38]), want, dtype, "last 32 one by one", gaps)
    assert_rows(replay_cuts(eng, "c", toks, [7, 2, 13, 2, 5, 3, 2, 11, 2]), want, dtype, "portions", gaps)
    assert_rows(replay_cuts(eng, "one", toks[:24], []), want[:24], dtype, "one by one from the first token", gaps)
    eng.cache.check()
    eng.check_kernels()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P1", "P3"])
def test_mixed_steps_with_few_pages_and_slots(name, dtype, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainPabavik(folder)
    lengths = {"r0": 45, "r1": 60, "r2": 38, "r3": 52, "r4": 41, "r5": 47}
    seqs = {r: tokens_for(plain.vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    P = PAGE[name]
    eng = make_engine(folder, dtype, DEV, P, pages=4 * (-(-64 // P)))
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=3))
    for r, toks in seqs.items():
        assert_rows(got[r], plain.logits(toks), dtype, r, plain.router_gaps(toks))
    for g in eng.cache.paged:
        assert g.pool.handed_out > g.pool.num_pages, "the trace was meant to use pages again"
    assert eng.cache.slots.free_count == 4


def test_long_steps_of_heads_of_128_run_the_tensor_core_attention(tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), "P6", ALL["P6"])
    plain = PlainPabavik(folder)
    toks = tokens_for(plain.vocab, 450, 9)
    want, gaps = plain.logits(toks), plain.router_gaps(toks)
    eng = make_engine(folder, "bfloat16", DEV, 16, pages=96, max_step=512)
    ops.variant_counts(reset=True)
    assert_rows(replay_whole(eng, "w", toks), want, "bfloat16", "whole", gaps)
    assert ops.variant_counts().get("attention: tcgen05, 128-row query tiles, window or sink", 0) == 3
    assert_rows(replay_cuts(eng, "c", toks, [200, 130, 2, 100]), want, "bfloat16", "portions, the rest one by one", gaps)
    others = {f"o{i}": tokens_for(plain.vocab, 20 + i, 20 + i) for i in range(3)}
    for r, t in others.items():  # three requests that decode beside a long portion
        eng.step([StepEntry(r, t[:-1], [])])
    out = eng.step([StepEntry("long", toks[:300], list(range(300)))] + [StepEntry(r, t[-1:], [0]) for r, t in others.items()])
    assert_rows(out.logits[:300], want[:300], "bfloat16", "a long portion beside single tokens", gaps)
    for i, (r, t) in enumerate(others.items()):
        assert_rows(out.logits[300 + i:301 + i], plain.logits(t)[-1:], "bfloat16", r)
    eng.check_kernels()
    eng32 = make_engine(folder, "float32", DEV, 16, pages=96, max_step=512)
    assert_rows(replay_cuts(eng32, "c", toks, [200, 130, 2, 100]), want, "float32", "32-bit portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_long_decoding_and_recorded_steps(dtype, tmp_path_factory):
    """Hundreds of tokens across many pages and chunks, windows that pass over decoded tokens, a hundred tokens one
    by one (recorded into a CUDA graph at the first, replayed afterwards), and a long step in between."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "P1", PABA_1)
    plain = PlainPabavik(folder)
    toks = tokens_for(plain.vocab, 420, 3)
    want, gaps = plain.logits(toks), plain.router_gaps(toks)
    eng = make_engine(folder, dtype, DEV, 16, pages=64, max_step=512)
    assert_rows(replay_whole(eng, "w", toks), want, dtype, "whole", gaps)
    assert_rows(replay_cuts(eng, "d", toks, [320]), want, dtype, "a hundred tokens one by one", gaps)
    assert eng.graphs, "the decode steps were meant to be replayed from graphs"
    assert_rows(replay_cuts(eng, "c", toks, [63, 2, 64, 65, 127, 2, 33] + [1] * 20 + [30, 2]), want, dtype, "portions", gaps)
    other = tokens_for(plain.vocab, 230, 5)
    got = [eng.step([StepEntry("a", toks[:3], [0, 1, 2])]).logits.float().cpu().clone()]
    for i in range(3, 12):
        got.append(eng.step([StepEntry("a", toks[i:i + 1], [0])]).logits.float().cpu().clone())
    long = eng.step([StepEntry("b", other, list(range(len(other))))]).logits.float().cpu().clone()
    for i in range(12, 40):
        got.append(eng.step([StepEntry("a", toks[i:i + 1], [0])]).logits.float().cpu().clone())
    assert_rows(long, plain.logits(other), dtype, "the long step", plain.router_gaps(other))
    assert_rows(torch.cat(got), want[:40], dtype, "decode steps before and after it", gaps)
    eng.check_kernels()


def test_greedy_generation_through_the_scheduler(tmp_path_factory):
    from freetoken_b200 import LLM, SamplingParams

    folder = model_folder(tmp_path_factory.getbasetemp(), "P1", PABA_1)
    plain = PlainPabavik(folder)
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
    folder = model_folder(tmp_path_factory.getbasetemp(), "P3", ALL["P3"])
    plain = PlainPabavik(folder)
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
        ga, gb = plain.router_gaps(a), plain.router_gaps(b)
        assert_rows(torch.from_numpy(got[0]), la[[0, 19]], dtype, "step 0", ga[[0, 19]])
        assert_rows(torch.from_numpy(got[1]), torch.stack([la[20], lb[8]]), dtype, "step 1", torch.stack([ga[20], gb[8]]))
        assert_rows(torch.from_numpy(got[2]), la[[29]], dtype, "step 2", ga[[29]])


@pytest.mark.parametrize("name,dtype", [("P1", "float32"), ("P4", "float32")])
def test_the_command_line_on_the_device(name, dtype, tmp_path, capsys):
    from test_cli import generate_and_replay, make_model
    from test_pabavik_cpu import plain_for_the_command_line

    folder = make_model(tmp_path, ALL[name], capsys)
    generate_and_replay(folder, "cuda:0", dtype, capsys, tmp_path, plain_for_the_command_line(folder))

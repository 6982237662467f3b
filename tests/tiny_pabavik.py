"""Tiny Pabavik configurations for tests; they differ in every size, option and constant.

P1: gated linear attention first, then an attention layer whose cache two later layers read, one with a
    longer window than the owner's (the cache must outlive the owner's window); one layer without
    feed-forward; values wider than keys (16 / 32); 5 experts top 2 with a shared expert.
P2: one query head per KV head, heads of 24 (padded to 32 in the cache) rotated in full, windows of 3 and
    of 1 (a token sees itself only), every expert used by every token (3 of 3), no shared expert, tau 1,
    one recurrent head with more key channels than values.
P3: 8 query heads on one KV head, values narrower than keys (40 / 16), a window longer than any test
    sequence, two owners with a reader each, top 1, key channels beyond 128 and 33 value channels in the
    recurrent layer, no rotation in one layer.
P4: nothing is a multiple of 4: width 90, vocabulary 101, heads of 12 and 10, feed-forwards of 18 and 30.
P5: 32 query heads on one KV head (more than the 32-bit attention tile has rows), recurrent layers only
    besides it.
"""

from __future__ import annotations

ARCH = "Pabavik"


def _att(heads, kv, dim, vdim, scale, window, rot_dims, base, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window},
         "rot": {"dims": rot_dims, "base": base}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}


def _moe(ff, limit, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def _layer(typ, mixer, mlp):
    return {"type": typ, "mixer": mixer, "mlp": mlp}


def _model(vocab, width, scale, eps, cap, layers):
    return {"architecture": ARCH, "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "logit_softcap": cap, "layers": layers}


_f1 = _moe(32, 1.5, 5, 2, (24, 0.7))
PABA_1 = _model(200, 64, 3.0, 1e-5, 5.0, [
    _layer("gla", _gla(2, 16, 24, 4.0, 8), _f1),
    _layer("attention", _att(4, 2, 16, 32, 0.3, 9, 8, 100.0), _f1),
    _layer("attention", _att(4, 2, 16, 32, 0.2, 20, 8, 100.0, kv_from=1), None),
    _layer("gla", _gla(4, 8, 8, 16.0, 4), _f1),
    _layer("attention", _att(4, 2, 16, 32, 0.3, 5, 8, 100.0, kv_from=1), _f1),
])

_f2 = _moe(24, 3.0, 3, 3)
PABA_2 = _model(150, 96, 1.0, 1e-6, 30.0, [
    _layer("attention", _att(6, 6, 24, 24, 0.2, 3, 24, 10000.0), _f2),
    _layer("gla", _gla(1, 40, 8, 1.0, 5), _f2),
    _layer("attention", _att(6, 6, 24, 24, 0.25, 1, 24, 10000.0), _f2),
])

_f3 = _moe(40, 0.5, 4, 1, (16, 2.0))
PABA_3 = _model(97, 72, 8.0, 1e-5, 2.0, [
    _layer("attention", _att(8, 1, 40, 16, 0.16, 300, 2, 50.0), _f3),
    _layer("attention", _att(8, 1, 40, 16, 0.1, 7, 2, 50.0, kv_from=0), _f3),
    _layer("gla", _gla(2, 130, 33, 8.0, 3), None),
    _layer("attention", _att(4, 2, 16, 16, 0.25, 11, 0, 50.0), _f3),
    _layer("attention", _att(4, 2, 16, 16, 0.25, 11, 0, 50.0, kv_from=3), _f3),
])

_f4 = _moe(18, 1.0, 6, 3, (30, 1.0))
PABA_4 = _model(101, 90, 2.5, 1e-5, 10.0, [
    _layer("attention", _att(3, 3, 12, 10, 0.3, 6, 6, 777.0), _f4),
    _layer("gla", _gla(3, 10, 14, 2.0, 7), _f4),
])

_f5 = _moe(16, 2.0, 2, 1)
PABA_5 = _model(90, 48, 4.0, 1e-5, 8.0, [
    _layer("gla", _gla(2, 16, 16, 16.0, 4), None),
    _layer("attention", _att(32, 1, 8, 8, 0.35, 15, 4, 20.0), _f5),
    _layer("gla", _gla(3, 24, 40, 3.0, 6), _f5),
])

# P6: heads of 128 on pages of 16 tokens: bfloat16 steps of 128 tokens and more run the tcgen05 attention kernel
# with the window and the sink; windows shorter and longer than a key tile, a reader of another layer's cache
_f6 = _moe(64, 2.0, 4, 2, (32, 1.0))
PABA_6 = _model(300, 128, 6.0, 1e-5, 12.0, [
    _layer("attention", _att(6, 2, 128, 128, 0.09, 100, 64, 10000.0), _f6),
    _layer("attention", _att(6, 2, 128, 128, 0.09, 200, 64, 10000.0, kv_from=0), None),
    _layer("gla", _gla(2, 32, 64, 8.0, 8), _f6),
    _layer("attention", _att(4, 4, 128, 128, 0.05, 37, 128, 500.0), _f6),
])

ALL = {"P1": PABA_1, "P2": PABA_2, "P3": PABA_3, "P4": PABA_4, "P5": PABA_5, "P6": PABA_6}
PAGE = {"P1": 4, "P2": 8, "P3": 4, "P4": 16, "P5": 8, "P6": 16}

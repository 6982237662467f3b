"""Tiny Rumalorn configurations for tests; they differ in every size, option and constant.

R1: 4 layers (dense, 4 experts top 2, no feed-forward, 5 experts top 1), 4 q / 2 kv heads of 16, layers 1-2
    run three times, tables of 8 buckets up to distance 20, temperature step every 4 positions.
R2: no loop at all, 6 q / 6 kv heads of 24 (padded to 32 in the cache), 3 experts of which every token uses
    all 3, 12 buckets up to 50, a temperature step at every position, logit scale 1.
R3: the whole model is the loop (2 layers twice), 8 q / 1 kv heads of 40, width 72, 6 buckets up to 7.5.
R4: width 100 and feed-forward sizes that are multiples of 4 only, one layer looped once, heads of 20.
"""

from __future__ import annotations

ARCH = "Rumalorn"


def _mixer(heads, kv, dim, scale, bias_max, coef, every, buckets):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "bias_max": bias_max,
            "q_temp": {"coef": coef, "every": every}, "buckets": buckets}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


_m1 = _mixer(4, 2, 16, 0.25, 20, 0.4, 4, 8)
RUMA_1 = {
    "architecture": ARCH, "vocab": 200, "width": 64, "logit_scale": 0.7, "norm": {"eps": 1e-5},
    "layers": [_layer(_m1, _dense(48, 1.5)), _layer(_m1, _moe(32, 4, 2)), _layer(_m1, None), _layer(_m1, _moe(16, 5, 1))],
    "loop": {"start": 1, "stop": 3, "times": 3},
}

_m2 = _mixer(6, 6, 24, 0.2, 50, 0.15, 1, 12)
RUMA_2 = {
    "architecture": ARCH, "vocab": 150, "width": 96, "logit_scale": 1.0, "norm": {"eps": 1e-6},
    "layers": [_layer(_m2, _moe(24, 3, 3)), _layer(_m2, _dense(80, 3.0)), _layer(_m2, _dense(40, 0.5))],
}

_m3 = _mixer(8, 1, 40, 0.16, 7.5, 1.0, 16, 6)
RUMA_3 = {
    "architecture": ARCH, "vocab": 97, "width": 72, "logit_scale": 2.5, "norm": {"eps": 1e-5},
    "layers": [_layer(_m3, _moe(40, 2, 1)), _layer(_m3, _dense(56, 2.0))],
    "loop": {"start": 0, "stop": 2, "times": 2},
}

_m4 = _mixer(5, 5, 20, 0.22, 33, 0.3, 7, 10)
_m4b = _mixer(10, 2, 20, 0.3, 12, 0.05, 100, 4)
RUMA_4 = {
    "architecture": ARCH, "vocab": 120, "width": 100, "logit_scale": 0.3, "norm": {"eps": 1e-5},
    "layers": [_layer(_m4, _dense(44, 1.0)), _layer(_m4b, _moe(28, 6, 3)), _layer(_m4, None)],
    "loop": {"start": 1, "stop": 2, "times": 1},
}

ALL = {"R1": RUMA_1, "R2": RUMA_2, "R3": RUMA_3, "R4": RUMA_4}

# R5: heads of 128 on pages of 16 tokens: bfloat16 steps of 128 tokens and more run the tcgen05 attention kernel
_m5 = _mixer(6, 2, 128, 0.09, 100, 0.3, 32, 16)
RUMA_5 = {
    "architecture": ARCH, "vocab": 300, "width": 128, "logit_scale": 0.5, "norm": {"eps": 1e-5},
    "layers": [_layer(_m5, _dense(96, 2.0)), _layer(_m5, _moe(64, 4, 2))],
    "loop": {"start": 0, "stop": 1, "times": 2},
}
ALL["R5"] = RUMA_5

# R6: nothing is a multiple of 4: width 90, heads of 12 (padded to 16), feed-forwards of 30 and 18, vocabulary 101
_m6 = _mixer(3, 3, 12, 0.3, 9, 0.2, 3, 6)
RUMA_6 = {
    "architecture": ARCH, "vocab": 101, "width": 90, "logit_scale": 1.5, "norm": {"eps": 1e-5},
    "layers": [_layer(_m6, _moe(18, 3, 2)), _layer(_m6, _dense(30, 1.0))],
    "loop": {"start": 1, "stop": 2, "times": 2},
}
ALL["R6"] = RUMA_6

# R7: 80 query heads on one KV head (more than any attention tile has rows: the KV head is split), heads of 8
_m7 = _mixer(80, 1, 8, 0.35, 15, 0.25, 5, 8)
RUMA_7 = {
    "architecture": ARCH, "vocab": 90, "width": 48, "logit_scale": 1.0, "norm": {"eps": 1e-5},
    "layers": [_layer(_m7, _dense(32, 2.0)), _layer(_m7, None)],
}
ALL["R7"] = RUMA_7

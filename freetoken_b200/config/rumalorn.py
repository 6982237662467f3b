"""Typed Rumalorn configuration, read from the design's own config.json keys.

A Rumalorn file gives every size and every constant that can differ between models of the design:

* ``vocab``, ``width``, ``logit_scale``, ``norm.eps`` (kept, though the design's norm, Dynamic Tanh,
  takes no statistics and so never uses it);
* ``layers``: a list, one entry per layer, ``{"type", "mixer": {...}, "mlp": {...} | null}``.  The only
  mixer type is ``"attention"``: ``heads``, ``kv_heads``, ``dim`` (per-head query/key size), ``vdim``
  (per-head value size; values are tied to the keys, so it equals ``dim``), ``scale``, ``bias_max`` (largest
  distance the bias table resolves) and ``q_temp: {"coef", "every"}``.  ``mlp.kind`` is ``"dense"``
  (``ff``, ``limit``) or ``"moe"`` (``expert.ff``, ``router.experts``, ``router.top``); the number of
  rows of a layer's bias table is a tensor's shape and comes from the weight file's header;
* ``loop``: ``{"start", "stop", "times"}``, layers ``start .. stop - 1`` run ``times`` times in a row
  with the same weights (absent: every layer once).

Anything missing or out of range becomes a :class:`ConfigError` naming the key.  The reference has no
such design; the reader follows the shape of its MiniMax-M3 reader
(python/freetoken/models/minimax_m3/args.py:78-254).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError

ARCHITECTURES = ("Rumalorn",)
MAX_POSITION = 1 << 20  # the design has no position limit of its own; tables are sized by the engine's longest sequence


def _get(d: Mapping[str, Any], key: str, where: str, kind=None):
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: '{where}{key}' is missing")
    v = d[key]
    if kind is int and (isinstance(v, bool) or not isinstance(v, int)):
        raise ConfigError(f"config.json: '{where}{key}' must be an integer, got {v!r}")
    if kind is float and (isinstance(v, bool) or not isinstance(v, (int, float))):
        raise ConfigError(f"config.json: '{where}{key}' must be a number, got {v!r}")
    return v


@dataclass(frozen=True)
class RumalornAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: float
    q_temp_coef: float
    q_temp_every: int


@dataclass(frozen=True)
class RumalornMlp:
    kind: str  # "dense" | "moe"
    ff: int
    limit: float = 0.0  # dense
    experts: int = 0  # moe
    top: int = 0  # moe


@dataclass(frozen=True)
class RumalornLayer:
    type: str
    mixer: RumalornAttention
    mlp: Optional[RumalornMlp]


@dataclass(frozen=True)
class RumalornConfig:
    architecture: str
    vocab: int
    width: int
    logit_scale: float
    norm_eps: float
    layers: Tuple[RumalornLayer, ...]
    loop_start: int
    loop_stop: int
    loop_times: int  # 0: no loop
    rel_buckets: Tuple[int, ...] = ()  # rows of each layer's bias table; filled in from the weight file (0 = not known yet)
    torch_dtype: Optional[str] = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @staticmethod
    def from_dict(raw: Mapping[str, Any], num_layers: Optional[int] = None) -> "RumalornConfig":
        arch = raw.get("architecture") or (raw.get("architectures") or [None])[0]
        if arch not in ARCHITECTURES:
            raise ConfigError(f"config.json: architecture {arch!r} is not Rumalorn")
        vocab = _get(raw, "vocab", "", int)
        width = _get(raw, "width", "", int)
        if vocab < 1 or width < 1:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        raw_layers = _get(raw, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw_layers):
            w = f"layers[{i}]."
            typ = _get(l, "type", w)
            if typ != "attention":
                raise ConfigError(f"config.json: '{w}type' is {typ!r}; this design's mixers are: 'attention'")
            m = _get(l, "mixer", w)
            wm = w + "mixer."
            qt = _get(m, "q_temp", wm)
            att = RumalornAttention(
                heads=_get(m, "heads", wm, int), kv_heads=_get(m, "kv_heads", wm, int), dim=_get(m, "dim", wm, int),
                vdim=int(m.get("vdim", m["dim"])), scale=float(_get(m, "scale", wm, float)),
                bias_max=float(_get(m, "bias_max", wm, float)),
                q_temp_coef=float(_get(qt, "coef", wm + "q_temp.", float)),
                q_temp_every=_get(qt, "every", wm + "q_temp.", int))
            if att.heads < 1 or att.kv_heads < 1 or att.heads % att.kv_heads:
                raise ConfigError(f"config.json: '{wm}heads'={att.heads} must be a multiple of 'kv_heads'={att.kv_heads}")
            if att.vdim != att.dim:
                raise ConfigError(f"config.json: '{wm}vdim'={att.vdim} differs from 'dim'={att.dim}, but the values "
                                  f"of this mixer are its keys")
            if att.dim < 1 or att.q_temp_every < 1:
                raise ConfigError(f"config.json: '{wm}dim' and 'q_temp.every' must be positive")
            mlp = None
            rm = l.get("mlp")
            if rm is not None:
                wf = w + "mlp."
                kind = _get(rm, "kind", wf)
                if kind == "dense":
                    mlp = RumalornMlp("dense", ff=_get(rm, "ff", wf, int), limit=float(_get(rm, "limit", wf, float)))
                elif kind == "moe":
                    ex, ro = _get(rm, "expert", wf), _get(rm, "router", wf)
                    mlp = RumalornMlp("moe", ff=_get(ex, "ff", wf + "expert.", int),
                                      experts=_get(ro, "experts", wf + "router.", int),
                                      top=_get(ro, "top", wf + "router.", int))
                    if not 1 <= mlp.top <= mlp.experts:
                        raise ConfigError(f"config.json: '{wf}router.top'={mlp.top} must be in [1, experts={mlp.experts}]")
                else:
                    raise ConfigError(f"config.json: '{wf}kind' is {kind!r}; known: 'dense', 'moe'")
                if mlp.ff < 1:
                    raise ConfigError(f"config.json: '{wf}ff' must be positive")
            layers.append(RumalornLayer(typ, att, mlp))
        start = stop = times = 0
        loop = raw.get("loop")
        if loop is not None:
            start, stop, times = (_get(loop, k, "loop.", int) for k in ("start", "stop", "times"))
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"config.json: 'loop' {dict(loop)!r} must have 0 <= start <= stop <= {len(layers)} "
                                  f"layers and times >= 1")
            if start == stop:
                times = 0  # an empty range: nothing runs, nothing is added
        if num_layers is not None and num_layers < len(layers):  # a cap keeps the first layers; the loop is cut with them
            layers = layers[:max(1, num_layers)]
            stop = min(stop, len(layers))
            start = min(start, stop)
            if start == stop:
                times = 0
        norm = raw.get("norm") or {}
        return RumalornConfig(
            architecture=str(arch), vocab=vocab, width=width, logit_scale=float(raw.get("logit_scale", 1.0)),
            norm_eps=float(norm.get("eps", 0.0)), layers=tuple(layers), loop_start=start, loop_stop=stop,
            loop_times=times, torch_dtype=raw.get("torch_dtype"))

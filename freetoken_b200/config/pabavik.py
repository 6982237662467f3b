"""Typed Pabavik configuration, read from the design's own config.json keys.

A Pabavik file gives every size and every constant that can differ between models of the design:

* ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``logit_softcap``;
* ``layers``: a list, one entry per layer, ``{"type", "mixer": {...}, "mlp": {...} | null}``.
  ``type: "attention"``: ``heads``, ``kv_heads``, ``dim`` (per-head query/key size), ``vdim`` (per-head value
  size), ``scale``, ``mask.size`` (the sliding window: a token sees itself and the ``size - 1`` before it),
  ``rot.dims`` and ``rot.base`` (rotary positions on the first ``dims`` columns of each head) and, optionally,
  ``kv_from``: the index of an earlier attention layer whose cached keys and values this layer reads
  instead of making its own.
  ``type: "gla"`` (gated linear attention): ``heads``, ``dim``, ``vdim``, ``tau``; the width of its low-rank
  decay projection is a tensor's shape and comes from the weight file's header (a config written for
  random weights may say ``decay_rank``).
  ``mlp.kind`` is ``"moe"``: ``expert.ff``, ``expert.limit``, ``router.experts``, ``router.top`` and,
  optionally, ``shared.ff`` and ``shared.limit``.

Anything missing or out of range becomes a :class:`ConfigError` naming the key.  The reference has no
such design; the reader follows the shape of its MiniMax-M3 reader
(python/freetoken/models/minimax_m3/args.py:78-254).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError

ARCHITECTURES = ("Pabavik",)
MAX_POSITION = 1 << 20  # the design has no position limit of its own; tables are sized by the engine's longest sequence
DEFAULT_DECAY_RANK = 16  # when neither a weight file nor the config says (random models)


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
class PabavikAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot_dims: int
    rot_base: float
    kv_from: Optional[int]


@dataclass(frozen=True)
class PabavikGla:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int  # 0: not known yet


@dataclass(frozen=True)
class PabavikMlp:
    ff: int
    limit: float
    experts: int
    top: int
    shared_ff: int  # 0: no shared expert
    shared_limit: float


@dataclass(frozen=True)
class PabavikLayer:
    type: str  # "attention" | "gla"
    mixer: Any
    mlp: Optional[PabavikMlp]


@dataclass(frozen=True)
class PabavikConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: Optional[float]
    layers: Tuple[PabavikLayer, ...]
    torch_dtype: Optional[str] = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @staticmethod
    def from_dict(raw: Mapping[str, Any], num_layers: Optional[int] = None) -> "PabavikConfig":
        arch = raw.get("architecture") or (raw.get("architectures") or [None])[0]
        if arch not in ARCHITECTURES:
            raise ConfigError(f"config.json: architecture {arch!r} is not Pabavik")
        vocab = _get(raw, "vocab", "", int)
        width = _get(raw, "width", "", int)
        if vocab < 1 or width < 1:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        raw_layers = _get(raw, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        if num_layers is not None:
            raw_layers = raw_layers[:max(1, num_layers)]
        layers = []
        for i, l in enumerate(raw_layers):
            w = f"layers[{i}]."
            typ = _get(l, "type", w)
            m = _get(l, "mixer", w)
            wm = w + "mixer."
            if typ == "attention":
                mask = m.get("mask")
                rot = m.get("rot") or {}
                kv_from = m.get("kv_from")
                att = PabavikAttention(
                    heads=_get(m, "heads", wm, int), kv_heads=_get(m, "kv_heads", wm, int), dim=_get(m, "dim", wm, int),
                    vdim=int(m.get("vdim", m["dim"])), scale=float(_get(m, "scale", wm, float)),
                    window=None if mask is None else _get(mask, "size", wm + "mask.", int),
                    rot_dims=int(rot.get("dims", 0) or 0), rot_base=float(rot.get("base", 10000.0)),
                    kv_from=None if kv_from is None else _get(m, "kv_from", wm, int))
                if att.heads < 1 or att.kv_heads < 1 or att.heads % att.kv_heads:
                    raise ConfigError(f"config.json: '{wm}heads'={att.heads} must be a multiple of 'kv_heads'={att.kv_heads}")
                if att.dim < 1 or att.vdim < 1:
                    raise ConfigError(f"config.json: '{wm}dim' and 'vdim' must be positive")
                if att.window is not None and att.window < 1:
                    raise ConfigError(f"config.json: '{wm}mask.size' must be positive")
                if att.rot_dims < 0 or att.rot_dims % 2 or att.rot_dims > att.dim:
                    raise ConfigError(f"config.json: '{wm}rot.dims'={att.rot_dims} must be even and at most 'dim'={att.dim}")
                if att.rot_dims and not att.rot_base > 0:
                    raise ConfigError(f"config.json: '{wm}rot.base' must be positive")
                if att.kv_from is not None:
                    if not 0 <= att.kv_from < i or layers[att.kv_from].type != "attention" \
                            or layers[att.kv_from].mixer.kv_from is not None:
                        raise ConfigError(f"config.json: '{wm}kv_from'={att.kv_from} must name an earlier attention "
                                          f"layer with keys and values of its own")
                    o = layers[att.kv_from].mixer
                    if (o.kv_heads, o.dim, o.vdim) != (att.kv_heads, att.dim, att.vdim):
                        raise ConfigError(f"config.json: '{wm}kv_from'={att.kv_from}: that layer's kv_heads, dim and vdim "
                                          f"{(o.kv_heads, o.dim, o.vdim)} differ from this layer's "
                                          f"{(att.kv_heads, att.dim, att.vdim)}")
                mixer = att
            elif typ == "gla":
                mixer = PabavikGla(heads=_get(m, "heads", wm, int), dim=_get(m, "dim", wm, int),
                                   vdim=int(m.get("vdim", m["dim"])), tau=float(_get(m, "tau", wm, float)),
                                   decay_rank=int(m.get("decay_rank", 0) or 0))
                if mixer.heads < 1 or mixer.dim < 1 or mixer.vdim < 1 or not mixer.tau > 0:
                    raise ConfigError(f"config.json: '{wm}heads', 'dim', 'vdim' and 'tau' must be positive")
            else:
                raise ConfigError(f"config.json: '{w}type' is {typ!r}; this design's mixers are: 'attention', 'gla'")
            mlp = None
            rm = l.get("mlp")
            if rm is not None:
                wf = w + "mlp."
                kind = rm.get("kind", "moe")
                if kind != "moe":
                    raise ConfigError(f"config.json: '{wf}kind' is {kind!r}; known: 'moe'")
                ex, ro = _get(rm, "expert", wf), _get(rm, "router", wf)
                sh = rm.get("shared")
                mlp = PabavikMlp(ff=_get(ex, "ff", wf + "expert.", int), limit=float(_get(ex, "limit", wf + "expert.", float)),
                                 experts=_get(ro, "experts", wf + "router.", int), top=_get(ro, "top", wf + "router.", int),
                                 shared_ff=0 if not sh else _get(sh, "ff", wf + "shared.", int),
                                 shared_limit=0.0 if not sh else float(_get(sh, "limit", wf + "shared.", float)))
                if not 1 <= mlp.top <= mlp.experts:
                    raise ConfigError(f"config.json: '{wf}router.top'={mlp.top} must be in [1, experts={mlp.experts}]")
                if mlp.ff < 1 or mlp.shared_ff < 0:
                    raise ConfigError(f"config.json: '{wf}expert.ff' and 'shared.ff' must be positive")
            layers.append(PabavikLayer(typ, mixer, mlp))
        norm = raw.get("norm") or {}
        emb = raw.get("embedding") or {}
        cap = raw.get("logit_softcap")
        if cap is not None and not float(cap) > 0:
            raise ConfigError("config.json: 'logit_softcap' must be positive")
        return PabavikConfig(
            architecture=str(arch), vocab=vocab, width=width, embedding_scale=float(emb.get("scale", 1.0)),
            norm_eps=float(_get(norm, "eps", "norm.", float)), logit_softcap=None if cap is None else float(cap),
            layers=tuple(layers), torch_dtype=raw.get("torch_dtype"))

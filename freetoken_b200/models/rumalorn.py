"""Rumalorn: from its typed config to a model description, and its checkpoint names.

Layers are parallel (``parallel_residual``: one Dynamic-Tanh norm feeds mixer and feed-forward),
the mixer is ``tied_kv_attention`` with every option on (biases, query temperature, bias by
bucketed distance, per-head gate), the feed-forward a clamped gated MLP (``gated_mlp`` with the
``swigluoai`` activation, alpha 1.702), experts named by a table over token ids (``moe`` with
``router="token_table"``, plain silu experts), or none.  A looped range of layers becomes repeated
schedule entries, each owning a cache; the first entry of every pass adds the pass's vector, and of
every pass but the first the input embedding too.  The logits are scaled (``linear_head`` with
``scale``).

Checkpoint names: ``embed``, ``head``, ``final.norm{,.b,.alpha}``, ``loop.step`` and, per layer
``l<i>``: ``norm1{,.b,.alpha}``, ``mix.{q,q.b,k,k.b,g,rel,o,o.b}``, ``mlp.{gate,up,down}`` or
``mlp.e<j>.{gate,up,down}`` with ``mlp.table``.  ``q``, ``k`` and ``g`` are concatenated into
``qkg_proj``; gate/up pairs and experts are stacked as for every other architecture here.
The reference has no such design.
"""

from __future__ import annotations

from dataclasses import replace
from typing import Any, List, Mapping, Optional, Tuple

from ..config.rumalorn import ARCHITECTURES, MAX_POSITION, RumalornConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..errors import ConfigError
from ..registry import Architecture, register_architecture
from ..weights.binder import FusionRule

DEFAULT_BUCKETS = 32  # rows of a bias table when neither a weight file nor the config says (random models)


def layer_passes(cfg: RumalornConfig) -> List[Tuple[int, bool, Optional[int]]]:
    """The order layers run in: (layer, add the input embedding first, pass vector to add first)."""
    n = len(cfg.layers)
    out: List[Tuple[int, bool, Optional[int]]] = []
    if not cfg.loop_times:
        return [(l, False, None) for l in range(n)]
    for l in range(cfg.loop_start):
        out.append((l, False, None))
    for t in range(cfg.loop_times):
        for l in range(cfg.loop_start, cfg.loop_stop):
            first = l == cfg.loop_start
            out.append((l, first and t > 0, t if first else None))
    for l in range(cfg.loop_stop, n):
        out.append((l, False, None))
    return out


def build_spec(cfg: RumalornConfig) -> ModelSpec:
    norm = PartSpec("dynamic_tanh", dict(size=cfg.width))
    block = PartSpec("parallel_residual", dict(hidden=cfg.width, norm=norm, norm_name="norm1"))
    layers: List[LayerSpec] = []
    # random models: spreads that keep every activation of order one, so that a fault anywhere shows in the logits
    w_in = cfg.width ** -0.5
    for i, l in enumerate(cfg.layers):
        a = l.mixer
        buckets = cfg.rel_buckets[i] if i < len(cfg.rel_buckets) and cfg.rel_buckets[i] else DEFAULT_BUCKETS
        mixer = PartSpec("tied_kv_attention", dict(
            hidden=cfg.width, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale,
            proj_bias=True, gate=True, buckets=buckets, max_distance=a.bias_max,
            position=PartSpec("log_temperature", dict(coef=a.q_temp_coef, every=a.q_temp_every)), window=None,
            init_std=(w_in, 0.5 * (a.heads * a.dim) ** -0.5)))
        if l.mlp is None:
            ffn = PartSpec("none")
        elif l.mlp.kind == "dense":
            ffn = PartSpec("gated_mlp", dict(hidden=cfg.width, inter=l.mlp.ff, act="swigluoai", alpha=1.702,
                                             limit=l.mlp.limit, init_std=(w_in, 0.5 * l.mlp.ff ** -0.5)))
        else:
            ffn = PartSpec("moe", dict(hidden=cfg.width, inter=l.mlp.ff, n_experts=l.mlp.experts, top_k=l.mlp.top,
                                       router="token_table", vocab=cfg.vocab, act="silu", scale=1.0,
                                       init_std=(w_in, 0.5 * l.mlp.ff ** -0.5)))
        layers.append(LayerSpec(name=f"l{i}", block=block, mixer=mixer, ffn=ffn, mixer_name="mix", ffn_name="mlp"))
    schedule = tuple(ScheduleEntry(l, None, emb, vec) for l, emb, vec in layer_passes(cfg))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
        schedule=schedule,
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=cfg.width, init_std=1.0)),
        final_norm=norm,
        head=PartSpec("linear_head", dict(tied=False, scale=cfg.logit_scale, init_std=w_in)),
        max_position=MAX_POSITION,
        embedding_name="embed_tokens", final_norm_name="final.norm", head_name="head",
        pass_vectors=PartSpec("pass_vectors", dict(passes=cfg.loop_times, name="step")) if cfg.loop_times else None,
        pass_vectors_name="loop",
        source=cfg,
    )


def fusion_rules(cfg: RumalornConfig) -> List[FusionRule]:
    """How checkpoint tensors combine into (or are renamed to) the model's tensors."""
    one = lambda target, source: FusionRule(target, [source], "cat0")  # noqa: E731  (a plain rename)
    rules = [one("embed_tokens.weight", "embed"), one("head.weight", "head"),
             one("final.norm.weight", "final.norm"), one("final.norm.bias", "final.norm.b")]
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        a = l.mixer
        rules += [one(f"{p}.norm1.weight", f"{p}.norm1"), one(f"{p}.norm1.bias", f"{p}.norm1.b"),
                  FusionRule(f"{p}.mix.qkg_proj.weight", [f"{p}.mix.q", f"{p}.mix.k", f"{p}.mix.g"], "cat0",
                             [a.heads * a.dim, a.kv_heads * a.dim, a.heads]),
                  one(f"{p}.mix.q_bias", f"{p}.mix.q.b"), one(f"{p}.mix.k_bias", f"{p}.mix.k.b"),
                  one(f"{p}.mix.o_proj.weight", f"{p}.mix.o"), one(f"{p}.mix.o_proj.bias", f"{p}.mix.o.b")]
        if l.mlp is None:
            continue
        if l.mlp.kind == "dense":
            rules += [FusionRule(f"{p}.mlp.gate_up_proj.weight", [f"{p}.mlp.gate", f"{p}.mlp.up"], "cat0"),
                      one(f"{p}.mlp.down_proj.weight", f"{p}.mlp.down")]
        else:
            E = l.mlp.experts
            rules += [FusionRule(f"{p}.mlp.experts.gate_up_proj",
                                 [f"{p}.mlp.e{e}.{w}" for e in range(E) for w in ("gate", "up")], "stack_pairs"),
                      FusionRule(f"{p}.mlp.experts.down_proj", [f"{p}.mlp.e{e}.down" for e in range(E)], "stack")]
    return rules


def parse(raw: Mapping[str, Any], num_layers: Optional[int] = None) -> RumalornConfig:
    cfg = RumalornConfig.from_dict(raw, num_layers=num_layers)
    # a config written for a random model may say how many rows its bias tables have
    given = tuple(int((l.get("mixer") or {}).get("buckets", 0) or 0) for l in raw["layers"][: len(cfg.layers)])
    return replace(cfg, rel_buckets=given) if any(given) else cfg


def sizes_from_weights(cfg: RumalornConfig, shapes: Mapping[str, Tuple[int, ...]]) -> RumalornConfig:
    """The number of rows of each layer's bias table is the shape of ``l<i>.mix.rel``."""
    rows = []
    for i in range(len(cfg.layers)):
        shape = shapes.get(f"l{i}.mix.rel")
        if shape is None:
            rows.append(cfg.rel_buckets[i] if i < len(cfg.rel_buckets) else 0)
            continue
        if len(shape) != 2 or shape[0] < 2:
            raise ConfigError(f"l{i}.mix.rel has shape {list(shape)}: [buckets >= 2, heads] expected")
        rows.append(int(shape[0]))
    return replace(cfg, rel_buckets=tuple(rows))


ARCH = Architecture(
    names=ARCHITECTURES,
    parse_config=parse,
    build_spec=build_spec,
    fusion_rules=fusion_rules,
    sizes_from_weights=sizes_from_weights,
)
register_architecture(ARCH)

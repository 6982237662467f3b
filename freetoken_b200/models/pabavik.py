"""Pabavik: from its typed config to a model description, and its checkpoint names.

Layers are ``sandwich_residual`` blocks (an RMS norm of the ``1 + w`` form on both sides of every
sub-layer).  The mixer is either ``gqa_attention`` with a sliding window, a sink of logit 0 in the softmax's
denominator, per-head RMS norm of queries and keys (plain weight), rotary positions on a part of each
head, an element-wise sigmoid output gate and, for a layer with ``kv_from``, the cache of an earlier
layer (its schedule entry reads that layer's entry); or ``gated_linear_attention``.  The feed-forward is
``moe`` with the router's bias inside the logits and the softmax taken over the chosen experts only
(``softmax_of_chosen``), clamped experts (``swigluoai``, alpha 1.702) and a shared expert with a clamp of
its own, or none.  The embedding is scaled, the logits are soft-capped.

Checkpoint names: ``embed``, ``head``, ``final.norm`` and, per layer ``l<i>``: ``norm1``, ``norm1b``,
``norm2``, ``norm2b``; attention ``mix.{q,k,v,g,o}``, ``mix.q.norm``, ``mix.k.norm`` (a layer with
``kv_from`` has no ``k``, ``v``, ``k.norm``); gated linear attention ``mix.{q,k,v,g,a1,a2,a2.b,norm,o}``;
``mlp.e<j>.{gate,up,down}``, ``mlp.router``, ``mlp.router.b``, ``mlp.shared.{gate,up,down}``.  The
projections of a mixer's input are concatenated into one matrix; gate/up pairs and experts are stacked as
for every other architecture here.  The reference has no such design.
"""

from __future__ import annotations

from dataclasses import replace
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..config.pabavik import ARCHITECTURES, DEFAULT_DECAY_RANK, MAX_POSITION, PabavikConfig, PabavikGla
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..errors import ConfigError
from ..registry import Architecture, register_architecture
from ..weights.binder import FusionRule

SINK_LOGIT = 0.0       # the design's sink adds e^0 = 1 to the softmax's denominator
EXPERT_ALPHA = 1.702   # g sigmoid(alpha g) (u + 1)


def cache_windows(cfg: PabavikConfig) -> Dict[int, Optional[int]]:
    """How long each owning attention layer's cache keeps a token: the longest window among the layer
    itself and the layers that read its keys and values (None: for ever)."""
    out: Dict[int, Optional[int]] = {}
    for i, l in enumerate(cfg.layers):
        if l.type != "attention":
            continue
        owner = i if l.mixer.kv_from is None else l.mixer.kv_from
        w = l.mixer.window
        if owner not in out:
            out[owner] = w
        elif out[owner] is not None:
            out[owner] = None if w is None else max(out[owner], w)
    return out


def build_spec(cfg: PabavikConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.norm_eps, gemma=True))
    block = PartSpec("sandwich_residual", dict(hidden=cfg.width, norm=norm,
                                               norm_names=("norm1", "norm1b", "norm2", "norm2b")))
    keep = cache_windows(cfg)
    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    # random models: spreads that keep every activation of order one, so that a fault anywhere shows in the logits
    w_in = cfg.width ** -0.5
    for i, l in enumerate(cfg.layers):
        a = l.mixer
        if l.type == "attention":
            position = (PartSpec("rope_neox", dict(rotary_dim=a.rot_dims, theta=a.rot_base, precise=True))
                        if a.rot_dims else PartSpec("none"))
            own = a.kv_from is None
            params = dict(hidden=cfg.width, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim, v_head_dim=a.vdim,
                          qk_norm=True, eps=cfg.norm_eps, gemma=False, position=position, window=a.window,
                          scale=a.scale, sink=SINK_LOGIT, out_gate="sigmoid", own_kv=own,
                          init_std=(2.0 * w_in, (a.heads * a.vdim) ** -0.5))
            if own:
                params["cache_window"] = keep[i]
            mixer = PartSpec("gqa_attention", params)
            schedule.append(ScheduleEntry(i, None if own else a.kv_from))
        else:
            mixer = PartSpec("gated_linear_attention", dict(
                hidden=cfg.width, n_heads=a.heads, head_dim=a.dim, v_head_dim=a.vdim, tau=a.tau,
                decay_rank=a.decay_rank or DEFAULT_DECAY_RANK, eps=cfg.norm_eps,
                init_std=(w_in, (a.heads * a.vdim) ** -0.5)))
            schedule.append(ScheduleEntry(i, None))
        if l.mlp is None:
            ffn = PartSpec("none")
        else:
            f = l.mlp
            ffn = PartSpec("moe", dict(hidden=cfg.width, inter=f.ff, n_experts=f.experts, top_k=f.top,
                                       scoring="softmax_of_chosen", bias=True, scale=1.0, act="swigluoai",
                                       alpha=EXPERT_ALPHA, limit=f.limit, shared_inter=f.shared_ff,
                                       shared_limit=f.shared_limit if f.shared_ff else f.limit,
                                       init_std=(w_in, f.ff ** -0.5)))
        layers.append(LayerSpec(name=f"l{i}", block=block, mixer=mixer, ffn=ffn, mixer_name="mix", ffn_name="mlp"))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
        schedule=tuple(schedule),
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=cfg.width, init_std=1.0,
                                                   scale=cfg.embedding_scale)),
        final_norm=norm,
        head=PartSpec("linear_head", dict(tied=False, softcap=cfg.logit_softcap, init_std=w_in)),
        max_position=MAX_POSITION,
        embedding_name="embed_tokens", final_norm_name="final.norm", head_name="head",
        source=cfg,
    )


def fusion_rules(cfg: PabavikConfig) -> List[FusionRule]:
    """How checkpoint tensors combine into (or are renamed to) the model's tensors."""
    one = lambda target, source: FusionRule(target, [source], "cat0")  # noqa: E731  (a plain rename)
    rules = [one("embed_tokens.weight", "embed"), one("head.weight", "head"), one("final.norm.weight", "final.norm")]
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        a = l.mixer
        rules += [one(f"{p}.norm1.weight", f"{p}.norm1"), one(f"{p}.norm1b.weight", f"{p}.norm1b")]
        if l.type == "attention":
            own = a.kv_from is None
            names = ["q"] + (["k", "v"] if own else []) + ["g"]
            sizes = [a.heads * a.dim] + ([a.kv_heads * a.dim, a.kv_heads * a.vdim] if own else []) + [a.heads * a.vdim]
            rules += [FusionRule(f"{p}.mix.qkv_proj.weight", [f"{p}.mix.{n}" for n in names], "cat0", sizes),
                      one(f"{p}.mix.q_norm.weight", f"{p}.mix.q.norm"), one(f"{p}.mix.o_proj.weight", f"{p}.mix.o")]
            if own:
                rules.append(one(f"{p}.mix.k_norm.weight", f"{p}.mix.k.norm"))
        else:
            rank = a.decay_rank or DEFAULT_DECAY_RANK
            rules += [FusionRule(f"{p}.mix.in_proj.weight", [f"{p}.mix.{n}" for n in ("q", "k", "v", "g", "a1")], "cat0",
                                 [a.heads * a.dim, a.heads * a.dim, a.heads * a.vdim, a.heads * a.vdim, rank]),
                      one(f"{p}.mix.decay_proj.weight", f"{p}.mix.a2"), one(f"{p}.mix.decay_proj.bias", f"{p}.mix.a2.b"),
                      one(f"{p}.mix.norm.weight", f"{p}.mix.norm"), one(f"{p}.mix.o_proj.weight", f"{p}.mix.o")]
        if l.mlp is None:
            continue
        E = l.mlp.experts
        rules += [one(f"{p}.norm2.weight", f"{p}.norm2"), one(f"{p}.norm2b.weight", f"{p}.norm2b"),
                  FusionRule(f"{p}.mlp.experts.gate_up_proj",
                             [f"{p}.mlp.e{e}.{w}" for e in range(E) for w in ("gate", "up")], "stack_pairs"),
                  FusionRule(f"{p}.mlp.experts.down_proj", [f"{p}.mlp.e{e}.down" for e in range(E)], "stack"),
                  one(f"{p}.mlp.gate.weight", f"{p}.mlp.router"),
                  one(f"{p}.mlp.e_score_correction_bias", f"{p}.mlp.router.b")]
        if l.mlp.shared_ff:
            rules += [FusionRule(f"{p}.mlp.shared_experts.gate_up_proj.weight",
                                 [f"{p}.mlp.shared.gate", f"{p}.mlp.shared.up"], "cat0"),
                      one(f"{p}.mlp.shared_experts.down_proj.weight", f"{p}.mlp.shared.down")]
    return rules


def parse(raw: Mapping[str, Any], num_layers: Optional[int] = None) -> PabavikConfig:
    return PabavikConfig.from_dict(raw, num_layers=num_layers)


def sizes_from_weights(cfg: PabavikConfig, shapes: Mapping[str, Tuple[int, ...]]) -> PabavikConfig:
    """The width of a gated-linear-attention layer's low-rank decay projection is the first size of ``l<i>.mix.a1``."""
    layers = list(cfg.layers)
    for i, l in enumerate(layers):
        if l.type != "gla":
            continue
        shape = shapes.get(f"l{i}.mix.a1")
        if shape is None:
            continue
        if len(shape) != 2 or shape[0] < 1 or shape[1] != cfg.width:
            raise ConfigError(f"l{i}.mix.a1 has shape {list(shape)}: [rank >= 1, {cfg.width}] expected")
        layers[i] = replace(l, mixer=replace(l.mixer, decay_rank=int(shape[0])))
    return replace(cfg, layers=tuple(layers))


ARCH = Architecture(
    names=ARCHITECTURES,
    parse_config=parse,
    build_spec=build_spec,
    fusion_rules=fusion_rules,
    sizes_from_weights=sizes_from_weights,
)
register_architecture(ARCH)

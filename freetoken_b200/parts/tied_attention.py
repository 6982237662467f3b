"""Softmax attention whose values are its keys, with positions entering through the scores only.

Per token: one projection gives the queries, the keys and one gate logit per query head
(``qkg_proj``, rows q, k, g); biases of q and k are added to the projected heads, the queries are
multiplied by a factor of their position (a :class:`PositionEncoding` with ``scale_table``), keys go to
the paged cache, and the only cached slab serves the score product and the value product alike
(``v = k``).  The score of query ``i`` and key ``j <= i`` is ``(q_i . k_j) scale + rel[bucket(i - j), head]``
with a learned table ``rel [buckets, heads]``: distances below ``buckets / 2`` have a row each, the
others share rows that are evenly spaced in the logarithm up to ``max_distance``
(:func:`distance_buckets`).  Each head's output is multiplied by the sigmoid of its gate logit and the
output projection has a bias.  Every option (biases, gate, temperature, distance bias) can be left
out, which leaves plain grouped-query attention over a key-only cache.

Heads whose size is not a multiple of 16 are padded with zeros in the cache and in q (a zero column
changes neither scores nor, with ``v = k``, the output's live columns); the output projection's
columns are padded to match when the weights are bound.

No counterpart in the reference, whose attention layers all rotate and keep values
(python/freetoken/models/minimax_m3/attention.py:79-119 is the closest); the kernels are the
framework's own (``norm_rope_store`` with bias and position factor, ``paged_attention`` with
``dist_bias`` and ``v_slab is k_slab``).
"""

from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from ..config.spec import PagedKVNeed, ParamSpec, PartSpec
from ..engine.attention_plan import DEAL_MOST_PIECES
from ..errors import ConfigError
from ..kernels import ops
from .attention import attention_kernel_form
from .base import MIXERS, BuildEnv, Mixer, StepState
from .rope import shared_position


def distance_buckets(n_buckets: int, max_distance: float) -> List[int]:
    """Bucket of every distance up to the first one that lands in the last bucket (all longer ones
    do too).  ``bucket(n) = n`` below ``half = n_buckets // 2``; above,
    ``min(n_buckets - 1, half + floor(ln(n / half) / ln(max_distance / half) * (n_buckets - half)))``."""
    half = n_buckets // 2
    if n_buckets < 2 or half < 1 or max_distance <= half:
        raise ConfigError(f"distance bias: {n_buckets} buckets up to distance {max_distance}: needs two buckets "
                          f"at least and a largest distance beyond half of them")
    out: List[int] = []
    n = 0
    while True:
        if n < half:
            b = n
        else:
            b = min(n_buckets - 1, half + int(math.floor(math.log(n / half) / math.log(max_distance / half)
                                                         * (n_buckets - half))))
        out.append(b)
        if b == n_buckets - 1 or n > 1 << 24:
            return out
        n += 1


@MIXERS.register("tied_kv_attention")
class TiedKVAttention(Mixer):
    """params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``, ``scale`` (None = head_dim^-0.5),
    ``proj_bias`` (bool: q, k and output projection have biases), ``gate`` (bool), ``buckets`` and
    ``max_distance`` (0 buckets = no distance bias), ``position`` (PartSpec with a ``scale_table``, or
    None), ``window`` (None or tokens), ``init_std``."""

    graph_safe = True  # running a step twice writes the same keys again

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden"])
        self.n_heads = int(spec["n_heads"])
        self.n_kv_heads = int(spec["n_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        if self.n_heads < 1 or self.n_kv_heads < 1 or self.n_heads % self.n_kv_heads:
            raise ConfigError("tied_kv_attention: n_heads must be a multiple of n_kv_heads")
        if not 1 <= self.head_dim <= 256:
            raise ConfigError(f"tied_kv_attention: head_dim={self.head_dim} must be in [1, 256]")
        self.pad_dim = -(-self.head_dim // 16) * 16  # what the attention kernels take
        self.group = self.n_heads // self.n_kv_heads
        self.scale = float(spec.get("scale") or self.head_dim ** -0.5)
        self.proj_bias = bool(spec.get("proj_bias", False))
        self.gate = bool(spec.get("gate", False))
        self.buckets = int(spec.get("buckets", 0) or 0)
        self.max_distance = float(spec.get("max_distance", 0) or 0)
        self.window: Optional[int] = spec.get("window")
        self._bucket_of = distance_buckets(self.buckets, self.max_distance) if self.buckets else None
        pos = spec.get("position")
        self.position = shared_position(pos, env) if pos is not None else None
        if self.position is not None and not hasattr(self.position, "scale_table"):
            raise ConfigError("tied_kv_attention: the position encoding must give a factor per position")
        # more query heads per KV head than the kernels' tiles have rows: every KV head is taken as `kv_split` heads of
        # the same keys (the smallest split that fits), and the work is planned for that many heads
        rows, _ = attention_kernel_form(env.dtype)
        most = rows if env.dtype != torch.bfloat16 else 64
        self.kv_split = next(s for s in range(1, self.group + 1) if self.group % s == 0 and self.group // s <= most)
        self.plan_group = self.group // self.kv_split
        self.plan_kv_heads = self.n_kv_heads * self.kv_split
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv_heads * self.head_dim
        self.proj_rows = self.q_dim + self.kv_dim + (self.n_heads if self.gate else 0)
        self._dist_bias: Optional[torch.Tensor] = None
        self._o_weight: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        std = self.spec.get("init_std")  # spread of random weights: (projections of the input, output projection)
        std_in, std_out = (float(std[0]), float(std[1])) if std else (0.02, 0.02)
        out = {
            "qkg_proj.weight": ParamSpec((self.proj_rows, self.hidden), init=("normal", 0.0, std_in)),
            "o_proj.weight": ParamSpec((self.hidden, self.q_dim), init=("normal", 0.0, std_out)),
        }
        if self.proj_bias:
            out["q_bias"] = ParamSpec((self.q_dim,), "float32", ("normal", 0.0, 0.3), store="bfloat16")
            out["k_bias"] = ParamSpec((self.kv_dim,), "float32", ("normal", 0.0, 0.3), store="bfloat16")
            out["o_proj.bias"] = ParamSpec((self.hidden,), "compute", ("normal", 0.0, 0.1))
        if self.buckets:
            out["rel"] = ParamSpec((self.buckets, self.n_heads), "float32", ("normal", 0.0, 0.5), store="bfloat16")
        return out

    def bind(self, tensors) -> None:
        super().bind(tensors)
        self._dist_bias = None
        if self.buckets:  # the table by distance, one row per head: what the kernels index
            idx = torch.tensor(self._bucket_of, dtype=torch.long, device=self.params["rel"].device)
            self._dist_bias = self.params["rel"].index_select(0, idx).t().contiguous()
        w = self.params["o_proj.weight"]
        if self.pad_dim != self.head_dim:  # zero columns where the attention output has its padding
            wp = torch.zeros((self.hidden, self.n_heads, self.pad_dim), dtype=w.dtype, device=w.device)
            wp[:, :, : self.head_dim] = w.view(self.hidden, self.n_heads, self.head_dim)
            w = wp.view(self.hidden, self.n_heads * self.pad_dim)
        self._o_weight = w

    def cache_need(self):
        return PagedKVNeed((("k", self.n_kv_heads, self.pad_dim),), self.window)

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        rows = n_tokens * (self.proj_rows + 2 * self.n_heads * self.pad_dim + self.hidden) * item
        return rows + DEAL_MOST_PIECES * 148 * 256 * (self.pad_dim + 2) * 4

    # ------------------------------------------------------------------ step
    def kernel_form(self, decode_only: bool, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0):
        # (of the tcgen05 kernels the ones with a single query tile a piece take a bias by distance)
        return attention_kernel_form(self.env.dtype, decode_only, self.plan_group, n_tokens,
                                     self.pad_dim if self.kv_split == 1 and self.window is None else 0, page_size,
                                     self.window, longest_span,
                                     one_tile_only=True)

    def plan_key(self, decode_only: bool = False, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0):
        rows, few_rows = self.kernel_form(decode_only, n_tokens, page_size, longest_span)
        return ("attention", self.plan_group, rows, self.window, self.plan_kv_heads, self.pad_dim, few_rows)

    def prepare(self, builder) -> None:
        n_tokens = sum(q for q, _ in builder.seg_lens)
        page_size = builder.engine.config.page_size if builder.engine is not None else 0
        rows, few_rows = self.kernel_form(builder.decode_only, n_tokens, page_size, builder.longest_span())
        self._step_plan = builder.attention_plan(self.plan_group, rows, self.window, self.plan_kv_heads, self.pad_dim,
                                                 few_rows)

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        D, Dp, H, G = self.head_dim, self.pad_dim, self.n_heads, self.n_kv_heads
        qkg = ws.get("tied.qkg", (T, self.proj_rows), dt, (cap, self.proj_rows))
        ops.linear(h, self.params["qkg_proj.weight"], qkg)
        q = ws.get("tied.q", (T, H, Dp), dt, (cap, H, Dp))
        q_sec = dict(first_head=0, n_heads=H, norm_weight=None, rotate=False, dense_out=q, dst_head_dim=Dp,
                     bias=self.params.get("q_bias"),
                     pos_scale=self.position.scale_table() if self.position is not None else None)
        sections = [q_sec]
        if writes_cache:
            sections.append(dict(first_head=H, n_heads=G, norm_weight=None, rotate=False, slab=cache.slabs["k"],
                                 slot_map=cache.slot_map, dst_head_dim=Dp, bias=self.params.get("k_bias")))
        ops.norm_rope_store(qkg, D, 0, step.positions, None, 0.0, False, sections)
        plan = step.attention_plans[self._step_plan]
        o = ws.get("tied.o", (T, H, Dp), dt, (cap, H, Dp))
        k = cache.slabs["k"]
        ops.paged_attention(q, k, k, cache.block_table, step.seg_info, len(step.segments), plan.items_dev,
                            plan.n_items, plan.part_o, plan.part_ml, o, self._step_plan[2], self.scale, self.window,
                            few_rows=self._step_plan[6], dist_bias=self._dist_bias, kv_split=self.kv_split)
        if self.gate:
            ops.head_gate(o, qkg[:, self.q_dim + self.kv_dim:])
        out = ws.get("tied.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(o.view(T, H * Dp), self._o_weight, out, bias=self.params.get("o_proj.bias"))
        return out

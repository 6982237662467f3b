"""Gated linear attention: a recurrent mixer with a matrix state per head and a decay per key channel.

Per token and head, with ``q, k`` of size ``D`` and ``v`` of size ``Dv``::

    a_t = sigmoid(W_a2 (W_a1 h_t) + b)^(1 / tau)          one decay per key channel, through a low rank
    S_t = diag(a_t) S_(t-1) + k_t v_t^T                   [D, Dv], 32-bit, carried from token to token
    o_t = S_t^T (q_t D^-1/2)

Each head's ``o_t`` is RMS-normed over ``Dv`` (one plain weight for all heads), multiplied element by element
by ``silu(W_g h_t)`` and projected.  One library product gives q, k, v, the gate and the low-rank decay
input (``in_proj``, rows in that order); the decay logits are a second, 32-bit product; decays, state and
outputs are 32-bit (``ops.gla_scan``), norm and gate one more kernel (``ops.gated_heads``).

The state lives in a slot of the cache manager's state pool (:class:`StateNeed`), starts from zero for a
request's first tokens, and a step may bring any number of a request's tokens: they are cut into chunks
that the kernel runs side by side (:func:`chunk_list`).  The reference has no recurrent mixer in the
models it serves; its state pool (python/freetoken/kvcache/linear_state_pool.py:32-183) is the
counterpart of the slots used here.
"""

from __future__ import annotations

from typing import Any, Dict, List, Sequence, Tuple

import numpy as np
import torch

from ..config.spec import ParamSpec, PartSpec, StateNeed
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, BuildEnv, Mixer, StepState

DEFAULT_CHUNK = 64


def chunk_list(seg_lens: Sequence[Tuple[int, int]], chunk: int) -> Tuple[np.ndarray, np.ndarray, bool, bool]:
    """A step's segments ``(q_len, kv_len)`` cut into chunks of at most ``chunk`` tokens.

    Returns ``chunks [n, 4]`` (segment, first token within the segment's tokens, tokens, place among the
    segment's chunks), ``seg_chunks [S, 2]`` (first chunk, chunks), and whether any segment has one chunk /
    several chunks."""
    chunks: List[Tuple[int, int, int, int]] = []
    per_seg = np.zeros((len(seg_lens), 2), dtype=np.int32)
    single = multi = False
    for s, (q_len, _) in enumerate(seg_lens):
        n = max(1, -(-q_len // chunk))
        per_seg[s] = (len(chunks), n)
        single |= n == 1
        multi |= n > 1
        for c in range(n):
            chunks.append((s, c * chunk, min(chunk, q_len - c * chunk), c))
    return np.asarray(chunks, dtype=np.int32).reshape(-1, 4), per_seg, single, multi


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    """params: ``hidden``, ``n_heads``, ``head_dim`` (keys and queries), ``v_head_dim``, ``tau``, ``decay_rank``
    (width of the low-rank decay projection), ``eps`` (of the output norm), ``q_scale`` (None = head_dim^-0.5),
    ``chunk`` (tokens per chunk of a long portion), ``init_std``."""

    graph_safe = False  # running a step twice would advance the state twice
    graph_recordable = True  # but everything a step does is decided on the device: a decode step can be recorded

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden"])
        self.n_heads = int(spec["n_heads"])
        self.head_dim = int(spec["head_dim"])
        self.v_dim = int(spec.get("v_head_dim") or self.head_dim)
        self.tau = float(spec.get("tau", 1.0))
        self.rank = int(spec["decay_rank"])
        self.eps = float(spec.get("eps", 1e-5))
        self.chunk = int(spec.get("chunk", DEFAULT_CHUNK))
        if self.n_heads < 1 or not 1 <= self.head_dim <= 256 or self.v_dim < 1 or self.rank < 1 or self.chunk < 1:
            raise ConfigError("gated_linear_attention: heads, head sizes (keys at most 256), decay rank and chunk "
                              "must be positive")
        if not self.tau > 0:
            raise ConfigError("gated_linear_attention: tau must be positive")
        self.q_scale = float(spec.get("q_scale") or self.head_dim ** -0.5)
        H, D, Dv = self.n_heads, self.head_dim, self.v_dim
        self.k_row = H * D
        self.v_row = 2 * H * D
        self.g_row = self.v_row + H * Dv
        self.a_row = self.g_row + H * Dv
        self.proj_rows = self.a_row + self.rank

    # ------------------------------------------------------------------ tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        std = self.spec.get("init_std")  # spread of random weights: (projections of the input, output projection)
        std_in, std_out = (float(std[0]), float(std[1])) if std else (0.02, 0.02)
        H, D, Dv = self.n_heads, self.head_dim, self.v_dim
        return {
            "in_proj.weight": ParamSpec((self.proj_rows, self.hidden), init=("normal", 0.0, std_in)),
            "decay_proj.weight": ParamSpec((H * D, self.rank), init=("normal", 0.0, self.rank ** -0.5 if std else 0.02)),
            "decay_proj.bias": ParamSpec((H * D,), "float32", ("normal", 2.0 if std else 0.0, 1.0 if std else 0.02),
                                         store="bfloat16"),
            "norm.weight": ParamSpec((Dv,), "float32", ("normal", 1.0, 0.2 if std else 0.02), store="bfloat16"),
            "o_proj.weight": ParamSpec((self.hidden, H * Dv), init=("normal", 0.0, std_out)),
        }

    def cache_need(self):
        return StateNeed((("s", (self.n_heads, self.head_dim, self.v_dim), "float32"),))

    def max_chunks(self, n_tokens: int) -> int:
        return n_tokens // self.chunk + self.env.max_decode_rows + 1

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        H, D, Dv = self.n_heads, self.head_dim, self.v_dim
        rows = n_tokens * ((self.proj_rows + H * Dv + self.hidden) * item + (H * D + H * Dv) * 4)
        return rows + self.max_chunks(n_tokens) * H * D * (Dv + 1) * 4

    # ------------------------------------------------------------------ step
    def prepare(self, builder) -> None:
        """Put the step's chunk lists into its metadata (once per chunk size, whatever the number of layers)."""
        name = f"gla.chunks.{self.chunk}"
        found = getattr(builder, "_gla_lists", None)
        if found is None:
            found = builder._gla_lists = {}
        if name not in found:
            chunks, per_seg, single, multi = chunk_list(builder.seg_lens, self.chunk)
            builder.add(name, chunks)
            builder.add(name + ".segments", per_seg)
            found[name] = (chunks.shape[0], single, multi)
        self._step_lists = (name,) + found[name]

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        if not writes_cache:
            raise ConfigError("gated_linear_attention: a state cannot be shared between layers")
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        H, D, Dv = self.n_heads, self.head_dim, self.v_dim
        proj = ws.get("gla.proj", (T, self.proj_rows), dt, (cap, self.proj_rows))
        ops.linear(h, self.params["in_proj.weight"], proj)
        z = ws.get("gla.z", (T, H * D), torch.float32, (cap, H * D))
        ops.linear_f32(proj[:, self.a_row:], self.params["decay_proj.weight"], z)
        name, n_chunks, single, multi = self._step_lists
        tensors = step.extras["tensors"]
        carry = decay = None
        if multi:
            most = self.max_chunks(cap)
            carry = ws.get("gla.carry", (n_chunks, H, D, Dv), torch.float32, (most, H, D, Dv))
            decay = ws.get("gla.decay", (n_chunks, H, D), torch.float32, (most, H, D))
        o32 = ws.get("gla.o32", (T, H, Dv), torch.float32, (cap, H, Dv))
        ops.gla_scan(proj[:, : self.k_row], proj[:, self.k_row: self.v_row], proj[:, self.v_row: self.g_row], z,
                     self.params["decay_proj.bias"], self.tau, self.q_scale, cache.tensors["s"], step.state_slots,
                     step.seg_info, len(step.segments), tensors[name], n_chunks, tensors[name + ".segments"],
                     single, multi, carry, decay, o32)
        o = ws.get("gla.o", (T, H, Dv), dt, (cap, H, Dv))
        ops.gated_heads(o32, proj[:, self.g_row: self.a_row], o, Dv, "silu", self.params["norm.weight"], self.eps)
        out = ws.get("gla.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(o.view(T, H * Dv), self.params["o_proj.weight"], out)
        return out

"""Plain, slow Rumalorn: whole sequences, no cache, no batching, one function per mechanism.

Rumalorn is a decoder whose layers are *parallel* (one Dynamic-Tanh norm feeds mixer and
feed-forward, both outputs are added to the stream), whose attention has no rotation (positions
enter through a query temperature and a learned bias by bucketed distance), uses its keys as values,
and gates every head's output; feed-forwards are a clamped gated MLP or experts chosen by a table
over token ids; a range of layers may run several times, each pass with a cache of its own.

The file shares no code with ``freetoken_b200``: it parses config.json and reads the safetensors
file (through the ``safetensors`` package) itself.  Everything is computed in the working dtype
(float64 by default).
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- mechanisms
def dynamic_tanh(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    """``tanh(alpha x) w + b``: no mean, no variance."""
    return torch.tanh(alpha * x) * w + b


def distance_bucket(n: int, n_buckets: int, max_distance: float) -> int:
    """Row of the bias table for a key ``n`` positions back: one row per distance in the first
    half of the table, then rows spaced evenly in the logarithm up to ``max_distance``."""
    half = n_buckets // 2
    if n < half:
        return n
    x = math.log(n / half) / math.log(max_distance / half) * (n_buckets - half)
    return min(n_buckets - 1, half + int(math.floor(x)))


def distance_bias(rel: torch.Tensor, q_pos: Sequence[int], n_keys: int, max_distance: float) -> torch.Tensor:
    """``[heads, queries, keys]`` bias from the table ``rel [buckets, heads]`` (future keys get 0 here;
    the causal mask removes them)."""
    B, H = rel.shape
    far = max(q_pos) + 1
    row_of = torch.tensor([distance_bucket(n, B, max_distance) for n in range(far)])  # by distance
    out = torch.zeros(H, len(q_pos), n_keys, dtype=rel.dtype)
    for a, i in enumerate(q_pos):
        n = min(i + 1, n_keys)
        out[:, a, :n] = rel[row_of[i - torch.arange(n)]].T
    return out


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def tied_value_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, positions: Sequence[int],
                         past_k: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal softmax attention whose values are its keys.  ``h [T, width]`` are the tokens at
    ``positions``; ``past_k [P, kv_heads, dim]`` the keys of positions ``0..P-1`` before them."""
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = (h @ w["q"].T + w["q.b"]).view(T, H, D)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, D)
    temp = torch.tensor([query_temperature(p, m["q_temp"]["coef"], m["q_temp"]["every"]) for p in positions],
                        dtype=h.dtype)
    q = q * temp[:, None, None]
    keys = k if past_k is None else torch.cat([past_k, k], dim=0)
    n_keys = keys.shape[0]
    bias = distance_bias(w["rel"], positions, n_keys, m["bias_max"])
    gate = torch.sigmoid(h @ w["g"].T)  # [T, H]
    per = H // G
    out = torch.zeros(T, H, D, dtype=h.dtype)
    for hd in range(H):
        kh = keys[:, hd // per]  # [n_keys, D]
        s = (q[:, hd] @ kh.T) * m["scale"] + bias[hd]
        for a, i in enumerate(positions):
            s[a, i + 1:] = -math.inf
        p = torch.softmax(s, dim=-1)
        out[:, hd] = (p @ kh) * gate[:, hd:hd + 1]
    return out.reshape(T, H * D) @ w["o"].T + w["o.b"]


def clamped_gated_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    z = h @ gate.T
    return ((z * torch.sigmoid(z)) * (h @ up.T)) @ down.T


def table_routed_experts(h: torch.Tensor, token_ids: Sequence[int], w: Dict[str, torch.Tensor], top: int) -> torch.Tensor:
    """Each token's experts are listed in row ``token id`` of the table; each weighs ``1 / top``."""
    out = torch.zeros_like(h)
    table = w["table"]
    for t, tok in enumerate(token_ids):
        for j in range(top):
            e = int(table[tok, j])
            out[t] += expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0] / top
    return out


# --------------------------------------------------------------------------- the model
class PlainRumalorn:
    def __init__(self, folder: str, dtype: torch.dtype = torch.float64):
        from safetensors import safe_open

        with open(os.path.join(folder, "config.json")) as f:
            self.cfg = json.load(f)
        self.dtype = dtype
        self.w: Dict[str, torch.Tensor] = {}
        with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                self.w[name] = t.to(dtype) if t.is_floating_point() else t.long()
        self.vocab = int(self.cfg["vocab"])
        self.width = int(self.cfg["width"])

    def sub(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def layer_order(self) -> List[List[int]]:
        """Passes of layer indices: ``[[before...], [looped...] x times, [after...]]`` flattened per pass."""
        n = len(self.cfg["layers"])
        loop = self.cfg.get("loop")
        if not loop:
            return [list(range(n))]
        a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
        return [list(range(0, a))] + [list(range(a, b)) for _ in range(times)] + [list(range(b, n))]

    def norm(self, name: str, x: torch.Tensor) -> torch.Tensor:
        return dynamic_tanh(x, self.w[name], self.w[name + ".b"], self.w[name + ".alpha"])

    def layer(self, i: int, x: torch.Tensor, tokens: Sequence[int], positions: Sequence[int]) -> torch.Tensor:
        spec = self.cfg["layers"][i]
        assert spec["type"] == "attention"
        h = self.norm(f"l{i}.norm1", x)
        y = tied_value_attention(h, self.sub(f"l{i}.mix."), spec["mixer"], positions)
        mlp = spec.get("mlp")
        if mlp is not None:
            w = self.sub(f"l{i}.mlp.")
            if mlp["kind"] == "dense":
                y = y + clamped_gated_mlp(h, w, float(mlp["limit"]))
            else:
                y = y + table_routed_experts(h, tokens, w, int(mlp["router"]["top"]))
        return x + y

    def run(self, tokens: Sequence[int], trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        tokens = [int(t) for t in tokens]
        positions = list(range(len(tokens)))
        emb = self.w["embed"][torch.tensor(tokens)]
        x = emb.clone()
        passes = self.layer_order()
        loop = self.cfg.get("loop")
        for pi, layers in enumerate(passes):
            looped = bool(loop) and 1 <= pi <= int(loop["times"])
            if looped and layers:
                t = pi - 1
                if t > 0:
                    x = x + emb
                x = x + self.w["loop.step"][t]
            for i in layers:
                x = self.layer(i, x, tokens, positions)
                if trace is not None:
                    trace.append(x.clone())
        return x

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        x = self.run(tokens)
        return (self.norm("final.norm", x) @ self.w["head"].T) * float(self.cfg["logit_scale"])

    def layer_trace(self, tokens: Sequence[int]) -> torch.Tensor:
        tr: List[torch.Tensor] = []
        self.run(tokens, tr)
        return torch.stack(tr)

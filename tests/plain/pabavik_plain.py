"""Plain, slow Pabavik: whole sequences, no cache, no batching, one function per mechanism.

Pabavik is a decoder whose layers norm every sub-layer on both sides (``x += N_b(f(N_a(x)))``), whose
mixers are either windowed softmax attention with a sink in the denominator, rotary positions on a part
of each head, an element-wise output gate and, optionally, the keys and values of an earlier layer, or
gated linear attention with a decay per key channel; feed-forwards are experts chosen by the largest
router logits (weights: softmax over the chosen logits) plus a shared expert; the logits are soft-capped.

The file shares no code with ``freetoken_b200``: it parses config.json and reads the safetensors
file (through the ``safetensors`` package) itself.  Everything is computed in the working dtype
(float64 by default).
"""

from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- mechanisms
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, one_plus: bool) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` times ``w`` or ``1 + w``, over the last axis."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y * (1.0 + w) if one_plus else y * w


def rotate_part(x: torch.Tensor, positions: Sequence[int], n_rot: int, base: float) -> torch.Tensor:
    """``x [T, heads, dim]``: the first ``n_rot`` columns of each head turn, column ``i`` with column
    ``i + n_rot/2`` by the angle ``p base^(-2i/n_rot)``; the others stay."""
    half = n_rot // 2
    out = x.clone()
    p = torch.tensor(list(positions), dtype=x.dtype)
    for i in range(half):
        ang = p * base ** (-2.0 * i / n_rot)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = a * c - b * s
        out[:, :, i + half] = b * c + a * s
    return out


def attention_keys_values(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """Keys (normed per head, rotated) and values of a whole sequence: ``[T, kv_heads, dim]``, ``[T, kv_heads, vdim]``."""
    T = h.shape[0]
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w["k"].T).view(T, G, D)
    k = rms_norm(k, w["k.norm"], eps, one_plus=False)
    k = rotate_part(k, range(T), m["rot"]["dims"], m["rot"]["base"])
    v = (h @ w["v"].T).view(T, G, Dv)
    return k, v


def sink_window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                          k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Softmax attention of every token over itself and the ``mask.size - 1`` tokens before it, with a 1
    added to the softmax's denominator, the heads gated element by element and projected."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, D)
    q = rms_norm(q, w["q.norm"], eps, one_plus=False)
    q = rotate_part(q, range(T), m["rot"]["dims"], m["rot"]["base"])
    span = int(m["mask"]["size"])
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        lo = max(0, t - span + 1)
        for a in range(H):
            g = a // (H // G)
            s = (k[lo:t + 1, g] @ q[t, a]) * m["scale"]
            e = torch.exp(s)
            p = e / (1.0 + e.sum())
            out[t, a] = p @ v[lo:t + 1, g]
    gate = torch.sigmoid(h @ w["g"].T)
    return (out.reshape(T, H * Dv) * gate) @ w["o"].T


def gated_linear_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """A matrix state per head, ``S <- diag(a_t) S + k_t v_t^T`` with ``a_t = sigmoid(z_t)^(1/tau)`` per key
    channel, read out as ``S^T q_t``; each head's output normed, the heads gated by ``silu`` and projected."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, Dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, D)
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = rms_norm(out, w["norm"], eps, one_plus=False)
    gate = h @ w["g"].T
    return (out.reshape(T, H * Dv) * (gate * torch.sigmoid(gate))) @ w["o"].T


def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, bias: torch.Tensor, top: int):
    """Experts with the largest logits (ties: the lower index) and the softmax over their logits."""
    z = h @ router.T + bias
    order = sorted(range(z.shape[-1]), key=lambda e: (-float(z[e]), e))[:top]
    zz = z[order]
    p = torch.exp(zz - zz.max())
    return order, p / p.sum()


def expert_mixture(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict, gaps: Optional[List] = None) -> torch.Tensor:
    """``gaps`` collects, per token, how far the last chosen expert's logit lies above the best one left out."""
    T = h.shape[0]
    out = torch.zeros(T, w["e0.down"].shape[0], dtype=h.dtype)
    if gaps is not None:
        z = torch.sort(h @ w["router"].T + w["router.b"], dim=-1, descending=True).values
        top = f["router"]["top"]
        gaps.append(z[:, top - 1] - z[:, top] if top < z.shape[1] else torch.full((T,), float("inf"), dtype=h.dtype))
    for t in range(T):
        ids, ps = route(h[t], w["router"], w["router.b"], f["router"]["top"])
        for e, p in zip(ids, ps):
            out[t] += p * clamped_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"],
                                         f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], f["shared"]["limit"])
    return out


def soft_cap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(x / cap)


# --------------------------------------------------------------------------- the model
def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], streams: Optional[List] = None,
            gaps: Optional[List] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence; ``streams`` collects the residual stream after every layer,
    ``gaps`` every router's margins (see :func:`expert_mixture`)."""
    eps = cfg["norm"]["eps"]
    x = weights["embed"][torch.as_tensor(list(tokens))] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, weights[p + "norm1"], eps, one_plus=True)
        wm = sub(weights, p + "mix.")
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(h, wm, m, eps)
            k, v = kept[i if m.get("kv_from") is None else m["kv_from"]]
            a = sink_window_attention(h, wm, m, eps, k, v)
        elif layer["type"] == "gla":
            a = gated_linear_attention(h, wm, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(a, weights[p + "norm1b"], eps, one_plus=True)
        if layer.get("mlp") is not None:
            h = rms_norm(x, weights[p + "norm2"], eps, one_plus=True)
            x = x + rms_norm(expert_mixture(h, sub(weights, p + "mlp."), layer["mlp"], gaps), weights[p + "norm2b"], eps,
                             one_plus=True)
        if streams is not None:
            streams.append(x.clone())
    y = rms_norm(x, weights["final.norm"], eps, one_plus=True)
    return soft_cap(y @ weights["head"].T, cfg["logit_softcap"])


def load(folder: str, dtype: torch.dtype = torch.float64):
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights = {k: (v if v.dtype == torch.int32 else v.to(dtype))
               for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, weights


class PlainPabavik:
    """A model folder as the tests use one: ``vocab`` and float64 ``logits`` of a whole sequence."""

    def __init__(self, folder: str, dtype: torch.dtype = torch.float64):
        self.cfg, self.weights = load(folder, dtype)
        self.vocab = int(self.cfg["vocab"])

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        return forward(self.cfg, self.weights, tokens)

    def router_gaps(self, tokens: Sequence[int]) -> torch.Tensor:
        """Per token, the smallest margin by which any layer's router made its choice: where it is within the
        rounding of a bfloat16 run, such a run may choose another expert and its logits differ by more than rounding."""
        gaps: List[torch.Tensor] = []
        forward(self.cfg, self.weights, tokens, gaps=gaps)
        if not gaps:
            return torch.full((len(tokens),), float("inf"), dtype=torch.float64)
        return torch.stack(gaps).min(0).values

"""Plain, slow Kekopel: whole sequences, no cache, no batching, one function per mechanism.

Kekopel is a decoder whose sub-layers read the stream itself and are normed on their way out only
(``x += ls * g * unit(f(x + conv(x)))``, ``g`` one number, ``ls`` a vector, ``conv`` a short causal
convolution over time on every channel), and whose layers hand on a learned mix of the outputs of all
layers so far.  Mixers are latent attention (queries and keys/values through low-rank latents, one
rotated key part shared by all heads, a sliding window and a learned sink per head in the softmax's
denominator) or the matrix memory of xLSTM with its running maximum.  Feed-forwards are dense
(squared ReLU, biases) or experts chosen by the largest sigmoid scores, whose weight scales the
expert's *input*.

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
import torch.nn.functional as F


# --------------------------------------------------------------------------- mechanisms
def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def short_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``h [T, C]``, ``w [C, taps]``: ``h_t + sum_j w[:, j] h_(t - taps + 1 + j)``, zeros before the start."""
    T, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] = out[t] + w[:, j] * h[s]
    return out


def rotate_pairs(x: torch.Tensor, positions: Sequence[int], n_rot: int, base: float) -> torch.Tensor:
    """``x [T, ..., dim]``: among the first ``n_rot`` columns, column ``2i`` turns with column ``2i + 1`` by
    the angle ``p base^(-2i / n_rot)``; the others stay."""
    out = x.clone()
    p = torch.tensor(list(positions), dtype=x.dtype)
    shape = [len(positions)] + [1] * (x.dim() - 2)
    for i in range(n_rot // 2):
        ang = p * base ** (-2.0 * i / n_rot)
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n_rot, base = int(m["rot"]["dims"]), float(m["rot"]["base"])
    cq = unit(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).view(T, H, D + R)
    q_flat, q_rot = q[..., :D], rotate_pairs(q[..., D:], range(T), n_rot, base)
    kv = h @ w["dkv"].T
    c = unit(kv[:, :C], eps) * w["dkv.norm"]
    k_rot = rotate_pairs(kv[:, C:], range(T), n_rot, base)  # [T, R], one for all heads
    k_flat = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, Dv)
    span = m.get("mask", {}).get("size") if m.get("mask") else None
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        lo = 0 if span is None else max(0, t - int(span) + 1)
        for a in range(H):
            s = (k_flat[lo:t + 1, a] @ q_flat[t, a] + k_rot[lo:t + 1] @ q_rot[t, a]) * m["scale"]
            top = torch.maximum(s.max(), w["sink"][a])
            e = torch.exp(s - top)
            p = e / (e.sum() + torch.exp(w["sink"][a] - top))
            out[t, a] = p @ v[lo:t + 1, a]
    return out.reshape(T, H * Dv) @ w["o"].T


def matrix_memory(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, Dv)
    gi = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    gf = F.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    mx = torch.zeros(H, dtype=h.dtype)
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    out = unit(out, eps).reshape(T, H * Dv) * w["norm"]
    return (out * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    a = torch.relu(h @ w["up"].T + w["up.b"])
    return (a * a) @ w["down"].T + w["down.b"]


def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    g = h @ gate.T
    return (g * torch.sigmoid(g) * (h @ up.T)) @ down.T


def expert_mixture(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict, gaps: Optional[List] = None) -> torch.Tensor:
    E, top = int(f["router"]["experts"]), int(f["router"]["top"])
    s = torch.sigmoid(h @ w["router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = torch.argsort(s[t], descending=True, stable=True)
        if gaps is not None:
            z = (h[t] @ w["router"].T)[order]
            gaps.append(float(z[top - 1] - z[top]) if top < E else math.inf)
        for e in order[:top].tolist():
            out[t] += expert(s[t, e] * h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])
    return out


# --------------------------------------------------------------------------- the model
def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], streams: Optional[List] = None,
            gaps: Optional[List] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of a whole sequence.  ``streams`` receives what every layer hands on,
    ``gaps`` per expert layer and token the router logits' gap between the last chosen and the first
    unchosen expert."""
    eps = float(cfg["norm"]["eps"])
    x = weights["embed"][torch.tensor(list(tokens))]
    outputs = [x]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = short_conv(x, weights[p + "canon1"])
        mix = {"latent_attention": latent_attention, "mlstm": matrix_memory}[layer["type"]]
        a = mix(h, sub(weights, p + "mix."), layer["mixer"], eps)
        x = x + unit(a, eps) * weights[p + "norm1"] * weights[p + "ls1"]
        f = layer.get("mlp")
        if f is not None:
            h = short_conv(x, weights[p + "canon2"])
            if f["kind"] == "dense":
                y = dense_ff(h, sub(weights, p + "mlp."))
            else:
                per_layer = [] if gaps is not None else None
                y = expert_mixture(h, sub(weights, p + "mlp."), f, per_layer)
                if gaps is not None:
                    gaps.append(per_layer)
            x = x + unit(y, eps) * weights[p + "norm2"] * weights[p + "ls2"]
        outputs.append(x)
        mixw = weights[p + "dwa"]
        x = sum(mixw[j] * outputs[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x.clone())
    x = unit(x, eps) * weights["final.norm"]
    return x @ weights["head"].T


def load(folder: str, dtype: torch.dtype = torch.float64):
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            weights[k] = t if t.dtype in (torch.int32, torch.int64) else t.to(dtype)
    return cfg, weights


class PlainKekopel:
    def __init__(self, folder: str, dtype: torch.dtype = torch.float64):
        self.cfg, self.weights = load(folder, dtype)
        self.dtype = dtype
        self.vocab = int(self.cfg["vocab"])

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        return forward(self.cfg, self.weights, tokens).float()

    def streams(self, tokens: Sequence[int]) -> torch.Tensor:
        out: List[torch.Tensor] = []
        forward(self.cfg, self.weights, tokens, streams=out)
        return torch.stack(out).float()

    def router_gaps(self, tokens: Sequence[int]) -> torch.Tensor:
        """Per token, the smallest gap of any expert layer's choice (infinite without such a layer)."""
        gaps: List = []
        forward(self.cfg, self.weights, tokens, gaps=gaps)
        if not gaps:
            return torch.full((len(tokens),), math.inf)
        return torch.tensor(gaps, dtype=torch.float32).min(0).values

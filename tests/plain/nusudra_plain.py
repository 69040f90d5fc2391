"""Plain, slow Nusudra: whole sequences, no cache, no batching, one function per mechanism.

Nusudra is a decoder whose residual is carried in several streams (hyper-connections): a sub-layer reads a
weighted sum of the streams, and its result is written back to every stream while the streams are mixed among
themselves.  What a mixer reads is first blended, channel by channel, with what it read for the token before
(token shift).  Mixers: latent attention (one cached latent and one rotated key part under all heads, a
sigmoid gate per head), a pair of mixers side by side (softmax attention with projection biases, a bias by the
logarithm of the distance and a sink per head; a Mamba-2 state-space layer) whose normed results are averaged,
or the gated delta rule.  Feed-forward: dense, squared ReLU.

The file shares no code with ``freetoken_b200``: it parses config.json and reads the safetensors file itself.
Everything is computed in the working dtype (float64 by default).
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- mechanisms
def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def token_shift(h: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """``h [T, C]``: row ``t`` becomes ``h_t + (h_(t-1) - h_t) * mu`` with the rows as they were (zeros before row 0)."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]])
    return h + (prev - h) * mu


def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [T, C]``, ``w [C, taps]``: ``sum_j w[:, j] x_(t - taps + 1 + j) (+ bias)``, zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] = out[t] + w[:, j] * x[s]
    return out if bias is None else out + bias


def rotate_half(x: torch.Tensor, positions: Sequence[int], n_rot: int, base: float) -> torch.Tensor:
    """``x [T, ..., dim]``: among the first ``n_rot`` columns, column ``i`` turns with column ``i + n_rot / 2`` by
    the angle ``p base^(-2i / n_rot)``; the others stay."""
    out = x.clone()
    p = torch.tensor(list(positions), dtype=x.dtype)
    shape = [len(positions)] + [1] * (x.dim() - 2)
    half = n_rot // 2
    for i in range(half):
        ang = p * base ** (-2.0 * i / n_rot)
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {}
    n_rot, base = int(rot.get("dims", R)), float(rot.get("base", 10000.0))
    q = (h @ w["q"].T).view(T, H, D + R)
    q_flat, q_rot = q[..., :D], rotate_half(q[..., D:], range(T), n_rot, base)
    kv = h @ w["dkv"].T
    c = unit(kv[:, :C], eps) * w["dkv.norm"]
    k_rot = rotate_half(kv[:, C:], range(T), n_rot, base)  # [T, R], one for all heads
    k_flat = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, Dv)
    gate = torch.sigmoid(h @ w["g"].T)  # [T, H]
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        for a in range(H):
            s = (k_flat[: t + 1, a] @ q_flat[t, a] + k_rot[: t + 1] @ q_rot[t, a]) * m["scale"]
            p = torch.softmax(s, 0)
            out[t, a] = (p[:, None] * v[: t + 1, a]).sum(0) * gate[t, a]
    return out.reshape(T, H * Dv) @ w["o"].T


def sink_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    """Softmax attention with projection biases, a bias by the logarithm of the distance and a sink per head."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T + w["q.b"]).view(T, H, D)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, D)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, Dv)
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        dist = torch.arange(t, -1, -1, dtype=h.dtype)  # i - j for j = 0 .. t
        for a in range(H):
            g = a // (H // G)
            s = (k[: t + 1, g] @ q[t, a]) * m["scale"] - w["r1"][a] * torch.log1p(w["r2"][a] * dist)
            top = torch.maximum(s.max(), w["sink"][a])
            e = torch.exp(s - top)
            den = e.sum() + torch.exp(w["sink"][a] - top)
            out[t, a] = (e[:, None] * v[: t + 1, g]).sum(0) / den
    return out.reshape(T, H * Dv) @ w["o"].T


def state_space(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Mamba-2, token by token."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = F.silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner: inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = F.softplus(dt + w["dt_bias"])  # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for t in range(T):
        for a in range(H):
            g = a // (H // G)
            S[a] = decay[t, a] * S[a] + dt[t, a] * torch.outer(B[t, g], x[t, a])
            y[t, a] = S[a].T @ Cm[t, g] + w["D"][a] * x[t, a]
    y = y.reshape(T, inner) * F.silu(z)
    parts = int(m["norm_groups"])
    y = unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    left = {k[len("left."):]: v for k, v in w.items() if k.startswith("left.")}
    right = {k[len("right."):]: v for k, v in w.items() if k.startswith("right.")}
    a = unit(sink_attention(h, left, m["left"]), eps) * w["left.out"]
    b = unit(state_space(h, right, m["right"], eps), eps) * w["right.out"]
    return 0.5 * (a + b)


def delta_rule(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Gated delta rule, token by token."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.silu(causal_conv(h @ w["q"].T, w["q.conv"])).view(T, G, D)
    k = F.silu(causal_conv(h @ w["k"].T, w["k.conv"])).view(T, G, D)
    v = F.silu(causal_conv(h @ w["v"].T, w["v.conv"])).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)  # [T, H]
    g = torch.exp(-torch.exp(w["A_log"]) * F.softplus(h @ w["a"].T + w["dt_bias"]))
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    o = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        for a in range(H):
            j = a // (H // G)
            S[a] = g[t, a] * S[a]
            u = beta[t, a] * (v[t, a] - S[a].T @ k[t, j])
            S[a] = S[a] + torch.outer(k[t, j], u)
            o[t, a] = S[a].T @ q[t, j]
    o = unit(o, eps) * w["norm"]
    o = o.reshape(T, H * Dv) * F.silu(h @ w["g"].T)
    return o @ w["o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return (torch.relu(h @ w["up"].T) ** 2) @ w["down"].T


MIXERS = {"latent_attention": latent_attention, "parallel": parallel_mixer, "delta": delta_rule}


# --------------------------------------------------------------------------- files
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
        data = f.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    out = {}
    for name, info in meta.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[lo:hi]), dtype=kinds[info["dtype"]]).view(info["shape"]).clone()
    return out


class PlainNusudra:
    def __init__(self, folder: Optional[str] = None, raw: Optional[dict] = None,
                 weights: Optional[Dict[str, torch.Tensor]] = None, dtype: torch.dtype = torch.float64):
        if raw is None:
            with open(os.path.join(folder, "config.json")) as f:
                raw = json.load(f)
        if weights is None:
            weights = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.raw = raw
        self.dtype = dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
        self.eps = float(raw["norm"]["eps"])
        self.streams = int(raw.get("streams", 0) or 0)
        self.vocab = int(raw["vocab"])

    def sub(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def forward(self, tokens: Sequence[int], layers_out: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """Logits ``[T, vocab]``; with ``layers_out`` the stream (the sum of the streams) after every layer."""
        w, eps = self.w, self.eps
        x = w["embed"][torch.tensor(list(tokens))] * float(self.raw["embedding"]["scale"])
        S = self.streams
        xs = [x.clone() for _ in range(S)] if S else None
        for i, layer in enumerate(self.raw["layers"]):
            p = f"l{i}."
            subs = [(1, "mix")] + ([(2, "mlp")] if layer.get("mlp") is not None else [])
            for q, what in subs:
                if S:
                    hc = self.sub(f"{p}hc{q}.")
                    u = sum(hc["in"][s] * xs[s] for s in range(S))
                else:
                    u = x
                h = unit(u, eps) * w[f"{p}norm{q}"]
                if what == "mix":
                    h = token_shift(h, w[p + "shift"])
                    y = MIXERS[layer["type"]](h, self.sub(p + "mix."), layer["mixer"], eps)
                else:
                    y = dense_ff(h, self.sub(p + "mlp."))
                if S:
                    xs = [sum(hc["mix"][s, t] * xs[s] for s in range(S)) + hc["out"][t] * y for t in range(S)]
                else:
                    x = x + y
            if layers_out is not None:
                layers_out.append(sum(xs) if S else x.clone())
        if S:
            x = sum(xs)
        return (unit(x, eps) * w["final.norm"]) @ w["head"].T

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        return self.forward(tokens).float()

    def layer_sums(self, tokens: Sequence[int]) -> List[torch.Tensor]:
        """The stream (the sum of the copies) after every layer, float32."""
        out: List[torch.Tensor] = []
        self.forward(tokens, out)
        return [x.float() for x in out]

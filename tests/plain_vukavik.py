"""A plain, slow Vukavik: whole sequences, no cache, no batching, float32 or float64 on the CPU.

One function per mechanism, written as loops over tokens from the design's equations.  Nothing
here imports the package under test; configuration and weights are read directly.

Notation: ``h`` [T, W] is a sublayer's input (already normed), rows are tokens of one sequence
whose first row sits at position 0.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_weights(model_dir: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            out[k] = t.to(dtype) if t.is_floating_point() else t
    return out


# ---- small pieces ------------------------------------------------------------------------
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], taps [C, L]: out[t, c] = sum_j taps[c, j] * x[t - (L-1) + j, c], zeros before
    the start (the last column of the taps belongs to the current token)."""
    T, C = x.shape
    L = taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(L):
            s = t - (L - 1) + j
            if s >= 0:
                out[t] += taps[:, j] * x[s]
    if bias is not None:
        out = out + bias
    return out


# ---- rotary frequencies --------------------------------------------------------------------
def rotary_frequencies(rot: dict) -> tuple:
    """(frequency per pair, multiplier of cos and sin) for a ``rot`` description with optional
    YaRN ``scaling``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def corr(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(corr(float(sc["fast"]))), 0)
    hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x: torch.Tensor, pos: int, freqs: Sequence[float], mult: float) -> torch.Tensor:
    """x [heads, dim]: pairs (2i, 2i+1) of the first 2*len(freqs) dimensions are turned."""
    y = x.clone()
    for i, f in enumerate(freqs):
        a = pos * f
        c, s = math.cos(a) * mult, math.sin(a) * mult
        u, v = x[:, 2 * i], x[:, 2 * i + 1]
        y[:, 2 * i] = u * c - v * s
        y[:, 2 * i + 1] = v * c + u * s
    return y


# ---- mixers ----------------------------------------------------------------------------------
def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot")
    if rot:
        freqs, mult = rotary_frequencies(rot)
        q = torch.stack([rotate_interleaved(q[t], t, freqs, mult) for t in range(T)])
        k = torch.stack([rotate_interleaved(k[t], t, freqs, mult) for t in range(T)])
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [T, H]
    size = int(m["mask"]["size"]) if m.get("mask") else 0
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        first = (t // size) * size if size > 0 else 0
        for hh in range(H):
            g = hh // (H // G)
            s = (k[first:t + 1, g] @ q[t, hh]) * m["scale"]
            sink = w[p + "sink"][hh]
            mx = torch.maximum(s.max(), sink)
            e = torch.exp(s - mx)
            den = e.sum() + torch.exp(sink - mx)
            out[t, hh] = (e / den) @ v[first:t + 1, g] * gate[t, hh]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def delta_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                       # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hh] = S.T @ q[t, g]
    o = rms(o, eps) * w[p + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def mamba2_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    zxbcdt = h @ w[p + "in"].T
    z = zxbcdt[:, :inner]
    xbc = silu(causal_conv(zxbcdt[:, inner:2 * inner + 2 * G * N], w[p + "conv"], w[p + "conv.b"]))
    dt = softplus(zxbcdt[:, 2 * inner + 2 * G * N:] + w[p + "dt_bias"])          # [T, H]
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    A = torch.exp(w[p + "A_log"])
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-A[hh] * dt[t, hh]) * S + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S.T @ C[t, g] + w[p + "D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


MIXERS = {"attention": attention_mixer, "delta": delta_mixer, "mamba2": mamba2_mixer}


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    if mlp["kind"] != "dense":
        raise ValueError(f"feed-forward kind {mlp['kind']!r}")
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ---- the model ---------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[List] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; ``layers_out`` collects the stream after each layer."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](rms(x, eps) * w[p + "norm1"], w, p + "mix.", layer["mixer"], eps)
        x = x + mult * (rms(y, eps) * w[p + "norm1b"])
        if layer.get("mlp"):
            y = feed_forward(rms(x, eps) * w[p + "norm2"], w, p + "mlp.", layer["mlp"])
            x = x + mult * (rms(y, eps) * w[p + "norm2b"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T * float(cfg["logit_scale"])

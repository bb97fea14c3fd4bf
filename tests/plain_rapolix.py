"""Rapolix, plainly: one function per mechanism, loops over tokens, float64 by default.

Nothing here is shared with the package: the folder is read with a few lines of its own, the model is
a function of (configuration, weights, tokens) without cache or state, and every mechanism is
written from its equations.

The model.  ``x = embed[token] + sinusoid(position)``; ``streams`` copies of x run through the layers
as hyper-connections (a sublayer reads a weighted sum of the copies and writes its output back into
each of them with a weight, while a small matrix mixes the copies); a layer's mixer is two mixers side
by side on the same input (windowed attention that also keeps the first tokens, with an output gate;
and a gated linear recurrence behind a short convolution), each RMS-normed, then averaged; its
feed-forward is a dense SwiGLU with biases, a mixture of squared-ReLU experts with a shared expert and
identity experts, or absent; norms before sublayers are layer norms with a weight and no bias; the
logits pass ``cap * tanh(logits / cap)``.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Any, Dict, List, Optional, Sequence

import torch

# ---- the folder -------------------------------------------------------------------------------------

_DT = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64, "I32": torch.int32,
       "I64": torch.int64}


def read_config(folder: str) -> Dict[str, Any]:
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
        return json.load(f)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    """Eight bytes of length, that much json (name -> dtype, shape, data_offsets), then the data."""
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in head.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=_DT[e["dtype"]]).reshape(e["shape"])
        out[name] = t.to(dtype) if t.dtype.is_floating_point else t
    return out


# ---- small functions ----------------------------------------------------------------------------------

def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    m = x.mean(-1, keepdim=True)
    d = x - m
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def sinusoid(position: int, width: int, dtype) -> torch.Tensor:
    """Entry 2i is the sine, entry 2i+1 the cosine, of position * 10000^(-2i/width)."""
    out = torch.zeros(width, dtype=dtype)
    for j in range(width):
        angle = position * 10000.0 ** (-2.0 * (j // 2) / width)
        out[j] = math.sin(angle) if j % 2 == 0 else math.cos(angle)
    return out


def visible(i: int, j: int, size: Optional[int], keep_first: int) -> bool:
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    if size is None:
        return True
    return i - j < size or j < keep_first


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], taps [C, L] (the last column weighs the current token); zeros before the start."""
    T, C = x.shape
    L = taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for l in range(L):
            s = t - (L - 1 - l)
            if s >= 0:
                out[t] += taps[:, l] * x[s]
        if bias is not None:
            out[t] += bias
    return out


# ---- the mixers ---------------------------------------------------------------------------------------

def windowed_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict[str, Any]) -> torch.Tensor:
    """Grouped-query attention without rotation; a window that keeps the first tokens; the
    concatenated heads times sigmoid(W_g h) before the output projection."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    mask = m.get("mask") or {}
    size, keep = mask.get("size"), int(mask.get("keep_first", 0) or 0)
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, size, keep)]
        for hd in range(H):
            g = hd // (H // G)
            s = (k[js, g] @ q[i, hd]) * m["scale"]
            out[i, hd] = torch.softmax(s, 0) @ v[js, g]
    gate = sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


def gated_recurrence(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict[str, Any]) -> torch.Tensor:
    """y = gelu(W_y h + b); u = conv(W_x h + b); per block of channels r = sigmoid(R_a u + b) and
    i = sigmoid(R_i u + b); a = exp(-8 r softplus(lam)); S <- a S + sqrt(1 - a^2) i u; W_o (S y)."""
    T = h.shape[0]
    C, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    bs = C // B
    S = torch.zeros(C, dtype=h.dtype)
    out = torch.zeros(T, C, dtype=h.dtype)
    sp = softplus(w[p + "lam"])
    for t in range(T):
        r = torch.zeros(C, dtype=h.dtype)
        i = torch.zeros(C, dtype=h.dtype)
        for b in range(B):
            ub = u[t, b * bs:(b + 1) * bs]
            r[b * bs:(b + 1) * bs] = sigmoid(w[p + "ra"][b] @ ub + w[p + "ra.b"][b])
            i[b * bs:(b + 1) * bs] = sigmoid(w[p + "ri"][b] @ ub + w[p + "ri.b"][b])
        a = torch.exp(-8.0 * r * sp)
        S = a * S + torch.sqrt(1.0 - a * a) * i * u[t]
        out[t] = S * y[t]
    return out @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = windowed_attention(h, w, p + "left.", m["left"])
    right = gated_recurrence(h, w, p + "right.", m["right"])
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


# ---- the feed-forwards --------------------------------------------------------------------------------

def dense_ff(h, w, p):
    g = h @ w[p + "gate"].T + w[p + "gate.b"]
    u = h @ w[p + "up"].T + w[p + "up.b"]
    return (silu(g) * u) @ w[p + "down"].T + w[p + "down.b"]


def expert(h, w, p):
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def route(z: torch.Tensor, correction: torch.Tensor, top: int, count: int, keep: int):
    """For one token's router logits: the chosen outputs and their weights."""
    n = z.numel()
    s = torch.softmax(z, 0)
    choice = s + correction
    allowed = [True] * n
    if count > 1 and keep < count:
        per = n // count
        best = sorted(range(count), key=lambda g: (-float(choice[g * per:(g + 1) * per].max()), g))[:keep]
        allowed = [(e // per) in best for e in range(n)]
    order = sorted((e for e in range(n) if allowed[e]), key=lambda e: (-float(choice[e]), e))[:top]
    total = sum(s[e] for e in order) + 1e-20
    return order, [s[e] / total for e in order]


def moe_ff(h, w, p, mlp):
    r = mlp["router"]
    E, I, top = r["experts"], int(r.get("identity", 0) or 0), r["top"]
    groups = r.get("groups") or {}
    count, keep = int(groups.get("count", 1) or 1), int(groups.get("keep", 1) or 1)
    out = torch.zeros_like(h)
    z = h @ w[p + "router"].T
    for t in range(h.shape[0]):
        chosen, weights = route(z[t], w[p + "correction"], top, count, keep)
        for e, g in zip(chosen, weights):
            out[t] += g * (h[t] if e >= E else expert(h[t], w, f"{p}e{e}."))
    if mlp.get("shared"):
        out = out + expert(h, w, p + "shared.")
    return out


# ---- the model ----------------------------------------------------------------------------------------

def forward(cfg: Dict[str, Any], w: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[List] = None
            ) -> torch.Tensor:
    """Logits [tokens, vocab] of one sequence from position 0.  ``layers_out`` collects the residual
    stream (the sum of the copies) after every layer."""
    W, eps = cfg["width"], cfg["norm"]["eps"]
    dtype = w["embed"].dtype
    x = torch.stack([w["embed"][t] + sinusoid(p, W, dtype) for p, t in enumerate(tokens)])
    hyper = "streams" in cfg
    S = int(cfg.get("streams", 1))
    xs = [x.clone() for _ in range(S)]

    def sublayer(q: int, lp: str, fn):
        nonlocal xs
        if hyper:
            hc = f"{lp}hc{q}."
            u = sum(w[hc + "in"][s] * xs[s] for s in range(S))
            y = fn(layer_norm(u, w[f"{lp}norm{q}"], eps))
            xs = [sum(w[hc + "mix"][s, t] * xs[s] for s in range(S)) + w[hc + "out"][t] * y for t in range(S)]
        else:
            xs = [xs[0] + fn(layer_norm(xs[0], w[f"{lp}norm{q}"], eps))]

    for li, layer in enumerate(cfg["layers"]):
        lp = f"l{li}."
        if layer["type"] != "parallel":
            raise ValueError(f"layer type {layer['type']}")
        sublayer(1, lp, lambda h: parallel_mixer(h, w, lp + "mix.", layer["mixer"], eps))
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                sublayer(2, lp, lambda h: dense_ff(h, w, lp + "mlp."))
            else:
                sublayer(2, lp, lambda h: moe_ff(h, w, lp + "mlp.", mlp))
        if layers_out is not None:
            layers_out.append(sum(xs))
    x = sum(xs)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits

"""Mixers that carry a fixed-size state per request: the gated delta rule, Mamba-2 and the real-gated
linear recurrent unit.

Both keep two things in the request's state slot, as one float32 row: the last ``taps - 1``
inputs of their short causal convolution, and the recurrent matrices of every head.  Their
kernels (``csrc/recurrent.cu``) walk each sequence of the step in order from the state that
earlier steps left, so a prompt may be cut anywhere and a decode step is the same call with
one token per sequence.  Decays, step sizes, gates, unit norms and the state are float32
whatever the activation dtype.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import CacheView, Mixer, StateSpec, TensorSpec, register_mixer


def _taps(t: torch.Tensor) -> torch.Tensor:
    """[channels, taps] as stored -> [taps, channels], oldest tap first (the last column of the stored
    form belongs to the current token)."""
    return t.t().contiguous()


class GatedDeltaMixer(Mixer):
    """The gated delta rule.

    ``q = W_q x`` and ``k = W_k x`` (``n_kv_heads`` heads of ``head_dim``), ``v = W_v x`` (``n_heads``
    heads of ``v_head_dim``); each passes a causal convolution of ``conv`` taps per channel (no
    bias) and SiLU; q and k become unit vectors per head (``x / sqrt(sum x^2 + 1e-6)``), q also
    times ``head_dim^-1/2``.  Head h reads q/k head ``h // (n_heads / n_kv_heads)``.  Per head and
    token, with ``beta = sigmoid(W_b x)`` and ``g = exp(-exp(A_log) softplus(W_a x + dt_bias))``:

        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

    (the read-out sees the token's own write).  Each head's o is RMS-normed over ``v_head_dim``
    with one weight shared by the heads, multiplied by ``silu(W_g x)``, and projected by ``W_o``.
    All six input projections are one product.
    """

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, conv: int,
                 norm_eps: float, *, unit_eps: float = 1e-6, names: Optional[Dict[str, str]] = None,
                 weight_suffix: str = ".weight"):
        if n_heads <= 0 or n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} key heads")
        if not 1 <= conv <= 8:
            raise ValueError(f"convolution of {conv} taps is outside 1..8")
        if not 1 <= head_dim <= 256:
            raise ValueError(f"key size {head_dim} is outside 1..256")
        self.hidden, self.nh, self.nkv, self.dk, self.dv = int(hidden), int(n_heads), int(n_kv_heads), int(head_dim), int(v_head_dim)
        self.L, self.eps, self.unit_eps, self.sfx = int(conv), float(norm_eps), float(unit_eps), weight_suffix
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "a": "a_proj", "b": "b_proj", "g": "g_proj",
                      "o": "o_proj", "conv": ".conv", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm"}
        if names:
            self.names.update(names)
        self.channels = 2 * self.nkv * self.dk + self.nh * self.dv
        self.conv_elems = (self.L - 1) * self.channels
        self.w_in = self.w_o = self.taps = self.A_log = self.dt_bias = self.norm_w = None

    def cache_spec(self):
        return StateSpec("gated_delta", (self.conv_elems + self.nh * self.dk * self.dv,), torch.float32)

    def _proj(self, prefix: str, role: str) -> str:
        return f"{prefix}{self.names[role]}{self.sfx}"

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, h = self.names, self.hidden
        qk, vv = self.nkv * self.dk, self.nh * self.dv
        return [TensorSpec(self._proj(prefix, "q"), (qk, h)), TensorSpec(self._proj(prefix, "k"), (qk, h)),
                TensorSpec(self._proj(prefix, "v"), (vv, h)),
                TensorSpec(f"{prefix}{n['q']}{n['conv']}", (qk, self.L), role="vector"),
                TensorSpec(f"{prefix}{n['k']}{n['conv']}", (qk, self.L), role="vector"),
                TensorSpec(f"{prefix}{n['v']}{n['conv']}", (vv, self.L), role="vector"),
                TensorSpec(self._proj(prefix, "a"), (self.nh, h)), TensorSpec(self._proj(prefix, "b"), (self.nh, h)),
                TensorSpec(f"{prefix}{n['A_log']}", (self.nh,), role="vector", init="zeros"),
                TensorSpec(f"{prefix}{n['dt_bias']}", (self.nh,), role="vector"),
                TensorSpec(f"{prefix}{n['norm']}", (self.dv,), role="vector", init="ones"),
                TensorSpec(self._proj(prefix, "g"), (vv, h)), TensorSpec(self._proj(prefix, "o"), (h, vv))]

    def bind(self, tensors, prefix, dtype):
        n = self.names
        parts = [tensors[self._proj(prefix, r)] for r in ("q", "k", "v", "g", "a", "b")]
        wd = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
        self.w_in = torch.cat([p.to(wd) for p in parts], 0).contiguous()      # q | k | v | g | a | b
        self.w_o = tensors[self._proj(prefix, "o")].contiguous()
        self.taps = _taps(torch.cat([tensors[f"{prefix}{n[r]}{n['conv']}"] for r in ("q", "k", "v")], 0))
        self.A_log = tensors[f"{prefix}{n['A_log']}"].contiguous()
        self.dt_bias = tensors[f"{prefix}{n['dt_bias']}"].contiguous()
        self.norm_w = tensors[f"{prefix}{n['norm']}"].contiguous()

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        C, vv, nh = self.channels, self.nh * self.dv, self.nh
        h = ops.linear(a, self.w_in)
        state = cache.tensor
        qkv = ops.causal_conv_silu(h[:, :C], self.taps, None, state, ctx.state_slots, ctx.tok_seq, ctx.cu_q,
                                   ctx.positions, ctx.max_q, ctx.status)
        o = ops.gated_delta(qkv, h[:, C + vv:C + vv + 2 * nh], self.A_log, self.dt_bias, state, self.conv_elems,
                            ctx.state_slots, ctx.cu_q, ctx.positions, nh, self.nkv, self.dk, self.dv, self.unit_eps,
                            ctx.status, max_q=ctx.max_q)
        y = ops.gated_group_rmsnorm(o, h[:, C:C + vv], self.norm_w, self.eps, self.dv, False, h.dtype)
        return ops.linear(y, self.w_o)


class Mamba2Mixer(Mixer):
    """Mamba-2 (state-space duality).

    With ``inner = n_heads * head_dim``, N = ``n_state`` and G = ``groups``, ``W_in x`` is
    ``[z: inner | x: inner | B: G N | C: G N | dt: n_heads]``.  x, B and C together pass a causal
    convolution of ``conv`` taps per channel (with bias) and SiLU.  Per head (head h reads group
    ``h // (n_heads / G)``), with ``step = softplus(dt + dt_bias)`` (no clamp):

        S <- exp(-exp(A_log) step) S + step B x^T   (S is N x head_dim);   y = S^T C + D x

    y times ``silu(z)`` is RMS-normed in ``norm_groups`` equal parts (the gate comes first), multiplied
    by the norm's weight, and projected by ``W_o``.
    """

    def __init__(self, hidden: int, n_heads: int, head_dim: int, n_state: int, groups: int, conv: int,
                 norm_groups: int, norm_eps: float, *, names: Optional[Dict[str, str]] = None,
                 weight_suffix: str = ".weight"):
        if n_heads <= 0 or groups <= 0 or n_heads % groups:
            raise ValueError(f"{n_heads} heads are not a multiple of {groups} groups")
        if not 1 <= conv <= 8:
            raise ValueError(f"convolution of {conv} taps is outside 1..8")
        if not 1 <= n_state <= 256:
            raise ValueError(f"state size {n_state} is outside 1..256")
        self.hidden, self.nh, self.p, self.N, self.G = int(hidden), int(n_heads), int(head_dim), int(n_state), int(groups)
        self.inner = self.nh * self.p
        if norm_groups <= 0 or self.inner % norm_groups:
            raise ValueError(f"{norm_groups} norm groups do not divide {self.inner} channels")
        self.L, self.norm_groups, self.eps, self.sfx = int(conv), int(norm_groups), float(norm_eps), weight_suffix
        self.names = {"in": "in_proj", "conv": "conv1d.weight", "conv_bias": "conv1d.bias", "dt_bias": "dt_bias",
                      "A_log": "A_log", "D": "D", "norm": "norm.weight", "o": "out_proj"}
        if names:
            self.names.update(names)
        self.channels = self.inner + 2 * self.G * self.N
        self.conv_elems = (self.L - 1) * self.channels
        self.w_in = self.w_o = self.taps = self.conv_b = self.A_log = self.dt_bias = self.D = self.norm_w = None

    def cache_spec(self):
        return StateSpec("mamba2", (self.conv_elems + self.nh * self.N * self.p,), torch.float32)

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, h = self.names, self.hidden
        return [TensorSpec(f"{prefix}{n['in']}{self.sfx}", (2 * self.inner + 2 * self.G * self.N + self.nh, h)),
                TensorSpec(f"{prefix}{n['conv']}", (self.channels, self.L), role="vector"),
                TensorSpec(f"{prefix}{n['conv_bias']}", (self.channels,), role="vector"),
                TensorSpec(f"{prefix}{n['dt_bias']}", (self.nh,), role="vector"),
                TensorSpec(f"{prefix}{n['A_log']}", (self.nh,), role="vector", init="zeros"),
                TensorSpec(f"{prefix}{n['D']}", (self.nh,), role="vector", init="ones"),
                TensorSpec(f"{prefix}{n['norm']}", (self.inner,), role="vector", init="ones"),
                TensorSpec(f"{prefix}{n['o']}{self.sfx}", (h, self.inner))]

    def bind(self, tensors, prefix, dtype):
        n = self.names
        self.w_in = tensors[f"{prefix}{n['in']}{self.sfx}"].contiguous()
        self.w_o = tensors[f"{prefix}{n['o']}{self.sfx}"].contiguous()
        self.taps = _taps(tensors[f"{prefix}{n['conv']}"])
        self.conv_b = tensors[f"{prefix}{n['conv_bias']}"].contiguous()
        self.dt_bias = tensors[f"{prefix}{n['dt_bias']}"].contiguous()
        self.A_log = tensors[f"{prefix}{n['A_log']}"].contiguous()
        self.D = tensors[f"{prefix}{n['D']}"].contiguous()
        self.norm_w = tensors[f"{prefix}{n['norm']}"].contiguous()

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        inner, C = self.inner, self.channels
        h = ops.linear(a, self.w_in)
        state = cache.tensor
        xbc = ops.causal_conv_silu(h[:, inner:inner + C], self.taps, self.conv_b, state, ctx.state_slots, ctx.tok_seq,
                                   ctx.cu_q, ctx.positions, ctx.max_q, ctx.status)
        y = ops.state_space(xbc, h[:, inner + C:inner + C + self.nh], self.A_log, self.dt_bias, self.D, state,
                            self.conv_elems, ctx.state_slots, ctx.cu_q, ctx.positions, self.nh, self.G, self.N, self.p,
                            ctx.status, max_q=ctx.max_q)
        out = ops.gated_group_rmsnorm(y, h[:, :inner], self.norm_w, self.eps, inner // self.norm_groups, True, h.dtype)
        return ops.linear(out, self.w_o)


class RGLRUMixer(Mixer):
    """A recurrent block around the real-gated linear recurrent unit (De et al., "Griffin").

    Two branches of ``width`` channels: ``y = gelu_tanh(W_y x + b_y)`` and ``u = conv(W_x x + b_x)``, a causal
    convolution of ``conv`` taps per channel with bias and no activation.  u is cut into ``blocks`` equal
    parts; in part b, ``r = sigmoid(R_a[b] u_b + b_a[b])`` and ``i = sigmoid(R_i[b] u_b + b_i[b])`` with square
    matrices stored [out, in].  Per channel

        log a = -decay_c * r * softplus(lam);   S <- exp(log a) S + sqrt(1 - a^2) (i u)

    from S = 0 at position 0, and the block returns ``W_o (S * y)``.  The request's state slot holds the
    convolution's last ``conv - 1`` inputs and S, as one float32 row.  The two in-projections are one product.
    """

    def __init__(self, hidden: int, width: int, blocks: int, conv: int, *, decay_c: float = 8.0,
                 names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight", bias_suffix: str = ".bias"):
        if width <= 0 or blocks <= 0 or width % blocks:
            raise ValueError(f"{width} channels do not split into {blocks} equal parts")
        if not 1 <= conv <= 8:
            raise ValueError(f"convolution of {conv} taps is outside 1..8")
        self.hidden, self.C, self.B, self.L = int(hidden), int(width), int(blocks), int(conv)
        self.decay_c, self.sfx, self.bsfx = float(decay_c), weight_suffix, bias_suffix
        self.names = {"y": "y_proj", "x": "x_proj", "conv": "conv1d", "a": "a_gate", "i": "input_gate", "lam": "a_param",
                      "o": "out_proj"}
        if names:
            self.names.update(names)
        self.conv_elems = (self.L - 1) * self.C
        self.w_in = self.b_in = self.taps = self.conv_b = self.w_a = self.b_a = self.w_i = self.b_i = self.lam = self.w_o = None

    def cache_spec(self):
        return StateSpec("rglru", (self.conv_elems + self.C,), torch.float32)

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, h, C, B, x, b = self.names, self.hidden, self.C, self.B, self.sfx, self.bsfx
        bs = C // B
        return [TensorSpec(f"{prefix}{n['y']}{x}", (C, h)), TensorSpec(f"{prefix}{n['y']}{b}", (C,), role="vector"),
                TensorSpec(f"{prefix}{n['x']}{x}", (C, h)), TensorSpec(f"{prefix}{n['x']}{b}", (C,), role="vector"),
                TensorSpec(f"{prefix}{n['conv']}{x}", (C, self.L), role="vector"),
                TensorSpec(f"{prefix}{n['conv']}{b}", (C,), role="vector"),
                TensorSpec(f"{prefix}{n['a']}{x}", (B, bs, bs)), TensorSpec(f"{prefix}{n['a']}{b}", (B, bs), role="vector"),
                TensorSpec(f"{prefix}{n['i']}{x}", (B, bs, bs)), TensorSpec(f"{prefix}{n['i']}{b}", (B, bs), role="vector"),
                TensorSpec(f"{prefix}{n['lam']}", (C,), role="vector"),
                TensorSpec(f"{prefix}{n['o']}{x}", (h, C))]

    def bind(self, tensors, prefix, dtype):
        n, x, b = self.names, self.sfx, self.bsfx
        wy, wx = tensors[f"{prefix}{n['y']}{x}"], tensors[f"{prefix}{n['x']}{x}"]
        wd = wy.dtype if wy.dtype == wx.dtype else torch.float32
        self.w_in = torch.cat([wy.to(wd), wx.to(wd)], 0).contiguous()                     # y | x
        self.b_in = torch.cat([tensors[f"{prefix}{n['y']}{b}"], tensors[f"{prefix}{n['x']}{b}"]], 0).contiguous()
        self.taps = _taps(tensors[f"{prefix}{n['conv']}{x}"])
        self.conv_b = tensors[f"{prefix}{n['conv']}{b}"].contiguous()
        # the gates are computed in float32 from matrices kept in the activation dtype
        self.w_a = tensors[f"{prefix}{n['a']}{x}"].to(dtype).contiguous()
        self.w_i = tensors[f"{prefix}{n['i']}{x}"].to(dtype).contiguous()
        self.b_a = tensors[f"{prefix}{n['a']}{b}"].reshape(-1).contiguous()
        self.b_i = tensors[f"{prefix}{n['i']}{b}"].reshape(-1).contiguous()
        self.lam = tensors[f"{prefix}{n['lam']}"].contiguous()
        self.w_o = tensors[f"{prefix}{n['o']}{x}"].contiguous()

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        C = self.C
        h = ops.linear(a, self.w_in, self.b_in)
        if h.dtype != a.dtype:
            h = h.to(a.dtype)
        state = cache.tensor
        u = ops.causal_conv(h[:, C:], self.taps, self.conv_b, state, ctx.state_slots, ctx.tok_seq, ctx.cu_q,
                            ctx.positions, ctx.max_q, ctx.status, act="none")
        s = ops.rglru(u, h[:, :C], self.w_a, self.b_a, self.w_i, self.b_i, self.lam, self.decay_c, state, self.conv_elems,
                      ctx.state_slots, ctx.cu_q, ctx.positions, ctx.status, max_q=ctx.max_q)
        return ops.linear(s, self.w_o)


register_mixer("gated_delta", GatedDeltaMixer)
register_mixer("rglru", RGLRUMixer)
register_mixer("mamba2", Mamba2Mixer)

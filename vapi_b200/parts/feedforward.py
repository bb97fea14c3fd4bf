"""Dense SwiGLU feed-forward."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import FeedForward, StreamState, TensorSpec, register_feed_forward


class SwiGLU(FeedForward):
    """``down( silu(gate f) * (up f) )`` without biases; gate and up are stacked into one
    matrix at bind time so they are one product
    (crates/vapi-backend-candle/src/models/lfm2.rs:568-595).  ``names`` maps gate/up/down to
    the checkpoint's sub-names (LFM2: w1 / w3 / w2).  ``bias``: ``down(silu(gate f + b_g) * (up f + b_u)) + b_d``."""

    def __init__(self, hidden: int, ff: int, names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight",
                 bias: bool = False, bias_suffix: str = ".bias"):
        self.hidden, self.ff, self.sfx = int(hidden), int(ff), weight_suffix
        #: with ``bias`` every projection adds a bias vector (``<name><bias_suffix>``)
        self.bias, self.bsfx = bool(bias), bias_suffix
        self.b_gate_up = self.b_down = None
        self.names = {"gate": "w1", "up": "w3", "down": "w2"}
        if names:
            self.names.update(names)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n = self.names
        specs = [TensorSpec(f"{prefix}{n['gate']}{self.sfx}", (self.ff, self.hidden)),
                 TensorSpec(f"{prefix}{n['up']}{self.sfx}", (self.ff, self.hidden)),
                 TensorSpec(f"{prefix}{n['down']}{self.sfx}", (self.hidden, self.ff))]
        if self.bias:
            specs += [TensorSpec(f"{prefix}{n['gate']}{self.bsfx}", (self.ff,), role="vector"),
                      TensorSpec(f"{prefix}{n['up']}{self.bsfx}", (self.ff,), role="vector"),
                      TensorSpec(f"{prefix}{n['down']}{self.bsfx}", (self.hidden,), role="vector")]
        return specs

    def bind(self, tensors, prefix, dtype):
        n = self.names
        g, u = tensors[f"{prefix}{n['gate']}{self.sfx}"], tensors[f"{prefix}{n['up']}{self.sfx}"]
        wd = g.dtype if g.dtype == u.dtype else torch.float32
        self.w_gate_up = torch.cat([g.to(wd), u.to(wd)], 0).contiguous()
        self.w_down = tensors[f"{prefix}{n['down']}{self.sfx}"].contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([tensors[f"{prefix}{n['gate']}{self.bsfx}"], tensors[f"{prefix}{n['up']}{self.bsfx}"]], 0).contiguous()
            self.b_down = tensors[f"{prefix}{n['down']}{self.bsfx}"].contiguous()

    def forward(self, f: torch.Tensor, ctx: Any) -> torch.Tensor:
        if self.bias:
            return ops.linear(ops.swiglu(ops.linear(f, self.w_gate_up, self.b_gate_up)), self.w_down, self.b_down)
        return ops.linear(ops.linear_swiglu(f, self.w_gate_up), self.w_down)

    def forward_stream(self, f, ctx, x, next_weight):
        if self.bias:
            return NotImplemented
        n = x.shape[0]
        if not (ops.few_rows_applies(n, self.w_gate_up) and ops.few_rows_applies(n, self.w_down)):
            return NotImplemented
        s = ops.few_rows_linear(self.w_gate_up, xw=f.xw, ss_in=f.ss, eps=f.eps, epilogue="swiglu")
        ss, xw = ops.few_rows_linear(self.w_down, act=s, epilogue="resid", resid=x, next_weight=next_weight)
        return StreamState(xw, ss)


register_feed_forward("swiglu", SwiGLU)

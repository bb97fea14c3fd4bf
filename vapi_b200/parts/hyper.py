"""Hyper-connections: several copies of the residual stream, and the block that reads and writes them."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import CacheView, FeedForward, Mixer, Norm, Part, TensorSpec
from .block import register_block
from .parallel import DeferredBranches


@dataclass
class HyperPending:
    """A sublayer's output that is still to be written into the residual streams:
    ``x_t <- sum_s mix[s, t] x_s + write[t] * y`` for all copies t at once.  The kernel that reads the streams
    next (for the following sublayer, or for the model's final norm) applies it while it reads the row."""

    y: torch.Tensor
    mix: torch.Tensor          # [S, S] float32, indexed [from, to]
    write: torch.Tensor        # [S] float32
    #: ``(y2 | None, w_y, w_y2 | None, eps, scale)``: what is written is ``scale * (rms(y) w_y + rms(y2) w_y2)``,
    #: the outputs of mixers side by side whose norms and mean the reading kernel takes on
    branch: Any = None


class HyperBlock(Part):
    """A pre-norm layer over ``streams`` copies x_1 .. x_S of the residual stream.  For each sublayer
    (the mixer, then the feed-forward, which may be absent):

        u = sum_s read[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + write[t] y

    ``read`` [S], ``write`` [S] and ``mix`` [S, S] are the sublayer's own tensors (``sub["mixer_hc"]`` /
    ``sub["ffn_hc"]`` + ``names``).  With ``learned`` False the block has no such tensors and one stream:
    the ordinary ``x <- x + sublayer(norm(x))``.  The streams are one float32 tensor [n, S, H]; a sublayer's
    output travels as a :class:`HyperPending` to whichever kernel reads the streams next.
    """

    def __init__(self, streams: int, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm],
                 ffn: Optional[FeedForward], sub: Dict[str, str], *, learned: bool = True,
                 names: Optional[Dict[str, str]] = None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward comes with its norm or not at all")
        if streams < 1 or streams > 8:
            raise ValueError(f"{streams} streams are outside 1..8")
        if not learned and streams != 1:
            raise ValueError("several streams need their read, write and mix tensors")
        self.S, self.learned = int(streams), bool(learned)
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.sub = dict(sub)
        self.names = {"read": "in", "write": "out", "mix": "mix"}
        if names:
            self.names.update(names)
        self.hc: Dict[str, Dict[str, torch.Tensor]] = {}

    def _subs(self):
        out = [("mixer", self.mixer_norm, self.mixer)]
        if self.ffn is not None:
            out.append(("ffn", self.ffn_norm, self.ffn))
        return out

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for key, norm, part in self._subs():
            out += norm.tensor_specs(prefix + self.sub.get(key + "_norm", ""))
            out += part.tensor_specs(prefix + self.sub.get(key, ""))
            if self.learned:
                hp = prefix + self.sub[key + "_hc"]
                out += [TensorSpec(hp + self.names["read"], (self.S,), role="vector", init="ones"),
                        TensorSpec(hp + self.names["write"], (self.S,), role="vector", init="ones"),
                        TensorSpec(hp + self.names["mix"], (self.S, self.S), role="vector", init="normal")]
        return out

    def bind(self, tensors, prefix, dtype):
        for key, norm, part in self._subs():
            norm.bind(tensors, prefix + self.sub.get(key + "_norm", ""), dtype)
            part.bind(tensors, prefix + self.sub.get(key, ""), dtype)
            if self.learned:
                hp = prefix + self.sub[key + "_hc"]
                self.hc[key] = {r: tensors[hp + self.names[r]].contiguous() for r in ("read", "write", "mix")}
            else:
                one = torch.ones(1, dtype=torch.float32, device=norm.weight.device)
                self.hc[key] = {"read": one, "write": one, "mix": one.view(1, 1)}

    def first_norm(self) -> Norm:
        return self.mixer_norm

    def _read(self, key: str, norm: Norm, x: torch.Tensor, pending: Optional[HyperPending], ctx: Any) -> torch.Tensor:
        if pending is not None and not isinstance(pending, HyperPending):
            raise TypeError("a block over several streams takes a HyperPending from the block before it")
        y, mix, write = (pending.y, pending.mix, pending.write) if pending is not None else (None, None, None)
        return ops.hyper_read_norm(x, y, mix, write, self.hc[key]["read"], norm.weight, norm.eps, ctx.dtype, None,
                                   norm.kind, pending.branch if pending is not None else None)

    def forward(self, x: torch.Tensor, delta: Optional[HyperPending], ctx: Any, cache: CacheView) -> HyperPending:
        a = self._read("mixer", self.mixer_norm, x, delta, ctx)
        y = self.mixer.forward(a, ctx, cache)
        branch = None
        if isinstance(y, DeferredBranches):          # mixers side by side: their norms and mean ride on the next read
            branch = (y.outs[1] if len(y.outs) > 1 else None, y.weights[0], y.weights[1] if len(y.outs) > 1 else None,
                      y.eps, y.scale)
            y = y.outs[0]
        pending = HyperPending(y, self.hc["mixer"]["mix"], self.hc["mixer"]["write"], branch)
        if self.ffn is None:
            return pending
        f = self._read("ffn", self.ffn_norm, x, pending, ctx)
        return HyperPending(self.ffn.forward(f, ctx), self.hc["ffn"]["mix"], self.hc["ffn"]["write"])


register_block("hyper", HyperBlock)

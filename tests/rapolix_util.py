"""Small Rapolix configurations and model folders whose small parameters make faults show."""
from __future__ import annotations

import zlib
from typing import Dict, Optional, Sequence, Tuple

import torch

import plain_rapolix as plain


def left(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, size: Optional[int] = 20, keep_first: Optional[int] = 3) -> dict:
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return m


def right(width=48, blocks=3, conv=4) -> dict:
    return {"width": width, "blocks": blocks, "conv": conv}


def dense(ff=96) -> dict:
    return {"kind": "dense", "ff": ff}


def moe(ff=40, experts=6, identity=2, top=2, count: Optional[int] = 4, keep=2, shared: Optional[int] = 56) -> dict:
    r = {"experts": experts, "identity": identity, "top": top}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(l: dict, r: dict, mlp: Optional[dict]) -> dict:
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def config(layers: Sequence[dict], width=64, vocab=200, streams: Optional[int] = 3, softcap: Optional[float] = 20.0,
           eps=1e-5) -> dict:
    c = {"architecture": "Rapolix", "layers": list(layers), "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if streams is not None:
        c["streams"] = streams
    if softcap is not None:
        c["logit_softcap"] = softcap
    return c


#: sizes that all differ from one another; every kind of feed-forward; a layer without one; windows that end inside
#: pages of 16; keys and values of unlike widths; convolutions of 1, 2 and 4 taps; 1, 2 and 3 parts
MIXED = config([layer(left(), right(), dense()),
                layer(left(heads=3, kv_heads=3, dim=24, vdim=16, size=33, keep_first=0), right(width=64, blocks=1, conv=1), moe()),
                layer(left(heads=2, kv_heads=1, dim=32, vdim=32, size=None), right(width=32, blocks=2, conv=2), None),
                layer(left(heads=2, kv_heads=2, dim=8, vdim=8, size=7, keep_first=9), right(width=24, blocks=3, conv=3),
                      moe(ff=24, experts=5, identity=0, top=1, count=None, shared=None))])
#: tiny, for runs where plain Python stands in for the kernels
TINY = config([layer(left(heads=2, kv_heads=1, dim=8, vdim=12, size=6, keep_first=2), right(width=16, blocks=2, conv=3), dense(40)),
               layer(left(heads=2, kv_heads=2, dim=8, vdim=8, size=9, keep_first=1), right(width=8, blocks=1, conv=2),
                     moe(ff=12, experts=3, identity=1, top=2, count=2, keep=1, shared=16))], width=32, vocab=61, streams=2)
#: one ordinary residual stream (no `streams` key, so no read / write / mix tensors) and no cap on the logits
ONE_STREAM = config([layer(left(size=12, keep_first=None), right(width=32, blocks=2, conv=2), moe(count=1, keep=1, identity=0)),
                     layer(left(heads=2, kv_heads=2, dim=16, vdim=16, size=5, keep_first=4), right(), dense(48))],
                    streams=None, softcap=None)
#: a single learned stream: hyper-connections whose matrices are 1 x 1
SINGLE_LEARNED = config([layer(left(), right(), dense(48))], streams=1)
#: keys and values of 64 and of 128, the widths of the tensor-core attention kernels; windows that end inside pages of 64
SERVING_HEADS = config([layer(left(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, size=100, keep_first=5), right(width=128, blocks=2, conv=3), dense(128)),
                        layer(left(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, size=70, keep_first=66), right(width=64, blocks=1, conv=4),
                              moe(ff=64, experts=8, identity=0, top=3, count=2, keep=1, shared=64))], width=128, streams=2)


#: sizes that fit no vector width: a model width of 100, five streams, heads of 12 and 20, a window of one token, a
#: window shorter than the kept count, parts of 10 channels, seven experts that are all chosen, an odd vocabulary
ODD = config([layer(left(heads=5, kv_heads=5, dim=12, vdim=20, scale=0.4, size=1, keep_first=0), right(width=50, blocks=5, conv=1),
                    moe(ff=10, experts=7, identity=0, top=7, count=None, shared=6)),
              layer(left(heads=6, kv_heads=2, dim=20, vdim=12, scale=0.2, size=3, keep_first=30), right(width=36, blocks=2, conv=8), dense(34)),
              layer(left(heads=1, kv_heads=1, dim=4, vdim=4, scale=1.0, size=200, keep_first=1), right(width=4, blocks=4, conv=2),
                    moe(ff=6, experts=2, identity=4, top=3, count=3, keep=2, shared=None))],
             width=100, vocab=133, streams=5, softcap=7.5, eps=1e-6)


def write_model(folder: str, cfg: dict, seed: int = 0, dtype=torch.float32, std: float = 0.12) -> str:
    """A model folder whose small parameters are far from their neutral values: slow and unlike decays, gate
    matrices that make the gates move, corrections of both signs, stream matrices that are no identity."""
    from vapi_b200.config.model import resolve_architecture
    from vapi_b200.weights import write_random_model
    arch = resolve_architecture(cfg)
    specs = arch.plan(arch.parse(cfg)).tensor_specs()
    over = {}
    for s in specs:
        g = torch.Generator().manual_seed(seed * 7919 + zlib.crc32(s.name.encode()) % 100003)
        parts = s.name.split(".")
        last = parts[-1]
        if last == "lam":
            over[s.name] = -1.0 - 5.0 * torch.rand(s.shape, generator=g)          # decays from 0.1 to 0.999 a token
        elif last in ("ra", "ri"):
            over[s.name] = 0.5 * torch.randn(s.shape, generator=g)
        elif last == "conv":
            over[s.name] = 0.5 * torch.randn(s.shape, generator=g)
        elif last == "b":
            over[s.name] = 0.3 * torch.randn(s.shape, generator=g)
        elif last == "correction":
            over[s.name] = 0.1 * torch.randn(s.shape, generator=g)
        elif last == "router":
            over[s.name] = 0.5 * torch.randn(s.shape, generator=g)
        elif len(parts) >= 2 and parts[-2] in ("hc1", "hc2"):
            S = s.shape[0]
            if last == "mix":
                over[s.name] = torch.eye(S) + 0.2 * torch.randn(s.shape, generator=g)
            elif last == "in":
                over[s.name] = 1.0 / S + 0.3 * torch.randn(s.shape, generator=g)
            else:
                over[s.name] = 1.0 + 0.3 * torch.randn(s.shape, generator=g)
    return write_random_model(folder, cfg, seed, std=std, norm_init="perturbed", dtype=dtype, overrides=over)


class Oracle:
    """The plain model on a folder, float64."""

    def __init__(self, folder: str):
        self.cfg = plain.read_config(folder)
        self.w = plain.read_weights(folder, torch.float64)
        self._memo: Dict[Tuple[int, ...], torch.Tensor] = {}

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(self.cfg, self.w, tokens)
        return self._memo[key]

    def greedy(self, tokens: Sequence[int], n: int):
        toks, out = list(tokens), []
        for _ in range(n):
            t = int(torch.argmax(self.logits(toks)[-1]))
            out.append(t)
            toks.append(t)
        return out

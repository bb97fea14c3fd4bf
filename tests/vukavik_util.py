"""Small Vukavik configurations, model folders with weights that make faults show, and the means
to push a schedule through the framework's step function and compare with the plain model."""
from __future__ import annotations

import zlib
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

import plain_vukavik as plain


def attention(heads=4, kv_heads=2, dim=16, vdim=24, chunk: Optional[int] = 40, rot_dims: Optional[int] = None,
              scaling: Optional[dict] = "default", scale=0.3, base=10000.0, ff: Optional[int] = 64) -> dict:
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot_dims != 0:
        rot = {"base": base, "dims": rot_dims or dim}
        if scaling == "default":
            scaling = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
        if scaling:
            rot["scaling"] = scaling
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, ff: Optional[int] = None) -> dict:
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def mamba2(heads=4, vdim=16, state=24, groups=2, conv=4, norm_groups=2, ff: Optional[int] = None) -> dict:
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers: Sequence[dict], width=64, vocab=200, residual_mult=0.5, logit_scale=0.7, eps=1e-5) -> dict:
    return {"architecture": "Vukavik", "layers": list(layers), "logit_scale": logit_scale, "norm": {"eps": eps},
            "residual_mult": residual_mult, "vocab": vocab, "width": width}


#: every mixer kind, sizes that differ from one another, a feed-forward on some layers only
MIXED = config([delta(ff=96), attention(), mamba2(), attention(heads=3, kv_heads=3, dim=24, vdim=16, chunk=17, rot_dims=12, ff=None),
                delta(heads=2, kv_heads=2, dim=24, vdim=16, conv=2), mamba2(heads=2, vdim=24, state=16, groups=1, conv=2, norm_groups=1, ff=64)])
#: tiny, for runs where plain Python stands in for the kernels
TINY = config([attention(heads=2, kv_heads=1, dim=8, vdim=12, chunk=9, ff=48), delta(heads=2, kv_heads=1, dim=8, vdim=12),
               mamba2(heads=2, vdim=8, state=8, groups=1, conv=3, norm_groups=1)], width=32, vocab=61)
#: no attention at all (no paged cache), multipliers of one
NO_ATTENTION = config([mamba2(ff=64), delta()], residual_mult=1.0, logit_scale=1.0)
#: attention only, no mask and no frequency scaling, a partial rotation
PLAIN_ATTENTION = config([attention(chunk=None, scaling=None, rot_dims=8), attention(chunk=None, scaling=None, rot_dims=0, heads=2, kv_heads=1, dim=32, vdim=32)])


#: keys and values of 64 and of 128, the widths of the tensor-core attention kernels; chunks that end inside pages of 64
SERVING_HEADS = config([attention(heads=4, kv_heads=2, dim=64, vdim=64, chunk=100, rot_dims=32, ff=128), delta(heads=2, kv_heads=1, dim=32, vdim=32),
                        attention(heads=2, kv_heads=1, dim=128, vdim=128, chunk=None, rot_dims=128, ff=None)], width=128)


def write_model(folder: str, cfg: dict, seed: int = 0, dtype=torch.float32, std: float = 0.12) -> str:
    """A model folder whose small parameters are far from their neutral values (decays, step
    biases, sinks, skips, taps, norm weights), so that leaving one out shows."""
    from vapi_b200.config.model import resolve_architecture
    from vapi_b200.weights import write_random_model
    arch = resolve_architecture(cfg)
    specs = arch.plan(arch.parse(cfg)).tensor_specs()
    over = {}
    for s in specs:
        g = torch.Generator().manual_seed(seed * 7919 + zlib.crc32(s.name.encode()) % 100003)
        last = s.name.split(".")[-1]
        if last == "A_log":
            over[s.name] = torch.rand(s.shape, generator=g) * 2.5 - 1.0
        elif last in ("dt_bias", "sink"):
            over[s.name] = torch.randn(s.shape, generator=g)
        elif last == "D":
            over[s.name] = 1.0 + 0.5 * torch.randn(s.shape, generator=g)
        elif last == "conv":
            over[s.name] = 0.5 * torch.randn(s.shape, generator=g)
        elif last == "b" and s.name.endswith("conv.b"):
            over[s.name] = 0.3 * torch.randn(s.shape, generator=g)
    return write_random_model(folder, cfg, seed, std=std, norm_init="perturbed", dtype=dtype, overrides=over)


def prompt(cfg: dict, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


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

    def greedy(self, tokens: Sequence[int], n: int) -> List[int]:
        toks, out = list(tokens), []
        for _ in range(n):
            t = int(torch.argmax(self.logits(toks)[-1]))
            out.append(t)
            toks.append(t)
        return out


def make_runner(folder: str, dtype: str, device: str, num_pages: int = 16, page_size: int = 16, max_requests: int = 4,
                max_tokens: int = 256):
    from vapi_b200.engine.runner import ModelRunner
    return ModelRunner.from_dir(folder, dtype=dtype, device=device, page_size=page_size, num_pages=num_pages,
                                max_requests=max_requests, max_batched_tokens=max_tokens,
                                max_context=num_pages * page_size, watermark=0.0)


def run_schedule(runner, requests: Dict[str, Sequence[int]], schedule: Sequence[Sequence[Tuple[str, int]]]) -> Dict[str, np.ndarray]:
    """``schedule``: steps of (request, how many of its next tokens).  A request is opened at its first
    entry and closed when its tokens are used up.  Returns request -> logits [tokens, vocab] at
    every position."""
    from vapi_b200.engine.step import StepEntry
    live, at = {}, {k: 0 for k in requests}
    rows: Dict[str, List[Optional[np.ndarray]]] = {k: [None] * len(v) for k, v in requests.items()}
    for step in schedule:
        entries, where = [], []
        for rid, count in step:
            toks = list(requests[rid][at[rid]:at[rid] + count])
            rc = live.get(rid)
            if rc is None:
                rc = live[rid] = runner.cache.open(rid)
            assert runner.cache.reserve(rc, rc.num_tokens + len(toks)), "the test's pool is too small"
            entries.append(StepEntry(rc, toks, list(range(len(toks)))))
            where += [(rid, at[rid] + i) for i in range(len(toks))]
            at[rid] += len(toks)
        out = runner.step(entries).float().cpu().numpy()
        runner.check_status()
        for (rid, pos), row in zip(where, out):
            rows[rid][pos] = row
        for rid, _ in step:
            if at[rid] == len(requests[rid]):
                runner.cache.close(live.pop(rid))
    assert not live and all(r is not None for v in rows.values() for r in v), "the schedule must use every token"
    runner.cache.check_invariants()
    return {k: np.stack(v) for k, v in rows.items()}


def worst(got: np.ndarray, want: torch.Tensor) -> Tuple[float, int]:
    """Largest difference of the logits as a fraction of their range, and the position that has it."""
    w = want.numpy()
    assert np.isfinite(got).all()
    d = np.abs(got - w).max(-1) / float(w.max() - w.min())
    return float(d.max()), int(d.argmax())


def limit(dtype: str) -> float:
    """float32: rounding of a few dozen operations.  bfloat16: four per cent of the logit range for
    narrow layers with strong weights, as the other tiny models of this suite get."""
    return 2e-5 if dtype == "float32" else 0.04


def cuts(total: int, sizes: Sequence[int]) -> List[int]:
    out, i = [], 0
    while total > 0:
        q = min(sizes[i % len(sizes)], total)
        out.append(q)
        total -= q
        i += 1
    return out

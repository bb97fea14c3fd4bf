"""Several mixers side by side on one input."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from .base import CacheView, Mixer, TensorSpec, register_mixer


@dataclass
class DeferredBranches:
    """The branches' outputs before their norms and their mean: ``scale * sum_b rmsnorm(outs[b]) * weights[b]``.
    A block whose next kernel reads every row anyway (:class:`~vapi_b200.parts.hyper.HyperBlock`) takes the
    norms and the mean on there; :meth:`tensor` computes them with a kernel of their own."""

    outs: List[torch.Tensor]
    weights: List[torch.Tensor]
    eps: float
    scale: float

    def tensor(self) -> torch.Tensor:
        return ops.branch_rmsnorm_mean(self.outs, self.weights, self.eps, self.scale)


class ParallelMixer(Mixer):
    """``mean_b rmsnorm(branch_b(a)) * w_b``: every branch reads the same normed input; each output is
    RMS-normed over the model width with a plain weight of its own (``<sub_b><norm_name>``) and the results
    are averaged.  ``branches`` is a sequence of ``(sub-prefix, mixer)``.  Each branch keeps the cache it
    asks for: the mixer's ``cache_spec`` is the tuple of the branches' specs, and it is handed a ``multi``
    view with one part per branch.  With ``deferred`` (and at most two branches) ``forward`` returns a
    :class:`DeferredBranches` instead of a tensor, for a block that folds the norms and the mean into its next read."""

    def __init__(self, hidden: int, branches: Sequence[Tuple[str, Mixer]], eps: float, norm_name: str = "out",
                 deferred: bool = False):
        if not 1 <= len(branches) <= 4:
            raise ValueError("one to four branches")
        self.hidden, self.eps, self.norm_name = int(hidden), float(eps), norm_name
        self.deferred = bool(deferred) and len(branches) <= 2
        self.subs = [s for s, _ in branches]
        self.branches: List[Mixer] = [m for _, m in branches]
        self.weights: List[torch.Tensor] = []

    def members(self):
        return tuple(self.branches)

    def cache_spec(self):
        return tuple(m.cache_spec() for m in self.branches)

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for sub, m in zip(self.subs, self.branches):
            out += m.tensor_specs(prefix + sub)
            out.append(TensorSpec(f"{prefix}{sub}{self.norm_name}", (self.hidden,), role="vector", init="ones"))
        return out

    def bind(self, tensors, prefix, dtype):
        self.weights = []
        for sub, m in zip(self.subs, self.branches):
            m.bind(tensors, prefix + sub, dtype)
            self.weights.append(tensors[f"{prefix}{sub}{self.norm_name}"].contiguous())

    def decode_splits(self, batch, max_context, page_size, dtype):
        return max(m.decode_splits(batch, max_context, page_size, dtype) for m in self.branches)

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        views = cache.parts if cache.kind == "multi" else [cache] * len(self.branches)
        outs = [m.forward(a, ctx, v) for m, v in zip(self.branches, views)]
        if self.deferred:
            return DeferredBranches(outs, self.weights, self.eps, 1.0 / len(outs))
        return ops.branch_rmsnorm_mean(outs, self.weights, self.eps, 1.0 / len(outs))


register_mixer("parallel", ParallelMixer)

"""Mixers side by side: several mixers read the same normalised input and their outputs are added
with one constant factor each, ``y = sum_b factor_b * mixer_b(h)``.

Each branch is an ordinary mixer part named by its own spec; at most one of them may keep pages and
at most one a per-request state, which then are this part's needs towards the cache manager.  The
weighted sum is one small kernel over the branches' partial sums (32-bit).
"""

from __future__ import annotations

from typing import Mapping, Sequence

import torch

from mini_engine_b200.config.model_spec import PartSpec
from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import LayerCache, Mixer, PagedCacheSpec, StateSpec, StepContext, build_part, register
from mini_engine_b200.weights.loader import WeightSpec


@register("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, prefix: str, hidden_size: int, *, branches: Sequence[Mapping]):
        """``branches``: mappings with ``mixer`` (a :class:`PartSpec`), ``factor`` and ``prefix`` (what
        the branch's tensor names start with, behind the layer's prefix)."""
        if not 1 <= len(branches) <= 4:
            raise ValueError("parallel_mixers takes one to four branches")
        self.hidden = hidden_size
        self.branches: list[Mixer] = []
        self.factors: list[float] = []
        for branch in branches:
            spec: PartSpec = branch["mixer"]
            self.branches.append(build_part("mixer", spec, prefix + branch.get("prefix", ""), hidden_size))
            self.factors.append(float(branch.get("factor", 1.0)))
        if sum(b.paged_cache() is not None for b in self.branches) > 1 or sum(b.state() is not None for b in self.branches) > 1:
            raise ValueError("at most one branch may keep pages and at most one a state of its own")

    @property
    def capturable(self) -> bool:  # type: ignore[override]
        return all(getattr(branch, "capturable", False) for branch in self.branches)

    @property
    def programmatic_launch(self) -> bool:  # type: ignore[override]
        return all(getattr(branch, "programmatic_launch", True) for branch in self.branches)

    def paged_cache(self) -> PagedCacheSpec | None:
        return next((b.paged_cache() for b in self.branches if b.paged_cache() is not None), None)

    def state(self) -> StateSpec | None:
        return next((b.state() for b in self.branches if b.state() is not None), None)

    def weight_specs(self) -> list[WeightSpec]:
        return [spec for branch in self.branches for spec in branch.weight_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for branch in self.branches:
            branch.load(tensors)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        outputs = [(branch.forward(h, ctx, cache), factor) for branch, factor in zip(self.branches, self.factors)]
        out = ctx.buffer("parallel.out", (h.shape[0], self.hidden), torch.float32)
        ops.branch_sum(outputs, out)
        return out.unsqueeze(0)

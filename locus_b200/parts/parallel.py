"""Mixers side by side: every branch reads the same input, and their outputs are added with fixed factors.

``branches``: (name, mixer spec, factor) each; a branch's tensors live under ``<prefix>.<name>`` and the branch gets
its factor as its ``out_scale``.  The branches share the layer's cache: at most one of them may keep pages and at most
one a per-request state (the layer's cache entry has one of each).

A branch behind the first that can run in two steps (``prepare``: all but its last product, on buffers and state of its
own; ``finish``: the product that adds into the output) is prepared on the runtime's side stream while the first branch
runs, and finished when both are done.
"""
from __future__ import annotations

from typing import Sequence, Tuple

from .base import Mixer, PartSpec, make_part, register_mixer


class ParallelMixers(Mixer):
    can_overwrite = True

    def __init__(self, prefix: str, *, branches: Sequence[Tuple[str, PartSpec, float]]) -> None:
        super().__init__(prefix)
        if not branches:
            raise ValueError("parallel: no branches")
        self.branches = [make_part("mixer", PartSpec(spec.kind, {**spec.args, "out_scale": float(scale)}), f"{prefix}.{name}")
                         for name, spec, scale in branches]
        paged = [b for b in self.branches if b.cache_needs()[0] is not None]
        state = [b for b in self.branches if b.cache_needs()[1] is not None]
        if len(paged) > 1 or len(state) > 1:
            raise ValueError("parallel: at most one branch may keep pages and at most one a per-request state")

    def sub_parts(self):
        return list(self.branches)

    def cache_needs(self):
        paged = state = None
        for b in self.branches:
            p, s = b.cache_needs()
            paged, state = paged or p, state or s
        return paged, state

    def step_plans(self):
        return [pl for b in self.branches for pl in b.step_plans()]

    def forward(self, h, batch, cache, residual, rt, accumulate=True) -> None:
        early = {}
        for i, b in enumerate(self.branches[1:], 1):
            if hasattr(b, "prepare") and hasattr(b, "finish"):
                with rt.side():
                    early[i] = b.prepare(h, batch, cache, rt)
        for i, b in enumerate(self.branches):
            if i in early:
                if i == min(early):   # the side stream's work is done in order: one wait covers every branch on it
                    rt.join()
                b.finish(early[i], residual, rt, accumulate=True)
            elif i == 0 and not accumulate and not b.can_overwrite:
                residual.zero_()
                b.forward(h, batch, cache, residual, rt)
            elif b.can_overwrite:
                b.forward(h, batch, cache, residual, rt, accumulate=accumulate or i > 0)
            else:
                b.forward(h, batch, cache, residual, rt)


register_mixer("parallel", ParallelMixers)

"""Several mixers side by side: every branch reads the same input, and the result is
sum_i scale_i * branch_i(x), or, with ``branch_norms``, sum_i scale_i * n_i(branch_i(x)) where n_i is
an RMS norm over the model width with a weight of its own (``branch_norms``: one entry per branch,
``dict(name=, eps=)`` with the checkpoint name of the weight, or None for a branch that joins as it
is).  The sum is left to the reader (the float32 residual stream norms and adds the branches'
outputs in float32, in branch order).  Each branch keeps the cache of its own kind; the schedule
entry's cache is a composite with one member per branch."""

from __future__ import annotations

from typing import Optional

from ..kernels import ops
from .base import Mixer
from .registry import MIXERS, register_mixer
from .spec import CompositeSpec, StateSpec, TensorSpec


def _keeps_state(spec) -> bool:
    if isinstance(spec, CompositeSpec):
        return any(_keeps_state(m) for m in spec.members)
    return isinstance(spec, StateSpec)


@register_mixer("parallel")
class ParallelMixers(Mixer):
    def __init__(self, ctx, branches: list, scales: list, branch_norms: Optional[list] = None,
                 hidden_size: Optional[int] = None):
        if len(branches) != len(scales) or not branches:
            raise ValueError(f"parallel mixers: {len(branches)} branches and {len(scales)} scales")
        self.branches = [MIXERS.build(spec, ctx) for spec in branches]
        self.scales = [float(s) for s in scales]
        self.branch_norms = None
        if branch_norms is not None:
            if len(branch_norms) != len(branches) or hidden_size is None:
                raise ValueError("parallel mixers: a norm entry (or None) per branch and the model width are needed")
            self.branch_norms = [None if n is None else dict(name=str(n["name"]), eps=float(n["eps"]))
                                 for n in branch_norms]
        self.hidden_size = None if hidden_size is None else int(hidden_size)
        self.norm_weights = [None] * len(self.branches)

    @property
    def state_on_device(self) -> bool:
        return all(getattr(b, "state_on_device", False) or not _keeps_state(b.cache_spec())
                   for b in self.branches)

    def tensor_specs(self):
        specs = [s for b in self.branches for s in b.tensor_specs()]
        for n in self.branch_norms or ():
            if n is not None:
                specs.append(TensorSpec(n["name"], (self.hidden_size,), role="vector", init="one_plus_normal"))
        return specs

    def load(self, tensors):
        for b in self.branches:
            b.load(tensors)
        for i, n in enumerate(self.branch_norms or ()):
            if n is not None:
                self.norm_weights[i] = tensors[n["name"]]

    def cache_spec(self):
        return CompositeSpec(tuple(b.cache_spec() for b in self.branches))

    def forward(self, x, step, cache):
        outs = [b.forward(x, step, cache.members[i]) for i, b in enumerate(self.branches)]
        if self.branch_norms is not None:
            outs = [o if n is None else ops.NormedTerm(o, self.norm_weights[i], n["eps"])
                    for i, (o, n) in enumerate(zip(outs, self.branch_norms))]
        return ops.WeightedSum(list(zip(self.scales, outs)))

"""Several mixers side by side on the same input, as one mixer.

    x += weight * sum_i rmsnorm(branch_i(h)) * n_i            (each branch's result normed over the model width with its own gain)

The branches are any registered mixers; each is built under its own prefix and keeps its own cache: a branch that wants
paged keys and values gets the run's paged group, a branch with a state of fixed size gets its share of the run's states,
in the order of the branches (the cache manager gives a run one paged group at most, so one branch at most may page).
Every branch writes its result into a float32 buffer of its own; one kernel norms them, adds them up and puts the sum
where the block wants it.

Without norms (`spec.weights`: one factor per branch) the result is the weighted sum of the branches' results as they are:

    x += sum_i weights[i] * branch_i(h)

Every branch then applies its factor itself in front of its last product (`takes_out_scale`), and the products add into the
stream one after the other: no buffer and no launch of this part's own.
"""
from __future__ import annotations

import torch

from ..cache.manager import FixedState, needs_of
from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Mixer, RunCache, part_class, register_mixer


class ParallelMixers(Mixer):
    can_overwrite = True
    wants_position_encodings = True        # the block hands over the model's position tables; the branches pick theirs

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime, position_encodings=()):
        self.spec, self.dim, self.rt = spec, dim, runtime
        self.overwrite = False
        self.branches, self.state_counts = [], []
        for b, p in zip(spec.branches, spec.prefixes):
            cls = part_class("mixer", b.kind)
            table = getattr(b, "rope_table", -1)
            extra = {"rope": position_encodings[table]} if table is not None and table >= 0 and position_encodings else {}
            part = cls(b, dim, tensors, prefix + p, runtime, **extra)
            if not getattr(part, "can_overwrite", False):
                raise ValueError(f"a {b.kind} mixer cannot be a branch: it only adds to the stream it is given")
            part.overwrite = not spec.weights
            if spec.weights:
                if not getattr(part, "takes_out_scale", False):
                    raise ValueError(f"a {b.kind} mixer cannot be a weighted branch: it takes no factor on its result")
                part.out_scale = float(spec.weights[len(self.branches)])
            self.branches.append(part)
            self.state_counts.append(sum(isinstance(n, FixedState) for n in needs_of(cls.cache_need(b))))
        self.gains = [tensors.pop(prefix + n) for n in spec.out_norms if n]
        if len(self.branches) != 2 or spec.weights:
            self.forward_branches = None      # (one branch: the block norms the mixer's own result)

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        out = {}
        for b, p, n in zip(spec.branches, spec.prefixes, spec.out_norms):
            out.update(part_class("mixer", b.kind).wants(b, dim, prefix + p))
            if n:
                out[prefix + n] = TensorWant((dim,), "vector", init="gain")
        return out

    @classmethod
    def cache_need(cls, spec):
        return tuple(n for b in spec.branches for n in needs_of(part_class("mixer", b.kind).cache_need(b)))

    @property
    def graph_safe(self) -> bool:
        return all(getattr(b, "graph_safe", False) for b in self.branches)

    def decode_bucket_cap(self, rows: int) -> int:
        return max(b.decode_bucket_cap(rows) for b in self.branches)

    def _run_branches(self, xb, batch, cache, into=None) -> list:
        """Every branch on the same rows; `into`: where the branches add their results (else each writes a buffer of its own)."""
        rows, outs, at = xb.shape[0], [], 0
        for i, (part, n) in enumerate(zip(self.branches, self.state_counts)):
            states = tuple(cache.states[at:at + n])
            at += n
            mine = RunCache(cache.run, cache.writes, cache.group, cache.keys, cache.values, states[0] if states else None, states)
            y = into if into is not None else self.rt.buffer(f"parallel_branch{i}", self.dim, torch.float32)[:rows]
            part.forward(xb, y, batch, mine)
            outs.append(y)
        return outs

    def forward_branches(self, xb, batch, cache):
        """The branches' results as they are, for a block that norms and adds them up in a launch of its own:
        (a, gain_a, b, gain_b, weight), the result being weight * (rmsnorm(a) * gain_a + rmsnorm(b) * gain_b). None where
        there is one branch only (the block then takes `forward`)."""
        outs = self._run_branches(xb, batch, cache)
        return outs[0], self.gains[0], outs[1], self.gains[1], self.spec.weight

    def forward(self, xb, x, batch, cache) -> None:
        s = self.spec
        if s.weights:
            if self.overwrite:
                x.zero_()
            self._run_branches(xb, batch, cache, into=x)
            return
        outs = self._run_branches(xb, batch, cache)
        b, gb = (outs[1], self.gains[1]) if len(outs) > 1 else (None, None)
        ops.norm_sum(x, outs[0], self.gains[0], s.norm_eps, b, gb, scale=s.weight, accumulate=not self.overwrite)


register_mixer("parallel_mixers", ParallelMixers, replace=True)

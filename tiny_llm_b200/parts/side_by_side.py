"""Several mixers side by side on the same normed input.  Each branch's output is RMS-normed over the model width
with a weight of its own and the branches are averaged with a fixed weight:
    y = weight * sum_b  rms(mixer_b(h)) * w_b.
Every branch keeps its own cache, so the part's cache need is the tuple of its branches' needs (flattened: a branch
may itself keep several things) and it hands each branch its share of the views.
With `norm=False` the branches are not normed: y = sum_b weights[b] * mixer_b(h), every branch with a factor of its own
(applied in 32-bit to the branch's sum, not folded into its matrices).  A branch is then (prefix, PartSpec) only."""
from __future__ import annotations

import torch

from .. import ops
from ..weights import FLOAT32, WeightSpec
from .registry import build_part, register_part


class SideBySide:

    def __init__(self, hidden_size: int, eps: float = 0.0, branches=(), weight: float = 1.0, out_scale: float = 1.0,
                 norm: bool = True, weights=None, shares_cache: bool = False):
        """`branches`: (weight-name prefix, PartSpec of a mixer, name of the branch's norm weight) each; without norms
        (prefix, PartSpec) each, and `weights` gives every branch's factor."""
        if shares_cache:
            raise ValueError("mixers side by side do not read another layer call's cache")
        self.hidden_size, self.eps = hidden_size, float(eps)
        self.weight = float(weight) * float(out_scale)
        self.norm = norm
        if not norm:
            if weights is None or len(weights) != len(branches):
                raise ValueError("branches without norms need one factor each")
            self.factors = [float(w) * float(out_scale) for w in weights]
            branches = [(b[0], b[1], None) for b in branches]
        self.branches = [(prefix, build_part("mixer", spec), norm_name) for prefix, spec, norm_name in branches]
        self.graph_safe = all(getattr(m, "graph_safe", False) for _, m, _ in self.branches)
        self.norm_weights = []
        self._needs = []
        for _, m, _ in self.branches:
            need = m.cache_need()
            self._needs.append(need if isinstance(need, (tuple, list)) else (need,))

    def cache_need(self):
        return tuple(one for need in self._needs for one in need)

    def weight_specs(self, prefix: str):
        specs = []
        for bp, m, norm_name in self.branches:
            specs += m.weight_specs(prefix + bp)
            if self.norm:
                specs.append(WeightSpec(prefix + norm_name, (self.hidden_size,), FLOAT32))
        return specs

    def load(self, prefix: str, weights) -> None:
        self.norm_weights = []
        for bp, m, norm_name in self.branches:
            m.load(prefix + bp, weights)
            self.norm_weights.append(weights[prefix + norm_name] if self.norm else None)

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        at = 0
        for i, ((bp, m, _), need, w) in enumerate(zip(self.branches, self._needs, self.norm_weights)):
            views = cache[at: at + len(need)]
            at += len(need)
            # a buffer of this part's own: `resid` may itself be the zeroed buffer of a block that norms the branch
            branch = ctx.workspace.get_zeroed("side_out", (t, self.hidden_size))
            m.forward(ctx, h, branch, views if isinstance(m.cache_need(), (tuple, list)) else views[0])
            if self.norm:
                ops.rms_norm_add(branch, w, self.eps, self.weight, resid)
            else:
                ops.scaled_add(branch, self.factors[i], resid)


register_part("mixer", "side_by_side", SideBySide)

"""Several mixers side by side on the same input: out = mean_i rmsnorm_i(mixer_i(h)), every
branch normalised over the model width with a weight of its own before the mean.  The branches
are any registered mixers; at most one of them may keep a paged cache and at most one a state
(a run-order entry names one cache entry and one state entry)."""
from __future__ import annotations

from ..kernels import ops
from .base import Mixer, ParamSpec, build_mixer, register_mixer


class SideBySide(Mixer):
    tree_name = "mixer"

    def __init__(self, hidden_size, branches, eps):
        """``branches``: ((name, PartSpec), ...); branch ``name`` lives under that name in the
        checkpoint and its output weight is ``name``.out.weight."""
        super().__init__()
        self.hidden_size, self.eps = hidden_size, float(eps)
        self.branches = [(name, build_mixer(spec)) for name, spec in branches]
        if not 1 <= len(self.branches) <= 4:
            raise ValueError("side by side: one to four branches")
        if sum(m.cache_spec() is not None for _, m in self.branches) > 1 or \
                sum(m.state_spec() is not None for _, m in self.branches) > 1:
            raise ValueError("side by side: at most one branch with a cache and one with a state")
        self.capturable = all(m.capturable for _, m in self.branches)

    def children(self):
        return dict(self.branches)

    def param_specs(self):
        return {f"{name}.out.weight": ParamSpec((self.hidden_size,), role="vector", init="norm_weight")
                for name, _ in self.branches}

    def cache_spec(self):
        return next((m.cache_spec() for _, m in self.branches if m.cache_spec() is not None), None)

    def state_spec(self):
        return next((m.state_spec() for _, m in self.branches if m.state_spec() is not None), None)

    def work_tile_queries(self, dtype, page_size):
        return max(m.work_tile_queries(dtype, page_size) for _, m in self.branches)

    def forward(self, h, ctx, call):
        outs = [m.forward(h, ctx, call) for _, m in self.branches]
        return ops.mean_of_normed(outs, [self.w[f"{name}.out.weight"] for name, _ in self.branches], self.eps)


register_mixer("side_by_side", SideBySide)

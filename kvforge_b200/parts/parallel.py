"""Mixers side by side: every branch reads the same normed input; each result is RMS-normed over the
model width with a weight of its own (a plain weight, not one-plus), and the mixer's result is the
mean of the normed results.

The branches are ordinary mixers.  At most one of them may keep pages of keys and values (the
block's cache group is that branch's); their per-request states lie side by side in one row of
floats, and each branch is handed its columns.
"""

from __future__ import annotations

from .. import ops
from .base import CacheNeed, Mixer, PartSpec, WeightDecl, build_part, register_mixer


def _spec(v) -> PartSpec:
    return v if isinstance(v, PartSpec) else PartSpec(v["kind"], v.get("params", {}))


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    """params: ``hidden_size``, ``eps``, ``branches``: a list of ``(name, PartSpec)``; branch
    ``name`` has its tensors under ``<prefix><name>.`` and its norm weight is ``<prefix><name>.out``."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.names = [name for name, _ in params["branches"]]
        if not 0 < len(self.names) <= ops.MAX_BRANCHES:
            raise ValueError(f"between 1 and {ops.MAX_BRANCHES} branches")
        self.branches: list[Mixer] = [build_part("mixer", _spec(spec), f"{prefix}{name}.") for name, spec in params["branches"]]
        paged = [b for b in self.branches if b.cache_need().kind != "none"]
        if len(paged) > 1:
            raise ValueError("only one branch of parallel mixers may keep pages of keys and values")
        self._need = paged[0].cache_need() if paged else CacheNeed("none")
        self._state_cols: list[tuple[int, int] | None] = []
        at = 0
        for b in self.branches:
            shape = b.state_shape()
            if shape is None:
                self._state_cols.append(None)
                continue
            if len(shape) != 1:
                raise ValueError("a branch's state must be a flat row of floats")
            self._state_cols.append((at, at + shape[0]))
            at += shape[0]
        self._state_floats = at

    @classmethod
    def weight_decls(cls, params):
        h = int(params["hidden_size"])
        return {f"{name}.out": WeightDecl((h,), kind="vector", init="ones") for name, _ in params["branches"]}

    def sub_parts(self):
        return list(self.branches)

    def cache_need(self) -> CacheNeed:
        return self._need

    def state_shape(self):
        return (self._state_floats,) if self._state_floats else None

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.out_w = [weights[f"{name}.out"] for name in self.names]

    def forward(self, ctx, x, cache):
        keep, ctx.residual = ctx.residual, None  # a branch's result is normed before it is added anywhere
        try:
            results = []
            for branch, cols in zip(self.branches, self._state_cols):
                view = cache
                if cache is not None and cache.state is not None:
                    view = cache.with_state(*cols) if cols else cache.with_state(0, 0)
                y = branch.forward(ctx, x, view)
                t = y.t if isinstance(y, ops.Partials) else y
                if any(t.data_ptr() == (o.t if isinstance(o, ops.Partials) else o).data_ptr() for o in results):
                    # two branches of one kind hand back the same persistent buffer: keep this one's result apart
                    kept = self.rt.buf(f"parallel.keep{len(results)}", t.numel() // t.shape[-1], t.shape[-1], t.dtype).view(t.shape)
                    kept.copy_(t)
                    y = ops.Partials(kept) if isinstance(y, ops.Partials) else kept
                results.append(y)
        finally:
            ctx.residual = keep
        out = self.rt.buf("parallel.out", x.shape[0], self.hidden)
        ops.branch_norm_mean(results, self.out_w, self.eps, out)
        return out

"""Two mixers side by side on the same input, as one mixer:

    y = left_scale * left(x) + right_scale * right(x)

`left` and `right` are any registered mixers, named in the parameters as {"kind": ..., "params": {...}}; their
tensors are this part's tensors under "left." and "right.".  The cache entry of the layer holds what both need:
the paged keys and values of the one and the per-sequence state of the other (two sides that both want pages, or
both want state, are refused).  The position encoding of the layer goes to both sides; a side that rotates
nothing ignores it.  Upstream has no such layer.
"""
from __future__ import annotations

from ..cache import EntryRequirement, split_requirement
from ..ops import kernels
from .base import Mixer, part_class, register_part


class _SideLoader:
    """The loader of one side: its local names are the parent's with a prefix."""

    def __init__(self, load, prefix: str):
        self.load, self.prefix = load, prefix

    def dtype(self, *names):
        return self.load.dtype(*(self.prefix + n for n in names))

    def __call__(self, name, out=None):
        return self.load(self.prefix + name, out=out)


class ParallelMixers(Mixer):
    kind = "parallel_mixers"

    @classmethod
    def wanted(cls, params):
        out = {}
        for side in ("left", "right"):
            spec = params[side]
            for n, w in part_class(spec["kind"]).wanted(spec["params"]).items():
                out[f"{side}.{n}"] = w
        return out

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        make = lambda side: part_class(params[side]["kind"])(params[side]["params"], _SideLoader(load, side + "."), rt)
        self.left, self.right = make("left"), make("right")
        self.left_scale, self.right_scale = float(params.get("left_scale", 1.0)), float(params.get("right_scale", 1.0))

    @property
    def graph_safe(self):
        return self.left.graph_safe and self.right.graph_safe

    def cache_requirement(self):
        (kv_l, st_l), (kv_r, st_r) = (split_requirement(m.cache_requirement()) for m in (self.left, self.right))
        if (kv_l is not None and kv_r is not None) or (st_l is not None and st_r is not None):
            raise ValueError("two mixers side by side that both want cache pages, or both want state rows")
        kv, st = kv_l or kv_r, st_l or st_r
        if kv is not None and st is not None:
            return EntryRequirement(kv, st)
        return kv if kv is not None else st

    def step_arrays(self, shape, cache):
        return {**self.left.step_arrays(shape, cache), **self.right.step_arrays(shape, cache)}

    def step(self, x, ctx, cache, position, writes_cache=True):
        a = self.left.step(x, ctx, cache, position, writes_cache)
        b = self.right.step(x, ctx, cache, position, writes_cache)
        return kernels.scaled_sum(a, self.left_scale, b, self.right_scale)


register_part(ParallelMixers.kind, ParallelMixers)

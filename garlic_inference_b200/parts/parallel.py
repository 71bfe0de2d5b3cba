"""Two mixers side by side on the same input, as one mixer:

    y = left_scale * left(x) + right_scale * right(x)

`left` and `right` are any registered mixers, named in the parameters as {"kind": ..., "params": {...}}; their
tensors are this part's tensors under "left." and "right.".  The cache entry of the layer holds what both need:
the paged keys and values of the one and the per-sequence state of the other (two sides that both want pages, or
both want state, are refused).  The position encoding of the layer goes to both sides; a side that rotates
nothing ignores it.

When both sides end in an output projection of their own and can hand over what goes into it (`pre_output`,
`w_o`), the two projections and the weighted sum are one product: each side writes its activations, times its
factor, into its columns of one matrix, and the two output weights lie side by side,
    y = [ left_scale a_left | right_scale a_right ] . [ Wo_left | Wo_right ]^T,
summed in float32 inside the product.  Otherwise the sides run whole and a kernel adds their results.
Upstream has no such layer.
"""
from __future__ import annotations

from ..cache import EntryRequirement, split_requirement
import torch

from ..ops import kernels, linear
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
        self.w_o = None
        sides = (self.left, self.right)
        if all(hasattr(m, "pre_output") and getattr(m, "w_o", None) is not None for m in sides) and \
                self.left.w_o.dtype == self.right.w_o.dtype and self.left.w_o.shape[1] % 8 == 0:
            self.k_left = self.left.w_o.shape[1]
            self.w_o = torch.cat([self.left.w_o, self.right.w_o], dim=1).contiguous()
            self.left.w_o = self.right.w_o = None                # the sides' own copies are let go: only pre_output runs

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
        if self.w_o is not None:
            acts = torch.empty((x.shape[0], self.w_o.shape[1]), dtype=self.rt.dtype, device=x.device)
            self.left.pre_output(x, ctx, cache, position, writes_cache, out=acts[:, :self.k_left], out_mul=self.left_scale)
            self.right.pre_output(x, ctx, cache, position, writes_cache, out=acts[:, self.k_left:], out_mul=self.right_scale)
            return linear(acts, self.w_o)
        a = self.left.step(x, ctx, cache, position, writes_cache)
        b = self.right.step(x, ctx, cache, position, writes_cache)
        return kernels.scaled_sum(a, self.left_scale, b, self.right_scale)


register_part(ParallelMixers.kind, ParallelMixers)

"""A routed feed-forward (mixture of experts), as a feed-forward part.

    z = Wr x                                   router logits, float32 (the weight is widened, the product is this
                                               package's float32 kernel; x may be its 16-bit rounding)
    the `top` experts with the largest z are chosen; their weights are the softmax over the chosen z alone
    y = sum_e weight_e Wd_e act(Wu_e x)        act: the square of relu ("relu_squared") or silu; no biases

The experts' matrices are stacked at load time ([experts, ff, hidden] and [experts, hidden, ff]).  Two ways to
run them.  A step of a few rows (a decode step; such a step may be recorded, so nothing may come back to the
host): two kernels that read the chosen experts' matrices only, a warp per matrix row, the experts taken from
device memory.  More rows: the (token, choice) pairs are sorted by expert on the device, the counts come to the
host once, every expert that was chosen runs two matrix products over its own rows, and one kernel sums each
token's `top` results with its weights in the router's order.  Either way a token's result does not depend on
the other tokens of the step beyond the rounding of the products.
NikolayBlagoev/garlic-inference's mixture-of-experts model is a different design (src/models/qwen3/qwen3-moe.cpp).
"""
from __future__ import annotations

import torch

from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .base import FeedForward, register_part

# Up to how many rows of a step the row-by-row kernels run (beyond: expert by expert through matrix products).
ROWWISE_MAX_ROWS = 32


class RoutedExperts(FeedForward):
    kind = "routed_experts"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        hid, ff, E = params["hidden_size"], params["expert_size"], params["n_experts"]
        w = {"router": TensorWant((E, hid))}
        for e in range(E):
            w[f"e{e}.up"], w[f"e{e}.down"] = TensorWant((ff, hid)), TensorWant((hid, ff))
        return w

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.ff = int(params["hidden_size"]), int(params["expert_size"])
        self.E, self.top = int(params["n_experts"]), int(params["top"])
        self.activation = params.get("activation", "relu_squared")
        if not 0 < self.top <= self.E:
            raise ValueError(f"{self.top} of {self.E} experts")
        if self.activation not in ("relu_squared", "silu"):
            raise ValueError(f"expert activation {self.activation!r} is neither 'relu_squared' nor 'silu'")
        self.w_router = load("router").to(torch.float32)
        names = [f"e{e}.up" for e in range(self.E)]
        dtype = load.dtype(*names, *(f"e{e}.down" for e in range(self.E)))
        self.w_up = torch.empty((self.E, self.ff, self.hidden), dtype=dtype, device=rt.device)
        self.w_down = torch.empty((self.E, self.hidden, self.ff), dtype=dtype, device=rt.device)
        for e in range(self.E):
            load(f"e{e}.up", out=self.w_up[e])
            load(f"e{e}.down", out=self.w_down[e])

    def step(self, x, ctx):
        n = x.shape[0]
        logits = linear(x, self.w_router, out_dtype=torch.float32)
        idx, wt = kernels.router_topk(logits, self.top)
        if ctx.captured or n <= ROWWISE_MAX_ROWS or self.activation != "relu_squared":
            return kernels.moe_rowwise(x, self.w_up, self.w_down, idx, wt, self.activation)
        # expert by expert: pairs (token, choice) sorted by expert; `where` is each pair's row in that order
        flat = idx.reshape(-1)
        order = torch.sort(flat.to(torch.int64), stable=True).indices
        where = torch.empty_like(order)
        where[order] = torch.arange(order.numel(), device=order.device)
        counts = torch.bincount(flat, minlength=self.E).tolist()           # the one trip to the host
        rows = x.index_select(0, order // self.top)
        buf = torch.empty((n * self.top, self.hidden), dtype=x.dtype, device=x.device)
        at = 0
        for e, c in enumerate(counts):
            if c:
                a = kernels.relu_squared(linear(rows[at:at + c], self.w_up[e]))
                buf[at:at + c] = linear(a, self.w_down[e])
                at += c
        return kernels.moe_combine(buf, where.to(torch.int32).view(n, self.top), wt)


register_part(RoutedExperts.kind, RoutedExperts)

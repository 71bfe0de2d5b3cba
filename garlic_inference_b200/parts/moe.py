"""A routed feed-forward (mixture of experts), as a feed-forward part.

    z = Wr x                                   router logits, float32 (the weight is widened, the product is a
                                               float32 kernel of its own; x may be its 16-bit rounding)
    the `top` experts with the largest z are chosen; their weights are the softmax over the chosen z alone
    y = sum_e weight_e Wd_e act(Wu_e x)        act: the square of relu ("relu_squared") or silu; no biases

The experts' matrices are stacked at load time ([experts, ff, hidden] and [experts, hidden, ff]).  Two ways to
run them.  A step of a few rows (a decode step; such a step may be recorded, so nothing may come back to the
host): kernels that read the chosen experts' matrices only, a warp per matrix row, the experts taken from
device memory.  More rows: the (token, choice) pairs are put in the order of their experts by a counting sort on
the device (which also gathers the tokens' vectors into that order), the experts run two matrix products over
their own rows, and one kernel sums each token's `top` results with its weights in the router's order.  In bfloat16 the two products are the library's grouped product (`torch._grouped_mm`: the rows
of every expert in one launch, the groups' ends read from device memory, nothing comes to the host); in float32,
or where the library has no grouped product, the counts come to the host once and every chosen expert runs this
package's products over its rows.  Either way a token's result does not depend on the other tokens of the step
beyond the rounding of the products.
NikolayBlagoev/garlic-inference's mixture-of-experts model is a different design (src/models/qwen3/qwen3-moe.cpp).
"""
from __future__ import annotations

import torch

from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .base import FeedForward, register_part

# Up to how many rows of a step the row-by-row kernels run (beyond: expert by expert through matrix products).
# The row-by-row kernels read an expert's matrices once per (token, choice) pair, the grouped product once per
# expert: from a few tokens on, pairs share experts.
ROWWISE_MAX_ROWS = 8


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
        logits = kernels.router_logits(x, self.w_router)
        idx, wt = kernels.router_topk(logits, self.top)
        grouped = self._grouped(x)
        if n <= ROWWISE_MAX_ROWS or self.activation != "relu_squared" or (ctx.captured and not grouped):
            return kernels.moe_rowwise(x, self.w_up, self.w_down, idx, wt, self.activation)
        # expert by expert: the pairs (token, choice) in the order of their experts; `where` is each pair's row
        where, ends, rows = kernels.moe_group(idx, x, self.E)
        if grouped:
            a = kernels.relu_squared(torch._grouped_mm(rows, self.w_up.transpose(1, 2), offs=ends))
            buf = torch._grouped_mm(a, self.w_down.transpose(1, 2), offs=ends)
        else:
            buf = torch.empty((n * self.top, self.hidden), dtype=x.dtype, device=x.device)
            at = 0
            bounds = [0] + ends.tolist()                                   # the one trip to the host
            for e in range(self.E):
                c = bounds[e + 1] - bounds[e]
                if c:
                    a = kernels.relu_squared(linear(rows[at:at + c], self.w_up[e]))
                    buf[at:at + c] = linear(a, self.w_down[e])
                    at += c
        return kernels.moe_combine(buf.contiguous(), where, wt)

    def _grouped(self, x) -> bool:
        """Whether the library's grouped product takes these operands: bfloat16, rows of 16-byte multiples."""
        return (x.dtype == torch.bfloat16 and self.w_up.dtype == torch.bfloat16 and hasattr(torch, "_grouped_mm")
                and self.hidden % 8 == 0 and self.ff % 8 == 0)


register_part(RoutedExperts.kind, RoutedExperts)

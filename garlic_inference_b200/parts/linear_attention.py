"""Linear attention with a fixed decay per head, as a mixer with a matrix of state per head.

    q, k, v = f(Wq x), f(Wk x), f(Wv x)          heads x key_dim, heads x key_dim, heads x value_dim
    S_t = lam_h S_(t-1) + k_t v_t^T              float32, from zero at a sequence's start
    o_t = S_t^T q_t                              no other scale
    y   = Wo( rmsnorm(concat_h o_t) * w * sigmoid(Wg x) )

`decay` (lam, one per head), the sizes and the norm's eps are parameters; the
feature map f is silu and the output gate a sigmoid, the only ones the kernel
computes.  The four projections that read x are one packed product.  The
state lives in the cache's per-slot state rows and is walked by one kernel for
prompts, portions of prompts and single tokens alike.  Upstream has no
recurrent mixer.
"""
from __future__ import annotations

import torch

from ..cache import StateRequirement
from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .base import Mixer, register_part, seq_spans_array


def scan_state_floats(key_dim: int, value_dim: int) -> int:
    """Floats of one head's state in the scan kernels' layout [value column][key, padded]: the keys are padded
    to 16, 32, 64, 128 or 256 (csrc/recurrent.cu holds the same rule)."""
    for regs in (4, 8, 16, 32, 64):
        if 4 * regs >= key_dim:
            return value_dim * 4 * regs
    raise ValueError(f"a key dimension of {key_dim} is beyond the scan kernels' 256")


def pack_rows(load, names_rows, hidden: int, rt, pad_to: int = 8):
    """The [rows, hidden] tensors listed as (name, rows) stacked into one weight (rows padded with zeros to a
    multiple of `pad_to`, so that the product's output rows stay aligned); returns (weight, first row of each)."""
    names, shapes = [n for n, _ in names_rows], [int(r) for _, r in names_rows]
    total = -(-sum(shapes) // pad_to) * pad_to
    w = torch.zeros((total, hidden), dtype=load.dtype(*names), device=rt.device)
    offsets, at = [], 0
    for n, rows in zip(names, shapes):
        load(n, out=w[at:at + rows])
        offsets.append(at)
        at += rows
    return w, offsets


class DecayLinearAttention(Mixer):
    kind = "decay_linear_attention"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        hid, H, d, dv = (params[k] for k in ("hidden_size", "n_heads", "key_dim", "value_dim"))
        return {"q": TensorWant((H * d, hid)), "k": TensorWant((H * d, hid)), "v": TensorWant((H * dv, hid)),
                "g": TensorWant((H * dv, hid)), "o": TensorWant((hid, H * dv)), "norm": TensorWant((H * dv,), "norm")}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.H = int(params["hidden_size"]), int(params["n_heads"])
        self.d, self.dv = int(params["key_dim"]), int(params["value_dim"])
        self.eps = float(params["eps"])
        if params.get("feature_map", "silu") != "silu" or params.get("out_gate", "sigmoid") != "sigmoid":
            raise ValueError("decay_linear_attention computes the silu feature map and a sigmoid output gate only")
        decay = [float(v) for v in params["decay"]]
        if len(decay) != self.H:
            raise ValueError(f"{len(decay)} decays for {self.H} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=rt.device)
        self.w_in, (self.q_off, self.k_off, self.v_off, self.g_off) = pack_rows(
            load, (("q", self.H * self.d), ("k", self.H * self.d), ("v", self.H * self.dv), ("g", self.H * self.dv)),
            self.hidden, rt)
        self.w_o, self.norm = load("o"), load("norm")
        self.state_floats = self.H * scan_state_floats(self.d, self.dv)

    def cache_requirement(self):
        return StateRequirement((self.state_floats,), torch.float32)

    def step_arrays(self, shape, cache):
        return {} if shape.all_single else {"seq_spans": lambda: seq_spans_array(shape)}

    def step(self, x, ctx, cache, position, writes_cache=True):
        if not writes_cache:
            raise ValueError("a mixer with state of its own cannot read another layer's")
        proj = linear(x, self.w_in)
        o = kernels.decay_scan(proj, (self.q_off, self.k_off, self.v_off), self.decay, cache.state, ctx.seq_spans(),
                               ctx.tok_slot, self.H, self.d, self.dv)
        y = kernels.gated_group_rmsnorm(o, proj[:, self.g_off:self.g_off + self.H * self.dv], self.norm, self.eps,
                                        groups=1, gate_kind="sigmoid")
        return linear(y, self.w_o)


register_part(DecayLinearAttention.kind, DecayLinearAttention)

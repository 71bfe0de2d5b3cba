"""Attention whose keys and values are expanded from a cached low-rank latent, as a mixer.

    q = Wq x = per head [ plain_dim unrotated | rot_dim rotated ]
    [c | kr] = Wdkv x;  c <- rmsnorm(c) * w  (kv_rank);  kr (rot_dim): one rotated key part shared by all heads
    head h:  key = [ Wuk,h c | rot(kr) ],  value = Wuv,h c
    score = (q_plain . Wuk,h c + rot(q_rot) . rot(kr)) * softmax_scale,  causal
    softmax whose denominator also holds exp(sink_h) (optional, one learned number per head)
    y = Wo concat_h( sum_j p_j Wuv,h c_j )

Only c and rot(kr) are cached: one row per position in a single-plane paged entry.  The expansion is never
materialised: q'_h = Wuk,h^T q_plain,h is made by a per-head product, attention runs over the cached rows for
all heads (score q'_h . c_j + rot(q_rot) . rot(kr_j), values c_j), and Wuv,h is applied to the result.

Which attention runs.  Everything under float32, and short portions: the exact-order kernel (scores, softmax
and weighted sum float32, one block per token and head).  Decode steps in bfloat16: the shared-rows kernel,
which stages the cached rows in shared memory once for 32 heads (asynchronous copies, a chunk ahead), cuts the
keys into slices and does both products on tensor cores (mma.sync; float32 scores, softmax and sums, the
weights rounded to bfloat16 as the second product's operand).  Portions of `PRODUCT_MIN_ROWS`
tokens and more in bfloat16: because all heads share the cached rows, the scores of a block of tokens are one
matrix product [tokens x heads, row] . [row, keys] with float32 results, the softmax (causal, with the sink,
float32) is this package's kernel, and the weighted sum is a second product [tokens x heads, keys] . [keys,
kv_rank]; the sequence's rows are gathered from its pages once per step and the tokens are cut into blocks
whose scores fit `SCORE_BYTES`.  Tensor cores do both products; the weights are rounded to bfloat16 only as
the second product's operand.
The rotation is the position part's (its frequencies, magnitude and layout; this mixer's kernel pairs
dimension 2i with 2i+1).  Upstream has grouped-query attention only (src/models/qwen3/qwen3.cpp:140-179).
"""
from __future__ import annotations

import torch

from ..cache import KVRequirement
from ..ops import kernels, linear, per_head_linear
from ..weights.loader import TensorWant
from .base import Mixer, register_part
from .linear_attention import pack_rows


# From how many new tokens of a sequence on a bfloat16 step runs attention as product - softmax - product.
PRODUCT_MIN_ROWS = 32
SCORE_BYTES = 256 << 20        # float32 scores of one block of tokens (all heads, all keys)


class LatentAttention(Mixer):
    kind = "latent_attention"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        hid, H, d, dr, dv, r = (params[k] for k in ("hidden_size", "n_heads", "plain_dim", "rot_dim", "value_dim",
                                                    "kv_rank"))
        w = {"q": TensorWant((H * (d + dr), hid)), "dkv": TensorWant((r + dr, hid)), "dkv.norm": TensorWant((r,), "norm"),
             "uk": TensorWant((H * d, r)), "uv": TensorWant((H * dv, r)), "o": TensorWant((hid, H * dv))}
        if params.get("sink", False):
            w["sink"] = TensorWant((H,), std_scale=20.0)
        return w

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.H = int(params["hidden_size"]), int(params["n_heads"])
        self.d, self.dr, self.dv, self.rank = (int(params[k]) for k in ("plain_dim", "rot_dim", "value_dim", "kv_rank"))
        self.scale, self.eps = float(params["softmax_scale"]), float(params["eps"])
        self.row = -(-(self.rank + self.dr) // 8) * 8             # a cache row, padded for the kernel's 16-byte loads
        self.w_in, (self.q_off, self.c_off) = pack_rows(
            load, (("q", self.H * (self.d + self.dr)), ("dkv", self.rank + self.dr)), self.hidden, rt)
        self.c_norm = load("dkv.norm")
        # Wuk per head as [rank, plain_dim]: the product q'_h = Wuk,h^T q_h in the [out, in] form of the others
        self.w_uk_t = load("uk").view(self.H, self.d, self.rank).transpose(1, 2).contiguous()
        self.w_uv = load("uv").view(self.H, self.dv, self.rank)
        self.w_o = load("o")
        self.sink = load("sink") if params.get("sink", False) else None
        self._no_rotation = None

    def cache_requirement(self):
        return KVRequirement(1, self.row, None, planes=1)

    def _rotation(self, position, device):
        if position is not None:
            freq, magnitude, n_rot, layout = position.rotary_frequencies()
            if layout != "interleaved":
                raise ValueError("latent_attention rotates pairs (2i, 2i+1): the position part must be 'interleaved'")
            if n_rot > self.dr:
                raise ValueError(f"{n_rot} rotated dimensions of a key part of {self.dr}")
            return freq, magnitude, n_rot
        if self._no_rotation is None:
            self._no_rotation = torch.zeros(0, dtype=torch.float32, device=device)
        return self._no_rotation, 1.0, 0

    def step(self, x, ctx, cache, position, writes_cache=True):
        kv = cache.kv
        n = x.shape[0]
        freq, magnitude, n_rot = self._rotation(position, x.device)
        proj = linear(x, self.w_in)
        q = proj[:, self.q_off:self.q_off + self.H * (self.d + self.dr)].view(n, self.H, self.d + self.dr)
        q_lat = per_head_linear(q[:, :, :self.d], self.w_uk_t)                       # [n, H, rank]
        q_rows = kernels.latent_prepare(proj, self.q_off, self.c_off, q_lat, self.c_norm, self.eps, freq, magnitude,
                                        n_rot, ctx.tok_pos, ctx.tok_slot, kv.block_table, kv.k_pool, self.H, self.d,
                                        self.dr, self.rank, ctx.status, append=writes_cache)
        o_lat = self.attend(q_rows, kv, ctx)
        o = per_head_linear(o_lat.view(n, self.H, self.rank), self.w_uv)             # [n, H, value_dim]
        return linear(o.view(n, self.H * self.dv), self.w_o)


    def attend(self, q_rows, kv, ctx):
        """Attention of q_rows [n, H, row] over the cached rows; returns [n, H * kv_rank]."""
        by_products = (q_rows.dtype == torch.bfloat16 and not ctx.all_single and not ctx.captured and ctx.seq_lens
                       and max(ctx.seq_lens) >= PRODUCT_MIN_ROWS)
        if ctx.all_single and kernels.latent_decode_takes(q_rows.dtype, q_rows.shape[2], self.rank, self.H):
            return kernels.latent_decode(q_rows, kv.k_pool, kv.block_table, ctx.tok_pos, ctx.tok_slot, self.scale,
                                         self.sink, self.rank, ctx.status)
        if not by_products:
            return kernels.attention_generic(q_rows, kv.k_pool, kv.k_pool, kv.block_table, ctx.tok_pos, ctx.tok_slot,
                                             self.scale, 0, ctx.status, sinks=self.sink, value_dim=self.rank)
        n, H, row = q_rows.shape
        out = torch.empty((n, H * self.rank), dtype=q_rows.dtype, device=q_rows.device)
        page = kv.page_size
        pool = kv.k_pool.view(kv.k_pool.shape[0], page, row)
        short = [(s, st, m, p) for s, st, m, p in zip(ctx.seq_slots, ctx.seq_starts, ctx.seq_lens, ctx.seq_past)
                 if m < PRODUCT_MIN_ROWS]
        for slot, start, n_new, past in zip(ctx.seq_slots, ctx.seq_starts, ctx.seq_lens, ctx.seq_past):
            if n_new < PRODUCT_MIN_ROWS:
                continue
            n_pages = -(-(past + n_new) // page)
            rows = pool.index_select(0, kv.block_table[slot, :n_pages].long()).view(n_pages * page, row)
            block = max(1, min(n_new, SCORE_BYTES // (4 * H * n_pages * page)))
            for q0 in range(0, n_new, block):
                tq = min(block, n_new - q0)
                keys = min(-(-(past + q0 + tq) // 8) * 8, n_pages * page)      # what this block sees, padded to 8
                q = q_rows[start + q0:start + q0 + tq].view(tq * H, row)
                scores = torch.mm(q, rows[:keys].t(), out_dtype=torch.float32)
                weights = kernels.causal_sink_softmax(scores, H, past + q0, self.scale, self.sink, q_rows.dtype)
                out[start + q0:start + q0 + tq] = torch.mm(weights, rows[:keys, :self.rank]).view(tq, H * self.rank)
        if short:                                  # sequences that bring a few tokens: the exact-order kernel
            idx = torch.cat([torch.arange(st, st + m) for _, st, m, _ in short]).to(q_rows.device)
            part = kernels.attention_generic(q_rows.index_select(0, idx).contiguous(), kv.k_pool, kv.k_pool,
                                             kv.block_table, ctx.tok_pos.index_select(0, idx).contiguous(),
                                             ctx.tok_slot.index_select(0, idx).contiguous(), self.scale, 0,
                                             ctx.status, sinks=self.sink, value_dim=self.rank)
            out.index_copy_(0, idx, part)
        return out


register_part(LatentAttention.kind, LatentAttention)

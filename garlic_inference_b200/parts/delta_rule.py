"""The gated delta rule behind short causal convolutions, as a mixer with a matrix of state per head.

    q, k, v = silu(conv(Wq x)), silu(conv(Wk x)), silu(conv(Wv x))     conv: per channel over time, `conv_taps`
                                                                        taps, the last on the current token
    q, k <- q / sqrt(|q|^2 + unit_eps) * key_dim^-1/2,  k / sqrt(|k|^2 + unit_eps)        per head
    beta = sigmoid(Wb x),   g = exp(-exp(A_h) softplus(Wa x + dt_h))                        one per head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q       float32; the read-out sees this token's write
    y = Wo( o / rms(o over value_dim) * w * silu(Wg x) )

Variants, by parameter: `decay_per` "channel" gives a decay per head and key channel (the logits and dt have
heads x key_dim elements and row c of S is multiplied by g[c]); `decay_rank` r makes the decay's projection the
product of two thin ones, Wa2 (Wa1 x) with Wa1 [r, hidden] (tensors `a1`, `a2` instead of `a`); `gate_rank` the
same for the output gate (`g1`, `g2` instead of `g`); `out_gate` is "silu" or "sigmoid".

q and k have `n_kv_heads` heads; head h of v reads q/k head h // (n_heads // n_kv_heads).  The projections of q,
k, v and the output gate are one packed product; those of beta and of the decay (two rows per head) are a
second one whose result stays float32, because the decay's logit is multiplied by exp(A_h) and passes two
exponentials, which would magnify a 16-bit rounding.  A slot's state row holds the matrices of all heads and, behind them, the
last conv_taps - 1 inputs of the convolutions.  Upstream has no recurrent mixer.
"""
from __future__ import annotations

import torch

from ..cache import StateRequirement
from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .base import Mixer, register_part, seq_spans_array
from .linear_attention import pack_rows, scan_state_floats


class GatedDeltaRule(Mixer):
    kind = "gated_delta_rule"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        hid, H, Hk, d, dv, K = (params[k] for k in ("hidden_size", "n_heads", "n_kv_heads", "key_dim", "value_dim",
                                                    "conv_taps"))
        taps = lambda rows: TensorWant((rows, K), std_scale=8.0)
        n_decay = H * d if params.get("decay_per", "head") == "channel" else H
        ra, rg = params.get("decay_rank"), params.get("gate_rank")
        w = {"q": TensorWant((Hk * d, hid)), "k": TensorWant((Hk * d, hid)), "v": TensorWant((H * dv, hid)),
             "q.conv": taps(Hk * d), "k.conv": taps(Hk * d), "v.conv": taps(H * dv),
             "b": TensorWant((H, hid)), "A_log": TensorWant((H,), std_scale=10.0),
             "dt_bias": TensorWant((n_decay,), std_scale=10.0), "o": TensorWant((hid, H * dv)),
             "norm": TensorWant((dv,), "norm")}
        if ra:
            w["a1"], w["a2"] = TensorWant((ra, hid)), TensorWant((n_decay, ra), std_scale=4.0)
        else:
            w["a"] = TensorWant((n_decay, hid))
        if rg:
            w["g1"], w["g2"] = TensorWant((rg, hid)), TensorWant((H * dv, rg), std_scale=4.0)
        else:
            w["g"] = TensorWant((H * dv, hid))
        return w

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.H, self.Hk = int(params["hidden_size"]), int(params["n_heads"]), int(params["n_kv_heads"])
        self.d, self.dv, self.K = int(params["key_dim"]), int(params["value_dim"]), int(params["conv_taps"])
        self.eps, self.unit_eps = float(params["eps"]), float(params.get("unit_eps", 1e-6))
        if self.H % self.Hk:
            raise ValueError(f"{self.H} heads are no multiple of {self.Hk} key heads")
        self.channel_decay = params.get("decay_per", "head") == "channel"
        if params.get("decay_per", "head") not in ("head", "channel"):
            raise ValueError(f"decay_per {params['decay_per']!r} is neither 'head' nor 'channel'")
        self.n_decay = self.H * self.d if self.channel_decay else self.H
        self.decay_rank, self.gate_rank = params.get("decay_rank"), params.get("gate_rank")
        self.out_gate = params.get("out_gate", "silu")
        if self.out_gate not in ("silu", "sigmoid"):
            raise ValueError(f"out_gate {self.out_gate!r} is neither 'silu' nor 'sigmoid'")
        # one packed product in the activation type: q, k, v, the gate (or its thin first factor) and the thin first
        # factor of the decay; a second one whose result stays float32: beta and a full-rank decay
        first = [("q", self.Hk * self.d), ("k", self.Hk * self.d), ("v", self.H * self.dv),
                 ("g1", int(self.gate_rank)) if self.gate_rank else ("g", self.H * self.dv)]
        if self.decay_rank:
            first.append(("a1", int(self.decay_rank)))
        self.w_in, offs = pack_rows(load, first, self.hidden, rt)
        self.q_off, self.k_off, self.v_off, self.g_off = offs[:4]
        self.a1_off = offs[4] if self.decay_rank else None
        second = [("b", self.H)] + ([] if self.decay_rank else [("a", self.n_decay)])
        self.w_ba, offs = pack_rows(load, second, self.hidden, rt)
        self.b_off, self.a_off = offs[0], (offs[1] if not self.decay_rank else 0)
        self.w_a2 = load("a2") if self.decay_rank else None
        self.w_g2 = load("g2") if self.gate_rank else None
        self.C = 2 * self.Hk * self.d + self.H * self.dv              # channels that pass the convolution
        self.taps = torch.cat([load("q.conv"), load("k.conv"), load("v.conv")]).contiguous()
        self.A_log, self.dt_bias = load("A_log"), load("dt_bias")
        self.w_o, self.norm = load("o"), load("norm")
        self.scan_floats = self.H * scan_state_floats(self.d, self.dv)
        self.state_floats = -(-(self.scan_floats + (self.K - 1) * self.C) // 4) * 4

    def cache_requirement(self):
        return StateRequirement((self.state_floats,), torch.float32)

    def step_arrays(self, shape, cache):
        return {} if shape.all_single else {"seq_spans": lambda: seq_spans_array(shape)}

    def pre_output(self, x, ctx, cache, position, writes_cache=True, out=None, out_mul=1.0):
        """Everything before the output projection: [n, n_heads * value_dim] in the activation type, times
        `out_mul`, written into `out` (columns of a wider matrix) when given."""
        if not writes_cache:
            raise ValueError("a mixer with state of its own cannot read another layer's")
        proj = linear(x, self.w_in)
        conv_in = proj[:, :self.C]
        conv_state = cache.state[:, self.scan_floats:]
        qkv = kernels.causal_conv_silu(conv_in, self.taps, conv_state, ctx.tok_slot, renew_state=ctx.all_single)
        if not ctx.all_single:
            kernels.conv_state_update(conv_in, self.K, conv_state, ctx.tok_slot)
        ba = linear(x, self.w_ba, out_dtype=torch.float32)
        decay = None
        if self.decay_rank:                          # the decay's logits stay float32 out of the second thin product
            decay = linear(proj[:, self.a1_off:self.a1_off + self.decay_rank].contiguous(), self.w_a2,
                           out_dtype=torch.float32)
        o = kernels.delta_scan(qkv, (self.q_off, self.k_off, self.v_off), ba, (self.b_off, self.a_off), self.A_log,
                               self.dt_bias, cache.state, ctx.seq_spans(), ctx.tok_slot, self.H, self.Hk, self.d,
                               self.dv, self.unit_eps, channel_decay=self.channel_decay, decay_logits=decay)
        if self.gate_rank:
            gate = linear(proj[:, self.g_off:self.g_off + self.gate_rank].contiguous(), self.w_g2)
        else:
            gate = proj[:, self.g_off:self.g_off + self.H * self.dv]
        return kernels.gated_group_rmsnorm(o, gate, self.norm, self.eps, groups=self.H, gate_kind=self.out_gate,
                                           mul=out_mul, out=out)

    def step(self, x, ctx, cache, position, writes_cache=True):
        return linear(self.pre_output(x, ctx, cache, position, writes_cache), self.w_o)


register_part(GatedDeltaRule.kind, GatedDeltaRule)

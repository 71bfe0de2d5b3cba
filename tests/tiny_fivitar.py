"""Tiny Fivitar configurations for the tests, and traces that cut prompts into portions.

The configurations differ from one another in every size: width, vocabulary, heads and key heads, key and value
sizes that are no multiples of the kernels' tiles, filters of 1 to 4 taps, rotation with and without YaRN and over
a part of the rotated dimensions, layers with and without feed-forward, the order of the mixers, and layers that
run another layer's tensors.
"""
from __future__ import annotations

import copy
from pathlib import Path

import numpy as np
import torch


def _latent(heads, dim, rot_dim, vdim, rank, dims=None, base=10000.0, scaling=None, scale=None):
    rot = {"base": base, "dims": dims or rot_dim}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "rot": rot,
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def _with(layer, ff=None, weights_of=None):
    out = dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


YARN = {"factor": 8.0, "original": 48, "fast": 16.0, "slow": 2.0}

TINY = {
    # one mixer each, no feed-forward: each mechanism alone
    "lightning": dict(vocab=300, width=64, eps=1e-5, seed=11, std=0.08, norm_std=0.1,
                      layers=[_with(_lightning(3, 72, 40, [0.5, 0.93, 0.999]))]),
    "latent": dict(vocab=300, width=64, eps=1e-6, seed=12, std=0.08, norm_std=0.1,
                   layers=[_with(_latent(3, 16, 8, 24, 20, scaling=YARN, scale=0.3))]),
    "delta": dict(vocab=300, width=64, eps=1e-5, seed=13, std=0.08, norm_std=0.1,
                  layers=[_with(_delta(4, 2, 24, 40, 3))]),
    # all mixers, every layer with a feed-forward, two layers on another layer's tensors
    "mix": dict(vocab=411, width=96, eps=2e-6, seed=14, std=0.06, norm_std=0.15,
                layers=[_with(_latent(2, 24, 16, 16, 40, dims=8, base=5000.0), ff=160),
                        _with(_delta(2, 2, 32, 24, 4), ff=128),
                        _with(_lightning(2, 40, 72, [0.9, 0.995]), ff=64),
                        _with(_delta(2, 2, 32, 24, 4), ff=128, weights_of=1),
                        _with(_latent(2, 24, 16, 16, 40, dims=8, base=5000.0), ff=160, weights_of=0),
                        _with(_lightning(1, 130, 8, [0.97]))]),
    # one head, one key head, a filter of one tap (no filter state), a rotated part without scaling
    "ones": dict(vocab=257, width=48, eps=1e-5, seed=15, std=0.1, norm_std=0.2,
                 layers=[_with(_delta(1, 1, 16, 16, 1), ff=48),
                         _with(_latent(1, 8, 4, 8, 8), ff=48),
                         _with(_lightning(1, 16, 16, [0.8])),
                         _with(_delta(3, 1, 8, 36, 2))]),
}

# Float32 is judged against the float64 run of the plain model, by the plain model's own float32 error: the
# engine may be `F32_FACTOR` times as far from the float64 logits as the plain float32 run is (and never closer
# than F32_FLOOR is asked of it).  Random models differ in how much they magnify rounding, and this bound moves
# with them.  Bfloat16 shares every kernel's logic with float32 and differs in the products' types, the cache
# rows and the rounded copy of the stream; a fault there moves every position, so it is judged by the median
# over positions of the root-mean-square error of a row relative to the logits' own, and the worst row by a
# loose bound.
F32_FACTOR, F32_FLOOR = 4.0, 2e-6
BF16_MEDIAN, BF16_WORST = 2e-2, 0.5


def row_errors(got, want64):
    """{(request, position): (largest difference / largest logit, rms difference / rms logit)}."""
    out = {}
    for rid in got:
        ref = want64[rid]
        top, rms = float(np.abs(ref).max()), float(np.sqrt((ref ** 2).mean()))
        for p, row in got[rid].items():
            assert np.isfinite(row).all(), f"request {rid} position {p}: non-finite logits"
            d = row.astype(np.float64) - ref[p]
            out[(rid, p)] = (float(np.abs(d).max()) / top, float(np.sqrt((d ** 2).mean())) / rms)
    return out


def judge(got, want64, plain32, dtype: str, what: str) -> float:
    """Assert that the engine's logits `got` {request: {position: row}} are as close to the float64 logits as
    the rules above ask; returns the worst largest-difference error."""
    errs = row_errors(got, want64)
    worst_at = max(errs, key=lambda k: errs[k][0])
    worst = errs[worst_at][0]
    if dtype == "float32":
        own = row_errors({r: dict(enumerate(plain32[r])) for r in got}, want64)
        bound = max(F32_FACTOR * max(e[0] for e in own.values()), F32_FLOOR)
        assert worst <= bound, (f"{what}: request {worst_at[0]} position {worst_at[1]} is {worst:.2e} of the largest "
                                f"logit from the float64 result; the plain float32 run allows {bound:.2e}")
    else:
        rms = sorted(e[1] for e in errs.values())
        assert rms[len(rms) // 2] <= BF16_MEDIAN and rms[-1] <= BF16_WORST, (
            f"{what}: median rms error {rms[len(rms) // 2]:.2e} (allowed {BF16_MEDIAN:.0e}), worst {rms[-1]:.2e} "
            f"(allowed {BF16_WORST})")
    return worst


def config_dict(name: str) -> dict:
    t = TINY[name]
    return {"architecture": "Fivitar", "vocab": t["vocab"], "width": t["width"], "norm": {"eps": t["eps"]},
            "layers": copy.deepcopy(t["layers"])}


def make_config(name: str):
    from garlic_inference_b200.config import FivitarConfig
    return FivitarConfig.from_dict(config_dict(name))


def write_model(name: str, folder) -> Path:
    from garlic_inference_b200 import write_random_model
    t = TINY[name]
    return write_random_model(folder, make_config(name), seed=t["seed"], std=t["std"], norm_std=t["norm_std"])


def plain_logits(model_dir, requests, dtype=torch.float32) -> dict:
    import plain_fivitar as plain
    cfg, weights = plain.read_model_dir(model_dir)
    return {rid: plain.forward(cfg, weights, toks, dtype).to(torch.float64).numpy() for rid, toks in requests.items()}


def plain_pair(model_dir, requests):
    """(float64 logits, float32 logits) of the plain model for every request."""
    return plain_logits(model_dir, requests, torch.float64), plain_logits(model_dir, requests, torch.float32)


def trace_portions(requests, sizes, together=False):
    """Prompts cut into portions whose sizes cycle through `sizes`; every position wanted.  Alone: one request
    after the other.  Together: all requests start in one step, and each later step brings the next portion of
    every request that still has tokens (each step's entries either all start or all go on)."""
    steps = []
    groups = [list(requests)] if together else [[rid] for rid in requests]
    for group in groups:
        at = {rid: 0 for rid in group}
        k = 0
        while any(at[rid] < len(requests[rid]) for rid in group):
            n = sizes[k % len(sizes)]
            entries, end = [], []
            for rid in group:
                toks = requests[rid]
                if at[rid] >= len(toks):
                    continue
                part = toks[at[rid]:at[rid] + n]
                entries.append({"id": rid, "tokens": part, "want": list(range(len(part)))})
                at[rid] += len(part)
                if at[rid] == len(toks):
                    end.append(rid)
            steps.append({"step": len(steps), "entries": entries, "end": end})
            k += 1
    return steps

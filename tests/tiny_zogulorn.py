"""Tiny Zogulorn configurations for the tests.

They differ from one another in every size: width, vocabulary, heads and key/value heads (equal, a fraction, one),
key and value sizes that are equal, smaller or larger and no multiples of the kernels' tiles, rotation over all
or a part of a head, chunks of 1 to 48 positions, filters of 1 to 4 taps, experts of which all, some or one are
chosen, layers with and without a feed-forward, the order of the mixers, and layers that read another layer's
keys and values.
"""
from __future__ import annotations

import copy
from pathlib import Path

import torch

from tiny_fivitar import BF16_MEDIAN, judge, row_errors, trace_portions  # noqa: F401  (the same rules of judgement)


def _left(heads, kv, dim, vdim, chunk, dims=None, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
            "rot": {"base": base, "dims": dim if dims is None else dims}, "scale": scale or dim ** -0.5}


def _right(heads, kv, dim, vdim, conv, rank=8):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "rank": rank}


def _parallel(left, right, a=0.7, b=1.2):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": a, "right_scale": b}}


def _attention(heads, kv, dim, vdim, chunk, conv, diff=0.5, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": chunk}, "conv": conv, "diff": diff,
         "scale": scale or dim ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _with(layer, mlp=None):
    return dict(layer, mlp=mlp)


TINY = {
    # each mechanism alone: one side of the parallel mixer switched off by its factor, no feed-forward
    "left": dict(vocab=300, width=64, eps=1e-5, emb=4.0, seed=21, std=0.08, norm_std=0.1,
                 layers=[_with(_parallel(_left(4, 2, 16, 24, 48, dims=8, base=100.0, scale=2.0), _right(2, 1, 8, 8, 2), a=1.3, b=0.0))]),
    "right": dict(vocab=300, width=64, eps=1e-5, emb=2.0, seed=22, std=0.08, norm_std=0.1,
                  layers=[_with(_parallel(_left(1, 1, 8, 8, 4), _right(4, 2, 24, 40, 3, rank=16), a=0.0, b=0.9))]),
    "diff": dict(vocab=300, width=64, eps=1e-6, emb=3.0, seed=23, std=0.08, norm_std=0.1,
                 layers=[_with(_attention(3, 3, 24, 40, 20, 3, diff=0.3))]),
    "dense": dict(vocab=280, width=48, eps=1e-5, emb=1.0, seed=24, std=0.1, norm_std=0.1,
                  layers=[_with(_attention(2, 1, 16, 16, 7, 2), _dense(100))]),
    "moe": dict(vocab=280, width=48, eps=1e-5, emb=5.0, seed=25, std=0.1, norm_std=0.1,
                layers=[_with(_attention(2, 2, 8, 16, 64, 4, diff=0.7), _moe(40, 5, 2))]),
    # everything, in another order than any other configuration's; two layers on an earlier layer's keys and values
    "mix": dict(vocab=411, width=96, eps=2e-6, emb=8.0, seed=26, std=0.06, norm_std=0.15,
                layers=[_with(_attention(4, 2, 16, 24, 33, 4, diff=0.4), _moe(48, 6, 3)),
                        _with(_parallel(_left(6, 3, 24, 16, 40, dims=12, base=5000.0), _right(3, 3, 40, 24, 4, rank=24)), _dense(128)),
                        _with(_attention(4, 2, 16, 24, 17, 2, diff=0.6, kv_from=0), _dense(64)),
                        _with(_parallel(_left(2, 2, 32, 32, 25), _right(4, 1, 16, 36, 3)), _moe(32, 4, 4)),
                        _with(_attention(4, 2, 16, 24, 50, 3, diff=0.2, kv_from=0))]),
    # heads of 128 (the prompt kernel on tcgen05 when the cache's pages are multiples of 64 tokens), chunks that are
    # no multiple of its tiles
    "wide": dict(vocab=300, width=64, eps=1e-5, emb=2.0, seed=28, std=0.08, norm_std=0.1,
                 layers=[_with(_parallel(_left(2, 1, 128, 128, 70, dims=64, scale=1.0), _right(2, 1, 8, 8, 2), a=1.1, b=0.4),
                               _dense(64))]),
    # one head, one key head, one tap (no filter state), chunks of one position, one expert of one, rotation of
    # the whole head and of none of it
    "ones": dict(vocab=257, width=48, eps=1e-5, emb=1.5, seed=27, std=0.1, norm_std=0.2,
                 layers=[_with(_parallel(_left(1, 1, 16, 16, 1), _right(1, 1, 16, 16, 1)), _moe(24, 1, 1)),
                         _with(_attention(1, 1, 8, 8, 5, 1), _dense(48)),
                         _with(_parallel(_left(2, 1, 8, 24, 9, dims=0), _right(3, 1, 8, 36, 2))),
                         _with(_attention(1, 1, 8, 8, 1, 2, kv_from=1), _moe(16, 3, 3))]),
}


def config_dict(name: str) -> dict:
    t = TINY[name]
    return {"architecture": "Zogulorn", "vocab": t["vocab"], "width": t["width"], "embedding": {"scale": t["emb"]},
            "norm": {"eps": t["eps"]}, "layers": copy.deepcopy(t["layers"])}


def make_config(name: str):
    from garlic_inference_b200.config import ZogulornConfig
    return ZogulornConfig.from_dict(config_dict(name))


def write_model(name: str, folder) -> Path:
    from garlic_inference_b200 import write_random_model
    t = TINY[name]
    return write_random_model(folder, make_config(name), seed=t["seed"], std=t["std"], norm_std=t["norm_std"])


def plain_logits(model_dir, requests, dtype=torch.float32) -> dict:
    import plain_zogulorn as plain
    cfg, weights = plain.read_model_dir(model_dir)
    return {rid: plain.forward(cfg, weights, toks, dtype).to(torch.float64).numpy() for rid, toks in requests.items()}


def plain_pair(model_dir, requests):
    """(float64 logits, float32 logits) of the plain model for every request."""
    return plain_logits(model_dir, requests, torch.float64), plain_logits(model_dir, requests, torch.float32)

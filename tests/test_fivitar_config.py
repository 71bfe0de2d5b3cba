"""Fivitar on the CPU: its configuration, plan and tensors, and the plain implementation against closed forms."""
import json
import math
import warnings

import numpy as np
import pytest
import torch

import plain_fivitar as plain
import tiny_fivitar as tf


def test_registry_reads_the_architecture_string_and_round_trips(tmp_path):
    from garlic_inference_b200 import load_config
    from garlic_inference_b200.config import FivitarConfig, known_architectures
    assert "Fivitar" in known_architectures()
    (tmp_path / "config.json").write_text(json.dumps(tf.config_dict("mix")))
    cfg = load_config(tmp_path)
    assert type(cfg) is FivitarConfig and cfg.width == 96 and cfg.vocab == 411 and cfg.norm_eps == 2e-6
    assert FivitarConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.to_dict()["architecture"] == "Fivitar" and len(cfg.to_dict()["layers"]) == 6


def test_plan_shares_weights_but_not_cache_entries():
    from garlic_inference_b200.engine.model import wanted_tensors
    plan = tf.make_config("mix").plan()
    assert [(e.layer, e.cache) for e in plan.schedule] == [(0, 0), (1, 1), (2, 2), (1, 3), (0, 4), (3, 5)]
    assert len(plan.layers) == 4 and plan.n_cache_entries() == 6
    names = wanted_tensors(plan)
    assert not any(n.startswith(("l3.", "l4.")) for n in names), "layers that use another layer's tensors have none"
    assert tuple(names["l0.mix.q"].shape) == (2 * (24 + 16), 96) and tuple(names["l0.mix.dkv"].shape) == (40 + 16, 96)
    assert tuple(names["l1.mix.q.conv"].shape) == (2 * 32, 4) and tuple(names["l1.mix.norm"].shape) == (24,)
    assert tuple(names["l2.mix.norm"].shape) == (2 * 72,) and tuple(names["l5.mix.q"].shape) == (130, 96)
    assert "l5.mlp.up" not in names and "l5.norm2" not in names and "l5.rg2" not in names, "a layer without feed-forward"
    assert tuple(names["l0.rg1.b"].shape) == (96,) and tuple(names["l0.mlp.act"].shape) == (2,)
    assert len(plan.positions) == 1, "equal rotary constants are one part"


def test_refusals_and_warnings():
    from garlic_inference_b200.config import ConfigError, FivitarConfig
    bad = tf.config_dict("ones")
    bad["layers"][0] = dict(bad["layers"][0], type="convolution")
    with pytest.raises(ConfigError, match="convolution"):
        FivitarConfig.from_dict(bad)
    bad = tf.config_dict("mix")
    bad["layers"][3] = dict(bad["layers"][3], mixer=dict(bad["layers"][3]["mixer"], conv=2))
    with pytest.raises(ConfigError, match="differs"):
        FivitarConfig.from_dict(bad)
    bad = tf.config_dict("lightning")
    bad["layers"][0]["mixer"] = dict(bad["layers"][0]["mixer"], decay=[0.5])
    with pytest.raises(ConfigError, match="decays"):
        FivitarConfig.from_dict(bad)
    bad = tf.config_dict("ones")
    bad["layers"][0]["mlp"] = {"kind": "experts", "ff": 8}
    with pytest.raises(ConfigError, match="experts"):
        FivitarConfig.from_dict(bad)
    odd = tf.config_dict("ones")
    odd["layers"][1] = dict(odd["layers"][1], mixer=dict(odd["layers"][1]["mixer"], window=7))
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        FivitarConfig.from_dict(odd)
    assert any("window" in str(w.message) for w in seen)


def test_random_folder_loads_and_fits(tmp_path):
    from garlic_inference_b200.engine.model import wanted_tensors
    from garlic_inference_b200.weights import Checkpoint
    d = tf.write_model("ones", tmp_path / "ones")
    Checkpoint(d).check(wanted_tensors(tf.make_config("ones").plan()))
    cfg, w = plain.read_model_dir(d)
    assert cfg == tf.config_dict("ones") and w["l0.mix.q.conv"].shape == (16, 1)
    logits = plain.forward(cfg, w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 257) and torch.isfinite(logits).all()


def test_state_layout_rule():
    from garlic_inference_b200.parts.linear_attention import scan_state_floats
    assert [scan_state_floats(d, 10) for d in (1, 16, 17, 64, 65, 128, 129, 256)] == \
        [160, 160, 320, 640, 1280, 1280, 2560, 2560]
    with pytest.raises(ValueError):
        scan_state_floats(257, 1)


def test_rotary_part_frequencies_match_the_plain_ones():
    from garlic_inference_b200.parts.rotary import RotaryPositions
    for dims, base, yarn in ((8, 5000.0, None), (16, 250000.0, tf.YARN), (4, 100.0, {"factor": 2.0, "original": 8,
                                                                                  "fast": 4.0, "slow": 1.0})):
        f, mag = RotaryPositions.frequencies(dims, base, yarn)
        pf, pmag = plain.yarn_frequencies(dims, base, yarn)
        np.testing.assert_allclose(f.numpy(), np.asarray(pf), rtol=1e-14)
        assert mag == pytest.approx(pmag, rel=1e-15)
    f, mag = plain.yarn_frequencies(16, 1e4, {"factor": 1.0, "original": 64, "fast": 32.0, "slow": 1.0})
    assert mag == 1.0 and f == [1e4 ** (-2.0 * i / 16) for i in range(8)], "factor 1 changes nothing"


# ---- the plain implementation against closed forms of the same equations -------------------------
def test_plain_lightning_equals_the_sum_over_earlier_tokens():
    torch.manual_seed(0)
    T, H, d, dv, hid = 9, 2, 5, 3, 7
    m = {"heads": H, "dim": d, "vdim": dv, "decay": [0.7, 0.95]}
    w = {"q": torch.randn(H * d, hid), "k": torch.randn(H * d, hid), "v": torch.randn(H * dv, hid),
         "g": torch.randn(H * dv, hid), "o": torch.randn(hid, H * dv), "norm": torch.rand(H * dv) + 0.5}
    h = torch.randn(T, hid, dtype=torch.float64)
    w = {k: v.double() for k, v in w.items()}
    got = plain.lightning_mixer(h, w, m, 1e-5)
    q, k, v = (plain.silu(h @ w[n].T).view(T, H, -1) for n in "qkv")
    o = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        for j in range(t + 1):
            for hh in range(H):
                o[t, hh] += m["decay"][hh] ** (t - j) * (q[t, hh] @ k[j, hh]) * v[j, hh]
    want = (plain.rms_norm(o.reshape(T, -1), w["norm"], 1e-5) * plain.sigmoid(h @ w["g"].T)) @ w["o"].T
    torch.testing.assert_close(got, want, rtol=1e-10, atol=1e-10)


def test_plain_sink_softmax_and_first_token():
    """With one key the weight of the token on itself is e^s / (e^s + e^sink): the sink counts once, unscaled."""
    torch.manual_seed(1)
    hid, H, d, dr, dv, r = 6, 2, 4, 2, 3, 5
    m = {"heads": H, "dim": d, "rot_dim": dr, "vdim": dv, "kv_rank": r, "scale": 0.37,
         "rot": {"base": 100.0, "dims": dr}}
    w = {"q": torch.randn(H * (d + dr), hid), "dkv": torch.randn(r + dr, hid), "dkv.norm": torch.rand(r) + 0.5,
         "uk": torch.randn(H * d, r), "uv": torch.randn(H * dv, r), "sink": torch.tensor([0.3, -1.2]),
         "o": torch.eye(H * dv)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(1, hid, dtype=torch.float64)
    got = plain.latent_attention_mixer(h, w, m, 1e-6)[0].view(H, dv)
    q = (h @ w["q"].T).view(H, d + dr)
    ckr = (h @ w["dkv"].T)[0]
    c = ckr[:r] / torch.sqrt((ckr[:r] ** 2).mean() + 1e-6) * w["dkv.norm"]
    for hh in range(H):
        k = w["uk"].view(H, d, r)[hh] @ c
        s = (q[hh, :d] @ k + q[hh, d:] @ ckr[r:]) * 0.37          # position 0: no rotation
        p = math.exp(s) / (math.exp(s) + math.exp(float(w["sink"][hh])))
        torch.testing.assert_close(got[hh], p * (w["uv"].view(H, dv, r)[hh] @ c), rtol=1e-10, atol=1e-12)


def test_plain_delta_rule_writes_then_reads():
    """One token from an empty state: S = k u^T with u = beta v, so o = (q . k) beta v."""
    torch.manual_seed(2)
    hid, H, Hk, d, dv = 5, 2, 1, 4, 3
    m = {"heads": H, "kv_heads": Hk, "dim": d, "vdim": dv, "conv": 2}
    w = {"q": torch.randn(Hk * d, hid), "k": torch.randn(Hk * d, hid), "v": torch.randn(H * dv, hid),
         "q.conv": torch.randn(Hk * d, 2), "k.conv": torch.randn(Hk * d, 2), "v.conv": torch.randn(H * dv, 2),
         "b": torch.randn(H, hid), "a": torch.randn(H, hid), "A_log": torch.randn(H), "dt_bias": torch.randn(H),
         "g": torch.randn(H * dv, hid), "o": torch.eye(H * dv), "norm": torch.ones(dv)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(1, hid, dtype=torch.float64)
    got = plain.delta_mixer(h, w, m, 1e-5)[0].view(H, dv)
    q = plain.silu((h @ w["q"].T)[0] * w["q.conv"][:, -1])
    k = plain.silu((h @ w["k"].T)[0] * w["k.conv"][:, -1])
    v = plain.silu((h @ w["v"].T)[0] * w["v.conv"][:, -1]).view(H, dv)
    q = q / torch.sqrt(q @ q + 1e-6) * d ** -0.5
    k = k / torch.sqrt(k @ k + 1e-6)
    beta = plain.sigmoid(h @ w["b"].T)[0]
    for hh in range(H):
        o = (q @ k) * beta[hh] * v[hh]
        o = o / torch.sqrt((o * o).mean() + 1e-5) * plain.silu(h @ w["g"].T)[0].view(H, dv)[hh]
        torch.testing.assert_close(got[hh], o, rtol=1e-10, atol=1e-12)


def test_plain_xielu_branches():
    z = torch.tensor([-2.0, -1e-3, 0.0, 1e-3, 3.0], dtype=torch.float64)
    p, q = 0.4, -0.7
    sp = lambda x: math.log1p(math.exp(x))
    want = [((0.5 + sp(q)) * (math.exp(v) - 1 - v) + v / 2) if v <= 0 else (sp(p) * v * v + v / 2) for v in z.tolist()]
    torch.testing.assert_close(plain.xielu(z, p, q), torch.tensor(want, dtype=torch.float64), rtol=1e-12, atol=1e-15)

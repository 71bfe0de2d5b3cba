"""Zogulorn on the CPU: its configuration, plan and tensors, and the plain implementation against closed forms."""
import json
import math
import warnings

import pytest
import torch

import plain_zogulorn as plain
import tiny_zogulorn as tz


def test_registry_reads_the_architecture_string_and_round_trips(tmp_path):
    from garlic_inference_b200 import load_config
    from garlic_inference_b200.config import ZogulornConfig, known_architectures
    assert "Zogulorn" in known_architectures()
    (tmp_path / "config.json").write_text(json.dumps(tz.config_dict("mix")))
    cfg = load_config(tmp_path)
    assert type(cfg) is ZogulornConfig and cfg.width == 96 and cfg.vocab == 411 and cfg.embedding_scale == 8.0
    assert ZogulornConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict() == tz.config_dict("mix")


def test_plan_tensors_and_borrowed_keys():
    from garlic_inference_b200.engine.model import wanted_tensors
    plan = tz.make_config("mix").plan()
    assert [(e.layer, e.cache, e.kv_cache) for e in plan.schedule] == [(0, 0, None), (1, 1, None), (2, 2, 0), (3, 3, None),
                                                                      (4, 4, 0)]
    names = wanted_tensors(plan)
    shape = lambda n: tuple(names[n].shape)
    assert shape("l0.mix.q") == (4 * 2 * 16, 96) and shape("l0.mix.k") == (2 * 2 * 16, 96) and shape("l0.mix.v") == (2 * 24, 96)
    assert shape("l0.mix.q.conv") == (128, 4) and shape("l0.mix.lq2") == (16,) and shape("l0.mix.g") == (4, 96)
    assert shape("l0.mix.o") == (96, 4 * 24) and shape("l0.norm1.alpha") == () and shape("l0.norm1.b") == (96,)
    assert "l2.mix.k" not in names and "l2.mix.v.conv" not in names and shape("l2.mix.q.conv") == (128, 2)
    assert "l4.mlp.router" not in names and "l4.norm2" not in names and "l4.ls2" not in names and "l4.ls1" in names
    assert shape("l1.mix.left.q") == (6 * 24, 96) and shape("l1.mix.left.v") == (3 * 16, 96) and shape("l1.mix.left.g") == (6, 96)
    assert shape("l1.mix.right.a1") == (24, 96) and shape("l1.mix.right.a2") == (3 * 40, 24)
    assert shape("l1.mix.right.dt_bias") == (3 * 40,) and shape("l1.mix.right.A_log") == (3,)
    assert shape("l1.mix.right.g2") == (3 * 24, 24) and shape("l1.mix.right.norm") == (24,)
    assert shape("l3.mix.right.q") == (1 * 16, 96) and shape("l3.mix.right.v") == (4 * 36, 96)
    assert shape("l0.mlp.e5.up") == (48, 96) and shape("l0.mlp.e0.down") == (96, 48) and shape("l0.mlp.router") == (6, 96)
    assert shape("l1.mlp.gate") == (128, 96) and shape("final.norm.alpha") == () and shape("head") == (411, 96)
    assert len(plan.positions) == 2, "two sets of rotary constants, two parts"


def test_the_thin_products_inner_size_comes_from_the_tensors():
    cfg = tz.make_config("mix")
    for layer in cfg.layers:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("rank")
    seen = cfg.with_shapes({"l1.mix.right.a1": (40, 96), "l3.mix.right.a1": (8, 96)})
    from garlic_inference_b200.engine.model import wanted_tensors
    names = wanted_tensors(seen.plan())
    assert tuple(names["l1.mix.right.a2"].shape) == (120, 40) and tuple(names["l3.mix.right.g1"].shape) == (8, 96)


def test_refusals_and_warnings():
    from garlic_inference_b200.config import ConfigError, ZogulornConfig
    bad = tz.config_dict("ones")
    bad["layers"][0] = dict(bad["layers"][0], type="convolution")
    with pytest.raises(ConfigError, match="convolution"):
        ZogulornConfig.from_dict(bad)
    bad = tz.config_dict("mix")
    bad["layers"][2]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError, match="kv_from"):
        ZogulornConfig.from_dict(bad)
    bad = tz.config_dict("mix")
    bad["layers"][2]["mixer"]["kv_heads"] = 4
    with pytest.raises(ConfigError, match="differ"):
        ZogulornConfig.from_dict(bad)
    bad = tz.config_dict("moe")
    bad["layers"][0]["mlp"]["router"]["top"] = 6
    with pytest.raises(ConfigError, match="experts"):
        ZogulornConfig.from_dict(bad)
    bad = tz.config_dict("dense")
    bad["layers"][0]["mlp"] = {"kind": "sparse", "ff": 8}
    with pytest.raises(ConfigError, match="sparse"):
        ZogulornConfig.from_dict(bad)
    odd = tz.config_dict("dense")
    odd["layers"][0]["mixer"]["window"] = 7
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        ZogulornConfig.from_dict(odd)
    assert any("window" in str(w.message) for w in seen)


def test_cache_entries_hold_pages_and_state_and_lend_their_pages():
    from garlic_inference_b200.cache import EntryRequirement, KVRequirement, PagedCache, StateRequirement
    kv = KVRequirement(4, 16, None, 2, value_heads=2, value_dim=24)
    reqs = [EntryRequirement(kv, StateRequirement((12,))), StateRequirement((8,)), EntryRequirement(None, StateRequirement((5,)))]
    c = PagedCache(reqs, max_tokens=128, max_positions=1024, dtype=torch.float32, device="cpu", page_size=16)
    own, lent = c.view(0), c.view(2, kv_entry=0)
    assert tuple(own.kv.k_pool.shape[1:]) == (4, 16, 16) and tuple(own.kv.v_pool.shape[1:]) == (2, 16, 24)
    assert own.state.shape[1:] == (12,) and lent.state.shape[1:] == (5,) and lent.kv.k_pool.data_ptr() == own.kv.k_pool.data_ptr()
    assert c.view(1).kv is None and c.view(2).kv is None
    assert c.bytes_per_token() == 4 * (4 * 16 + 2 * 24)


def test_random_folder_loads_and_fits(tmp_path):
    from garlic_inference_b200.engine.model import wanted_tensors
    from garlic_inference_b200.weights import Checkpoint
    d = tz.write_model("ones", tmp_path / "ones")
    Checkpoint(d).check(wanted_tensors(tz.make_config("ones").plan()))
    cfg, w = plain.read_model_dir(d)
    assert cfg == tz.config_dict("ones") and w["l0.mix.right.q.conv"].shape == (16, 1) and w["l0.norm1.alpha"].shape == ()
    logits = plain.forward(cfg, w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 257) and torch.isfinite(logits).all()


# ---- the plain functions against closed forms ----------------------------------------------------
def test_plain_norm_activations_and_filter():
    x = torch.tensor([[0.5, -2.0, 0.0]])
    got = plain.dyt(x, torch.tensor([2.0, 1.0, 3.0]), torch.tensor([0.1, 0.2, 0.3]), torch.tensor(0.7))
    want = [math.tanh(0.35) * 2 + 0.1, math.tanh(-1.4) + 0.2, 0.3]
    assert torch.allclose(got, torch.tensor([want]), atol=1e-6)
    z = torch.tensor([1.0, -1.0, 0.0])
    g = lambda v: 0.5 * v * (1 + math.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))
    assert torch.allclose(plain.gelu_tanh(z), torch.tensor([g(1.0), g(-1.0), 0.0]), atol=1e-6)
    x = torch.arange(1.0, 6.0)[:, None]                      # one channel: 1 2 3 4 5
    y = plain.causal_conv(x, torch.tensor([[100.0, 10.0, 1.0]]))
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0], "the last tap is the current token's"


def test_plain_rotation_and_chunks():
    x = torch.zeros(3, 1, 6)
    x[:, 0, 0] = 1.0
    x[:, 0, 2] = 1.0
    x[:, 0, 5] = 7.0
    y = plain.rotate_pairs(x, 4, 100.0)
    for p in range(3):
        assert torch.allclose(y[p, 0, :2], torch.tensor([math.cos(p), math.sin(p)]), atol=1e-6)
        assert torch.allclose(y[p, 0, 2:4], torch.tensor([math.cos(p * 0.1), math.sin(p * 0.1)]), atol=1e-6)
        assert y[p, 0, 4] == 0.0 and y[p, 0, 5] == 7.0, "dimensions beyond the rotated ones pass"
    seen = plain.chunk_mask(7, 3)
    assert seen[4].tolist() == [False, False, False, True, True, False, False]
    assert seen[3].tolist() == [False, False, False, True, False, False, False] and seen[2, :3].all()
    q = torch.zeros(5, 2, 4)
    k = torch.randn(5, 1, 4)
    v = torch.arange(5.0)[:, None, None].expand(5, 1, 3).clone()
    o = plain.attend(q, k, v, 1.0, plain.chunk_mask(5, 2))     # equal scores: the mean of the visible values
    assert torch.allclose(o[:, 0, 0], torch.tensor([0.0, 0.5, 2.0, 2.5, 4.0])) and torch.equal(o[:, 0], o[:, 1])


def test_plain_delta_rule_and_router():
    # one head, two keys; orthonormal keys write their values, a repeated key with beta 1 overwrites, decay scales rows
    e0, e1 = torch.tensor([1.0, 0.0]), torch.tensor([0.0, 1.0])
    k = torch.stack([e0, e1, e0])[:, None, :]
    v = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])[:, None, :]
    beta = torch.ones(3, 1)
    g = torch.ones(3, 1, 2)
    g[2, 0] = torch.tensor([1.0, 0.5])
    q = torch.stack([e0, e0 + e1, e0 + e1])[:, None, :]
    o = plain.delta_rule(q, k, v, beta, g)[:, 0]
    assert torch.allclose(o, torch.tensor([[1.0, 2.0], [4.0, 6.0], [5.0 + 1.5, 6.0 + 2.0]]))
    idx, w = plain.route(torch.tensor([[0.0, 3.0, 1.0, 3.0 - math.log(3.0)]]), 2)
    assert idx.tolist() == [[1, 3]] and torch.allclose(w, torch.tensor([[0.75, 0.25]]))


def test_what_the_comparisons_rest_on_shows_in_the_plain_model(tmp_path):
    """Dropping the state of the recurrence and the filters, moving a chunk's edge by one, or leaving out the
    second map changes the plain logits by far more than any tolerance used against it."""
    d = tz.write_model("mix", tmp_path / "mix")
    cfg, w = plain.read_model_dir(d)
    toks = torch.randint(0, 411, (80,), generator=torch.Generator().manual_seed(1)).tolist()
    want = plain.forward(cfg, w, toks)
    scale = float(want.abs().max())
    cut = plain.forward(cfg, w, toks[40:])
    assert float((cut - want[40:]).abs().max()) / scale > 1e-2
    for layer, path in ((0, ("mask", "size")), (1, ("left", "mask", "size"))):
        moved = json.loads(json.dumps(cfg))
        m = moved["layers"][layer]["mixer"]
        for key in path[:-1]:
            m = m[key]
        m[path[-1]] += 1
        assert float((plain.forward(moved, w, toks) - want).abs().max()) / scale > 1e-2
    one_map = dict(w, **{"l0.mix.lq1": torch.full_like(w["l0.mix.lq1"], -30.0), "l0.mix.lk1": torch.ones_like(w["l0.mix.lk1"])})
    assert float((plain.forward(cfg, one_map, toks) - want).abs().max()) / scale > 1e-3

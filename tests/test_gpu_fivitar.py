"""Fivitar through the engine against the plain implementation: each mixer alone, prompts against token-by-token
decoding, portions, batches, slots and pages used again, far keys and page borders, long decoding, generation."""
import json

import numpy as np
import pytest
import torch

import plain_fivitar as plain
import tiny
import tiny_fivitar as tf

pytestmark = pytest.mark.gpu

_DIRS, _MODELS = {}, {}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    def get(name):
        if name not in _DIRS:
            _DIRS[name] = tf.write_model(name, tmp_path_factory.mktemp(f"fivitar_{name}"))
        return _DIRS[name]
    return get


@pytest.fixture(scope="module")
def model(folder):
    def get(name, dtype, max_tokens=4096, page_size=16, **kw):
        key = (name, dtype, max_tokens, page_size, tuple(sorted(kw.items())))
        if key not in _MODELS:
            from garlic_inference_b200 import AutoModel
            _MODELS[key] = AutoModel.from_pretrained(folder(name), device=0, dtype=dtype, max_tokens=max_tokens,
                                                     page_size=page_size, **kw)
        return _MODELS[key]
    return get


def _requests(name, lengths, seed):
    return tiny.random_requests(tf.TINY[name]["vocab"], lengths, seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["lightning", "latent", "delta", "mix", "ones"])
def test_prompts_decoding_portions_and_batches_agree_with_the_plain_model(name, dtype, model, folder):
    """Every way of cutting the same requests gives the plain logits: whole prompts; all but 40 tokens, then one
    at a time; portions of 2, 7, 33 and 3 tokens; the same portions with all requests in one batch; unequal
    requests that start together and decode together.  The cache has room for one batch only, so slots, state
    rows and pages are given back and used again by later requests."""
    m = model(name, dtype, max_tokens=512, page_size=16, max_slots=4)
    reqs = _requests(name, [70, 1, 37, 150], seed=5)
    want, own = tf.plain_pair(folder(name), reqs)
    for what, steps in (("whole", tiny.trace_whole(reqs)),
                        ("tail", tiny.trace_tail_by_one(reqs, tail=40)),
                        ("portions", tf.trace_portions(reqs, [2, 7, 33, 3])),
                        ("portions together", tf.trace_portions(reqs, [5, 2, 64], together=True)),
                        ("batched", tiny.trace_batched(reqs, [["r3", "r1"], ["r0", "r2", "r1"]], prompt_frac=0.6))):
        got = tiny.run_trace_in_process(m, steps)
        tiny.assert_covers(got, reqs)
        tf.judge(got, want, own, dtype, f"{name} {dtype} {what}")
    assert m.engine.cache.slots.n_free == 4, "every slot came back"


def test_float32_logits_do_not_depend_on_the_cut_or_the_batch(model):
    """The same position gives the same bits whole, in portions, decoded, alone or in a batch (float32 engine:
    its products, scans and attention walk every row in an order that depends on the row alone)."""
    m = model("mix", "float32", max_tokens=1024, page_size=16)
    reqs = _requests("mix", [90, 33], seed=6)
    base = tiny.run_trace_in_process(m, tiny.trace_whole(reqs))
    for steps in (tf.trace_portions(reqs, [2, 31, 8]), tiny.trace_tail_by_one(reqs, tail=20),
                  tf.trace_portions(reqs, [16, 3], together=True)):
        got = tiny.run_trace_in_process(m, steps)
        for rid in reqs:
            for p in range(len(reqs[rid])):
                assert np.array_equal(got[rid][p], base[rid][p]), f"request {rid} position {p} differs in its bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_at_page_borders_and_the_first_tokens(dtype, folder, tmp_path):
    """A token whose embedding is six times the others' stands at positions 0, 15, 16, 17 and 63 (cache pages of
    16) of a prompt of 260 and again as the query at its end and in decoding: the rotated score of those pairs
    stands out by a factor of 36 and turns with the distance.  The plain model says how much a lost or misplaced
    key would show (the same prompt without the far tokens), and the engine has to be far closer than that."""
    from garlic_inference_b200 import AutoModel
    from garlic_inference_b200.weights.safetensors_io import SafetensorsFile, write_safetensors_lazy
    src = folder("latent")
    f = SafetensorsFile(src / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    needle = 7
    tensors["embed"][needle] *= 6.0
    dst = tmp_path / "needle"
    dst.mkdir()
    (dst / "config.json").write_text((src / "config.json").read_text())
    write_safetensors_lazy(dst / "model.safetensors", {n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()},
                           lambda n: tensors[n])
    rng = np.random.default_rng(3)
    toks = [int(t) for t in rng.integers(8, 300, size=260)]
    plainer = list(toks)
    for p in (0, 15, 16, 17, 63):
        toks[p] = needle
    for p in (200, 255, 259):
        toks[p] = plainer[p] = needle
    cfg, w = plain.read_model_dir(dst)
    want = plain.forward(cfg, w, toks, torch.float64).numpy()
    own = plain.forward(cfg, w, toks, torch.float32).double().numpy()
    without = plain.forward(cfg, w, plainer, torch.float64).numpy()
    shows = min(np.sqrt(((want[p] - without[p]) ** 2).mean()) for p in (200, 255, 259)) / np.sqrt((want ** 2).mean())
    assert shows > 5 * tf.BF16_MEDIAN, f"the far keys move the logits by only {shows:.2e}"
    m = AutoModel.from_pretrained(dst, device=0, dtype=dtype, max_tokens=512, page_size=16)
    reqs = {"n": toks}
    for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=62), tf.trace_portions(reqs, [17, 2])):
        got = tiny.run_trace_in_process(m, steps)
        tf.judge(got, {"n": want}, {"n": own}, dtype, f"far key {dtype}")
        if dtype == "bfloat16":                   # the rows that look far back, one by one
            errs = tf.row_errors(got, {"n": want})
            assert max(errs[("n", p)][1] for p in (200, 255, 259)) <= shows / 5


def test_the_sink_and_the_state_show_in_the_plain_model(folder):
    """What the comparisons above rest on: dropping the sink, the filters' state or the decayed state changes the
    plain logits by far more than the tolerance, so an engine that lost one of them would not pass."""
    cfg, w = plain.read_model_dir(folder("mix"))
    toks = _requests("mix", [60], seed=8)["r0"]
    want = plain.forward(cfg, w, toks)
    scale = float(want.abs().max())
    no_sink = dict(w, **{"l0.mix.sink": torch.full_like(w["l0.mix.sink"], -1e9)})
    assert float((plain.forward(cfg, no_sink, toks) - want).abs().max()) / scale > 1e-2
    cut = plain.forward(cfg, w, toks[30:])                 # the last 30 tokens without what came before
    assert float((cut - want[30:]).abs().max()) / scale > 1e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "delta", "lightning"])
def test_long_decoding(name, dtype, model, folder):
    """300 tokens decoded one at a time after a prompt of 5, two requests together, through the recorded decode
    step: state carried 300 times, cache pages taken one after the other."""
    m = model(name, dtype, max_tokens=1024, page_size=16)
    reqs = _requests(name, [305, 280], seed=9)
    want, own = tf.plain_pair(folder(name), reqs)
    steps = tiny.trace_batched(reqs, [["r0", "r1"]], prompt_frac=5 / 305)
    got = tiny.run_trace_in_process(m, steps)
    tiny.assert_covers(got, reqs)
    tf.judge(got, want, own, dtype, f"long decoding {name} {dtype}")
    assert m.engine.graphs is not None and 2 in m.engine.graphs._graphs, "decode steps ran from a recorded graph"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype, model, folder):
    m = model("mix", dtype, max_tokens=512, page_size=16, max_slots=3)
    prompts = list(_requests("mix", [9, 1, 30, 17, 5], seed=10).values())
    got = m.generate(prompts, max_new_tokens=10)
    assert m.last_stats.batches == 2
    cfg, w = plain.read_model_dir(folder("mix"))
    for prompt, new in zip(prompts, got):
        ids = list(prompt)
        assert len(new) == 10
        for k, tok in enumerate(new):
            logits = plain.forward(cfg, w, ids)[-1]
            best = int(logits.argmax())
            if tok != best:
                gap = float(logits[best] - logits[tok]) / float(logits.abs().max())
                assert dtype == "bfloat16" and gap <= 0.1, \
                    f"prompt of {len(prompt)}, new token {k}: engine chose {tok}, plain {best} (gap {gap:.2e})"
                break
            ids.append(tok)


def test_trace_program_and_command_line_serve_the_design(folder, tmp_path):
    import subprocess
    import sys
    reqs = _requests("ones", [20, 3], seed=12)
    want, own = tf.plain_pair(folder("ones"), reqs)
    steps = tiny.trace_batched(reqs, [["r0", "r1"]])
    got = tiny.run_trace_program(folder("ones"), "float32", steps, tmp_path / "out", 256, tf.TINY["ones"]["vocab"])
    tf.judge(got, want, own, "float32", "trace program")
    r = subprocess.run([sys.executable, str(tiny.REPO / "bin" / "runner"), str(folder("ones")), "--prompt-ids", "5,6,7",
                        "--max-new-tokens", "4", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [int(t) for t in r.stdout.splitlines()[0].split()]
    cfg, w = plain.read_model_dir(folder("ones"))
    seq = [5, 6, 7]
    for tok in ids:
        assert tok == int(plain.forward(cfg, w, seq)[-1].argmax())
        seq.append(tok)


# ---- kernels alone -----------------------------------------------------------------------------
def test_xielu_and_gate_norm_add_kernels():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(0)
    z = torch.randn(37, 100, device="cuda") * 3
    pq = torch.tensor([0.3, -0.8], device="cuda")
    torch.testing.assert_close(kernels.xielu(z, pq).cpu(), plain.xielu(z.cpu(), 0.3, -0.8), rtol=2e-6, atol=2e-6)
    wide = torch.randn(37, 140, device="cuda")
    torch.testing.assert_close(kernels.xielu(wide[:, 20:120], pq).cpu(), plain.xielu(wide[:, 20:120].cpu(), 0.3, -0.8),
                               rtol=2e-6, atol=2e-6)
    y, g, b, w = (torch.randn(s, device="cuda") for s in ((37, 100), (37, 100), (100,), (100,)))
    res = torch.randn(37, 100, device="cuda")
    want = res.cpu() + plain.rms_norm(y.cpu() * plain.sigmoid(g.cpu() + b.cpu()), w.cpu(), 1e-5)
    assert kernels.gate_norm_add(y, g, b, w, 1e-5, res, False) is None
    torch.testing.assert_close(res.cpu(), want, rtol=1e-5, atol=1e-5)
    yb, gb = y.bfloat16(), g.bfloat16()
    res2 = torch.zeros(37, 100, device="cuda")
    copy = kernels.gate_norm_add(yb, gb, b, w, 1e-5, res2, True)
    want = plain.rms_norm(yb.float().cpu() * plain.sigmoid(gb.float().cpu() + b.cpu()), w.cpu(), 1e-5)
    torch.testing.assert_close(res2.cpu(), want, rtol=1e-5, atol=1e-5)
    assert torch.equal(copy, res2.bfloat16())


def test_filter_kernel_carries_its_state_across_cuts():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(1)
    C, K, T = 70, 4, 23
    x = torch.randn(T, C + 9, device="cuda")[:, 4:4 + C]            # rows that lie apart
    taps = torch.randn(C, K, device="cuda")
    want = plain.silu(plain.causal_conv(x.cpu(), taps.cpu()))
    for cuts in ([T], [1] * T, [2, 1, 5, 3, 12], [3, 20]):
        state = torch.zeros(3, (K - 1) * C + 2, device="cuda")
        out, at = [], 0
        for n in cuts:
            # the sequence lives in slot 1; a one-token neighbour in slot 2 and a padding row share each step
            rows = torch.cat([x[at:at + n], x[:1], x[:1]])
            slots = torch.tensor([1] * n + [2, -1], dtype=torch.int32, device="cuda")
            out.append(kernels.causal_conv_silu(rows, taps, state, slots)[:n])
            kernels.conv_state_update(rows, K, state, slots)
            at += n
        torch.testing.assert_close(torch.cat(out).cpu(), want, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(state[1, :(K - 1) * C].view(K - 1, C).cpu(), x[T - (K - 1):].cpu())
        assert float(state[0].abs().max()) == 0.0


def test_attention_sinks_and_narrow_values():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(2)
    H, d, dv, page, T = 3, 24, 16, 8, 21
    pool = torch.randn(4, 1, page, d, device="cuda")
    table = torch.tensor([[2, 0, 3, -1]], dtype=torch.int32, device="cuda")
    q = torch.randn(T, H, d, device="cuda")
    sinks = torch.tensor([0.5, -2.0, 3.0], device="cuda")
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    slot = torch.zeros(T, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = kernels.attention_generic(q, pool, pool, table, pos, slot, 0.4, 0, status, sinks=sinks, value_dim=dv)
    rows = torch.cat([pool[2, 0], pool[0, 0], pool[3, 0]]).cpu()[:T]
    s = torch.einsum("thd,jd->htj", q.cpu(), rows) * 0.4
    s = s.masked_fill(torch.arange(T)[None, None, :] > torch.arange(T)[None, :, None], float("-inf"))
    e = torch.exp(s)
    p = e / (e.sum(-1, keepdim=True) + torch.exp(sinks.cpu())[:, None, None])
    want = torch.einsum("htj,jv->thv", p, rows[:, :dv]).reshape(T, H * dv)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-5)
    assert int(status.item()) == 0


def test_causal_sink_softmax_kernel():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(3)
    H, T, first, keys = 3, 5, 9, 16
    wide = torch.randn(T * H, keys + 5, device="cuda") * 4
    scores = wide[:, :keys]
    sinks = torch.tensor([0.2, -3.0, 2.5], device="cuda")
    for sk in (sinks, None):
        got = kernels.causal_sink_softmax(scores, H, first, 0.7, sk, torch.float32).cpu().view(T, H, keys)
        s = scores.cpu().view(T, H, keys) * 0.7
        seen = torch.arange(keys)[None, None, :] <= (first + torch.arange(T))[:, None, None]
        e = torch.where(seen, torch.exp(s), torch.zeros(()))
        extra = torch.exp(sinks.cpu())[None, :, None] if sk is not None else 0.0
        torch.testing.assert_close(got, e / (e.sum(-1, keepdim=True) + extra), rtol=1e-5, atol=1e-7)
    got = kernels.causal_sink_softmax(scores, H, first, 0.7, sinks, torch.bfloat16)
    assert got.dtype == torch.bfloat16 and float(got.view(T, H, keys)[0, :, first + 1:].abs().max()) == 0.0

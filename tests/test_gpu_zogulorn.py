"""Zogulorn through the engine against the plain implementation: each mechanism alone, prompts against
token-by-token decoding, portions, batches, slots and pages used again, keys at chunk edges and page borders,
long decoding, generation, the two programs, and the kernels alone."""
import json

import numpy as np
import pytest
import torch

import plain_zogulorn as plain
import tiny
import tiny_zogulorn as tz

pytestmark = pytest.mark.gpu

_DIRS, _MODELS = {}, {}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    def get(name):
        if name not in _DIRS:
            _DIRS[name] = tz.write_model(name, tmp_path_factory.mktemp(f"zogulorn_{name}"))
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
    return tiny.random_requests(tz.TINY[name]["vocab"], lengths, seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["left", "right", "diff", "dense", "moe", "mix", "ones"])
def test_prompts_decoding_portions_and_batches_agree_with_the_plain_model(name, dtype, model, folder):
    """Every way of cutting the same requests gives the plain logits: whole prompts; all but 40 tokens, then one
    at a time; portions of 2, 7, 33 and 3 tokens; portions with all requests in one batch; unequal requests that
    start together and decode together.  The cache has room for one batch only, so slots, state rows and pages
    are given back and used again by later requests."""
    m = model(name, dtype, max_tokens=512, page_size=16, max_slots=4)
    reqs = _requests(name, [70, 1, 37, 150], seed=5)
    want, own = tz.plain_pair(folder(name), reqs)
    for what, steps in (("whole", tiny.trace_whole(reqs)),
                        ("tail", tiny.trace_tail_by_one(reqs, tail=40)),
                        ("portions", tz.trace_portions(reqs, [2, 7, 33, 3])),
                        ("portions together", tz.trace_portions(reqs, [5, 2, 64], together=True)),
                        ("batched", tiny.trace_batched(reqs, [["r3", "r1"], ["r0", "r2", "r1"]], prompt_frac=0.6))):
        got = tiny.run_trace_in_process(m, steps)
        tiny.assert_covers(got, reqs)
        tz.judge(got, want, own, dtype, f"{name} {dtype} {what}")
    assert m.engine.cache.slots.n_free == 4, "every slot came back"


def test_float32_logits_do_not_depend_on_the_cut_or_the_batch(model):
    """Without routed experts (whose few-row and many-row paths sum in different orders) the same position gives
    the same bits whole, in portions, decoded, alone or in a batch."""
    for name in ("left", "right", "diff", "dense"):
        m = model(name, "float32", max_tokens=1024, page_size=16)
        reqs = _requests(name, [90, 33], seed=6)
        base = tiny.run_trace_in_process(m, tiny.trace_whole(reqs))
        for steps in (tz.trace_portions(reqs, [2, 31, 8]), tiny.trace_tail_by_one(reqs, tail=20),
                      tz.trace_portions(reqs, [16, 3], together=True)):
            got = tiny.run_trace_in_process(m, steps)
            for rid in reqs:
                for p in range(len(reqs[rid])):
                    assert np.array_equal(got[rid][p], base[rid][p]), f"{name}: request {rid} position {p} differs in its bits"


def _with_needle(src, dst, needle, factor):
    from garlic_inference_b200.weights.safetensors_io import SafetensorsFile, write_safetensors_lazy
    f = SafetensorsFile(src / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["embed"][needle] *= factor
    dst.mkdir()
    (dst / "config.json").write_text((src / "config.json").read_text())
    write_safetensors_lazy(dst / "model.safetensors", {n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()},
                           lambda n: tensors[n])
    return dst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,chunk", [("left", 48), ("diff", 20)])
def test_keys_at_chunk_edges_and_page_borders(name, chunk, dtype, folder, tmp_path):
    """A token whose embedding is five times the others' stands at the first position of a chunk, at the last of
    the chunk before, at cache-page borders inside a chunk (pages of 16) and as a query at chunk ends and in
    decoding.  With a needle just inside its chunk a query's logits move, with one just outside they must not:
    the plain model says how much a key that is lost, or seen from the wrong side of an edge, would show, and
    the engine has to be far closer than that.  Both prompts (with the needles, and with ordinary tokens in
    their place) are compared, whole, with a decoded tail that crosses two chunk edges, and in portions."""
    from garlic_inference_b200 import AutoModel
    needle = 7
    dst = _with_needle(folder(name), tmp_path / "needle", needle, 5.0)
    rng = np.random.default_rng(3)
    n = 5 * chunk + 9
    plainer = [int(t) for t in rng.integers(8, tz.TINY[name]["vocab"], size=n)]
    toks, ends = list(plainer), []
    for c in (1, 3):                           # a page border inside a chunk (pages of 16): needles around it
        start = c * chunk
        border = -(-(start + 1) // 16) * 16
        assert border + 1 < start + chunk - 1
        for p in (border - 1, border, border + 1):
            toks[p] = needle
        ends.append(border + 3)
    for e in (2 * chunk, 4 * chunk):
        toks[e] = needle                       # just inside: the first key of its chunk
        toks[e - 1] = needle                   # just outside: the last key of the chunk before
        ends += [e + 1, e + chunk - 1]         # the next query, and the chunk's last, far from its first key
    for p in ends:
        toks[p] = plainer[p] = needle
    cfg, w = plain.read_model_dir(dst)
    want = plain.forward(cfg, w, toks, torch.float64).numpy()
    own = plain.forward(cfg, w, toks, torch.float32).double().numpy()
    without = plain.forward(cfg, w, plainer, torch.float64).numpy()
    rms = np.sqrt((want ** 2).mean())
    shows = {p: np.sqrt(((want[p] - without[p]) ** 2).mean()) / rms for p in ends}
    clear = [p for p in ends if shows[p] > 3 * tz.BF16_MEDIAN]
    assert len(clear) >= 4, f"the needles move the logits too little: {shows}"
    m = AutoModel.from_pretrained(dst, device=0, dtype=dtype, max_tokens=1024, page_size=16)
    for what, prompt, ref, ref32 in (("needles", toks, want, own),
                                     ("plain", plainer, without, plain.forward(cfg, w, plainer, torch.float32).double().numpy())):
        reqs = {"n": prompt}
        for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=2 * chunk + 12),
                      tz.trace_portions(reqs, [17, 2, chunk])):
            got = tiny.run_trace_in_process(m, steps)
            tz.judge(got, {"n": ref}, {"n": ref32}, dtype, f"chunk edges {name} {dtype} {what}")
            if dtype == "bfloat16":
                errs = tz.row_errors(got, {"n": ref})
                for p in clear:
                    assert errs[("n", p)][1] <= shows[p] / 3, f"position {p}"


def test_heads_of_128_on_pages_of_64_run_the_tcgen05_prompt_kernel(model, folder):
    """bfloat16, heads of 128, pages of 64 tokens: prompts and portions go through the tcgen05 kernel with the chunk
    mask in it (chunks of 70: edges inside its tiles of 64 keys and 128 queries), decode steps through the split-KV
    kernel; all against the plain model."""
    from garlic_inference_b200.ops import counters
    m = model("wide", "bfloat16", max_tokens=2048, page_size=64, max_slots=4)
    reqs = _requests("wide", [300, 1, 141, 70], seed=15)
    want, own = tz.plain_pair(folder("wide"), reqs)
    for what, steps in (("whole", tiny.trace_whole(reqs)), ("tail", tiny.trace_tail_by_one(reqs, tail=80)),
                        ("portions", tz.trace_portions(reqs, [129, 3, 64], together=True))):
        got = tiny.run_trace_in_process(m, steps)
        tiny.assert_covers(got, reqs)
        tz.judge(got, want, own, "bfloat16", f"wide {what}")
    mixer = m.model.blocks[0].mixer.left
    assert mixer._run_rows(m.engine.cache.view(0).kv) == 128
    from garlic_inference_b200.ops import kernels
    kernels.check_bounded_waits(torch.device("cuda", 0))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "right", "moe"])
def test_long_decoding(name, dtype, model, folder):
    """300 tokens decoded one at a time after a prompt of 5, two requests together, through the recorded decode
    step: recurrent and filter state carried 300 times, chunks begun and left, cache pages taken one by one."""
    m = model(name, dtype, max_tokens=1024, page_size=16)
    reqs = _requests(name, [305, 280], seed=9)
    want, own = tz.plain_pair(folder(name), reqs)
    steps = tiny.trace_batched(reqs, [["r0", "r1"]], prompt_frac=5 / 305)
    got = tiny.run_trace_in_process(m, steps)
    tiny.assert_covers(got, reqs)
    tz.judge(got, want, own, dtype, f"long decoding {name} {dtype}")
    assert m.engine.graphs is not None and 2 in m.engine.graphs._graphs, "decode steps ran from a recorded graph"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["moe", "mix"])
def test_a_dozen_requests_decode_together(name, dtype, model, folder):
    """Twelve unequal requests start together and decode together through a recorded step of 16 rows (four of them
    padding): the routed feed-forward then runs expert by expert inside the recording, the attention kernels see
    padding rows, and requests leave one after the other."""
    m = model(name, dtype, max_tokens=2048, page_size=16, max_slots=12)
    reqs = _requests(name, [31 + 3 * i for i in range(12)], seed=21)
    want, own = tz.plain_pair(folder(name), reqs)
    got = tiny.run_trace_in_process(m, tiny.trace_batched(reqs, [list(reqs)], prompt_frac=0.5))
    tiny.assert_covers(got, reqs)
    tz.judge(got, want, own, dtype, f"twelve together {name} {dtype}")
    assert m.engine.graphs is not None and 16 in m.engine.graphs._graphs


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
    want, own = tz.plain_pair(folder("ones"), reqs)
    steps = tiny.trace_batched(reqs, [["r0", "r1"]])
    got = tiny.run_trace_program(folder("ones"), "float32", steps, tmp_path / "out", 256, tz.TINY["ones"]["vocab"])
    tz.judge(got, want, own, "float32", "trace program")
    r = subprocess.run([sys.executable, str(tiny.REPO / "bin" / "runner"), str(folder("ones")), "--prompt-ids", "5,6,7",
                        "--max-new-tokens", "4", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [int(t) for t in r.stdout.splitlines()[0].split()]
    cfg, w = plain.read_model_dir(folder("ones"))
    seq = [5, 6, 7]
    for tok in ids:
        assert tok == int(plain.forward(cfg, w, seq)[-1].argmax())
        seq.append(tok)


def test_the_stored_inner_size_of_the_thin_products_wins(folder, tmp_path):
    """A folder whose config.json does not say how thin the delta rule's two-matrix projections are: the tensors do."""
    from garlic_inference_b200 import AutoModel
    src = folder("right")
    dst = tmp_path / "norank"
    dst.mkdir()
    cfg = json.loads((src / "config.json").read_text())
    assert cfg["layers"][0]["mixer"]["right"].pop("rank") == 16
    (dst / "config.json").write_text(json.dumps(cfg))
    (dst / "model.safetensors").write_bytes((src / "model.safetensors").read_bytes())
    m = AutoModel.from_pretrained(dst, device=0, dtype="float32", max_tokens=256, page_size=16)
    reqs = _requests("right", [30], seed=2)
    want, own = tz.plain_pair(dst, reqs)
    tz.judge(tiny.run_trace_in_process(m, tiny.trace_whole(reqs)), want, own, "float32", "rank from the tensors")


# ---- kernels alone -----------------------------------------------------------------------------
def test_dyt_glu_and_sums():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(0)
    res, delta, ls, w, b = (torch.randn(s, device="cuda") for s in ((37, 100), (37, 100), (100,), (100,), (100,)))
    alpha = torch.tensor([0.6], device="cuda")
    keep = res.clone()
    out = kernels.add_dyt(delta, ls, res, w, b, alpha, torch.float32)
    s = keep.cpu() + delta.cpu() * ls.cpu()
    torch.testing.assert_close(res.cpu(), s, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out.cpu(), plain.dyt(s, w.cpu(), b.cpu(), 0.6), rtol=1e-5, atol=1e-5)
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device="cuda")
    before = res.clone()
    picked = kernels.add_dyt(delta, None, res, w, b, alpha, torch.float32, rows=rows)
    assert torch.equal(res, before), "gathered rows write nothing back"
    torch.testing.assert_close(picked.cpu(), plain.dyt((before + delta).cpu()[[5, 0, 36]], w.cpu(), b.cpu(), 0.6), rtol=1e-5, atol=1e-5)
    few = kernels.add_dyt(None, None, res[:3].contiguous(), w, b, alpha, torch.bfloat16)
    torch.testing.assert_close(few.float().cpu(), plain.dyt(res[:3].cpu(), w.cpu(), b.cpu(), 0.6), rtol=1e-2, atol=1e-2)
    r2 = keep.clone()
    kernels.residual_add_scaled(delta, ls, r2)
    torch.testing.assert_close(r2.cpu(), s, rtol=1e-6, atol=1e-6)
    gu = torch.randn(9, 140, device="cuda") * 2
    torch.testing.assert_close(kernels.glu(gu, "gelu_tanh").cpu(), plain.gelu_tanh(gu[:, :70].cpu()) * gu[:, 70:].cpu(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(kernels.glu(gu, "silu").cpu(), plain.silu(gu[:, :70].cpu()) * gu[:, 70:].cpu(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(kernels.relu_squared(gu).cpu(), torch.relu(gu.cpu()) ** 2)
    a, c = torch.randn(7, 33, device="cuda"), torch.randn(7, 33, device="cuda")
    torch.testing.assert_close(kernels.scaled_sum(a, 0.6, c, 1.1).cpu(), 0.6 * a.cpu() + 1.1 * c.cpu(), rtol=1e-6, atol=1e-6)
    table = torch.randn(11, 20, device="cuda").bfloat16()
    ids = torch.tensor([3, 10, 0], dtype=torch.int32, device="cuda")
    torch.testing.assert_close(kernels.embedding(ids, table, scale=3.0).cpu(), table.float().cpu()[[3, 10, 0]] * 3.0)


def test_router_and_expert_kernels():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(1)
    n, E, top, hid, ff = 45, 7, 3, 40, 24
    z = torch.randn(n, E, device="cuda")
    z[0, 2] = z[0, 5] = 9.0                               # a tie: the lower index first
    idx, wt = kernels.router_topk(z, top)
    ri, rw = plain.route(z.cpu(), top)
    assert idx[0, :2].tolist() == [2, 5]
    assert torch.equal(idx[1:].cpu().long(), ri[1:]) and torch.allclose(wt.cpu(), rw, atol=1e-6)
    x = torch.randn(n, hid, device="cuda")
    up, down = torch.randn(E, ff, hid, device="cuda") * 0.3, torch.randn(E, hid, ff, device="cuda") * 0.3
    w = {"router": torch.zeros(E, hid)}
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = up[e].cpu(), down[e].cpu()
    want = torch.zeros(n, hid)
    for e in range(E):
        y = (torch.relu(x.cpu() @ up[e].cpu().T) ** 2) @ down[e].cpu().T
        want += y * (wt.cpu() * (idx.cpu() == e)).sum(-1, keepdim=True)
    torch.testing.assert_close(kernels.moe_rowwise(x, up, down, idx, wt, "relu_squared").cpu(), want, rtol=1e-4, atol=1e-4)
    for rows_n, experts in ((45, 7), (1500, 3), (700, 70)):       # one block of pairs, several, more experts than a warp
        ids = torch.randint(0, experts, (rows_n, 2), device="cuda", dtype=torch.int32)
        xs = torch.randn(rows_n, 24, device="cuda")
        where, ends, rows = kernels.moe_group(ids, xs, experts)
        flat = ids.reshape(-1).long().cpu()
        order = torch.sort(flat, stable=True).indices
        want_where = torch.empty_like(order)
        want_where[order] = torch.arange(order.numel())
        assert torch.equal(where.reshape(-1).long().cpu(), want_where), "pairs in the order of their experts, stable"
        assert torch.equal(ends.long().cpu(), torch.cumsum(torch.bincount(flat, minlength=experts), 0))
        assert torch.equal(rows.cpu(), xs.cpu()[order // 2])
    buf = torch.randn(n * top, hid, device="cuda")
    where = torch.randperm(n * top, device="cuda").to(torch.int32).view(n, top)
    got = kernels.moe_combine(buf, where, wt)
    torch.testing.assert_close(got.cpu(), (buf.cpu()[where.cpu().long()] * wt.cpu()[..., None]).sum(1), rtol=1e-5, atol=1e-5)


def test_routed_experts_few_rows_and_many_rows_agree(folder):
    """The part's two ways (row by row for a few tokens, expert by expert for many) on the same rows."""
    from garlic_inference_b200.parts import Runtime, StepContext, part_class
    from garlic_inference_b200.weights import Checkpoint
    ck = Checkpoint(folder("moe"))
    params = dict(hidden_size=48, expert_size=40, n_experts=5, top=2, activation="relu_squared")
    names = {n: "l0.mlp." + n for n in ["router"] + [f"e{e}.{s}" for e in range(5) for s in ("up", "down")]}

    class Load:
        def dtype(self, *a):
            return torch.float32

        def __call__(self, n, out=None):
            t = ck.tensor(names[n]).float().cuda()
            return t if out is None else out.copy_(t)

    part = part_class("routed_experts")(params, Load(), Runtime(torch.float32, torch.device("cuda")))
    x = torch.randn(70, 48, device="cuda")
    z = torch.zeros(70, dtype=torch.int32, device="cuda")
    many = part.step(x, StepContext(70, z, z, z))
    few = torch.cat([part.step(x[i:i + 7].contiguous(), StepContext(7, z, z, z)) for i in range(0, 70, 7)])
    torch.testing.assert_close(many, few, rtol=1e-5, atol=1e-6)
    w = {n[len("l0.mlp."):]: ck.tensor(n).float() for n in ck.names() if n.startswith("l0.mlp.")}
    torch.testing.assert_close(many.cpu(), plain.moe_ff(x.cpu(), w, {"router": {"experts": 5, "top": 2}}), rtol=1e-4, atol=1e-5)


def test_rotation_append_and_masked_attention_kernels():
    """Keys and values of different shapes in pools of their own, pages out of order, chunks, two maps."""
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(2)
    H, G, d, dv, page, T, chunk, maps = 4, 2, 12, 20, 8, 27, 10, 2
    C = H * maps * d + G * maps * d + G * dv
    src = torch.randn(T, C + 6, device="cuda")[:, 3:3 + C]
    k_pool = torch.zeros(5, G * maps, page, d, device="cuda")
    v_pool = torch.zeros(5, G, page, dv, device="cuda")
    table = torch.tensor([[3, 0, 4, 1]], dtype=torch.int32, device="cuda")
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    slot = torch.zeros(T, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    n_rot, base = 8, 50.0
    freq = torch.tensor([base ** (-2.0 * r / n_rot) for r in range(n_rot // 2)], dtype=torch.float32, device="cuda")
    Cq, Ck = H * maps * d, G * maps * d
    q = kernels.attn_prepare(src, 0, Cq, Cq + Ck, freq, n_rot, False, pos, slot, table, k_pool, v_pool, H * maps, d,
                             torch.float32, status)
    s = src.cpu()
    qr = plain.rotate_pairs(s[:, :Cq].reshape(T, H * maps, d), n_rot, base)
    kr = plain.rotate_pairs(s[:, Cq:Cq + Ck].reshape(T, G * maps, d), n_rot, base)
    torch.testing.assert_close(q.cpu(), qr, rtol=1e-5, atol=1e-5)
    order = [3, 0, 4, 1]
    keys = torch.cat([k_pool[p] for p in order], dim=1).transpose(0, 1).cpu()[:T]      # [T, G maps, d]
    vals = torch.cat([v_pool[p] for p in order], dim=1).transpose(0, 1).cpu()[:T]
    torch.testing.assert_close(keys, kr, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(vals, s[:, Cq + Ck:].reshape(T, G, dv))
    got = kernels.attention_masked(q, k_pool, v_pool, table, pos, slot, 0.3, status, chunk=chunk, maps=maps, out_float32=True)
    seen = plain.chunk_mask(T, chunk)
    qm, km = qr.view(T, H, maps, d), kr.view(T, G, maps, d)
    want = torch.stack([plain.attend(qm[:, :, i], km[:, :, i], vals, 0.3, seen) for i in range(maps)], dim=2)
    torch.testing.assert_close(got.cpu().view(T, H, maps, dv), want, rtol=1e-5, atol=1e-5)
    lam = torch.tensor([0.4], device="cuda")
    gate = torch.randn(T, H, device="cuda")
    fin = kernels.attn_finish(got, H, maps, lam, 1e-5, 0.7, gate, torch.float32)
    o = plain.rms_div(want[:, :, 0] - 0.4 * want[:, :, 1], 1e-5) * 0.7 * plain.sigmoid(gate.cpu())[:, :, None]
    torch.testing.assert_close(fin.cpu(), o.reshape(T, H * dv), rtol=1e-4, atol=1e-5)
    win = kernels.attention_masked(q[:, ::2].contiguous(), k_pool[:, ::2].contiguous(), v_pool, table, pos, slot, 0.3, status, window=5)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    torch.testing.assert_close(win.cpu().view(T, H, dv), plain.attend(qm[:, :, 0], km[:, :, 0], vals, 0.3, (j <= i) & (j > i - 5)),
                               rtol=1e-5, atol=1e-5)
    assert int(status.item()) == 0


@pytest.mark.parametrize("d,dv", [(32, 32), (16, 32), (64, 32), (96, 96)])
def test_tensor_core_attention_with_chunks_two_maps_and_values_of_another_size(d, dv):
    """The tensor-core kernels (bfloat16) with a chunk mask, two maps per head and values of a size of their own:
    the prompt kernel for two sequences of unequal lengths of which one goes on from cached keys, and the decode
    kernel for the last token of each."""
    from garlic_inference_b200.ops import kernels
    from garlic_inference_b200.parts import StepShape
    from garlic_inference_b200.parts.attention import query_runs
    torch.manual_seed(4)
    H, G, page, maps, chunk = 4, 2, 16, 2, 50
    lens, past = [150, 70], [0, 90]
    n_pages = 24
    k_pool = (torch.randn(n_pages, G * maps, page, d, device="cuda") * 0.7).bfloat16()
    v_pool = torch.randn(n_pages, G, page, dv, device="cuda").bfloat16()
    table = torch.full((2, 12), -1, dtype=torch.int32, device="cuda")
    table[0, :10] = torch.arange(10, dtype=torch.int32) * 2 + 1
    table[1, :10] = torch.arange(10, dtype=torch.int32) * 2
    n = sum(lens)
    q = torch.randn(n, H * maps, d, device="cuda").bfloat16()
    runs = torch.from_numpy(query_runs(StepShape([0, 1], [0, 150], lens, past, False), 64)).cuda()
    last = torch.tensor([149, 150 + 69], device="cuda")
    pos1 = torch.tensor([149, 159], dtype=torch.int32, device="cuda")
    slot1 = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    for ch, win in ((chunk, 0), (0, 0), (7, 0), (0, 40)):
        got = kernels.attention_prefill_masked_bf16(q, k_pool, v_pool, table, runs, 0.2, window=win, chunk=ch, maps=maps,
                                                    rows_covered=True).float().cpu().view(n, H, maps, dv)
        one = kernels.attention_decode_masked_bf16(q[last].contiguous(), k_pool, v_pool, table, pos1, slot1, 0.2, window=win,
                                                   chunk=ch, maps=maps, n_splits=3).float().cpu().view(2, H, maps, dv)
        for s, (start, m, p0) in enumerate(zip([0, 150], lens, past)):
            T = p0 + m
            pages = table[s, :-(-T // page)].long()
            keys = k_pool[pages].float().cpu().permute(0, 2, 1, 3).reshape(-1, G, maps, d)[:T]
            vals = v_pool[pages].float().cpu().permute(0, 2, 1, 3).reshape(-1, G, dv)[:T]
            i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
            seen = plain.chunk_mask(T, ch) if ch else ((j <= i) & (j > i - win) if win else j <= i)
            qs = torch.zeros(T, H, maps, d)
            qs[p0:] = q[start:start + m].float().cpu().view(m, H, maps, d)
            for mp in range(maps):
                want = plain.attend(qs[:, :, mp], keys[:, :, mp], vals, 0.2, seen)[p0:]
                torch.testing.assert_close(got[start:start + m, :, mp], want, rtol=2e-2, atol=2e-2)
                torch.testing.assert_close(one[s, :, mp], want[-1], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("chunk", [1, 64, 100, 128, 200, 1000])
def test_tcgen05_prompt_attention_with_chunks(chunk):
    """The tcgen05 prompt kernel (heads of 128, pages of 64) with chunks smaller than, equal to and larger than its
    tiles of 64 keys and 128 queries, for a sequence that starts and one that goes on from cached keys."""
    from garlic_inference_b200.ops import kernels
    from garlic_inference_b200.parts import StepShape
    from garlic_inference_b200.parts.attention import query_runs
    torch.manual_seed(5)
    H, G, d, page = 4, 2, 128, 64
    lens, past = [300, 150], [0, 210]
    k_pool = (torch.randn(16, G, page, d, device="cuda") * 0.5).bfloat16()
    v_pool = torch.randn(16, G, page, d, device="cuda").bfloat16()
    table = torch.full((2, 8), -1, dtype=torch.int32, device="cuda")
    table[0, :5] = torch.tensor([9, 2, 11, 4, 13], dtype=torch.int32)
    table[1, :6] = torch.tensor([0, 7, 1, 8, 3, 15], dtype=torch.int32)
    n = sum(lens)
    q = torch.randn(n, H, d, device="cuda").bfloat16()
    runs = torch.from_numpy(query_runs(StepShape([0, 1], [0, 300], lens, past, False), 128)).cuda()
    got = kernels.attention_prefill_tcgen05(q, k_pool, v_pool, table, runs, 0.1, 0, rows_covered=True, chunk=chunk)
    kernels.check_bounded_waits(torch.device("cuda", 0))
    got = got.float().cpu().view(n, H, d)
    for s, (start, m, p0) in enumerate(zip([0, 300], lens, past)):
        T = p0 + m
        pages = table[s, :-(-T // page)].long()
        keys = k_pool[pages].float().cpu().permute(0, 2, 1, 3).reshape(-1, G, d)[:T]
        vals = v_pool[pages].float().cpu().permute(0, 2, 1, 3).reshape(-1, G, d)[:T]
        qs = torch.zeros(T, H, d)
        qs[p0:] = q[start:start + m].float().cpu()
        want = plain.attend(qs, keys, vals, 0.1, plain.chunk_mask(T, chunk))[p0:]
        torch.testing.assert_close(got[start:start + m], want, rtol=2e-2, atol=2e-2)


def test_delta_scan_with_a_decay_per_key_channel_and_plain_filters():
    from garlic_inference_b200.ops import kernels
    from garlic_inference_b200.parts.linear_attention import scan_state_floats
    torch.manual_seed(3)
    H, Hk, d, dv, T = 4, 2, 24, 40, 50
    qkv = torch.randn(T, 2 * Hk * d + H * dv, device="cuda")
    b, a = torch.randn(T, H, device="cuda"), torch.randn(T, H * d, device="cuda")
    A_log, dt = torch.randn(H, device="cuda") * 0.5, torch.randn(H * d, device="cuda")
    sf = H * scan_state_floats(d, dv)
    spans = torch.tensor([[1, 0, T]], dtype=torch.int32, device="cuda")
    slots = torch.ones(T, dtype=torch.int32, device="cuda")
    q, k, v = (t.cpu() for t in (qkv[:, :Hk * d].view(T, Hk, d), qkv[:, Hk * d:2 * Hk * d].view(T, Hk, d), qkv[:, 2 * Hk * d:].view(T, H, dv)))
    q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5).repeat_interleave(H // Hk, 1)
    k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(H // Hk, 1)
    g = torch.exp(-torch.exp(A_log.cpu())[None, :, None] * plain.softplus((a.cpu() + dt.cpu()).view(T, H, d)))
    want = plain.delta_rule(q, k, v, plain.sigmoid(b.cpu()), g).reshape(T, H * dv)
    state = torch.zeros(3, sf, device="cuda")
    whole = kernels.delta_scan(qkv, (0, Hk * d, 2 * Hk * d), b, (0, 0), A_log, dt, state, spans, slots, H, Hk, d, dv, 1e-6,
                               channel_decay=True, decay_logits=a)
    torch.testing.assert_close(whole.cpu(), want, rtol=1e-4, atol=1e-5)
    state2 = torch.zeros(3, sf, device="cuda")
    one = torch.ones(1, dtype=torch.int32, device="cuda")
    steps = torch.cat([kernels.delta_scan(qkv[t:t + 1], (0, Hk * d, 2 * Hk * d), b[t:t + 1], (0, 0), A_log, dt, state2, None, one,
                                          H, Hk, d, dv, 1e-6, channel_decay=True, decay_logits=a[t:t + 1]) for t in range(T)])
    assert torch.equal(steps, whole) and torch.equal(state, state2), "token by token: the same bits"
    C, K = 70, 3
    x, taps = torch.randn(T, C, device="cuda"), torch.randn(C, K, device="cuda")
    st = torch.zeros(3, (K - 1) * C, device="cuda")
    y = kernels.causal_conv_silu(x, taps, st, slots, activation="none")
    torch.testing.assert_close(y.cpu(), plain.causal_conv(x.cpu(), taps.cpu()), rtol=1e-5, atol=1e-5)

"""Toretar on the GPU against the plain implementation: each mechanism's kernels alone, then
whole models through the trace runner, the step function and the generation entry point, with
prompts cut in every way, batches of unequal requests, reused slots and pages, planted far keys
and keys at page borders, long decoding and the first tokens of a sequence."""
import json
import os

import numpy as np
import pytest
import torch

import plain_toretar as plain
from replay_util import Trace, run_trace
from tiny_configs import TORETAR_A, TORETAR_B, TORETAR_C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_F32 = 2e-5
# bfloat16 engine against the float64 plain implementation, as a fraction of the largest logit
TOL_BF16 = 1.5e-2
PAGE = 64


def _within(errors, tol, dtype, what):
    """float32: every position within ``tol``.  bfloat16: rounding the router's input moves a token
    whose two candidate experts have nearly equal logits to the other expert now and then, which
    changes that position's logits by far more than rounding; random weights have such tokens, so up
    to 3 % of the positions (at least one) may be over, and the rest must be within ``tol``."""
    errors = np.asarray(errors)
    over = int((errors > tol).sum())
    allowed = 0 if dtype == "float32" else max(1, int(0.03 * errors.size))
    assert over <= allowed, f"{what}: {over} of {errors.size} positions are over {tol:.2e} (worst {errors.max():.2e})"


def _dt(name):
    return torch.float32 if name == "float32" else torch.bfloat16


def _rand(rng, shape, dtype, scale=1.0):
    """Random values that ``dtype`` holds exactly, as (device tensor, float64 numpy)."""
    t = torch.from_numpy(rng.standard_normal(shape) * scale).to(dtype)
    return t.to(DEV), t.double().numpy()


def _batch(starts, lens, slots):
    """Packed-token index tensors of a step: (tok_pos, tok_seq, seq_slot)."""
    pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lens)])
    seq = np.repeat(np.arange(len(lens)), lens)
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    return i32(pos), i32(seq), i32(slots), pos, seq


# ------------------------------------------------------------------ mechanisms alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotation_of_interleaved_pairs(dtype):
    from gemmars_b200 import kernels
    rng = np.random.default_rng(1)
    x, xr = _rand(rng, (7, 3, 10), _dt(dtype))
    pos = [0, 1, 5, 63, 64, 1000, 40000]
    dims, base = 6, 30000.0
    inv = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32, device=DEV)
    kernels.rope_pairs(x, torch.tensor(pos, dtype=torch.int32, device=DEV), inv, dims)
    want = plain.rotate_pairs(xr, pos, dims, base)
    tol = 2e-3 if dtype == "float32" else 2e-2     # the angle itself is float32: 40000 * f has 2^-8 of slack
    assert np.abs(x.double().cpu().numpy() - want).max() < tol
    assert np.array_equal(x.double().cpu().numpy()[..., dims:], xr[..., dims:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,rd,rank,rot", [(3, 20, 6, 36, 4), (1, 0, 8, 16, 8), (5, 8, 4, 24, 0)])
def test_prepare_norms_rotates_and_places_the_cache_rows(dtype, heads, dim, rd, rank, rot):
    from gemmars_b200 import kernels
    rng = np.random.default_rng(2)
    dt = _dt(dtype)
    starts, lens, slots = [60, 0, 127], [9, 3, 2], [2, 0, 1]
    tok_pos, tok_seq, seq_slot, pos, seq = _batch(starts, lens, slots)
    t = len(pos)
    q, qn = _rand(rng, (t, heads * (dim + rd)), torch.float32)
    kv, kvn = _rand(rng, (t, rank + rd), torch.float32)
    g, gn = _rand(rng, (t, heads), torch.float32)
    w, wn = _rand(rng, (rank,), torch.float32)
    table = torch.tensor([[3, 1, 0], [5, 2, 0], [4, 6, 7], [0, 0, 0]], dtype=torch.int32, device=DEV)
    cache = torch.zeros((8, PAGE, rank + rd), dtype=dt, device=DEV)
    q_nope = torch.empty((t, heads * dim), dtype=dt, device=DEV)
    qa = torch.zeros((t, heads * (rank + rd)), dtype=dt, device=DEV)
    gate = torch.empty((t, heads), dtype=torch.float32, device=DEV)
    base, eps, scale = 777.0, 1e-5, 0.37
    inv = torch.tensor([base ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32, device=DEV)
    kernels.latent_prepare(q, kv, g, w, eps, inv if rot else None, rot, scale, q_nope, qa, gate, cache, table, PAGE,
                           tok_pos, tok_seq, seq_slot, heads, dim, rd, rank)
    tol = 1e-5 if dtype == "float32" else 2e-2
    c = plain.rms_norm(kvn[:, :rank], wn, eps)
    kr = plain.rotate_pairs(kvn[:, rank:], pos, rot, base)
    table_h = table.cpu().numpy()
    got = cache.double().cpu().numpy()
    written = np.zeros((8, PAGE), dtype=bool)
    for i in range(t):
        page = table_h[slots[seq[i]], pos[i] // PAGE]
        row = got[page, pos[i] % PAGE]
        written[page, pos[i] % PAGE] = True
        assert np.abs(row - np.concatenate([c[i], kr[i]])).max() < tol * 4
    assert not got[~written].any()                       # nothing else was touched
    q3 = qn.reshape(t, heads, dim + rd)
    if dim:
        assert np.abs(q_nope.double().cpu().numpy() - (q3[:, :, :dim] * scale).reshape(t, -1)).max() < tol * 4
    qr = plain.rotate_pairs(q3[:, :, dim:], pos, rot, base) * scale
    assert np.abs(qa.double().cpu().numpy().reshape(t, heads, rank + rd)[:, :, rank:] - qr).max() < tol * 4
    assert np.abs(gate.double().cpu().numpy() - plain.sigmoid(gn)).max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("t,heads,n,k", [(5, 3, 36, 20), (130, 2, 24, 48), (1, 9, 128, 16), (70, 4, 48, 64)])
def test_products_per_head(dtype, t, heads, n, k):
    from gemmars_b200 import kernels
    rng = np.random.default_rng(3)
    dt = _dt(dtype)
    x, xn = _rand(rng, (t, heads * (k + 5)), dt)          # heads lie k + 5 apart: a view into wider rows
    w, wn = _rand(rng, (heads, n, k), dt)
    s, sn = _rand(rng, (t, heads), torch.float32)
    y = torch.zeros((t, heads * (n + 3)), dtype=dt, device=DEV)
    xv = x.view(t, heads, k + 5)[:, :, :k]
    yv = y.view(t, heads, n + 3)[:, :, :n]
    for scale, sc in ((None, None), (s, sn)):
        kernels.heads_gemm(xv, w, yv, heads, scale=scale)
        want = np.einsum("thk,hnk->thn", xn.reshape(t, heads, k + 5)[:, :, :k], wn)
        if sc is not None:
            want = want * sc[:, :, None]
        got = y.double().cpu().numpy().reshape(t, heads, n + 3)
        tol = 1e-5 if dtype == "float32" else 1e-2
        assert np.abs(got[:, :, :n] - want).max() <= tol * np.abs(want).max()
        assert not got[:, :, n:].any()


def _plain_latent_attention(qa, rows_of_seq, pos, seq, heads, rank, rd, window=None):
    out = np.zeros((len(pos), heads, rank))
    q3 = qa.reshape(len(pos), heads, rank + rd)
    for i in range(len(pos)):
        rows = rows_of_seq[seq[i]][:pos[i] + 1]
        if window:
            rows = rows[max(0, pos[i] + 1 - window):]
        for h in range(heads):
            out[i, h] = plain.softmax(rows @ q3[i, h]) @ rows[:, :rank]
    return out.reshape(len(pos), heads * rank)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,rank,rd", [(3, 36, 6), (7, 112, 16), (1, 64, 32), (17, 48, 16), (4, 256, 32), (2, 512, 64)])
@pytest.mark.parametrize("decoding", [False, True], ids=["prompt", "decoding"])
def test_attention_over_latents_finds_planted_keys(dtype, heads, rank, rd, decoding):
    """Sequences of several pages in shuffled pages.  Every query is made to point at one key, the
    rest being noise: far back, at a page's last and first position, its own position, and, for a
    query pointed at the position after its own, the result must not see that key."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(4)
    dt = _dt(dtype)
    kd = rank + rd
    lengths = [333, 70, 129]
    n_pages = sum(-(-n // PAGE) for n in lengths) + 1
    order = rng.permutation(np.arange(1, n_pages))
    table = np.zeros((4, 6), dtype=np.int32)
    cache = torch.zeros((n_pages, PAGE, kd), dtype=dt, device=DEV)
    rows_of_seq, at = [], 0
    for s, n in enumerate(lengths):
        rows, rown = _rand(rng, (n, kd), dt, 0.3)
        rows_of_seq.append(rown)
        for lp in range(-(-n // PAGE)):
            table[s, lp] = order[at]
            m = min(PAGE, n - lp * PAGE)
            cache[order[at], :m] = rows[lp * PAGE:lp * PAGE + m]
            at += 1
    # (sequence, query position, key the query points at)
    plant = [(0, 332, 1), (0, 332, 63), (0, 332, 64), (0, 200, 127), (0, 200, 128), (0, 200, 200), (0, 200, 201),
             (1, 69, 0), (1, 64, 63), (1, 64, 65), (2, 128, 128), (2, 128, 64), (2, 127, 128), (0, 0, 0), (0, 1, 0)]
    if decoding:
        groups = [[p] for p in plant if p[1] == lengths[p[0]] - 1 or p[1] < 2]     # one position of a sequence a step
    else:   # all sequences whole in one step; a query position is planted once a step
        groups = []
        for item in plant:
            for grp in groups:
                if all(item[:2] != other[:2] for other in grp):
                    grp.append(item)
                    break
            else:
                groups.append([item])
    for group in groups:
        if decoding:
            starts, lens, slots = [group[0][1]], [1], [group[0][0]]
            want_rows = [0]
        else:
            starts, lens, slots = [0, 0, 0], lengths, [0, 1, 2]
            offs = np.cumsum([0] + lengths)
            want_rows = [offs[s] + p for s, p, _ in group]
        tok_pos, tok_seq, seq_slot, pos, seq = _batch(starts, lens, slots)
        t = len(pos)
        qa, _ = _rand(rng, (t, heads * kd), dt, 0.3)
        for r, (s, p, key) in zip(want_rows, group):
            k = rows_of_seq[s][key] if key < lengths[s] else rng.standard_normal(kd)
            qa.view(t, heads, kd)[r] = torch.from_numpy(k * 40.0 / (k @ k) ** 0.5).to(dt).to(DEV)   # score ~ 40 |k|
        qan = qa.double().cpu().numpy()
        out = torch.zeros((t, heads * rank), dtype=dt, device=DEV)
        ctx = type("Ctx", (), dict(tok_pos=tok_pos, tok_seq=tok_seq, seq_slot=seq_slot, host=None, n_tokens=t,
                                   max_new=max(lens), pad_slot=None, cu_seqlens=None, seq_start=None))()
        ctx.cu_seqlens = torch.tensor(np.cumsum([0] + lens), dtype=torch.int32, device=DEV)
        ctx.seq_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        ctx.n_seqs, ctx.max_total = len(lens), max(a + b for a, b in zip(starts, lens))
        kernels.latent_attention(ctx, qa, out, heads, rank, rd, cache, torch.from_numpy(table).to(DEV), PAGE)
        seqmap = {i: rows_of_seq[s] for i, s in enumerate(slots)}
        want = _plain_latent_attention(qan, seqmap, pos, seq, heads, rank, rd)
        got = out.double().cpu().numpy()
        tol = 2e-5 if dtype == "float32" else 1.5e-2
        assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())
        for r, (s, p, key) in zip(want_rows, group):
            if key <= p:    # the planted key dominates: the output is its latent
                assert np.abs(got[r].reshape(heads, rank) - rows_of_seq[s][key][:rank]).max() < 0.05


@pytest.mark.parametrize("t,experts,top", [(9, 5, 2), (70, 8, 8), (3, 3, 1), (33, 40, 6), (5, 300, 32)])
def test_expert_choice_from_the_logits(t, experts, top):
    from gemmars_b200 import kernels
    rng = np.random.default_rng(5)
    z, zn = _rand(rng, (t, experts + 1), torch.float32)
    b, bn = _rand(rng, (experts,), torch.float32)
    idx, wts, gate = kernels.moe_topk(z, b, experts, top, has_gate=True)
    logits = zn[:, :experts] + bn
    want_idx = np.argsort(-logits, axis=-1, kind="stable")[:, :top]
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert np.abs(wts.double().cpu().numpy() - plain.softmax(np.take_along_axis(logits, want_idx, -1))).max() < 1e-6
    assert np.abs(gate.double().cpu().numpy() - plain.sigmoid(zn[:, experts])).max() < 1e-6
    z[:, 1] = z[:, 0]                               # a tie goes to the lower index
    idx2, _, none = kernels.moe_topk(z, None, experts, top)
    order = np.argsort(-z.cpu().numpy()[:, :experts], axis=-1, kind="stable")[:, :top]
    assert none is None and np.array_equal(idx2.cpu().numpy(), order)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("t,width,experts,top,ff,ffs", [(9, 72, 5, 2, 40, 56), (200, 128, 6, 3, 64, 96), (2, 40, 3, 1, 24, 0),
                                                      (130, 64, 2, 2, 32, 16), (300, 128, 6, 3, 64, 96),
                                                      (700, 64, 40, 1, 72, 0), (257, 256, 3, 2, 200, 136)])
def test_routed_feed_forward(dtype, t, width, experts, top, ff, ffs):
    """The whole feed-forward part against the plain one; inputs large enough that both clamps act."""
    from gemmars_b200.parts.base import build_part
    from gemmars_b200.parts.plan import PartSpec
    rng = np.random.default_rng(6)
    dt = _dt(dtype)
    names, w, wn = {}, {}, {}
    def add(short, shape, scale, f32=False):
        w[short], wn["p." + short.replace("router_bias", "router.b")] = _rand(rng, shape, dt, scale)
        names[short] = short
    add("router", (experts, width), 0.3)
    add("router_bias", (experts,), 0.3)
    for e in range(experts):
        add(f"e{e}.gate", (ff, width), 0.2)
        add(f"e{e}.up", (ff, width), 0.2)
        add(f"e{e}.down", (width, ff), 0.2)
    if ffs:
        add("shared.gate", (ffs, width), 0.2)
        add("shared.up", (ffs, width), 0.2)
        add("shared.down", (width, ffs), 0.2)
        add("shared.sg", (1, width), 0.3)
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": 0.8},
           "shared": {"ff": ffs, "limit": 1.7} if ffs else None}
    part = build_part("ffn", PartSpec("moe", {"hidden_size": width, "experts": experts, "top": top, "ff": ff, "limit": 0.8,
                                              "shared": {"ff": ffs, "limit": 1.7} if ffs else None}, names), dtype)
    part.load({k: (v.float() if part.wants()[k].role == "vector" else v.to(dt)) for k, v in w.items()})
    h, hn = _rand(rng, (t, width), dt)
    res, resn = _rand(rng, (t, width), torch.float32)
    ctx = type("Ctx", (), dict(host=None))()
    part.forward(ctx, h, res)
    want = resn + plain.moe(hn, wn, "p.", mlp)
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    assert np.abs(res.double().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    g = hn @ wn["p.e0.gate"].T
    assert (g > 0.8).any() and (np.abs(hn @ wn["p.e0.up"].T) > 0.8).any()


# ------------------------------------------------------------------ whole models

def _sharp_folder(tmp_path_factory, raw, seed, factor):
    """Random weights whose latent norm weights are scaled by ``factor``: scores grow with its
    square, attention picks single keys far back, and a wrong key, page or slot shows."""
    from gemmars_b200.weights import random_weights, write_safetensors
    tensors = random_weights(raw, seed=seed)
    for name in tensors:
        if name.endswith("dkv.norm"):
            tensors[name] = (tensors[name].float() * factor).bfloat16()
    d = str(tmp_path_factory.mktemp("toretar"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d


REQUESTS = {"A": (TORETAR_A, [15, 21, 9, 70, 40, 131]), "B": (TORETAR_B, [17, 33, 3, 80, 150, 65])}
GROUPS = [[0, 1, 2], [3, 4, 5]]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (raw, lengths) in REQUESTS.items():
        folder = _sharp_folder(tmp_path_factory, raw, seed=11 + len(name), factor=2.0)
        cfg, w = plain.load_folder(folder)
        rng = np.random.default_rng(lengths[0])
        reqs = [rng.integers(0, raw["vocab"], n).tolist() for n in lengths]
        out[name] = (folder, cfg, w, reqs, [plain.forward(cfg, w, r) for r in reqs])
    return out


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_cuttings_match_the_plain_implementation(name, dtype, models, tmp_path):
    """Through bin/trace_run: each request whole, with its last 32 tokens one by one, and in two
    batches of unequal requests that follow one another in a cache sized to the peak, so that the
    second batch lives in the slots and pages the first gave back."""
    folder, cfg, w, reqs, ref = models[name]
    tr = Trace()
    tr.whole("w", reqs)
    tr.tail("t", reqs)
    prompt_lens = [max(1, len(r) - 8 - 3 * i) for i, r in enumerate(reqs)]
    prompt_lens[2] = len(reqs[2])
    prompt_lens[1] = 1
    tr.batches("b", reqs, GROUPS, prompt_lens)
    got = run_trace(tr, folder, dtype, str(tmp_path / "out"))
    scale = max(float(np.abs(r).max()) for r in ref)
    tol = (TOL_F32 if dtype == "float32" else TOL_BF16) * scale
    for tag in "wtb":
        _within([np.abs(got[(f"{tag}{i}", p)] - r[p]).max() for i, r in enumerate(ref) for p in range(len(r))], tol, dtype,
               f"cutting {tag!r}")
    if dtype == "float32":
        for i, r in enumerate(ref):
            for p in range(len(r)):
                assert np.array_equal(got[(f"w{i}", p)], got[(f"t{i}", p)]) and np.array_equal(got[(f"w{i}", p)], got[(f"b{i}", p)])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_residual_after_every_layer(dtype, models):
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, cfg, w, reqs, _ = models["A"]
    toks = reqs[3]
    want = []
    plain.forward(cfg, w, toks, want)
    model = build_model(folder, dtype=dtype)
    seen = []
    for block in model.blocks:
        def run(ctx, x, caches, writes_cache=True, _inner=block.forward):
            _inner(ctx, x, caches, writes_cache=writes_cache)
            seen.append(x.double().cpu().numpy())
        block.forward = run
    runner = Runner(model, max_tokens=256, max_batch=1, use_graphs=False)
    runner.step([StepItem(runner.open(), toks, [])])
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        tol = (1e-5 if dtype == "float32" else 2e-2) * np.abs(b).max()
        _within(np.abs(a - b).max(axis=1), tol, dtype, f"layer {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_long_decoding_and_reused_slots(dtype, models):
    """One runner, a cache of six pages.  A prompt in portions of 2, 3, 64, 1, 65 and the rest;
    another from its first token one by one for 200 steps across three page borders beside a
    neighbour that comes and goes; then the same again in the slots and pages given back."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, cfg, w, reqs, ref = models["B"]
    model = build_model(folder, dtype=dtype)
    runner = Runner(model, max_tokens=6 * PAGE, max_batch=3)
    rng = np.random.default_rng(8)
    long_toks = rng.integers(0, cfg["vocab"], 200).tolist()
    long_ref = plain.forward(cfg, w, long_toks)
    scale = float(np.abs(long_ref).max())
    tol = (TOL_F32 if dtype == "float32" else TOL_BF16) * scale
    first_round = None
    for round_ in range(2):
        got = {}
        a = runner.open()
        at = 0
        for n in (2, 3, 64, 1, 65, 15):
            part = reqs[4][at:at + n]
            got.update({("a", at + i): r for i, r in enumerate(runner.step([StepItem(a, part, range(len(part)))]).cpu().numpy())})
            at += len(part)
        assert at == len(reqs[4])
        runner.close(a)
        b = runner.open()
        c = None
        for p, tok in enumerate(long_toks):
            items = [StepItem(b, [tok], [0])]
            if p == 20:
                c = runner.open()
                items.append(StepItem(c, reqs[0], range(len(reqs[0]))))     # a prompt beside a decoded token
            elif c is not None and p < 20 + 30:
                items.append(StepItem(c, [reqs[1][p - 21]], [0]))
            out = runner.step(items).cpu().numpy()
            got[("b", p)] = out[0]
            if p == 20:
                got.update({("c", i): r for i, r in enumerate(out[1:])})
            if p == 49:
                runner.close(c)
                c = None
        runner.close(b)
        assert runner.cache.pages_held() == 0
        _within([np.abs(got[("a", p)] - ref[4][p]).max() for p in range(len(reqs[4]))], tol, dtype, "portions")
        _within([np.abs(got[("b", p)] - long_ref[p]).max() for p in range(len(long_toks))], tol, dtype, "decoded")
        _within([np.abs(got[("c", p)] - ref[0][p]).max() for p in range(len(reqs[0]))], tol, dtype, "neighbour")
        if first_round is None:
            first_round = got
        elif dtype == "float32":
            assert all(np.array_equal(got[k], first_round[k]) for k in got)


def test_prompts_over_expanded_heads(tmp_path_factory):
    """Prompt steps whose sequences all start at position 0 may expand keys and values per head.
    Three unequal prompts in one step, then decoding from the cache the step left: both ways of
    running the prompt agree with the plain implementation, and a continued prompt (a cached prefix)
    takes the other way by itself."""
    from gemmars_b200 import kernels
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder = _sharp_folder(tmp_path_factory, TORETAR_C, seed=5, factor=2.0)
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(12)
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (150, 65, 3)]
    ref = [plain.forward(cfg, w, r + [7, 8]) for r in reqs]
    scale = max(float(np.abs(r).max()) for r in ref)
    was = kernels.LATENT_EXPAND_MIN_TOKENS
    got = {}
    try:
        for name, threshold in (("expanded", 32), ("latent", 1 << 30)):
            kernels.LATENT_EXPAND_MIN_TOKENS = threshold
            before = kernels.launch_count()
            model = build_model(folder, dtype="bfloat16")
            runner = Runner(model, max_tokens=1024, max_batch=4)
            slots = [runner.open() for _ in reqs]
            out = runner.step([StepItem(s, r, range(len(r))) for s, r in zip(slots, reqs)]).cpu().numpy()
            nxt = runner.step([StepItem(s, [7], [0]) for s in slots]).cpu().numpy()           # decoding reads the cache
            more = runner.step([StepItem(s, [8, 9], [0]) for s in slots]).cpu().numpy()       # a continued prompt
            got[name] = (out, nxt, more)
            errs, at = [], 0
            for i, r in enumerate(reqs):
                errs += list(np.abs(out[at:at + len(r)] - ref[i][:len(r)]).max(axis=1))
                errs.append(np.abs(nxt[i] - ref[i][len(r)]).max())
                errs.append(np.abs(more[i] - ref[i][len(r) + 1]).max())
                at += len(r)
            _within(errs, TOL_BF16 * scale, "bfloat16", name)
    finally:
        kernels.LATENT_EXPAND_MIN_TOKENS = was
    assert not np.array_equal(got["expanded"][0], got["latent"][0])     # the two ways are different arithmetic
    assert np.abs(got["expanded"][0] - got["latent"][0]).max() <= 2 * TOL_BF16 * scale


def test_greedy_generation_through_the_engine(models):
    from gemmars_b200 import Engine
    folder, cfg, w, reqs, _ = models["A"]
    eng = Engine.load(folder, "dtype=float32;max_batch=3;max_tokens=2048")
    prompts = [reqs[0], reqs[2], [5], reqs[4][:33], reqs[3]]
    free_run, _ = plain.generate(cfg, w, prompts[0], 10)
    stop = [free_run[4]]
    res = eng.generate(prompts, max_tokens=10, stop_ids=stop)
    for p, r in zip(prompts, res):
        want, reason = plain.generate(cfg, w, p, 10, stop=stop)
        assert r.tokens == want and r.reason == reason
    assert eng.runner.cache.pages_held() == 0
    again = eng.generate(list(reversed(prompts)), max_tokens=10, stop_ids=stop)
    assert [r.tokens for r in reversed(again)] == [r.tokens for r in res]
    # bfloat16 decodes through captured steps: the tokens it picks are the plain model's best or within
    # rounding of it (but for the few that follow a token routed to another expert, see _within)
    eng16 = Engine.load(folder, "dtype=bfloat16;max_batch=4;max_tokens=2048")
    near, total = 0, 0
    for p, r in zip(prompts, eng16.generate(prompts, max_tokens=8, stop_ids=[])):
        assert len(r.tokens) == 8
        for i, tok in enumerate(r.tokens):
            row = plain.forward(cfg, w, list(p) + r.tokens[:i])[-1]
            near += bool(row[tok] >= row.max() - TOL_BF16 * np.abs(row).max())
            total += 1
    assert near >= 0.9 * total
    assert eng16.runner.cache.pages_held() == 0

"""Kuporax on the GPU against the plain implementation: each mechanism's kernels alone, then whole
models through the trace runner, the step function and the generation entry point, with prompts
cut in every way, batches of unequal requests, reused slots and pages, planted keys far back, at
page borders and on both sides of a window's edge, long decoding and the first tokens of a
sequence."""
import json
import os

import numpy as np
import pytest
import torch

import plain_kuporax as plain
from replay_util import Trace, run_trace
from tiny_configs import KUPORAX_A, KUPORAX_B, KUPORAX_C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_F32 = 3e-5
# bfloat16 engine against the float64 plain implementation, as a fraction of the largest logit
TOL_BF16 = 3e-2
PAGE = 64


def _dt(name):
    return torch.float32 if name == "float32" else torch.bfloat16


def _rand(rng, shape, dtype=torch.float32, scale=1.0):
    """Random values that ``dtype`` holds exactly, as (device tensor, float64 numpy)."""
    t = torch.from_numpy(rng.standard_normal(shape) * scale).to(dtype)
    return t.to(DEV), t.double().numpy()


def _i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def _packed(lens, slots, starts=None):
    """Index tensors of a packed step: (cu_seqlens, tok_seq, seq_slot, tok_pos)."""
    starts = starts or [0] * len(lens)
    cu = np.concatenate([[0], np.cumsum(lens)])
    seq = np.repeat(np.arange(len(lens)), lens)
    pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lens)])
    return _i32(cu), _i32(seq), _i32(slots), _i32(pos)


def _cuts(total, sizes):
    """[(start, end)] covering 0..total in portions of ``sizes`` (the last size repeats)."""
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[min(i, len(sizes) - 1)], total - at)
        out.append((at, at + n))
        at, i = at + n, i + 1
    return out


# ------------------------------------------------------------------ mechanisms alone

def test_row_kernels():
    from gemmars_b200 import kernels
    rng = np.random.default_rng(1)
    table, tn = _rand(rng, (37, 52), torch.bfloat16)
    x, xn = _rand(rng, (9, 52))
    idx = [0, 36, 5, 5, 1, 2, 3, 4, 20]
    kernels.gather_add(table, _i32(idx), x)
    assert np.abs(x.double().cpu().numpy() - (xn + tn[idx])).max() < 1e-6
    for n in (52, 700, 4100):
        y, yn = _rand(rng, (5, n), scale=3.0)
        r, rn = _rand(rng, (5, n))
        w, wn = _rand(rng, (n,))
        kernels.rmsnorm_add(y, w, r, 1e-5)
        want = rn + plain.rms_scale(yn, 1e-5) * wn
        assert np.abs(r.double().cpu().numpy() - want).max() < 2e-5
        # with the norm that reads the stream next taken in the same pass
        w2, w2n = _rand(rng, (n,))
        for dtype in ("float32", "bfloat16"):
            r2 = torch.from_numpy(rn).float().to(DEV)
            h = torch.empty((5, n), dtype=_dt(dtype), device=DEV)
            kernels.rmsnorm_add(y, w, r2, 1e-5, (w2, 1e-6, h))
            assert torch.equal(r2, r)
            assert np.abs(h.double().cpu().numpy() - plain.rms_scale(want, 1e-6) * w2n).max() < (2e-5 if dtype == "float32" else 8e-2)
    for dtype in ("float32", "bfloat16"):
        gu, gn = _rand(rng, (11, 2 * 36), _dt(dtype), scale=2.0)
        out = torch.empty((11, 36), dtype=_dt(dtype), device=DEV)
        kernels.gated_act(gu, out, "gelu_tanh")
        want = plain.gelu_tanh(gn[:, :36]) * gn[:, 36:]
        assert np.abs(out.double().cpu().numpy() - want).max() < (1e-5 if dtype == "float32" else 1e-2) * max(1.0, np.abs(want).max())
    z, zn = _rand(rng, (3, 97))
    kernels.scale_rows(z, 1.7)
    assert np.allclose(z.cpu().numpy(), (zn * np.float32(1.7)).astype(np.float32), rtol=1e-6)


@pytest.mark.parametrize("tokens", [1, 8, 40, 100, 300])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_product_with_gelu(tokens, dtype):
    """act(x gate^T) * (x up^T): in bfloat16 the activation rides on the tensor-core product's epilogue."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(tokens)
    x, xn = _rand(rng, (tokens, 128), _dt(dtype))
    w, wn = _rand(rng, (2 * 200, 128), _dt(dtype), scale=0.2)
    out = torch.empty((tokens, 200), dtype=_dt(dtype), device=DEV)
    kernels.gemm_gated(x, w, out, "gelu_tanh")
    want = plain.gelu_tanh(xn @ wn[:200].T) * (xn @ wn[200:].T)
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert np.abs(out.double().cpu().numpy() - want).max() < tol * max(1.0, np.abs(want).max())
    kernels.check_status()


@pytest.mark.parametrize("taps,bias,act", [(1, False, False), (2, True, True), (4, False, True), (5, True, False), (8, True, True)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_filter_carries_its_last_inputs(taps, bias, act, dtype):
    """Three sequences in other slots than their order; portions of 1, 2, 3 and 7 rows, so that a
    portion is shorter than the filter's memory; a slot that is cleared and used again."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(taps)
    c, lens, slots = 70, [23, 1, 9], [2, 0, 3]
    w, wn = _rand(rng, (c, taps))
    b, bn = _rand(rng, (c,)) if bias else (None, None)
    state = torch.zeros((5, taps - 1, c), dtype=torch.float32, device=DEV)
    state[1] = 7.0                                   # a slot nobody uses keeps what it held
    seqs = [_rand(rng, (n, c + 6), _dt(dtype)) for n in lens]
    want = [plain.short_conv(s[1][:, 3:3 + c], wn, bn) for s in seqs]
    if act:
        want = [plain.silu(x) for x in want]
    for round_ in range(2):
        got = [np.zeros((n, c)) for n in lens]
        cuts = [_cuts(n, [1, 2, 3, 7]) for n in lens]
        for step in range(max(len(x) for x in cuts)):
            live = [i for i in range(3) if step < len(cuts[i])]
            rows = torch.cat([seqs[i][0][cuts[i][step][0]:cuts[i][step][1]] for i in live])
            cu, seq, slot, _ = _packed([cuts[i][step][1] - cuts[i][step][0] for i in live], [slots[i] for i in live])
            out = torch.full((rows.shape[0], c + 2), -5.0, dtype=_dt(dtype), device=DEV)
            kernels.short_filter(rows[:, 3:3 + c], w, b, state, cu, seq, slot, out[:, 1:1 + c], act=act)
            res, at = out.double().cpu().numpy(), 0
            assert (res[:, 0] == -5.0).all() and (res[:, -1] == -5.0).all()
            for i in live:
                lo, hi = cuts[i][step]
                got[i][lo:hi] = res[at:at + hi - lo, 1:1 + c]
                at += hi - lo
        tol = 1e-5 if dtype == "float32" else 3e-2
        for g, x in zip(got, want):
            assert np.abs(g - x).max() < tol * max(1.0, np.abs(x).max())
        if taps > 1:
            assert (state[1] == 7.0).all()
            last = seqs[0][1][-(taps - 1):, 3:3 + c]
            assert np.abs(state[2].double().cpu().numpy() - last).max() < 1e-6
        for s in slots:
            state[s].zero_()                          # what opening a sequence does


@pytest.mark.parametrize("taps", [2, 4, 7])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_filter_over_a_long_step_of_several_sequences(taps, dtype):
    """A step of more than 512 rows, in which a thread walks sixteen rows with the window in its
    registers: sequences of 300, 5, 260, 1 and 40 rows that each go on from a memory of earlier
    inputs, so the window has to be read anew wherever the rows pass to the next sequence; then
    the same rows one sequence a step, which must give the same bits."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(taps)
    c, lens, slots = 300, [300, 5, 260, 1, 40], [3, 0, 4, 1, 2]
    w, wn = _rand(rng, (c, taps))
    b, bn = _rand(rng, (c,))
    before = [_rand(rng, (taps - 1, c), _dt(dtype)) for _ in lens]        # what each sequence brought earlier
    rows = [_rand(rng, (n, c), _dt(dtype)) for n in lens]
    want = [plain.silu(plain.short_conv(np.concatenate([h[1], x[1]]), wn, bn))[taps - 1:] for h, x in zip(before, rows)]

    def fresh_state():
        state = torch.zeros((6, taps - 1, c), dtype=torch.float32, device=DEV)
        for h, s_ in zip(before, slots):
            state[s_] = h[0].float()
        return state

    state = fresh_state()
    cu, seq, slot, _ = _packed(lens, slots)
    out = torch.empty((sum(lens), c), dtype=_dt(dtype), device=DEV)
    kernels.short_filter(torch.cat([x[0] for x in rows]), w, b, state, cu, seq, slot, out, act=True)
    tol = 2e-5 if dtype == "float32" else 3e-2
    got = out.double().cpu().numpy()
    assert np.abs(got - np.concatenate(want)).max() < tol * max(1.0, np.abs(np.concatenate(want)).max())
    for x, s_, n in zip(rows, slots, lens):
        tail = np.concatenate([before[slots.index(s_)][1], x[1]])[-(taps - 1):]
        assert np.abs(state[s_].double().cpu().numpy() - tail).max() < 1e-6
    state2 = fresh_state()
    at = 0
    for x, s_, n in zip(rows, slots, lens):
        cu1, seq1, slot1, _ = _packed([n], [s_])
        one = torch.empty((n, c), dtype=_dt(dtype), device=DEV)
        kernels.short_filter(x[0], w, b, state2, cu1, seq1, slot1, one, act=True)
        assert torch.equal(one, out[at:at + n])
        at += n
    assert torch.equal(state, state2)


@pytest.mark.parametrize("heads,groups,dim,vdim", [(4, 4, 16, 24), (6, 2, 8, 40), (3, 1, 64, 64), (2, 2, 128, 128), (1, 1, 20, 7), (2, 1, 200, 72)])
def test_delta_rule_alone(heads, groups, dim, vdim):
    """Whole sequences against portions of 1, 2, 5 and 33 tokens, in slots out of order; the unit
    norms, the decay and beta are the kernel's work.  One k of a sequence is made large and its v
    distinctive, and a later q points at it: the read-out must find that write."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(heads * 100 + dim)
    lens, slots = [71, 2, 40], [1, 3, 0]
    a_log, an = _rand(rng, (heads,), scale=0.5)
    dt_bias, dn = _rand(rng, (heads,), scale=0.5)
    data, want = [], []
    for n in lens:
        x, xn = _rand(rng, (n, 2 * groups * dim + heads * vdim + 3))
        gates, gn = _rand(rng, (n, 2 * heads + 1), scale=2.0)
        if n > 30:
            xn[5, groups * dim:2 * groups * dim] *= 6.0                      # a loud key at token 5 ...
            xn[30, :groups * dim] = xn[5, groups * dim:2 * groups * dim]     # ... that the query at 30 asks for
            x = torch.from_numpy(xn).float().to(DEV)
            xn = x.double().cpu().numpy()
        data.append((x, gates))
        q = xn[:, :groups * dim].reshape(n, groups, dim)
        k = xn[:, groups * dim:2 * groups * dim].reshape(n, groups, dim)
        v = xn[:, 2 * groups * dim:2 * groups * dim + heads * vdim].reshape(n, heads, vdim)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        beta = plain.sigmoid(gn[:, :heads])
        decay = np.exp(-np.exp(an) * plain.softplus(gn[:, heads:2 * heads] + dn))
        want.append(plain.delta_scan(q, k, v, beta, decay))
    qk = groups * dim
    for sizes in ([1000], [1, 2, 5, 33], [1]):
        state = torch.zeros((5, heads, kernels.recurrent_state_floats(dim, vdim)), dtype=torch.float32, device=DEV)
        got = [np.zeros((n, heads * vdim)) for n in lens]
        cuts = [_cuts(n, sizes) for n in lens]
        for step in range(max(len(c) for c in cuts)):
            live = [i for i in range(3) if step < len(cuts[i])]
            x = torch.cat([data[i][0][cuts[i][step][0]:cuts[i][step][1]] for i in live])
            g = torch.cat([data[i][1][cuts[i][step][0]:cuts[i][step][1]] for i in live])
            cu, seq, slot, _ = _packed([cuts[i][step][1] - cuts[i][step][0] for i in live], [slots[i] for i in live])
            y = torch.empty((x.shape[0], heads * vdim), dtype=torch.float32, device=DEV)
            kernels.delta_rule(x[:, :qk], x[:, qk:2 * qk], x[:, 2 * qk:2 * qk + heads * vdim], g[:, :heads], g[:, heads:2 * heads],
                               a_log, dt_bias, state, cu, slot, y, heads, groups, dim, vdim, dim ** -0.5)
            res, at = y.double().cpu().numpy(), 0
            for i in live:
                lo, hi = cuts[i][step]
                got[i][lo:hi] = res[at:at + hi - lo]
                at += hi - lo
        for i, (out, final) in enumerate(want):
            assert np.abs(got[i] - out.reshape(lens[i], -1)).max() < 2e-5 * max(1.0, np.abs(out).max())
            held = torch.stack([kernels.recurrent_state_matrix(state[slots[i], h], dim, vdim) for h in range(heads)])
            assert np.abs(held.double().cpu().numpy() - final).max() < 2e-5 * max(1.0, np.abs(final).max())
        assert not state[2].any() and not state[4].any()


@pytest.mark.parametrize("heads,groups,n_state,vdim", [(3, 1, 12, 16), (4, 4, 20, 8), (2, 1, 64, 64), (5, 5, 7, 33), (2, 2, 128, 96)])
def test_state_space_scan_alone(heads, groups, n_state, vdim):
    from gemmars_b200 import kernels
    rng = np.random.default_rng(heads * 100 + n_state)
    lens, slots = [60, 1, 35], [2, 0, 1]
    a_log, an = _rand(rng, (heads,), scale=0.5)
    dt_bias, dn = _rand(rng, (heads,), scale=0.5)
    skip, sn = _rand(rng, (heads,))
    inner, gn_ = heads * vdim, groups * n_state
    data, want = [], []
    for n in lens:
        x, xn = _rand(rng, (n, inner + 2 * gn_ + 5))
        d, dd = _rand(rng, (n, heads + 2))
        data.append((x, d))
        dt = plain.softplus(dd[:, 1:1 + heads] + dn)
        want.append(plain.ssd_scan(xn[:, :inner].reshape(n, heads, vdim), xn[:, inner:inner + gn_].reshape(n, groups, n_state),
                                   xn[:, inner + gn_:inner + 2 * gn_].reshape(n, groups, n_state), dt, np.exp(an), sn))
    for sizes in ([1000], [2, 1, 9], [1]):
        state = torch.zeros((4, heads, kernels.recurrent_state_floats(n_state, vdim)), dtype=torch.float32, device=DEV)
        got = [np.zeros((n, inner)) for n in lens]
        cuts = [_cuts(n, sizes) for n in lens]
        for step in range(max(len(c) for c in cuts)):
            live = [i for i in range(3) if step < len(cuts[i])]
            x = torch.cat([data[i][0][cuts[i][step][0]:cuts[i][step][1]] for i in live])
            d = torch.cat([data[i][1][cuts[i][step][0]:cuts[i][step][1]] for i in live])
            cu, seq, slot, _ = _packed([cuts[i][step][1] - cuts[i][step][0] for i in live], [slots[i] for i in live])
            y = torch.empty((x.shape[0], inner), dtype=torch.float32, device=DEV)
            kernels.ssd_scan(x[:, :inner], x[:, inner:inner + gn_], x[:, inner + gn_:inner + 2 * gn_], d[:, 1:1 + heads], a_log,
                             dt_bias, skip, state, cu, slot, y, heads, groups, n_state, vdim)
            res, at = y.double().cpu().numpy(), 0
            for i in live:
                lo, hi = cuts[i][step]
                got[i][lo:hi] = res[at:at + hi - lo]
                at += hi - lo
        for i, (out, final) in enumerate(want):
            assert np.abs(got[i] - out.reshape(lens[i], -1)).max() < 2e-5 * max(1.0, np.abs(out).max())
            held = torch.stack([kernels.recurrent_state_matrix(state[slots[i], h], n_state, vdim) for h in range(heads)])
            assert np.abs(held.double().cpu().numpy() - final).max() < 2e-5 * max(1.0, np.abs(final).max())
        assert not state[3].any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,group,wn,first", [(48, 16, 48, True), (160, 40, 40, False), (72, 72, 72, True), (66, 33, 33, False)])
def test_gated_norm_over_groups(dtype, n, group, wn, first):
    from gemmars_b200 import kernels
    rng = np.random.default_rng(n)
    y, yn = _rand(rng, (7, n), scale=3.0)
    gate, gn = _rand(rng, (7, n + 4))
    w, wv = _rand(rng, (wn,))
    out = torch.empty((7, n), dtype=_dt(dtype), device=DEV)
    kernels.gated_group_norm(y, gate[:, 2:2 + n], w, out, group, 1e-5, first, 0.8)
    gt = plain.silu(gn[:, 2:2 + n])
    weights = np.tile(wv, n // wn)
    if first:
        want = plain.rms_scale((yn * gt).reshape(7, n // group, group), 1e-5).reshape(7, n) * weights
    else:
        want = plain.rms_scale(yn.reshape(7, n // group, group), 1e-5).reshape(7, n) * weights * gt
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert np.abs(out.double().cpu().numpy() - 0.8 * want).max() < tol * max(1.0, np.abs(want).max())


class _Ctx:
    """What attention_capped reads of a step's context: every query a sequence of its own that
    brings one token, all of them reading the same slot."""

    def __init__(self, positions, slot):
        n = len(positions)
        self.tok_pos, self.tok_seq, self.seq_slot = _i32(positions), _i32(np.arange(n)), _i32([slot] * n)
        self.cu_seqlens, self.seq_start, self.n_seqs = _i32(np.arange(n + 1)), _i32(positions), n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,groups,dim,vdim,rot,taps,window,cap",
                         [(4, 2, 24, 40, 16, 2, 50, 7.5), (3, 3, 32, 16, 32, 1, 9, 11.0), (8, 2, 64, 128, 32, 4, 130, 30.0),
                          (2, 1, 48, 80, 0, 3, 64, 0.0), (2, 2, 80, 256, 8, 0, None, 25.0), (5, 1, 16, 300, 16, 2, 200, 3.0)])
def test_capped_attention_finds_planted_keys(dtype, heads, groups, dim, vdim, rot, taps, window, cap):
    """One sequence of 300 tokens in shuffled pages beside a short one.  The filter and the rotation
    are checked through the cache rows; then queries are built that point at single keys: far back,
    on both sides of page borders, the query's own position, and the keys just inside and just
    outside the window.  Run as one prompt, as a prompt in portions, and token by token."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(dim + vdim)
    dt = _dt(dtype)
    n, short = 300, 5
    channels = (heads + groups) * dim + groups * vdim
    base, scale = 5000.0, 0.2
    inv = torch.tensor([base ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32, device=DEV)
    w, wn = _rand(rng, (channels, taps)) if taps else (None, None)
    table = torch.tensor([[7, 2, 9, 4, 1], [3, 0, 0, 0, 0], [0, 0, 0, 0, 0]], dtype=torch.int32, device=DEV)
    u, un = _rand(rng, (n + short, channels + 8), dt)
    f = [plain.short_conv(x, wn) if taps else x for x in (un[:n, 4:4 + channels], un[n:, 4:4 + channels])]
    want_q, want_k, want_v = [], [], []
    for x in f:
        t = len(x)
        pos = np.arange(t)
        want_q.append(plain.rotate_half(x[:, :heads * dim].reshape(t, heads, dim), pos, base, rot))
        want_k.append(plain.rotate_half(x[:, heads * dim:(heads + groups) * dim].reshape(t, groups, dim), pos, base, rot))
        want_v.append(x[:, (heads + groups) * dim:].reshape(t, groups, vdim))
    tol = 2e-5 if dtype == "float32" else 3e-2
    for sizes in ([1000], [2, 3, 64, 1, 65], [1]):
        kc = torch.zeros((11, groups, PAGE, dim), dtype=dt, device=DEV)
        vc = torch.zeros((11, groups, vdim, PAGE), dtype=dt, device=DEV)
        state = torch.zeros((3, max(taps - 1, 0), channels), dtype=torch.float32, device=DEV)
        q_all = torch.zeros((n + short, heads * dim), dtype=dt, device=DEV)
        cuts = [_cuts(n, sizes), _cuts(short, sizes)]
        for step in range(max(len(c) for c in cuts)):
            live = [i for i in range(2) if step < len(cuts[i])]
            spans = [(cuts[i][step][0] + (n if i else 0), cuts[i][step][1] + (n if i else 0)) for i in live]
            rows = torch.cat([u[lo:hi] for lo, hi in spans])
            cu, seq, slot, pos = _packed([cuts[i][step][1] - cuts[i][step][0] for i in live], [0 if i == 0 else 1 for i in live],
                                         [cuts[i][step][0] for i in live])
            q = torch.empty((rows.shape[0], heads * dim), dtype=dt, device=DEV)
            kernels.filter_rope_cache(rows[:, 4:4 + channels], w, state if taps > 1 else None, inv if rot else None, rot, pos, seq,
                                      slot, cu, table, PAGE, q, kc, vc, heads, groups, dim, vdim)
            if taps > 1:
                kernels.short_filter_state(rows[:, 4:4 + channels], state, cu, slot, taps)
            at = 0
            for lo, hi in spans:
                q_all[lo:hi] = q[at:at + hi - lo]
                at += hi - lo
        got_q = q_all.double().cpu().numpy()
        assert np.abs(got_q[:n].reshape(n, heads, dim) - want_q[0]).max() < tol * 4
        assert np.abs(got_q[n:].reshape(short, heads, dim) - want_q[1]).max() < tol * 4
        kh, vh, th = kc.double().cpu().numpy(), vc.double().cpu().numpy(), table.cpu().numpy()
        for p in (0, 1, 63, 64, 65, 127, 128, 255, 256, 299):
            assert np.abs(kh[th[0, p // PAGE], :, p % PAGE] - want_k[0][p]).max() < tol * 4
            assert np.abs(vh[th[0, p // PAGE], :, :, p % PAGE] - want_v[0][p]).max() < tol * 4
        assert not kh[5].any() and not kh[6].any() and not kh[0].any()       # pages nobody owns
    # queries that point at single keys of the long sequence, as the cache holds them
    keys = kc.double().cpu().numpy()
    size = window or 10 ** 9
    targets = []
    for p in (299, 200, 128, 64, 17):
        for back in (0, 1, p % PAGE, p % PAGE + 1, p, size - 1, size, size + 1, size - 2):
            if 0 <= p - back:
                targets.append((p, p - back))
    qn = np.zeros((len(targets), heads, dim))
    for i, (p, j) in enumerate(targets):
        for h in range(heads):
            key = keys[th[0, j // PAGE], h // (heads // groups), j % PAGE]
            qn[i, h] = key * (40.0 / scale / max((key * key).sum(), 1e-3))    # a score of 40 for key j before the cap
    q = torch.from_numpy(qn.reshape(len(targets), -1)).to(dt).to(DEV)
    gate, gn = _rand(rng, (len(targets), heads * vdim + 2), dt)
    out = torch.empty((len(targets), heads * vdim), dtype=dt, device=DEV)
    ctx = _Ctx([p for p, _ in targets], 0)
    gate_cols = gate[:, 2:2 + heads * vdim]
    kernels.attention_capped(ctx, q, out, heads, kc, vc, table, PAGE, window, scale, cap, gate_cols, 0.7)
    if kernels.attention_capped_mma_usable(dt, dim, vdim, PAGE):
        # the tensor-core kernel ran; the plain kernel on the same inputs agrees with it
        other = torch.empty_like(out)
        kernels.CAPPED_ATTENTION_MMA = False
        try:
            kernels.attention_capped(ctx, q, other, heads, kc, vc, table, PAGE, window, scale, cap, gate_cols, 0.7)
        finally:
            kernels.CAPPED_ATTENTION_MMA = True
        assert (out.double() - other.double()).abs().max() < 2e-2 * max(1.0, float(other.abs().max()))
    kall = np.stack([keys[th[0, j // PAGE], :, j % PAGE] for j in range(n)])
    vall = np.stack([vc.double().cpu().numpy()[th[0, j // PAGE], :, :, j % PAGE] for j in range(n)])
    want = plain.capped_attention(q.double().cpu().numpy().reshape(len(targets), heads, dim), kall, vall, [p for p, _ in targets],
                                  np.arange(n), scale, cap, window)
    want = want.reshape(len(targets), -1) * plain.sigmoid(gn[:, 2:2 + heads * vdim]) * 0.7
    assert np.abs(out.double().cpu().numpy() - want).max() < (2e-5 if dtype == "float32" else 2e-2) * max(1.0, np.abs(want).max())
    if cap == 0.0 or cap >= 30.0:
        # the planted key decides: outside the window the output is never its value; inside it is,
        # unless a neighbour that shares the filter's inputs is louder still (the plain implementation
        # says which)
        found = 0
        for i, (p, j) in enumerate(targets):
            mine = vall[j].repeat(heads // groups, axis=0).reshape(-1) * plain.sigmoid(gn[i, 2:2 + heads * vdim]) * 0.7
            close = np.abs(out[i].double().cpu().numpy() - mine).max() < 0.1 * np.abs(mine).max()
            assert close == (np.abs(want[i] - mine).max() < 0.1 * np.abs(mine).max())
            if p - j >= size:
                assert not close, f"query {p} saw key {j} outside its window of {window}"
            found += bool(close)
        assert found >= 0.5 * sum(p - j < size for p, j in targets)


# ------------------------------------------------------------------ whole models

def _sharp_folder(tmp_path_factory, raw, seed):
    """Random weights whose q and k projections are large enough that attention prefers single keys
    and the delta rule's reads depend on which writes came before, and whose decay and step
    projections vary from token to token: a wrong key, window, state or slot then shows."""
    from gemmars_b200.weights import random_weights, write_safetensors
    tensors = random_weights(raw, seed=seed)
    for name in tensors:
        tail = name.split(".")[-1]
        if name.endswith(("left.q", "left.k")):
            tensors[name] = (tensors[name].float() * 6.0).bfloat16()
        elif tail in ("a", "b") and ".mix." in name and tensors[name].dim() == 2:
            tensors[name] = (tensors[name].float() * 8.0).bfloat16()
        elif tail in ("v", "in", "q", "k") and ".mix." in name:
            tensors[name] = (tensors[name].float() * 3.0).bfloat16()
    d = str(tmp_path_factory.mktemp("kuporax"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d


REQUESTS = {"A": (KUPORAX_A, [15, 21, 9, 70, 40, 131]), "B": (KUPORAX_B, [17, 33, 3, 80, 150, 65]),
            "C": (KUPORAX_C, [5, 30, 1, 66, 12, 90])}
GROUPS = [[0, 1, 2], [3, 4, 5]]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (raw, lengths) in REQUESTS.items():
        folder = _sharp_folder(tmp_path_factory, raw, seed=7 + len(out))
        cfg, w = plain.load_folder(folder)
        rng = np.random.default_rng(lengths[0])
        reqs = [rng.integers(0, raw["vocab"], n).tolist() for n in lengths]
        out[name] = (folder, cfg, w, reqs, [plain.forward(cfg, w, r) for r in reqs])
    return out


def _check(errors, tol, what, dtype="float32"):
    """float32: every position within ``tol``.  bfloat16: the sharpened weights put several keys'
    scores close to one another, and rounding q and k moves the softmax's weights between them by
    more than rounding moves anything else: 5 % of the positions (at least two) may be over ``tol``,
    none over four times it."""
    errors = np.asarray(errors)
    over = int((errors > tol).sum())
    allowed = 0 if dtype == "float32" else max(2, int(0.05 * errors.size))
    assert over <= allowed and errors.max() <= 4 * tol, \
        f"{what}: {over} of {errors.size} positions are over {tol:.2e} (worst {errors.max():.2e})"


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_cuttings_match_the_plain_implementation(name, dtype, models, tmp_path):
    """Through bin/trace_run: each request whole, with its last 32 tokens one by one, and in two
    batches of unequal requests that follow one another in a cache sized to the peak, so that the
    second batch lives in the slots, pages and states the first gave back."""
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
        _check([np.abs(got[(f"{tag}{i}", p)] - r[p]).max() for i, r in enumerate(ref) for p in range(len(r))], tol, f"cutting {tag!r}", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_residual_after_every_layer(dtype, models):
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, cfg, w, reqs, _ = models["A"]
    toks = reqs[3]
    _, want = plain.forward(cfg, w, toks, return_layers=True)
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
        tol = (2e-5 if dtype == "float32" else 3e-2) * np.abs(b).max()
        _check(np.abs(a - b).max(axis=1), tol, f"layer {i}", dtype)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_long_decoding_and_reused_slots(name, dtype, models):
    """One runner with a small cache.  A prompt in portions of 2, 3, 64, 1, 65 and the rest; another
    from its first token one by one for 400 steps, far past every window (a window's pages are a
    ring that is written over) and across page borders, beside a neighbour that comes and goes;
    then the same again in the slots, pages and states given back."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, cfg, w, reqs, ref = models[name]
    model = build_model(folder, dtype=dtype)
    runner = Runner(model, max_tokens=8 * PAGE, max_batch=3, prefill_chunk=70)
    rng = np.random.default_rng(8)
    long_toks = rng.integers(0, cfg["vocab"], 400).tolist()
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
            if part:
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
                items.append(StepItem(c, [reqs[3][p - 21]], [0]))
            out = runner.step(items).cpu().numpy()
            got[("b", p)] = out[0]
            if p == 20:
                got.update({("c", i): r for i, r in enumerate(out[1:])})
            if p == 49:
                runner.close(c)
                c = None
        runner.close(b)
        assert runner.cache.pages_held() == 0
        _check([np.abs(got[("a", p)] - ref[4][p]).max() for p in range(len(reqs[4]))], tol, "portions", dtype)
        _check([np.abs(got[("b", p)] - long_ref[p]).max() for p in range(len(long_toks))], tol, "decoded", dtype)
        _check([np.abs(got[("c", p)] - ref[0][p]).max() for p in range(len(reqs[0]))], tol, "neighbour", dtype)
        if first_round is None:
            first_round = got
        elif dtype == "float32":
            assert all(np.array_equal(got[k], first_round[k]) for k in got)


def test_prompt_chunks_of_the_step_function(models):
    """A prompt longer than the runner's chunk is cut by the step function itself; the states and
    the filters' memories pass from chunk to chunk.  Chunks of 2 tokens, the smallest that still
    is a prompt step."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, cfg, w, reqs, ref = models["A"]
    model = build_model(folder, dtype="float32")
    for chunk in (2, 7, 64):
        runner = Runner(model, max_tokens=4 * PAGE, max_batch=2, prefill_chunk=chunk)
        s0, s1 = runner.open(), runner.open()
        out = runner.step([StepItem(s0, reqs[5], range(len(reqs[5]))), StepItem(s1, reqs[1], range(len(reqs[1])))]).cpu().numpy()
        scale = float(np.abs(ref[5]).max())
        assert np.abs(out[:len(reqs[5])] - ref[5]).max() < TOL_F32 * scale
        assert np.abs(out[len(reqs[5]):] - ref[1]).max() < TOL_F32 * scale


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
    # bfloat16 decodes through captured steps: the tokens it picks are the plain model's best or
    # within rounding of it
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


def test_a_conversation_keeps_its_states_between_turns(models):
    """``Engine.send``: the slot lives on between turns, so the recurrent states, the filters'
    memories and the window's pages are carried; two turns give what one long sequence gives."""
    from gemmars_b200 import Engine
    folder, cfg, w, reqs, _ = models["A"]
    eng = Engine.load(folder, "dtype=float32;max_batch=2;max_tokens=1024")
    eng.set("max_tokens", 5)
    eng.set("stop", "")
    first, second = reqs[0], reqs[2]
    a = eng.send(first)
    want_a, _ = plain.generate(cfg, w, first, 5)
    assert a.tokens == want_a
    b = eng.send(second)
    want_b, _ = plain.generate(cfg, w, list(first) + want_a + list(second), 5)
    assert b.tokens == want_b
    eng.reset()
    assert eng.runner.cache.pages_held() == 0
    assert eng.send(first).tokens == want_a              # the slot taken again starts from zero states

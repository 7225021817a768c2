"""Ninisun on the GPU against the plain float64 oracle (tests/ninisun_oracle.py): every mechanism alone through the
C ABI, then whole models of several shapes through the engine, the slot cache, the state slots and the scheduler."""
import json
import math
import os

import pytest
import torch

import ninisun_oracle as O

pytestmark = pytest.mark.gpu
F64 = torch.float64
PAGE = 64


def _lib():
    from pg_b200 import _cabi as cabi
    return cabi, cabi.lib(), cabi.stream()


def _engine(cfg, seed=0, dtype=torch.float32, pool_tokens=1024, lora=6, **kw):
    from pg_b200.ninisun import NinisunEngine
    ck = O.make_checkpoint(cfg, seed, lora=lora)
    return NinisunEngine(cfg, ck, device="cuda:0", dtype=dtype, kv_pool_tokens=pool_tokens, **kw), ck


def _close(got, want, rel):
    got, want = got.detach().cpu().to(F64), want.to(F64)
    err = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt().clamp_min(1e-30))
    assert err <= rel, f"relative rms error {err:.3g} > {rel}"


def _rows_close(got, want, rel, stray=0.0):
    """Every row within `rel` (relative rms).  stray > 0 (16-bit runs of whole models): that fraction of the rows may
    differ.  At the first positions of a sequence a recurrent head's output is v (k . r) divided by its own rms, so
    with k . r near zero the sign of the whole head's contribution is a matter of rounding the projections."""
    got, want = got.detach().cpu().to(F64), want.to(F64)
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)
    bad = int((err > rel).sum())
    assert bad <= stray * err.numel(), \
        f"{bad} of {err.numel()} rows over {rel}: worst relative rms error {float(err.max()):.3g} (row {int(err.argmax())})"


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


_KEEP = []


def _i32(v):
    """Device copy that outlives the asynchronous launch it is passed to."""
    _KEEP.append(torch.tensor(v, dtype=torch.int32, device="cuda"))
    del _KEEP[:-64]
    return _KEEP[-1]


TOL = {torch.float32: 3e-5, torch.bfloat16: 5e-2}
STRAY = {torch.float32: 0.0, torch.bfloat16: 0.015}
CT = {torch.float32: 0, torch.bfloat16: 1}


# ------------------------------------------------------------------ mechanisms alone (C ABI)
@pytest.mark.parametrize("D,with_scale,with_next", [(48, True, True), (100, False, True), (256, True, False),
                                                    (1500, True, True), (4096, True, True), (4100, False, True)])
@pytest.mark.parametrize("R", [9, 70])       # a CTA per row for a handful of rows, a warp per row beyond
def test_output_norm_layer_scale_residual_next_norm(D, with_scale, with_next, R):
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(2)
    x, y = torch.randn(R, D, generator=g) * 2, torch.randn(R, D + 8, generator=g) * 5
    wp, sc, wn = (torch.randn(D, generator=g) for _ in range(3))
    xd, yd, out = x.cuda(), y.cuda(), torch.zeros(R, D, device="cuda")
    wpd, scd, wnd = wp.cuda(), sc.cuda(), wn.cuda()
    cabi.check(L.pg_postnorm_residual(out.data_ptr() if with_next else None, xd.data_ptr(), yd.data_ptr(), D + 8,
                                      wpd.data_ptr(), scd.data_ptr() if with_scale else None,
                                      wnd.data_ptr() if with_next else None, R, D, 1e-3, cabi.PG_F32, st))
    want = x.to(F64) + O.rms_norm(y[:, :D], wp, 1e-3) * (sc.to(F64) if with_scale else 1.0)
    _close(xd, want, 1e-6)
    if with_next:
        _close(out, O.rms_norm(want, wn, 1e-3), 1e-5)


def test_gelu_pairing():
    cabi, L, st = _lib()
    gu = (torch.randn(5, 2 * 24, generator=torch.Generator().manual_seed(3)) * 3).cuda()
    out = torch.empty(5, 24, device="cuda")
    cabi.check(L.pg_geglu(out.data_ptr(), gu.data_ptr(), 5, 24, cabi.PG_F32, st))
    g = gu.cpu().to(F64)
    _close(out, O.gelu_tanh(g[:, :24]) * g[:, 24:], 1e-6)


class Paged:
    """Shuffled pages for `lens` sequences: pools [pages, 64, cols], page table [slots, max_pages]."""

    def __init__(self, lens, kcols, vcols, dtype=torch.float32, seed=0):
        per = [(n + PAGE - 1) // PAGE for n in lens]
        total = sum(per) + 3
        order = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
        self.max_pages = max(per) + 1
        table = torch.full((len(lens), self.max_pages), order[-1], dtype=torch.int32)
        at = 0
        for s, n in enumerate(per):
            table[s, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
            at += n
        self.table_host, self.table = table, table.cuda()
        self.k = torch.full((total, PAGE, kcols), 7.0, dtype=dtype, device="cuda")    # stale rows would show
        self.v = torch.full((total, PAGE, vcols), -9.0, dtype=dtype, device="cuda")

    def rows(self, slot, positions):
        return [int(self.table_host[slot, p // PAGE]) * PAGE + p % PAGE for p in positions]

    def fill(self, slot, k, v):
        r = torch.tensor(self.rows(slot, range(k.shape[0])), device="cuda")
        self.k.view(-1, self.k.shape[-1])[r] = k.reshape(k.shape[0], -1).to(self.k.dtype).cuda()
        self.v.view(-1, self.v.shape[-1])[r] = v.reshape(v.shape[0], -1).to(self.v.dtype).cuda()


@pytest.mark.parametrize("dim,rot_dims,scaling,biased,mix", [
    (8, 4, None, False, True), (16, 16, (4.0, 64, 16.0, 1.0), True, False), (12, 0, None, True, True),
    (32, 10, (2.5, 100, 8.0, 0.5), False, False)])
def test_rotary_append_bias_value_mixing(dim, rot_dims, scaling, biased, mix):
    cabi, L, st = _lib()
    from pg_b200.ninisun import RotaryCfg
    H, G, vdim, T = 3, 1, 20, 6
    g = torch.Generator().manual_seed(5)
    nq, nk, nv = H * dim, G * dim, G * vdim
    ld = 8 + nq + nk + nv + 3
    proj = torch.randn(T, ld, generator=g)
    qb, kb, vb = torch.randn(nq, generator=g), torch.randn(nk, generator=g), torch.randn(nv, generator=g)
    vf = torch.randn(T, nv + 5, generator=g)
    positions, slots = [70, 71, 0, 1, 2, 300], [1, 1, 0, 0, 0, 2]
    pg = Paged([3, 72, 301], nk, nv)
    freq, mag = (None, 1.0)
    if rot_dims:
        f, mag = RotaryCfg(rot_dims, 777.0, dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None).table()
        freq = f.to(torch.float32).cuda()
    projd, q_out = proj.cuda(), torch.empty(T, nq, device="cuda")
    dev = [t.cuda() for t in (qb, kb, vb, vf)]
    cabi.check(L.pg_rotary_append(
        q_out.data_ptr(), projd.data_ptr(), ld, 8, H, 8 + nq, G, dim, 8 + nq + nk, vdim,
        dev[0].data_ptr() if biased else None, dev[1].data_ptr() if biased else None, dev[2].data_ptr() if biased else None,
        None if freq is None else freq.data_ptr(), rot_dims, mag, 1, dev[3].data_ptr() if mix else None, nv + 5, 0.3,
        pg.k.data_ptr(), pg.v.data_ptr(), pg.table.data_ptr(), pg.max_pages, PAGE, _i32(slots).data_ptr(),
        _i32(positions).data_ptr(), T, cabi.PG_F32, st))
    q = proj[:, 8:8 + nq].to(F64) + (qb.to(F64) if biased else 0)
    k = proj[:, 8 + nq:8 + nq + nk].to(F64) + (kb.to(F64) if biased else 0)
    v = proj[:, 8 + nq + nk:8 + nq + nk + nv].to(F64) + (vb.to(F64) if biased else 0)
    q, k = q.view(T, H, dim), k.view(T, G, dim)
    if rot_dims:
        r = O.rot(rot_dims, 777.0, scaling)
        cos, sin = O.rotary_table(r, positions)
        q, k = O.rotate_pairs(q, cos, sin), O.rotate_pairs(k, cos, sin)
    if mix:
        v = 0.7 * v + 0.3 * vf[:, :nv].to(F64)
    _close(q_out, q.reshape(T, nq), 2e-6)
    rows = [pg.rows(s, [p])[0] for s, p in zip(slots, positions)]
    _close(pg.k.view(-1, nk)[rows], k.reshape(T, nk), 2e-6)
    _close(pg.v.view(-1, nv)[rows], v, 2e-6)
    untouched = torch.ones(pg.k.shape[0] * PAGE, dtype=torch.bool)
    untouched[rows] = False
    assert bool((pg.k.view(-1, nk).cpu()[untouched] == 7.0).all())


def _attention_case(H, G, dim, vdim, window, keep, lens, new, sigmoid, dtype=torch.float32, tower=None, seed=0, tc=False):
    """Sequences of lens[s] cached tokens of which the last new[s] are this step's queries; returns (got, want).
    tc: through the tensor-core kernel (query tiles of up to 128 consecutive tokens of one sequence)."""
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(seed)
    pg = Paged(lens, G * dim, G * vdim, dtype)
    scale = 0.4
    qs, want, slots, positions = [], [], [], []
    pb = torch.randn(H, generator=g)
    gate_rows = []
    for s, (n, m) in enumerate(zip(lens, new)):
        q, k, v = torch.randn(n, H, dim, generator=g), torch.randn(n, G, dim, generator=g), torch.randn(n, G, vdim, generator=g)
        if tower is not None:                     # one key whose score stands far out for the last query
            j = tower(n - 1)
            if 0 <= j < n:
                k[j] = 12.0 * q[n - 1, ::H // G] / scale / dim
                v[j] += 50.0
        if dtype != torch.float32:
            q, k, v = (t.to(dtype).float() for t in (q, k, v))
        pg.fill(s, k, v)
        if sigmoid:
            o = O.causal_sigmoid_attention(q.to(F64), k.to(F64), v.to(F64), scale, pb.to(F64))
            gt = torch.randn(n, H, generator=g)
            if dtype != torch.float32:
                gt = gt.to(dtype).float()
            o = o * O.sigmoid(gt.to(F64))[:, :, None] * 0.65
            gate_rows.append(gt[n - m:])
        else:
            o = O.window_softmax_attention(q.to(F64), k.to(F64), v.to(F64), scale, window, keep)
        qs.append(q[n - m:].reshape(m, H * dim))
        want.append(o[n - m:].reshape(m, H * vdim))
        slots += [s] * m
        positions += list(range(n - m, n))
    q_all = torch.cat(qs).to(dtype).cuda()
    T = q_all.shape[0]
    out = torch.zeros(T, H * vdim + 8, dtype=dtype, device="cuda")
    gate = torch.cat(gate_rows).to(dtype).cuda() if sigmoid else None
    pbd = pb.cuda()
    ws = torch.empty(1 << 20, device="cuda")
    if tc:
        tiles, t0 = [], 0
        while t0 < T:
            t1 = t0 + 1
            while t1 < T and t1 - t0 < 128 and slots[t1] == slots[t0]:
                t1 += 1
            tiles += [t0, t1 - t0, slots[t0], positions[t0]]
            t0 = t1
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        cabi.check(L.pg_attention_ragged_tc_ex(
            out.data_ptr(), H * vdim + 8, q_all.data_ptr(), H * dim, None if gate is None else gate.data_ptr(), H,
            1 if sigmoid else 0, pg.k.data_ptr(), pg.v.data_ptr(), pg.k.shape[0] * PAGE, pg.table.data_ptr(), pg.max_pages,
            PAGE, _i32(tiles).data_ptr(), len(tiles) // 4, T, H, G, dim, vdim, scale, window, keep, None,
            1 if sigmoid else 0, pbd.data_ptr() if sigmoid else None, 0.65 if sigmoid else 1.0, err.data_ptr(), CT[dtype], st))
        torch.cuda.synchronize()
        assert int(err) == 0
        return out[:, :H * vdim].float(), torch.cat(want)
    cabi.check(L.pg_attention_ragged_ex(
        out.data_ptr(), H * vdim + 8, q_all.data_ptr(), H * dim, None if gate is None else gate.data_ptr(), H,
        1 if sigmoid else 0, pg.k.data_ptr(), pg.v.data_ptr(), pg.table.data_ptr(), pg.max_pages, PAGE,
        _i32(slots).data_ptr(), _i32(positions).data_ptr(), T, H, G, dim, vdim, scale, window, keep, None,
        1 if sigmoid else 0, pbd.data_ptr() if sigmoid else None, 0.65 if sigmoid else 1.0, ws.data_ptr(), ws.numel(),
        CT[dtype], st))
    torch.cuda.synchronize()
    return out[:, :H * vdim].float(), torch.cat(want)


@pytest.mark.parametrize("H,G,dim,vdim", [(4, 2, 8, 16), (6, 1, 12, 20), (2, 2, 64, 32), (8, 2, 32, 40), (8, 1, 16, 128)])
@pytest.mark.parametrize("window,keep", [(0, 0), (5, 0), (5, 3), (3, 7), (64, 4), (75, 5), (130, 70), (1, 1)])
def test_windowed_attention_with_kept_first_tokens(H, G, dim, vdim, window, keep):
    # prompt portions that start in the middle of a page and single decoded tokens far into their sequences
    got, want = _attention_case(H, G, dim, vdim, window, keep, lens=[150, 1, 201, 66], new=[40, 1, 1, 2], sigmoid=False)
    _rows_close(got, want, 2e-5)


@pytest.mark.parametrize("window,keep", [(5, 3), (75, 5), (100, 64), (70, 0)])
@pytest.mark.parametrize("where", ["window_in", "window_out", "first_in", "first_out"])
@pytest.mark.parametrize("decode", [True, False])
def test_a_towering_key_at_every_edge(window, keep, where, decode):
    """The last query's score for ONE key is far above the rest: just inside / outside the window, the last kept
    first token / the one after it.  A mask that is off by one changes the result completely."""
    tower = {"window_in": lambda i: i - window + 1, "window_out": lambda i: i - window,
             "first_in": lambda i: keep - 1, "first_out": lambda i: keep}[where]
    for n in (window + keep + 9, 257):
        got, want = _attention_case(8, 2, 16, 24, window, keep, lens=[n, 90], new=[1 if decode else min(33, n), 1], sigmoid=False,
                                    tower=tower, seed=n)
        _rows_close(got, want, 2e-5)


@pytest.mark.parametrize("H,G,dim,vdim", [(4, 2, 8, 16), (3, 3, 12, 20), (8, 2, 64, 64), (8, 8, 16, 32)])
def test_sigmoid_attention_head_bias_head_gate(H, G, dim, vdim):
    got, want = _attention_case(H, G, dim, vdim, 0, 0, lens=[150, 1, 300, 66], new=[40, 1, 1, 2], sigmoid=True)
    _rows_close(got, want, 2e-5)
    got, want = _attention_case(H, G, dim, vdim, 0, 0, lens=[700], new=[1], sigmoid=True, tower=lambda i: 3)
    _rows_close(got, want, 2e-5)


@pytest.mark.parametrize("H,G,dim,vdim", [(4, 2, 64, 128), (2, 1, 128, 64), (2, 2, 64, 64)])
@pytest.mark.parametrize("window,keep", [(0, 0), (100, 3), (70, 66), (64, 130), (200, 0), (5, 1)])
@pytest.mark.parametrize("sigmoid", [False, True])
def test_tensor_core_attention_portions_windows_kept_tokens(H, G, dim, vdim, window, keep, sigmoid):
    """16-bit prompt portions on the tcgen05 kernel: a portion that starts in the middle of a page and a window, a
    two-token portion and single tokens in one launch; softmax weights are rounded to 16 bits as the operand of P V."""
    if sigmoid and (window or keep):
        pytest.skip("the sigmoid attention of this design is unmasked")
    got, want = _attention_case(H, G, dim, vdim, window, keep, lens=[300, 1, 150, 66], new=[200, 1, 40, 2], sigmoid=sigmoid,
                                dtype=torch.bfloat16, tc=True)
    _rows_close(got, want, 2e-2)


@pytest.mark.parametrize("window,keep", [(75, 5), (100, 64), (70, 0), (130, 65)])
@pytest.mark.parametrize("where", ["window_in", "window_out", "first_in", "first_out"])
def test_tensor_core_attention_towering_key_at_every_edge(window, keep, where):
    tower = {"window_in": lambda i: i - window + 1, "window_out": lambda i: i - window,
             "first_in": lambda i: keep - 1, "first_out": lambda i: keep}[where]
    for n in (window + keep + 9, 257, 400):
        got, want = _attention_case(4, 2, 64, 64, window, keep, lens=[n, 90], new=[min(150, n), 1], sigmoid=False,
                                    dtype=torch.bfloat16, tower=tower, seed=n, tc=True)
        _rows_close(got, want, 2e-2)


@pytest.mark.parametrize("heads,dim,lora", [(3, 8, 6), (1, 44, 12), (2, 64, 5), (2, 100, 8), (1, 130, 4)])
def test_delta_rule_prep_recurrence_head_norm(heads, dim, lora):
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(11)
    nd = heads * dim
    lens = [19, 1, 30]                               # three sequences in one step, in slots 2, 0, 3
    slot_of = [2, 0, 3]
    T = sum(lens)
    ld = 5 * nd + lora + 4
    proj = torch.randn(T, ld, generator=g)
    w2, w0, ab = torch.randn(nd, lora, generator=g), torch.randn(nd, generator=g), torch.randn(nd, generator=g)
    nw, gate_w = 1 + 0.1 * torch.randn(nd, generator=g), None
    c_r, c_k, c_v, c_g, c_a, c_l = 0, nd, 2 * nd, 3 * nd, 4 * nd, 5 * nd
    state0 = torch.randn(4, heads, dim, dim, generator=g) * 0.3
    state = state0.clone().cuda()
    projd = proj.cuda()
    o = torch.empty(T, nd, device="cuda")
    rec = torch.empty(int(L.pg_delta_record_floats(T, heads, dim)), device="cuda")
    dw = [t.cuda() for t in (w2, w0, ab, nw)]
    cabi.check(L.pg_delta_prep(rec.data_ptr(), projd.data_ptr(), ld, c_r, c_k, c_v, c_a, c_l, lora, dw[0].data_ptr(),
                               dw[1].data_ptr(), dw[2].data_ptr(), T, heads, dim, math.exp(-0.5), 1e-6, cabi.PG_F32, st))
    segs, row = [], 0
    for s, n in zip(slot_of, lens):
        segs += [s, row, n]
        row += n
    segs += [0, 0, 0]                                # a padded empty segment leaves slot 0 alone
    cabi.check(L.pg_delta_rule(o.data_ptr(), state.data_ptr(), rec.data_ptr(), _i32(segs).data_ptr(), len(segs) // 3, heads,
                               dim, st))
    out = torch.zeros(T, nd + 8, device="cuda")
    cabi.check(L.pg_headnorm_gate(out.data_ptr(), nd + 8, o.data_ptr(), dw[3].data_ptr(), projd[:, c_g:].data_ptr(), ld, T,
                                  heads, dim, 1e-4, 1.3, cabi.PG_F32, st))
    p64 = proj.to(F64)
    w = torch.exp(-math.exp(-0.5) * O.sigmoid(O.lin(w2, torch.tanh(p64[:, c_l:c_l + lora])) + w0.to(F64)))
    a = O.sigmoid(p64[:, c_a:c_a + nd] + ab.to(F64))
    dp = (dim + 3) // 4 * 4
    recs = rec.view(T, heads, 6, dp)                 # [r | k | w | u | a*u | v], padded columns zero
    _close(recs[:, :, 2, :dim], w.reshape(T, heads, dim), 1e-6)
    assert dp == dim or float(recs[..., dim:].abs().max()) == 0.0
    row = 0
    for s, n in zip(slot_of, lens):
        sl = slice(row, row + n)
        view = lambda t: t[sl].reshape(n, heads, dim)
        want_o, want_S = O.delta_rule(view(p64[:, c_r:c_r + nd]), view(p64[:, c_k:c_k + nd]), view(p64[:, c_v:c_v + nd]),
                                      view(w), view(a), state0[s].to(F64))
        _close(o[sl], want_o.reshape(n, nd), 2e-5)
        _close(state[s], want_S, 2e-5)
        want = O.rms_norm(want_o, None, 1e-4).reshape(n, nd) * nw.to(F64) * O.sigmoid(p64[sl, c_g:c_g + nd]) * 1.3
        _close(out[sl, :nd], want, 2e-5)
        row += n
    assert torch.equal(state[1].cpu(), state0[1])    # a slot without tokens keeps its state


# ------------------------------------------------------------------ whole models
SC = (4.0, 64, 16.0, 1.0)
CONFIGS = {
    "small": O.make_config(layers=[
        O.layer(O.attn(window=9, keep_first=2)), O.layer(O.parallel()), O.layer(O.attn(window=9, keep_first=2)),
        O.layer(O.attn(window=30, keep_first=0, v_mix=False), 0)]),
    # a recurrent layer first, two of them, full attention without a mask, rotation of the whole head, no grouping
    "parallel_first": O.make_config(width=64, vocab=80, eps=1e-3, layers=[
        O.layer(O.parallel(heads=2, kv_heads=2, dim=16, vdim=16, rot_dims=16, r_heads=1, r_dim=40, left_scale=1.0, right_scale=1.0), 0),
        O.layer(O.attn(heads=4, kv_heads=4, dim=16, vdim=16, rot_dims=16, window=0, v_mix=False), 72),
        O.layer(O.parallel(heads=4, kv_heads=1, dim=8, vdim=24, rot_dims=2, scaling=(8.0, 32, 4.0, 2.0), r_heads=4, r_dim=16), 24)]),
    # sizes off every vector width, one key/value head under six query heads, more kept tokens than the window
    "odd": O.make_config(width=52, vocab=67, layers=[
        O.layer(O.attn(heads=6, kv_heads=1, dim=12, vdim=20, rot_dims=6, window=3, keep_first=5, v_mix=False), 20),
        O.layer(O.attn(heads=3, kv_heads=3, dim=10, vdim=6, rot_dims=0, window=70, keep_first=1)),
        O.layer(O.parallel(heads=3, kv_heads=1, dim=12, vdim=20, rot_dims=0, r_heads=1, r_dim=20), 36),
        O.layer(O.attn(heads=9, kv_heads=3, dim=4, vdim=6, rot_dims=4, window=1, keep_first=0))]),
    # head sizes of real models: 64 / 128 wide keys and values, 64 and 128 wide recurrent heads
    "wide": O.make_config(width=128, vocab=120, layers=[
        O.layer(O.attn(heads=4, kv_heads=2, dim=64, vdim=128, rot_dims=32, scale=0.12, window=100, keep_first=3), 64),
        O.layer(O.parallel(heads=2, kv_heads=1, dim=128, vdim=64, scale=0.09, rot_dims=64, r_heads=2, r_dim=64), 64),
        O.layer(O.attn(heads=4, kv_heads=2, dim=64, vdim=128, rot_dims=32, scale=0.12, window=70, keep_first=66), 0),
        O.layer(O.parallel(heads=2, kv_heads=2, dim=64, vdim=64, scale=0.12, rot_dims=16, r_heads=1, r_dim=128), 32)]),
    # nothing a multiple of anything: odd width, odd head sizes, one recurrent head of odd size, decay rank 1
    "ragged_sizes": O.make_config(width=50, vocab=33, eps=1e-6, layers=[
        O.layer(O.parallel(heads=5, kv_heads=5, dim=9, vdim=7, rot_dims=4, scaling=(2.0, 16, 3.0, 0.7), r_heads=1, r_dim=9,
                           left_scale=1.7, right_scale=0.2), 19),
        O.layer(O.attn(heads=5, kv_heads=1, dim=7, vdim=3, rot_dims=6, window=65, keep_first=64, v_mix=False), 0)]),
    # a width at which the 16-bit run crosses the tensor-core GEMM kernels (fused projections, GeGLU epilogue, split-K)
    "mid": O.make_config(width=384, vocab=600, layers=[
        O.layer(O.attn(heads=6, kv_heads=2, dim=64, vdim=64, rot_dims=64, scale=0.12, window=80, keep_first=2), 1024),
        O.layer(O.parallel(heads=6, kv_heads=3, dim=64, vdim=64, scale=0.1, rot_dims=32, r_heads=6, r_dim=64), 1024),
        O.layer(O.attn(heads=6, kv_heads=2, dim=64, vdim=64, rot_dims=64, scale=0.12, window=80, keep_first=2), 1024)]),
}
LORA = {"small": 6, "parallel_first": 16, "odd": 3, "wide": 32, "ragged_sizes": 1, "mid": 24}
_ORACLE_CACHE = {}


def _oracle(name, n, seed=0):
    """(tokens, logits, residual stream after every layer) of `n` random tokens (token seed `seed`; weights seed 0)."""
    key = (name, n, seed)
    if key not in _ORACLE_CACHE:
        cfg = CONFIGS[name]
        ck = O.make_checkpoint(cfg, 0, lora=LORA[name])
        toks = _tokens(n, cfg["vocab"], 100 + seed)
        sink = []
        _ORACLE_CACHE[key] = (toks, O.forward(cfg, ck, toks, sink), sink)
    return _ORACLE_CACHE[key]


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_logits_and_every_layer(name, dtype):
    n = 150
    toks, want, layers = _oracle(name, n)
    eng, _ = _engine(CONFIGS[name], dtype=dtype, lora=LORA[name])
    b = eng.new_batcher(slots=2)
    b.admit("a")
    sink = []
    got = b.run_entries([("a", toks, list(range(n)))], layer_sink=sink)
    eng.check_errors(sync=True)
    assert len(sink) == len(layers)
    for x, ref in zip(sink, layers):
        _rows_close(x, ref, TOL[dtype], STRAY[dtype])
    _rows_close(got, want, TOL[dtype] * 2, STRAY[dtype])
    b.close()


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_then_token_by_token_and_portions(name, dtype):
    n = 150
    toks, want, _ = _oracle(name, n)
    eng, _ = _engine(CONFIGS[name], dtype=dtype, lora=LORA[name], pool_tokens=448)
    b = eng.new_batcher(slots=2)
    # most of it in one step, the rest one by one
    b.admit("a")
    rows = [b.run_entries([("a", toks[:100], [99])])]
    rows += [b.run_entries([("a", [t], [0])]) for t in toks[100:]]
    _rows_close(torch.cat(rows), want[99:], TOL[dtype] * 2, STRAY[dtype])
    b.finish("a")
    # portions of changing size, down to two tokens and single ones, cut inside pages and windows
    b.admit("b")
    at, got = 0, []
    for size in [2, 37, 2, 1, 31, 13, 1, 1, 2, 50, 3, 7]:
        got.append(b.run_entries([("b", toks[at:at + size], list(range(size)))]))
        at += size
    assert at == n
    _rows_close(torch.cat(got), want, TOL[dtype] * 2, STRAY[dtype])
    eng.check_errors(sync=True)
    b.close()


@pytest.mark.parametrize("name", ["small", "odd", "wide"])
def test_unequal_requests_in_one_batch_with_slots_and_pages_used_again(name):
    cfg = CONFIGS[name]
    lens = {"a": 131, "b": 23, "c": 97, "d": 150, "e": 70}
    ref = {k: _oracle(name, n, seed=i) for i, (k, n) in enumerate(lens.items())}
    eng, _ = _engine(cfg, lora=LORA[name], pool_tokens=6 * PAGE)          # a pool that forces pages to be handed on
    b = eng.new_batcher(slots=3)
    fed = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    plan = [  # portions of some beside single tokens of others; b, c end early and d, e take over their slots and pages
        [("a", 64), ("b", 21), ("c", 2)], [("a", 3), ("b", 1), ("c", 90)], [("a", 1), ("b", 1), ("c", 1)],
        [("a", 60), ("c", 1)], [("c", 1), ("a", 1)], [("c", 2)], [("a", 2), ("d", 65)], [("d", 2), ("e", 64)],
        [("d", 80), ("e", 1)], [("e", 5), ("d", 1)], [("d", 2)]]
    for step in plan:
        entries = []
        for k, n in step:
            if k not in b.slot_of:
                b.admit(k)
            entries.append((k, ref[k][0][fed[k]:fed[k] + n], list(range(n))))
            fed[k] += n
        out = b.run_entries(entries)
        at = 0
        for k, n in step:
            got[k].append(out[at:at + n])
            at += n
        for k, _ in step:
            if fed[k] == lens[k] and k in b.slot_of:
                b.finish(k)
    eng.check_errors(sync=True)
    for k in lens:
        assert fed[k] == lens[k]
        _rows_close(torch.cat(got[k]), ref[k][1], TOL[torch.float32] * 2)
    b.close()
    assert eng.pages_in_use() == 0


def test_long_decoding_through_windows_pages_and_state():
    name, n = "small", 330
    toks, want, _ = _oracle(name, n)
    for dtype in (torch.float32, torch.bfloat16):
        eng, _ = _engine(CONFIGS[name], dtype=dtype, lora=LORA[name])
        b = eng.new_batcher(slots=1)
        b.admit("a")
        rows = [b.run_entries([("a", toks[:5], list(range(5)))])]
        rows += [b.run_entries([("a", [t], [0])]) for t in toks[5:]]
        _rows_close(torch.cat(rows), want, TOL[dtype] * 2, STRAY[dtype])
        b.close()


def test_greedy_generation_through_the_scheduler():
    name = "small"
    cfg = CONFIGS[name]
    ck = O.make_checkpoint(cfg, 0, lora=LORA[name])
    eng, _ = _engine(cfg, lora=LORA[name])
    prompts = [_tokens(n, cfg["vocab"], 40 + n) for n in (3, 70, 18)]
    b = eng.new_batcher(slots=2, token_budget=32)
    rids = [b.submit(p, max_new_tokens=6) for p in prompts]
    done = b.run()
    for rid, p in zip(rids, prompts):
        seq = list(p)
        for _ in range(6):                                     # the oracle's own greedy loop
            seq.append(int(O.forward(cfg, ck, seq)[-1].argmax()))
        assert done[rid].tokens == seq[len(p):]
    b.close()
    assert eng.pages_in_use() == 0
    # the framework's top-p kernel on the same scheduler: tokens of the vocabulary, the same seed gives the same tokens
    runs = []
    for _ in range(2):
        b = eng.new_batcher(slots=2, token_budget=32, do_sample=True, temperature=0.9, top_p=0.8, seed=5)
        rids = [b.submit(p, max_new_tokens=5) for p in prompts[:2]]
        done = b.run()
        runs.append([done[r].tokens for r in rids])
        b.close()
    assert runs[0] == runs[1] and all(0 <= t < cfg["vocab"] for seq in runs[0] for t in seq)
    assert all(len(seq) == 5 for seq in runs[0])


def test_model_folder_through_the_registry(tmp_path):
    from pg_b200.checkpoint import write_safetensors
    from pg_b200.registry import load_engine
    cfg = CONFIGS["odd"]
    ck = O.make_checkpoint(cfg, 3, lora=LORA["odd"])
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "model.safetensors"), ck)
    eng = load_engine(str(tmp_path), device="cuda:0", dtype=torch.float32, kv_pool_tokens=256)
    assert type(eng).__name__ == "NinisunEngine"
    toks = _tokens(40, cfg["vocab"], 9)
    b = eng.new_batcher(slots=1)
    b.admit(0)
    _rows_close(b.run_entries([(0, toks, [39, 0])]), O.forward(cfg, ck, toks)[[39, 0]], 1e-4)
    b.close()
    more = dict(ck)
    more["l0.mix.extra"] = torch.zeros(3)                  # a tensor the config does not call for: reported, or refused
    with pytest.warns(UserWarning):
        type(eng)(cfg, more, device="cuda:0", dtype=torch.float32, kv_pool_tokens=64)
    with pytest.raises(ValueError):
        type(eng)(cfg, more, device="cuda:0", dtype=torch.float32, kv_pool_tokens=64, strict=True)
    less = {k: v for k, v in ck.items() if k != "l1.mix.q"}
    with pytest.raises(KeyError):
        type(eng)(cfg, less, device="cuda:0", dtype=torch.float32, kv_pool_tokens=64)
    wrong = dict(ck)
    wrong["l1.mix.q"] = torch.zeros(5, cfg["width"])
    with pytest.raises(ValueError):
        type(eng)(cfg, wrong, device="cuda:0", dtype=torch.float32, kv_pool_tokens=64)


def test_command_line_replay_and_generation(tmp_path):
    """bin/trace_run replays a schedule (portions beside single tokens, a slot handed on) and bin/generate generates,
    both on a model folder picked up through the registry."""
    import subprocess
    import sys
    import numpy as np
    from pg_b200.checkpoint import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = CONFIGS["small"]
    ck = O.make_checkpoint(cfg, 0, lora=LORA["small"])
    model = tmp_path / "model"
    model.mkdir()
    with open(model / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(model / "model.safetensors"), ck)
    seq = {k: _tokens(n, cfg["vocab"], 60 + n) for k, n in (("a", 22), ("b", 5), ("c", 70))}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": seq["a"][:20], "want": [19]}, {"id": "b", "tokens": seq["b"], "want": [0, 4]}],
         "end": ["b"]},
        {"step": 1, "entries": [{"id": "a", "tokens": seq["a"][20:21], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "c", "tokens": seq["c"], "want": [69]}, {"id": "a", "tokens": seq["a"][21:], "want": [0]}],
         "end": ["a", "c"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()                      # nothing was asked for in step 1
    ref = {k: O.forward(cfg, ck, v) for k, v in seq.items()}
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, cfg["vocab"]))
    _rows_close(got0, torch.stack([ref["a"][19], ref["b"][0], ref["b"][4]]), 1e-4)
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    _rows_close(got2, torch.stack([ref["c"][69], ref["a"][21]]), 1e-4)
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "generate"), "--model", str(model), "--dtype", "float32",
                        "--prompt-ids", ",".join(map(str, seq["b"])), "--prompt-ids", ",".join(map(str, seq["a"])),
                        "--max-new-tokens", "4", "--max-tokens", "256", "--slots", "2"], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    for i, key in enumerate(("b", "a")):
        s = list(seq[key])
        for _ in range(4):
            s.append(int(O.forward(cfg, ck, s)[-1].argmax()))
        assert lines[i] == {"request": i, "tokens": s[len(seq[key]):]}

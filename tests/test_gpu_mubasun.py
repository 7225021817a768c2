"""Mubasun on the GPU against the plain float64 oracle (tests/mubasun_oracle.py): every mechanism alone through the
C ABI, then whole models of several shapes through the engine, the slot cache and the scheduler."""
import math

import pytest
import torch

import mubasun_oracle as O

pytestmark = pytest.mark.gpu
F64 = torch.float64


def _engine(cfg, seed=0, dtype=torch.float32, pool_tokens=1024, **kw):
    from pg_b200.mubasun import MubasunEngine
    ck = O.make_checkpoint(cfg, seed)
    return MubasunEngine(cfg, ck, device="cuda:0", dtype=dtype, kv_pool_tokens=pool_tokens, **kw), O.Oracle(cfg, ck)


def _close(got, want, rel):
    """rms of the difference against the rms of the reference."""
    got, want = got.detach().cpu().to(F64), want.to(F64)
    err = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt().clamp_min(1e-30))
    assert err <= rel, f"relative rms error {err:.3g} > {rel}"


def _rows_close(got, want, rel, stray=0.0):
    """Every row within `rel` (relative rms).  stray > 0 (16-bit runs of models with routers): that fraction of the
    rows may differ, because rounding the router's input can flip a near tie between two experts."""
    got, want = got.detach().cpu().to(F64), want.to(F64)
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)
    bad = int((err > rel).sum())
    assert bad <= stray * err.numel(), \
        f"{bad} of {err.numel()} rows over {rel}: worst relative rms error {float(err.max()):.3g} (row {int(err.argmax())})"


_KEEP = []


def _dev(t):
    """Device copy that outlives the asynchronous launch it is passed to."""
    _KEEP.append(t.cuda())
    del _KEEP[:-64]
    return _KEEP[-1]


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


TOL = {torch.float32: 2e-5, torch.bfloat16: 4e-2}

SMALL = O.make_config(layers=[O.layer(O.attn(), O.dense()), O.layer(O.attn(window=9), O.moe()),
                              O.layer(O.attn(window=9, kv_from=1), O.moe(top=1, identity=0, shared=0))])

# shapes that differ in everything a checkpoint can vary: head grouping, key vs value width, norm groups, windows,
# layer order, feed-forward kinds, expert counts, shared / identity experts, cache sharing
CONFIGS = {
    "small": SMALL,
    "mha_equal_dims": O.make_config(width=64, groups=1, vocab=80, layers=[
        O.layer(O.attn(heads=4, kv_heads=4, dim=16, vdim=16, window=0), None),
        O.layer(O.attn(heads=4, kv_heads=4, dim=16, vdim=16, window=33, kv_from=0), O.dense(72))]),
    "mqa_wide_values": O.make_config(width=40, groups=5, vocab=120, eps=1e-3, layers=[
        O.layer(O.attn(heads=6, kv_heads=1, dim=8, vdim=24, window=17, scale=0.5), O.moe(experts=3, identity=2, top=3, ff=16)),
        O.layer(O.attn(heads=2, kv_heads=2, dim=24, vdim=8, window=70), O.moe(experts=9, identity=0, top=2, ff=8, shared=0)),
        O.layer(O.attn(heads=6, kv_heads=1, dim=8, vdim=24, window=5, kv_from=0), O.dense(16)),
        O.layer(O.attn(heads=2, kv_heads=2, dim=24, vdim=8, window=1, kv_from=1), None)]),
    "wide_heads": O.make_config(width=64, groups=2, vocab=72, max_positions=512, layers=[   # the tensor-core attention's sizes
        O.layer(O.attn(heads=2, kv_heads=1, dim=64, vdim=128, window=100, scale=0.12), O.dense(32)),
        O.layer(O.attn(heads=2, kv_heads=1, dim=64, vdim=128, window=0, scale=0.12, kv_from=0), O.moe(experts=4, top=2, ff=16))]),
    "odd_head_dim": O.make_config(width=56, groups=7, vocab=64, layers=[
        O.layer(O.attn(heads=3, kv_heads=3, dim=12, vdim=20, window=40, scale=1.0), O.moe(experts=2, identity=1, top=1, ff=32, shared=8)),
        O.layer(O.attn(heads=8, kv_heads=2, dim=4, vdim=36, window=3), O.dense(24))]),
}


# ------------------------------------------------------------------ mechanisms alone (C ABI)
def _lib():
    from pg_b200 import _cabi as cabi
    return cabi, cabi.lib(), cabi.stream()


@pytest.mark.parametrize("groups,D", [(1, 48), (3, 48), (4, 64), (8, 8)])
def test_group_rmsnorm_and_residual_sum(groups, D):
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, D, generator=g) * 3
    a, b, w = torch.randn(7, D, generator=g), torch.randn(7, D, generator=g), torch.randn(D, generator=g)
    xd, out = x.cuda(), torch.empty(7, D, device="cuda")
    cabi.check(L.pg_group_rmsnorm(out.data_ptr(), xd.data_ptr(), _dev(a).data_ptr(), D, _dev(b).data_ptr(), D,
                                  _dev(w).data_ptr(), None, 7, D, groups, 1e-2, cabi.PG_F32, st))
    s = x.to(F64) + a.to(F64) + b.to(F64)
    _close(xd, s, 1e-6)                                               # the sum is written back in fp32
    _close(out, O.group_rms_norm(s, w.to(F64), groups, 1e-2), 1e-5)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")    # packed output of picked rows, no sum
    out2 = torch.empty(3, D, device="cuda")
    cabi.check(L.pg_group_rmsnorm(out2.data_ptr(), xd.data_ptr(), None, 0, None, 0, _dev(w).data_ptr(), rows.data_ptr(),
                                  3, D, groups, 1e-2, cabi.PG_F32, st))
    _close(out2, O.group_rms_norm(s[[5, 0, 5]], w.to(F64), groups, 1e-2), 1e-5)


def test_xielu_both_branches():
    cabi, L, st = _lib()
    z = torch.linspace(-6, 6, 241)
    for p, q in ((0.3, -1.2), (-2.0, 2.5)):
        pq = torch.tensor([p, q]).cuda()
        out = torch.empty_like(z).cuda()
        cabi.check(L.pg_xielu(out.data_ptr(), _dev(z).data_ptr(), pq.data_ptr(), z.numel(), cabi.PG_F32, st))
        _close(out, O.xielu(z.to(F64), p, q), 1e-5)


def _attention_case(H, G, dim, vdim, window, scale, positions, seq_len, page_size=8, dtype=torch.float32, k_boost=None,
                    use_ws=True):
    """One sequence whose cache rows are scattered over shuffled pages; queries at `positions`."""
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(3)
    n = len(positions)
    q = torch.randn(n, H * dim, generator=g)
    kc, vc = torch.randn(seq_len, G * dim, generator=g), torch.randn(seq_len, G * vdim, generator=g)
    gate = torch.randn(n, H * vdim, generator=g)
    if k_boost is not None:                 # make one (query, key) score stand out: the key is seen or it is not
        qi, kj = k_boost
        kc[kj] = 0
        kc[kj, :dim] = q[qi, :dim] * 4 / (q[qi, :dim].norm() ** 2 * scale) * 6
        vc[kj] = 50.0
    q, kc, vc, gate = (t.to(dtype) for t in (q, kc, vc, gate))
    n_pages = (seq_len + page_size - 1) // page_size
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    kp = torch.zeros(n_pages + 3, page_size, G * dim, dtype=dtype)
    vp = torch.zeros(n_pages + 3, page_size, G * vdim, dtype=dtype)
    for j in range(seq_len):
        kp[perm[j // page_size], j % page_size] = kc[j]
        vp[perm[j // page_size], j % page_size] = vc[j]
    table = torch.zeros(2, n_pages, dtype=torch.int32)
    table[1] = perm.to(torch.int32)
    slot = torch.ones(n, dtype=torch.int32)
    pos = torch.tensor(positions, dtype=torch.int32)
    slopes = torch.tensor(O.head_slopes(H), dtype=torch.float32)
    out = torch.empty(n, H * vdim, dtype=dtype, device="cuda")
    ws = torch.empty(1 << 20, dtype=torch.float32, device="cuda") if use_ws else None
    dev = [t.cuda() for t in (q, gate, kp, vp, table, slot, pos, slopes)]
    cabi.check(L.pg_attention_ragged(out.data_ptr(), H * vdim, dev[0].data_ptr(), H * dim, dev[1].data_ptr(), H * vdim,
                                     dev[2].data_ptr(), dev[3].data_ptr(), dev[4].data_ptr(), n_pages, page_size,
                                     dev[5].data_ptr(), dev[6].data_ptr(), n, H, G, dim, vdim, scale, window,
                                     dev[7].data_ptr(), ws.data_ptr() if ws is not None else None,
                                     0 if ws is None else ws.numel(), cabi.DTYPE_CODE[dtype], st))
    want = O.window_attention(q.to(F64), kc.to(F64), vc.to(F64), positions, H, G, dim, vdim, scale, window)
    return out, want * torch.sigmoid(gate.to(F64))


@pytest.mark.parametrize("H,G,dim,vdim", [(4, 2, 8, 16), (3, 3, 12, 20), (8, 1, 4, 36), (2, 2, 64, 64), (1, 1, 40, 72)])
@pytest.mark.parametrize("window", [0, 1, 7, 32, 33, 200])
def test_attention_windows_and_head_layouts(H, G, dim, vdim, window):
    positions = [0, 1, 2, 6, 7, 8, 31, 32, 33, 63, 64, 65, 99]      # first tokens, page borders (8), window edges
    out, want = _attention_case(H, G, dim, vdim, window, 0.37, positions, 100)
    _rows_close(out, want, 2e-5)


@pytest.mark.parametrize("n_queries", [1, 3])           # a handful of tokens: the split kernel of decode steps
def test_attention_decode_sized_batches(n_queries):
    out, want = _attention_case(4, 2, 16, 16, 150, 0.2, [299, 150, 64][:n_queries], 300)
    _rows_close(out, want, 2e-5)
    for dims in ((2, 1, 32, 64), (2, 2, 16, 128), (1, 1, 8, 256), (3, 1, 8, 72)):     # vector loads of the value rows
        out, want = _attention_case(*dims, 0, 0.2, [1499, 700, 64][:n_queries], 1500, page_size=64)   # key slices + merge
        _rows_close(out, want, 2e-5)
        out, want = _attention_case(*dims, 0, 0.2, [1499, 700, 64][:n_queries], 1500, page_size=64, use_ws=False)
        _rows_close(out, want, 2e-5)
    out, want = _attention_case(4, 2, 16, 16, 0, 0.2, [299, 150, 64][:n_queries], 300, dtype=torch.bfloat16)
    _rows_close(out, want, 2e-2)


def _tc_attention_case(H, G, dim, vdim, window, segments, seed=4):
    """segments: (start position, count) runs of one sequence each (slot = run index + 1, own shuffled pages)."""
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(seed)
    ps, dtype = 64, torch.bfloat16
    n = sum(c for _, c in segments)
    q = torch.randn(n, H * dim, generator=g).to(dtype)
    gate = torch.randn(n, H * vdim, generator=g).to(dtype)
    max_len = max(s0 + c for s0, c in segments)
    pages_per = (max_len + ps - 1) // ps
    n_pages = pages_per * len(segments) + 2
    perm = torch.randperm(n_pages, generator=g)
    kp, vp = torch.zeros(n_pages, ps, G * dim, dtype=dtype), torch.zeros(n_pages, ps, G * vdim, dtype=dtype)
    table = torch.zeros(len(segments) + 1, pages_per, dtype=torch.int32)
    tiles, want, row = [], [], 0
    for si, (s0, c) in enumerate(segments):
        kc = torch.randn(s0 + c, G * dim, generator=g).to(dtype)
        vc = torch.randn(s0 + c, G * vdim, generator=g).to(dtype)
        pg = perm[si * pages_per:(si + 1) * pages_per]
        table[si + 1] = pg.to(torch.int32)
        for j in range(s0 + c):
            kp[pg[j // ps], j % ps], vp[pg[j // ps], j % ps] = kc[j], vc[j]
        pos = list(range(s0, s0 + c))
        want.append(O.window_attention(q[row:row + c].to(F64), kc.to(F64), vc.to(F64), pos, H, G, dim, vdim, 0.11, window))
        for a in range(0, c, 128):
            tiles += [row + a, min(128, c - a), si + 1, s0 + a]
        row += c
    want = torch.cat(want) * torch.sigmoid(gate.to(F64))
    out = torch.zeros(n, H * vdim, dtype=dtype, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    d = [_dev(t) for t in (q, gate, kp, vp, table, torch.tensor(tiles, dtype=torch.int32),
                           torch.tensor(O.head_slopes(H), dtype=torch.float32))]
    assert L.pg_attention_ragged_tc_ok(dim, vdim, ps, H * dim, H * vdim, H * vdim, cabi.PG_BF16)
    cabi.check(L.pg_attention_ragged_tc(out.data_ptr(), H * vdim, d[0].data_ptr(), H * dim, d[1].data_ptr(), H * vdim,
                                        d[2].data_ptr(), d[3].data_ptr(), n_pages * ps, d[4].data_ptr(), pages_per, ps,
                                        d[5].data_ptr(), len(tiles) // 4, n, H, G, dim, vdim, 0.11, window, d[6].data_ptr(),
                                        err.data_ptr(), cabi.PG_BF16, st))
    assert int(err) == 0
    return out, want


@pytest.mark.parametrize("H,G,dim,vdim", [(2, 1, 64, 64), (4, 2, 128, 64), (2, 2, 64, 192), (1, 1, 256, 256)])
@pytest.mark.parametrize("window", [0, 1, 64, 65, 130, 700])
def test_tensor_core_attention_windows_tiles_and_portions(H, G, dim, vdim, window):
    """Whole prompts (several query tiles), a portion that starts in the middle of a page and of a window, a portion
    of two tokens, a single decoded token, all in one launch."""
    out, want = _tc_attention_case(H, G, dim, vdim, window, [(0, 300), (190, 135), (63, 2), (500, 1), (0, 1)])
    _rows_close(out, want, 2e-2)


@pytest.mark.parametrize("window,delta,seen", [(25, 24, True), (25, 25, False), (64, 63, True), (64, 64, False),
                                               (130, 129, True), (130, 130, False)])
def test_attention_key_just_inside_or_outside_the_window(window, delta, seen):
    """A key whose score towers over the rest sits `delta` positions back: inside the window it owns the output of
    head 0, one step further it must not be read at all."""
    pos = 290
    out, want = _attention_case(2, 1, 16, 8, window, 0.5, [pos], 300, k_boost=(0, pos - delta))
    _rows_close(out, want, 2e-5)
    gate_free = want[0, :8].abs().max()
    assert (gate_free > 1.0) == seen        # the boosted value row is 50 before the gate: seen or not is unmistakable


def test_router_topk_correction_and_identity_weights():
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(5)
    T_, D, R, top = 33, 24, 7, 3
    h, wr = torch.randn(T_, D, generator=g), torch.randn(R, D, generator=g) * 0.5
    corr, wsg = torch.randn(R, generator=g) * 0.3, torch.randn(D, generator=g) * 0.3
    idx = torch.empty(T_, top, dtype=torch.int32, device="cuda")
    wt = torch.empty(T_, top, dtype=torch.float32, device="cuda")
    sg = torch.empty(T_, dtype=torch.float32, device="cuda")
    cabi.check(L.pg_moe_route(idx.data_ptr(), wt.data_ptr(), sg.data_ptr(), _dev(h).data_ptr(), D, _dev(wr).data_ptr(),
                              _dev(corr).data_ptr(), _dev(wsg).data_ptr(), T_, D, R, top, 1.7, cabi.PG_F32, st))
    widx, wwt = O.route(h.to(F64), wr.to(F64), corr.to(F64), top, 1.7)
    assert idx.cpu().tolist() == widx.tolist()
    _close(wt, wwt, 1e-5)
    _close(sg, torch.sigmoid(h.to(F64) @ wsg.to(F64)), 1e-5)
    # the correction changes the choice, never the weight
    s = torch.softmax(h.to(F64) @ wr.to(F64).t(), -1)
    assert (widx != torch.argsort(s, -1, descending=True)[:, :top]).any()


@pytest.mark.parametrize("dtype,impl", [(torch.float32, 1), (torch.bfloat16, 1), (torch.bfloat16, 2)])
@pytest.mark.parametrize("T_,D,ff", [(150, 64, 32), (700, 200, 120), (5, 72, 264)])
def test_moe_grouped_gemms_and_combine(dtype, impl, T_, D, ff):
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(7)
    E, I, top = 5, 2, 3
    h = torch.randn(T_, D, generator=g).to(dtype)
    gu = (torch.randn(E, 2 * ff, D, generator=g) / math.sqrt(D)).to(dtype)
    dn = (torch.randn(E, D, ff, generator=g) / math.sqrt(ff)).to(dtype)
    idx = torch.stack([torch.randperm(E + I, generator=g)[:top] for _ in range(T_)]).to(torch.int32)
    idx[:T_ // 3, 0] = 2                                       # an expert with many tokens, one with none
    idx[idx == 4] = 3
    wt = torch.rand(T_, top, generator=g)
    x0 = torch.randn(T_, D, generator=g)
    dt = cabi.DTYPE_CODE[dtype]
    d_idx, d_wt, d_h, d_gu, d_dn, x = idx.cuda(), wt.cuda(), h.cuda(), gu.cuda(), dn.cuda(), x0.cuda()
    P = T_ * top
    off = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    rows, pos = torch.empty(P, dtype=torch.int32, device="cuda"), torch.empty(P, dtype=torch.int32, device="cuda")
    cabi.check(L.pg_moe_sort(off.data_ptr(), rows.data_ptr(), pos.data_ptr(), d_idx.data_ptr(), P, top, E, st))
    counts = [(idx == e).sum().item() for e in range(E)]
    assert off.cpu().tolist() == [sum(counts[:e]) for e in range(E + 1)]
    act, y = torch.empty(P, ff, dtype=dtype, device="cuda"), torch.empty(P, D, dtype=dtype, device="cuda")
    a, row_map = d_h, rows.data_ptr()
    if impl == 2:                                              # the tensor-core kernel takes rows in expert order
        a, row_map = torch.zeros(P, D, dtype=dtype, device="cuda"), None
        cabi.check(L.pg_gather_rows(a.data_ptr(), d_h.data_ptr(), D, rows.data_ptr(), off[E:].data_ptr(), P, D, dt, st))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    cabi.check(L.pg_moe_gemm(act.data_ptr(), ff, a.data_ptr(), D, row_map, d_gu.data_ptr(), off.data_ptr(), P, E,
                             ff, D, 1, impl, err.data_ptr(), dt, st))
    cabi.check(L.pg_moe_gemm(y.data_ptr(), D, act.data_ptr(), ff, None, d_dn.data_ptr(), off.data_ptr(), P, E, D, ff, 0,
                             impl, err.data_ptr(), dt, st))
    assert int(err) == 0
    cabi.check(L.pg_moe_combine(x.data_ptr(), y.data_ptr(), D, pos.data_ptr(), d_wt.data_ptr(), d_h.data_ptr(), D, None, 0,
                                None, T_, D, top, dt, st))
    want = x0.to(F64).clone()
    hh = h.to(F64)
    for t in range(T_):
        for k in range(top):
            e = int(idx[t, k])
            o = O.gated_expert(hh[t:t + 1], gu[e, :ff].to(F64), gu[e, ff:].to(F64), dn[e].to(F64))[0] if e < E else hh[t]
            want[t] += float(wt[t, k]) * o
    _rows_close(x - x0.cuda(), want - x0.to(F64), TOL[dtype])


def test_qk_norm_is_over_the_whole_projection_and_append_lands_in_the_right_page():
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(9)
    n, nq, nk, nv, ps = 5, 24, 12, 20, 4
    proj = torch.randn(n, nq + nk + nv + 7, generator=g)
    qw, kw = torch.randn(nq, generator=g), torch.randn(nk, generator=g)
    kp, vp = torch.zeros(6, ps, nk, device="cuda"), torch.zeros(6, ps, nv, device="cuda")
    table = torch.tensor([[5, 1, 3], [2, 0, 4]], dtype=torch.int32)
    slot = torch.tensor([1, 1, 0, 1, 0], dtype=torch.int32)
    pos = torch.tensor([3, 4, 0, 11, 9], dtype=torch.int32)
    q = torch.empty(n, nq, device="cuda")
    cabi.check(L.pg_qknorm_append(q.data_ptr(), _dev(proj).data_ptr(), proj.shape[1], 0, nq, nq, nk, nq + nk, nv,
                                  _dev(qw).data_ptr(), _dev(kw).data_ptr(), 1e-3, kp.data_ptr(), vp.data_ptr(),
                                  _dev(table).data_ptr(), 3, ps, _dev(slot).data_ptr(), _dev(pos).data_ptr(), n,
                                  cabi.PG_F32, st))
    p64 = proj.to(F64)
    _close(q, O.whole_rms_norm(p64[:, :nq], qw.to(F64), 1e-3), 1e-5)
    wk = O.whole_rms_norm(p64[:, nq:nq + nk], kw.to(F64), 1e-3)
    for t in range(n):
        page = int(table[slot[t], pos[t] // ps])
        _close(kp[page, pos[t] % ps], wk[t], 1e-5)
        _close(vp[page, pos[t] % ps], p64[t, nq + nk:nq + nk + nv], 1e-6)
    assert int((kp.abs().sum(-1) > 0).sum()) == n                 # nothing else was written


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_logits_and_layer_streams(name, dtype):
    cfg = CONFIGS[name]
    eng, orc = _engine(cfg, seed=11, dtype=dtype)
    b = eng.new_batcher(slots=2)
    toks = _tokens(200 if name == "wide_heads" else 90, cfg["vocab"], 1)
    b.admit("a")
    sink = []
    got = b.run_entries([("a", toks, list(range(len(toks))))], layer_sink=sink)
    want_layers = []
    want = orc.run(toks, orc.new_cache(), 0, want_layers)
    stray = 0.0 if dtype == torch.float32 else 0.2
    _rows_close(got, want, TOL[dtype], stray)
    for li, (x, wx) in enumerate(zip(sink, want_layers)):
        _rows_close(x, wx, TOL[dtype], stray)
    b.close()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_equals_token_by_token_and_portions(name):
    cfg = CONFIGS[name]
    eng, orc = _engine(cfg, seed=13)
    toks = _tokens(75, cfg["vocab"], 2)
    want = orc.logits(toks)
    b = eng.new_batcher(slots=3)
    b.admit("one")                                     # one token per step from the first token on
    one = torch.cat([b.run_entries([("one", [t], [0])]) for t in toks])
    _rows_close(one, want, 2e-5)
    for key, sizes in (("p2", [2] * 37 + [1]), ("mix", [1, 2, 3, 5, 7, 11, 13, 2, 31])):
        b.admit(key)
        at, parts = 0, []
        for n in sizes:
            parts.append(b.run_entries([(key, toks[at:at + n], list(range(n)))]))
            at += n
        assert at == len(toks)
        _rows_close(torch.cat(parts), want, 2e-5)
    b.close()


MID = O.make_config(width=384, groups=2, vocab=600, max_positions=512, layers=[
    O.layer(O.attn(heads=6, kv_heads=3, dim=64, vdim=64, window=150, scale=0.125), O.dense(640)),
    O.layer(O.attn(heads=6, kv_heads=3, dim=64, vdim=64, window=40, scale=0.125, kv_from=0),
            O.moe(experts=6, identity=1, top=2, ff=128, shared=192)),
    O.layer(O.attn(heads=4, kv_heads=1, dim=128, vdim=64, window=0, scale=0.09), O.moe(experts=3, identity=0, top=1, ff=256, shared=0))])


WIDE = O.make_config(width=1024, groups=8, vocab=1000, max_positions=512, layers=[
    O.layer(O.attn(heads=8, kv_heads=2, dim=128, vdim=128, window=200, scale=0.088), O.moe(experts=4, identity=1, top=2, ff=512, shared=256)),
    O.layer(O.attn(heads=8, kv_heads=2, dim=128, vdim=128, window=64, scale=0.088, kv_from=0), O.dense(2048))])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which", ["mid", "wide"])
def test_mid_size_model_portions_of_every_gemm_regime(dtype, which):
    """Wide enough that the 16-bit run takes every projection path of the library: CTA-pair / single-CTA tiles for
    the whole prompt, the skinny and split-K kernels for portions of 4..128 tokens, the weight-streaming kernel for
    1..3 tokens, the tensor-core attention from 48 tokens on and the CUDA-graph step below 17."""
    cfg = MID if which == "mid" else WIDE
    eng, orc = _engine(cfg, seed=37, dtype=dtype, pool_tokens=1024)
    toks = _tokens(330, cfg["vocab"], 12)
    want = orc.logits(toks)
    stray = 0.0 if dtype == torch.float32 else 0.2
    b = eng.new_batcher(slots=2)
    b.admit("whole")
    _rows_close(b.run_entries([("whole", toks, list(range(len(toks))))]), want, TOL[dtype], stray)
    b.admit("parts")
    at, parts = 0, []
    for n in (5, 17, 64, 100, 3, 48, 1, 2, 70, 4, 16):
        parts.append(b.run_entries([("parts", toks[at:at + n], list(range(n)))]))
        at += n
    assert at == len(toks)
    _rows_close(torch.cat(parts), want, TOL[dtype], stray)
    eng.check_errors(sync=True)
    b.close()


def test_unequal_requests_in_one_batch_equal_each_alone_and_slots_and_pages_are_reused():
    cfg = CONFIGS["small"]
    eng, orc = _engine(cfg, seed=17, pool_tokens=4 * 64)               # four pages for everything
    b = eng.new_batcher(slots=2)
    free0 = len(eng._free)
    reqs = {k: _tokens(n, cfg["vocab"], s) for k, n, s in (("a", 100, 3), ("b", 37, 4), ("c", 129, 5), ("d", 2, 6), ("e", 64, 7))}
    want = {k: orc.logits(v) for k, v in reqs.items()}
    got = {k: [] for k in reqs}

    def run(step):          # step: list of (key, count)
        ents = []
        for k, n in step:
            if k not in b.slot_of:
                b.admit(k)
            lo = b.length(k)
            ents.append((k, reqs[k][lo:lo + n], list(range(n))))
        out = b.run_entries(ents)
        at = 0
        for k, n in step:
            got[k].append(out[at:at + n])
            at += n
            if b.length(k) == len(reqs[k]):
                b.finish(k)

    run([("a", 60), ("b", 1)])                  # a prompt portion beside a first token
    run([("b", 30), ("a", 1)])                  # ... and the other way round
    run([("a", 39), ("b", 6)])                  # both end: their slots and pages go back
    assert len(eng._free) == free0
    run([("c", 100)])                           # takes over pages that a and b used
    run([("c", 1), ("d", 2)])
    run([("c", 28), ("e", 3)])                  # d's slot, again
    run([("e", 61)])
    assert len(eng._free) == free0 and not b.slot_of
    for k in reqs:
        _rows_close(torch.cat(got[k]), want[k], 2e-5)
    b.close()


def test_long_decoding_through_windows_and_page_borders():
    cfg = O.make_config(width=32, groups=2, vocab=50, max_positions=400, layers=[
        O.layer(O.attn(heads=2, kv_heads=1, dim=16, vdim=16, window=70), O.dense(32)),
        O.layer(O.attn(heads=2, kv_heads=1, dim=16, vdim=16, window=130, kv_from=0), O.moe(experts=3, identity=1, top=2, ff=16))])
    eng, orc = _engine(cfg, seed=19, pool_tokens=384)
    toks = _tokens(330, cfg["vocab"], 8)
    want = orc.logits(toks)
    b = eng.new_batcher(slots=1)
    b.admit("s")
    parts = [b.run_entries([("s", toks[:50], list(range(50)))])]
    parts += [b.run_entries([("s", [t], [0])]) for t in toks[50:]]     # 280 single tokens: both windows slide past them
    _rows_close(torch.cat(parts), want, 3e-5)
    b.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_scheduler(dtype):
    cfg = CONFIGS["small"]
    eng, orc = _engine(cfg, seed=23, dtype=dtype, pool_tokens=512)
    b = eng.new_batcher(slots=2, token_budget=16)                     # prompts are read in portions of <= 16 tokens
    prompts = [_tokens(n, cfg["vocab"], 30 + n) for n in (5, 40, 23)]
    rids = [b.submit(p, 12) for p in prompts]
    done = b.run()
    assert len(eng._free) == eng.num_pages - 1                        # all pages back (one is the parking page)
    for rid, p in zip(rids, prompts):
        if dtype == torch.float32:
            assert done[rid].tokens == orc.greedy(p, 12)
        else:   # bf16: teacher-forced comparison (a near tie may flip a token, never the distribution)
            seq = p + done[rid].tokens
            lg = orc.logits(seq[:-1])[len(p) - 1:]
            top2 = lg.topk(2, -1)
            sure = (top2.values[:, 0] - top2.values[:, 1]) > 0.25 * lg.std()
            picks = torch.tensor(done[rid].tokens)
            assert bool((picks[sure] == top2.indices[sure, 0]).all())
    b.close()


def test_sampling_uses_the_framework_sampler_and_eos_frees_the_slot():
    cfg = CONFIGS["small"]
    eng, orc = _engine(cfg, seed=29, pool_tokens=256)
    p = _tokens(9, cfg["vocab"], 40)
    first = orc.greedy(p, 3)
    b = eng.new_batcher(slots=1)
    rid = b.submit(p, 10, eos_token_id=first[1])
    assert b.run()[rid].tokens == first[:2]                           # stops at EOS, EOS included
    b2 = eng.new_batcher(slots=1, do_sample=True, temperature=0.7, top_p=0.9, seed=5)
    r1 = b2.submit(p, 8)
    t1 = b2.run()[r1].tokens
    assert len(t1) == 8 and all(0 <= t < cfg["vocab"] for t in t1)
    b.close(), b2.close()


def test_registry_loads_a_model_folder(tmp_path):
    import json
    from pg_b200.checkpoint import write_safetensors
    from pg_b200.registry import load_engine
    cfg = CONFIGS["odd_head_dim"]
    ck = O.make_checkpoint(cfg, 31)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(tmp_path / "model.safetensors"), ck)
    eng = load_engine(str(tmp_path), device="cuda:0", dtype=torch.float32, kv_pool_tokens=128)
    b = eng.new_batcher(slots=1)
    toks = _tokens(20, cfg["vocab"], 9)
    b.admit(0)
    _rows_close(b.run_entries([(0, toks, [19])]), O.Oracle(cfg, ck).logits(toks)[19:], 2e-5)
    b.close()

"""Galirax on the GPU against the plain float64 statement in galirax_ref.py: every mechanism alone through the C ABI, then whole
models through the loader, the batch step, the sequence cache and the engine (prefill against decoding, portions, mixed
batches, cells and slots that are used again, windows passing over prompts and decoded tokens, greedy generation)."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import pytest

import galirax_ref as R
import koboldcpp_b200.host as H
from koboldcpp_b200.lib import BF16, F32, I32, LinearAttnArgs, QkvStoreArgs, SinkAttnArgs, Tensor, check, lib

pytestmark = pytest.mark.gpu


def dev(a, dtype=np.float32):
    return H.DeviceBuffer.from_numpy(np.ascontiguousarray(a, dtype=dtype), pad=256)


def rel(got, want):
    return float(np.abs(got - want).max() / (np.abs(want).max() + 1e-30))


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("n,rows", [(40, 5), (320, 3), (5000, 2), (20000, 2)])
def test_norm_with_bias_and_output_gate(kind, n, rows):
    rng = np.random.default_rng(n + kind)
    x = rng.standard_normal((rows, n)) * 3 + 0.7
    w, b = 1 + 0.2 * rng.standard_normal(n), rng.standard_normal(n)
    gate, res = rng.standard_normal((rows, n)), rng.standard_normal((rows, n))
    eps = 1e-5
    base = R.layer_norm(x, w, b, eps) if kind == 0 else R.rms_norm(x, w, eps) + b
    dx, dw, db, dg, dr, dout = dev(x), dev(w), dev(b), dev(gate), dev(res), H.DeviceBuffer(4 * rows * n + 256)
    tx, tg, tr, td = (Tensor.contiguous(t.ptr, F32, (n, rows)) for t in (dx, dg, dr, dout))
    check(lib().b200_op_norm_affine(C.byref(tx), dw.ptr, 1, db.ptr, None, None, 0, None, C.byref(td), eps, kind, None))
    assert rel(dout.to_numpy(np.float32, (rows, n)), base) < 3e-6
    check(lib().b200_op_norm_affine(C.byref(tx), dw.ptr, 1, db.ptr, C.byref(tg), None, 1, C.byref(tr), C.byref(td), eps, kind, None))
    assert rel(dout.to_numpy(np.float32, (rows, n)), res + base * R.sigmoid(gate)) < 3e-6


def run_qkv_store(q, k, v, vecs, pos, cells, rot, n_cells, eps, lead=3):
    """q, k, v [T, heads, size] are handed over as column ranges of one wider row, as the fused projection leaves them."""
    T, Hh, D = q.shape
    G, V = k.shape[1], v.shape[2]
    row = lead + Hh * D + G * D + G * V + 5
    buf = np.random.default_rng(0).standard_normal((T, row))
    oq, ok, ov = lead, lead + Hh * D, lead + Hh * D + G * D
    buf[:, oq:ok], buf[:, ok:ov], buf[:, ov:ov + G * V] = q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)
    d = dev(buf)
    dv = {n: dev(a) for n, a in vecs.items()}
    dp, dc, df = dev(pos, np.int32), dev(cells, np.int32), dev(R.rotation_freqs(rot) if rot["dims"] else np.zeros(1))
    kc, vc = dev(np.full((n_cells, G * D + 2), 7.0)), dev(np.full((n_cells, G * V + 1), 7.0))
    g = lambda n: dv[n].ptr if n in dv else None
    a = QkvStoreArgs(q=d.ptr + 4 * oq, q_stride=row, k=d.ptr + 4 * ok, k_stride=row, v=d.ptr + 4 * ov, v_stride=row, q_bias=g("q.b"), k_bias=g("k.b"), v_bias=g("v.b"),
                     q_norm=g("q.norm"), k_norm=g("k.norm"), pos=dp.ptr, cells=dc.ptr, freqs=df.ptr, k_cache=kc.ptr, k_cache_stride=G * D + 2, v_cache=vc.ptr,
                     v_cache_stride=G * V + 1, n_head=Hh, n_head_kv=G, dim=D, vdim=V, n_dims=rot["dims"], n_tokens=T, eps=eps)
    check(lib().b200_op_qkv_store(C.byref(a), None))
    out = d.to_numpy(np.float32, (T, row))
    assert np.array_equal(out[:, :lead], buf[:, :lead].astype(np.float32)) and np.array_equal(out[:, ok:], buf[:, ok:].astype(np.float32))  # only q is rewritten
    return out[:, oq:ok].reshape(T, Hh, D), kc.to_numpy(np.float32, (n_cells, G * D + 2)), vc.to_numpy(np.float32, (n_cells, G * V + 1))


@pytest.mark.parametrize("Hh,G,D,V,dims,extra", [(4, 2, 16, 24, 8, True), (3, 3, 10, 6, 10, False), (1, 1, 64, 64, 32, True), (6, 2, 96, 40, 0, True)])
def test_qkv_store_bias_norm_rotation_cells(Hh, G, D, V, dims, extra):
    rng = np.random.default_rng(Hh * D + V)
    T, n_cells, eps = 7, 20, 1e-5
    q, k, v = rng.standard_normal((T, Hh, D)), rng.standard_normal((T, G, D)), rng.standard_normal((T, G, V))
    pos, cells = np.array([0, 1, 2, 95, 96, 4000, 3]), np.array([5, 0, 19, 7, 8, 2, 11])
    rot = {"base": 3000.0, "dims": dims, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    vecs = {}
    if extra:
        vecs = {"q.b": rng.standard_normal(Hh * D), "k.b": rng.standard_normal(G * D), "v.b": rng.standard_normal(G * V),
                "q.norm": 1 + 0.3 * rng.standard_normal(Hh * D), "k.norm": 1 + 0.3 * rng.standard_normal(G * D)}
    gq, kc, vc = run_qkv_store(q, k, v, vecs, pos, cells, rot, n_cells, eps)
    wq, wk, wv = q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)
    if extra:
        wq, wk, wv = R.rms_norm(wq + vecs["q.b"], vecs["q.norm"], eps), R.rms_norm(wk + vecs["k.b"], vecs["k.norm"], eps), wv + vecs["v.b"]
    wq, wk = R.rotate_pairs(wq.reshape(T, Hh, D), pos, rot), R.rotate_pairs(wk.reshape(T, G, D), pos, rot)
    tol = 3e-4  # an f32 angle at position 4000 is rounded by up to 4000 * 2^-24 rad
    assert rel(gq, wq) < tol
    assert rel(kc[cells, :G * D], wk.reshape(T, -1)) < tol and rel(vc[cells, :G * V], wv) < 3e-6
    untouched = np.setdiff1d(np.arange(n_cells), cells)
    assert (kc[untouched] == 7.0).all() and (vc[untouched] == 7.0).all() and (kc[:, G * D:] == 7.0).all() and (vc[:, G * V:] == 7.0).all()


def run_sink_attn(q, kc, vc, cell_seq, cell_pos, tok_seq, tok_pos, sink, scale, G, window=0, keep_first=0, bf16=0):
    T, Hh, D = q.shape
    V = vc.shape[1] // G
    bufs = [dev(q), dev(kc), dev(vc), dev(cell_seq, np.int32), dev(cell_pos, np.int32), dev(tok_seq, np.int32), dev(tok_pos, np.int32)]
    dsink = dev(sink) if sink is not None else None
    out = H.DeviceBuffer(4 * T * Hh * V + 256)
    a = SinkAttnArgs(q=bufs[0].ptr, q_stride=Hh * D, k_cache=bufs[1].ptr, k_cache_stride=kc.shape[1], v_cache=bufs[2].ptr, v_cache_stride=vc.shape[1], cell_seq=bufs[3].ptr,
                     cell_pos=bufs[4].ptr, tok_seq=bufs[5].ptr, tok_pos=bufs[6].ptr, sink=dsink.ptr if dsink else None, dst=out.ptr, dst_stride=Hh * V, n_head=Hh, n_head_kv=G,
                     dim=D, vdim=V, n_tokens=T, n_kv=len(cell_seq), window=window, keep_first=keep_first, scale=scale, bf16_products=bf16)
    need = int(lib().b200_sink_attn_workspace_bytes(C.byref(a)))  # > 0: few tokens and many cells, the cells are split over CTAs
    ws = H.DeviceBuffer(need + 256) if need else None
    check(lib().b200_op_sink_attn_ws(C.byref(a), ws.ptr if ws else None, need, None))
    got = out.to_numpy(np.float32, (T, Hh, V))
    if need:  # without a workspace the unsplit form must give the same
        check(lib().b200_op_sink_attn(C.byref(a), None))
        assert np.allclose(out.to_numpy(np.float32, (T, Hh, V)), got, rtol=1e-5, atol=1e-6, equal_nan=True)
    return got


def one_token_reference(q_t, kc, vc, cell_seq, cell_pos, s, p, sink, scale, G, window, keep_first):
    """The sequence's rows in position order, then the dense reference; returns the row of position p."""
    D, V = q_t.shape[1], vc.shape[1] // G
    idx = [int(np.where((cell_seq == s) & (cell_pos == j))[0][0]) for j in range(p + 1)]
    k, v = kc[idx].reshape(p + 1, G, D), vc[idx].reshape(p + 1, G, V)
    q = np.repeat(q_t[None], p + 1, 0)
    return R.sink_attention(q, k, v, scale, sink, window, keep_first)[p]


@pytest.mark.parametrize("Hh,G,D,V", [(4, 2, 16, 24), (3, 3, 40, 8), (8, 1, 64, 64), (2, 2, 96, 130), (1, 1, 200, 33)])
@pytest.mark.parametrize("window,keep_first", [(0, 0), (5, 0), (6, 3)])
@pytest.mark.parametrize("n_cells", [96, 2304])
def test_sink_attn_scattered_cells_two_sequences(Hh, G, D, V, window, keep_first, n_cells):
    """Two sequences share the cell table in shuffled order, with free cells (NaN rows) between; few tokens: the decode form
    (with 2304 cells: split over several CTAs per (token, head) and merged)."""
    rng = np.random.default_rng(D + V + window)
    n_a, n_b = 37, 21
    kc, vc = rng.standard_normal((n_cells, G * D)), rng.standard_normal((n_cells, G * V))
    perm = rng.permutation(n_cells)
    cell_seq, cell_pos = np.full(n_cells, -1), np.full(n_cells, -1)
    cell_seq[perm[:n_a]], cell_pos[perm[:n_a]] = 4, np.arange(n_a)
    cell_seq[perm[n_a:n_a + n_b]], cell_pos[perm[n_a:n_a + n_b]] = 9, np.arange(n_b)
    kc[cell_seq < 0], vc[cell_seq < 0] = np.nan, np.nan
    toks = [(4, 0), (4, 1), (4, 36), (9, 20), (9, 5), (4, 17), (9, 6), (4, 8)]
    q, sink = rng.standard_normal((len(toks), Hh, D)), rng.standard_normal(Hh)
    scale = 1.5 / math.sqrt(D)
    got = run_sink_attn(q, kc, vc, cell_seq, cell_pos, [s for s, _ in toks], [p for _, p in toks], sink, scale, G, window, keep_first)
    for i, (s, p) in enumerate(toks):
        want = one_token_reference(q[i], kc, vc, cell_seq, cell_pos, s, p, sink, scale, G, window, keep_first)
        assert rel(got[i], want) < 1e-5, (i, s, p)


@pytest.mark.parametrize("bf16", [0, 1])
@pytest.mark.parametrize("Hh,G,D,V,T", [(4, 2, 16, 32, 150), (2, 1, 64, 64, 300), (3, 3, 96, 48, 70), (2, 2, 40, 24, 40), (4, 4, 128, 128, 129)])
@pytest.mark.parametrize("window,keep_first", [(0, 0), (33, 4)])
def test_sink_attn_prompt_batches(Hh, G, D, V, T, window, keep_first, bf16):
    """A prompt of T tokens behind 19 cached ones, beside a second sequence's prompt; free cells hold NaN.  With bf16 products the
    reference gets q, k, v rounded the same way (the weights' rounding is bounded by the tolerance)."""
    rng = np.random.default_rng(T + D + bf16)
    past, T2 = 19, 23
    n_cells = (past + T + T2 + 40 + 31) // 32 * 32
    kc, vc = np.full((n_cells, G * D), np.nan), np.full((n_cells, G * V), np.nan)
    cells_a = np.sort(rng.choice(n_cells, past + T, replace=False))
    free = np.setdiff1d(np.arange(n_cells), cells_a)
    cells_b = free[:T2]
    cell_seq, cell_pos = np.full(n_cells, -1), np.full(n_cells, -1)
    cell_seq[cells_a], cell_pos[cells_a] = 2, np.arange(past + T)
    cell_seq[cells_b], cell_pos[cells_b] = 5, np.arange(T2)
    ka, va, kb, vb = rng.standard_normal((past + T, G, D)), rng.standard_normal((past + T, G, V)), rng.standard_normal((T2, G, D)), rng.standard_normal((T2, G, V))
    qa, qb = rng.standard_normal((T, Hh, D)), rng.standard_normal((T2, Hh, D))
    if bf16:
        ka, va, kb, vb, qa, qb = (R.bf16_round(z).astype(np.float64) for z in (ka, va, kb, vb, qa, qb))
    kc[cells_a], vc[cells_a], kc[cells_b], vc[cells_b] = ka.reshape(past + T, -1), va.reshape(past + T, -1), kb.reshape(T2, -1), vb.reshape(T2, -1)
    sink, scale = rng.standard_normal(Hh), 1.2 / math.sqrt(D)
    q = np.concatenate([qa, qb])
    tok_seq, tok_pos = [2] * T + [5] * T2, list(range(past, past + T)) + list(range(T2))
    got = run_sink_attn(q, kc, vc, cell_seq, cell_pos, tok_seq, tok_pos, sink, scale, G, window, keep_first, bf16)
    qfull = np.concatenate([np.zeros((past, Hh, D)), qa])
    want_a = R.sink_attention(qfull, ka, va, scale, sink, window, keep_first)[past:]
    want_b = R.sink_attention(qb, kb, vb, scale, sink, window, keep_first)
    tol = 1.5e-2 if bf16 else 1e-5
    assert np.isfinite(got).all() and rel(got[:T], want_a) < tol and rel(got[T:], want_b) < tol


@pytest.mark.parametrize("T", [3, 200])
def test_sink_attn_far_key_window_edge_and_sink(T):
    """One key is made to dominate.  At distance window - 1 it owns the output, at distance window it must be gone, below
    keep_first it is back, and a large sink takes the weight away from all of them."""
    rng = np.random.default_rng(T)
    Hh, G, D, V, n, window, keep = 2, 1, 32, 16, 600, 100, 3
    k, v = rng.standard_normal((n, G, D)) * 0.1, rng.standard_normal((n, G, V))
    cell_seq, cell_pos = np.zeros(n, dtype=np.int64), np.arange(n)
    qdir = rng.standard_normal(D)
    qdir /= np.linalg.norm(qdir)
    sink = np.array([-30.0, -30.0])
    for far, expect_far in [(599 - 99, True), (599 - 100, False), (2, True), (3, False)]:
        kk = k.copy()
        kk[far, 0] = 40.0 * qdir  # score 40 against the query below, all others near 0
        q = np.tile(qdir, (T, Hh, 1)).astype(np.float64)
        tok_pos = [599] * T
        got = run_sink_attn(q, kk.reshape(n, -1), v.reshape(n, -1), cell_seq, cell_pos, [0] * T, tok_pos, sink, 1.0, G, window, keep)
        close = np.abs(got[0, 0] - v[far, 0]).max() < 1e-3
        assert close == expect_far, (far, expect_far)
        want = R.sink_attention(np.concatenate([np.zeros((599, Hh, D)), q[:1]]), kk, v, 1.0, sink, window, keep)[599]
        assert rel(got[0], want) < 1e-5 and rel(got[-1], want) < 1e-5
    got = run_sink_attn(q, k.reshape(n, -1), v.reshape(n, -1), cell_seq, cell_pos, [0] * T, [599] * T, np.array([30.0, -30.0]), 1.0, G, window, keep)
    assert np.abs(got[0, 0]).max() < 1e-6 and np.abs(got[0, 1]).max() > 1e-3  # head 0: the sink has (almost) all the weight and no value


def run_linear_attn(q, k, v, decay, runs, state, slot_stride, act=1):
    T, Hh, D = q.shape
    V = v.shape[2]
    info = np.array([[r[i] for r in runs] for i in range(4)], dtype=np.int32)  # first, count, slot, fresh
    bufs = [dev(q), dev(k), dev(v), dev(decay), dev(info, np.int32)]
    out = H.DeviceBuffer(4 * T * Hh * V + 256, zero=True)
    a = LinearAttnArgs(q=bufs[0].ptr, k=bufs[1].ptr, v=bufs[2].ptr, q_stride=Hh * D, k_stride=Hh * D, v_stride=Hh * V, decay=bufs[3].ptr, seq_info=bufs[4].ptr, n_seq=len(runs),
                       state=state.ptr, slot_stride=slot_stride, dst=out.ptr, dst_stride=Hh * V, heads=Hh, dim=D, vdim=V, act=act)
    check(lib().b200_op_linear_attn_scan(C.byref(a), None))
    return out.to_numpy(np.float32, (T, Hh, V))


@pytest.mark.parametrize("Hh,D,V", [(2, 32, 32), (3, 8, 12), (1, 100, 21), (2, 130, 64)])
def test_linear_attn_whole_against_portions_across_slots(Hh, D, V):
    rng = np.random.default_rng(D + V)
    Ta, Tb = 45, 18
    q, k, v = (rng.standard_normal((Ta + Tb, Hh, n)) for n in (D, D, V))
    decay = np.array([0.999, 0.6, 0.9][:Hh])
    stride = Hh * D * V + 5
    state = dev(np.full((3, stride), np.nan))  # stale contents: fresh sequences must not read them
    want_a, Sa = R.decayed_outer_product_scan(R.silu(q[:Ta]), R.silu(k[:Ta]), R.silu(v[:Ta]), decay)
    want_b, _ = R.decayed_outer_product_scan(R.silu(q[Ta:]), R.silu(k[Ta:]), R.silu(v[Ta:]), decay)
    got = run_linear_attn(q, k, v, decay, [(0, Ta, 2, 1), (Ta, Tb, 0, 1)], state, stride)
    assert rel(got[:Ta], want_a) < 2e-5 and rel(got[Ta:], want_b) < 2e-5
    S = state.to_numpy(np.float32, (3, stride))[2, :Hh * D * V].reshape(Hh, V, D)
    assert rel(S, Sa.transpose(0, 2, 1)) < 2e-5
    # the same sequence in portions of 17, 1, 2, ... tokens through slot 1 gives the same outputs
    state2 = dev(np.full((3, stride), np.nan))
    at, rows = 0, []
    for n in [17, 1, 2, 16, 9]:
        rows.append(run_linear_attn(q[at:at + n], k[at:at + n], v[at:at + n], decay, [(0, n, 1, int(at == 0))], state2, stride))
        at += n
    assert at == Ta and rel(np.concatenate(rows), want_a) < 2e-5


def run_route(z, corr, top, n_group, n_keep, scale):
    T, E = z.shape
    dz, dc, di, dw = dev(z), dev(corr), H.DeviceBuffer(4 * T * top + 256), H.DeviceBuffer(4 * T * top + 256)
    check(lib().b200_op_moe_route_grouped(dz.ptr, E, dc.ptr, di.ptr, top, dw.ptr, top, E, top, n_group, n_keep, scale, T, None))
    return di.to_numpy(np.int32, (T, top)), dw.to_numpy(np.float32, (T, top))


@pytest.mark.parametrize("E,top,n_group,n_keep", [(16, 3, 4, 3), (6, 2, 3, 2), (8, 1, 1, 1), (64, 8, 8, 2), (256, 6, 8, 4), (12, 4, 12, 5), (40, 5, 4, 4)])
def test_router_groups_correction_and_ties(E, top, n_group, n_keep):
    rng = np.random.default_rng(E + top)
    T = 50
    z = rng.standard_normal((T, E)).astype(np.float32) * 2
    corr = (rng.standard_normal(E) * 0.5 - 1.5).astype(np.float32)  # all choice scores negative: a group that is out must not count as 0
    z[7] = 0.0          # equal scores: the correction alone decides
    ids, w = run_route(z, corr, top, n_group, n_keep, 2.5)
    for t in range(T):
        s32 = (1.0 / (1.0 + np.exp(-z[t].astype(np.float32)))).astype(np.float32)
        chosen, ww = R.route(z[t].astype(np.float64), corr.astype(np.float64), top, n_group, n_keep, 2.5)
        if list(ids[t]) != chosen:  # only a near tie of two f32 choice scores may differ
            c = s32 + corr
            a, b = sorted(set(ids[t]) ^ set(chosen))[:2]
            assert abs(c[a] - c[b]) < 1e-6, (t, ids[t], chosen)
            continue
        assert rel(w[t], ww) < 1e-5
    # all choice scores equal: the lowest groups and, inside them, the lowest indices
    ids, w = run_route(np.zeros((1, E), dtype=np.float32), np.zeros(E, dtype=np.float32), top, n_group, n_keep, 1.0)
    assert list(ids[0]) == list(range(top))
    assert abs(w[0].sum() - 1.0) < 1e-6


@pytest.mark.parametrize("wt", [F32, BF16])
@pytest.mark.parametrize("K,M,E,top,T", [(40, 24, 6, 2, 5), (64, 48, 4, 3, 1), (320, 128, 16, 3, 30), (72, 10, 3, 1, 9), (128, 320, 8, 2, 70)])
def test_expert_products_dense_weights(wt, K, M, E, top, T):
    rng = np.random.default_rng(K + M + T)
    w = R.bf16_round(rng.standard_normal((E, M, K)))
    x = rng.standard_normal((T, top, K)).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:top] for _ in range(T)]).astype(np.int32)
    raw = (w.view(np.uint32) >> 16).astype(np.uint16) if wt == BF16 else w
    dw, dx, di, dd = dev(raw, raw.dtype), dev(x), dev(ids, np.int32), H.DeviceBuffer(4 * T * top * M + 256)
    want = np.einsum("tsk,tsmk->tsm", x.astype(np.float64), w[ids].astype(np.float64))
    for nbr in (top, 1):  # a row per slot, or one row shared by the slots of a token
        tw, tx = Tensor.contiguous(dw.ptr, wt, (K, M, E)), Tensor.contiguous(dx.ptr, F32, (K, nbr, T))
        tx.nb[2] = 4 * K * top
        ti, td = Tensor.contiguous(di.ptr, I32, (top, T)), Tensor.contiguous(dd.ptr, F32, (M, top, T))
        check(lib().b200_op_mul_mat_id_float(C.byref(tw), C.byref(tx), C.byref(ti), C.byref(td), None))
        ref = want if nbr == top else np.einsum("tk,tsmk->tsm", x[:, 0].astype(np.float64), w[ids].astype(np.float64))
        assert rel(dd.to_numpy(np.float32, (T, top, M)), ref) < 3e-6


@pytest.mark.parametrize("K,M,E,top,T", [(64, 48, 4, 3, 40), (320, 128, 16, 3, 300), (128, 320, 8, 2, 70), (192, 130, 5, 1, 100)])
def test_expert_products_bf16_batches_on_the_tensor_cores(K, M, E, top, T):
    rng = np.random.default_rng(K + M + T)
    w = R.bf16_round(rng.standard_normal((E, M, K)))
    x = rng.standard_normal((T, top, K)).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:top] for _ in range(T)]).astype(np.int32)
    bits = (w.view(np.uint32) >> 16).astype(np.uint16)
    got = H.mul_mat_id_q(BF16, bits.view(np.uint8), ids, x, K, M, E)
    want = np.einsum("tsk,tsmk->tsm", R.bf16_round(x).astype(np.float64), w[ids].astype(np.float64))
    assert rel(got, want) < 3e-6


@pytest.mark.parametrize("K,M,N", [(4096, 8, 1), (512, 64, 5), (1001, 3, 40), (640, 256, 9), (320, 16, 7)])
def test_f32_product_with_few_outputs(K, M, N):
    """Router-shaped products: f32 weights, a handful of rows over the model width (long rows take the CTA-per-output kernel)."""
    rng = np.random.default_rng(K + M + N)
    w, x = rng.standard_normal((M, K)).astype(np.float32), rng.standard_normal((N, K + 3)).astype(np.float32)
    dw, dx, dd = dev(w), dev(x), H.DeviceBuffer(4 * N * (M + 2) + 256)
    tw, tx, td = Tensor.contiguous(dw.ptr, F32, (K, M)), Tensor.contiguous(dx.ptr, F32, (K, N)), Tensor.contiguous(dd.ptr, F32, (M, N))
    tx.nb[1], td.nb[1] = 4 * (K + 3), 4 * (M + 2)  # rows of a wider buffer
    check(lib().b200_op_mul_mat_float(C.byref(tw), C.byref(tx), C.byref(td), None))
    got = dd.to_numpy(np.float32, (N, M + 2))[:, :M]
    assert rel(got, x[:, :K].astype(np.float64) @ w.astype(np.float64).T) < 3e-6


def test_silu_mul_halves_combine_and_softcap():
    rng = np.random.default_rng(11)
    F, NU, T, Wd = 24, 3, 7, 40
    gu = rng.standard_normal((T, NU, 2 * F))
    dgu, dact = dev(gu), H.DeviceBuffer(4 * T * NU * F + 256)
    ta, tb = Tensor.contiguous(dgu.ptr, F32, (F, NU, T)), Tensor.contiguous(dgu.ptr + 4 * F, F32, (F, NU, T))
    for t in (ta, tb):
        t.nb[1], t.nb[2] = 8 * F, 8 * F * NU
    td = Tensor.contiguous(dact.ptr, F32, (F, NU, T))
    check(lib().b200_op_silu_mul_strided(C.byref(ta), C.byref(tb), C.byref(td), None))
    assert rel(dact.to_numpy(np.float32, (T, NU, F)), R.silu(gu[..., :F]) * gu[..., F:]) < 2e-6
    y, w, x0, x1 = rng.standard_normal((T, NU, Wd)), rng.standard_normal((T, NU)), rng.standard_normal((T, Wd)), rng.standard_normal((T, Wd))
    dy, dw, d0, d1, dout = dev(y), dev(w), dev(x0), dev(x1), H.DeviceBuffer(4 * T * Wd + 256)
    check(lib().b200_op_moe_combine(dy.ptr, Wd, NU * Wd, dw.ptr, NU, d0.ptr, Wd, d1.ptr, Wd, dout.ptr, Wd, Wd, NU, T, None))
    assert rel(dout.to_numpy(np.float32, (T, Wd)), x0 + x1 + np.einsum("tk,tkn->tn", w, y)) < 2e-6
    z = rng.standard_normal(500) * 40
    dz, dc = dev(z), H.DeviceBuffer(2000 + 256)
    tz, tc = Tensor.contiguous(dz.ptr, F32, (500,)), Tensor.contiguous(dc.ptr, F32, (500,))
    check(lib().b200_op_unary(9, C.byref(tz), C.byref(tc), 30.0, 0.0, None))
    assert rel(dc.to_numpy(np.float32, (500,)), 30.0 * np.tanh(z / 30.0)) < 2e-6


# ------------------------------------------------------------------------------------------------ whole models
from koboldcpp_b200 import galirax as G  # noqa: E402
from koboldcpp_b200.engine import Engine, Request  # noqa: E402

CONFIGS = {
    # a looped stretch (layers 1 and 2 run twice, each run with its own cache / state), a window shorter than the prompts
    "mixed": lambda: R.make_config([R.attn_layer(), R.attn_layer("attention_2", window=9, keep_first=2, scaling=False), R.lightning_layer(),
                                    R.attn_layer("attention_2", heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=8, window=30, keep_first=1, mlp=None)], loop=(1, 3, 2)),
    # one head, one group, one expert per token, dim != vdim everywhere, rotation over the whole head, no soft cap, no loop
    "odd": lambda: R.make_config([R.attn_layer(heads=1, kv_heads=1, dim=24, vdim=40, rot_dims=24, scaling=False, base=500.0, mlp=R.moe(ff=40, experts=5, top=1, groups=1, keep=1, scale=1.0)),
                                  R.lightning_layer(heads=1, dim=24, vdim=40, decay=[0.97], mlp=None),
                                  R.attn_layer("attention_2", heads=6, kv_heads=2, dim=8, vdim=4, rot_dims=2, window=4, keep_first=0, mlp=R.moe(ff=8, experts=8, top=4, groups=4, keep=2, scale=0.7))],
                                 width=72, vocab=70, eps=1e-6, softcap=0.0),
    "lightning_only": lambda: R.make_config([R.lightning_layer(heads=2, dim=32, vdim=64), R.lightning_layer(mlp=None)], width=32, vocab=50, loop=(0, 2, 2)),
    # sizes that take the 16-byte paths: width and ff multiples of 64
    "aligned": lambda: R.make_config([R.attn_layer(heads=4, kv_heads=4, dim=32, vdim=32, rot_dims=32, mlp=R.moe(ff=64, experts=8, top=2, groups=2, keep=1)),
                                      R.attn_layer("attention_2", heads=4, kv_heads=1, dim=64, vdim=32, rot_dims=16, window=20, keep_first=3, mlp=R.moe(ff=64, experts=4, top=2, groups=1, keep=1))],
                                     width=128, vocab=96, loop=(1, 2, 3)),
}


@pytest.fixture(scope="module", params=list(CONFIGS))
def model(request):
    cfg = CONFIGS[request.param]()
    W = R.random_weights(cfg, seed=len(request.param))
    m = G.build(cfg, R.as_tensors(W), dtype="float32", n_ctx=768, n_seq_max=4, max_batch=400)
    yield cfg, W, m
    m.close()


def logits_err(got, want):
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return float((np.sqrt((d ** 2).mean(-1)) / want.std()).max())


def test_prompt_logits_first_tokens_and_every_position(model):
    cfg, W, m = model
    rng = np.random.default_rng(1)
    toks = rng.integers(0, cfg["vocab"], 70).tolist()
    want = R.forward(cfg, W, toks)
    eng = Engine(m)
    got = eng.step([("a", toks, range(len(toks)))])
    eng.finish("a")
    assert logits_err(got, want) < 1e-4
    one = eng.step([("b", toks[:1], [0])])  # a sequence of one token
    eng.finish("b")
    assert logits_err(one, want[:1]) < 1e-4


@pytest.mark.parametrize("portion", [2, 3, 7, 33])
def test_portions_and_decoding_match_the_whole_prompt(model, portion):
    cfg, W, m = model
    rng = np.random.default_rng(portion)
    toks = rng.integers(0, cfg["vocab"], 60).tolist()
    want = R.forward(cfg, W, toks)
    eng = Engine(m)
    rows = []
    for a in range(0, 40, portion):
        b = min(a + portion, 40)
        rows.append(eng.step([("p", toks[a:b], range(b - a))]))
    for t in range(40, 60):  # the windows (4, 9, 20, 30) pass over decoded tokens here
        rows.append(eng.step([("p", [toks[t]], [0])]))
    eng.finish("p")
    assert logits_err(np.concatenate(rows), want) < 1e-4


def test_unequal_batch_then_decode_together_and_reuse(model):
    """Three requests of different lengths start in one batch and decode together; the shortest ends first and its cells and
    slot go to a new request that joins while the others still decode."""
    cfg, W, m = model
    rng = np.random.default_rng(4)
    lens = {"a": (1, 12), "b": (23, 30), "c": (57, 70)}  # prompt length, total length
    toks = {k: rng.integers(0, cfg["vocab"], n).tolist() for k, (_, n) in lens.items()}
    toks["d"] = rng.integers(0, cfg["vocab"], 31).tolist()
    want = {k: R.forward(cfg, W, v) for k, v in toks.items()}
    eng = Engine(m)
    got = {k: [] for k in toks}
    out = eng.step([(k, toks[k][:lens[k][0]], [lens[k][0] - 1]) for k in "abc"])
    for i, k in enumerate("abc"):
        got[k].append((lens[k][0] - 1, out[i]))
    at = {k: lens[k][0] for k in "abc"}
    live = ["a", "b", "c"]
    d_started = False
    while live:
        out = eng.step([(k, [toks[k][at[k]]], [0]) for k in live])
        for i, k in enumerate(live):
            got[k].append((at[k], out[i])); at[k] += 1
        for k in [k for k in live if at[k] == len(toks[k])]:
            live.remove(k); eng.finish(k)
            if k == "a" and not d_started:  # "d" takes over what "a" held, as a prompt beside the decoding tokens
                d_started = True
                o = eng.step([("d", toks["d"][:20], [19])] + [(x, [toks[x][at[x]]], [0]) for x in live])
                got["d"].append((19, o[0]))
                for i, x in enumerate(live):
                    got[x].append((at[x], o[1 + i])); at[x] += 1
                at["d"] = 20; live.append("d")
    for k, rows in got.items():
        pos = [p for p, _ in rows]
        assert logits_err(np.stack([r for _, r in rows]), want[k][pos]) < 1e-4, k
    assert m.seq_length(0) == -1  # everything was given back


def test_long_decoding_across_cache_padding(model):
    cfg, W, m = model
    rng = np.random.default_rng(6)
    toks = rng.integers(0, cfg["vocab"], 300).tolist()
    want = R.forward(cfg, W, toks)
    eng = Engine(m)
    rows = [eng.step([("x", toks[:230], [0, 1, 229])])]
    places = [0, 1, 229]
    for t in range(230, 300):  # passes 256 cells
        rows.append(eng.step([("x", [toks[t]], [0])])); places.append(t)
    eng.finish("x")
    assert logits_err(np.concatenate(rows), want[places]) < 2e-4


def test_greedy_generation_through_the_engine(model):
    cfg, W, m = model
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (5, 17, 1, 40)]
    eng = Engine(m, max_step_tokens=24)  # prompts are cut into portions beside decoding requests
    outs = eng.generate([Request(p, 10) for p in prompts])
    for p, out in zip(prompts, outs):
        seq = list(p)
        for tok in out:  # every generated token is the reference's argmax given what came before, or a near tie
            lg = R.forward(cfg, W, seq)[-1]
            top = np.sort(lg)[-2:]
            assert tok == int(np.argmax(lg)) or lg[tok] > top[1] - 1e-3 * (abs(top[1]) + 1), (len(seq), tok)
            seq.append(tok)
        assert len(out) == 10


@pytest.mark.parametrize("name", ["mixed", "aligned"])
def test_bfloat16_portions_batches_and_decoding_agree_with_float32(name):
    """bf16 serving mode: prompt portions of 16 tokens or more take the tensor-core kernels (attention and expert products), over
    cells that earlier portions wrote and beside another request's tokens; shorter portions and single tokens take the f32 kernels.
    All of them must give the logits of the float64 reference up to bf16 rounding."""
    cfg = CONFIGS[name]()
    W = R.random_weights(cfg, seed=5)
    rng = np.random.default_rng(1)
    ta, tb = rng.integers(0, cfg["vocab"], 75).tolist(), rng.integers(0, cfg["vocab"], 41).tolist()
    want = R.forward(cfg, W, ta)
    m = G.build(cfg, R.as_tensors(W), dtype="bfloat16", n_ctx=256, n_seq_max=2, max_batch=128)
    eng = Engine(m)
    whole = eng.step([("a", ta, range(75))])
    eng.finish("a")
    parts = [eng.step([("b", tb, []), ("a", ta[:33], range(33))])]  # the freed cells are used again, in another order
    parts.append(eng.step([("a", ta[33:53], range(20))]))
    parts.append(eng.step([("a", ta[53:70], range(17))]))
    parts.append(eng.step([("a", ta[70:73], range(3))]))
    parts += [eng.step([("a", [t], [0])]) for t in ta[73:]]
    m.close()
    for got in (whole, np.concatenate(parts)):
        d = got - want
        d = d - d.mean(-1, keepdims=True)
        e = np.sqrt((d ** 2).mean(-1)) / want.std()
        # a rounded activation can move a router choice at a near tie; the bound is on the bulk of the rows, with a loose cap
        assert np.isfinite(e).all() and np.quantile(e, 0.8) < 3e-2 and e.max() < 0.7


def test_far_key_through_the_model():
    """Weights make the attention sharp (large score scale), so a wrong position, mask or cell would show in the logits; the
    second layer's window edge and its kept first tokens lie inside the prompt and inside the decoded stretch."""
    cfg = R.make_config([R.attn_layer(heads=2, kv_heads=1, dim=16, vdim=16, rot_dims=16, scale=3.0, mlp=None),
                         R.attn_layer("attention_2", heads=2, kv_heads=2, dim=16, vdim=8, rot_dims=8, window=300, keep_first=5, scale=3.0, scaling=False)])
    W = R.random_weights(cfg, seed=21)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], 640).tolist()
    want = R.forward(cfg, W, toks)
    m = G.build(cfg, R.as_tensors(W), dtype="float32", n_ctx=768, n_seq_max=2, max_batch=640)
    eng = Engine(m)
    places = [0, 1, 2, 255, 256, 257, 299, 300, 301, 304, 305, 306, 511, 512, 600]
    rows = [eng.step([("a", toks[:601], places)])]
    for t in range(601, 640):
        rows.append(eng.step([("a", [toks[t]], [0])])); places.append(t)
    m.close()
    assert logits_err(np.concatenate(rows), want[places]) < 2e-4


# ------------------------------------------------------------------------------------------------ a model folder, the registry, the command line, the trace runner
def write_model_folder(path, cfg, W):
    import json
    import struct
    meta, blobs, at = {}, [], 0
    for name, (dt, shape, raw) in R.as_tensors(W).items():
        b = raw.tobytes()
        meta[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [at, at + len(b)]}
        blobs.append(b); at += len(b)
    head = json.dumps(meta).encode()
    (path / "model.safetensors").write_bytes(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    (path / "config.json").write_text(json.dumps(cfg))


def test_model_folder_command_line_and_trace_runner(tmp_path, capsys):
    import json
    import subprocess
    import sys
    from pathlib import Path
    from koboldcpp_b200 import __main__ as cli
    cfg = CONFIGS["mixed"]()
    W = R.random_weights(cfg, seed=2)
    write_model_folder(tmp_path, cfg, W)
    rng = np.random.default_rng(3)
    pa, pb = rng.integers(0, cfg["vocab"], 9).tolist(), rng.integers(0, cfg["vocab"], 4).tolist()
    # generate: greedy tokens of two prompts through registry, loader, engine and sampler
    assert cli.main(["generate", "--model", str(tmp_path), "--dtype", "float32", "--max-new-tokens", "6", "--prompt", ",".join(map(str, pa)), "--prompt", ",".join(map(str, pb))]) == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines() if x.startswith("{")]
    assert [x["prompt"] for x in lines] == [pa, pb]
    for x in lines:
        seq = list(x["prompt"])
        for tok in x["tokens"]:
            lg = R.forward(cfg, W, seq)[-1]
            top = np.sort(lg)[-2:]
            assert tok == int(np.argmax(lg)) or lg[tok] > top[1] - 1e-3 * (abs(top[1]) + 1)
            seq.append(tok)
    # the trace runner: two requests start together, decode together, the shorter one ends first
    ta, tb = rng.integers(0, cfg["vocab"], 14).tolist(), rng.integers(0, cfg["vocab"], 8).tolist()
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": ta[:11], "want": [0, 10]}, {"id": "y", "tokens": tb[:6], "want": [5]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": ta[11:12], "want": []}, {"id": "y", "tokens": tb[6:7], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": ta[12:13], "want": [0]}, {"id": "y", "tokens": tb[7:8], "want": [0]}], "end": ["y"]},
             {"step": 3, "entries": [{"id": "x", "tokens": ta[13:14], "want": [0]}], "end": ["x"]}]
    out = tmp_path / "out"
    root = Path(__file__).resolve().parent.parent
    p = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    wa, wb = R.forward(cfg, W, ta), R.forward(cfg, W, tb)
    want = {0: np.stack([wa[0], wa[10], wb[5]]), 1: wb[6:7], 2: np.stack([wa[12], wb[7]]), 3: wa[13:14]}
    for n, w in want.items():
        got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        assert got.shape == w.shape and logits_err(got, w) < 1e-4, n

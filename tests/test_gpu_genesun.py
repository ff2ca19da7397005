"""Genesun on the GPU against the plain float64 statement in genesun_ref.py: every mechanism alone through the C ABI, then whole
models through the loader, the batch step, the sequence cache and the engine (prefill against decoding, portions, mixed
batches, cells and slots that are used again, long decoding, greedy generation)."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import pytest

import genesun_ref as R
import koboldcpp_b200.host as H
from koboldcpp_b200.lib import BF16, F32, I32, LatentAttnArgs, MlstmArgs, Tensor, check, lib

pytestmark = pytest.mark.gpu


def dev(a, dtype=np.float32):
    return H.DeviceBuffer.from_numpy(np.ascontiguousarray(a, dtype=dtype), pad=256)


def rel(got, want):
    return float(np.abs(got - want).max() / (np.abs(want).max() + 1e-30))


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("n,rows", [(64, 5), (320, 3), (1000, 2), (5000, 2)])
def test_norm_with_gate_and_residual(kind, n, rows):
    rng = np.random.default_rng(n + kind)
    x = rng.standard_normal((rows, n)) * 3 + 0.7
    w = 1 + 0.2 * rng.standard_normal(n)
    gate, bias, res = rng.standard_normal((rows, n)), rng.standard_normal(n), rng.standard_normal((rows, n))
    eps = 1e-5
    f = (lambda z: R.layer_norm(z, 1.0, eps)) if kind == 0 else (lambda z: R.unit_rms(z, eps))
    dx, dw, dg, db, dr, dout = dev(x), dev(w), dev(gate), dev(bias), dev(res), H.DeviceBuffer(4 * rows * n + 256)
    tx, tg, tr, td = (Tensor.contiguous(b.ptr, F32, (n, rows)) for b in (dx, dg, dr, dout))
    check(lib().b200_op_norm(C.byref(tx), dw.ptr, 1, None, None, None, C.byref(td), eps, kind, None))
    assert rel(dout.to_numpy(np.float32, (rows, n)), f(x) * w) < 2e-6
    check(lib().b200_op_norm(C.byref(tx), dw.ptr, 1, C.byref(tg), db.ptr, C.byref(tr), C.byref(td), eps, kind, None))
    assert rel(dout.to_numpy(np.float32, (rows, n)), res + f(x * R.sigmoid(gate + bias)) * w) < 2e-6


def test_norm_weight_per_head():
    rng = np.random.default_rng(3)
    Hh, V, T = 3, 40, 4  # rows are (token, head); the weight has one row per head
    x, w = rng.standard_normal((T * Hh, V)), rng.standard_normal((Hh, V))
    dx, dw, dout = dev(x), dev(w), H.DeviceBuffer(4 * T * Hh * V + 256)
    tx, td = Tensor.contiguous(dx.ptr, F32, (V, T * Hh)), Tensor.contiguous(dout.ptr, F32, (V, T * Hh))
    check(lib().b200_op_norm(C.byref(tx), dw.ptr, Hh, None, None, None, C.byref(td), 1e-6, 1, None))
    want = (R.unit_rms(x, 1e-6).reshape(T, Hh, V) * w[None]).reshape(T * Hh, V)
    assert rel(dout.to_numpy(np.float32, (T * Hh, V)), want) < 2e-6


@pytest.mark.parametrize("n", [48, 320, 2049])
def test_polynorm(n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal((4, n)) * 2
    coef = np.array([0.7, -0.3, 0.25, 0.1])
    dx, dc, dout = dev(x), dev(coef), H.DeviceBuffer(16 * n + 256)
    tx, td = Tensor.contiguous(dx.ptr, F32, (n, 4)), Tensor.contiguous(dout.ptr, F32, (n, 4))
    check(lib().b200_op_polynorm(C.byref(tx), dc.ptr, C.byref(td), 1e-5, None))
    assert rel(dout.to_numpy(np.float32, (4, n)), R.polynorm(x, coef, 1e-5)) < 3e-6


@pytest.mark.parametrize("dims,n", [(8, 8), (6, 10), (16, 16)])
def test_rope_table_in_place_on_a_strided_view(dims, n):
    rng = np.random.default_rng(dims)
    Hh, T, lead = 3, 5, 7  # rows of lead + n values per head; only the last n are rotated (in place)
    pos = np.array([0, 1, 17, 300, 4000])
    x = rng.standard_normal((T, Hh, lead + n))
    scaling = {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 1.0}
    cos, sin = R.rotation_table(dims, 10000.0, scaling, pos)
    freqs = np.arctan2(*R.rotation_table(dims, 10000.0, scaling, [1.0])[::-1])[0]  # angles at position 1 (all below pi)
    want = x.copy()
    want[..., lead:] = R.rotate_interleaved(x[..., lead:], cos, sin, dims)
    dx, dp, df = dev(x), dev(pos, np.int32), dev(freqs)
    t = Tensor.contiguous(dx.ptr + 4 * lead, F32, (n, Hh, T))
    t.nb[1], t.nb[2] = 4 * (lead + n), 4 * (lead + n) * Hh
    mag = 0.1 * math.log(4.0) + 1.0
    check(lib().b200_op_rope_table(C.byref(t), dp.ptr, df.ptr, C.byref(t), dims, 0, mag, None))
    assert rel(dx.to_numpy(np.float32, x.shape), want) < 3e-4  # an f32 angle at position 4000 is rounded by up to 4000 * 2^-24 rad


def test_weighted_sum_and_sigmoid_mul():
    rng = np.random.default_rng(5)
    xs, w = rng.standard_normal((5, 300)), rng.standard_normal(5)
    dxs, dw, dout = dev(xs), dev(w), H.DeviceBuffer(1200 + 256)
    check(lib().b200_op_weighted_sum(dxs.ptr, 300, 3, dw.ptr, dout.ptr, 300, None))  # only the first 3 slices
    assert rel(dout.to_numpy(np.float32, (300,)), w[:3] @ xs[:3]) < 2e-6
    a, b = rng.standard_normal((4, 3, 6)), rng.standard_normal((3, 4, 6))  # a is read through a permuted view
    da, db, dd = dev(a), dev(b), H.DeviceBuffer(4 * 72 + 256)
    ta = Tensor.contiguous(da.ptr, F32, (6, 3, 4))
    ta.ne[1], ta.ne[2], ta.nb[1], ta.nb[2] = 4, 3, ta.nb[2], ta.nb[1]
    tb, td = Tensor.contiguous(db.ptr, F32, (6, 4, 3)), Tensor.contiguous(dd.ptr, F32, (6, 4, 3))
    check(lib().b200_op_sigmoid_mul(C.byref(ta), C.byref(tb), C.byref(td), None))
    assert rel(dd.to_numpy(np.float32, (3, 4, 6)), a.transpose(1, 0, 2) * R.sigmoid(b)) < 2e-6


def run_latent_attn(q_lat, q_rot, rows, cell_seq, cell_pos, tok_seq, tok_pos, sink, scale, window=0, bf16=0):
    T, Hh, KR = q_lat.shape
    Rr = q_rot.shape[-1]
    bufs = [dev(q_lat), dev(q_rot), dev(rows), dev(cell_seq, np.int32), dev(cell_pos, np.int32), dev(tok_seq, np.int32), dev(tok_pos, np.int32)]
    dsink = dev(sink) if sink is not None else None
    out = H.DeviceBuffer(4 * T * Hh * KR + 256)
    a = LatentAttnArgs(q_lat=bufs[0].ptr, q_lat_s_head=KR, q_lat_s_tok=Hh * KR, q_rot=bufs[1].ptr, q_rot_s_head=Rr, q_rot_s_tok=Hh * Rr, cache=bufs[2].ptr,
                       cache_stride=rows.shape[1], cell_seq=bufs[3].ptr, cell_pos=bufs[4].ptr, tok_seq=bufs[5].ptr, tok_pos=bufs[6].ptr,
                       sink=dsink.ptr if dsink else None, dst=out.ptr, dst_s_head=KR, dst_s_tok=Hh * KR, kv_rank=KR, rot_dim=Rr, n_head=Hh, n_tokens=T,
                       n_kv=len(cell_seq), window=window, scale=scale, bf16_products=bf16)
    check(lib().b200_op_latent_attn(C.byref(a), None))
    return out.to_numpy(np.float32, (T, Hh, KR))


@pytest.mark.parametrize("KR,Rr,Hh", [(32, 8, 2), (80, 0, 3), (128, 16, 1), (200, 40, 2)])
@pytest.mark.parametrize("window", [0, 5])
def test_latent_attn_scattered_cells_two_sequences(KR, Rr, Hh, window):
    """Two sequences share the cell table in shuffled order, with free cells between; queries sit at several positions."""
    rng = np.random.default_rng(KR + Rr)
    n_a, n_b, n_cells = 37, 21, 96
    rows = rng.standard_normal((n_cells, KR + Rr))
    perm = rng.permutation(n_cells)
    cell_seq, cell_pos = np.full(n_cells, -1), np.full(n_cells, -1)
    cell_seq[perm[:n_a]], cell_pos[perm[:n_a]] = 4, np.arange(n_a)
    cell_seq[perm[n_a:n_a + n_b]], cell_pos[perm[n_a:n_a + n_b]] = 9, np.arange(n_b)
    toks = [(4, 0), (4, 1), (4, 36), (9, 20), (9, 5), (4, 17)]
    q_lat, q_rot = rng.standard_normal((len(toks), Hh, KR)), rng.standard_normal((len(toks), Hh, max(Rr, 1)))[..., :Rr]
    sink = rng.standard_normal(Hh)
    scale = 0.3 / math.sqrt(KR)
    got = run_latent_attn(q_lat, q_rot, rows, cell_seq, cell_pos, [s for s, _ in toks], [p for _, p in toks], sink, scale, window)
    for i, (s, p) in enumerate(toks):
        seq_rows = np.stack([rows[np.where((cell_seq == s) & (cell_pos == j))[0][0]] for j in range(p + 1)])
        k = np.repeat(seq_rows[:, None, :], Hh, 1)
        q = np.concatenate([q_lat[i], q_rot[i]], -1)[None].repeat(p + 1, 0)
        want = R.sink_softmax_attention(q, k, k[..., :KR], scale, sink, window)[p]
        assert rel(got[i], want) < 1e-5, (i, s, p)


@pytest.mark.parametrize("KR,Rr,Hh,T", [(64, 16, 3, 150), (40, 4, 9, 40), (64, 8, 1, 300), (30, 3, 2, 160)])
def test_latent_attn_prompt_batches(KR, Rr, Hh, T):
    """Many (token, head) pairs: the kernels for prompt batches (heads of a token share staged rows; one head, or rows that are
    not a multiple of 4 floats, take the plain kernel).  Two sequences interleaved in the cell table, every token a query."""
    rng = np.random.default_rng(KR * 7 + Hh)
    n_a = T - T // 3
    n_b = T - n_a
    n_cells = T + 11
    rows = rng.standard_normal((n_cells, KR + Rr))
    perm = rng.permutation(n_cells)
    cell_seq, cell_pos = np.full(n_cells, -1), np.full(n_cells, -1)
    cell_seq[perm[:n_a]], cell_pos[perm[:n_a]] = 1, np.arange(n_a)
    cell_seq[perm[n_a:T]], cell_pos[perm[n_a:T]] = 0, np.arange(n_b)
    toks = [(1, p) for p in range(n_a)] + [(0, p) for p in range(n_b)]
    q_lat, q_rot = rng.standard_normal((T, Hh, KR)), rng.standard_normal((T, Hh, Rr))
    sink = rng.standard_normal(Hh)
    scale = 0.5 / math.sqrt(KR)
    got = run_latent_attn(q_lat, q_rot, rows, cell_seq, cell_pos, [s for s, _ in toks], [p for _, p in toks], sink, scale)
    at = 0
    for sq, n in ((1, n_a), (0, n_b)):
        seq_rows = np.stack([rows[np.where((cell_seq == sq) & (cell_pos == j))[0][0]] for j in range(n)])
        k = np.repeat(seq_rows[:, None, :], Hh, 1)
        q = np.concatenate([q_lat[at:at + n], q_rot[at:at + n]], -1)
        want = R.sink_softmax_attention(q, k, k[..., :KR], scale, sink)
        assert rel(got[at:at + n], want) < 1e-5, sq
        at += n


@pytest.mark.parametrize("KR,Rr,Hh,T,window", [(64, 16, 3, 150, 0), (16, 0, 2, 16, 0), (48, 4, 5, 77, 9), (128, 40, 1, 300, 0), (80, 8, 2, 33, 0), (320, 24, 2, 50, 17)])
def test_latent_attn_prompt_batches_bf16_products(KR, Rr, Hh, T, window):
    """16 tokens or more with bf16 products allowed: the tensor-core kernel (16-token tiles, 16-cell tiles, the last of either
    ragged).  Inputs are bf16 values already, so what remains against the plain statement is the rounding of the weights.
    Two sequences interleaved in a shuffled cell table; free cells hold NaN and must not reach any sum."""
    rng = np.random.default_rng(KR * 5 + T)
    n_a = T - T // 3
    n_b = T - n_a
    n_cells = T + 13
    rows = R.bf16_round(rng.standard_normal((n_cells, KR + Rr))).astype(np.float64)
    perm = rng.permutation(n_cells)
    cell_seq, cell_pos = np.full(n_cells, -1), np.full(n_cells, -1)
    cell_seq[perm[:n_a]], cell_pos[perm[:n_a]] = 1, np.arange(n_a)
    cell_seq[perm[n_a:T]], cell_pos[perm[n_a:T]] = 0, np.arange(n_b)
    toks = [(1, p) for p in range(n_a)] + [(0, p) for p in range(n_b)]
    q_lat = R.bf16_round(rng.standard_normal((T, Hh, KR))).astype(np.float64)
    q_rot = R.bf16_round(rng.standard_normal((T, Hh, max(Rr, 1)))).astype(np.float64)[..., :Rr]
    sink = rng.standard_normal(Hh)
    scale = 1.5 / math.sqrt(KR)
    dirty = rows.copy()
    dirty[perm[T:]] = np.nan
    got = run_latent_attn(q_lat, q_rot, dirty, cell_seq, cell_pos, [s for s, _ in toks], [p for _, p in toks], sink, scale, window, bf16=1)
    exact = run_latent_attn(q_lat, q_rot, dirty, cell_seq, cell_pos, [s for s, _ in toks], [p for _, p in toks], sink, scale, window, bf16=0)
    assert np.isfinite(got).all()
    at = 0
    for sq, n in ((1, n_a), (0, n_b)):
        seq_rows = np.stack([rows[np.where((cell_seq == sq) & (cell_pos == j))[0][0]] for j in range(n)])
        k = np.repeat(seq_rows[:, None, :], Hh, 1)
        q = np.concatenate([q_lat[at:at + n], q_rot[at:at + n]], -1)
        want = R.sink_softmax_attention(q, k, k[..., :KR], scale, sink, window)
        assert rel(exact[at:at + n], want) < 1e-5, sq
        assert rel(got[at:at + n], want) < 6e-3, sq
        assert np.abs(got[at:at + n] - want).mean() < 1e-3 * np.abs(want).mean() + 1e-4, sq  # a wrong cell or row moves far more than rounding does
        at += n


def test_latent_attn_far_key_and_sink_show():
    """One key far back is made to dominate; with the sink left out, or the key masked, the result would move by far more."""
    rng = np.random.default_rng(11)
    KR, Rr, Hh, n = 64, 8, 2, 700
    rows = rng.standard_normal((n, KR + Rr)) * 0.1
    q_lat, q_rot = rng.standard_normal((1, Hh, KR)), rng.standard_normal((1, Hh, Rr))
    rows[3, :KR] = 6.0 * q_lat[0, 0] / np.linalg.norm(q_lat[0, 0])  # head 0 looks at cell 3
    sink = np.array([2.0, 5.0])
    seq, pos = np.zeros(n, int), np.arange(n)
    got = run_latent_attn(q_lat, q_rot, rows, seq, pos, [0], [n - 1], sink, 1.0)
    k = np.repeat(rows[:, None, :], Hh, 1)
    q = np.concatenate([q_lat, q_rot], -1).repeat(n, 0)
    want = R.sink_softmax_attention(q, k, k[..., :KR], 1.0, sink)[n - 1]
    no_sink = R.sink_softmax_attention(q, k, k[..., :KR], 1.0, None)[n - 1]
    assert rel(got[0], want) < 1e-5
    assert rel(no_sink, want) > 1e-2  # the test would see a missing sink


def test_latent_kv_store_rows():
    rng = np.random.default_rng(2)
    KR, Rr, dims, T, n_cells = 48, 12, 8, 6, 20
    dkv, w = rng.standard_normal((T, KR + Rr + 5)), 1 + 0.1 * rng.standard_normal(KR)  # rows with a stride
    pos, cells = np.array([0, 1, 2, 3, 100, 101]), np.array([7, 3, 19, 0, 1, 12])
    freqs = 10000.0 ** (-2.0 * np.arange(dims // 2) / dims)
    ddkv, dw, dp, df, dc, cache = dev(dkv), dev(w), dev(pos, np.int32), dev(freqs), dev(cells, np.int32), H.DeviceBuffer(4 * n_cells * (KR + Rr) + 256, zero=True)
    check(lib().b200_op_latent_kv_store(ddkv.ptr, dkv.shape[1], dw.ptr, dp.ptr, df.ptr, dc.ptr, cache.ptr, KR + Rr, KR, Rr, dims, 1.0, 1e-6, T, None))
    got = cache.to_numpy(np.float32, (n_cells, KR + Rr))
    cos, sin = R.rotation_table(dims, 10000.0, None, pos)
    want = np.zeros_like(got, dtype=np.float64)
    want[cells, :KR] = R.unit_rms(dkv[:, :KR], 1e-6) * w
    want[cells, KR:] = R.rotate_interleaved(dkv[:, KR:KR + Rr], cos, sin, dims)
    assert rel(got, want) < 1e-5


def run_mlstm(q, k, v, ig, fg, ib, fb, cap, info, state, slot_stride):
    T, Hh, D = q.shape
    V = v.shape[-1]
    bufs = [dev(q), dev(k), dev(v), dev(ig), dev(fg), dev(ib), dev(fb), dev(np.asarray(info).T, np.int32)]
    out = H.DeviceBuffer(4 * T * Hh * V + 256)
    a = MlstmArgs(q=bufs[0].ptr, k=bufs[1].ptr, v=bufs[2].ptr, ig=bufs[3].ptr, fg=bufs[4].ptr, q_stride=Hh * D, k_stride=Hh * D, v_stride=Hh * V, g_stride=Hh,
                  i_bias=bufs[5].ptr, f_bias=bufs[6].ptr, seq_info=bufs[7].ptr, n_seq=len(info), state=state.ptr, slot_stride=slot_stride, dst=out.ptr,
                  dst_stride=Hh * V, heads=Hh, dim=D, vdim=V, gate_cap=cap, q_scale=D ** -0.5)
    check(lib().b200_op_mlstm_scan(C.byref(a), None))
    return out.to_numpy(np.float32, (T, Hh, V))


@pytest.mark.parametrize("Hh,D,V", [(2, 16, 24), (1, 32, 64), (3, 24, 40), (2, 80, 33), (1, 160, 8), (4, 8, 500), (9, 40, 450)])
def test_mlstm_scan_whole_against_steps_and_slots(Hh, D, V):
    """Two sequences in one launch (slots 2 and 0), then the same tokens one by one through the carried state, then a slot that
    is used again by a fresh sequence.  The large shapes give enough (head, column tile) pairs for 4 state columns per warp:
    with (4, 8, 500) two sequences in a launch take that form and one sequence the form with 2, on the same state."""
    rng = np.random.default_rng(Hh * 100 + D + V)
    lens = [9, 5]
    T = sum(lens)
    q, k, v = rng.standard_normal((T, Hh, D)), rng.standard_normal((T, Hh, D)), rng.standard_normal((T, Hh, V))
    ig, fg = rng.standard_normal((T, Hh)) * 4, rng.standard_normal((T, Hh)) * 4 + 2
    ib, fb, cap = rng.standard_normal(Hh), rng.standard_normal(Hh), 6.0
    stride = int(lib().b200_mlstm_state_floats(Hh, D, V)) + 3
    want = np.concatenate([R.mlstm_recurrence(q[a:b] * D ** -0.5, k[a:b], v[a:b], ig[a:b] + ib, fg[a:b] + fb, cap)[0] for a, b in ((0, 9), (9, 14))])
    state = H.DeviceBuffer(4 * stride * 3, zero=False)  # never cleared: fresh sequences must not read it
    check(lib().b200_memset(state.ptr, 0x7f, 4 * stride * 3, None))
    got = run_mlstm(q, k, v, ig, fg, ib, fb, cap, [(0, 9, 2, 1), (9, 5, 0, 1)], state, stride)
    assert rel(got, want) < 2e-5
    # token by token: both sequences advance by one token per launch, the shorter one ends earlier
    check(lib().b200_memset(state.ptr, 0x7f, 4 * stride * 3, None))
    steps = np.zeros_like(want)
    for t in range(9):
        idx = [t] + ([9 + t] if t < 5 else [])
        info = [(i, 1, slot, int(t == 0)) for i, slot in zip(range(len(idx)), (2, 0))]
        steps[idx] = run_mlstm(q[idx], k[idx], v[idx], ig[idx], fg[idx], ib, fb, cap, info, state, stride)
    assert rel(steps, want) < 2e-5
    # slot 2 again, by a new sequence
    again = run_mlstm(q[9:], k[9:], v[9:], ig[9:], fg[9:], ib, fb, cap, [(0, 5, 2, 1)], state, stride)
    assert rel(again, want[9:]) < 2e-5


def test_mlstm_scan_column_split_changes_between_launches():
    """A sequence starts alone (few CTAs: 2 state columns per warp), goes on beside a new one (4 per warp), then alone again:
    the state that one form leaves is the state the other reads."""
    rng = np.random.default_rng(77)
    Hh, D, V, na, nb = 4, 8, 500, 8, 4
    T = na + nb
    q, k, v = rng.standard_normal((T, Hh, D)), rng.standard_normal((T, Hh, D)), rng.standard_normal((T, Hh, V))
    ig, fg = rng.standard_normal((T, Hh)) * 3, rng.standard_normal((T, Hh)) * 3 + 1
    ib, fb, cap = rng.standard_normal(Hh), rng.standard_normal(Hh), 9.0
    want = np.concatenate([R.mlstm_recurrence(q[a:b] * D ** -0.5, k[a:b], v[a:b], ig[a:b] + ib, fg[a:b] + fb, cap)[0] for a, b in ((0, na), (na, T))])
    stride = int(lib().b200_mlstm_state_floats(Hh, D, V))
    state = H.DeviceBuffer(4 * stride * 2, zero=False)
    check(lib().b200_memset(state.ptr, 0x7f, 4 * stride * 2, None))
    got = np.zeros_like(want)
    got[0:3] = run_mlstm(q[0:3], k[0:3], v[0:3], ig[0:3], fg[0:3], ib, fb, cap, [(0, 3, 1, 1)], state, stride)
    idx = list(range(3, 6)) + list(range(na, T))
    got[idx] = run_mlstm(q[idx], k[idx], v[idx], ig[idx], fg[idx], ib, fb, cap, [(0, 3, 1, 0), (3, nb, 0, 1)], state, stride)
    got[6:na] = run_mlstm(q[6:na], k[6:na], v[6:na], ig[6:na], fg[6:na], ib, fb, cap, [(0, na - 6, 1, 0)], state, stride)
    assert rel(got, want) < 2e-5


def test_mlstm_gates_saturate_without_overflow():
    rng = np.random.default_rng(8)
    Hh, D, V, T = 1, 16, 16, 300
    q, k, v = rng.standard_normal((T, Hh, D)), rng.standard_normal((T, Hh, D)), rng.standard_normal((T, Hh, V))
    ig, fg = rng.standard_normal((T, Hh)) * 50, rng.standard_normal((T, Hh)) * 50  # far beyond the cap
    stride = int(lib().b200_mlstm_state_floats(Hh, D, V))
    state = H.DeviceBuffer(4 * stride, zero=True)
    got = run_mlstm(q, k, v, ig, fg, np.zeros(Hh), np.zeros(Hh), 8.0, [(0, T, 0, 1)], state, stride)
    want = R.mlstm_recurrence(q * D ** -0.5, k, v, ig, fg, 8.0)[0]
    assert np.isfinite(got).all() and rel(got, want) < 5e-5


@pytest.mark.parametrize("K,M,N", [(64, 5, 1), (320, 37, 3), (4096, 130, 8), (200, 9, 2), (100, 7, 1), (128, 300, 9), (320, 257, 40), (2048, 512, 300), (192, 64, 513),
                                   (96, 21, 5), (200, 9, 4), (32, 16, 8), (2048, 47, 6), (104, 33, 7)])
def test_dense_bf16_matmul(K, M, N):
    """N <= 2: the GEMV with f32 activations (K not a multiple of 8 falls back to the plain kernel); N = 3..8: the tensor-core
    GEMV when K is a multiple of 32 (activations rounded to bf16), else the f32 one; larger N: the tensor-core GEMM, whose
    activations are rounded to bf16."""
    rng = np.random.default_rng(K + M + N)
    w = R.bf16_round(rng.standard_normal((M, K)))
    x = rng.standard_normal((N, K)).astype(np.float32)
    bits = (w.view(np.uint32) >> 16).astype(np.uint16)
    if N <= 8:
        dw, dx, dd = dev(bits, np.uint16), dev(x), H.DeviceBuffer(4 * N * M + 256)
        tw, tx, td = Tensor.contiguous(dw.ptr, BF16, (K, M)), Tensor.contiguous(dx.ptr, F32, (K, N)), Tensor.contiguous(dd.ptr, F32, (M, N))
        check(lib().b200_op_mul_mat_float(C.byref(tw), C.byref(tx), C.byref(td), None))
        xr = R.bf16_round(x) if N >= 3 and K % 32 == 0 else x
        got, want = dd.to_numpy(np.float32, (N, M)), xr.astype(np.float64) @ w.astype(np.float64).T
        assert rel(got, want) < 2e-6
    else:
        got = H.mul_mat_q(BF16, bits.view(np.uint8), x, K, M)
        want = R.bf16_round(x).astype(np.float64) @ w.astype(np.float64).T
        assert rel(got, want) < 2e-6


@pytest.mark.parametrize("K,M,N,B", [(64, 40, 9, 3), (128, 256, 70, 5), (192, 130, 300, 2)])
def test_dense_bf16_matmul_batched(K, M, N, B):
    """One launch for B products; the activations of product b are a strided slice (rows of B * K values), as a per-head view is."""
    rng = np.random.default_rng(K + M + N + B)
    w = R.bf16_round(rng.standard_normal((B, M, K)))
    x = rng.standard_normal((N, B, K)).astype(np.float32)
    bits = (w.view(np.uint32) >> 16).astype(np.uint16)
    dw, dx, dd = dev(bits, np.uint16), dev(x), H.DeviceBuffer(4 * B * N * M + 256)
    ws_bytes = B * int(lib().b200_mul_mat_q_workspace_bytes(BF16, K, M, N))
    ws = H.DeviceBuffer(ws_bytes + 16)
    check(lib().b200_mul_mat_bf16_batched(dw.ptr, 2 * K, 2 * K * M, dx.ptr, B * K, K, dd.ptr, M, N * M, K, M, N, B, ws.ptr, ws_bytes, None))
    got = dd.to_numpy(np.float32, (B, N, M))
    want = np.einsum("nbk,bmk->bnm", R.bf16_round(x).astype(np.float64), w.astype(np.float64))
    assert rel(got, want) < 2e-6
    # the same batch with 1..8 columns goes through the GEMV, one grid row per product
    n8 = min(N, 5)
    tw, tx, td = Tensor.contiguous(dw.ptr, BF16, (K, M, B)), Tensor.contiguous(dx.ptr, F32, (K, n8, B)), Tensor.contiguous(dd.ptr, F32, (M, n8, B))
    tx.nb[1], tx.nb[2] = 4 * B * K, 4 * K
    check(lib().b200_op_mul_mat_float(C.byref(tw), C.byref(tx), C.byref(td), None))
    got = dd.to_numpy(np.float32, (B, n8, M))
    xr = R.bf16_round(x[:n8]) if n8 >= 3 and K % 32 == 0 else x[:n8]
    want = np.einsum("nbk,bmk->bnm", xr.astype(np.float64), w.astype(np.float64))
    assert rel(got, want) < 2e-6


# ------------------------------------------------------------------------------------------------ whole models
from koboldcpp_b200 import genesun as G  # noqa: E402
from koboldcpp_b200.engine import Engine, Request  # noqa: E402

CONFIGS = {
    "mixed": lambda: R.make_config([R.mlstm_layer(), R.attn_layer(), R.attn_layer(kv_from=1, ff=0), R.mlstm_layer(ff=40)]),
    # values the layers could have in common are all different here; one head; rotation over a part of the rotated size; no scaling
    "odd": lambda: R.make_config([R.attn_layer(heads=1, dim=24, rot_dim=12, vdim=40, kv_rank=48, q_rank=20, ff=72, rot_dims=8, scaling=False, base=500.0),
                                  R.mlstm_layer(heads=3, dim=24, vdim=40, gate_cap=4.0, ff=56),
                                  R.attn_layer(heads=3, dim=8, rot_dim=4, vdim=8, kv_rank=40, q_rank=36, ff=0)], width=96, vocab=70, eps=1e-6),
    "attn_only": lambda: R.make_config([R.attn_layer(), R.attn_layer(kv_from=0), R.attn_layer(kv_from=0, ff=0)], width=48),
    "mlstm_only": lambda: R.make_config([R.mlstm_layer(heads=1, dim=32, vdim=64), R.mlstm_layer(ff=32)], width=32, vocab=50),
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
    for t in range(40, 60):
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
    toks = rng.integers(0, cfg["vocab"], 530).tolist()
    want = R.forward(cfg, W, toks)
    eng = Engine(m)
    rows = [eng.step([("x", toks[:250], [0, 1, 249])])]
    places = [0, 1, 249]
    for t in range(250, 530):  # passes 256 and 512 cells
        rows.append(eng.step([("x", [toks[t]], [0])])); places.append(t)
    eng.finish("x")
    assert logits_err(np.concatenate(rows), want[places]) < 2e-4


def test_greedy_generation_through_the_engine(model):
    cfg, W, m = model
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (5, 17, 1, 40)]
    eng = Engine(m, max_step_tokens=24)  # prompts are cut into portions beside decoding requests
    outs = eng.generate([Request(p, 12) for p in prompts])
    for p, out in zip(prompts, outs):
        seq = list(p)
        for tok in out:  # every generated token is the reference's argmax given what came before, or a near tie
            lg = R.forward(cfg, W, seq)[-1]
            top = np.sort(lg)[-2:]
            assert tok == int(np.argmax(lg)) or lg[tok] > top[1] - 1e-3 * (abs(top[1]) + 1), (len(seq), tok)
            seq.append(tok)
        assert len(out) == 12


def test_bfloat16_weights_close_to_float32():
    cfg = CONFIGS["mixed"]()
    W = R.random_weights(cfg, seed=3)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 50).tolist()
    want = R.forward(cfg, W, toks)
    m = G.build(cfg, R.as_tensors(W), dtype="bfloat16", n_ctx=256, n_seq_max=1, max_batch=64)
    eng = Engine(m)
    got = eng.step([("a", toks[:44], range(44))])  # the prompt goes through the tensor-core GEMM ...
    rows = [got] + [eng.step([("a", [t], [0])]) for t in toks[44:]]  # ... single tokens through the GEMV
    m.close()
    # Rounding an activation to bf16 moves a logit row by a few 1e-3 of its spread; a token whose mLSTM normaliser sits at its
    # threshold (the first token of a sequence can) amplifies that, so the bound is on the bulk of the rows, with a loose cap.
    d = np.concatenate(rows) - want
    d = d - d.mean(-1, keepdims=True)
    e = np.sqrt((d ** 2).mean(-1)) / want.std()
    assert np.quantile(e, 0.9) < 2e-2 and e.max() < 0.5


def test_bfloat16_portions_and_batches_agree_with_the_whole_prompt():
    """bf16 serving mode: prompt portions of 16 tokens or more take the tensor-core attention, over cells that earlier portions
    wrote and beside another request's tokens; shorter portions and single tokens take the f32 kernels.  All of them must
    give the logits of the whole prompt up to bf16 rounding."""
    cfg = CONFIGS["mixed"]()
    W = R.random_weights(cfg, seed=5)
    rng = np.random.default_rng(1)
    ta, tb = rng.integers(0, cfg["vocab"], 75).tolist(), rng.integers(0, cfg["vocab"], 41).tolist()
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
    d = np.concatenate(parts) - whole
    d = d - d.mean(-1, keepdims=True)
    e = np.sqrt((d ** 2).mean(-1)) / whole.std()
    assert np.isfinite(e).all() and np.quantile(e, 0.9) < 2e-2 and e.max() < 0.5


def test_far_key_through_the_model():
    """Weights make the attention sharp (large score scale), so a wrong position, mask or cell would show in the logits."""
    cfg = R.make_config([R.attn_layer(heads=2, dim=16, rot_dim=8, kv_rank=32, q_rank=32, ff=0), R.attn_layer(kv_from=0, ff=32)])
    for layer in cfg["layers"]:
        layer["mixer"]["scale"] = 3.0
    W = R.random_weights(cfg, seed=21)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], 640).tolist()
    want = R.forward(cfg, W, toks)
    m = G.build(cfg, R.as_tensors(W), dtype="float32", n_ctx=768, n_seq_max=2, max_batch=640)
    eng = Engine(m)
    places = [0, 1, 2, 255, 256, 257, 511, 512, 600]
    rows = [eng.step([("a", toks[:601], places)])]
    for t in range(601, 640):
        rows.append(eng.step([("a", [toks[t]], [0])])); places.append(t)
    m.close()
    assert logits_err(np.concatenate(rows), want[places]) < 2e-4

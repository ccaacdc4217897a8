"""Medodra on the GPU against the plain float64 statement in medodra_ref.py: every mechanism alone through the C ABI, then whole
models through the loader, the batch step, the sequence cache and the engine (prefill against decoding, portions, mixed
batches, cells and slots that are used again, far keys and bucket edges, greedy generation)."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import pytest

import koboldcpp_b200.host as H
import medodra_ref as R
from koboldcpp_b200.lib import F32, DeltaRuleArgs, MinGruArgs, QkvStoreArgs, ShortConvArgs, SinkAttnArgs, Tensor, check, lib

pytestmark = pytest.mark.gpu


def dev(a, dtype=np.float32):
    return H.DeviceBuffer.from_numpy(np.ascontiguousarray(a, dtype=dtype), pad=256)


def rel(got, want):
    return float(np.abs(got - want).max() / (np.abs(want).max() + 1e-30))


def seq_info(runs):
    """runs: [(first token, count, slot, fresh)] -> the int32 [4][n] table the scans read."""
    return np.array(runs, dtype=np.int32).T.copy()


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("n,T", [(6, 3), (7, 5), (160, 40)])
def test_sinusoid_positions(n, T):
    rng = np.random.default_rng(n)
    x, pos = rng.standard_normal((T, n)), rng.integers(0, 3000, T)
    pos[0] = 0
    freqs = np.array([10000.0 ** (-2.0 * i / n) for i in range((n + 1) // 2)])
    dx, dp, df, dout = dev(x), dev(pos, np.int32), dev(freqs), H.DeviceBuffer(4 * T * n + 256)
    tx, to = Tensor.contiguous(dx.ptr, F32, (n, T)), Tensor.contiguous(dout.ptr, F32, (n, T))
    check(lib().b200_op_add_sinusoid(C.byref(tx), dp.ptr, df.ptr, C.byref(to), None))
    got = dout.to_numpy(np.float32, (T, n))
    assert np.abs(got - (x + R.sinusoid(pos, n))).max() < 3e-4  # an f32 angle near 3000 rad is rounded by up to 3000 * 2^-24
    assert np.abs(got[0] - (x[0] + R.sinusoid([0], n)[0])).max() < 1e-6


def run_short_conv(u, w, bias, portions, taps, act, lead=2):
    """u [T, C] of one sequence, fed in the given portions beside a second sequence that owns another slot; returns y [T, C]."""
    T, Cn = u.shape
    rng = np.random.default_rng(1)
    other = rng.standard_normal((3, Cn))
    tail = dev(np.full((3, max(taps - 1, 1) * Cn + 4), 9.0))  # stale values in every slot: a fresh sequence must not read them
    dw, db = dev(w), dev(bias) if bias is not None else None
    out, done, first_call = np.zeros((T, Cn)), 0, True
    for n in portions:
        row = lead + Cn + 3
        buf = rng.standard_normal((n + 3, row))
        buf[:3, lead:lead + Cn], buf[3:, lead:lead + Cn] = other, u[done:done + n]
        dx, dy = dev(buf), H.DeviceBuffer(4 * (n + 3) * Cn + 256)
        info = dev(seq_info([(0, 3, 0, 1), (3, n, 2, 1 if first_call else 0)]), np.int32)
        a = ShortConvArgs(x=dx.ptr + 4 * lead, x_stride=row, bias=db.ptr if db else None, w=dw.ptr, seq_info=info.ptr, n_seq=2, tail=tail.ptr, slot_stride=max(taps - 1, 1) * Cn + 4,
                          dst=dy.ptr, dst_stride=Cn, channels=Cn, taps=taps, act=act, n_tokens=n + 3)
        check(lib().b200_op_short_conv(C.byref(a), None))
        out[done:done + n] = dy.to_numpy(np.float32, (n + 3, Cn))[3:]
        done, first_call = done + n, False
    return out


@pytest.mark.parametrize("Cn,taps,portions,act", [(5, 4, [11], 0), (130, 4, [1, 1, 1, 2, 3, 40, 1], 1), (70, 2, [33, 2], 0), (9, 1, [4, 3], 1), (40, 7, [2, 2, 2, 70], 0),
                                                  (300, 3, [64, 1, 32], 1), (24, 11, [3, 30, 5, 1], 1), (24, 17, [40], 0)])
def test_short_convolution_whole_and_in_portions(Cn, taps, portions, act):
    rng = np.random.default_rng(Cn + taps)
    T = sum(portions)
    u, w, bias = rng.standard_normal((T, Cn)), rng.standard_normal((Cn, taps)), rng.standard_normal(Cn)
    want, _ = R.short_conv(u + bias, w, np.zeros((taps - 1, Cn)))
    if act:
        want = R.silu(want)
    assert rel(run_short_conv(u, w, bias, portions, taps, act), want) < 3e-6
    assert rel(run_short_conv(u, w, bias, [T], taps, act), want) < 3e-6


def run_delta(q, k, v, a, b, a_log, dt_bias, portions, eps=1e-6):
    """q, k [T, G, D]; v [T, H, V]; a, b [T, H]; one sequence in portions in slot 1 of 2, the other slot full of stale values."""
    T, G, D = q.shape
    Hh, V = v.shape[1], v.shape[2]
    state = dev(np.full((2, Hh * D * V + 8), 5.0))
    dal, ddt = dev(a_log), dev(dt_bias)
    out, done = np.zeros((T, Hh, V)), 0
    for n in portions:
        sl = slice(done, done + n)
        dq, dk, dv, da, db = dev(q[sl].reshape(n, -1)), dev(k[sl].reshape(n, -1)), dev(v[sl].reshape(n, -1)), dev(a[sl]), dev(b[sl])
        dy = H.DeviceBuffer(4 * n * Hh * V + 256)
        info = dev(seq_info([(0, n, 1, 1 if done == 0 else 0)]), np.int32)
        args = DeltaRuleArgs(q=dq.ptr, k=dk.ptr, v=dv.ptr, q_stride=G * D, k_stride=G * D, v_stride=Hh * V, a=da.ptr, b=db.ptr, a_stride=Hh, b_stride=Hh, a_log=dal.ptr, dt_bias=ddt.ptr,
                             seq_info=info.ptr, n_seq=1, state=state.ptr, slot_stride=Hh * D * V + 8, dst=dy.ptr, dst_stride=Hh * V, heads=Hh, kv_heads=G, dim=D, vdim=V, unit_qk=1,
                             unit_eps=eps, q_scale=D ** -0.5)
        check(lib().b200_op_delta_rule_scan(C.byref(args), None))
        out[sl] = dy.to_numpy(np.float32, (n, Hh, V))
        done += n
    return out


def delta_oracle(q, k, v, a, b, a_log, dt_bias):
    T, G, D = q.shape
    Hh, V = v.shape[1], v.shape[2]
    qn, kn = R.unit_vector(q) * D ** -0.5, R.unit_vector(k)
    beta, g = R.sigmoid(b), np.exp(-np.exp(a_log) * R.softplus(a + dt_bias))
    S, o = np.zeros((Hh, D, V)), np.zeros((T, Hh, V))
    for t in range(T):
        for h in range(Hh):
            S[h], o[t, h] = R.delta_rule_step(S[h], qn[t, h // (Hh // G)], kn[t, h // (Hh // G)], v[t, h], beta[t, h], g[t, h])
    return o


@pytest.mark.parametrize("Hh,G,D,V,portions", [(2, 1, 8, 4, [5]), (8, 2, 64, 16, [21]), (4, 4, 40, 20, [1, 1, 2, 17, 16, 1]), (3, 1, 130, 9, [20, 3]), (2, 2, 32, 48, [64, 1, 1])])
def test_gated_delta_rule_whole_and_in_portions(Hh, G, D, V, portions):
    rng = np.random.default_rng(Hh * D + V)
    T = sum(portions)
    q, k, v = rng.standard_normal((T, G, D)), rng.standard_normal((T, G, D)), rng.standard_normal((T, Hh, V))
    a, b, a_log, dt_bias = rng.standard_normal((T, Hh)), rng.standard_normal((T, Hh)), rng.standard_normal(Hh) * 0.5, rng.standard_normal(Hh)
    want = delta_oracle(q, k, v, a, b, a_log, dt_bias)
    assert rel(run_delta(q, k, v, a, b, a_log, dt_bias, portions), want) < 2e-5
    assert rel(run_delta(q, k, v, a, b, a_log, dt_bias, [T]), want) < 2e-5


def test_delta_rule_overwrites_what_a_key_holds():
    """With beta = 1 and no decay, writing v2 under a key that already holds v1 must leave v2 there, not v1 + v2."""
    D, V = 16, 4
    k = np.zeros((3, 1, D)); k[:, 0, 3] = 1.0
    v = np.array([[[1.0, 2.0, 3.0, 4.0]], [[-5.0, 0.5, 7.0, 1.0]], [[0.0, 0.0, 0.0, 0.0]]])
    big = np.full((3, 1), 40.0)  # sigmoid(40) = 1; softplus(-40) = 0: no decay
    got = run_delta(k * 3.0, k * 2.0, v, -big, big, np.zeros(1), np.zeros(1), [3])
    want = np.stack([v[0], v[1], v[2]]) * D ** -0.5
    assert np.abs(got - want).max() < 1e-5


def run_mingru(z, x, g, zb, xb, portions):
    T, Wd = z.shape
    state = dev(np.full((3, Wd + 2), 4.0))
    dzb, dxb = dev(zb), dev(xb)
    out, done = np.zeros((T, Wd)), 0
    for n in portions:
        sl = slice(done, done + n)
        row = 3 * Wd + 1
        buf = np.concatenate([z[sl], x[sl], g[sl], np.zeros((n, 1))], 1)
        dx, dy = dev(buf), H.DeviceBuffer(4 * n * Wd + 256)
        info = dev(seq_info([(0, n, 2, 1 if done == 0 else 0)]), np.int32)
        args = MinGruArgs(z=dx.ptr, x=dx.ptr + 4 * Wd, g=dx.ptr + 8 * Wd, z_stride=row, x_stride=row, g_stride=row, z_bias=dzb.ptr, x_bias=dxb.ptr, seq_info=info.ptr, n_seq=1,
                          state=state.ptr, slot_stride=Wd + 2, dst=dy.ptr, dst_stride=Wd, width=Wd, n_tokens=n)
        check(lib().b200_op_mingru_scan(C.byref(args), None))
        out[sl] = dy.to_numpy(np.float32, (n, Wd))
        done += n
    return out


@pytest.mark.parametrize("Wd,portions", [(5, [7]), (320, [19]), (70, [1, 1, 3, 40, 33, 1]), (33, [200, 2])])
def test_mingru_whole_and_in_portions(Wd, portions):
    rng = np.random.default_rng(Wd)
    T = sum(portions)
    z, x, g, zb, xb = (rng.standard_normal(s) * 2 for s in ((T, Wd), (T, Wd), (T, Wd), (Wd,), (Wd,)))
    zz, cc = R.sigmoid(z + zb), R.mingru_candidate(x + xb)
    S, want = np.zeros(Wd), np.zeros((T, Wd))
    for t in range(T):
        S = (1 - zz[t]) * S + zz[t] * cc[t]
        want[t] = S * R.silu(g[t])
    assert rel(run_mingru(z, x, g, zb, xb, portions), want) < 1e-5
    assert rel(run_mingru(z, x, g, zb, xb, [T]), want) < 1e-5


def test_mingru_candidate_is_continuous_at_zero():
    assert R.mingru_candidate(np.array([0.0]))[0] == 0.5 and abs(R.mingru_candidate(np.array([-1e-9]))[0] - 0.5) < 1e-8


@pytest.mark.parametrize("V,Hh,T", [(16, 5, 5), (20, 3, 2), (130, 2, 3)])
def test_head_norm_with_silu_gate(V, Hh, T):
    """Every head's row: x / rms(x) * w * silu(gate), the gate read from a wider row."""
    rng = np.random.default_rng(V)
    x, gate, w, eps = rng.standard_normal((T, Hh, V)) * 3, rng.standard_normal((T, Hh, V)) * 2, 1 + 0.3 * rng.standard_normal(V), 1e-6
    row = Hh * V + 5
    gbuf = rng.standard_normal((T, row)); gbuf[:, 2:2 + Hh * V] = gate.reshape(T, -1)
    dx, dg, dw, dout = dev(x), dev(gbuf), dev(w), H.DeviceBuffer(4 * T * Hh * V + 256)
    tx, to = Tensor.contiguous(dx.ptr, F32, (V, Hh, T)), Tensor.contiguous(dout.ptr, F32, (V, Hh, T))
    tg = Tensor.contiguous(dg.ptr + 8, F32, (V, Hh, T)); tg.nb[2] = 4 * row
    check(lib().b200_op_norm_affine(C.byref(tx), dw.ptr, 1, None, C.byref(tg), None, 2, None, C.byref(to), eps, 1, None))
    assert rel(dout.to_numpy(np.float32, (T, Hh, V)), R.rms_unit(x, eps) * w * R.silu(gate)) < 3e-6


@pytest.mark.parametrize("n,T", [(40, 3), (70, 1), (1024, 4), (5000, 2)])
def test_two_sides_joined_behind_their_norms(n, T):
    """N(a + bias) * wa + N(b) * wb in one launch, the second input read from a wider row."""
    rng = np.random.default_rng(n)
    a, b2, bias, wa, wb, eps = rng.standard_normal((T, n)) * 4, rng.standard_normal((T, n + 6)), rng.standard_normal(n), rng.standard_normal(n), rng.standard_normal(n), 1e-5
    da, db, dbias, dwa, dwb, dout = dev(a), dev(b2), dev(bias), dev(wa), dev(wb), H.DeviceBuffer(4 * T * n + 256)
    ta, to = Tensor.contiguous(da.ptr, F32, (n, T)), Tensor.contiguous(dout.ptr, F32, (n, T))
    tb = Tensor.contiguous(db.ptr + 8, F32, (n, T)); tb.nb[1] = 4 * (n + 6)
    check(lib().b200_op_norm_pair(C.byref(ta), dwa.ptr, dbias.ptr, C.byref(tb), dwb.ptr, C.byref(to), eps, None))
    want = R.rms_unit(a + bias, eps) * wa + R.rms_unit(b2[:, 2:2 + n], eps) * wb
    assert rel(dout.to_numpy(np.float32, (T, n)), want) < 3e-6


# ------------------------------------------------------------------------------------------------ sigmoid attention with a bias by distance
def distance_table(rel_tab, pb, bias_max):
    """[heads, bias_max + 1]: what the loader hands the kernel (computed here from the oracle's bucket function)."""
    B = rel_tab.shape[0]
    return np.ascontiguousarray(np.stack([rel_tab[R.distance_bucket(n, B, bias_max)] + pb for n in range(bias_max + 1)]).T)


def run_sigmoid_attn(q, kc, vc, cell_seq, cell_pos, tok_seq, tok_pos, scale, G, table, bf16=0):
    T, Hh, D = q.shape
    V = vc.shape[1] // G
    bufs = [dev(q), dev(kc), dev(vc), dev(cell_seq, np.int32), dev(cell_pos, np.int32), dev(tok_seq, np.int32), dev(tok_pos, np.int32), dev(table)]
    out = H.DeviceBuffer(4 * T * Hh * V + 256)
    a = SinkAttnArgs(q=bufs[0].ptr, q_stride=Hh * D, k_cache=bufs[1].ptr, k_cache_stride=kc.shape[1], v_cache=bufs[2].ptr, v_cache_stride=vc.shape[1], cell_seq=bufs[3].ptr,
                     cell_pos=bufs[4].ptr, tok_seq=bufs[5].ptr, tok_pos=bufs[6].ptr, sink=None, dst=out.ptr, dst_stride=Hh * V, n_head=Hh, n_head_kv=G, dim=D, vdim=V, n_tokens=T,
                     n_kv=len(cell_seq), scale=scale, bf16_products=bf16, weights=1, dist_bias=bufs[7].ptr, n_dist=table.shape[1])
    need = int(lib().b200_sink_attn_workspace_bytes(C.byref(a)))  # > 0: few tokens and many cells, the cells are split over CTAs
    ws = H.DeviceBuffer(need + 256) if need else None
    check(lib().b200_op_sink_attn_ws(C.byref(a), ws.ptr if ws else None, need, None))
    got = out.to_numpy(np.float32, (T, Hh, V))
    if need:  # without a workspace the unsplit form must give the same
        check(lib().b200_op_sink_attn(C.byref(a), None))
        assert np.allclose(out.to_numpy(np.float32, (T, Hh, V)), got, rtol=1e-5, atol=1e-6, equal_nan=True)
    return got


def scattered_cache(rng, n_cells, lens, width_k, width_v):
    """Sequences of the given lengths shuffled into one cache; free cells hold NaN."""
    total = sum(lens)
    order = rng.permutation(n_cells)[:total]
    cell_seq, cell_pos = np.full(n_cells, -1), np.full(n_cells, -1)
    at = 0
    for s, n in enumerate(lens):
        cell_seq[order[at:at + n]], cell_pos[order[at:at + n]] = s, np.arange(n)
        at += n
    kc, vc = np.full((n_cells, width_k), np.nan), np.full((n_cells, width_v), np.nan)
    kc[order], vc[order] = rng.standard_normal((total, width_k)), rng.standard_normal((total, width_v))
    return cell_seq, cell_pos, kc, vc


def rows_of_sequence(cell_seq, cell_pos, s, n):
    return [int(np.where((cell_seq == s) & (cell_pos == j))[0][0]) for j in range(n)]


@pytest.mark.parametrize("Hh,G,D,V", [(4, 2, 16, 24), (3, 3, 40, 8), (8, 1, 64, 64), (1, 1, 200, 33)])
@pytest.mark.parametrize("n_cells", [96, 2304])
def test_sigmoid_attn_single_tokens_scattered_cells_two_sequences(Hh, G, D, V, n_cells):
    """The decode form (split over CTAs at 2304 cells): weights are sigmoids, nothing is normalised, the bias follows the distance."""
    rng = np.random.default_rng(Hh + D)
    La, Lb, B, far = 41, 52, 6, 30
    cell_seq, cell_pos, kc, vc = scattered_cache(rng, n_cells, [La, Lb], G * D, G * V)
    rel_tab, pb = rng.standard_normal((B, Hh)) * 2, rng.standard_normal(Hh) - 1
    toks = [(0, La - 1), (1, Lb - 1), (0, 0), (1, 29), (1, 30), (1, 31), (0, 2), (0, 3), (1, 1)]
    q, scale = rng.standard_normal((len(toks), Hh, D)), 1.7 / math.sqrt(D)
    got = run_sigmoid_attn(q, kc, vc, cell_seq, cell_pos, [s for s, _ in toks], [p for _, p in toks], scale, G, distance_table(rel_tab, pb, far))
    for i, (s, p) in enumerate(toks):
        idx = rows_of_sequence(cell_seq, cell_pos, s, p + 1)
        want = R.sigmoid_attention(q[i:i + 1], kc[idx].reshape(-1, G, D), vc[idx].reshape(-1, G, V), [p], np.arange(p + 1), scale, rel_tab, pb, far)[0]
        assert rel(got[i], want) < 2e-5, (i, s, p)


@pytest.mark.parametrize("Hh,G,D,V,T", [(4, 2, 16, 24, 70), (2, 2, 64, 64, 129), (3, 1, 40, 72, 33), (1, 1, 128, 128, 64)])
@pytest.mark.parametrize("bf16", [0, 1])
def test_sigmoid_attn_prompt_batches_behind_cached_tokens(Hh, G, D, V, T, bf16):
    """A portion of T tokens behind P0 cached ones, beside a second sequence in the same cache; f32 products and the tensor cores."""
    rng = np.random.default_rng(T)
    P0, Lb, B, far = 23, 30, 10, 50
    cell_seq, cell_pos, kc, vc = scattered_cache(rng, 256, [Lb, P0 + T], G * D, G * V)
    rel_tab, pb = rng.standard_normal((B, Hh)), rng.standard_normal(Hh) - 2
    q, scale = rng.standard_normal((T, Hh, D)), 1.3 / math.sqrt(D)
    pos = list(range(P0, P0 + T))
    got = run_sigmoid_attn(q, kc, vc, cell_seq, cell_pos, [1] * T, pos, scale, G, distance_table(rel_tab, pb, far), bf16)
    idx = rows_of_sequence(cell_seq, cell_pos, 1, P0 + T)
    src = (lambda a: R.bf16_round(a).astype(np.float64)) if bf16 else (lambda a: a)
    want = R.sigmoid_attention(src(q), src(kc[idx]).reshape(-1, G, D), src(vc[idx]).reshape(-1, G, V), pos, np.arange(P0 + T), scale, rel_tab, pb, far)
    assert rel(got, want) < (2e-2 if bf16 else 2e-5)


@pytest.mark.parametrize("T,bf16", [(1, 0), (40, 0), (40, 1)])
def test_sigmoid_attn_bucket_edges_and_a_far_key(T, bf16):
    """All scores are far below zero except where one bucket's bias lifts them: the result is the sum of the values at exactly the
    distances of that bucket.  Then one loud key hundreds of positions back, beyond the table's last row."""
    rng = np.random.default_rng(5)
    G, D, V, n, B, far = 1, 32, 16, 700, 8, 64
    k, v = np.zeros((n, G, D)), rng.standard_normal((n, G, V))
    q = np.zeros((T, 1, D))
    cell_seq, cell_pos = np.zeros(n, dtype=np.int64), np.arange(n)
    edges = [R.distance_bucket(d, B, far) for d in range(n)]
    for bucket in range(B):
        rel_tab = np.full((B, 1), -60.0); rel_tab[bucket] = 60.0
        got = run_sigmoid_attn(q, k.reshape(n, -1), v.reshape(n, -1), cell_seq, cell_pos, [0] * T, [n - 1] * T, 1.0, G, distance_table(rel_tab, np.zeros(1), far), bf16)
        members = [n - 1 - d for d in range(n) if edges[d] == bucket]
        want = v[members, 0].sum(0)
        assert np.abs(got[:, 0] - want).max() < (0.05 * len(members) ** 0.5 if bf16 else 1e-3), bucket
    rel_tab = np.zeros((B, 1))
    qv = rng.standard_normal(D)
    q[:] = qv
    k[37, 0] = qv * 3.0  # position 37 seen from position 699
    got = run_sigmoid_attn(q, k.reshape(n, -1), v.reshape(n, -1), cell_seq, cell_pos, [0] * T, [n - 1] * T, 1.0, G, distance_table(rel_tab, np.full(1, -30.0), far), bf16)
    assert np.abs(got[:, 0] - v[37, 0]).max() < (2e-2 if bf16 else 1e-4)


def test_store_with_query_temperature_and_value_norm():
    rng = np.random.default_rng(2)
    T, Hh, G, D, V, n_cells, eps = 6, 4, 2, 12, 20, 16, 1e-5
    q, k, v = rng.standard_normal((T, Hh, D)), rng.standard_normal((T, G, D)), rng.standard_normal((T, G, V)) * 3
    v[:, 0] *= 10.0  # a loud head must not move the other head's scale
    pos, cells = np.array([0, 5, 6, 12, 13, 700]), np.array([5, 0, 15, 7, 8, 2])
    coef, every = 0.5, 7
    dq, dk, dv, dp, dc = dev(q), dev(k), dev(v), dev(pos, np.int32), dev(cells, np.int32)
    kc, vc = dev(np.full((n_cells, G * D), 7.0)), dev(np.full((n_cells, G * V), 7.0))
    a = QkvStoreArgs(q=dq.ptr, q_stride=Hh * D, k=dk.ptr, k_stride=G * D, v=dv.ptr, v_stride=G * V, pos=dp.ptr, cells=dc.ptr, freqs=None, k_cache=kc.ptr, k_cache_stride=G * D,
                     v_cache=vc.ptr, v_cache_stride=G * V, n_head=Hh, n_head_kv=G, dim=D, vdim=V, n_dims=0, n_tokens=T, eps=eps, v_unit_rms=1, q_temp_coef=coef, q_temp_every=every)
    check(lib().b200_op_qkv_store(C.byref(a), None))
    temp = np.array([R.query_temperature(p, coef, every) for p in pos])
    assert temp[0] == temp[1] == 1.0 and temp[2] > 1.0 and temp[3] == temp[2] and temp[4] > temp[3]  # a step wherever pos + 1 is a multiple of `every`
    assert rel(dq.to_numpy(np.float32, (T, Hh, D)), q * temp[:, None, None]) < 3e-6
    assert rel(kc.to_numpy(np.float32, (n_cells, G, D))[cells], k) < 1e-6
    assert rel(vc.to_numpy(np.float32, (n_cells, G, V))[cells], R.rms_unit(v, eps)) < 3e-6


def test_scaled_activation_and_combine_with_shared_expert():
    rng = np.random.default_rng(8)
    F, NU, T, n = 24, 3, 5, 40
    gu, w = rng.standard_normal((T, NU, 2 * F)), rng.uniform(0.1, 1.0, (T, NU))
    dgu, dw, dact = dev(gu), dev(w), H.DeviceBuffer(4 * T * NU * F + 256)
    ta, tb = (Tensor.contiguous(dgu.ptr + off, F32, (F, NU, T)) for off in (0, 4 * F))
    for t in (ta, tb):
        t.nb[1], t.nb[2] = 8 * F, 8 * F * NU
    tw, td = Tensor.contiguous(dw.ptr, F32, (NU, T)), Tensor.contiguous(dact.ptr, F32, (F, NU, T))
    check(lib().b200_op_glu_scaled(0, C.byref(ta), C.byref(tb), C.byref(tw), C.byref(td), 0.0, 0.0, None))
    g, u = gu[..., :F] * w[..., None], gu[..., F:] * w[..., None]
    assert rel(dact.to_numpy(np.float32, (T, NU, F)), R.silu(g) * u) < 3e-6
    y, res, mix, sh, sg, mult = rng.standard_normal((T, NU, n)), rng.standard_normal((T, n)), rng.standard_normal((T, n)), rng.standard_normal((T, n)), rng.standard_normal((T, 3)), 0.6
    dy, dr, dm, dsh, dsg, dout = dev(y), dev(res), dev(mix), dev(sh), dev(sg), H.DeviceBuffer(4 * T * (n + 2) + 256)
    check(lib().b200_op_moe_combine_shared(dy.ptr, n, NU * n, None, 0, dr.ptr, n, dm.ptr, n, dsh.ptr, n, dsg.ptr + 4, 3, mult, dout.ptr, n + 2, n, NU, T, None))
    want = res + mult * (mix + y.sum(1) + sh * R.sigmoid(sg[:, 1:2]))
    assert rel(dout.to_numpy(np.float32, (T, n + 2))[:, :n], want) < 3e-6
    check(lib().b200_op_moe_combine_shared(None, 0, 0, None, 0, dr.ptr, n, dm.ptr, n, None, 0, None, 0, mult, dout.ptr, n + 2, n, 0, T, None))  # a layer without a feed-forward
    assert rel(dout.to_numpy(np.float32, (T, n + 2))[:, :n], res + mult * mix) < 3e-6


# ------------------------------------------------------------------------------------------------ whole models
from koboldcpp_b200 import medodra as M  # noqa: E402
from koboldcpp_b200.engine import Engine, Request  # noqa: E402

CONFIGS = {
    # the looped stretch holds one layer of each kind; bias tables shorter than the prompts; 4 heads over 2 kv heads
    "looped": lambda: R.make_config([R.parallel_layer(), R.delta_layer(), R.parallel_layer(heads=2, kv_heads=2, dim=8, vdim=8, conv=2, bias_max=9, every=5, mlp=None),
                                     R.delta_layer(heads=2, kv_heads=1, dim=8, vdim=12, conv=3)], loop=(1, 3, 4)),
    # a delta layer first and the loop from layer 0, run once; one head, one kv head, one expert per token and all experts per token, no
    # shared expert, a convolution of one tap and of six, dim != vdim, multipliers of exactly one, a width that is no multiple of 8
    "odd": lambda: R.make_config([R.delta_layer(heads=1, kv_heads=1, dim=24, vdim=40, conv=1, mlp=R.moe_cfg(ff=40, experts=5, top=1, shared=0)),
                                  R.parallel_layer(heads=1, kv_heads=1, dim=40, vdim=6, conv=6, bias_max=300, coef=0.0, every=1, side=5, mlp=R.moe_cfg(ff=8, experts=3, top=3, shared=10)),
                                  R.delta_layer(heads=6, kv_heads=6, dim=10, vdim=6, conv=2, mlp=None)],
                                 width=70, vocab=70, eps=1e-6, embed_scale=1.0, residual_mult=1.0, loop=(0, 2, 1)),
    # sizes that take the 16-byte and tensor-core paths: width and ff multiples of 64; no loop at all
    "aligned": lambda: R.make_config([R.parallel_layer(heads=4, kv_heads=4, dim=32, vdim=32, conv=4, bias_max=24, side=128, mlp=R.moe_cfg(ff=64, experts=8, top=2, shared=64)),
                                      R.delta_layer(heads=4, kv_heads=1, dim=64, vdim=32, conv=4, mlp=R.moe_cfg(ff=64, experts=4, top=1, shared=128))], width=128, vocab=96,
                                     residual_mult=1.5),
}


@pytest.fixture(scope="module", params=list(CONFIGS))
def model(request):
    cfg = CONFIGS[request.param]()
    W = R.random_weights(cfg, seed=len(request.param))
    m = M.build(cfg, R.as_tensors(W), dtype="float32", n_ctx=768, n_seq_max=4, max_batch=400)
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
    want = R.logits(cfg, W, toks)
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
    toks = rng.integers(0, cfg["vocab"], 70).tolist()
    want = R.logits(cfg, W, toks)
    eng = Engine(m)
    rows = []
    for a in range(0, 40, portion):  # portions shorter than a convolution's tail, and longer than a scan's chunk
        b = min(a + portion, 40)
        rows.append(eng.step([("p", toks[a:b], range(b - a))]))
    for t in range(40, 70):
        rows.append(eng.step([("p", [toks[t]], [0])]))
    eng.finish("p")
    assert logits_err(np.concatenate(rows), want) < 1e-4


def test_unequal_batch_then_decode_together_and_reuse(model):
    """Three requests of different lengths start in one batch and decode together; the shortest ends first and its cells and
    slot (convolution tails and recurrent states with what it left there) go to a new request that joins while the others decode."""
    cfg, W, m = model
    rng = np.random.default_rng(4)
    lens = {"a": (1, 12), "b": (23, 30), "c": (57, 70)}  # prompt length, total length
    toks = {k: rng.integers(0, cfg["vocab"], n).tolist() for k, (_, n) in lens.items()}
    toks["d"] = rng.integers(0, cfg["vocab"], 31).tolist()
    want = {k: R.logits(cfg, W, v) for k, v in toks.items()}
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
    want = R.logits(cfg, W, toks)
    eng = Engine(m)
    rows = [eng.step([("x", toks[:230], [0, 1, 229])])]
    places = [0, 1, 229]
    for t in range(230, 300):  # passes 256 cells; every distance bucket's edge is crossed by decoded tokens
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
            lg = R.logits(cfg, W, seq)[-1]
            top = np.sort(lg)[-2:]
            assert tok == int(np.argmax(lg)) or lg[tok] > top[1] - 1e-3 * (abs(top[1]) + 1), (len(seq), tok)
            seq.append(tok)
        assert len(out) == 10


@pytest.mark.parametrize("name", ["looped", "aligned"])
def test_bfloat16_portions_batches_and_decoding_agree_with_float32(name):
    """bf16 serving mode: prompt portions of 16 tokens or more take the tensor-core kernels (attention and expert products), over
    cells that earlier portions wrote and beside another request's tokens; shorter portions and single tokens take the f32 kernels.
    All of them must give the logits of the float64 reference up to bf16 rounding."""
    cfg = CONFIGS[name]()
    W = R.random_weights(cfg, seed=5)
    rng = np.random.default_rng(1)
    ta, tb = rng.integers(0, cfg["vocab"], 75).tolist(), rng.integers(0, cfg["vocab"], 41).tolist()
    want = R.logits(cfg, W, ta)
    m = M.build(cfg, R.as_tensors(W), dtype="bfloat16", n_ctx=256, n_seq_max=2, max_batch=128)
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


def test_far_key_and_bucket_edges_through_the_model():
    """A large score scale makes the attention side sharp, so a wrong position, distance row or cell would show in the logits; the
    table's last row (distance 100) lies inside the prompt, the prompt's end is no multiple of any block size, and the decoded stretch
    crosses the cache padding."""
    cfg = R.make_config([R.parallel_layer(heads=2, kv_heads=1, dim=16, vdim=16, conv=2, bias_max=100, scale=2.0, every=64, mlp=None),
                         R.delta_layer(heads=2, kv_heads=2, dim=16, vdim=8, conv=4, mlp=None),
                         R.parallel_layer(heads=2, kv_heads=2, dim=16, vdim=8, conv=4, bias_max=17, scale=2.0, every=3)])
    W = R.random_weights(cfg, seed=21, rel_rows=12)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], 290).tolist()
    want = R.logits(cfg, W, toks)
    m = M.build(cfg, R.as_tensors(W), dtype="float32", n_ctx=512, n_seq_max=2, max_batch=300)
    eng = Engine(m)
    places = [0, 1, 2, 5, 6, 7, 17, 18, 99, 100, 101, 102, 200, 201, 241]
    rows = [eng.step([("a", toks[:242], places)])]
    for t in range(242, 290):
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
    cfg = CONFIGS["looped"]()
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
            lg = R.logits(cfg, W, seq)[-1]
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
    wa, wb = R.logits(cfg, W, ta), R.logits(cfg, W, tb)
    want = {0: np.stack([wa[0], wa[10], wb[5]]), 1: wb[6:7], 2: np.stack([wa[12], wb[7]]), 3: wa[13:14]}
    for n, w in want.items():
        got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        assert got.shape == w.shape and logits_err(got, w) < 1e-4, n

"""Zevopel on the GPU against the plain float64 statement in zevopel_ref.py: every mechanism alone through the C ABI, then whole
models through the loader, the batch step, the sequence cache and the engine (prefill against decoding, portions, mixed
batches, cells and slots that are used again, chunk borders inside prompts and inside decoded stretches, greedy generation)."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import pytest

import koboldcpp_b200.host as H
import zevopel_ref as R
from koboldcpp_b200.lib import F32, QkvStoreArgs, SinkAttnArgs, Tensor, check, lib

pytestmark = pytest.mark.gpu


def dev(a, dtype=np.float32):
    return H.DeviceBuffer.from_numpy(np.ascontiguousarray(a, dtype=dtype), pad=256)


def rel(got, want):
    return float(np.abs(got - want).max() / (np.abs(want).max() + 1e-30))


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("n,rows", [(40, 5), (72, 1), (320, 3), (5000, 2)])
def test_norm_behind_a_sublayer_with_scales_and_residual(n, rows):
    """res + c * a * (1 + w) * y / rms(y): the product hands the norm op ONE weight vector c * a * (1 + w)."""
    rng = np.random.default_rng(n)
    y, res = rng.standard_normal((rows, n)) * 3 + 0.4, rng.standard_normal((rows, n))
    w, a, c, eps = 0.2 * rng.standard_normal(n), 1 + 0.3 * rng.standard_normal(n), 0.6, 1e-6
    want = res + c * a * R.rms_norm_one_plus(y, w, eps)
    folded = ((1.0 + w.astype(np.float32)) * a.astype(np.float32) * np.float32(c)).astype(np.float32)
    dy, dr, dw, dout = dev(y), dev(res), dev(folded), H.DeviceBuffer(4 * rows * n + 256)
    ty, tr, td = (Tensor.contiguous(t.ptr, F32, (n, rows)) for t in (dy, dr, dout))
    check(lib().b200_op_norm_affine(C.byref(ty), dw.ptr, 1, None, None, None, 0, C.byref(tr), C.byref(td), eps, 1, None))
    assert rel(dout.to_numpy(np.float32, (rows, n)), want) < 3e-6


def run_qkv_store(q, k, v, qn, kn, pos, cells, rot, n_cells, eps, lead=3):
    """q, k, v [T, heads, size] are handed over as column ranges of one wider row, as the fused projection leaves them."""
    T, Hh, D = q.shape
    G, V = k.shape[1], v.shape[2]
    row = lead + Hh * D + G * D + G * V + 5
    buf = np.random.default_rng(0).standard_normal((T, row))
    oq, ok, ov = lead, lead + Hh * D, lead + Hh * D + G * D
    buf[:, oq:ok], buf[:, ok:ov], buf[:, ov:ov + G * V] = q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)
    d, dqn, dkn = dev(buf), dev(qn), dev(kn)
    dp, dc, df = dev(pos, np.int32), dev(cells, np.int32), dev(R.rotation_freqs(rot) if rot["dims"] else np.zeros(1))
    kc, vc = dev(np.full((n_cells, G * D + 2), 7.0)), dev(np.full((n_cells, G * V + 1), 7.0))
    a = QkvStoreArgs(q=d.ptr + 4 * oq, q_stride=row, k=d.ptr + 4 * ok, k_stride=row, v=d.ptr + 4 * ov, v_stride=row, q_norm=dqn.ptr, k_norm=dkn.ptr, pos=dp.ptr, cells=dc.ptr,
                     freqs=df.ptr, k_cache=kc.ptr, k_cache_stride=G * D + 2, v_cache=vc.ptr, v_cache_stride=G * V + 1, n_head=Hh, n_head_kv=G, dim=D, vdim=V, n_dims=rot["dims"],
                     n_tokens=T, eps=eps, norm_per_head=1, rope_halves=1)
    check(lib().b200_op_qkv_store(C.byref(a), None))
    out = d.to_numpy(np.float32, (T, row))
    assert np.array_equal(out[:, :lead], buf[:, :lead].astype(np.float32)) and np.array_equal(out[:, ok:], buf[:, ok:].astype(np.float32))  # only q is rewritten
    return out[:, oq:ok].reshape(T, Hh, D), kc.to_numpy(np.float32, (n_cells, G * D + 2)), vc.to_numpy(np.float32, (n_cells, G * V + 1))


@pytest.mark.parametrize("Hh,G,D,V,dims", [(4, 2, 16, 24, 8), (3, 3, 10, 6, 10), (1, 1, 64, 64, 32), (6, 2, 96, 40, 0), (40, 8, 12, 4, 6), (2, 1, 130, 8, 64)])
def test_qkv_store_norm_per_head_and_rotation_of_halves(Hh, G, D, V, dims):
    rng = np.random.default_rng(Hh * D + V)
    T, n_cells, eps = 7, 20, 1e-5
    q, k, v = rng.standard_normal((T, Hh, D)), rng.standard_normal((T, G, D)), rng.standard_normal((T, G, V))
    q[:, 0] *= 9.0  # one loud head must not leak into the scale of the others
    pos, cells = np.array([0, 1, 2, 95, 96, 4000, 3]), np.array([5, 0, 19, 7, 8, 2, 11])
    rot = {"base": 3000.0, "dims": dims, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    qn, kn = 1 + 0.3 * rng.standard_normal(D), 1 + 0.3 * rng.standard_normal(D)
    gq, kc, vc = run_qkv_store(q, k, v, qn, kn, pos, cells, rot, n_cells, eps)
    wq, wk = R.rotate_halves(R.rms_norm_plain(q, qn, eps), pos, rot), R.rotate_halves(R.rms_norm_plain(k, kn, eps), pos, rot)
    tol = 3e-4  # an f32 angle at position 4000 is rounded by up to 4000 * 2^-24 rad
    assert rel(gq, wq) < tol
    assert rel(kc[cells, :G * D], wk.reshape(T, -1)) < tol and rel(vc[cells, :G * V], v.reshape(T, -1)) < 3e-6
    untouched = np.setdiff1d(np.arange(n_cells), cells)
    assert (kc[untouched] == 7.0).all() and (vc[untouched] == 7.0).all() and (kc[:, G * D:] == 7.0).all() and (vc[:, G * V:] == 7.0).all()


def test_rotation_frequencies_by_band():
    """All three bands occur with these numbers; the values are written out by hand from the rule."""
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}}
    f = [1.0, 100 ** -0.25, 0.1, 100 ** -0.75]  # wavelengths 6.28, 19.9, 62.8, 198.7 against the borders 10 and 40
    s = (40 / (2 * math.pi / f[1]) - 1.0) / 3.0
    want = [f[0], (1 - s) * f[1] / 4 + s * f[1], f[2] / 4, f[3] / 4]
    assert np.allclose(R.rotation_freqs(rot), want, rtol=1e-12)


def run_sink_attn(q, kc, vc, cell_seq, cell_pos, tok_seq, tok_pos, sink, scale, G, chunk=0, gate=None, bf16=0):
    T, Hh, D = q.shape
    V = vc.shape[1] // G
    bufs = [dev(q), dev(kc), dev(vc), dev(cell_seq, np.int32), dev(cell_pos, np.int32), dev(tok_seq, np.int32), dev(tok_pos, np.int32)]
    dsink = dev(sink) if sink is not None else None
    gs = Hh + 3  # the gates are columns of a wider row
    dgate = dev(np.concatenate([gate, np.full((T, 3), np.nan)], 1)) if gate is not None else None
    out = H.DeviceBuffer(4 * T * Hh * V + 256)
    a = SinkAttnArgs(q=bufs[0].ptr, q_stride=Hh * D, k_cache=bufs[1].ptr, k_cache_stride=kc.shape[1], v_cache=bufs[2].ptr, v_cache_stride=vc.shape[1], cell_seq=bufs[3].ptr,
                     cell_pos=bufs[4].ptr, tok_seq=bufs[5].ptr, tok_pos=bufs[6].ptr, sink=dsink.ptr if dsink else None, dst=out.ptr, dst_stride=Hh * V, n_head=Hh, n_head_kv=G,
                     dim=D, vdim=V, n_tokens=T, n_kv=len(cell_seq), scale=scale, bf16_products=bf16, chunk=chunk, gate=dgate.ptr if dgate else None, gate_stride=gs)
    need = int(lib().b200_sink_attn_workspace_bytes(C.byref(a)))  # > 0: few tokens and many cells, the cells are split over CTAs
    ws = H.DeviceBuffer(need + 256) if need else None
    check(lib().b200_op_sink_attn_ws(C.byref(a), ws.ptr if ws else None, need, None))
    got = out.to_numpy(np.float32, (T, Hh, V))
    if need:  # without a workspace the unsplit form must give the same
        check(lib().b200_op_sink_attn(C.byref(a), None))
        assert np.allclose(out.to_numpy(np.float32, (T, Hh, V)), got, rtol=1e-5, atol=1e-6, equal_nan=True)
    return got


def one_token_reference(q_t, kc, vc, cell_seq, cell_pos, s, p, sink, scale, G, chunk):
    """The sequence's rows in position order, then the dense reference; returns the row of position p."""
    D, V = q_t.shape[1], vc.shape[1] // G
    idx = [int(np.where((cell_seq == s) & (cell_pos == j))[0][0]) for j in range(p + 1)]
    k, v = kc[idx].reshape(p + 1, G, D), vc[idx].reshape(p + 1, G, V)
    return R.sink_attention(np.repeat(q_t[None], p + 1, 0), k, v, scale, sink, chunk)[p]


@pytest.mark.parametrize("Hh,G,D,V", [(4, 2, 16, 24), (3, 3, 40, 8), (8, 1, 64, 64), (1, 1, 200, 33)])
@pytest.mark.parametrize("chunk", [0, 1, 5, 37])
@pytest.mark.parametrize("n_cells", [96, 2304])
def test_sink_attn_chunks_gates_scattered_cells_two_sequences(Hh, G, D, V, chunk, n_cells):
    """Single tokens (the decode form, split over CTAs at 2304 cells) of two sequences whose cells are shuffled into one cache;
    free cells hold NaN."""
    rng = np.random.default_rng(Hh + D + chunk)
    La, Lb = 41, 52
    order = rng.permutation(n_cells)[:La + Lb]
    cell_seq, cell_pos = np.full(n_cells, -1), np.full(n_cells, -1)
    cell_seq[order[:La]], cell_pos[order[:La]] = 0, np.arange(La)
    cell_seq[order[La:]], cell_pos[order[La:]] = 1, np.arange(Lb)
    kc, vc = np.full((n_cells, G * D), np.nan), np.full((n_cells, G * V), np.nan)
    kc[order], vc[order] = rng.standard_normal((La + Lb, G * D)), rng.standard_normal((La + Lb, G * V))
    toks = [(0, La - 1), (1, Lb - 1), (0, 0), (1, 36), (1, 37), (0, 4), (0, 5), (1, 1)]
    q = rng.standard_normal((len(toks), Hh, D))
    sink, gate, scale = rng.standard_normal(Hh), rng.standard_normal((len(toks), Hh)) * 2, 1.7 / math.sqrt(D)
    got = run_sink_attn(q, kc, vc, cell_seq, cell_pos, [s for s, _ in toks], [p for _, p in toks], sink, scale, G, chunk, gate)
    for i, (s, p) in enumerate(toks):
        want = one_token_reference(q[i], kc, vc, cell_seq, cell_pos, s, p, sink, scale, G, chunk) * R.sigmoid(gate[i])[:, None]
        assert rel(got[i], want) < 2e-5, (i, s, p)


@pytest.mark.parametrize("Hh,G,D,V,T", [(4, 2, 16, 24, 70), (2, 2, 64, 64, 129), (3, 1, 40, 72, 33), (1, 1, 128, 128, 64)])
@pytest.mark.parametrize("chunk", [0, 16, 29])
@pytest.mark.parametrize("bf16", [0, 1])
def test_sink_attn_prompt_batches_behind_cached_tokens(Hh, G, D, V, T, chunk, bf16):
    """A portion of T tokens at positions P0 .. P0 + T - 1 behind P0 cached ones, beside a second sequence in the same cache."""
    rng = np.random.default_rng(T + chunk)
    P0, Lb = 23, 30
    n_cells = 256
    order = rng.permutation(n_cells)[:P0 + T + Lb]
    cell_seq, cell_pos = np.full(n_cells, -1), np.full(n_cells, -1)
    cell_seq[order[:P0 + T]], cell_pos[order[:P0 + T]] = 1, np.arange(P0 + T)
    cell_seq[order[P0 + T:]], cell_pos[order[P0 + T:]] = 0, np.arange(Lb)
    kc, vc = np.full((n_cells, G * D), np.nan), np.full((n_cells, G * V), np.nan)
    kc[order], vc[order] = rng.standard_normal((P0 + T + Lb, G * D)), rng.standard_normal((P0 + T + Lb, G * V))
    q = rng.standard_normal((T, Hh, D))
    sink, gate, scale = rng.standard_normal(Hh), rng.standard_normal((T, Hh)), 1.3 / math.sqrt(D)
    got = run_sink_attn(q, kc, vc, cell_seq, cell_pos, [1] * T, list(range(P0, P0 + T)), sink, scale, G, chunk, gate, bf16)
    idx = order[:P0 + T]
    qq = np.concatenate([np.zeros((P0, Hh, D)), q])
    src = (lambda a: R.bf16_round(a).astype(np.float64)) if bf16 else (lambda a: a)
    want = R.sink_attention(src(qq), src(kc[idx]).reshape(-1, G, D), src(vc[idx]).reshape(-1, G, V), scale, sink, chunk)[P0:] * R.sigmoid(gate)[:, :, None]
    assert rel(got, want) < (2e-2 if bf16 else 2e-5)


@pytest.mark.parametrize("T,bf16", [(1, 0), (40, 0), (40, 1)])
def test_sink_attn_one_loud_key_at_the_chunk_border_and_a_sink_that_takes_all(T, bf16):
    """The key of one position scores far above the rest, so whether it is seen decides the result: the first position of the
    query's chunk is seen, the one before it is not; T = 1 is the decode form, T = 40 the prompt form (all queries at one place),
    with f32 products and on the tensor cores."""
    rng = np.random.default_rng(3)
    G, D, V, n, chunk = 1, 32, 16, 600, 128
    k, v = rng.standard_normal((n, G, D)) * 0.1, rng.standard_normal((n, G, V))
    qv = rng.standard_normal(D)
    q = np.repeat(qv[None, None], T, 0).reshape(T, 1, D)
    cell_seq, cell_pos = np.zeros(n, dtype=np.int64), np.arange(n)
    for query_pos, loud, seen in [(599, 512, True), (599, 511, False), (512, 512, True), (511, 384, True), (511, 383, False), (127, 0, True), (128, 127, False)]:
        kk = k.copy()
        kk[loud, 0] = qv * 4.0
        got = run_sink_attn(q, kk.reshape(n, -1), v.reshape(n, -1), cell_seq, cell_pos, [0] * T, [query_pos] * T, np.array([-1.0]), 1.0, G, chunk, None, bf16)
        if seen:
            assert rel(got[:, 0], np.repeat(v[loud], T, 0)) < (1e-2 if bf16 else 1e-3), (query_pos, loud)
        else:
            assert np.abs(got[:, 0] - v[loud, 0]).max() > 0.3, (query_pos, loud)
    got = run_sink_attn(q, k.reshape(n, -1), v.reshape(n, -1), cell_seq, cell_pos, [0] * T, [599] * T, np.array([40.0]), 1.0, G, chunk, None, bf16)
    assert np.abs(got).max() < 1e-9  # the sink holds the whole weight and has no value


def run_route(z, top, score, keep, scale=1.0):
    T, E = z.shape
    dz, di, dw = dev(z), H.DeviceBuffer(4 * T * top + 256), H.DeviceBuffer(4 * T * top + 256)
    check(lib().b200_op_moe_route_scored(dz.ptr, E, None, di.ptr, top, dw.ptr, top, E, top, 1, 1, scale, score, keep, T, None))
    return di.to_numpy(np.int32, (T, top)), dw.to_numpy(np.float32, (T, top))


@pytest.mark.parametrize("E,top", [(16, 3), (6, 2), (8, 1), (5, 5), (64, 8), (256, 6), (40, 32), (33, 4)])
def test_router_softmax_over_all_experts_scores_kept(E, top):
    rng = np.random.default_rng(E + top)
    T = 50
    z = (rng.standard_normal((T, E)) * 3).astype(np.float32)
    z[7] = 0.25  # all equal: the lowest indices, each with weight 1 / E
    z[8, :] = -80.0; z[8, E - 1] = 60.0  # one expert holds everything
    ids, w = run_route(z, top, 1, 1)
    for t in range(T):
        chosen, ww = R.softmax_router(z[t].astype(np.float64), top)
        if list(ids[t]) != chosen:  # only a near tie of two f32 scores may differ
            a, b = sorted(set(ids[t]) ^ set(chosen))[:2]
            assert abs(z[t, a] - z[t, b]) < 1e-5 or max(z[t, a], z[t, b]) < z[t].max() - 80, (t, ids[t], chosen)
            continue
        assert np.allclose(w[t], ww, rtol=2e-5, atol=1e-30)
    assert list(ids[7]) == list(range(top)) and np.allclose(w[7], 1.0 / E, rtol=1e-6)
    assert w.sum(1).max() <= 1.0 + 1e-5 and (top == E or abs(w[7].sum() - top / E) < 1e-6)  # the weights are not brought back to sum 1
    # the same op with the division switched on sums to one
    _, wn = run_route(z, top, 1, 0)
    assert np.allclose(wn.sum(1), 1.0, rtol=1e-5)


def test_gated_activations_gelu_and_clamped_swish():
    rng = np.random.default_rng(11)
    F, NU, T = 24, 3, 7
    gu = rng.standard_normal((T, NU, 2 * F)) * 2.5
    gu[0, 0, :4] = [1.25, -1.25, 40.0, -40.0]; gu[0, 0, F:F + 4] = [1.25, -1.25, 40.0, -40.0]
    dgu, dact = dev(gu), H.DeviceBuffer(4 * T * NU * F + 256)
    ta, tb = Tensor.contiguous(dgu.ptr, F32, (F, NU, T)), Tensor.contiguous(dgu.ptr + 4 * F, F32, (F, NU, T))
    for t in (ta, tb):
        t.nb[1], t.nb[2] = 8 * F, 8 * F * NU
    td = Tensor.contiguous(dact.ptr, F32, (F, NU, T))
    a, u = gu[..., :F], gu[..., F:]
    check(lib().b200_op_glu_strided(1, C.byref(ta), C.byref(tb), C.byref(td), 0.0, 0.0, None))
    assert rel(dact.to_numpy(np.float32, (T, NU, F)), R.gelu_tanh(a) * u) < 2e-6
    limit = 1.25
    g, c = np.minimum(a, limit), np.clip(u, -limit, limit)
    check(lib().b200_op_glu_strided(2, C.byref(ta), C.byref(tb), C.byref(td), limit, 1.702, None))
    assert rel(dact.to_numpy(np.float32, (T, NU, F)), g * R.sigmoid(1.702 * g) * (c + 1.0)) < 2e-6
    check(lib().b200_op_glu_strided(0, C.byref(ta), C.byref(tb), C.byref(td), 0.0, 0.0, None))
    assert rel(dact.to_numpy(np.float32, (T, NU, F)), a * R.sigmoid(a) * u) < 2e-6


@pytest.mark.parametrize("n,NU,T", [(40, 3, 7), (70, 1, 2), (1024, 2, 5), (12288, 4, 2), (16384, 2, 3)])
def test_expert_sum_norm_and_residual_in_one_launch(n, NU, T):
    rng = np.random.default_rng(n + NU)
    y, w, res, nw = rng.standard_normal((T, NU, n)) * 2, rng.random((T, NU)), rng.standard_normal((T, n)), 1 + 0.3 * rng.standard_normal(n)
    eps = 1e-6
    dy, dw, dr, dn, dout = dev(y), dev(w), dev(res), dev(nw), H.DeviceBuffer(4 * T * n + 256)
    check(lib().b200_op_moe_combine_norm(dy.ptr, n, NU * n, dw.ptr, NU, dn.ptr, eps, dr.ptr, n, dout.ptr, n, n, NU, T, None))
    s = np.einsum("tk,tkn->tn", w, y)
    assert rel(dout.to_numpy(np.float32, (T, n)), res + R.rms_norm_plain(s, nw, eps)) < 3e-6
    check(lib().b200_op_moe_combine_norm(dy.ptr, n, NU * n, dw.ptr, NU, None, eps, None, 0, dout.ptr, n, n, NU, T, None))
    assert rel(dout.to_numpy(np.float32, (T, n)), R.rms_unit(s, eps)) < 3e-6


def test_clamped_expert_matches_its_parts():
    rng = np.random.default_rng(5)
    x, Wg, Wu, Wd = rng.standard_normal(12) * 2, rng.standard_normal((7, 12)), rng.standard_normal((7, 12)), rng.standard_normal((12, 7))
    g, u = Wg @ x, Wu @ x
    assert (g > 1.0).any() and (np.abs(u) > 1.0).any()
    y = np.array([min(gi, 1.0) / (1 + math.exp(-1.702 * min(gi, 1.0))) * (max(-1.0, min(ui, 1.0)) + 1.0) for gi, ui in zip(g, u)])
    assert np.allclose(R.clamped_expert(x, Wg, Wu, Wd, 1.0), Wd @ y, rtol=1e-12)


# ------------------------------------------------------------------------------------------------ whole models
from koboldcpp_b200 import zevopel as Z  # noqa: E402
from koboldcpp_b200.engine import Engine, Request  # noqa: E402

CONFIGS = {
    # dense, routed and no feed-forward; chunks shorter than the prompts, a layer without chunks; 4 heads over 2 kv heads
    "mixed": lambda: R.make_config([R.attn_layer(chunk=9), R.attn_layer(mlp="moe", chunk=30), R.attn_layer(heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=8, mlp=None),
                                    R.attn_layer(mlp="moe", chunk=16, scaling=False)]),
    # one head, one kv head, one expert per token and all experts per token, dim != vdim, rotation over the whole head or none of it,
    # multipliers of exactly one, a width that is no multiple of 8
    "odd": lambda: R.make_config([R.attn_layer(heads=1, kv_heads=1, dim=24, vdim=40, rot_dims=24, scaling=False, base=500.0, chunk=1, mlp=R.moe(ff=40, experts=5, top=1, limit=0.5)),
                                  R.attn_layer(heads=6, kv_heads=2, dim=8, vdim=4, rot_dims=0, chunk=4, mlp=R.moe(ff=8, experts=3, top=3, limit=4.0)),
                                  R.attn_layer(heads=3, kv_heads=3, dim=10, vdim=6, rot_dims=2, chunk=1000, mlp=R.dense(20))],
                                 width=70, vocab=70, eps=1e-6, embed_scale=1.0, residual_mult=1.0),
    # sizes that take the 16-byte and tensor-core paths: width and ff multiples of 64
    "aligned": lambda: R.make_config([R.attn_layer(heads=4, kv_heads=4, dim=32, vdim=32, rot_dims=32, chunk=20, mlp=R.moe(ff=64, experts=8, top=2)),
                                      R.attn_layer(heads=4, kv_heads=1, dim=64, vdim=32, rot_dims=16, chunk=64, mlp=R.dense(192))], width=128, vocab=96, residual_mult=1.5),
}


@pytest.fixture(scope="module", params=list(CONFIGS))
def model(request):
    cfg = CONFIGS[request.param]()
    W = R.random_weights(cfg, seed=len(request.param))
    m = Z.build(cfg, R.as_tensors(W), dtype="float32", n_ctx=768, n_seq_max=4, max_batch=400)
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
    want = R.forward(toks, W, cfg)
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
    want = R.forward(toks, W, cfg)
    eng = Engine(m)
    rows = []
    for a in range(0, 40, portion):  # the cuts of the portions do not fall on the chunk borders (4, 9, 16, 20, 30, 64)
        b = min(a + portion, 40)
        rows.append(eng.step([("p", toks[a:b], range(b - a))]))
    for t in range(40, 70):  # the chunk borders 45, 48, 60, 64 are crossed by decoded tokens
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
    want = {k: R.forward(v, W, cfg) for k, v in toks.items()}
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
    want = R.forward(toks, W, cfg)
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
            lg = R.forward(seq, W, cfg)[-1]
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
    want = R.forward(ta, W, cfg)
    m = Z.build(cfg, R.as_tensors(W), dtype="bfloat16", n_ctx=256, n_seq_max=2, max_batch=128)
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


def test_sharp_attention_through_the_model_with_chunk_borders():
    """Weights make the attention sharp (large score scale), so a wrong position, border or cell would show in the logits; the
    chunk borders lie inside the prompt, at the prompt's end and inside the decoded stretch, and at the cache padding."""
    cfg = R.make_config([R.attn_layer(heads=2, kv_heads=1, dim=16, vdim=16, rot_dims=16, scale=3.0, chunk=256, mlp=None),
                         R.attn_layer(heads=2, kv_heads=2, dim=16, vdim=8, rot_dims=8, chunk=101, scale=3.0, scaling=False)])
    W = R.random_weights(cfg, seed=21)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], 640).tolist()
    want = R.forward(toks, W, cfg)
    m = Z.build(cfg, R.as_tensors(W), dtype="float32", n_ctx=768, n_seq_max=2, max_batch=640)
    eng = Engine(m)
    places = [0, 1, 2, 100, 101, 102, 201, 202, 255, 256, 257, 302, 303, 304, 511, 512, 513, 599, 600, 605]
    rows = [eng.step([("a", toks[:606], places)])]  # 606 = 6 * 101: the next token opens a chunk of the second layer
    for t in range(606, 640):
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
            lg = R.forward(seq, W, cfg)[-1]
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
    wa, wb = R.forward(ta, W, cfg), R.forward(tb, W, cfg)
    want = {0: np.stack([wa[0], wa[10], wb[5]]), 1: wb[6:7], 2: np.stack([wa[12], wb[7]]), 3: wa[13:14]}
    for n, w in want.items():
        got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        assert got.shape == w.shape and logits_err(got, w) < 1e-4, n

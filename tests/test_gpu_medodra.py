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
                                                  (300, 3, [64, 1, 32], 1)])
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

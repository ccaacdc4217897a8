"""Medodra without a GPU: configuration -> layer parameters and run order, the registry, and the oracle's own consistency (a
continued sequence against the whole one, distance buckets, the convolution's tail, the delta rule as an overwrite)."""
from __future__ import annotations

import math

import numpy as np

import medodra_ref as R
from koboldcpp_b200 import medodra
from koboldcpp_b200.galirax import run_order
from koboldcpp_b200.models import ARCHITECTURES


def test_registry_knows_the_architecture():
    assert ARCHITECTURES["Medodra"] is medodra.load


def test_layer_parameters_from_the_configuration():
    d = medodra.layer_params(R.delta_layer(heads=6, kv_heads=2, dim=24, vdim=8, conv=5, mlp=R.moe_cfg(ff=40, experts=7, top=3, shared=0)), loop_input=True)
    assert (d.mixer, d.heads, d.kv_heads, d.dim, d.vdim, d.conv_taps, d.loop_input) == (medodra.MIXER_DELTA, 6, 2, 24, 8, 5, 1)
    assert (d.mlp, d.ff, d.n_expert, d.n_expert_used, d.shared_ff, d.router_keep_scores, d.router_scale_input) == (medodra.MLP_MOE_GATED, 40, 7, 3, 0, 1, 1)
    p = medodra.layer_params(R.parallel_layer(heads=3, kv_heads=1, dim=10, vdim=12, conv=2, bias_max=99, coef=0.25, every=7, scale=0.4, side=33, mlp=None))
    assert (p.mixer, p.heads, p.kv_heads, p.dim, p.vdim, p.conv_taps, p.loop_input) == (medodra.MIXER_SIGMOID_ATTENTION_GRU, 3, 1, 10, 12, 2, 0)
    assert (p.dist_bias_max, p.q_temp_every, p.side_width, p.mlp) == (99, 7, 33, medodra.MLP_NONE)
    assert abs(p.q_temp_coef - 0.25) < 1e-7 and abs(p.scale - 0.4) < 1e-7


def test_run_order_of_a_looped_stretch():
    assert run_order(5, {"start": 2, "stop": 4, "times": 3}) == [0, 1, 2, 3, 2, 3, 2, 3, 4]
    assert [il for il, _ in R.run_order(R.make_config([0] * 5, loop=(2, 4, 3)))] == [0, 1, 2, 3, 2, 3, 2, 3, 4]
    assert [s for _, s in R.run_order(R.make_config([0] * 3, loop=(0, 2, 2)))] == [True, False, True, False, False]
    assert R.run_order(R.make_config([0] * 2)) == [(0, False), (1, False)]


def test_distance_buckets():
    B, D = 8, 40
    b = [R.distance_bucket(n, B, D) for n in range(200)]
    assert b[:4] == [0, 1, 2, 3] and b[4] == 4 and b[39] <= 7 and b[40] == 7 and b[199] == 7
    assert all(x <= y for x, y in zip(b, b[1:])) and set(b) == set(range(8))
    # where the logarithm lands on a whole number the bucket starts there: half 4, far 64, 4 log buckets: 4 * 2^j starts bucket 4 + j
    assert [R.distance_bucket(n, 8, 64) for n in (7, 8, 15, 16, 31, 32, 63, 64)] == [4, 5, 5, 6, 6, 7, 7, 7]


def test_query_temperature_steps():
    assert R.query_temperature(0, 0.5, 4) == 1.0 and R.query_temperature(2, 0.5, 4) == 1.0
    assert abs(R.query_temperature(3, 0.5, 4) - (1 + 0.5 * math.log(2))) < 1e-12 and abs(R.query_temperature(10, 0.5, 4) - (1 + 0.5 * math.log(3))) < 1e-12


def test_short_convolution_tail():
    rng = np.random.default_rng(0)
    u, w = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    whole, _ = R.short_conv(u, w, np.zeros((3, 3)))
    a, tail = R.short_conv(u[:2], w, np.zeros((3, 3)))
    b, tail = R.short_conv(u[2:3], w, tail)
    c, _ = R.short_conv(u[3:], w, tail)
    assert np.allclose(np.concatenate([a, b, c]), whole)
    assert np.allclose(whole[0], w[:, 3] * u[0]) and np.allclose(whole[1], w[:, 3] * u[1] + w[:, 2] * u[0])


def test_delta_rule_step_overwrites():
    k = np.zeros(4); k[1] = 1.0
    S, _ = R.delta_rule_step(np.zeros((4, 2)), k, k, np.array([1.0, 2.0]), 1.0, 1.0)
    S, o = R.delta_rule_step(S, k, k, np.array([5.0, -1.0]), 1.0, 1.0)
    assert np.allclose(o, [5.0, -1.0]) and np.allclose(S[1], [5.0, -1.0])
    S, o = R.delta_rule_step(S, k, k, np.array([0.0, 0.0]), 0.0, 0.5)  # beta 0 writes nothing; the decay halves what is there
    assert np.allclose(o, [2.5, -0.5])


def test_continued_sequence_equals_the_whole_one():
    cfg = R.make_config([R.parallel_layer(), R.delta_layer(), R.parallel_layer(heads=2, kv_heads=2, conv=2, mlp=None)], loop=(1, 3, 2))
    W = R.random_weights(cfg, seed=3)
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], 17).tolist()
    whole = R.logits(cfg, W, toks)
    a, st = R.forward(cfg, W, toks[:5])
    b, st = R.forward(cfg, W, toks[5:6], st)
    c, st = R.forward(cfg, W, toks[6:], st)
    assert np.allclose(np.concatenate([a, b, c]), whole, atol=1e-9)

"""Host-side pieces of the Zevopel path that need no GPU: the configuration reader, the registry and the reference's own
consistency (rotation bands and pairs, chunked visibility, router, clamps, prefill against a continued sequence)."""
from __future__ import annotations

import math

import numpy as np
import pytest

import zevopel_ref as R
from koboldcpp_b200 import models
from koboldcpp_b200 import zevopel as Z
from koboldcpp_b200.lib import B200Error


def test_layer_params_from_config():
    a = Z.layer_params(R.attn_layer(heads=6, kv_heads=3, dim=8, vdim=4, rot_dims=2, chunk=5, mlp=R.moe(ff=8, experts=12, top=4, limit=0.75)))
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.rope_dims, a.chunk, a.window, a.keep_first) == (Z.MIXER_ATTENTION, 6, 3, 8, 4, 2, 5, 0, 0)
    assert (a.qk_norm, a.qk_norm_per_head, a.rope_halves, a.head_gate, a.qkv_bias) == (1, 1, 1, 1, 0)
    assert (a.mlp, a.ff, a.n_expert, a.n_expert_used, a.glu_kind, a.router_score, a.router_keep_scores) == (Z.MLP_MOE_GATED, 8, 12, 4, Z.GLU_SWISH_CLAMPED, Z.ROUTER_SOFTMAX, 1)
    assert abs(a.glu_limit - 0.75) < 1e-7 and abs(a.glu_alpha - 1.702) < 1e-6 and a.router_scale == 1.0
    assert a.rope_scaling == Z.ROPE_SCALING_BANDS and (a.yarn_factor, a.band_low, a.band_high, a.yarn_original) == (4.0, 1.0, 3.0, 48)
    b = Z.layer_params(R.attn_layer(scaling=False, mlp=None))
    assert (b.chunk, b.rope_scaling, b.mlp, b.ff) == (0, Z.ROPE_SCALING_NONE, Z.MLP_NONE, 0)
    c = Z.layer_params(R.attn_layer(mlp=R.dense(56)))
    assert (c.mlp, c.ff, c.glu_kind) == (Z.MLP_DENSE_GATED, 56, Z.GLU_GELU_TANH)
    with pytest.raises(B200Error):
        Z.layer_params({"type": "convolution", "mixer": {}, "mlp": None})
    with pytest.raises(B200Error):
        Z.layer_params(R.attn_layer(mlp={"kind": "maxout"}))


def test_registry_knows_the_architecture():
    assert models.ARCHITECTURES["Zevopel"] is Z.load


def test_reference_rotation_pairs_and_bands():
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    f, plain = R.rotation_freqs(rot), R.rotation_freqs({"base": 10000.0, "dims": 32})
    wl = 2 * np.pi / plain
    assert np.allclose(f[wl < 16], plain[wl < 16]) and np.allclose(f[wl > 64], plain[wl > 64] / 8.0)
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and (f[mid] <= plain[mid] + 1e-15).all() and (f[mid] >= plain[mid] / 8.0 - 1e-15).all()
    # entry i turns with entry i + n/2; entries from n on stay; position 0 changes nothing; lengths are kept
    x = np.random.default_rng(0).standard_normal((3, 2, 12))
    y = R.rotate_halves(x, [0, 5, 9], {"base": 50.0, "dims": 8})
    assert np.array_equal(y[0], x[0]) and np.array_equal(y[:, :, 8:], x[:, :, 8:])
    a = 5 * 50.0 ** (-2.0 / 8)
    assert np.allclose(y[1, :, 1], x[1, :, 1] * math.cos(a) - x[1, :, 5] * math.sin(a)) and np.allclose(y[1, :, 5], x[1, :, 5] * math.cos(a) + x[1, :, 1] * math.sin(a))
    assert np.allclose((y[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1))


def test_reference_chunks_sink_and_router():
    assert [j for j in range(10) if R.sees(7, j, 4)] == [4, 5, 6, 7] and [j for j in range(10) if R.sees(8, j, 4)] == [8]
    assert [j for j in range(10) if R.sees(3, j, 0)] == [0, 1, 2, 3]
    # the sink takes weight and gives nothing: with one visible key the output is v * e^s / (e^s + e^sink)
    q, k, v = np.ones((1, 1, 2)), np.ones((1, 1, 2)), np.array([[[3.0, -1.0]]])
    out = R.sink_attention(q, k, v, 0.5, np.array([1.0]), 0)
    assert np.allclose(out[0, 0], v[0, 0] * math.e / (math.e + math.e))
    ids, w = R.softmax_router(np.array([0.0, 2.0, 2.0, -1.0]), 2)
    assert ids == [1, 2] and abs(w[0] - w[1]) < 1e-15 and sum(w) < 1.0
    s = np.exp([0.0, 2.0, 2.0, -1.0])
    assert abs(w[0] - s[1] / s.sum()) < 1e-15


def test_reference_whole_prompt_against_a_continued_sequence():
    """The attention of a portion that continues a sequence must use positions and chunks counted from the sequence's start."""
    cfg = R.make_config([R.attn_layer(chunk=5, mlp="moe"), R.attn_layer(chunk=0)])
    W = R.random_weights(cfg, seed=3)
    toks = list(range(3, 20))
    whole = R.forward(toks, W, cfg)
    # a chunk border at position 10: what comes from there on is a function of tokens 10.. alone in a model whose layers all use
    # the same chunk
    cfg1 = R.make_config([R.attn_layer(chunk=5, mlp="moe")])
    W1 = {k: v for k, v in W.items() if not k.startswith("l1.")}
    a = R.forward(toks, W1, cfg1)
    b = R.forward(toks[10:], W1, cfg1, pos0=10)
    assert np.allclose(a[10:], b, rtol=1e-9, atol=1e-9)
    c = R.forward(toks[9:], W1, cfg1, pos0=9)  # one token earlier the cut is inside a chunk: position 9 has lost what it saw
    assert not np.allclose(a[9], c[0], rtol=1e-3)
    assert whole.shape == (17, cfg["vocab"])

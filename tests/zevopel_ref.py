"""Zevopel in plain float64 numpy, one function per mechanism, written from the equations and sharing no code with the product
path.  Everything is token by token or dense and slow on purpose.

Notation: x is the residual stream [T, W] and c the residual multiplier.  A layer is
    x <- x + c * a1 * N1(mixer(x)),   x <- x + c * a2 * N2(ff(x))
with N an RMS norm whose stored weight w acts as (1 + w), and a1, a2 per-channel scales.  Neither sublayer sees a normalised
input: the norm sits behind it.
"""
from __future__ import annotations

import math

import numpy as np


def bf16_round(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rms_norm_plain(x, w, eps):
    """The weight multiplies as stored."""
    return rms_unit(x, eps) * w


def rms_norm_one_plus(x, w, eps):
    """The weight is stored as its distance from one."""
    return rms_unit(x, eps) * (1.0 + w)


# ------------------------------------------------------------------------------------------------ rotation
def rotation_freqs(rot):
    """f_i = base^(-2i/n), i < n/2.  With scaling {factor, low, high, original}: the wavelength L = 2 pi / f decides.  L below
    original / high: f stays.  L above original / low: f / factor.  Between: s = (original / L - low) / (high - low) and the
    result is (1 - s) f / factor + s f."""
    n = rot["dims"]
    out = []
    sc = rot.get("scaling")
    for i in range(n // 2):
        f = float(rot["base"]) ** (-2.0 * i / n)
        if sc:
            L = 2.0 * math.pi / f
            if L < sc["original"] / sc["high"]:
                pass
            elif L > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            else:
                s = (sc["original"] / L - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return np.array(out)


def rotate_halves(x, pos, rot):
    """x [T, heads, dim].  Among the first n = rot.dims entries of a head, entry i pairs with entry i + n/2 and the pair turns
    by the angle pos * f_i; entries from n on stay."""
    n = rot["dims"]
    y = np.array(x, dtype=np.float64, copy=True)
    if n == 0:
        return y
    f = rotation_freqs(rot)
    for t in range(x.shape[0]):
        for i in range(n // 2):
            a = pos[t] * f[i]
            u, v = x[t, :, i], x[t, :, i + n // 2]
            y[t, :, i] = u * math.cos(a) - v * math.sin(a)
            y[t, :, i + n // 2] = v * math.cos(a) + u * math.sin(a)
    return y


# ------------------------------------------------------------------------------------------------ attention
def sees(i, j, chunk):
    """Position i sees j when j is not later and, with chunks, both lie in the same chunk counted from position 0."""
    return j <= i and (chunk <= 0 or i // chunk == j // chunk)


def sink_attention(q, k, v, scale, sink, chunk, pos0=0):
    """q [T, H, D], k [T, G, D], v [T, G, V] of one sequence that starts at position pos0.  For every row
    p_j = exp(s_j) / (exp(sink_h) + sum_j' exp(s_j')), out = sum_j p_j v_j; the sink takes weight and gives nothing."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[-1]))
    for i in range(T):
        js = [j for j in range(T) if sees(pos0 + i, pos0 + j, chunk)]
        for h in range(H):
            g = h // (H // G)
            s = np.array([scale * (q[i, h] @ k[j, g]) for j in js])
            m = max(s.max(), sink[h])
            e = np.exp(s - m)
            out[i, h] = (e / (e.sum() + math.exp(sink[h] - m))) @ np.stack([v[j, g] for j in js])
    return out


def attention_mixer(x, W, pre, mx, eps, pos0=0):
    T = x.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (x @ W[pre + "q"].T).reshape(T, H, D)
    k = (x @ W[pre + "k"].T).reshape(T, G, D)
    v = (x @ W[pre + "v"].T).reshape(T, G, V)
    q, k = rms_norm_plain(q, W[pre + "q.norm"], eps), rms_norm_plain(k, W[pre + "k.norm"], eps)  # per head, one weight for all heads
    pos = np.arange(pos0, pos0 + T)
    rot = mx.get("rot") or {"dims": 0}
    q, k = rotate_halves(q, pos, rot), rotate_halves(k, pos, rot)
    o = sink_attention(q, k, v, mx["scale"], W[pre + "sink"], int((mx.get("mask") or {}).get("size", 0)), pos0)
    o = o * sigmoid(x @ W[pre + "g"].T)[:, :, None]  # one gate per head, from the mixer's input
    return o.reshape(T, H * V) @ W[pre + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_ff(x, W, pre):
    return (gelu_tanh(x @ W[pre + "gate"].T) * (x @ W[pre + "up"].T)) @ W[pre + "down"].T


def softmax_router(z, top):
    """z [E]: scores are the softmax over all experts; the `top` largest are chosen (lowest index among equals) and keep their
    scores as weights, without renormalisation."""
    s = np.exp(z - z.max())
    s = s / s.sum()
    ids = sorted(range(len(z)), key=lambda e: (-s[e], e))[:top]
    return ids, [s[e] for e in ids]


def clamped_expert(x, Wg, Wu, Wd, limit):
    g = np.minimum(x @ Wg.T, limit)
    u = np.clip(x @ Wu.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ Wd.T


def moe_ff(x, W, pre, mlp):
    E, top, limit = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["limit"]
    out = np.zeros((x.shape[0], W[pre + "e0.down"].shape[0]))
    for t in range(x.shape[0]):
        ids, ws = softmax_router(W[pre + "router"] @ x[t], top)
        for e, w in zip(ids, ws):
            out[t] += w * clamped_expert(x[t], W[pre + f"e{e}.gate"], W[pre + f"e{e}.up"], W[pre + f"e{e}.down"], limit)
    return out


# ------------------------------------------------------------------------------------------------ the model
def layer(x, W, il, cfg, pos0=0):
    L = cfg["layers"][il]
    eps, c = cfg["norm"]["eps"], cfg["residual_mult"]
    pre = f"l{il}."
    if L["type"] != "attention":
        raise ValueError(L["type"])
    y = attention_mixer(x, W, pre + "mix.", L["mixer"], eps, pos0)
    x = x + c * W[pre + "ls1"] * rms_norm_one_plus(y, W[pre + "norm1"], eps)
    mlp = L.get("mlp")
    if mlp is not None:
        y = dense_ff(x, W, pre + "mlp.") if mlp["kind"] == "dense" else moe_ff(x, W, pre + "mlp.", mlp)
        x = x + c * W[pre + "ls2"] * rms_norm_one_plus(y, W[pre + "norm2"], eps)
    return x


def forward(tokens, W, cfg, pos0=0, streams=None):
    """Logits [T, vocab] of one sequence given whole (float64 weights W by name).  streams, a list, receives x after every layer."""
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    for il in range(len(cfg["layers"])):
        x = layer(x, W, il, cfg, pos0)
        if streams is not None:
            streams.append(x.copy())
    return rms_norm_one_plus(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T


# ------------------------------------------------------------------------------------------------ random models for tests
def dense(ff=48):
    return {"kind": "dense", "ff": ff}


def moe(ff=24, experts=6, top=2, limit=1.25):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def attn_layer(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, base=1000.0, scaling=True, chunk=0, scale=None, mlp="dense"):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 48}
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale if scale is not None else 1.3 / math.sqrt(dim)}
    if chunk:
        mx["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": mx, "mlp": dense() if mlp == "dense" else moe() if mlp == "moe" else mlp}


def make_config(layers, width=40, vocab=61, eps=1e-5, embed_scale=2.0, residual_mult=0.8):
    return {"architecture": "Zevopel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "residual_mult": residual_mult, "layers": layers}


def random_weights(cfg, seed=0, gain=1.0):
    """name -> float64 arrays whose values bfloat16 holds exactly, so that the served (bf16) and the exact (f32) modes read the same
    model.  The experts' products are large enough for both clamps to act."""
    rng = np.random.default_rng(seed)
    Wd, Vc = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, rows, cols, g=1.0):
        W[name] = bf16_round(rng.standard_normal((rows, cols)) * g * gain / math.sqrt(cols)).astype(np.float64)

    def vec(name, n, mean=0.0, spread=0.3):
        W[name] = bf16_round(mean + spread * rng.standard_normal(n)).astype(np.float64)

    W["embed"] = bf16_round(rng.standard_normal((Vc, Wd))).astype(np.float64)
    mat("head", Vc, Wd, 3.0)
    vec("final.norm", Wd, 0.0, 0.2)
    for il, L in enumerate(cfg["layers"]):
        p, mx = f"l{il}.", L["mixer"]
        H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        mat(p + "mix.q", H * D, Wd); mat(p + "mix.k", G * D, Wd); mat(p + "mix.v", G * V, Wd); mat(p + "mix.g", H, Wd, 1.5); mat(p + "mix.o", Wd, H * V)
        vec(p + "mix.q.norm", D, 1.0, 0.3); vec(p + "mix.k.norm", D, 1.0, 0.3); vec(p + "mix.sink", H, 0.5, 1.0)
        vec(p + "norm1", Wd, 0.0, 0.2); vec(p + "ls1", Wd, 1.0, 0.3)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        vec(p + "norm2", Wd, 0.0, 0.2); vec(p + "ls2", Wd, 1.0, 0.3)
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            mat(p + "mlp.gate", F, Wd); mat(p + "mlp.up", F, Wd); mat(p + "mlp.down", Wd, F)
        else:
            F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            mat(p + "mlp.router", E, Wd, 1.5)
            for e in range(E):
                mat(p + f"mlp.e{e}.gate", F, Wd, 0.7); mat(p + f"mlp.e{e}.up", F, Wd, 0.7); mat(p + f"mlp.e{e}.down", Wd, F)
    return W


def as_tensors(W):
    """name -> (dtype, shape, raw bytes), the form the loader takes: matrices and vectors as bf16 bits."""
    out = {}
    for name, a in W.items():
        bits = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
        out[name] = ("BF16", tuple(a.shape), bits.view(np.uint8).reshape(-1))
    return out

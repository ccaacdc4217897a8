"""Medodra in plain float64 numpy, one function per mechanism, written from the equations and sharing no code with the product
path.  Everything is token by token or dense and slow on purpose.

Notation: x is the residual stream [T, W], c the residual multiplier, N an RMS norm whose stored weight w acts as (1 + w).
A layer is   x <- x + c * (mixer(N1(x)) + ff(N2(x)))   with both sublayers reading the same x.
The stream starts as  x0 = scale * embed[token] + sinusoid(position);  a looped stretch of layers runs several times with the same
weights and, before the first layer of every pass,  x <- W_in [x ; x0].

A `state` dict carries what a sequence needs to go on: per layer run the conv tails, the recurrent states and the cached keys and
values, and the number of tokens seen.  forward() with a state continues that sequence.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


# ------------------------------------------------------------------------------------------------ embedding
def sinusoid(pos, width):
    """Entry 2i is sin(p f_i), entry 2i + 1 is cos(p f_i), f_i = 10000^(-2i / width)."""
    out = np.zeros((len(pos), width))
    for t, p in enumerate(pos):
        for j in range(width):
            i = j // 2
            a = p * 10000.0 ** (-2.0 * i / width)
            out[t, j] = math.sin(a) if j % 2 == 0 else math.cos(a)
    return out


def embed(tokens, table, scale, pos):
    return table[np.asarray(tokens)] * scale + sinusoid(pos, table.shape[1])


# ------------------------------------------------------------------------------------------------ short convolution
def short_conv(u, w, tail):
    """u [T, C] inputs in time order, w [C, taps] (last column multiplies the current input), tail [taps - 1, C] the inputs before
    u (zeros at the start of a sequence).  Returns y [T, C] and the new tail."""
    taps = w.shape[1]
    ext = np.concatenate([tail, u], 0)  # ext[taps - 1 + t] = u[t]
    y = np.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            y[t] += w[:, j] * ext[t + j]
    return y, ext[ext.shape[0] - (taps - 1):] if taps > 1 else ext[:0]


# ------------------------------------------------------------------------------------------------ gated delta rule
def unit_vector(x, eps=1e-6):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + eps)


def delta_rule_step(S, q, k, v, beta, g):
    """One token of one head.  S [dim, vdim]: decay, then write the difference between v and what k reads, then read with q."""
    S = g * S
    u = beta * (v - S.T @ k)
    S = S + np.outer(k, u)
    return S, S.T @ q


def delta_mixer(h, W, mx, eps, st):
    """h [T, width].  W: the layer's 'mix.*' tensors by leaf name.  st: {'conv_q', 'conv_k', 'conv_v', 'S'} or empty."""
    H, G, D, V, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
    T = h.shape[0]
    parts = {}
    for leaf, rows in (("q", G * D), ("k", G * D), ("v", H * V)):
        tail = st.get("conv_" + leaf, np.zeros((taps - 1, rows)))
        y, st["conv_" + leaf] = short_conv(h @ W[leaf].T, W[leaf + ".conv"], tail)
        parts[leaf] = silu(y)
    q = unit_vector(parts["q"].reshape(T, G, D)) * D ** -0.5
    k = unit_vector(parts["k"].reshape(T, G, D))
    v = parts["v"].reshape(T, H, V)
    beta = sigmoid(h @ W["b"].T)
    g = np.exp(-np.exp(W["A_log"]) * softplus(h @ W["a"].T + W["dt_bias"]))
    gate = silu(h @ W["g"].T).reshape(T, H, V)
    S = st.get("S", np.zeros((H, D, V)))
    o = np.zeros((T, H, V))
    for t in range(T):
        for hh in range(H):
            kv = hh // (H // G)
            S[hh], o[t, hh] = delta_rule_step(S[hh], q[t, kv], k[t, kv], v[t, hh], beta[t, hh], g[t, hh])
    st["S"] = S
    o = rms_unit(o, eps) * W["norm"] * gate
    return o.reshape(T, H * V) @ W["o"].T


# ------------------------------------------------------------------------------------------------ sigmoid attention with distance bias
def distance_bucket(n, B, D):
    """Distances below B // 2 have a bucket each; the rest share B - B // 2 buckets spaced evenly in log distance up to D."""
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half) + 1e-9)))


def query_temperature(p, coef, every):
    return 1.0 + coef * math.log((p + 1) // every + 1)


def sigmoid_attention(q, k, v, pos_q, pos_k, scale, rel, pb, bias_max):
    """q [T, H, D]; k [N, G, D], v [N, G, V] everything cached including the new tokens; rel [B, H]; pb [H].  A key at position j <= i
    has the weight sigmoid(scale q.k + rel[bucket(i - j)] + pb); the weights are not normalised."""
    T, H, _ = q.shape
    G = k.shape[1]
    o = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        for hh in range(H):
            kv = hh // (H // G)
            for n in range(k.shape[0]):
                if pos_k[n] > pos_q[t]:
                    continue
                s = scale * (q[t, hh] @ k[n, kv]) + rel[distance_bucket(pos_q[t] - pos_k[n], rel.shape[0], bias_max), hh] + pb[hh]
                o[t, hh] += sigmoid(s) * v[n, kv]
    return o


def attention_side(h, W, mx, eps, pos, st):
    H, G, D, V, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
    T = h.shape[0]
    parts = {}
    for leaf, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
        tail = st.get("conv_" + leaf, np.zeros((taps - 1, rows)))
        parts[leaf], st["conv_" + leaf] = short_conv(h @ W[leaf].T + W[leaf + ".b"], W[leaf + ".conv"], tail)
    q = parts["q"].reshape(T, H, D)
    for t in range(T):
        q[t] *= query_temperature(pos[t], mx["q_temp"]["coef"], mx["q_temp"]["every"])
    k = parts["k"].reshape(T, G, D)
    v = rms_unit(parts["v"].reshape(T, G, V), eps)
    st["k"] = np.concatenate([st["k"], k], 0) if "k" in st else k
    st["v"] = np.concatenate([st["v"], v], 0) if "v" in st else v
    st["pos"] = np.concatenate([st.get("pos", np.zeros(0, dtype=np.int64)), np.asarray(pos)])
    o = sigmoid_attention(q, st["k"], st["v"], pos, st["pos"], mx["scale"], W["rel"], W["pb"], mx["bias_max"])
    return o.reshape(T, H * V) @ W["o"].T + W["o.b"]


# ------------------------------------------------------------------------------------------------ minGRU
def mingru_candidate(u):
    return np.where(u >= 0, u + 0.5, sigmoid(u))


def mingru_side(h, W, st):
    z = sigmoid(h @ W["z"].T + W["z.b"])
    c = mingru_candidate(h @ W["x"].T + W["x.b"])
    gate = silu(h @ W["g"].T)
    S = st.get("S", np.zeros(z.shape[1]))
    out = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        out[t] = S * gate[t]
    st["S"] = S
    return out @ W["o"].T


def parallel_mixer(h, W, mx, eps, pos, st):
    left = attention_side(h, sub(W, "left."), mx["left"], eps, pos, st.setdefault("left", {}))
    right = mingru_side(h, sub(W, "right."), st.setdefault("right", {}))
    return 0.5 * (rms_unit(left, eps) * W["left.out"] + rms_unit(right, eps) * W["right.out"])


# ------------------------------------------------------------------------------------------------ feed-forward
def gated_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, top):
    """Scores sigmoid(W h); the `top` largest are chosen (lowest index among equals) and used as they are."""
    s = sigmoid(h @ router.T)
    ids = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return ids, np.take_along_axis(s, ids, -1)


def moe(h, W, mlp):
    ids, w = route(h, W["router"], mlp["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(ids[t], w[t]):
            out[t] += gated_expert(we * h[t], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])  # the weight scales the expert's input
    if mlp.get("shared"):
        out += gated_expert(h, W["shared.gate"], W["shared.up"], W["shared.down"]) * sigmoid(h @ W["shared.sg"].T)
    return out


# ------------------------------------------------------------------------------------------------ the model
def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def run_order(cfg):
    """[(layer, starts a pass)]: layers loop.start .. loop.stop - 1 run loop.times times in a row, the rest once."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    a, b = lp["start"], lp["stop"]
    out = [(i, False) for i in range(a)]
    for _ in range(lp["times"]):
        out += [(i, i == a) for i in range(a, b)]
    return out + [(i, False) for i in range(b, n)]


def layer(x, W, lc, cfg, pos, st):
    eps, c = cfg["norm"]["eps"], cfg["residual_mult"]
    h1 = norm_one_plus(x, W["norm1"], eps)
    if lc["type"] == "delta":
        y = delta_mixer(h1, sub(W, "mix."), lc["mixer"], eps, st)
    elif lc["type"] == "parallel":
        y = parallel_mixer(h1, sub(W, "mix."), lc["mixer"], eps, pos, st)
    else:
        raise ValueError(lc["type"])
    if lc.get("mlp"):
        y = y + moe(norm_one_plus(x, W["norm2"], eps), sub(W, "mlp."), lc["mlp"])
    return x + c * y


def forward(cfg, weights, tokens, state=None, want_layers=False):
    """tokens: the next tokens of one sequence.  Returns logits [T, vocab] (and the stream after every layer run) and the state."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    state = state if state is not None else {"n": 0, "runs": {}}
    pos = list(range(state["n"], state["n"] + len(tokens)))
    state["n"] += len(tokens)
    x0 = embed(tokens, W["embed"], cfg["embedding"]["scale"], pos)
    x = x0
    streams = []
    for r, (il, starts) in enumerate(run_order(cfg)):
        if starts:
            x = np.concatenate([x, x0], -1) @ W["loop.in"].T
        x = layer(x, sub(W, f"l{il}."), cfg["layers"][il], cfg, pos, state["runs"].setdefault(r, {}))
        streams.append(x)
    logits = norm_one_plus(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T
    if want_layers:
        return logits, np.stack(streams), state
    return logits, state


def logits(cfg, weights, tokens):
    return forward(cfg, weights, tokens)[0]


# ------------------------------------------------------------------------------------------------ small random models for the tests
def bf16_round(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32)


def moe_cfg(ff=24, experts=6, top=2, shared=16):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=8, conv=4, mlp="moe"):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": moe_cfg() if mlp == "moe" else mlp}


def parallel_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, bias_max=40, coef=0.7, every=16, scale=None, side=48, mlp="moe"):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "bias_max": bias_max, "q_temp": {"coef": coef, "every": every},
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": side}}, "mlp": moe_cfg() if mlp == "moe" else mlp}


def make_config(layers, width=40, vocab=61, eps=1e-5, embed_scale=3.0, residual_mult=0.7, loop=None):
    cfg = {"architecture": "Medodra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "residual_mult": residual_mult, "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed=0, rel_rows=8):
    """name -> float64 arrays whose values bfloat16 holds exactly, so that the served (bf16) and the exact (f32) modes read the same
    model."""
    rng = np.random.default_rng(seed)
    Wd, Vc = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, rows, cols, g=1.0):
        W[name] = bf16_round(rng.standard_normal((rows, cols)) * g / math.sqrt(cols)).astype(np.float64)

    def vec(name, n, mean=0.0, spread=0.3):
        W[name] = bf16_round(mean + spread * rng.standard_normal(n)).astype(np.float64)

    W["embed"] = bf16_round(rng.standard_normal((Vc, Wd))).astype(np.float64)
    mat("head", Vc, Wd, 3.0)
    vec("final.norm", Wd, 0.0, 0.2)
    if cfg.get("loop"):
        mat("loop.in", Wd, 2 * Wd, 1.5)
    for il, L in enumerate(cfg["layers"]):
        p, mx = f"l{il}.", L["mixer"]
        vec(p + "norm1", Wd, 0.0, 0.2)
        if L["type"] == "delta":
            H, G, D, V, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
            for leaf, rows in (("q", G * D), ("k", G * D), ("v", H * V)):
                mat(p + "mix." + leaf, rows, Wd, 1.5)
                W[p + "mix." + leaf + ".conv"] = bf16_round(rng.standard_normal((rows, taps)) * 0.6).astype(np.float64)
            mat(p + "mix.b", H, Wd, 2.0); mat(p + "mix.a", H, Wd, 2.0); mat(p + "mix.g", H * V, Wd, 1.5); mat(p + "mix.o", Wd, H * V)
            vec(p + "mix.A_log", H, -0.5, 0.7); vec(p + "mix.dt_bias", H, 0.0, 1.0); vec(p + "mix.norm", V, 1.0, 0.3)
        else:
            a, side = mx["left"], mx["right"]["width"]
            H, G, D, V, taps = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["conv"]
            for leaf, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                mat(p + "mix.left." + leaf, rows, Wd, 1.5)
                vec(p + "mix.left." + leaf + ".b", rows, 0.0, 0.3)
                W[p + "mix.left." + leaf + ".conv"] = bf16_round(rng.standard_normal((rows, taps)) * 0.6).astype(np.float64)
            W[p + "mix.left.rel"] = bf16_round(rng.standard_normal((rel_rows, H))).astype(np.float64)
            vec(p + "mix.left.pb", H, -1.0, 0.7)
            mat(p + "mix.left.o", Wd, H * V); vec(p + "mix.left.o.b", Wd, 0.0, 0.3)
            for leaf in ("z", "x", "g"):
                mat(p + "mix.right." + leaf, side, Wd, 2.0)
            vec(p + "mix.right.z.b", side, 0.0, 0.5); vec(p + "mix.right.x.b", side, 0.0, 0.5)
            mat(p + "mix.right.o", Wd, side)
            vec(p + "mix.left.out", Wd, 1.0, 0.3); vec(p + "mix.right.out", Wd, 1.0, 0.3)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        vec(p + "norm2", Wd, 0.0, 0.2)
        F = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            mat(p + f"mlp.e{e}.gate", F, Wd, 1.5); mat(p + f"mlp.e{e}.up", F, Wd, 1.5); mat(p + f"mlp.e{e}.down", Wd, F, 1.5)
        mat(p + "mlp.router", mlp["router"]["experts"], Wd, 3.0)
        if mlp.get("shared"):
            FS = mlp["shared"]["ff"]
            mat(p + "mlp.shared.gate", FS, Wd, 1.5); mat(p + "mlp.shared.up", FS, Wd, 1.5); mat(p + "mlp.shared.down", Wd, FS, 1.5); mat(p + "mlp.shared.sg", 1, Wd, 2.0)
    return W


def as_tensors(W):
    """name -> (dtype, shape, raw bytes), the form the loader takes: matrices and vectors as bf16 bits."""
    out = {}
    for name, a in W.items():
        bits = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
        out[name] = ("BF16", tuple(a.shape), bits.view(np.uint8).reshape(-1))
    return out

// host_medodra.cu -- the Medodra architecture for the decoder of host_llama.cu: where its tensors go and the graph of one batch
// step.  The decoder owns the model object, the sequence cache, the inputs and the step; this file adds no loop of its own.
//
// The stream starts as  x0 = scale * embed[token] + s(pos)  with s the sine / cosine position vector (entries 2i, 2i + 1 turn with
// the frequency 10000^(-2i / width)).  A layer reads the stream through two RMS norms (stored weight w acts as 1 + w) and adds both
// sublayers at once:   x <- x + c * (mixer(N1(x)) + ff(N2(x))),   c the model's residual multiplier.  The first layer of the looped
// stretch replaces the stream by  W_in [x ; x0]  every time it is about to run.  Mixers (b200_layer_params):
//   * delta: q, k (kv_heads) and v (heads) pass a short causal convolution and silu, q and k become unit vectors per head, and a
//     state per head follows the gated delta rule (decay from softplus / exp, write strength from a sigmoid); every head's read-out
//     is RMS-normalised, gated by silu(W_g h) and projected;
//   * sigmoid attention + minGRU side by side: the attention side has biases, the same convolution (no activation), a query
//     temperature that grows with ln(position), values normalised per head before they are cached, a learned score bias by
//     bucketed distance and sigmoid weights that are not normalised over the keys; the minGRU side is an element-wise gated state.
//     Each side is RMS-normalised over the width with its own weight and the two are averaged.
// The feed-forward is a mixture of gated experts with sigmoid router scores used as they are, the weight applied to the expert's
// input, plus a shared expert scaled by a sigmoid gate per token.  The output is the norm and the head.
//
// Graph choices: everything a mixer projects from its input is ONE product over row-concatenated weights (rows padded to a multiple
// of 8); q, k, v are adjacent there so that one convolution launch covers them; (1 + w), the halves of the averaged sides and the
// embedding scale are folded into f32 vectors / the f32 table when the model is finalised; rel[bucket(n)] + pb becomes a table by
// distance n = 0 .. bias_max (computed in double, one row for everything further away); an expert's weight joins behind its linear
// gate / up products (inside the activation kernel) instead of in front of them; the experts' sum, the gated shared expert, the
// mixer's result, the multiplier and the residual are one launch, which writes straight into the first half of [x ; x0] when the
// next run starts a pass; the router is an f32 product of f32 weights with the unrounded input in every mode.
#include "host_fused.h"

namespace {

constexpr float kUnitEps = 1e-6f;  // q and k of the delta rule: x / sqrt(sum(x^2) + 1e-6)

struct MdLayer {
    ggml_tensor *pre1 = nullptr, *pre12 = nullptr;     // 1 + norm1 alone (no feed-forward), or 1 + norm1 over 1 + norm2 as one [2][width] tensor
    ggml_tensor *proj1 = nullptr, *convw = nullptr, *convb = nullptr, *wo = nullptr;
    int64_t proj1_rows = 0, conv_channels = 0;
    // delta
    ggml_tensor *a_log = nullptr, *dt_bias = nullptr, *onorm = nullptr;
    // sigmoid attention + minGRU
    ggml_tensor *wo_bias = nullptr, *dist = nullptr, *zb = nullptr, *xb = nullptr, *wo_side = nullptr, *out_l = nullptr, *out_r = nullptr;
    // feed-forward
    ggml_tensor *gate_up = nullptr, *down = nullptr, *router = nullptr, *sh_gate_up = nullptr, *sh_down = nullptr;
    int64_t sh_rows = 0;
};
struct MdRun {
    ggml_tensor *k_cache = nullptr, *v_cache = nullptr;  // attention side: [kv_heads * dim, n_ctx], [kv_heads * vdim, n_ctx] f32
    ggml_tensor *tail = nullptr;                         // the convolution's last taps - 1 inputs per slot
    ggml_tensor *state = nullptr;                        // delta: S [heads * vdim * dim] per slot; minGRU: [side_width] per slot
};
struct MdData {
    std::map<std::string, std::vector<float>> host_vecs;  // vectors that finalize folds or expands
    std::map<std::string, int64_t> host_rows;             // rows of a 2-D one among them
    std::vector<MdLayer> layers;
    std::vector<MdRun> runs;
    ggml_tensor *embed = nullptr, *final_scale = nullptr, *head = nullptr, *loop_in = nullptr, *pos_freqs = nullptr;
};
MdData *md(b200_llama *m) {
    if (!m->arch_data) m->arch_data = std::shared_ptr<void>(new MdData(), [](void *p) { delete (MdData *)p; });
    return (MdData *)m->arch_data.get();
}

int64_t pad8(int64_t v) { return (v + 7) / 8 * 8; }
bool is_delta(const b200_layer_params &lp) { return lp.mixer == B200_MIXER_DELTA; }
// everything the mixer projects from its input, in the order of the rows of the fused matrix; q, k, v come first
int parts_proj1(const b200_layer_params &lp, Part out[8]) {
    int n = 0;
    const int64_t H = lp.heads, G = lp.kv_heads, D = lp.dim, V = lp.vdim;
    if (is_delta(lp)) {
        out[n++] = {"mix.q", G * D}; out[n++] = {"mix.k", G * D}; out[n++] = {"mix.v", H * V};
        out[n++] = {"mix.g", H * V}; out[n++] = {"mix.b", H}; out[n++] = {"mix.a", H};
    } else {
        out[n++] = {"mix.left.q", H * D}; out[n++] = {"mix.left.k", G * D}; out[n++] = {"mix.left.v", G * V};
        out[n++] = {"mix.right.z", lp.side_width}; out[n++] = {"mix.right.x", lp.side_width}; out[n++] = {"mix.right.g", lp.side_width};
    }
    return n;
}
// the first three parts with another suffix: "<leaf>.conv" (rows of the fused convolution weights) or "<leaf>.b"
int parts_qkv(const b200_layer_params &lp, const char *suffix, std::string names[3], Part out[3]) {
    Part p[8];
    parts_proj1(lp, p);
    for (int i = 0; i < 3; i++) { names[i] = std::string(p[i].leaf) + suffix; out[i] = {names[i].c_str(), p[i].rows}; }
    return 3;
}
int parts_shared(const b200_layer_params &lp, Part out[8]) {
    out[0] = {"mlp.shared.gate", lp.shared_ff}; out[1] = {"mlp.shared.up", lp.shared_ff}; out[2] = {"mlp.shared.sg", 1};
    return 3;
}
bool is_host_vec(const b200_layer_params &lp, const char *leaf) {
    if (!strcmp(leaf, "norm1") || !strcmp(leaf, "norm2")) return true;
    if (is_delta(lp)) return false;
    return !strcmp(leaf, "mix.left.out") || !strcmp(leaf, "mix.right.out") || !strcmp(leaf, "mix.left.rel") || !strcmp(leaf, "mix.left.pb");
}

int md_place_tensor(b200_llama *m, const char *name, int type, int64_t ne0, int64_t ne1, int64_t ne2, const void *data) {
    const b200_llama_params &hp = m->hp;
    const int64_t W = hp.n_embd;
    if (!strcmp(name, "embed")) {  // the scale of the embedding is part of the table
        LL_REQUIRE(type == GGML_TYPE_F32 && ne0 == W && ne1 == hp.n_vocab && ne2 == 1, B200_ERR_INVALID, "b200_llama_set_tensor: embed must be f32 [%d, %d]", hp.n_vocab, hp.n_embd);
        const float sc = hp.embed_scale == 0.0f ? 1.0f : hp.embed_scale;
        std::vector<float> t((size_t)(ne0 * ne1));
        for (size_t i = 0; i < t.size(); i++) t[i] = ((const float *)data)[i] * sc;
        return upload_tensor(m, name, type, ne0, ne1, ne2, t.data());
    }
    if (!strcmp(name, "final.norm")) {
        LL_REQUIRE(type == GGML_TYPE_F32 && ne0 == W && ne1 == 1 && ne2 == 1, B200_ERR_INVALID, "b200_llama_set_tensor: %s must be %lld f32 values", name, (long long)W);
        md(m)->host_vecs[name].assign((const float *)data, (const float *)data + W);
        return B200_OK;
    }
    int il = -1;
    const char *leaf = nullptr;
    if (!split_name(name, &il, &leaf)) return upload_tensor(m, name, type, ne0, ne1, ne2, data);
    LL_REQUIRE(il >= 0 && il < hp.n_layer, B200_ERR_INVALID, "b200_llama_set_tensor: %s names a layer outside 0..%d", name, hp.n_layer - 1);
    const b200_layer_params &lp = m->layer_hp[(size_t)il];
    LL_REQUIRE(lp.mixer != 0, B200_ERR_INVALID, "b200_llama_set_tensor: %s before b200_llama_set_layer(%d)", name, il);
    const TypeTraits tt = type_traits(type);
    LL_REQUIRE(tt.blck == 1 && ne2 == 1, B200_ERR_UNSUPPORTED, "b200_llama_set_tensor: %s: dense 1-D / 2-D tensors only", name);
    const std::string pre = "l" + std::to_string(il) + ".";
    const size_t es = (size_t)tt.size;
    if (is_host_vec(lp, leaf)) {
        LL_REQUIRE(type == GGML_TYPE_F32, B200_ERR_INVALID, "b200_llama_set_tensor: %s must be uploaded as f32", name);
        LL_REQUIRE(!md(m)->host_vecs.count(name), B200_ERR_INVALID, "b200_llama_set_tensor: duplicate tensor %s", name);
        md(m)->host_vecs[name].assign((const float *)data, (const float *)data + ne0 * ne1);
        md(m)->host_rows[name] = ne1;
        return B200_OK;
    }
    int e = -1;
    const char *which = nullptr;
    if (lp.mlp == B200_MLP_MOE_GATED && split_expert(leaf, &e, &which)) {
        LL_REQUIRE(e >= 0 && e < lp.n_expert, B200_ERR_INVALID, "b200_llama_set_tensor: %s names an expert outside 0..%d", name, lp.n_expert - 1);
        const int64_t F = lp.ff;
        if (!strcmp(which, "gate") || !strcmp(which, "up")) {
            LL_REQUIRE(ne0 == W && ne1 == F, B200_ERR_INVALID, "b200_llama_set_tensor: %s is [%lld, %lld], expected [%lld, %lld]", name, (long long)ne1, (long long)ne0, (long long)F, (long long)W);
            const size_t off = ((size_t)e * 2 * (size_t)F + (which[0] == 'u' ? (size_t)F : 0)) * (size_t)W * es;
            return place_into(m, pre + "mlp.gate_up", name, type, W, 2 * F, lp.n_expert, off, (size_t)(F * W) * es, data);
        }
        if (!strcmp(which, "down")) {
            LL_REQUIRE(ne0 == F && ne1 == W, B200_ERR_INVALID, "b200_llama_set_tensor: %s is [%lld, %lld], expected [%lld, %lld]", name, (long long)ne1, (long long)ne0, (long long)W, (long long)F);
            return place_into(m, pre + "mlp.down", name, type, F, W, lp.n_expert, (size_t)e * (size_t)(F * W) * es, (size_t)(F * W) * es, data);
        }
    }
    // a part of a fused matrix whose rows are padded to a multiple of 8 with zero weights (their results are zeros nobody reads)
    auto place_rows = [&](const Part *parts, int n, const std::string &fused) -> int {
        int64_t total = 0, rows = 0;
        const int64_t off = part_offset(parts, n, leaf, &total, &rows);
        if (off < 0) return -1;
        LL_REQUIRE(ne0 == W && ne1 == rows, B200_ERR_INVALID, "b200_llama_set_tensor: %s is [%lld, %lld], expected [%lld, %lld]", name, (long long)ne1, (long long)ne0, (long long)rows, (long long)W);
        const bool first = find_w(m, fused) == nullptr;
        const int rc = place_into(m, fused, name, type, W, pad8(total), 1, (size_t)(off * W) * es, (size_t)(rows * W) * es, data);
        if (rc == B200_OK && first && pad8(total) > total) {
            ggml_tensor *f = find_w(m, fused);
            const std::vector<char> z((size_t)((pad8(total) - total) * W) * es, 0);
            f->buffer->iface.set_tensor(f->buffer, f, z.data(), (size_t)(total * W) * es, z.size());
        }
        return rc;
    };
    Part parts[8];
    int rc = place_rows(parts, parts_proj1(lp, parts), pre + "proj1");
    if (rc >= 0) return rc;
    if (lp.mlp == B200_MLP_MOE_GATED && lp.shared_ff > 0) {
        rc = place_rows(parts, parts_shared(lp, parts), pre + "mlp.shared.gate_up");
        if (rc >= 0) return rc;
    }
    std::string names[3];
    Part qkv[3];
    int64_t total = 0, rows = 0;
    parts_qkv(lp, ".conv", names, qkv);
    int64_t off = part_offset(qkv, 3, leaf, &total, &rows);
    if (off >= 0) {  // [channels, taps] each: the fused tensor keeps a channel's taps together
        const int64_t taps = lp.conv_taps;
        LL_REQUIRE(type == GGML_TYPE_F32 && ne0 == taps && ne1 == rows, B200_ERR_INVALID, "b200_llama_set_tensor: %s must be f32 [%lld, %lld]", name, (long long)rows, (long long)taps);
        return place_into(m, pre + "mix.convw", name, type, taps, total, 1, (size_t)(off * taps) * 4, (size_t)(rows * taps) * 4, data);
    }
    if (!is_delta(lp)) {
        parts_qkv(lp, ".b", names, qkv);
        off = part_offset(qkv, 3, leaf, &total, &rows);
        if (off >= 0) {
            LL_REQUIRE(type == GGML_TYPE_F32 && ne0 == rows && ne1 == 1, B200_ERR_INVALID, "b200_llama_set_tensor: %s must be %lld f32 values", name, (long long)rows);
            return place_into(m, pre + "mix.convb", name, type, total, 1, 1, (size_t)off * 4, (size_t)rows * 4, data);
        }
    }
    return upload_tensor(m, name, type, ne0, ne1, ne2, data);
}

// the row of the distance table a key `n` positions back reads: distances below rows / 2 have a row each, the others share the rest
// evenly in ln(distance) up to `far`; a sum that lands on a whole number in exact arithmetic must not fall below it in floating point
int distance_bucket(int64_t n, int64_t rows, int64_t far) {
    const int64_t half = rows / 2;
    if (n < half) return (int)n;
    const double v = log((double)n / (double)half) / log((double)far / (double)half) * (double)(rows - half);
    const int64_t b = half + (int64_t)floor(v + 1e-9);
    return (int)(b < rows - 1 ? b : rows - 1);
}

int md_finalize(b200_llama *m) {
    const b200_llama_params &hp = m->hp;
    MdData *g = md(m);
    g->layers.assign((size_t)hp.n_layer, MdLayer());
    const int64_t W = hp.n_embd;
    g->embed = find_w(m, "embed"); g->head = find_w(m, "head"); g->loop_in = find_w(m, "loop.in");
    LL_REQUIRE(g->embed && g->head && g->host_vecs.count("final.norm"), B200_ERR_INVALID, "b200_llama_finalize: embed / final.norm / head missing");
    LL_REQUIRE(g->head->ne[0] == W && g->head->ne[1] == hp.n_vocab, B200_ERR_INVALID, "b200_llama_finalize: head does not fit width %d and vocabulary %d", hp.n_embd, hp.n_vocab);
    // a vector w on the host becomes the device vector mult * (plus_one + w)
    auto fold = [&](const std::string &out, const std::string &src, float plus_one, float mult, int64_t n, ggml_tensor **dst) -> int {
        auto it = g->host_vecs.find(src);
        LL_REQUIRE(it != g->host_vecs.end() && (int64_t)it->second.size() == n, B200_ERR_INVALID, "b200_llama_finalize: tensor %s missing or not %lld values", src.c_str(), (long long)n);
        std::vector<float> v((size_t)n);
        for (int64_t i = 0; i < n; i++) v[(size_t)i] = mult * (plus_one + it->second[(size_t)i]);
        const int rc = upload_tensor(m, out.c_str(), GGML_TYPE_F32, n, 1, 1, v.data());
        if (rc != B200_OK) return rc;
        *dst = find_w(m, out);
        return B200_OK;
    };
    int rc = fold("final.scale", "final.norm", 1.0f, 1.0f, W, &g->final_scale);
    if (rc != B200_OK) return rc;
    {   // position frequencies 10000^(-2i / width), in double, rounded once
        std::vector<float> f((size_t)((W + 1) / 2));
        for (size_t i = 0; i < f.size(); i++) f[i] = (float)pow(10000.0, -2.0 * (double)i / (double)W);
        rc = upload_tensor(m, "pos_freqs", GGML_TYPE_F32, (int64_t)f.size(), 1, 1, f.data());
        if (rc != B200_OK) return rc;
        g->pos_freqs = find_w(m, "pos_freqs");
    }
    bool any_loop = false;
    for (int il = 0; il < hp.n_layer; il++) {
        const b200_layer_params &lp = m->layer_hp[(size_t)il];
        MdLayer &L = g->layers[(size_t)il];
        const std::string pre = "l" + std::to_string(il) + ".";
        auto need = [&](const char *leaf, int64_t ne0, int64_t ne1, int64_t ne2 = 1) -> ggml_tensor * {
            ggml_tensor *t = find_w(m, pre + leaf);
            if (!t) { b200::set_error("b200_llama_finalize: tensor %s%s missing", pre.c_str(), leaf); return nullptr; }
            if (t->ne[0] != ne0 || t->ne[1] != ne1 || t->ne[2] != ne2) {
                b200::set_error("b200_llama_finalize: tensor %s%s has shape [%lld, %lld, %lld], the layer's sizes give [%lld, %lld, %lld]", pre.c_str(), leaf, (long long)t->ne[2],
                                (long long)t->ne[1], (long long)t->ne[0], (long long)ne2, (long long)ne1, (long long)ne0);
                return nullptr;
            }
            return t;
        };
#define MD_NEED(dst, ...) do { dst = need(__VA_ARGS__); if (!(dst)) return B200_ERR_INVALID; } while (0)
        LL_REQUIRE(lp.mixer == B200_MIXER_DELTA || lp.mixer == B200_MIXER_SIGMOID_ATTENTION_GRU, B200_ERR_INVALID, "b200_llama_finalize: layer %d has no mixer of this architecture", il);
        const int64_t H = lp.heads, G = lp.kv_heads, D = lp.dim, V = lp.vdim;
        LL_REQUIRE(H > 0 && G > 0 && H % G == 0 && D > 0 && D <= 256 && V > 0 && V <= 256, B200_ERR_INVALID, "b200_llama_finalize: layer %d: heads %d over %d kv heads, dim %d and vdim %d (<= 256)", il,
                   lp.heads, lp.kv_heads, lp.dim, lp.vdim);
        LL_REQUIRE(lp.conv_taps >= 1 && lp.conv_taps <= 17, B200_ERR_UNSUPPORTED, "b200_llama_finalize: layer %d: a convolution of 1 to 17 taps", il);
        any_loop |= lp.loop_input != 0;
        if (lp.mlp == B200_MLP_NONE) {
            rc = fold(pre + "pre1", pre + "norm1", 1.0f, 1.0f, W, &L.pre1);
        } else {  // both norms read the same row: one launch over [width, 2, tokens] with the weight chosen by the middle index
            auto n1 = g->host_vecs.find(pre + "norm1"), n2 = g->host_vecs.find(pre + "norm2");
            LL_REQUIRE(n1 != g->host_vecs.end() && n2 != g->host_vecs.end() && (int64_t)n1->second.size() == W && (int64_t)n2->second.size() == W, B200_ERR_INVALID,
                       "b200_llama_finalize: %snorm1 / norm2 missing or not %lld values", pre.c_str(), (long long)W);
            std::vector<float> v((size_t)(2 * W));
            for (int64_t i = 0; i < W; i++) { v[(size_t)i] = 1.0f + n1->second[(size_t)i]; v[(size_t)(W + i)] = 1.0f + n2->second[(size_t)i]; }
            rc = upload_tensor(m, (pre + "pre12").c_str(), GGML_TYPE_F32, W, 2, 1, v.data());
            L.pre12 = find_w(m, pre + "pre12");
        }
        if (rc != B200_OK) return rc;
        Part parts[8];
        int np = parts_proj1(lp, parts);
        int64_t total = 0;
        part_offset(parts, np, "", &total);
        for (int i = 0; i < np; i++) LL_REQUIRE(find_w(m, pre + parts[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), parts[i].leaf);
        L.proj1_rows = pad8(total);
        L.conv_channels = parts[0].rows + parts[1].rows + parts[2].rows;
        MD_NEED(L.proj1, "proj1", W, L.proj1_rows);
        std::string names[3];
        Part qkv[3];
        parts_qkv(lp, ".conv", names, qkv);
        for (int i = 0; i < 3; i++) LL_REQUIRE(find_w(m, pre + qkv[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), qkv[i].leaf);
        MD_NEED(L.convw, "mix.convw", lp.conv_taps, L.conv_channels);
        if (is_delta(lp)) {
            MD_NEED(L.wo, "mix.o", H * V, W);
            MD_NEED(L.a_log, "mix.A_log", H, 1);
            MD_NEED(L.dt_bias, "mix.dt_bias", H, 1);
            MD_NEED(L.onorm, "mix.norm", V, 1);
        } else {
            parts_qkv(lp, ".b", names, qkv);
            for (int i = 0; i < 3; i++) LL_REQUIRE(find_w(m, pre + qkv[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), qkv[i].leaf);
            MD_NEED(L.convb, "mix.convb", L.conv_channels, 1);
            MD_NEED(L.wo, "mix.left.o", H * V, W);
            MD_NEED(L.wo_bias, "mix.left.o.b", W, 1);
            LL_REQUIRE(lp.side_width > 0, B200_ERR_INVALID, "b200_llama_finalize: layer %d: the minGRU needs a width", il);
            MD_NEED(L.zb, "mix.right.z.b", lp.side_width, 1);
            MD_NEED(L.xb, "mix.right.x.b", lp.side_width, 1);
            MD_NEED(L.wo_side, "mix.right.o", lp.side_width, W);
            // the two sides are averaged behind their norms: the half joins their weights
            rc = fold(pre + "mix.out_l", pre + "mix.left.out", 0.0f, 0.5f, W, &L.out_l);
            if (rc != B200_OK) return rc;
            rc = fold(pre + "mix.out_r", pre + "mix.right.out", 0.0f, 0.5f, W, &L.out_r);
            if (rc != B200_OK) return rc;
            // per head rel[bucket(n)][h] + pb[h] for n = 0 .. bias_max; the last entry serves every greater distance
            auto rel = g->host_vecs.find(pre + "mix.left.rel"), pb = g->host_vecs.find(pre + "mix.left.pb");
            LL_REQUIRE(rel != g->host_vecs.end() && pb != g->host_vecs.end() && (int64_t)pb->second.size() == H, B200_ERR_INVALID, "b200_llama_finalize: %smix.left.rel / pb missing", pre.c_str());
            const int64_t rows = g->host_rows[pre + "mix.left.rel"], far = lp.dist_bias_max;
            LL_REQUIRE(rows >= 2 && (int64_t)rel->second.size() == rows * H && far > rows / 2, B200_ERR_INVALID,
                       "b200_llama_finalize: layer %d: a distance table of [rows >= 2, %lld] with the farthest distance beyond rows / 2", il, (long long)H);
            std::vector<float> tab((size_t)((far + 1) * H));
            for (int64_t n = 0; n <= far; n++)
                for (int64_t h = 0; h < H; h++) tab[(size_t)(h * (far + 1) + n)] = rel->second[(size_t)(distance_bucket(n, rows, far) * H + h)] + pb->second[(size_t)h];
            rc = upload_tensor(m, (pre + "mix.dist").c_str(), GGML_TYPE_F32, far + 1, H, 1, tab.data());
            if (rc != B200_OK) return rc;
            L.dist = find_w(m, pre + "mix.dist");
        }
        if (lp.mlp == B200_MLP_NONE) continue;
        LL_REQUIRE(lp.mlp == B200_MLP_MOE_GATED && lp.ff > 0 && lp.n_expert > 0 && lp.n_expert <= 256 && lp.n_expert_used > 0 && lp.n_expert_used <= 32 && lp.n_expert_used <= lp.n_expert,
                   B200_ERR_UNSUPPORTED, "b200_llama_finalize: layer %d: feed-forward kind / expert counts (at most 256 experts, 32 per token)", il);
        for (int e = 0; e < lp.n_expert; e++)
            for (const char *w : {"gate", "up", "down"}) {
                const std::string nm = pre + "mlp.e" + std::to_string(e) + "." + w;
                LL_REQUIRE(find_w(m, nm), B200_ERR_INVALID, "b200_llama_finalize: tensor %s missing", nm.c_str());
            }
        MD_NEED(L.gate_up, "mlp.gate_up", W, 2 * (int64_t)lp.ff, lp.n_expert);
        MD_NEED(L.down, "mlp.down", lp.ff, W, lp.n_expert);
        MD_NEED(L.router, "mlp.router", W, lp.n_expert);
        LL_REQUIRE(L.router->type == GGML_TYPE_F32, B200_ERR_INVALID, "b200_llama_finalize: %smlp.router must be uploaded as f32 (the router runs in f32 in every mode)", pre.c_str());
        if (lp.shared_ff > 0) {
            np = parts_shared(lp, parts);
            for (int i = 0; i < np; i++) LL_REQUIRE(find_w(m, pre + parts[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), parts[i].leaf);
            L.sh_rows = pad8(2 * (int64_t)lp.shared_ff + 1);
            MD_NEED(L.sh_gate_up, "mlp.shared.gate_up", W, L.sh_rows);
            MD_NEED(L.sh_down, "mlp.shared.down", lp.shared_ff, W);
        }
#undef MD_NEED
    }
    LL_REQUIRE(!any_loop || (g->loop_in && g->loop_in->ne[0] == 2 * W && g->loop_in->ne[1] == W), B200_ERR_INVALID, "b200_llama_finalize: loop.in must be [%lld, %lld]", (long long)W, (long long)(2 * W));
    g->host_vecs.clear();
    g->host_rows.clear();
    // every run of a layer owns its cache rows, its convolution tail and its state
    if (m->run_layer.empty()) for (int il = 0; il < hp.n_layer; il++) m->run_layer.push_back(il);
    g->runs.resize(m->run_layer.size());
    for (size_t r = 0; r < m->run_layer.size(); r++) {
        const int il = m->run_layer[r];
        const b200_layer_params &lp = m->layer_hp[(size_t)il];
        MdRun &R = g->runs[r];
        const std::string pre = "run" + std::to_string(r) + ".";
        const int64_t tail_floats = (int64_t)(lp.conv_taps - 1) * g->layers[(size_t)il].conv_channels;
        R.tail = new_device_tensor(m, (pre + "tail").c_str(), GGML_TYPE_F32, tail_floats > 0 ? tail_floats : 1, hp.n_seq_max, true);
        if (is_delta(lp)) {
            R.state = new_device_tensor(m, (pre + "state").c_str(), GGML_TYPE_F32, (int64_t)lp.heads * lp.dim * lp.vdim, hp.n_seq_max, true);
        } else {
            R.state = new_device_tensor(m, (pre + "state").c_str(), GGML_TYPE_F32, lp.side_width, hp.n_seq_max, true);
            R.k_cache = new_device_tensor(m, (pre + "k").c_str(), GGML_TYPE_F32, (int64_t)lp.kv_heads * lp.dim, hp.n_ctx, true);
            R.v_cache = new_device_tensor(m, (pre + "v").c_str(), GGML_TYPE_F32, (int64_t)lp.kv_heads * lp.vdim, hp.n_ctx, true);
            LL_REQUIRE(R.k_cache && R.v_cache, B200_ERR_NOMEM, "b200_llama_finalize: out of device memory for the cache of run %zu", r);
            m->kv_bytes += (int64_t)(nbytes(R.k_cache) + nbytes(R.v_cache));
        }
        LL_REQUIRE(R.tail && R.state, B200_ERR_NOMEM, "b200_llama_finalize: out of device memory for the state of run %zu", r);
        m->kv_bytes += (int64_t)(nbytes(R.tail) + nbytes(R.state));
    }
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ graph of one batch step
enum { R_HEAD = 0, R_EVEN = 1, R_ODD = 2, R_TAIL = 3 };

int md_build(b200_llama *m, const BatchShape &bs) {
    const b200_llama_params &hp = m->hp;
    MdData *g = md(m);
    const int64_t T = bs.n_tokens, W = hp.n_embd;
    const float eps = hp.rms_eps, mult = hp.residual_mult == 0.0f ? 1.0f : hp.residual_mult;
    m->arena.reset();
    Builder b;
    b.arena = &m->arena;
    for (Bump &r : m->regions) r.off = 0;
    auto input_view = [&](const ggml_tensor &base, int64_t ne0, int64_t ne1 = 1) {
        ggml_tensor *t = m->arena.get();
        *t = base;
        set_shape(t, base.type, ne0, ne1, 1, 1);
        return t;
    };
    ggml_tensor *tokens = input_view(m->inp_tokens, T), *pos = input_view(m->inp_pos, T), *cells = input_view(m->inp_cells, T), *tok_seq = input_view(m->inp_tok_seq, T);
    ggml_tensor *cell_seq = input_view(m->inp_cell_seq, bs.n_kv), *cell_pos = input_view(m->inp_cell_pos, bs.n_kv), *seq_info = input_view(m->inp_seq_info, bs.n_seq, 4);

    // RMS norm with a weight; optionally a gate on the result (2: silu) and a residual operand
    auto norm = [&](ggml_tensor *x, ggml_tensor *w, ggml_tensor *gate = nullptr, int gate_kind = 0, ggml_tensor *res = nullptr) {
        ggml_tensor *dst = b.alloc_result(GGML_TYPE_F32, x->ne[0], x->ne[1], x->ne[2], 1);
        b.ext(dst, B200_EXT_NORM, {x, w, gate, nullptr, res, nullptr});
        dst->op_params[2] = B200_NORM_RMS; Builder::set_f(dst, 3, eps); dst->op_params[4] = 1; dst->op_params[5] = gate ? gate_kind : 0;
        return dst;
    };
    // rows [row0, row0 + rows) of a stacked tensor [2 W, T] as a [rows, T] tensor the producing node writes directly
    auto rows_of = [&](ggml_tensor *stack, int64_t row0, int64_t rows) {
        ggml_tensor *t = b.result_at(stack, (size_t)row0 * 4, GGML_TYPE_F32, rows, T);
        t->nb[1] = stack->nb[1]; t->nb[2] = t->nb[3] = t->nb[1] * (size_t)T;
        return t;
    };

    b.bump = &m->regions[R_HEAD];
    bool any_loop = false;
    for (int il : m->run_layer) any_loop |= m->layer_hp[(size_t)il].loop_input != 0;
    // with a looped stretch the stream and its first value wait side by side as [x ; x0] for the input projection of a pass
    ggml_tensor *cat = any_loop ? b.alloc_result(GGML_TYPE_F32, 2 * W, T) : nullptr;
    ggml_tensor *e = b.op(b.alloc_result(GGML_TYPE_F32, W, T), GGML_OP_GET_ROWS, g->embed, tokens);
    ggml_tensor *x0 = b.ext(cat ? rows_of(cat, W, W) : b.alloc_result(GGML_TYPE_F32, W, T), B200_EXT_ADD_SINUSOID, {e, pos, g->pos_freqs});
    ggml_tensor *x = x0;
    bool x_in_cat = false;  // x was written straight into the first half of cat

    for (size_t r = 0; r < m->run_layer.size(); r++) {
        const int il = m->run_layer[r];
        const b200_layer_params &lp = m->layer_hp[(size_t)il];
        MdLayer &L = g->layers[(size_t)il];
        MdRun &R = g->runs[r];
        b.bump = &m->regions[(r & 1) ? R_ODD : R_EVEN];
        b.bump->off = 0;
        const int64_t H = lp.heads, G = lp.kv_heads, D = lp.dim, V = lp.vdim;
        if (lp.loop_input) {
            ggml_tensor *last = x;  // the node that completes [x ; x0]
            if (!x_in_cat) last = b.cpy(x, rows_of(cat, 0, W));
            ggml_tensor *both = b.view_of(last, GGML_OP_VIEW, 0);
            set_shape(both, GGML_TYPE_F32, 2 * W, T, 1, 1);
            both->data = cat->data; both->view_src = cat; both->view_offs = 0;
            x = b.mul_mat(g->loop_in, both);
        }
        ggml_tensor *h1, *h2 = nullptr, *h2_3d = nullptr;
        if (L.pre12) {
            ggml_tensor *hh = b.alloc_result(GGML_TYPE_F32, W, 2, T);
            b.ext(hh, B200_EXT_NORM, {b.view_3d(x, W, 2, T, 0, x->nb[1], 0), L.pre12, nullptr, nullptr, nullptr, nullptr});
            hh->op_params[2] = B200_NORM_RMS; Builder::set_f(hh, 3, eps); hh->op_params[4] = 2; hh->op_params[5] = 0;
            h1 = b.view_2d(hh, W, T, hh->nb[2], 0);
            h2 = b.view_2d(hh, W, T, hh->nb[2], (size_t)W * 4);
            h2_3d = b.view_3d(hh, W, 1, T, hh->nb[2], hh->nb[2], (size_t)W * 4);
        } else {
            h1 = norm(x, L.pre1);
        }
        ggml_tensor *P = b.mul_mat(L.proj1, h1);
        Part parts[8];
        const int np = parts_proj1(lp, parts);
        auto part = [&](ggml_tensor *src, const char *leaf) {
            int64_t rows = 0;
            const int64_t off = part_offset(parts, np, leaf, nullptr, &rows);
            return b.view_2d(src, rows, T, src->nb[1], (size_t)off * 4);
        };
        // q, k, v are the first rows of P: one convolution over all their channels, then the same offsets hold in its result
        const int64_t CC = L.conv_channels;
        ggml_tensor *C = b.ext(b.alloc_result(GGML_TYPE_F32, CC, T), B200_EXT_SHORT_CONV, {b.view_2d(P, CC, T, P->nb[1], 0), L.convw, L.convb, seq_info, R.tail});
        C->op_params[2] = is_delta(lp) ? 1 : 0;
        ggml_tensor *y;  // the mixer's result [W, T]
        if (is_delta(lp)) {
            ggml_tensor *o = b.alloc_result(GGML_TYPE_F32, H * V, T);
            b.ext(o, B200_EXT_DELTA_RULE_SCAN, {part(C, "mix.q"), part(C, "mix.k"), part(C, "mix.v"), part(P, "mix.a"), part(P, "mix.b"), L.a_log, L.dt_bias, seq_info, R.state});
            o->op_params[2] = (int32_t)H; o->op_params[3] = (int32_t)G; o->op_params[4] = (int32_t)D; o->op_params[5] = (int32_t)V; o->op_params[6] = 1;
            Builder::set_f(o, 7, kUnitEps); Builder::set_f(o, 8, 1.0f / sqrtf((float)D));
            // every head's read-out: RMS norm over vdim, the shared weight, times silu of the gate projection
            int64_t g_rows = 0;
            const int64_t g_off = part_offset(parts, np, "mix.g", nullptr, &g_rows);
            ggml_tensor *gate = b.view_3d(P, V, H, T, (size_t)V * 4, P->nb[1], (size_t)g_off * 4);
            ggml_tensor *on = norm(b.reshape(o, V, H, T), L.onorm, gate, 2);
            y = b.mul_mat(L.wo, b.reshape(on, H * V, T));
        } else {
            ggml_tensor *kc_all = b.view_2d(R.k_cache, G * D, hp.n_ctx, R.k_cache->nb[1], 0), *vc_all = b.view_2d(R.v_cache, G * V, hp.n_ctx, R.v_cache->nb[1], 0);
            ggml_tensor *q = part(C, "mix.left.q");
            ggml_tensor *qo = part(C, "mix.left.q");  // the store rewrites q in place
            b.ext(qo, B200_EXT_QKV_STORE, {q, part(C, "mix.left.k"), part(C, "mix.left.v"), nullptr, pos, nullptr, cells, kc_all, vc_all});
            qo->op_params[2] = (int32_t)D; qo->op_params[3] = (int32_t)V; qo->op_params[4] = 0; Builder::set_f(qo, 5, eps);
            qo->op_params[6] = 0; qo->op_params[7] = 0; qo->op_params[8] = 0;
            qo->op_params[9] = 1; Builder::set_f(qo, 10, lp.q_temp_coef); qo->op_params[11] = lp.q_temp_every;
            ggml_tensor *o = b.alloc_result(GGML_TYPE_F32, H * V, T);
            b.ext(o, B200_EXT_SINK_ATTN, {qo, b.view_2d(R.k_cache, G * D, bs.n_kv, R.k_cache->nb[1], 0), b.view_2d(R.v_cache, G * V, bs.n_kv, R.v_cache->nb[1], 0), nullptr, tok_seq, pos,
                                           cell_seq, cell_pos, nullptr, L.dist});
            o->op_params[2] = (int32_t)D; Builder::set_f(o, 3, lp.scale); o->op_params[4] = 0; o->op_params[5] = 0;
            // bf16 weights: the attention products of a prompt batch may be bf16 as well (B200_ATTN_F32=1 keeps them in f32)
            static const bool attn_f32 = getenv("B200_ATTN_F32") != nullptr;
            o->op_params[6] = L.proj1->type == GGML_TYPE_BF16 && !attn_f32;
            o->op_params[7] = (int32_t)V; o->op_params[8] = 0; o->op_params[9] = B200_ATTN_SIGMOID;
            ggml_tensor *ya = b.mul_mat(L.wo, o);
            ggml_tensor *s = b.alloc_result(GGML_TYPE_F32, lp.side_width, T);
            b.ext(s, B200_EXT_MINGRU_SCAN, {part(P, "mix.right.z"), part(P, "mix.right.x"), part(P, "mix.right.g"), L.zb, L.xb, seq_info, R.state});
            ggml_tensor *yg = b.mul_mat(L.wo_side, s);
            // the output bias of the attention side, both sides' norms, their weights (halved) and the sum: one launch
            if (W <= 16384) {
                y = b.ext(b.alloc_result(GGML_TYPE_F32, W, T), B200_EXT_NORM_PAIR, {ya, L.out_l, L.wo_bias, yg, L.out_r});
                Builder::set_f(y, 3, eps);
            } else {
                y = norm(yg, L.out_r, nullptr, 0, norm(b.binary(GGML_OP_ADD, ya, L.wo_bias), L.out_l));
            }
        }
        // where the layer's result goes: the first half of [x ; x0] when the next run starts a pass
        const bool next_starts = r + 1 < m->run_layer.size() && m->layer_hp[(size_t)m->run_layer[r + 1]].loop_input != 0;
        ggml_tensor *nx = next_starts ? rows_of(cat, 0, W) : b.alloc_result(GGML_TYPE_F32, W, T);
        if (lp.mlp == B200_MLP_MOE_GATED) {
            const int64_t F = lp.ff, NU = lp.n_expert_used;
            // the router's result: per token NU weights, then NU expert ids (as i32) in the same row
            ggml_tensor *rt = b.alloc_result(GGML_TYPE_F32, 2 * NU, T);
            b.ext(rt, B200_EXT_MOE_ROUTE, {b.mul_mat(L.router, h2), nullptr});
            rt->op_params[2] = 1; rt->op_params[3] = 1; Builder::set_f(rt, 4, lp.router_scale == 0.0f ? 1.0f : lp.router_scale); rt->op_params[5] = (int32_t)NU;
            rt->op_params[6] = lp.router_score; rt->op_params[7] = lp.router_keep_scores ? 1 : 0;
            ggml_tensor *wts = b.view_2d(rt, NU, T, rt->nb[1], 0), *ids = b.view_2d(rt, NU, T, rt->nb[1], (size_t)NU * 4);
            ids->type = GGML_TYPE_I32;
            ggml_tensor *gu = b.ext(b.alloc_result(GGML_TYPE_F32, 2 * F, NU, T), B200_EXT_MUL_MAT_ID, {L.gate_up, h2_3d, ids});
            // an expert's weight scales its input: the same factor on both of its linear products, applied where they are read
            ggml_tensor *act = b.ext(b.alloc_result(GGML_TYPE_F32, F, NU, T), B200_EXT_SILU_MUL,
                                     {b.view_3d(gu, F, NU, T, gu->nb[1], gu->nb[2], 0), b.view_3d(gu, F, NU, T, gu->nb[1], gu->nb[2], (size_t)F * 4), lp.router_scale_input ? wts : nullptr});
            act->op_params[2] = B200_GLU_SILU;
            ggml_tensor *dn = b.ext(b.alloc_result(GGML_TYPE_F32, W, NU, T), B200_EXT_MUL_MAT_ID, {L.down, act, ids});
            ggml_tensor *sdn = nullptr, *sg = nullptr;
            if (lp.shared_ff > 0) {
                const int64_t FS = lp.shared_ff;
                ggml_tensor *sgu = b.mul_mat(L.sh_gate_up, h2);
                ggml_tensor *sact = b.ext(b.alloc_result(GGML_TYPE_F32, FS, T), B200_EXT_SILU_MUL, {b.view_2d(sgu, FS, T, sgu->nb[1], 0), b.view_2d(sgu, FS, T, sgu->nb[1], (size_t)FS * 4)});
                sact->op_params[2] = B200_GLU_SILU;
                sdn = b.mul_mat(L.sh_down, sact);
                sg = b.view_2d(sgu, 1, T, sgu->nb[1], (size_t)(2 * FS) * 4);
            }
            b.ext(nx, B200_EXT_MOE_COMBINE, {dn, lp.router_scale_input ? nullptr : wts, x, y, nullptr, sdn, sg});
        } else {
            b.ext(nx, B200_EXT_MOE_COMBINE, {nullptr, nullptr, x, y, nullptr, nullptr, nullptr});
        }
        nx->op_params[2] = 0; Builder::set_f(nx, 4, mult);
        x = nx;
        x_in_cat = next_starts;
    }
    b.bump = &m->regions[R_TAIL];
    ggml_tensor *out = x;
    if (bs.n_outputs > 0) {
        if (bs.n_outputs < T) out = b.get_rows(out, input_view(m->inp_out_ids, bs.n_outputs));
        out = b.mul_mat(g->head, norm(out, g->final_scale));
    }
    b.expand(out);
    for (Bump &r : m->regions) LL_REQUIRE(m->measuring || r.off <= r.size, B200_ERR_NOMEM, "b200_llama_decode_batch: compute buffer too small for this batch");
    LL_REQUIRE(!b.oom, B200_ERR_NOMEM, "b200_llama_decode_batch: compute buffer too small for this batch");
    m->logits_t = bs.n_outputs > 0 ? out : nullptr;
    m->graph_nodes.swap(b.nodes);
    memset(&m->graph, 0, sizeof(m->graph));
    m->graph.size = m->graph.n_nodes = (int)m->graph_nodes.size();
    m->graph.nodes = m->graph_nodes.data();
    return B200_OK;
}

const Arch k_medodra = {"medodra", md_place_tensor, md_finalize, nullptr, md_build, nullptr};

}  // namespace

const Arch *b200::host::medodra_arch() { return &k_medodra; }

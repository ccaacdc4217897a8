// host_zevopel.cu -- the Zevopel architecture for the decoder of host_llama.cu: where its tensors go and the graph of one batch
// step.  The decoder owns the model object, the sequence cache, the inputs and the step; this file adds no loop of its own.
//
// A Zevopel layer normalises what a sublayer returns, not what it reads:
//     x <- x + c * a1 * N1(mixer(x)),   x <- x + c * a2 * N2(ff(x))
// with c the model's residual multiplier, a1 / a2 per-channel scales ("ls1", "ls2") and N an RMS norm whose stored weight w acts
// as (1 + w).  The mixer is grouped-query attention (b200_layer_params): an RMS norm per head on q and k with one weight vector for
// all heads, rotation of pairs (i, i + n/2) by a band-scaled frequency table, a per-head sink in the softmax denominator, positions
// cut into chunks that do not see each other, and a sigmoid gate per head computed from the mixer's input.  The feed-forward is
// dense (gelu(gate x) * up x -> down) or a mixture of experts with clamped gate / up products, a softmax router over all experts
// and the chosen experts' scores as weights.  The embedding is scaled; the output is the same norm and the head.
//
// Graph choices: q, k, v and the head gates are ONE product over row-concatenated weights (rows padded to a multiple of 8 so that
// every slice of the result starts 16-byte aligned when the sizes allow it); gate and up are one product; per-head norm, rotation
// and the cache store are one launch; sink, chunks and the head gate live inside the attention kernels; c * a * (1 + w) is folded
// into ONE weight vector per norm when the model is finalised, so "norm, scale, add to the stream" is one launch (behind the
// experts the weighted sum over the chosen ones is part of that launch too); the embedding
// scale is folded into the f32 table; the router is an f32 product of f32 weights with the unrounded stream in every mode.
#include "host_fused.h"

namespace {

struct ZvLayer {
    ggml_tensor *proj1 = nullptr, *wo = nullptr, *qknorm = nullptr, *sink = nullptr, *freqs = nullptr, *post1 = nullptr, *post2 = nullptr;
    ggml_tensor *gate_up = nullptr, *down = nullptr, *router = nullptr;
    int64_t proj1_rows = 0;
};
struct ZvRun {
    ggml_tensor *k_cache = nullptr, *v_cache = nullptr;  // [kv_heads * dim, n_ctx], [kv_heads * vdim, n_ctx] f32
};
struct ZvData {
    std::map<std::string, std::vector<float>> host_vecs;  // the vectors that finalize folds into one weight per norm
    std::vector<ZvLayer> layers;
    std::vector<ZvRun> runs;
    ggml_tensor *embed = nullptr, *final_scale = nullptr, *head = nullptr;
};
ZvData *zv(b200_llama *m) {
    if (!m->arch_data) m->arch_data = std::shared_ptr<void>(new ZvData(), [](void *p) { delete (ZvData *)p; });
    return (ZvData *)m->arch_data.get();
}

int64_t pad8(int64_t v) { return (v + 7) / 8 * 8; }
int parts_proj1(const b200_layer_params &lp, Part out[8]) {
    int n = 0;
    const int64_t H = lp.heads, G = lp.kv_heads, D = lp.dim, V = lp.vdim;
    out[n++] = {"mix.q", H * D};
    out[n++] = {"mix.k", G * D};
    out[n++] = {"mix.v", G * V};
    if (lp.head_gate) out[n++] = {"mix.g", H};
    return n;
}
int parts_qknorm(const b200_layer_params &lp, Part out[8]) {
    if (!lp.qk_norm) return 0;
    const int64_t nq = lp.qk_norm_per_head ? lp.dim : (int64_t)lp.heads * lp.dim, nk = lp.qk_norm_per_head ? lp.dim : (int64_t)lp.kv_heads * lp.dim;
    out[0] = {"mix.q.norm", nq};
    out[1] = {"mix.k.norm", nk};
    return 2;
}
bool is_folded_vec(const char *leaf) { return !strcmp(leaf, "norm1") || !strcmp(leaf, "norm2") || !strcmp(leaf, "ls1") || !strcmp(leaf, "ls2"); }

int zv_place_tensor(b200_llama *m, const char *name, int type, int64_t ne0, int64_t ne1, int64_t ne2, const void *data) {
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
        zv(m)->host_vecs[name].assign((const float *)data, (const float *)data + W);
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
    if (is_folded_vec(leaf)) {
        LL_REQUIRE(type == GGML_TYPE_F32 && ne0 == W && ne1 == 1, B200_ERR_INVALID, "b200_llama_set_tensor: %s must be %lld f32 values", name, (long long)W);
        LL_REQUIRE(!zv(m)->host_vecs.count(name), B200_ERR_INVALID, "b200_llama_set_tensor: duplicate tensor %s", name);
        zv(m)->host_vecs[name].assign((const float *)data, (const float *)data + W);
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
    if (lp.mlp == B200_MLP_DENSE_GATED && (!strcmp(leaf, "mlp.gate") || !strcmp(leaf, "mlp.up"))) {
        const int64_t F = lp.ff;
        LL_REQUIRE(ne0 == W && ne1 == F, B200_ERR_INVALID, "b200_llama_set_tensor: %s is [%lld, %lld], expected [%lld, %lld]", name, (long long)ne1, (long long)ne0, (long long)F, (long long)W);
        return place_into(m, pre + "mlp.gate_up", name, type, W, 2 * F, 1, leaf[4] == 'u' ? (size_t)(F * W) * es : 0, (size_t)(F * W) * es, data);
    }
    Part parts[8];
    int64_t total = 0, rows = 0;
    int n = parts_proj1(lp, parts);
    int64_t off = part_offset(parts, n, leaf, &total, &rows);
    if (off >= 0) {
        LL_REQUIRE(ne0 == W && ne1 == rows, B200_ERR_INVALID, "b200_llama_set_tensor: %s is [%lld, %lld], expected [%lld, %lld]", name, (long long)ne1, (long long)ne0, (long long)rows, (long long)W);
        const bool first = find_w(m, pre + "proj1") == nullptr;
        const int rc = place_into(m, pre + "proj1", name, type, W, pad8(total), 1, (size_t)(off * W) * es, (size_t)(rows * W) * es, data);
        if (rc == B200_OK && first && pad8(total) > total) {  // the padding rows are zero weights: their results are zeros nobody reads
            ggml_tensor *f = find_w(m, pre + "proj1");
            const std::vector<char> z((size_t)((pad8(total) - total) * W) * es, 0);
            f->buffer->iface.set_tensor(f->buffer, f, z.data(), (size_t)(total * W) * es, z.size());
        }
        return rc;
    }
    n = parts_qknorm(lp, parts);
    off = part_offset(parts, n, leaf, &total, &rows);
    if (off >= 0) {
        LL_REQUIRE(type == GGML_TYPE_F32 && ne0 == rows && ne1 == 1, B200_ERR_INVALID, "b200_llama_set_tensor: %s must be %lld f32 values", name, (long long)rows);
        return place_into(m, pre + "mix.qknorm", name, type, total, 1, 1, (size_t)off * 4, (size_t)rows * 4, data);
    }
    return upload_tensor(m, name, type, ne0, ne1, ne2, data);
}

int zv_finalize(b200_llama *m) {
    const b200_llama_params &hp = m->hp;
    ZvData *g = zv(m);
    g->layers.assign((size_t)hp.n_layer, ZvLayer());
    const int64_t W = hp.n_embd;
    const float c = hp.residual_mult == 0.0f ? 1.0f : hp.residual_mult;
    g->embed = find_w(m, "embed"); g->head = find_w(m, "head");
    LL_REQUIRE(g->embed && g->head && g->host_vecs.count("final.norm"), B200_ERR_INVALID, "b200_llama_finalize: embed / final.norm / head missing");
    LL_REQUIRE(g->head->ne[0] == W && g->head->ne[1] == hp.n_vocab, B200_ERR_INVALID, "b200_llama_finalize: head does not fit width %d and vocabulary %d", hp.n_embd, hp.n_vocab);
    // a norm's weight acts as (1 + w); the per-channel scale and the residual multiplier behind it join the same vector (f32)
    auto fold = [&](const std::string &out, const std::string &norm, const std::string &scale, float mult, ggml_tensor **dst) -> int {
        auto wn = g->host_vecs.find(norm);
        LL_REQUIRE(wn != g->host_vecs.end(), B200_ERR_INVALID, "b200_llama_finalize: tensor %s missing", norm.c_str());
        std::vector<float> v((size_t)W);
        for (int64_t i = 0; i < W; i++) v[(size_t)i] = 1.0f + wn->second[(size_t)i];
        if (!scale.empty()) {
            auto ws = g->host_vecs.find(scale);
            LL_REQUIRE(ws != g->host_vecs.end(), B200_ERR_INVALID, "b200_llama_finalize: tensor %s missing", scale.c_str());
            for (int64_t i = 0; i < W; i++) v[(size_t)i] = v[(size_t)i] * ws->second[(size_t)i] * mult;
        }
        const int rc = upload_tensor(m, out.c_str(), GGML_TYPE_F32, W, 1, 1, v.data());
        if (rc != B200_OK) return rc;
        *dst = find_w(m, out);
        return B200_OK;
    };
    int rc = fold("final.scale", "final.norm", "", 1.0f, &g->final_scale);
    if (rc != B200_OK) return rc;
    for (int il = 0; il < hp.n_layer; il++) {
        const b200_layer_params &lp = m->layer_hp[(size_t)il];
        ZvLayer &L = g->layers[(size_t)il];
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
#define ZV_NEED(dst, ...) do { dst = need(__VA_ARGS__); if (!(dst)) return B200_ERR_INVALID; } while (0)
        LL_REQUIRE(lp.mixer == B200_MIXER_ATTENTION, B200_ERR_INVALID, "b200_llama_finalize: layer %d has no mixer of this architecture", il);
        const int64_t H = lp.heads, G = lp.kv_heads, D = lp.dim, V = lp.vdim;
        LL_REQUIRE(H > 0 && G > 0 && H % G == 0 && D > 0 && D <= 256 && V > 0 && V <= 256, B200_ERR_INVALID, "b200_llama_finalize: layer %d: heads %d over %d kv heads, dim %d and vdim %d (<= 256)", il,
                   lp.heads, lp.kv_heads, lp.dim, lp.vdim);
        LL_REQUIRE(lp.rope_dims >= 0 && lp.rope_dims % 2 == 0 && lp.rope_dims <= D && (lp.rope_dims == 0 || lp.rope_base > 0.0f), B200_ERR_INVALID, "b200_llama_finalize: layer %d: rotation does not fit dim", il);
        LL_REQUIRE(lp.rope_scaling == B200_ROPE_SCALING_NONE || (lp.rope_scaling == B200_ROPE_SCALING_BANDS && lp.yarn_factor > 0.0f && lp.yarn_original > 0 && lp.band_low > 0.0f &&
                   lp.band_high > lp.band_low), B200_ERR_INVALID, "b200_llama_finalize: layer %d: frequency scaling parameters", il);
        LL_REQUIRE(lp.window >= 0 && lp.keep_first >= 0 && lp.chunk >= 0, B200_ERR_INVALID, "b200_llama_finalize: layer %d: window / kept first positions / chunk must not be negative", il);
        Part parts[8];
        int np = parts_proj1(lp, parts);
        int64_t total = 0;
        part_offset(parts, np, "", &total);
        for (int i = 0; i < np; i++) LL_REQUIRE(find_w(m, pre + parts[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), parts[i].leaf);
        L.proj1_rows = pad8(total);
        ZV_NEED(L.proj1, "proj1", W, L.proj1_rows);
        ZV_NEED(L.wo, "mix.o", H * V, W);
        ZV_NEED(L.sink, "mix.sink", H, 1);
        np = parts_qknorm(lp, parts);
        if (np > 0) {
            part_offset(parts, np, "", &total);
            for (int i = 0; i < np; i++) LL_REQUIRE(find_w(m, pre + parts[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), parts[i].leaf);
            ZV_NEED(L.qknorm, "mix.qknorm", total, 1);
        }
        std::vector<float> f;
        rope_freqs(lp, f);
        if (f.empty()) f.push_back(0.0f);
        const std::string fname = pre + "rope_freqs";
        rc = upload_tensor(m, fname.c_str(), GGML_TYPE_F32, (int64_t)f.size(), 1, 1, f.data());
        if (rc != B200_OK) return rc;
        L.freqs = find_w(m, fname);
        rc = fold(pre + "post1", pre + "norm1", pre + "ls1", c, &L.post1);
        if (rc != B200_OK) return rc;
        if (lp.mlp == B200_MLP_NONE) continue;
        rc = fold(pre + "post2", pre + "norm2", pre + "ls2", c, &L.post2);
        if (rc != B200_OK) return rc;
        LL_REQUIRE(lp.ff > 0 && (lp.glu_kind == B200_GLU_SILU || lp.glu_kind == B200_GLU_GELU_TANH || lp.glu_kind == B200_GLU_SWISH_CLAMPED), B200_ERR_INVALID,
                   "b200_llama_finalize: layer %d: feed-forward size / activation", il);
        if (lp.mlp == B200_MLP_DENSE_GATED) {
            for (const char *w : {"mlp.gate", "mlp.up"}) LL_REQUIRE(find_w(m, pre + w), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), w);
            ZV_NEED(L.gate_up, "mlp.gate_up", W, 2 * (int64_t)lp.ff);
            ZV_NEED(L.down, "mlp.down", lp.ff, W);
        } else {
            LL_REQUIRE(lp.mlp == B200_MLP_MOE_GATED && lp.n_expert > 0 && lp.n_expert <= 256 && lp.n_expert_used > 0 && lp.n_expert_used <= 32 && lp.n_expert_used <= lp.n_expert,
                       B200_ERR_UNSUPPORTED, "b200_llama_finalize: layer %d: feed-forward kind / expert counts (at most 256 experts, 32 per token)", il);
            for (int e = 0; e < lp.n_expert; e++)
                for (const char *w : {"gate", "up", "down"}) {
                    const std::string nm = pre + "mlp.e" + std::to_string(e) + "." + w;
                    LL_REQUIRE(find_w(m, nm), B200_ERR_INVALID, "b200_llama_finalize: tensor %s missing", nm.c_str());
                }
            ZV_NEED(L.gate_up, "mlp.gate_up", W, 2 * (int64_t)lp.ff, lp.n_expert);
            ZV_NEED(L.down, "mlp.down", lp.ff, W, lp.n_expert);
            ZV_NEED(L.router, "mlp.router", W, lp.n_expert);
            LL_REQUIRE(L.router->type == GGML_TYPE_F32, B200_ERR_INVALID, "b200_llama_finalize: %smlp.router must be uploaded as f32 (the router runs in f32 in every mode)", pre.c_str());
        }
#undef ZV_NEED
    }
    g->host_vecs.clear();
    if (m->run_layer.empty()) for (int il = 0; il < hp.n_layer; il++) m->run_layer.push_back(il);
    g->runs.resize(m->run_layer.size());
    for (size_t r = 0; r < m->run_layer.size(); r++) {
        const b200_layer_params &lp = m->layer_hp[(size_t)m->run_layer[r]];
        ZvRun &R = g->runs[r];
        const std::string pre = "run" + std::to_string(r) + ".";
        R.k_cache = new_device_tensor(m, (pre + "k").c_str(), GGML_TYPE_F32, (int64_t)lp.kv_heads * lp.dim, hp.n_ctx, true);
        R.v_cache = new_device_tensor(m, (pre + "v").c_str(), GGML_TYPE_F32, (int64_t)lp.kv_heads * lp.vdim, hp.n_ctx, true);
        LL_REQUIRE(R.k_cache && R.v_cache, B200_ERR_NOMEM, "b200_llama_finalize: out of device memory for the cache of run %zu", r);
        m->kv_bytes += (int64_t)(nbytes(R.k_cache) + nbytes(R.v_cache));
    }
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ graph of one batch step
enum { R_HEAD = 0, R_EVEN = 1, R_ODD = 2, R_TAIL = 3 };

int zv_build(b200_llama *m, const BatchShape &bs) {
    const b200_llama_params &hp = m->hp;
    ZvData *g = zv(m);
    const int64_t T = bs.n_tokens, W = hp.n_embd;
    const float eps = hp.rms_eps;
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
    ggml_tensor *cell_seq = input_view(m->inp_cell_seq, bs.n_kv), *cell_pos = input_view(m->inp_cell_pos, bs.n_kv);

    // res + RMSnorm(y) * w: the norm behind a sublayer, its scales and the residual add in one launch
    auto post_norm = [&](ggml_tensor *y, ggml_tensor *w, ggml_tensor *res) {
        ggml_tensor *dst = b.alloc_result(GGML_TYPE_F32, y->ne[0], y->ne[1], y->ne[2], 1);
        b.ext(dst, B200_EXT_NORM, {y, w, nullptr, nullptr, res, nullptr});
        dst->op_params[2] = B200_NORM_RMS; Builder::set_f(dst, 3, eps); dst->op_params[4] = 1; dst->op_params[5] = 0;
        return dst;
    };
    auto glu = [&](ggml_tensor *dst, ggml_tensor *a, ggml_tensor *u, const b200_layer_params &lp) {
        b.ext(dst, B200_EXT_SILU_MUL, {a, u});
        dst->op_params[2] = lp.glu_kind; Builder::set_f(dst, 3, lp.glu_limit); Builder::set_f(dst, 4, lp.glu_alpha);
        return dst;
    };

    b.bump = &m->regions[R_HEAD];
    ggml_tensor *x = b.op(b.alloc_result(GGML_TYPE_F32, W, T), GGML_OP_GET_ROWS, g->embed, tokens);

    for (size_t r = 0; r < m->run_layer.size(); r++) {
        const int il = m->run_layer[r];
        const b200_layer_params &lp = m->layer_hp[(size_t)il];
        ZvLayer &L = g->layers[(size_t)il];
        ZvRun &R = g->runs[r];
        b.bump = &m->regions[(r & 1) ? R_ODD : R_EVEN];
        b.bump->off = 0;
        const int64_t H = lp.heads, G = lp.kv_heads, D = lp.dim, V = lp.vdim;
        ggml_tensor *P = b.mul_mat(L.proj1, x);
        Part parts[8];
        const int np = parts_proj1(lp, parts);
        auto part = [&](const char *leaf) {
            int64_t rows = 0;
            const int64_t off = part_offset(parts, np, leaf, nullptr, &rows);
            return b.view_2d(P, rows, T, P->nb[1], (size_t)off * 4);
        };
        ggml_tensor *kc_all = b.view_2d(R.k_cache, G * D, hp.n_ctx, R.k_cache->nb[1], 0), *vc_all = b.view_2d(R.v_cache, G * V, hp.n_ctx, R.v_cache->nb[1], 0);
        ggml_tensor *q = part("mix.q");
        ggml_tensor *qo = part("mix.q");  // the store rewrites q in place
        b.ext(qo, B200_EXT_QKV_STORE, {q, part("mix.k"), part("mix.v"), L.qknorm, pos, L.freqs, cells, kc_all, vc_all});
        qo->op_params[2] = (int32_t)D; qo->op_params[3] = (int32_t)V; qo->op_params[4] = lp.rope_dims; Builder::set_f(qo, 5, eps);
        qo->op_params[6] = 0; qo->op_params[7] = lp.qk_norm ? (lp.qk_norm_per_head ? 2 : 1) : 0; qo->op_params[8] = lp.rope_halves ? 1 : 0;
        ggml_tensor *o = b.alloc_result(GGML_TYPE_F32, H * V, T);
        b.ext(o, B200_EXT_SINK_ATTN, {qo, b.view_2d(R.k_cache, G * D, bs.n_kv, R.k_cache->nb[1], 0), b.view_2d(R.v_cache, G * V, bs.n_kv, R.v_cache->nb[1], 0), L.sink, tok_seq, pos,
                                       cell_seq, cell_pos, lp.head_gate ? part("mix.g") : nullptr});
        o->op_params[2] = (int32_t)D; Builder::set_f(o, 3, lp.scale); o->op_params[4] = lp.window; o->op_params[5] = lp.keep_first;
        // bf16 weights: the attention products of a prompt batch may be bf16 as well (B200_ATTN_F32=1 keeps them in f32)
        static const bool attn_f32 = getenv("B200_ATTN_F32") != nullptr;
        o->op_params[6] = L.proj1->type == GGML_TYPE_BF16 && !attn_f32;
        o->op_params[7] = (int32_t)V; o->op_params[8] = lp.chunk;
        x = post_norm(b.mul_mat(L.wo, o), L.post1, x);
        if (lp.mlp == B200_MLP_DENSE_GATED) {
            const int64_t F = lp.ff;
            ggml_tensor *gu = b.mul_mat(L.gate_up, x);
            ggml_tensor *act = glu(b.alloc_result(GGML_TYPE_F32, F, T), b.view_2d(gu, F, T, gu->nb[1], 0), b.view_2d(gu, F, T, gu->nb[1], (size_t)F * 4), lp);
            x = post_norm(b.mul_mat(L.down, act), L.post2, x);
        } else if (lp.mlp == B200_MLP_MOE_GATED) {
            const int64_t F = lp.ff, NU = lp.n_expert_used;
            // the router's result: per token NU weights, then NU expert ids (as i32) in the same row
            ggml_tensor *rt = b.alloc_result(GGML_TYPE_F32, 2 * NU, T);
            b.ext(rt, B200_EXT_MOE_ROUTE, {b.mul_mat(L.router, x), nullptr});
            rt->op_params[2] = 1; rt->op_params[3] = 1; Builder::set_f(rt, 4, lp.router_scale == 0.0f ? 1.0f : lp.router_scale); rt->op_params[5] = (int32_t)NU;
            rt->op_params[6] = lp.router_score; rt->op_params[7] = lp.router_keep_scores ? 1 : 0;
            ggml_tensor *wts = b.view_2d(rt, NU, T, rt->nb[1], 0), *ids = b.view_2d(rt, NU, T, rt->nb[1], (size_t)NU * 4);
            ids->type = GGML_TYPE_I32;
            ggml_tensor *gu = b.ext(b.alloc_result(GGML_TYPE_F32, 2 * F, NU, T), B200_EXT_MUL_MAT_ID, {L.gate_up, b.reshape(x, W, 1, T), ids});
            ggml_tensor *act = glu(b.alloc_result(GGML_TYPE_F32, F, NU, T), b.view_3d(gu, F, NU, T, gu->nb[1], gu->nb[2], 0), b.view_3d(gu, F, NU, T, gu->nb[1], gu->nb[2], (size_t)F * 4), lp);
            ggml_tensor *dn = b.ext(b.alloc_result(GGML_TYPE_F32, W, NU, T), B200_EXT_MUL_MAT_ID, {L.down, act, ids});
            if (W <= B200_MOE_COMBINE_NORM_MAX) {  // the weighted sum over the chosen experts, the norm behind it and the residual in one launch
                ggml_tensor *nx = b.ext(b.alloc_result(GGML_TYPE_F32, W, T), B200_EXT_MOE_COMBINE, {dn, wts, x, nullptr, L.post2});
                nx->op_params[2] = 1; Builder::set_f(nx, 3, eps);
                x = nx;
            } else {
                x = post_norm(b.ext(b.alloc_result(GGML_TYPE_F32, W, T), B200_EXT_MOE_COMBINE, {dn, wts, nullptr, nullptr}), L.post2, x);
            }
        }
    }
    b.bump = &m->regions[R_TAIL];
    ggml_tensor *out = x;
    if (bs.n_outputs > 0) {
        if (bs.n_outputs < T) out = b.get_rows(out, input_view(m->inp_out_ids, bs.n_outputs));
        out = b.mul_mat(g->head, post_norm(out, g->final_scale, nullptr));
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

const Arch k_zevopel = {"zevopel", zv_place_tensor, zv_finalize, nullptr, zv_build, nullptr};

}  // namespace

const Arch *b200::host::zevopel_arch() { return &k_zevopel; }

// host_galirax.cu -- the Galirax architecture for the decoder of host_llama.cu: where its tensors go and the graph of one batch
// step.  The decoder owns the model object, the sequence cache, the inputs and the step; this file adds no loop of its own.
//
// A Galirax model is a list of layers, run in an order that may repeat a stretch of them (every run has its own cache rows or
// recurrent state, b200_llama_set_layer_order).  A layer is parallel: h = LayerNorm(x) with weight and bias feeds both the mixer
// and the feed-forward, and x <- x + (mixer(h) + ff(h)).  Mixers (b200_layer_params):
//   * attention: heads query heads over kv_heads key / value heads, optional biases and an RMS norm over the whole q / k projection,
//     interleaved rotation by a frequency table (band-wise scaled or plain), a per-head sink in the softmax denominator, and an
//     optional sliding window that keeps the first positions visible;
//   * lightning: linear attention with silu on q, k, v, a fixed decay per head, an RMS norm over all heads and a sigmoid gate.
// The feed-forward is a mixture of gated experts with a sigmoid router, a choice bias and group-limited choice.  The output is
// LayerNorm, the head, and a tanh soft cap.
//
// Graph choices: q, k, v (and the gate) are ONE product over row-concatenated weights; the router is a small f32 product of its
// own (f32 weights, unrounded input, in every mode); bias, norm, rotation and the cache store are one launch; the experts of a
// layer are two stacked tensors (gate over up per expert, and down) used through expert-indexed products; the weighted sum over
// the chosen experts adds the mixer's result and the residual in the same launch.
#include "host_fused.h"

namespace {

struct GxLayer {
    ggml_tensor *norm1 = nullptr, *norm1b = nullptr, *proj1 = nullptr, *wo = nullptr;
    ggml_tensor *qkvec = nullptr, *sink = nullptr, *freqs = nullptr;     // attention
    ggml_tensor *lnorm = nullptr, *decay = nullptr;                       // lightning
    ggml_tensor *router = nullptr, *gate_up = nullptr, *down = nullptr, *correction = nullptr;  // experts
};
struct GxRun {
    ggml_tensor *k_cache = nullptr, *v_cache = nullptr;  // attention: [kv_heads * dim, n_ctx], [kv_heads * vdim, n_ctx] f32
    ggml_tensor *state = nullptr;                         // lightning: [heads * vdim * dim, n_seq_max] f32
};
struct GxData {
    std::vector<GxLayer> layers;
    std::vector<GxRun> runs;
    ggml_tensor *embed = nullptr, *final_norm = nullptr, *final_norm_b = nullptr, *head = nullptr;
};
GxData *gx(b200_llama *m) { return (GxData *)m->arch_data.get(); }

int parts_proj1(const b200_layer_params &lp, Part out[8]) {
    int n = 0;
    const int64_t H = lp.heads, D = lp.dim, V = lp.vdim;
    if (lp.mixer == B200_MIXER_ATTENTION) {
        out[n++] = {"mix.q", H * D};
        out[n++] = {"mix.k", (int64_t)lp.kv_heads * D};
        out[n++] = {"mix.v", (int64_t)lp.kv_heads * V};
    } else {
        out[n++] = {"mix.q", H * D};
        out[n++] = {"mix.k", H * D};
        out[n++] = {"mix.v", H * V};
        out[n++] = {"mix.g", H * V};
    }
    return n;
}
// the optional vectors of an attention layer, packed in one f32 tensor in this order
int parts_qkvec(const b200_layer_params &lp, Part out[8]) {
    int n = 0;
    if (lp.mixer != B200_MIXER_ATTENTION) return 0;
    const int64_t nq = (int64_t)lp.heads * lp.dim, nk = (int64_t)lp.kv_heads * lp.dim, nv = (int64_t)lp.kv_heads * lp.vdim;
    if (lp.qkv_bias) { out[n++] = {"mix.q.b", nq}; out[n++] = {"mix.k.b", nk}; out[n++] = {"mix.v.b", nv}; }
    if (lp.qk_norm) { out[n++] = {"mix.q.norm", nq}; out[n++] = {"mix.k.norm", nk}; }
    return n;
}
int gx_place_tensor(b200_llama *m, const char *name, int type, int64_t ne0, int64_t ne1, int64_t ne2, const void *data) {
    int il = -1;
    const char *leaf = nullptr;
    if (!split_name(name, &il, &leaf)) return upload_tensor(m, name, type, ne0, ne1, ne2, data);
    LL_REQUIRE(il >= 0 && il < m->hp.n_layer, B200_ERR_INVALID, "b200_llama_set_tensor: %s names a layer outside 0..%d", name, m->hp.n_layer - 1);
    const b200_layer_params &lp = m->layer_hp[(size_t)il];
    LL_REQUIRE(lp.mixer != 0, B200_ERR_INVALID, "b200_llama_set_tensor: %s before b200_llama_set_layer(%d)", name, il);
    const TypeTraits tt = type_traits(type);
    LL_REQUIRE(tt.blck == 1 && ne2 == 1, B200_ERR_UNSUPPORTED, "b200_llama_set_tensor: %s: dense 1-D / 2-D tensors only", name);
    const int64_t W = m->hp.n_embd;
    const std::string pre = "l" + std::to_string(il) + ".";
    const size_t es = (size_t)tt.size;
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
    Part parts[8];
    int64_t total = 0, rows = 0;
    int n = parts_proj1(lp, parts);
    int64_t off = part_offset(parts, n, leaf, &total, &rows);
    if (off >= 0) {
        LL_REQUIRE(ne0 == W && ne1 == rows, B200_ERR_INVALID, "b200_llama_set_tensor: %s is [%lld, %lld], expected [%lld, %lld]", name, (long long)ne1, (long long)ne0, (long long)rows, (long long)W);
        return place_into(m, pre + "proj1", name, type, W, total, 1, (size_t)(off * W) * es, (size_t)(rows * W) * es, data);
    }
    n = parts_qkvec(lp, parts);
    off = part_offset(parts, n, leaf, &total, &rows);
    if (off >= 0) {
        LL_REQUIRE(type == GGML_TYPE_F32 && ne0 == rows && ne1 == 1, B200_ERR_INVALID, "b200_llama_set_tensor: %s must be %lld f32 values", name, (long long)rows);
        return place_into(m, pre + "mix.qkvec", name, type, total, 1, 1, (size_t)off * 4, (size_t)rows * 4, data);
    }
    return upload_tensor(m, name, type, ne0, ne1, ne2, data);
}

int gx_finalize(b200_llama *m) {
    const b200_llama_params &hp = m->hp;
    m->arch_data = std::shared_ptr<void>(new GxData(), [](void *p) { delete (GxData *)p; });
    GxData *g = gx(m);
    g->layers.resize((size_t)hp.n_layer);
    g->embed = find_w(m, "embed"); g->final_norm = find_w(m, "final.norm"); g->final_norm_b = find_w(m, "final.norm.b"); g->head = find_w(m, "head");
    LL_REQUIRE(g->embed && g->final_norm && g->final_norm_b && g->head, B200_ERR_INVALID, "b200_llama_finalize: embed / final.norm / final.norm.b / head missing");
    LL_REQUIRE(g->embed->ne[0] == hp.n_embd && g->embed->ne[1] == hp.n_vocab && g->head->ne[0] == hp.n_embd && g->head->ne[1] == hp.n_vocab &&
               g->final_norm->ne[0] == hp.n_embd && g->final_norm_b->ne[0] == hp.n_embd, B200_ERR_INVALID,
               "b200_llama_finalize: embed / head / final.norm do not fit width %d and vocabulary %d", hp.n_embd, hp.n_vocab);
    const int64_t W = hp.n_embd;
    for (int il = 0; il < hp.n_layer; il++) {
        const b200_layer_params &lp = m->layer_hp[(size_t)il];
        GxLayer &L = g->layers[(size_t)il];
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
#define GX_NEED(dst, ...) do { dst = need(__VA_ARGS__); if (!(dst)) return B200_ERR_INVALID; } while (0)
        LL_REQUIRE(lp.mixer == B200_MIXER_ATTENTION || lp.mixer == B200_MIXER_LIGHTNING, B200_ERR_INVALID, "b200_llama_finalize: layer %d has no mixer of this architecture", il);
        LL_REQUIRE(lp.heads > 0 && lp.dim > 0 && lp.vdim > 0 && lp.dim <= 256, B200_ERR_INVALID, "b200_llama_finalize: layer %d: heads, dim (<= 256), vdim must be positive", il);
        const int64_t H = lp.heads, D = lp.dim, V = lp.vdim;
        GX_NEED(L.norm1, "norm1", W, 1); GX_NEED(L.norm1b, "norm1.b", W, 1);
        Part parts[8];
        int np = parts_proj1(lp, parts);
        int64_t total = 0;
        part_offset(parts, np, "", &total);
        for (int i = 0; i < np; i++) LL_REQUIRE(find_w(m, pre + parts[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), parts[i].leaf);
        GX_NEED(L.proj1, "proj1", W, total);
        GX_NEED(L.wo, "mix.o", H * V, W);
        if (lp.mixer == B200_MIXER_ATTENTION) {
            LL_REQUIRE(lp.kv_heads > 0 && H % lp.kv_heads == 0 && V <= 256, B200_ERR_INVALID, "b200_llama_finalize: layer %d: heads %d do not divide over %d kv heads (vdim <= 256)", il, lp.heads, lp.kv_heads);
            LL_REQUIRE(lp.rope_dims >= 0 && lp.rope_dims % 2 == 0 && lp.rope_dims <= D && (lp.rope_dims == 0 || lp.rope_base > 0.0f), B200_ERR_INVALID, "b200_llama_finalize: layer %d: rotation does not fit dim", il);
            LL_REQUIRE(lp.rope_scaling == B200_ROPE_SCALING_NONE || (lp.rope_scaling == B200_ROPE_SCALING_BANDS && lp.yarn_factor > 0.0f && lp.yarn_original > 0 && lp.band_low > 0.0f &&
                       lp.band_high > lp.band_low), B200_ERR_INVALID, "b200_llama_finalize: layer %d: frequency scaling parameters", il);
            LL_REQUIRE(lp.window >= 0 && lp.keep_first >= 0, B200_ERR_INVALID, "b200_llama_finalize: layer %d: window / kept first positions must not be negative", il);
            GX_NEED(L.sink, "mix.sink", H, 1);
            np = parts_qkvec(lp, parts);
            if (np > 0) {
                part_offset(parts, np, "", &total);
                for (int i = 0; i < np; i++) LL_REQUIRE(find_w(m, pre + parts[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), parts[i].leaf);
                GX_NEED(L.qkvec, "mix.qkvec", total, 1);
            }
            std::vector<float> f;
            rope_freqs(lp, f);
            if (f.empty()) f.push_back(0.0f);
            const std::string fname = pre + "rope_freqs";
            const int rc = upload_tensor(m, fname.c_str(), GGML_TYPE_F32, (int64_t)f.size(), 1, 1, f.data());
            if (rc != B200_OK) return rc;
            L.freqs = find_w(m, fname);
        } else {
            GX_NEED(L.lnorm, "mix.norm", H * V, 1); GX_NEED(L.decay, "mix.decay", H, 1);
        }
        if (lp.mlp != B200_MLP_NONE) {
            LL_REQUIRE(lp.mlp == B200_MLP_MOE_GATED && lp.ff > 0 && lp.n_expert > 0 && lp.n_expert <= 256 && lp.n_expert_used > 0 && lp.n_expert_used <= 32 && lp.n_expert_used <= lp.n_expert,
                       B200_ERR_UNSUPPORTED, "b200_llama_finalize: layer %d: feed-forward kind / expert counts (at most 256 experts, 32 per token)", il);
            const int ng = lp.n_group < 1 ? 1 : lp.n_group, nk = lp.n_group_used < 1 ? ng : lp.n_group_used;
            LL_REQUIRE(ng <= 32 && lp.n_expert % ng == 0 && nk <= ng && (int64_t)nk * (lp.n_expert / ng) >= lp.n_expert_used, B200_ERR_INVALID, "b200_llama_finalize: layer %d: expert groups do not fit", il);
            for (int e = 0; e < lp.n_expert; e++)
                for (const char *w : {"gate", "up", "down"}) {
                    const std::string nm = pre + "mlp.e" + std::to_string(e) + "." + w;
                    LL_REQUIRE(find_w(m, nm), B200_ERR_INVALID, "b200_llama_finalize: tensor %s missing", nm.c_str());
                }
            GX_NEED(L.gate_up, "mlp.gate_up", W, 2 * (int64_t)lp.ff, lp.n_expert); GX_NEED(L.down, "mlp.down", lp.ff, W, lp.n_expert);
            GX_NEED(L.router, "mlp.router", W, lp.n_expert);
            LL_REQUIRE(L.router->type == GGML_TYPE_F32, B200_ERR_INVALID, "b200_llama_finalize: %smlp.router must be uploaded as f32 (the router runs in f32 in every mode)", pre.c_str());
            L.correction = find_w(m, pre + "mlp.correction");
            LL_REQUIRE(!L.correction || L.correction->ne[0] == lp.n_expert, B200_ERR_INVALID, "b200_llama_finalize: %smlp.correction does not fit %d experts", pre.c_str(), lp.n_expert);
        }
#undef GX_NEED
    }
    // every run of a layer owns its cache rows or its state
    if (m->run_layer.empty()) for (int il = 0; il < hp.n_layer; il++) m->run_layer.push_back(il);
    g->runs.resize(m->run_layer.size());
    for (size_t r = 0; r < m->run_layer.size(); r++) {
        const b200_layer_params &lp = m->layer_hp[(size_t)m->run_layer[r]];
        GxRun &R = g->runs[r];
        const std::string pre = "run" + std::to_string(r) + ".";
        if (lp.mixer == B200_MIXER_ATTENTION) {
            R.k_cache = new_device_tensor(m, (pre + "k").c_str(), GGML_TYPE_F32, (int64_t)lp.kv_heads * lp.dim, hp.n_ctx, true);
            R.v_cache = new_device_tensor(m, (pre + "v").c_str(), GGML_TYPE_F32, (int64_t)lp.kv_heads * lp.vdim, hp.n_ctx, true);
            LL_REQUIRE(R.k_cache && R.v_cache, B200_ERR_NOMEM, "b200_llama_finalize: out of device memory for the cache of run %zu", r);
            m->kv_bytes += (int64_t)(nbytes(R.k_cache) + nbytes(R.v_cache));
        } else {
            R.state = new_device_tensor(m, (pre + "state").c_str(), GGML_TYPE_F32, (int64_t)lp.heads * lp.dim * lp.vdim, hp.n_seq_max, true);
            LL_REQUIRE(R.state, B200_ERR_NOMEM, "b200_llama_finalize: out of device memory for the state of run %zu", r);
            m->kv_bytes += (int64_t)nbytes(R.state);
        }
    }
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ graph of one batch step
enum { R_HEAD = 0, R_EVEN = 1, R_ODD = 2, R_TAIL = 3 };

int gx_build(b200_llama *m, const BatchShape &bs) {
    const b200_llama_params &hp = m->hp;
    GxData *g = gx(m);
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
    ggml_tensor *cell_seq = input_view(m->inp_cell_seq, bs.n_kv), *cell_pos = input_view(m->inp_cell_pos, bs.n_kv), *seq_info = input_view(m->inp_seq_info, bs.n_seq, 4);

    // LayerNorm / RMS norm with weight, optional bias, optional sigmoid gate on the result
    auto norm = [&](ggml_tensor *x, ggml_tensor *w, int kind, ggml_tensor *bias = nullptr, ggml_tensor *out_gate = nullptr) {
        ggml_tensor *dst = b.alloc_result(GGML_TYPE_F32, x->ne[0], x->ne[1], x->ne[2], 1);
        b.ext(dst, B200_EXT_NORM, {x, w, out_gate, nullptr, nullptr, bias});
        dst->op_params[2] = kind; Builder::set_f(dst, 3, eps); dst->op_params[4] = 1; dst->op_params[5] = out_gate ? 1 : 0;
        return dst;
    };

    b.bump = &m->regions[R_HEAD];
    ggml_tensor *x = b.op(b.alloc_result(GGML_TYPE_F32, W, T), GGML_OP_GET_ROWS, g->embed, tokens);

    for (size_t r = 0; r < m->run_layer.size(); r++) {
        const int il = m->run_layer[r];
        const b200_layer_params &lp = m->layer_hp[(size_t)il];
        GxLayer &L = g->layers[(size_t)il];
        GxRun &R = g->runs[r];
        b.bump = &m->regions[(r & 1) ? R_ODD : R_EVEN];
        b.bump->off = 0;
        const int64_t H = lp.heads, D = lp.dim, V = lp.vdim;
        ggml_tensor *h = norm(x, L.norm1, B200_NORM_LAYER, L.norm1b);
        ggml_tensor *P = b.mul_mat(L.proj1, h);
        Part parts[8];
        const int np = parts_proj1(lp, parts);
        auto part = [&](const char *leaf) {
            int64_t rows = 0;
            const int64_t off = part_offset(parts, np, leaf, nullptr, &rows);
            return b.view_2d(P, rows, T, P->nb[1], (size_t)off * 4);
        };
        ggml_tensor *y;  // the mixer's result, [W, T]
        if (lp.mixer == B200_MIXER_ATTENTION) {
            const int64_t G = lp.kv_heads;
            ggml_tensor *kc_all = b.view_2d(R.k_cache, G * D, hp.n_ctx, R.k_cache->nb[1], 0), *vc_all = b.view_2d(R.v_cache, G * V, hp.n_ctx, R.v_cache->nb[1], 0);
            ggml_tensor *q = part("mix.q");
            ggml_tensor *qo = part("mix.q");  // the store rewrites q in place
            b.ext(qo, B200_EXT_QKV_STORE, {q, part("mix.k"), part("mix.v"), L.qkvec, pos, L.freqs, cells, kc_all, vc_all});
            qo->op_params[2] = (int32_t)D; qo->op_params[3] = (int32_t)V; qo->op_params[4] = lp.rope_dims; Builder::set_f(qo, 5, eps);
            qo->op_params[6] = lp.qkv_bias ? 1 : 0; qo->op_params[7] = lp.qk_norm ? 1 : 0;
            ggml_tensor *o = b.alloc_result(GGML_TYPE_F32, H * V, T);
            b.ext(o, B200_EXT_SINK_ATTN, {qo, b.view_2d(R.k_cache, G * D, bs.n_kv, R.k_cache->nb[1], 0), b.view_2d(R.v_cache, G * V, bs.n_kv, R.v_cache->nb[1], 0), L.sink, tok_seq, pos,
                                           cell_seq, cell_pos});
            o->op_params[2] = (int32_t)D; Builder::set_f(o, 3, lp.scale); o->op_params[4] = lp.window; o->op_params[5] = lp.keep_first;
            // bf16 weights: the attention products of a prompt batch may be bf16 as well (B200_ATTN_F32=1 keeps them in f32)
            static const bool attn_f32 = getenv("B200_ATTN_F32") != nullptr;
            o->op_params[6] = L.proj1->type == GGML_TYPE_BF16 && !attn_f32;
            o->op_params[7] = (int32_t)V;
            y = b.mul_mat(L.wo, o);
        } else {
            ggml_tensor *o = b.alloc_result(GGML_TYPE_F32, H * V, T);
            b.ext(o, B200_EXT_LINEAR_ATTN_SCAN, {part("mix.q"), part("mix.k"), part("mix.v"), L.decay, seq_info, R.state});
            o->op_params[2] = (int32_t)H; o->op_params[3] = (int32_t)D; o->op_params[4] = (int32_t)V; o->op_params[5] = 1;
            y = b.mul_mat(L.wo, norm(o, L.lnorm, B200_NORM_RMS, nullptr, part("mix.g")));
        }
        if (lp.mlp == B200_MLP_MOE_GATED) {
            const int64_t F = lp.ff, NU = lp.n_expert_used;
            // the router's result: per token NU weights, then NU expert ids (as i32) in the same row
            ggml_tensor *rt = b.alloc_result(GGML_TYPE_F32, 2 * NU, T);
            b.ext(rt, B200_EXT_MOE_ROUTE, {b.mul_mat(L.router, h), L.correction});  // f32 weights times the unrounded h: the choice does not hang on a rounded input
            rt->op_params[2] = lp.n_group < 1 ? 1 : lp.n_group; rt->op_params[3] = lp.n_group_used < 1 ? rt->op_params[2] : lp.n_group_used;
            Builder::set_f(rt, 4, lp.router_scale); rt->op_params[5] = (int32_t)NU;
            ggml_tensor *wts = b.view_2d(rt, NU, T, rt->nb[1], 0), *ids = b.view_2d(rt, NU, T, rt->nb[1], (size_t)NU * 4);
            ids->type = GGML_TYPE_I32;
            ggml_tensor *gu = b.ext(b.alloc_result(GGML_TYPE_F32, 2 * F, NU, T), B200_EXT_MUL_MAT_ID, {L.gate_up, b.reshape(h, W, 1, T), ids});
            ggml_tensor *act = b.ext(b.alloc_result(GGML_TYPE_F32, F, NU, T), B200_EXT_SILU_MUL,
                                     {b.view_3d(gu, F, NU, T, gu->nb[1], gu->nb[2], 0), b.view_3d(gu, F, NU, T, gu->nb[1], gu->nb[2], (size_t)F * 4)});
            ggml_tensor *dn = b.ext(b.alloc_result(GGML_TYPE_F32, W, NU, T), B200_EXT_MUL_MAT_ID, {L.down, act, ids});
            x = b.ext(b.alloc_result(GGML_TYPE_F32, W, T), B200_EXT_MOE_COMBINE, {dn, wts, x, y});
        } else {
            x = b.binary(GGML_OP_ADD, x, y);
        }
    }
    b.bump = &m->regions[R_TAIL];
    ggml_tensor *out = x;
    if (bs.n_outputs > 0) {
        if (bs.n_outputs < T) out = b.get_rows(out, input_view(m->inp_out_ids, bs.n_outputs));
        out = b.mul_mat(g->head, norm(out, g->final_norm, B200_NORM_LAYER, g->final_norm_b));
        if (hp.logit_softcap > 0.0f) {
            ggml_tensor *c = b.ext(b.alloc_result(GGML_TYPE_F32, out->ne[0], out->ne[1]), B200_EXT_UNARY, {out});
            c->op_params[2] = B200_UN_SOFTCAP; Builder::set_f(c, 3, hp.logit_softcap);
            out = c;
        }
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

const Arch k_galirax = {"galirax", gx_place_tensor, gx_finalize, nullptr, gx_build, nullptr};

}  // namespace

const Arch *b200::host::galirax_arch() { return &k_galirax; }

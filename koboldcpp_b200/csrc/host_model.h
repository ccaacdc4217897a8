// host_model.h -- what the decoders above the ggml_backend boundary share: the node constructors that fill struct ggml_tensor the
// way the ggml_* builders do, the bump allocator of the compute buffer, the model / context object behind b200_llama.h, the
// sequence cache (cells and state slots) and the table of architectures.  No compute happens in the host_*.cu files.
#pragma once
#include <chrono>
#include <cmath>
#include <deque>
#include <map>
#include <memory>
#include <unordered_set>

#include "../../include/b200_comm.h"
#include "../../include/b200_llama.h"
#include "../../include/b200_ggml_ops.h"
#include "backend_internal.h"
#include "host_cache.h"

namespace b200 {
void set_error(const char *fmt, ...);
}

namespace b200 {
namespace host {


constexpr int KV_PAD = 256;  // llama_kv_cache_get_padding with flash attention, src/llama.cpp:4143-4146

// ------------------------------------------------------------------------------------------------ tensor arena
struct Arena {
    std::deque<ggml_tensor> pool;  // stable addresses
    size_t used = 0;
    void reset() { used = 0; }
    ggml_tensor *get() {
        if (used == pool.size()) pool.emplace_back();
        ggml_tensor *t = &pool[used++];
        memset(t, 0, sizeof(*t));
        return t;
    }
};

inline void set_shape(ggml_tensor *t, int type, int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3) {
    const TypeTraits tt = type_traits(type);
    t->type = (ggml_type)type;
    t->ne[0] = ne0; t->ne[1] = ne1; t->ne[2] = ne2; t->ne[3] = ne3;
    t->nb[0] = (size_t)tt.size;
    t->nb[1] = t->nb[0] * (size_t)(ne0 / tt.blck);
    t->nb[2] = t->nb[1] * (size_t)ne1;
    t->nb[3] = t->nb[2] * (size_t)ne2;
}

// bump allocator over one backend buffer (stands in for ggml-alloc: every graph gets the same addresses again)
struct Bump {
    ggml_backend_buffer_t buf = nullptr;
    char *base = nullptr;
    size_t size = 0, off = 0, align = 128, peak = 0;  // peak: the furthest any take() reached since it was cleared
    void *take(size_t bytes) {
        off = (off + align - 1) / align * align;
        if (off + bytes > size) return nullptr;
        void *p = base + off;
        off += bytes;
        if (off > peak) peak = off;
        return p;
    }
};

struct Builder {
    Arena *arena;
    Bump *bump;
    std::vector<ggml_tensor *> nodes;
    std::unordered_set<const ggml_tensor *> visited;
    bool oom = false;

    // ggml_build_forward_expand: post-order DFS over src[], left to right (ggml_visit_parents, ggml.c:19020-19070);
    // tensors with op NONE are leafs and not part of the node list
    void expand(ggml_tensor *t) {
        if (!t || !visited.insert(t).second) return;
        for (int i = 0; i < GGML_MAX_SRC; i++) expand(t->src[i]);
        if (t->op != GGML_OP_NONE) nodes.push_back(t);
    }

    ggml_tensor *alloc_result(int type, int64_t ne0, int64_t ne1 = 1, int64_t ne2 = 1, int64_t ne3 = 1) {
        ggml_tensor *t = arena->get();
        set_shape(t, type, ne0, ne1, ne2, ne3);
        t->data = bump->take(nbytes(t));
        if (!t->data) oom = true;
        t->buffer = bump->buf;
        return t;
    }
    ggml_tensor *op(ggml_tensor *t, int o, ggml_tensor *a, ggml_tensor *b = nullptr, ggml_tensor *c = nullptr, ggml_tensor *d = nullptr) {
        t->op = (ggml_op)o;
        t->src[0] = a; t->src[1] = b; t->src[2] = c; t->src[3] = d;
        return t;
    }
    // views share the data of their source (ggml_view_impl)
    ggml_tensor *view_of(ggml_tensor *a, int o, size_t offs) {
        ggml_tensor *t = arena->get();
        t->type = a->type;
        t->buffer = a->buffer;
        t->view_src = a->view_src ? a->view_src : a;
        t->view_offs = (a->view_src ? a->view_offs : 0) + offs;
        t->data = a->data ? (char *)a->data + offs : nullptr;
        t->op = (ggml_op)o;
        t->src[0] = a;
        return t;
    }
    ggml_tensor *reshape(ggml_tensor *a, int64_t ne0, int64_t ne1 = 1, int64_t ne2 = 1, int64_t ne3 = 1) {
        ggml_tensor *t = view_of(a, GGML_OP_RESHAPE, 0);
        set_shape(t, a->type, ne0, ne1, ne2, ne3);
        return t;
    }
    ggml_tensor *view_1d(ggml_tensor *a, int64_t ne0, size_t offs) {
        ggml_tensor *t = view_of(a, GGML_OP_VIEW, offs);
        set_shape(t, a->type, ne0, 1, 1, 1);
        memcpy(t->op_params, &offs, sizeof(offs));
        return t;
    }
    ggml_tensor *view_2d(ggml_tensor *a, int64_t ne0, int64_t ne1, size_t nb1, size_t offs) {
        ggml_tensor *t = view_of(a, GGML_OP_VIEW, offs);
        set_shape(t, a->type, ne0, ne1, 1, 1);
        t->nb[1] = nb1; t->nb[2] = nb1 * (size_t)ne1; t->nb[3] = t->nb[2];
        memcpy(t->op_params, &offs, sizeof(offs));
        return t;
    }
    ggml_tensor *view_3d(ggml_tensor *a, int64_t ne0, int64_t ne1, int64_t ne2, size_t nb1, size_t nb2, size_t offs) {
        ggml_tensor *t = view_of(a, GGML_OP_VIEW, offs);
        set_shape(t, a->type, ne0, ne1, ne2, 1);
        t->nb[1] = nb1; t->nb[2] = nb2; t->nb[3] = nb2 * (size_t)ne2;
        memcpy(t->op_params, &offs, sizeof(offs));
        return t;
    }
    ggml_tensor *permute(ggml_tensor *a, int ax0, int ax1, int ax2, int ax3) {
        ggml_tensor *t = view_of(a, GGML_OP_PERMUTE, 0);
        const int ax[4] = {ax0, ax1, ax2, ax3};
        for (int i = 0; i < 4; i++) { t->ne[ax[i]] = a->ne[i]; t->nb[ax[i]] = a->nb[i]; }
        for (int i = 0; i < 4; i++) t->op_params[i] = ax[i];
        return t;
    }
    ggml_tensor *rms_norm(ggml_tensor *a, float eps) {
        ggml_tensor *t = alloc_result(GGML_TYPE_F32, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        memcpy(t->op_params, &eps, 4);
        return op(t, GGML_OP_RMS_NORM, a);
    }
    ggml_tensor *binary(int o, ggml_tensor *a, ggml_tensor *b) {
        return op(alloc_result(GGML_TYPE_F32, a->ne[0], a->ne[1], a->ne[2], a->ne[3]), o, a, b);
    }
    ggml_tensor *mul_mat(ggml_tensor *w, ggml_tensor *x) {
        return op(alloc_result(GGML_TYPE_F32, w->ne[1], x->ne[1], x->ne[2], x->ne[3]), GGML_OP_MUL_MAT, w, x);
    }
    // as [K, M, n_expert], b [K, n_b_rows, T], ids [n_used, T] -> [M, n_used, T]   (ggml.c:5693-5729)
    ggml_tensor *mul_mat_id(ggml_tensor *as, ggml_tensor *b, ggml_tensor *ids) {
        return op(alloc_result(GGML_TYPE_F32, as->ne[1], ids->ne[0], b->ne[2], 1), GGML_OP_MUL_MAT_ID, as, b, ids);
    }
    ggml_tensor *rope(ggml_tensor *a, ggml_tensor *pos, ggml_tensor *ff, int n_dims, int mode, int n_ctx_orig, float freq_base, float freq_scale) {
        ggml_tensor *t = alloc_result(GGML_TYPE_F32, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        const float ext_factor = 0.0f, attn_factor = 1.0f, beta_fast = 32.0f, beta_slow = 1.0f;  // llama_context_default_params
        int32_t p[11] = {0, n_dims, mode, 0, n_ctx_orig};
        memcpy(p + 5, &freq_base, 4); memcpy(p + 6, &freq_scale, 4); memcpy(p + 7, &ext_factor, 4);
        memcpy(p + 8, &attn_factor, 4); memcpy(p + 9, &beta_fast, 4); memcpy(p + 10, &beta_slow, 4);
        memcpy(t->op_params, p, sizeof(p));
        return op(t, GGML_OP_ROPE, a, pos, ff);
    }
    // CPY(a, b): the result is a view of b (ggml_cpy_impl, ggml.c:5982-6005)
    ggml_tensor *cpy(ggml_tensor *a, ggml_tensor *b) {
        ggml_tensor *t = arena->get();
        *t = *b;
        t->view_src = b->view_src ? b->view_src : b;
        t->view_offs = b->view_src ? b->view_offs : 0;
        memset(t->op_params, 0, sizeof(t->op_params));
        memset(t->src, 0, sizeof(t->src));
        return op(t, GGML_OP_CPY, a, b);
    }
    ggml_tensor *cast(ggml_tensor *a, int type) {  // ggml_cast: CPY into a fresh tensor of `type`
        ggml_tensor *t = alloc_result(type, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        return op(t, GGML_OP_CPY, a, t);
    }
    ggml_tensor *get_rows(ggml_tensor *a, ggml_tensor *ids) {
        return op(alloc_result(GGML_TYPE_F32, a->ne[0], ids->ne[0], ids->ne[1], 1), GGML_OP_GET_ROWS, a, ids);
    }
    ggml_tensor *flash_attn(ggml_tensor *q, ggml_tensor *k, ggml_tensor *v, ggml_tensor *mask, float scale) {
        // result [D, n_head, N] (ggml.c:7165: ne = { v->ne[0], q->ne[2], q->ne[1], q->ne[3] })
        ggml_tensor *t = alloc_result(GGML_TYPE_F32, v->ne[0], q->ne[2], q->ne[1], q->ne[3]);
        const float p[3] = {scale, 0.0f, 0.0f};
        memcpy(t->op_params, p, sizeof(p));
        return op(t, GGML_OP_FLASH_ATTN_EXT, q, k, v, mask);
    }
    ggml_tensor *silu(ggml_tensor *a) {
        ggml_tensor *t = alloc_result(GGML_TYPE_F32, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        t->op_params[0] = GGML_UNARY_OP_SILU;
        return op(t, GGML_OP_UNARY, a);
    }
    ggml_tensor *soft_max(ggml_tensor *a) {
        ggml_tensor *t = alloc_result(GGML_TYPE_F32, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        const float p[2] = {1.0f, 0.0f};
        memcpy(t->op_params, p, sizeof(p));
        return op(t, GGML_OP_SOFT_MAX, a);
    }
    ggml_tensor *top_k(ggml_tensor *a, int k) {  // ggml_top_k = argsort(desc) + view (ggml.c:7080-7095)
        ggml_tensor *s = alloc_result(GGML_TYPE_I32, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        s->op_params[0] = GGML_SORT_ORDER_DESC;
        op(s, GGML_OP_ARGSORT, a);
        ggml_tensor *t = view_of(s, GGML_OP_VIEW, 0);
        set_shape(t, GGML_TYPE_I32, k, s->ne[1], s->ne[2], s->ne[3]);
        t->nb[1] = s->nb[1]; t->nb[2] = s->nb[2]; t->nb[3] = s->nb[3];
        return t;
    }
    // an exchange between the ranks of a tensor-parallel model (b200_comm.h): all-reduce in place, or all-gather along ne0
    ggml_tensor *collective(ggml_tensor *a, int kind, int world) {
        ggml_tensor *t;
        if (kind == B200_COLLECTIVE_ALL_REDUCE_SUM) {
            t = view_of(a, GGML_OP_MAP_CUSTOM1, 0);
            set_shape(t, a->type, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        } else {
            t = alloc_result(GGML_TYPE_F32, a->ne[0] * world, a->ne[1], a->ne[2], a->ne[3]);
            op(t, GGML_OP_MAP_CUSTOM1, a);
        }
        t->op_params[0] = (int32_t)B200_COLLECTIVE_TAG;
        t->op_params[1] = kind;
        return t;
    }
    // an extension op (include/b200_ggml_ops.h, enum b200_ext_op): `t` is the result tensor, which may alias an operand (in place)
    ggml_tensor *ext(ggml_tensor *t, int kind, std::initializer_list<ggml_tensor *> srcs) {
        t->op = GGML_OP_MAP_CUSTOM1;
        memset(t->src, 0, sizeof(t->src));
        int i = 0;
        for (ggml_tensor *s : srcs) t->src[i++] = s;
        t->op_params[0] = (int32_t)B200_EXT_TAG;
        t->op_params[1] = kind;
        return t;
    }
    static void set_f(ggml_tensor *t, int i, float v) { memcpy(t->op_params + i, &v, 4); }
    // a result tensor that lives inside another tensor's memory (a slice the node writes directly): not a ggml view
    ggml_tensor *result_at(ggml_tensor *parent, size_t offs, int type, int64_t ne0, int64_t ne1 = 1, int64_t ne2 = 1) {
        ggml_tensor *t = arena->get();
        set_shape(t, type, ne0, ne1, ne2, 1);
        t->data = (char *)parent->data + offs;
        t->buffer = parent->buffer;
        return t;
    }
    ggml_tensor *sum_rows(ggml_tensor *a) { return op(alloc_result(GGML_TYPE_F32, 1, a->ne[1], a->ne[2], a->ne[3]), GGML_OP_SUM_ROWS, a); }
};


}  // namespace host
}  // namespace b200

struct b200_llama;
namespace b200 {
namespace host {

// What an architecture adds to the shared decoder: where an uploaded tensor goes, what finalize resolves and allocates, and the
// graph of one step over a batch of sequences.
struct BatchShape { int32_t n_tokens, n_kv, n_outputs, n_seq; };
struct Arch {
    const char *name;
    // an uploaded tensor may land inside a larger fused tensor (rows appended) and / or be re-laid out on the host first
    int (*place_tensor)(b200_llama *m, const char *name, int type, int64_t ne0, int64_t ne1, int64_t ne2, const void *data);
    int (*finalize)(b200_llama *m);
    size_t (*compute_bytes)(b200_llama *m, int32_t max_batch);
    int (*build)(b200_llama *m, const BatchShape &bs);
    void (*release)(b200_llama *m);
};
const Arch *find_arch(int32_t id);
const Arch *genesun_arch();
const Arch *galirax_arch();
const Arch *zevopel_arch();
const Arch *medodra_arch();

}  // namespace host
}  // namespace b200
using namespace b200;
using namespace b200::host;

struct LayerW {
    ggml_tensor *attn_norm = nullptr, *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *ffn_norm = nullptr;
    ggml_tensor *ffn_gate = nullptr, *ffn_up = nullptr, *ffn_down = nullptr;
    ggml_tensor *ffn_gate_inp = nullptr, *ffn_gate_exps = nullptr, *ffn_up_exps = nullptr, *ffn_down_exps = nullptr;
};

struct b200_llama {
    b200_llama_params hp;
    ggml_backend_t be = nullptr;
    ggml_backend_buffer_type_t buft = nullptr, split_buft = nullptr;
    std::map<std::string, ggml_tensor *> weights;
    std::deque<ggml_tensor> weight_pool;
    std::vector<ggml_backend_buffer_t> buffers;  // everything to free
    int64_t weight_bytes = 0, kv_bytes = 0;
    // resolved weights
    ggml_tensor *tok_embd = nullptr, *output_norm = nullptr, *output = nullptr, *rope_freqs = nullptr;
    std::vector<LayerW> layers;
    // KV cache (one tensor per layer, [n_embd_gqa * n_ctx], src/llama.cpp:3583-3584)
    std::vector<ggml_tensor *> k_l, v_l;
    // compute
    int32_t max_batch = 0;
    Bump bump;
    size_t region_inputs = 0, region_half = 0;  // layout of the compute buffer: [inputs | half A | half B | tail]
    ggml_tensor inp_tokens, inp_pos, inp_mask, inp_out_ids;
    // pinned staging of the per-call inputs: [tokens | positions | out ids | mask], reused every call behind `in_ev`
    unsigned char *pin = nullptr;
    size_t pin_bytes = 0;
    cudaEvent_t in_ev = nullptr;   // recorded behind the input copies of the last call
    bool in_ev_pending = false;
    // what the device-side KQ mask currently holds (single-token decode only moves one element per call)
    // the graph of the previous call, reusable when only the KV write position moved (single-token decode): per layer the two
    // destination views of the cache stores and the CPY nodes that alias them
    struct KvStore { ggml_tensor *view, *cpy; char *base; size_t row; };
    std::vector<KvStore> kv_stores;
    int32_t g_n_tokens = 0, g_n_outputs = 0;
    int64_t g_n_kv = -1;
    double t_build = 0, t_inputs = 0, t_compute = 0, t_sync = 0;  // host seconds per phase (B200_LLAMA_TIMING=1 prints them at free)
    int64_t t_calls = 0;
    int64_t mk_n_kv = -1, mk_rows = -1;
    int32_t mk_n_tokens = 0, mk_n_past = -1;
    Arena arena;
    ggml_cgraph graph;
    std::vector<ggml_tensor *> graph_nodes;
    ggml_tensor *logits_t = nullptr;
    int64_t last_launches = 0;
    bool finalized = false;
    // architectures with their own graph (hp.arch != 0): per-layer shapes, resolved weights and caches (arch_data), the
    // sequence cache, the inputs of a batch step and the regions of the compute buffer the architecture's builder fills
    const b200::host::Arch *arch = nullptr;
    std::vector<b200_layer_params> layer_hp;
    std::vector<int32_t> run_layer;          // the layer of every run, in execution order (empty: every layer once)
    std::shared_ptr<void> arch_data;
    b200::host::SeqCache cache;
    ggml_tensor inp_cells, inp_tok_seq, inp_cell_seq, inp_cell_pos, inp_seq_info;
    b200::host::BatchShape g_shape = {0, 0, 0, 0};
    static constexpr int N_REGIONS = 4;      // stacked layer results | layers with even index | odd index | output head
    b200::host::Bump regions[N_REGIONS];
    bool measuring = false;                  // the builder runs over fake addresses to size the regions
    std::vector<int32_t> st_cells, st_pos, st_seq, st_out, st_info;  // host staging of a batch step
};

namespace b200 {
namespace host {


#define LL_REQUIRE(cond, code, ...)      \
    do {                                 \
        if (!(cond)) {                   \
            b200::set_error(__VA_ARGS__); \
            return code;                 \
        }                                \
    } while (0)

inline bool is_matrix_weight(const std::string &name) {
    // what llama.cpp places in the split buffer type: the 2-D weight matrices of the layers and the output head
    // (llm_load_tensors uses buft_matrix for them, src/llama.cpp:7039-7062); norms, router and token_embd are not split
    if (name == "output.weight") return true;
    if (name.compare(0, 4, "blk.") != 0) return false;
    static const char *const k[] = {"attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight", "ffn_gate.weight", "ffn_up.weight", "ffn_down.weight"};
    for (const char *s : k) {
        const size_t n = strlen(s);
        if (name.size() > n && name.compare(name.size() - n, n, s) == 0) return true;
    }
    return false;
}

inline ggml_tensor *alloc_in_buft(b200_llama *m, ggml_backend_buffer_type_t buft, ggml_tensor *t, int usage) {
    const size_t sz = buft->iface.get_alloc_size ? buft->iface.get_alloc_size(buft, t) : nbytes(t);
    ggml_backend_buffer_t buf = buft->iface.alloc_buffer(buft, sz);
    if (!buf) return nullptr;
    buf->usage = (ggml_backend_buffer_usage)usage;
    m->buffers.push_back(buf);
    t->buffer = buf;
    t->data = buf->iface.get_base(buf);
    if (buf->iface.init_tensor) buf->iface.init_tensor(buf, t);
    return t;
}

inline ggml_tensor *find_w(b200_llama *m, const std::string &name) {
    auto it = m->weights.find(name);
    return it == m->weights.end() ? nullptr : it->second;
}

// a weight tensor with its own device buffer (what b200_llama_set_tensor does for a plain tensor)
int upload_tensor(b200_llama *m, const char *name, int type, int64_t ne0, int64_t ne1, int64_t ne2, const void *data);
// a zero-initialised device tensor owned by the model (caches, recurrent state)
ggml_tensor *new_device_tensor(b200_llama *m, const char *name, int type, int64_t ne0, int64_t ne1, bool clear);

}  // namespace host
}  // namespace b200

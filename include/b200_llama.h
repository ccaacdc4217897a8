/* b200_llama.h -- C ABI of the host-side decoder that sits ABOVE the ggml_backend boundary (libkcpp_b200.so).
 *
 * This is the caller side of the hot path ("the callers either side of the path"): it does what
 * llama.cpp does for a llama / mixtral model -- builds the per-batch ggml graph node for node like build_llama
 * (/root/reference/src/llama.cpp:10453-10617, llm_build_kv :9648-9680, llm_build_kv_store :9161-9203, llm_build_kqv
 * :9517-9646, llm_build_ffn :9289-9414, llm_build_moe_ffn :9416-9515), places weights / KV cache / activations in
 * buffers obtained through the backend's buffer-type vtable, feeds the graph inputs with set_tensor, and calls the
 * backend's graph_compute -- the same five vtables llama.cpp would call (b200_ggml_backend.h).  It exists so that
 * bench.py and the tests can run whole-token decode through the reference-facing plugin interface on a machine that
 * has no reference checkout; under koboldcpp the caller is llama.cpp itself.
 *
 * All functions return 0 or a b200_status; b200_last_error() describes the failure.  Not thread safe per model.
 */
#ifndef B200_LLAMA_H
#define B200_LLAMA_H

#include "b200_ggml.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int32_t n_embd, n_layer, n_head, n_head_kv, n_embd_head, n_ff, n_vocab;
    int32_t n_expert, n_expert_used; /* 0 / 0 for dense models */
    int32_t n_ctx;                   /* KV cells */
    int32_t type_k, type_v;          /* B200_TYPE_F16 or B200_TYPE_Q8_0 (llama_context_params.type_k/type_v) */
    int32_t rope_neox;               /* 0: LLAMA_ROPE_TYPE_NORM (llama, mixtral) */
    int32_t n_ctx_orig;
    float   rms_eps, rope_freq_base, rope_freq_scale;
    int32_t main_device;             /* device that runs the graph */
    int32_t n_split_devices;         /* 0/1: everything on main_device; >1: weight matrices in the row-split buffer type */
    float   tensor_split[16];        /* all zero: equal split */
    /* tensor-parallel mode, one process per GPU (b200_comm.h; a communicator of tp_world ranks must exist): the caller uploads
     * this rank's SHARD of every matrix -- attn_q/k/v, ffn_gate/up and output split by output rows (heads r*n_head/W ..,
     * ffn columns, vocabulary rows), attn_output and ffn_down split along K (their ne0 is n_embd/W resp. n_ff/W) -- while
     * token_embd and the norm vectors are replicated.  The graph then holds n_head/W heads and n_head_kv/W KV heads per rank,
     * one all-reduce after attn_output and one after ffn_down, and an all-gather of the logits.  0 / 1 = off. */
    int32_t tp_rank, tp_world;
    /* Architecture of the graph: 0 = llama / mixtral (everything above), else one of enum b200_arch.  Architectures whose layers
     * differ from one another describe them with b200_llama_set_layer before the weights are uploaded; of the fields above they
     * read n_embd, n_layer, n_vocab, n_ctx (cache cells, a multiple of 256), rms_eps (the eps of every norm) and main_device. */
    int32_t arch;
    int32_t n_seq_max;               /* sequences (and recurrent-state slots) that can be open at a time; 0 = 1 */
    float   logit_softcap;           /* > 0: logits = cap * tanh(logits / cap) (architectures with their own graph) */
    float   embed_scale;             /* the embedding row is multiplied by this (0 reads as 1) */
    float   residual_mult;           /* architectures that scale a sublayer's result before it joins the residual stream (0 reads as 1) */
} b200_llama_params;

enum b200_arch { B200_ARCH_LLAMA = 0, B200_ARCH_GENESUN = 1, B200_ARCH_GALIRAX = 2, B200_ARCH_ZEVOPEL = 3, B200_ARCH_MEDODRA = 4 };
enum b200_mixer {
    B200_MIXER_LATENT_ATTENTION = 1, B200_MIXER_MLSTM = 2,
    B200_MIXER_ATTENTION = 3, /* softmax attention of heads over kv_heads cached keys / values, per-head sink, optional window */
    B200_MIXER_LIGHTNING = 4, /* linear attention: a decayed outer-product state per head */
    B200_MIXER_DELTA = 5,     /* gated delta rule: the state forgets by a per-token decay and is corrected towards v along k */
    B200_MIXER_SIGMOID_ATTENTION_GRU = 6, /* two mixers side by side: attention with sigmoid weights and a distance bias, and a minGRU */
};
enum b200_mlp {
    B200_MLP_NONE = 0, B200_MLP_DENSE_POLYNORM = 1, B200_MLP_MOE_GATED = 2 /* routed gated experts */,
    B200_MLP_DENSE_GATED = 3, /* down(act(gate x) * up x), act by glu_kind */
};
enum b200_rope_scaling { B200_ROPE_SCALING_NONE = 0, B200_ROPE_SCALING_YARN = 1, B200_ROPE_SCALING_BANDS = 2 /* per wavelength band */ };

/* One layer of an architecture with per-layer shapes (Genesun: config.json "layers"). */
typedef struct {
    int32_t mixer;                   /* enum b200_mixer */
    int32_t heads, dim, vdim;        /* per head: (unrotated) query / key size and value size */
    int32_t rot_dim, kv_rank, q_rank;/* latent attention: rotated size per head, latent sizes of keys / values and of queries */
    int32_t kv_from;                 /* latent attention: layer whose cache this layer reads (-1: its own) */
    int32_t window;                  /* attention window in tokens (0: every earlier token) */
    float   scale;                   /* attention score scale */
    int32_t rope_dims;               /* rotated dimensions (<= rot_dim) */
    float   rope_base;
    float   yarn_factor;             /* 0 or 1: no frequency scaling */
    float   yarn_fast, yarn_slow;
    int32_t yarn_original;
    float   gate_cap;                /* mLSTM: soft cap of the gate pre-activations */
    int32_t mlp, ff;                 /* enum b200_mlp and its hidden size (per expert for B200_MLP_MOE_GATED) */
    /* B200_MIXER_ATTENTION */
    int32_t kv_heads;                /* key / value heads; query head h reads kv head h / (heads / kv_heads) */
    int32_t keep_first;              /* with a window: positions below this stay visible whatever the distance */
    int32_t qkv_bias;                /* 1: q, k, v have biases ("<leaf>.b") */
    int32_t qk_norm;                 /* 1: RMS norm over the whole q (and k) projection with weights "q.norm" / "k.norm", before rotation */
    int32_t rope_scaling;            /* enum b200_rope_scaling; BANDS: wavelengths below original / band_high keep their frequency,
                                        above original / band_low are divided by yarn_factor, between the two blended linearly in
                                        original / wavelength (yarn_factor, yarn_original give factor and original) */
    float   band_low, band_high;
    /* B200_MLP_MOE_GATED: n_expert experts silu(gate x) * (up x) -> down, n_expert_used per token.  Router: s = sigmoid(W x);
     * choice by s + correction, limited to the n_group_used best of n_group equal groups of neighbouring experts (a group scores
     * the sum of its two largest choice scores); weights s / sum(s over the chosen) * router_scale. */
    int32_t n_expert, n_expert_used, n_group, n_group_used;
    float   router_scale;
    /* B200_MIXER_ATTENTION, further switches */
    int32_t chunk;                   /* > 0: positions are cut into chunks of this many, counted from 0; a token sees its own chunk only */
    int32_t qk_norm_per_head;        /* 1 (with qk_norm): the RMS norm runs over every head by itself, weights "q.norm" / "k.norm" of dim values */
    int32_t rope_halves;             /* 1: entry i turns with entry i + rope_dims / 2 instead of the neighbours (2i, 2i + 1) */
    int32_t head_gate;               /* 1: every head's result is multiplied by sigmoid(W_g x)_h, weights "g" [heads, width] */
    /* feed-forward, further switches */
    int32_t glu_kind;                /* enum b200_glu_kind (b200_ggml_ops.h) of the dense feed-forward or of the experts */
    float   glu_limit, glu_alpha;    /* B200_GLU_SWISH_CLAMPED */
    int32_t router_score;            /* enum b200_router_score */
    int32_t router_keep_scores;      /* 1: an expert's weight is its score, not divided by the sum over the chosen */
    /* mixers with a short causal convolution over time on q, k, v (tensors "<leaf>.conv" [channels, taps]); the last taps - 1 inputs of a
     * sequence are part of its state */
    int32_t conv_taps;               /* 0 / 1: none */
    /* B200_MIXER_SIGMOID_ATTENTION_GRU */
    float   q_temp_coef;             /* queries are multiplied by 1 + coef * ln(floor((pos + 1) / q_temp_every) + 1) */
    int32_t q_temp_every;
    int32_t dist_bias_max;           /* the rows of the distance table "rel" [rows, heads]: distances below rows / 2 have a row each, the
                                        others share the rest evenly in log distance up to this distance */
    int32_t side_width;              /* size of the minGRU state */
    /* feed-forward, further switches */
    int32_t router_scale_input;      /* 1: a chosen expert's weight multiplies its input, not its result */
    int32_t shared_ff;               /* > 0: a shared expert of this hidden size runs for every token ("mlp.shared.*"), times sigmoid(W_sg x) */
    int32_t loop_input;              /* 1: every time this layer is about to run, the stream x is first replaced by W_in [x ; x0] ("loop.in" [width, 2 width]),
                                        x0 being the stream as the embedding left it: the first layer of a looped stretch */
} b200_layer_params;


typedef struct b200_llama b200_llama; /* opaque */

B200_API int  b200_llama_new(const b200_llama_params *p, b200_llama **out);
B200_API void b200_llama_free(b200_llama *m);

/* Upload one weight tensor under its GGUF name ("token_embd.weight", "blk.3.attn_q.weight", "blk.3.ffn_gate_exps.weight",
 * "output_norm.weight", "output.weight", ...; names as written by convert_hf_to_gguf.py / gguf-py/gguf/constants.py).
 * data: ggml_nbytes of the tensor in host memory, GGUF layout (ne0 contiguous).  Goes through buft->alloc_buffer,
 * buffer->init_tensor and buffer->set_tensor exactly like llama_model_loader::load_all_data (src/llama.cpp:5024-5219). */
B200_API int b200_llama_set_tensor(b200_llama *m, const char *name, int type, int64_t ne0, int64_t ne1, int64_t ne2, const void *data);
/* Same tensor contents as an already uploaded tensor but its own device memory (synthetic models: one generated layer
 * replicated device-to-device instead of 80 host uploads). */
B200_API int b200_llama_clone_tensor(b200_llama *m, const char *name, const char *from);

/* Allocate KV cache + compute buffers once all weights are set (llama_new_context_with_model, src/llama.cpp:19507-19594). */
B200_API int b200_llama_finalize(b200_llama *m, int32_t max_batch);

/* Per-layer hyper-parameters (architectures other than llama), before any b200_llama_set_tensor. */
B200_API int b200_llama_set_layer(b200_llama *m, int32_t il, const b200_layer_params *lp);

/* The order in which the layers run: order[r] is the layer (weights) of run r; a layer may run several times, and every run has
 * its own cache rows or recurrent state.  Default: every layer once, in index order.  Before any b200_llama_set_tensor. */
B200_API int b200_llama_set_layer_order(b200_llama *m, const int32_t *order, int32_t n_runs);

/* Sequences: a batch step names the sequence of every token; the decoder keeps each sequence's cache cells, positions and
 * recurrent state.  open returns a free sequence id (B200_ERR_NOMEM when n_seq_max are open); close gives its cells and its
 * state slot back (llama_kv_cache_seq_rm over the whole sequence). */
B200_API int b200_llama_seq_open(b200_llama *m, int32_t *seq_id);
B200_API int b200_llama_seq_close(b200_llama *m, int32_t seq_id);
B200_API int b200_llama_seq_length(b200_llama *m, int32_t seq_id);

/* One step over a batch (llama_decode with a llama_batch of several sequences): tokens[i] continues sequence seq_ids[i] at that
 * sequence's next position; the tokens of one sequence are adjacent and in order.  want[i] != 0 asks for the logits at token i;
 * logits receives them in batch order, n_vocab floats each (want == NULL: none).  Synchronous on return. */
B200_API int b200_llama_decode_batch(b200_llama *m, const int32_t *tokens, const int32_t *seq_ids, const int8_t *want, int32_t n_tokens, float *logits);

/* Raw access to KV cells [cell0, cell0+n) of layer il (is_v: 0 = K, 1 = V): rows of n_embd_gqa values in type_k / type_v,
 * as llama_state_seq_set_data would write them (ggml_backend_tensor_set with an offset). */
B200_API int b200_llama_kv_write(b200_llama *m, int32_t il, int32_t is_v, int32_t cell0, int32_t n, const void *data);
B200_API int b200_llama_kv_read(b200_llama *m, int32_t il, int32_t is_v, int32_t cell0, int32_t n, void *data);

/* llama_decode for one sequence: tokens[n_tokens] at positions n_past .. n_past+n_tokens-1, stored in KV cells of the same
 * index.  logits: host buffer receiving n_vocab floats of the LAST token (logits_all == 0) or n_tokens*n_vocab (!= 0).
 * Synchronous on return (like llama_decode + llama_get_logits).  logits may be NULL (then nothing is copied back). */
B200_API int b200_llama_decode(b200_llama *m, const int32_t *tokens, int32_t n_tokens, int32_t n_past, float *logits, int32_t logits_all);

/* Asynchronous halves of the same call, for device-side timing: enqueue copies + graph, then wait. */
B200_API int b200_llama_decode_async(b200_llama *m, const int32_t *tokens, int32_t n_tokens, int32_t n_past, float *logits, int32_t logits_all);
B200_API int b200_llama_synchronize(b200_llama *m);
/* Replay the last decoded graph again with inputs already resident (no H2D / D2H): the HBM-resident leg of bench.py. */
B200_API int b200_llama_replay(b200_llama *m);
B200_API b200_stream_t b200_llama_stream(b200_llama *m); /* the backend's stream (for CUDA-event timing) */

/* Introspection for tests: number of graph nodes / kernels launched by the last decode, bytes of weights resident. */
B200_API int b200_llama_stats(b200_llama *m, int64_t *n_nodes, int64_t *n_kernels, int64_t *weight_bytes, int64_t *kv_bytes);

#ifdef __cplusplus
}
#endif
#endif

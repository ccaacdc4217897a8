/* b200_ggml_ops.h -- C ABI of the hot-path-adjacent ops: everything else a llama / mixtral
 * graph contains, so that a whole decode graph stays on the device (no CPU fallback, CUDA-graph capturable).
 * Tensors are described the way ggml does: element counts ne[4] and BYTE strides nb[4] (ggml.h:584-619).
 * Each entry cites the reference CUDA kernel it replaces and the CPU function that defines its semantics
 * (paths under /root/reference/ggml/src/).
 */
#ifndef B200_GGML_OPS_H
#define B200_GGML_OPS_H

#include "b200_ggml.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    void   *data;
    int32_t type; /* enum b200_type / ggml_type */
    int32_t _pad;
    int64_t ne[4];
    size_t  nb[4];
} b200_tensor;

enum b200_binary_op { B200_BIN_ADD = 0, B200_BIN_SUB = 1, B200_BIN_MUL = 2, B200_BIN_DIV = 3 };
enum b200_unary_op {
    B200_UN_SILU = 0, B200_UN_GELU = 1, B200_UN_GELU_QUICK = 2, B200_UN_RELU = 3, B200_UN_TANH = 4, B200_UN_SIGMOID = 5,
    B200_UN_SQR = 6, B200_UN_SCALE = 7 /* p0 = factor */, B200_UN_CLAMP = 8 /* p0 = min, p1 = max */,
    B200_UN_SOFTCAP = 9 /* p0 * tanh(x / p0) */,
};

/* RMS_NORM (+ optional fused MUL by a per-column weight): y = x / sqrt(mean(x^2) + eps) [* w]
 * replaces rms_norm_f32, ggml-cuda/norm.cu:101-140; semantics ggml_compute_forward_rms_norm_f32, ggml.c:12060-12110.
 * x, dst: f32, rows contiguous (nb[0] == 4).  w: f32 [ne0] or NULL. */
B200_API int b200_op_rms_norm(const b200_tensor *x, const float *w, const b200_tensor *dst, float eps, b200_stream_t stream);

/* Fused RMS_NORM -> MUL(weight) pair as llama graphs emit it (src/llama.cpp:9130-9160 llm_build_norm): dst = norm(x) * w;
 * norm_out (optional, contiguous rows) also receives norm(x), the intermediate node's value. */
B200_API int b200_op_rms_norm_mul(const b200_tensor *x, const float *w, float *norm_out, const b200_tensor *dst, float eps, b200_stream_t stream);
/* Fused UNARY(SILU) -> MUL pair of the gated FFN (src/llama.cpp:9416-9515 llm_build_ffn, LLM_FFN_SILU + LLM_FFN_PAR):
 * dst = silu(gate) * up over n contiguous floats; act_out (optional) also receives silu(gate). */
B200_API int b200_op_silu_mul(const float *gate, const float *up, float *act_out, float *dst, int64_t n, b200_stream_t stream);

/* ADD / SUB / MUL / DIV with ggml broadcasting of src1 over src0 (ggml_can_repeat): f32 only.
 * replaces k_bin_bcast, ggml-cuda/binbcast.cu:26-120; semantics ggml_compute_forward_{add,sub,mul,div}_f32, ggml.c:10241-10900 */
B200_API int b200_op_binary(int op, const b200_tensor *a, const b200_tensor *b, const b200_tensor *dst, b200_stream_t stream);

/* elementwise f32 -> f32 on a contiguous tensor.  replaces ggml-cuda/unary.cu, scale.cu, clamp.cu */
B200_API int b200_op_unary(int op, const b200_tensor *x, const b200_tensor *dst, float p0, float p1, b200_stream_t stream);

/* ROPE (normal and NeoX ordering, YaRN extrapolation mix, optional frequency factors), f32.
 * replaces rope_norm / rope_neox, ggml-cuda/rope.cu:32-120; semantics ggml_compute_forward_rope_f32, ggml.c:14272-14400.
 * x: [ne0 = head dim, ne1 = heads, ne2 = tokens]; pos: i32 [ne2]; freq_factors: f32 [n_dims/2] or NULL. */
typedef struct {
    int32_t n_dims, mode, n_ctx_orig;
    float   freq_base, freq_scale, ext_factor, attn_factor, beta_fast, beta_slow;
} b200_rope_params;
B200_API int b200_op_rope(const b200_tensor *x, const int32_t *pos, const float *freq_factors, const b200_tensor *dst,
                          const b200_rope_params *rp, b200_stream_t stream);

/* CPY / CONT / DUP: same element count, arbitrary strides; f32->f32, f32->f16, f16->f16, f16->f32, f32->q8_0 (the KV-cache
 * store; quantize_row_q8_0_ref arithmetic, ggml-quants.c:849-872).  For q8_0 destinations src rows must be contiguous.
 * replaces ggml-cuda/cpy.cu:34-440 */
B200_API int b200_op_cpy(const b200_tensor *src, const b200_tensor *dst, b200_stream_t stream);
/* Same, but the destination base pointer is read on the device from *dst_slot when the kernel runs (dst->data is ignored
 * when dst_slot != NULL).  Used for the KV-cache store inside a replayed CUDA graph: the write position moves every token
 * (reference: cudaGraphExecKernelNodeSetParams patching of the cpy nodes, ggml-cuda.cu:2593-2650). */
B200_API int b200_op_cpy_indirect(const b200_tensor *src, const b200_tensor *dst, void *const *dst_slot, b200_stream_t stream);

/* The four nodes llm_build_kv emits per layer in one launch (src/llama.cpp:9161-9203, 10504-10523): q_dst = ROPE(q),
 * k_dst = ROPE(k), cache_k[new rows] = CPY(k_dst), cache_v[new rows] = CPY(v).  q [D, n_head, T], k [D, n_head_kv, T],
 * v [D*n_head_kv, T]: contiguous f32.  kv_type: F16 or Q8_0; the T new cache rows are contiguous at k_cache / v_cache, or at
 * *k_slot / *v_slot read on the device (CUDA-graph replay with a moving write position).  NORM rope ordering only. */
B200_API int b200_op_rope_kv_store(const b200_tensor *q, const b200_tensor *q_dst, const b200_tensor *k, const b200_tensor *k_dst,
                                   const b200_tensor *v, const int32_t *pos, const float *freq_factors, const b200_rope_params *rp,
                                   int kv_type, void *k_cache, void *v_cache, void *const *k_slot, void *const *v_slot, b200_stream_t stream);

/* GET_ROWS: dst[i] = dequantise(src row ids[i]); src f32 / f16 / q4_0 / q8_0 / q4_K / q5_K / q6_K (K-quant token embeddings
 * stay on the device -- the reference falls back to the CPU for them, ggml-cuda.cu:3033-3047).
 * replaces k_get_rows / k_get_rows_float, ggml-cuda/getrows.cu:5-120 */
B200_API int b200_op_get_rows(const b200_tensor *src, const b200_tensor *ids, const b200_tensor *dst, b200_stream_t stream);

/* SOFT_MAX over ne0 with optional f16/f32 mask [ne0, >= ne1] broadcast over heads, scale and ALiBi max_bias.
 * replaces soft_max_f32, ggml-cuda/softmax.cu:15-120; semantics ggml_compute_forward_soft_max_f32, ggml.c:13900-14005 */
B200_API int b200_op_soft_max(const b200_tensor *x, const b200_tensor *mask, const b200_tensor *dst, float scale, float max_bias,
                              b200_stream_t stream);

/* ARGSORT of every row (ne0 <= 1024), i32 indices out; order: 0 ascending, 1 descending (ties keep index order).
 * replaces k_argsort_f32_i32, ggml-cuda/argsort.cu:11-100 */
/* The router of llm_build_moe_ffn (src/llama.cpp:9416-9470) in one launch, replacing SOFT_MAX -> ARGSORT(desc) + VIEW(top n_used) ->
 * GET_ROWS -> SUM_ROWS -> DIV: per token, probs = softmax(logits[n_expert]); ids[k] = index of the k-th largest prob (ties: lowest
 * index); w_gather[k] = probs[ids[k]]; wsum = sum_k w_gather[k]; w_out[k] = w_gather[k] / wsum.  ld_* are row strides in elements;
 * w_gather / w_out are [n_tok][n_used] contiguous (they may alias); n_expert <= 256, n_used <= 32. */
B200_API int b200_op_moe_router(const float *logits, int64_t ld_logits, float *probs, int64_t ld_probs, int32_t *ids, int64_t ld_ids, float *w_gather,
                                float *wsum, float *w_out, int32_t n_expert, int32_t n_used, int64_t n_tok, b200_stream_t stream);
B200_API int b200_op_argsort(const b200_tensor *x, const b200_tensor *dst, int order, b200_stream_t stream);

/* SUM_ROWS: dst[row] = sum over ne0.  replaces k_sum_rows_f32, ggml-cuda/sumrows.cu:3-30 */
B200_API int b200_op_sum_rows(const b200_tensor *x, const b200_tensor *dst, b200_stream_t stream);

/* MUL_MAT with an f32, f16 or bf16 weight matrix (MoE router, small dense layers): dst[n][m] = sum_k W[m][k] X[n][k], with ggml's
 * broadcast over dims 2 and 3.  A bandwidth-oriented warp-per-output kernel; the quantised hot path lives in b200_ggml.h.
 * replaces the cuBLAS / mul_mat_vec_nc paths for float weights, ggml-cuda.cu:1042-1284 */
B200_API int b200_op_mul_mat_float(const b200_tensor *w, const b200_tensor *x, const b200_tensor *dst, b200_stream_t stream);


/* ------------------------------------------------------------------------------------------------------------------------
 * Ops beyond the llama / mixtral graph (no counterpart in the reference): normalisation with a gate and a residual, a
 * polynomial activation, rotation by a frequency table, a weighted sum over stacked activations, attention over a latent
 * cache with a per-head sink, and a matrix-memory recurrence.  In a graph they travel as GGML_OP_MAP_CUSTOM1 nodes tagged
 * B200_EXT_TAG in op_params[0] with the kind in op_params[1] (the tensor-parallel collectives use the same carrier).
 * Everything here is computed in f32. */
#define B200_EXT_TAG 0xB200E7A5u
enum b200_ext_op {
    B200_EXT_NORM = 1,         /* src: x, w, [gate, gate_bias, res, bias]; op_params: [2] kind, [3] eps, [4] w_period, [5] gate: 0 sigmoid in front of the norm,
                                  1 sigmoid on the output, 2 silu on the output */
    B200_EXT_POLYNORM = 2,     /* src: x, coef[4]; op_params: [3] eps */
    B200_EXT_ROPE_TABLE = 3,   /* src: x, pos, freqs; in place; op_params: [2] n_dims, [3] mscale, [4] neox */
    B200_EXT_WEIGHTED_SUM = 4, /* src: xs [n, J], w [J] */
    B200_EXT_SIGMOID_MUL = 5,  /* src: a, b: dst = a * sigmoid(b), any strides */
    B200_EXT_LATENT_KV_STORE = 6, /* src: dkv, norm w, pos, freqs, cells, cache; op_params: [2] kv_rank, [3] eps, [4] mscale, [5] n_dims */
    B200_EXT_LATENT_ATTN = 7,  /* src: q_lat, q_rot, cache, sink, tok_seq, tok_pos, cell_seq, cell_pos; op_params: [2] kv_rank, [3] scale, [4] window */
    B200_EXT_MLSTM_SCAN = 8,   /* src: q, k, v, ig, fg, i_bias, f_bias, seq_info, state; op_params: [2] heads, [3] dim, [4] vdim, [5] gate_cap */
    B200_EXT_QKV_STORE = 9,    /* src: q, k, v, vecs (the present ones of q.b, k.b, v.b, q.norm, k.norm packed in one tensor, or NULL), pos, freqs,
                                  cells, k cache, v cache; q in place; op_params: [2] dim, [3] vdim, [4] n_dims, [5] eps, [6] biases present, [7] norms present
                                  (1: over the whole row, 2: per head with one weight vector of dim values), [8] pairs are (i, i + n_dims / 2), [9] every head of v is divided
                                  by its root mean square, [10] q temperature coefficient, [11] its period in positions; freqs may be NULL without rotation */
    B200_EXT_SINK_ATTN = 10,   /* src: q, k cache, v cache, sink, tok_seq, tok_pos, cell_seq, cell_pos, [head gate [heads, T]]; op_params: [2] dim, [3] scale,
                                  [4] window, [5] keep_first, [6] bf16 products, [7] vdim, [8] chunk, [9] enum b200_attn_weights; src[9]: score bias by distance
                                  [n_dist, heads] (optional) */
    B200_EXT_LINEAR_ATTN_SCAN = 11, /* src: q, k, v, decay, seq_info, state; op_params: [2] heads, [3] dim, [4] vdim, [5] silu on q / k / v */
    B200_EXT_MOE_ROUTE = 12,   /* src: logits, correction; dst [2 n_used, T]: per token n_used weights (f32), then n_used expert ids (i32);
                                  op_params: [2] n_group, [3] n_group_used, [4] scale, [5] n_used, [6] enum b200_router_score, [7] weights are the
                                  scores as they are (no division by their sum) */
    B200_EXT_SILU_MUL = 13,    /* src: a, b, [scale [ne1, ne2]]: dst = act(s a) * (s b), any strides; op_params: [2] enum b200_glu_kind (0: silu), [3] limit, [4] alpha */
    B200_EXT_MOE_COMBINE = 14, /* src: y [n, n_used, T], weights [n_used, T], add0, add1 (optional [n, T]), [norm weight [n]]: dst = add0 + add1 + sum_k w_k y_k;
                                  op_params[2] != 0: an RMS norm with eps op_params[3] and the norm weight runs over the sum before add0 joins (no add1);
                                  else src[5], src[6] (optional): a shared result [n, T] and its gate logit per token, and op_params[4] the multiplier (0 reads
                                  as 1): dst = add0 + mult * (add1 + sum_k w_k y_k + sigmoid(gate) * shared); y and the weights may be absent */
    B200_EXT_UNARY = 15,       /* src: x; op_params: [2] enum b200_unary_op, [3] p0, [4] p1 */
    B200_EXT_MUL_MAT_ID = 16,  /* src: experts [K, M, E] f32 / bf16, b [K, n_b_rows, T], ids [n_used, T]: dense-weight form of MUL_MAT_ID */
    B200_EXT_ADD_SINUSOID = 17, /* src: x [n, T], pos, freqs [ceil(n / 2)]: dst[2i] = x[2i] + sin(pos f_i), dst[2i + 1] = x[2i + 1] + cos(pos f_i) */
    B200_EXT_SHORT_CONV = 18,  /* src: x [channels, T], w [taps, channels], bias (optional), seq_info, tail [(taps - 1) * channels, slots]; op_params: [2] activation
                                  (0 none, 1 silu) */
    B200_EXT_DELTA_RULE_SCAN = 19, /* src: q, k, v, a, b, a_log, dt_bias, seq_info, state; op_params: [2] heads, [3] kv_heads, [4] dim, [5] vdim, [6] q and k become
                                  unit vectors, [7] the eps of that, [8] q scale */
    B200_EXT_MINGRU_SCAN = 20, /* src: z, x, g (optional), z bias, x bias (optional), seq_info, state [width, slots] */
    B200_EXT_NORM_PAIR = 21,   /* src: x1, w1, b1 (optional), x2, w2: dst = N(x1 + b1) * w1 + N(x2) * w2, N the RMS norm; op_params: [3] eps */
};
/* how attention turns scores into weights: SOFTMAX over the visible keys (with the sink in the denominator), or SIGMOID of every score by
 * itself with no normalisation over the keys (a sink has no meaning then) */
enum b200_attn_weights { B200_ATTN_SOFTMAX = 0, B200_ATTN_SIGMOID = 1 };

enum b200_router_score { B200_ROUTER_SIGMOID = 0, B200_ROUTER_SOFTMAX = 1 /* over all experts */ };
/* gated activations dst = f(a, b): SILU a sigmoid(a) b; GELU_TANH gelu(a) b with the tanh form of gelu; SWISH_CLAMPED with g = min(a, limit),
 * u = clamp(b, -limit, limit): g sigmoid(alpha g) (u + 1) */
enum b200_glu_kind { B200_GLU_SILU = 0, B200_GLU_GELU_TANH = 1, B200_GLU_SWISH_CLAMPED = 2 };
enum b200_norm_kind { B200_NORM_LAYER = 0 /* (x - mean) / sqrt(var + eps) */, B200_NORM_RMS = 1 /* x / sqrt(mean(x^2) + eps) */ };

/* dst[row] = (res ? res[row] : 0) + N(x[row] * (gate ? sigmoid(gate[row] + gate_bias) : 1)) * w[(row % w_period)], N the layer
 * norm or the RMS norm over ne0.  x, gate, res, dst: f32 rows (nb[0] == 4), any row strides; w: [w_period][ne0] f32 or NULL;
 * gate_bias: [ne0] or NULL.  One block per row, statistics in f32 (variance = mean of squared deviations, two passes). */
B200_API int b200_op_norm(const b200_tensor *x, const float *w, int64_t w_period, const b200_tensor *gate, const float *gate_bias,
                          const b200_tensor *res, const b200_tensor *dst, float eps, int kind, b200_stream_t stream);

/* The same with a bias behind the weight (dst = res + N(..) * w + bias) and the gate either in front of the norm (gate_on_output
 * == 0, as above) or behind it: dst = res + (N(x) * w + bias) * f(gate + gate_bias), f the sigmoid (gate_on_output == 1) or silu
 * z sigmoid(z) (gate_on_output == 2). */
B200_API int b200_op_norm_affine(const b200_tensor *x, const float *w, int64_t w_period, const float *bias, const b200_tensor *gate, const float *gate_bias,
                                 int gate_on_output, const b200_tensor *res, const b200_tensor *dst, float eps, int kind, b200_stream_t stream);

/* Two results joined behind their own RMS norms, one row per block: dst = N(x1 + b1) * w1 + N(x2) * w2 with N(z) = z / sqrt(mean(z^2) + eps)
 * over ne0; b1 optional; x1, x2, dst f32 rows of one shape with any row strides; ne0 <= 16384. */
B200_API int b200_op_norm_pair(const b200_tensor *x1, const float *w1, const float *b1, const b200_tensor *x2, const float *w2, const b200_tensor *dst, float eps,
                               b200_stream_t stream);

/* PolyNorm: dst = c0 N(x) + c1 N(x^2) + c2 N(x^3) + c3 with N(z) = z / sqrt(mean(z^2) + eps) over ne0, powers element by
 * element; coef: 4 floats on the device. */
B200_API int b200_op_polynorm(const b200_tensor *x, const float *coef, const b200_tensor *dst, float eps, b200_stream_t stream);

/* Rotation by a table of frequencies: for pair i < n_dims/2 of every row of x [ne0, ne1 (heads), ne2 (tokens)] the angle is
 * pos[token] * freqs[i]; (u, v) -> mscale * (u cos - v sin, v cos + u sin).  Pairs are (2i, 2i+1), or (i, i + n_dims/2) with
 * neox != 0; elements from n_dims on are copied.  x and dst may be the same view.  The table carries any frequency scaling
 * (linear, NTK, YaRN ramps) computed once by the caller. */
B200_API int b200_op_rope_table(const b200_tensor *x, const int32_t *pos, const float *freqs, const b200_tensor *dst, int32_t n_dims,
                                int32_t neox, float mscale, b200_stream_t stream);

/* dst[i] = sum_j w[j] * xs[j * slice_stride + i], j ascending, i < n. */
B200_API int b200_op_weighted_sum(const float *xs, int64_t slice_stride, int32_t n_slices, const float *w, float *dst, int64_t n, b200_stream_t stream);

/* dst = a * sigmoid(b); a, b, dst f32 of one shape with any strides (a permuted view is fine). */
B200_API int b200_op_sigmoid_mul(const b200_tensor *a, const b200_tensor *b, const b200_tensor *dst, b200_stream_t stream);

/* Latent KV cache (one row per cell: kv_rank normalised latent values, then rot_dim rotated key values, f32).
 * store: row cells[t] = [ RMSnorm(dkv[t][:kv_rank]) * w , rope_table(dkv[t][kv_rank:]) ]. */
B200_API int b200_op_latent_kv_store(const float *dkv, int64_t dkv_stride, const float *w, const int32_t *pos, const float *freqs, const int32_t *cells,
                                     float *cache, int64_t cache_stride, int32_t kv_rank, int32_t rot_dim, int32_t n_dims, float mscale, float eps,
                                     int32_t n_tokens, b200_stream_t stream);

/* Attention of H query heads over the latent cache (every head reads the same rows: the key is the whole row, the value its
 * first kv_rank entries).  score = scale * (q_lat . row[:kv_rank] + q_rot . row[kv_rank:]); a token sees the cells of its own
 * sequence with cell_pos <= tok_pos (and cell_pos > tok_pos - window when window > 0); softmax in f32 whose denominator also
 * holds exp(sink[h]) when sink != NULL.  Strides are in floats.  dst[h][t][:kv_rank] = sum_c p_c row_c[:kv_rank].
 * bf16_products != 0 allows the two contractions of a prompt batch (16 tokens or more) to take queries, rows and weights rounded
 * to bf16 with f32 accumulation (scores, maxima, exponentials and sums stay f32); 0 keeps every product in f32. */
typedef struct {
    const float *q_lat; int64_t q_lat_s_head, q_lat_s_tok;
    const float *q_rot; int64_t q_rot_s_head, q_rot_s_tok;
    const float *cache; int64_t cache_stride;
    const int32_t *cell_seq, *cell_pos, *tok_seq, *tok_pos;
    const float *sink;
    float *dst; int64_t dst_s_head, dst_s_tok;
    int32_t kv_rank, rot_dim, n_head, n_tokens, n_kv, window;
    float scale;
    int32_t bf16_products;
} b200_latent_attn_args;
B200_API int b200_op_latent_attn(const b200_latent_attn_args *a, b200_stream_t stream);

/* Matrix-memory recurrence (mLSTM) over the tokens of n_seq sequences, state per (slot, head) in f32:
 *   i = cap tanh((ig + i_bias) / cap),  f = logsigmoid(cap tanh((fg + f_bias) / cap)),  m' = max(f + m, i),
 *   S' = exp(f + m - m') S + exp(i - m') k v^T,  n' likewise with k,  o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6),  q scaled by q_scale.
 * seq_info: int32 [4][n_seq] = first token, token count, state slot, fresh (1: start from S = 0, n = 0, m = 0).
 * State: slot_stride floats per slot, of which the first b200_mlstm_state_floats(heads, dim, vdim) are used: S [head][vdim][dim],
 * then n and m once per column tile of the kernel (a tile never reads what another tile of the same launch writes).
 * Strides in floats; dst [heads * vdim] per token. */
B200_API int64_t b200_mlstm_state_floats(int32_t heads, int32_t dim, int32_t vdim);
typedef struct {
    const float *q, *k, *v, *ig, *fg; int64_t q_stride, k_stride, v_stride, g_stride;
    const float *i_bias, *f_bias;
    const int32_t *seq_info; int32_t n_seq;
    float *state; int64_t slot_stride;
    float *dst; int64_t dst_stride;
    int32_t heads, dim, vdim;
    float gate_cap, q_scale;
} b200_mlstm_args;
B200_API int b200_op_mlstm_scan(const b200_mlstm_args *a, b200_stream_t stream);


/* dst = silu(a) * b; a, b, dst f32 of one shape with any strides (the two halves of a fused gate / up product are fine). */
B200_API int b200_op_silu_mul_strided(const b200_tensor *a, const b200_tensor *b, const b200_tensor *dst, b200_stream_t stream);
/* The same for any enum b200_glu_kind; limit and alpha are read by B200_GLU_SWISH_CLAMPED only. */
B200_API int b200_op_glu_strided(int kind, const b200_tensor *a, const b200_tensor *b, const b200_tensor *dst, float limit, float alpha, b200_stream_t stream);
/* The same with both inputs multiplied by scale[i1, i2] first (f32, any strides; NULL: none): an expert whose weight scales its input,
 * applied behind the linear gate / up products instead of in front of them. */
B200_API int b200_op_glu_scaled(int kind, const b200_tensor *a, const b200_tensor *b, const b200_tensor *scale, const b200_tensor *dst, float limit, float alpha,
                                b200_stream_t stream);

/* Softmax attention of n_head query heads over cached keys and values of n_head_kv heads (query head h reads kv head
 * h / (n_head / n_head_kv)); one cache row per cell holds all kv heads of a token: k rows [n_head_kv * dim], v rows
 * [n_head_kv * vdim], f32.
 * store: per token t, q (and k) += bias; q, k <- RMS norm * weight (when given) over the whole row, or with norm_per_head over
 * every head by itself with one weight vector of dim values for all heads; the first n_dims values of every head of q and k are
 * rotated by pos[t] * freqs[i] as interleaved pairs (2i, 2i + 1), or with rope_halves as pairs (i, i + n_dims / 2); q is written
 * back in place, k and v (+ bias) go to row cells[t] of the caches.  Strides in floats. */
typedef struct {
    float *q; int64_t q_stride;            /* [n_tokens][n_head * dim], rotated in place */
    const float *k; int64_t k_stride;      /* [n_tokens][n_head_kv * dim] */
    const float *v; int64_t v_stride;      /* [n_tokens][n_head_kv * vdim] */
    const float *q_bias, *k_bias, *v_bias; /* NULL: none */
    const float *q_norm, *k_norm;          /* NULL: no norm */
    const int32_t *pos, *cells;
    const float *freqs;                    /* [n_dims / 2] */
    float *k_cache; int64_t k_cache_stride;
    float *v_cache; int64_t v_cache_stride;
    int32_t n_head, n_head_kv, dim, vdim, n_dims, n_tokens;
    float eps;
    int32_t norm_per_head, rope_halves;
    int32_t v_unit_rms;                    /* 1: every head of v is divided by sqrt(mean(v^2) + eps) before it is stored (behind the bias) */
    float   q_temp_coef;                   /* != 0: q is multiplied by 1 + coef * ln(floor((pos + 1) / q_temp_every) + 1) */
    int32_t q_temp_every;
} b200_qkv_store_args;
B200_API int b200_op_qkv_store(const b200_qkv_store_args *a, b200_stream_t stream);

/* score = scale * q . k (+ dist_bias, see below); a token sees the cells of its own sequence with cell_pos <= tok_pos and (window == 0 or
 * tok_pos - cell_pos < window or cell_pos < keep_first) and (chunk == 0 or tok_pos / chunk == cell_pos / chunk: positions are cut
 * into chunks counted from 0 and nothing is seen across a cut); softmax in f32 whose denominator also holds exp(sink[h]) when
 * sink != NULL (the sink has no key and no value).  gate != NULL: head h of token t is multiplied by sigmoid(gate[t * gate_stride
 * + h]).  dst [n_tokens][n_head * vdim].  bf16_products as for b200_op_latent_attn. */
typedef struct {
    const float *q; int64_t q_stride;
    const float *k_cache; int64_t k_cache_stride;
    const float *v_cache; int64_t v_cache_stride;
    const int32_t *cell_seq, *cell_pos, *tok_seq, *tok_pos;
    const float *sink;
    float *dst; int64_t dst_stride;
    int32_t n_head, n_head_kv, dim, vdim, n_tokens, n_kv, window, keep_first;
    float scale;
    int32_t bf16_products;
    int32_t chunk;
    const float *gate; int64_t gate_stride;
    int32_t weights;                       /* enum b200_attn_weights */
    const float *dist_bias; int32_t n_dist; /* [n_head][n_dist] added to the scaled score of a key min(tok_pos - cell_pos, n_dist - 1) positions back (NULL: none) */
} b200_sink_attn_args;
B200_API int b200_op_sink_attn(const b200_sink_attn_args *a, b200_stream_t stream);
/* The same with a workspace of b200_sink_attn_workspace_bytes(a) bytes (16-byte aligned; 0: none needed): with few tokens and
 * many cells (decode) the cells of a (token, head) pair are split over several CTAs whose partial results meet there. */
B200_API size_t b200_sink_attn_workspace_bytes(const b200_sink_attn_args *a);
B200_API int b200_op_sink_attn_ws(const b200_sink_attn_args *a, void *workspace, size_t workspace_bytes, b200_stream_t stream);

/* Linear attention with a decayed state per (slot, head), f32: S' = decay[h] S + k v^T, o = S'^T q, over the tokens of n_seq
 * sequences; act != 0 applies silu to q, k and v first.  seq_info as for b200_op_mlstm_scan.  State [head][vdim][dim] per slot.
 * q, k: [n_tokens][heads * dim], v and dst: [n_tokens][heads * vdim]; strides in floats. */
typedef struct {
    const float *q, *k, *v; int64_t q_stride, k_stride, v_stride;
    const float *decay;                    /* [heads] */
    const int32_t *seq_info; int32_t n_seq;
    float *state; int64_t slot_stride;
    float *dst; int64_t dst_stride;
    int32_t heads, dim, vdim, act;
} b200_linear_attn_args;
B200_API int b200_op_linear_attn_scan(const b200_linear_attn_args *a, b200_stream_t stream);

/* Router with sigmoid scores, a choice bias and group-limited choice, one token per warp: s = sigmoid(logits); c = s + correction
 * (NULL: none); with n_group > 1 the n_expert experts form n_group equal groups of neighbours, a group scores the sum of its two
 * largest c, and only experts of the n_group_used best groups can be chosen; ids[k] = the n_used largest c (ties: lowest index);
 * w[k] = s[ids[k]] / (sum_k s[ids[k]] + 1e-20) * scale.  n_expert <= 256, n_used <= 32.  ld_* in elements. */
B200_API int b200_op_moe_route_grouped(const float *logits, int64_t ld_logits, const float *correction, int32_t *ids, int64_t ld_ids, float *w, int64_t ld_w,
                                       int32_t n_expert, int32_t n_used, int32_t n_group, int32_t n_group_used, float scale, int64_t n_tok, b200_stream_t stream);
/* The same router with the score function as a parameter (enum b200_router_score: sigmoid per expert, or softmax over all
 * experts) and, with keep_scores != 0, weights w[k] = s[ids[k]] * scale without the division by their sum. */
B200_API int b200_op_moe_route_scored(const float *logits, int64_t ld_logits, const float *correction, int32_t *ids, int64_t ld_ids, float *w, int64_t ld_w,
                                      int32_t n_expert, int32_t n_used, int32_t n_group, int32_t n_group_used, float scale, int32_t score, int32_t keep_scores,
                                      int64_t n_tok, b200_stream_t stream);

/* dst[t] = add0[t] + add1[t] + sum_k w[t][k] * y[t][k]; y [n, n_used, T] f32, w [n_used, T], add0 / add1 / dst [n, T] (add0, add1
 * optional); strides in floats. */
B200_API int b200_op_moe_combine(const float *y, int64_t y_s_slot, int64_t y_s_tok, const float *w, int64_t w_s_tok, const float *add0, int64_t add0_stride,
                                 const float *add1, int64_t add1_stride, float *dst, int64_t dst_stride, int64_t n, int32_t n_used, int64_t n_tok, b200_stream_t stream);

/* dst[t] = add0[t] + mult * (add1[t] + sum_k w[t][k] * y[t][k] + sigmoid(gate[t * gate_stride]) * shared[t]): the chosen experts, a shared
 * expert gated per token, the other sublayer's result and the scaled residual connection in one launch.  w NULL: weights of one; y
 * NULL (n_used 0), add0, add1, shared: optional. */
B200_API int b200_op_moe_combine_shared(const float *y, int64_t y_s_slot, int64_t y_s_tok, const float *w, int64_t w_s_tok, const float *add0, int64_t add0_stride,
                                        const float *add1, int64_t add1_stride, const float *shared, int64_t shared_stride, const float *gate, int64_t gate_stride,
                                        float mult, float *dst, int64_t dst_stride, int64_t n, int32_t n_used, int64_t n_tok, b200_stream_t stream);

/* The same sum followed by an RMS norm over it and a residual: dst[t] = res[t] + s / sqrt(mean(s^2) + eps) * norm_w with s = sum_k w[t][k] * y[t][k];
 * norm_w and res are optional; n <= B200_MOE_COMBINE_NORM_MAX (the summed row waits in the registers of one CTA), n_used <= 32. */
#define B200_MOE_COMBINE_NORM_MAX 16384
B200_API int b200_op_moe_combine_norm(const float *y, int64_t y_s_slot, int64_t y_s_tok, const float *w, int64_t w_s_tok, const float *norm_w, float eps, const float *res,
                                      int64_t res_stride, float *dst, int64_t dst_stride, int64_t n, int32_t n_used, int64_t n_tok, b200_stream_t stream);

/* MUL_MAT_ID over dense f32 or bf16 expert matrices: as [K, M, n_expert], b [K, n_b_rows, T] f32, ids [n_used, T]:
 * dst[:, s, t] = as[:, :, ids[s, t]] . b[:, s % n_b_rows, t].  Any K and M; f32 accumulation; products in f32 (bf16 weights are
 * widened).  The batched tensor-core form for bf16 weights is b200_mul_mat_id_q (b200_ggml.h). */
B200_API int b200_op_mul_mat_id_float(const b200_tensor *as, const b200_tensor *b, const b200_tensor *ids, const b200_tensor *dst, b200_stream_t stream);

/* dst[t][2i] = x[t][2i] + sin(pos[t] * freqs[i]), dst[t][2i + 1] = x[t][2i + 1] + cos(pos[t] * freqs[i]); x, dst [n, T] f32 rows with any
 * row strides (they may be the same); angles pos * f in f32. */
B200_API int b200_op_add_sinusoid(const b200_tensor *x, const int32_t *pos, const float *freqs, const b200_tensor *dst, b200_stream_t stream);

/* Short causal convolution over time, every channel by itself: y[t] = act(sum_j w[c][j] * u[t - taps + 1 + j]), u = x + bias, zeros before
 * the start of a sequence.  The last taps - 1 values of u of a sequence wait in its slot of `tail` ([taps - 1][channels] per slot) for
 * its next tokens.  seq_info as for b200_op_mlstm_scan.  x, dst [n_tokens][channels] (not the same memory), strides in floats; w
 * [channels][taps]; taps <= 17. */
typedef struct {
    const float *x; int64_t x_stride;
    const float *bias;                     /* [channels] or NULL */
    const float *w;
    const int32_t *seq_info; int32_t n_seq;
    float *tail; int64_t slot_stride;
    float *dst; int64_t dst_stride;
    int32_t channels, taps, act;           /* act: 0 none, 1 silu */
    int32_t n_tokens;
} b200_short_conv_args;
B200_API int b200_op_short_conv(const b200_short_conv_args *a, b200_stream_t stream);

/* Gated delta rule over the tokens of n_seq sequences, a state S [dim, vdim] per (slot, head) in f32:
 *   g = exp(-exp(a_log[h]) * softplus(a[t][h] + dt_bias[h])),  beta = sigmoid(b[t][h]),
 *   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
 * Head h reads q / k head h / (heads / kv_heads).  With unit_qk, q and k are first divided by sqrt(sum(x^2) + unit_eps) per head; q is
 * multiplied by q_scale.  State [head][vdim][dim] per slot; seq_info as for b200_op_mlstm_scan; strides in floats. */
typedef struct {
    const float *q, *k, *v; int64_t q_stride, k_stride, v_stride;  /* q, k [n_tokens][kv_heads * dim], v [n_tokens][heads * vdim] */
    const float *a, *b; int64_t a_stride, b_stride;                /* [n_tokens][heads] */
    const float *a_log, *dt_bias;                                  /* [heads] */
    const int32_t *seq_info; int32_t n_seq;
    float *state; int64_t slot_stride;
    float *dst; int64_t dst_stride;                                /* [n_tokens][heads * vdim] */
    int32_t heads, kv_heads, dim, vdim, unit_qk;
    float unit_eps, q_scale;
} b200_delta_rule_args;
B200_API int b200_op_delta_rule_scan(const b200_delta_rule_args *a, b200_stream_t stream);

/* minGRU, element by element over `width` channels: zg = sigmoid(z + z_bias), u = x + x_bias, c = u + 1/2 where u >= 0 and sigmoid(u)
 * elsewhere, S <- (1 - zg) S + zg c, dst = S * silu(g) (g NULL: dst = S).  State [width] per slot in f32; seq_info as above. */
typedef struct {
    const float *z, *x, *g; int64_t z_stride, x_stride, g_stride;
    const float *z_bias, *x_bias;
    const int32_t *seq_info; int32_t n_seq;
    float *state; int64_t slot_stride;
    float *dst; int64_t dst_stride;
    int32_t width, n_tokens;
} b200_mingru_args;
B200_API int b200_op_mingru_scan(const b200_mingru_args *a, b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif

// gattn.cu -- grouped-query softmax attention with a per-head sink over f32 key / value caches, and linear attention with a
// decayed state (include/b200_ggml_ops.h: b200_op_qkv_store, b200_op_sink_attn, b200_op_linear_attn_scan).
//
// Cache rows are indexed by cell, one row per token holding all kv heads; which cells a token sees follows from the (sequence,
// position) pairs of token and cell, so a batch may mix sequences, cells may be scattered, and a sliding window with kept first
// positions needs no mask tensor.  The sink only enters the softmax denominator.  A table of score biases by distance (per head) may
// join the scaled score, and the weights may be sigmoids of the scores instead of a softmax over them (nothing is normalised then).
#include "ops_util.cuh"
#include <cuda_bf16.h>

namespace b200 {
using namespace opx;

// ------------------------------------------------------------------------------------------------ bias + norm + rotation + cache store
// One CTA per token.  The RMS statistics run over the whole projection (all heads at once) or, with norm_per_head, over every
// head by itself (a warp per head, the scales parked in shared memory); q is rewritten in place, k and v go to the token's cache
// rows.  A rotated pair is (2i, 2i + 1) or, with rope_halves, (i, i + n_dims / 2).
__global__ void __launch_bounds__(1024) qkv_store_kernel(const b200_qkv_store_args a) {
    __shared__ float sh[32];
    extern __shared__ float head_scale[];  // norm_per_head: [n_head + n_head_kv]
    const int t = blockIdx.x;
    const int nq = a.n_head * a.dim, nk = a.n_head_kv * a.dim, nv = a.n_head_kv * a.vdim;
    float *q = a.q + (int64_t)t * a.q_stride;
    const float *k = a.k + (int64_t)t * a.k_stride, *v = a.v + (int64_t)t * a.v_stride;
    const int64_t cell = a.cells[t];
    float *kc = a.k_cache + cell * a.k_cache_stride, *vc = a.v_cache + cell * a.v_cache_stride;
    float qs = 1.f, ks = 1.f;
    const bool per_head = a.norm_per_head != 0;
    if (per_head) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
        for (int hh = warp; hh < a.n_head + a.n_head_kv; hh += n_warps) {
            const bool is_k = hh >= a.n_head;
            if (!(is_k ? a.k_norm : a.q_norm)) continue;  // warp-uniform
            const int e0 = (is_k ? hh - a.n_head : hh) * a.dim;
            const float *src = is_k ? k : q, *bias = is_k ? a.k_bias : a.q_bias;
            float s = 0.f;
            for (int i = lane; i < a.dim; i += 32) { const float x = src[e0 + i] + (bias ? bias[e0 + i] : 0.f); s += x * x; }
            s = warp_sum(s);
            if (lane == 0) head_scale[hh] = 1.0f / sqrtf(s / (float)a.dim + a.eps);
        }
        __syncthreads();
    } else {
        if (a.q_norm) {
            float s = 0.f;
            for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float x = q[i] + (a.q_bias ? a.q_bias[i] : 0.f); s += x * x; }
            qs = 1.0f / sqrtf(block_sum(s, sh) / (float)nq + a.eps);
        }
        if (a.k_norm) {
            float s = 0.f;
            for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float x = k[i] + (a.k_bias ? a.k_bias[i] : 0.f); s += x * x; }
            ks = 1.0f / sqrtf(block_sum(s, sh) / (float)nk + a.eps);
        }
    }
    const float p = (float)a.pos[t];
    // queries grow with the logarithm of the position, in steps of q_temp_every positions
    const float q_temp = a.q_temp_coef != 0.f ? 1.0f + a.q_temp_coef * logf((float)((a.pos[t] + 1) / max(a.q_temp_every, 1) + 1)) : 1.0f;
    const int half = a.n_dims / 2, per_head_items = half + (a.dim - a.n_dims);  // work items of a head: rotated pairs, then single values
    for (int which = 0; which < 2; which++) {
        const float *src = which ? k : q;
        float *dst = which ? kc : q;
        const float *bias = which ? a.k_bias : a.q_bias, *nw = which ? a.k_norm : a.q_norm;
        const int heads = which ? a.n_head_kv : a.n_head;
        for (int idx = threadIdx.x; idx < heads * per_head_items; idx += blockDim.x) {
            const int hh = idx / per_head_items, j = idx - hh * per_head_items;
            const float sc = (per_head && nw) ? head_scale[which * a.n_head + hh] : (which ? ks : qs);
            const int wb = per_head ? hh * a.dim : 0;  // the weight of entry e is nw[e - wb]
            if (j >= half) {
                const int e = hh * a.dim + a.n_dims + (j - half);
                float x = src[e] + (bias ? bias[e] : 0.f);
                if (nw) x = x * sc * nw[e - wb];
                dst[e] = which ? x : x * q_temp;
                continue;
            }
            const int e0 = hh * a.dim + (a.rope_halves ? j : 2 * j), e1 = a.rope_halves ? e0 + half : e0 + 1;
            float u = src[e0] + (bias ? bias[e0] : 0.f), w = src[e1] + (bias ? bias[e1] : 0.f);
            if (nw) { u = u * sc * nw[e0 - wb]; w = w * sc * nw[e1 - wb]; }
            float sn, cs;
            sincosf(p * a.freqs[j], &sn, &cs);
            const float tq = which ? 1.0f : q_temp;
            dst[e0] = (u * cs - w * sn) * tq;
            dst[e1] = (w * cs + u * sn) * tq;
        }
    }
    if (a.v_unit_rms) {  // a warp per head of v: statistics, then the scaled row
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
        for (int hh = warp; hh < a.n_head_kv; hh += n_warps) {
            const int e0 = hh * a.vdim;
            float ss = 0.f;
            for (int i = lane; i < a.vdim; i += 32) { const float x = v[e0 + i] + (a.v_bias ? a.v_bias[e0 + i] : 0.f); ss += x * x; }
            const float sc = 1.0f / sqrtf(warp_sum(ss) / (float)a.vdim + a.eps);
            for (int i = lane; i < a.vdim; i += 32) vc[e0 + i] = (v[e0 + i] + (a.v_bias ? a.v_bias[e0 + i] : 0.f)) * sc;
        }
        return;
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) vc[i] = v[i] + (a.v_bias ? a.v_bias[i] : 0.f);
}

// lo: the first position of the token's chunk (0 without chunks): nothing before it is seen
__device__ __forceinline__ bool sa_visible(int cell_seq, int cell_pos, int seq, int pos, int window, int keep_first, int lo) {
    return cell_seq == seq && cell_pos <= pos && cell_pos >= lo && (window <= 0 || pos - cell_pos < window || cell_pos < keep_first);
}
__device__ __forceinline__ int sa_chunk_start(int pos, int chunk) { return chunk > 0 ? pos - pos % chunk : 0; }
// the bias of a key `dist` positions behind the query (0 without a table)
__device__ __forceinline__ float sa_dist_bias(const b200_sink_attn_args &a, int dist, int h) {
    return a.dist_bias ? a.dist_bias[(int64_t)h * a.n_dist + min(dist, a.n_dist - 1)] : 0.f;  // a head's row is contiguous: neighbouring keys share cache lines
}
__device__ __forceinline__ float sa_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
// for weights that are rounded to bf16 right away (8 bits of mantissa): the fast exponential and division are exact enough
__device__ __forceinline__ float sa_sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float sa_head_gate(const b200_sink_attn_args &a, int64_t t, int h) {
    return a.gate ? 1.0f / (1.0f + expf(-a.gate[t * a.gate_stride + h])) : 1.0f;
}

// ------------------------------------------------------------------------------------------------ attention, f32 products
// One CTA per (token, head); its warps stride over the cells 32 at a time (one visibility test per lane, one ballot), then work
// through the visible ones SA_UNROLL at a time with all loads of a round issued before the first dot product.  Each warp keeps an
// online softmax and an accumulator; they meet in shared memory, where the sink joins the denominator.
// ND = ceil(dim / 32), NV = ceil(vdim / 32): values per lane.  WARPS is 16 when there are few (token, head) pairs (decode).
constexpr int SA_UNROLL = 4;
// With n_split > 1 (few tokens, many cells) blockIdx.z takes one stretch of the cells and leaves (maximum, sum, unnormalised
// accumulator) in `part`; sink_attn_merge_kernel joins the stretches and the sink.
template <int ND, int NV, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) sink_attn_kernel(const b200_sink_attn_args a, float *__restrict__ part, int n_split) {
    extern __shared__ float smem[];  // [WARPS][vdim] accumulators, then m[WARPS], l[WARPS]
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = a.dim, V = a.vdim;
    const int g = h / (a.n_head / a.n_head_kv);
    const float *qp = a.q + (int64_t)t * a.q_stride + (int64_t)h * D;
    const float *kb = a.k_cache + (int64_t)g * D, *vb = a.v_cache + (int64_t)g * V;
    float q[ND], acc[NV];
#pragma unroll
    for (int i = 0; i < ND; i++) { const int j = lane + 32 * i; q[i] = j < D ? qp[j] * a.scale : 0.f; }
#pragma unroll
    for (int i = 0; i < NV; i++) acc[i] = 0.f;
    const int seq = a.tok_seq[t], pos = a.tok_pos[t], lo = sa_chunk_start(pos, a.chunk);
    const bool sig = a.weights == B200_ATTN_SIGMOID;
    float m = sig ? 0.f : -INFINITY, l = 0.f;  // sigmoid weights: no maximum, no sum; the warps' accumulators simply add up
    const int per_split = ((a.n_kv + n_split - 1) / n_split + 31) & ~31;
    const int c_begin = (int)blockIdx.z * per_split, c_end = min(a.n_kv, c_begin + per_split);
    for (int cb = c_begin + warp * 32; cb < c_end; cb += WARPS * 32) {
        bool mine = false;
        int my_dist = 0;
        if (cb + lane < c_end) {
            const int cp = a.cell_pos[cb + lane];
            mine = sa_visible(a.cell_seq[cb + lane], cp, seq, pos, a.window, a.keep_first, lo);
            my_dist = pos - cp;
        }
        const float my_bias = mine ? sa_dist_bias(a, my_dist, h) : 0.f;  // lane j holds the bias of cell cb + j
        unsigned rest = __ballot_sync(0xffffffffu, mine);
        while (rest) {
            bool vis[SA_UNROLL];  // warp-uniform
            int cu[SA_UNROLL];
            float kv[SA_UNROLL][ND], vv[SA_UNROLL][NV];
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) {
                vis[u] = rest != 0u;
                cu[u] = vis[u] ? cb + __ffs(rest) - 1 : 0;
                rest &= rest - 1;  // 0 stays 0
            }
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) {
                if (!vis[u]) continue;
                const float *kr = kb + (int64_t)cu[u] * a.k_cache_stride, *vr = vb + (int64_t)cu[u] * a.v_cache_stride;
#pragma unroll
                for (int i = 0; i < ND; i++) { const int j = lane + 32 * i; kv[u][i] = j < D ? kr[j] : 0.f; }
#pragma unroll
                for (int i = 0; i < NV; i++) { const int j = lane + 32 * i; vv[u][i] = j < V ? vr[j] : 0.f; }
            }
            float s[SA_UNROLL];
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) {
                s[u] = 0.f;
                if (!vis[u]) continue;
#pragma unroll
                for (int i = 0; i < ND; i++) s[u] += q[i] * kv[u][i];
            }
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) if (vis[u]) s[u] = warp_sum(s[u]) + __shfl_sync(0xffffffffu, my_bias, cu[u] - cb);
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) {
                if (!vis[u]) continue;
                if (sig) {
                    const float p = sa_sigmoid(s[u]);
#pragma unroll
                    for (int i = 0; i < NV; i++) acc[i] += p * vv[u][i];
                    continue;
                }
                const float mn = fmaxf(m, s[u]);
                const float corr = expf(m - mn), p = expf(s[u] - mn);  // m = -inf at the first cell: corr = 0
                l = l * corr + p;
#pragma unroll
                for (int i = 0; i < NV; i++) acc[i] = acc[i] * corr + p * vv[u][i];
                m = mn;
            }
        }
    }
    float *sacc = smem + (size_t)warp * V, *sm = smem + (size_t)WARPS * V, *sl = sm + WARPS;
#pragma unroll
    for (int i = 0; i < NV; i++) { const int j = lane + 32 * i; if (j < V) sacc[j] = acc[i]; }
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
    __syncthreads();
    const float sink = (a.sink && n_split == 1 && !sig) ? a.sink[h] : -INFINITY;  // split: the merge adds the sink
    float M = sink;
    for (int w = 0; w < WARPS; w++) M = fmaxf(M, sm[w]);
    float L = sink != -INFINITY ? expf(sink - M) : 0.f;
    for (int w = 0; w < WARPS; w++) if (sm[w] != -INFINITY) L += sl[w] * expf(sm[w] - M);
    __syncthreads();
    if (threadIdx.x < WARPS) sl[threadIdx.x] = sm[threadIdx.x] == -INFINITY ? 0.f : expf(sm[threadIdx.x] - M);  // the warp's weight in the merge
    __syncthreads();
    if (n_split > 1) {
        float *pp = part + (((int64_t)t * a.n_head + h) * n_split + blockIdx.z) * (V + 2);
        if (threadIdx.x == 0) { pp[0] = M; pp[1] = L; }
        for (int j = threadIdx.x; j < V; j += blockDim.x) {
            float o = 0.f;
            for (int w = 0; w < WARPS; w++) o += smem[(size_t)w * V + j] * sl[w];
            pp[2 + j] = o;
        }
        return;
    }
    // sigmoid weights: every warp's maximum is 0, so M = 0, the warps' merge weights are 1 and nothing is divided
    const float inv = (sig ? 1.0f : (L > 0.f ? 1.0f / L : 0.f)) * sa_head_gate(a, t, h);
    float *out = a.dst + (int64_t)t * a.dst_stride + (int64_t)h * V;
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < WARPS; w++) o += smem[(size_t)w * V + j] * sl[w];
        out[j] = o * inv;
    }
}

// one CTA per (token, head), a thread per output column: the stretches' (maximum, sum, accumulator) and the sink become the output row
__global__ void __launch_bounds__(128) sink_attn_merge_kernel(const b200_sink_attn_args a, const float *__restrict__ part, int n_split) {
    const int64_t pair = blockIdx.x;
    const int V = a.vdim, h = (int)(pair % a.n_head);
    const int64_t t = pair / a.n_head;
    const float *pp = part + pair * n_split * (V + 2);
    const bool sig = a.weights == B200_ATTN_SIGMOID;  // every stretch reports the maximum 0: the stretches add up
    const float sink = (a.sink && !sig) ? a.sink[h] : -INFINITY;
    float M = sink;
    for (int z = 0; z < n_split; z++) M = fmaxf(M, pp[(int64_t)z * (V + 2)]);
    float L = sink != -INFINITY ? expf(sink - M) : 0.f;
    for (int z = 0; z < n_split; z++) { const float mz = pp[(int64_t)z * (V + 2)]; if (mz != -INFINITY) L += pp[(int64_t)z * (V + 2) + 1] * expf(mz - M); }
    const float inv = (sig ? 1.0f : (L > 0.f ? 1.0f / L : 0.f)) * sa_head_gate(a, t, h);
    float *out = a.dst + t * a.dst_stride + (int64_t)h * V;
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
        float o = 0.f;
        for (int z = 0; z < n_split; z++) { const float mz = pp[(int64_t)z * (V + 2)]; if (mz != -INFINITY) o += pp[(int64_t)z * (V + 2) + 2 + j] * expf(mz - M); }
        out[j] = o * inv;
    }
}

// stretches of cells per (token, head) when there are too few pairs to fill the device (decode) and a workspace to merge through
static int sink_attn_splits(const b200_sink_attn_args *a) {
    const int64_t pairs = (int64_t)a->n_tokens * a->n_head;
    // a batch of several sequences fills the device by itself, and its stretches would be unequal; below a few thousand cells a
    // pair's CTA is bound by its fixed costs, not by the cells, and the merge would only add a launch
    if (pairs * 2 > 148 || a->n_kv < 2048) return 1;
    int s = (int)((2 * 148 + pairs - 1) / pairs);
    const int most = a->n_kv / 128;  // at least 128 cells per stretch
    if (s > most) s = most;
    if (s > 64) s = 64;
    return s < 1 ? 1 : s;
}
template <int ND, int NV, int WARPS>
static int launch_sink_attn3(const b200_sink_attn_args *a, float *part, int n_split, cudaStream_t st) {
    const dim3 grid((unsigned)a->n_tokens, (unsigned)a->n_head, (unsigned)n_split);
    const size_t smem = ((size_t)WARPS * a->vdim + 2 * WARPS) * 4;
    sink_attn_kernel<ND, NV, WARPS><<<grid, WARPS * 32, smem, st>>>(*a, part, n_split);
    B200_CUDA_TRY(cudaGetLastError());
    if (n_split > 1) {
        sink_attn_merge_kernel<<<(unsigned)(a->n_tokens * a->n_head), 128, 0, st>>>(*a, part, n_split);
        B200_CUDA_TRY(cudaGetLastError());
    }
    return B200_OK;
}
template <int ND, int NV>
static int launch_sink_attn2(const b200_sink_attn_args *a, float *part, int n_split, cudaStream_t st) {
    if ((int64_t)a->n_tokens * a->n_head < 2 * 148 && a->n_kv > 64) return launch_sink_attn3<ND, NV, 16>(a, part, n_split, st);
    return launch_sink_attn3<ND, NV, 4>(a, part, 1, st);
}
template <int ND>
static int launch_sink_attn(const b200_sink_attn_args *a, float *part, int n_split, cudaStream_t st) {
    const int nv = (a->vdim + 31) / 32;
    if (nv <= 1) return launch_sink_attn2<ND, 1>(a, part, n_split, st);
    if (nv <= 2) return launch_sink_attn2<ND, 2>(a, part, n_split, st);
    if (nv <= 4) return launch_sink_attn2<ND, 4>(a, part, n_split, st);
    return launch_sink_attn2<ND, 8>(a, part, n_split, st);
}

// ------------------------------------------------------------------------------------------------ attention, bf16 products (prompts)
// The tensor cores take both contractions (mma.sync.m16n8k16, bf16 in, f32 accumulators).  One CTA per (GM_TOK consecutive tokens
// of the batch, head), a warp per 16 tokens: its query rows stay in registers as A fragments for the whole pass, the scores of a
// tile of GM_CELLS cells stay in accumulator registers through scale, visibility and the online softmax (all f32), and are
// repacked in place as the A fragments of the second product, so a warp never exchanges anything with another warp.  Keys and
// values of a tile are converted to bf16 on the way into shared memory (free cells are read as zeros: zero weight times whatever
// an unwritten row holds must not reach the sum).  Before a tile is loaded every warp tests its 16 tokens against the tile's 32
// cells (a lane per cell): a tile nobody sees is skipped by the CTA, and a warp whose rows see nothing in it skips the products.
// KS = ceil(dim / 16), VS = ceil(vdim / 16): head sizes are padded with zeros in shared memory, so any size up to 128 runs.
constexpr int GM_TOK = 64, GM_CELLS = 32, GM_WARPS = 4;
__device__ __forceinline__ void gm_ldsm4(unsigned addr, unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void gm_ldsm4_t(unsigned addr, unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void gm_mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned gm_pack_bf2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned *>(&v);
}
// ROWS rows of an f32 matrix -> bf16 rows of `stride` bytes in shared memory: `width` values kept, the rest of the padded row
// (GROUPS groups of 4 values) zero.  row_of(r) gives the source row or nullptr (a row of zeros) and is called by every thread the
// same number of times (it may exchange values within the warp).  All loads of a thread are issued before the first store, so a
// tile costs one trip to L2.
template <int ROWS, int GROUPS, typename RowOf>
__device__ __forceinline__ void gm_stage(unsigned char *dst, int stride, int width, bool vec4, RowOf row_of) {
    constexpr int TOTAL = ROWS * GROUPS, TRIPS = (TOTAL + GM_WARPS * 32 - 1) / (GM_WARPS * 32);
    float4 v[TRIPS];
#pragma unroll
    for (int k = 0; k < TRIPS; k++) {
        const int idx = threadIdx.x + k * GM_WARPS * 32, r = min(idx / GROUPS, ROWS - 1), j = (idx % GROUPS) * 4;
        const float *src = row_of(r);
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (src && idx < TOTAL) {
            if (vec4 && j + 3 < width) v[k] = *reinterpret_cast<const float4 *>(src + j);
            else {
                if (j < width) v[k].x = src[j];
                if (j + 1 < width) v[k].y = src[j + 1];
                if (j + 2 < width) v[k].z = src[j + 2];
                if (j + 3 < width) v[k].w = src[j + 3];
            }
        }
    }
#pragma unroll
    for (int k = 0; k < TRIPS; k++) {
        const int idx = threadIdx.x + k * GM_WARPS * 32, r = idx / GROUPS, j = (idx % GROUPS) * 4;
        if (idx < TOTAL) *reinterpret_cast<uint2 *>(dst + r * stride + j * 2) = make_uint2(gm_pack_bf2(v[k].x, v[k].y), gm_pack_bf2(v[k].z, v[k].w));
    }
}

template <int KS, int VS>
__global__ void __launch_bounds__(GM_WARPS * 32) sink_attn_mma_kernel(const b200_sink_attn_args a) {
    constexpr int QSTRIDE = KS * 32 + 16, VSTRIDE = VS * 32 + 16;  // bytes per bf16 row: 8 consecutive rows start in 8 different 16-byte bank groups
    __shared__ __align__(16) unsigned char qs[GM_TOK * QSTRIDE];
    __shared__ __align__(16) unsigned char ks[GM_CELLS * QSTRIDE];
    __shared__ __align__(16) unsigned char vs[GM_CELLS * VSTRIDE];
    __shared__ int cseq[GM_CELLS], cpos[GM_CELLS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int t0 = blockIdx.x * GM_TOK, h = blockIdx.y;
    const int D = a.dim, V = a.vdim, kvh = h / (a.n_head / a.n_head_kv);
    const float *kb = a.k_cache + (int64_t)kvh * D, *vb = a.v_cache + (int64_t)kvh * V;
    const bool q4 = D % 4 == 0 && a.q_stride % 4 == 0 && ((uintptr_t)a.q & 15) == 0;
    const bool k4 = D % 4 == 0 && a.k_cache_stride % 4 == 0 && ((uintptr_t)a.k_cache & 15) == 0;
    const bool v4 = V % 4 == 0 && a.v_cache_stride % 4 == 0 && ((uintptr_t)a.v_cache & 15) == 0;

    gm_stage<GM_TOK, KS * 4>(qs, QSTRIDE, D, q4, [&](int r) { return t0 + r < a.n_tokens ? a.q + (int64_t)(t0 + r) * a.q_stride + (int64_t)h * D : nullptr; });
    // the warp's 16 tokens: lane i < 16 holds token i (for the tile test); every lane the two rows of its accumulator fragments
    const int wt = t0 + warp * 16;
    int my_seq = -2, my_pos = 0;
    if (lane < 16 && wt + lane < a.n_tokens) { my_seq = a.tok_seq[wt + lane]; my_pos = a.tok_pos[wt + lane]; }
    const int my_lo = sa_chunk_start(my_pos, a.chunk);
    const int rs0 = __shfl_sync(0xffffffffu, my_seq, g), rp0 = __shfl_sync(0xffffffffu, my_pos, g), rl0 = __shfl_sync(0xffffffffu, my_lo, g);
    const int rs1 = __shfl_sync(0xffffffffu, my_seq, g + 8), rp1 = __shfl_sync(0xffffffffu, my_pos, g + 8), rl1 = __shfl_sync(0xffffffffu, my_lo, g + 8);
    __syncthreads();

    const int mi = lane >> 3, mr = lane & 7;
    const unsigned qs_u = (unsigned)__cvta_generic_to_shared(qs), ks_u = (unsigned)__cvta_generic_to_shared(ks), vs_u = (unsigned)__cvta_generic_to_shared(vs);
    const unsigned a_off = (unsigned)(((mi & 1) * 8 + mr) * QSTRIDE + (mi >> 1) * 16);   // A (queries): rows (mi&1)*8.., columns (mi>>1)*8..
    const unsigned k_off = (unsigned)(((mi >> 1) * 8 + mr) * QSTRIDE + (mi & 1) * 16);   // B (keys): cells (mi>>1)*8.., values (mi&1)*8..
    const unsigned v_off = (unsigned)(((mi & 1) * 8 + mr) * VSTRIDE + (mi >> 1) * 16);   // transposed B (values): cells (mi&1)*8.., columns (mi>>1)*8..
    unsigned qa[KS][4];
#pragma unroll
    for (int kk = 0; kk < KS; kk++) gm_ldsm4(qs_u + warp * 16 * QSTRIDE + a_off + kk * 32, qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
    float o[2 * VS][4];
#pragma unroll
    for (int j = 0; j < 2 * VS; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g + 8; l: this lane's share of the row sum
    const bool sig = a.weights == B200_ATTN_SIGMOID;

    for (int c0 = 0; c0 < a.n_kv; c0 += GM_CELLS) {
        // does any of the warp's tokens see any of the tile's cells?  lane = cell
        int cs = -1, cp = 0;
        if (c0 + lane < a.n_kv) { cs = a.cell_seq[c0 + lane]; cp = a.cell_pos[c0 + lane]; }
        bool see = false;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int ts = __shfl_sync(0xffffffffu, my_seq, i), tp = __shfl_sync(0xffffffffu, my_pos, i), tl = __shfl_sync(0xffffffffu, my_lo, i);
            see |= cs >= 0 && sa_visible(cs, cp, ts, tp, a.window, a.keep_first, tl);
        }
        const bool warp_sees = __any_sync(0xffffffffu, see);
        if (!__syncthreads_or(warp_sees)) continue;  // (also: the previous tile has been read by every warp)
        if (warp == 0) { cseq[lane] = cs; cpos[lane] = cp; }
        // lane r of every warp holds cell c0 + r's owner: a row's owner comes by shuffle, not by another load
        gm_stage<GM_CELLS, KS * 4>(ks, QSTRIDE, D, k4, [&](int r) { return __shfl_sync(0xffffffffu, cs, r) >= 0 ? kb + (int64_t)(c0 + r) * a.k_cache_stride : nullptr; });
        gm_stage<GM_CELLS, VS * 4>(vs, VSTRIDE, V, v4, [&](int r) { return __shfl_sync(0xffffffffu, cs, r) >= 0 ? vb + (int64_t)(c0 + r) * a.v_cache_stride : nullptr; });
        __syncthreads();
        if (!warp_sees) continue;
        float s[GM_CELLS / 8][4];
#pragma unroll
        for (int j = 0; j < GM_CELLS / 8; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KS; kk++) {
#pragma unroll
            for (int half = 0; half < GM_CELLS / 16; half++) {
                unsigned b0, b1, b2, b3;
                gm_ldsm4(ks_u + half * 16 * QSTRIDE + k_off + kk * 32, b0, b1, b2, b3);
                gm_mma_bf16(s[2 * half], qa[kk], b0, b1);
                gm_mma_bf16(s[2 * half + 1], qa[kk], b2, b3);
            }
        }
        // scale, visibility, running maximum per row (a row lives in the 4 lanes of a quad)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < GM_CELLS / 8; j++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int c = j * 8 + 2 * t4 + e;
                const int xs = cseq[c], xp = cpos[c];
                s[j][e] = sa_visible(xs, xp, rs0, rp0, a.window, a.keep_first, rl0) ? s[j][e] * a.scale + sa_dist_bias(a, rp0 - xp, h) : -INFINITY;
                s[j][2 + e] = sa_visible(xs, xp, rs1, rp1, a.window, a.keep_first, rl1) ? s[j][2 + e] * a.scale + sa_dist_bias(a, rp1 - xp, h) : -INFINITY;
                mx0 = fmaxf(mx0, s[j][e]); mx1 = fmaxf(mx1, s[j][2 + e]);
            }
        }
        if (sig) {  // every visible key's weight is the sigmoid of its own score (0 for the others: the sigmoid of -inf); nothing is rescaled
            unsigned pa[GM_CELLS / 16][4];
#pragma unroll
            for (int j = 0; j < GM_CELLS / 8; j++) {
                pa[j >> 1][(j & 1) * 2] = gm_pack_bf2(sa_sigmoid_fast(s[j][0]), sa_sigmoid_fast(s[j][1]));
                pa[j >> 1][(j & 1) * 2 + 1] = gm_pack_bf2(sa_sigmoid_fast(s[j][2]), sa_sigmoid_fast(s[j][3]));
            }
#pragma unroll
            for (int kk = 0; kk < GM_CELLS / 16; kk++) {
#pragma unroll
                for (int j = 0; j < VS; j++) {
                    unsigned b0, b1, b2, b3;
                    gm_ldsm4_t(vs_u + kk * 16 * VSTRIDE + v_off + j * 32, b0, b1, b2, b3);
                    gm_mma_bf16(o[2 * j], pa[kk], b0, b1);
                    gm_mma_bf16(o[2 * j + 1], pa[kk], b2, b3);
                }
            }
            continue;
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float al0 = n0 == -INFINITY ? 1.f : expf(m0 - n0), al1 = n1 == -INFINITY ? 1.f : expf(m1 - n1);  // nothing seen yet: keep the zeros
        m0 = n0; m1 = n1;
        float ps0 = 0.f, ps1 = 0.f;
        unsigned pa[GM_CELLS / 16][4];
#pragma unroll
        for (int j = 0; j < GM_CELLS / 8; j++) {
            const float p0 = n0 == -INFINITY ? 0.f : expf(s[j][0] - n0), p1 = n0 == -INFINITY ? 0.f : expf(s[j][1] - n0);
            const float p2 = n1 == -INFINITY ? 0.f : expf(s[j][2] - n1), p3 = n1 == -INFINITY ? 0.f : expf(s[j][3] - n1);
            ps0 += p0 + p1; ps1 += p2 + p3;
            pa[j >> 1][(j & 1) * 2] = gm_pack_bf2(p0, p1);
            pa[j >> 1][(j & 1) * 2 + 1] = gm_pack_bf2(p2, p3);
        }
        l0 = l0 * al0 + ps0; l1 = l1 * al1 + ps1;
        const bool rescale = __any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f);
        if (rescale) {
#pragma unroll
            for (int j = 0; j < 2 * VS; j++) { o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1; }
        }
#pragma unroll
        for (int kk = 0; kk < GM_CELLS / 16; kk++) {
#pragma unroll
            for (int j = 0; j < VS; j++) {
                unsigned b0, b1, b2, b3;
                gm_ldsm4_t(vs_u + kk * 16 * VSTRIDE + v_off + j * 32, b0, b1, b2, b3);
                gm_mma_bf16(o[2 * j], pa[kk], b0, b1);      // columns 16 j .. 16 j + 7
                gm_mma_bf16(o[2 * j + 1], pa[kk], b2, b3);  // columns 16 j + 8 .. 16 j + 15
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float sink = a.sink ? a.sink[h] : -INFINITY;
    float w[2];
    if (sig) {
        w[0] = w[1] = 1.0f;
    } else {
        const float M0 = fmaxf(m0, sink), M1 = fmaxf(m1, sink);
        const float f0 = m0 == -INFINITY ? 0.f : expf(m0 - M0), f1 = m1 == -INFINITY ? 0.f : expf(m1 - M1);
        const float d0 = l0 * f0 + (a.sink ? expf(sink - M0) : 0.f), d1 = l1 * f1 + (a.sink ? expf(sink - M1) : 0.f);
        w[0] = d0 > 0.f ? f0 / d0 : 0.f; w[1] = d1 > 0.f ? f1 / d1 : 0.f;
    }
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        const int t = wt + g + 8 * hh;
        if (t >= a.n_tokens) continue;
        w[hh] *= sa_head_gate(a, t, h);
        float *out = a.dst + (int64_t)t * a.dst_stride + (int64_t)h * V;
#pragma unroll
        for (int j = 0; j < 2 * VS; j++) {
            const int c = 8 * j + 2 * t4;
            if (c < V) out[c] = o[j][2 * hh] * w[hh];
            if (c + 1 < V) out[c + 1] = o[j][2 * hh + 1] * w[hh];
        }
    }
}

template <int KS, int VS>
static int launch_sink_attn_mma2(const b200_sink_attn_args *a, cudaStream_t st) {
    const dim3 grid((unsigned)((a->n_tokens + GM_TOK - 1) / GM_TOK), (unsigned)a->n_head);
    sink_attn_mma_kernel<KS, VS><<<grid, GM_WARPS * 32, 0, st>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
template <int KS>
static int launch_sink_attn_mma1(const b200_sink_attn_args *a, cudaStream_t st) {
    const int vs = (a->vdim + 15) / 16;
    if (vs <= 2) return launch_sink_attn_mma2<KS, 2>(a, st);
    if (vs <= 4) return launch_sink_attn_mma2<KS, 4>(a, st);
    if (vs <= 6) return launch_sink_attn_mma2<KS, 6>(a, st);
    return launch_sink_attn_mma2<KS, 8>(a, st);
}
// bf16 products were asked for, there are enough tokens to fill 16-row tiles, and the head sizes fit the register budget
static bool sink_attn_mma_ok(const b200_sink_attn_args *a) { return a->bf16_products && a->n_tokens >= 16 && a->dim <= 128 && a->vdim <= 128; }
static int launch_sink_attn_mma(const b200_sink_attn_args *a, cudaStream_t st) {
    const int ks = (a->dim + 15) / 16;
    if (ks <= 2) return launch_sink_attn_mma1<2>(a, st);
    if (ks <= 4) return launch_sink_attn_mma1<4>(a, st);
    if (ks <= 6) return launch_sink_attn_mma1<6>(a, st);
    return launch_sink_attn_mma1<8>(a, st);
}

// ------------------------------------------------------------------------------------------------ linear attention with decay
// The columns of the state never interact: a warp owns LA_CW columns of one (sequence, head) and keeps them in registers over
// the whole token loop, a lane the rows d = lane, lane + 32, ...  The inputs of LA_CHUNK tokens are staged in shared memory
// (activation applied once) while the serial loop only does the decayed rank-one update and the column sums.
constexpr int LA_CW = 4, LA_WARPS = 4, LA_COLS = LA_CW * LA_WARPS, LA_CHUNK = 16, LA_RG = 8;
static_assert(LA_RG * LA_CW == 32 && LA_CW == 4, "one partial sum per lane");
__device__ __forceinline__ float la_act(float x, int act) { return act ? x / (1.0f + expf(-x)) : x; }
template <int DPL>
__global__ void __launch_bounds__(LA_WARPS * 32) linear_attn_scan_kernel(const b200_linear_attn_args a) {
    extern __shared__ float sm_[];  // q [LA_CHUNK][32 DPL], k [LA_CHUNK][32 DPL], v [LA_CHUNK][LA_COLS]
    const int h = blockIdx.y, s = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int D = a.dim, V = a.vdim;
    const int first = a.seq_info[s], count = a.seq_info[a.n_seq + s], slot = a.seq_info[2 * a.n_seq + s], fresh = a.seq_info[3 * a.n_seq + s];
    if (count <= 0) return;
    const int cb = blockIdx.x * LA_COLS, col0 = cb + warp * LA_CW;
    float *sq = sm_, *sk = sq + LA_CHUNK * 32 * DPL, *sv = sk + LA_CHUNK * 32 * DPL;  // rows padded to 32 DPL values
    float *Sp = a.state + (int64_t)slot * a.slot_stride + ((int64_t)h * V + col0) * D;
    const float decay = a.decay[h];
    float S[LA_CW][DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < LA_CW; c++) S[c][i] = (!fresh && d < D && col0 + c < V) ? Sp[(int64_t)c * D + d] : 0.f;
    }
    // the inputs of the next chunk travel to registers while the current chunk is worked on: a chunk costs one trip to L2 / HBM that
    // overlaps the serial loop instead of standing in front of it
    constexpr int DP = 32 * DPL, NQ = LA_CHUNK * DP / (LA_WARPS * 32), NVV = LA_CHUNK * LA_COLS / (LA_WARPS * 32);
    float pq[NQ], pk[NQ], pv[NVV];
    auto fetch = [&](int t0) {
        const int nt = min(LA_CHUNK, count - t0);
#pragma unroll
        for (int j = 0; j < NQ; j++) {
            const int idx = tid + j * LA_WARPS * 32, tt = idx / DP, d = idx - tt * DP;
            const bool ok = tt < nt && d < D;
            const int64_t tok = first + t0 + tt;
            pq[j] = ok ? a.q[tok * a.q_stride + (int64_t)h * D + d] : 0.f;
            pk[j] = ok ? a.k[tok * a.k_stride + (int64_t)h * D + d] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < NVV; j++) {
            const int idx = tid + j * LA_WARPS * 32, tt = idx / LA_COLS, c = idx - tt * LA_COLS;
            pv[j] = (tt < nt && cb + c < V) ? a.v[(int64_t)(first + t0 + tt) * a.v_stride + (int64_t)h * V + cb + c] : 0.f;
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < count; t0 += LA_CHUNK) {
        const int nt = min(LA_CHUNK, count - t0);
        __syncthreads();  // the previous chunk has been read
#pragma unroll
        for (int j = 0; j < NQ; j++) { sq[tid + j * LA_WARPS * 32] = la_act(pq[j], a.act); sk[tid + j * LA_WARPS * 32] = la_act(pk[j], a.act); }
#pragma unroll
        for (int j = 0; j < NVV; j++) sv[tid + j * LA_WARPS * 32] = la_act(pv[j], a.act);
        __syncthreads();
        if (t0 + LA_CHUNK < count) fetch(t0 + LA_CHUNK);
        for (int tt0 = 0; tt0 < nt; tt0 += LA_RG) {
            // the row sums do not feed the recurrence: LA_RG tokens x LA_CW columns = 32 partial sums per lane are added up across
            // the warp in one halving exchange (31 shuffles) that leaves sum p in lane p, instead of a full reduction per sum
            float part[LA_RG * LA_CW];
#pragma unroll
            for (int u = 0; u < LA_RG; u++) {
                const int tt = tt0 + u;
                if (tt < nt) {  // warp-uniform
                    float qv[DPL], kv[DPL];
#pragma unroll
                    for (int i = 0; i < DPL; i++) { const int d = lane + 32 * i; qv[i] = sq[tt * DP + d]; kv[i] = sk[tt * DP + d]; }
#pragma unroll
                    for (int c = 0; c < LA_CW; c++) {
                        const float vc = sv[tt * LA_COLS + warp * LA_CW + c];
                        float acc = 0.f;
#pragma unroll
                        for (int i = 0; i < DPL; i++) { S[c][i] = decay * S[c][i] + kv[i] * vc; acc += S[c][i] * qv[i]; }
                        part[u * LA_CW + c] = acc;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < LA_CW; c++) part[u * LA_CW + c] = 0.f;
                }
            }
#pragma unroll
            for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < n / 2; i++) {
                    const float send = upper ? part[i] : part[i + n / 2], keep = upper ? part[i + n / 2] : part[i];
                    part[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            const int tt = tt0 + (lane >> 2), c = lane & 3;  // LA_CW == 4
            if (tt < nt && col0 + c < V) a.dst[(int64_t)(first + t0 + tt) * a.dst_stride + (int64_t)h * V + col0 + c] = part[0];
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < LA_CW; c++) if (d < D && col0 + c < V) Sp[(int64_t)c * D + d] = S[c][i];
    }
}

template <int DPL>
static int launch_linear_attn(const b200_linear_attn_args *a, cudaStream_t st) {
    const dim3 grid((unsigned)((a->vdim + LA_COLS - 1) / LA_COLS), (unsigned)a->heads, (unsigned)a->n_seq);
    const size_t smem = (size_t)LA_CHUNK * (2 * 32 * DPL + LA_COLS) * 4;
    linear_attn_scan_kernel<DPL><<<grid, LA_WARPS * 32, smem, st>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_op_qkv_store(const b200_qkv_store_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q && a->k && a->v && a->pos && a->cells && a->k_cache && a->v_cache && (a->freqs || a->n_dims == 0), B200_ERR_INVALID, "b200_op_qkv_store: NULL argument");
    OPX_REQUIRE(a->n_head > 0 && a->n_head_kv > 0 && a->n_head % a->n_head_kv == 0 && a->dim > 0 && a->vdim > 0 && a->n_dims >= 0 && a->n_dims % 2 == 0 && a->n_dims <= a->dim &&
                a->n_tokens >= 0 && a->k_cache_stride >= (int64_t)a->n_head_kv * a->dim && a->v_cache_stride >= (int64_t)a->n_head_kv * a->vdim, B200_ERR_INVALID,
                "b200_op_qkv_store: bad sizes");
    if (a->n_tokens == 0) return B200_OK;
    // few tokens (decode): a token's row is all the parallelism there is, so its CTA is wide
    const int threads = a->n_tokens <= 64 ? 1024 : 256;
    const size_t smem = a->norm_per_head ? (size_t)(a->n_head + a->n_head_kv) * sizeof(float) : 0;
    OPX_REQUIRE(smem <= 32 * 1024, B200_ERR_UNSUPPORTED, "b200_op_qkv_store: per-head norms over at most 8192 heads");
    qkv_store_kernel<<<(unsigned)a->n_tokens, threads, smem, (cudaStream_t)stream>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" size_t b200_sink_attn_workspace_bytes(const b200_sink_attn_args *a) {
    if (!a || a->n_tokens <= 0 || a->n_head <= 0 || a->vdim <= 0) return 0;
    if (a->bf16_products && a->n_tokens >= 16 && a->dim <= 128 && a->vdim <= 128) return 0;
    const int s = sink_attn_splits(a);
    return s > 1 ? (size_t)a->n_tokens * a->n_head * s * (a->vdim + 2) * sizeof(float) : 0;
}

extern "C" int b200_op_sink_attn(const b200_sink_attn_args *a, b200_stream_t stream) { return b200_op_sink_attn_ws(a, nullptr, 0, stream); }

extern "C" int b200_op_sink_attn_ws(const b200_sink_attn_args *a, void *workspace, size_t workspace_bytes, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q && a->k_cache && a->v_cache && a->cell_seq && a->cell_pos && a->tok_seq && a->tok_pos && a->dst, B200_ERR_INVALID, "b200_op_sink_attn: NULL argument");
    OPX_REQUIRE(a->n_head > 0 && a->n_head <= 65535 && a->n_head_kv > 0 && a->n_head % a->n_head_kv == 0 && a->dim > 0 && a->dim <= 256 && a->vdim > 0 && a->vdim <= 256 &&
                a->n_tokens >= 0 && a->n_kv >= 0 && a->window >= 0 && a->keep_first >= 0 && a->chunk >= 0, B200_ERR_UNSUPPORTED, "b200_op_sink_attn: head sizes up to 256, heads up to 65535");
    OPX_REQUIRE((a->weights == B200_ATTN_SOFTMAX || a->weights == B200_ATTN_SIGMOID) && (!a->dist_bias || a->n_dist > 0), B200_ERR_INVALID, "b200_op_sink_attn: weight kind / distance table");
    if (a->n_tokens == 0) return B200_OK;
    const cudaStream_t st = (cudaStream_t)stream;
    if (sink_attn_mma_ok(a)) return launch_sink_attn_mma(a, st);
    int n_split = sink_attn_splits(a);
    if (n_split > 1 && (!workspace || workspace_bytes < b200_sink_attn_workspace_bytes(a) || ((uintptr_t)workspace & 15))) n_split = 1;  // no room to merge through
    float *part = (float *)workspace;
    const int nd = (a->dim + 31) / 32;
    if (nd <= 1) return launch_sink_attn<1>(a, part, n_split, st);
    if (nd <= 2) return launch_sink_attn<2>(a, part, n_split, st);
    if (nd <= 4) return launch_sink_attn<4>(a, part, n_split, st);
    return launch_sink_attn<8>(a, part, n_split, st);
}

extern "C" int b200_op_linear_attn_scan(const b200_linear_attn_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q && a->k && a->v && a->decay && a->seq_info && a->state && a->dst, B200_ERR_INVALID, "b200_op_linear_attn_scan: NULL argument");
    OPX_REQUIRE(a->heads > 0 && a->heads <= 65535 && a->dim > 0 && a->dim <= 256 && a->vdim > 0 && a->n_seq >= 0 && a->n_seq <= 65535 &&
                a->slot_stride >= (int64_t)a->heads * a->dim * a->vdim, B200_ERR_UNSUPPORTED, "b200_op_linear_attn_scan: dim up to 256");
    if (a->n_seq == 0) return B200_OK;
    const cudaStream_t st = (cudaStream_t)stream;
    const int dpl = (a->dim + 31) / 32;
    if (dpl <= 1) return launch_linear_attn<1>(a, st);
    if (dpl <= 2) return launch_linear_attn<2>(a, st);
    if (dpl <= 4) return launch_linear_attn<4>(a, st);
    return launch_linear_attn<8>(a, st);
}

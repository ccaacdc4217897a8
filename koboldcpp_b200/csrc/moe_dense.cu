// moe_dense.cu -- routed experts over dense (f32 / bf16) weights (include/b200_ggml_ops.h: b200_op_moe_route_grouped,
// b200_op_mul_mat_id_float, b200_op_silu_mul_strided, b200_op_moe_combine).  The quantised expert products live in mmvq.cu /
// mmq.cu; the batched tensor-core product over bf16 experts is the grouped GEMM of mmq.cu with a bf16 producer.
#include "ops_util.cuh"
#include <cuda_bf16.h>

namespace b200 {
using namespace opx;

// ------------------------------------------------------------------------------------------------ router
// (value, index) maximum over the warp; among equal values the lowest index wins
__device__ __forceinline__ void warp_argmax(float &v, int &i) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, off);
        const int oi = __shfl_xor_sync(0xffffffffu, i, off);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

constexpr int RG_WARPS = 4, RG_MAX_PER_LANE = 8;  // 256 experts
// SCORE: enum b200_router_score.  The softmax runs over all experts of the token (maximum and sum across the warp); keep_scores
// leaves the chosen experts' scores as they are instead of dividing them by their sum.
template <int SCORE>
__global__ void __launch_bounds__(RG_WARPS * 32) moe_route_grouped_kernel(const float *__restrict__ logits, int64_t ld_logits, const float *__restrict__ correction,
                                                                          int32_t *__restrict__ ids, int64_t ld_ids, float *__restrict__ w, int64_t ld_w, int n_expert,
                                                                          int n_used, int n_group, int n_group_used, float scale, int keep_scores, int64_t n_tok) {
    const int64_t t = (int64_t)blockIdx.x * RG_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= n_tok) return;
    float s[RG_MAX_PER_LANE], c[RG_MAX_PER_LANE];
    if (SCORE == B200_ROUTER_SOFTMAX) {
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < RG_MAX_PER_LANE; i++) {
            const int e = lane + 32 * i;
            s[i] = e < n_expert ? logits[t * ld_logits + e] : -INFINITY;
            mx = fmaxf(mx, s[i]);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        float den = 0.f;
#pragma unroll
        for (int i = 0; i < RG_MAX_PER_LANE; i++) { s[i] = lane + 32 * i < n_expert ? expf(s[i] - mx) : 0.f; den += s[i]; }
        den = warp_sum(den);
#pragma unroll
        for (int i = 0; i < RG_MAX_PER_LANE; i++) s[i] = s[i] / den;
    }
#pragma unroll
    for (int i = 0; i < RG_MAX_PER_LANE; i++) {
        const int e = lane + 32 * i;
        if (e < n_expert) {
            if (SCORE == B200_ROUTER_SIGMOID) s[i] = 1.0f / (1.0f + expf(-logits[t * ld_logits + e]));
            c[i] = s[i] + (correction ? correction[e] : 0.f);
        } else {
            s[i] = 0.f; c[i] = -INFINITY;
        }
    }
    if (n_group > 1 && n_group_used < n_group) {
        const int per = n_expert / n_group;
        // lane g ends up with the score of group g (n_group <= 32): the sum of the group's two largest choice scores
        float gscore = -INFINITY;
        for (int g = 0; g < n_group; g++) {
            float v1 = -INFINITY; int i1 = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < RG_MAX_PER_LANE; i++) {
                const int e = lane + 32 * i;
                if (e < n_expert && e / per == g && (c[i] > v1 || (c[i] == v1 && e < i1))) { v1 = c[i]; i1 = e; }
            }
            warp_argmax(v1, i1);
            float v2 = -INFINITY; int i2 = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < RG_MAX_PER_LANE; i++) {
                const int e = lane + 32 * i;
                if (e < n_expert && e / per == g && e != i1 && (c[i] > v2 || (c[i] == v2 && e < i2))) { v2 = c[i]; i2 = e; }
            }
            warp_argmax(v2, i2);
            const float sc = per >= 2 ? v1 + v2 : v1;
            if (lane == g) gscore = sc;
        }
        unsigned keep = 0u;
        for (int r = 0; r < n_group_used; r++) {
            float v = (lane < n_group && !((keep >> lane) & 1u)) ? gscore : -INFINITY;
            int gi = (lane < n_group && !((keep >> lane) & 1u)) ? lane : 0x7fffffff;
            // a kept group must not be found again even when every remaining score is -inf: order by (taken, value, index)
            warp_argmax(v, gi);
            if (gi != 0x7fffffff) keep |= 1u << gi;
        }
#pragma unroll
        for (int i = 0; i < RG_MAX_PER_LANE; i++) {
            const int e = lane + 32 * i;
            if (e < n_expert && !((keep >> (e / per)) & 1u)) c[i] = -INFINITY;
        }
    }
    float sum = 0.f, mine_w = 0.f;
    int mine_id = 0;
    unsigned taken = 0u;  // bit i: this lane's expert lane + 32 i has been chosen
    for (int r = 0; r < n_used; r++) {
        float v = -INFINITY; int bi = 0x7fffffff; float bs = 0.f;
#pragma unroll
        for (int i = 0; i < RG_MAX_PER_LANE; i++) {
            const int e = lane + 32 * i;
            if (e < n_expert && !((taken >> i) & 1u) && (bi == 0x7fffffff || c[i] > v)) { v = c[i]; bi = e; bs = s[i]; }
        }
        float rv = v; int ri = bi;
        // lanes without a candidate carry index INT_MAX and lose every comparison among equal values
        warp_argmax(rv, ri);
        // several lanes may hold -inf candidates (experts outside the kept groups): the lowest index wins, as among any equals
        const float ws = __shfl_sync(0xffffffffu, bs, ri & 31);
        if (bi == ri && ri != 0x7fffffff) taken |= 1u << (ri >> 5);
        sum += ws;
        if (lane == r) { mine_id = ri; mine_w = ws; }
    }
    if (lane < n_used) {
        ids[t * ld_ids + lane] = mine_id;
        w[t * ld_w + lane] = keep_scores ? mine_w * scale : mine_w / (sum + 1e-20f) * scale;
    }
}

// ------------------------------------------------------------------------------------------------ expert products, dense weights
__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
// one warp per output element (m, slot, token)
template <typename W>
__global__ void mul_mat_id_float_kernel(TD as, TD b, TD ids, TD dst) {
    const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t M = dst.ne[0], NU = dst.ne[1], T = dst.ne[2];
    if (gw >= M * NU * T) return;
    const int64_t m = gw % M, sl = (gw / M) % NU, t = gw / (M * NU);
    const int e = *(const int32_t *)(ids.data + sl * ids.nb[0] + t * ids.nb[1]);
    if (e < 0 || e >= as.ne[2]) return;
    const W *wr = (const W *)(as.data + m * as.nb[1] + (int64_t)e * as.nb[2]);
    const float *xr = (const float *)(b.data + (sl % b.ne[1]) * b.nb[1] + t * b.nb[2]);
    float s = 0.f;
    for (int64_t k = lane; k < as.ne[0]; k += 32) s += widen(wr[k]) * xr[k];
    s = warp_sum(s);
    if (lane == 0) *(float *)(dst.data + m * dst.nb[0] + sl * dst.nb[1] + t * dst.nb[2]) = s;
}

// Decode over bf16 experts: a warp owns two output rows of one (slot, token) job, 16-byte weight loads that bypass L1, f32
// activations and sums -- the expert form of the dense bf16 GEMV.
__device__ __forceinline__ uint4 mid_ld_stream16(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__global__ void __launch_bounds__(128) gemv_id_bf16_kernel(TD as, TD b, TD ids, TD dst) {
    const int64_t M = dst.ne[0];
    const int64_t m0 = ((int64_t)blockIdx.x * 4 + (threadIdx.x >> 5)) * 2;
    const int lane = threadIdx.x & 31, sl = blockIdx.y, t = blockIdx.z;
    if (m0 >= M) return;
    const int e = *(const int32_t *)(ids.data + sl * ids.nb[0] + t * ids.nb[1]);
    if (e < 0 || e >= as.ne[2]) return;
    const uint4 *w0 = (const uint4 *)(as.data + m0 * as.nb[1] + (int64_t)e * as.nb[2]);
    const uint4 *w1 = (const uint4 *)(as.data + (m0 + 1 < M ? m0 + 1 : m0) * as.nb[1] + (int64_t)e * as.nb[2]);
    const float *xr = (const float *)(b.data + (sl % b.ne[1]) * b.nb[1] + t * b.nb[2]);
    float a0 = 0.f, a1 = 0.f;
    const int64_t nv = as.ne[0] / 8;
#pragma unroll 2
    for (int64_t i = lane; i < nv; i += 32) {
        const uint4 u0 = mid_ld_stream16(w0 + i), u1 = mid_ld_stream16(w1 + i);
        const float4 x0 = reinterpret_cast<const float4 *>(xr + i * 8)[0], x1 = reinterpret_cast<const float4 *>(xr + i * 8)[1];
        const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        const unsigned wa[4] = {u0.x, u0.y, u0.z, u0.w}, wb[4] = {u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            a0 += __uint_as_float(wa[j] << 16) * xs[2 * j] + __uint_as_float(wa[j] & 0xffff0000u) * xs[2 * j + 1];
            a1 += __uint_as_float(wb[j] << 16) * xs[2 * j] + __uint_as_float(wb[j] & 0xffff0000u) * xs[2 * j + 1];
        }
    }
    a0 = warp_sum(a0); a1 = warp_sum(a1);
    if (lane == 0) {
        float *d = (float *)(dst.data + sl * dst.nb[1] + t * dst.nb[2]);
        d[m0] = a0;
        if (m0 + 1 < M) d[m0 + 1] = a1;
    }
}

// enum b200_glu_kind
template <int KIND>
__device__ __forceinline__ float glu_value(float x, float u, float limit, float alpha) {
    if (KIND == B200_GLU_GELU_TANH) return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x))) * u;
    if (KIND == B200_GLU_SWISH_CLAMPED) {
        const float g = fminf(x, limit), c = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-alpha * g)) * (c + 1.0f);
    }
    return x / (1.0f + expf(-x)) * u;
}
template <int KIND>
__global__ void glu_strided_kernel(TD a, TD b, TD sc, bool has_scale, TD dst, int64_t n, float limit, float alpha) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t i0 = i % dst.ne[0], i1 = (i / dst.ne[0]) % dst.ne[1], i2 = (i / (dst.ne[0] * dst.ne[1])) % dst.ne[2], i3 = i / (dst.ne[0] * dst.ne[1] * dst.ne[2]);
    float x = *(const float *)(a.data + i0 * a.nb[0] + i1 * a.nb[1] + i2 * a.nb[2] + i3 * a.nb[3]);
    float u = *(const float *)(b.data + i0 * b.nb[0] + i1 * b.nb[1] + i2 * b.nb[2] + i3 * b.nb[3]);
    if (has_scale) {  // the two products are linear in their input: a factor on the input is a factor on both
        const float f = *(const float *)(sc.data + i1 * sc.nb[0] + i2 * sc.nb[1]);
        x *= f; u *= f;
    }
    *(float *)(dst.data + i0 * dst.nb[0] + i1 * dst.nb[1] + i2 * dst.nb[2] + i3 * dst.nb[3]) = glu_value<KIND>(x, u, limit, alpha);
}

__global__ void moe_combine_kernel(const float *__restrict__ y, int64_t y_s_slot, int64_t y_s_tok, const float *__restrict__ w, int64_t w_s_tok,
                                   const float *__restrict__ add0, int64_t add0_stride, const float *__restrict__ add1, int64_t add1_stride, float *__restrict__ dst,
                                   int64_t dst_stride, int64_t n, int n_used, int64_t total) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t t = idx / n, i = idx - t * n;
    float s = 0.f;
    for (int k = 0; k < n_used; k++) s += w[t * w_s_tok + k] * y[t * y_s_tok + k * y_s_slot + i];
    if (add1) s += add1[t * add1_stride + i];  // the two sublayers first, then the residual stream
    if (add0) s += add0[t * add0_stride + i];
    dst[t * dst_stride + i] = s;
}

// The chosen experts' results (weights optional), a shared expert's result times the sigmoid of its per-token gate logit, the other
// sublayer's result; their sum times the residual multiplier joins the stream.  VEC values per thread (4: 16-byte loads and stores).
template <int VEC>
__global__ void moe_combine_shared_kernel(const float *__restrict__ y, int64_t y_s_slot, int64_t y_s_tok, const float *__restrict__ w, int64_t w_s_tok,
                                          const float *__restrict__ add0, int64_t add0_stride, const float *__restrict__ add1, int64_t add1_stride,
                                          const float *__restrict__ shared, int64_t shared_stride, const float *__restrict__ gate, int64_t gate_stride, float mult,
                                          float *__restrict__ dst, int64_t dst_stride, int64_t n, int n_used, int64_t total) {
    const int64_t idx = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (idx >= total) return;
    const int64_t t = idx / n, i = idx - t * n;
    float s[VEC];
    auto load = [&](const float *p, float (&v)[VEC]) {
        if (VEC == 4) { const float4 q = *reinterpret_cast<const float4 *>(p); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
        else v[0] = *p;
    };
#pragma unroll
    for (int e = 0; e < VEC; e++) s[e] = 0.f;
    for (int k = 0; k < n_used; k++) {
        float v[VEC];
        load(y + t * y_s_tok + k * y_s_slot + i, v);
        const float wk = w ? w[t * w_s_tok + k] : 1.0f;
#pragma unroll
        for (int e = 0; e < VEC; e++) s[e] += wk * v[e];
    }
    if (shared) {
        float v[VEC];
        load(shared + t * shared_stride + i, v);
        const float gs = gate ? sigmoidf_(gate[t * gate_stride]) : 1.0f;
#pragma unroll
        for (int e = 0; e < VEC; e++) s[e] += gs * v[e];
    }
    if (add1) {
        float v[VEC];
        load(add1 + t * add1_stride + i, v);
#pragma unroll
        for (int e = 0; e < VEC; e++) s[e] += v[e];
    }
#pragma unroll
    for (int e = 0; e < VEC; e++) s[e] *= mult;
    if (add0) {
        float v[VEC];
        load(add0 + t * add0_stride + i, v);
#pragma unroll
        for (int e = 0; e < VEC; e++) s[e] += v[e];
    }
    if (VEC == 4) *reinterpret_cast<float4 *>(dst + t * dst_stride + i) = make_float4(s[0], s[1], s[2], s[3]);
    else dst[t * dst_stride + i] = s[0];
}

// The weighted sum of a token's expert results, an RMS norm over it with a weight, and the residual stream, one CTA per token.
// The summed row stays in registers (VPT values per thread) between the statistics and the output, and every load of a thread
// -- expert rows, norm weight, residual -- is issued before the block-wide sum, so a token costs one trip to memory.
template <int VPT>
__global__ void __launch_bounds__(1024) moe_combine_norm_kernel(const float *__restrict__ y, int64_t y_s_slot, int64_t y_s_tok, const float *__restrict__ w, int64_t w_s_tok,
                                                                const float *__restrict__ nw, float eps, const float *__restrict__ res, int64_t res_stride,
                                                                float *__restrict__ dst, int64_t dst_stride, int n, int n_used) {
    __shared__ float sh[32], sw[32];
    const int64_t t = blockIdx.x;
    if ((int)threadIdx.x < n_used) sw[threadIdx.x] = w[t * w_s_tok + threadIdx.x];
    __syncthreads();
    float v[VPT], wv[VPT], rv[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = 0.f;
        wv[k] = (nw && i < n) ? nw[i] : 1.f;
        rv[k] = (res && i < n) ? res[t * res_stride + i] : 0.f;
    }
    for (int kk = 0; kk < n_used; kk++) {
        const float wk = sw[kk];
        const float *yk = y + t * y_s_tok + kk * y_s_slot;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n) v[k] += wk * yk[i];
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; k++) ss += v[k] * v[k];
    const float scale = 1.0f / sqrtf(block_sum(ss, sh) / (float)n + eps);
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n) dst[t * dst_stride + i] = v[k] * scale * wv[k] + rv[k];
    }
}

static unsigned grid1d(int64_t n, int block) { return (unsigned)((n + block - 1) / block); }

}  // namespace b200

using namespace b200;
using namespace b200::opx;

extern "C" int b200_op_moe_route_grouped(const float *logits, int64_t ld_logits, const float *correction, int32_t *ids, int64_t ld_ids, float *w, int64_t ld_w,
                                         int32_t n_expert, int32_t n_used, int32_t n_group, int32_t n_group_used, float scale, int64_t n_tok, b200_stream_t stream) {
    return b200_op_moe_route_scored(logits, ld_logits, correction, ids, ld_ids, w, ld_w, n_expert, n_used, n_group, n_group_used, scale, B200_ROUTER_SIGMOID, 0, n_tok, stream);
}

extern "C" int b200_op_moe_route_scored(const float *logits, int64_t ld_logits, const float *correction, int32_t *ids, int64_t ld_ids, float *w, int64_t ld_w,
                                        int32_t n_expert, int32_t n_used, int32_t n_group, int32_t n_group_used, float scale, int32_t score, int32_t keep_scores,
                                        int64_t n_tok, b200_stream_t stream) {
    OPX_REQUIRE(logits && ids && w, B200_ERR_INVALID, "b200_op_moe_route_grouped: NULL argument");
    OPX_REQUIRE(score == B200_ROUTER_SIGMOID || score == B200_ROUTER_SOFTMAX, B200_ERR_INVALID, "b200_op_moe_route_scored: unknown score function %d", score);
    OPX_REQUIRE(n_expert > 0 && n_expert <= 32 * RG_MAX_PER_LANE && n_used > 0 && n_used <= 32 && n_used <= n_expert && n_tok >= 0, B200_ERR_UNSUPPORTED,
                "b200_op_moe_route_grouped: at most 256 experts, 32 per token");
    if (n_group < 1) n_group = 1;
    OPX_REQUIRE(n_group <= 32 && n_expert % n_group == 0 && n_group_used >= 1 && n_group_used <= n_group && (int64_t)n_group_used * (n_expert / n_group) >= n_used, B200_ERR_INVALID,
                "b200_op_moe_route_grouped: %d groups (%d kept) do not fit %d experts, %d per token", n_group, n_group_used, n_expert, n_used);
    if (n_tok == 0) return B200_OK;
    if (score == B200_ROUTER_SOFTMAX)
        moe_route_grouped_kernel<B200_ROUTER_SOFTMAX><<<grid1d(n_tok, RG_WARPS), RG_WARPS * 32, 0, (cudaStream_t)stream>>>(logits, ld_logits, correction, ids, ld_ids, w, ld_w, n_expert,
                                                                                                                          n_used, n_group, n_group_used, scale, keep_scores, n_tok);
    else
        moe_route_grouped_kernel<B200_ROUTER_SIGMOID><<<grid1d(n_tok, RG_WARPS), RG_WARPS * 32, 0, (cudaStream_t)stream>>>(logits, ld_logits, correction, ids, ld_ids, w, ld_w, n_expert,
                                                                                                                          n_used, n_group, n_group_used, scale, keep_scores, n_tok);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_mul_mat_id_float(const b200_tensor *as, const b200_tensor *b, const b200_tensor *ids, const b200_tensor *dst, b200_stream_t stream) {
    OPX_REQUIRE(as && b && ids && dst && as->data && b->data && ids->data && dst->data, B200_ERR_INVALID, "b200_op_mul_mat_id_float: NULL argument");
    OPX_REQUIRE((as->type == B200_TYPE_F32 || as->type == B200_TYPE_BF16) && b->type == B200_TYPE_F32 && ids->type == B200_TYPE_I32 && dst->type == B200_TYPE_F32, B200_ERR_UNSUPPORTED,
                "b200_op_mul_mat_id_float: f32 / bf16 experts, f32 activations, i32 ids");
    OPX_REQUIRE(as->nb[0] == (size_t)type_block_bytes(as->type) && b->nb[0] == 4 && as->ne[3] == 1 && b->ne[3] == 1, B200_ERR_UNSUPPORTED, "b200_op_mul_mat_id_float: rows must be contiguous");
    OPX_REQUIRE(as->ne[0] == b->ne[0] && dst->ne[0] == as->ne[1] && dst->ne[1] == ids->ne[0] && dst->ne[2] == ids->ne[1] && b->ne[2] == ids->ne[1] && b->ne[1] >= 1, B200_ERR_INVALID,
                "b200_op_mul_mat_id_float: shape mismatch");
    const int64_t total = dst->ne[0] * dst->ne[1] * dst->ne[2];
    if (total == 0) return B200_OK;
    const cudaStream_t st = (cudaStream_t)stream;
    if (as->type == B200_TYPE_BF16 && dst->ne[1] * dst->ne[2] <= 64 && dst->ne[1] <= 65535 && dst->ne[2] <= 65535 && as->ne[0] % 8 == 0 && dst->nb[0] == 4 &&
        (((uintptr_t)as->data | as->nb[1] | as->nb[2] | (uintptr_t)b->data | b->nb[1] | b->nb[2]) & 15) == 0) {
        const dim3 grid((unsigned)((dst->ne[0] + 7) / 8), (unsigned)dst->ne[1], (unsigned)dst->ne[2]);
        gemv_id_bf16_kernel<<<grid, 128, 0, st>>>(td(as), td(b), td(ids), td(dst));
    } else if (as->type == B200_TYPE_F32) {
        mul_mat_id_float_kernel<float><<<grid1d(total * 32, 256), 256, 0, st>>>(td(as), td(b), td(ids), td(dst));
    } else {
        mul_mat_id_float_kernel<__nv_bfloat16><<<grid1d(total * 32, 256), 256, 0, st>>>(td(as), td(b), td(ids), td(dst));
    }
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_silu_mul_strided(const b200_tensor *a, const b200_tensor *b, const b200_tensor *dst, b200_stream_t stream) {
    return b200_op_glu_strided(B200_GLU_SILU, a, b, dst, 0.0f, 0.0f, stream);
}

extern "C" int b200_op_glu_strided(int kind, const b200_tensor *a, const b200_tensor *b, const b200_tensor *dst, float limit, float alpha, b200_stream_t stream) {
    return b200_op_glu_scaled(kind, a, b, nullptr, dst, limit, alpha, stream);
}

extern "C" int b200_op_glu_scaled(int kind, const b200_tensor *a, const b200_tensor *b, const b200_tensor *scale, const b200_tensor *dst, float limit, float alpha,
                                  b200_stream_t stream) {
    OPX_REQUIRE(a && b && dst && a->data && b->data && dst->data, B200_ERR_INVALID, "b200_op_glu_strided: NULL argument");
    OPX_REQUIRE(!scale || (scale->data && scale->type == B200_TYPE_F32 && scale->ne[0] == dst->ne[1] && scale->ne[1] == dst->ne[2] && dst->ne[3] == 1), B200_ERR_INVALID,
                "b200_op_glu_scaled: the scale is one f32 value per (i1, i2)");
    const TD tsc = scale ? td(scale) : td(dst);
    OPX_REQUIRE(a->type == B200_TYPE_F32 && b->type == B200_TYPE_F32 && dst->type == B200_TYPE_F32 && same_shape(a, dst) && same_shape(b, dst), B200_ERR_UNSUPPORTED,
                "b200_op_glu_strided: f32 tensors of one shape only");
    OPX_REQUIRE(kind == B200_GLU_SILU || kind == B200_GLU_GELU_TANH || kind == B200_GLU_SWISH_CLAMPED, B200_ERR_INVALID, "b200_op_glu_strided: unknown kind %d", kind);
    const int64_t n = nelements(dst);
    if (n == 0) return B200_OK;
    const cudaStream_t st = (cudaStream_t)stream;
    if (kind == B200_GLU_GELU_TANH) glu_strided_kernel<B200_GLU_GELU_TANH><<<grid1d(n, 256), 256, 0, st>>>(td(a), td(b), tsc, scale != nullptr, td(dst), n, limit, alpha);
    else if (kind == B200_GLU_SWISH_CLAMPED) glu_strided_kernel<B200_GLU_SWISH_CLAMPED><<<grid1d(n, 256), 256, 0, st>>>(td(a), td(b), tsc, scale != nullptr, td(dst), n, limit, alpha);
    else glu_strided_kernel<B200_GLU_SILU><<<grid1d(n, 256), 256, 0, st>>>(td(a), td(b), tsc, scale != nullptr, td(dst), n, limit, alpha);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_moe_combine_norm(const float *y, int64_t y_s_slot, int64_t y_s_tok, const float *w, int64_t w_s_tok, const float *norm_w, float eps, const float *res,
                                        int64_t res_stride, float *dst, int64_t dst_stride, int64_t n, int32_t n_used, int64_t n_tok, b200_stream_t stream) {
    OPX_REQUIRE(y && w && dst && n >= 0 && n <= B200_MOE_COMBINE_NORM_MAX && n_used > 0 && n_tok >= 0, B200_ERR_INVALID, "b200_op_moe_combine_norm: bad argument (rows of at most %d values)",
                B200_MOE_COMBINE_NORM_MAX);
    if (n == 0 || n_tok == 0) return B200_OK;
    OPX_REQUIRE(n_used <= 32, B200_ERR_UNSUPPORTED, "b200_op_moe_combine_norm: at most 32 experts per token");
    const int rb = n <= 512 ? 128 : n <= 1024 ? 256 : n <= 2048 ? 512 : 1024, vpt = (int)((n + rb - 1) / rb);
#define B200_MCN(V) moe_combine_norm_kernel<V><<<(unsigned)n_tok, rb, 0, (cudaStream_t)stream>>>(y, y_s_slot, y_s_tok, w, w_s_tok, norm_w, eps, res, res_stride, dst, dst_stride, (int)n, n_used)
    if (vpt <= 4) B200_MCN(4); else if (vpt <= 8) B200_MCN(8); else B200_MCN(16);
#undef B200_MCN
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_moe_combine(const float *y, int64_t y_s_slot, int64_t y_s_tok, const float *w, int64_t w_s_tok, const float *add0, int64_t add0_stride,
                                   const float *add1, int64_t add1_stride, float *dst, int64_t dst_stride, int64_t n, int32_t n_used, int64_t n_tok, b200_stream_t stream) {
    OPX_REQUIRE(y && w && dst && n >= 0 && n_used > 0 && n_tok >= 0, B200_ERR_INVALID, "b200_op_moe_combine: bad argument");
    const int64_t total = n * n_tok;
    if (total == 0) return B200_OK;
    moe_combine_kernel<<<grid1d(total, 256), 256, 0, (cudaStream_t)stream>>>(y, y_s_slot, y_s_tok, w, w_s_tok, add0, add0_stride, add1, add1_stride, dst, dst_stride, n, n_used, total);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_moe_combine_shared(const float *y, int64_t y_s_slot, int64_t y_s_tok, const float *w, int64_t w_s_tok, const float *add0, int64_t add0_stride,
                                          const float *add1, int64_t add1_stride, const float *shared, int64_t shared_stride, const float *gate, int64_t gate_stride,
                                          float mult, float *dst, int64_t dst_stride, int64_t n, int32_t n_used, int64_t n_tok, b200_stream_t stream) {
    OPX_REQUIRE(dst && n >= 0 && n_used >= 0 && n_tok >= 0 && (y || n_used == 0), B200_ERR_INVALID, "b200_op_moe_combine_shared: bad argument");
    const int64_t total = n * n_tok;
    if (total == 0) return B200_OK;
    // 16-byte accesses when every row of every operand starts on a 16-byte boundary
    auto al = [](const float *p, int64_t stride) { return !p || ((((uintptr_t)p) & 15) == 0 && stride % 4 == 0); };
    const bool vec = n % 4 == 0 && al(y, y_s_slot) && y_s_tok % 4 == 0 && al(add0, add0_stride) && al(add1, add1_stride) && al(shared, shared_stride) && al(dst, dst_stride);
    if (vec)
        moe_combine_shared_kernel<4><<<grid1d(total / 4, 256), 256, 0, (cudaStream_t)stream>>>(y, y_s_slot, y_s_tok, w, w_s_tok, add0, add0_stride, add1, add1_stride, shared,
                                                                                          shared_stride, gate, gate_stride, mult, dst, dst_stride, n, n_used, total);
    else
        moe_combine_shared_kernel<1><<<grid1d(total, 256), 256, 0, (cudaStream_t)stream>>>(y, y_s_slot, y_s_tok, w, w_s_tok, add0, add0_stride, add1, add1_stride, shared,
                                                                                      shared_stride, gate, gate_stride, mult, dst, dst_stride, n, n_used, total);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

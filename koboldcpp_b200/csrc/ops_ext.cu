// ops_ext.cu -- row and elementwise ops beyond the llama / mixtral graph (include/b200_ggml_ops.h, "Ops beyond ..."): a norm
// with an optional sigmoid gate in front and a residual behind, PolyNorm, rotation by a frequency table, a weighted sum over
// stacked activations, and a * sigmoid(b) over strided views.  All f32, one pass over HBM per op (rows stay in L1 / L2 between
// the statistics pass and the output pass).
#include "ops_util.cuh"

namespace b200 {
using namespace opx;

// ------------------------------------------------------------------------------------------------ norm (+ gate, + residual)
template <int KIND, bool GATE>
__global__ void norm_kernel(TD x, const float *__restrict__ w, int64_t w_period, const float *__restrict__ bias, TD gate, const float *__restrict__ gate_bias,
                            int gate_out, TD res, bool has_res, TD dst, float eps) {
    __shared__ float sh[32];
    extern __shared__ float rowbuf[];  // the gated row (GATE only)
    const int64_t r = blockIdx.x;
    const float *xr = (const float *)row_ptr(x, r);
    float *yr = (float *)row_ptr(dst, r);
    const float *gr = GATE ? (const float *)row_ptr(gate, r) : nullptr;
    const float *rr = has_res ? (const float *)row_ptr(res, r) : nullptr;
    const float *wr = w ? w + (r % w_period) * x.ne[0] : nullptr;
    const int n = (int)x.ne[0];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = xr[i];
        if (GATE && !gate_out) {
            v *= sigmoidf_(gr[i] + (gate_bias ? gate_bias[i] : 0.f));
            rowbuf[i] = v;
        }
        s += KIND == B200_NORM_RMS ? v * v : v;
    }
    if (GATE) __syncthreads();
    const float *src = (GATE && !gate_out) ? rowbuf : xr;
    float mean = 0.f, var;
    if (KIND == B200_NORM_RMS) {
        var = block_sum(s, sh) / (float)n;
    } else {
        mean = block_sum(s, sh) / (float)n;
        float q = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) { const float d = src[i] - mean; q += d * d; }
        var = block_sum(q, sh) / (float)n;
    }
    const float scale = 1.0f / sqrtf(var + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = (src[i] - mean) * scale;
        if (wr) v *= wr[i];
        if (bias) v += bias[i];
        if (GATE && gate_out) { const float z = gr[i] + (gate_bias ? gate_bias[i] : 0.f); v *= gate_out == 2 ? z * sigmoidf_(z) : sigmoidf_(z); }
        if (rr) v += rr[i];
        yr[i] = v;
    }
}

// ------------------------------------------------------------------------------------------------ PolyNorm
__global__ void polynorm_kernel(TD x, const float *__restrict__ coef, TD dst, float eps) {
    __shared__ float sh[32];
    const int64_t r = blockIdx.x;
    const float *xr = (const float *)row_ptr(x, r);
    float *yr = (float *)row_ptr(dst, r);
    const int n = (int)x.ne[0];
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float z = xr[i], z2 = z * z, z3 = z2 * z;
        s2 += z2; s4 += z2 * z2; s6 += z3 * z3;
    }
    s2 = block_sum(s2, sh); s4 = block_sum(s4, sh); s6 = block_sum(s6, sh);
    const float inv = 1.0f / (float)n;
    const float r1 = coef[0] / sqrtf(s2 * inv + eps), r2 = coef[1] / sqrtf(s4 * inv + eps), r3 = coef[2] / sqrtf(s6 * inv + eps), c3 = coef[3];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float z = xr[i], z2 = z * z;
        yr[i] = r1 * z + r2 * z2 + r3 * (z2 * z) + c3;
    }
}


// Rows of up to blockDim * VPT values stay in registers: every load of the row (and of its gate) is issued before the first
// reduction, so a row costs one memory latency for the statistics and one for the weight / residual, whatever its length.
template <int KIND, bool GATE, int VPT>
__global__ void __launch_bounds__(1024) norm_reg_kernel(TD x, const float *__restrict__ w, int64_t w_period, const float *__restrict__ bias, TD gate,
                                                        const float *__restrict__ gate_bias, int gate_out, TD res, bool has_res, TD dst, float eps) {
    __shared__ float sh[32];
    const int64_t r = blockIdx.x;
    const float *xr = (const float *)row_ptr(x, r);
    float *yr = (float *)row_ptr(dst, r);
    const float *gr = GATE ? (const float *)row_ptr(gate, r) : nullptr;
    const float *rr = has_res ? (const float *)row_ptr(res, r) : nullptr;
    const float *wr = w ? w + (r % w_period) * x.ne[0] : nullptr;
    const int n = (int)x.ne[0];
    float v[VPT], g[VPT], wv[VPT], rv[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = i < n ? xr[i] : 0.f;
        if (GATE) g[k] = i < n ? gr[i] + (gate_bias ? gate_bias[i] : 0.f) : 0.f;
        wv[k] = (wr && i < n) ? wr[i] : 1.f;
        rv[k] = (rr && i < n) ? rr[i] : 0.f;
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        if (GATE && !gate_out) v[k] *= sigmoidf_(g[k]);
        s += KIND == B200_NORM_RMS ? v[k] * v[k] : v[k];
    }
    float mean = 0.f, var;
    if (KIND == B200_NORM_RMS) {
        var = block_sum(s, sh) / (float)n;
    } else {
        mean = block_sum(s, sh) / (float)n;
        float q = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; k++) { const float d = threadIdx.x + k * blockDim.x < n ? v[k] - mean : 0.f; q += d * d; }
        var = block_sum(q, sh) / (float)n;
    }
    const float scale = 1.0f / sqrtf(var + eps);
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n) {
            float y = (v[k] - mean) * scale * wv[k];
            if (bias) y += bias[i];
            if (GATE && gate_out) y *= gate_out == 2 ? g[k] * sigmoidf_(g[k]) : sigmoidf_(g[k]);
            yr[i] = y + rv[k];
        }
    }
}

template <int VPT>
__global__ void __launch_bounds__(1024) polynorm_reg_kernel(TD x, const float *__restrict__ coef, TD dst, float eps) {
    __shared__ float sh[32];
    const int64_t r = blockIdx.x;
    const float *xr = (const float *)row_ptr(x, r);
    float *yr = (float *)row_ptr(dst, r);
    const int n = (int)x.ne[0];
    float z[VPT], s2 = 0.f, s4 = 0.f, s6 = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; k++) { const int i = threadIdx.x + k * blockDim.x; z[k] = i < n ? xr[i] : 0.f; }
#pragma unroll
    for (int k = 0; k < VPT; k++) { const float z2 = z[k] * z[k], z3 = z2 * z[k]; s2 += z2; s4 += z2 * z2; s6 += z3 * z3; }
    s2 = block_sum(s2, sh); s4 = block_sum(s4, sh); s6 = block_sum(s6, sh);
    const float inv = 1.0f / (float)n;
    const float r1 = coef[0] / sqrtf(s2 * inv + eps), r2 = coef[1] / sqrtf(s4 * inv + eps), r3 = coef[2] / sqrtf(s6 * inv + eps), c3 = coef[3];
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        const float z2 = z[k] * z[k];
        if (i < n) yr[i] = r1 * z[k] + r2 * z2 + r3 * (z2 * z[k]) + c3;
    }
}

// ------------------------------------------------------------------------------------------------ rotation by a table
__global__ void rope_table_kernel(TD x, const int32_t *__restrict__ pos, const float *__restrict__ freqs, TD dst, int n_dims, int neox, float mscale,
                                  int64_t total) {
    // one thread per pair of the rotated part, or per element of the pass-through part
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int half = n_dims / 2;
    const int64_t per_row = half + (x.ne[0] - n_dims);
    const int64_t row = idx / per_row;
    const int j = (int)(idx % per_row);
    const int64_t i1 = row % x.ne[1], i2 = row / x.ne[1];
    const float *xr = (const float *)(x.data + i1 * x.nb[1] + i2 * x.nb[2]);
    float *yr = (float *)(dst.data + i1 * dst.nb[1] + i2 * dst.nb[2]);
    if (j >= half) {
        const int e = n_dims + (j - half);
        const float v = xr[e];
        yr[e] = v;
        return;
    }
    const int a = neox ? j : 2 * j, b = neox ? j + half : 2 * j + 1;
    const float ang = (float)pos[i2] * freqs[j];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    sn *= mscale; cs *= mscale;
    const float u = xr[a], v = xr[b];
    yr[a] = u * cs - v * sn;
    yr[b] = v * cs + u * sn;
}

// ------------------------------------------------------------------------------------------------ weighted sum of slices
__global__ void weighted_sum_kernel(const float *__restrict__ xs, int64_t slice_stride, int n_slices, const float *__restrict__ w, float *__restrict__ dst,
                                    int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.f;
    for (int j = 0; j < n_slices; j++) s += w[j] * xs[(int64_t)j * slice_stride + i];
    dst[i] = s;
}

__global__ void sigmoid_mul_kernel(TD a, TD b, TD dst, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t i0 = i % dst.ne[0], i1 = (i / dst.ne[0]) % dst.ne[1], i2 = (i / (dst.ne[0] * dst.ne[1])) % dst.ne[2], i3 = i / (dst.ne[0] * dst.ne[1] * dst.ne[2]);
    const float x = *(const float *)(a.data + i0 * a.nb[0] + i1 * a.nb[1] + i2 * a.nb[2] + i3 * a.nb[3]);
    const float g = *(const float *)(b.data + i0 * b.nb[0] + i1 * b.nb[1] + i2 * b.nb[2] + i3 * b.nb[3]);
    *(float *)(dst.data + i0 * dst.nb[0] + i1 * dst.nb[1] + i2 * dst.nb[2] + i3 * dst.nb[3]) = x * sigmoidf_(g);
}

static unsigned grid1d(int64_t n, int block) { return (unsigned)((n + block - 1) / block); }

// two rows, each divided by its own root mean square and multiplied by its own weight, added: both rows wait in registers, the two
// sums of squares share the block-wide exchange
template <int VPT>
__global__ void __launch_bounds__(1024) norm_pair_kernel(TD x1, const float *__restrict__ w1, const float *__restrict__ b1, TD x2, const float *__restrict__ w2, TD dst, float eps) {
    __shared__ float sh[32];
    const int64_t r = blockIdx.x;
    const float *p1 = (const float *)row_ptr(x1, r), *p2 = (const float *)row_ptr(x2, r);
    float *yr = (float *)row_ptr(dst, r);
    const int n = (int)x1.ne[0];
    float u[VPT], v[VPT], a[VPT], c[VPT], s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        u[k] = i < n ? p1[i] + (b1 ? b1[i] : 0.f) : 0.f;
        v[k] = i < n ? p2[i] : 0.f;
        a[k] = i < n ? w1[i] : 0.f;
        c[k] = i < n ? w2[i] : 0.f;
        s1 += u[k] * u[k]; s2 += v[k] * v[k];
    }
    s1 = block_sum(s1, sh); s2 = block_sum(s2, sh);
    const float f1 = 1.0f / sqrtf(s1 / (float)n + eps), f2 = 1.0f / sqrtf(s2 / (float)n + eps);
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n) yr[i] = u[k] * f1 * a[k] + v[k] * f2 * c[k];
    }
}

// position vector of sines and cosines added to every row: a thread per pair (2i, 2i + 1), the angle pos * f_i in f32
__global__ void add_sinusoid_kernel(TD x, const int32_t *__restrict__ pos, const float *__restrict__ freqs, TD dst, int64_t pairs, int64_t total) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t t = idx / pairs, i = idx - t * pairs;
    const float *xr = (const float *)(x.data + t * x.nb[1]);
    float *yr = (float *)(dst.data + t * dst.nb[1]);
    float sn, cs;
    sincosf((float)pos[t] * freqs[i], &sn, &cs);
    yr[2 * i] = xr[2 * i] + sn;
    if (2 * i + 1 < x.ne[0]) yr[2 * i + 1] = xr[2 * i + 1] + cs;
}

}  // namespace b200

using namespace b200;
using namespace b200::opx;

extern "C" int b200_op_norm_pair(const b200_tensor *x1, const float *w1, const float *b1, const b200_tensor *x2, const float *w2, const b200_tensor *dst, float eps,
                                 b200_stream_t stream) {
    OPX_REQUIRE(x1 && x2 && dst && w1 && w2 && x1->data && x2->data && dst->data, B200_ERR_INVALID, "b200_op_norm_pair: NULL argument");
    OPX_REQUIRE(x1->type == B200_TYPE_F32 && x2->type == B200_TYPE_F32 && dst->type == B200_TYPE_F32 && x1->nb[0] == 4 && x2->nb[0] == 4 && dst->nb[0] == 4 && same_shape(x1, dst) &&
                same_shape(x2, dst) && x1->ne[0] <= 16384, B200_ERR_UNSUPPORTED, "b200_op_norm_pair: f32 rows of one shape, at most 16384 values each");
    const int64_t rows = nrows(dst);
    if (rows == 0 || dst->ne[0] == 0) return B200_OK;
    const int n = (int)dst->ne[0];
    const int rb = n <= 256 ? 64 : n <= 1024 ? 128 : n <= 2048 ? 256 : n <= 4096 ? 512 : 1024, vpt = (n + rb - 1) / rb;
#define B200_NP(V) norm_pair_kernel<V><<<(unsigned)rows, rb, 0, (cudaStream_t)stream>>>(td(x1), w1, b1, td(x2), w2, td(dst), eps)
    if (vpt <= 4) B200_NP(4); else if (vpt <= 8) B200_NP(8); else B200_NP(16);
#undef B200_NP
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_add_sinusoid(const b200_tensor *x, const int32_t *pos, const float *freqs, const b200_tensor *dst, b200_stream_t stream) {
    OPX_REQUIRE(x && dst && pos && freqs && x->data && dst->data, B200_ERR_INVALID, "b200_op_add_sinusoid: NULL argument");
    OPX_REQUIRE(x->type == B200_TYPE_F32 && dst->type == B200_TYPE_F32 && x->nb[0] == 4 && dst->nb[0] == 4 && same_shape(x, dst) && x->ne[2] == 1 && x->ne[3] == 1, B200_ERR_UNSUPPORTED,
                "b200_op_add_sinusoid: f32 [n, tokens] rows only");
    const int64_t pairs = (x->ne[0] + 1) / 2, total = pairs * x->ne[1];
    if (total == 0) return B200_OK;
    add_sinusoid_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(td(x), pos, freqs, td(dst), pairs, total);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_norm(const b200_tensor *x, const float *w, int64_t w_period, const b200_tensor *gate, const float *gate_bias, const b200_tensor *res,
                            const b200_tensor *dst, float eps, int kind, b200_stream_t stream) {
    return b200_op_norm_affine(x, w, w_period, nullptr, gate, gate_bias, 0, res, dst, eps, kind, stream);
}

extern "C" int b200_op_norm_affine(const b200_tensor *x, const float *w, int64_t w_period, const float *bias, const b200_tensor *gate, const float *gate_bias,
                                   int gate_on_output, const b200_tensor *res, const b200_tensor *dst, float eps, int kind, b200_stream_t stream) {
    const int gate_out = gate ? gate_on_output : 0;  // 0: in front of the norm; 1: sigmoid on the output; 2: silu on the output
    OPX_REQUIRE(gate_out >= 0 && gate_out <= 2, B200_ERR_INVALID, "b200_op_norm: unknown gate placement %d", gate_on_output);
    OPX_REQUIRE(x && dst && x->data && dst->data, B200_ERR_INVALID, "b200_op_norm: NULL argument");
    OPX_REQUIRE(x->type == B200_TYPE_F32 && dst->type == B200_TYPE_F32 && x->nb[0] == 4 && dst->nb[0] == 4 && same_shape(x, dst), B200_ERR_UNSUPPORTED,
                "b200_op_norm: f32 rows of one shape only");
    OPX_REQUIRE(kind == B200_NORM_LAYER || kind == B200_NORM_RMS, B200_ERR_INVALID, "b200_op_norm: unknown kind %d", kind);
    OPX_REQUIRE(!gate || (gate->data && gate->type == B200_TYPE_F32 && gate->nb[0] == 4 && same_shape(gate, x)), B200_ERR_INVALID, "b200_op_norm: gate shape");
    OPX_REQUIRE(!res || (res->data && res->type == B200_TYPE_F32 && res->nb[0] == 4 && same_shape(res, x)), B200_ERR_INVALID, "b200_op_norm: residual shape");
    OPX_REQUIRE(!gate || x->ne[0] * 4 <= 160 * 1024, B200_ERR_UNSUPPORTED, "b200_op_norm: gated rows longer than 40960 values");
    const int64_t rows = nrows(x);
    if (rows == 0 || x->ne[0] == 0) return B200_OK;
    if (w_period < 1) w_period = 1;
    const int block = x->ne[0] >= 4096 ? 512 : (x->ne[0] >= 1024 ? 256 : 128);
    const cudaStream_t st = (cudaStream_t)stream;
    TD tg = gate ? td(gate) : td(x), tr = res ? td(res) : td(x);
    if (x->ne[0] <= 16384) {  // the row fits the registers of one block
        const int n = (int)x->ne[0];
        const int rb = n <= 256 ? 64 : n <= 1024 ? 128 : n <= 2048 ? 256 : n <= 4096 ? 512 : 1024;
#define B200_NORM_REG(K, G, V) norm_reg_kernel<K, G, V><<<(unsigned)rows, rb, 0, st>>>(td(x), w, w_period, bias, tg, gate_bias, gate_out, tr, res != nullptr, td(dst), eps)
#define B200_NORM_REG_V(K, G) do { if ((n + rb - 1) / rb <= 4) B200_NORM_REG(K, G, 4); else if ((n + rb - 1) / rb <= 8) B200_NORM_REG(K, G, 8); else B200_NORM_REG(K, G, 16); } while (0)
        if (kind == B200_NORM_RMS) { if (gate) B200_NORM_REG_V(B200_NORM_RMS, true); else B200_NORM_REG_V(B200_NORM_RMS, false); }
        else { if (gate) B200_NORM_REG_V(B200_NORM_LAYER, true); else B200_NORM_REG_V(B200_NORM_LAYER, false); }
#undef B200_NORM_REG_V
#undef B200_NORM_REG
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    const size_t smem = gate && !gate_out ? (size_t)x->ne[0] * 4 : 0;
#define B200_NORM_LAUNCH(K, G)                                                                                                                   \
    do {                                                                                                                                         \
        if (smem > 48 * 1024) B200_CUDA_TRY(cudaFuncSetAttribute(norm_kernel<K, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
        norm_kernel<K, G><<<(unsigned)rows, block, smem, st>>>(td(x), w, w_period, bias, tg, gate_bias, gate_out, tr, res != nullptr, td(dst), eps);             \
    } while (0)
    if (kind == B200_NORM_RMS) { if (gate) B200_NORM_LAUNCH(B200_NORM_RMS, true); else B200_NORM_LAUNCH(B200_NORM_RMS, false); }
    else { if (gate) B200_NORM_LAUNCH(B200_NORM_LAYER, true); else B200_NORM_LAUNCH(B200_NORM_LAYER, false); }
#undef B200_NORM_LAUNCH
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_polynorm(const b200_tensor *x, const float *coef, const b200_tensor *dst, float eps, b200_stream_t stream) {
    OPX_REQUIRE(x && dst && coef && x->data && dst->data, B200_ERR_INVALID, "b200_op_polynorm: NULL argument");
    OPX_REQUIRE(x->type == B200_TYPE_F32 && dst->type == B200_TYPE_F32 && x->nb[0] == 4 && dst->nb[0] == 4 && same_shape(x, dst), B200_ERR_UNSUPPORTED,
                "b200_op_polynorm: f32 rows of one shape only");
    const int64_t rows = nrows(x);
    if (rows == 0 || x->ne[0] == 0) return B200_OK;
    if (x->ne[0] <= 16384) {
        const int n = (int)x->ne[0];
        const int rb = n <= 256 ? 64 : n <= 1024 ? 128 : n <= 2048 ? 256 : n <= 4096 ? 512 : 1024;
        const int vpt = (n + rb - 1) / rb;
        if (vpt <= 4) polynorm_reg_kernel<4><<<(unsigned)rows, rb, 0, (cudaStream_t)stream>>>(td(x), coef, td(dst), eps);
        else if (vpt <= 8) polynorm_reg_kernel<8><<<(unsigned)rows, rb, 0, (cudaStream_t)stream>>>(td(x), coef, td(dst), eps);
        else polynorm_reg_kernel<16><<<(unsigned)rows, rb, 0, (cudaStream_t)stream>>>(td(x), coef, td(dst), eps);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    const int block = x->ne[0] >= 4096 ? 512 : (x->ne[0] >= 1024 ? 256 : 128);
    polynorm_kernel<<<(unsigned)rows, block, 0, (cudaStream_t)stream>>>(td(x), coef, td(dst), eps);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_rope_table(const b200_tensor *x, const int32_t *pos, const float *freqs, const b200_tensor *dst, int32_t n_dims, int32_t neox,
                                  float mscale, b200_stream_t stream) {
    OPX_REQUIRE(x && dst && pos && freqs && x->data && dst->data, B200_ERR_INVALID, "b200_op_rope_table: NULL argument");
    OPX_REQUIRE(x->type == B200_TYPE_F32 && dst->type == B200_TYPE_F32 && x->nb[0] == 4 && dst->nb[0] == 4 && same_shape(x, dst) && x->ne[3] == 1,
                B200_ERR_UNSUPPORTED, "b200_op_rope_table: f32 [ne0, heads, tokens] only");
    OPX_REQUIRE(n_dims >= 0 && n_dims % 2 == 0 && n_dims <= x->ne[0], B200_ERR_INVALID, "b200_op_rope_table: n_dims %d does not fit rows of %lld", n_dims, (long long)x->ne[0]);
    const int64_t per_row = n_dims / 2 + (x->ne[0] - n_dims);
    const int64_t total = per_row * x->ne[1] * x->ne[2];
    if (total == 0) return B200_OK;
    rope_table_kernel<<<grid1d(total, 256), 256, 0, (cudaStream_t)stream>>>(td(x), pos, freqs, td(dst), n_dims, neox, mscale, total);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_weighted_sum(const float *xs, int64_t slice_stride, int32_t n_slices, const float *w, float *dst, int64_t n, b200_stream_t stream) {
    OPX_REQUIRE(xs && w && dst && n_slices > 0 && n >= 0, B200_ERR_INVALID, "b200_op_weighted_sum: bad argument");
    if (n == 0) return B200_OK;
    weighted_sum_kernel<<<grid1d(n, 256), 256, 0, (cudaStream_t)stream>>>(xs, slice_stride, n_slices, w, dst, n);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_sigmoid_mul(const b200_tensor *a, const b200_tensor *b, const b200_tensor *dst, b200_stream_t stream) {
    OPX_REQUIRE(a && b && dst && a->data && b->data && dst->data, B200_ERR_INVALID, "b200_op_sigmoid_mul: NULL argument");
    OPX_REQUIRE(a->type == B200_TYPE_F32 && b->type == B200_TYPE_F32 && dst->type == B200_TYPE_F32 && same_shape(a, dst) && same_shape(b, dst), B200_ERR_UNSUPPORTED,
                "b200_op_sigmoid_mul: f32 tensors of one shape only");
    const int64_t n = nelements(dst);
    if (n == 0) return B200_OK;
    sigmoid_mul_kernel<<<grid1d(n, 256), 256, 0, (cudaStream_t)stream>>>(td(a), td(b), td(dst), n);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

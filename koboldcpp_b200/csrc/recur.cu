// recur.cu -- mixers that carry a fixed-size state per sequence instead of a cache row per token (include/b200_ggml_ops.h:
// b200_op_short_conv, b200_op_delta_rule_scan, b200_op_mingru_scan).  A batch names its sequences through seq_info (first token,
// token count, state slot, fresh); a fresh sequence starts from zeros whatever its slot held before.  Everything is f32.
#include "ops_util.cuh"

namespace b200 {
using namespace opx;

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
// ln(1 + e^x) without overflow for large x and without cancellation for very negative x
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// ------------------------------------------------------------------------------------------------ short causal convolution
// A thread per channel, a CTA per (128 channels, SC_TOK tokens of one sequence).  Input i of a sequence's portion is x[first + i]
// (+ bias) for i >= 0 and the tail's entry taps - 1 + i before that; only the CTA of the portion's first tokens reads the tail, and
// it alone rewrites it afterwards (thread = channel, so nobody else touches the same values): the new tail is the last taps - 1
// inputs, which are old tail entries shifted down where the portion is shorter than the tail.
// KMAX >= taps is the compile-time window: the weights are padded with zeros in front, the SC_TOK + KMAX - 1 inputs of the CTA's
// tokens travel to registers with all loads in flight at once, and every output is KMAX multiply-adds on registers.  KMAX == 0 is
// the general form for longer filters (every input read where it is used).
constexpr int SC_TOK = 16, SC_MAX_TAPS = SC_TOK + 1;
template <int KMAX>
__global__ void __launch_bounds__(128) short_conv_kernel(const b200_short_conv_args a) {
    const int c = blockIdx.x * 128 + threadIdx.x, s = blockIdx.z;
    const int first = a.seq_info[s], count = a.seq_info[a.n_seq + s], slot = a.seq_info[2 * a.n_seq + s], fresh = a.seq_info[3 * a.n_seq + s];
    const int t0 = blockIdx.y * SC_TOK;
    if (c >= a.channels || t0 >= count) return;
    const int taps = a.taps, nt = min(SC_TOK, count - t0);
    const float bias = a.bias ? a.bias[c] : 0.f;
    float *tail = a.tail + (int64_t)slot * a.slot_stride + c;  // entry j at tail[j * channels]
    const float *w = a.w + (int64_t)c * taps;
    auto input = [&](int i) -> float {
        if (i >= 0) return a.x[(int64_t)(first + i) * a.x_stride + c] + bias;
        return (fresh || i < -(taps - 1)) ? 0.f : tail[(int64_t)(taps - 1 + i) * a.channels];
    };
    if (KMAX > 0) {
        float wp[KMAX > 0 ? KMAX : 1], win[SC_TOK + (KMAX > 0 ? KMAX : 1) - 1];
#pragma unroll
        for (int j = 0; j < KMAX; j++) wp[j] = j >= KMAX - taps ? w[j - (KMAX - taps)] : 0.f;
#pragma unroll
        for (int i = 0; i < SC_TOK + KMAX - 1; i++) win[i] = i - (KMAX - 1) < nt ? input(t0 + i - (KMAX - 1)) : 0.f;  // win[i] = input t0 + i - (KMAX - 1)
#pragma unroll
        for (int t = 0; t < SC_TOK; t++) {
            float y = 0.f;
#pragma unroll
            for (int j = 0; j < KMAX; j++) y += wp[j] * win[t + j];
            if (t < nt) a.dst[(int64_t)(first + t0 + t) * a.dst_stride + c] = a.act ? silu_f(y) : y;
        }
    } else {
        for (int t = t0; t < t0 + nt; t++) {
            float y = 0.f;
            for (int j = 0; j < taps; j++) y += w[j] * input(t - taps + 1 + j);
            a.dst[(int64_t)(first + t) * a.dst_stride + c] = a.act ? silu_f(y) : y;
        }
    }
    if (t0 == 0) {
        // entry j of the new tail is input count - (taps - 1) + j: an old entry of higher index, or a value of x; ascending j never
        // reads what it has written
        for (int j = 0; j < taps - 1; j++) tail[(int64_t)j * a.channels] = input(count - (taps - 1) + j);
    }
}

// ------------------------------------------------------------------------------------------------ gated delta rule
// The columns of the state never interact: column j of S [dim, vdim] sees  S_j <- g S_j + k u_j  with  u_j = beta (v_j - g k.S_j),
// and the read-out is  o_j = q.S_j(new) = g q.S_j(old) + (q.k) u_j,  so one pass over the old column gives both sums a token
// needs.  A warp owns DR_CW * DR_CPL columns of one (sequence, head); 8 lanes share DR_CPL columns, lane r of them keeping the rows
// 4 (r + 8 i) .. + 3 of each in registers over the whole token loop, so a sum over a column is three exchanges among 8 lanes and
// the q and k values a lane reads from shared memory serve DR_CPL columns (the loads, not the arithmetic, are what two CTAs on one
// SM compete for).
// The inputs of DR_CHUNK tokens are staged in shared memory: q and k as unit vectors (q scaled), q.k, the decay and beta once per
// token; the next chunk's values travel to registers while the current chunk is worked on.
constexpr int DR_CW = 4, DR_CPL = 1, DR_WARPS = 8, DR_COLS = DR_CW * DR_CPL * DR_WARPS, DR_CHUNK = 16, DR_TPW = DR_CHUNK / DR_WARPS;
template <int DQ>  // float4 groups per lane: dim <= 32 DQ
__global__ void __launch_bounds__(DR_WARPS * 32) delta_rule_scan_kernel(const b200_delta_rule_args a) {
    constexpr int DP = 32 * DQ;
    __shared__ __align__(16) float sq[DR_CHUNK][DP], sk[DR_CHUNK][DP];
    __shared__ float sv[DR_CHUNK][DR_COLS], sqk[DR_CHUNK], sg[DR_CHUNK], sbeta[DR_CHUNK];
    const int h = blockIdx.y, s = blockIdx.z, kvh = h / (a.heads / a.kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int D = a.dim, V = a.vdim;
    const int first = a.seq_info[s], count = a.seq_info[a.n_seq + s], slot = a.seq_info[2 * a.n_seq + s], fresh = a.seq_info[3 * a.n_seq + s];
    if (count <= 0) return;
    const int cb = blockIdx.x * DR_COLS, cw = lane >> 3, r = lane & 7, lc0 = warp * DR_CW * DR_CPL + cw;  // the lane's columns: cb + lc0 + DR_CW c
    float *Sp = a.state + (int64_t)slot * a.slot_stride + ((int64_t)h * V + cb + lc0) * D;                // column c at Sp + DR_CW c D
    float S[DR_CPL][DQ][4];
#pragma unroll
    for (int c = 0; c < DR_CPL; c++)
#pragma unroll
        for (int i = 0; i < DQ; i++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int d = 4 * (r + 8 * i) + e;
                S[c][i][e] = (!fresh && d < D && cb + lc0 + DR_CW * c < V) ? Sp[(int64_t)DR_CW * c * D + d] : 0.f;
            }
    const float decay_rate = expf(a.a_log[h]), dtb = a.dt_bias ? a.dt_bias[h] : 0.f;
    // staging: the raw values of a chunk travel to registers (every thread a slice of the chunk), are parked in shared memory, and
    // warp w then turns the tokens w, w + DR_WARPS, ... into unit vectors in place
    constexpr int NQ = DR_CHUNK * DP / (DR_WARPS * 32), NVV = (DR_CHUNK * DR_COLS) / (DR_WARPS * 32);
    float pq[NQ], pk[NQ], pv[NVV], pa = 0.f, pb = 0.f;
    auto fetch = [&](int t0) {
        const int nt = min(DR_CHUNK, count - t0);
#pragma unroll
        for (int j = 0; j < NQ; j++) {
            const int idx = tid + j * DR_WARPS * 32, tt = idx / DP, d = idx - tt * DP;
            const bool ok = tt < nt && d < D;
            const int64_t tok = first + t0 + tt;
            pq[j] = ok ? a.q[tok * a.q_stride + (int64_t)kvh * D + d] : 0.f;
            pk[j] = ok ? a.k[tok * a.k_stride + (int64_t)kvh * D + d] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < NVV; j++) {
            const int idx = tid + j * DR_WARPS * 32, tt = idx / DR_COLS, c = idx - tt * DR_COLS;
            pv[j] = (tt < nt && cb + c < V) ? a.v[(int64_t)(first + t0 + tt) * a.v_stride + (int64_t)h * V + cb + c] : 0.f;
        }
        if (tid < DR_CHUNK) {
            pa = tid < nt ? a.a[(int64_t)(first + t0 + tid) * a.a_stride + h] : 0.f;
            pb = tid < nt ? a.b[(int64_t)(first + t0 + tid) * a.b_stride + h] : 0.f;
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < count; t0 += DR_CHUNK) {
        const int nt = min(DR_CHUNK, count - t0);
        __syncthreads();  // the previous chunk has been read
#pragma unroll
        for (int j = 0; j < NQ; j++) { (&sq[0][0])[tid + j * DR_WARPS * 32] = pq[j]; (&sk[0][0])[tid + j * DR_WARPS * 32] = pk[j]; }
#pragma unroll
        for (int j = 0; j < NVV; j++) (&sv[0][0])[tid + j * DR_WARPS * 32] = pv[j];
        if (tid < DR_CHUNK) {
            sg[tid] = expf(-decay_rate * softplus_f(pa + dtb));
            sbeta[tid] = sigmoidf_(pb);
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < DR_TPW; u++) {
            const int tt = warp + u * DR_WARPS;
            float qv[DQ], kv[DQ], qq = 0.f, kk = 0.f, qk = 0.f;
#pragma unroll
            for (int j = 0; j < DQ; j++) {
                qv[j] = sq[tt][lane + 32 * j]; kv[j] = sk[tt][lane + 32 * j];
                qq += qv[j] * qv[j]; kk += kv[j] * kv[j];
            }
            qq = warp_sum(qq); kk = warp_sum(kk);
            const float fq = (a.unit_qk ? 1.0f / sqrtf(qq + a.unit_eps) : 1.0f) * a.q_scale, fk = a.unit_qk ? 1.0f / sqrtf(kk + a.unit_eps) : 1.0f;
#pragma unroll
            for (int j = 0; j < DQ; j++) {
                qv[j] *= fq; kv[j] *= fk;
                qk += qv[j] * kv[j];
                sq[tt][lane + 32 * j] = qv[j]; sk[tt][lane + 32 * j] = kv[j];
            }
            qk = warp_sum(qk);
            if (lane == 0) sqk[tt] = qk;
        }
        __syncthreads();
        if (t0 + DR_CHUNK < count) fetch(t0 + DR_CHUNK);
        // unrolled so that the shared-memory loads of the following tokens are issued ahead of the chain S -> sums -> u -> S
#pragma unroll 4
        for (int tt = 0; tt < nt; tt++) {
            float ks[DR_CPL], qs[DR_CPL];
            float4 kv[DQ];
#pragma unroll
            for (int c = 0; c < DR_CPL; c++) ks[c] = qs[c] = 0.f;
#pragma unroll
            for (int i = 0; i < DQ; i++) {
                kv[i] = *reinterpret_cast<const float4 *>(&sk[tt][4 * (r + 8 * i)]);
                const float4 qv = *reinterpret_cast<const float4 *>(&sq[tt][4 * (r + 8 * i)]);
#pragma unroll
                for (int c = 0; c < DR_CPL; c++) {
                    ks[c] += (kv[i].x * S[c][i][0] + kv[i].z * S[c][i][2]) + (kv[i].y * S[c][i][1] + kv[i].w * S[c][i][3]);
                    qs[c] += (qv.x * S[c][i][0] + qv.z * S[c][i][2]) + (qv.y * S[c][i][1] + qv.w * S[c][i][3]);
                }
            }
#pragma unroll
            for (int off = 4; off >= 1; off >>= 1)
#pragma unroll
                for (int c = 0; c < DR_CPL; c++) { ks[c] += __shfl_xor_sync(0xffffffffu, ks[c], off); qs[c] += __shfl_xor_sync(0xffffffffu, qs[c], off); }
            const float g = sg[tt];
#pragma unroll
            for (int c = 0; c < DR_CPL; c++) {
                const float u = sbeta[tt] * (sv[tt][lc0 + DR_CW * c] - g * ks[c]);
#pragma unroll
                for (int i = 0; i < DQ; i++) {
                    S[c][i][0] = g * S[c][i][0] + kv[i].x * u; S[c][i][1] = g * S[c][i][1] + kv[i].y * u;
                    S[c][i][2] = g * S[c][i][2] + kv[i].z * u; S[c][i][3] = g * S[c][i][3] + kv[i].w * u;
                }
                if (r == 0 && cb + lc0 + DR_CW * c < V) a.dst[(int64_t)(first + t0 + tt) * a.dst_stride + (int64_t)h * V + cb + lc0 + DR_CW * c] = g * qs[c] + sqk[tt] * u;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < DR_CPL; c++)
#pragma unroll
        for (int i = 0; i < DQ; i++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int d = 4 * (r + 8 * i) + e;
                if (d < D && cb + lc0 + DR_CW * c < V) Sp[(int64_t)DR_CW * c * D + d] = S[c][i][e];
            }
}

template <int DQ>
static int launch_delta_rule(const b200_delta_rule_args *a, cudaStream_t st) {
    const dim3 grid((unsigned)((a->vdim + DR_COLS - 1) / DR_COLS), (unsigned)a->heads, (unsigned)a->n_seq);
    delta_rule_scan_kernel<DQ><<<grid, DR_WARPS * 32, 0, st>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ minGRU
// S_t = (1 - z_t) S_(t-1) + z_t c_t is linear in S, so a stretch of tokens acts on the state as S -> A S + B.  A CTA takes 32
// channels of one sequence (a warp row reads 128 contiguous bytes of a token) and blockDim.y stretches of MG_TPT tokens at a time:
// every thread loads its stretch with all loads in flight, turns the pre-activations into gates once, finds its (A, B), reads the
// state in front of its stretch off the earlier stretches' (A, B) in shared memory, and runs its tokens again from registers to
// write the outputs.  With few tokens (decoding) the launch has one stretch per CTA and the middle step is empty.
constexpr int MG_TPT = 8, MG_SEG_MAX = 32;
__global__ void __launch_bounds__(32 * MG_SEG_MAX) mingru_scan_kernel(const b200_mingru_args a) {
    __shared__ float sA[MG_SEG_MAX][32], sB[MG_SEG_MAX][32], sS[32];
    const int lane = threadIdx.x, seg = threadIdx.y, n_seg = blockDim.y, c = blockIdx.x * 32 + lane, s = blockIdx.y;
    const int first = a.seq_info[s], count = a.seq_info[a.n_seq + s], slot = a.seq_info[2 * a.n_seq + s], fresh = a.seq_info[3 * a.n_seq + s];
    if (count <= 0) return;
    const bool live = c < a.width;
    const float zb = (a.z_bias && live) ? a.z_bias[c] : 0.f, xb = (a.x_bias && live) ? a.x_bias[c] : 0.f;
    float *Sp = a.state + (int64_t)slot * a.slot_stride + c;
    if (seg == 0) sS[lane] = (live && !fresh) ? *Sp : 0.f;
    for (int base = 0; base < count; base += n_seg * MG_TPT) {
        const int t_lo = base + seg * MG_TPT;
        float z[MG_TPT], cand[MG_TPT], g[MG_TPT];
#pragma unroll
        for (int u = 0; u < MG_TPT; u++) {
            const bool ok = live && t_lo + u < count;
            const int64_t tok = first + t_lo + u;
            z[u] = ok ? a.z[tok * a.z_stride + c] : 0.f;
            cand[u] = ok ? a.x[tok * a.x_stride + c] : 0.f;
            g[u] = (ok && a.g) ? a.g[tok * a.g_stride + c] : 0.f;
        }
        float A = 1.f, B = 0.f;
#pragma unroll
        for (int u = 0; u < MG_TPT; u++) {
            const bool ok = t_lo + u < count;
            const float zz = ok ? sigmoidf_(z[u] + zb) : 0.f, uu = cand[u] + xb;  // a token beyond the end leaves the state as it is
            z[u] = zz; cand[u] = uu >= 0.f ? uu + 0.5f : sigmoidf_(uu);
            A *= 1.f - zz; B = (1.f - zz) * B + zz * cand[u];
        }
        sA[seg][lane] = A; sB[seg][lane] = B;
        __syncthreads();  // (also: sS holds the state in front of these stretches)
        float S = sS[lane];
        for (int j = 0; j < seg; j++) S = sA[j][lane] * S + sB[j][lane];
#pragma unroll
        for (int u = 0; u < MG_TPT; u++) {
            S = (1.f - z[u]) * S + z[u] * cand[u];
            if (live && t_lo + u < count) a.dst[(int64_t)(first + t_lo + u) * a.dst_stride + c] = a.g ? S * silu_f(g[u]) : S;
        }
        __syncthreads();  // everybody has read sS, sA, sB
        if (seg == n_seg - 1) sS[lane] = S;
    }
    __syncthreads();
    if (seg == 0 && live) *Sp = sS[lane];
}

}  // namespace b200

using namespace b200;

extern "C" int b200_op_short_conv(const b200_short_conv_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->x && a->w && a->seq_info && a->dst && (a->tail || a->taps <= 1), B200_ERR_INVALID, "b200_op_short_conv: NULL argument");
    OPX_REQUIRE(a->channels > 0 && a->taps >= 1 && a->taps <= SC_MAX_TAPS && a->n_seq >= 0 && a->n_seq <= 65535 && a->n_tokens >= 0 &&
                (a->taps <= 1 || a->slot_stride >= (int64_t)(a->taps - 1) * a->channels), B200_ERR_UNSUPPORTED, "b200_op_short_conv: at most %d taps", SC_MAX_TAPS);
    OPX_REQUIRE(a->x != a->dst, B200_ERR_INVALID, "b200_op_short_conv: not in place");
    if (a->n_seq == 0 || a->n_tokens == 0) return B200_OK;
    const dim3 grid((unsigned)((a->channels + 127) / 128), (unsigned)((a->n_tokens + SC_TOK - 1) / SC_TOK), (unsigned)a->n_seq);
    OPX_REQUIRE(grid.y <= 65535, B200_ERR_UNSUPPORTED, "b200_op_short_conv: at most %d tokens in a batch", 65535 * SC_TOK);
    if (a->taps <= 4) short_conv_kernel<4><<<grid, 128, 0, (cudaStream_t)stream>>>(*a);
    else if (a->taps <= 8) short_conv_kernel<8><<<grid, 128, 0, (cudaStream_t)stream>>>(*a);
    else short_conv_kernel<0><<<grid, 128, 0, (cudaStream_t)stream>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_delta_rule_scan(const b200_delta_rule_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q && a->k && a->v && a->a && a->b && a->a_log && a->seq_info && a->state && a->dst, B200_ERR_INVALID, "b200_op_delta_rule_scan: NULL argument");
    OPX_REQUIRE(a->heads > 0 && a->heads <= 65535 && a->kv_heads > 0 && a->heads % a->kv_heads == 0 && a->dim > 0 && a->dim <= 256 && a->vdim > 0 && a->n_seq >= 0 &&
                a->n_seq <= 65535 && a->slot_stride >= (int64_t)a->heads * a->dim * a->vdim, B200_ERR_UNSUPPORTED, "b200_op_delta_rule_scan: dim up to 256");
    if (a->n_seq == 0) return B200_OK;
    const cudaStream_t st = (cudaStream_t)stream;
    const int dq = (a->dim + 31) / 32;
    if (dq <= 1) return launch_delta_rule<1>(a, st);
    if (dq <= 2) return launch_delta_rule<2>(a, st);
    if (dq <= 4) return launch_delta_rule<4>(a, st);
    return launch_delta_rule<8>(a, st);
}

extern "C" int b200_op_mingru_scan(const b200_mingru_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->z && a->x && a->seq_info && a->state && a->dst, B200_ERR_INVALID, "b200_op_mingru_scan: NULL argument");
    OPX_REQUIRE(a->width > 0 && a->n_seq >= 0 && a->n_seq <= 65535 && a->slot_stride >= a->width, B200_ERR_INVALID, "b200_op_mingru_scan: bad sizes");
    if (a->n_seq == 0) return B200_OK;
    const dim3 grid((unsigned)((a->width + 31) / 32), (unsigned)a->n_seq);
    // stretches per CTA: as many as the longest sequence of the batch can fill (a sequence has at most n_tokens tokens)
    int segs = (a->n_tokens + MG_TPT - 1) / MG_TPT;
    segs = a->n_tokens <= 0 ? MG_SEG_MAX : segs < 1 ? 1 : segs > MG_SEG_MAX ? MG_SEG_MAX : segs;
    mingru_scan_kernel<<<grid, dim3(32, (unsigned)segs), 0, (cudaStream_t)stream>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

// The generalized delta rule: a recurrent mixer whose state per request and head is a matrix
// S [key channel, value channel] in 32-bit,
//
//     S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T,     o_t = S_t^T r_t,
//
// with a decay w_t and a removal rate a_t per key channel, and u_t = k_t / sqrt(|k_t|^2 + eps)
// the unit key.  Both terms read the old state.  A column of S (one value channel) never meets
// another column: s <- w * s - (a * u) (u . s) + k v_c, o_c = s . r.
//
// Layout: a column is spread over LANES neighbouring lanes of a warp, each with EPL = 16 of
// its elements in registers (the key size D is padded to LANES * 16; the padding stays zero).
// Lane l owns the float4 units l, l + LANES, l + 2 LANES, ... of the column, so that the lanes
// of a column read consecutive 16-byte words of shared memory.  A CTA of 256 threads owns
// 256 / LANES columns of one (row, head) and walks the row's tokens in chunks: the chunk's
// r, k, w, a are staged in shared memory (all 256 threads load, the unit key is formed there,
// a * u is stored beside u), then every thread runs the chunk's tokens.  Per token the only
// chain is (partial dot of 16 products) -> log2(LANES) shuffles -> one multiply-add per
// element; the read-out s . r is kept as a partial sum per token and summed across the lanes
// after the chunk, off the chain.  Rows of one token (decode steps) take the same path with a
// chunk of one.
//
// state: float32 [slots, H, V, DP] with DP = the padded key size; a fresh slot holds zeros.
// Compiled once per key size (-DSLLM_HEAD_DIM=D).
#include "common.cuh"

#ifndef SLLM_HEAD_DIM
#define SLLM_HEAD_DIM 64
#endif

namespace sllm {

constexpr int D = SLLM_HEAD_DIM;
constexpr int EPL = 16;                       // elements of a column per lane
constexpr int lanes_for(int d) {
    int l = 1;
    while (l * EPL < d) l *= 2;
    return l;
}
constexpr int LANES = lanes_for(D);
static_assert(LANES <= 32, "key sizes up to 512");
constexpr int DP = LANES * EPL;               // padded key size
constexpr int THREADS = 256;
constexpr int COLS = THREADS / LANES;         // columns of S per CTA
constexpr int UNITS = EPL / 4;                // float4 units per lane
// tokens per chunk: five vectors of DP floats per token, within 40 KB
constexpr int CHUNK = (40 * 1024 / (5 * DP * 4)) >= 16 ? 16 : (40 * 1024 / (5 * DP * 4));
static_assert(CHUNK >= 2, "chunk too small");

// rkv: [N, ld] with the heads' r at column r0, k at k0, v at v0 (each heads x D or heads x V);
// wa: float32 [N, ldwa] with the decays at column 0 and the removal rates at column H * D.
template <typename T>
__global__ void __launch_bounds__(THREADS)
general_delta_kernel(const T* __restrict__ rkv, int64_t ld, int r0, int k0, int v0,
                     const float* __restrict__ wa, int64_t ldwa, float* __restrict__ state,
                     const int* __restrict__ row_start, const int* __restrict__ row_slot,
                     float* __restrict__ out, int H, int V, float unit_eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ __align__(16) float sr[CHUNK][DP], sk[CHUNK][DP], sw[CHUNK][DP], su[CHUNK][DP],
        sau[CHUNK][DP];
    __shared__ float sv[CHUNK][COLS];
    __shared__ float sinv[CHUNK];
    const int row = blockIdx.z, head = blockIdx.y;
    const int t0 = row_start[row], n_new = row_start[row + 1] - t0;
    if (n_new <= 0) return;
    const int tid = threadIdx.x, lane_in_col = tid % LANES;
    const int col_local = tid / LANES, col = blockIdx.x * COLS + col_local;
    const bool live = col < V;
    float* sp = state + (((int64_t)row_slot[row] * H + head) * V + (live ? col : 0)) * DP;
    float s[EPL];
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const float4 x = live ? *reinterpret_cast<const float4*>(sp + 4 * (lane_in_col + LANES * u))
                              : make_float4(0.f, 0.f, 0.f, 0.f);
        s[4 * u] = x.x; s[4 * u + 1] = x.y; s[4 * u + 2] = x.z; s[4 * u + 3] = x.w;
    }
    const int HD = H * D;
    for (int c0 = 0; c0 < n_new; c0 += CHUNK) {
        const int n = min(CHUNK, n_new - c0);
        __syncthreads();    // the chunk before is done with
        for (int i = tid; i < n * DP; i += THREADS) {
            const int t = i / DP, e = i - t * DP;
            const int64_t tok = t0 + c0 + t;
            float r = 0.f, k = 0.f, w = 0.f, a = 0.f;
            if (e < D) {
                r = to_float(rkv[tok * ld + r0 + head * D + e]);
                k = to_float(rkv[tok * ld + k0 + head * D + e]);
                w = wa[tok * ldwa + head * D + e];
                a = wa[tok * ldwa + HD + head * D + e];
            }
            sr[t][e] = r; sk[t][e] = k; sw[t][e] = w; sau[t][e] = a;
        }
        for (int i = tid; i < n * COLS; i += THREADS) {
            const int t = i / COLS, c = i - t * COLS;
            const int cc = blockIdx.x * COLS + c;
            sv[t][c] = cc < V ? to_float(rkv[(int64_t)(t0 + c0 + t) * ld + v0 + head * V + cc]) : 0.f;
        }
        __syncthreads();
        for (int t = tid >> 5; t < n; t += THREADS / 32) {   // a warp per token: |k|^2
            float ss = 0.f;
            for (int e = tid & 31; e < D; e += 32) ss = fmaf(sk[t][e], sk[t][e], ss);
            ss = warp_sum(ss);
            if ((tid & 31) == 0) sinv[t] = 1.0f / sqrtf(ss + unit_eps);
        }
        __syncthreads();
        for (int i = tid; i < n * DP; i += THREADS) {
            const int t = i / DP, e = i - t * DP;
            const float u = sk[t][e] * sinv[t];
            su[t][e] = u;
            sau[t][e] *= u;
        }
        __syncthreads();
        float o_part[CHUNK];
#pragma unroll
        for (int t = 0; t < CHUNK; ++t) {
            if (t < n) {
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
                for (int u = 0; u < UNITS; ++u) {
                    const float4 x = *reinterpret_cast<const float4*>(&su[t][4 * (lane_in_col + LANES * u)]);
                    d0 = fmaf(x.x, s[4 * u], d0);
                    d1 = fmaf(x.y, s[4 * u + 1], d1);
                    d2 = fmaf(x.z, s[4 * u + 2], d2);
                    d3 = fmaf(x.w, s[4 * u + 3], d3);
                }
                float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
                for (int o = LANES >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                const float v = sv[t][col_local];
                float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
                for (int u = 0; u < UNITS; ++u) {
                    const int e = 4 * (lane_in_col + LANES * u);
                    const float4 w = *reinterpret_cast<const float4*>(&sw[t][e]);
                    const float4 au = *reinterpret_cast<const float4*>(&sau[t][e]);
                    const float4 k = *reinterpret_cast<const float4*>(&sk[t][e]);
                    const float4 r = *reinterpret_cast<const float4*>(&sr[t][e]);
                    s[4 * u] = fmaf(k.x, v, fmaf(-au.x, dot, w.x * s[4 * u]));
                    s[4 * u + 1] = fmaf(k.y, v, fmaf(-au.y, dot, w.y * s[4 * u + 1]));
                    s[4 * u + 2] = fmaf(k.z, v, fmaf(-au.z, dot, w.z * s[4 * u + 2]));
                    s[4 * u + 3] = fmaf(k.w, v, fmaf(-au.w, dot, w.w * s[4 * u + 3]));
                    p0 = fmaf(s[4 * u], r.x, p0);
                    p1 = fmaf(s[4 * u + 1], r.y, p1);
                    p2 = fmaf(s[4 * u + 2], r.z, p2);
                    p3 = fmaf(s[4 * u + 3], r.w, p3);
                }
                o_part[t] = (p0 + p1) + (p2 + p3);
            }
        }
#pragma unroll
        for (int t = 0; t < CHUNK; ++t) {
            if (t < n) {
                float o = o_part[t];
#pragma unroll
                for (int sh = LANES >> 1; sh > 0; sh >>= 1) o += __shfl_xor_sync(0xffffffffu, o, sh);
                if (lane_in_col == 0 && live)
                    out[(int64_t)(t0 + c0 + t) * H * V + head * V + col] = o;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int u = 0; u < UNITS; ++u)
            *reinterpret_cast<float4*>(sp + 4 * (lane_in_col + LANES * u)) =
                make_float4(s[4 * u], s[4 * u + 1], s[4 * u + 2], s[4 * u + 3]);
    }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_general_delta_padded_dim() { return DP; }

// dtype of rkv: 0 = float32, 1 = bfloat16.
SLLM_EXPORT int sllm_general_delta(const void* rkv, int64_t ld, int r0, int k0, int v0,
                                   const float* wa, int64_t ldwa, float* state,
                                   const int* row_start, const int* row_slot, float* out,
                                   int n_rows, int H, int V, float unit_eps, int dtype,
                                   cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || V <= 0 || H > 65535 || n_rows > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((V + COLS - 1) / COLS, H, n_rows);
    if (dtype == 0)
        return (int)sllm_launch_pdl(general_delta_kernel<float>, grid, dim3(THREADS), 0, stream,
                                    (const float*)rkv, ld, r0, k0, v0, wa, ldwa, state, row_start,
                                    row_slot, out, H, V, unit_eps);
    if (dtype == 1)
        return (int)sllm_launch_pdl(general_delta_kernel<__nv_bfloat16>, grid, dim3(THREADS), 0,
                                    stream, (const __nv_bfloat16*)rkv, ld, r0, k0, v0, wa, ldwa,
                                    state, row_start, row_slot, out, H, V, unit_eps);
    return (int)cudaErrorInvalidValue;
}

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
// its elements in registers (a thread holds such slices of CPT = 2 columns: the five vectors it
// reads from shared memory per token serve both, and shared-memory bandwidth is what a token
// costs an SM) (the key size D is padded to LANES * 16; the padding stays zero).
// Lane l owns the float4 units l, l + LANES, l + 2 LANES, ... of the column, so that the lanes
// of a column read consecutive 16-byte words of shared memory.  A CTA has one COMPUTE warp,
// which owns 2 * 32 / LANES columns of one (row, head), and two LOADER warps; a head's columns are
// spread over several CTAs (many SMs work on one sequence, and the shared-memory reads of a
// token, five vectors per thread, are shared out with them).  The row's tokens come in chunks
// through two buffers: while the compute warps run chunk c, the loader warps fetch chunk c + 1
// (r, k, w, a of the head, v of the CTA's columns), form the unit key and a * u, and all
// warps meet once per chunk.  Per token the only chain is (partial dot of 16 products) ->
// log2(LANES) shuffles -> one multiply-add per element; the read-out s . r is kept as a partial
// sum per token and summed across the lanes after the chunk, off the chain.  Rows of one token
// (decode steps) take the same path with a chunk of one.
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
constexpr int COMPUTE = 64, LOADERS = 64, THREADS = COMPUTE + LOADERS;
// columns per compute thread (measured at 32 heads of 64 x 64, 2,048 tokens: 1 column and two
// compute warps 571 us; 2 columns and one warp 844 us; a warp's issue rate, not shared memory,
// is what a token costs)
constexpr int CPT = 1;
constexpr int COLS = COMPUTE / LANES * CPT;   // columns of S per CTA
constexpr int UNITS = EPL / 4;                // float4 units per lane
// tokens per chunk: two buffers of five vectors of DP floats per token, within 40 KB
constexpr int CHUNK = (20 * 1024 / (5 * DP * 4)) >= 16 ? 16 : (20 * 1024 / (5 * DP * 4));
static_assert(CHUNK >= 2, "chunk too small");

struct __align__(16) Staged {
    float r[CHUNK][DP], k[CHUNK][DP], w[CHUNK][DP], u[CHUNK][DP], au[CHUNK][DP];
    float v[CHUNK][COLS];
    float inv[CHUNK];
};

__device__ __forceinline__ void loaders_sync() {
    asm volatile("bar.sync 1, %0;\n" ::"n"(LOADERS) : "memory");
}

__device__ __forceinline__ float4 load4(const float* p) {
    return *reinterpret_cast<const float4*>(p);
}
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
    return make_float4(__low2float(h[0]), __high2float(h[0]), __low2float(h[1]), __high2float(h[1]));
}

constexpr int QUADS = CHUNK * DP / 4;                       // units of 4 elements in a chunk
constexpr int QPT = (QUADS + LOADERS - 1) / LOADERS;        // of which a loader thread takes
// a token's units fit the lanes of one warp (and LOADERS is a multiple of them): the unit key is
// formed in registers
constexpr bool FUSED_UNIT = DP / 4 <= 32;

// The loader warps fetch the tokens [tok0, tok0 + n) of one head into `st`.  VEC: every row of
// every operand starts on a multiple of 4 elements, so four elements come per load; a thread
// requests all its loads before it stores any (the chunk costs one round trip, not one per
// element).
template <typename T, bool VEC>
__device__ __forceinline__ void stage_chunk(Staged& st, int lt, const T* __restrict__ rkv,
                                            int64_t ld, int r0, int k0, int v0,
                                            const float* __restrict__ wa, int64_t ldwa, int HD,
                                            int head, int V, int col0, int64_t tok0, int n,
                                            float unit_eps) {
    if (VEC) {
        float4 r[QPT], k[QPT], w[QPT], a[QPT];
#pragma unroll
        for (int j = 0; j < QPT; ++j) {
            const int i = lt + j * LOADERS;
            const int t = i / (DP / 4), e = (i - t * (DP / 4)) * 4;
            r[j] = k[j] = w[j] = a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < QUADS && t < n && e < D) {
                const int64_t tok = tok0 + t;
                r[j] = load4(rkv + tok * ld + r0 + head * D + e);
                k[j] = load4(rkv + tok * ld + k0 + head * D + e);
                w[j] = load4(wa + tok * ldwa + head * D + e);
                a[j] = load4(wa + tok * ldwa + HD + head * D + e);
            }
        }
        if (FUSED_UNIT) {
            // a token's DP / 4 units lie in neighbouring lanes of one warp: |k|^2 is summed
            // across them and the unit key and a * u are stored at once (no second pass)
            for (int i = lt; i < n * COLS; i += LOADERS) {
                const int t = i / COLS, c = i - t * COLS;
                st.v[t][c] = col0 + c < V
                    ? to_float(rkv[(tok0 + t) * ld + v0 + head * V + col0 + c]) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < QPT; ++j) {
                const int i = lt + j * LOADERS;
                const int t = i / (DP / 4), e = (i - t * (DP / 4)) * 4;
                float ss = fmaf(k[j].x, k[j].x, fmaf(k[j].y, k[j].y,
                                fmaf(k[j].z, k[j].z, k[j].w * k[j].w)));
#pragma unroll
                for (int o = (DP / 4) >> 1; o > 0; o >>= 1)
                    ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float inv = 1.0f / sqrtf(ss + unit_eps);
                if (i < QUADS && t < n) {
                    const float4 u = make_float4(k[j].x * inv, k[j].y * inv, k[j].z * inv,
                                                 k[j].w * inv);
                    *reinterpret_cast<float4*>(&st.r[t][e]) = r[j];
                    *reinterpret_cast<float4*>(&st.k[t][e]) = k[j];
                    *reinterpret_cast<float4*>(&st.w[t][e]) = w[j];
                    *reinterpret_cast<float4*>(&st.u[t][e]) = u;
                    *reinterpret_cast<float4*>(&st.au[t][e]) =
                        make_float4(a[j].x * u.x, a[j].y * u.y, a[j].z * u.z, a[j].w * u.w);
                }
            }
        } else {
#pragma unroll
        for (int j = 0; j < QPT; ++j) {
            const int i = lt + j * LOADERS;
            const int t = i / (DP / 4), e = (i - t * (DP / 4)) * 4;
            if (i < QUADS && t < n) {
                *reinterpret_cast<float4*>(&st.r[t][e]) = r[j];
                *reinterpret_cast<float4*>(&st.k[t][e]) = k[j];
                *reinterpret_cast<float4*>(&st.w[t][e]) = w[j];
                *reinterpret_cast<float4*>(&st.au[t][e]) = a[j];
            }
        }
        }
    } else {
        for (int i = lt; i < n * DP; i += LOADERS) {
            const int t = i / DP, e = i - t * DP;
            const int64_t tok = tok0 + t;
            float r = 0.f, k = 0.f, w = 0.f, a = 0.f;
            if (e < D) {
                r = to_float(rkv[tok * ld + r0 + head * D + e]);
                k = to_float(rkv[tok * ld + k0 + head * D + e]);
                w = wa[tok * ldwa + head * D + e];
                a = wa[tok * ldwa + HD + head * D + e];
            }
            st.r[t][e] = r; st.k[t][e] = k; st.w[t][e] = w; st.au[t][e] = a;
        }
    }
    if (!(VEC && FUSED_UNIT)) {     // (else stored above, unit key and all)
        for (int i = lt; i < n * COLS; i += LOADERS) {
            const int t = i / COLS, c = i - t * COLS;
            st.v[t][c] = col0 + c < V
                ? to_float(rkv[(tok0 + t) * ld + v0 + head * V + col0 + c]) : 0.f;
        }
        loaders_sync();
        for (int t = lt >> 5; t < n; t += LOADERS / 32) {   // a warp per token: |k|^2
            float ss = 0.f;
            for (int e = lt & 31; e < D; e += 32) ss = fmaf(st.k[t][e], st.k[t][e], ss);
            ss = warp_sum(ss);
            if ((lt & 31) == 0) st.inv[t] = 1.0f / sqrtf(ss + unit_eps);
        }
        loaders_sync();
        for (int i = lt; i < n * DP; i += LOADERS) {
            const int t = i / DP, e = i - t * DP;
            const float u = st.k[t][e] * st.inv[t];
            st.u[t][e] = u;
            st.au[t][e] *= u;
        }
    }
}

// The compute warps' part of a chunk: n tokens of `st` through this thread's slices of its
// columns.  out_head: the output row of the chunk's first token at this head, rows ld_out apart.
// (A variant without the `t < n` conditions for whole chunks, which lets a token's loads be
// requested during the chain of the one before, gained 8 % at key size 64 and lost 70 % at 128,
// where it held too many values in flight; it was dropped.)
__device__ __forceinline__ void run_chunk(const Staged& st, float (&s)[CPT][EPL], int n,
                                          int lane_in_col, int col_local, int col0, int V,
                                          float* __restrict__ out_head, int64_t ld_out) {
    float o_part[CHUNK][CPT];
#pragma unroll
    for (int t = 0; t < CHUNK; ++t) {
        if (t < n) {
            float dot[CPT];
            {
                float d[CPT][4];
#pragma unroll
                for (int c = 0; c < CPT; ++c) d[c][0] = d[c][1] = d[c][2] = d[c][3] = 0.f;
#pragma unroll
                for (int u = 0; u < UNITS; ++u) {
                    const float4 x = *reinterpret_cast<const float4*>(
                        &st.u[t][4 * (lane_in_col + LANES * u)]);
#pragma unroll
                    for (int c = 0; c < CPT; ++c) {
                        d[c][0] = fmaf(x.x, s[c][4 * u], d[c][0]);
                        d[c][1] = fmaf(x.y, s[c][4 * u + 1], d[c][1]);
                        d[c][2] = fmaf(x.z, s[c][4 * u + 2], d[c][2]);
                        d[c][3] = fmaf(x.w, s[c][4 * u + 3], d[c][3]);
                    }
                }
#pragma unroll
                for (int c = 0; c < CPT; ++c)
                    dot[c] = (d[c][0] + d[c][1]) + (d[c][2] + d[c][3]);
            }
#pragma unroll
            for (int o = LANES >> 1; o > 0; o >>= 1)
#pragma unroll
                for (int c = 0; c < CPT; ++c)
                    dot[c] += __shfl_xor_sync(0xffffffffu, dot[c], o);
            float v[CPT], p[CPT][4];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                v[c] = st.v[t][col_local + c];
                p[c][0] = p[c][1] = p[c][2] = p[c][3] = 0.f;
            }
#pragma unroll
            for (int u = 0; u < UNITS; ++u) {
                const int e = 4 * (lane_in_col + LANES * u);
                const float4 w = *reinterpret_cast<const float4*>(&st.w[t][e]);
                const float4 au = *reinterpret_cast<const float4*>(&st.au[t][e]);
                const float4 k = *reinterpret_cast<const float4*>(&st.k[t][e]);
                const float4 r = *reinterpret_cast<const float4*>(&st.r[t][e]);
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    float* sc = &s[c][4 * u];
                    sc[0] = fmaf(k.x, v[c], fmaf(-au.x, dot[c], w.x * sc[0]));
                    sc[1] = fmaf(k.y, v[c], fmaf(-au.y, dot[c], w.y * sc[1]));
                    sc[2] = fmaf(k.z, v[c], fmaf(-au.z, dot[c], w.z * sc[2]));
                    sc[3] = fmaf(k.w, v[c], fmaf(-au.w, dot[c], w.w * sc[3]));
                    p[c][0] = fmaf(sc[0], r.x, p[c][0]);
                    p[c][1] = fmaf(sc[1], r.y, p[c][1]);
                    p[c][2] = fmaf(sc[2], r.z, p[c][2]);
                    p[c][3] = fmaf(sc[3], r.w, p[c][3]);
                }
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c)
                o_part[t][c] = (p[c][0] + p[c][1]) + (p[c][2] + p[c][3]);
        }
    }
#pragma unroll
    for (int t = 0; t < CHUNK; ++t) {
        if (t < n) {
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float o = o_part[t][c];
#pragma unroll
                for (int sh = LANES >> 1; sh > 0; sh >>= 1)
                    o += __shfl_xor_sync(0xffffffffu, o, sh);
                const int col = col0 + col_local + c;
                if (lane_in_col == 0 && col < V)
                    out_head[(int64_t)t * ld_out + col] = o;
            }
        }
    }
}

// rkv: [N, ld] with the heads' r at column r0, k at k0, v at v0 (each heads x D or heads x V);
// wa: float32 [N, ldwa] with the decays at column 0 and the removal rates at column H * D.
template <typename T, bool VEC>
__global__ void __launch_bounds__(THREADS)
general_delta_kernel(const T* __restrict__ rkv, int64_t ld, int r0, int k0, int v0,
                     const float* __restrict__ wa, int64_t ldwa, float* __restrict__ state,
                     const int* __restrict__ row_start, const int* __restrict__ row_slot,
                     float* __restrict__ out, int H, int V, float unit_eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ Staged stage[2];
    const int row = blockIdx.z, head = blockIdx.y;
    const int t0 = row_start[row], n_new = row_start[row + 1] - t0;
    if (n_new <= 0) return;
    const int tid = threadIdx.x;
    const bool loader = tid >= COMPUTE;
    const int lane_in_col = tid % LANES;
    const int col_local = (tid % COMPUTE) / LANES * CPT, col0 = blockIdx.x * COLS;
    // this thread's columns: col0 + col_local + c, c < CPT
    float* sp = state + (((int64_t)row_slot[row] * H + head) * V) * DP;
    float s[CPT][EPL];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int col = col0 + col_local + c;
        const bool live = !loader && col < V;
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
            const float4 x = live ? *reinterpret_cast<const float4*>(
                                        sp + (int64_t)col * DP + 4 * (lane_in_col + LANES * u))
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
            s[c][4 * u] = x.x; s[c][4 * u + 1] = x.y; s[c][4 * u + 2] = x.z; s[c][4 * u + 3] = x.w;
        }
    }
    const int HD = H * D;
    if (loader)
        stage_chunk<T, VEC>(stage[0], tid - COMPUTE, rkv, ld, r0, k0, v0, wa, ldwa, HD, head, V, col0,
                    (int64_t)t0, min(CHUNK, n_new), unit_eps);
    __syncthreads();
    int buf = 0;
    for (int c0 = 0; c0 < n_new; c0 += CHUNK, buf ^= 1) {
        const int n = min(CHUNK, n_new - c0);
        if (loader) {
            if (c0 + CHUNK < n_new)
                stage_chunk<T, VEC>(stage[buf ^ 1], tid - COMPUTE, rkv, ld, r0, k0, v0, wa, ldwa, HD, head,
                            V, col0, (int64_t)t0 + c0 + CHUNK, min(CHUNK, n_new - c0 - CHUNK),
                            unit_eps);
        } else {
            run_chunk(stage[buf], s, n, lane_in_col, col_local, col0, V,
                      out + (int64_t)(t0 + c0) * H * V + head * V, (int64_t)H * V);
        }
        __syncthreads();    // chunk c is done with, chunk c + 1 is staged
    }
    if (!loader) {
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int col = col0 + col_local + c;
            if (col >= V) continue;
#pragma unroll
            for (int u = 0; u < UNITS; ++u)
                *reinterpret_cast<float4*>(sp + (int64_t)col * DP + 4 * (lane_in_col + LANES * u)) =
                    make_float4(s[c][4 * u], s[c][4 * u + 1], s[c][4 * u + 2], s[c][4 * u + 3]);
        }
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
    // four elements per load where every operand's rows start on multiples of four elements
    const bool vec = D % 4 == 0 && ld % 4 == 0 && r0 % 4 == 0 && k0 % 4 == 0 && ldwa % 4 == 0 &&
                     !(((uintptr_t)rkv | (uintptr_t)wa) & 15);
    typedef __nv_bfloat16 bf16;
#define SLLM_GD_LAUNCH(T, VEC)                                                                  \
    return (int)sllm_launch_pdl(general_delta_kernel<T, VEC>, grid, dim3(THREADS), 0, stream,   \
                                (const T*)rkv, ld, r0, k0, v0, wa, ldwa, state, row_start,      \
                                row_slot, out, H, V, unit_eps)
    if (dtype == 0) {
        if (vec) SLLM_GD_LAUNCH(float, true);
        SLLM_GD_LAUNCH(float, false);
    }
    if (dtype == 1) {
        if (vec) SLLM_GD_LAUNCH(bf16, true);
        SLLM_GD_LAUNCH(bf16, false);
    }
#undef SLLM_GD_LAUNCH
    return (int)cudaErrorInvalidValue;
}

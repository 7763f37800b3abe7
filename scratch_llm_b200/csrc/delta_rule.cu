// The gated delta rule: a linear recurrence whose state is one matrix S [D, V] per head and
// request, carried in 32-bit from token to token.  Per token, with a unit key k and a scaled
// unit query q of size D, a value v of size V, a decay g in (0, 1) and a step size beta:
//
//     S  <-  g S
//     u   =  beta (v - S^T k)
//     S  <-  S + k u^T
//     o   =  S^T q                       (the read-out sees the token's own write)
//
// with, computed here in 32-bit from what the projections and the short convolution left:
//     k = k_raw / sqrt(sum(k_raw^2) + 1e-6),   q = q_raw / sqrt(sum(q_raw^2) + 1e-6) * D^(-1/2)
//     beta = sigmoid(b),   g = exp(-exp(A_log) * softplus(a + dt_bias))
// Head h of H reads key/query head h / (H / G).
//
// Columns of S are independent of each other: u_j and o_j need column j of S only.  A CTA
// takes COLS columns of one (row, head); R threads share a column, each holding D / R of its
// elements in registers, and two shuffles rounds give both dot products of a token (S^T k and
// S^T q of the decayed state; o = S'^T q + u (k . q)).  Tokens are staged in chunks of TC: the
// CTA norms the chunk's keys and queries and evaluates its gates, then walks the chunk without
// a block-wide barrier.  The same kernel serves portions of prompts (many tokens per row) and
// decoding (one): a row reads its state from its slot and writes it back; rows without tokens
// touch nothing.
//
// Compiled once per key size: -DSLLM_HEAD_DIM=<D>.
#include "common.cuh"

#ifndef SLLM_HEAD_DIM
#error "compile with -DSLLM_HEAD_DIM=<key size>"
#endif

namespace sllm {

constexpr int D = SLLM_HEAD_DIM;
static_assert(D >= 1 && D <= 256, "key size: 1 to 256 (a chunk of keys and queries is staged in shared memory)");
constexpr int R = D > 128 ? 8 : (D > 8 ? 4 : 1);   // threads that share a column
constexpr int DP = (D + R - 1) / R;                 // elements of a column per thread
constexpr int THREADS = 128;
constexpr int COLS = THREADS / R;
constexpr int TC = 16;                              // tokens staged at a time

struct DeltaArgs {
    const void* act; int64_t ld_act;     // [tokens, >= 2 G D + H V]: q heads, k heads, v heads
    const float* ab; int64_t ld_ab;      // [tokens, >= 2 H]: a (decay input) then b (step input)
    const float* A_log; const float* dt_bias;   // [H]
    float* state;                        // [slots, H, V, D]
    const int* row_start; const int* row_slot;
    float* out;                          // [tokens, H * V]
    int H; int G; int V;
};

template <typename T>
__global__ void __launch_bounds__(THREADS) delta_rule_kernel(const DeltaArgs a) {
    __shared__ float ks[TC][D];
    __shared__ float qs[TC][D];
    __shared__ float vs[TC][COLS];
    __shared__ float gate_s[TC], beta_s[TC], kq_s[TC];

    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.z, head = blockIdx.y;
    const int t0 = a.row_start[r], n_new = a.row_start[r + 1] - t0;
    if (n_new <= 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = head / (a.H / a.G);
    const int col0 = blockIdx.x * COLS;
    const int col = col0 + tid / R, part = tid % R;
    const bool live = col < a.V;
    const T* act = reinterpret_cast<const T*>(a.act);
    const int64_t k_col0 = (int64_t)a.G * D, v_col0 = 2 * (int64_t)a.G * D;

    float S[DP];
    float* st = a.state + (((int64_t)a.row_slot[r] * a.H + head) * a.V + (live ? col : 0)) * D;
#pragma unroll
    for (int i = 0; i < DP; ++i) {
        const int e = i * R + part;
        S[i] = (live && e < D) ? st[e] : 0.f;
    }
    const float decay_rate = expf(a.A_log[head]), dt_bias = a.dt_bias[head];
    const float q_scale = rsqrtf((float)D);

    for (int c0 = 0; c0 < n_new; c0 += TC) {
        const int nt = min(TC, n_new - c0);
        __syncthreads();   // the previous chunk's staging is no longer read
        for (int idx = tid; idx < nt * D; idx += THREADS) {
            const int t = idx / D, e = idx - t * D;
            const T* row = act + (int64_t)(t0 + c0 + t) * a.ld_act + (int64_t)g * D;
            qs[t][e] = to_float(row[e]);
            ks[t][e] = to_float(row[k_col0 + e]);
        }
        for (int idx = tid; idx < nt * COLS; idx += THREADS) {
            const int t = idx / COLS, j = idx - t * COLS;
            vs[t][j] = col0 + j < a.V
                ? to_float(act[(int64_t)(t0 + c0 + t) * a.ld_act + v_col0 + (int64_t)head * a.V +
                               col0 + j]) : 0.f;
        }
        if (tid < nt) {
            const float* ab = a.ab + (int64_t)(t0 + c0 + tid) * a.ld_ab;
            const float x = ab[head] + dt_bias;
            const float softplus = x > 20.f ? x : log1pf(expf(x));
            gate_s[tid] = expf(-decay_rate * softplus);
            beta_s[tid] = 1.0f / (1.0f + expf(-ab[a.H + head]));
        }
        __syncthreads();
        // unit vectors, the query's scale, and k . q: one warp per token
        for (int t = warp; t < nt; t += THREADS / 32) {
            float sk = 0.f, sq = 0.f;
            for (int e = lane; e < D; e += 32) {
                sk += ks[t][e] * ks[t][e];
                sq += qs[t][e] * qs[t][e];
            }
            sk = warp_sum(sk);
            sq = warp_sum(sq);
            const float ik = 1.0f / sqrtf(sk + 1e-6f), iq = q_scale / sqrtf(sq + 1e-6f);
            float kq = 0.f;
            for (int e = lane; e < D; e += 32) {
                const float kk = ks[t][e] * ik, qq = qs[t][e] * iq;
                ks[t][e] = kk;
                qs[t][e] = qq;
                kq += kk * qq;
            }
            kq = warp_sum(kq);
            if (lane == 0) kq_s[t] = kq;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float decay = gate_s[t];
            float sk = 0.f, sq = 0.f;
#pragma unroll
            for (int i = 0; i < DP; ++i) {
                const int e = i * R + part;
                if (e < D) {
                    S[i] *= decay;
                    sk = fmaf(S[i], ks[t][e], sk);
                    sq = fmaf(S[i], qs[t][e], sq);
                }
            }
#pragma unroll
            for (int o = R / 2; o > 0; o >>= 1) {
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
            }
            const float u = beta_s[t] * (vs[t][tid / R] - sk);
#pragma unroll
            for (int i = 0; i < DP; ++i) {
                const int e = i * R + part;
                if (e < D) S[i] = fmaf(ks[t][e], u, S[i]);
            }
            if (live && part == 0)
                a.out[(int64_t)(t0 + c0 + t) * a.H * a.V + (int64_t)head * a.V + col] =
                    sq + u * kq_s[t];
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DP; ++i) {
            const int e = i * R + part;
            if (e < D) st[e] = S[i];
        }
    }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_delta_rule_head_dim() { return D; }

// dtype: 0 = float32, 1 = bfloat16 (of act).  n_rows rows of the packed batch (row_start has
// n_rows + 1 entries); state slots are indexed by row_slot.
SLLM_EXPORT int sllm_delta_rule(const void* act, int64_t ld_act, const float* ab, int64_t ld_ab,
                                const float* A_log, const float* dt_bias, float* state,
                                const int* row_start, const int* row_slot, float* out, int n_rows,
                                int H, int G, int V, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || V <= 0 || n_rows > 65535 || H > 65535 ||
        ld_act < 2 * (int64_t)G * D + (int64_t)H * V || ld_ab < 2 * H)
        return (int)cudaErrorInvalidValue;
    DeltaArgs a;
    a.act = act; a.ld_act = ld_act; a.ab = ab; a.ld_ab = ld_ab; a.A_log = A_log;
    a.dt_bias = dt_bias; a.state = state; a.row_start = row_start; a.row_slot = row_slot;
    a.out = out; a.H = H; a.G = G; a.V = V;
    dim3 grid((V + COLS - 1) / COLS, H, n_rows);
    if (dtype == 0)
        delta_rule_kernel<float><<<grid, THREADS, 0, stream>>>(a);
    else if (dtype == 1)
        delta_rule_kernel<__nv_bfloat16><<<grid, THREADS, 0, stream>>>(a);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}

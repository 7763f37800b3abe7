// Per-head RMS norm of queries and keys, an optional position-dependent factor on the
// queries, and the write of the new keys and values into the paged cache, for attention
// mixers without a rotation.
//
// x is [n_tokens, ld]: H query heads, then G key heads, each `hd` wide, then whatever else the
// fused projection holds (not touched).
//   q[t, h]  <-  q / sqrt(mean(q^2) + eps) * q_gain * temp(p)       (in place)
//   temp(p)  =   1 + coef * ln(floor((p + 1) / every) + 1)           (coef = 0: no factor)
//   K page   <-  k / sqrt(mean(k^2) + eps) * k_gain
//   V page   <-  v[t, g] if the projection has value heads (v_col0 >= 0), else k as projected,
//                before its norm (a mixer whose values ARE its keys)
// with gains of size hd shared by all heads; q_gain / k_gain null: no norm of that side.
// pages: [n_pages, 2 (K, V), G, page_size, hd]; page = block_table[row, p / page_size].
// A token whose row is -1 is padding: nothing of it is normed or stored.  Norms and the
// factor are 32-bit arithmetic with one rounding.
#include "common.cuh"

namespace sllm {

constexpr int QN_WARPS = 4;

// grid (tokens, ceil((H + G) / QN_WARPS)); one warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(QN_WARPS * 32)
qk_norm_kv_write_kernel(T* __restrict__ x, int64_t ld, const int* __restrict__ positions,
                        const int* __restrict__ token_row, const float* __restrict__ q_gain,
                        const float* __restrict__ k_gain, float eps, float temp_coef,
                        float temp_every, int v_col0, T* __restrict__ pages,
                        const int* __restrict__ block_table, int table_stride, int page_size,
                        int H, int G, int hd, int write) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    const int row = token_row[n];
    if (row < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * QN_WARPS + warp;
    if (head >= H + G) return;
    const bool is_k = head >= H;
    if (is_k && !write) return;
    const int pos = positions[n];
    T* h = x + n * ld + (int64_t)head * hd;
    const float* gain = is_k ? k_gain : q_gain;
    float inv = 1.f;
    if (gain) {
        float ss = 0.f;
        for (int d = lane; d < hd; d += 32) {
            const float v = to_float(h[d]);
            ss += v * v;
        }
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    if (!is_k) {
        float temp = 1.f;
        if (temp_coef != 0.f) {
            const float k = temp_every == floorf(temp_every) && temp_every >= 1.f
                                ? (float)((pos + 1) / (int)temp_every)
                                : floorf((float)(pos + 1) / temp_every);
            temp = 1.0f + temp_coef * logf(k + 1.0f);
        }
        if (!gain && temp == 1.f) return;
        for (int d = lane; d < hd; d += 32)
            h[d] = from_float<T>(to_float(h[d]) * inv * (gain ? gain[d] : 1.f) * temp);
        return;
    }
    const int g = head - H;
    const int page = block_table[(int64_t)row * table_stride + pos / page_size];
    T* k_dst = pages + (((int64_t)page * 2 * G + g) * page_size + pos % page_size) * hd;
    T* v_dst = k_dst + (int64_t)G * page_size * hd;
    const T* v_src = v_col0 >= 0 ? x + n * ld + v_col0 + (int64_t)g * hd : h;
    for (int d = lane; d < hd; d += 32) {
        const T raw = h[d];
        v_dst[d] = v_col0 >= 0 ? v_src[d] : raw;
        k_dst[d] = from_float<T>(to_float(raw) * inv * (gain ? gain[d] : 1.f));
    }
}

// The same for bfloat16 and head sizes 8 * 2^k up to 256 with 16-byte accesses: hd / 8 lanes
// share a head (8 consecutive elements each), so a warp takes 256 / hd heads of a token at once.
// The arithmetic is the scalar kernel's; the sum of squares is added up in another order.
// grid (tokens, ceil((H + G) / (heads per warp * QN_WARPS))).
__global__ void __launch_bounds__(QN_WARPS * 32)
qk_norm_kv_write_vec_kernel(__nv_bfloat16* __restrict__ x, int64_t ld,
                            const int* __restrict__ positions, const int* __restrict__ token_row,
                            const float* __restrict__ q_gain, const float* __restrict__ k_gain,
                            float eps, float temp_coef, float temp_every, int v_col0,
                            __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table,
                            int table_stride, int page_size, int H, int G, int hd, int write) {
    pdl_wait();
    pdl_trigger();
    typedef __nv_bfloat16 bf16;
    const int64_t n = blockIdx.x;
    const int row = token_row[n];
    if (row < 0) return;
    const int group = hd >> 3;                       // lanes per head
    const int per_warp = 32 / group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = (blockIdx.y * QN_WARPS + warp) * per_warp + lane / group;
    const int piece = lane % group;                  // which 8 elements of the head
    const bool is_k = head >= H;
    const bool active = head < H + G && !(is_k && !write);
    const int pos = positions[n];
    bf16* h = x + n * ld + (int64_t)(active ? head : 0) * hd + piece * 8;
    const float* gain = is_k ? k_gain : q_gain;
    float v[8];
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (active) raw = *reinterpret_cast<const uint4*>(h);
    {
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __low2float(p2[i]);
            v[2 * i + 1] = __high2float(p2[i]);
        }
    }
    float inv = 1.f;
    if (gain) {                                      // (the same for every lane of the launch)
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
        for (int o = group >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        inv = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    if (!active) return;
    float scale[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) scale[i] = inv * (gain ? gain[piece * 8 + i] : 1.f);
    auto pack = [&](float factor) {
        uint4 out;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            o2[i] = __floats2bfloat162_rn(v[2 * i] * scale[2 * i] * factor,
                                          v[2 * i + 1] * scale[2 * i + 1] * factor);
        return out;
    };
    if (!is_k) {
        float temp = 1.f;
        if (temp_coef != 0.f) {
            const float k = temp_every == floorf(temp_every) && temp_every >= 1.f
                                ? (float)((pos + 1) / (int)temp_every)
                                : floorf((float)(pos + 1) / temp_every);
            temp = 1.0f + temp_coef * logf(k + 1.0f);
        }
        if (!gain && temp == 1.f) return;
        *reinterpret_cast<uint4*>(h) = pack(temp);
        return;
    }
    const int g = head - H;
    const int page = block_table[(int64_t)row * table_stride + pos / page_size];
    bf16* k_dst = pages + (((int64_t)page * 2 * G + g) * page_size + pos % page_size) * hd + piece * 8;
    bf16* v_dst = k_dst + (int64_t)G * page_size * hd;
    *reinterpret_cast<uint4*>(v_dst) =
        v_col0 >= 0 ? *reinterpret_cast<const uint4*>(x + n * ld + v_col0 + (int64_t)g * hd + piece * 8)
                    : raw;
    *reinterpret_cast<uint4*>(k_dst) = pack(1.f);
}

}  // namespace sllm

using namespace sllm;

// dtype: 0 = float32, 1 = bfloat16 (of x and pages).
SLLM_EXPORT int sllm_qk_norm_kv_write(void* x, int64_t ld, const int* positions,
                                      const int* token_row, const float* q_gain,
                                      const float* k_gain, float eps, float temp_coef,
                                      float temp_every, int v_col0, void* pages,
                                      const int* block_table, int table_stride, int page_size,
                                      int n_tokens, int H, int G, int hd, int write, int dtype,
                                      cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || hd <= 0 || page_size <= 0 || ld < (int64_t)(H + G) * hd ||
        (temp_coef != 0.f && !(temp_every > 0.f)) || (v_col0 >= 0 && v_col0 + (int64_t)G * hd > ld))
        return (int)cudaErrorInvalidValue;
    const bool pow2 = hd >= 8 && hd <= 256 && (hd & (hd - 1)) == 0;
    if (dtype == 1 && pow2 && ld % 8 == 0 && (v_col0 < 0 || v_col0 % 8 == 0) &&
        (q_gain != nullptr) == (k_gain != nullptr) &&
        !(((uintptr_t)x | (uintptr_t)pages) & 15)) {
        const int per_block = (256 / hd) * QN_WARPS;
        dim3 vgrid(n_tokens, (H + G + per_block - 1) / per_block);
        qk_norm_kv_write_vec_kernel<<<vgrid, QN_WARPS * 32, 0, stream>>>(
            (__nv_bfloat16*)x, ld, positions, token_row, q_gain, k_gain, eps, temp_coef, temp_every,
            v_col0, (__nv_bfloat16*)pages, block_table, table_stride, page_size, H, G, hd, write);
        SLLM_LAUNCH_CHECK();
        return 0;
    }
    dim3 grid(n_tokens, (H + G + QN_WARPS - 1) / QN_WARPS);
    if (dtype == 0)
        qk_norm_kv_write_kernel<float><<<grid, QN_WARPS * 32, 0, stream>>>(
            (float*)x, ld, positions, token_row, q_gain, k_gain, eps, temp_coef, temp_every, v_col0,
            (float*)pages, block_table, table_stride, page_size, H, G, hd, write);
    else if (dtype == 1)
        qk_norm_kv_write_kernel<__nv_bfloat16><<<grid, QN_WARPS * 32, 0, stream>>>(
            (__nv_bfloat16*)x, ld, positions, token_row, q_gain, k_gain, eps, temp_coef, temp_every,
            v_col0, (__nv_bfloat16*)pages, block_table, table_stride, page_size, H, G, hd, write);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}

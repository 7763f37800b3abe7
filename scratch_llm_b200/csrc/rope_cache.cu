// Rotary position encoding of q and k (32-bit angles and arithmetic) fused with the write of
// the new keys and values into the paged cache.
//
// Restates src/scratch_llm/model.py:204-220 (rotation of adjacent pairs by the angles of the
// token's absolute position), :284-285 (q and k are rotated, v is not) and the page scatter of
// src/scratch_llm/kv_cache.py:423-428 of the reference.
//
// qkv is [n_tokens, (H + 2G) * hd]: q heads, then k heads, then v heads.  q is rotated in
// place.  k is rotated and stored, v is copied, into
//   pages[page, 0 (K) | 1 (V), g, offset, :]     pages: [n_pages, 2, G, page_size, hd]
// where page = block_table[row, position / page_size], offset = position % page_size.
// A token whose row is -1 is padding: it is neither rotated nor stored.
//
// Two options of the plain kernel: `bias` (float32 [(H + 2G) * hd], may be null) is added to q,
// k and v before anything else (projections with biases); `rot` < hd rotates only the first
// `rot` entries of a head (pairs (2j, 2j + 1) or (j, j + rot / 2), tables of rot / 2 columns)
// and passes the rest on as they are.
#include "common.cuh"

namespace sllm {

// grid (tokens, blocks of heads); a block of 256 threads takes as many heads as fit, one thread
// per rotated pair (for v heads: per copied pair).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_row,
                                     const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, T* __restrict__ pages,
                                     const int* __restrict__ block_table, int table_stride,
                                     int page_size, int H, int G, int hd, int rotate,
                                     int interleaved, int write, int heads_per_block,
                                     const float* __restrict__ bias, int rot) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    if (token_row[n] < 0) return;   // a padding token: it belongs to no row
    const int half = hd >> 1, rhalf = rot >> 1;
    const int local = threadIdx.x / half, j = threadIdx.x - local * half;
    const int head = blockIdx.y * heads_per_block + local;
    if (local >= heads_per_block || head >= H + 2 * G) return;
    if (head >= H && !write) return;
    const int pos = positions[n];
    T* h = qkv + n * (int64_t)(H + 2 * G) * hd + (int64_t)head * hd;
    // pair j of the rotated part, or, beyond it, two neighbouring entries that pass unchanged
    const bool turns = j < rhalf;
    const int i0 = turns ? (interleaved ? 2 * j : j) : rot + 2 * (j - rhalf);
    const int i1 = turns ? (interleaved ? 2 * j + 1 : j + rhalf) : i0 + 1;
    float r0 = to_float(h[i0]), r1 = to_float(h[i1]);
    if (bias != nullptr) {
        r0 += bias[(int64_t)head * hd + i0];
        r1 += bias[(int64_t)head * hd + i1];
    }
    if (rotate && turns && head < H + G) {
        const float cj = cos_t[(int64_t)pos * rhalf + j], sj = sin_t[(int64_t)pos * rhalf + j];
        const float x0 = r0, x1 = r1;
        r0 = x0 * cj - x1 * sj;
        r1 = x0 * sj + x1 * cj;
    }
    if (head < H) {
        if (rotate || bias != nullptr) {
            h[i0] = from_float<T>(r0);
            h[i1] = from_float<T>(r1);
        }
        return;
    }
    const int page = block_table[(int64_t)token_row[n] * table_stride + pos / page_size];
    const int off = pos % page_size;
    const bool is_v = head >= H + G;
    const int g = head - H - (is_v ? G : 0);
    T* dst = pages + (((int64_t)page * 2 + (is_v ? 1 : 0)) * G + g) * page_size * hd +
             (int64_t)off * hd;
    // (v is never rotated: r0 and r1 are its entries, with the bias if there is one)
    dst[i0] = from_float<T>(r0);
    dst[i1] = from_float<T>(r1);
}


// The same for bfloat16 with 16-byte accesses: a thread takes 8 consecutive elements of a head
// (adjacent pairing: 4 pairs) or 8 elements of each half of the rotated part (split pairing: 8
// pairs).  Arithmetic and rounding are those of the kernel above.  hd % 16 == 0.
constexpr int ROPE_HEAD_GROUPS = 4;   // threads that share a token's heads between them (plain form)

__device__ __forceinline__ void unpack8(const uint4& r, float* v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __low2float(h[i]);
        v[2 * i + 1] = __high2float(h[i]);
    }
}
__device__ __forceinline__ uint4 pack8(const float* v) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return r;
}

// A thread takes one 8-element unit (adjacent pairing, and entries beyond the rotated part) or
// one pair of units (split pairing) of a token and walks a quarter of the token's heads with
// it: the angles are fetched once and serve every head.  With rot < hd (a multiple of 16, of 8
// for the adjacent pairing) the units beyond the rotated part only pass (with the bias, if
// there is one).
__global__ void rope_kv_write_vec_kernel(__nv_bfloat16* __restrict__ qkv,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ token_row,
                                         const float* __restrict__ cos_t,
                                         const float* __restrict__ sin_t,
                                         __nv_bfloat16* __restrict__ pages,
                                         const int* __restrict__ block_table, int table_stride,
                                         int page_size, int H, int G, int hd, int rotate,
                                         int interleaved, int write, int64_t n_items,
                                         const float* __restrict__ bias, int rot, int groups) {
    pdl_wait();
    pdl_trigger();
    typedef __nv_bfloat16 bf16;
    const int rhalf = rot >> 1;
    const int rot_units = interleaved ? rot / 8 : rot / 16;          // units that turn
    const int per_head = interleaved ? hd / 8 : rot_units + (hd - rot) / 8;
    const int n_heads = write ? H + 2 * G : H;
    const int heads_per_group = (n_heads + groups - 1) / groups;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_items;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int u = (int)(i % per_head);
        const int64_t t = i / per_head;
        const int group = (int)(t % groups);
        const int64_t n = t / groups;
        const int row = token_row[n];
        if (row < 0) continue;   // a padding token: it belongs to no row
        const int pos = positions[n];
        const bool turns = rotate && u < rot_units;
        const bool two = turns && !interleaved;       // a second unit, rot / 2 further on
        // first and second group of 8 elements this thread owns in every head
        const int e0 = (interleaved || u < rot_units) ? 8 * u : rot + 8 * (u - rot_units);
        const int e1 = rhalf + 8 * u;
        float c[8], sn[8];
        if (turns) {
            const float* cp = cos_t + (int64_t)pos * rhalf + (interleaved ? 4 * u : 8 * u);
            const float* sp = sin_t + (int64_t)pos * rhalf + (interleaved ? 4 * u : 8 * u);
            *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cp);
            *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sp);
            if (!interleaved) {
                *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cp + 4);
                *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sp + 4);
            }
        }
        int64_t page_base = 0;
        if (write) {
            const int page = block_table[(int64_t)row * table_stride + pos / page_size];
            page_base = (int64_t)page * 2 * G * page_size * hd + (int64_t)(pos % page_size) * hd;
        }
        bf16* tok = qkv + n * (int64_t)(H + 2 * G) * hd;
        const int head_end = min(n_heads, (group + 1) * heads_per_group);
#pragma unroll 2
        for (int head = group * heads_per_group; head < head_end; ++head) {
            const bool is_v = head >= H + G;
            if (head < H && !turns && bias == nullptr) continue;   // a query's passing entries
            bf16* h = tok + (int64_t)head * hd;
            float xa[8], xb[8];
            unpack8(*reinterpret_cast<const uint4*>(h + e0), xa);
            if (two) unpack8(*reinterpret_cast<const uint4*>(h + e1), xb);
            if (bias != nullptr) {
                const float* bh = bias + (int64_t)head * hd;
                float ba[8];
                *reinterpret_cast<float4*>(ba) = *reinterpret_cast<const float4*>(bh + e0);
                *reinterpret_cast<float4*>(ba + 4) = *reinterpret_cast<const float4*>(bh + e0 + 4);
#pragma unroll
                for (int q = 0; q < 8; ++q) xa[q] += ba[q];
                if (two) {
                    *reinterpret_cast<float4*>(ba) = *reinterpret_cast<const float4*>(bh + e1);
                    *reinterpret_cast<float4*>(ba + 4) = *reinterpret_cast<const float4*>(bh + e1 + 4);
#pragma unroll
                    for (int q = 0; q < 8; ++q) xb[q] += ba[q];
                }
            }
            if (turns && !is_v) {
                if (interleaved) {
#pragma unroll
                    for (int p = 0; p < 4; ++p) {    // 4 adjacent pairs inside one group of 8
                        const float x0 = xa[2 * p], x1 = xa[2 * p + 1];
                        xa[2 * p] = x0 * c[p] - x1 * sn[p];
                        xa[2 * p + 1] = x0 * sn[p] + x1 * c[p];
                    }
                } else {
#pragma unroll
                    for (int p = 0; p < 8; ++p) {
                        const float x0 = xa[p], x1 = xb[p];
                        xa[p] = x0 * c[p] - x1 * sn[p];
                        xb[p] = x0 * sn[p] + x1 * c[p];
                    }
                }
            }
            const uint4 a = pack8(xa);
            uint4 b;
            if (two) b = pack8(xb);
            if (head < H) {
                *reinterpret_cast<uint4*>(h + e0) = a;
                if (two) *reinterpret_cast<uint4*>(h + e1) = b;
                continue;
            }
            const int g = head - H - (is_v ? G : 0);
            bf16* dst = pages + page_base + ((int64_t)(is_v ? G : 0) + g) * page_size * hd;
            *reinterpret_cast<uint4*>(dst + e0) = a;
            if (two) *reinterpret_cast<uint4*>(dst + e1) = b;
        }
    }
}

}  // namespace sllm

using namespace sllm;

// rotate = 0 stores k unrotated (a position encoding that is not rotary applies itself first).
SLLM_EXPORT int sllm_rope_kv_write(void* qkv, const int* positions, const int* token_row,
                                   const float* cos_t, const float* sin_t, void* pages,
                                   const int* block_table, int table_stride, int page_size,
                                   int n_tokens, int H, int G, int hd, int rotate,
                                   int interleaved, int write, int dtype, const float* bias,
                                   int rot, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!rotate || rot <= 0) rot = rotate ? hd : 0;
    if (rot > hd || (rot & 1)) return (int)cudaErrorInvalidValue;
    if (H <= 0 || G <= 0 || hd <= 0 || (hd & 1) || page_size <= 0) return (int)cudaErrorInvalidValue;
    if (hd / 2 > 256) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    const int heads_per_block = threads / (hd / 2);
    const int n_heads = write ? H + 2 * G : H;
    dim3 grid(n_tokens, (n_heads + heads_per_block - 1) / heads_per_block);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    if (dtype == 0)
        return (int)sllm_launch_pdl(rope_kv_write_kernel<float>, grid, dim3(threads), 0, stream,
                                    (float*)qkv, positions, token_row, cos_t, sin_t, (float*)pages,
                                    block_table, table_stride, page_size, H, G, hd, rotate,
                                    interleaved, write, heads_per_block, bias, rot);
    // (with a bias or a partial rotation a thread's walk over the heads is longer: steps of few
    // tokens, which cannot fill the device with it, take the plain kernel's many small blocks)
    const bool plain_form = bias == nullptr && (!rotate || rot == hd);
    if (dtype == 1 && hd % 16 == 0 && rot % (interleaved ? 8 : 16) == 0 &&
        (plain_form || n_tokens >= 64) &&
        !((uintptr_t)qkv & 15) && !((uintptr_t)pages & 15) && !((uintptr_t)bias & 15) &&
        (!rotate || (!((uintptr_t)cos_t & 15) && !((uintptr_t)sin_t & 15)))) {
        const int per_head = interleaved ? hd / 8 : rot / 16 + (hd - rot) / 8;
        // (with a bias every head brings loads of its own: the heads are shared out wider)
        const int n_heads_all = write ? H + 2 * G : H;
        const int groups = plain_form ? ROPE_HEAD_GROUPS
                                      : (n_heads_all < 64 ? n_heads_all : 64);
        const int64_t n_units = (int64_t)n_tokens * groups * per_head;
        int64_t blocks = (n_units + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        return (int)sllm_launch_pdl(rope_kv_write_vec_kernel, dim3((unsigned)blocks), dim3(256), 0,
                                    stream, (__nv_bfloat16*)qkv, positions, token_row, cos_t, sin_t,
                                    (__nv_bfloat16*)pages, block_table, table_stride, page_size, H,
                                    G, hd, rotate, interleaved, write, n_units, bias, rot, groups);
    }
    if (dtype == 1)
        return (int)sllm_launch_pdl(rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(threads), 0,
                                    stream, (__nv_bfloat16*)qkv, positions, token_row, cos_t, sin_t,
                                    (__nv_bfloat16*)pages, block_table, table_stride, page_size, H,
                                    G, hd, rotate, interleaved, write, heads_per_block, bias, rot);
    return (int)cudaErrorInvalidValue;
}

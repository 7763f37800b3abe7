// Dynamic Tanh in the place of a norm: dyt(x) = tanh(alpha * x) * w + b, element by element,
// with one scalar alpha and two vectors per norm.  No mean and no variance is computed, so
// every element is independent of its row and several norms chain inside one kernel.
//
//   * sllm_dyt_norm: out = dyt(stream) for all tokens or for a gathered list of rows, and,
//     with a mixing vector mu, the token shift on the way:
//         h_t <- h_t + (h_{t-1} - h_t) * mu
//     where h_{t-1} is the previous token's dyt(stream) (recomputed from the previous row of
//     the stream inside a step, read from the request's state slot for a row's first token;
//     zeros at a sequence's start, which is what a fresh slot holds).  A row that brings one
//     token stores its h into the slot itself; rows of several tokens are stored by
//     sllm_dyt_state_update, a launch of its own, because a row's first token reads the slot
//     that its last token replaces.
//   * sllm_dyt_add: stream += dyt_a(delta) and, optionally, out = dyt_b(stream): the norm on
//     a branch's output and the norm in front of the next branch in one pass.
//
// The stream is 32-bit, all arithmetic is 32-bit with one rounding to T (float or bfloat16).
#include "common.cuh"

namespace sllm {

// tanh in 32-bit.  FAST (the serving path, whose results are rounded to bfloat16 or join a
// stream that bfloat16 products feed): 1 - 2 / (exp(2x) + 1) with the hardware's exponential
// and reciprocal, absolute error about 1e-7, a sixth of the instructions of tanhf (which took
// as long as the kernels' memory traffic).  The 32-bit path keeps tanhf.
template <bool FAST>
__device__ __forceinline__ float tanh32(float x) {
    if (FAST) return 1.0f - __fdividef(2.0f, __expf(2.0f * x) + 1.0f);
    return tanhf(x);
}
template <typename T> struct Serving { static constexpr bool value = false; };
template <> struct Serving<__nv_bfloat16> { static constexpr bool value = true; };

struct Dyt {
    float alpha;
    const float* w;
    const float* b;
    template <bool FAST>
    __device__ __forceinline__ float eval(float x, int e) const {
        return fmaf(tanh32<FAST>(alpha * x), w[e], b[e]);
    }
};

// One thread per element.  index (may be null): the rows of the stream to norm into out[0..n).
template <typename T>
__global__ void dyt_norm_kernel(const float* __restrict__ resid, const int* __restrict__ index,
                                int64_t n_elems, int d, Dyt norm, const float* __restrict__ mu,
                                float* __restrict__ state, const int* __restrict__ token_row,
                                const int* __restrict__ row_start,
                                const int* __restrict__ row_slot, T* __restrict__ out,
                                int write) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_elems;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / d;
        const int e = (int)(i - n * d);
        const int64_t src = index ? index[n] : n;
        constexpr bool FAST = Serving<T>::value;
        float h = norm.eval<FAST>(resid[src * d + e], e);
        if (mu != nullptr) {
            const int r = token_row[n];
            if (r >= 0) {   // (a padding token belongs to no row: nothing is mixed in)
                const int t0 = row_start[r];
                float* st = state + (int64_t)row_slot[r] * d + e;
                const float prev = n == t0 ? *st : norm.eval<FAST>(resid[(n - 1) * d + e], e);
                if (write && row_start[r + 1] - t0 == 1) *st = h;
                h = fmaf(prev - h, mu[e], h);
            }
        }
        out[i] = from_float<T>(h);
    }
}

// grid (ceil(d / 256), rows): rows of two tokens or more store dyt(stream) of their last token.
template <bool FAST>
__global__ void dyt_state_update_kernel(const float* __restrict__ resid, int d, Dyt norm,
                                        float* __restrict__ state,
                                        const int* __restrict__ row_start,
                                        const int* __restrict__ row_slot) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int t0 = row_start[r], t1 = row_start[r + 1];
    if (e >= d || t1 - t0 < 2) return;
    state[(int64_t)row_slot[r] * d + e] = norm.eval<FAST>(resid[(int64_t)(t1 - 1) * d + e], e);
}

template <typename T>
__global__ void dyt_add_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                               int64_t n_elems, int d, Dyt post, int has_next, Dyt next,
                               T* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_elems;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int e = (int)(i % d);
        constexpr bool FAST = Serving<T>::value;
        const float x = resid[i] + post.eval<FAST>(to_float(delta[i]), e);
        resid[i] = x;
        if (has_next) out[i] = from_float<T>(next.eval<FAST>(x, e));
    }
}

// Four elements per thread with 16-byte accesses of the stream (d % 4 == 0).
template <typename T> struct Out4;
template <> struct Out4<float> {
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
};
template <> struct Out4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        uint2 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
        h[0] = __floats2bfloat162_rn(v[0], v[1]);
        h[1] = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = r;
    }
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
        v[0] = __low2float(h[0]); v[1] = __high2float(h[0]);
        v[2] = __low2float(h[1]); v[3] = __high2float(h[1]);
    }
};

// (The gain, the offset and the mixing vector come as 16-byte loads, and the previous token's
// row of the stream is requested together with the token's own, before the row's bookkeeping
// says whether it is needed: a thread's loads make one round trip, two for a row's first token.)
template <typename T>
__global__ void dyt_norm_vec_kernel(const float* __restrict__ resid,
                                    const int* __restrict__ index, int d,
                                    Dyt norm, const float* __restrict__ mu,
                                    float* __restrict__ state, const int* __restrict__ token_row,
                                    const int* __restrict__ row_start,
                                    const int* __restrict__ row_slot, T* __restrict__ out,
                                    int write) {
    pdl_wait();
    pdl_trigger();
    constexpr bool FAST = Serving<T>::value;
    // grid (tokens, blocks of 4-feature units): no thread divides to find its place
    const int64_t n = blockIdx.x;
    const int e = (int)(blockIdx.y * blockDim.x + threadIdx.x) << 2;
    if (e < d) {
        const int64_t src = index ? index[n] : n;
        float x[4], h[4], w[4], b[4], prev[4] = {0.f, 0.f, 0.f, 0.f}, m[4];
        Out4<float>::load(resid + src * d + e, x);
        Out4<float>::load(norm.w + e, w);
        Out4<float>::load(norm.b + e, b);
        int r = -1;
        if (mu != nullptr) {
            r = token_row[n];
            if (n > 0) Out4<float>::load(resid + (n - 1) * d + e, prev);
            Out4<float>::load(mu + e, m);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) h[q] = fmaf(tanh32<FAST>(norm.alpha * x[q]), w[q], b[q]);
        if (r >= 0) {   // (a padding token belongs to no row: nothing is mixed in)
            const int t0 = row_start[r];
            float* st = state + (int64_t)row_slot[r] * d + e;
            if (n == t0) {
                Out4<float>::load(st, prev);
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    prev[q] = fmaf(tanh32<FAST>(norm.alpha * prev[q]), w[q], b[q]);
            }
            if (write && row_start[r + 1] - t0 == 1) Out4<float>::store(st, h);
#pragma unroll
            for (int q = 0; q < 4; ++q) h[q] = fmaf(prev[q] - h[q], m[q], h[q]);
        }
        Out4<T>::store(out + n * d + e, h);
    }
}

template <typename T>
__global__ void dyt_add_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   int d, Dyt post, int has_next, Dyt next, T* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    const int e = (int)(blockIdx.y * blockDim.x + threadIdx.x) << 2;
    if (e >= d) return;
    const int64_t at = (int64_t)blockIdx.x * d + e;
    float x[4], y[4], w[4], b[4];
    Out4<float>::load(resid + at, x);
    Out4<T>::load(delta + at, y);
    Out4<float>::load(post.w + e, w);
    Out4<float>::load(post.b + e, b);
#pragma unroll
    for (int q = 0; q < 4; ++q)
        x[q] += fmaf(tanh32<Serving<T>::value>(post.alpha * y[q]), w[q], b[q]);
    Out4<float>::store(resid + at, x);
    if (has_next) {
        Out4<float>::load(next.w + e, w);
        Out4<float>::load(next.b + e, b);
#pragma unroll
        for (int q = 0; q < 4; ++q)
            y[q] = fmaf(tanh32<Serving<T>::value>(next.alpha * x[q]), w[q], b[q]);
        Out4<T>::store(out + at, y);
    }
}

// Blocks of up to 256 threads over the 4-feature units of a row.
static inline void row_launch(int d, dim3& grid, dim3& block, int n_rows) {
    const int units = d / 4;
    int threads = 32;
    while (threads < 256 && threads < units) threads <<= 1;
    block = dim3(threads);
    grid = dim3(n_rows, (units + threads - 1) / threads);
}

static inline int grid_for(int64_t n_items) {
    int64_t blocks = (n_items + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace sllm

using namespace sllm;

// dtype of out: 0 = float32, 1 = bfloat16.  index (may be null) gathers rows and excludes mu.
SLLM_EXPORT int sllm_dyt_norm(const float* resid, const int* index, int n_out, int d, float alpha,
                              const float* w, const float* b, const float* mu, float* state,
                              const int* token_row, const int* row_start, const int* row_slot,
                              void* out, int write, int dtype, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (d <= 0 || (mu != nullptr && (index != nullptr || state == nullptr || token_row == nullptr ||
                                     row_start == nullptr || row_slot == nullptr)))
        return (int)cudaErrorInvalidValue;
    const Dyt norm{alpha, w, b};
    const bool vec = d % 4 == 0 &&
        !(((uintptr_t)resid | (uintptr_t)out | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)w |
           (uintptr_t)b) & 15);
    cudaError_t err;
    if (vec) {
        dim3 grid, block;
        row_launch(d, grid, block, n_out);
        if (grid.y > 65535) return (int)cudaErrorInvalidValue;
        if (dtype == 0)
            err = sllm_launch_pdl(dyt_norm_vec_kernel<float>, grid, block, 0, stream, resid, index,
                                  d, norm, mu, state, token_row, row_start, row_slot, (float*)out,
                                  write);
        else if (dtype == 1)
            err = sllm_launch_pdl(dyt_norm_vec_kernel<__nv_bfloat16>, grid, block, 0, stream, resid,
                                  index, d, norm, mu, state, token_row, row_start, row_slot,
                                  (__nv_bfloat16*)out, write);
        else
            return (int)cudaErrorInvalidValue;
        return (int)err;
    }
    const int64_t elems = (int64_t)n_out * d;
    if (dtype == 0)
        err = sllm_launch_pdl(dyt_norm_kernel<float>, dim3(grid_for(elems)), dim3(256), 0, stream,
                              resid, index, elems, d, norm, mu, state, token_row, row_start,
                              row_slot, (float*)out, write);
    else if (dtype == 1)
        err = sllm_launch_pdl(dyt_norm_kernel<__nv_bfloat16>, dim3(grid_for(elems)), dim3(256), 0,
                              stream, resid, index, elems, d, norm, mu, state, token_row,
                              row_start, row_slot, (__nv_bfloat16*)out, write);
    else
        return (int)cudaErrorInvalidValue;
    return (int)err;
}

SLLM_EXPORT int sllm_dyt_state_update(const float* resid, int d, float alpha, const float* w,
                                      const float* b, float* state, const int* row_start,
                                      const int* row_slot, int n_rows, int dtype,
                                      cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0 || n_rows > 65535) return (int)cudaErrorInvalidValue;
    const Dyt norm{alpha, w, b};
    // (dtype: that of the norm's output in this model, so that what is carried is bit for bit
    // what the norm kernel forms for a token inside a step)
    if (dtype == 1)
        return (int)sllm_launch_pdl(dyt_state_update_kernel<true>, dim3((d + 255) / 256, n_rows),
                                    dim3(256), 0, stream, resid, d, norm, state, row_start,
                                    row_slot);
    return (int)sllm_launch_pdl(dyt_state_update_kernel<false>, dim3((d + 255) / 256, n_rows),
                                dim3(256), 0, stream, resid, d, norm, state, row_start, row_slot);
}

// next_w null: no second norm, out is not written.
SLLM_EXPORT int sllm_dyt_add(float* resid, const void* delta, int n_tokens, int d, float alpha,
                             const float* w, const float* b, float next_alpha,
                             const float* next_w, const float* next_b, void* out, int dtype,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || (next_w != nullptr && (next_b == nullptr || out == nullptr)))
        return (int)cudaErrorInvalidValue;
    const Dyt post{alpha, w, b}, next{next_alpha, next_w, next_b};
    const int has_next = next_w != nullptr;
    const bool vec = d % 4 == 0 &&
        !(((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)out | (uintptr_t)w | (uintptr_t)b |
           (uintptr_t)next_w | (uintptr_t)next_b) & 15);
    cudaError_t err;
    if (vec) {
        dim3 grid, block;
        row_launch(d, grid, block, n_tokens);
        if (grid.y > 65535) return (int)cudaErrorInvalidValue;
        if (dtype == 0)
            err = sllm_launch_pdl(dyt_add_vec_kernel<float>, grid, block, 0, stream, resid,
                                  (const float*)delta, d, post, has_next, next, (float*)out);
        else if (dtype == 1)
            err = sllm_launch_pdl(dyt_add_vec_kernel<__nv_bfloat16>, grid, block, 0, stream, resid,
                                  (const __nv_bfloat16*)delta, d, post, has_next, next,
                                  (__nv_bfloat16*)out);
        else
            return (int)cudaErrorInvalidValue;
        return (int)err;
    }
    const int64_t elems = (int64_t)n_tokens * d;
    if (dtype == 0)
        err = sllm_launch_pdl(dyt_add_kernel<float>, dim3(grid_for(elems)), dim3(256), 0, stream,
                              resid, (const float*)delta, elems, d, post, has_next, next,
                              (float*)out);
    else if (dtype == 1)
        err = sllm_launch_pdl(dyt_add_kernel<__nv_bfloat16>, dim3(grid_for(elems)), dim3(256), 0,
                              stream, resid, (const __nv_bfloat16*)delta, elems, d, post, has_next,
                              next, (__nv_bfloat16*)out);
    else
        return (int)cudaErrorInvalidValue;
    return (int)err;
}

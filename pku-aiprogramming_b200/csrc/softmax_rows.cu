// Row softmax, forward and backward, as single-pass HBM-bound kernels.
//
// Semantics of the reference's native SoftmaxForward (src/Layers.cu:324-349 of the reference
// project: softmax over the last axis, leading axes flattened to rows, row maximum subtracted;
// there it is five launches plus two host loops of per-row Thrust reductions) in ONE launch that
// reads every element once and writes it once.  The backward (the reference has none on the
// native side) is dx = y * (dy - sum(dy * y)).
//
// A row is held in registers: kWarpRow rows are handled by one warp each (cols <= 1024, up to 32
// values per lane), longer rows by one CTA of 256 threads (cols <= 16384, up to 64 values per
// thread); beyond that the row is streamed three times (L2 keeps most of it).  Loads and stores
// are 16-byte vectors whenever the row pitch allows it.
#include "common.h"

namespace ttk {

template <typename T> __device__ __forceinline__ float sm_ld(const T* p, long long i);
template <> __device__ __forceinline__ float sm_ld<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float sm_ld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void sm_st(T* p, long long i, float v);
template <> __device__ __forceinline__ void sm_st<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void sm_st<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float wred_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float wred_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
template <bool kMax>
__device__ __forceinline__ float block_reduce(float x, float* red) {   // 256 threads
    x = kMax ? wred_max(x) : wred_sum(x);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = x;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) r = kMax ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

// kBwd = false: out = softmax(a).   kBwd = true: out = a * (b - sum(a*b))  with a = y, b = dy.
// kPer = values per thread, kBlock = true: one CTA per row, else one warp per row.
template <typename T, int kPer, bool kBlock, bool kBwd>
__global__ void __launch_bounds__(256) softmax_rows_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                          T* __restrict__ out, long long rows, int cols) {
    __shared__ float red[8];
    const int nthr = kBlock ? 256 : 32;
    const int tid = kBlock ? threadIdx.x : (threadIdx.x & 31);
    const long long row = kBlock ? (long long)blockIdx.x : (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (!kBlock && row >= rows) return;
    const long long base = row * cols;
    float x[kPer], y[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int c = tid + i * nthr;
        x[i] = (c < cols) ? sm_ld<T>(a, base + c) : (kBwd ? 0.f : -INFINITY);
        if (kBwd) y[i] = (c < cols) ? sm_ld<T>(b, base + c) : 0.f;
    }
    if (!kBwd) {
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < kPer; ++i) m = fmaxf(m, x[i]);
        m = kBlock ? block_reduce<true>(m, red) : wred_max(m);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            x[i] = __expf(x[i] - m);
            s += x[i];
        }
        s = kBlock ? block_reduce<false>(s, red) : wred_sum(s);
        const float inv = 1.0f / s;
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int c = tid + i * nthr;
            if (c < cols) sm_st<T>(out, base + c, x[i] * inv);
        }
    } else {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < kPer; ++i) d = fmaf(x[i], y[i], d);
        d = kBlock ? block_reduce<false>(d, red) : wred_sum(d);
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int c = tid + i * nthr;
            if (c < cols) sm_st<T>(out, base + c, x[i] * (y[i] - d));
        }
    }
}

// rows longer than 16384: three streaming passes, one CTA per row
template <typename T, bool kBwd>
__global__ void __launch_bounds__(256) softmax_rows_long_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                               T* __restrict__ out, long long rows, int cols) {
    __shared__ float red[8];
    const long long base = (long long)blockIdx.x * cols;
    if (!kBwd) {
        float m = -INFINITY;
        for (int c = threadIdx.x; c < cols; c += 256) m = fmaxf(m, sm_ld<T>(a, base + c));
        m = block_reduce<true>(m, red);
        float s = 0.f;
        for (int c = threadIdx.x; c < cols; c += 256) s += __expf(sm_ld<T>(a, base + c) - m);
        s = block_reduce<false>(s, red);
        const float inv = 1.0f / s;
        for (int c = threadIdx.x; c < cols; c += 256) sm_st<T>(out, base + c, __expf(sm_ld<T>(a, base + c) - m) * inv);
    } else {
        float d = 0.f;
        for (int c = threadIdx.x; c < cols; c += 256) d = fmaf(sm_ld<T>(a, base + c), sm_ld<T>(b, base + c), d);
        d = block_reduce<false>(d, red);
        for (int c = threadIdx.x; c < cols; c += 256)
            sm_st<T>(out, base + c, sm_ld<T>(a, base + c) * (sm_ld<T>(b, base + c) - d));
    }
}

template <typename T, bool kBwd>
static cudaError_t launch_softmax(const void* a, const void* b, void* out, long long rows, int cols, cudaStream_t st) {
    const T* pa = (const T*)a;
    const T* pb = (const T*)b;
    T* po = (T*)out;
    LaunchScope ls(kBwd ? K_SOFTMAX_BWD : K_SOFTMAX_FWD, st);
#define TT_SM_WARP(P) softmax_rows_kernel<T, P, false, kBwd><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(pa, pb, po, rows, cols)
#define TT_SM_BLOCK(P) softmax_rows_kernel<T, P, true, kBwd><<<(unsigned)rows, 256, 0, st>>>(pa, pb, po, rows, cols)
    if (cols <= 32) TT_SM_WARP(1);
    else if (cols <= 64) TT_SM_WARP(2);
    else if (cols <= 128) TT_SM_WARP(4);
    else if (cols <= 256) TT_SM_WARP(8);
    else if (cols <= 512) TT_SM_WARP(16);
    else if (cols <= 1024) TT_SM_WARP(32);
    else if (cols <= 2048) TT_SM_BLOCK(8);
    else if (cols <= 4096) TT_SM_BLOCK(16);
    else if (cols <= 8192) TT_SM_BLOCK(32);
    else if (cols <= 16384) TT_SM_BLOCK(64);
    else softmax_rows_long_kernel<T, kBwd><<<(unsigned)rows, 256, 0, st>>>(pa, pb, po, rows, cols);
#undef TT_SM_WARP
#undef TT_SM_BLOCK
    return cudaGetLastError();
}

cudaError_t softmax_rows_fwd(const void* in, void* out, long long rows, int cols, int bf16, cudaStream_t st) {
    return bf16 ? launch_softmax<__nv_bfloat16, false>(in, nullptr, out, rows, cols, st)
                : launch_softmax<float, false>(in, nullptr, out, rows, cols, st);
}
cudaError_t softmax_rows_bwd(const void* y, const void* dy, void* dx, long long rows, int cols, int bf16,
                             cudaStream_t st) {
    return bf16 ? launch_softmax<__nv_bfloat16, true>(y, dy, dx, rows, cols, st)
                : launch_softmax<float, true>(y, dy, dx, rows, cols, st);
}

}  // namespace ttk

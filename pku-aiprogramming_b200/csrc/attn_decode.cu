// Split-KV single-query attention (decode): out[bh] = softmax(scale * q[bh] K[bh]^T) V[bh].
//
// The work is HBM-bound (one FMA per byte of K/V), so the kernel is organised around
// streaming every K and V row exactly once with 16-byte loads that bypass L1:
//   - a unit = (slice, key range); units are laid out so that neighbouring CTAs read
//     neighbouring memory; the number of key ranges per slice is chosen so that there are
//     many more units than resident CTAs (small tail);
//   - D/8 lanes share one key row (each lane owns a 16-byte segment = 8 bf16), so a warp
//     load instruction covers 2 (D=128) or 4 (D=64) whole rows, fully coalesced;
//   - each lane keeps kUnroll K vectors and kUnroll V vectors in flight;
//   - scores are reduced across the lanes of a row with xor shuffles, then an online
//     softmax (base 2, fp32) updates the lane's 8 output accumulators;
//   - lanes/warps of a CTA are merged through shared memory; with more than one key range
//     per slice the unnormalised (max, sum, out) partials go to the workspace and a small
//     second kernel merges them.
#include "common.h"
#include <atomic>

namespace ttk {

constexpr int kDecThreads = 256;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ float dot8(const uint4& a, const float (&q)[8]) {
    float s = bf_lo(a.x) * q[0];
    s = fmaf(bf_hi(a.x), q[1], s);
    s = fmaf(bf_lo(a.y), q[2], s);
    s = fmaf(bf_hi(a.y), q[3], s);
    s = fmaf(bf_lo(a.z), q[4], s);
    s = fmaf(bf_hi(a.z), q[5], s);
    s = fmaf(bf_lo(a.w), q[6], s);
    s = fmaf(bf_hi(a.w), q[7], s);
    return s;
}
__device__ __forceinline__ void axpy8(float p, const uint4& a, float (&o)[8]) {
    o[0] = fmaf(p, bf_lo(a.x), o[0]);
    o[1] = fmaf(p, bf_hi(a.x), o[1]);
    o[2] = fmaf(p, bf_lo(a.y), o[2]);
    o[3] = fmaf(p, bf_hi(a.y), o[3]);
    o[4] = fmaf(p, bf_lo(a.z), o[4]);
    o[5] = fmaf(p, bf_hi(a.z), o[5]);
    o[6] = fmaf(p, bf_lo(a.w), o[6]);
    o[7] = fmaf(p, bf_hi(a.w), o[7]);
}

// Merges two online-softmax states (base-2 exponent domain).
__device__ __forceinline__ void merge_state(float& m, float& l, float (&o)[8], float m2, float l2,
                                            const float (&o2)[8]) {
    float mn = fmaxf(m, m2);
    float a = (m == -INFINITY) ? 0.f : exp2f(m - mn);
    float b = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
    l = l * a + l2 * b;
#pragma unroll
    for (int t = 0; t < 8; ++t) o[t] = o[t] * a + o2[t] * b;
    m = mn;
}

// partial layout in the workspace, per unit: [m, l, o[D]] floats
template <int D>
__global__ void __launch_bounds__(kDecThreads, 4)
attn_decode_bf16_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                        const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ lse, float* __restrict__ partial, int L, int splits, int chunk,
                        float scale_log2) {
    constexpr int LPR = D / 8;        // lanes per key row
    constexpr int RPI = 32 / LPR;     // rows per warp load instruction
    __shared__ float sm_m[kDecWarps], sm_l[kDecWarps];
    __shared__ float sm_o[kDecWarps][D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPR, seg = lane % LPR;
    const long long unit = blockIdx.x;
    const long long bh = unit / splits;
    const int split = (int)(unit - bh * splits);
    const int k0 = split * chunk;
    const int k1 = min(L, k0 + chunk);

    float qf[8];
    {
        uint4 qv = *reinterpret_cast<const uint4*>(q + bh * D + seg * 8);
        qf[0] = bf_lo(qv.x) * scale_log2; qf[1] = bf_hi(qv.x) * scale_log2;
        qf[2] = bf_lo(qv.y) * scale_log2; qf[3] = bf_hi(qv.y) * scale_log2;
        qf[4] = bf_lo(qv.z) * scale_log2; qf[5] = bf_hi(qv.z) * scale_log2;
        qf[6] = bf_lo(qv.w) * scale_log2; qf[7] = bf_hi(qv.w) * scale_log2;
    }
    const __nv_bfloat16* kb = k + (bh * (long long)L) * D + seg * 8;
    const __nv_bfloat16* vb = v + (bh * (long long)L) * D + seg * 8;
    float m = -INFINITY, l = 0.f, o[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) o[t] = 0.f;

    constexpr int kRowsPerIter = kDecWarps * RPI * kUnroll;   // rows a CTA consumes per iteration
    for (int base = k0 + warp * (RPI * kUnroll); base < k1; base += kRowsPerIter) {
        uint4 kv[kUnroll], vv[kUnroll];
        bool ok[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int r = base + u * RPI + sub;
            ok[u] = r < k1;
            int rr = ok[u] ? r : k0;   // any valid row; its score is discarded below
            kv[u] = ld_stream16(kb + (long long)rr * D);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int r = base + u * RPI + sub;
            int rr = ok[u] ? r : k0;
            vv[u] = ld_stream16(vb + (long long)rr * D);
        }
        float s[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            float x = dot8(kv[u], qf);
#pragma unroll
            for (int off = LPR / 2; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
            s[u] = ok[u] ? x : -INFINITY;
        }
        float mx = s[0];
#pragma unroll
        for (int u = 1; u < kUnroll; ++u) mx = fmaxf(mx, s[u]);
        if (mx > m) {   // uniform across the lanes of a row group
            float corr = (m == -INFINITY) ? 0.f : exp2f(m - mx);
            l *= corr;
#pragma unroll
            for (int t = 0; t < 8; ++t) o[t] *= corr;
            m = mx;
        }
        if (m != -INFINITY) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                float pu = exp2f(s[u] - m);
                l += pu;
                axpy8(pu, vv[u], o);
            }
        }
    }
    // merge the RPI row groups of the warp (states live at lanes with equal `seg`)
#pragma unroll
    for (int off = 16; off >= LPR; off >>= 1) {
        float m2 = __shfl_xor_sync(0xffffffffu, m, off);
        float l2 = __shfl_xor_sync(0xffffffffu, l, off);
        float o2[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) o2[t] = __shfl_xor_sync(0xffffffffu, o[t], off);
        merge_state(m, l, o, m2, l2, o2);
    }
    if (lane < LPR) {
        if (lane == 0) {
            sm_m[warp] = m;
            sm_l[warp] = l;
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) sm_o[warp][seg * 8 + t] = o[t];
    }
    __syncthreads();
    if (threadIdx.x < D) {
        const int d = threadIdx.x;
        float M = sm_m[0];
#pragma unroll
        for (int w = 1; w < kDecWarps; ++w) M = fmaxf(M, sm_m[w]);
        float Lsum = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            float a = (sm_m[w] == -INFINITY) ? 0.f : exp2f(sm_m[w] - M);
            Lsum = fmaf(sm_l[w], a, Lsum);
            O = fmaf(sm_o[w][d], a, O);
        }
        if (splits == 1) {
            out[bh * D + d] = __float2bfloat16_rn(O / Lsum);
            if (d == 0 && lse != nullptr) lse[bh] = (M + log2f(Lsum)) * 0.6931471805599453f;
        } else {
            float* pu = partial + unit * (D + 2);
            pu[2 + d] = O;
            if (d == 0) {
                pu[0] = M;
                pu[1] = Lsum;
            }
        }
    }
}

template <int D>
__global__ void attn_decode_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                         float* __restrict__ lse, int splits) {
    const long long bh = blockIdx.x;
    const int d = threadIdx.x;
    const float* pb = partial + bh * splits * (D + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, pb[s * (D + 2)]);
    float Lsum = 0.f, O = 0.f;
    for (int s = 0; s < splits; ++s) {
        float ms = pb[s * (D + 2)];
        float a = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
        Lsum = fmaf(pb[s * (D + 2) + 1], a, Lsum);
        O = fmaf(pb[s * (D + 2) + 2 + d], a, O);
    }
    out[bh * D + d] = __float2bfloat16_rn(O / Lsum);
    if (d == 0 && lse != nullptr) lse[bh] = (M + log2f(Lsum)) * 0.6931471805599453f;
}

static int env_int(const char* name, int dflt);

DecodePlan attn_decode_plan(const AttnArgs& a) {
    DecodePlan pl{1, a.L, 0};
    if (!(a.bf16 && (a.D == 64 || a.D == 128) && a.S == 1)) return pl;   // SIMT forward handles it
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    const long long resident = (long long)n_sm * 4;
    const long long target = resident * 12;
    long long splits = (target + a.BH - 1) / a.BH;
    long long max_splits = a.L / 256;
    if (max_splits < 1) max_splits = 1;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    int forced = env_int("TT_DECODE_SPLITS", 0);
    if (forced > 0) splits = forced;
    int chunk = (int)((a.L + splits - 1) / splits);
    chunk = (chunk + 63) / 64 * 64;
    splits = (a.L + chunk - 1) / chunk;
    pl.splits = (int)splits;
    pl.chunk = chunk;
    pl.ws_bytes = splits > 1 ? align256((size_t)splits * a.BH * (a.D + 2) * sizeof(float)) : 0;
    return pl;
}

template <int D>
static cudaError_t launch_decode(const AttnArgs& a, const DecodePlan& pl, void* ws, cudaStream_t st,
                                 bool allow_timing = true) {
    const long long units = a.BH * pl.splits;
    {
        LaunchScope ls(K_DECODE, st, allow_timing);
        attn_decode_bf16_kernel<D><<<(unsigned)units, kDecThreads, 0, st>>>(
            (const __nv_bfloat16*)a.q, (const __nv_bfloat16*)a.k, (const __nv_bfloat16*)a.v, (__nv_bfloat16*)a.out,
            a.lse, (float*)ws, a.L, pl.splits, pl.chunk, a.scale * 1.4426950408889634f);
    }
    if (pl.splits > 1) {
        LaunchScope ls(K_DECODE_MERGE, st, allow_timing);
        attn_decode_merge_kernel<D><<<(unsigned)a.BH, D, 0, st>>>((const float*)ws, (__nv_bfloat16*)a.out, a.lse,
                                                                  pl.splits);
    }
    return cudaGetLastError();
}

cudaError_t attn_decode(const AttnArgs& a, const DecodePlan& pl, void* ws, cudaStream_t st) {
    if (a.bf16 && a.S == 1 && a.D == 128) return launch_decode<128>(a, pl, ws, st);
    if (a.bf16 && a.S == 1 && a.D == 64) return launch_decode<64>(a, pl, ws, st);
    return attn_fwd_simt(a, st);
}

// ------------------------------------------------------------------------------------------
// Variant for callers that must not allocate device memory: the split-KV partials live in a
// fixed array that is part of this library's device image.  Every context that loads the
// library carries these bytes until it exits, whether or not this path is ever called.
constexpr size_t kStaticScratchBytes = (size_t)8 << 20;   // 8 MiB
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not a device address: the
// address a kernel can use has to be asked for, per device, with that device current.
constexpr int kMaxDevices = 64;
static void* g_static_scratch_addr[kMaxDevices];
static std::atomic<int> g_static_scratch_ready[kMaxDevices];

size_t attn_decode_static_capacity() { return kStaticScratchBytes; }

cudaError_t attn_decode_static(const AttnArgs& a, const DecodePlan& pl, cudaStream_t st, bool* too_big) {
    *too_big = pl.ws_bytes > kStaticScratchBytes;
    if (*too_big) return cudaSuccess;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!g_static_scratch_ready[dev].load(std::memory_order_acquire)) {
        // first call on this device: resolve the device address of the array
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_scratch_addr[dev] = p;
        g_static_scratch_ready[dev].store(1, std::memory_order_release);
    }
    void* scratch = g_static_scratch_addr[dev];
    // Nothing in the array has to start at zero: every partial the merge kernel reads is
    // written by the first kernel of the same call.
    if (a.D == 128) return launch_decode<128>(a, pl, scratch, st, /*allow_timing=*/false);
    return launch_decode<64>(a, pl, scratch, st, /*allow_timing=*/false);
}

}  // namespace ttk

#include <stdlib.h>
namespace ttk {
static int env_int(const char* name, int dflt) {
    const char* s = getenv(name);
    return (s && *s) ? atoi(s) : dflt;
}
}  // namespace ttk

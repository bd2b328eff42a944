// SIMT attention kernels with true fp32 FMA arithmetic (no TF32, no tensor cores).
//
// They serve the fp32 dtype, whose tolerance (1e-5 relative) rules out tensor-core
// formats, and every bf16 shape the tcgen05 kernels do not cover (head dims other than
// 64/128).  Inputs of either dtype are widened to fp32 in shared memory; all dot
// products, the softmax and the accumulators are fp32.
//
// Two forms of each kernel (forward, dQ pass, dK/dV pass):
//   register-tiled (head dims that are multiples of 4 up to 128, vector-aligned tensors): a block owns
//     64 "rows" and walks the "columns" in tiles of 64; each of its 16 x 16 threads holds a 4 x 4 patch
//     of scores, so a 128-bit shared-memory load feeds 16 FMAs; see the sections further down;
//   row-per-lane (any D <= 256): a block owns 32 rows, a warp 4 of them, columns in tiles of 32; lane j
//     of a warp computes the score of its 4 rows against column j; row statistics are warp-shuffle
//     reductions; the D-wide accumulators live in registers, D/32 values per lane.
#include "common.h"
#include <cstdlib>

namespace ttk {

constexpr int kRowsPerBlock = 32;
constexpr int kRowsPerWarp = 4;
constexpr int kColsPerTile = 32;
constexpr int kSimtThreads = 256;

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Copies up to 32 rows of a [n_rows, D] matrix (starting at row0) into shared memory as
// fp32 with row pitch D+1; rows past n_rows are zero-filled.
template <typename T>
__device__ __forceinline__ void stage_rows(float* dst, const T* src, long long row0, long long n_rows, int D,
                                           float mul) {
    const int pitch = D + 1;
    for (int idx = threadIdx.x; idx < 32 * D; idx += blockDim.x) {
        int r = idx / D, d = idx - r * D;
        long long gr = row0 + r;
        float x = 0.f;
        if (gr < n_rows) x = to_f32<T>(src[gr * D + d]) * mul;
        dst[r * pitch + d] = x;
    }
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// ------------------------------------------------------------------------------- forward
template <typename T, int NV>
__global__ void __launch_bounds__(kSimtThreads) attn_fwd_simt_kernel(const T* __restrict__ q,
                                                                      const T* __restrict__ k,
                                                                      const T* __restrict__ v, T* __restrict__ out,
                                                                      float* __restrict__ lse, int S, int L, int D,
                                                                      int causal, float scale, int group, const int* __restrict__ kv_lens, int H) {
    extern __shared__ float smem[];
    const int pitch = D + 1;
    float* sQ = smem;
    float* sK = sQ + 32 * pitch;
    float* sV = sK + 32 * pitch;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = (S + kRowsPerBlock - 1) / kRowsPerBlock;
    const long long bh = blockIdx.x / nblk;
    const int row0 = (int)(blockIdx.x % nblk) * kRowsPerBlock;
    const int off = L - S;
    q += bh * (long long)S * D;
    k += (bh / group) * (long long)L * D;   // grouped heads: query slice bh reads key/value slice bh / group
    v += (bh / group) * (long long)L * D;
    out += bh * (long long)S * D;

    stage_rows<T>(sQ, q, row0, S, D, 1.0f);
    float m[kRowsPerWarp], l[kRowsPerWarp], o[kRowsPerWarp][NV];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int t = 0; t < NV; ++t) o[r][t] = 0.f;
    }
    const int Lv = valid_keys(kv_lens, bh / H, L);            // keys beyond it are padding
    int last_row = min(row0 + kRowsPerBlock, S) - 1;
    int col_end = causal ? min(Lv, last_row + off + 1) : Lv;  // exclusive
    for (int c0 = 0; c0 < col_end; c0 += kColsPerTile) {
        __syncthreads();
        stage_rows<T>(sK, k, c0, L, D, 1.0f);
        stage_rows<T>(sV, v, c0, L, D, 1.0f);
        __syncthreads();
        float s[kRowsPerWarp] = {0.f, 0.f, 0.f, 0.f};
        const float* kr = sK + lane * pitch;
        for (int d = 0; d < D; ++d) {
            float kd = kr[d];
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) s[r] = fmaf(sQ[(warp * kRowsPerWarp + r) * pitch + d], kd, s[r]);
        }
        const int col = c0 + lane;
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int row = row0 + warp * kRowsPerWarp + r;
            float sv = s[r] * scale;
            bool valid = col < Lv && (!causal || col <= row + off);
            sv = valid ? sv : -INFINITY;
            float mnew = fmaxf(m[r], warp_max(sv));
            float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - mnew);
            float p = (mnew == -INFINITY) ? 0.f : expf(sv - mnew);
            l[r] = l[r] * corr + warp_sum(p);
            m[r] = mnew;
#pragma unroll
            for (int t = 0; t < NV; ++t) o[r][t] *= corr;
            for (int jj = 0; jj < kColsPerTile; ++jj) {
                float pj = __shfl_sync(0xffffffffu, p, jj);
#pragma unroll
                for (int t = 0; t < NV; ++t) {
                    int d = lane + 32 * t;
                    if (d < D) o[r][t] = fmaf(pj, sV[jj * pitch + d], o[r][t]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int row = row0 + warp * kRowsPerWarp + r;
        if (row >= S) continue;
        float inv = 1.0f / l[r];
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            int d = lane + 32 * t;
            if (d < D) out[(long long)row * D + d] = from_f32<T>(o[r][t] * inv);
        }
        if (lse != nullptr && lane == 0) lse[bh * S + row] = m[r] + logf(l[r]);
    }
}

// --------------------------------------------------------------- backward: delta = rowsum(dO * O)
template <typename T>
__global__ void attn_bwd_delta_kernel(const T* __restrict__ out, const T* __restrict__ dout,
                                      float* __restrict__ delta, long long n_rows, int D) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long row = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= n_rows) return;
    float acc = 0.f;
    for (int d = lane; d < D; d += 32) acc = fmaf(to_f32<T>(out[row * D + d]), to_f32<T>(dout[row * D + d]), acc);
    acc = warp_sum(acc);
    if (lane == 0) delta[row] = acc;
}

// --------------------------------------------------------------- backward: dQ (rows = queries)
template <typename T, int NV>
__global__ void __launch_bounds__(kSimtThreads) attn_bwd_dq_simt_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ dout,
    const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dq, int S, int L, int D,
    int causal, float scale, int group, const int* __restrict__ kv_lens, int H) {
    extern __shared__ float smem[];
    const int pitch = D + 1;
    float* sQ = smem;
    float* sdO = sQ + 32 * pitch;
    float* sK = sdO + 32 * pitch;
    float* sV = sK + 32 * pitch;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = (S + kRowsPerBlock - 1) / kRowsPerBlock;
    const long long bh = blockIdx.x / nblk;
    const int row0 = (int)(blockIdx.x % nblk) * kRowsPerBlock;
    const int off = L - S;
    q += bh * (long long)S * D;
    dout += bh * (long long)S * D;
    dq += bh * (long long)S * D;
    k += (bh / group) * (long long)L * D;
    v += (bh / group) * (long long)L * D;
    lse += bh * S;
    delta += bh * S;

    stage_rows<T>(sQ, q, row0, S, D, 1.0f);
    stage_rows<T>(sdO, dout, row0, S, D, 1.0f);
    float acc[kRowsPerWarp][NV], row_lse[kRowsPerWarp], row_delta[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        int row = row0 + warp * kRowsPerWarp + r;
        row_lse[r] = row < S ? lse[row] : 0.f;
        row_delta[r] = row < S ? delta[row] : 0.f;
#pragma unroll
        for (int t = 0; t < NV; ++t) acc[r][t] = 0.f;
    }
    const int Lv = valid_keys(kv_lens, bh / H, L);
    int last_row = min(row0 + kRowsPerBlock, S) - 1;
    int col_end = causal ? min(Lv, last_row + off + 1) : Lv;
    for (int c0 = 0; c0 < col_end; c0 += kColsPerTile) {
        __syncthreads();
        stage_rows<T>(sK, k, c0, L, D, 1.0f);
        stage_rows<T>(sV, v, c0, L, D, 1.0f);
        __syncthreads();
        float s[kRowsPerWarp] = {0.f, 0.f, 0.f, 0.f}, dp[kRowsPerWarp] = {0.f, 0.f, 0.f, 0.f};
        const float* kr = sK + lane * pitch;
        const float* vr = sV + lane * pitch;
        for (int d = 0; d < D; ++d) {
            float kd = kr[d], vd = vr[d];
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                int rr = (warp * kRowsPerWarp + r) * pitch + d;
                s[r] = fmaf(sQ[rr], kd, s[r]);
                dp[r] = fmaf(sdO[rr], vd, dp[r]);
            }
        }
        const int col = c0 + lane;
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int row = row0 + warp * kRowsPerWarp + r;
            bool valid = col < Lv && row < S && (!causal || col <= row + off);
            float p = valid ? expf(s[r] * scale - row_lse[r]) : 0.f;
            float ds = p * (dp[r] - row_delta[r]);
            for (int jj = 0; jj < kColsPerTile; ++jj) {
                float dsj = __shfl_sync(0xffffffffu, ds, jj);
#pragma unroll
                for (int t = 0; t < NV; ++t) {
                    int d = lane + 32 * t;
                    if (d < D) acc[r][t] = fmaf(dsj, sK[jj * pitch + d], acc[r][t]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int row = row0 + warp * kRowsPerWarp + r;
        if (row >= S) continue;
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            int d = lane + 32 * t;
            if (d < D) dq[(long long)row * D + d] = from_f32<T>(acc[r][t] * scale);
        }
    }
}

// --------------------------------------------------------------- backward: dK, dV (rows = keys)
template <typename T, int NV>
__global__ void __launch_bounds__(kSimtThreads) attn_bwd_dkv_simt_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ dout,
    const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dk, T* __restrict__ dv, int S,
    int L, int D, int causal, float scale, int group, const int* __restrict__ kv_lens, int H) {
    extern __shared__ float smem[];
    const int pitch = D + 1;
    float* sK = smem;
    float* sV = sK + 32 * pitch;
    float* sQ = sV + 32 * pitch;
    float* sdO = sQ + 32 * pitch;
    float* sLse = sdO + 32 * pitch;
    float* sDelta = sLse + 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = (L + kRowsPerBlock - 1) / kRowsPerBlock;
    const long long bh = blockIdx.x / nblk;
    const int key0 = (int)(blockIdx.x % nblk) * kRowsPerBlock;
    const int off = L - S;
    // bh is the key/value slice; its `group` query heads are slices bh*group .. bh*group+group-1
    q += bh * group * (long long)S * D;
    dout += bh * group * (long long)S * D;
    k += bh * (long long)L * D;
    v += bh * (long long)L * D;
    dk += bh * (long long)L * D;
    dv += bh * (long long)L * D;
    lse += bh * group * S;
    delta += bh * group * S;

    const int Lv = valid_keys(kv_lens, (bh * group) / H, L);   // padded keys get zero gradients
    stage_rows<T>(sK, k, key0, L, D, 1.0f);
    stage_rows<T>(sV, v, key0, L, D, 1.0f);
    float aK[kRowsPerWarp][NV], aV[kRowsPerWarp][NV];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
        for (int t = 0; t < NV; ++t) aK[r][t] = aV[r][t] = 0.f;
    // first query that can see the first key of this block: i >= key0 - off
    int i_begin = causal ? max(0, key0 - off) : 0;
    i_begin = (i_begin / kColsPerTile) * kColsPerTile;
    for (int hh = 0; hh < group; ++hh, q += (long long)S * D, dout += (long long)S * D, lse += S, delta += S)
    for (int i0 = i_begin; i0 < S; i0 += kColsPerTile) {
        __syncthreads();
        stage_rows<T>(sQ, q, i0, S, D, 1.0f);
        stage_rows<T>(sdO, dout, i0, S, D, 1.0f);
        if (threadIdx.x < 32) {
            int i = i0 + threadIdx.x;
            sLse[threadIdx.x] = i < S ? lse[i] : 0.f;
            sDelta[threadIdx.x] = i < S ? delta[i] : 0.f;
        }
        __syncthreads();
        float s[kRowsPerWarp] = {0.f, 0.f, 0.f, 0.f}, dp[kRowsPerWarp] = {0.f, 0.f, 0.f, 0.f};
        const float* qr = sQ + lane * pitch;
        const float* dor = sdO + lane * pitch;
        for (int d = 0; d < D; ++d) {
            float qd = qr[d], dod = dor[d];
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                int rr = (warp * kRowsPerWarp + r) * pitch + d;
                s[r] = fmaf(sK[rr], qd, s[r]);
                dp[r] = fmaf(sV[rr], dod, dp[r]);
            }
        }
        const int i = i0 + lane;
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int key = key0 + warp * kRowsPerWarp + r;
            bool valid = i < S && key < Lv && (!causal || key <= i + off);
            float p = valid ? expf(s[r] * scale - sLse[lane]) : 0.f;
            float ds = p * (dp[r] - sDelta[lane]);
            for (int jj = 0; jj < kColsPerTile; ++jj) {
                float pj = __shfl_sync(0xffffffffu, p, jj);
                float dsj = __shfl_sync(0xffffffffu, ds, jj);
#pragma unroll
                for (int t = 0; t < NV; ++t) {
                    int d = lane + 32 * t;
                    if (d < D) {
                        aV[r][t] = fmaf(pj, sdO[jj * pitch + d], aV[r][t]);
                        aK[r][t] = fmaf(dsj, sQ[jj * pitch + d], aK[r][t]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int key = key0 + warp * kRowsPerWarp + r;
        if (key >= L) continue;
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            int d = lane + 32 * t;
            if (d < D) {
                dk[(long long)key * D + d] = from_f32<T>(aK[r][t] * scale);
                dv[(long long)key * D + d] = from_f32<T>(aV[r][t]);
            }
        }
    }
}

// ------------------------------------------------------------------- forward, register-tiled
// The forward for head dims that are multiples of 4 up to 128.  A block owns 64 query rows and walks
// the keys in tiles of 64; thread (ty, tx) of the 16 x 16 block holds the 4 x 4 scores of rows
// ty + 16 i against keys tx + 16 j, so every 128-bit shared-memory load feeds 16 FMAs (the
// row-per-lane kernel above fetches one operand per FMA).  The 16 lanes that share a row reduce its
// statistics with shuffles, P goes through shared memory (in place of the K tile), and the same thread accumulates
// O[rows ty + 16 i][4 tx + 64 jj .. + 3], so the rescale factors never leave registers.
constexpr int kTiledM = 64, kTiledN = 64, kTiledThreads = 256, kTiledPPitch = kTiledN + 4;

template <typename T>
__device__ __forceinline__ float4 load4_f32(const T* p);
template <>
__device__ __forceinline__ float4 load4_f32<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load4_f32<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xffff0000u));
}
template <typename T>
__device__ __forceinline__ void store4_f32(T* p, float4 x);
template <>
__device__ __forceinline__ void store4_f32<float>(float* p, float4 x) { *reinterpret_cast<float4*>(p) = x; }
template <>
__device__ __forceinline__ void store4_f32<__nv_bfloat16>(__nv_bfloat16* p, float4 x) {
    __nv_bfloat162 a = __floats2bfloat162_rn(x.x, x.y), b = __floats2bfloat162_rn(x.z, x.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}
// 64 rows of a [n_rows, D] matrix from row0 on into shared memory (pitch DP floats), zero past n_rows
template <typename T>
__device__ __forceinline__ void stage_tile64(float* dst, const T* src, long long row0, long long n_rows, int D, int DP) {
    const int d4 = D >> 2;
    for (int idx = threadIdx.x; idx < 64 * d4; idx += kTiledThreads) {
        const int r = idx / d4, c = (idx - r * d4) << 2;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < n_rows) x = load4_f32<T>(src + (row0 + r) * D + c);
        *reinterpret_cast<float4*>(dst + r * DP + c) = x;
    }
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(kTiledThreads, 2) attn_fwd_simt_tiled_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ out,
    float* __restrict__ lse, int S, int L, int D, int causal, float scale, int group, const int* __restrict__ kv_lens,
    int H) {
    constexpr int DP = DMAX + 4;        // pitch: rows 16 bytes apart modulo 128, 128-bit loads conflict-free
    constexpr int NJ = DMAX / 64;       // float4 column groups of O per thread
    extern __shared__ __align__(16) float smem[];
    float* sQ = smem;
    float* sK = sQ + kTiledM * DP;
    float* sV = sK + kTiledN * DP;
    float* sP = sK;   // P takes the K tile's place once the scores are done: three tiles in all, two blocks per SM at D = 128
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int nblk = (S + kTiledM - 1) / kTiledM;
    const long long bh = blockIdx.x / nblk;
    const int row0 = (int)(blockIdx.x % nblk) * kTiledM;
    const int off = L - S;
    q += bh * (long long)S * D;
    k += (bh / group) * (long long)L * D;
    v += (bh / group) * (long long)L * D;
    out += bh * (long long)S * D;

    // columns of sV at and past D are read by the O accumulation (and discarded): keep them finite
    for (int idx = threadIdx.x; idx < kTiledN * DP; idx += kTiledThreads) sV[idx] = 0.f;
    stage_tile64<T>(sQ, q, row0, S, D, DP);
    float m[4], l[4];
    float4 o[4][NJ];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) o[i][jj] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int Lv = valid_keys(kv_lens, bh / H, L);
    const int last_row = min(row0 + kTiledM, S) - 1;
    const int col_end = causal ? min(Lv, last_row + off + 1) : Lv;   // exclusive
    for (int c0 = 0; c0 < col_end; c0 += kTiledN) {
        __syncthreads();   // the previous tile's P V is done (and sQ / the zeroed sV are in place)
        stage_tile64<T>(sK, k, c0, L, D, DP);
        stage_tile64<T>(sV, v, c0, L, D, DP);
        __syncthreads();
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll 2
        for (int d = 0; d < D; d += 4) {
            float4 qa[4], kb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) qa[i] = *reinterpret_cast<const float4*>(sQ + (ty + 16 * i) * DP + d);
#pragma unroll
            for (int j = 0; j < 4; ++j) kb[j] = *reinterpret_cast<const float4*>(sK + (tx + 16 * j) * DP + d);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[i][j] = fmaf(qa[i].x, kb[j].x, s[i][j]);
                    s[i][j] = fmaf(qa[i].y, kb[j].y, s[i][j]);
                    s[i][j] = fmaf(qa[i].z, kb[j].z, s[i][j]);
                    s[i][j] = fmaf(qa[i].w, kb[j].w, s[i][j]);
                }
        }
        __syncthreads();   // every thread has read its K rows: the tile's space now holds P
        float corr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = row0 + ty + 16 * i;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = c0 + tx + 16 * j;
                const bool valid = col < Lv && (!causal || col <= row + off);
                s[i][j] = valid ? s[i][j] * scale : -INFINITY;
                mx = fmaxf(mx, s[i][j]);
            }
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
            const float mnew = fmaxf(m[i], mx);
            corr[i] = (m[i] == -INFINITY) ? 0.f : expf(m[i] - mnew);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p = (mnew == -INFINITY) ? 0.f : expf(s[i][j] - mnew);
                sum += p;
                sP[(ty + 16 * i) * kTiledPPitch + tx + 16 * j] = p;
            }
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
            l[i] = l[i] * corr[i] + sum;
            m[i] = mnew;
#pragma unroll
            for (int jj = 0; jj < NJ; ++jj) {
                o[i][jj].x *= corr[i]; o[i][jj].y *= corr[i]; o[i][jj].z *= corr[i]; o[i][jj].w *= corr[i];
            }
        }
        __syncthreads();   // P complete
#pragma unroll 2
        for (int n = 0; n < kTiledN; n += 4) {
            float pa[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 t = *reinterpret_cast<const float4*>(sP + (ty + 16 * i) * kTiledPPitch + n);
                pa[i][0] = t.x; pa[i][1] = t.y; pa[i][2] = t.z; pa[i][3] = t.w;
            }
#pragma unroll
            for (int nn = 0; nn < 4; ++nn)
#pragma unroll
                for (int jj = 0; jj < NJ; ++jj) {
                    const float4 vb = *reinterpret_cast<const float4*>(sV + (n + nn) * DP + 4 * tx + 64 * jj);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        o[i][jj].x = fmaf(pa[i][nn], vb.x, o[i][jj].x);
                        o[i][jj].y = fmaf(pa[i][nn], vb.y, o[i][jj].y);
                        o[i][jj].z = fmaf(pa[i][nn], vb.z, o[i][jj].z);
                        o[i][jj].w = fmaf(pa[i][nn], vb.w, o[i][jj].w);
                    }
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + ty + 16 * i;
        if (row >= S) continue;
        const float inv = 1.0f / l[i];
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) {
            const int d = 4 * tx + 64 * jj;
            if (d < D)
                store4_f32<T>(out + (long long)row * D + d,
                              make_float4(o[i][jj].x * inv, o[i][jj].y * inv, o[i][jj].z * inv, o[i][jj].w * inv));
        }
        if (lse != nullptr && tx == 0) lse[bh * S + row] = m[i] + logf(l[i]);
    }
}

// ------------------------------------------------------------------ backward, register-tiled
// Same 16 x 16 thread layout as the tiled forward.  A block owns a 64-row tile (queries for dQ, keys
// for dK/dV) held in shared memory together with its partner tensor (dO resp. V) and streams the
// other side in 64-row tiles.  Both score products of a tile pair, S and dP, come out of one pass
// over d; P and dS go through shared memory into the accumulating products.
//
// s[i][j] = a1[row_i] . b1[col_j],  dp[i][j] = a2[row_i] . b2[col_j]   (rows ty + 16 i, cols tx + 16 j)
template <int DP>
__device__ __forceinline__ void tiled_two_products(const float* a1, const float* a2, const float* b1, const float* b2,
                                                   int ty, int tx, int D, float (&s)[4][4], float (&dp)[4][4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.f;
    for (int d = 0; d < D; d += 4) {
        float4 xa[4], xb[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) xa[i] = *reinterpret_cast<const float4*>(a1 + (ty + 16 * i) * DP + d);
#pragma unroll
        for (int j = 0; j < 4; ++j) xb[j] = *reinterpret_cast<const float4*>(b1 + (tx + 16 * j) * DP + d);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                s[i][j] = fmaf(xa[i].x, xb[j].x, s[i][j]);
                s[i][j] = fmaf(xa[i].y, xb[j].y, s[i][j]);
                s[i][j] = fmaf(xa[i].z, xb[j].z, s[i][j]);
                s[i][j] = fmaf(xa[i].w, xb[j].w, s[i][j]);
            }
#pragma unroll
        for (int i = 0; i < 4; ++i) xa[i] = *reinterpret_cast<const float4*>(a2 + (ty + 16 * i) * DP + d);
#pragma unroll
        for (int j = 0; j < 4; ++j) xb[j] = *reinterpret_cast<const float4*>(b2 + (tx + 16 * j) * DP + d);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                dp[i][j] = fmaf(xa[i].x, xb[j].x, dp[i][j]);
                dp[i][j] = fmaf(xa[i].y, xb[j].y, dp[i][j]);
                dp[i][j] = fmaf(xa[i].z, xb[j].z, dp[i][j]);
                dp[i][j] = fmaf(xa[i].w, xb[j].w, dp[i][j]);
            }
    }
}
// acc[i][jj] += sum_n w[row_i][n] * b[n][4 tx + 64 jj ..]   (w: 64 x 64 in shared memory, pitch kTiledPPitch)
template <int DP, int NJ>
__device__ __forceinline__ void tiled_accumulate(const float* w, const float* b, int ty, int tx, float4 (&acc)[4][NJ]) {
#pragma unroll 2
    for (int n = 0; n < kTiledN; n += 4) {
        float pa[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 t = *reinterpret_cast<const float4*>(w + (ty + 16 * i) * kTiledPPitch + n);
            pa[i][0] = t.x; pa[i][1] = t.y; pa[i][2] = t.z; pa[i][3] = t.w;
        }
#pragma unroll
        for (int nn = 0; nn < 4; ++nn)
#pragma unroll
            for (int jj = 0; jj < NJ; ++jj) {
                const float4 vb = *reinterpret_cast<const float4*>(b + (n + nn) * DP + 4 * tx + 64 * jj);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[i][jj].x = fmaf(pa[i][nn], vb.x, acc[i][jj].x);
                    acc[i][jj].y = fmaf(pa[i][nn], vb.y, acc[i][jj].y);
                    acc[i][jj].z = fmaf(pa[i][nn], vb.z, acc[i][jj].z);
                    acc[i][jj].w = fmaf(pa[i][nn], vb.w, acc[i][jj].w);
                }
            }
    }
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(kTiledThreads) attn_bwd_dq_simt_tiled_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ dout,
    const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dq, int S, int L, int D,
    int causal, float scale, int group, const int* __restrict__ kv_lens, int H) {
    constexpr int DP = DMAX + 4, NJ = DMAX / 64;
    extern __shared__ __align__(16) float smem[];
    float* sQ = smem;
    float* sdO = sQ + kTiledM * DP;
    float* sK = sdO + kTiledM * DP;
    float* sV = sK + kTiledN * DP;
    float* sW = sV + kTiledN * DP;       // dS
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int nblk = (S + kTiledM - 1) / kTiledM;
    const long long bh = blockIdx.x / nblk;
    const int row0 = (int)(blockIdx.x % nblk) * kTiledM;
    const int off = L - S;
    q += bh * (long long)S * D;
    dout += bh * (long long)S * D;
    dq += bh * (long long)S * D;
    k += (bh / group) * (long long)L * D;
    v += (bh / group) * (long long)L * D;
    lse += bh * S;
    delta += bh * S;

    // columns of sK at and past D are read by the dQ accumulation (and discarded): keep them finite
    for (int idx = threadIdx.x; idx < kTiledN * DP; idx += kTiledThreads) sK[idx] = 0.f;
    stage_tile64<T>(sQ, q, row0, S, D, DP);
    stage_tile64<T>(sdO, dout, row0, S, D, DP);
    float row_lse[4], row_delta[4];
    float4 acc[4][NJ];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + ty + 16 * i;
        row_lse[i] = row < S ? lse[row] : 0.f;
        row_delta[i] = row < S ? delta[row] : 0.f;
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) acc[i][jj] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int Lv = valid_keys(kv_lens, bh / H, L);
    const int last_row = min(row0 + kTiledM, S) - 1;
    const int col_end = causal ? min(Lv, last_row + off + 1) : Lv;
    for (int c0 = 0; c0 < col_end; c0 += kTiledN) {
        __syncthreads();
        stage_tile64<T>(sK, k, c0, L, D, DP);
        stage_tile64<T>(sV, v, c0, L, D, DP);
        __syncthreads();
        float s[4][4], dp[4][4];
        tiled_two_products<DP>(sQ, sdO, sK, sV, ty, tx, D, s, dp);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = row0 + ty + 16 * i;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = c0 + tx + 16 * j;
                const bool valid = col < Lv && row < S && (!causal || col <= row + off);
                const float p = valid ? expf(s[i][j] * scale - row_lse[i]) : 0.f;
                sW[(ty + 16 * i) * kTiledPPitch + tx + 16 * j] = p * (dp[i][j] - row_delta[i]);
            }
        }
        __syncthreads();
        tiled_accumulate<DP, NJ>(sW, sK, ty, tx, acc);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + ty + 16 * i;
        if (row >= S) continue;
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) {
            const int d = 4 * tx + 64 * jj;
            if (d < D)
                store4_f32<T>(dq + (long long)row * D + d, make_float4(acc[i][jj].x * scale, acc[i][jj].y * scale,
                                                                        acc[i][jj].z * scale, acc[i][jj].w * scale));
        }
    }
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(kTiledThreads) attn_bwd_dkv_simt_tiled_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ dout,
    const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dk, T* __restrict__ dv, int S,
    int L, int D, int causal, float scale, int group, const int* __restrict__ kv_lens, int H) {
    constexpr int DP = DMAX + 4, NJ = DMAX / 64;
    extern __shared__ __align__(16) float smem[];
    float* sK = smem;
    float* sV = sK + kTiledM * DP;
    float* sQ = sV + kTiledM * DP;
    float* sdO = sQ + kTiledN * DP;
    float* sP = sdO + kTiledN * DP;                  // P^T   [key][query]
    float* sW = sP + kTiledM * kTiledPPitch;         // dS^T  [key][query]
    float* sLse = sW + kTiledM * kTiledPPitch;       // [64] of the streamed queries
    float* sDelta = sLse + kTiledN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int nblk = (L + kTiledM - 1) / kTiledM;
    const long long bh = blockIdx.x / nblk;          // key/value slice; its query heads are bh*group ...
    const int key0 = (int)(blockIdx.x % nblk) * kTiledM;
    const int off = L - S;
    q += bh * group * (long long)S * D;
    dout += bh * group * (long long)S * D;
    k += bh * (long long)L * D;
    v += bh * (long long)L * D;
    dk += bh * (long long)L * D;
    dv += bh * (long long)L * D;
    lse += bh * group * S;
    delta += bh * group * S;

    const int Lv = valid_keys(kv_lens, (bh * group) / H, L);   // padded keys get zero gradients
    // columns of sQ / sdO at and past D are read by the accumulations (and discarded): keep them finite
    for (int idx = threadIdx.x; idx < 2 * kTiledN * DP; idx += kTiledThreads) sQ[idx] = 0.f;
    stage_tile64<T>(sK, k, key0, L, D, DP);
    stage_tile64<T>(sV, v, key0, L, D, DP);
    float4 aK[4][NJ], aV[4][NJ];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) aK[i][jj] = aV[i][jj] = make_float4(0.f, 0.f, 0.f, 0.f);
    int i_begin = causal ? max(0, key0 - off) : 0;   // first query that can see this block's first key
    i_begin = (i_begin / kTiledN) * kTiledN;
    for (int hh = 0; hh < group; ++hh, q += (long long)S * D, dout += (long long)S * D, lse += S, delta += S)
        for (int i0 = i_begin; i0 < S; i0 += kTiledN) {
            __syncthreads();
            stage_tile64<T>(sQ, q, i0, S, D, DP);
            stage_tile64<T>(sdO, dout, i0, S, D, DP);
            if (threadIdx.x < kTiledN) {
                const int qi = i0 + threadIdx.x;
                sLse[threadIdx.x] = qi < S ? lse[qi] : 0.f;
                sDelta[threadIdx.x] = qi < S ? delta[qi] : 0.f;
            }
            __syncthreads();
            float s[4][4], dp[4][4];
            tiled_two_products<DP>(sK, sV, sQ, sdO, ty, tx, D, s, dp);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int qi = i0 + tx + 16 * j;
                const float ql = sLse[tx + 16 * j], qd = sDelta[tx + 16 * j];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = key0 + ty + 16 * i;
                    const bool valid = qi < S && key < Lv && (!causal || key <= qi + off);
                    const float p = valid ? expf(s[i][j] * scale - ql) : 0.f;
                    sP[(ty + 16 * i) * kTiledPPitch + tx + 16 * j] = p;
                    sW[(ty + 16 * i) * kTiledPPitch + tx + 16 * j] = p * (dp[i][j] - qd);
                }
            }
            __syncthreads();
            tiled_accumulate<DP, NJ>(sP, sdO, ty, tx, aV);
            tiled_accumulate<DP, NJ>(sW, sQ, ty, tx, aK);
        }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int key = key0 + ty + 16 * i;
        if (key >= L) continue;
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) {
            const int d = 4 * tx + 64 * jj;
            if (d < D) {
                store4_f32<T>(dk + (long long)key * D + d, make_float4(aK[i][jj].x * scale, aK[i][jj].y * scale,
                                                                        aK[i][jj].z * scale, aK[i][jj].w * scale));
                store4_f32<T>(dv + (long long)key * D + d, aV[i][jj]);
            }
        }
    }
}

// ------------------------------------------------------------------------------- launchers
template <typename K>
static cudaError_t set_smem(K kernel, size_t bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <typename T, int NV>
static cudaError_t launch_fwd_simt(const AttnArgs& a, cudaStream_t st) {
    size_t smem = (size_t)3 * 32 * (a.D + 1) * sizeof(float);
    cudaError_t e = set_smem(attn_fwd_simt_kernel<T, NV>, smem);
    if (e != cudaSuccess) return e;
    unsigned grid = (unsigned)(((a.S + kRowsPerBlock - 1) / kRowsPerBlock) * a.BH);
    {
        LaunchScope ls(K_FWD_SIMT, st);
        attn_fwd_simt_kernel<T, NV><<<grid, kSimtThreads, smem, st>>>((const T*)a.q, (const T*)a.k, (const T*)a.v,
                                                                      (T*)a.out, a.lse, a.S, a.L, a.D, a.causal,
                                                                      a.scale, a.group, a.kv_lens, a.H);
    }
    return cudaGetLastError();
}

// the tiled backward kernels: same vector requirements as the tiled forward, for every tensor they touch
static bool simt_tiled_bwd_ok(const AttnArgs& a) {
    const char* e = getenv("TT_SIMT_BWD");
    if (e && e[0] == 'r') return false;
    const uintptr_t mask = a.bf16 ? 7 : 15;
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) |
                           reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.dout) |
                           reinterpret_cast<uintptr_t>(a.dq) | reinterpret_cast<uintptr_t>(a.dk) |
                           reinterpret_cast<uintptr_t>(a.dv);
    return a.D % 4 == 0 && a.D <= 128 && (ptrs & mask) == 0;
}
template <typename T, int DMAX>
static cudaError_t launch_bwd_simt_tiled(const AttnArgs& a, float* delta, cudaStream_t st) {
    const size_t tile = (size_t)64 * (DMAX + 4) * sizeof(float), w = (size_t)64 * kTiledPPitch * sizeof(float);
    const size_t smem_q = 4 * tile + w, smem_kv = 4 * tile + 2 * w + 2 * kTiledN * sizeof(float);
    cudaError_t e = set_smem(attn_bwd_dq_simt_tiled_kernel<T, DMAX>, smem_q);
    if (e != cudaSuccess) return e;
    e = set_smem(attn_bwd_dkv_simt_tiled_kernel<T, DMAX>, smem_kv);
    if (e != cudaSuccess) return e;
    const unsigned gq = (unsigned)(((a.S + kTiledM - 1) / kTiledM) * a.BH);
    {
        LaunchScope ls(K_BWD_SIMT_DQ, st);
        attn_bwd_dq_simt_tiled_kernel<T, DMAX><<<gq, kTiledThreads, smem_q, st>>>(
            (const T*)a.q, (const T*)a.k, (const T*)a.v, (const T*)a.dout, a.lse, delta, (T*)a.dq, a.S, a.L, a.D,
            a.causal, a.scale, a.group, a.kv_lens, a.H);
    }
    const unsigned gk = (unsigned)(((a.L + kTiledM - 1) / kTiledM) * (a.BH / a.group));
    {
        LaunchScope ls(K_BWD_SIMT_DKV, st);
        attn_bwd_dkv_simt_tiled_kernel<T, DMAX><<<gk, kTiledThreads, smem_kv, st>>>(
            (const T*)a.q, (const T*)a.k, (const T*)a.v, (const T*)a.dout, a.lse, delta, (T*)a.dk, (T*)a.dv, a.S,
            a.L, a.D, a.causal, a.scale, a.group, a.kv_lens, a.H);
    }
    return cudaGetLastError();
}

template <typename T, int NV>
static cudaError_t launch_bwd_simt(const AttnArgs& a, float* delta, cudaStream_t st) {
    long long n_rows = a.BH * (long long)a.S;
    {
        LaunchScope ls(K_BWD_SIMT_DELTA, st);
        attn_bwd_delta_kernel<T><<<(unsigned)((n_rows + 7) / 8), 256, 0, st>>>((const T*)a.out, (const T*)a.dout,
                                                                              delta, n_rows, a.D);
    }
    if (simt_tiled_bwd_ok(a)) return a.D <= 64 ? launch_bwd_simt_tiled<T, 64>(a, delta, st) : launch_bwd_simt_tiled<T, 128>(a, delta, st);
    size_t smem_q = (size_t)4 * 32 * (a.D + 1) * sizeof(float);
    size_t smem_kv = smem_q + 64 * sizeof(float);
    cudaError_t e = set_smem(attn_bwd_dq_simt_kernel<T, NV>, smem_q);
    if (e != cudaSuccess) return e;
    e = set_smem(attn_bwd_dkv_simt_kernel<T, NV>, smem_kv);
    if (e != cudaSuccess) return e;
    unsigned gq = (unsigned)(((a.S + kRowsPerBlock - 1) / kRowsPerBlock) * a.BH);
    {
        LaunchScope ls(K_BWD_SIMT_DQ, st);
        attn_bwd_dq_simt_kernel<T, NV><<<gq, kSimtThreads, smem_q, st>>>(
            (const T*)a.q, (const T*)a.k, (const T*)a.v, (const T*)a.dout, a.lse, delta, (T*)a.dq, a.S, a.L, a.D,
            a.causal, a.scale, a.group, a.kv_lens, a.H);
    }
    unsigned gk = (unsigned)(((a.L + kRowsPerBlock - 1) / kRowsPerBlock) * (a.BH / a.group));
    {
        LaunchScope ls(K_BWD_SIMT_DKV, st);
        attn_bwd_dkv_simt_kernel<T, NV><<<gk, kSimtThreads, smem_kv, st>>>(
            (const T*)a.q, (const T*)a.k, (const T*)a.v, (const T*)a.dout, a.lse, delta, (T*)a.dk, (T*)a.dv, a.S,
            a.L, a.D, a.causal, a.scale, a.group, a.kv_lens, a.H);
    }
    return cudaGetLastError();
}

template <typename T, int DMAX>
static cudaError_t launch_fwd_simt_tiled(const AttnArgs& a, cudaStream_t st) {
    const size_t smem = (size_t)(kTiledM + 2 * kTiledN) * (DMAX + 4) * sizeof(float);   // Q, K (then P), V
    cudaError_t e = set_smem(attn_fwd_simt_tiled_kernel<T, DMAX>, smem);
    if (e != cudaSuccess) return e;
    const unsigned grid = (unsigned)(((a.S + kTiledM - 1) / kTiledM) * a.BH);
    {
        LaunchScope ls(K_FWD_SIMT, st);
        attn_fwd_simt_tiled_kernel<T, DMAX><<<grid, kTiledThreads, smem, st>>>(
            (const T*)a.q, (const T*)a.k, (const T*)a.v, (T*)a.out, a.lse, a.S, a.L, a.D, a.causal, a.scale, a.group,
            a.kv_lens, a.H);
    }
    return cudaGetLastError();
}
// the register-tiled forward needs 4-element vectors: D a multiple of 4 and 16-byte (fp32) or 8-byte
// (bf16) aligned tensors; TT_SIMT_FWD=rows keeps the row-per-lane kernel
static bool simt_tiled_ok(const AttnArgs& a) {
    const char* e = getenv("TT_SIMT_FWD");
    if (e && e[0] == 'r') return false;
    const uintptr_t mask = a.bf16 ? 7 : 15;
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) |
                           reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.out);
    return a.D % 4 == 0 && a.D <= 128 && (ptrs & mask) == 0;
}

template <typename T>
static cudaError_t dispatch_fwd(const AttnArgs& a, cudaStream_t st) {
    if (simt_tiled_ok(a)) return a.D <= 64 ? launch_fwd_simt_tiled<T, 64>(a, st) : launch_fwd_simt_tiled<T, 128>(a, st);
    if (a.D <= 32) return launch_fwd_simt<T, 1>(a, st);
    if (a.D <= 64) return launch_fwd_simt<T, 2>(a, st);
    if (a.D <= 128) return launch_fwd_simt<T, 4>(a, st);
    return launch_fwd_simt<T, 8>(a, st);
}
template <typename T>
static cudaError_t dispatch_bwd(const AttnArgs& a, float* delta, cudaStream_t st) {
    if (a.D <= 32) return launch_bwd_simt<T, 1>(a, delta, st);
    if (a.D <= 64) return launch_bwd_simt<T, 2>(a, delta, st);
    if (a.D <= 128) return launch_bwd_simt<T, 4>(a, delta, st);
    return launch_bwd_simt<T, 8>(a, delta, st);
}

cudaError_t attn_fwd_simt(const AttnArgs& a, cudaStream_t st) {
    return a.bf16 ? dispatch_fwd<__nv_bfloat16>(a, st) : dispatch_fwd<float>(a, st);
}
cudaError_t attn_bwd_simt(const AttnArgs& a, float* delta, cudaStream_t st) {
    return a.bf16 ? dispatch_bwd<__nv_bfloat16>(a, delta, st) : dispatch_bwd<float>(a, delta, st);
}
size_t attn_bwd_simt_workspace(const AttnArgs& a) { return align256((size_t)a.BH * a.S * sizeof(float)); }

}  // namespace ttk

// SIMT attention kernels with true fp32 FMA arithmetic (no TF32, no tensor cores).
//
// They serve the fp32 dtype, whose tolerance (1e-5 relative) rules out tensor-core
// formats, and every bf16 shape the tcgen05 kernels do not cover (head dims other than
// 64/128).  Inputs of either dtype are widened to fp32 in shared memory; all dot
// products, the softmax and the accumulators are fp32.
//
// Structure (forward and both backward kernels share it): a block owns 32 "rows", a warp
// owns 4 of them, and the block walks over "columns" in tiles of 32.  Lane j of a warp
// computes the score of its 4 rows against column j; row statistics are warp-shuffle
// reductions; the D-wide accumulators live in registers, D/32 values per lane.
#include "common.h"

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

template <typename T, int NV>
static cudaError_t launch_bwd_simt(const AttnArgs& a, float* delta, cudaStream_t st) {
    long long n_rows = a.BH * (long long)a.S;
    {
        LaunchScope ls(K_BWD_SIMT_DELTA, st);
        attn_bwd_delta_kernel<T><<<(unsigned)((n_rows + 7) / 8), 256, 0, st>>>((const T*)a.out, (const T*)a.dout,
                                                                              delta, n_rows, a.D);
    }
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

template <typename T>
static cudaError_t dispatch_fwd(const AttnArgs& a, cudaStream_t st) {
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

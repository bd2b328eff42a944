// Fully connected layer GEMMs for sm_100a: C[M,N] = op(A) op(B) (+ bias), bf16 in, fp32
// accumulation in tensor memory, bf16 out.
//
// The reference's FcForward / FcBackward (src/Layers.cu:9-79 of the reference project) are
// cublasSgemm calls that create and destroy a handle and synchronise the device per call
// (src/Layers_kernels.cu:10-30), with the bias added by a second rank-1 GEMM against a ones
// vector.  Here one persistent kernel serves the three products of the layer
//     forward   y  = x W + b        A = x  [M,K]  K-major,   B = W  [K,N]  MN-major
//     backward  dx = dy W^T         A = dy [M,N]  K-major,   B = W  [K,N]  K-major (as [N_out rows of K])
//               dW = x^T dy         A = x  [M,K]  MN-major,  B = dy [M,N]  MN-major
// straight from the row-major tensors (no transposed copies), the bias joins in the epilogue,
// and db = column sums of dy is one small HBM-bound reduction.
//
// Kernel structure (192 threads, one CTA per SM, static round-robin over 128x256 output tiles in
// bands of 16 tile rows so that one wave of CTAs shares its operand panels in L2):
//   warp 0      TMA producer: 4-stage ring of {A 128x64, B 256x64} bf16 tiles, 128-byte swizzle
//   warp 1      issues tcgen05.mma (M128 N256 K16, 4 per stage); a commit frees the stage, a
//               commit per tile hands the accumulator to the epilogue
//   warps 2-5   epilogue: accumulator (256 tensor-memory columns, double buffered so the next
//               tile's MMAs run meanwhile) -> registers -> + bias -> bf16 -> global
// Every wait is bounded (see sm100_ptx.cuh); an expired wait aborts the CTA through the common exit.
#include <cuda.h>

#include <algorithm>

#include "common.h"
#include "sm100_ptx.cuh"

namespace ttk {
using namespace sm100;

namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4;
constexpr int kABytes = kBM * kBK * 2;          // 16 KB
constexpr int kBBytes = kBN * kBK * 2;          // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;  // 48 KB
constexpr int kSubBytes = 64 * 128;             // one 64-wide MN-major sub-block: 64 K-rows x 128 B
constexpr int kGemmSmem = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int kBandRows = 16;

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
    const int per_band = kBandRows * tiles_n;
    const int band = t / per_band;
    const int first = band * kBandRows;
    const int rows = min(kBandRows, tiles_m - first);
    const int r = t - band * per_band;
    mb = first + r % rows;
    nb = r / rows;
}

// One thread's accumulator row (256 fp32 columns of tensor memory starting at `taddr`) -> + bias -> bf16 ->
// row `row` of C, columns n0...  Hands the accumulator buffer back (one arrival: on `acc_empty` of this CTA,
// or, in a CTA pair, on the barrier at `acc_empty_cluster` in the pair's rank-0 CTA) as soon as the row has
// been read.
template <bool kPair>
__device__ __forceinline__ void store_acc_row(uint32_t taddr, long long row, int n0, __nv_bfloat16* __restrict__ C,
                                              const __nv_bfloat16* __restrict__ bias, int M, int N, int wide,
                                              uint64_t* acc_empty, uint32_t acc_empty_cluster) {
    __nv_bfloat16* crow = C + row * (long long)N;
#pragma unroll 1
    for (int c = 0; c < kBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), r);
        tmem_wait_ld();
        if (c == kBN / 32 - 1) {   // this thread has read its whole accumulator row
            tc_fence_before();
            if (kPair) mbar_arrive_cluster(acc_empty_cluster);
            else mbar_arrive(acc_empty);
        }
        const int col0 = n0 + c * 32;
        if (row < M) {
#pragma unroll
            for (int g2 = 0; g2 < 2; ++g2) {
                uint32_t o8[8];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int g = g2 * 2 + h;
                    const int col = col0 + g * 8;
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[g * 8 + e]);
                    if (bias && col < N) {
                        const uint4 bb = *reinterpret_cast<const uint4*>(bias + col);
                        const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            v[2 * e] += __uint_as_float(bw[e] << 16);
                            v[2 * e + 1] += __uint_as_float(bw[e] & 0xffff0000u);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) o8[h * 4 + e] = pack_bf16x2(v[2 * e], v[2 * e + 1]);
                }
                // N % 8 == 0: a group of 8 columns is inside or outside as a whole
                const int col = col0 + g2 * 16;
                if (wide && col + 16 <= N) {
                    st_global_32B(crow + col, o8);   // one full sector per lane and instruction
                } else {
                    if (col < N) *reinterpret_cast<uint4*>(crow + col) = make_uint4(o8[0], o8[1], o8[2], o8[3]);
                    if (col + 8 < N) *reinterpret_cast<uint4*>(crow + col + 8) = make_uint4(o8[4], o8[5], o8[6], o8[7]);
                }
            }
        }
    }
}

template <bool kAMn, bool kBMn>
__global__ void __launch_bounds__(192, 1)
fc_gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                     int tiles_m, int tiles_n, int wide, unsigned int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* full = bars;                    // [kStages] producer -> MMA
    uint64_t* empty = bars + kStages;         // [kStages] MMA -> producer
    uint64_t* acc_full = bars + 2 * kStages;  // [2] MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;       // [2] epilogue -> MMA (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 128);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncwarp();
    if (warp == 0) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
        if (elect_one()) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    WaitCtx wctx{status, abort_flag, warp};

    const int total = tiles_m * tiles_n;
    const int kblocks = (K + kBK - 1) / kBK;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        int it = 0;
        bool live = true;
        for (int t = blockIdx.x; t < total && live; t += gridDim.x) {
            int mb, nb;
            tile_coords(t, tiles_m, tiles_n, mb, nb);
            const int m0 = mb * kBM, n0 = nb * kBN;
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % kStages;
                const uint32_t ph = (uint32_t)(it / kStages) & 1u;
                if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, wctx, 10 + s, it))) {
                    live = false;
                    break;
                }
                if (elect_one()) {
                    unsigned char* sA = smem + s * kStageBytes;
                    unsigned char* sB = sA + kABytes;
                    const int k0 = kb * kBK;
                    mbar_arrive_expect_tx(&full[s], kStageBytes);
                    if (kAMn) {
                        tma_load_3d(sA, &tmA, &full[s], m0, k0, 0);
                        tma_load_3d(sA + kSubBytes, &tmA, &full[s], m0 + 64, k0, 0);
                    } else {
                        tma_load_3d(sA, &tmA, &full[s], k0, m0, 0);
                    }
                    if (kBMn) {
#pragma unroll
                        for (int j = 0; j < kBN / 64; ++j) tma_load_3d(sB + j * kSubBytes, &tmB, &full[s], n0 + 64 * j, k0, 0);
                    } else {
                        tma_load_3d(sB, &tmB, &full[s], k0, n0, 0);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = umma_idesc_bf16(kBM, kBN, kAMn, kBMn);
        constexpr uint32_t a_step = kAMn ? 2048u : 32u;   // one K=16 step inside the stage
        constexpr uint32_t b_step = kBMn ? 2048u : 32u;
        int it = 0, lt = 0;
        bool live = true;
        for (int t = blockIdx.x; t < total && live; t += gridDim.x, ++lt) {
            const int buf = lt & 1;
            const uint32_t use = (uint32_t)(lt >> 1) & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(&acc_empty[buf], use ^ 1u, wctx, 30 + buf, lt))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)buf * kBN;
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % kStages;
                const uint32_t ph = (uint32_t)(it / kStages) & 1u;
                if (!__all_sync(0xffffffffu, mbar_wait(&full[s], ph, wctx, 20 + s, it))) {
                    live = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sA = smem_u32(smem + s * kStageBytes);
                const uint32_t sB = sA + kABytes;
                const uint64_t a0 = umma_smem_desc(sA, kAMn ? kSubBytes : 16, 1024);
                const uint64_t b0 = umma_smem_desc(sB, kBMn ? kSubBytes : 16, 1024);
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)
                    umma_ss(d_tmem, umma_desc_advance(a0, kk * a_step), umma_desc_advance(b0, kk * b_step), idesc,
                            (uint32_t)((kb | kk) != 0));
                tc_commit(&empty[s]);
            }
            if (live) tc_commit(&acc_full[buf]);
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int lane_group = warp & 3;                 // tensor-memory lanes 32*lane_group .. +31
        const uint32_t lane_off = (uint32_t)(lane_group * 32) << 16;
        int lt = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++lt) {
            int mb, nb;
            tile_coords(t, tiles_m, tiles_n, mb, nb);
            const int buf = lt & 1;
            const uint32_t use = (uint32_t)(lt >> 1) & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[buf], use, wctx, 40 + buf, lt))) break;
            tc_fence_after();
            const long long row = (long long)mb * kBM + lane_group * 32 + lane;
            store_acc_row<false>(tmem_base + lane_off + (uint32_t)(buf * kBN), row, nb * kBN, C, bias, M, N, wide,
                                 &acc_empty[buf], 0u);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- the same GEMM on CTA pairs (clusters of two, tcgen05 cta_group::2) ----------------------------------
// A pair owns a 256x256 output tile: CTA r of the pair holds rows [128r, 128r+128) of the A tile and
// rows [128r, 128r+128) of the B tile's N extent, so every K=64 stage is 16 KB + 16 KB per CTA and a
// M256 N256 K16 instruction reads 8 KB of shared memory per SM in its 128 cycles (64 B/clk, against
// 96 B/clk for the one-CTA 128x256 tile).  Both CTAs run the TMA producer (their loads count on the
// rank-0 CTA's `full` barrier) and the epilogue (each drains its own 128 accumulator rows); only the
// rank-0 CTA issues MMAs, and hands stages and accumulators back to both CTAs with one commit each.
constexpr int kPStages = 6;
constexpr int kPABytes = 128 * kBK * 2;             // 16 KB: this CTA's 128 rows of A
constexpr int kPBBytes = 128 * kBK * 2;             // 16 KB: this CTA's half of the 256 B rows
constexpr int kPStageBytes = kPABytes + kPBBytes;   // 32 KB
constexpr int kPairSmem = kPStages * kPStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

template <bool kAMn, bool kBMn>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
fc_gemm_pair_sm100_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                          int tiles_m, int tiles_n, int wide, unsigned int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPStages * kPStageBytes);
    uint64_t* full = bars;                     // [kPStages] both producers -> MMA (the rank-0 CTA's copy is used)
    uint64_t* empty = bars + kPStages;         // [kPStages] MMA -> this CTA's producer
    uint64_t* acc_full = bars + 2 * kPStages;  // [2] MMA -> this CTA's epilogue
    uint64_t* acc_empty = acc_full + 2;        // [2] both epilogues -> MMA (256 arrivals; rank-0 CTA's copy)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kPStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 256);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncwarp();
    if (warp == 0) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
        if (elect_one()) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers are initialised and its tensor memory allocated
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    WaitCtx wctx{status, abort_flag, warp};

    const int total = tiles_m * tiles_n;   // 256x256 tiles
    const int kblocks = (K + kBK - 1) / kBK;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        int it = 0;
        bool live = true;
        for (int t = pair; t < total && live; t += n_pairs) {
            int mb, nb;
            tile_coords(t, tiles_m, tiles_n, mb, nb);
            const int m0 = mb * 256 + (int)rank * 128, n0 = nb * 256 + (int)rank * 128;
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % kPStages;
                const uint32_t ph = (uint32_t)(it / kPStages) & 1u;
                if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, wctx, 10 + s, it))) {
                    live = false;
                    break;
                }
                if (elect_one()) {
                    unsigned char* sA = smem + s * kPStageBytes;
                    unsigned char* sB = sA + kPABytes;
                    const int k0 = kb * kBK;
                    if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * kPStageBytes);   // both CTAs' bytes
                    const uint32_t full0 = map_to_cta(smem_u32(&full[s]), 0);
                    if (kAMn) {
                        tma_load_3d_pair(sA, &tmA, full0, m0, k0, 0);
                        tma_load_3d_pair(sA + kSubBytes, &tmA, full0, m0 + 64, k0, 0);
                    } else {
                        tma_load_3d_pair(sA, &tmA, full0, k0, m0, 0);
                    }
                    if (kBMn) {
                        tma_load_3d_pair(sB, &tmB, full0, n0, k0, 0);
                        tma_load_3d_pair(sB + kSubBytes, &tmB, full0, n0 + 64, k0, 0);
                    } else {
                        tma_load_3d_pair(sB, &tmB, full0, k0, n0, 0);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (rank-0 CTA only)
        if (rank == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(256, 256, kAMn, kBMn);
            constexpr uint32_t a_step = kAMn ? 2048u : 32u;   // one K=16 step inside the stage
            constexpr uint32_t b_step = kBMn ? 2048u : 32u;
            int it = 0, lt = 0;
            bool live = true;
            for (int t = pair; t < total && live; t += n_pairs, ++lt) {
                const int buf = lt & 1;
                const uint32_t use = (uint32_t)(lt >> 1) & 1u;
                if (!__all_sync(0xffffffffu, mbar_wait(&acc_empty[buf], use ^ 1u, wctx, 30 + buf, lt))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * kBN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % kPStages;
                    const uint32_t ph = (uint32_t)(it / kPStages) & 1u;
                    if (!__all_sync(0xffffffffu, mbar_wait(&full[s], ph, wctx, 20 + s, it))) {
                        live = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sA = smem_u32(smem + s * kPStageBytes);
                    const uint32_t sB = sA + kPABytes;
                    const uint64_t a0 = umma_smem_desc(sA, kAMn ? kSubBytes : 16, 1024);
                    const uint64_t b0 = umma_smem_desc(sB, kBMn ? kSubBytes : 16, 1024);
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk)
                        umma_ss_pair(d_tmem, umma_desc_advance(a0, kk * a_step), umma_desc_advance(b0, kk * b_step), idesc,
                                     (uint32_t)((kb | kk) != 0));
                    const uint32_t e0 = smem_u32(&empty[s]);
                    tc_commit_pair(e0);                  // this CTA's producer may refill the stage ...
                    tc_commit_pair(map_to_cta(e0, 1));   // ... and so may the peer's
                }
                if (live) {
                    const uint32_t f0 = smem_u32(&acc_full[buf]);
                    tc_commit_pair(f0);
                    tc_commit_pair(map_to_cta(f0, 1));
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int lane_group = warp & 3;                 // tensor-memory lanes 32*lane_group .. +31
        const uint32_t lane_off = (uint32_t)(lane_group * 32) << 16;
        int lt = 0;
        for (int t = pair; t < total; t += n_pairs, ++lt) {
            int mb, nb;
            tile_coords(t, tiles_m, tiles_n, mb, nb);
            const int buf = lt & 1;
            const uint32_t use = (uint32_t)(lt >> 1) & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[buf], use, wctx, 40 + buf, lt))) break;
            tc_fence_after();
            const long long row = (long long)mb * 256 + (int)rank * 128 + lane_group * 32 + lane;
            store_acc_row<true>(tmem_base + lane_off + (uint32_t)(buf * kBN), row, nb * kBN, C, bias, M, N, wide,
                                nullptr, map_to_cta(smem_u32(&acc_empty[buf]), 0));
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // neither CTA leaves while the other may still read its shared memory or signal its barriers
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// fp32-arithmetic SIMT GEMM for float tensors and for shapes the tensor-core kernel does not
// take (row pitches that are not multiples of 16 bytes).  64x64 tiles, 4x4 outputs per thread.
template <typename T> __device__ __forceinline__ float g_ld(const T* p, long long i);
template <> __device__ __forceinline__ float g_ld<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float g_ld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void g_st(T* p, long long i, float v);
template <> __device__ __forceinline__ void g_st<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void g_st<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) fc_gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ B,
                                                          T* __restrict__ C, const T* __restrict__ bias, int M, int N,
                                                          int K, int a_mn, int b_mn) {
    __shared__ float sA[16][64 + 1];
    __shared__ float sB[16][64 + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long m0 = (long long)blockIdx.y * 64;
    const int n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 16 * 64; i += 256) {
            // the faster-running index follows the contiguous axis of each operand
            const int kk_a = a_mn ? i / 64 : i % 16, mm = a_mn ? i % 64 : i / 16;
            const long long m = m0 + mm;
            const int k = k0 + kk_a;
            sA[kk_a][mm] = (m < M && k < K) ? g_ld<T>(A, a_mn ? (long long)k * M + m : m * K + k) : 0.f;
            const int kk_b = b_mn ? i / 64 : i % 16, nn = b_mn ? i % 64 : i / 16;
            const int n = n0 + nn, kb = k0 + kk_b;
            sB[kk_b][nn] = (n < N && kb < K) ? g_ld<T>(B, b_mn ? (long long)kb * N + n : (long long)n * K + kb) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = sA[kk][ty * 4 + i];
                b[i] = sB[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) g_st<T>(C, m * N + n, acc[i][j] + (bias ? g_ld<T>(bias, n) : 0.f));
        }
    }
}

// Column sums of a row-major [M,N] matrix: partial[split][n] over a fixed row range per split,
// then a second pass adds the splits in order (deterministic).
template <typename T>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const T* __restrict__ X, float* __restrict__ partial,
                                                            long long M, int N, int rows_per_split) {
    const int col = blockIdx.x * 64 + (threadIdx.x & 63);
    const int sub = threadIdx.x >> 6;   // 4 row phases per CTA
    const long long r0 = (long long)blockIdx.y * rows_per_split;
    const long long r1 = min(M, r0 + rows_per_split);
    float s = 0.f;
    if (col < N)
        for (long long r = r0 + sub; r < r1; r += 4) s += g_ld<T>(X, r * N + col);
    __shared__ float red[4][64];
    red[sub][threadIdx.x & 63] = s;
    __syncthreads();
    if (sub == 0 && col < N)
        partial[(long long)blockIdx.y * N + col] = red[0][threadIdx.x] + red[1][threadIdx.x] + red[2][threadIdx.x] + red[3][threadIdx.x];
}
template <typename T>
__global__ void colsum_final_kernel(const float* __restrict__ partial, T* __restrict__ out, int N, int splits,
                                    int scalar_bias) {
    if (scalar_bias) {   // one CTA: the reference's single-value bias gets the sum over all columns too
        __shared__ float red[256];
        float s = 0.f;
        for (int n = threadIdx.x; n < N; n += 256)
            for (int p = 0; p < splits; ++p) s += partial[(long long)p * N + n];
        red[threadIdx.x] = s;
        __syncthreads();
        for (int o = 128; o > 0; o >>= 1) {
            if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
            __syncthreads();
        }
        if (threadIdx.x == 0) g_st<T>(out, 0, red[0]);
        return;
    }
    const int n = blockIdx.x * 256 + threadIdx.x;
    if (n >= N) return;
    float s = 0.f;
    for (int p = 0; p < splits; ++p) s += partial[(long long)p * N + n];
    g_st<T>(out, n, s);
}

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev] > 0 ? cached[dev] : 148;
}

template <bool kAMn, bool kBMn>
cudaError_t launch_tc(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, cudaStream_t st) {
    TmapStorage ta, tb;
    const char* why = nullptr;
    if (!make_tmap_bf16(&ta, A, kAMn ? (uint64_t)M : (uint64_t)K, kAMn ? (uint64_t)K : (uint64_t)M, 1, kAMn ? 64 : kBM, &why))
        return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tb, B, kBMn ? (uint64_t)N : (uint64_t)K, kBMn ? (uint64_t)K : (uint64_t)N, 1, kBMn ? 64 : kBN, &why))
        return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(fc_gemm_sm100_kernel<kAMn, kBMn>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
    if (e != cudaSuccess) return e;
    const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + kBN - 1) / kBN;
    const int grid = std::min(tiles_m * tiles_n, sm_count());
    LaunchScope ls(K_FC_GEMM, st);
    fc_gemm_sm100_kernel<kAMn, kBMn><<<grid, 192, kGemmSmem, st>>>(
        *reinterpret_cast<CUtensorMap*>(ta.bytes), *reinterpret_cast<CUtensorMap*>(tb.bytes), (__nv_bfloat16*)C,
        (const __nv_bfloat16*)bias, M, N, K, tiles_m, tiles_n,
        ((reinterpret_cast<uintptr_t>(C) & 31) == 0 && N % 16 == 0) ? 1 : 0,   // 32-byte stores possible
        device_status_word());
    return cudaGetLastError();
}


// true: the CTA-pair kernel takes this launch.  It needs enough 256x256 tiles to fill the pairs; smaller
// problems spread better as 128x256 tiles over single CTAs.  TT_FC_PATH=1cta / 2cta forces either (tests).
bool use_pair_kernel(int M, int N) {
    const char* f = getenv("TT_FC_PATH");
    if (f && f[0] == '1') return false;
    if (f && f[0] == '2') return true;
    const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    return tiles >= sm_count();   // two or more tiles per pair
}

template <bool kAMn, bool kBMn>
cudaError_t launch_tc_pair(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, cudaStream_t st) {
    TmapStorage ta, tb;
    const char* why = nullptr;
    if (!make_tmap_bf16(&ta, A, kAMn ? (uint64_t)M : (uint64_t)K, kAMn ? (uint64_t)K : (uint64_t)M, 1, kAMn ? 64 : 128, &why))
        return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tb, B, kBMn ? (uint64_t)N : (uint64_t)K, kBMn ? (uint64_t)K : (uint64_t)N, 1, kBMn ? 64 : 128, &why))
        return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(fc_gemm_pair_sm100_kernel<kAMn, kBMn>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
    if (e != cudaSuccess) return e;
    const int tiles_m = (M + 255) / 256, tiles_n = (N + 255) / 256;
    // pairs that can be resident at once (a GPC with an odd number of usable SMs leaves one without a partner)
    static int max_pairs[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!max_pairs[dev]) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)sm_count() & ~1u);
        cfg.blockDim = dim3(192);
        cfg.dynamicSmemBytes = kPairSmem;
        cudaLaunchAttribute at;
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = 2;
        at.val.clusterDim.y = 1;
        at.val.clusterDim.z = 1;
        cfg.attrs = &at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, fc_gemm_pair_sm100_kernel<kAMn, kBMn>, &cfg) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = sm_count() / 2;
        }
        max_pairs[dev] = n;
    }
    const int pairs = std::min(tiles_m * tiles_n, max_pairs[dev]);
    LaunchScope ls(K_FC_GEMM, st);
    fc_gemm_pair_sm100_kernel<kAMn, kBMn><<<2 * pairs, 192, kPairSmem, st>>>(
        *reinterpret_cast<CUtensorMap*>(ta.bytes), *reinterpret_cast<CUtensorMap*>(tb.bytes), (__nv_bfloat16*)C,
        (const __nv_bfloat16*)bias, M, N, K, tiles_m, tiles_n,
        ((reinterpret_cast<uintptr_t>(C) & 31) == 0 && N % 16 == 0) ? 1 : 0, device_status_word());
    return cudaGetLastError();
}

}  // namespace

bool fc_gemm_tc_supported(const void* A, const void* B, const void* C, const void* bias, long long M, int N, int K,
                          int a_mn, int b_mn, int bf16) {
    if (!bf16 || M < 1 || M > 0x7fffffffLL || N < 1 || K < 1) return false;
    const long long a_cols = a_mn ? M : K, b_cols = b_mn ? N : K;
    if (a_cols % 8 || b_cols % 8 || N % 8) return false;
    if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C | (uintptr_t)bias) & 15) return false;
    const char* f = getenv("TT_FC_PATH");
    if (f && f[0] == 's') return false;   // "simt": force the fp32-arithmetic kernel (tests)
    return true;
}

cudaError_t fc_gemm(const void* A, const void* B, void* C, const void* bias, long long M, int N, int K, int a_mn,
                    int b_mn, int bf16, cudaStream_t st) {
    if (fc_gemm_tc_supported(A, B, C, bias, M, N, K, a_mn, b_mn, bf16)) {
        if (use_pair_kernel((int)M, N)) {
            if (!a_mn && b_mn) return launch_tc_pair<false, true>(A, B, C, bias, (int)M, N, K, st);
            if (!a_mn && !b_mn) return launch_tc_pair<false, false>(A, B, C, bias, (int)M, N, K, st);
            if (a_mn && b_mn) return launch_tc_pair<true, true>(A, B, C, bias, (int)M, N, K, st);
            return launch_tc_pair<true, false>(A, B, C, bias, (int)M, N, K, st);
        }
        if (!a_mn && b_mn) return launch_tc<false, true>(A, B, C, bias, (int)M, N, K, st);
        if (!a_mn && !b_mn) return launch_tc<false, false>(A, B, C, bias, (int)M, N, K, st);
        if (a_mn && b_mn) return launch_tc<true, true>(A, B, C, bias, (int)M, N, K, st);
        return launch_tc<true, false>(A, B, C, bias, (int)M, N, K, st);
    }
    dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64));
    if (grid.y > 65535u) return cudaErrorInvalidValue;
    LaunchScope ls(K_FC_SIMT, st);
    if (bf16)
        fc_gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)B,
                                                                (__nv_bfloat16*)C, (const __nv_bfloat16*)bias, (int)M, N, K, a_mn, b_mn);
    else
        fc_gemm_simt_kernel<float><<<grid, 256, 0, st>>>((const float*)A, (const float*)B, (float*)C, (const float*)bias,
                                                        (int)M, N, K, a_mn, b_mn);
    return cudaGetLastError();
}

int fc_colsum_splits(long long M) { return (int)std::max<long long>(1, std::min<long long>(64, (M + 255) / 256)); }
size_t fc_colsum_workspace(long long M, int N) { return align256((size_t)fc_colsum_splits(M) * (size_t)N * sizeof(float)); }

cudaError_t fc_colsum(const void* X, void* out, long long M, int N, int bf16, int scalar_bias, void* workspace,
                      cudaStream_t st) {
    const int splits = fc_colsum_splits(M);
    const int rows_per_split = (int)((M + splits - 1) / splits);
    float* partial = (float*)workspace;
    dim3 grid((unsigned)((N + 63) / 64), (unsigned)splits);
    {
        LaunchScope ls(K_FC_COLSUM, st);
        if (bf16) colsum_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)X, partial, M, N, rows_per_split);
        else colsum_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)X, partial, M, N, rows_per_split);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    LaunchScope ls(K_FC_COLSUM, st, false);
    const unsigned fgrid = scalar_bias ? 1u : (unsigned)((N + 255) / 256);
    if (bf16) colsum_final_kernel<__nv_bfloat16><<<fgrid, 256, 0, st>>>(partial, (__nv_bfloat16*)out, N, splits, scalar_bias);
    else colsum_final_kernel<float><<<fgrid, 256, 0, st>>>(partial, (float*)out, N, splits, scalar_bias);
    return cudaGetLastError();
}

}  // namespace ttk

// Single-query attention (decode) on the tensor cores with keys on the accumulator rows, single or grouped heads.
// bf16, head dim 128 or 64, 1..16 query heads per key/value head, dense, ragged or paged cache.
//
// Run as a forward problem with the G query heads of a key/value head as G query rows, the general
// forward kernel spends a whole 128-row query tile on G rows: its softmax threads are rows, so per
// key tile ONE warp evaluates 128 exponentials per lane while the other rows hold nothing, and the
// chain scores -> softmax -> P V of the single busy tile takes longer than HBM needs to deliver the
// next K/V tile (measured 75-82 % of the copy bandwidth).  Here the problem is transposed:
//     S^T [128 keys x 16] = K_j Q^T          A = K tile (shared memory, K-major), B = Q (16 rows, K-major)
//     O^T [128 d    x 16] += V_j^T P_j       A = V tile read MN-major (M = d), B = P_j (16 rows, K-major)
// so a softmax thread is a KEY: per tile it scales its G scores, takes part in one maximum over the
// tile (redux.sync over the warp, shared memory over the four warps), evaluates G exponentials and
// writes G bf16 probabilities into the shared-memory P tile.  The MMAs have N = 16 and take a few
// hundred cycles per tile; S^T and P are double buffered, so the next tile's scores are computed under
// this tile's softmax.  The running maximum is raised lazily (only when a tile's maximum exceeds it
// by more than 2^8), in which case every thread -- now as a row d of O^T -- rescales its 16 accumulator
// columns in tensor memory.
//
// One CTA per (key/value slice, key range); two CTAs per SM (110 KB of shared memory, 64 tensor-memory
// columns each) so that one CTA's set-up and tail overlap the other's stream.  Results per range are
// normalised (out bf16 [slices*ranges, G, D], log-sum-exp fp32): with more than one range a merge
// kernel combines them, exactly as for the forward-kernel route this replaces.
//   warps 0-3  softmax (thread = key of the tile = row d of O^T),  warp 4  MMA issuer,  warp 5  TMA loader
// Every mbarrier wait is bounded (sm100_ptx.cuh); the one bar.sync per tile among the softmax warps is reached
// by all 128 threads whatever the waits returned (they never leave the tile loop early).
#include "common.h"
#include "sm100_ptx.cuh"

#include <stdlib.h>
#include <algorithm>

namespace ttk {
using namespace sm100;

namespace {

constexpr int kSubBytes = 128 * 128;          // [128 rows x 128 B]
constexpr int kPBytes = 4096;                 // [16 query rows x 128 keys]: two sub-blocks of [16 rows x 128 B]
constexpr int kAuxBytes = 2048;               // barriers, reduction scratch
constexpr int kThreads = 192;
constexpr int kTmemCols = 64;                 // S^T buffers at [0,16) and [16,32), O^T at [32,48)
template <int kD>
struct GqCfg {
    static constexpr int kSub = kD / 64;                       // 64-column sub-blocks per K/V tile
    static constexpr int kTileBytes = kSub * kSubBytes;        // 32 KB (D = 128), 16 KB (D = 64)
    static constexpr int kStages = 96 * 1024 / kTileBytes;     // ring of K/V tiles: K_0, V_0, K_1, V_1, ...
    static constexpr int kQBytes = kSub * 2048;                // [16 query rows x D]: sub-blocks of [16 rows x 128 B]
    static constexpr int kSmemBytes = kStages * kTileBytes + 4096 /*Q*/ + 2 * kPBytes + kAuxBytes + 1024;   // +1024: alignment slack
};

struct GqParams {
    __nv_bfloat16* out;
    float* lse;
    int G;              // query heads per key/value head = query rows of a slice
    int L;              // keys per key/value slice of the K/V tensor maps
    int q_div;          // output slices (key ranges) per query slice
    int kv_chunk;       // cache mode: keys per range (0: one range)
    const int* kv_lens; // cache mode: keys per batch entry (may hold 0)
    int H;              // cache mode: key/value heads per batch entry
    const int* block_table;
    int page_size, max_pages;
    float scale_log2;
    unsigned int* status;
};

// order-preserving map float -> int, so that redux.sync.max.s32 yields the float maximum
__device__ __forceinline__ int float_key(float x) {
    const int i = __float_as_int(x);
    return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float key_float(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7fffffff)); }
__device__ __forceinline__ void bar_sync_128(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

// kD: head dim, 128 or 64.  At 64 the accumulator still has 128 rows: the V tile is one 64-wide block, and the
// descriptor's stride to the "second" block is 0, so rows 64..127 of O^T repeat rows 0..63 and are never read.
// kG: columns of S^T / O^T the softmax evaluates (G <= kG <= 16).  kCache: ragged and/or paged cache.
template <int kD, int kG, bool kCache>
__global__ void __launch_bounds__(kThreads, 2)
attn_decode_gq_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, const GqParams p) {
    using Cfg = GqCfg<kD>;
    constexpr int kStages = Cfg::kStages, kTileBytes = Cfg::kTileBytes, kSub = Cfg::kSub, kQBytes = Cfg::kQBytes;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sKV = smem;
    unsigned char* sQ = smem + kStages * kTileBytes;
    unsigned char* sP = sQ + 4096;
    unsigned char* aux = sP + 2 * kPBytes;
    uint64_t* bar_q_full = reinterpret_cast<uint64_t*>(aux);
    uint64_t* bar_kv_full = bar_q_full + 1;          // [kStages]
    uint64_t* bar_kv_empty = bar_kv_full + kStages;  // [kStages]
    uint64_t* bar_s_full = bar_kv_empty + kStages;   // [2] MMA -> softmax
    uint64_t* bar_s_free = bar_s_full + 2;           // [2] softmax (scores in registers) -> MMA
    uint64_t* bar_p_full = bar_s_free + 2;           // [2] softmax (P in shared memory) -> MMA
    uint64_t* bar_p_free = bar_p_full + 2;           // [2] MMA (P consumed) -> softmax
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_p_free + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* red_max = reinterpret_cast<int*>(aux + 512);        // [2 buffers][4 warps][16]
    float* red_sum = reinterpret_cast<float*>(aux + 1024);   // [4 warps][16]

    const int warp = uniform_warp_idx();
    const int lane = threadIdx.x & 31;

    // ---- this CTA's key range
    const int bh = blockIdx.x;                 // output slice
    const int qslice = bh / p.q_div;
    int zslice = bh, key0 = 0, Lv = p.L;
    if (kCache) {
        zslice = qslice;                       // key/value slice
        key0 = (bh - qslice * p.q_div) * p.kv_chunk;
        const int len = p.kv_lens ? min(p.L, max(0, p.kv_lens[zslice / p.H])) : p.L;
        Lv = p.kv_chunk > 0 ? max(0, min(len - key0, p.kv_chunk)) : len;
    }
    const int n_tiles = (Lv + 127) >> 7;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bar_kv_full[s], 1);
            mbar_init(&bar_kv_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_s_full[b], 1);
            mbar_init(&bar_s_free[b], 4);
            mbar_init(&bar_p_full[b], 4);
            mbar_init(&bar_p_free[b], 1);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 4) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    if (warp == 5 && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    WaitCtx wctx{p.status, abort_flag, warp};
    constexpr uint32_t kColO = 32;

    if (warp < 4) {
        // =========================================================== softmax: thread = key of the tile / row d of O^T
        const int t = threadIdx.x;
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        const float c = p.scale_log2;
        if (n_tiles == 0) {   // an empty range (cache mode): zero output, log-sum-exp -inf; the merge gives it no weight
            if (t < kD)
                for (int g = 0; g < p.G; ++g) p.out[((long long)bh * p.G + g) * kD + t] = __float2bfloat16_rn(0.f);
            if (t < p.G && p.lse != nullptr) p.lse[(long long)bh * p.G + t] = -INFINITY;
        } else {
            float m_ref[kG], l_t[kG];
#pragma unroll
            for (int g = 0; g < kG; ++g) {
                m_ref[g] = -INFINITY;
                l_t[g] = 0.f;
            }
            // where this key's probabilities go in a P buffer: row g, 16-byte chunk ((t & 63) >> 3) ^ (g & 7)
            const uint32_t p_off = (uint32_t)((t >> 6) * 2048 + (t & 7) * 2);
            const uint32_t p_chunk = (uint32_t)((t & 63) >> 3);
            // Every thread runs every tile, even after a wait has given up (all later waits then return at
            // once and the results are void): the named barriers below need all 128 threads each time.
            for (int j = 0; j < n_tiles; ++j) {
                const int b = j & 1;
                mbar_wait(&bar_s_full[b], (j >> 1) & 1, wctx, 10 + b, j);
                __syncwarp();
                tc_fence_after();
                uint32_t sr[16];
                tmem_ld16(tmem_base + lane_off + (uint32_t)(b * 16), sr);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_s_free[b]);   // this warp's scores are in registers
                const bool valid = j * 128 + t < Lv;
                float x[kG];
                int wkey[kG];
#pragma unroll
                for (int g = 0; g < kG; ++g) {
                    x[g] = valid ? __uint_as_float(sr[g]) * c : -INFINITY;
                    wkey[g] = __reduce_max_sync(0xffffffffu, float_key(x[g]));
                }
                if (lane == 0) {
#pragma unroll
                    for (int g = 0; g < kG; ++g) red_max[(b * 4 + warp) * 16 + g] = wkey[g];
                }
                bar_sync_128(1);
                // Both buffers of red_max are safe without a second barrier: a thread writes buffer b again
                // only at tile j + 2, after the barrier of tile j + 1, which every thread reaches after
                // reading buffer b here.
                bool need = (j == 0);
                float tmax[kG];
#pragma unroll
                for (int g = 0; g < kG; ++g) {
                    const int* r = red_max + b * 64 + g;
                    tmax[g] = key_float(max(max(r[0], r[16]), max(r[32], r[48])));
                    need = need || (tmax[g] > m_ref[g] + 8.0f);
                }
                if (need) {   // the same decision in every thread of the CTA: all see the same maxima
                    float f[kG];
#pragma unroll
                    for (int g = 0; g < kG; ++g) {
                        const float m_new = fmaxf(m_ref[g], tmax[g]);
                        f[g] = (m_ref[g] == -INFINITY) ? 0.f : ex2_approx(m_ref[g] - m_new);
                        l_t[g] *= f[g];
                        m_ref[g] = m_new;
                    }
                    if (j > 0) {
                        // O^T *= f, once every MMA up to tile j - 1 has completed: that is the next phase of the
                        // other P buffer's `free` barrier (a thread waits for every phase of these two barriers in
                        // turn, so a phase's parity is never mistaken for an older one's)
                        mbar_wait(&bar_p_free[(j - 1) & 1], ((j - 1) >> 1) & 1, wctx, 30, j);
                        __syncwarp();
                        tc_fence_after();
                        uint32_t o[16];
                        tmem_ld16(tmem_base + lane_off + kColO, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int g = 0; g < kG; ++g) o[g] = __float_as_uint(__uint_as_float(o[g]) * f[g]);
                        tmem_st16(tmem_base + lane_off + kColO, o);
                        tmem_wait_st();
                    }
                }
                mbar_wait(&bar_p_free[b], ((j >> 1) & 1) ^ 1, wctx, 20 + b, j);   // MMAs of tile j - 2 have read this P buffer
                unsigned char* pb = sP + b * kPBytes + p_off;
#pragma unroll
                for (int g = 0; g < kG; ++g) {
                    const float pv = ex2_approx(x[g] - m_ref[g]);
                    l_t[g] += pv;
                    *reinterpret_cast<__nv_bfloat16*>(pb + (g >> 3) * 1024 + (g & 7) * 128 + ((p_chunk ^ (uint32_t)(g & 7)) << 4)) =
                        __float2bfloat16_rn(pv);
                }
                fence_proxy_async_smem();   // the MMA reads P through the async proxy
                tc_fence_before();          // (orders the rescale's tensor-memory stores, when there were any)
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_p_full[b]);
            }
            // ---- result: O^T / l -> bf16, log-sum-exp
            mbar_wait(&bar_p_free[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, wctx, 31, n_tiles);   // the last tile's MMAs have completed
            __syncwarp();
            tc_fence_after();
            uint32_t o[16];
            tmem_ld16(tmem_base + lane_off + kColO, o);
            tmem_wait_ld();
#pragma unroll
            for (int g = 0; g < kG; ++g) {
                float v = l_t[g];
#pragma unroll
                for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
                if (lane == 0) red_sum[warp * 16 + g] = v;
            }
            bar_sync_128(1);
#pragma unroll
            for (int g = 0; g < kG; ++g) {
                const float l = red_sum[g] + red_sum[16 + g] + red_sum[32 + g] + red_sum[48 + g];
                if (g < p.G) {
                    if (t < kD) p.out[((long long)bh * p.G + g) * kD + t] = __float2bfloat16_rn(__uint_as_float(o[g]) / l);
                    if (t == g && p.lse != nullptr) p.lse[(long long)bh * p.G + g] = (m_ref[g] + log2f(l)) * 0.6931471805599453f;
                }
            }
        }
    } else if (warp == 5) {
        // =========================================================== TMA loader
        if (n_tiles > 0) {
            if (elect_one()) {
                mbar_arrive_expect_tx(bar_q_full, kQBytes);
                // 16 query rows from row qslice * G of q viewed as [rows, D]; rows past the group belong to other
                // heads (or are zero past the end): their columns of S^T and O^T are never read
#pragma unroll
                for (int sb = 0; sb < kSub; ++sb) tma_load_3d(sQ + sb * 2048, &tmQ, bar_q_full, sb * 64, qslice * p.G, 0);
            }
            __syncwarp();
            // paged cache: lane i fetches the i-th page (or 128-row part of a larger page) of a tile.  The table
            // entry of the NEXT tile is read while this tile's two entries wait for their ring slots, so the
            // look-up's latency stays off the loader's critical path; K and V of a tile share it.
            const bool paged = kCache && p.block_table != nullptr;
            const int box_rows = paged ? min(p.page_size, 128) : 128;
            auto page_of = [&](int tile) -> int {
                const int key = key0 + tile * 128 + lane * box_rows;
                if (!paged || tile >= n_tiles || lane * box_rows >= 128 || tile * 128 + lane * box_rows >= Lv) return 0;
                return __ldg(p.block_table + (long long)(zslice / p.H) * p.max_pages + key / p.page_size);
            };
            int page_next = page_of(0);
            for (int e = 0; e < 2 * n_tiles; ++e) {   // entry e: K of tile e/2 (even), V (odd)
                const int st = e % kStages;
                const int tile = e >> 1;
                const int page = page_next;
                if (e & 1) page_next = page_of(tile + 1);             // issued now, consumed two entries later
                if (!mbar_wait(&bar_kv_empty[st], ((e / kStages) & 1) ^ 1, wctx, 40 + st, e)) break;
                __syncwarp();
                const CUtensorMap* tm = (e & 1) ? &tmV : &tmK;
                unsigned char* dst = sKV + st * kTileBytes;
                const int k_first = tile * 128;                       // first key of the tile inside the range
                if (paged) {
                    // Only pages that hold counted keys are fetched: what the rest of the tile holds is masked
                    // in S^T and zeroed in V.
                    const int n_box = min(128 / box_rows, (Lv - k_first + box_rows - 1) / box_rows);
                    if (lane == 0) mbar_arrive_expect_tx(&bar_kv_full[st], (uint32_t)(n_box * box_rows * kD * 2));
                    __syncwarp();
                    if (lane < n_box) {
                        const int key = key0 + k_first + lane * box_rows;
                        const int z = page * p.H + (zslice % p.H);
#pragma unroll
                        for (int sb = 0; sb < kSub; ++sb)
                            tma_load_3d(dst + sb * kSubBytes + lane * box_rows * 128, tm, &bar_kv_full[st], sb * 64,
                                        key % p.page_size, z);
                    }
                    __syncwarp();
                } else {
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&bar_kv_full[st], kTileBytes);
#pragma unroll
                        for (int sb = 0; sb < kSub; ++sb)
                            tma_load_3d(dst + sb * kSubBytes, tm, &bar_kv_full[st], sb * 64, key0 + k_first, zslice);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (n_tiles > 0) {
        // =========================================================== MMA issuer (warp 4)
        constexpr uint32_t idesc_s = umma_idesc_bf16(128, 16, false, false);   // S^T = K Q^T
        constexpr uint32_t idesc_o = umma_idesc_bf16(128, 16, true, false);    // O^T += V^T P: A = V read MN-major
        const uint32_t sKV_addr = __shfl_sync(0xffffffffu, smem_u32(sKV), 0);
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
        const uint64_t dK_base = umma_smem_desc(sKV_addr, 16, 1024);             // K-major A, 128 key rows
        const uint64_t dV_base = umma_smem_desc(sKV_addr, kSub == 2 ? kSubBytes : 0, 1024);   // MN-major A: M = d over two 64-wide blocks (D = 64: the same block twice)
        const uint64_t dQ = umma_smem_desc(__shfl_sync(0xffffffffu, smem_u32(sQ), 0), 16, 1024);   // K-major B, 16 rows
        const uint64_t dP_base = umma_smem_desc(__shfl_sync(0xffffffffu, smem_u32(sP), 0), 16, 1024);
        auto issue_s = [&](int j) {
            const uint64_t a0 = umma_desc_advance(dK_base, ((2 * j) % kStages) * kTileBytes);
#pragma unroll
            for (int kk = 0; kk < kD / 16; ++kk)
                umma_ss(tmem_u + (uint32_t)((j & 1) * 16), umma_desc_advance(a0, (kk >> 2) * kSubBytes + (kk & 3) * 32),
                        umma_desc_advance(dQ, (kk >> 2) * 2048 + (kk & 3) * 32), idesc_s, kk > 0);
        };
        auto issue_o = [&](int j) {
            const uint64_t a0 = umma_desc_advance(dV_base, ((2 * j + 1) % kStages) * kTileBytes);
            const uint64_t b0 = umma_desc_advance(dP_base, (j & 1) * kPBytes);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)   // 16 keys per step
                umma_ss(tmem_u + kColO, umma_desc_advance(a0, kk * 2048), umma_desc_advance(b0, (kk >> 2) * 2048 + (kk & 3) * 32),
                        idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        };
        auto wait_entry = [&](int e) -> bool {
            const bool ok = mbar_wait(&bar_kv_full[e % kStages], (e / kStages) & 1, wctx, 50 + e % kStages, e);
            __syncwarp();
            return ok;
        };
        bool live = mbar_wait(bar_q_full, 0, wctx, 60, 0);
        __syncwarp();
        live = live && wait_entry(0);
        tc_fence_after();
        if (live) {
            issue_s(0);
            tc_commit(&bar_s_full[0]);
            tc_commit(&bar_kv_empty[0]);
        }
        for (int j = 0; j < n_tiles && live; ++j) {
            const int b = j & 1;
            if (j + 1 < n_tiles) {   // next tile's scores, under this tile's softmax
                live = wait_entry(2 * j + 2);
                if (j + 1 >= 2) live = live && mbar_wait(&bar_s_free[(j + 1) & 1], (((j + 1) >> 1) & 1) ^ 1, wctx, 61, j);
                __syncwarp();
                tc_fence_after();
                if (!live) break;
                issue_s(j + 1);
                tc_commit(&bar_s_full[(j + 1) & 1]);
                tc_commit(&bar_kv_empty[(2 * j + 2) % kStages]);
            }
            live = wait_entry(2 * j + 1);   // V_j
            const int rv = Lv - j * 128;
            if (rv < 128) {
                // Rows of the last V tile past the range's end hold whatever memory (or the ring slot) held;
                // their P is exactly 0, but 0 x NaN is not, so they are zeroed.
                unsigned char* vt = sKV + ((2 * j + 1) % kStages) * kTileBytes;
#pragma unroll
                for (int sb = 0; sb < kSub; ++sb)
                    for (int o = rv * 128 + lane * 16; o < 128 * 128; o += 32 * 16)
                        *reinterpret_cast<uint4*>(vt + sb * kSubBytes + o) = make_uint4(0u, 0u, 0u, 0u);
                fence_proxy_async_smem();
                __syncwarp();
            }
            live = live && mbar_wait(&bar_p_full[b], (j >> 1) & 1, wctx, 62 + b, j);
            __syncwarp();
            tc_fence_after();
            if (!live) break;
            issue_o(j);
            tc_commit(&bar_kv_empty[(2 * j + 1) % kStages]);
            tc_commit(&bar_p_free[b]);   // P consumed; also: every MMA issued so far has completed
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int kD, int kG, bool kCache>
cudaError_t launch_gq(const AttnArgs& a, cudaStream_t st) {
    TmapStorage tq, tk, tv;
    const char* why = nullptr;
    const int q_div = a.q_div > 0 ? a.q_div : 1;
    const long long q_rows = (a.BH / q_div) * (long long)a.S;   // q viewed as [rows, D]
    if (!make_tmap_bf16(&tq, a.q, kD, (uint64_t)q_rows, 1, 16, &why)) return cudaErrorInvalidValue;
    if (kCache && a.block_table != nullptr) {
        // the pools' page count is not known here; the extent only bounds what TMA may touch, and the block
        // table names the pages that exist
        const uint64_t slices = 0x7fffffffull;
        const uint32_t box_rows = (uint32_t)std::min(a.page_size, 128);
        if (!make_tmap_bf16(&tk, a.k, kD, (uint64_t)a.page_size, slices, box_rows, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16(&tv, a.v, kD, (uint64_t)a.page_size, slices, box_rows, &why)) return cudaErrorInvalidValue;
    } else {
        const long long kv_slices = kCache ? a.BH / q_div : a.BH;
        if (!make_tmap_bf16(&tk, a.k, kD, a.L, kv_slices, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16(&tv, a.v, kD, a.L, kv_slices, 128, &why)) return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaFuncSetAttribute(attn_decode_gq_sm100_kernel<kD, kG, kCache>, cudaFuncAttributeMaxDynamicSharedMemorySize, GqCfg<kD>::kSmemBytes);
    if (e != cudaSuccess) return e;
    GqParams p;
    p.out = (__nv_bfloat16*)a.out;
    p.lse = a.lse;
    p.G = a.S;
    p.L = a.L;
    p.q_div = q_div;
    p.kv_chunk = a.kv_chunk;
    p.kv_lens = a.kv_lens;
    p.H = a.H > 0 ? a.H : 1;
    p.block_table = a.block_table;
    p.page_size = a.page_size;
    p.max_pages = a.max_pages;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = device_status_word();
    LaunchScope ls(K_DECODE_GQ, st);
    attn_decode_gq_sm100_kernel<kD, kG, kCache><<<(unsigned)a.BH, kThreads, GqCfg<kD>::kSmemBytes, st>>>(
        *reinterpret_cast<CUtensorMap*>(tq.bytes), *reinterpret_cast<CUtensorMap*>(tk.bytes),
        *reinterpret_cast<CUtensorMap*>(tv.bytes), p);
    return cudaGetLastError();
}

}  // namespace

// `a` is the forward view of a grouped decode (see decode_as_forward / paged_as_forward in
// attn_decode.cu): S = query heads per key/value head, BH = key/value slices x key ranges.
// TT_DECODE_GQA_PATH=fwd keeps such problems on the general forward kernel (tests, measurements).
bool attn_decode_gq_sm100_supported(const AttnArgs& a) {
    if (!a.bf16 || (a.D != 128 && a.D != 64) || a.causal || a.group != 1 || a.S < 1 || a.S > 16 || a.L < 1 || a.cu_q != nullptr) return false;
    if (a.BH < 1 || a.BH >= (1LL << 31)) return false;
    if (a.cache_mode) {
        if (a.q_div > 1 ? !(a.kv_chunk >= 128 && a.kv_chunk % 128 == 0) : a.kv_chunk != 0) return false;
        const int ps = a.page_size;   // paged: whole pages per TMA box
        if (a.block_table != nullptr && !(ps >= 8 && (128 % ps == 0 || ps % 128 == 0) && a.max_pages >= 1)) return false;
    } else if (a.block_table != nullptr || a.kv_lens != nullptr) {
        return false;
    }
    const char* f = getenv("TT_DECODE_GQA_PATH");
    return !(f && f[0] == 'f');
}

template <int kD>
static cudaError_t dispatch_gq(const AttnArgs& a, cudaStream_t st) {
    const bool cache = a.cache_mode != 0;
    if (a.S <= 4) return cache ? launch_gq<kD, 4, true>(a, st) : launch_gq<kD, 4, false>(a, st);
    if (a.S <= 8) return cache ? launch_gq<kD, 8, true>(a, st) : launch_gq<kD, 8, false>(a, st);
    return cache ? launch_gq<kD, 16, true>(a, st) : launch_gq<kD, 16, false>(a, st);
}
cudaError_t attn_decode_gq_sm100(const AttnArgs& a, cudaStream_t st) {
    return a.D == 128 ? dispatch_gq<128>(a, st) : dispatch_gq<64>(a, st);
}

}  // namespace ttk

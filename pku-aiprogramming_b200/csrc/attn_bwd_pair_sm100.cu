// dK/dV pass of the two-pass attention backward on CTA pairs (clusters of two, tcgen05 cta_group::2)
// for B200: bf16, head dim 128, dense [B,H,S,D] tensors.  Same arithmetic, roles and tensor-memory
// layout as the keys-resident instantiation of attn_bwd_sm100.cu; bit-identical results.
//
// A pair owns two consecutive key tiles of one key/value slice: the CTA of cluster rank r keeps
// K and V of key tile 2*pair + r in shared memory and accumulates that tile's dV and dK in its own
// tensor memory.  Both CTAs stream the same query tiles (Q_t, dO_t), and every MMA spans the pair
// (M = 256: 128 key rows per CTA), issued by one thread of the rank-0 CTA:
//     G1: S^T  = K Q_t^T    A = each CTA's K;   B = Q_t,  query rows [64r, 64r+64) from CTA r   (K-major)
//     G2: dP^T = V dO_t^T   A = each CTA's V;   B = dO_t, query rows [64r, 64r+64) from CTA r   (K-major)
//     G3: dV  += P^T dO_t   A = P^T  (tensor memory); B = dO_t, columns [64r, 64r+64) from CTA r (MN-major)
//     G4: dK  += dS^T Q_t   A = dS^T (tensor memory); B = Q_t,  columns [64r, 64r+64) from CTA r (MN-major)
// The hardware splits B along N over the pair, and N is the query index in G1/G2 but the head
// dimension in G3/G4, so a CTA holds two views of each streamed tile -- a row half for the score GEMMs
// and a column half for the accumulation GEMMs, 16 KB each: it loads as many bytes as the one-CTA
// kernel, but every MMA reads half as much B from each SM's shared memory.  (That traffic turned out
// not to be what paces the one-CTA pass: see the measurements at attn_bwd_dkv_pair_supported below.
// The kernel is kept as an opt-in path.)
//
// Under the causal mask the pair streams the query tiles its earlier key tile (rank 0) can see; for
// the rank-1 CTA the first of them is fully masked, which its compute threads turn into P = dS = 0.
// A key tile past the end of the keys (odd tile count) holds zeros and its rows are never stored.
#include "attn_bwd_common.cuh"

#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <type_traits>

namespace ttk {
using namespace sm100;

namespace {

struct BwdPairCfg : BwdRegs {
    static constexpr int D = 128;
    static constexpr int kSubBytes = 128 * 128;              // 16 KB: [128 rows x 128 B]
    static constexpr int kTileBytes = 2 * kSubBytes;         // 32 KB: a resident tile, or one streamed entry (row half + column half)
    static constexpr int kN0 = 3, kN1 = 2;                   // ring lengths of Q and dO entries
    static constexpr int kTmemCols = 512;
    static constexpr int kAuxBytes = 3072;                   // 1 KB barriers + 2 KB lse/delta staging
    static constexpr int kSmemBytes = (2 + kN0 + kN1) * kTileBytes + kAuxBytes;
    static_assert(kSmemBytes <= 227 * 1024, "exceeds the shared memory of one CTA");
};

// Work item = (key/value slice, pair of key tiles); numbered like the one-CTA pass (early key tiles
// first: under the causal mask they are the heavy ones; the lightest quarter in a second phase).
struct PairBwdItem {
    int bh;        // key/value slice
    int r0;        // first key row of THIS CTA's tile
    int t_begin, nt, n_it;
    int Lv;
};
__device__ __forceinline__ PairBwdItem pair_bwd_decode(int item, const BwdParams& p, int rank) {
    PairBwdItem w;
    int pos;   // position of the tile pair among its slice's pairs, heaviest first
    if (item < p.n_items_heavy) {
        const int n_heavy = p.n_tiles - p.n_light;
        w.bh = item / n_heavy;
        pos = item - w.bh * n_heavy;
    } else {
        const int r = item - p.n_items_heavy;
        w.bh = r / p.n_light;
        pos = (p.n_tiles - p.n_light) + (r - w.bh * p.n_light);
    }
    w.Lv = valid_keys(p.kv_lens, ((long long)w.bh * p.group) / p.H, p.L);
    const int off = p.L - p.S;
    const int k0 = pos * 256;                                  // first key of the pair
    int t_end = (p.S + 127) >> 7;
    w.t_begin = p.causal ? (max(0, k0 - off) >> 7) : 0;
    if (k0 >= w.Lv) t_end = min(t_end, w.t_begin + 1);         // all padding: one tile keeps the hand-offs alive
    w.r0 = k0 + 128 * rank;
    w.nt = max(0, t_end - w.t_begin);
    w.n_it = w.nt * p.group;
    return w;
}
// u-th streamed tile of an item: query tile index and query slice (the group's heads one after the other)
__device__ __forceinline__ void pair_bwd_stream_tile(const PairBwdItem& w, int u, int group, int& t, int& slice) {
    const int hh = u / w.nt;
    t = w.t_begin + (u - hh * w.nt);
    slice = w.bh * group + hh;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(BwdPairCfg::kThreads, 1)
attn_bwd_dkv_pair_sm100_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                               const __grid_constant__ CUtensorMap tmQrows, const __grid_constant__ CUtensorMap tmQcols,
                               const __grid_constant__ CUtensorMap tmDOrows, const __grid_constant__ CUtensorMap tmDOcols,
                               const BwdParams p) {
    using Cfg = BwdPairCfg;
    constexpr int D = Cfg::D;
    constexpr int kN0 = Cfg::kN0, kN1 = Cfg::kN1;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = smem_raw;
    if ((smem_u32(smem_raw) & 1023u) != 0u) {   // the 128-byte swizzle of TMA and UMMA needs 1024-byte aligned tiles
        if (threadIdx.x == 0 && atomicCAS(p.status, 0u, (8u << 16) | (blockIdx.x & 0xffffu)) == 0u) {
            p.status[1] = 0xA116u;   // "alignment"
            p.status[2] = smem_u32(smem_raw);
            p.status[3] = 0u;
        }
        return;                      // every thread of every CTA takes this exit together: nothing was started
    }
    unsigned char* sR = smem;                                 // K, V of this CTA's key tile
    unsigned char* sT = smem + 2 * Cfg::kTileBytes;           // kN0 Q entries, then kN1 dO entries
    unsigned char* aux = smem + (2 + kN0 + kN1) * Cfg::kTileBytes;
    // (R0) = only the rank-0 CTA's copy is waited on
    uint64_t* bar_res_full = reinterpret_cast<uint64_t*>(aux);   // both loaders -> MMA (R0)
    uint64_t* bar_res_empty = bar_res_full + 1;                  // MMA -> this CTA's loader
    uint64_t* bar_t0_full = bar_res_empty + 1;                   // [3] (R0)
    uint64_t* bar_t0_empty = bar_t0_full + 3;                    // [3]
    uint64_t* bar_t1_full = bar_t0_empty + 3;                    // [2] (R0)
    uint64_t* bar_t1_empty = bar_t1_full + 2;                    // [2]
    uint64_t* bar_s_full = bar_t1_empty + 2;                     // MMA -> this CTA's compute threads
    uint64_t* bar_dp_full = bar_s_full + 1;
    uint64_t* bar_p_full = bar_dp_full + 1;                      // compute warps of both CTAs -> MMA (R0)
    uint64_t* bar_ds_full = bar_p_full + 1;                      // (R0)
    uint64_t* bar_final = bar_ds_full + 1;
    uint64_t* bar_acc_free = bar_final + 1;                      // (R0)
    uint64_t* bar_sched_full = bar_acc_free + 1;                 // [2]
    uint64_t* bar_sched_empty = bar_sched_full + 2;              // [2] (R0)
    uint64_t* bar_stat = bar_sched_empty + 2;                    // [2] per warpgroup: a tile's statistics are staged
    int* sched_item = reinterpret_cast<int*>(bar_stat + 2);      // [2]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(sched_item + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    float* s_stat = reinterpret_cast<float*>(aux + 1024);     // [2 buffers][2: -lse2, -delta][128]

    const int warp = uniform_warp_idx();
    const int lane = threadIdx.x & 31;
    const int rank = (int)cluster_cta_rank();

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_res_full, 1);
        mbar_init(bar_res_empty, 1);
        for (int s = 0; s < kN0; ++s) {
            mbar_init(&bar_t0_full[s], 1);
            mbar_init(&bar_t0_empty[s], 1);
        }
        for (int s = 0; s < kN1; ++s) {
            mbar_init(&bar_t1_full[s], 1);
            mbar_init(&bar_t1_empty[s], 1);
        }
        mbar_init(bar_s_full, 1);
        mbar_init(bar_dp_full, 1);
        mbar_init(bar_p_full, 16);       // 8 compute warps in each CTA
        mbar_init(bar_ds_full, 16);
        mbar_init(bar_final, 1);
        mbar_init(bar_acc_free, 16);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_stat[i], 128);
            mbar_init(&bar_sched_full[i], 1);
            mbar_init(&bar_sched_empty[i], 18);   // rank 0: 8 compute warps + MMA warp; rank 1: 8 compute warps + loader
        }
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 8) {
        tmem_alloc_pair(tmem_base_slot, Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    if (warp == 9 && lane == 0) {
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmQrows);
        tma_prefetch_desc(&tmQcols);
        tma_prefetch_desc(&tmDOrows);
        tma_prefetch_desc(&tmDOcols);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers exist and its tensor memory is allocated
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    WaitCtx wctx{p.status, abort_flag, warp};
    constexpr uint32_t kColS = 0, kColDP = 128, kColAcc0 = 256, kColAcc1 = 256 + D;

    auto next_item = [&](int k) -> int {
        const int slot = k & 1;
        if (!mbar_wait_cluster(&bar_sched_full[slot], (k >> 1) & 1, wctx, 80 + slot, k)) return -1;
        return sched_item[slot];
    };
    const uint32_t sched_empty_r0 = map_to_cta(smem_u32(&bar_sched_empty[0]), 0);   // [slot]: + 8 * slot

    if (warp < 8) {
        // ============================================================ compute warpgroups (both CTAs)
        setmaxnreg_inc<Cfg::kRegsCompute>();
        const int wg = warp >> 2;
        const int wq = warp & 3;
        const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_off + kColS + wg * 64;
        const uint32_t tDP = tmem_base + lane_off + kColDP + wg * 64;
        const int ctid = threadIdx.x;                          // 0..255 among compute threads
        const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2);
        const uint32_t p_full_r0 = map_to_cta(smem_u32(bar_p_full), 0);
        const uint32_t ds_full_r0 = map_to_cta(smem_u32(bar_ds_full), 0);
        const uint32_t acc_free_r0 = map_to_cta(smem_u32(bar_acc_free), 0);
        const int off = p.L - p.S;
        uint32_t git = 0;      // streamed tiles processed so far, over all items (barrier phases)
        for (int k = 0;; ++k) {
            const int item = next_item(k);
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(sched_empty_r0 + 8u * (uint32_t)(k & 1));
            if (item < 0) break;
            const PairBwdItem w = pair_bwd_decode(item, p, rank);
            const int bh = w.bh;
            const int rrow = w.r0 + wq * 32 + lane;            // this thread's key row
            // per-column statistics: each warpgroup stages the statistics of ITS 64 streamed queries
            // (columns wg*64..+63), one tile ahead of their use -- thread j of the warpgroup fetches
            // -lse2 (j < 64) or -delta (j >= 64) of query wg*64 + (j & 63)
            const int stat_j = ctid & 127;
            const int stat_q = wg * 64 + (stat_j & 63);          // query inside the streamed tile
            const int stat_slot = (stat_j >> 6) * 128 + stat_q;  // [-lse2 | -delta][128]
            const float* stat_src = (stat_j < 64 ? p.lse2 : p.delta);
            const float stat_oob = (stat_j < 64) ? -INFINITY : 0.f;
            // The load of the next tile's statistic is issued a whole iteration before its value is
            // used: nothing may consume `stat_raw` until the store at the top of the next iteration.
            float stat_raw = 0.f;
            bool stat_ok = false;
            auto stat_issue = [&](int u) {   // this thread's statistic of streamed tile u
                int tt, qs;
                pair_bwd_stream_tile(w, u, p.group, tt, qs);
                const int qrow = tt * 128 + stat_q;
                stat_ok = qrow < p.S;
                if (stat_ok) stat_raw = stat_src[(long long)qs * p.S + qrow];
            };
            auto stat_publish = [&](uint32_t g) {
                s_stat[(g & 1) * 256 + stat_slot] = stat_ok ? -stat_raw : stat_oob;
                mbar_arrive(&bar_stat[wg]);
            };
            if (w.n_it > 0) {
                stat_issue(0);
                stat_publish(git);            // first tile of the item: the one exposed load
                if (w.n_it > 1) stat_issue(1);
            }
            for (int u = 0; u < w.n_it; ++u, ++git) {
                const int t = w.t_begin + u % w.nt;
                const int c0 = t * 128;                            // first streamed query of this tile
                const float* st_nlse = s_stat + (git & 1) * 256;   // -lse2 of the 128 streamed queries
                const float* st_ndelta = st_nlse + 128;            // -delta
                mbar_wait(&bar_stat[wg], git & 1, wctx, 35, u);    // tile u's statistics are staged
                // visible columns (queries) of this thread's key row inside the tile: [vis_lo, 128)
                const int vis_lo = p.causal ? max(0, rrow - off - c0) : 0;   // query >= key - off
                const bool need_mask = vis_lo > 0;
                uint64_t stat_reg[2][16];
                auto load_stats = [&](const float* src) {
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc)
#pragma unroll
                        for (int e4 = 0; e4 < 8; ++e4) {
                            const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(src + wg * 64 + cc * 32 + e4 * 4);
                            stat_reg[cc][2 * e4] = v.x;
                            stat_reg[cc][2 * e4 + 1] = v.y;
                        }
                };
                // ---------------- phase A: P = exp2(S*c - lse2)
                load_stats(st_nlse);
                mbar_wait(bar_s_full, git & 1, wctx, 30, u);
                __syncwarp();
                tc_fence_after();
                uint64_t pf2[32];     // this thread's 64 probabilities, fp32 pairs
                uint32_t sr[2][32], dr[2][32];
                auto phase_a_body = [&](auto masked_c, int cc) {
                    constexpr bool kMasked = decltype(masked_c)::value;
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const int col = wg * 64 + cc * 32 + e;
                        const uint64_t x = fma_f32x2(pack_f32x2(__uint_as_float(sr[cc][e]), __uint_as_float(sr[cc][e + 1])), c2,
                                                     stat_reg[cc][e >> 1]);
                        float a0, a1;
                        unpack_f32x2(x, a0, a1);
                        float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
                        if (kMasked) {
                            p0 = (col >= vis_lo) ? p0 : 0.f;
                            p1 = (col + 1 >= vis_lo) ? p1 : 0.f;
                        }
                        pf2[cc * 16 + (e >> 1)] = pack_f32x2(p0, p1);
                    }
                };
                auto phase_a = [&](int cc) {
                    if (need_mask) phase_a_body(std::true_type{}, cc);
                    else phase_a_body(std::false_type{}, cc);
                };
                // dS = P * (dP - delta) for one chunk; the 32 fp32 dP columns just read then hold 16
                // columns of bf16 P^T and 16 of dS^T
                auto phase_b = [&](int cc) {
                    uint32_t pk[16], pkp[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const uint64_t tdiff = add_f32x2(pack_f32x2(__uint_as_float(dr[cc][e]), __uint_as_float(dr[cc][e + 1])),
                                                         stat_reg[cc][e >> 1]);
                        const uint64_t ds = mul_f32x2(pf2[cc * 16 + (e >> 1)], tdiff);
                        float x0, x1, q0, q1;
                        unpack_f32x2(ds, x0, x1);
                        pk[e >> 1] = pack_bf16x2(x0, x1);
                        unpack_f32x2(pf2[cc * 16 + (e >> 1)], q0, q1);
                        pkp[e >> 1] = pack_bf16x2(q0, q1);
                    }
                    tmem_st16(tDP + cc * 32, pkp);
                    tmem_st16(tDP + cc * 32 + 16, pk);
                };
                tmem_ld32(tS, sr[0]);
                tmem_wait_ld();
                phase_a(0);
                tmem_ld32(tS + 32, sr[1]);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(p_full_r0);   // this warp's S(t) is in registers: its columns are free
                phase_a(1);
                load_stats(st_ndelta);
                if (u + 1 < w.n_it) {
                    stat_publish(git + 1);                     // its load was issued a tile ago
                    if (u + 2 < w.n_it) stat_issue(u + 2);
                }
                mbar_wait(bar_dp_full, git & 1, wctx, 31, u);
                __syncwarp();
                tc_fence_after();
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    tmem_ld32(tDP + cc * 32, dr[cc]);
                    tmem_wait_ld();
                    phase_b(cc);
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(ds_full_r0);
            }
            // ---------------- epilogue: accumulators out of tensor memory (then the issuer may start
            // the next item in them) -> bf16 -> global; warpgroup w owns columns [w*D/2, +D/2)
            mbar_wait(bar_final, k & 1, wctx, 34, k);
            __syncwarp();
            tc_fence_after();
            constexpr int kHalf = D / 2;
            uint32_t acc[2][kHalf / 32][32];
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                const uint32_t tA = tmem_base + lane_off + (a == 0 ? kColAcc0 : kColAcc1) + wg * kHalf;
#pragma unroll
                for (int cc = 0; cc < kHalf / 32; ++cc) tmem_ld32(tA + cc * 32, acc[a][cc]);
            }
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_free_r0);
            if (rrow < p.L) {
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    __nv_bfloat16* dst = (a == 0 ? p.out0 : p.out1) + ((long long)bh * p.L + rrow) * D + wg * kHalf;
                    if (rrow >= w.Lv) {   // gradients of padded keys are zero
#pragma unroll
                        for (int cc = 0; cc < kHalf / 32; ++cc)
#pragma unroll
                            for (int e = 0; e < 32; ++e) acc[a][cc][e] = 0u;
                    }
                    bwd_store_row<kHalf / 32>(dst, acc[a], a == 0 ? 1.0f : p.scale, p.wide_stores);
                }
            }
            __syncwarp();
        }
    } else {
        setmaxnreg_dec<Cfg::kRegsOther>();
        if (warp == 9) {
            // ============================================================ TMA loader (both CTAs; the rank-0
            // CTA's also takes the work items and publishes them to both)
            // a streamed entry: the row half (2 sub-blocks of 64 rows) then the column half (1 sub-block of 128 rows)
            auto load_entry = [&](unsigned char* dst, const CUtensorMap* rows, const CUtensorMap* cols, uint32_t full0, int t, int slice) {
#pragma unroll
                for (int sb = 0; sb < 2; ++sb) tma_load_3d_pair(dst + sb * (Cfg::kSubBytes / 2), rows, full0, sb * 64, t * 128 + 64 * rank, slice);
                tma_load_3d_pair(dst + Cfg::kSubBytes, cols, full0, 64 * rank, t * 128, slice);
            };
            uint32_t git = 0;
            for (int k = 0;; ++k) {
                int item = 0;
                const int slot = k & 1;
                if (rank == 0) {
                    if (lane == 0) item = (int)atomicAdd(p.sched_counter, 1u);
                    item = __shfl_sync(0xffffffffu, item, 0);
                    if (item >= p.n_items || *abort_flag) item = -1;   // an aborted pair takes no further items
                    mbar_wait(&bar_sched_empty[slot], ((k >> 1) & 1) ^ 1, wctx, 90 + slot, k);
                    __syncwarp();
                    if (lane == 0) {
                        sched_item[slot] = item;
                        st_shared_cluster_u32(map_to_cta(smem_u32(&sched_item[slot]), 1), (uint32_t)item);
                        mbar_arrive(&bar_sched_full[slot]);
                        mbar_arrive_cluster_release(map_to_cta(smem_u32(&bar_sched_full[slot]), 1));
                    }
                    __syncwarp();
                } else {
                    item = next_item(k);
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(sched_empty_r0 + 8u * (uint32_t)slot);
                    __syncwarp();
                }
                if (item < 0) break;
                const PairBwdItem w = pair_bwd_decode(item, p, rank);
                mbar_wait(bar_res_empty, (k & 1) ^ 1, wctx, 1, k);
                __syncwarp();
                if (elect_one()) {
                    if (rank == 0) mbar_arrive_expect_tx(bar_res_full, 4 * Cfg::kTileBytes);   // K and V of both CTAs
                    const uint32_t full0 = map_to_cta(smem_u32(bar_res_full), 0);
#pragma unroll
                    for (int sb = 0; sb < 2; ++sb) {
                        tma_load_3d_pair(sR + sb * Cfg::kSubBytes, &tmK, full0, sb * 64, w.r0, w.bh);
                        tma_load_3d_pair(sR + Cfg::kTileBytes + sb * Cfg::kSubBytes, &tmV, full0, sb * 64, w.r0, w.bh);
                    }
                }
                __syncwarp();
                for (int u = 0; u < w.n_it; ++u, ++git) {
                    const int s0 = git % kN0, s1 = git % kN1;
                    int t, ts;
                    pair_bwd_stream_tile(w, u, p.group, t, ts);
                    mbar_wait(&bar_t0_empty[s0], ((git / kN0) & 1) ^ 1, wctx, 20 + s0, (int)git);
                    __syncwarp();
                    if (elect_one()) {
                        if (rank == 0) mbar_arrive_expect_tx(&bar_t0_full[s0], 2 * Cfg::kTileBytes);
                        load_entry(sT + s0 * Cfg::kTileBytes, &tmQrows, &tmQcols, map_to_cta(smem_u32(&bar_t0_full[s0]), 0), t, ts);
                    }
                    __syncwarp();
                    mbar_wait(&bar_t1_empty[s1], ((git / kN1) & 1) ^ 1, wctx, 26 + s1, (int)git);
                    __syncwarp();
                    if (elect_one()) {
                        if (rank == 0) mbar_arrive_expect_tx(&bar_t1_full[s1], 2 * Cfg::kTileBytes);
                        load_entry(sT + (kN0 + s1) * Cfg::kTileBytes, &tmDOrows, &tmDOcols, map_to_cta(smem_u32(&bar_t1_full[s1]), 0), t, ts);
                    }
                    __syncwarp();
                }
            }
        } else if (warp == 8 && rank == 0) {
            // ============================================================ MMA issuer (rank-0 CTA)
            constexpr uint32_t idesc_s = umma_idesc_bf16(256, 128, false, false);
            constexpr uint32_t idesc_acc = umma_idesc_bf16(256, D, false, true);
            const uint32_t sR_addr = __shfl_sync(0xffffffffu, smem_u32(sR), 0);
            const uint32_t sT_addr = __shfl_sync(0xffffffffu, smem_u32(sT), 0);
            const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
            const uint64_t dR_base = umma_smem_desc(sR_addr, 16, 1024);                                   // K-major, 128 rows
            const uint64_t dT_rows_base = umma_smem_desc(sT_addr, 16, 1024);                              // K-major, 64 rows
            const uint64_t dT_cols_base = umma_smem_desc(sT_addr + Cfg::kSubBytes, Cfg::kSubBytes, 1024); // MN-major, 64 columns
            auto commit_both = [&](uint64_t* bar) {   // one arrival on this barrier in each CTA of the pair
                const uint32_t a = smem_u32(bar);
                tc_commit_pair(a);
                tc_commit_pair(map_to_cta(a, 1));
            };
            // G1 / G2: tmem[col] = R_which T^T for the streamed entry `entry`
            auto issue_score = [&](int which, int entry, uint32_t col) {
                const uint64_t a0 = umma_desc_advance(dR_base, which * Cfg::kTileBytes);
                const uint64_t b0 = umma_desc_advance(dT_rows_base, entry * Cfg::kTileBytes);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t oa = (kk >> 2) * Cfg::kSubBytes + (kk & 3) * 32;
                    const uint32_t ob = (kk >> 2) * (Cfg::kSubBytes / 2) + (kk & 3) * 32;
                    umma_ss_pair(tmem_u + col, umma_desc_advance(a0, oa), umma_desc_advance(b0, ob), idesc_s, kk > 0);
                }
            };
            // G3 / G4: tmem[acc] (+)= bf16 A in tensor memory (per 32-column chunk of the dP columns: 16 columns of
            // P^T (part 0) then 16 of dS^T (part 1)) times the streamed entry's column half
            auto issue_acc = [&](int entry, int part, uint32_t acc_col, bool accumulate) {
                const uint64_t b0 = umma_desc_advance(dT_cols_base, entry * Cfg::kTileBytes);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t in_wg = (uint32_t)(((kk & 3) >> 1) * 32 + part * 16 + (kk & 1) * 8);
                    const uint32_t a = tmem_u + kColDP + (kk >> 2) * 64 + in_wg;
                    umma_ts_pair(tmem_u + acc_col, a, umma_desc_advance(b0, kk * 2048), idesc_acc, (accumulate || kk > 0) ? 1u : 0u);
                }
            };
            uint32_t git = 0;      // streamed tiles issued before the current item
            for (int k = 0;; ++k) {
                const int item = next_item(k);
                __syncwarp();
                if (elect_one()) mbar_arrive(&bar_sched_empty[k & 1]);
                __syncwarp();
                if (item < 0) break;
                const PairBwdItem w = pair_bwd_decode(item, p, rank);
                const int n_it = w.n_it;
                mbar_wait(bar_res_full, k & 1, wctx, 0, k);
                __syncwarp();
                if (n_it > 0) {
                    // first scores of the item; the S / dP columns are free because the G3 / G4 of the
                    // previous item were issued earlier by this warp and execute in order
                    const int f0 = git % kN0, f1 = git % kN1;
                    mbar_wait(&bar_t0_full[f0], (git / kN0) & 1, wctx, 10 + f0, (int)git);
                    __syncwarp();
                    tc_fence_after();
                    issue_score(0, f0, kColS);
                    commit_both(bar_s_full);
                    mbar_wait(&bar_t1_full[f1], (git / kN1) & 1, wctx, 16 + f1, (int)git);
                    __syncwarp();
                    tc_fence_after();
                    issue_score(1, kN0 + f1, kColDP);
                    commit_both(bar_dp_full);
                    if (n_it == 1) commit_both(bar_res_empty);   // those were the item's last reads of the resident pair
                }
                for (int it = 0; it < n_it; ++it) {
                    const uint32_t g = git + it;
                    const int a0s = g % kN0, a1s = g % kN1;                  // entries of this tile
                    const bool has_next = it + 1 < n_it;
                    const int n0s = (g + 1) % kN0, n1s = (g + 1) % kN1;      // entries of the next tile
                    mbar_wait(bar_p_full, g & 1, wctx, 32, it);   // S(t) is in registers in both CTAs: its columns are free
                    __syncwarp();
                    tc_fence_after();
                    if (has_next) {
                        mbar_wait(&bar_t0_full[n0s], ((g + 1) / kN0) & 1, wctx, 10 + n0s, it + 1);
                        __syncwarp();
                        tc_fence_after();
                        issue_score(0, n0s, kColS);
                        commit_both(bar_s_full);
                    }
                    mbar_wait(bar_ds_full, g & 1, wctx, 33, it);  // dS^T and P^T are in the dP columns of both CTAs
                    __syncwarp();
                    tc_fence_after();
                    if (it == 0) {
                        // the accumulator columns must have been read out by the previous item's epilogues
                        mbar_wait(bar_acc_free, (k & 1) ^ 1, wctx, 36, k);
                        __syncwarp();
                    }
                    issue_acc(kN0 + a1s, 0, kColAcc0, it > 0);                       // dV += P^T dO
                    commit_both(&bar_t1_empty[a1s]);                                 // last read of dO(t)
                    issue_acc(a0s, 1, kColAcc1, it > 0);                             // dK += dS^T Q
                    commit_both(&bar_t0_empty[a0s]);                                 // last read of Q(t)
                    if (has_next) {
                        mbar_wait(&bar_t1_full[n1s], ((g + 1) / kN1) & 1, wctx, 16 + n1s, it + 1);
                        __syncwarp();
                        tc_fence_after();
                        issue_score(1, kN0 + n1s, kColDP);
                        commit_both(bar_dp_full);
                        if (it + 2 == n_it) commit_both(bar_res_empty);   // last reads of the resident pair
                    }
                }
                commit_both(bar_final);
                git += (uint32_t)n_it;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // neither CTA leaves while the other may still read its shared memory or arrive on its barriers
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

int max_resident_pairs() {
    static int cached[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!cached[dev]) {
        int n_sm = 148;
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        cudaFuncSetAttribute(attn_bwd_dkv_pair_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdPairCfg::kSmemBytes);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)n_sm & ~1u);
        cfg.blockDim = dim3(BwdPairCfg::kThreads);
        cfg.dynamicSmemBytes = BwdPairCfg::kSmemBytes;
        cudaLaunchAttribute at;
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = 2;
        at.val.clusterDim.y = 1;
        at.val.clusterDim.z = 1;
        cfg.attrs = &at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, attn_bwd_dkv_pair_sm100_kernel, &cfg) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = n_sm / 2;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace

// Takes dense bf16 tensors with head dim 128.  Not chosen by default: measured on B200 it computes the
// same bits as the one-CTA pass at the same speed on long sequences (S = 32768, 16 heads: backward 11.6
// against 11.5 ms) and 8 % slower at S = 4096 (1.67 against 1.54 ms) -- a tile's step is paced by the
// chain dS -> dV, dK, next dP -> next dS through the shared dP columns of tensor memory, not by the
// shared-memory reads the pair halves, and the pair's items are twice as coarse.  TT_BWD_DKV=2cta
// selects it (tests, measurements).
bool attn_bwd_dkv_pair_supported(const AttnArgs& a) {
    const char* f = getenv("TT_BWD_DKV");
    if (!(f && f[0] == '2')) return false;
    if (!a.bf16 || a.D != 128 || a.cu_q != nullptr || a.S < 1 || a.L < 1) return false;
    return (a.BH / a.group) * (long long)((((a.L + 127) / 128) + 1) / 2) < (1LL << 31);
}

cudaError_t attn_bwd_dkv_pair(const AttnArgs& a, const float* delta, const float* lse2, cudaStream_t st) {
    using Cfg = BwdPairCfg;
    constexpr int D = Cfg::D;
    TmapStorage tk, tv, tq64, tq128, tdo64, tdo128;
    const char* why = nullptr;
    if (!make_tmap_bf16(&tk, a.k, D, a.L, a.BH / a.group, 128, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tv, a.v, D, a.L, a.BH / a.group, 128, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tq64, a.q, D, a.S, a.BH, 64, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tq128, a.q, D, a.S, a.BH, 128, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tdo64, a.dout, D, a.S, a.BH, 64, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tdo128, a.dout, D, a.S, a.BH, 128, &why)) return cudaErrorInvalidValue;
    auto M = [](TmapStorage& t) -> CUtensorMap& { return *reinterpret_cast<CUtensorMap*>(t.bytes); };
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkv_pair_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    BwdParams p;
    memset(&p, 0, sizeof(p));
    p.lse2 = lse2;
    p.delta = delta;
    p.S = a.S;
    p.L = a.L;
    p.causal = a.causal;
    p.scale = a.scale;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = device_status_word();
    p.out0 = (__nv_bfloat16*)a.dv;
    p.out1 = (__nv_bfloat16*)a.dk;
    p.group = a.group;
    p.kv_lens = a.kv_lens;
    p.H = a.H;
    p.Hkv = a.H / a.group;
    const uintptr_t al = reinterpret_cast<uintptr_t>(a.dk) | reinterpret_cast<uintptr_t>(a.dv);
    p.wide_stores = (al & 31) == 0 ? 1 : 0;
    p.n_tiles = (((a.L + 127) / 128) + 1) / 2;   // pairs of key tiles per slice
    p.n_items = (int)(a.BH / a.group * p.n_tiles);
    p.n_light = a.causal ? p.n_tiles / 4 : 0;
    p.n_items_heavy = (int)(a.BH / a.group * (p.n_tiles - p.n_light));
    SchedCounter sc;
    e = sched_counter_acquire(st, &sc);
    if (e != cudaSuccess) return e;
    p.sched_counter = sc.ptr;
    const unsigned pairs = (unsigned)std::min<long long>(p.n_items, max_resident_pairs());
    {
        LaunchScope ls(K_BWD_DKV, st);
        attn_bwd_dkv_pair_sm100_kernel<<<2 * pairs, Cfg::kThreads, Cfg::kSmemBytes, st>>>(M(tk), M(tv), M(tq64), M(tq128), M(tdo64),
                                                                                          M(tdo128), p);
    }
    sched_counter_release(sc, st);
    return cudaGetLastError();
}

}  // namespace ttk

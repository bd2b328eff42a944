// Fused attention backward for B200 (sm_100a): bf16 tensors, fp32 accumulation, head dim 64
// or 128.  P is recomputed from Q, K and the forward's log-sum-exp; nothing of size S x L
// is ever stored.
//
//   delta = rowsum(dO * O)                      (small preprocessing kernel, also lse*log2e)
//   P  = exp(scale*Q K^T - lse)      dP = dO V^T       dS = P * (dP - delta)
//   dV = P^T dO      dK = scale * dS^T Q      dQ = scale * dS K
//
// Two launches of ONE kernel template, both free of atomics (bit-reproducible):
//   kKeysResident = true : a CTA owns 128 keys (K,V tiles stay in shared memory) and streams
//                          the query tiles (Q_i, dO_i) that can see them; it accumulates dV and
//                          dK in tensor memory.  Scores are computed transposed (keys on the
//                          TMEM lanes) so that P^T and dS^T are directly the A operands.
//   kKeysResident = false: a CTA owns 128 queries (Q,dO tiles resident) and streams (K_j,V_j);
//                          it accumulates dQ.
// With R = resident pair and T = streamed pair the four GEMMs of an iteration are
//   G1: S  = R0 T0^T   (A,B shared memory, K-major)        G2: dP = R1 T1^T
//   G3: acc0 += P  T1  (A tensor memory, B MN-major)  [keys resident only: dV]
//   G4: acc1 += dS T0  (A tensor memory, B MN-major)  [dK or dQ]
//
// Roles: warps 0-7 = two compute warpgroups (thread <-> resident row; warpgroup w owns
// score columns [64w, 64w+64)), warp 8 = MMA issuer, warp 9 = TMA loader.
// Tensor memory: S [0,128), dP [128,256), acc0 [256,256+D), acc1 [256+D,256+2D); the bf16
// P / dS written by warpgroup w overlay columns [64w,64w+32) of S / dP.
#include "common.h"
#include "sm100_ptx.cuh"
#include <stdlib.h>

namespace ttk {
using namespace sm100;

template <int D>
struct BwdCfg {
    static constexpr int kSub = D / 64;
    static constexpr int kSubBytes = 128 * 128;
    static constexpr int kTileBytes = kSub * kSubBytes;
    static constexpr int kStages = (D == 128) ? 2 : 4;              // streamed (T0,T1) pairs in flight
    static constexpr int kThreads = 384;
    static constexpr int kTmemCols = 512;
    static constexpr int kAuxBytes = 4096;                           // barriers + lse/delta staging
    static constexpr int kSmemBytes = (2 + 2 * kStages) * kTileBytes + kAuxBytes + 1024;
};

enum BwdBarId { BB_RES = 0, BB_STFULL = 10, BB_STEMPTY = 20, BB_SFULL = 30, BB_DPFULL = 31, BB_PFULL = 32,
                BB_DSFULL = 33, BB_FINAL = 34, BB_PREAD = 35 };

struct BwdParams {
    __nv_bfloat16* out0;   // keys resident: dV ; else unused
    __nv_bfloat16* out1;   // keys resident: dK ; else dQ
    const float* lse2;     // [BH,S]  lse * log2(e)
    const float* delta;    // [BH,S]
    int S, L;
    int n_tiles;           // resident tiles per slice
    int causal;
    float scale, scale_log2;
    unsigned int* status;
    long long* trace;   // optional cycle trace of one CTA (debug aid): [3 roles][64 iterations][8 stamps]
    int trace_block;
};

#define TT_BTRACE(role, iter, slot)                                                                 \
    do {                                                                                           \
        if (p.trace != nullptr && (int)blockIdx.x == p.trace_block && (iter) < 64)                 \
            p.trace[((role) * 64 + (iter)) * 8 + (slot)] = clock64();                              \
    } while (0)

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// kPoly: of every 8 pairs of exponentials, kPoly are evaluated by a polynomial on the FMA pipes
// instead of the special-function unit.
template <int D, bool kKeysResident, int kPoly>
__global__ void __launch_bounds__(BwdCfg<D>::kThreads, 1)
attn_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmR0, const __grid_constant__ CUtensorMap tmR1,
                      const __grid_constant__ CUtensorMap tmT0, const __grid_constant__ CUtensorMap tmT1,
                      const BwdParams p) {
    using Cfg = BwdCfg<D>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sR = smem;                                 // R0, R1
    unsigned char* sT = smem + 2 * Cfg::kTileBytes;           // kStages x (T0, T1)
    unsigned char* aux = smem + (2 + 2 * kStages) * Cfg::kTileBytes;
    uint64_t* bar_res = reinterpret_cast<uint64_t*>(aux);     // [1]
    uint64_t* bar_st_full = bar_res + 1;                      // [kStages]
    uint64_t* bar_st_empty = bar_st_full + kStages;           // [kStages]
    uint64_t* bar_s_full = bar_st_empty + kStages;
    uint64_t* bar_dp_full = bar_s_full + 1;
    uint64_t* bar_p_full = bar_dp_full + 1;
    uint64_t* bar_ds_full = bar_p_full + 1;
    uint64_t* bar_final = bar_ds_full + 1;
    uint64_t* bar_p_read = bar_final + 1;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bar_p_read + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    float* s_stat = reinterpret_cast<float*>(aux + 1024);     // [2 buffers][2: lse2, delta][128]

    const int warp = uniform_warp_idx();
    const int lane = threadIdx.x & 31;
    const int off = p.L - p.S;
    const int bh = blockIdx.x / p.n_tiles;
    int rt;            // resident tile index
    int t_begin, t_end;  // streamed tile range [t_begin, t_end)
    if (kKeysResident) {
        rt = (int)(blockIdx.x % p.n_tiles);                           // early key tiles are the heavy ones
        t_end = (p.S + 127) >> 7;
        t_begin = p.causal ? (max(0, rt * 128 - off) >> 7) : 0;
    } else {
        rt = p.n_tiles - 1 - (int)(blockIdx.x % p.n_tiles);           // late query tiles are the heavy ones
        const int n_kv = (p.L + 127) >> 7;
        t_begin = 0;
        t_end = p.causal ? min(n_kv, ((min(rt * 128 + 127, p.S - 1) + off) >> 7) + 1) : n_kv;
    }
    const int r0 = rt * 128;   // first resident row (key or query index)

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_res, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bar_st_full[s], 1);
            mbar_init(&bar_st_empty[s], 1);
        }
        mbar_init(bar_s_full, 1);
        mbar_init(bar_dp_full, 1);
        mbar_init(bar_p_full, 256);
        mbar_init(bar_ds_full, 256);
        mbar_init(bar_p_read, 1);
        mbar_init(bar_final, 1);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 8) {
        tmem_alloc(tmem_base_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    if (warp == 9 && lane == 0) {
        tma_prefetch_desc(&tmR0);
        tma_prefetch_desc(&tmR1);
        tma_prefetch_desc(&tmT0);
        tma_prefetch_desc(&tmT1);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    WaitCtx wctx{p.status, abort_flag, warp};
    constexpr uint32_t kColS = 0, kColDP = 128, kColAcc0 = 256, kColAcc1 = 256 + D;

    if (warp < 8) {
        // ============================================================ compute warpgroups
        setmaxnreg_inc<224>();
        const int wg = warp >> 2;
        const int wq = warp & 3;
        const int rrow = r0 + wq * 32 + lane;                  // this thread's resident row
        const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_off + kColS + wg * 64;
        const uint32_t tDP = tmem_base + lane_off + kColDP + wg * 64;
        const int ctid = threadIdx.x;                          // 0..255 among compute threads
        // row constants (queries resident) as packed pairs of the NEGATED values
        uint64_t row_nlse2 = 0, row_ndelta2 = 0;
        if (!kKeysResident) {
            const bool ok = rrow < p.S;
            const float nl = ok ? -p.lse2[(long long)bh * p.S + rrow] : -INFINITY;
            const float nd = ok ? -p.delta[(long long)bh * p.S + rrow] : 0.f;
            row_nlse2 = pack_f32x2(nl, nl);
            row_ndelta2 = pack_f32x2(nd, nd);
        }
        // per-column statistics (keys resident): thread ctid fetches -lse2 (ctid < 128) or -delta of
        // streamed query (ctid & 127), one tile ahead of its use
        const float* stat_src = (ctid < 128 ? p.lse2 : p.delta) + (long long)bh * p.S;
        const float stat_oob = (ctid < 128) ? -INFINITY : 0.f;
        float stat_next = stat_oob;
        if (kKeysResident && t_begin < t_end) {
            const int qrow = t_begin * 128 + (ctid & 127);
            stat_next = qrow < p.S ? -stat_src[qrow] : stat_oob;
        }
        const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2);
        for (int t = t_begin; t < t_end; ++t) {
            const int it = t - t_begin;
            const int c0 = t * 128;                            // first streamed row of this tile
            if (wq == 0 && lane == 0) TT_BTRACE(wg, it, 0);
            const float* st_nlse = s_stat + (it & 1) * 256;    // -lse2 of the 128 streamed queries
            const float* st_ndelta = st_nlse + 128;            // -delta
            if (kKeysResident) {
                s_stat[(it & 1) * 256 + ctid] = stat_next;
                named_bar_sync(1, 256);
                if (t + 1 < t_end) {
                    const int qrow = (t + 1) * 128 + (ctid & 127);
                    stat_next = qrow < p.S ? -stat_src[qrow] : stat_oob;
                }
            }
            // visible columns of this thread's row inside the tile: [vis_lo, vis_hi)
            int vis_lo = 0, vis_hi = 128;
            if (kKeysResident) {
                if (p.causal) vis_lo = max(0, rrow - off - c0);           // query >= key - off
            } else {
                vis_hi = p.L - c0;
                if (p.causal) vis_hi = min(vis_hi, rrow + off + 1 - c0);  // key <= query + off
                vis_hi = min(vis_hi, 128);
            }
            const bool need_mask = (vis_lo > 0) || (vis_hi < 128);
            // ---------------- phase A: P = exp2(S*c - lse2)
            if (wq == 0 && lane == 0) TT_BTRACE(wg, it, 1);
            mbar_wait(bar_s_full, it & 1, wctx, BB_SFULL, it);
            __syncwarp();
            tc_fence_after();
            if (wq == 0 && lane == 0) TT_BTRACE(wg, it, 2);
            uint64_t pf2[32];     // this thread's 64 probabilities, fp32 pairs
            uint32_t sr[2][32];
            if (!kKeysResident) {
                // nothing is written back into the S columns in this pass: release them as soon as
                // they are in registers so that the next tile's scores overlap these exponentials
                tmem_ld32(tS, sr[0]);
                tmem_ld32(tS + 32, sr[1]);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(bar_p_full);
            }
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                if (kKeysResident) {
                    tmem_ld32(tS + cc * 32, sr[cc]);
                    tmem_wait_ld();
                }
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const int col = wg * 64 + cc * 32 + e;
                    const uint64_t nl = kKeysResident ? *reinterpret_cast<const uint64_t*>(st_nlse + col) : row_nlse2;
                    const uint64_t x = fma_f32x2(pack_f32x2(__uint_as_float(sr[cc][e]), __uint_as_float(sr[cc][e + 1])), c2, nl);
                    float p0, p1;
                    if ((((e >> 1) * kPoly) % 8) < kPoly) {   // kPoly of every 8 pairs on the FMA pipes
                        ex2_poly_x2(x, p0, p1);
                    } else {
                        float a0, a1;
                        unpack_f32x2(x, a0, a1);
                        p0 = ex2_approx(a0);
                        p1 = ex2_approx(a1);
                    }
                    if (need_mask) {
                        p0 = (col >= vis_lo && col < vis_hi) ? p0 : 0.f;
                        p1 = (col + 1 >= vis_lo && col + 1 < vis_hi) ? p1 : 0.f;
                    }
                    pf2[cc * 16 + (e >> 1)] = pack_f32x2(p0, p1);
                    if (kKeysResident) pk[e >> 1] = pack_bf16x2(p0, p1);
                }
                if (kKeysResident) tmem_st16(tS + cc * 16, pk);
            }
            if (kKeysResident) {
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar_p_full);
            }
            if (wq == 0 && lane == 0) TT_BTRACE(wg, it, 3);
            // ---------------- phase B: dS = P * (dP - delta)
            mbar_wait(bar_dp_full, it & 1, wctx, BB_DPFULL, it);
            __syncwarp();
            tc_fence_after();
            if (wq == 0 && lane == 0) TT_BTRACE(wg, it, 4);
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t dr[32];
                tmem_ld32(tDP + cc * 32, dr);
                tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const int col = wg * 64 + cc * 32 + e;
                    const uint64_t nd = kKeysResident ? *reinterpret_cast<const uint64_t*>(st_ndelta + col) : row_ndelta2;
                    const uint64_t tdiff = add_f32x2(pack_f32x2(__uint_as_float(dr[e]), __uint_as_float(dr[e + 1])), nd);
                    const uint64_t ds = mul_f32x2(pf2[cc * 16 + (e >> 1)], tdiff);
                    float x0, x1;
                    unpack_f32x2(ds, x0, x1);
                    pk[e >> 1] = pack_bf16x2(x0, x1);
                }
                tmem_st16(tDP + cc * 16, pk);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar_ds_full);
            if (wq == 0 && lane == 0) TT_BTRACE(wg, it, 5);
        }
        // ---------------- epilogue: accumulators -> bf16 -> global (warpgroup w: columns [w*D/2, +D/2))
        mbar_wait(bar_final, 0, wctx, BB_FINAL, 0);
        __syncwarp();
        tc_fence_after();
        const int n_rows = kKeysResident ? p.L : p.S;
        const bool row_ok = rrow < n_rows;
        constexpr int kHalf = D / 2;
#pragma unroll
        for (int a = (kKeysResident ? 0 : 1); a < 2; ++a) {
            __nv_bfloat16* dst = (a == 0 ? p.out0 : p.out1) + ((long long)bh * n_rows + rrow) * D + wg * kHalf;
            const float mul = (a == 0) ? 1.0f : p.scale;
            const uint32_t tA = tmem_base + lane_off + (a == 0 ? kColAcc0 : kColAcc1) + wg * kHalf;
#pragma unroll
            for (int cc = 0; cc < kHalf / 32; ++cc) {
                uint32_t orr[32];
                __syncwarp();
                tmem_ld32(tA + cc * 32, orr);
                tmem_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint4 w;
                        w.x = pack_bf16x2(__uint_as_float(orr[e + 0]) * mul, __uint_as_float(orr[e + 1]) * mul);
                        w.y = pack_bf16x2(__uint_as_float(orr[e + 2]) * mul, __uint_as_float(orr[e + 3]) * mul);
                        w.z = pack_bf16x2(__uint_as_float(orr[e + 4]) * mul, __uint_as_float(orr[e + 5]) * mul);
                        w.w = pack_bf16x2(__uint_as_float(orr[e + 6]) * mul, __uint_as_float(orr[e + 7]) * mul);
                        *reinterpret_cast<uint4*>(dst + cc * 32 + e) = w;
                    }
                }
            }
        }
    } else {
        setmaxnreg_dec<56>();
        if (warp == 9) {
            // ============================================================ TMA loader (whole warp runs the
            // control flow, one elected lane issues)
            auto load_tile = [&](unsigned char* dst, const CUtensorMap* tm, uint64_t* bar, int row_start) {
#pragma unroll
                for (int sb = 0; sb < Cfg::kSub; ++sb) tma_load_3d(dst + sb * Cfg::kSubBytes, tm, bar, sb * 64, row_start, bh);
            };
            if (elect_one()) {
                mbar_arrive_expect_tx(bar_res, 2 * Cfg::kTileBytes);
                load_tile(sR, &tmR0, bar_res, r0);
                load_tile(sR + Cfg::kTileBytes, &tmR1, bar_res, r0);
            }
            __syncwarp();
            for (int t = t_begin; t < t_end; ++t) {
                const int it = t - t_begin;
                const int slot = it % kStages;
                mbar_wait(&bar_st_empty[slot], ((it / kStages) & 1) ^ 1, wctx, BB_STEMPTY + slot, it);
                __syncwarp();
                if (elect_one()) {
                    mbar_arrive_expect_tx(&bar_st_full[slot], 2 * Cfg::kTileBytes);
                    unsigned char* dst = sT + slot * 2 * Cfg::kTileBytes;
                    load_tile(dst, &tmT0, &bar_st_full[slot], t * 128);
                    load_tile(dst + Cfg::kTileBytes, &tmT1, &bar_st_full[slot], t * 128);
                }
                __syncwarp();
            }
        } else if (warp == 8) {
            // ============================================================ MMA issuer (whole warp runs the
            // control flow; each tcgen05.mma / commit is issued by one elected lane, so descriptors and
            // addresses stay on the uniform datapath)
            constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);
            constexpr uint32_t idesc_acc = umma_idesc_bf16(128, D, false, true);
            const uint32_t sR_addr = __shfl_sync(0xffffffffu, smem_u32(sR), 0);
            const uint32_t sT_addr = __shfl_sync(0xffffffffu, smem_u32(sT), 0);
            const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
            const uint64_t dR_base = umma_smem_desc(sR_addr, 16, 1024);                   // K-major
            const uint64_t dT_base = umma_smem_desc(sT_addr, 16, 1024);                   // K-major
            const uint64_t dT_mn_base = umma_smem_desc(sT_addr, Cfg::kSubBytes, 1024);    // MN-major
            // G1 / G2: tmem[col] = R_which T_which^T for the pair in `slot`
            auto issue_score = [&](int which, int slot, uint32_t col) {
                const uint64_t a0 = umma_desc_advance(dR_base, which * Cfg::kTileBytes);
                const uint64_t b0 = umma_desc_advance(dT_base, (slot * 2 + which) * Cfg::kTileBytes);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t o = (kk >> 2) * Cfg::kSubBytes + (kk & 3) * 32;
                    umma_ss(tmem_u + col, umma_desc_advance(a0, o), umma_desc_advance(b0, o), idesc_s, kk > 0);
                }
            };
            // G3 / G4: tmem[acc] (+)= bf16 A at tmem[a_col] (two 32-column halves) times T_which (MN-major)
            auto issue_acc = [&](int which, int slot, uint32_t a_col, uint32_t acc_col, bool accumulate) {
                const uint64_t b0 = umma_desc_advance(dT_mn_base, (slot * 2 + which) * Cfg::kTileBytes);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t a = tmem_u + a_col + (kk >> 2) * 64 + (kk & 3) * 8;
                    umma_ts(tmem_u + acc_col, a, umma_desc_advance(b0, kk * 2048), idesc_acc,
                            (accumulate || kk > 0) ? 1u : 0u);
                }
            };
            const int n_it = t_end - t_begin;
            mbar_wait(bar_res, 0, wctx, BB_RES, 0);
            __syncwarp();
            if (n_it > 0) {
                mbar_wait(&bar_st_full[0], 0, wctx, BB_STFULL, 0);
                __syncwarp();
                tc_fence_after();
                issue_score(0, 0, kColS);
                tc_commit(bar_s_full);
                issue_score(1, 0, kColDP);
                tc_commit(bar_dp_full);
            }
            for (int it = 0; it < n_it; ++it) {
                const int slot = it % kStages;
                const bool has_next = it + 1 < n_it;
                const int nslot = (it + 1) % kStages;
                if (lane == 0) TT_BTRACE(2, it, 0);
                mbar_wait(bar_p_full, it & 1, wctx, BB_PFULL, it);
                __syncwarp();
                tc_fence_after();
                if (lane == 0) TT_BTRACE(2, it, 1);
                if (kKeysResident) issue_acc(1, slot, kColS, kColAcc0, it > 0);     // dV += P^T dO
                if (has_next) {
                    mbar_wait(&bar_st_full[nslot], ((it + 1) / kStages) & 1, wctx, BB_STFULL + nslot, it + 1);
                    __syncwarp();
                    tc_fence_after();
                    issue_score(0, nslot, kColS);
                    tc_commit(bar_s_full);
                }
                if (lane == 0) TT_BTRACE(2, it, 2);
                mbar_wait(bar_ds_full, it & 1, wctx, BB_DSFULL, it);
                __syncwarp();
                tc_fence_after();
                if (lane == 0) TT_BTRACE(2, it, 3);
                issue_acc(0, slot, kColDP, kColAcc1, it > 0);                        // dK += dS^T Q | dQ += dS K
                tc_commit(&bar_st_empty[slot]);
                if (has_next) {
                    issue_score(1, nslot, kColDP);
                    tc_commit(bar_dp_full);
                }
                if (lane == 0) TT_BTRACE(2, it, 4);
            }
            tc_commit(bar_final);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---------------------------------------------------------------- preprocessing
// delta[row] = sum_d dO*O ; lse2[row] = lse[row] * log2(e).  One warp per row.
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                     const float* __restrict__ lse, float* __restrict__ delta,
                                     float* __restrict__ lse2, long long n_rows, int D) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= n_rows) return;
    const uint2* o2 = reinterpret_cast<const uint2*>(out + row * D);
    const uint2* d2 = reinterpret_cast<const uint2*>(dout + row * D);
    float acc = 0.f;
    for (int i = lane; i < D / 4; i += 32) {
        uint2 a = o2[i], b = d2[i];
        acc = fmaf(__uint_as_float(a.x << 16), __uint_as_float(b.x << 16), acc);
        acc = fmaf(__uint_as_float(a.x & 0xffff0000u), __uint_as_float(b.x & 0xffff0000u), acc);
        acc = fmaf(__uint_as_float(a.y << 16), __uint_as_float(b.y << 16), acc);
        acc = fmaf(__uint_as_float(a.y & 0xffff0000u), __uint_as_float(b.y & 0xffff0000u), acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        delta[row] = acc;
        lse2[row] = lse[row] * 1.4426950408889634f;
    }
}

// ---------------------------------------------------------------- host side
bool attn_bwd_sm100_supported(const AttnArgs& a) {
    long long tiles = ((long long)(a.S > a.L ? a.S : a.L) + 127) / 128;
    return a.bf16 && (a.D == 64 || a.D == 128) && a.BH * tiles < (1LL << 31);
}
size_t attn_bwd_sm100_workspace(const AttnArgs& a) { return 2 * align256((size_t)a.BH * a.S * sizeof(float)); }

static long long* g_bwd_trace = nullptr;
static int g_bwd_trace_block = 0, g_bwd_trace_mode = 0;   // mode 1: dK/dV pass, 2: dQ pass
void attn_bwd_set_trace(long long* device_buf, int block, int pass) {
    g_bwd_trace = device_buf;
    g_bwd_trace_block = block;
    g_bwd_trace_mode = device_buf ? pass : 0;
}

template <int D, int kPoly>
static cudaError_t launch_bwd(const AttnArgs& a, void* ws, cudaStream_t st) {
    using Cfg = BwdCfg<D>;
    float* delta = reinterpret_cast<float*>(ws);
    float* lse2 = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(ws) + align256((size_t)a.BH * a.S * sizeof(float)));
    const long long n_rows = a.BH * (long long)a.S;
    {
        LaunchScope ls(K_BWD_PREP, st);
        attn_bwd_prep_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, st>>>(
            (const __nv_bfloat16*)a.out, (const __nv_bfloat16*)a.dout, a.lse, delta, lse2, n_rows, D);
    }
    TmapStorage tq, tk, tv, tdo;
    const char* why = nullptr;
    if (!make_tmap_bf16(&tq, a.q, D, a.S, a.BH, 128, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tk, a.k, D, a.L, a.BH, 128, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tv, a.v, D, a.L, a.BH, 128, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tdo, a.dout, D, a.S, a.BH, 128, &why)) return cudaErrorInvalidValue;
    auto M = [](TmapStorage& t) -> CUtensorMap& { return *reinterpret_cast<CUtensorMap*>(t.bytes); };
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_sm100_kernel<D, true, kPoly>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(attn_bwd_sm100_kernel<D, false, kPoly>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    BwdParams p;
    p.lse2 = lse2;
    p.delta = delta;
    p.S = a.S;
    p.L = a.L;
    p.causal = a.causal;
    p.scale = a.scale;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = device_status_word();
    p.trace = g_bwd_trace_mode == 1 ? g_bwd_trace : nullptr;
    p.trace_block = g_bwd_trace_block;
    // dK, dV: keys resident, stream (Q, dO)
    p.out0 = (__nv_bfloat16*)a.dv;
    p.out1 = (__nv_bfloat16*)a.dk;
    p.n_tiles = (a.L + 127) / 128;
    {
        LaunchScope ls(K_BWD_DKV, st);
        attn_bwd_sm100_kernel<D, true, kPoly><<<(unsigned)(a.BH * p.n_tiles), Cfg::kThreads, Cfg::kSmemBytes, st>>>(
            M(tk), M(tv), M(tq), M(tdo), p);
    }
    // dQ: queries resident, stream (K, V)
    p.trace = g_bwd_trace_mode == 2 ? g_bwd_trace : nullptr;
    p.out0 = nullptr;
    p.out1 = (__nv_bfloat16*)a.dq;
    p.n_tiles = (a.S + 127) / 128;
    {
        LaunchScope ls(K_BWD_DQ, st);
        attn_bwd_sm100_kernel<D, false, kPoly><<<(unsigned)(a.BH * p.n_tiles), Cfg::kThreads, Cfg::kSmemBytes, st>>>(
            M(tq), M(tdo), M(tk), M(tv), p);
    }
    return cudaGetLastError();
}

static int bwd_poly_setting() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("TT_BWD_POLY");
        v = (e && *e) ? atoi(e) : 0;
        if (v != 0 && v != 2 && v != 4 && v != 6) v = 0;
    }
    return v;
}
template <int D>
static cudaError_t launch_bwd_d(const AttnArgs& a, void* ws, cudaStream_t st) {
    switch (bwd_poly_setting()) {
        case 2: return launch_bwd<D, 2>(a, ws, st);
        case 4: return launch_bwd<D, 4>(a, ws, st);
        case 6: return launch_bwd<D, 6>(a, ws, st);
        default: return launch_bwd<D, 0>(a, ws, st);
    }
}
cudaError_t attn_bwd_sm100(const AttnArgs& a, void* ws, cudaStream_t st) {
    return a.D == 128 ? launch_bwd_d<128>(a, ws, st) : launch_bwd_d<64>(a, ws, st);
}

}  // namespace ttk

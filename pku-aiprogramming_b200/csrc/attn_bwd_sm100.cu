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
// score columns [64w, 64w+64)), warp 8 = MMA issuer, warp 9 = TMA loader and work-item scheduler.
// Tensor memory: S [0,128), dP [128,256), acc0 [256,256+D), acc1 [256+D,256+2D).  A compute
// thread reads its S values (which frees the S columns for the next tile's G1 at once), forms P in
// registers, reads its dP values, and writes the bf16 dS^T -- with keys resident also the bf16
// P^T -- over the dP columns it has just read; G3, G4 and the next G2 follow back to back.
// With queries resident acc0 is not needed: its columns hold a copy of the resident pair, which
// from an item's second tile on is the A operand of G1 and G2 (tensor memory instead of shared
// memory, which is the scarcer bandwidth).
// Shared memory: the resident pair plus rings of 3 (T0) and 2 (T1) streamed tiles at D = 128,
// barriers and 2 KB of per-column statistics: exactly 227 KB.
#include "attn_bwd_common.cuh"
#include <string.h>
#include <algorithm>

namespace ttk {
using namespace sm100;

template <int D>
struct BwdCfg : BwdRegs {
    static constexpr int kSub = D / 64;
    static constexpr int kSubBytes = 128 * 128;
    static constexpr int kTileBytes = kSub * kSubBytes;
    // Streamed tiles held in shared memory.  At D = 128 (32 KB tiles) the two resident tiles, five
    // streamed ones and 3 KB of barriers and staging are EXACTLY the 227 KB a CTA may have, so there
    // is no slack for aligning the base by hand: the kernel declares the dynamic array 1024-byte
    // aligned and refuses to run (status word) if the base is not.
    static constexpr int kStreamTiles = (D == 128) ? 5 : 8;
    static constexpr int kTmemCols = 512;
    static constexpr int kAuxBytes = 3072;                           // 1 KB barriers + 2 KB lse/delta staging
    static constexpr int kSmemBytes = (2 + kStreamTiles) * kTileBytes + kAuxBytes;
    static_assert(kSmemBytes <= 227 * 1024, "exceeds the shared memory of one CTA");
};

enum BwdBarId { BB_RES = 0, BB_STFULL = 10, BB_STEMPTY = 20, BB_SFULL = 30, BB_DPFULL = 31, BB_PFULL = 32,
                BB_DSFULL = 33, BB_FINAL = 34, BB_STAT = 35 };

#define TT_BTRACE(role, iter, slot)                                                                 \
    do {                                                                                           \
        if (p.trace != nullptr && (int)blockIdx.x == p.trace_block && (iter) < 64)                 \
            p.trace[((role) * 64 + (iter)) * 8 + (slot)] = clock64();                              \
    } while (0)

// Persistent like the forward: one CTA per SM takes (slice, resident tile) items from a global
// counter, heavy items of a slice first; the loader runs up to two items ahead and the first
// MMAs of the next item overlap the write-out of the accumulators of the current one.
// kTrace: compiled with the cycle stamps (debug aid; launched only while a trace buffer is set).
// kVarlen: packed variable-length batches (per-item sequence geometry, token-major addressing).
template <int D, bool kKeysResident, bool kTrace, bool kVarlen>
__global__ void __launch_bounds__(BwdCfg<D>::kThreads, 1)
attn_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmR0, const __grid_constant__ CUtensorMap tmR1,
                      const __grid_constant__ CUtensorMap tmT0, const __grid_constant__ CUtensorMap tmT1,
                      const BwdParams p) {
    using Cfg = BwdCfg<D>;
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
    unsigned char* sR = smem;                                 // R0, R1
    unsigned char* sT = smem + 2 * Cfg::kTileBytes;           // kStreamTiles streamed tiles: T0 ring, then T1 ring
    unsigned char* aux = smem + (2 + Cfg::kStreamTiles) * Cfg::kTileBytes;
    uint64_t* bar_res_full = reinterpret_cast<uint64_t*>(aux);   // TMA -> MMA (resident pair)
    uint64_t* bar_res_empty = bar_res_full + 1;                  // MMA (last score GEMMs of the item) -> TMA
    // The two streamed tensors have rings of their own.  T0 (Q | K) is read by the first score GEMM of
    // a tile, which is issued as soon as the PREVIOUS tile's scores are in registers, and by the last
    // accumulation GEMM of the tile: T0(t+1) must have landed when tile t has barely begun, while
    // T0(t-1) was needed until the end of tile t-1 -- three slots.  T1 (dO | V) is read by the second
    // score GEMM (end of the previous tile) and, with keys resident, by dV: two slots.  With two T0
    // slots the MMA warp waited ~1300 cycles per tile for the load (measured, both passes).
    constexpr int kN0 = (D == 128) ? 3 : (kKeysResident ? 4 : 6);
    constexpr int kN1 = Cfg::kStreamTiles - kN0;                 // D = 128: 2;  D = 64: 4 | 2
    static_assert(kN0 <= 6 && kN1 <= 4 && kN1 >= 1, "barrier arrays below are sized for these ring lengths");
    uint64_t* bar_t0_full = bar_res_empty + 1;                   // [6]
    uint64_t* bar_t0_empty = bar_t0_full + 6;                    // [6]
    uint64_t* bar_t1_full = bar_t0_empty + 6;                    // [4]
    uint64_t* bar_t1_empty = bar_t1_full + 4;                    // [4]
    uint64_t* bar_s_full = bar_t1_empty + 4;
    uint64_t* bar_dp_full = bar_s_full + 1;
    uint64_t* bar_p_full = bar_dp_full + 1;
    uint64_t* bar_ds_full = bar_p_full + 1;
    uint64_t* bar_final = bar_ds_full + 1;
    uint64_t* bar_acc_free = bar_final + 1;                      // compute (accumulators read out) -> MMA
    uint64_t* bar_sched_full = bar_acc_free + 1;                 // [2]
    uint64_t* bar_sched_empty = bar_sched_full + 2;              // [2]
    uint64_t* bar_stat = bar_sched_empty + 2;                    // [2] per warpgroup: a tile's statistics are staged
    uint64_t* bar_res_tmem = bar_stat + 2;                       // compute -> MMA: resident pair copied to tensor memory
    int* sched_item = reinterpret_cast<int*>(bar_res_tmem + 1);  // [2]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(sched_item + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    float* s_stat = reinterpret_cast<float*>(aux + 1024);     // [2 buffers][2: -lse2, -delta][128]

    const int warp = uniform_warp_idx();
    const int lane = threadIdx.x & 31;
    // With queries resident only one accumulator (dQ) is needed, which leaves 128 tensor-memory
    // columns free.  The compute threads copy the resident Q and dO tiles there at the start of an
    // item (bf16, D/2 columns each), and from the item's second tile on they are the A operands of
    // the two score GEMMs, which then read only the streamed tile from shared memory: half the
    // bytes of an MMA with both operands in shared memory, whose 8 KB per 64 cycles are all an SM
    // can deliver (measured: 2040 -> 1810 cycles per tile).  The first tile's score GEMMs still take
    // both operands from shared memory so that they can be issued under the previous item's epilogue.
    constexpr bool kResidentInTmem = !kKeysResident;
    constexpr uint32_t kColRes = 256;   // Q at [256, 256 + D/2), dO at [256 + D/2, 256 + D)

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_res_full, 1);
        // the resident pair may be reloaded when the MMA warp has issued its last reads of it and, where
        // the compute threads copy it to tensor memory, when all of them have done so (short items
        // release it in their prologue, before the compute threads have even begun the item)
        mbar_init(bar_res_empty, kResidentInTmem ? 257 : 1);
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
        mbar_init(bar_p_full, 256);
        mbar_init(bar_ds_full, 256);
        mbar_init(bar_final, 1);
        mbar_init(bar_acc_free, 256);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_stat[i], 128);
            if (i == 0) mbar_init(bar_res_tmem, 256);
            mbar_init(&bar_sched_full[i], 1);
            mbar_init(&bar_sched_empty[i], 257);   // MMA warp (1) + 256 compute threads
        }
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

    auto next_item = [&](int k) -> int {
        const int slot = k & 1;
        // a wait that gave up (this CTA has aborted) ends the sequence: the slot may hold anything
        if (!mbar_wait(&bar_sched_full[slot], (k >> 1) & 1, wctx, 80 + slot, k)) return -1;
        return sched_item[slot];
    };

    if (warp < 8) {
        // ============================================================ compute warpgroups
        setmaxnreg_inc<Cfg::kRegsCompute>();
        const int wg = warp >> 2;
        const int wq = warp & 3;
        const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_off + kColS + wg * 64;
        const uint32_t tDP = tmem_base + lane_off + kColDP + wg * 64;
        const int ctid = threadIdx.x;                          // 0..255 among compute threads
        const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2);
        uint32_t git = 0;      // streamed tiles processed so far, over all items (barrier phases)
        for (int k = 0;; ++k) {
            const int item = next_item(k);
            __syncwarp();
            mbar_arrive(&bar_sched_empty[k & 1]);
            if (item < 0) break;
            const BwdItem w = bwd_decode_item<kKeysResident, kVarlen>(item, p);
            const int bh = w.bh;
            const int rrow = w.r0 + wq * 32 + lane;            // this thread's resident row
            const int off = w.L - w.S;
            // where the statistics of query row r of query slice qs live: [slices, S] for dense tensors,
            // [H, total_q] for packed ones (qs is then the query head and the row is offset by the sequence start)
            auto stat_index = [&](int qs, int r) -> long long {
                return kVarlen ? (long long)qs * p.total_q + w.q_lo + r : (long long)qs * p.S + r;
            };
            // per-item stamps of the traced CTA: row k of warpgroup wg, slots 6 (start) and 7 (tiles)
            if (kTrace && p.trace != nullptr && (int)blockIdx.x == p.trace_block && wq == 0 && lane == 0 && k < 64) {
                p.trace[(wg * 64 + k) * 8 + 6] = clock64();
                p.trace[(wg * 64 + k) * 8 + 7] = w.n_it;
            }
            if (kResidentInTmem) {
                // warpgroup 0 copies this thread's row of Q, warpgroup 1 its row of dO, out of the
                // 128-byte-swizzled shared-memory tile (16-byte chunk j of row r sits at chunk j ^ (r & 7));
                // two consecutive bf16 values per 32-bit column, low half first, as the MMA expects.
                // The previous item's GEMMs are done with these columns: its epilogue waited for them.
                mbar_wait(bar_res_full, k & 1, wctx, BB_RES, k);
                const int r_in = wq * 32 + lane;
                const unsigned char* tile = sR + wg * Cfg::kTileBytes + r_in * 128;
                const uint32_t tdst = tmem_base + lane_off + kColRes + wg * (D / 2);
#pragma unroll
                for (int sb = 0; sb < Cfg::kSub; ++sb) {
                    uint32_t r[32];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint4 v4 = *reinterpret_cast<const uint4*>(tile + sb * Cfg::kSubBytes + ((j ^ (r_in & 7)) << 4));
                        r[4 * j + 0] = v4.x; r[4 * j + 1] = v4.y; r[4 * j + 2] = v4.z; r[4 * j + 3] = v4.w;
                    }
                    tmem_st32(tdst + sb * 32, r);
                }
                mbar_arrive(bar_res_empty);   // this thread's reads of the shared-memory tiles are done
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar_res_tmem);
            }
            // row constants (queries resident) as packed pairs of the NEGATED values
            uint64_t row_nlse2 = 0, row_ndelta2 = 0;
            if (!kKeysResident) {
                const bool ok = rrow < w.S;
                const long long si = stat_index(kVarlen ? w.head : bh, rrow);
                const float nl = ok ? -p.lse2[si] : -INFINITY;
                const float nd = ok ? -p.delta[si] : 0.f;
                row_nlse2 = pack_f32x2(nl, nl);
                row_ndelta2 = pack_f32x2(nd, nd);
            }
            // per-column statistics (keys resident): each warpgroup stages the statistics of ITS 64
            // streamed queries (columns wg*64..+63), one tile ahead of their use -- thread j of the
            // warpgroup fetches -lse2 (j < 64) or -delta (j >= 64) of query wg*64 + (j & 63) -- so the
            // hand-over needs only a barrier among the warpgroup's own 128 threads and the two
            // warpgroups are free to drift apart (they share the special-function units)
            const int stat_j = ctid & 127;
            const int stat_q = wg * 64 + (stat_j & 63);          // query inside the streamed tile
            const int stat_slot = (stat_j >> 6) * 128 + stat_q;  // [-lse2 | -delta][128]
            const float* stat_src = (stat_j < 64 ? p.lse2 : p.delta);
            const float stat_oob = (stat_j < 64) ? -INFINITY : 0.f;
            // The load of the next tile's statistic is issued a whole iteration before its value is
            // used: nothing may consume `stat_raw` (not even a negation or a select) until the store
            // at the top of the next iteration, or the warp waits out the load latency right here
            // (measured: ~1100 cycles per tile).
            float stat_raw = 0.f;
            bool stat_ok = false;
            auto stat_issue = [&](int u) {   // this thread's statistic of streamed tile u
                int tt, qs;
                bwd_stream_tile<kKeysResident, kVarlen>(w, u, p.group, tt, qs);
                const int qrow = tt * 128 + stat_q;
                stat_ok = qrow < w.S;
                if (stat_ok) stat_raw = stat_src[stat_index(qs, qrow)];
            };
            // Staging runs one tile ahead and is split-phase: the statistic of tile u+1 is written to
            // the other half of the double buffer in the MIDDLE of tile u, followed by an arrive on the
            // warpgroup's mbarrier; the matching wait at the top of tile u+1 then finds the phase long
            // complete.  (A bar.sync at the top of every tile made each warp wait for the slowest of
            // its warpgroup: ~500 cycles per tile.)  A thread's own reads of a buffer all precede its
            // next arrive, so nobody overwrites a buffer that is still being read.
            auto stat_publish = [&](uint32_t g) {
                s_stat[(g & 1) * 256 + stat_slot] = stat_ok ? -stat_raw : stat_oob;
                mbar_arrive(&bar_stat[wg]);
            };
            if (kKeysResident && w.n_it > 0) {
                stat_issue(0);
                stat_publish(git);            // first tile of the item: the one exposed load
                if (w.n_it > 1) stat_issue(1);
            }
            for (int u = 0; u < w.n_it; ++u, ++git) {
                const int it = u;
                const int t = kKeysResident ? w.t_begin + u % w.nt : w.t_begin + u;
                const bool tr = kTrace && (k == 0 && wq == 0 && lane == 0);
                const int c0 = t * 128;                            // first streamed row of this tile
                if (tr) TT_BTRACE(wg, it, 0);
                const float* st_nlse = s_stat + (git & 1) * 256;   // -lse2 of the 128 streamed queries
                const float* st_ndelta = st_nlse + 128;            // -delta
                if (kKeysResident) mbar_wait(&bar_stat[wg], git & 1, wctx, BB_STAT, it);   // tile u's statistics are staged
                // visible columns of this thread's row inside the tile: [vis_lo, vis_hi)
                int vis_lo = 0, vis_hi = 128;
                if (kKeysResident) {
                    if (p.causal) vis_lo = max(0, rrow - off - c0);           // query >= key - off
                } else {
                    vis_hi = w.Lv - c0;
                    if (p.causal) vis_hi = min(vis_hi, rrow + off + 1 - c0);  // key <= query + off
                    vis_hi = min(vis_hi, 128);
                }
                const bool need_mask = (vis_lo > 0) || (vis_hi < 128);
                // With keys resident the per-column statistics come from shared memory.  They are fetched
                // into registers BEFORE each wait on the tensor pipe (16-byte loads): inside the phases
                // they would sit behind the tensor-memory waits, and shared memory is busy feeding the
                // score GEMMs just then (measured: 850 cycles per 32-column chunk against 625 in the
                // other pass, which keeps its statistics in registers).
                uint64_t stat_reg[2][16];
                auto load_stats = [&](const float* src) {
                    if (kKeysResident) {
#pragma unroll
                        for (int cc = 0; cc < 2; ++cc)
#pragma unroll
                            for (int e4 = 0; e4 < 8; ++e4) {
                                const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(src + wg * 64 + cc * 32 + e4 * 4);
                                stat_reg[cc][2 * e4] = v.x;
                                stat_reg[cc][2 * e4 + 1] = v.y;
                            }
                    }
                };
                // ---------------- phase A: P = exp2(S*c - lse2)
                load_stats(st_nlse);
                if (tr) TT_BTRACE(wg, it, 1);
                mbar_wait(bar_s_full, git & 1, wctx, BB_SFULL, it);
                __syncwarp();
                tc_fence_after();
                if (tr) TT_BTRACE(wg, it, 2);
                uint64_t pf2[32];     // this thread's 64 probabilities, fp32 pairs
                uint32_t sr[2][32], dr[2][32];
                // Nothing is written back into the S columns: they are released as soon as they are in
                // registers, so the next tile's score GEMM runs under these exponentials.  (With keys
                // resident the bf16 P^T that dV needs joins dS^T in the dP columns in phase B.)
                // The mask test must stay OUT of the unrolled loop: a branch per pair makes every pair a
                // basic block of its own, nothing is scheduled across them and each pair then pays its
                // shared-memory, FMA and special-function latencies in full (measured: 55 cycles per pair
                // against 32 at the special-function unit's rate).
                auto phase_a_body = [&](auto masked_c, int cc) {
                    constexpr bool kMasked = decltype(masked_c)::value;
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const int col = wg * 64 + cc * 32 + e;
                        const uint64_t nl = kKeysResident ? stat_reg[cc][e >> 1] : row_nlse2;
                        const uint64_t x = fma_f32x2(pack_f32x2(__uint_as_float(sr[cc][e]), __uint_as_float(sr[cc][e + 1])), c2, nl);
                        float a0, a1;
                        unpack_f32x2(x, a0, a1);
                        float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
                        if (kMasked) {
                            p0 = (col >= vis_lo && col < vis_hi) ? p0 : 0.f;
                            p1 = (col + 1 >= vis_lo && col + 1 < vis_hi) ? p1 : 0.f;
                        }
                        pf2[cc * 16 + (e >> 1)] = pack_f32x2(p0, p1);
                    }
                };
                auto phase_a = [&](int cc) {
                    if (need_mask) phase_a_body(std::true_type{}, cc);
                    else phase_a_body(std::false_type{}, cc);
                };
                // dS = P * (dP - delta) for one chunk, written over the dP columns just read
                auto phase_b = [&](int cc) {
                    uint32_t pk[16], pkp[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const uint64_t nd = kKeysResident ? stat_reg[cc][e >> 1] : row_ndelta2;
                        const uint64_t tdiff = add_f32x2(pack_f32x2(__uint_as_float(dr[cc][e]), __uint_as_float(dr[cc][e + 1])), nd);
                        const uint64_t ds = mul_f32x2(pf2[cc * 16 + (e >> 1)], tdiff);
                        float x0, x1;
                        unpack_f32x2(ds, x0, x1);
                        pk[e >> 1] = pack_bf16x2(x0, x1);
                        if (kKeysResident) {
                            float q0, q1;
                            unpack_f32x2(pf2[cc * 16 + (e >> 1)], q0, q1);
                            pkp[e >> 1] = pack_bf16x2(q0, q1);
                        }
                    }
                    if (kKeysResident) {
                        // the 32 fp32 dP columns just read now hold 16 columns of bf16 P^T and 16 of dS^T
                        tmem_st16(tDP + cc * 32, pkp);
                        tmem_st16(tDP + cc * 32 + 16, pk);
                    } else {
                        tmem_st16(tDP + cc * 16, pk);
                    }
                };
                // (Issuing these loads further ahead of their use -- both chunks at once, or one chunk
                // ahead under the previous chunk's arithmetic -- was measured slower, twice.)
                tmem_ld32(tS, sr[0]);
                tmem_wait_ld();
                phase_a(0);
                tmem_ld32(tS + 32, sr[1]);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(bar_p_full);                // all of S(t) is in registers: its columns are free
                phase_a(1);
                if (tr) TT_BTRACE(wg, it, 3);
                load_stats(st_ndelta);
                if (kKeysResident && u + 1 < w.n_it) {
                    stat_publish(git + 1);                     // its load was issued a tile ago
                    if (u + 2 < w.n_it) stat_issue(u + 2);
                }
                mbar_wait(bar_dp_full, git & 1, wctx, BB_DPFULL, it);
                __syncwarp();
                tc_fence_after();
                if (tr) TT_BTRACE(wg, it, 4);
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    tmem_ld32(tDP + cc * 32, dr[cc]);
                    tmem_wait_ld();
                    phase_b(cc);
                }
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar_ds_full);
                if (tr) TT_BTRACE(wg, it, 5);
            }
            // ---------------- epilogue: accumulators out of tensor memory (then the MMA warp may start
            // the next item in them) -> bf16 -> global; warpgroup w owns columns [w*D/2, +D/2)
            mbar_wait(bar_final, k & 1, wctx, BB_FINAL, k);
            __syncwarp();
            tc_fence_after();
            const int n_rows = kKeysResident ? w.L : w.S;
            constexpr int kHalf = D / 2;
            constexpr int kAccs = kKeysResident ? 2 : 1;
            uint32_t acc[kAccs][kHalf / 32][32];
#pragma unroll
            for (int a = 0; a < kAccs; ++a) {
                const uint32_t tA = tmem_base + lane_off + ((kKeysResident && a == 0) ? kColAcc0 : kColAcc1) + wg * kHalf;
#pragma unroll
                for (int cc = 0; cc < kHalf / 32; ++cc) tmem_ld32(tA + cc * 32, acc[a][cc]);
            }
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(bar_acc_free);
            if (rrow < n_rows) {
#pragma unroll
                for (int a = 0; a < kAccs; ++a) {
                    const bool is_acc0 = kKeysResident && a == 0;
                    // dense: row rrow of slice bh of [slices, rows, D]; packed: token (first token + rrow), head
                    const long long o_el = kVarlen
                        ? ((long long)((kKeysResident ? w.k_lo : w.q_lo) + rrow) * (kKeysResident ? p.Hkv : p.H) + w.head) * D
                        : ((long long)bh * n_rows + rrow) * D;
                    __nv_bfloat16* dst = (is_acc0 ? p.out0 : p.out1) + o_el + wg * kHalf;
                    const float mul = is_acc0 ? 1.0f : p.scale;
                    if (kKeysResident && rrow >= w.Lv) {   // gradients of padded keys are zero
#pragma unroll
                        for (int cc = 0; cc < kHalf / 32; ++cc)
#pragma unroll
                            for (int e = 0; e < 32; ++e) acc[a][cc][e] = 0u;
                    }
#pragma unroll
                    for (int cc = 0; cc < kHalf / 32; ++cc) {
#pragma unroll
                        for (int e = 0; e < 32; e += 16) {
                            uint32_t o8[8];
#pragma unroll
                            for (int q2 = 0; q2 < 8; ++q2)
                                o8[q2] = pack_bf16x2(__uint_as_float(acc[a][cc][e + 2 * q2]) * mul,
                                                     __uint_as_float(acc[a][cc][e + 2 * q2 + 1]) * mul);
                            if (p.wide_stores) {
                                st_global_32B(dst + cc * 32 + e, o8);
                            } else {
                                *reinterpret_cast<uint4*>(dst + cc * 32 + e) = make_uint4(o8[0], o8[1], o8[2], o8[3]);
                                *reinterpret_cast<uint4*>(dst + cc * 32 + e + 8) = make_uint4(o8[4], o8[5], o8[6], o8[7]);
                            }
                        }
                    }
                }
            }
            __syncwarp();
        }
    } else {
        setmaxnreg_dec<Cfg::kRegsOther>();
        if (warp == 9) {
            // ============================================================ TMA loader + scheduler (whole
            // warp runs the control flow, one elected lane issues)
            auto load_tile = [&](unsigned char* dst, const CUtensorMap* tm, uint64_t* bar, int row_start, int bh) {
#pragma unroll
                for (int sb = 0; sb < Cfg::kSub; ++sb) tma_load_3d(dst + sb * Cfg::kSubBytes, tm, bar, sb * 64, row_start, bh);
            };
            uint32_t git = 0;
            for (int k = 0;; ++k) {
                int item = 0;
                BwdItem w;
                for (;;) {
                    if (lane == 0) item = (int)atomicAdd(p.sched_counter, 1u);
                    item = __shfl_sync(0xffffffffu, item, 0);
                    if (item >= p.n_items || *abort_flag) item = -1;   // an aborted CTA takes no further items
                    if (item < 0) break;
                    w = bwd_decode_item<kKeysResident, kVarlen>(item, p);
                    // packed batches number their items for the longest sequence: what lies past a shorter
                    // sequence's end, or sees nothing under the causal mask, is never published (the
                    // outputs were cleared before the launch)
                    if (!kVarlen || w.n_it > 0) break;
                }
                const int slot = k & 1;
                mbar_wait(&bar_sched_empty[slot], ((k >> 1) & 1) ^ 1, wctx, 90 + slot, k);
                __syncwarp();
                if (lane == 0) {
                    sched_item[slot] = item;
                    mbar_arrive(&bar_sched_full[slot]);
                }
                __syncwarp();
                if (item < 0) break;
                // TMA coordinates: (row, slice) of [slices, rows, D] for dense tensors; for packed ones the row is
                // offset by the sequence's first token and the slice is the head
                const int res_y0 = kVarlen ? (kKeysResident ? w.k_lo : w.q_lo) : 0;
                const int str_y0 = kVarlen ? (kKeysResident ? w.q_lo : w.k_lo) : 0;
                const int res_z = kVarlen ? w.head : w.bh;
                mbar_wait(bar_res_empty, (k & 1) ^ 1, wctx, BB_RES + 1, k);
                __syncwarp();
                if (elect_one()) {
                    mbar_arrive_expect_tx(bar_res_full, 2 * Cfg::kTileBytes);
                    load_tile(sR, &tmR0, bar_res_full, res_y0 + w.r0, res_z);
                    load_tile(sR + Cfg::kTileBytes, &tmR1, bar_res_full, res_y0 + w.r0, res_z);
                }
                __syncwarp();
                for (int u = 0; u < w.n_it; ++u, ++git) {
                    const int s0 = git % kN0, s1 = git % kN1;
                    int t, ts;
                    bwd_stream_tile<kKeysResident, kVarlen>(w, u, p.group, t, ts);
                    mbar_wait(&bar_t0_empty[s0], ((git / kN0) & 1) ^ 1, wctx, BB_STEMPTY + s0, (int)git);
                    __syncwarp();
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&bar_t0_full[s0], Cfg::kTileBytes);
                        load_tile(sT + s0 * Cfg::kTileBytes, &tmT0, &bar_t0_full[s0], str_y0 + t * 128, ts);
                    }
                    __syncwarp();
                    mbar_wait(&bar_t1_empty[s1], ((git / kN1) & 1) ^ 1, wctx, BB_STEMPTY + 6 + s1, (int)git);
                    __syncwarp();
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&bar_t1_full[s1], Cfg::kTileBytes);
                        load_tile(sT + (kN0 + s1) * Cfg::kTileBytes, &tmT1, &bar_t1_full[s1], str_y0 + t * 128, ts);
                    }
                    __syncwarp();
                }
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
            // G1 / G2: tmem[col] = R_which T^T for the streamed tile at index `tile` of the stream buffers
            auto issue_score = [&](int which, int tile, uint32_t col, bool a_in_tmem = false) {
                const uint64_t a0 = umma_desc_advance(dR_base, which * Cfg::kTileBytes);
                const uint64_t b0 = umma_desc_advance(dT_base, tile * Cfg::kTileBytes);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t o = (kk >> 2) * Cfg::kSubBytes + (kk & 3) * 32;
                    if (kResidentInTmem && a_in_tmem)   // A = resident tile in tensor memory: 8 columns per K step of 16
                        umma_ts(tmem_u + col, tmem_u + kColRes + which * (D / 2) + kk * 8, umma_desc_advance(b0, o), idesc_s,
                                kk > 0);
                    else
                        umma_ss(tmem_u + col, umma_desc_advance(a0, o), umma_desc_advance(b0, o), idesc_s, kk > 0);
                }
            };
            // G3 / G4: tmem[acc] (+)= bf16 A in tensor memory times the streamed tile (MN-major).  A is what
            // phase B left in the dP columns: with queries resident, each warpgroup's 64 dS values in the
            // first 32 of its 64 columns; with keys resident, per 32-column chunk 16 columns of P^T
            // (part = 0) then 16 of dS^T (part = 1).  K step kk covers 16 streamed rows = 8 columns.
            auto issue_acc = [&](int tile, int part, uint32_t acc_col, bool accumulate) {
                const uint64_t b0 = umma_desc_advance(dT_mn_base, tile * Cfg::kTileBytes);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t in_wg = kKeysResident ? (uint32_t)(((kk & 3) >> 1) * 32 + part * 16 + (kk & 1) * 8)
                                                         : (uint32_t)((kk & 3) * 8);
                    const uint32_t a = tmem_u + kColDP + (kk >> 2) * 64 + in_wg;
                    umma_ts(tmem_u + acc_col, a, umma_desc_advance(b0, kk * 2048), idesc_acc,
                            (accumulate || kk > 0) ? 1u : 0u);
                }
            };
            uint32_t git = 0;      // streamed tiles issued before the current item
            for (int k = 0;; ++k) {
                const int item = next_item(k);
                __syncwarp();
                if (elect_one()) mbar_arrive(&bar_sched_empty[k & 1]);
                __syncwarp();
                if (item < 0) break;
                const BwdItem w = bwd_decode_item<kKeysResident, kVarlen>(item, p);
                const int n_it = w.n_it;
                mbar_wait(bar_res_full, k & 1, wctx, BB_RES, k);
                __syncwarp();
                if (n_it > 0) {
                    // first scores of the item; the S / dP columns are free because the G3 / G4 of the
                    // previous item were issued earlier by this warp and execute in order
                    const int f0 = git % kN0, f1 = git % kN1;
                    mbar_wait(&bar_t0_full[f0], (git / kN0) & 1, wctx, BB_STFULL + f0, (int)git);
                    __syncwarp();
                    tc_fence_after();
                    issue_score(0, f0, kColS);
                    tc_commit(bar_s_full);
                    mbar_wait(&bar_t1_full[f1], (git / kN1) & 1, wctx, BB_STFULL + 6 + f1, (int)git);
                    __syncwarp();
                    tc_fence_after();
                    issue_score(1, kN0 + f1, kColDP);
                    tc_commit(bar_dp_full);
                    if (!kKeysResident) tc_commit(&bar_t1_empty[f1]);   // dP was the only use of this V tile
                    if (n_it == 1) tc_commit(bar_res_empty);   // those were the item's last reads of the resident pair
                }
                for (int it = 0; it < n_it; ++it) {
                    const uint32_t g = git + it;
                    const int a0s = g % kN0, a1s = g % kN1;                  // slots of this tile
                    const bool has_next = it + 1 < n_it;
                    const int n0s = (g + 1) % kN0, n1s = (g + 1) % kN1;      // slots of the next tile
                    const bool tr = kTrace && (k == 0 && lane == 0);
                    if (tr) TT_BTRACE(2, it, 0);
                    mbar_wait(bar_p_full, g & 1, wctx, BB_PFULL, it);   // S(t) is in registers: its columns are free
                    __syncwarp();
                    tc_fence_after();
                    if (tr) TT_BTRACE(2, it, 1);
                    if (kResidentInTmem && it == 0) {   // complete long ago: the copy precedes the compute threads' first tile
                        mbar_wait(bar_res_tmem, k & 1, wctx, BB_RES + 2, k);
                        __syncwarp();
                        tc_fence_after();
                    }
                    if (has_next) {
                        mbar_wait(&bar_t0_full[n0s], ((g + 1) / kN0) & 1, wctx, BB_STFULL + n0s, it + 1);
                        __syncwarp();
                        tc_fence_after();
                        issue_score(0, n0s, kColS, true);
                        tc_commit(bar_s_full);
                    }
                    if (tr) TT_BTRACE(2, it, 2);
                    mbar_wait(bar_ds_full, g & 1, wctx, BB_DSFULL, it);  // dS^T (and P^T) are in the dP columns
                    __syncwarp();
                    tc_fence_after();
                    if (tr) TT_BTRACE(2, it, 3);
                    if (it == 0) {
                        // the accumulator columns must have been read out by the previous item's epilogue
                        mbar_wait(bar_acc_free, (k & 1) ^ 1, wctx, BB_FINAL + 1, k);
                        __syncwarp();
                    }
                    if (kKeysResident) {
                        issue_acc(kN0 + a1s, 0, kColAcc0, it > 0);                       // dV += P^T dO
                        tc_commit(&bar_t1_empty[a1s]);                                   // last read of dO(t)
                    }
                    issue_acc(a0s, kKeysResident ? 1 : 0, kColAcc1, it > 0);             // dK += dS^T Q | dQ += dS K
                    tc_commit(&bar_t0_empty[a0s]);                                       // last read of Q(t) | K(t)
                    if (has_next) {
                        mbar_wait(&bar_t1_full[n1s], ((g + 1) / kN1) & 1, wctx, BB_STFULL + 6 + n1s, it + 1);
                        __syncwarp();
                        tc_fence_after();
                        issue_score(1, kN0 + n1s, kColDP, true);
                        tc_commit(bar_dp_full);
                        if (!kKeysResident) tc_commit(&bar_t1_empty[n1s]);   // dP was the only use of V(t+1)
                        if (it + 2 == n_it) tc_commit(bar_res_empty);   // last reads of the resident pair
                    }
                    if (tr) TT_BTRACE(2, it, 4);
                }
                tc_commit(bar_final);
                git += (uint32_t)n_it;
            }
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
// delta[row] = sum_d dO*O ; lse2[row] = lse[row] * log2(e).  HBM-bound: D/8 lanes share a row (16 bytes
// of O and of dO per lane), a warp covers 32/(D/8) rows per load instruction and keeps kPrepUnroll of
// them in flight before it starts to add.
constexpr int kPrepUnroll = 4;
__device__ __forceinline__ uint4 ld_nc16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
// kVarlen: packed batches -- out, dout are [total_q, H, D] (row = token * H + head), lse, delta, lse2 are
// [H, total_q]; a row that saw no key has lse = -inf: +inf in lse2 makes its recomputed probabilities
// exp2(-inf) = 0.
template <int D, bool kVarlen>
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                                            const float* __restrict__ lse, float* __restrict__ delta,
                                                            float* __restrict__ lse2, long long n_rows, long long total_q, int H) {
    constexpr int kLanesPerRow = D / 8, kRowsPerStep = 32 / kLanesPerRow;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / kLanesPerRow, li = lane % kLanesPerRow;
    const long long row0 = ((long long)blockIdx.x * (blockDim.x >> 5) + warp) * (kRowsPerStep * kPrepUnroll) + sub;
    uint4 a[kPrepUnroll], b[kPrepUnroll];
#pragma unroll
    for (int u = 0; u < kPrepUnroll; ++u) {
        const long long row = row0 + u * kRowsPerStep;
        a[u] = b[u] = make_uint4(0u, 0u, 0u, 0u);
        if (row < n_rows) {
            a[u] = ld_nc16(out + row * D + li * 8);
            b[u] = ld_nc16(dout + row * D + li * 8);
        }
    }
#pragma unroll
    for (int u = 0; u < kPrepUnroll; ++u) {
        const long long row = row0 + u * kRowsPerStep;
        const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            acc = fmaf(__uint_as_float(aw[e] << 16), __uint_as_float(bw[e] << 16), acc);
            acc = fmaf(__uint_as_float(aw[e] & 0xffff0000u), __uint_as_float(bw[e] & 0xffff0000u), acc);
        }
#pragma unroll
        for (int o = kLanesPerRow / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (li == 0 && row < n_rows) {
            if (kVarlen) {
                const long long tok = row / H;
                const long long i = (row - tok * H) * total_q + tok;
                const float l = lse[i];
                delta[i] = acc;
                lse2[i] = (l == -INFINITY) ? INFINITY : l * 1.4426950408889634f;
            } else {
                delta[row] = acc;
                lse2[row] = lse[row] * 1.4426950408889634f;
            }
        }
    }
}
template <int D, bool kVarlen>
static void launch_prep(const AttnArgs& a, float* delta, float* lse2, long long n_rows, cudaStream_t st) {
    const long long per_cta = 8LL * (32 / (D / 8)) * kPrepUnroll;
    attn_bwd_prep_kernel<D, kVarlen><<<(unsigned)((n_rows + per_cta - 1) / per_cta), 256, 0, st>>>(
        (const __nv_bfloat16*)a.out, (const __nv_bfloat16*)a.dout, a.lse, delta, lse2, n_rows, a.total_q, a.H);
}
cudaError_t attn_bwd_prep(const AttnArgs& a, float* delta, float* lse2, cudaStream_t st) {
    LaunchScope ls(K_BWD_PREP, st);
    const bool varlen = a.cu_q != nullptr;
    const long long n_rows = varlen ? a.total_q * a.H : a.BH * (long long)a.S;
    if (a.D == 128) {
        if (varlen) launch_prep<128, true>(a, delta, lse2, n_rows, st);
        else launch_prep<128, false>(a, delta, lse2, n_rows, st);
    } else {
        if (varlen) launch_prep<64, true>(a, delta, lse2, n_rows, st);
        else launch_prep<64, false>(a, delta, lse2, n_rows, st);
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------- host side
bool attn_bwd_sm100_supported(const AttnArgs& a) {
    long long tiles = ((long long)(a.S > a.L ? a.S : a.L) + 127) / 128;
    return a.bf16 && (a.D == 64 || a.D == 128) && a.BH * tiles < (1LL << 31);
}
// statistics: one float per query row of every slice, twice (delta, lse2)
static size_t stats_rows(const AttnArgs& a) { return a.cu_q ? (size_t)a.total_q * a.H : (size_t)a.BH * a.S; }
static size_t stats_bytes(const AttnArgs& a) { return 2 * align256(stats_rows(a) * sizeof(float)); }
size_t attn_bwd_sm100_workspace(const AttnArgs& a) {
    return stats_bytes(a) + ((attn_bwd_fused_supported(a) && !a.cu_q) ? attn_bwd_fused_workspace(a) : 0);
}

static long long* g_bwd_trace = nullptr;
static int g_bwd_trace_block = 0, g_bwd_trace_mode = 0;   // mode 1: dK/dV pass, 2: dQ pass
void attn_bwd_set_trace(long long* device_buf, int block, int pass) {
    g_bwd_trace = device_buf;
    g_bwd_trace_block = block;
    g_bwd_trace_mode = device_buf ? pass : 0;
}

template <int D, bool kTrace, bool kVarlen = false>
static cudaError_t launch_bwd(const AttnArgs& a, void* ws, cudaStream_t st) {
    using Cfg = BwdCfg<D>;
    float* delta = reinterpret_cast<float*>(ws);
    float* lse2 = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(ws) + align256(stats_rows(a) * sizeof(float)));
    cudaError_t e = attn_bwd_prep(a, delta, lse2, st);
    if (e != cudaSuccess) return e;
    TmapStorage tq, tk, tv, tdo;
    const char* why = nullptr;
    const int hkv = a.H / a.group;
    if (kVarlen) {
        // work items are numbered for the longest sequence and skipped where a sequence is shorter or sees
        // nothing: whatever no item writes must read as zero
        const size_t es = sizeof(__nv_bfloat16);
        if ((e = cudaMemsetAsync(a.dq, 0, (size_t)a.total_q * a.H * D * es, st)) != cudaSuccess) return e;
        if ((e = cudaMemsetAsync(a.dk, 0, (size_t)a.total_k * hkv * D * es, st)) != cudaSuccess) return e;
        if ((e = cudaMemsetAsync(a.dv, 0, (size_t)a.total_k * hkv * D * es, st)) != cudaSuccess) return e;
        if (!make_tmap_bf16_strided(&tq, a.q, D, a.total_q, a.H, (uint64_t)a.H * D, D, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16_strided(&tdo, a.dout, D, a.total_q, a.H, (uint64_t)a.H * D, D, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16_strided(&tk, a.k, D, a.total_k, hkv, (uint64_t)hkv * D, D, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16_strided(&tv, a.v, D, a.total_k, hkv, (uint64_t)hkv * D, D, 128, &why)) return cudaErrorInvalidValue;
    } else {
        if (!make_tmap_bf16(&tq, a.q, D, a.S, a.BH, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16(&tk, a.k, D, a.L, a.BH / a.group, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16(&tv, a.v, D, a.L, a.BH / a.group, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16(&tdo, a.dout, D, a.S, a.BH, 128, &why)) return cudaErrorInvalidValue;
    }
    auto M = [](TmapStorage& t) -> CUtensorMap& { return *reinterpret_cast<CUtensorMap*>(t.bytes); };
    e = cudaFuncSetAttribute(attn_bwd_sm100_kernel<D, true, kTrace, kVarlen>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(attn_bwd_sm100_kernel<D, false, kTrace, kVarlen>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
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
    p.trace = g_bwd_trace_mode == 1 ? g_bwd_trace : nullptr;
    p.trace_block = g_bwd_trace_block;
    // dK, dV: keys resident, stream (Q, dO)
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    p.out0 = (__nv_bfloat16*)a.dv;
    p.out1 = (__nv_bfloat16*)a.dk;
    p.group = a.group;
    p.kv_lens = a.kv_lens;
    p.H = a.H;
    p.Hkv = hkv;
    p.cu_q = a.cu_q;
    p.cu_k = a.cu_k;
    p.total_q = (int)a.total_q;
    const uintptr_t al = reinterpret_cast<uintptr_t>(a.dq) | reinterpret_cast<uintptr_t>(a.dk) | reinterpret_cast<uintptr_t>(a.dv);
    p.wide_stores = (al & 31) == 0 ? 1 : 0;
    p.n_tiles = (a.L + 127) / 128;
    p.n_items = (int)(a.BH / a.group * p.n_tiles);
    p.n_light = a.causal ? p.n_tiles / 4 : 0;
    p.n_items_heavy = (int)(a.BH / a.group * (p.n_tiles - p.n_light));
    SchedCounter sc;
    if (D == 128 && !kTrace && !kVarlen && attn_bwd_dkv_pair_supported(a)) {
        // same pass on CTA pairs: each MMA reads half of its streamed operand per SM
        if ((e = attn_bwd_dkv_pair(a, delta, lse2, st)) != cudaSuccess) return e;
    } else {
        e = sched_counter_acquire(st, &sc);
        if (e != cudaSuccess) return e;
        p.sched_counter = sc.ptr;
        {
            LaunchScope ls(K_BWD_DKV, st);
            attn_bwd_sm100_kernel<D, true, kTrace, kVarlen><<<(unsigned)std::min(p.n_items, n_sm), Cfg::kThreads, Cfg::kSmemBytes, st>>>(
                M(tk), M(tv), M(tq), M(tdo), p);
        }
        sched_counter_release(sc, st);
    }
    // dQ: queries resident, stream (K, V)
    p.trace = g_bwd_trace_mode == 2 ? g_bwd_trace : nullptr;
    p.out0 = nullptr;
    p.out1 = (__nv_bfloat16*)a.dq;
    p.n_tiles = (a.S + 127) / 128;
    p.n_items = (int)(a.BH * p.n_tiles);
    p.n_light = a.causal ? p.n_tiles / 4 : 0;
    p.n_items_heavy = (int)(a.BH * (p.n_tiles - p.n_light));
    e = sched_counter_acquire(st, &sc);
    if (e != cudaSuccess) return e;
    p.sched_counter = sc.ptr;
    {
        LaunchScope ls(K_BWD_DQ, st);
        attn_bwd_sm100_kernel<D, false, kTrace, kVarlen><<<(unsigned)std::min(p.n_items, n_sm), Cfg::kThreads, Cfg::kSmemBytes, st>>>(
            M(tq), M(tdo), M(tk), M(tv), p);
    }
    sched_counter_release(sc, st);
    return cudaGetLastError();
}

template <int D>
static cudaError_t launch_bwd_d(const AttnArgs& a, void* ws, cudaStream_t st) {
    if (a.cu_q != nullptr) return launch_bwd<D, false, true>(a, ws, st);
    if (g_bwd_trace_mode != 0) return launch_bwd<D, true>(a, ws, st);
    return launch_bwd<D, false>(a, ws, st);
}
cudaError_t attn_bwd_two_pass(const AttnArgs& a, void* ws, cudaStream_t st) {
    return a.D == 128 ? launch_bwd_d<128>(a, ws, st) : launch_bwd_d<64>(a, ws, st);
}

}  // namespace ttk

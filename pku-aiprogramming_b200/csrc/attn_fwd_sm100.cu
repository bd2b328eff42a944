// Flash-style fused attention forward for B200 (sm_100a), bf16 in / bf16 out, fp32
// softmax and accumulation.  Head dim 64 or 128.
//
// One CTA owns 256 consecutive query rows of one (batch, head) slice as two 128-row
// tiles and walks over the keys in tiles of 128.
//
//   warps 0-3   softmax warpgroup of query tile 0   (thread <-> one query row)
//   warps 4-7   softmax warpgroup of query tile 1
//   warp  8     MMA issuer (one elected lane issues every tcgen05.mma)
//   warp  9     TMA loader (one elected lane issues every cp.async.bulk.tensor)
//   warps 10-11 idle (they only complete the third warpgroup for setmaxnreg)
//
// Tensor memory (512 columns x 128 lanes x 32 bit):
//   S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [256+D,256+2D)
//   P_i (bf16, packed two per column) overlays columns [0,64) of S_i.
//
// Per key tile j and query tile i:  S_i = Q_i K_j^T (A,B from shared memory, K-major) ->
// softmax warpgroup reads S_i row-per-thread, keeps the running max/sum, rescales O_i in
// tensor memory only when the max grew by more than 2^8, writes P_i as bf16 into tensor
// memory -> O_i += P_i V_j (A from tensor memory, B = V_j from shared memory, MN-major).
// The issuer alternates the two query tiles so the tensor pipe works on one tile while
// the other tile's softmax runs.
//
// Shared memory: Q tiles (2) + a ring of K/V tiles, each tile stored by TMA as D/64
// sub-blocks of [128 rows x 128 bytes] with the 128-byte swizzle.
#include "attn_fwd_common.cuh"
#include <algorithm>

namespace ttk {
using namespace sm100;

#ifndef TT_FWD_REGS_SOFTMAX
#define TT_FWD_REGS_SOFTMAX 216
#define TT_FWD_REGS_OTHER 72
#endif

template <int D>
struct FwdCfg {
    static constexpr int kTile = 128;                     // rows per Q tile and keys per K/V tile
    static constexpr int kSub = D / 64;                   // 64-column sub-blocks per tile
    static constexpr int kSubBytes = kTile * 128;         // 16 KiB
    static constexpr int kTileBytes = kSub * kSubBytes;   // 32 KiB (D=128), 16 KiB (D=64)
    static constexpr int kStages = (D == 128) ? 4 : 8;    // K/V ring depth (tiles)
    static constexpr int kThreads = 384;
    // Register split after setmaxnreg: the two softmax warpgroups grow to kRegsSoftmax, the third
    // warpgroup (loader, MMA issuer, two idle warps) shrinks to kRegsOther.  The pool a CTA can draw
    // from is what the launch allocated (kRegsLaunch per thread, the __launch_bounds__ figure rounded
    // down to a multiple of 8); a split that asks for more than the pool never completes.
    static constexpr int kRegsLaunch = 168;
    static constexpr int kRegsSoftmax = TT_FWD_REGS_SOFTMAX;
    static constexpr int kRegsOther = TT_FWD_REGS_OTHER;
    static_assert(256 * kRegsSoftmax + 128 * kRegsOther <= kThreads * kRegsLaunch, "register split exceeds the CTA's pool");
    static_assert(kRegsSoftmax % 8 == 0 && kRegsOther % 8 == 0, "setmaxnreg takes multiples of 8");
    static constexpr int kTmemCols = 512;
    static constexpr int kBarBytes = 1024;
    static constexpr int kSmemBytes = (2 + kStages) * kTileBytes + kBarBytes + 1024;  // +1024: alignment slack
};

enum FwdBarId { BAR_QFULL = 0, BAR_KVFULL = 10, BAR_KVEMPTY = 30, BAR_SFULL = 50, BAR_PFULL = 60, BAR_OFINAL = 70 };

#define TT_TRACE(role, iter, slot)                                                                  \
    do {                                                                                           \
        if (p.trace != nullptr && (int)blockIdx.x == p.trace_block && (iter) < 64)                 \
            p.trace[((role) * 64 + (iter)) * 8 + (slot)] = clock64();                              \
    } while (0)

// The kernel is persistent: one CTA per SM takes work items (slice, 256-row query block) from a
// global counter until none are left.  Items are numbered slice-major with the heavy (late)
// query blocks of a slice first, so that concurrently running CTAs share a slice's K/V in L2.
// Causal launches keep the lightest quarter of every slice's blocks for a second pass over the
// slices, so that the tail of the launch consists of light items.  The loader runs up to two items ahead; the
// first MMAs of item n+1 overlap the epilogue (normalise, store O) of item n.
struct FwdItem {
    int bh, q0, n_tiles[2], n_max;
    int Lv;   // keys that count for this slice (<= L; fewer with key padding)
    int kvs, key0;   // kPaged: key/value slice and first key of this item
    // geometry of the item's slice: queries and causal offset (L - S), which are the launch's own for dense
    // tensors and the sequence's for packed ones; TMA coordinates (first row, slice index) of its Q and K/V
    // rows; where its output rows and log-sum-exps go
    int S, off;
    int qy0, qz, ky0, kz;
    long long out_row0;   // output row r of the slice is row out_row0 + r of a [rows, out_pitch] matrix, at column out_col
    int out_pitch, out_col;
    long long lse0;       // lse[lse0 + r]
};
template <bool kPaged = false, bool kVarlen = false>
__device__ __forceinline__ FwdItem fwd_decode_item(int item, const FwdParams& p, int D) {
    FwdItem w;
    int qb;
    if (item < p.n_items_heavy) {
        const int n_heavy = p.n_qblk - p.n_light;
        w.bh = item / n_heavy;
        qb = p.n_qblk - 1 - (item - w.bh * n_heavy);
    } else {   // second phase: the light (early) query blocks, again slice-major and heavy first
        const int r = item - p.n_items_heavy;
        w.bh = r / p.n_light;
        qb = p.n_light - 1 - (r - w.bh * p.n_light);
    }
    w.q0 = qb * 256;
    int S = p.S, L = p.L;
    if (kVarlen) {
        const int b = w.bh / p.H, h = w.bh - b * p.H;
        const int q_lo = p.cu_q[b], k_lo = p.cu_k[b];
        S = p.cu_q[b + 1] - q_lo;
        L = p.cu_k[b + 1] - k_lo;
        w.qy0 = q_lo; w.qz = h; w.ky0 = k_lo; w.kz = h / p.group;
        w.out_row0 = q_lo; w.out_pitch = p.H * D; w.out_col = h * D;
        w.lse0 = (long long)h * p.total_q + q_lo;
    } else {
        w.qy0 = 0; w.qz = w.bh / p.q_div; w.ky0 = 0; w.kz = w.bh / p.group;
        w.out_row0 = (long long)w.bh * p.S; w.out_pitch = D; w.out_col = 0;
        w.lse0 = (long long)w.bh * p.S;
    }
    w.S = S;
    const int off = L - S;
    w.off = off;
    if (kPaged) {   // a paged cache may hold empty sequences, and an item may cover one key range of its slice
        w.kvs = w.bh / p.q_div;
        w.key0 = (w.bh - w.kvs * p.q_div) * p.kv_chunk;
        const int len = p.kv_lens ? min(p.L, max(0, p.kv_lens[w.kvs / p.H])) : p.L;
        w.Lv = p.kv_chunk > 0 ? max(0, min(len - w.key0, p.kv_chunk)) : len;
    } else if (kVarlen) {
        w.Lv = L;
    } else {
        w.Lv = valid_keys(p.kv_lens, w.bh / p.H, p.L);
    }
    const int n_kv_total = (w.Lv + 127) >> 7;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r0 = w.q0 + 128 * i;
        if (r0 >= S) {
            w.n_tiles[i] = 0;
        } else if (p.causal) {
            const int last_row = min(r0 + 127, S - 1);
            w.n_tiles[i] = max(0, min(n_kv_total, ((last_row + off) >> 7) + 1));   // off < 0: early rows may see no key
        } else {
            w.n_tiles[i] = n_kv_total;
        }
    }
    w.n_max = max(w.n_tiles[0], w.n_tiles[1]);
    return w;
}

// kTrace: compiled with the cycle stamps (debug aid; costs registers in every role, so the
// product launches the kTrace = false instantiation unless a trace buffer is set).
// kPaged: decode over a ragged and/or paged cache run as a [batch x key/value heads, group, D]
// forward problem: sequences may be empty, an item may cover one key range of its slice, rows
// behind a sequence's end are zeroed in V, and with a block table the K and V tiles are gathered
// page by page.
// kVarlen: packed variable-length batches (see FwdParams): per-item sequence geometry, token-major addressing.
template <int D, bool kTrace, bool kPaged, bool kVarlen>
__global__ void __launch_bounds__(FwdCfg<D>::kThreads, 1)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
    using Cfg = FwdCfg<D>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle pattern shared by TMA and UMMA.
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem;                                  // 2 tiles
    unsigned char* sKV = smem + 2 * Cfg::kTileBytes;           // kStages tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + kStages) * Cfg::kTileBytes);
    uint64_t* bar_q_full = bars;                     // [2]  TMA -> MMA
    uint64_t* bar_q_empty = bar_q_full + 2;          // [2]  MMA (last S of the item) -> TMA
    uint64_t* bar_kv_full = bar_q_empty + 2;         // [kStages]
    uint64_t* bar_kv_empty = bar_kv_full + kStages;  // [kStages]
    uint64_t* bar_s_full = bar_kv_empty + kStages;   // [2]  MMA -> softmax
    uint64_t* bar_p_full = bar_s_full + 2;           // [2 tiles][2 halves of the key tile] softmax -> MMA
    uint64_t* bar_o_final = bar_p_full + 4;          // [2]  MMA -> softmax (epilogue)
    uint64_t* bar_o_free = bar_o_final + 2;          // [2]  softmax (O read out) -> MMA
    uint64_t* bar_sched_full = bar_o_free + 2;       // [2]  loader -> MMA + softmax
    uint64_t* bar_sched_empty = bar_sched_full + 2;  // [2]
    int* sched_item = reinterpret_cast<int*>(bar_sched_empty + 2);   // [2]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(sched_item + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = uniform_warp_idx();
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_q_full[i], 1);
            mbar_init(&bar_q_empty[i], 1);
            mbar_init(&bar_s_full[i], 1);
            mbar_init(&bar_p_full[2 * i], 128);
            mbar_init(&bar_p_full[2 * i + 1], 128);
            mbar_init(&bar_o_final[i], 1);
            mbar_init(&bar_o_free[i], 128);
            mbar_init(&bar_sched_full[i], 1);
            mbar_init(&bar_sched_empty[i], 257);   // MMA warp (1) + 256 softmax threads
        }
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bar_kv_full[s], 1);
            mbar_init(&bar_kv_empty[s], 1);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 8) {
        tmem_alloc(tmem_base_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    if (warp == 9 && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    WaitCtx wctx{p.status, abort_flag, warp};

    // Every role walks the same item sequence.  Items are published by the loader in a two-slot
    // ring; a negative value ends the sequence.
    auto next_item = [&](int k) -> int {
        const int slot = k & 1;
        // a wait that gave up (this CTA has aborted) ends the sequence: the slot may hold anything
        if (!mbar_wait(&bar_sched_full[slot], (k >> 1) & 1, wctx, 80 + slot, k)) return -1;
        return sched_item[slot];
    };

    if (warp < 8) {
        // =========================================================== softmax warpgroups
        setmaxnreg_inc<Cfg::kRegsSoftmax>();
        const int i = warp >> 2;                    // query tile
        const int wq = warp & 3;                    // TMEM lane quarter of this warp
        const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_off + (uint32_t)(i * 128);
        const uint32_t tP = tS;
        const uint32_t tO = tmem_base + lane_off + (uint32_t)(256 + i * D);
        const float c = p.scale_log2;
        uint32_t s_cnt = 0;    // S tiles of this query-tile slot consumed so far (barrier phase)
        uint32_t o_cnt = 0;    // items in which this slot was active
        for (int k = 0;; ++k) {
            const int item = next_item(k);
            __syncwarp();
            mbar_arrive(&bar_sched_empty[k & 1]);
            if (item < 0) break;
            const FwdItem w = fwd_decode_item<kPaged, kVarlen>(item, p, D);
            const int nt = w.n_tiles[i];
            // per-item stamps of the traced CTA (role slot 0/1 = query tile, row = item number k)
            if (kTrace && p.trace != nullptr && (int)blockIdx.x == p.trace_block && wq == 0 && (threadIdx.x & 31) == 0 && k < 64) {
                p.trace[(i * 64 + k) * 8 + 6] = clock64();
                p.trace[(i * 64 + k) * 8 + 7] = nt;
            }
            const int row = w.q0 + 128 * i + wq * 32 + lane;
            const int off = w.off;
            if ((kPaged || kVarlen) && nt == 0 && row < w.S) {   // no key at all for this tile's rows: zero output, log-sum-exp -inf
                uint4* orow = reinterpret_cast<uint4*>(p.out + (w.out_row0 + row) * w.out_pitch + w.out_col);
#pragma unroll
                for (int e = 0; e < D / 8; ++e) orow[e] = make_uint4(0u, 0u, 0u, 0u);
                if (p.lse != nullptr) p.lse[w.lse0 + row] = -INFINITY;
            }
            if (nt == 0) continue;
            float m2 = -INFINITY;   // running max in the scaled log2 domain
            float l = 0.f;          // running sum of exp2(s*c - m2)
            for (int j = 0; j < nt; ++j, ++s_cnt) {
                const bool tr = kTrace && (k == p.trace_item && wq == 0 && lane == 0);
                if (tr) TT_TRACE(i, j, 0);
                mbar_wait(&bar_s_full[i], s_cnt & 1, wctx, BAR_SFULL + i, j);
                __syncwarp();
                tc_fence_after();
                if (tr) TT_TRACE(i, j, 1);
                // visible columns of this row inside the tile: [0, lim)
                const int kv0 = j << 7;
                const bool need_mask = (kv0 + 128 > w.Lv) || (p.causal && (kv0 + 127 > (w.q0 + 128 * i) + off));
                int lim = 128;
                if (need_mask) {
                    lim = w.Lv;
                    if (p.causal) lim = min(lim, row + off + 1);
                    lim -= kv0;
                }
                uint32_t sr[4][32];
                load_s_row(tS, sr, need_mask, lim);
                if (tr) TT_TRACE(i, j, 2);
                const float mx = row_max_raw(sr) * c;
                float resc = 1.0f;
                bool grow = false;
                if (j == 0) {
                    m2 = mx;
                } else if (mx > m2 + 8.0f) {   // lazy rescale: only when the max grew by more than 2^8
                    resc = ex2_approx(m2 - mx);
                    m2 = mx;
                    l *= resc;
                    grow = true;
                }
                if (__any_sync(0xffffffffu, grow)) {
                    // O_i *= resc (the previous P V of this tile has completed: its commit precedes the
                    // S commit waited on above)
#pragma unroll
                    for (int cc = 0; cc < D / 32; ++cc) {
                        uint32_t orr[32];
                        tmem_ld32(tO + cc * 32, orr);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) orr[e] = __float_as_uint(__uint_as_float(orr[e]) * resc);
                        tmem_st32(tO + cc * 32, orr);
                    }
                }
                if (tr) TT_TRACE(i, j, 3);
                // P = exp2(S*c - m2) in two halves of 64 keys; the P V MMAs of a half start as soon as
                // that half is in tensor memory
                uint64_t acc = pack_f32x2(0.f, 0.f);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t pk[32];
                    // (packed batches: a row that has met no visible key yet has m2 = -inf; subtracting 0 instead keeps
                    // its probabilities at exp2(-inf) = 0 rather than NaN)
                    acc = add_f32x2(acc, softmax_exp_half(sr, h, c, (kVarlen && m2 == -INFINITY) ? 0.f : m2, pk));
#pragma unroll
                    for (int q4 = 0; q4 < 2; ++q4) {
                        uint32_t t16[16];
#pragma unroll
                        for (int e = 0; e < 16; ++e) t16[e] = pk[q4 * 16 + e];
                        tmem_st16(tP + h * 32 + q4 * 16, t16);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(&bar_p_full[2 * i + h]);
                    if (tr) TT_TRACE(i, j, 4 + h);
                }
                {
                    float t0, t1;
                    unpack_f32x2(acc, t0, t1);
                    l += t0 + t1;
                }
            }
            // ---- epilogue: O_i out of tensor memory (then the MMA warp may start the next item's
            // accumulation in it), O_i / l -> bf16 -> global, LSE
            mbar_wait(&bar_o_final[i], o_cnt & 1, wctx, BAR_OFINAL + i, k);
            ++o_cnt;
            __syncwarp();
            tc_fence_after();
            uint32_t orr[D / 32][32];
#pragma unroll
            for (int cc = 0; cc < D / 32; ++cc) tmem_ld32(tO + cc * 32, orr[cc]);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&bar_o_free[i]);
            // (a packed sequence with fewer keys than queries under the causal mask has rows that see no key:
            // their l is 0 and they get a zero output and log-sum-exp -inf)
            const float inv = (kVarlen && !(l > 0.f)) ? 0.f : 1.0f / l;
            if (row < w.S) {
                __nv_bfloat16* orow = p.out + (w.out_row0 + row) * w.out_pitch + w.out_col;
#pragma unroll
                for (int cc = 0; cc < D / 32; ++cc) {
#pragma unroll
                    for (int e = 0; e < 32; e += 16) {
                        uint32_t o8[8];
#pragma unroll
                        for (int q2 = 0; q2 < 8; ++q2)
                            o8[q2] = pack_bf16x2(__uint_as_float(orr[cc][e + 2 * q2]) * inv, __uint_as_float(orr[cc][e + 2 * q2 + 1]) * inv);
                        if (p.wide_stores) {
                            st_global_32B(orow + cc * 32 + e, o8);
                        } else {
                            *reinterpret_cast<uint4*>(orow + cc * 32 + e) = make_uint4(o8[0], o8[1], o8[2], o8[3]);
                            *reinterpret_cast<uint4*>(orow + cc * 32 + e + 8) = make_uint4(o8[4], o8[5], o8[6], o8[7]);
                        }
                    }
                }
                if (p.lse != nullptr) p.lse[w.lse0 + row] = (kVarlen && !(l > 0.f)) ? -INFINITY : (m2 + log2f(l)) * 0.6931471805599453f;
            }
            __syncwarp();
        }
    } else {
        setmaxnreg_dec<Cfg::kRegsOther>();
        if (warp == 9) {
            // ======================================================= TMA loader + scheduler (whole warp
            // runs the control flow, one elected lane issues)
            auto load_tile = [&](unsigned char* dst, const CUtensorMap* tm, uint64_t* bar, int row_start, int bh) {
                if (elect_one()) {
                    mbar_arrive_expect_tx(bar, Cfg::kTileBytes);
#pragma unroll
                    for (int sb = 0; sb < Cfg::kSub; ++sb)
                        tma_load_3d(dst + sb * Cfg::kSubBytes, tm, bar, sb * 64, row_start, bh);
                }
                __syncwarp();
            };
            uint32_t t = 0;                    // K/V ring item counter (runs across work items)
            uint32_t q_uses[2] = {0, 0};       // how often each Q buffer has been filled
            for (int k = 0;; ++k) {
                int item = 0;
                if (lane == 0) item = (int)atomicAdd(p.sched_counter, 1u);
                item = __shfl_sync(0xffffffffu, item, 0);
                if (item >= p.n_items || *abort_flag) item = -1;   // an aborted CTA takes no further items
                const int slot = k & 1;
                mbar_wait(&bar_sched_empty[slot], ((k >> 1) & 1) ^ 1, wctx, 90 + slot, k);
                __syncwarp();
                if (lane == 0) {
                    sched_item[slot] = item;
                    mbar_arrive(&bar_sched_full[slot]);
                }
                __syncwarp();
                if (item < 0) break;
                const FwdItem w = fwd_decode_item<kPaged, kVarlen>(item, p, D);
                auto load_q = [&](int i) {
                    mbar_wait(&bar_q_empty[i], (q_uses[i] & 1) ^ 1, wctx, 5 + i, k);
                    __syncwarp();
                    load_tile(sQ + i * Cfg::kTileBytes, &tmQ, &bar_q_full[i], w.qy0 + w.q0 + 128 * i, w.qz);
                    ++q_uses[i];
                };
                auto load_kv = [&](const CUtensorMap* tm, int j) {   // ring order: K_0, V_0, K_1, V_1, ...
                    const int st = t % kStages;
                    mbar_wait(&bar_kv_empty[st], ((t / kStages) & 1) ^ 1, wctx, BAR_KVEMPTY + st, (int)t);
                    __syncwarp();
                    if (kPaged && p.block_table != nullptr) {
                        // One TMA box per page (or one 128-row box out of a larger page); lanes issue
                        // side by side.  Only pages that hold counted keys are fetched: the rows after
                        // them are masked in S and zeroed in V by the MMA warp.
                        unsigned char* dst = sKV + st * Cfg::kTileBytes;
                        const int box_rows = min(p.page_size, 128);
                        const int key0 = j * 128;
                        const int n_box = min(128 / box_rows, (w.Lv - key0 + box_rows - 1) / box_rows);
                        if (lane == 0) mbar_arrive_expect_tx(&bar_kv_full[st], (uint32_t)(n_box * box_rows * D * 2));
                        __syncwarp();
                        if (lane < n_box) {
                            const int key = w.key0 + key0 + lane * box_rows;
                            const int lp = key / p.page_size;
                            const int page = __ldg(p.block_table + (long long)(w.kvs / p.H) * p.max_pages + lp);
                            const int z = page * p.H + (w.kvs % p.H);
#pragma unroll
                            for (int sb = 0; sb < Cfg::kSub; ++sb)
                                tma_load_3d(dst + sb * Cfg::kSubBytes + lane * box_rows * 128, tm, &bar_kv_full[st], sb * 64,
                                            key - lp * p.page_size, z);
                        }
                        __syncwarp();
                    } else if (kPaged) {   // dense ragged cache: this item's key range of its slice
                        load_tile(sKV + st * Cfg::kTileBytes, tm, &bar_kv_full[st], w.key0 + j * 128, w.kvs);
                    } else {
                        load_tile(sKV + st * Cfg::kTileBytes, tm, &bar_kv_full[st], w.ky0 + j * 128, w.kz);
                    }
                    ++t;
                };
                if (w.n_tiles[0] > 0) load_q(0);
                if (w.n_max > 0) load_kv(&tmK, 0);
                if (w.n_tiles[1] > 0) load_q(1);
                for (int j = 0; j < w.n_max; ++j) {
                    load_kv(&tmV, j);
                    if (j + 1 < w.n_max) load_kv(&tmK, j + 1);
                }
            }
        } else if (warp == 8) {
            // ======================================================= MMA issuer (whole warp runs the
            // control flow; each tcgen05.mma / commit is issued by one elected lane)
            constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);
            constexpr uint32_t idesc_pv = umma_idesc_bf16(128, D, false, true);
            const uint32_t sQ_addr = __shfl_sync(0xffffffffu, smem_u32(sQ), 0);
            const uint32_t sKV_addr = __shfl_sync(0xffffffffu, smem_u32(sKV), 0);
            const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);   // warp-uniform copy
            // descriptor templates; per MMA only the 14-bit start-address field moves
            const uint64_t dq_base = umma_smem_desc(sQ_addr, 16, 1024);
            const uint64_t dk_base = umma_smem_desc(sKV_addr, 16, 1024);                 // K-major (S = Q K^T)
            const uint64_t dv_base = umma_smem_desc(sKV_addr, Cfg::kSubBytes, 1024);     // MN-major (O += P V)
            uint32_t t = 0;                  // K/V ring items consumed before the current work item
            uint32_t q_uses[2] = {0, 0}, p_cnt[2] = {0, 0}, o_uses[2] = {0, 0};
            auto wait_item = [&](uint32_t ri) {
                const int st = ri % kStages;
                mbar_wait(&bar_kv_full[st], (ri / kStages) & 1, wctx, BAR_KVFULL + st, (int)ri);
                __syncwarp();
            };
            auto release_item = [&](uint32_t ri) { tc_commit(&bar_kv_empty[ri % kStages]); };
            auto issue_s = [&](int i, uint32_t ri) {   // S_i = Q_i K^T with K in ring item ri
                const uint64_t a0 = umma_desc_advance(dq_base, i * Cfg::kTileBytes);
                const uint64_t b0 = umma_desc_advance(dk_base, (ri % kStages) * Cfg::kTileBytes);
                const uint32_t d = tmem_u + (uint32_t)(i * 128);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t o = (kk >> 2) * Cfg::kSubBytes + (kk & 3) * 32;
                    umma_ss(d, umma_desc_advance(a0, o), umma_desc_advance(b0, o), idesc_s, kk > 0);
                }
            };
            auto issue_pv = [&](int i, uint32_t ri, bool accumulate, int half) {   // O_i (+)= P_i V
                const uint64_t b0 = umma_desc_advance(dv_base, (ri % kStages) * Cfg::kTileBytes);
                const uint32_t d = tmem_u + (uint32_t)(256 + i * D);
                const uint32_t a = tmem_u + (uint32_t)(i * 128);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                    const int kk = half * 4 + k4;
                    umma_ts(d, a + kk * 8, umma_desc_advance(b0, kk * 2048), idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
                }
            };
            // Causal items give query tile 1 one key/value tile more than tile 0, so in an item's last
            // iteration slot 0 has nothing to do.  That gap is used: the item that follows is fetched
            // early and its S_0(0) issued right there (`s0_ahead`), so that softmax warpgroup 0 finds
            // its first scores waiting instead of sitting out tile 1's last iteration plus a GEMM.
            int ahead_item = -2;       // next work item when fetched early (-2: not fetched)
            bool s0_ahead = false;     // S_0(0) of the current item was issued during the previous item
            for (int k = 0;; ++k) {
                const int item = (ahead_item != -2) ? ahead_item : next_item(k);
                ahead_item = -2;
                __syncwarp();
                if (elect_one()) mbar_arrive(&bar_sched_empty[k & 1]);
                __syncwarp();
                if (item < 0) break;
                const FwdItem w = fwd_decode_item<kPaged, kVarlen>(item, p, D);
                // S_i(0) for both tiles.  The S/P columns are free: the P V MMAs of the previous item
                // were issued earlier by this warp and execute in order.
                if (w.n_max > 0) {
                    wait_item(t);   // K_0
                    tc_fence_after();
                    for (int i = 0; i < 2; ++i) {
                        if (i == 0 && s0_ahead) {   // done already, including the bookkeeping of Q_0
                            s0_ahead = false;
                            continue;
                        }
                        if (w.n_tiles[i] > 0) {
                            mbar_wait(&bar_q_full[i], q_uses[i] & 1, wctx, BAR_QFULL + i, k);
                            ++q_uses[i];
                            __syncwarp();
                            tc_fence_after();
                            issue_s(i, t);
                            tc_commit(&bar_s_full[i]);
                            if (w.n_tiles[i] == 1) tc_commit(&bar_q_empty[i]);   // that was this tile's last S
                        }
                    }
                    release_item(t);
                }
                for (int j = 0; j < w.n_max; ++j) {
                    const uint32_t item_v = t + 2 * j + 1, item_k = t + 2 * j + 2;
                    wait_item(item_v);
                    if constexpr (kPaged) {
                        // Rows of the last V tile past the sequence's end hold whatever the pool (or the
                        // ring slot) held; their P is exactly 0, but 0 x NaN is not, so they are zeroed.
                        const int rv = w.Lv - j * 128;
                        if (rv < 128) {
                            unsigned char* vt = sKV + (item_v % kStages) * Cfg::kTileBytes;
#pragma unroll
                            for (int sb = 0; sb < Cfg::kSub; ++sb)
                                for (int o = rv * 128 + lane * 16; o < 128 * 128; o += 32 * 16)
                                    *reinterpret_cast<uint4*>(vt + sb * Cfg::kSubBytes + o) = make_uint4(0u, 0u, 0u, 0u);
                            fence_proxy_async_smem();
                            __syncwarp();
                        }
                    }
                    bool k_waited = false;
                    for (int i = 0; i < 2; ++i) {
                        if (j < w.n_tiles[i]) {
                            if (j == 0) {
                                // the accumulator columns must have been read out by the previous item's epilogue
                                mbar_wait(&bar_o_free[i], (o_uses[i] & 1) ^ 1, wctx, 75 + i, k);
                                ++o_uses[i];
                                __syncwarp();
                            }
                            const bool tr = kTrace && (k == p.trace_item && lane == 0);
                            if (tr) TT_TRACE(2, j, 4 * i + 0);
                            mbar_wait(&bar_p_full[2 * i], p_cnt[i] & 1, wctx, BAR_PFULL + 2 * i, j);
                            __syncwarp();
                            tc_fence_after();
                            if (tr) TT_TRACE(2, j, 4 * i + 1);
                            issue_pv(i, item_v, j > 0, 0);
                            mbar_wait(&bar_p_full[2 * i + 1], p_cnt[i] & 1, wctx, BAR_PFULL + 2 * i + 1, j);
                            ++p_cnt[i];
                            __syncwarp();
                            tc_fence_after();
                            if (tr) TT_TRACE(2, j, 4 * i + 2);
                            issue_pv(i, item_v, j > 0, 1);
                            if (j + 1 < w.n_tiles[i]) {
                                if (!k_waited) {
                                    wait_item(item_k);
                                    tc_fence_after();
                                    k_waited = true;
                                }
                                issue_s(i, item_k);
                                tc_commit(&bar_s_full[i]);
                                if (j + 2 == w.n_tiles[i]) tc_commit(&bar_q_empty[i]);   // this tile's last S
                                if (tr) TT_TRACE(2, j, 4 * i + 3);
                            } else {
                                tc_commit(&bar_o_final[i]);
                            }
                        }
                    }
                    if (p.s0_ahead && j + 1 == w.n_max && w.n_tiles[0] < w.n_max) {
                        // last iteration, slot 0 idle: S_0(0) of the next item (its K_0 is ring item t + 2 n_max)
                        ahead_item = next_item(k + 1);
                        __syncwarp();
                        if (ahead_item >= 0) {
                            const FwdItem wn = fwd_decode_item<kPaged, kVarlen>(ahead_item, p, D);
                            if (wn.n_tiles[0] > 0) {
                                const uint32_t tn = t + 2 * (uint32_t)w.n_max;
                                wait_item(tn);
                                tc_fence_after();
                                mbar_wait(&bar_q_full[0], q_uses[0] & 1, wctx, BAR_QFULL, k + 1);
                                ++q_uses[0];
                                __syncwarp();
                                tc_fence_after();
                                issue_s(0, tn);
                                tc_commit(&bar_s_full[0]);
                                if (wn.n_tiles[0] == 1) tc_commit(&bar_q_empty[0]);   // that was this tile's last S
                                s0_ahead = true;
                            }
                        }
                    }
                    release_item(item_v);
                    if (j + 1 < w.n_max) release_item(item_k);
                }
                t += 2 * (uint32_t)w.n_max;
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

// ------------------------------------------------------------------------------ host side
bool attn_fwd_sm100_supported(const AttnArgs& a) {
    if (a.block_table != nullptr && !a.cache_mode) return false;
    if (a.cache_mode) {   // decode over a cache: one query tile, no causal mask, key ranges of whole tiles
        if (!(a.causal == 0 && a.group == 1 && a.S <= 128)) return false;
        if (a.q_div > 1 ? !(a.kv_chunk >= 128 && a.kv_chunk % 128 == 0) : a.kv_chunk != 0) return false;
        const int ps = a.page_size;   // paged: whole pages per TMA box
        if (a.block_table != nullptr && !(ps >= 8 && (128 % ps == 0 || ps % 128 == 0) && a.max_pages >= 1)) return false;
    }
    return a.bf16 && (a.D == 64 || a.D == 128) && a.S >= 1 && a.L >= 1 && a.BH * (long long)((a.S + 255) / 256) < (1LL << 31);
}

static long long* g_fwd_trace = nullptr;
static int g_fwd_trace_block = 0, g_fwd_trace_item = 0;
void attn_fwd_set_trace(long long* device_buf, int block, int item) {
    g_fwd_trace = device_buf;
    g_fwd_trace_block = block;
    g_fwd_trace_item = item;
}

template <int D, bool kTrace, bool kPaged = false, bool kVarlen = false>
static cudaError_t launch_fwd(const AttnArgs& a, cudaStream_t st) {
    using Cfg = FwdCfg<D>;
    TmapStorage tq, tk, tv;
    const char* why = nullptr;
    const int q_div = a.q_div > 0 ? a.q_div : 1;
    if (kVarlen) {
        // token-major [tokens, heads, D]: row pitch heads*D elements, "slice" = head at pitch D
        if (!make_tmap_bf16_strided(&tq, a.q, D, a.total_q, a.H, (uint64_t)a.H * D, D, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16_strided(&tk, a.k, D, a.total_k, a.H / a.group, (uint64_t)(a.H / a.group) * D, D, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16_strided(&tv, a.v, D, a.total_k, a.H / a.group, (uint64_t)(a.H / a.group) * D, D, 128, &why)) return cudaErrorInvalidValue;
    } else if (!make_tmap_bf16(&tq, a.q, D, a.S, a.BH / q_div, 128, &why)) {
        return cudaErrorInvalidValue;
    } else if (kPaged && a.block_table != nullptr) {
        // The pools' page count is not known here; the extent only bounds what TMA may touch, and
        // the block table names the pages that exist.
        const uint64_t slices = 0x7fffffffull;
        const uint32_t box_rows = (uint32_t)std::min(a.page_size, 128);
        if (!make_tmap_bf16(&tk, a.k, D, (uint64_t)a.page_size, slices, box_rows, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16(&tv, a.v, D, (uint64_t)a.page_size, slices, box_rows, &why)) return cudaErrorInvalidValue;
    } else if (!kVarlen) {
        const long long kv_slices = kPaged ? a.BH / q_div : a.BH / a.group;
        if (!make_tmap_bf16(&tk, a.k, D, a.L, kv_slices, 128, &why)) return cudaErrorInvalidValue;
        if (!make_tmap_bf16(&tv, a.v, D, a.L, kv_slices, 128, &why)) return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_sm100_kernel<D, kTrace, kPaged, kVarlen>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    FwdParams p;
    p.out = (__nv_bfloat16*)a.out;
    p.lse = a.lse;
    p.S = a.S;
    p.L = a.L;
    p.n_qblk = (a.S + 255) / 256;
    p.causal = a.causal;
    p.group = a.group;
    p.kv_lens = a.kv_lens;
    p.H = a.H;
    p.q_div = q_div;
    p.block_table = a.block_table;
    p.page_size = a.page_size;
    p.max_pages = a.max_pages;
    p.kv_chunk = a.kv_chunk;
    p.cu_q = a.cu_q;
    p.cu_k = a.cu_k;
    p.total_q = (int)a.total_q;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = device_status_word();
    p.trace = g_fwd_trace;
    p.trace_block = g_fwd_trace_block;
    p.trace_item = g_fwd_trace_item;
    p.s0_ahead = (kPaged || kVarlen) ? 0 : 1;
    p.wide_stores = (reinterpret_cast<uintptr_t>(a.out) & 31) == 0 ? 1 : 0;
    p.n_items = (int)(a.BH * p.n_qblk);
    {
        // Causal items weigh in proportion to their query block's position.  With one slice-major
        // numbering the launch ends on the last slice's heaviest blocks while the other CTAs run dry;
        // keeping the lightest quarter of every slice's blocks (1/16 of the work) for a second phase
        // gives the CTAs that finish early something short to do.
        p.n_light = a.causal ? p.n_qblk / 4 : 0;
        p.n_items_heavy = (int)(a.BH * (p.n_qblk - p.n_light));
    }
    SchedCounter sc;
    e = sched_counter_acquire(st, &sc);
    if (e != cudaSuccess) return e;
    p.sched_counter = sc.ptr;
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    unsigned grid = (unsigned)std::min<long long>(p.n_items, n_sm);
    {
        LaunchScope ls(K_FWD_TC, st);
        attn_fwd_sm100_kernel<D, kTrace, kPaged, kVarlen><<<grid, Cfg::kThreads, Cfg::kSmemBytes, st>>>(
            *reinterpret_cast<CUtensorMap*>(tq.bytes), *reinterpret_cast<CUtensorMap*>(tk.bytes),
            *reinterpret_cast<CUtensorMap*>(tv.bytes), p);
    }
    sched_counter_release(sc, st);
    return cudaGetLastError();
}

template <int D>
static cudaError_t launch_fwd_d(const AttnArgs& a, cudaStream_t st) {
    if (a.cache_mode) return launch_fwd<D, false, true>(a, st);
    if (a.cu_q != nullptr) return launch_fwd<D, false, false, true>(a, st);
    if (g_fwd_trace != nullptr) return launch_fwd<D, true>(a, st);
    return launch_fwd<D, false>(a, st);
}
cudaError_t attn_fwd_sm100(const AttnArgs& a, cudaStream_t st) {
    if (g_fwd_trace == nullptr && attn_fwd_pair_sm100_supported(a)) return attn_fwd_pair_sm100(a, st);
    return a.D == 128 ? launch_fwd_d<128>(a, st) : launch_fwd_d<64>(a, st);
}

// ------------------------------------------------------------------------------ self test
// One CTA, 128 threads: S = A B^T (K = 128) from shared memory, S -> global; P = bf16(S)
// into tensor memory; O = P Vt (A from tensor memory, B MN-major) -> global.
template <int D>
__global__ void __launch_bounds__(128, 1)
umma_probe_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmV, float* s_out, float* o_out, unsigned int* status) {
    constexpr int kSubBytes = 128 * 128;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;
    unsigned char* sB = smem + 2 * kSubBytes;
    unsigned char* sV = smem + 4 * kSubBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kSubBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
    (void)lane;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_init(&bars[2], 1);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncwarp();
    if (warp == 0) {
        tmem_alloc(tmem_slot, 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    WaitCtx wctx{status, abort_flag, warp};
    if (warp == 0) {
        if (elect_one()) {
            mbar_arrive_expect_tx(&bars[0], (4 + D / 64) * kSubBytes);
            for (int sb = 0; sb < 2; ++sb) {
                tma_load_3d(sA + sb * kSubBytes, &tmA, &bars[0], sb * 64, 0, 0);
                tma_load_3d(sB + sb * kSubBytes, &tmB, &bars[0], sb * 64, 0, 0);
            }
            for (int sb = 0; sb < D / 64; ++sb) tma_load_3d(sV + sb * kSubBytes, &tmV, &bars[0], sb * 64, 0, 0);
        }
        __syncwarp();
        mbar_wait(&bars[0], 0, wctx, 0, 0);
        __syncwarp();
        tc_fence_after();
        constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);
        for (int kk = 0; kk < 8; ++kk) {
            const uint32_t o = (kk >> 2) * kSubBytes + (kk & 3) * 32;
            umma_ss(tmem_base, umma_smem_desc(smem_u32(sA) + o, 16, 1024), umma_smem_desc(smem_u32(sB) + o, 16, 1024),
                    idesc_s, kk > 0);
        }
        tc_commit(&bars[1]);
    }
    __syncwarp();
    mbar_wait(&bars[1], 0, wctx, 1, 0);
    __syncwarp();
    tc_fence_after();
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const int row = warp * 32 + lane;
    {
        uint32_t sr[4][32];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld32(tmem_base + lane_off + cc * 32, sr[cc]);
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                s_out[row * 128 + cc * 32 + e] = __uint_as_float(sr[cc][e]);
                s_out[row * 128 + cc * 32 + e + 1] = __uint_as_float(sr[cc][e + 1]);
                pk[e >> 1] = pack_bf16x2(__uint_as_float(sr[cc][e]), __uint_as_float(sr[cc][e + 1]));
            }
            tmem_st16(tmem_base + lane_off + cc * 16, pk);
        }
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        constexpr uint32_t idesc_pv = umma_idesc_bf16(128, D, false, true);
        for (int kk = 0; kk < 8; ++kk)
            umma_ts(tmem_base + 128, tmem_base + kk * 8, umma_smem_desc(smem_u32(sV) + kk * 2048, kSubBytes, 1024),
                    idesc_pv, kk > 0);
        tc_commit(&bars[2]);
    }
    __syncwarp();
    mbar_wait(&bars[2], 0, wctx, 2, 0);
    __syncwarp();
    tc_fence_after();
#pragma unroll
    for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t orr[32];
        tmem_ld32(tmem_base + lane_off + 128 + cc * 32, orr);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) o_out[row * D + cc * 32 + e] = __uint_as_float(orr[e]);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 256);
    }
}

template <int D>
static cudaError_t launch_probe(const void* a, const void* b, const void* vt, float* s_out, float* o_out,
                                cudaStream_t st) {
    TmapStorage ta, tb, tv;
    const char* why = nullptr;
    if (!make_tmap_bf16(&ta, a, 128, 128, 1, 128, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tb, b, 128, 128, 1, 128, &why)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16(&tv, vt, D, 128, 1, 128, &why)) return cudaErrorInvalidValue;
    const int smem = 6 * 128 * 128 + 1024 + 1024;
    cudaError_t e = cudaFuncSetAttribute(umma_probe_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    {
        LaunchScope ls(K_PROBE, st);
        umma_probe_kernel<D><<<1, 128, smem, st>>>(*reinterpret_cast<CUtensorMap*>(ta.bytes),
                                                   *reinterpret_cast<CUtensorMap*>(tb.bytes),
                                                   *reinterpret_cast<CUtensorMap*>(tv.bytes), s_out, o_out,
                                                   device_status_word());
    }
    return cudaGetLastError();
}

// Exercises the bounded-wait path: one warp waits on an mbarrier that nothing ever arrives on.
// The wait gives up after `budget_cycles`, records itself in the status word and the kernel
// returns normally (no trap, no hang); the host then sees TT_ERR_TIMEOUT.
__global__ void wait_timeout_kernel(unsigned int* status, long long budget_cycles) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    WaitCtx ctx{status, &abort_flag, 0, budget_cycles};
    mbar_wait(&bar, 0, ctx, 99, 7);
}
cudaError_t wait_timeout_probe(long long budget_cycles, cudaStream_t st) {
    LaunchScope ls(K_PROBE, st);
    wait_timeout_kernel<<<1, 32, 0, st>>>(device_status_word(), budget_cycles);
    return cudaGetLastError();
}

cudaError_t umma_probe(const void* a, const void* b, const void* vt, int D, float* s_out, float* o_out,
                       cudaStream_t st) {
    if (D == 128) return launch_probe<128>(a, b, vt, s_out, o_out, st);
    if (D == 64) return launch_probe<64>(a, b, vt, s_out, o_out, st);
    return cudaErrorInvalidValue;
}

}  // namespace ttk

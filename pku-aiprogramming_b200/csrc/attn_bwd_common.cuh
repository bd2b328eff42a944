// Pieces shared by the two tensor-core backward kernels (the two-pass kernel of attn_bwd_sm100.cu and the
// single-pass kernel of attn_bwd_fused_sm100.cu): launch parameters, the work-item numbering and the
// register split.
#pragma once
#include "common.h"
#include "sm100_ptx.cuh"

namespace ttk {

// Registers per thread after setmaxnreg (compute warpgroups / the loader-and-MMA warpgroup).
#ifndef TT_BWD_REGS_COMPUTE
#define TT_BWD_REGS_COMPUTE 216
#define TT_BWD_REGS_OTHER 72
#endif

struct BwdRegs {
    static constexpr int kThreads = 384;
    // The pool a CTA's setmaxnreg can draw from is what the launch allocated: kRegsLaunch per thread
    // (the __launch_bounds__ figure rounded down to a multiple of 8).  A split above it never completes.
    static constexpr int kRegsLaunch = 168;
    static constexpr int kRegsCompute = TT_BWD_REGS_COMPUTE;
    static constexpr int kRegsOther = TT_BWD_REGS_OTHER;
    static_assert(256 * kRegsCompute + 128 * kRegsOther <= kThreads * kRegsLaunch, "register split exceeds the CTA's pool");
    static_assert(kRegsCompute % 8 == 0 && kRegsOther % 8 == 0, "setmaxnreg takes multiples of 8");
};

struct BwdParams {
    __nv_bfloat16* out0;   // keys resident: dV ; else unused
    __nv_bfloat16* out1;   // keys resident: dK ; else dQ
    const float* lse2;     // [BH,S]  lse * log2(e)
    const float* delta;    // [BH,S]
    int S, L;
    int n_tiles;           // resident tiles per slice
    // causal: the n_light lightest resident tiles of every slice are numbered after all others, so that
    // CTAs that run out of heavy items near the end of the launch still find short ones (0: one phase)
    int n_light;
    int n_items_heavy;     // items of the first phase = slices * (n_tiles - n_light)
    int causal;
    float scale, scale_log2;
    unsigned int* status;
    unsigned int* sched_counter;   // zero at launch; work items are taken with atomicAdd
    int n_items;                   // resident slices * n_tiles
    int group;                     // query heads per key/value head (1 = ordinary multi-head attention)
    const int* kv_lens;            // optional key padding lengths per batch entry (see AttnArgs)
    int H;                         // query heads per batch entry
    int wide_stores;               // 1: the outputs are 32-byte aligned, the epilogue uses 32-byte stores
    // single-pass kernel only: fp32 dQ accumulator in global memory, one [D/4][128 rows][4] block per
    // (query slice, 128-row query tile), zero at launch; n_qt = query tiles per slice
    float* dq_acc;
    int n_qt;
    long long* trace;   // optional cycle trace of one CTA (debug aid): [3 roles][64 iterations][8 stamps]
    int trace_block;
    // packed variable-length batches (two-pass kernel only; see AttnArgs): per-sequence geometry from cu_q /
    // cu_k, token-major tensors, statistics as [H, total_q]; S and L above are the longest sequence's counts
    const int* cu_q;
    const int* cu_k;
    int total_q;
    int Hkv;                       // key/value heads per batch entry
};

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// One work item = one resident 128-row tile of one slice and the streamed tiles that meet it.
// With grouped heads (group g > 1) query slice bh reads key/value slice bh / g.  A pass that keeps
// queries resident streams the key/value slice of its query slice; a pass that keeps keys resident
// streams the query tiles of its g query heads one head after the other into the same accumulators,
// which is the sum over the group that dK and dV are.
struct BwdItem {
    int bh;        // resident slice (key/value slice when keys are resident, query slice otherwise)
    int r0, t_begin, t_end;
    int nt;        // streamed tiles per streamed slice
    int n_it;      // streamed tiles of the item (nt x group when keys are resident)
    int Lv;        // keys that count for this slice (<= L; fewer with key padding)
    // geometry of the item's slice: the launch's own S, L for dense tensors, the sequence's for packed ones
    int S, L;
    // packed batches only: first query / key token of the sequence, and the resident slice's head
    int q_lo, k_lo, head;
};
// The u-th streamed tile of an item: its tile index and the slice it belongs to (for packed batches the
// slice is a head: tensors are token-major and the sequence's first token is added to the row instead).
template <bool kKeysResident, bool kVarlen = false>
__device__ __forceinline__ void bwd_stream_tile(const BwdItem& w, int u, int group, int& t, int& slice) {
    if (kKeysResident) {
        const int hh = u / w.nt;
        t = w.t_begin + (u - hh * w.nt);
        slice = (kVarlen ? w.head : w.bh) * group + hh;
    } else {
        t = w.t_begin + u;
        slice = (kVarlen ? w.head : w.bh) / group;
    }
}
template <bool kKeysResident, bool kVarlen = false>
__device__ __forceinline__ BwdItem bwd_decode_item(int item, const BwdParams& p) {
    BwdItem w;
    int rank;   // position of the resident tile among its slice's tiles, heaviest first
    if (item < p.n_items_heavy) {
        const int n_heavy = p.n_tiles - p.n_light;
        w.bh = item / n_heavy;
        rank = item - w.bh * n_heavy;
    } else {
        const int r = item - p.n_items_heavy;
        w.bh = r / p.n_light;
        rank = (p.n_tiles - p.n_light) + (r - w.bh * p.n_light);
    }
    int S = p.S, L = p.L;
    if (kVarlen) {
        const int heads = kKeysResident ? p.Hkv : p.H;
        const int b = w.bh / heads;
        w.head = w.bh - b * heads;
        w.q_lo = p.cu_q[b];
        w.k_lo = p.cu_k[b];
        S = p.cu_q[b + 1] - w.q_lo;
        L = p.cu_k[b + 1] - w.k_lo;
        w.Lv = L;
    } else {
        // batch entry: a resident key/value slice is bh / (H / group), a resident query slice bh / H
        w.Lv = valid_keys(p.kv_lens, kKeysResident ? ((long long)w.bh * p.group) / p.H : (long long)w.bh / p.H, p.L);
        w.q_lo = w.k_lo = w.head = 0;
    }
    w.S = S;
    w.L = L;
    const int off = L - S;
    int rt;
    if (kKeysResident) {
        rt = rank;                                                    // early key tiles are the heavy ones
        w.t_end = (S + 127) >> 7;
        w.t_begin = p.causal ? (max(0, rt * 128 - off) >> 7) : 0;
        // a key tile that is all padding gets zero gradients: one streamed tile keeps the pipeline's
        // hand-offs alive, the epilogue writes zeros
        if (rt * 128 >= w.Lv) w.t_end = min(w.t_end, w.t_begin + 1);
    } else {
        rt = p.n_tiles - 1 - rank;                                    // late query tiles are the heavy ones
        const int n_kv = (w.Lv + 127) >> 7;
        w.t_begin = 0;
        w.t_end = p.causal ? min(n_kv, ((min(rt * 128 + 127, S - 1) + off) >> 7) + 1) : n_kv;
    }
    w.r0 = rt * 128;   // first resident row (key or query index)
    w.nt = max(0, w.t_end - w.t_begin);
    if (kVarlen && w.r0 >= (kKeysResident ? L : S)) w.nt = 0;   // the sequence is shorter than the longest one: nothing here
    w.n_it = kKeysResident ? w.nt * p.group : w.nt;
    return w;
}

// Writes the accumulators a compute thread holds for its resident row (kHalf fp32 columns as
// kHalf / 32 chunks) to `dst` as bf16, scaled by `mul`.
template <int kChunks>
__device__ __forceinline__ void bwd_store_row(__nv_bfloat16* dst, const uint32_t (&acc)[kChunks][32], float mul, int wide) {
#pragma unroll
    for (int cc = 0; cc < kChunks; ++cc) {
#pragma unroll
        for (int e = 0; e < 32; e += 16) {
            uint32_t o8[8];
#pragma unroll
            for (int q2 = 0; q2 < 8; ++q2)
                o8[q2] = sm100::pack_bf16x2(__uint_as_float(acc[cc][e + 2 * q2]) * mul, __uint_as_float(acc[cc][e + 2 * q2 + 1]) * mul);
            if (wide) {
                sm100::st_global_32B(dst + cc * 32 + e, o8);
            } else {
                *reinterpret_cast<uint4*>(dst + cc * 32 + e) = make_uint4(o8[0], o8[1], o8[2], o8[3]);
                *reinterpret_cast<uint4*>(dst + cc * 32 + e + 8) = make_uint4(o8[4], o8[5], o8[6], o8[7]);
            }
        }
    }
}

// Two-pass (bit-reproducible) backward and the single-pass one; both take the same workspace.
cudaError_t attn_bwd_two_pass(const AttnArgs& a, void* workspace, cudaStream_t st);
bool attn_bwd_fused_supported(const AttnArgs& a);
size_t attn_bwd_fused_workspace(const AttnArgs& a);
cudaError_t attn_bwd_fused(const AttnArgs& a, void* workspace, cudaStream_t st);
void attn_bwd_fused_set_trace(long long* device_buf, int block);

// dK/dV pass on CTA pairs (attn_bwd_pair_sm100.cu): same results as the one-CTA keys-resident pass.
bool attn_bwd_dkv_pair_supported(const AttnArgs& a);
cudaError_t attn_bwd_dkv_pair(const AttnArgs& a, const float* delta, const float* lse2, cudaStream_t st);

// delta[row] = sum_d dO*O ; lse2[row] = lse[row] * log2(e).  One warp per row.
cudaError_t attn_bwd_prep(const AttnArgs& a, float* delta, float* lse2, cudaStream_t st);

}  // namespace ttk

// Pieces shared by the forward attention kernels for sm_100a (the one-CTA kernel and the CTA-pair
// kernel): the launch parameters and the per-row softmax arithmetic of a softmax warpgroup thread.
#pragma once
#include "common.h"
#include "sm100_ptx.cuh"

namespace ttk {
using namespace sm100;

struct FwdParams {
    __nv_bfloat16* out;
    float* lse;
    int S, L;
    int n_qblk;       // 256-row query blocks per slice
    int n_light;      // causal: the n_light lightest query blocks of every slice are numbered after all others (0: one phase)
    int n_items_heavy;   // items of the first phase = slices * (n_qblk - n_light)
    int causal;
    float scale_log2; // scale * log2(e)
    unsigned int* status;
    unsigned int* sched_counter;   // zero at launch; work items are taken with atomicAdd
    int n_items;                   // slices * n_qblk
    int group;                     // query heads per key/value head: query slice bh reads key/value slice bh / group
    const int* kv_lens;            // optional key padding lengths per batch entry (see AttnArgs)
    int H;
    int q_div;                     // query slice = output slice / q_div
    const int* block_table;        // kPaged only: K and V are page pools (see AttnArgs)
    int page_size, max_pages;
    int kv_chunk;                  // kPaged: keys per output slice when a slice's keys are split (0: not split)
    // kVarlen: packed batches.  q/out are [total_q, H, D], k/v [total_k, H / group, D]; sequence b owns query
    // tokens [cu_q[b], cu_q[b+1]) and key tokens [cu_k[b], cu_k[b+1]); slices are (sequence, head) pairs,
    // S and L above are the LONGEST sequence's counts (they size the grid); lse is [H, total_q].
    const int* cu_q;
    const int* cu_k;
    int total_q;
    long long* trace;   // optional cycle trace of one CTA (debug aid): [3 roles][64 iterations][8 stamps]
    int trace_block;
    int trace_item;     // which of the CTA's work items gets the per-iteration stamps
    int s0_ahead;       // 1: issue the next item's S_0(0) in a causal item's idle last iteration
    int wide_stores;    // 1: `out` is 32-byte aligned, the epilogue uses 32-byte stores
};

// This thread's row of S (128 fp32 columns) from tensor memory; columns >= lim become -inf.
__device__ __forceinline__ void load_s_row(uint32_t tS, uint32_t (&sr)[4][32], bool need_mask, int lim) {
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) tmem_ld32(tS + cc * 32, sr[cc]);
    tmem_wait_ld();
    if (need_mask) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
#pragma unroll
            for (int e = 0; e < 32; ++e)
                if (cc * 32 + e >= lim) sr[cc][e] = 0xff800000u;   // -inf
    }
}
__device__ __forceinline__ float row_max_raw(const uint32_t (&sr)[4][32]) {
    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
        mx0 = fmax3(mx0, __uint_as_float(sr[0][e]), __uint_as_float(sr[0][e + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sr[1][e]), __uint_as_float(sr[1][e + 1]));
        mx2 = fmax3(mx2, __uint_as_float(sr[2][e]), __uint_as_float(sr[2][e + 1]));
        mx3 = fmax3(mx3, __uint_as_float(sr[3][e]), __uint_as_float(sr[3][e + 1]));
    }
    return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
}
// P = exp2(S*c - m) for one half (64 keys) of this thread's row: packs P to bf16 pairs and
// returns the two-lane partial row sum.
__device__ __forceinline__ uint64_t softmax_exp_half(const uint32_t (&sr)[4][32], int h, float c, float m,
                                                     uint32_t (&pk)[32]) {
    const float nm = -m;
    const uint64_t c2 = pack_f32x2(c, c), nm2 = pack_f32x2(nm, nm);
    uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
#pragma unroll
    for (int cq = 0; cq < 2; ++cq) {
        const int cc = h * 2 + cq;
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
            const uint64_t xa = fma_f32x2(pack_f32x2(__uint_as_float(sr[cc][e]), __uint_as_float(sr[cc][e + 1])), c2, nm2);
            const uint64_t xb = fma_f32x2(pack_f32x2(__uint_as_float(sr[cc][e + 2]), __uint_as_float(sr[cc][e + 3])), c2, nm2);
            float a0, a1, p2, p3;
            unpack_f32x2(xa, a0, a1);
            const float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
            {
                float b0, b1;
                unpack_f32x2(xb, b0, b1);
                p2 = ex2_approx(b0);
                p3 = ex2_approx(b1);
            }
            acc0 = add_f32x2(acc0, pack_f32x2(p0, p1));
            acc1 = add_f32x2(acc1, pack_f32x2(p2, p3));
            pk[cq * 16 + (e >> 1)] = pack_bf16x2(p0, p1);
            pk[cq * 16 + (e >> 1) + 1] = pack_bf16x2(p2, p3);
        }
    }
    return add_f32x2(acc0, acc1);
}

// ---- the CTA-pair forward (attn_fwd_pair_sm100.cu)
bool attn_fwd_pair_sm100_supported(const AttnArgs& a);
cudaError_t attn_fwd_pair_sm100(const AttnArgs& a, cudaStream_t st);

}  // namespace ttk

// Split-KV single-query attention (decode): out[bh] = softmax(scale * q[bh] K[bh]^T) V[bh].
//
// The work is HBM-bound (one FMA per byte of K/V), so the kernel is organised around
// streaming every K and V row exactly once with 16-byte loads that bypass L1:
//   - a unit = (slice, key range); units are laid out so that neighbouring CTAs read
//     neighbouring memory; the number of key ranges per slice is chosen so that there are
//     many more units than resident CTAs (small tail);
//   - D/8 lanes share one key row (each lane owns a 16-byte segment = 8 bf16), so a warp
//     load instruction covers 2 (D=128) or 4 (D=64) whole rows, fully coalesced;
//   - each lane keeps kUnroll K vectors and kUnroll V vectors in flight;
//   - scores are reduced across the lanes of a row with xor shuffles, then an online
//     softmax (base 2, fp32) updates the lane's 8 output accumulators;
//   - lanes/warps of a CTA are merged through shared memory; with more than one key range
//     per slice the unnormalised (max, sum, out) partials go to the workspace and a small
//     second kernel merges them.
#include <stdlib.h>

#include "common.h"
#include <atomic>

namespace ttk {

constexpr int kDecThreads = 256;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ float dot8(const uint4& a, const float (&q)[8]) {
    float s = bf_lo(a.x) * q[0];
    s = fmaf(bf_hi(a.x), q[1], s);
    s = fmaf(bf_lo(a.y), q[2], s);
    s = fmaf(bf_hi(a.y), q[3], s);
    s = fmaf(bf_lo(a.z), q[4], s);
    s = fmaf(bf_hi(a.z), q[5], s);
    s = fmaf(bf_lo(a.w), q[6], s);
    s = fmaf(bf_hi(a.w), q[7], s);
    return s;
}
__device__ __forceinline__ void axpy8(float p, const uint4& a, float (&o)[8]) {
    o[0] = fmaf(p, bf_lo(a.x), o[0]);
    o[1] = fmaf(p, bf_hi(a.x), o[1]);
    o[2] = fmaf(p, bf_lo(a.y), o[2]);
    o[3] = fmaf(p, bf_hi(a.y), o[3]);
    o[4] = fmaf(p, bf_lo(a.z), o[4]);
    o[5] = fmaf(p, bf_hi(a.z), o[5]);
    o[6] = fmaf(p, bf_lo(a.w), o[6]);
    o[7] = fmaf(p, bf_hi(a.w), o[7]);
}

// Merges two online-softmax states (base-2 exponent domain).
__device__ __forceinline__ void merge_state(float& m, float& l, float (&o)[8], float m2, float l2,
                                            const float (&o2)[8]) {
    float mn = fmaxf(m, m2);
    float a = (m == -INFINITY) ? 0.f : exp2f(m - mn);
    float b = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
    l = l * a + l2 * b;
#pragma unroll
    for (int t = 0; t < 8; ++t) o[t] = o[t] * a + o2[t] * b;
    m = mn;
}

// Where the key/value rows of a (batch, key/value head) slice live, and how many of them count.
//   dense:  k, v are [slices, L, D]                           (block_table == nullptr)
//   paged:  k, v are page pools [pages, hkv, page_size, D]; row r of batch entry b is in page
//           block_table[b * max_pages + r / page_size] at row r % page_size
//   seq_lens (optional): batch entry b has seq_lens[b] <= L keys; the rest is ignored
struct DecodeRows {
    const int* block_table;
    const int* seq_lens;
    int page_size, max_pages, hkv;
};

// partial layout in the workspace, per (unit, query head of the group): [m, l, o[D]] floats
//
// One CTA = one (key/value slice, key range) unit.  With grouped heads (G query heads share a
// key/value head) the CTA scores its rows against all G queries, so K and V cross HBM once for
// the whole group.  kMap: the generic fallback for group sizes without an instantiation -- one
// query per CTA, key/value slice = query slice / group (the group's CTAs are neighbours in the
// grid, so the re-reads mostly hit L2).
template <int D, int G>
__global__ void __launch_bounds__(kDecThreads, (G == 1 ? 4 : (G <= 4 ? 2 : 1)))
attn_decode_bf16_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                        const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ lse, float* __restrict__ partial, int L, int splits, int chunk,
                        float scale_log2, int map_group, DecodeRows rows) {
    constexpr int LPR = D / 8;        // lanes per key row
    constexpr int RPI = 32 / LPR;     // rows per warp load instruction
    __shared__ float sm_m[G][kDecWarps], sm_l[G][kDecWarps];
    __shared__ float sm_o[G][kDecWarps][D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPR, seg = lane % LPR;
    const long long unit = blockIdx.x;
    const long long slice = unit / splits;                 // query slice when G == 1, key/value slice otherwise
    const int split = (int)(unit - slice * splits);
    const long long kvs = (G == 1) ? slice / map_group : slice;
    const long long q0 = (G == 1) ? slice : slice * G;     // first query slice of this CTA
    const int b = (int)(kvs / rows.hkv), hk = (int)(kvs % rows.hkv);
    const int Lb = rows.seq_lens ? min(L, max(0, rows.seq_lens[b])) : L;
    const int k0 = split * chunk;
    const int k1 = min(Lb, k0 + chunk);

    float qf[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        uint4 qv = *reinterpret_cast<const uint4*>(q + (q0 + g) * D + seg * 8);
        qf[g][0] = bf_lo(qv.x) * scale_log2; qf[g][1] = bf_hi(qv.x) * scale_log2;
        qf[g][2] = bf_lo(qv.y) * scale_log2; qf[g][3] = bf_hi(qv.y) * scale_log2;
        qf[g][4] = bf_lo(qv.z) * scale_log2; qf[g][5] = bf_hi(qv.z) * scale_log2;
        qf[g][6] = bf_lo(qv.w) * scale_log2; qf[g][7] = bf_hi(qv.w) * scale_log2;
    }
    // element offset of key/value row r of this slice (without the lane's segment)
    const int* table = rows.block_table ? rows.block_table + (long long)b * rows.max_pages : nullptr;
    auto row_off = [&](int r) -> long long {
        if (table == nullptr) return (kvs * (long long)L + r) * D;
        const int pg = r / rows.page_size;
        const int page = table[pg];
        return (((long long)page * rows.hkv + hk) * rows.page_size + (r - pg * rows.page_size)) * D;
    };
    const __nv_bfloat16* kb = k + seg * 8;
    const __nv_bfloat16* vb = v + seg * 8;
    float m[G], l[G], o[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int t = 0; t < 8; ++t) o[g][t] = 0.f;
    }

    constexpr int kRowsPerIter = kDecWarps * RPI * kUnroll;   // rows a CTA consumes per iteration
    for (int base = k0 + warp * (RPI * kUnroll); base < k1; base += kRowsPerIter) {
        uint4 kv[kUnroll], vv[kUnroll];
        bool ok[kUnroll];
        long long ro[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int r = base + u * RPI + sub;
            ok[u] = r < k1;
            ro[u] = row_off(ok[u] ? r : k0);   // any valid row; its score is discarded below
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) kv[u] = ld_stream16(kb + ro[u]);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) vv[u] = ld_stream16(vb + ro[u]);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float s[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                float x = dot8(kv[u], qf[g]);
#pragma unroll
                for (int off = LPR / 2; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
                s[u] = ok[u] ? x : -INFINITY;
            }
            float mx = s[0];
#pragma unroll
            for (int u = 1; u < kUnroll; ++u) mx = fmaxf(mx, s[u]);
            // branch-free running-maximum update (a branch per query head would cut the unrolled
            // body into basic blocks and nothing would be scheduled across the heads): the
            // correction is exactly 1 when the maximum did not move and 0 for a state that was empty
            const float mnew = fmaxf(m[g], mx);
            const float mref = (mnew == -INFINITY) ? 0.f : mnew;   // no inf - inf when nothing is visible yet
            const float corr = exp2f(m[g] - mref);
            l[g] *= corr;
#pragma unroll
            for (int t = 0; t < 8; ++t) o[g][t] *= corr;
            m[g] = mnew;
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const float pu = exp2f(s[u] - mref);             // masked rows: exp2(-inf) = 0
                l[g] += pu;
                axpy8(pu, vv[u], o[g]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
        // merge the RPI row groups of the warp (states live at lanes with equal `seg`)
#pragma unroll
        for (int off = 16; off >= LPR; off >>= 1) {
            float m2 = __shfl_xor_sync(0xffffffffu, m[g], off);
            float l2 = __shfl_xor_sync(0xffffffffu, l[g], off);
            float o2[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) o2[t] = __shfl_xor_sync(0xffffffffu, o[g][t], off);
            merge_state(m[g], l[g], o[g], m2, l2, o2);
        }
        if (lane < LPR) {
            if (lane == 0) {
                sm_m[g][warp] = m[g];
                sm_l[g][warp] = l[g];
            }
#pragma unroll
            for (int t = 0; t < 8; ++t) sm_o[g][warp][seg * 8 + t] = o[g][t];
        }
    }
    __syncthreads();
    if (threadIdx.x < D) {
        const int d = threadIdx.x;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float M = sm_m[g][0];
#pragma unroll
            for (int w = 1; w < kDecWarps; ++w) M = fmaxf(M, sm_m[g][w]);
            float Lsum = 0.f, O = 0.f;
#pragma unroll
            for (int w = 0; w < kDecWarps; ++w) {
                float a = (sm_m[g][w] == -INFINITY) ? 0.f : exp2f(sm_m[g][w] - M);
                Lsum = fmaf(sm_l[g][w], a, Lsum);
                O = fmaf(sm_o[g][w][d], a, O);
            }
            if (splits == 1) {
                // a sequence without keys (seq_lens[b] == 0) has no distribution: output 0, lse -inf
                out[(q0 + g) * D + d] = __float2bfloat16_rn(Lsum > 0.f ? O / Lsum : 0.f);
                if (d == 0 && lse != nullptr) lse[q0 + g] = (M + log2f(Lsum)) * 0.6931471805599453f;
            } else {
                float* pu = partial + (unit * G + g) * (D + 2);
                pu[2 + d] = O;
                if (d == 0) {
                    pu[0] = M;
                    pu[1] = Lsum;
                }
            }
        }
    }
}

// out[bh] from the `splits` partial states of its key ranges.  G as in the kernel above: the
// partials of query head g of key/value slice kvs are at ((kvs * splits + s) * G + g).
template <int D>
__global__ void attn_decode_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                         float* __restrict__ lse, int splits, int G) {
    const long long bh = blockIdx.x;
    const int d = threadIdx.x;
    const long long kvs = bh / G;
    const int g = (int)(bh - kvs * G);
    const float* pb = partial + ((kvs * splits) * G + g) * (D + 2);
    const long long stride = (long long)G * (D + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, pb[s * stride]);
    float Lsum = 0.f, O = 0.f;
    for (int s = 0; s < splits; ++s) {
        float ms = pb[s * stride];
        float a = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
        Lsum = fmaf(pb[s * stride + 1], a, Lsum);
        O = fmaf(pb[s * stride + 2 + d], a, O);
    }
    out[bh * D + d] = __float2bfloat16_rn(Lsum > 0.f ? O / Lsum : 0.f);
    if (d == 0 && lse != nullptr) lse[bh] = (M + log2f(Lsum)) * 0.6931471805599453f;
}

static int env_int(const char* name, int dflt);

static bool decode_group_instantiated(int g) { return g == 1 || g == 2 || g == 4 || g == 8; }

// Grouped heads on a dense cache, as a tensor-core problem: the G query heads of a key/value head
// are contiguous in q [B, Hkv*G, 1, D], i.e. they ARE a [B, Hkv, G, D] tensor of G query rows per
// key/value head, and out / lse have the matching layout.  The forward kernel then computes the
// whole group against each K/V tile with two MMAs, which the SIMT kernel cannot keep up with from
// G = 4 on (it is instruction-bound: G dot products and G softmax updates per loaded row).
// With fewer (batch, key/value head) items than SMs the keys are split as well: K and V viewed as
// [slices * splits, L / splits, D] are `splits` independent problems per slice (the forward kernel
// reads the query rows of slice s / splits), whose normalised partial outputs and log-sum-exps a
// second kernel merges.
// The forward view of a grouped decode runs on the keys-on-rows decode kernel where that takes it (head
// dim 128, groups of up to 16), else on the general forward kernel.
static cudaError_t run_forward_view(const AttnArgs& g, cudaStream_t st) {
    return attn_decode_gq_sm100_supported(g) ? attn_decode_gq_sm100(g, st) : attn_fwd_sm100(g, st);
}
static AttnArgs decode_as_forward(const AttnArgs& a, int splits) {
    AttnArgs g = a;
    g.BH = a.BH / a.group * splits;
    g.S = a.group;
    g.L = a.L / splits;
    g.group = 1;
    g.causal = 0;
    g.q_div = splits;
    g.kv_lens = nullptr;
    return g;
}
// true: the tensor-core route of this decode is the keys-on-rows kernel.  It runs two CTAs per SM, one per
// (slice, key range).  As many slices as SMs already keep HBM busy (the CTAs share its bandwidth, so a
// partial last wave costs little: measured, 256 and 512 unsplit slices beat any split); with fewer, the
// keys are cut into about four ranges per SM of at least 512 keys.
static bool decode_on_gq_kernel(const AttnArgs& a) {
    const char* f = getenv("TT_DECODE_GQA_PATH");
    return a.bf16 && (a.D == 128 || a.D == 64) && a.S == 1 && a.group <= 16 && !(f && f[0] == 'f');
}
static int decode_tc_splits(const AttnArgs& a) {   // 0: do not use the forward kernel
    const char* f = getenv("TT_DECODE_GQA_PATH");
    // the keys-on-rows kernel takes every group size up to 16 (measured faster than the split-KV kernel even for
    // single heads); larger groups take the forward kernel
    const int min_group = decode_on_gq_kernel(a) ? 1 : 4;
    if (!(a.bf16 && a.S == 1 && a.group >= min_group)) return 0;
    if (f && f[0] == 's') return 0;                           // "simt"
    if (!attn_fwd_sm100_supported(decode_as_forward(a, 1))) return 0;
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    const long long slices = a.BH / a.group;
    const bool gq = decode_on_gq_kernel(a);
    const long long min_chunk = gq ? 512 : 256;
    if (slices >= n_sm) return 1;
    // about four (forward kernel: two) items per SM, ranges of at least min_chunk keys that divide L exactly
    const long long want = ((gq ? 4LL : 2LL) * n_sm + slices - 1) / slices;
    for (long long s = want; s <= 64 && a.L / s >= min_chunk; ++s)
        if (a.L % s == 0) return (int)s;
    for (long long s = want - 1; s >= 2; --s)
        if (a.L % s == 0 && a.L / s >= min_chunk) return (int)s;
    if (gq) return 1;                                         // short or indivisible key range: one range per slice
    return (f && f[0] == 't') ? 1 : 0;                        // "tc": unsplit rather than SIMT
}

DecodePlan attn_decode_plan(const AttnArgs& a, bool allow_tc) {
    DecodePlan pl{1, a.L, 0, 0};
    if (!(a.bf16 && (a.D == 64 || a.D == 128) && a.S == 1)) return pl;   // SIMT forward handles it
    if (allow_tc) {
        pl.tc_splits = decode_tc_splits(a);
        if (pl.tc_splits == 1) return pl;
        if (pl.tc_splits > 1) {   // partial outputs (bf16) and log-sum-exps (fp32) of every key range
            pl.splits = pl.tc_splits;
            pl.chunk = a.L / pl.tc_splits;
            pl.ws_bytes = align256((size_t)a.BH * pl.tc_splits * a.D * 2) + align256((size_t)a.BH * pl.tc_splits * 4);
            return pl;
        }
    }
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    const long long resident = (long long)n_sm * 4;
    const long long target = resident * 12;
    const long long cta_slices = decode_group_instantiated(a.group) ? a.BH / a.group : a.BH;
    long long splits = (target + cta_slices - 1) / cta_slices;
    long long max_splits = a.L / 256;
    if (max_splits < 1) max_splits = 1;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    int forced = env_int("TT_DECODE_SPLITS", 0);
    if (forced > 0) splits = forced;
    int chunk = (int)((a.L + splits - 1) / splits);
    chunk = (chunk + 63) / 64 * 64;
    splits = (a.L + chunk - 1) / chunk;
    pl.splits = (int)splits;
    pl.chunk = chunk;
    pl.ws_bytes = splits > 1 ? align256((size_t)splits * a.BH * (a.D + 2) * sizeof(float)) : 0;
    return pl;
}

// Merge of the forward kernel's per-range results: out[bh] = sum_c w_c O_c / sum_c w_c with
// w_c = exp(lse_c - max lse); partial O is [kvs, splits, G, D] bf16, partial lse [kvs, splits, G].
template <int D>
__global__ void attn_decode_tc_merge_kernel(const __nv_bfloat16* __restrict__ po, const float* __restrict__ plse,
                                            __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int splits, int G) {
    const long long bh = blockIdx.x;
    const int d = threadIdx.x;
    const long long kvs = bh / G;
    const int g = (int)(bh - kvs * G);
    float m = -INFINITY;
    for (int c = 0; c < splits; ++c) m = fmaxf(m, plse[(kvs * splits + c) * G + g]);
    if (m == -INFINITY) {   // no range held a key (an empty sequence of a paged cache)
        out[bh * D + d] = __float2bfloat16_rn(0.f);
        if (d == 0 && lse != nullptr) lse[bh] = -INFINITY;
        return;
    }
    float den = 0.f, acc = 0.f;
    for (int c = 0; c < splits; ++c) {
        const long long row = (kvs * splits + c) * G + g;
        const float w = expf(plse[row] - m);
        den += w;
        acc = fmaf(w, __bfloat162float(po[row * D + d]), acc);
    }
    out[bh * D + d] = __float2bfloat16_rn(acc / den);
    if (d == 0 && lse != nullptr) lse[bh] = m + logf(den);
}

template <int D, int G>
static void launch_decode_g(const AttnArgs& a, const DecodePlan& pl, void* ws, cudaStream_t st, const DecodeRows& rows) {
    const long long units = (a.BH / G) * pl.splits;
    attn_decode_bf16_kernel<D, G><<<(unsigned)units, kDecThreads, 0, st>>>(
        (const __nv_bfloat16*)a.q, (const __nv_bfloat16*)a.k, (const __nv_bfloat16*)a.v, (__nv_bfloat16*)a.out, a.lse,
        (float*)ws, a.L, pl.splits, pl.chunk, a.scale * 1.4426950408889634f, a.group, rows);
}

template <int D>
static cudaError_t launch_decode(const AttnArgs& a, const DecodePlan& pl, void* ws, cudaStream_t st,
                                 bool allow_timing = true, const DecodeView* view = nullptr) {
    DecodeRows rows{nullptr, nullptr, 0, 0, 1};
    if (view) rows = DecodeRows{view->block_table, view->seq_lens, view->page_size, view->max_pages, view->hkv};
    const int G = decode_group_instantiated(a.group) ? a.group : 1;
    {
        LaunchScope ls(K_DECODE, st, allow_timing);
        switch (G) {
            case 8: launch_decode_g<D, 8>(a, pl, ws, st, rows); break;
            case 4: launch_decode_g<D, 4>(a, pl, ws, st, rows); break;
            case 2: launch_decode_g<D, 2>(a, pl, ws, st, rows); break;
            default: launch_decode_g<D, 1>(a, pl, ws, st, rows); break;
        }
    }
    if (pl.splits > 1) {
        LaunchScope ls(K_DECODE_MERGE, st, allow_timing);
        attn_decode_merge_kernel<D><<<(unsigned)a.BH, D, 0, st>>>((const float*)ws, (__nv_bfloat16*)a.out, a.lse,
                                                                  pl.splits, G);
    }
    return cudaGetLastError();
}

// Decode over a ragged and/or paged cache as a forward problem: the same [batch x key/value heads, G, D] view as
// above, with sequence lengths per batch entry and, for a paged cache, the forward kernel's loader
// gathering each 128-key tile page by page through the block table.  With few slices the key range is cut into `splits` ranges of `chunk` keys (work
// items of their own, merged afterwards); a range past a sequence's end yields a zero partial with
// log-sum-exp -inf, which the merge gives no weight.
static AttnArgs paged_as_forward(const AttnArgs& a, const DecodeView& v, int splits, int chunk) {
    AttnArgs g = decode_as_forward(a, 1);
    g.BH = a.BH / a.group * splits;
    g.q_div = splits;
    g.kv_chunk = splits > 1 ? chunk : 0;
    g.cache_mode = 1;
    g.H = v.hkv;                    // key/value slices per batch entry
    g.kv_lens = v.seq_lens;
    g.block_table = v.block_table;
    g.page_size = v.page_size;
    g.max_pages = v.max_pages;
    return g;
}
static void paged_split(const AttnArgs& a, int* splits, int* chunk) {
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    const long long slices = a.BH / a.group;
    *splits = 1;
    *chunk = a.L;
    const bool gq = decode_on_gq_kernel(a);
    if (gq ? slices >= n_sm : 2 * slices >= n_sm) return;
    // about four (forward kernel: two) items per SM, ranges of whole 128-key tiles
    const long long want = ((gq ? 4LL : 2LL) * n_sm + slices - 1) / slices;
    const long long min_chunk = gq ? 512 : 256;
    long long c = ((a.L + want - 1) / want + 127) / 128 * 128;
    if (c < min_chunk) c = min_chunk;
    const long long n = (a.L + c - 1) / c;
    if (n < 2) return;
    *splits = (int)n;
    *chunk = (int)c;
}
int attn_decode_paged_on_forward(const AttnArgs& a, const DecodeView& v, size_t* ws_bytes) {
    *ws_bytes = 0;
    if (!(a.bf16 && a.S == 1 && a.group >= (decode_on_gq_kernel(a) ? 1 : 4) && (v.block_table != nullptr || v.seq_lens != nullptr))) return 0;
    const char* f = getenv("TT_DECODE_GQA_PATH");
    if (f && f[0] == 's') return 0;                           // "simt"
    int splits, chunk;
    paged_split(a, &splits, &chunk);
    if (!attn_fwd_sm100_supported(paged_as_forward(a, v, splits, chunk))) return 0;
    if (splits > 1) *ws_bytes = align256((size_t)a.BH * splits * a.D * 2) + align256((size_t)a.BH * splits * 4);
    return splits;
}
cudaError_t attn_decode_paged_forward(const AttnArgs& a, const DecodeView& v, int splits, void* ws, cudaStream_t st) {
    int s2, chunk;
    paged_split(a, &s2, &chunk);
    if (s2 != splits) return cudaErrorInvalidValue;
    AttnArgs g = paged_as_forward(a, v, splits, chunk);
    if (splits == 1) return run_forward_view(g, st);
    __nv_bfloat16* po = (__nv_bfloat16*)ws;
    float* plse = (float*)((unsigned char*)ws + align256((size_t)a.BH * splits * a.D * 2));
    g.out = po;
    g.lse = plse;
    cudaError_t e = run_forward_view(g, st);
    if (e != cudaSuccess) return e;
    LaunchScope ls(K_DECODE_MERGE, st);
    if (a.D == 128)
        attn_decode_tc_merge_kernel<128><<<(unsigned)a.BH, 128, 0, st>>>(po, plse, (__nv_bfloat16*)a.out, a.lse, splits, a.group);
    else
        attn_decode_tc_merge_kernel<64><<<(unsigned)a.BH, 64, 0, st>>>(po, plse, (__nv_bfloat16*)a.out, a.lse, splits, a.group);
    return cudaGetLastError();
}

cudaError_t attn_decode(const AttnArgs& a, const DecodePlan& pl, void* ws, cudaStream_t st, const DecodeView* view) {
    const bool plain = !(view && (view->block_table || view->seq_lens));
    if (plain && pl.tc_splits == 1) return run_forward_view(decode_as_forward(a, 1), st);
    if (plain && pl.tc_splits > 1) {
        AttnArgs g = decode_as_forward(a, pl.tc_splits);
        __nv_bfloat16* po = (__nv_bfloat16*)ws;
        float* plse = (float*)((unsigned char*)ws + align256((size_t)a.BH * pl.tc_splits * a.D * 2));
        g.out = po;
        g.lse = plse;
        cudaError_t e = run_forward_view(g, st);
        if (e != cudaSuccess) return e;
        LaunchScope ls(K_DECODE_MERGE, st);
        if (a.D == 128)
            attn_decode_tc_merge_kernel<128><<<(unsigned)a.BH, 128, 0, st>>>(po, plse, (__nv_bfloat16*)a.out, a.lse, pl.tc_splits, a.group);
        else
            attn_decode_tc_merge_kernel<64><<<(unsigned)a.BH, 64, 0, st>>>(po, plse, (__nv_bfloat16*)a.out, a.lse, pl.tc_splits, a.group);
        return cudaGetLastError();
    }
    if (a.bf16 && a.S == 1 && a.D == 128) return launch_decode<128>(a, pl, ws, st, true, view);
    if (a.bf16 && a.S == 1 && a.D == 64) return launch_decode<64>(a, pl, ws, st, true, view);
    if (view && (view->block_table || view->seq_lens)) return cudaErrorNotSupported;   // paged / ragged: bf16, D 64 or 128
    return attn_fwd_simt(a, st);
}

// ------------------------------------------------------------------------------------------
// Variant for callers that must not allocate device memory: the split-KV partials live in a
// fixed array that is part of this library's device image.  Every context that loads the
// library carries these bytes until it exits, whether or not this path is ever called.
constexpr size_t kStaticScratchBytes = (size_t)8 << 20;   // 8 MiB
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not a device address: the
// address a kernel can use has to be asked for, per device, with that device current.
constexpr int kMaxDevices = 64;
static void* g_static_scratch_addr[kMaxDevices];
static std::atomic<int> g_static_scratch_ready[kMaxDevices];

size_t attn_decode_static_capacity() { return kStaticScratchBytes; }

cudaError_t attn_decode_static(const AttnArgs& a, const DecodePlan& pl, cudaStream_t st, bool* too_big) {
    *too_big = pl.ws_bytes > kStaticScratchBytes;
    if (*too_big) return cudaSuccess;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!g_static_scratch_ready[dev].load(std::memory_order_acquire)) {
        // first call on this device: resolve the device address of the array
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_scratch_addr[dev] = p;
        g_static_scratch_ready[dev].store(1, std::memory_order_release);
    }
    void* scratch = g_static_scratch_addr[dev];
    // Nothing in the array has to start at zero: every partial the merge kernel reads is
    // written by the first kernel of the same call.
    if (a.D == 128) return launch_decode<128>(a, pl, scratch, st, /*allow_timing=*/false);
    return launch_decode<64>(a, pl, scratch, st, /*allow_timing=*/false);
}

}  // namespace ttk

#include <stdlib.h>
namespace ttk {
static int env_int(const char* name, int dflt) {
    const char* s = getenv(name);
    return (s && *s) ? atoi(s) : dflt;
}
}  // namespace ttk

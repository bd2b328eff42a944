// Internal declarations shared by the kernel translation units and the C-ABI layer.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stddef.h>
#include <stdint.h>

namespace ttk {

// Fully resolved launch arguments (device pointers, scale already defaulted).
struct AttnArgs {
    long long BH;   // B*H query slices
    int group;      // query heads per key/value head (>= 1); k, v, dk, dv have BH / group slices
    int S, L, D;
    int causal;
    int bf16;       // 1: __nv_bfloat16 tensors, 0: float
    float scale;
    const void *q, *k, *v, *dout;
    void* out;
    float* lse;     // forward: written (may be null); backward: read
    void *dq, *dk, *dv;
    // optional key padding: batch entry b attends to its first kv_lens[b] keys (1..L; device int32
    // [B]); null = all L.  H = query heads per batch entry (batch entry of query slice bh = bh / H).
    const int* kv_lens;
    int H;
    // forward kernel only: query slice = output slice / q_div (0 or 1: the same slice).  Lets several
    // key ranges of one slice run as work items of their own, each with its own output rows.
    int q_div;
    // forward kernel only, used by decode over a ragged and/or paged cache (cache_mode = 1): kv_lens
    // may hold 0 (an empty sequence: zero output, log-sum-exp -inf), and what lies behind a
    // sequence's end never reaches the result, whatever bits it holds.  block_table != null: k and v
    // are page pools [pages, H, page_size, D] (H = key/value heads here) and key r of batch entry b
    // is row r % page_size of page block_table[b * max_pages + r / page_size]; page_size divides
    // 128 or is a multiple of it.
    // With kv_chunk > 0 output slice s covers keys [c * kv_chunk, (c + 1) * kv_chunk) of key/value slice
    // s / q_div, c = s % q_div (kv_chunk a multiple of 128); L stays the whole key range.
    const int* block_table;
    int page_size, max_pages;
    int kv_chunk;
    int cache_mode;
    // packed variable-length batches (tensor-core kernels only): cu_q / cu_k are device int32 [n_seq + 1]
    // cumulative token counts; q, out, dout, dq are [total_q, H, D], k, v, dk, dv [total_k, H / group, D],
    // lse [H, total_q]; BH = n_seq * H slices; S and L hold the longest sequence's counts.
    const int* cu_q;
    const int* cu_k;
    long long total_q, total_k;
};
// keys that count for batch entry b (device side)
__device__ __forceinline__ int valid_keys(const int* kv_lens, long long b, int L) {
    return kv_lens ? min(L, max(1, kv_lens[b])) : L;
}

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// Error reporting of the C-ABI layer: records the message tt_last_error() returns on this thread and
// hands back `code` (a tt_status).
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
int check_device();   // TT_OK, or TT_ERR_BAD_DEVICE when the current device is not an sm_100 part

// Kernel families, for launch accounting and the optional per-kernel event timing.
enum KernelId {
    K_FWD_TC = 0, K_FWD_SIMT, K_BWD_PREP, K_BWD_DKV, K_BWD_DQ, K_BWD_SIMT_DELTA, K_BWD_SIMT_DQ, K_BWD_SIMT_DKV,
    K_DECODE, K_DECODE_MERGE, K_PROBE, K_SOFTMAX_FWD, K_SOFTMAX_BWD, K_FC_GEMM, K_FC_SIMT, K_FC_COLSUM, K_BWD_FUSED,
    K_BWD_DQ_CONVERT, K_DECODE_GQ, K_COUNT
};
// Scoped around ONE kernel launch: counts it and, when timing is enabled, brackets it with
// CUDA events on the launching stream.
struct LaunchScope {
    // allow_timing = false: count only (creates no events, so nothing is allocated)
    LaunchScope(KernelId id, cudaStream_t st, bool allow_timing = true);
    ~LaunchScope();
    KernelId id;
    cudaStream_t st;
    void* rec;
};
unsigned int* device_status_word();  // 4 x uint32 in global memory of the current device (zeroed)

// Work-item counter of one persistent launch: a slot of a small per-device set, cleared on the launch
// stream.  `release` records the launch's completion on the slot, so that a later launch that is handed
// the same slot while this one still runs is ordered behind it instead of sharing its counter.
struct SchedCounter {
    unsigned int* ptr = nullptr;
    int slot = -1;
};
cudaError_t sched_counter_acquire(cudaStream_t st, SchedCounter* c);
void sched_counter_release(const SchedCounter& c, cudaStream_t st);


// --- SIMT fp32-arithmetic kernels (any D <= 256, float or bf16 tensors)
cudaError_t attn_fwd_simt(const AttnArgs& a, cudaStream_t st);
cudaError_t attn_bwd_simt(const AttnArgs& a, float* delta, cudaStream_t st);
size_t attn_bwd_simt_workspace(const AttnArgs& a);

// --- grouped-head decode with keys on the accumulator rows (attn_decode_gq_sm100.cu); `a` is the forward
// view of the decode (S = query heads per key/value head)
bool attn_decode_gq_sm100_supported(const AttnArgs& a);
cudaError_t attn_decode_gq_sm100(const AttnArgs& a, cudaStream_t st);

// --- tcgen05 / TMA kernels (bf16, D in {64,128})
bool attn_fwd_sm100_supported(const AttnArgs& a);
cudaError_t attn_fwd_sm100(const AttnArgs& a, cudaStream_t st);
// Debug aid: when device_buf is non-null, CTA `block` of every later forward launch stamps
// clock64() at its hand-off points into device_buf ([3 roles][64 iterations][8 stamps]).
void attn_fwd_set_trace(long long* device_buf, int block, int item);
void attn_bwd_set_trace(long long* device_buf, int block, int pass);   // pass 1: dK/dV, 2: dQ
bool attn_bwd_sm100_supported(const AttnArgs& a);
size_t attn_bwd_sm100_workspace(const AttnArgs& a);
cudaError_t attn_bwd_sm100(const AttnArgs& a, void* workspace, cudaStream_t st);
// Which tensor-core backward runs: 0 = the faster one for the shape (the single pass -- dQ through fp32 adds
// in global memory, five GEMMs per tile pair, dQ reproducible to fp32 rounding -- or the two passes),
// 1 = always the two passes (seven GEMMs, every result bit-reproducible).
void attn_bwd_set_deterministic(int on);
int attn_bwd_deterministic();
cudaError_t wait_timeout_probe(long long budget_cycles, cudaStream_t st);
cudaError_t umma_probe(const void* a, const void* b, const void* vt, int D, float* s_out, float* o_out,
                       cudaStream_t st);

// --- row softmax (adjacent native op of the reference), fp32 or bf16 rows
cudaError_t softmax_rows_fwd(const void* in, void* out, long long rows, int cols, int bf16, cudaStream_t st);
cudaError_t softmax_rows_bwd(const void* y, const void* dy, void* dx, long long rows, int cols, int bf16,
                             cudaStream_t st);

// --- fully connected layer: C[M,N] = op(A) op(B) (+ bias[N]), row-major, fp32 accumulation.
//   a_mn = 0: A stored [M,K];  a_mn = 1: A stored [K,M] (the product uses its transpose)
//   b_mn = 1: B stored [K,N];  b_mn = 0: B stored [N,K] (the product uses its transpose)
// bf16 with 16-byte row pitches runs the tcgen05 kernel, everything else the fp32 SIMT kernel.
bool fc_gemm_tc_supported(const void* A, const void* B, const void* C, const void* bias, long long M, int N, int K,
                          int a_mn, int b_mn, int bf16);
cudaError_t fc_gemm(const void* A, const void* B, void* C, const void* bias, long long M, int N, int K, int a_mn,
                    int b_mn, int bf16, cudaStream_t st);
// out[n] = sum over rows of X[M,N] (scalar_bias: out[0] = sum of everything); workspace of
// fc_colsum_workspace(M, N) bytes holds the per-range partial sums.
size_t fc_colsum_workspace(long long M, int N);
cudaError_t fc_colsum(const void* X, void* out, long long M, int N, int bf16, int scalar_bias, void* workspace,
                      cudaStream_t st);

// --- split-KV decode (S == 1, bf16 or float)
struct DecodePlan {
    int splits;        // key ranges per slice
    int chunk;         // keys per range (multiple of 64)
    size_t ws_bytes;   // partials: splits * BH * (D + 2) floats (0 when splits == 1)
    // grouped heads on the tcgen05 forward kernel (see attn_decode.cu): 0 = not taken, 1 = whole key
    // range per (batch, key/value head), > 1 = that many key ranges each, merged by a second kernel
    int tc_splits;
};
// allow_tc = false: plan for the SIMT split-KV kernel whatever the shape (paged / ragged caches and
// the no-allocation entry point need it)
DecodePlan attn_decode_plan(const AttnArgs& a, bool allow_tc = true);
// Optional description of where the key/value rows live (bf16, D in {64,128} only):
//   block_table != null: k, v are page pools [pages, hkv, page_size, D] and row r of batch entry b
//                        is row r % page_size of page block_table[b * max_pages + r / page_size];
//   seq_lens != null:    batch entry b has seq_lens[b] (<= L) keys, the rest is ignored.
struct DecodeView {
    const int* block_table = nullptr;
    const int* seq_lens = nullptr;
    int page_size = 0, max_pages = 0;
    int hkv = 1;   // key/value heads per batch entry
};
cudaError_t attn_decode(const AttnArgs& a, const DecodePlan& plan, void* workspace, cudaStream_t st,
                        const DecodeView* view = nullptr);

// Paged decode with grouped heads (group >= 4) on the tcgen05 forward kernel; the SIMT split-KV
// kernel serves every other paged call.
// Returns the number of key ranges per slice (0: route not taken, 1: no merge, no workspace).
int attn_decode_paged_on_forward(const AttnArgs& a, const DecodeView& view, size_t* ws_bytes);
cudaError_t attn_decode_paged_forward(const AttnArgs& a, const DecodeView& view, int splits, void* workspace,
                                      cudaStream_t st);

// Same kernels, partials in the library's own fixed device array (no allocation anywhere).
// *too_big is set when the plan needs more than the array holds (nothing is launched then).
size_t attn_decode_static_capacity();
cudaError_t attn_decode_static(const AttnArgs& a, const DecodePlan& plan, cudaStream_t st, bool* too_big);

// Builds a 3-D bf16 tensor map over a dense [slices, rows, cols] array, box
// [1, box_rows, 64] with 128-byte swizzle.  Returns false (and sets `why`) on failure.
struct TmapStorage { alignas(64) unsigned char bytes[128]; };
bool make_tmap_bf16(TmapStorage* out, const void* base, uint64_t cols, uint64_t rows, uint64_t slices,
                    uint32_t box_rows, const char** why);
// Same box over an array whose rows are `row_pitch` elements apart and whose slices `slice_pitch` elements
// (token-major [rows, slices, cols]: row_pitch = slices * cols, slice_pitch = cols).
bool make_tmap_bf16_strided(TmapStorage* out, const void* base, uint64_t cols, uint64_t rows, uint64_t slices,
                            uint64_t row_pitch, uint64_t slice_pitch, uint32_t box_rows, const char** why);

}  // namespace ttk

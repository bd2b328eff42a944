/*
 * tt_attn.h -- C ABI of the B200 (sm_100a) attention kernels for TinyTensor.
 *
 * This is the boundary a host framework binds: plain pointers and sizes, no C++ or
 * torch types.  The reference project (TinyTensor) reaches its GPU code through C++
 * free functions over `TinyTensor<T>` bound with pybind11; each entry point below names
 * the reference interface it sits under.  Paths are relative to the reference project
 * root (`Task3/Tinytensor/`).
 *
 * Conventions
 *   - All tensors are dense row-major, contiguous: q/out/dout/dq `[B,H,S,D]`,
 *     k/v/dk/dv `[B,H,L,D]`, lse `[B,H,S]` (float, natural log of the softmax
 *     denominator including the row maximum).
 *   - Pointers are DEVICE pointers unless the function name ends in `_host`.
 *   - `stream` is a `cudaStream_t` passed as `void*`; calls are asynchronous on it.
 *   - `scale <= 0` selects `1/sqrt(D)`.
 *   - causal: query i attends to keys j <= i + (L - S) (bottom-right aligned);
 *     causal with L < S is rejected (some rows would have no key).
 *   - Every function returns a `tt_status`; none throws or aborts.  A human-readable
 *     message for the last failure on the calling thread is at `tt_last_error()`.
 *   - There is no CPU path: a call on a machine without a usable sm_100 device returns
 *     TT_ERR_BAD_DEVICE.
 */
#ifndef TT_ATTN_H
#define TT_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef enum tt_status {
    TT_OK = 0,
    TT_ERR_NULL = 1,        /* a required pointer is null */
    TT_ERR_BAD_SHAPE = 2,   /* non-positive extent, unsupported head dim, causal with L < S */
    TT_ERR_BAD_DTYPE = 3,
    TT_ERR_BAD_DEVICE = 4,  /* no CUDA device, or not compute capability 10.x */
    TT_ERR_WORKSPACE = 5,   /* workspace missing or smaller than *_workspace_bytes() */
    TT_ERR_CUDA = 6,        /* a CUDA runtime/driver call failed */
    TT_ERR_TIMEOUT = 7,     /* a bounded device-side wait expired (reported after a sync) */
    TT_ERR_UNSUPPORTED = 8,
    TT_ERR_NCCL = 9         /* the NCCL library is missing, or one of its calls failed */
} tt_status;

typedef enum tt_dtype { TT_F32 = 0, TT_BF16 = 1 } tt_dtype;

/* Problem description shared by every entry point. */
typedef struct tt_attn_desc {
    int32_t B, H;     /* batch, heads: B*H independent slices */
    int32_t S;        /* queries per slice */
    int32_t L;        /* keys/values per slice */
    int32_t D;        /* head dim: 1..256 (tensor-core path: 64 or 128, bf16) */
    int32_t dtype;    /* tt_dtype of q,k,v,out and gradients */
    int32_t causal;   /* 0 / 1 */
    float scale;      /* <= 0 -> 1/sqrt(D) */
    int32_t Hkv;      /* key/value heads; 0 or H: one per query head.  Hkv < H (H % Hkv == 0) is grouped
                       * (GQA / MQA) attention: k, v, dk, dv are [B,Hkv,L,D] and query head h reads
                       * key/value head h / (H/Hkv); dk, dv are summed over the group.  No counterpart
                       * in the reference. */
} tt_attn_desc;

/* ---- forward -------------------------------------------------------------------------
 * out = softmax(scale * q k^T [+ causal mask]) v, lse = log sum exp of the scaled scores.
 * Replaces the composition MatMul/Transpose/MulScalar/EWiseAdd/Exp/Summation/Reshape/
 * BroadcastTo/EWiseDiv/MatMul of optimizer/operators.py:194-199,234-242,289-298,323-340,
 * 348-380,388-408,416-429,464-470, and on the native side the cudaGemm + SoftmaxForward
 * sequence of src/Layers_kernels.cu:10-30 and src/Layers.cu:324-349.
 * `lse` may be null when no backward will follow.  Needs no workspace. */
int tt_attn_fwd(const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                void* out, float* lse, void* stream);

/* ---- backward ------------------------------------------------------------------------
 * dq, dk, dv of sum(out * dout); `out` and `lse` are the forward's results.
 * Replaces the reverse sweep of optimizer/autodiff.py:33-61 over the gradient methods of
 * the ops listed above (operators.py:198-199,241-242,296-298,338-340,356-358,373-380,
 * 400-408,421-429,469-470).
 * Workspace: tt_attn_bwd_workspace_bytes() bytes of device memory, 256-byte aligned;
 * contents on entry are ignored. */
size_t tt_attn_bwd_workspace_bytes(const tt_attn_desc* desc);
int tt_attn_bwd(const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                const void* out, const float* lse, const void* dout,
                void* dq, void* dk, void* dv,
                void* workspace, size_t workspace_bytes, void* stream);

/* The tensor-core backward (bf16, D = 64 or 128) exists twice.  Two passes (dk/dv with the keys resident,
 * then dq with the queries resident and the scores recomputed): seven GEMMs per tile pair, no atomics,
 * every result bit-reproducible.  One pass that produces dk, dv and dq together (five GEMMs), dq through
 * fp32 additions into the workspace; those arrive in no fixed order, so dq repeats to fp32 rounding (a few
 * 1e-7 relative) rather than bit for bit.  on = 0 (default): whichever measured faster for the shape (one
 * pass at D = 64, two passes at D = 128).  on = 1: always the two passes.  Process-wide; no counterpart in
 * the reference, whose NumPy reverse sweep (optimizer/autodiff.py:33-61) is deterministic and
 * single-threaded. */
int tt_attn_bwd_set_deterministic(int on);

/* ---- single-query decode (S == 1) ----------------------------------------------------
 * The memory-bound case: every K and V row is streamed once.  Same mathematics as
 * tt_attn_fwd with S == 1, no mask.  bf16 at D = 128 or 64 with up to 16 query heads per key/value
 * head runs a tensor-core kernel whose accumulator rows are the keys (K and V tiles by TMA,
 * the group's query heads as 16 B-operand rows, one CTA per (key/value slice, key range));
 * other shapes a split-KV kernel with 16-byte loads.  With more than one key range per slice
 * a second small kernel merges the partial results.
 * Workspace: tt_attn_decode_workspace_bytes() bytes (partials), 256-byte aligned.
 * `lse` may be null. */
size_t tt_attn_decode_workspace_bytes(const tt_attn_desc* desc);
int tt_attn_decode(const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                   void* out, float* lse, void* workspace, size_t workspace_bytes, void* stream);

/* Decode for callers that cannot allocate device memory.  No counterpart in the reference:
 * it exists for hosts that run with a frozen memory map -- a real-time serving loop that
 * pre-allocated everything at start-up and may not touch the allocator again, or a plugin sandbox
 * whose policy forbids cudaMalloc -- and therefore cannot supply the partials workspace
 * tt_attn_decode wants.  It always runs the split-KV kernels named above (tt_attn_decode prefers the
 * tensor-core decode kernel), so its results match tt_attn_decode within the bf16
 * tolerance, bit for bit where both take the same
 * kernels; the split-KV partials go to an 8 MiB array built into the library's device image (each
 * GPU that loads the library keeps those 8 MiB until the process exits).  The call itself performs
 * no cudaMalloc/cudaFree and calls no allocating library routine; q, k, v, out (and lse) are still the caller's.
 *   - bf16, D = 64 or 128, S = 1 only; problems whose partials exceed the array are refused
 *     with TT_ERR_WORKSPACE and a message naming both sizes (B*H*(D+2)*4*splits bytes; e.g.
 *     B*H up to ~4000 slices at D = 128 with 4 key ranges each).
 *   - The first call on each device looks up the array's device address (one runtime query);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the previous call
 *     left; nothing in it needs clearing because each call overwrites every partial it
 *     later reads.  Two calls that overlap on the GPU (different streams) race on it:
 *     serialise them. */
int tt_attn_decode_static(const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                          void* out, float* lse, void* stream);

/* ---- padded batches -------------------------------------------------------------------------
 * tt_attn_fwd / tt_attn_bwd with a key padding length per batch entry (no counterpart in the
 * reference): kv_lens is a device array of B int32; batch entry b attends to its first kv_lens[b]
 * keys (clamped to 1..L), the rest of its k, v rows is padding.  dk, dv rows of padded keys are
 * zero.  Query rows are all computed (give padded queries a zero dout).  The causal mask keeps its
 * alignment to the full L.  Padding rows must hold finite values (zeros are customary): a masked
 * probability of exactly 0 still meets them in the P.V and dS.K products.  kv_lens == NULL is the
 * unpadded call. */
int tt_attn_fwd_padded(const tt_attn_desc* desc, const void* q, const void* k, const void* v, const int32_t* kv_lens,
                       void* out, float* lse, void* stream);
int tt_attn_bwd_padded(const tt_attn_desc* desc, const void* q, const void* k, const void* v, const int32_t* kv_lens,
                       const void* out, const float* lse, const void* dout, void* dq, void* dk, void* dv,
                       void* workspace, size_t workspace_bytes, void* stream);

/* ---- packed variable-length batches ----------------------------------------------------------
 * n_seq sequences of different lengths stored back to back, token-major, without padding (no counterpart
 * in the reference, whose tensors are dense [B,H,S,D], src/TinyTensor.h:14-17): q, out, dout, dq are
 * [total_q, H, D]; k, v, dk, dv [total_k, Hkv, D]; lse [H, total_q].  cu_q, cu_k: device arrays of
 * n_seq + 1 int32, cumulative token counts (cu[0] = 0, cu[n_seq] = total): sequence b owns query tokens
 * [cu_q[b], cu_q[b+1]) and key tokens [cu_k[b], cu_k[b+1]).  max_q, max_k: upper bounds of the longest
 * sequence (host values: they size the launch; the kernels read the real lengths from cu_q / cu_k).
 * Every sequence is its own attention problem with the conventions above (causal: bottom-right aligned
 * per sequence; a row that sees no key -- an empty key sequence, or causal with fewer keys than queries --
 * gets out = 0, lse = -inf and zero gradients).  bf16 with D = 64 or 128 only (tensor-core kernels);
 * anything else returns TT_ERR_UNSUPPORTED.  The backward runs the two-pass kernels (bit-reproducible);
 * workspace: tt_attn_bwd_varlen_workspace_bytes(), 256-byte aligned. */
typedef struct tt_varlen_desc {
    int32_t n_seq, H, Hkv;   /* Hkv: 0 or H, or a divisor of H (grouped heads) */
    int32_t D, dtype, causal;
    float scale;             /* <= 0 -> 1/sqrt(D) */
    int32_t max_q, max_k;
    int64_t total_q, total_k;
} tt_varlen_desc;
int tt_attn_fwd_varlen(const tt_varlen_desc* desc, const void* q, const void* k, const void* v, const int32_t* cu_q,
                       const int32_t* cu_k, void* out, float* lse, void* stream);
size_t tt_attn_bwd_varlen_workspace_bytes(const tt_varlen_desc* desc);
int tt_attn_bwd_varlen(const tt_varlen_desc* desc, const void* q, const void* k, const void* v, const int32_t* cu_q,
                       const int32_t* cu_k, const void* out, const float* lse, const void* dout, void* dq, void* dk,
                       void* dv, void* workspace, size_t workspace_bytes, void* stream);

/* ---- decode over a paged and/or ragged key/value cache -----------------------------------
 * tt_attn_decode for serving-style caches (no counterpart in the reference).  bf16, D = 64 or
 * 128, S = 1; desc->L is the longest sequence any batch entry may have.
 *   block_table != NULL: k_pool, v_pool are page pools [pages, Hkv, page_size, D]; key r of batch
 *       entry b is row r % page_size of page block_table[b * max_pages + r / page_size]
 *       (device array of B * max_pages int32); page_size * max_pages >= L.
 *   block_table == NULL: k_pool, v_pool are dense [B, Hkv, L, D] as in tt_attn_decode.
 *   seq_lens != NULL: device array of B int32, batch entry b attends to its first seq_lens[b]
 *       keys (clamped to 0..L); an entry with no keys gets out = 0 and lse = -inf.
 * Grouped heads (desc->Hkv < H) read each key/value row once for the whole group: groups of up to
 * 16 on the tensor-core decode kernel, as in tt_attn_decode, larger ones on the tensor-core forward
 * kernel.  Over a paged cache the tensor-core
 * kernels need a page_size that divides 128 or is a multiple of it (>= 8) and gather the pages by
 * TMA; other page sizes take the split-KV kernel.  Rows that no sequence owns never reach the
 * result and may hold anything.  Workspace: tt_attn_decode_workspace_bytes(desc). */
int tt_attn_decode_paged(const tt_attn_desc* desc, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_table, const int32_t* seq_lens, int32_t page_size, int32_t max_pages,
                         void* out, float* lse, void* workspace, size_t workspace_bytes, void* stream);

/* ---- row softmax ------------------------------------------------------------------------
 * out[r,:] = softmax(in[r,:]) over `cols`, row maximum subtracted; rows = product of the leading
 * axes.  One launch that reads and writes every element once; replaces SoftmaxForward of
 * src/Layers.cu:324-349 with its five launches and per-row Thrust loops
 * (src/Layers_kernels.cu:189-257).  The backward, dx = y * (dy - sum(dy*y)), has no native
 * counterpart in the reference (its NumPy form is the Softmax part of optimizer/operators.py:
 * 610-626).  dtype: TT_F32 or TT_BF16 (fp32 arithmetic either way). */
int tt_softmax_fwd(const void* in, void* out, int64_t rows, int32_t cols, int32_t dtype, void* stream);
int tt_softmax_bwd(const void* y, const void* dy, void* dx, int64_t rows, int32_t cols, int32_t dtype, void* stream);

/* ---- fully connected layer ------------------------------------------------------------------
 * y[rows,out] = x[rows,in] . w[in,out] + bias[out]  (bias may be NULL), all row-major; replaces
 * FcForward of src/Layers.cu:9-40 (cublasSgemm through a handle created and destroyed per call
 * plus a rank-1 GEMM for the bias, src/Layers_kernels.cu:10-30).  tt_fc_bwd replaces FcBackward
 * of src/Layers.cu:42-79: dx = dy . w^T, dw = x^T . dy, db = column sums of dy (db_scalar != 0:
 * one value, the sum over all of dy, for the reference's single-value bias); each of dx, dw, db
 * may be NULL and is then skipped.  bf16 with in % 8 == 0 and out % 8 == 0 runs the tcgen05
 * kernel (fp32 accumulation), float and other shapes an fp32 SIMT kernel; tt_fc_path says
 * which (1 = tensor cores).  The workspace is only needed for db. */
int tt_fc_fwd(const void* x, const void* w, const void* bias, void* y, int64_t rows, int32_t in_features,
              int32_t out_features, int32_t dtype, void* stream);
size_t tt_fc_bwd_workspace_bytes(int64_t rows, int32_t in_features, int32_t out_features, int32_t dtype);
int tt_fc_bwd(const void* x, const void* w, const void* dy, void* dx, void* dw, void* db, int32_t db_scalar, int64_t rows,
              int32_t in_features, int32_t out_features, int32_t dtype, void* workspace, size_t workspace_bytes,
              void* stream);
int tt_fc_path(int64_t rows, int32_t in_features, int32_t out_features, int32_t dtype);

/* ---- host-buffer calls (what the reference's Python ops do around each native op:
 * upload NumPy -> run -> download, optimizer/operators.py:502-512) ----------------------
 * Pointers are HOST pointers (pinned memory gives the best copy rate).  Device buffers
 * come from the pool below; the call uploads, runs, downloads and synchronises. */
int tt_attn_fwd_host(const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                     void* out, float* lse);
int tt_attn_bwd_host(const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                     const void* out, const float* lse, const void* dout,
                     void* dq, void* dk, void* dv);
int tt_attn_decode_host(const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                        void* out, float* lse);
/* One training step from host buffers: forward and backward of every slice, with the slices cut
 * into chunks that flow through an upload stream, a compute stream and a download stream, so
 * the PCIe transfers of both directions overlap the kernels (use pinned host memory; with
 * pageable memory the copies serialise).  What the Python autograd op does in two calls
 * (compute, then gradient with the tensors kept on the device, optimizer/operators.py:498-527
 * pattern of the reference) in one.  `lse` may be null. */
int tt_attn_fwd_bwd_host(const tt_attn_desc* desc, const void* q, const void* k, const void* v, const void* dout,
                         void* out, float* lse, void* dq, void* dk, void* dv);

/* ---- pooled device storage -----------------------------------------------------------
 * Replaces the per-object cudaMalloc/cudaFree of src/Tinytensor.cu:17-22,85-93: freed
 * blocks go to size-bucketed free lists of the current device and are reused. */
int tt_alloc(size_t bytes, void** out_ptr);
int tt_free(void* ptr);   /* does not synchronise: free a block only after the work that uses it has completed */
/* Host storage of the tensor class goes through the library too (plain malloc/free underneath), so that
 * the two rules below cover host and device buffers alike. */
int tt_host_alloc(size_t bytes, void** out_ptr);
int tt_host_free(void* ptr);
/* Shared ownership for zero-copy views (DLPack exports of the tensor class, src/bind_Tensor.cpp of the
 * reference has no such export): while a buffer is retained, tt_free / tt_host_free of it only mark it;
 * the block goes back to the pool (or the heap) when the last holder releases it.  So a tensor may be
 * resized, moved between host and device or destroyed while a view of its old buffer is alive. */
int tt_buffer_retain(void* ptr);
int tt_buffer_release(void* ptr);
int tt_pool_trim(void);                                     /* return cached blocks to the driver */
int tt_pool_stats(size_t* bytes_in_use, size_t* bytes_cached, uint64_t* n_driver_allocs);

/* ---- sharding of the B*H independent slices over ranks -------------------------------
 * Contiguous ranges, remainder spread over the first ranks; pure host arithmetic.
 * (The reference has no multi-GPU path; Task2/mnist.py:53-54 is torch DataParallel.) */
int tt_shard_range(int64_t n_slices, int32_t world, int32_t rank, int64_t* begin, int64_t* count);

/* ---- several GPUs: one process (or thread) per GPU, slices sharded, outputs all-gathered -------
 * The B*H slices are independent in forward and backward, so rank r of `world` owns the contiguous
 * range tt_shard_range(B*H, world, r) of them, keeps q, k, v, out, lse and the gradients of that
 * range in its own memory, and runs the single-GPU kernels on it; nothing crosses between GPUs on the
 * data path.  The one exchange is the all-gather that gives every rank the full `out` (and, if asked
 * for, full gradients): because [B,H,S,D] is contiguous in the slice index, each rank's shard is one
 * contiguous block of the full tensor and a single ncclAllGather lands it in place, no repacking.
 * The communicator owns one ncclComm_t and one side stream on its device: gathers run on the side
 * stream, ordered behind the kernels that produce their data, so the gather of `out` overlaps the
 * backward.  NCCL is bound at run time (dlopen of libnccl.so.2, or the library TT_NCCL_LIB names);
 * no kernel of this library reads another GPU's memory.
 * No counterpart in the reference, whose only multi-GPU construct is torch's nn.DataParallel around
 * a PyTorch model (Task2/mnist.py:53-54).
 *
 *   tt_mgpu_unique_id   rank 0 calls it and hands the TT_MGPU_ID_BYTES bytes to every rank by its own
 *                       means (a file, a socket, MPI, torch.distributed).
 *   tt_mgpu_init        collective over the ranks; binds the communicator to the CURRENT device.
 *   tt_mgpu_attn_fwd    desc describes the WHOLE problem (all B*H slices); the tensor arguments are this
 *                       rank's shard ([count,S,D] / [count/group,L,D] / [count,S]).  out_full, if not
 *                       null, is [B*H,S,D] on this device and receives every rank's out.
 *                       B*H must divide evenly by world, and a shard must hold whole groups of query
 *                       heads, else TT_ERR_UNSUPPORTED.  Kernels run on `stream`; returns at once.
 *   tt_mgpu_attn_bwd    same for the backward; dq_full / dk_full / dv_full (each may be null) receive
 *                       the all-gathered gradients, otherwise gradients stay with their owners.
 *                       Workspace: tt_mgpu_bwd_workspace_bytes(comm, desc), 256-byte aligned.
 *   tt_mgpu_wait        makes `stream` wait (on the device) for every gather issued so far.
 *   tt_mgpu_destroy     collective; frees the communicator, the side stream and the events. */
#define TT_MGPU_ID_BYTES 128
typedef struct tt_mgpu* tt_mgpu_t;
int tt_mgpu_unique_id(void* id_bytes);
int tt_mgpu_init(tt_mgpu_t* comm, int32_t world, int32_t rank, const void* id_bytes);
int tt_mgpu_destroy(tt_mgpu_t comm);
int tt_mgpu_shard(tt_mgpu_t comm, const tt_attn_desc* desc, int64_t* first_slice, int64_t* n_slices);
int tt_mgpu_attn_fwd(tt_mgpu_t comm, const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                     void* out, float* lse, void* out_full, void* stream);
size_t tt_mgpu_bwd_workspace_bytes(tt_mgpu_t comm, const tt_attn_desc* desc);
int tt_mgpu_attn_bwd(tt_mgpu_t comm, const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                     const void* out, const float* lse, const void* dout, void* dq, void* dk, void* dv,
                     void* dq_full, void* dk_full, void* dv_full, void* workspace, size_t workspace_bytes, void* stream);
int tt_mgpu_wait(tt_mgpu_t comm, void* stream);

/* ---- diagnostics ---------------------------------------------------------------------*/
const char* tt_last_error(void);
/* Number of kernels this library has launched in this process (for launch accounting). */
uint64_t tt_kernel_launch_count(void);
/* Name of the kernel family the given problem dispatches to: "tcgen05" or "simt". */
const char* tt_attn_fwd_path(const tt_attn_desc* desc);
const char* tt_attn_bwd_path(const tt_attn_desc* desc);
/* Reads (and clears) the device-side status word after synchronising `stream`:
 * TT_OK, or TT_ERR_TIMEOUT with details in tt_last_error(). */
int tt_check_device_status(void* stream);

/* Optional per-kernel timing: while enabled, every kernel launch of this library is
 * bracketed by CUDA events on its launching stream.  tt_profile_read() waits for the
 * recorded events and returns the accumulated device time and launch count of one kernel
 * family (ids 0 .. tt_profile_kernel_count()-1, names from tt_profile_kernel_name()). */
int tt_profile_enable(int on);
int tt_profile_reset(void);
int tt_profile_kernel_count(void);
const char* tt_profile_kernel_name(int kernel_id);
int tt_profile_read(int kernel_id, double* total_ms, uint64_t* launches);

/* Launches a one-warp kernel whose only wait can never be satisfied and whose wait budget is
 * `budget_cycles` SM cycles (at most 4e9).  The wait expires, the kernel returns normally, and the
 * next tt_check_device_status() reports TT_ERR_TIMEOUT (barrier id 99, iteration 7) and clears
 * the status word: a way to test the failure-reporting path without faulting or hanging a GPU. */
int tt_debug_wait_timeout(int64_t budget_cycles, void* stream);

/* Building-block self test of the tensor-core plumbing (TMA load -> tcgen05.mma from
 * shared memory -> tcgen05.ld, tcgen05.st -> tcgen05.mma with A in tensor memory and an
 * MN-major B).  a,b: bf16 [128,128] row-major; vt: bf16 [128,D] row-major (D = 64|128).
 * Outputs: s = a b^T as float [128,128]; o = bf16(s) vt as float [128,D]. */
int tt_debug_umma_probe(const void* a, const void* b, const void* vt, int32_t D,
                        float* s_out, float* o_out, void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* TT_ATTN_H */

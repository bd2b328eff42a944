/*
 * tt_debug.h -- tuning aids of libtt_attn.so that are not part of the boundary a host framework binds
 * (include/tt_attn.h).  Exported for the tuning scripts only; signatures may change.
 */
#ifndef TT_DEBUG_H
#define TT_DEBUG_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* While `device_buf` (3*64*8 int64, device memory) is non-null, CTA number `block` of every forward
 * launch records clock64() at its hand-off points (softmax warpgroups: wait for S, S loaded, max known,
 * P half/whole written; MMA issuer: waits and issues) for its work item number `item`, and a start
 * stamp for each of its first 64 items.  Pass null to switch it off. */
int tt_debug_fwd_trace(void* device_buf, int32_t block, int32_t item);
/* Same for the tensor-core backward; pass = 1 traces the dK/dV launch of the two-pass kernels, 2 their dQ
 * launch, 3 the single-pass kernel. */
int tt_debug_bwd_trace(void* device_buf, int32_t block, int32_t pass);

/* A failure made on the host, for tests of the error exits of the host-buffer calls (tt_attn_*_host):
 * the (checks+1)-th CUDA runtime result those calls inspect from now on is reported as cudaErrorUnknown
 * although the runtime call was made and succeeded, so the entry point returns TT_ERR_CUDA in the middle
 * of its sequence with copies and kernels still queued.  Nothing fails on the device.  Negative = off;
 * the countdown disarms itself once it has fired.  Process-wide: not for use beside concurrent callers. */
int tt_debug_fail_host_call_after(int64_t checks);
/* How many times a host-buffer call has synchronised its streams on the way out before handing its
 * pooled device buffers back (every exit, successful or not, does). */
int64_t tt_debug_guard_syncs(void);

/* The collective calls tt_mgpu_* makes, as a table, so that a test can put stand-ins in their place
 * (each returns an ncclResult_t value: 0 = success).  tt_mgpu_set_collectives(NULL) restores the NCCL
 * library's own entry points; communicators made under one table must be destroyed under it. */
typedef struct tt_mgpu_collectives {
    int (*get_unique_id)(void* id_bytes);
    int (*comm_init_rank)(void** comm, int world, const void* id_bytes, int rank);
    int (*comm_destroy)(void* comm);
    /* dtype: 1 = bf16, 0 = float */
    int (*all_gather)(const void* send, void* recv, size_t count, int dtype, void* comm, void* stream);
    const char* (*error_string)(int result);
} tt_mgpu_collectives;
int tt_mgpu_set_collectives(const tt_mgpu_collectives* table);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* TT_DEBUG_H */

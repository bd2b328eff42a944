// Several GPUs, one rank each: the (batch, head) slices are sharded over the ranks, every rank runs the
// single-GPU kernels on its shard, and NCCL all-gathers the outputs on a side stream the communicator
// owns.  See the tt_mgpu_* block of include/tt_attn.h.  NCCL is bound at run time through its public C
// ABI (dlopen), so the library has no link-time dependency on it and a test can substitute the calls.
#include "../../include/tt_attn.h"
#include "tt_debug.h"
#include "common.h"

#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <mutex>

namespace ttk {
namespace {

// ---- the NCCL entry points used, by their public prototypes (nccl.h: ncclUniqueId is 128 bytes passed by
// value, ncclDataType_t ncclFloat32 = 7, ncclBfloat16 = 9, ncclSuccess = 0)
struct NcclId { char internal[TT_MGPU_ID_BYTES]; };
typedef int (*GetUniqueIdFn)(NcclId*);
typedef int (*CommInitRankFn)(void**, int, NcclId, int);
typedef int (*CommDestroyFn)(void*);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef const char* (*ErrorStringFn)(int);

struct NcclLib {
    void* handle = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    AllGatherFn all_gather = nullptr;
    ErrorStringFn error_string = nullptr;
    char why[256] = "";
};
NcclLib* nccl_lib() {
    static NcclLib lib;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[3] = {getenv("TT_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            if (!n || !*n) continue;
            lib.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (lib.handle) break;
            snprintf(lib.why, sizeof(lib.why), "%s", dlerror());
        }
        if (!lib.handle) return;
        lib.get_unique_id = (GetUniqueIdFn)dlsym(lib.handle, "ncclGetUniqueId");
        lib.comm_init_rank = (CommInitRankFn)dlsym(lib.handle, "ncclCommInitRank");
        lib.comm_destroy = (CommDestroyFn)dlsym(lib.handle, "ncclCommDestroy");
        lib.all_gather = (AllGatherFn)dlsym(lib.handle, "ncclAllGather");
        lib.error_string = (ErrorStringFn)dlsym(lib.handle, "ncclGetErrorString");
        if (!lib.get_unique_id || !lib.comm_init_rank || !lib.comm_destroy || !lib.all_gather || !lib.error_string) {
            snprintf(lib.why, sizeof(lib.why), "the NCCL library lacks one of ncclGetUniqueId, ncclCommInitRank, "
                     "ncclCommDestroy, ncclAllGather, ncclGetErrorString");
            lib.handle = nullptr;
        }
    });
    return &lib;
}

// the default table: thin adapters onto the library
int real_get_unique_id(void* id) { return nccl_lib()->get_unique_id(reinterpret_cast<NcclId*>(id)); }
int real_comm_init_rank(void** comm, int world, const void* id, int rank) {
    NcclId v;
    memcpy(&v, id, sizeof(v));
    return nccl_lib()->comm_init_rank(comm, world, v, rank);
}
int real_comm_destroy(void* comm) { return nccl_lib()->comm_destroy(comm); }
int real_all_gather(const void* send, void* recv, size_t count, int dtype, void* comm, void* stream) {
    return nccl_lib()->all_gather(send, recv, count, dtype ? 9 : 7, comm, (cudaStream_t)stream);
}
const char* real_error_string(int r) { return nccl_lib()->error_string(r); }
const tt_mgpu_collectives kRealTable = {real_get_unique_id, real_comm_init_rank, real_comm_destroy, real_all_gather,
                                        real_error_string};

std::mutex g_table_mu;
tt_mgpu_collectives g_table;
bool g_table_is_stub = false;

// The table in force; *rc = TT_OK, or TT_ERR_NCCL (message set) when NCCL itself is needed and missing.
const tt_mgpu_collectives* table(int* rc) {
    std::lock_guard<std::mutex> lk(g_table_mu);
    *rc = TT_OK;
    if (g_table_is_stub) return &g_table;
    NcclLib* lib = nccl_lib();
    if (!lib->handle) {
        *rc = fail(TT_ERR_NCCL, "the NCCL library could not be loaded (%s); set TT_NCCL_LIB to its path", lib->why);
        return nullptr;
    }
    return &kRealTable;
}
int nccl_fail(const tt_mgpu_collectives* t, int r, const char* what) {
    const char* s = (t && t->error_string) ? t->error_string(r) : nullptr;
    return fail(TT_ERR_NCCL, "%s: NCCL result %d (%s)", what, r, s ? s : "?");
}

}  // namespace
}  // namespace ttk

using namespace ttk;

struct tt_mgpu {
    void* comm = nullptr;
    int world = 1, rank = 0, device = -1;
    cudaStream_t side = nullptr;
    cudaEvent_t produced = nullptr;   // recorded on the caller's stream behind the kernels whose output is gathered
    cudaEvent_t gathered = nullptr;   // recorded on the side stream behind the gathers
    bool gathers_pending = false;
    tt_mgpu_collectives calls;
};

namespace {
// this rank's shard of the problem `d` describes; fills the shard-local descriptor
int shard_of(const tt_mgpu* c, const tt_attn_desc* d, const char* who, tt_attn_desc* local, int64_t* first, int64_t* count) {
    if (!c) return fail(TT_ERR_NULL, "%s: communicator is null", who);
    if (!d) return fail(TT_ERR_NULL, "%s: desc is null", who);
    if (d->B < 1 || d->H < 1) return fail(TT_ERR_BAD_SHAPE, "%s: B=%d H=%d must be >= 1", who, d->B, d->H);
    const int hkv = d->Hkv > 0 ? d->Hkv : d->H;
    if (hkv > d->H || d->H % hkv != 0) return fail(TT_ERR_BAD_SHAPE, "%s: Hkv=%d must divide H=%d", who, d->Hkv, d->H);
    const int group = d->H / hkv;
    const int64_t n = (int64_t)d->B * d->H;
    if (n % c->world != 0)
        return fail(TT_ERR_UNSUPPORTED, "%s: %lld slices do not divide evenly over %d ranks", who, (long long)n, c->world);
    const int64_t per = n / c->world;
    if (per % group != 0)
        return fail(TT_ERR_UNSUPPORTED, "%s: a shard of %lld query heads would split a group of %d that shares key/value heads",
                    who, (long long)per, group);
    if (per > 0x7fffffffLL) return fail(TT_ERR_BAD_SHAPE, "%s: shard too large", who);
    *first = per * c->rank;
    *count = per;
    *local = *d;
    local->B = 1;
    local->H = (int32_t)per;
    local->Hkv = (int32_t)(per / group);
    return TT_OK;
}
int on_device(const tt_mgpu* c, const char* who) {
    int rc = check_device();
    if (rc != TT_OK) return rc;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, who);
    if (dev != c->device)
        return fail(TT_ERR_BAD_DEVICE, "%s: the communicator belongs to device %d, the current device is %d", who, c->device, dev);
    return TT_OK;
}
// orders the side stream behind `stream` and all-gathers `count` elements per rank
int gather(tt_mgpu* c, const void* send, void* recv, size_t count, int bf16, cudaStream_t stream, const char* who) {
    cudaError_t e = cudaEventRecord(c->produced, stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->side, c->produced, 0);
    if (e != cudaSuccess) return cuda_fail(e, who);
    const int r = c->calls.all_gather(send, recv, count, bf16, c->comm, (void*)c->side);
    if (r != 0) return nccl_fail(&c->calls, r, who);
    c->gathers_pending = true;
    return TT_OK;
}
}  // namespace

extern "C" {

int tt_mgpu_set_collectives(const tt_mgpu_collectives* t) {
    std::lock_guard<std::mutex> lk(g_table_mu);
    if (!t) {
        g_table_is_stub = false;
        return TT_OK;
    }
    if (!t->get_unique_id || !t->comm_init_rank || !t->comm_destroy || !t->all_gather)
        return fail(TT_ERR_NULL, "tt_mgpu_set_collectives: a table entry is null");
    g_table = *t;
    g_table_is_stub = true;
    return TT_OK;
}

int tt_mgpu_unique_id(void* id_bytes) {
    if (!id_bytes) return fail(TT_ERR_NULL, "tt_mgpu_unique_id: id_bytes is null");
    int rc;
    const tt_mgpu_collectives* t = table(&rc);
    if (!t) return rc;
    const int r = t->get_unique_id(id_bytes);
    if (r != 0) return nccl_fail(t, r, "tt_mgpu_unique_id");
    return TT_OK;
}

int tt_mgpu_init(tt_mgpu_t* out, int32_t world, int32_t rank, const void* id_bytes) {
    if (!out || !id_bytes) return fail(TT_ERR_NULL, "tt_mgpu_init: null argument");
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world) return fail(TT_ERR_BAD_SHAPE, "tt_mgpu_init: world=%d rank=%d", world, rank);
    int rc;
    const tt_mgpu_collectives* t = table(&rc);
    if (!t) return rc;
    // Under a stand-in table a communicator may exist on a machine without a GPU (host-side tests of
    // the sharding rules and the error mapping); it has no stream, and its attention calls fail with
    // TT_ERR_BAD_DEVICE like every other entry point there.
    const bool have_device = check_device() == TT_OK;
    if (!have_device && t == &kRealTable) return check_device();
    tt_mgpu* c = new tt_mgpu();
    c->calls = *t;
    c->world = world;
    c->rank = rank;
    cudaError_t e = cudaSuccess;
    if (have_device) {
        e = cudaGetDevice(&c->device);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->produced, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->gathered, cudaEventDisableTiming);
    }
    rc = TT_OK;
    if (e != cudaSuccess) {
        rc = cuda_fail(e, "tt_mgpu_init");
    } else {
        const int r = c->calls.comm_init_rank(&c->comm, world, id_bytes, rank);
        if (r != 0) rc = nccl_fail(&c->calls, r, "tt_mgpu_init: ncclCommInitRank");
    }
    if (rc != TT_OK) {
        if (c->gathered) cudaEventDestroy(c->gathered);
        if (c->produced) cudaEventDestroy(c->produced);
        if (c->side) cudaStreamDestroy(c->side);
        delete c;
        return rc;
    }
    *out = c;
    return TT_OK;
}

int tt_mgpu_destroy(tt_mgpu_t c) {
    if (!c) return TT_OK;
    int rc = TT_OK;
    if (c->side) {
        cudaError_t e = cudaStreamSynchronize(c->side);   // no gather of ours may be in flight when the communicator goes
        if (e != cudaSuccess) rc = cuda_fail(e, "tt_mgpu_destroy: synchronize");
    }
    if (c->comm) {
        const int r = c->calls.comm_destroy(c->comm);
        if (r != 0 && rc == TT_OK) rc = nccl_fail(&c->calls, r, "tt_mgpu_destroy: ncclCommDestroy");
    }
    if (c->gathered) cudaEventDestroy(c->gathered);
    if (c->produced) cudaEventDestroy(c->produced);
    if (c->side) cudaStreamDestroy(c->side);
    delete c;
    return rc;
}

int tt_mgpu_shard(tt_mgpu_t c, const tt_attn_desc* desc, int64_t* first_slice, int64_t* n_slices) {
    if (!first_slice || !n_slices) return fail(TT_ERR_NULL, "tt_mgpu_shard: null output");
    tt_attn_desc local;
    return shard_of(c, desc, "tt_mgpu_shard", &local, first_slice, n_slices);
}

int tt_mgpu_attn_fwd(tt_mgpu_t c, const tt_attn_desc* desc, const void* q, const void* k, const void* v, void* out,
                     float* lse, void* out_full, void* stream) {
    tt_attn_desc local;
    int64_t first, count;
    int rc = shard_of(c, desc, "tt_mgpu_attn_fwd", &local, &first, &count);
    if (rc != TT_OK) return rc;
    if ((rc = on_device(c, "tt_mgpu_attn_fwd")) != TT_OK) return rc;
    if ((rc = tt_attn_fwd(&local, q, k, v, out, lse, stream)) != TT_OK) return rc;
    if (out_full) {
        const size_t n = (size_t)count * (size_t)desc->S * (size_t)desc->D;
        return gather(c, out, out_full, n, desc->dtype == TT_BF16, (cudaStream_t)stream, "tt_mgpu_attn_fwd: all-gather of out");
    }
    return TT_OK;
}

size_t tt_mgpu_bwd_workspace_bytes(tt_mgpu_t c, const tt_attn_desc* desc) {
    tt_attn_desc local;
    int64_t first, count;
    if (shard_of(c, desc, "tt_mgpu_bwd_workspace_bytes", &local, &first, &count) != TT_OK) return 0;
    return tt_attn_bwd_workspace_bytes(&local);
}

int tt_mgpu_attn_bwd(tt_mgpu_t c, const tt_attn_desc* desc, const void* q, const void* k, const void* v, const void* out,
                     const float* lse, const void* dout, void* dq, void* dk, void* dv, void* dq_full, void* dk_full,
                     void* dv_full, void* workspace, size_t workspace_bytes, void* stream) {
    tt_attn_desc local;
    int64_t first, count;
    int rc = shard_of(c, desc, "tt_mgpu_attn_bwd", &local, &first, &count);
    if (rc != TT_OK) return rc;
    if ((rc = on_device(c, "tt_mgpu_attn_bwd")) != TT_OK) return rc;
    if ((rc = tt_attn_bwd(&local, q, k, v, out, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream)) != TT_OK) return rc;
    const int bf16 = desc->dtype == TT_BF16;
    const size_t nq = (size_t)count * (size_t)desc->S * (size_t)desc->D;
    const size_t nk = (size_t)local.Hkv * (size_t)desc->L * (size_t)desc->D;
    if (dq_full && (rc = gather(c, dq, dq_full, nq, bf16, (cudaStream_t)stream, "tt_mgpu_attn_bwd: all-gather of dq")) != TT_OK) return rc;
    if (dk_full && (rc = gather(c, dk, dk_full, nk, bf16, (cudaStream_t)stream, "tt_mgpu_attn_bwd: all-gather of dk")) != TT_OK) return rc;
    if (dv_full && (rc = gather(c, dv, dv_full, nk, bf16, (cudaStream_t)stream, "tt_mgpu_attn_bwd: all-gather of dv")) != TT_OK) return rc;
    return TT_OK;
}

int tt_mgpu_wait(tt_mgpu_t c, void* stream) {
    if (!c) return fail(TT_ERR_NULL, "tt_mgpu_wait: communicator is null");
    if (!c->gathers_pending) return TT_OK;
    cudaError_t e = cudaEventRecord(c->gathered, c->side);
    if (e == cudaSuccess) e = cudaStreamWaitEvent((cudaStream_t)stream, c->gathered, 0);
    if (e != cudaSuccess) return cuda_fail(e, "tt_mgpu_wait");
    c->gathers_pending = false;
    return TT_OK;
}

}  // extern "C"

// C-ABI layer: argument validation, dispatch to the kernel families, pooled device
// storage, tensor-map construction, error reporting.  See include/tt_attn.h.
#include "../../include/tt_attn.h"
#include "tt_debug.h"
#include "common.h"
#include "attn_bwd_common.cuh"
#include "sched_slots.h"

#include <cuda.h>
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace ttk {

// ------------------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";
int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
int cuda_fail(cudaError_t e, const char* what) {
    return fail(TT_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

static std::atomic<uint64_t> g_launches{0};

// ------------------------------------------------------------------------------ per-kernel event timing
static const char* const kKernelNames[K_COUNT] = {
    "attn_fwd_sm100", "attn_fwd_simt", "attn_bwd_prep", "attn_bwd_sm100_dkv", "attn_bwd_sm100_dq",
    "attn_bwd_simt_delta", "attn_bwd_simt_dq", "attn_bwd_simt_dkv", "attn_decode", "attn_decode_merge",
    "umma_probe", "softmax_rows_fwd", "softmax_rows_bwd", "fc_gemm_sm100", "fc_gemm_simt",
    "fc_colsum", "attn_bwd_fused_sm100", "attn_bwd_dq_convert", "attn_decode_gq_sm100"};
struct TimedLaunch {
    KernelId id;
    cudaEvent_t start, stop;
};
static std::atomic<int> g_timing_on{0};
static std::mutex g_timing_mu;
static std::vector<TimedLaunch*> g_pending;          // recorded, not yet read back
static std::vector<TimedLaunch*> g_free_records;     // events are reused
static double g_total_ms[K_COUNT];
static uint64_t g_timed_launches[K_COUNT];

LaunchScope::LaunchScope(KernelId id_, cudaStream_t st_, bool allow_timing) : id(id_), st(st_), rec(nullptr) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (!allow_timing || !g_timing_on.load(std::memory_order_relaxed)) return;
    TimedLaunch* r = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_timing_mu);
        if (!g_free_records.empty()) {
            r = g_free_records.back();
            g_free_records.pop_back();
        }
    }
    if (!r) {
        r = new TimedLaunch();
        if (cudaEventCreate(&r->start) != cudaSuccess || cudaEventCreate(&r->stop) != cudaSuccess) {
            delete r;
            return;
        }
    }
    r->id = id;
    cudaEventRecord(r->start, st);
    rec = r;
}
LaunchScope::~LaunchScope() {
    if (!rec) return;
    TimedLaunch* r = static_cast<TimedLaunch*>(rec);
    cudaEventRecord(r->stop, st);
    std::lock_guard<std::mutex> lk(g_timing_mu);
    g_pending.push_back(r);
}

// ------------------------------------------------------------------------------ device status word
__device__ unsigned int g_device_status[4];
static std::mutex g_status_mu;
static std::unordered_map<int, unsigned int*> g_status_ptr;
unsigned int* device_status_word() {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_status_mu);
    auto it = g_status_ptr.find(dev);
    if (it != g_status_ptr.end()) return it->second;
    unsigned int* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_device_status) != cudaSuccess) p = nullptr;
    if (p) cudaMemset(p, 0, 4 * sizeof(unsigned int));
    g_status_ptr[dev] = p;
    return p;
}

// ------------------------------------------------------------------------------ work-item counters
// One set of counters and events per device.  The events exist from the first use of a device on, so a
// launch itself creates nothing.
constexpr int kSchedSlots = 64;
__device__ unsigned int g_sched_counters[kSchedSlots];
namespace {
struct DevSlots {
    SlotRing ring{kSchedSlots};
    cudaEvent_t ev[kSchedSlots] = {};
    unsigned int* base = nullptr;
    cudaError_t init_err = cudaSuccess;
};
std::mutex g_slots_mu;
std::unordered_map<int, DevSlots*> g_slots;
DevSlots* slots_for_current_device() {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_slots_mu);
    auto it = g_slots.find(dev);
    if (it != g_slots.end()) return it->second;
    DevSlots* d = new DevSlots();
    d->init_err = cudaGetSymbolAddress((void**)&d->base, g_sched_counters);
    for (int i = 0; i < kSchedSlots && d->init_err == cudaSuccess; ++i)
        d->init_err = cudaEventCreateWithFlags(&d->ev[i], cudaEventDisableTiming);
    g_slots[dev] = d;
    return d;
}
}  // namespace
cudaError_t sched_counter_acquire(cudaStream_t st, SchedCounter* c) {
    DevSlots* d = slots_for_current_device();
    if (d->init_err != cudaSuccess) return d->init_err;
    bool must_wait = false;
    const int s = d->ring.acquire([&](int i) { return cudaEventQuery(d->ev[i]) == cudaErrorNotReady; }, &must_wait);
    cudaError_t e = cudaSuccess;
    // the launch that last used this counter is still running: this one goes behind it
    if (must_wait) e = cudaStreamWaitEvent(st, d->ev[s], 0);
    if (e == cudaSuccess) e = cudaMemsetAsync(d->base + s, 0, sizeof(unsigned int), st);
    if (e != cudaSuccess) {
        d->ring.release(s);
        return e;
    }
    c->ptr = d->base + s;
    c->slot = s;
    return cudaSuccess;
}
void sched_counter_release(const SchedCounter& c, cudaStream_t st) {
    if (c.slot < 0) return;
    DevSlots* d = slots_for_current_device();
    cudaEventRecord(d->ev[c.slot], st);
    d->ring.release(c.slot);
}

// ------------------------------------------------------------------------------ device check
int check_device() {
    static thread_local int cached_dev = -1;
    static thread_local int cached_ok = 0;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(TT_ERR_BAD_DEVICE, "no usable CUDA device: %s", cudaGetErrorString(e));
    if (dev == cached_dev && cached_ok) return TT_OK;
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return fail(TT_ERR_BAD_DEVICE, "cannot query device %d: %s", dev, cudaGetErrorString(e));
    if (major != 10)
        return fail(TT_ERR_BAD_DEVICE, "device %d has compute capability %d.x; these kernels are built for sm_100a only",
                    dev, major);
    cached_dev = dev;
    cached_ok = 1;
    return TT_OK;
}

// ------------------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

bool make_tmap_bf16(TmapStorage* out, const void* base, uint64_t cols, uint64_t rows, uint64_t slices,
                    uint32_t box_rows, const char** why) {
    return make_tmap_bf16_strided(out, base, cols, rows, slices, cols, cols * rows, box_rows, why);
}

bool make_tmap_bf16_strided(TmapStorage* out, const void* base, uint64_t cols, uint64_t rows, uint64_t slices,
                            uint64_t row_pitch, uint64_t slice_pitch, uint32_t box_rows, const char** why) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        *why = "cuTensorMapEncodeTiled entry point not available";
        fail(TT_ERR_CUDA, "%s", *why);
        return false;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_pitch * 2) % 16 != 0 || (slice_pitch * 2) % 16 != 0) {
        *why = "tensor base or row pitch not 16-byte aligned";
        fail(TT_ERR_BAD_SHAPE, "%s", *why);
        return false;
    }
    cuuint64_t gdim[3] = {cols, rows, slices};
    cuuint64_t gstride[2] = {row_pitch * 2, slice_pitch * 2};
    cuuint32_t box[3] = {64, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap*>(out->bytes), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                    const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        *why = "cuTensorMapEncodeTiled failed";
        fail(TT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (cols=%llu rows=%llu slices=%llu)", (int)r,
             (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)slices);
        return false;
    }
    return true;
}

// ------------------------------------------------------------------------------ pooled storage
struct Pool {
    std::mutex mu;
    std::map<size_t, std::vector<void*>> free_by_size;   // bucket size -> cached blocks
    std::unordered_map<void*, size_t> live;               // ptr -> bucket size
    size_t in_use = 0, cached = 0;
    uint64_t driver_allocs = 0;
};
static std::mutex g_pools_mu;
static std::unordered_map<int, Pool*> g_pools;
static Pool* pool_for_current_device() {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_pools_mu);
    auto it = g_pools.find(dev);
    if (it != g_pools.end()) return it->second;
    Pool* p = new Pool();
    g_pools[dev] = p;
    return p;
}
// Buffers with live views (tt_buffer_retain): pointer -> holders, and what a free that arrived meanwhile
// asked for (0 nothing, 1 back to this pool, 2 host free).
struct Retained {
    int holders = 0;
    int pending = 0;
    Pool* pool = nullptr;
};
static std::mutex g_retained_mu;
static std::unordered_map<void*, Retained> g_retained;
// true: the buffer has holders, the free was recorded and must not happen now
static bool defer_free(void* ptr, int kind, Pool* pool) {
    std::lock_guard<std::mutex> lk(g_retained_mu);
    auto it = g_retained.find(ptr);
    if (it == g_retained.end() || it->second.holders <= 0) return false;
    it->second.pending = kind;
    it->second.pool = pool;
    return true;
}

// Buckets: powers of two up to 1 MiB, multiples of 2 MiB above.
static size_t bucket_of(size_t n) {
    if (n <= 512) return 512;
    if (n <= (1u << 20)) {
        size_t b = 512;
        while (b < n) b <<= 1;
        return b;
    }
    const size_t g = (size_t)2 << 20;
    return (n + g - 1) / g * g;
}

}  // namespace ttk

using namespace ttk;

extern "C" {

const char* tt_last_error(void) { return g_err; }
uint64_t tt_kernel_launch_count(void) { return g_launches.load(); }

int tt_alloc(size_t bytes, void** out_ptr) {
    if (!out_ptr) return fail(TT_ERR_NULL, "tt_alloc: out_ptr is null");
    *out_ptr = nullptr;
    if (bytes == 0) return TT_OK;
    Pool* pool = pool_for_current_device();
    const size_t b = bucket_of(bytes);
    {
        std::lock_guard<std::mutex> lk(pool->mu);
        auto it = pool->free_by_size.find(b);
        if (it != pool->free_by_size.end() && !it->second.empty()) {
            void* p = it->second.back();
            it->second.pop_back();
            pool->cached -= b;
            pool->in_use += b;
            pool->live[p] = b;
            *out_ptr = p;
            return TT_OK;
        }
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, b);
    if (e == cudaErrorMemoryAllocation) {   // give cached blocks back and retry once
        cudaGetLastError();
        tt_pool_trim();
        e = cudaMalloc(&p, b);
    }
    if (e != cudaSuccess) return cuda_fail(e, "tt_alloc: cudaMalloc");
    std::lock_guard<std::mutex> lk(pool->mu);
    pool->driver_allocs++;
    pool->in_use += b;
    pool->live[p] = b;
    *out_ptr = p;
    return TT_OK;
}

static int pool_put_back(Pool* pool, void* ptr) {
    std::lock_guard<std::mutex> lk(pool->mu);
    auto it = pool->live.find(ptr);
    if (it == pool->live.end()) return fail(TT_ERR_NULL, "tt_free: pointer %p was not allocated by tt_alloc on this device", ptr);
    size_t b = it->second;
    pool->live.erase(it);
    pool->in_use -= b;
    pool->cached += b;
    pool->free_by_size[b].push_back(ptr);
    return TT_OK;
}

int tt_host_alloc(size_t bytes, void** out_ptr) {
    if (!out_ptr) return fail(TT_ERR_NULL, "tt_host_alloc: out_ptr is null");
    *out_ptr = nullptr;
    if (bytes == 0) return TT_OK;
    void* p = malloc(bytes);
    if (!p) return fail(TT_ERR_CUDA, "tt_host_alloc: out of host memory (%zu bytes)", bytes);
    *out_ptr = p;
    return TT_OK;
}
int tt_host_free(void* ptr) {
    if (!ptr) return TT_OK;
    if (defer_free(ptr, 2, nullptr)) return TT_OK;
    free(ptr);
    return TT_OK;
}
int tt_buffer_retain(void* ptr) {
    if (!ptr) return TT_OK;
    std::lock_guard<std::mutex> lk(g_retained_mu);
    g_retained[ptr].holders += 1;
    return TT_OK;
}
int tt_buffer_release(void* ptr) {
    if (!ptr) return TT_OK;
    Retained r;
    {
        std::lock_guard<std::mutex> lk(g_retained_mu);
        auto it = g_retained.find(ptr);
        if (it == g_retained.end()) return fail(TT_ERR_NULL, "tt_buffer_release: pointer %p is not retained", ptr);
        if (--it->second.holders > 0) return TT_OK;
        r = it->second;
        g_retained.erase(it);
    }
    if (r.pending == 1) return pool_put_back(r.pool, ptr);   // the free that arrived while views were alive
    if (r.pending == 2) free(ptr);
    return TT_OK;
}

int tt_free(void* ptr) {
    if (!ptr) return TT_OK;
    Pool* pool = pool_for_current_device();
    if (defer_free(ptr, 1, pool)) return TT_OK;
    std::lock_guard<std::mutex> lk(pool->mu);
    auto it = pool->live.find(ptr);
    if (it == pool->live.end()) return fail(TT_ERR_NULL, "tt_free: pointer %p was not allocated by tt_alloc on this device", ptr);
    size_t b = it->second;
    pool->live.erase(it);
    pool->in_use -= b;
    pool->cached += b;
    pool->free_by_size[b].push_back(ptr);
    return TT_OK;
}

int tt_pool_trim(void) {
    Pool* pool = pool_for_current_device();
    std::vector<void*> victims;
    {
        std::lock_guard<std::mutex> lk(pool->mu);
        for (auto& kv : pool->free_by_size)
            for (void* p : kv.second) victims.push_back(p);
        pool->free_by_size.clear();
        pool->cached = 0;
    }
    for (void* p : victims) cudaFree(p);
    return TT_OK;
}

int tt_pool_stats(size_t* bytes_in_use, size_t* bytes_cached, uint64_t* n_driver_allocs) {
    Pool* pool = pool_for_current_device();
    std::lock_guard<std::mutex> lk(pool->mu);
    if (bytes_in_use) *bytes_in_use = pool->in_use;
    if (bytes_cached) *bytes_cached = pool->cached;
    if (n_driver_allocs) *n_driver_allocs = pool->driver_allocs;
    return TT_OK;
}

int tt_shard_range(int64_t n_slices, int32_t world, int32_t rank, int64_t* begin, int64_t* count) {
    if (!begin || !count) return fail(TT_ERR_NULL, "tt_shard_range: null output");
    if (n_slices < 0 || world < 1 || rank < 0 || rank >= world)
        return fail(TT_ERR_BAD_SHAPE, "tt_shard_range: n_slices=%lld world=%d rank=%d", (long long)n_slices, world, rank);
    int64_t base = n_slices / world, rem = n_slices % world;
    *begin = rank * base + (rank < rem ? rank : rem);
    *count = base + (rank < rem ? 1 : 0);
    return TT_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------ validation
namespace ttk {
int resolve(const tt_attn_desc* d, AttnArgs* a, const char* who) {
    if (!d) return fail(TT_ERR_NULL, "%s: desc is null", who);
    if (d->B < 1 || d->H < 1 || d->S < 1 || d->L < 1)
        return fail(TT_ERR_BAD_SHAPE, "%s: B=%d H=%d S=%d L=%d must all be >= 1", who, d->B, d->H, d->S, d->L);
    if (d->D < 1 || d->D > 256) return fail(TT_ERR_BAD_SHAPE, "%s: head dim D=%d outside 1..256", who, d->D);
    if (d->dtype != TT_F32 && d->dtype != TT_BF16) return fail(TT_ERR_BAD_DTYPE, "%s: dtype %d unknown", who, d->dtype);
    if (d->causal && d->L < d->S)
        return fail(TT_ERR_BAD_SHAPE, "%s: causal with L=%d < S=%d leaves query rows without keys", who, d->L, d->S);
    if (!std::isfinite(d->scale)) return fail(TT_ERR_BAD_SHAPE, "%s: scale is not finite", who);
    const int hkv = d->Hkv > 0 ? d->Hkv : d->H;
    if (hkv > d->H || d->H % hkv != 0)
        return fail(TT_ERR_BAD_SHAPE, "%s: Hkv=%d must divide H=%d", who, d->Hkv, d->H);
    memset(a, 0, sizeof(*a));
    a->BH = (long long)d->B * d->H;
    a->group = d->H / hkv;
    a->H = d->H;
    a->kv_lens = nullptr;
    a->S = d->S;
    a->L = d->L;
    a->D = d->D;
    a->causal = d->causal ? 1 : 0;
    a->bf16 = d->dtype == TT_BF16;
    a->scale = d->scale > 0.f ? d->scale : 1.0f / sqrtf((float)d->D);
    long long nblk = ((long long)(d->S > d->L ? d->S : d->L) + 31) / 32;
    if (a->BH * nblk >= (1LL << 31)) return fail(TT_ERR_BAD_SHAPE, "%s: problem too large for a 1-D grid", who);
    return TT_OK;
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
}  // namespace ttk

extern "C" {

const char* tt_attn_fwd_path(const tt_attn_desc* desc) {
    AttnArgs a;
    if (resolve(desc, &a, "tt_attn_fwd_path") != TT_OK) return "invalid";
    return attn_fwd_sm100_supported(a) ? "tcgen05" : "simt";
}
const char* tt_attn_bwd_path(const tt_attn_desc* desc) {
    AttnArgs a;
    if (resolve(desc, &a, "tt_attn_bwd_path") != TT_OK) return "invalid";
    return attn_bwd_sm100_supported(a) ? "tcgen05" : "simt";
}

static int attn_fwd_common(const char* who, const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                           const int32_t* kv_lens, void* out, float* lse, void* stream) {
    AttnArgs a;
    int rc = resolve(desc, &a, who);
    if (rc != TT_OK) return rc;
    if (!q || !k || !v || !out) return fail(TT_ERR_NULL, "%s: q, k, v and out must be non-null", who);
    if ((rc = check_device()) != TT_OK) return rc;
    g_err[0] = 0;
    a.q = q; a.k = k; a.v = v; a.out = out; a.lse = lse;
    a.kv_lens = kv_lens;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (attn_fwd_sm100_supported(a) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out)) {
        e = attn_fwd_sm100(a, st);
        if (e == cudaErrorInvalidValue && g_err[0]) return TT_ERR_CUDA;
    } else {
        e = attn_fwd_simt(a, st);
    }
    if (e != cudaSuccess) return cuda_fail(e, who);
    return TT_OK;
}
int tt_attn_fwd(const tt_attn_desc* desc, const void* q, const void* k, const void* v, void* out, float* lse,
                void* stream) {
    return attn_fwd_common("tt_attn_fwd", desc, q, k, v, nullptr, out, lse, stream);
}
int tt_attn_fwd_padded(const tt_attn_desc* desc, const void* q, const void* k, const void* v, const int32_t* kv_lens,
                       void* out, float* lse, void* stream) {
    return attn_fwd_common("tt_attn_fwd_padded", desc, q, k, v, kv_lens, out, lse, stream);
}

int tt_attn_bwd_set_deterministic(int on) {
    attn_bwd_set_deterministic(on);
    return TT_OK;
}

size_t tt_attn_bwd_workspace_bytes(const tt_attn_desc* desc) {
    AttnArgs a;
    if (resolve(desc, &a, "tt_attn_bwd_workspace_bytes") != TT_OK) return 0;
    size_t simt = attn_bwd_simt_workspace(a);
    size_t tc = attn_bwd_sm100_supported(a) ? attn_bwd_sm100_workspace(a) : 0;
    return simt > tc ? simt : tc;
}

static int attn_bwd_common(const char* who, const tt_attn_desc* desc, const void* q, const void* k, const void* v,
                           const int32_t* kv_lens, const void* out, const float* lse, const void* dout, void* dq, void* dk,
                           void* dv, void* workspace, size_t workspace_bytes, void* stream) {
    AttnArgs a;
    int rc = resolve(desc, &a, who);
    if (rc != TT_OK) return rc;
    if (!q || !k || !v || !out || !lse || !dout || !dq || !dk || !dv)
        return fail(TT_ERR_NULL, "%s: all tensor pointers must be non-null", who);
    size_t need = tt_attn_bwd_workspace_bytes(desc);
    if (!workspace || workspace_bytes < need)
        return fail(TT_ERR_WORKSPACE, "%s: workspace of %zu bytes required, %zu given", who, need, workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return fail(TT_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned", who);
    if ((rc = check_device()) != TT_OK) return rc;
    g_err[0] = 0;
    a.q = q; a.k = k; a.v = v; a.out = const_cast<void*>(out); a.lse = const_cast<float*>(lse); a.dout = dout;
    a.dq = dq; a.dk = dk; a.dv = dv;
    a.kv_lens = kv_lens;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    bool al = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(dout) && aligned16(dq) &&
              aligned16(dk) && aligned16(dv);
    if (attn_bwd_sm100_supported(a) && al) {
        e = attn_bwd_sm100(a, workspace, st);
        if (e == cudaErrorInvalidValue && g_err[0]) return TT_ERR_CUDA;
    } else {
        e = attn_bwd_simt(a, (float*)workspace, st);
    }
    if (e != cudaSuccess) return cuda_fail(e, who);
    return TT_OK;
}
int tt_attn_bwd(const tt_attn_desc* desc, const void* q, const void* k, const void* v, const void* out,
                const float* lse, const void* dout, void* dq, void* dk, void* dv, void* workspace,
                size_t workspace_bytes, void* stream) {
    return attn_bwd_common("tt_attn_bwd", desc, q, k, v, nullptr, out, lse, dout, dq, dk, dv, workspace, workspace_bytes,
                           stream);
}
int tt_attn_bwd_padded(const tt_attn_desc* desc, const void* q, const void* k, const void* v, const int32_t* kv_lens,
                       const void* out, const float* lse, const void* dout, void* dq, void* dk, void* dv,
                       void* workspace, size_t workspace_bytes, void* stream) {
    return attn_bwd_common("tt_attn_bwd_padded", desc, q, k, v, kv_lens, out, lse, dout, dq, dk, dv, workspace,
                           workspace_bytes, stream);
}

// ---- packed variable-length batches
static int resolve_varlen(const tt_varlen_desc* d, AttnArgs* a, const char* who) {
    if (!d) return fail(TT_ERR_NULL, "%s: desc is null", who);
    if (d->n_seq < 1 || d->H < 1 || d->max_q < 1 || d->max_k < 1 || d->total_q < 1 || d->total_k < 1)
        return fail(TT_ERR_BAD_SHAPE, "%s: n_seq=%d H=%d max_q=%d max_k=%d total_q=%lld total_k=%lld must all be >= 1", who,
                    d->n_seq, d->H, d->max_q, d->max_k, (long long)d->total_q, (long long)d->total_k);
    if (d->max_q > d->total_q || d->max_k > d->total_k)
        return fail(TT_ERR_BAD_SHAPE, "%s: the longest sequence (%d / %d) cannot exceed the token totals", who, d->max_q, d->max_k);
    if (d->total_q >= (1LL << 31) || d->total_k >= (1LL << 31))
        return fail(TT_ERR_BAD_SHAPE, "%s: more than 2^31-1 tokens", who);
    if (d->dtype != TT_F32 && d->dtype != TT_BF16) return fail(TT_ERR_BAD_DTYPE, "%s: dtype %d unknown", who, d->dtype);
    if (d->dtype != TT_BF16 || !(d->D == 64 || d->D == 128))
        return fail(TT_ERR_UNSUPPORTED, "%s: packed batches run on the tensor-core kernels only: bf16 with D = 64 or 128 "
                    "(got dtype %d, D=%d)", who, d->dtype, d->D);
    if (!std::isfinite(d->scale)) return fail(TT_ERR_BAD_SHAPE, "%s: scale is not finite", who);
    const int hkv = d->Hkv > 0 ? d->Hkv : d->H;
    if (hkv > d->H || d->H % hkv != 0) return fail(TT_ERR_BAD_SHAPE, "%s: Hkv=%d must divide H=%d", who, d->Hkv, d->H);
    memset(a, 0, sizeof(*a));
    a->BH = (long long)d->n_seq * d->H;
    a->group = d->H / hkv;
    a->H = d->H;
    a->S = d->max_q;
    a->L = d->max_k;
    a->D = d->D;
    a->causal = d->causal ? 1 : 0;
    a->bf16 = 1;
    a->scale = d->scale > 0.f ? d->scale : 1.0f / sqrtf((float)d->D);
    a->total_q = d->total_q;
    a->total_k = d->total_k;
    const long long tiles = ((long long)std::max(d->max_q, d->max_k) + 127) / 128;
    if (a->BH * tiles >= (1LL << 31)) return fail(TT_ERR_BAD_SHAPE, "%s: problem too large for the work-item numbering", who);
    return TT_OK;
}

int tt_attn_fwd_varlen(const tt_varlen_desc* desc, const void* q, const void* k, const void* v, const int32_t* cu_q,
                       const int32_t* cu_k, void* out, float* lse, void* stream) {
    AttnArgs a;
    int rc = resolve_varlen(desc, &a, "tt_attn_fwd_varlen");
    if (rc != TT_OK) return rc;
    if (!q || !k || !v || !out || !cu_q || !cu_k)
        return fail(TT_ERR_NULL, "tt_attn_fwd_varlen: q, k, v, out, cu_q and cu_k must be non-null");
    if (!(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out)))
        return fail(TT_ERR_BAD_SHAPE, "tt_attn_fwd_varlen: q, k, v, out must be 16-byte aligned");
    if ((rc = check_device()) != TT_OK) return rc;
    g_err[0] = 0;
    a.q = q; a.k = k; a.v = v; a.out = out; a.lse = lse;
    a.cu_q = cu_q; a.cu_k = cu_k;
    cudaError_t e = attn_fwd_sm100(a, (cudaStream_t)stream);
    if (e == cudaErrorInvalidValue && g_err[0]) return TT_ERR_CUDA;
    if (e != cudaSuccess) return cuda_fail(e, "tt_attn_fwd_varlen");
    return TT_OK;
}

size_t tt_attn_bwd_varlen_workspace_bytes(const tt_varlen_desc* desc) {
    AttnArgs a;
    if (resolve_varlen(desc, &a, "tt_attn_bwd_varlen_workspace_bytes") != TT_OK) return 0;
    static const int one = 0;
    a.cu_q = a.cu_k = &one;   // marks the packed layout for the size computation; never dereferenced
    return attn_bwd_sm100_workspace(a);
}

int tt_attn_bwd_varlen(const tt_varlen_desc* desc, const void* q, const void* k, const void* v, const int32_t* cu_q,
                       const int32_t* cu_k, const void* out, const float* lse, const void* dout, void* dq, void* dk,
                       void* dv, void* workspace, size_t workspace_bytes, void* stream) {
    AttnArgs a;
    int rc = resolve_varlen(desc, &a, "tt_attn_bwd_varlen");
    if (rc != TT_OK) return rc;
    if (!q || !k || !v || !out || !lse || !dout || !dq || !dk || !dv || !cu_q || !cu_k)
        return fail(TT_ERR_NULL, "tt_attn_bwd_varlen: all tensor pointers, cu_q and cu_k must be non-null");
    if (!(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(dout) && aligned16(dq) && aligned16(dk) &&
          aligned16(dv)))
        return fail(TT_ERR_BAD_SHAPE, "tt_attn_bwd_varlen: tensors must be 16-byte aligned");
    const size_t need = tt_attn_bwd_varlen_workspace_bytes(desc);
    if (!workspace || workspace_bytes < need)
        return fail(TT_ERR_WORKSPACE, "tt_attn_bwd_varlen: workspace of %zu bytes required, %zu given", need, workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return fail(TT_ERR_WORKSPACE, "tt_attn_bwd_varlen: workspace must be 256-byte aligned");
    if ((rc = check_device()) != TT_OK) return rc;
    g_err[0] = 0;
    a.q = q; a.k = k; a.v = v; a.out = const_cast<void*>(out); a.lse = const_cast<float*>(lse); a.dout = dout;
    a.dq = dq; a.dk = dk; a.dv = dv;
    a.cu_q = cu_q; a.cu_k = cu_k;
    cudaError_t e = attn_bwd_two_pass(a, workspace, (cudaStream_t)stream);
    if (e == cudaErrorInvalidValue && g_err[0]) return TT_ERR_CUDA;
    if (e != cudaSuccess) return cuda_fail(e, "tt_attn_bwd_varlen");
    return TT_OK;
}

size_t tt_attn_decode_workspace_bytes(const tt_attn_desc* desc) {
    AttnArgs a;
    if (resolve(desc, &a, "tt_attn_decode_workspace_bytes") != TT_OK) return 0;
    if (a.S != 1) return 0;
    // enough for every route a call with this descriptor can take (dense, paged or ragged)
    const size_t w1 = attn_decode_plan(a, true).ws_bytes, w2 = attn_decode_plan(a, false).ws_bytes;
    size_t w3 = 0;
    {   // the paged route on the forward kernel (its split depends on the shape only; page size 128 stands in)
        static const int one_page = 0;
        DecodeView v;
        v.block_table = &one_page;
        v.page_size = 128;
        v.max_pages = (a.L + 127) / 128;
        v.hkv = desc->Hkv > 0 ? desc->Hkv : desc->H;
        attn_decode_paged_on_forward(a, v, &w3);
    }
    return std::max(w1, std::max(w2, w3));
}

int tt_attn_decode(const tt_attn_desc* desc, const void* q, const void* k, const void* v, void* out, float* lse,
                   void* workspace, size_t workspace_bytes, void* stream) {
    AttnArgs a;
    int rc = resolve(desc, &a, "tt_attn_decode");
    if (rc != TT_OK) return rc;
    if (a.S != 1) return fail(TT_ERR_BAD_SHAPE, "tt_attn_decode: S must be 1, got %d", a.S);
    if (!q || !k || !v || !out) return fail(TT_ERR_NULL, "tt_attn_decode: q, k, v and out must be non-null");
    if ((rc = check_device()) != TT_OK) return rc;
    a.causal = 0;   // a single query aligned bottom-right sees every key
    DecodePlan pl = attn_decode_plan(a);
    if (pl.ws_bytes > 0) {
        if (!workspace || workspace_bytes < pl.ws_bytes)
            return fail(TT_ERR_WORKSPACE, "tt_attn_decode: workspace of %zu bytes required, %zu given", pl.ws_bytes,
                        workspace_bytes);
        if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
            return fail(TT_ERR_WORKSPACE, "tt_attn_decode: workspace must be 256-byte aligned");
    }
    if (a.bf16 && (a.D == 64 || a.D == 128) && !(aligned16(q) && aligned16(k) && aligned16(v)))
        return fail(TT_ERR_BAD_SHAPE, "tt_attn_decode: q, k, v must be 16-byte aligned");
    a.q = q; a.k = k; a.v = v; a.out = out; a.lse = lse;
    cudaError_t e = attn_decode(a, pl, workspace, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "tt_attn_decode: launch");
    return TT_OK;
}

int tt_attn_decode_static(const tt_attn_desc* desc, const void* q, const void* k, const void* v, void* out,
                          float* lse, void* stream) {
    AttnArgs a;
    int rc = resolve(desc, &a, "tt_attn_decode_static");
    if (rc != TT_OK) return rc;
    if (a.S != 1) return fail(TT_ERR_BAD_SHAPE, "tt_attn_decode_static: S must be 1, got %d", a.S);
    if (!(a.bf16 && (a.D == 64 || a.D == 128)))
        return fail(TT_ERR_UNSUPPORTED, "tt_attn_decode_static: bf16 with head dim 64 or 128 only (got dtype %d, D=%d)",
                    desc->dtype, a.D);
    if (!q || !k || !v || !out) return fail(TT_ERR_NULL, "tt_attn_decode_static: q, k, v and out must be non-null");
    if (!(aligned16(q) && aligned16(k) && aligned16(v)))
        return fail(TT_ERR_BAD_SHAPE, "tt_attn_decode_static: q, k, v must be 16-byte aligned");
    if ((rc = check_device()) != TT_OK) return rc;
    a.causal = 0;
    DecodePlan pl = attn_decode_plan(a, /*allow_tc=*/false);   // this entry point is the SIMT kernel on the fixed array
    a.q = q; a.k = k; a.v = v; a.out = out; a.lse = lse;
    bool too_big = false;
    cudaError_t e = attn_decode_static(a, pl, (cudaStream_t)stream, &too_big);
    if (too_big)
        return fail(TT_ERR_WORKSPACE,
                    "tt_attn_decode_static: this problem needs %zu bytes of partials but the built-in scratch array "
                    "holds %zu; use tt_attn_decode with a caller-provided workspace", pl.ws_bytes,
                    attn_decode_static_capacity());
    if (e != cudaSuccess) return cuda_fail(e, "tt_attn_decode_static");
    return TT_OK;
}

static int softmax_args(const char* who, const void* a, const void* out, int64_t rows, int32_t cols, int32_t dtype) {
    if ((!a || !out) && rows != 0) return fail(TT_ERR_NULL, "%s: null pointer", who);
    if (rows < 0 || cols < 1) return fail(TT_ERR_BAD_SHAPE, "%s: rows=%lld cols=%d", who, (long long)rows, cols);
    if (rows >= (1LL << 31)) return fail(TT_ERR_BAD_SHAPE, "%s: more than 2^31-1 rows", who);
    if (dtype != TT_F32 && dtype != TT_BF16) return fail(TT_ERR_BAD_DTYPE, "%s: dtype %d unknown", who, dtype);
    return check_device();
}
int tt_softmax_fwd(const void* in, void* out, int64_t rows, int32_t cols, int32_t dtype, void* stream) {
    int rc = softmax_args("tt_softmax_fwd", in, out, rows, cols, dtype);
    if (rc != TT_OK || rows == 0) return rc;
    cudaError_t e = softmax_rows_fwd(in, out, rows, cols, dtype == TT_BF16, (cudaStream_t)stream);
    return e == cudaSuccess ? TT_OK : cuda_fail(e, "tt_softmax_fwd: launch");
}
int tt_softmax_bwd(const void* y, const void* dy, void* dx, int64_t rows, int32_t cols, int32_t dtype, void* stream) {
    int rc = softmax_args("tt_softmax_bwd", y, dx, rows, cols, dtype);
    if (rc != TT_OK || rows == 0) return rc;
    if (!dy) return fail(TT_ERR_NULL, "tt_softmax_bwd: null pointer");
    cudaError_t e = softmax_rows_bwd(y, dy, dx, rows, cols, dtype == TT_BF16, (cudaStream_t)stream);
    return e == cudaSuccess ? TT_OK : cuda_fail(e, "tt_softmax_bwd: launch");
}

static int fc_args(const char* who, int64_t rows, int32_t in_f, int32_t out_f, int32_t dtype) {
    if (rows < 0 || in_f < 1 || out_f < 1)
        return fail(TT_ERR_BAD_SHAPE, "%s: rows=%lld in_features=%d out_features=%d", who, (long long)rows, in_f, out_f);
    if (rows >= (1LL << 31)) return fail(TT_ERR_BAD_SHAPE, "%s: more than 2^31-1 rows", who);
    if (dtype != TT_F32 && dtype != TT_BF16) return fail(TT_ERR_BAD_DTYPE, "%s: dtype %d unknown", who, dtype);
    return check_device();
}
int tt_fc_fwd(const void* x, const void* w, const void* bias, void* y, int64_t rows, int32_t in_features,
              int32_t out_features, int32_t dtype, void* stream) {
    int rc = fc_args("tt_fc_fwd", rows, in_features, out_features, dtype);
    if (rc != TT_OK || rows == 0) return rc;
    if (!x || !w || !y) return fail(TT_ERR_NULL, "tt_fc_fwd: null pointer");
    cudaError_t e = fc_gemm(x, w, y, bias, rows, out_features, in_features, 0, 1, dtype == TT_BF16, (cudaStream_t)stream);
    return e == cudaSuccess ? TT_OK : cuda_fail(e, "tt_fc_fwd: launch");
}
size_t tt_fc_bwd_workspace_bytes(int64_t rows, int32_t in_features, int32_t out_features, int32_t dtype) {
    (void)in_features; (void)dtype;
    if (rows < 1 || out_features < 1) return 0;
    return fc_colsum_workspace(rows, out_features);
}
int tt_fc_bwd(const void* x, const void* w, const void* dy, void* dx, void* dw, void* db, int32_t db_scalar, int64_t rows,
              int32_t in_features, int32_t out_features, int32_t dtype, void* workspace, size_t workspace_bytes,
              void* stream) {
    int rc = fc_args("tt_fc_bwd", rows, in_features, out_features, dtype);
    if (rc != TT_OK) return rc;
    if (rows && (!dy || (dx && !w) || (dw && !x)))
        return fail(TT_ERR_NULL, "tt_fc_bwd: null pointer (dy always, w for dx, x for dw)");
    cudaStream_t st = (cudaStream_t)stream;
    const int bf16 = dtype == TT_BF16;
    const size_t esz = bf16 ? 2 : 4;
    if (rows == 0) {   // empty batch: the parameter gradients are zero
        cudaError_t e = cudaSuccess;
        if (dw) e = cudaMemsetAsync(dw, 0, (size_t)in_features * out_features * esz, st);
        if (e == cudaSuccess && db) e = cudaMemsetAsync(db, 0, (db_scalar ? 1 : (size_t)out_features) * esz, st);
        return e == cudaSuccess ? TT_OK : cuda_fail(e, "tt_fc_bwd: memset");
    }
    cudaError_t e = cudaSuccess;
    // dx[rows,in] = dy[rows,out] . w[in,out]^T
    if (dx) e = fc_gemm(dy, w, dx, nullptr, rows, in_features, out_features, 0, 0, bf16, st);
    // dw[in,out] = x[rows,in]^T . dy[rows,out]
    if (e == cudaSuccess && dw) e = fc_gemm(x, dy, dw, nullptr, in_features, out_features, (int)rows, 1, 1, bf16, st);
    if (e == cudaSuccess && db) {
        const size_t need = fc_colsum_workspace(rows, out_features);
        if (!workspace || workspace_bytes < need)
            return fail(TT_ERR_WORKSPACE, "tt_fc_bwd: workspace of %zu bytes needed for the bias gradient, %zu given", need,
                        workspace_bytes);
        e = fc_colsum(dy, db, rows, out_features, bf16, db_scalar != 0, workspace, st);
    }
    return e == cudaSuccess ? TT_OK : cuda_fail(e, "tt_fc_bwd: launch");
}
int tt_fc_path(int64_t rows, int32_t in_features, int32_t out_features, int32_t dtype) {
    // alignment of the pointers is checked at the call; pools and torch hand out >= 256-byte alignment
    return fc_gemm_tc_supported(nullptr, nullptr, nullptr, nullptr, rows, out_features, in_features, 0, 1, dtype == TT_BF16) &&
                   fc_gemm_tc_supported(nullptr, nullptr, nullptr, nullptr, in_features, out_features, (int)rows, 1, 1, dtype == TT_BF16)
               ? 1 : 0;
}

int tt_attn_decode_paged(const tt_attn_desc* desc, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_table, const int32_t* seq_lens, int32_t page_size, int32_t max_pages,
                         void* out, float* lse, void* workspace, size_t workspace_bytes, void* stream) {
    AttnArgs a;
    int rc = resolve(desc, &a, "tt_attn_decode_paged");
    if (rc != TT_OK) return rc;
    if (a.S != 1) return fail(TT_ERR_BAD_SHAPE, "tt_attn_decode_paged: S must be 1, got %d", a.S);
    if (!a.bf16 || !(a.D == 64 || a.D == 128))
        return fail(TT_ERR_BAD_DTYPE, "tt_attn_decode_paged: bf16 with D = 64 or 128 only (dtype %d, D %d)", desc->dtype, a.D);
    if (!q || !k_pool || !v_pool || !out) return fail(TT_ERR_NULL, "tt_attn_decode_paged: q, k, v and out must be non-null");
    if (block_table) {
        if (page_size < 1 || max_pages < 1)
            return fail(TT_ERR_BAD_SHAPE, "tt_attn_decode_paged: page_size=%d max_pages=%d must be >= 1", page_size, max_pages);
        if ((long long)page_size * max_pages < a.L)
            return fail(TT_ERR_BAD_SHAPE, "tt_attn_decode_paged: L=%d exceeds page_size*max_pages=%lld", a.L,
                        (long long)page_size * max_pages);
    }
    if (!(aligned16(q) && aligned16(k_pool) && aligned16(v_pool)))
        return fail(TT_ERR_BAD_SHAPE, "tt_attn_decode_paged: q, k, v must be 16-byte aligned");
    if ((rc = check_device()) != TT_OK) return rc;
    a.causal = 0;
    DecodeView view;
    view.block_table = block_table;
    view.seq_lens = seq_lens;
    view.page_size = page_size;
    view.max_pages = max_pages;
    view.hkv = desc->Hkv > 0 ? desc->Hkv : desc->H;
    a.q = q; a.k = k_pool; a.v = v_pool; a.out = out; a.lse = lse;
    size_t paged_ws = 0;
    if (const int splits = attn_decode_paged_on_forward(a, view, &paged_ws)) {   // grouped heads over a paged cache
        if (paged_ws > 0) {
            if (!workspace || workspace_bytes < paged_ws)
                return fail(TT_ERR_WORKSPACE, "tt_attn_decode_paged: workspace of %zu bytes required, %zu given", paged_ws,
                            workspace_bytes);
            if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
                return fail(TT_ERR_WORKSPACE, "tt_attn_decode_paged: workspace must be 256-byte aligned");
        }
        cudaError_t e = attn_decode_paged_forward(a, view, splits, workspace, (cudaStream_t)stream);
        if (e != cudaSuccess) return cuda_fail(e, "tt_attn_decode_paged: launch");
        return TT_OK;
    }
    DecodePlan pl = attn_decode_plan(a, /*allow_tc=*/!(block_table || seq_lens));
    if (pl.ws_bytes > 0) {
        if (!workspace || workspace_bytes < pl.ws_bytes)
            return fail(TT_ERR_WORKSPACE, "tt_attn_decode_paged: workspace of %zu bytes required, %zu given", pl.ws_bytes,
                        workspace_bytes);
        if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
            return fail(TT_ERR_WORKSPACE, "tt_attn_decode_paged: workspace must be 256-byte aligned");
    }
    cudaError_t e = attn_decode(a, pl, workspace, (cudaStream_t)stream, &view);
    if (e != cudaSuccess) return cuda_fail(e, "tt_attn_decode_paged: launch");
    return TT_OK;
}

int tt_debug_wait_timeout(int64_t budget_cycles, void* stream) {
    if (budget_cycles < 1 || budget_cycles > 4000000000LL)
        return fail(TT_ERR_BAD_SHAPE, "tt_debug_wait_timeout: budget of %lld cycles outside 1..4e9", (long long)budget_cycles);
    int rc = check_device();
    if (rc != TT_OK) return rc;
    cudaError_t e = wait_timeout_probe(budget_cycles, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "tt_debug_wait_timeout: launch");
    return TT_OK;
}

int tt_debug_fwd_trace(void* device_buf, int32_t block, int32_t item) {
    attn_fwd_set_trace(reinterpret_cast<long long*>(device_buf), block, item);
    return TT_OK;
}

int tt_debug_bwd_trace(void* device_buf, int32_t block, int32_t pass) {
    if (pass == 3 || device_buf == nullptr) attn_bwd_fused_set_trace(reinterpret_cast<long long*>(device_buf), block);
    if (pass != 3) attn_bwd_set_trace(reinterpret_cast<long long*>(device_buf), block, pass);
    return TT_OK;
}

int tt_profile_enable(int on) {
    g_timing_on.store(on ? 1 : 0);
    return TT_OK;
}
int tt_profile_reset(void) {
    std::lock_guard<std::mutex> lk(g_timing_mu);
    for (TimedLaunch* r : g_pending) {
        cudaEventSynchronize(r->stop);
        g_free_records.push_back(r);
    }
    g_pending.clear();
    for (int i = 0; i < K_COUNT; ++i) {
        g_total_ms[i] = 0.0;
        g_timed_launches[i] = 0;
    }
    return TT_OK;
}
int tt_profile_kernel_count(void) { return K_COUNT; }
const char* tt_profile_kernel_name(int kernel_id) {
    return (kernel_id >= 0 && kernel_id < K_COUNT) ? kKernelNames[kernel_id] : "";
}
int tt_profile_read(int kernel_id, double* total_ms, uint64_t* launches) {
    if (kernel_id < 0 || kernel_id >= K_COUNT) return fail(TT_ERR_BAD_SHAPE, "tt_profile_read: kernel id %d", kernel_id);
    std::lock_guard<std::mutex> lk(g_timing_mu);
    for (TimedLaunch* r : g_pending) {
        float ms = 0.f;
        if (cudaEventSynchronize(r->stop) == cudaSuccess && cudaEventElapsedTime(&ms, r->start, r->stop) == cudaSuccess) {
            g_total_ms[r->id] += ms;
            g_timed_launches[r->id] += 1;
        }
        g_free_records.push_back(r);
    }
    g_pending.clear();
    if (total_ms) *total_ms = g_total_ms[kernel_id];
    if (launches) *launches = g_timed_launches[kernel_id];
    return TT_OK;
}

int tt_check_device_status(void* stream) {
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "tt_check_device_status: synchronize");
    unsigned int* dptr = device_status_word();
    if (!dptr) return fail(TT_ERR_CUDA, "tt_check_device_status: status word unavailable");
    unsigned int h[4] = {0, 0, 0, 0};
    e = cudaMemcpy(h, dptr, sizeof(h), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "tt_check_device_status: copy");
    if (h[0] == 0) return TT_OK;
    cudaMemset(dptr, 0, sizeof(h));
    if ((h[0] >> 16) == 8u)   // the backward kernel found its dynamic shared memory not 1024-byte aligned and did nothing
        return fail(TT_ERR_CUDA, "kernel refused to run: dynamic shared memory base 0x%x is not 1024-byte aligned (block %u)",
                    h[2], h[0] & 0xffffu);
    return fail(TT_ERR_TIMEOUT, "a device-side wait expired: block %u, barrier id %u, iteration %u, warp %u",
                h[0] & 0xffffu, h[1], h[2], h[3]);
}

int tt_debug_umma_probe(const void* a, const void* b, const void* vt, int32_t D, float* s_out, float* o_out,
                        void* stream) {
    if (!a || !b || !vt || !s_out || !o_out) return fail(TT_ERR_NULL, "tt_debug_umma_probe: null pointer");
    if (D != 64 && D != 128) return fail(TT_ERR_BAD_SHAPE, "tt_debug_umma_probe: D must be 64 or 128");
    int rc = check_device();
    if (rc != TT_OK) return rc;
    g_err[0] = 0;
    cudaError_t e = umma_probe(a, b, vt, D, s_out, o_out, (cudaStream_t)stream);
    if (e == cudaErrorInvalidValue && g_err[0]) return TT_ERR_CUDA;
    if (e != cudaSuccess) return cuda_fail(e, "tt_debug_umma_probe: launch");
    return TT_OK;
}

// ------------------------------------------------------------------------------ host-buffer calls
namespace {
struct DevBuf {
    void* p = nullptr;
    ~DevBuf() { if (p) tt_free(p); }
    int get(size_t n) { return tt_alloc(n, &p); }
};
cudaStream_t host_call_stream() {
    static thread_local cudaStream_t st = nullptr;
    static thread_local int st_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (!st || st_dev != dev) {
        if (st) {   // the thread moved to another device: give the old device's stream back
            cudaSetDevice(st_dev);
            cudaStreamDestroy(st);
            cudaSetDevice(dev);
            st = nullptr;
        }
        if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) st = nullptr;
        st_dev = dev;
    }
    return st;
}
// Synchronises the streams it was given when it goes out of scope, unless dismissed.  The host-buffer
// calls queue copies and kernels on non-blocking streams and then let pooled device buffers go: on an
// error exit in the middle of the sequence that work may still be queued, and tt_free hands a block to
// the next tt_alloc at once.  Declared AFTER the DevBufs, so that it runs before their destructors.
std::atomic<long long> g_guard_syncs{0};
struct SyncOnExit {
    cudaStream_t s[4] = {nullptr, nullptr, nullptr, nullptr};
    int n = 0;
    bool armed = true;
    void add(cudaStream_t st) { if (n < 4) s[n++] = st; }
    ~SyncOnExit() {
        if (!armed) return;
        for (int i = 0; i < n; ++i) cudaStreamSynchronize(s[i]);
        g_guard_syncs.fetch_add(1);
    }
};
// Host-made failure for tests: while the countdown is armed, the check that brings it to zero reports
// cudaErrorUnknown although the runtime call it guards was made and succeeded -- so the call returns in
// the middle of its sequence with copies and kernels still queued, which is the case SyncOnExit exists
// for.  Nothing on the device fails.
std::atomic<long long> g_fail_countdown{-1};
inline cudaError_t injected(cudaError_t e) {
    if (e != cudaSuccess || g_fail_countdown.load(std::memory_order_relaxed) < 0) return e;
    return g_fail_countdown.fetch_sub(1) == 0 ? cudaErrorUnknown : e;
}
#define TT_TRY(x) do { int rc__ = (x); if (rc__ != TT_OK) return rc__; } while (0)
#define TT_CUDA(x, what) do { cudaError_t e__ = injected(x); if (e__ != cudaSuccess) return cuda_fail(e__, what); } while (0)
}  // namespace

int tt_debug_fail_host_call_after(int64_t checks) {
    g_fail_countdown.store(checks < 0 ? -1 : (long long)checks);
    return TT_OK;
}
int64_t tt_debug_guard_syncs(void) { return (int64_t)g_guard_syncs.load(); }

int tt_attn_fwd_host(const tt_attn_desc* d, const void* q, const void* k, const void* v, void* out, float* lse) {
    AttnArgs a;
    TT_TRY(resolve(d, &a, "tt_attn_fwd_host"));
    if (!q || !k || !v || !out) return fail(TT_ERR_NULL, "tt_attn_fwd_host: q, k, v and out must be non-null");
    TT_TRY(check_device());
    const size_t es = a.bf16 ? 2 : 4;
    const size_t nq = (size_t)a.BH * a.S * a.D * es, nk = (size_t)(a.BH / a.group) * a.L * a.D * es;
    const size_t nl = (size_t)a.BH * a.S * sizeof(float);
    DevBuf dq_, dk_, dv_, do_, dl_;
    TT_TRY(dq_.get(nq)); TT_TRY(dk_.get(nk)); TT_TRY(dv_.get(nk)); TT_TRY(do_.get(nq)); TT_TRY(dl_.get(nl));
    cudaStream_t st = host_call_stream();
    SyncOnExit guard;
    guard.add(st);
    TT_CUDA(cudaMemcpyAsync(dq_.p, q, nq, cudaMemcpyHostToDevice, st), "upload q");
    TT_CUDA(cudaMemcpyAsync(dk_.p, k, nk, cudaMemcpyHostToDevice, st), "upload k");
    TT_CUDA(cudaMemcpyAsync(dv_.p, v, nk, cudaMemcpyHostToDevice, st), "upload v");
    TT_TRY(tt_attn_fwd(d, dq_.p, dk_.p, dv_.p, do_.p, (float*)dl_.p, st));
    TT_CUDA(cudaMemcpyAsync(out, do_.p, nq, cudaMemcpyDeviceToHost, st), "download out");
    if (lse) TT_CUDA(cudaMemcpyAsync(lse, dl_.p, nl, cudaMemcpyDeviceToHost, st), "download lse");
    return tt_check_device_status(st);
}

int tt_attn_bwd_host(const tt_attn_desc* d, const void* q, const void* k, const void* v, const void* out,
                     const float* lse, const void* dout, void* dq, void* dk, void* dv) {
    AttnArgs a;
    TT_TRY(resolve(d, &a, "tt_attn_bwd_host"));
    if (!q || !k || !v || !out || !lse || !dout || !dq || !dk || !dv)
        return fail(TT_ERR_NULL, "tt_attn_bwd_host: all tensor pointers must be non-null");
    TT_TRY(check_device());
    const size_t es = a.bf16 ? 2 : 4;
    const size_t nq = (size_t)a.BH * a.S * a.D * es, nk = (size_t)(a.BH / a.group) * a.L * a.D * es;
    const size_t nl = (size_t)a.BH * a.S * sizeof(float);
    const size_t nws = tt_attn_bwd_workspace_bytes(d);
    DevBuf bq, bk, bv, bo, bl, bdo, bdq, bdk, bdv, bws;
    TT_TRY(bq.get(nq)); TT_TRY(bk.get(nk)); TT_TRY(bv.get(nk)); TT_TRY(bo.get(nq)); TT_TRY(bl.get(nl));
    TT_TRY(bdo.get(nq)); TT_TRY(bdq.get(nq)); TT_TRY(bdk.get(nk)); TT_TRY(bdv.get(nk)); TT_TRY(bws.get(nws));
    cudaStream_t st = host_call_stream();
    SyncOnExit guard;
    guard.add(st);
    TT_CUDA(cudaMemcpyAsync(bq.p, q, nq, cudaMemcpyHostToDevice, st), "upload q");
    TT_CUDA(cudaMemcpyAsync(bk.p, k, nk, cudaMemcpyHostToDevice, st), "upload k");
    TT_CUDA(cudaMemcpyAsync(bv.p, v, nk, cudaMemcpyHostToDevice, st), "upload v");
    TT_CUDA(cudaMemcpyAsync(bo.p, out, nq, cudaMemcpyHostToDevice, st), "upload out");
    TT_CUDA(cudaMemcpyAsync(bl.p, lse, nl, cudaMemcpyHostToDevice, st), "upload lse");
    TT_CUDA(cudaMemcpyAsync(bdo.p, dout, nq, cudaMemcpyHostToDevice, st), "upload dout");
    TT_TRY(tt_attn_bwd(d, bq.p, bk.p, bv.p, bo.p, (const float*)bl.p, bdo.p, bdq.p, bdk.p, bdv.p, bws.p, nws, st));
    TT_CUDA(cudaMemcpyAsync(dq, bdq.p, nq, cudaMemcpyDeviceToHost, st), "download dq");
    TT_CUDA(cudaMemcpyAsync(dk, bdk.p, nk, cudaMemcpyDeviceToHost, st), "download dk");
    TT_CUDA(cudaMemcpyAsync(dv, bdv.p, nk, cudaMemcpyDeviceToHost, st), "download dv");
    return tt_check_device_status(st);
}

// ---- pipelined host-buffer training step ----------------------------------------------------
// The (batch, head) slices are independent, so the step is cut into chunks of slices that flow
// through the streams: upload (q,k,v,dout of chunk c+1) | forward+backward (chunk c) |
// download (out,lse,dq,dk,dv of chunk c-1).  With pinned host memory the PCIe transfers of both
// directions overlap the kernels instead of preceding and following them.  Chunks alternate between
// two compute streams: the kernels are persistent (one CTA per SM), so the next chunk's first CTAs
// take over SMs as the previous chunk's last items finish instead of waiting for its whole tail.
namespace {
struct PipeStreams {
    cudaStream_t in = nullptr, comp = nullptr, comp2 = nullptr, out = nullptr;
    int dev = -1;
};
int pipe_streams(PipeStreams** ps) {
    static thread_local PipeStreams s;
    int dev = 0;
    cudaGetDevice(&dev);
    if (s.dev != dev) {
        if (s.dev >= 0) {   // the thread moved to another device: give the old device's streams back
            cudaSetDevice(s.dev);
            for (cudaStream_t old : {s.in, s.comp, s.comp2, s.out})
                if (old) cudaStreamDestroy(old);
            cudaSetDevice(dev);
            s.in = s.comp = s.comp2 = s.out = nullptr;
            s.dev = -1;
        }
        TT_CUDA(cudaStreamCreateWithFlags(&s.in, cudaStreamNonBlocking), "stream");
        TT_CUDA(cudaStreamCreateWithFlags(&s.comp, cudaStreamNonBlocking), "stream");
        TT_CUDA(cudaStreamCreateWithFlags(&s.comp2, cudaStreamNonBlocking), "stream");
        TT_CUDA(cudaStreamCreateWithFlags(&s.out, cudaStreamNonBlocking), "stream");
        s.dev = dev;
    }
    *ps = &s;
    return TT_OK;
}
struct EventSet {
    static const int kN = 3;
    // per buffer set: q,k,v uploaded | dO uploaded | forward done | backward done | all downloaded
    cudaEvent_t in[kN] = {}, in_do[kN] = {}, fwd[kN] = {}, comp[kN] = {}, out[kN] = {};
    bool ok = false;
    int make() {
        for (cudaEvent_t* arr : {in, in_do, fwd, comp, out})
            for (int i = 0; i < kN; ++i) TT_CUDA(cudaEventCreateWithFlags(&arr[i], cudaEventDisableTiming), "event");
        ok = true;
        return TT_OK;
    }
    ~EventSet() {
        for (cudaEvent_t* arr : {in, in_do, fwd, comp, out})
            for (int i = 0; i < kN; ++i)
                if (arr[i]) cudaEventDestroy(arr[i]);
    }
};
}  // namespace

int tt_attn_fwd_bwd_host(const tt_attn_desc* d, const void* q, const void* k, const void* v, const void* dout,
                         void* out, float* lse, void* dq, void* dk, void* dv) {
    AttnArgs a;
    TT_TRY(resolve(d, &a, "tt_attn_fwd_bwd_host"));
    if (!q || !k || !v || !dout || !out || !dq || !dk || !dv)
        return fail(TT_ERR_NULL, "tt_attn_fwd_bwd_host: q, k, v, dout, out, dq, dk, dv must be non-null");
    TT_TRY(check_device());
    const size_t es = a.bf16 ? 2 : 4;
    const size_t q_slice = (size_t)a.S * a.D * es, k_slice = (size_t)a.L * a.D * es, l_slice = (size_t)a.S * sizeof(float);
    // chunk: about 32 MiB of q per chunk, at least 1 slice, at most an eighth of the slices: with few
    // slices (a rank's share of a sharded problem) the pipeline still gets eight stages, so that only
    // the first upload and the last download are exposed
    long long per = (long long)((32u << 20) / (q_slice ? q_slice : 1));
    if (per < 1) per = 1;
    if (per > a.BH / 8) per = a.BH / 8;
    if (per < 1) per = 1;
    per = (per + a.group - 1) / a.group * a.group;   // a chunk holds whole groups of query heads
    // Chunk sizes: `per` slices, but the first two and the last two chunks are a quarter and a half of that
    // (whole groups): the upload of the first chunk and the download of the last are the only transfers
    // nothing overlaps, and the two compute streams hide the short launches of small chunks.
    std::vector<long long> starts;   // first slice of every chunk, then BH
    {
        const long long g = a.group;
        const long long quarter = std::max<long long>(g, per / 4 / g * g), half = std::max<long long>(g, per / 2 / g * g);
        long long left = a.BH, at = 0;
        const long long back = quarter + half;
        auto push = [&](long long n) { starts.push_back(at); at += n; left -= n; };
        if (a.BH >= 2 * back + per) {
            push(quarter);
            push(half);
            while (left - back >= per) push(per);
            if (left > back) push(left - back);
            push(half);
            push(quarter);
        } else {
            while (left > 0) push(std::min(per, left));
        }
        starts.push_back(a.BH);
    }
    const long long n_chunks = (long long)starts.size() - 1;
    constexpr int NB = EventSet::kN;
    tt_attn_desc dc = *d;
    dc.B = 1;
    dc.H = (int32_t)per;
    dc.Hkv = (int32_t)(per / a.group);
    const size_t ws_bytes = tt_attn_bwd_workspace_bytes(&dc);
    DevBuf bq[NB], bk[NB], bv[NB], bdo[NB], bo[NB], bl[NB], bdq[NB], bdk[NB], bdv[NB], bws[NB];
    const int nb_used = (int)(n_chunks < NB ? n_chunks : NB);
    for (int i = 0; i < nb_used; ++i) {
        const long long perk = per / a.group;
        TT_TRY(bq[i].get(per * q_slice)); TT_TRY(bk[i].get(perk * k_slice)); TT_TRY(bv[i].get(perk * k_slice));
        TT_TRY(bdo[i].get(per * q_slice)); TT_TRY(bo[i].get(per * q_slice)); TT_TRY(bl[i].get(per * l_slice));
        TT_TRY(bdq[i].get(per * q_slice)); TT_TRY(bdk[i].get(perk * k_slice)); TT_TRY(bdv[i].get(perk * k_slice));
        TT_TRY(bws[i].get(ws_bytes));
    }
    PipeStreams* ps = nullptr;
    TT_TRY(pipe_streams(&ps));
    SyncOnExit guard;
    guard.add(ps->in);
    guard.add(ps->comp);
    guard.add(ps->comp2);
    guard.add(ps->out);
    EventSet ev;
    TT_TRY(ev.make());
    const char* hq = (const char*)q; const char* hk = (const char*)k; const char* hv = (const char*)v;
    const char* hdo = (const char*)dout;
    char* ho = (char*)out; char* hdq = (char*)dq; char* hdk = (char*)dk; char* hdv = (char*)dv;
    for (long long c = 0; c < n_chunks; ++c) {
        const int b = (int)(c % NB);
        const long long s0 = starts[(size_t)c];
        const long long cnt = starts[(size_t)c + 1] - s0;
        const long long k0 = s0 / a.group, kcnt = cnt / a.group;   // the chunk's key/value slices
        if (c >= NB) TT_CUDA(cudaStreamWaitEvent(ps->in, ev.out[b], 0), "wait buffer");   // chunk c-NB downloaded
        TT_CUDA(cudaMemcpyAsync(bq[b].p, hq + s0 * q_slice, cnt * q_slice, cudaMemcpyHostToDevice, ps->in), "upload q");
        TT_CUDA(cudaMemcpyAsync(bk[b].p, hk + k0 * k_slice, kcnt * k_slice, cudaMemcpyHostToDevice, ps->in), "upload k");
        TT_CUDA(cudaMemcpyAsync(bv[b].p, hv + k0 * k_slice, kcnt * k_slice, cudaMemcpyHostToDevice, ps->in), "upload v");
        // the forward needs q, k, v only: it starts while dO is still on its way, and its results go
        // back to the host while the backward runs
        TT_CUDA(cudaEventRecord(ev.in[b], ps->in), "record");
        TT_CUDA(cudaMemcpyAsync(bdo[b].p, hdo + s0 * q_slice, cnt * q_slice, cudaMemcpyHostToDevice, ps->in), "upload dout");
        TT_CUDA(cudaEventRecord(ev.in_do[b], ps->in), "record");
        const cudaStream_t cs = (c & 1) ? ps->comp2 : ps->comp;
        TT_CUDA(cudaStreamWaitEvent(cs, ev.in[b], 0), "wait upload");
        tt_attn_desc di = *d;
        di.B = 1;
        di.H = (int32_t)cnt;
        di.Hkv = (int32_t)kcnt;
        TT_TRY(tt_attn_fwd(&di, bq[b].p, bk[b].p, bv[b].p, bo[b].p, (float*)bl[b].p, cs));
        TT_CUDA(cudaEventRecord(ev.fwd[b], cs), "record");
        TT_CUDA(cudaStreamWaitEvent(cs, ev.in_do[b], 0), "wait upload");
        TT_TRY(tt_attn_bwd(&di, bq[b].p, bk[b].p, bv[b].p, bo[b].p, (const float*)bl[b].p, bdo[b].p, bdq[b].p, bdk[b].p,
                           bdv[b].p, bws[b].p, ws_bytes, cs));
        TT_CUDA(cudaEventRecord(ev.comp[b], cs), "record");
        TT_CUDA(cudaStreamWaitEvent(ps->out, ev.fwd[b], 0), "wait forward");
        TT_CUDA(cudaMemcpyAsync(ho + s0 * q_slice, bo[b].p, cnt * q_slice, cudaMemcpyDeviceToHost, ps->out), "download out");
        if (lse) TT_CUDA(cudaMemcpyAsync(lse + s0 * a.S, bl[b].p, cnt * l_slice, cudaMemcpyDeviceToHost, ps->out), "download lse");
        TT_CUDA(cudaStreamWaitEvent(ps->out, ev.comp[b], 0), "wait backward");
        TT_CUDA(cudaMemcpyAsync(hdq + s0 * q_slice, bdq[b].p, cnt * q_slice, cudaMemcpyDeviceToHost, ps->out), "download dq");
        TT_CUDA(cudaMemcpyAsync(hdk + k0 * k_slice, bdk[b].p, kcnt * k_slice, cudaMemcpyDeviceToHost, ps->out), "download dk");
        TT_CUDA(cudaMemcpyAsync(hdv + k0 * k_slice, bdv[b].p, kcnt * k_slice, cudaMemcpyDeviceToHost, ps->out), "download dv");
        TT_CUDA(cudaEventRecord(ev.out[b], ps->out), "record");
    }
    TT_CUDA(cudaStreamSynchronize(ps->in), "synchronize");
    TT_CUDA(cudaStreamSynchronize(ps->comp), "synchronize");
    TT_CUDA(cudaStreamSynchronize(ps->comp2), "synchronize");
    return tt_check_device_status(ps->out);
}

int tt_attn_decode_host(const tt_attn_desc* d, const void* q, const void* k, const void* v, void* out,
                        float* lse) {
    AttnArgs a;
    TT_TRY(resolve(d, &a, "tt_attn_decode_host"));
    if (a.S != 1) return fail(TT_ERR_BAD_SHAPE, "tt_attn_decode_host: S must be 1, got %d", a.S);
    if (!q || !k || !v || !out) return fail(TT_ERR_NULL, "tt_attn_decode_host: q, k, v and out must be non-null");
    TT_TRY(check_device());
    const size_t es = a.bf16 ? 2 : 4;
    const size_t nq = (size_t)a.BH * a.D * es, nk = (size_t)(a.BH / a.group) * a.L * a.D * es;
    const size_t nl = (size_t)a.BH * sizeof(float);
    const size_t nws = tt_attn_decode_workspace_bytes(d);
    DevBuf bq, bk, bv, bo, bl, bws;
    TT_TRY(bq.get(nq)); TT_TRY(bk.get(nk)); TT_TRY(bv.get(nk)); TT_TRY(bo.get(nq)); TT_TRY(bl.get(nl));
    TT_TRY(bws.get(nws));
    cudaStream_t st = host_call_stream();
    SyncOnExit guard;
    guard.add(st);
    TT_CUDA(cudaMemcpyAsync(bq.p, q, nq, cudaMemcpyHostToDevice, st), "upload q");
    TT_CUDA(cudaMemcpyAsync(bk.p, k, nk, cudaMemcpyHostToDevice, st), "upload k");
    TT_CUDA(cudaMemcpyAsync(bv.p, v, nk, cudaMemcpyHostToDevice, st), "upload v");
    TT_TRY(tt_attn_decode(d, bq.p, bk.p, bv.p, bo.p, (float*)bl.p, bws.p, nws, st));
    TT_CUDA(cudaMemcpyAsync(out, bo.p, nq, cudaMemcpyDeviceToHost, st), "download out");
    if (lse) TT_CUDA(cudaMemcpyAsync(lse, bl.p, nl, cudaMemcpyDeviceToHost, st), "download lse");
    return tt_check_device_status(st);
}

}  // extern "C"

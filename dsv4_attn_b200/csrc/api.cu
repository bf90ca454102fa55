// C ABI of the library: argument validation, parameter filling, launches.
// No allocation and no synchronisation.  Process-wide state is limited to: per-device flags that a
// kernel's shared-memory attribute has been set, the per-device address of the built-in scratch array of
// the entry point that allocates nothing (both written once, atomically), and the test switches of
// dsv4_debug_set_flags / dsv4_debug_set_wait, which are read once per call.
#include "../../include/dsv4_attn.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cmath>
#include <atomic>

#include "combine.cuh"
#include "compress_reduce.cuh"
#include "cache_write.cuh"
#include "rope_norm.cuh"
#include "indexer.cuh"
#include "decode_kernel.cuh"
#include "sched.cuh"
#include "decode_simt.cuh"

namespace dsv4 {
namespace {

constexpr int kMaxDevices = 64;

// Test switches (dsv4_debug_set_flags, dsv4_debug_set_wait); product behaviour when left alone.
std::atomic<int> g_dbg{0};
std::atomic<unsigned long long> g_wait_ns{kDefaultWaitNs};
std::atomic<int> g_drop_tile{-1};
#ifdef DSV4_TRACE
std::atomic<unsigned long long*> g_trace{nullptr};
#endif

thread_local const char* t_last_error = "";

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does
// not link against libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Q as a 2-D BF16 tensor [rows, cols], row-major; box = 64 columns x 128 rows, 128-byte swizzle.
cudaError_t make_q_map(CUtensorMap* map, const void* q, int64_t rows, int cols) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(cols) * 2};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Opt in to the large dynamic shared memory once per (kernel, device).  The flags are written once,
// atomically; two threads racing on the first call both set the attribute, which is harmless.
template <typename Kernel>
cudaError_t ensure_smem(Kernel kernel, int bytes, std::atomic<bool>* done_per_device) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!done_per_device[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        done_per_device[dev].store(true, std::memory_order_release);
    }
    return cudaSuccess;
}

int device_sms() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

// Layout of a schedule buffer (int32 words); a function of the batch shape only, so that the planner and
// the decode entry points agree on it without reading anything back.
struct SchedLayout {
    int64_t info, pair_begin, unit_nsplits, unit_slot, unit_prefix, items, words;
    int item_cap;
};
constexpr int kSchedInfoWords = 16;
SchedLayout sched_layout(int n_units, int item_cap) {
    SchedLayout l{};
    l.info = 0;
    l.pair_begin = kSchedInfoWords;
    l.unit_nsplits = l.pair_begin + ((kPlanMaxPairs + 1 + 3) / 4) * 4;
    l.unit_slot = l.unit_nsplits + ((n_units + 3) / 4) * 4;
    l.unit_prefix = l.unit_slot + ((n_units + 3) / 4) * 4;
    l.items = l.unit_prefix + 2 * int64_t((n_units + 1) / 2 * 2);
    l.item_cap = item_cap;
    l.words = l.items + int64_t(item_cap) * kItemWords;
    return l;
}
int sched_item_cap(int n_units, int num_splits, int num_pairs) {
    return n_units * (num_splits > 1 ? num_splits : 1) + num_pairs;
}
int64_t sched_slot_cap(int n_units, int num_splits, int num_pairs) {
    if (num_splits == 1) return 0;
    return num_splits > 1 ? int64_t(n_units) * num_splits : 2 * int64_t(num_pairs);
}

template <int NCHUNK, int SRC>
cudaError_t launch_mma(DecodeArgs& a, int rows, const void* sched, cudaStream_t stream) {
    cudaError_t e = make_q_map(&a.q_map, a.q, int64_t(rows) * a.H, NCHUNK * 64);
    if (e != cudaSuccess) return e;
    a.wait_ns = g_wait_ns.load(std::memory_order_relaxed);
    a.dbg_drop_tile = g_drop_tile.load(std::memory_order_relaxed);
#ifdef DSV4_TRACE
    a.trace = g_trace.load();
#endif
    const int head_groups = (a.H + kHeadsPerCta - 1) / kHeadsPerCta;
    dim3 grid(2 * head_groups, rows, a.num_splits);
    if (sched != nullptr) {
        // resident blocks, one pair per two SMs, each walking its slice of the plan
        const SchedLayout l = sched_layout(rows * head_groups, 0);
        const int32_t* base = static_cast<const int32_t*>(sched);
        a.sched_pair_begin = base + l.pair_begin;
        a.sched_items = base + l.items;
        int pairs = device_sms() / 2;
        if (pairs > kPlanMaxPairs) pairs = kPlanMaxPairs;
        grid = dim3(2 * (pairs > 0 ? pairs : 1), 1, 1);
    }
    static std::atomic<bool> done[kMaxDevices];
    constexpr int smem = SmemLayout<NCHUNK>::kTotal;
    e = ensure_smem(decode_mma_kernel<NCHUNK, SRC>, smem, done);
    if (e != cudaSuccess) return e;
    decode_mma_kernel<NCHUNK, SRC><<<grid, kNumThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int SRC>
cudaError_t launch_simt(const DecodeArgs& a, int rows, int max_tok, cudaStream_t stream) {
    static std::atomic<bool> done[kMaxDevices];
    const int smem = (576 + kSimtThreads + max_tok) * int(sizeof(float));
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = ensure_smem(decode_simt_kernel<SRC>, 200 * 1024, done);
    if (e != cudaSuccess) return e;
    dim3 grid(rows, a.H);
    decode_simt_kernel<SRC><<<grid, kSimtThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

// after_decode: the launch directly follows this library's decode launch on the same stream; the merge is then
// launched as its programmatic dependent, so that its blocks are resident (and waiting) when the last decode
// blocks are in their epilogue.
cudaError_t launch_combine(const CombineArgs& c, cudaStream_t stream, bool after_decode = false) {
    const int64_t units = int64_t(c.N) * c.H;
    const int blocks = int((units + kCombineWarps - 1) / kCombineWarps);
    if (after_decode && !(g_dbg.load(std::memory_order_relaxed) & 64)) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(blocks);
        cfg.blockDim = dim3(kCombineWarps * 32);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, combine_kernel, c);
    }
    combine_kernel<<<blocks, kCombineWarps * 32, 0, stream>>>(c);
    return cudaGetLastError();
}

CombineArgs contiguous_combine(int rows, int H, int S, const float* po, const float* pl, void* out, float* lse,
                               const float* sink, bool partial_bf16 = false) {
    CombineArgs c{};
    c.partial_bf16 = partial_bf16 ? 1 : 0;
    c.N = rows;  c.H = H;  c.num_splits = S;
    c.partial_o = po;  c.partial_lse = pl;
    c.out = static_cast<__nv_bfloat16*>(out);  c.lse = lse;  c.attn_sink = sink;
    c.stride_po_split = int64_t(rows) * H * 512;  c.stride_po_n = int64_t(H) * 512;  c.stride_po_h = 512;
    c.stride_pl_split = int64_t(rows) * H;  c.stride_pl_n = H;
    c.stride_out_n = int64_t(H) * 512;  c.stride_out_h = 512;
    c.stride_lse_n = H;
    return c;
}

bool common_ok(int B, int s_q, int H, int num_splits, float sm_scale, const void* q, const void* out,
               const float* po, const float* pl) {
    if (B <= 0 || s_q <= 0 || H <= 0) return false;
    if (int64_t(B) * s_q > 65535) return false;                 // grid.y
    if (num_splits < 1 || num_splits > DSV4_MAX_SPLITS) return false;
    if (!(sm_scale > 0.f) || !std::isfinite(sm_scale)) return false;
    if (q == nullptr || out == nullptr || !aligned(q, 16) || !aligned(out, 16)) return false;
    if (num_splits > 1 && (po == nullptr || pl == nullptr || !aligned(po, 16))) return false;
    return true;
}

bool fill_csa(const Dsv4CsaSparseDecodeParams* p, DecodeArgs& a) {
    if (p == nullptr) return false;
    if (!common_ok(p->B, p->s_q, p->H, p->sched != nullptr ? 2 : p->num_splits, p->sm_scale, p->q, p->out, p->partial_o, p->partial_lse))
        return false;
    if (p->topk <= 0 || p->max_pages <= 0 || p->num_pages <= 0 || !aligned(p->sched, 16)) return false;
    if (p->kv_pool == nullptr || p->block_table == nullptr || p->indices == nullptr) return false;
    if (!aligned(p->kv_pool, 16)) return false;
    a = DecodeArgs{};
    a.B = p->B;  a.s_q = p->s_q;  a.H = p->H;  a.topk = p->topk;  a.max_pages = p->max_pages;
    a.num_pages = p->num_pages;
    a.num_splits = p->sched != nullptr ? 1 : p->num_splits;
    a.scale_log2 = p->sm_scale * 1.4426950408889634f;
    a.q = static_cast<const __nv_bfloat16*>(p->q);
    a.kv_pool = static_cast<const uint8_t*>(p->kv_pool);
    a.block_table = p->block_table;  a.indices = p->indices;  a.kv_len = p->kv_len;  a.topk_len = p->topk_len;
    a.attn_sink = p->attn_sink;
    a.out = static_cast<__nv_bfloat16*>(p->out);  a.lse = p->lse;
    a.partial_o = p->partial_o;  a.partial_lse = p->partial_lse;  a.status = p->status;
    return true;
}

bool fill_hca(const Dsv4HcaDenseDecodeParams* p, DecodeArgs& a) {
    if (p == nullptr) return false;
    if (!common_ok(p->B, p->s_q, p->H, p->sched != nullptr ? 2 : p->num_splits, p->sm_scale, p->q, p->out, p->partial_o, p->partial_lse))
        return false;
    if (p->max_pages <= 0 || p->win_cap < 0 || p->num_pages <= 0 || !aligned(p->sched, 16)) return false;
    if (p->kv_pool == nullptr || p->block_table == nullptr || p->kv_len == nullptr || p->win_len == nullptr)
        return false;
    if (p->win_cap > 0 && p->win_pool == nullptr) return false;
    if (!aligned(p->kv_pool, 16) || !aligned(p->win_pool, 16)) return false;
    a = DecodeArgs{};
    a.B = p->B;  a.s_q = p->s_q;  a.H = p->H;  a.max_pages = p->max_pages;  a.win_cap = p->win_cap;
    a.num_pages = p->num_pages;
    a.num_splits = p->sched != nullptr ? 1 : p->num_splits;
    a.scale_log2 = p->sm_scale * 1.4426950408889634f;
    a.q = static_cast<const __nv_bfloat16*>(p->q);
    a.kv_pool = static_cast<const uint8_t*>(p->kv_pool);
    a.block_table = p->block_table;  a.kv_len = p->kv_len;
    a.win_pool = static_cast<const uint8_t*>(p->win_pool);  a.win_len = p->win_len;
    a.attn_sink = p->attn_sink;
    a.out = static_cast<__nv_bfloat16*>(p->out);  a.lse = p->lse;
    a.partial_o = p->partial_o;  a.partial_lse = p->partial_lse;  a.status = p->status;
    return true;
}

// Split-KV scratch for the entry point that must not allocate: partial outputs
// followed by partial LSEs, in device memory that belongs to the loaded library
// image.  32 MiB + 64 KiB per GPU that loads the library, held until exit.
constexpr size_t kNoAllocPartialFloats = size_t(8) << 20;                 // 8 Mi floats = 32 MiB of partial outputs
constexpr size_t kNoAllocLseFloats = kNoAllocPartialFloats / 512;         // one LSE per 512-wide partial row
__device__ __align__(256) float g_noalloc_scratch[kNoAllocPartialFloats + kNoAllocLseFloats];

// Device address of the scratch array on the current device.  In host code the
// array's name is only a handle for the runtime, not an address a kernel could
// use, so the address is asked for once per device and kept.
cudaError_t noalloc_scratch(float** ptr) {
    static std::atomic<float*> per_device[kMaxDevices];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    float* known = per_device[dev].load(std::memory_order_acquire);
    if (known == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        known = static_cast<float*>(p);
        per_device[dev].store(known, std::memory_order_release);     // racing threads store the same address
    }
    *ptr = known;
    return cudaSuccess;
}

// Records why a launch failed for dsv4_attn_last_error().
int launch_failed(cudaError_t e) {
    t_last_error = cudaGetErrorString(e);
    return int(e);
}

// Decode (+ merge when split) for the packed-entry sources.  With a plan, the resident blocks walk it and the
// merge adds up the units the plan cut.
template <int SRC>
int decode_fwd(DecodeArgs& a, const void* sched, cudaStream_t stream) {
    const int rows = a.B * a.s_q;
    cudaError_t e = launch_mma<9, SRC>(a, rows, sched, stream);
    if (e != cudaSuccess) return launch_failed(e);
    if (sched != nullptr) {
        const int hgs = (a.H + kHeadsPerCta - 1) / kHeadsPerCta;
        const SchedLayout l = sched_layout(rows * hgs, 0);
        CombineArgs c = contiguous_combine(rows, a.H, 1, a.partial_o, a.partial_lse, a.out, a.lse, a.attn_sink, true);
        c.unit_nsplits = static_cast<const int32_t*>(sched) + l.unit_nsplits;
        c.unit_slot = static_cast<const int32_t*>(sched) + l.unit_slot;
        c.hgs = hgs;
        e = launch_combine(c, stream, true);
    } else if (a.num_splits > 1) {
        CombineArgs c = contiguous_combine(rows, a.H, a.num_splits, a.partial_o, a.partial_lse, a.out, a.lse, a.attn_sink,
                                           true);
        e = launch_combine(c, stream, true);
    }
    return e == cudaSuccess ? 0 : launch_failed(e);
}

}  // namespace
}  // namespace dsv4

using namespace dsv4;

extern "C" int dsv4_attn_version(void) { return (0 << 16) | 2; }

extern "C" void dsv4_debug_set_flags(int flags) { g_dbg.store(flags); }

extern "C" void dsv4_debug_set_wait(unsigned long long wait_ns, int drop_tile) {
    g_wait_ns.store(wait_ns != 0 ? wait_ns : kDefaultWaitNs);
    g_drop_tile.store(drop_tile);
}

#ifdef DSV4_TRACE
extern "C" void dsv4_debug_set_trace(void* device_buffer) { g_trace.store(static_cast<unsigned long long*>(device_buffer)); }
#endif

extern "C" int64_t dsv4_attn_sched_bytes(int rows, int H, int num_splits, int num_sms, int64_t* partial_o_bytes,
                                         int64_t* partial_lse_bytes) {
    if (partial_o_bytes) *partial_o_bytes = 0;
    if (partial_lse_bytes) *partial_lse_bytes = 0;
    if (rows <= 0 || H <= 0 || num_splits < 0 || num_splits > DSV4_MAX_SPLITS) return 0;
    if (num_sms <= 0) num_sms = device_sms();
    int pairs = num_sms / 2;
    if (pairs < 1) pairs = 1;
    if (pairs > kPlanMaxPairs) pairs = kPlanMaxPairs;
    const int hgs = (H + kHeadsPerCta - 1) / kHeadsPerCta;
    if (int64_t(rows) * hgs > 0x3FFFFFFF / DSV4_MAX_SPLITS) return 0;
    const int n_units = rows * hgs;
    const SchedLayout l = sched_layout(n_units, sched_item_cap(n_units, num_splits, pairs));
    const int64_t slots = sched_slot_cap(n_units, num_splits, pairs);
    if (partial_o_bytes) *partial_o_bytes = slots * 128 * 512 * 2;       // BF16 rows
    if (partial_lse_bytes) *partial_lse_bytes = slots * 128 * 4;
    return l.words * 4;
}

namespace {
// Validates a plan request and fills the planner's arguments; `base` is where the schedule goes.
int fill_plan(const Dsv4PlanParams* p, int32_t* base, PlanArgs& a) {
    t_last_error = "invalid argument";
    if (p == nullptr || p->B <= 0 || p->s_q <= 0 || p->H <= 0 || base == nullptr || !aligned(base, 16)) return int(cudaErrorInvalidValue);
    if (p->num_splits < 0 || p->num_splits > DSV4_MAX_SPLITS || int64_t(p->B) * p->s_q > 65535) return int(cudaErrorInvalidValue);
    const int sms = device_sms();
    int num_sms = p->num_sms > 0 ? p->num_sms : sms;
    if (num_sms > sms && p->num_sms <= 0) num_sms = sms;
    int pairs = num_sms / 2;
    if (pairs < 1) pairs = 1;
    if (pairs > kPlanMaxPairs) pairs = kPlanMaxPairs;
    a = PlanArgs{};
    if (p->kind == DSV4_PLAN_CSA) {
        if (p->topk <= 0) return int(cudaErrorInvalidValue);
        a.kind = kSrcCsa;
    } else if (p->kind == DSV4_PLAN_HCA) {
        if (p->kv_len == nullptr || p->win_len == nullptr) return int(cudaErrorInvalidValue);
        a.kind = kSrcHca;
    } else {
        return int(cudaErrorInvalidValue);
    }
    a.rows = p->B * p->s_q;
    a.hgs = (p->H + kHeadsPerCta - 1) / kHeadsPerCta;
    const int n_units = a.rows * a.hgs;
    const SchedLayout l = sched_layout(n_units, sched_item_cap(n_units, p->num_splits, pairs));
    if (p->sched_bytes < l.words * 4) {
        t_last_error = "schedule buffer smaller than dsv4_attn_sched_bytes() for this shape";
        return int(cudaErrorInvalidValue);
    }
    a.topk = p->topk;  a.topk_len = p->topk_len;  a.kv_len = p->kv_len;  a.win_len = p->win_len;
    a.num_pairs = pairs;
    a.fixed_splits = p->num_splits;
    a.item_cap = l.item_cap;
    const int64_t slots = sched_slot_cap(n_units, p->num_splits, pairs);
    a.slot_cap = int(slots < 0x7FFFFFFF ? slots : 0x7FFFFFFF);
    a.info = base + l.info;
    a.pair_begin = base + l.pair_begin;
    a.unit_nsplits = base + l.unit_nsplits;
    a.unit_slot = base + l.unit_slot;
    a.unit_prefix = reinterpret_cast<long long*>(base + l.unit_prefix);
    a.items = base + l.items;
    t_last_error = "";
    return 0;
}
}  // namespace

extern "C" int dsv4_attn_plan(const Dsv4PlanParams* p, void* stream) {
    PlanArgs a;
    if (p != nullptr && p->num_sms > device_sms()) { t_last_error = "num_sms exceeds the device";  return int(cudaErrorInvalidValue); }
    const int rc = fill_plan(p, p ? static_cast<int32_t*>(p->sched) : nullptr, a);
    if (rc != 0) return rc;
    plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : launch_failed(e);
}

extern "C" int dsv4_attn_plan_host(const Dsv4PlanParams* p) {
    PlanArgs a;
    const int rc = fill_plan(p, p ? static_cast<int32_t*>(p->sched) : nullptr, a);
    if (rc != 0) return rc;
    plan_host(a);
    return 0;
}

extern "C" int dsv4_csa_sparse_decode_fwd(const Dsv4CsaSparseDecodeParams* p, void* stream) {
    DecodeArgs a;
    if (!fill_csa(p, a)) return int(cudaErrorInvalidValue);
    return decode_fwd<kSrcCsa>(a, p->sched, static_cast<cudaStream_t>(stream));
}

extern "C" const char* dsv4_attn_last_error(void) { return t_last_error; }

extern "C" int64_t dsv4_noalloc_scratch_bytes(void) {
    return int64_t(sizeof(float) * (kNoAllocPartialFloats + kNoAllocLseFloats));
}

extern "C" int dsv4_csa_sparse_decode_fwd_noalloc(const Dsv4CsaSparseDecodeParams* p, void* stream) {
    DecodeArgs a;
    t_last_error = "";
    if (p == nullptr) { t_last_error = "null parameter block";  return int(cudaErrorInvalidValue); }
    // the caller's workspace pointers are not used here; validate the rest as usual
    Dsv4CsaSparseDecodeParams q = *p;
    q.sched = nullptr;                        // this entry point always takes the caller's split count
    static float dummy;                       // stands in for the workspace during host-side validation only
    if (q.num_splits > 1) { q.partial_o = reinterpret_cast<float*>(uintptr_t(256));  q.partial_lse = &dummy; }
    if (!fill_csa(&q, a)) { t_last_error = "invalid argument";  return int(cudaErrorInvalidValue); }
    if (a.num_splits > 1) {
        const size_t rows = size_t(a.B) * a.s_q;
        const size_t need_o = size_t(a.num_splits) * rows * a.H * 512;
        const size_t need_l = size_t(a.num_splits) * rows * a.H;
        if (need_o > kNoAllocPartialFloats || need_l > kNoAllocLseFloats) {
            t_last_error = "num_splits * B * s_q * H * 512 partial floats exceed the built-in scratch "
                           "(8 Mi floats = 32 MiB): use fewer splits or rows, or the entry point that takes a workspace";
            return int(cudaErrorInvalidValue);
        }
        float* scratch = nullptr;
        const cudaError_t e = noalloc_scratch(&scratch);
        if (e != cudaSuccess) { t_last_error = "cudaGetSymbolAddress failed";  return int(e); }
        a.partial_o = scratch;
        a.partial_lse = scratch + kNoAllocPartialFloats;
    } else {
        a.partial_o = nullptr;
        a.partial_lse = nullptr;
    }
    return decode_fwd<kSrcCsa>(a, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int dsv4_hca_dense_decode_fwd(const Dsv4HcaDenseDecodeParams* p, void* stream) {
    DecodeArgs a;
    if (!fill_hca(p, a)) return int(cudaErrorInvalidValue);
    return decode_fwd<kSrcHca>(a, p->sched, static_cast<cudaStream_t>(stream));
}

extern "C" int dsv4_csa_sparse_decode_simt(const Dsv4CsaSparseDecodeParams* p, void* stream) {
    DecodeArgs a;
    if (!fill_csa(p, a) || p->num_splits != 1) return int(cudaErrorInvalidValue);
    return int(launch_simt<kSrcCsa>(a, a.B * a.s_q, a.topk, static_cast<cudaStream_t>(stream)));
}

extern "C" int dsv4_hca_dense_decode_simt(const Dsv4HcaDenseDecodeParams* p, void* stream) {
    DecodeArgs a;
    if (!fill_hca(p, a) || p->num_splits != 1) return int(cudaErrorInvalidValue);
    // the longest row bounds the logit scratch; the caller's block table bounds kv_len
    const int max_tok = p->max_pages * DSV4_PAGE_ENTRIES + p->win_cap;
    return int(launch_simt<kSrcHca>(a, a.B * a.s_q, max_tok, static_cast<cudaStream_t>(stream)));
}

extern "C" int dsv4_attn_combine(const Dsv4CombineParams* p, void* stream) {
    if (p == nullptr || p->N <= 0 || p->H <= 0 || p->D != 512) return int(cudaErrorInvalidValue);
    if (p->num_splits < 1 || p->num_splits > kCombineMaxSplits) return int(cudaErrorInvalidValue);
    if (p->partial_o == nullptr || p->partial_lse == nullptr || p->out == nullptr) return int(cudaErrorInvalidValue);
    if (!aligned(p->partial_o, 16) || !aligned(p->out, 16)) return int(cudaErrorInvalidValue);
    if ((p->stride_po_split | p->stride_po_n | p->stride_po_h) % 4 != 0) return int(cudaErrorInvalidValue);
    if ((p->stride_out_n | p->stride_out_h) % 8 != 0) return int(cudaErrorInvalidValue);
    CombineArgs c{};
    c.N = p->N;  c.H = p->H;  c.num_splits = p->num_splits;
    c.partial_o = p->partial_o;  c.partial_lse = p->partial_lse;
    c.out = static_cast<__nv_bfloat16*>(p->out);  c.lse = p->lse;  c.attn_sink = p->attn_sink;
    c.stride_po_split = p->stride_po_split;  c.stride_po_n = p->stride_po_n;  c.stride_po_h = p->stride_po_h;
    c.stride_pl_split = p->stride_pl_split;  c.stride_pl_n = p->stride_pl_n;
    c.stride_out_n = p->stride_out_n;  c.stride_out_h = p->stride_out_h;
    c.stride_lse_n = p->stride_lse_n;
    return int(launch_combine(c, static_cast<cudaStream_t>(stream)));
}

extern "C" int dsv4_attn_plan_splits(int rows, int H, int max_len, int num_sms) {
    if (rows <= 0 || H <= 0 || max_len < 0) return -int(cudaErrorInvalidValue);
    if (num_sms <= 0) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return -int(e);
    }
    const int tiles = (max_len + kTileN - 1) / kTileN;
    if (tiles <= 1) return 1;
    const int64_t units = int64_t(rows) * 2 * ((H + kHeadsPerCta - 1) / kHeadsPerCta);
    // Cost model in units of one tile's time: a block costs a fixed set-up (Q
    // load, tensor-memory allocation, epilogue) plus its tiles; blocks run in
    // waves of `num_sms`; splitting adds the partial write + merge read.
    // constants fitted to measurements on B200 (split sweep at 512 units x 32 tiles)
    const double fixed = 4.0, merge_per_split = 1.8, merge_launch = 2.0;
    double best = 1e300;
    int best_s = 1;
    const int max_s = tiles < DSV4_MAX_SPLITS ? tiles : DSV4_MAX_SPLITS;
    for (int s = 1; s <= max_s; ++s) {
        const int tps = (tiles + s - 1) / s;
        if (s > 1 && (tiles + tps - 1) / tps != s) continue;   // would leave an empty split
        const int64_t blocks = units * s;
        const double waves = std::ceil(double(blocks) / num_sms);
        double cost = waves * (fixed + tps);
        if (s > 1) cost += merge_per_split * s * (double(units) / num_sms) + merge_launch;   // partials written and re-read, one more launch
        if (cost < best - 1e-9) { best = cost;  best_s = s; }
    }
    return best_s;
}

extern "C" int64_t dsv4_attn_workspace_bytes(int rows, int H, int num_splits, int64_t* lse_offset) {
    if (rows <= 0 || H <= 0 || num_splits <= 1) {
        if (lse_offset) *lse_offset = 0;
        return 0;
    }
    const int64_t po = int64_t(num_splits) * rows * H * 512 * 4;
    const int64_t pl = int64_t(num_splits) * rows * H * 4;
    if (lse_offset) *lse_offset = po;
    return po + ((pl + 255) / 256) * 256;
}

extern "C" int hca_decode_fwd(const void* Q,
                              const void* Kc, const void* Kc_s, const void* Kc_rope,
                              const void* Kswa, const void* Kswa_s, const void* Kswa_rope,
                              const void* sink_logits,
                              void* O, void* partial_O, void* partial_lse,
                              float sm_scale,
                              int B, int n_h, int c, int n_rope,
                              int M_cur, int swa_len,
                              void* stream) {
    if (B <= 0 || B > 65535 || n_h <= 0 || c != 448 || n_rope != 64) return int(cudaErrorInvalidValue);
    if (M_cur < 0 || swa_len < 0 || M_cur + swa_len < 1) return int(cudaErrorInvalidValue);
    if (Q == nullptr || O == nullptr || !aligned(Q, 16) || !aligned(O, 16)) return int(cudaErrorInvalidValue);
    if (!(sm_scale > 0.f) || !std::isfinite(sm_scale)) return int(cudaErrorInvalidValue);
    if (M_cur > 0 && (Kc == nullptr || Kc_s == nullptr || Kc_rope == nullptr || !aligned(Kc, 16) || !aligned(Kc_rope, 16)))
        return int(cudaErrorInvalidValue);
    if (swa_len > 0 && (Kswa == nullptr || Kswa_s == nullptr || Kswa_rope == nullptr || !aligned(Kswa, 16) ||
                        !aligned(Kswa_rope, 16)))
        return int(cudaErrorInvalidValue);

    DecodeArgs a{};
    a.B = B;  a.s_q = 1;  a.H = n_h;
    a.scale_log2 = sm_scale * 1.4426950408889634f;
    a.q = static_cast<const __nv_bfloat16*>(Q);
    a.out = static_cast<__nv_bfloat16*>(O);
    a.attn_sink = static_cast<const float*>(sink_logits);
    a.ref_kc = static_cast<const uint8_t*>(Kc);  a.ref_kc_s = static_cast<const uint8_t*>(Kc_s);
    a.ref_kc_rope = static_cast<const __nv_bfloat16*>(Kc_rope);
    a.ref_ks = static_cast<const uint8_t*>(Kswa);  a.ref_ks_s = static_cast<const uint8_t*>(Kswa_s);
    a.ref_ks_rope = static_cast<const __nv_bfloat16*>(Kswa_rope);
    a.ref_m_cur = M_cur;  a.ref_swa_len = swa_len;
    // The caller sizes the workspaces for (M_cur + swa_len) / 128 splits; never use more.
    const int caller_splits = (M_cur + swa_len) / 128;
    int splits = dsv4_attn_plan_splits(B, n_h, M_cur + swa_len, 0);
    if (splits < 1) return -splits;
    if (splits > caller_splits) splits = caller_splits;
    if (splits < 1 || partial_O == nullptr || partial_lse == nullptr || !aligned(partial_O, 16)) splits = 1;
    a.num_splits = splits;
    a.partial_o = static_cast<float*>(partial_O);
    a.partial_lse = static_cast<float*>(partial_lse);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = launch_mma<8, kSrcRef>(a, B, nullptr, s);
    if (e != cudaSuccess) return int(e);
    if (splits > 1) {
        CombineArgs cb = contiguous_combine(B, n_h, splits, a.partial_o, a.partial_lse, O, nullptr, a.attn_sink, true);
        e = launch_combine(cb, s, true);
    }
    return int(e);
}


extern "C" int dsv4_csa_compress_reduce_fwd(const Dsv4CsaCompressReduceParams* p, void* stream) {
    if (p == nullptr || p->B <= 0 || p->n <= 0 || p->c_out <= 0 || p->m <= 0) return int(cudaErrorInvalidValue);
    if (p->n % p->m != 0) return int(cudaErrorInvalidValue);
    if (p->C_a == nullptr || p->C_b == nullptr || p->Z_a == nullptr || p->Z_b == nullptr || p->B_a == nullptr ||
        p->B_b == nullptr || p->out == nullptr)
        return int(cudaErrorInvalidValue);
    if (p->m != 4) return int(cudaErrorNotSupported);      // as in the reference, only m = 4 is instantiated
    CompressReduceArgs a{};
    a.B = p->B;  a.n = p->n;  a.n_blocks = p->n / p->m;  a.c_out = p->c_out;  a.m = p->m;
    a.C_a = static_cast<const __nv_bfloat16*>(p->C_a);  a.C_b = static_cast<const __nv_bfloat16*>(p->C_b);
    a.Z_a = static_cast<const __nv_bfloat16*>(p->Z_a);  a.Z_b = static_cast<const __nv_bfloat16*>(p->Z_b);
    a.B_a = static_cast<const __nv_bfloat16*>(p->B_a);  a.B_b = static_cast<const __nv_bfloat16*>(p->B_b);
    a.out = static_cast<__nv_bfloat16*>(p->out);
    a.stride_c_b = p->stride_C_b;  a.stride_c_n = p->stride_C_n;
    a.stride_out_b = p->stride_out_b;  a.stride_out_blk = p->stride_out_blk;
    const bool vec = (p->c_out % 8 == 0) && (p->stride_C_b % 8 == 0) && (p->stride_C_n % 8 == 0) &&
                     (p->stride_out_b % 8 == 0) && (p->stride_out_blk % 8 == 0) && aligned(p->C_a, 16) &&
                     aligned(p->C_b, 16) && aligned(p->Z_a, 16) && aligned(p->Z_b, 16) && aligned(p->B_a, 16) &&
                     aligned(p->B_b, 16) && aligned(p->out, 16);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t items = int64_t(a.B) * a.n_blocks * (vec ? a.c_out / 4 : a.c_out);
    const int64_t want = (items + kCompressThreads - 1) / kCompressThreads;
    // at most 8 blocks per SM (two waves of the 4 resident ones); beyond that the grid-stride loop takes over
    const int64_t cap = int64_t(sms) * 8;
    const int blocks = int(want < cap ? (want > 0 ? want : 1) : cap);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (vec) compress_reduce_kernel<4, 4><<<blocks, kCompressThreads, 0, s>>>(a);
    else compress_reduce_kernel<4, 1><<<blocks, kCompressThreads, 0, s>>>(a);
    return int(cudaGetLastError());
}


static bool fill_cache_dest(const Dsv4CacheDest* d, int B, CacheDest& out) {
    if (d == nullptr || d->kv_pool == nullptr || d->block_table == nullptr || d->insert_pos == nullptr) return false;
    if (d->max_pages <= 0 || d->num_pages <= 0 || !aligned(d->kv_pool, 16)) return false;
    (void)B;
    out.kv_pool = static_cast<uint8_t*>(d->kv_pool);
    out.block_table = d->block_table;
    out.insert_pos = d->insert_pos;
    out.max_pages = d->max_pages;
    out.num_pages = d->num_pages;
    out.status = d->status;
    return true;
}

extern "C" int dsv4_hca_compress_fwd(const Dsv4HcaCompressParams* p, void* stream) {
    if (p == nullptr || p->B <= 0 || p->n <= 0 || p->c <= 0 || p->m <= 0) return int(cudaErrorInvalidValue);
    if (p->n % p->m != 0 || p->c % 8 != 0) return int(cudaErrorInvalidValue);
    if (p->C == nullptr || p->Z == nullptr || p->bias == nullptr) return int(cudaErrorInvalidValue);
    if (p->out == nullptr && p->dst == nullptr) return int(cudaErrorInvalidValue);
    if (p->stride_b % 8 != 0 || p->stride_n % 8 != 0 || !aligned(p->C, 16) || !aligned(p->Z, 16) || !aligned(p->bias, 16) ||
        (p->out != nullptr && !aligned(p->out, 16)))
        return int(cudaErrorInvalidValue);
    HcaCompressArgs a{};
    a.B = p->B;  a.n = p->n;  a.n_blocks = p->n / p->m;  a.c = p->c;  a.m = p->m;
    a.C = static_cast<const __nv_bfloat16*>(p->C);
    a.Z = static_cast<const __nv_bfloat16*>(p->Z);
    a.bias = static_cast<const __nv_bfloat16*>(p->bias);
    a.stride_b = p->stride_b;  a.stride_n = p->stride_n;
    a.out = static_cast<__nv_bfloat16*>(p->out);
    a.stride_out_b = int64_t(a.n_blocks) * a.c;  a.stride_out_blk = a.c;
    if (p->dst != nullptr) {
        if (p->c != 576 || !fill_cache_dest(p->dst, p->B, a.dst)) return int(cudaErrorInvalidValue);
    }
    const int64_t rows_out = int64_t(a.B) * a.n_blocks;
    if (rows_out > 0x7FFFFFFF) return int(cudaErrorInvalidValue);
    const dim3 grid(unsigned(rows_out), unsigned((a.c / 8 + kHcaVecsPerBlock - 1) / kHcaVecsPerBlock), 1);
    if (grid.y > 65535u) return int(cudaErrorInvalidValue);
    hca_compress_kernel<<<grid, kHcaCompressThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return int(cudaGetLastError());
}

extern "C" int dsv4_kv_quantize_insert(const Dsv4KvQuantizeInsertParams* p, void* stream) {
    if (p == nullptr || p->B <= 0 || p->T <= 0 || p->rows == nullptr) return int(cudaErrorInvalidValue);
    if (p->stride_b % 8 != 0 || p->stride_t % 8 != 0 || !aligned(p->rows, 16)) return int(cudaErrorInvalidValue);
    KvInsertArgs a{};
    a.B = p->B;  a.T = p->T;
    a.rows = static_cast<const __nv_bfloat16*>(p->rows);
    a.stride_b = p->stride_b;  a.stride_t = p->stride_t;
    a.n_rows = p->n_rows;
    if (!fill_cache_dest(p->dst, p->B, a.dst)) return int(cudaErrorInvalidValue);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t rows = int64_t(a.B) * a.T;
    const int64_t want = (rows + kInsertThreads / 32 - 1) / (kInsertThreads / 32);
    const int64_t cap = int64_t(sms) * 8;
    const int blocks = int(want < cap ? want : cap);
    kv_quantize_insert_kernel<<<blocks, kInsertThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return int(cudaGetLastError());
}


extern "C" int dsv4_hca_packed_decode_fwd(const Dsv4HcaPackedDecodeParams* p, void* stream) {
    if (p == nullptr || p->B <= 0 || p->B > 65535 || p->H <= 0) return int(cudaErrorInvalidValue);
    if (p->page_size != 16 && p->page_size != 32 && p->page_size != 64) return int(cudaErrorInvalidValue);
    if (p->q == nullptr || p->out == nullptr || !aligned(p->q, 16) || !aligned(p->out, 16)) return int(cudaErrorInvalidValue);
    if (p->m_cur == nullptr || p->swa_len == nullptr) return int(cudaErrorInvalidValue);
    if (!(p->sm_scale > 0.f) || !std::isfinite(p->sm_scale)) return int(cudaErrorInvalidValue);
    // a leg may be absent altogether (null pool): its lengths must then be zero, which only the caller can know
    if (p->kv_pages != nullptr && (p->block_table == nullptr || p->max_pages <= 0 || p->num_pages <= 0 || !aligned(p->kv_pages, 64)))
        return int(cudaErrorInvalidValue);
    if (p->swa_pages != nullptr && (p->swa_block_table == nullptr || p->swa_max_pages <= 0 || p->swa_num_pages <= 0 ||
                                    !aligned(p->swa_pages, 64)))
        return int(cudaErrorInvalidValue);
    if (p->kv_pages == nullptr && p->swa_pages == nullptr) return int(cudaErrorInvalidValue);
    if (p->num_splits < 1 || p->num_splits > DSV4_MAX_SPLITS) return int(cudaErrorInvalidValue);
    if (p->num_splits > 1 && (p->partial_o == nullptr || p->partial_lse == nullptr || !aligned(p->partial_o, 16)))
        return int(cudaErrorInvalidValue);

    DecodeArgs a{};
    a.B = p->B;  a.s_q = 1;  a.H = p->H;
    a.scale_log2 = p->sm_scale * 1.4426950408889634f;
    a.q = static_cast<const __nv_bfloat16*>(p->q);
    a.out = static_cast<__nv_bfloat16*>(p->out);
    a.lse = p->lse;
    a.attn_sink = p->attn_sink;
    a.kv_len = p->m_cur;  a.win_len = p->swa_len;
    a.block_table = p->block_table;  a.max_pages = p->max_pages;
    a.pg_kv = static_cast<const uint8_t*>(p->kv_pages);
    a.pg_swa = static_cast<const uint8_t*>(p->swa_pages);
    a.pg_swa_table = p->swa_block_table;  a.pg_swa_max_pages = p->swa_max_pages;
    a.pg_page_shift = p->page_size == 64 ? 6 : (p->page_size == 32 ? 5 : 4);
    a.pg_page_bytes = int64_t(p->page_size) * 584;
    a.pg_num_pages = p->num_pages;  a.pg_swa_num_pages = p->swa_num_pages;
    a.num_splits = p->num_splits;
    a.partial_o = p->partial_o;  a.partial_lse = p->partial_lse;
    a.status = p->status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = launch_mma<8, kSrcRefPaged>(a, p->B, nullptr, s);
    if (e != cudaSuccess) return int(e);
    if (a.num_splits > 1) {
        CombineArgs cb = contiguous_combine(p->B, p->H, a.num_splits, a.partial_o, a.partial_lse, a.out, a.lse, a.attn_sink,
                                            true);
        e = launch_combine(cb, s, true);
    }
    return int(e);
}


extern "C" int dsv4_rope_norm_fwd(const Dsv4RopeNormParams* p, void* stream) {
    if (p == nullptr || p->n_rows <= 0 || p->vecs_per_row <= 0 || p->x == nullptr || p->out == nullptr || p->positions == nullptr)
        return int(cudaErrorInvalidValue);
    if (p->n_rope != 64 || p->c < p->n_rope || (p->c - p->n_rope) % 8 != 0 || p->c - p->n_rope > 512) return int(cudaErrorInvalidValue);
    if (!aligned(p->x, 16) || !aligned(p->out, 16) || (p->norm_weight != nullptr && !aligned(p->norm_weight, 16))) return int(cudaErrorInvalidValue);
    if (!(p->theta > 1.f) || !std::isfinite(p->theta) || !(p->eps >= 0.f)) return int(cudaErrorInvalidValue);
    RopeNormArgs a{};
    a.n_rows = p->n_rows;  a.vecs_per_row = p->vecs_per_row;  a.c = p->c;  a.n_rope = p->n_rope;  a.inverse = p->inverse ? 1 : 0;
    a.eps = p->eps;  a.theta = p->theta;
    a.x = static_cast<const __nv_bfloat16*>(p->x);
    a.out = static_cast<__nv_bfloat16*>(p->out);
    a.positions = p->positions;
    a.weight = static_cast<const __nv_bfloat16*>(p->norm_weight);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t items = a.n_rows * ((a.vecs_per_row + kRopeGroup - 1) / kRopeGroup);
    const int64_t want = (items + kRopeNormThreads / 32 - 1) / (kRopeNormThreads / 32);
    const int64_t cap = int64_t(sms) * 8;
    rope_norm_kernel<<<int(want < cap ? want : cap), kRopeNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return int(cudaGetLastError());
}


namespace {
cudaError_t make_byte_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows, bool swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {128, cuuint64_t(rows)};
    const cuuint64_t strides[1] = {128};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}
}  // namespace

extern "C" int dsv4_indexer_topk_fwd(const Dsv4IndexerTopkParams* p, void* stream) {
    if (p == nullptr || p->B <= 0 || p->B > 65535 || (p->s_q != 1 && p->s_q != 2) || p->max_pages <= 0 || p->num_pages <= 0 || p->k <= 0)
        return int(cudaErrorInvalidValue);
    if (p->q_fp8 == nullptr || p->q_weight == nullptr || p->key_pages == nullptr || p->block_table == nullptr || p->n_vis == nullptr ||
        p->scores == nullptr || p->out_indices == nullptr)
        return int(cudaErrorInvalidValue);
    if (!aligned(p->q_fp8, 128) || !aligned(p->key_pages, 128) || !aligned(p->scores, 16)) return int(cudaErrorInvalidValue);
    if (p->score_stride < int64_t(p->max_pages) * kIdxPageKeys) return int(cudaErrorInvalidValue);
    if (p->num_pages * kIdxPageRows > 0x7FFFFFFFll) return int(cudaErrorInvalidValue);      // TMA coordinates are 32-bit
    IndexerArgs a{};
    cudaError_t e = make_byte_map(&a.key_map, p->key_pages, uint64_t(p->num_pages) * kIdxPageRows, kIdxPageKeys, true);
    if (e == cudaSuccess) e = make_byte_map(&a.scale_map, p->key_pages, uint64_t(p->num_pages) * kIdxPageRows, 2, false);
    if (e == cudaSuccess) e = make_byte_map(&a.q_map, p->q_fp8, uint64_t(p->B) * p->s_q * kIdxHeads, uint32_t(p->s_q * kIdxHeads), true);
    if (e != cudaSuccess) return int(e);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles_cap = (p->max_pages + 1) / 2;
    // Blocks per request: two blocks are resident per SM; the time is (waves of resident blocks) x
    // (tiles per block + a fixed set-up of about two tiles).  Pick the count that minimises it.
    int ctas = 1;
    {
        const int64_t slots = 2 * int64_t(sms);
        double best = 1e300;
        const int c_max = tiles_cap < 64 ? tiles_cap : 64;
        for (int c = 1; c <= c_max; ++c) {
            const int tpc = (tiles_cap + c - 1) / c;
            const int64_t blocks = int64_t(p->B) * ((tiles_cap + tpc - 1) / tpc);
            const double cost = double((blocks + slots - 1) / slots) * (tpc + 2.0);
            if (cost < best - 1e-9) { best = cost;  ctas = c; }
        }
    }
    a.tiles_per_cta = (tiles_cap + ctas - 1) / ctas;
    const int grid_x = (tiles_cap + a.tiles_per_cta - 1) / a.tiles_per_cta;
    a.B = p->B;  a.s_q = p->s_q;  a.max_pages = p->max_pages;  a.num_pages = p->num_pages;
    a.q_weight = p->q_weight;  a.block_table = p->block_table;  a.n_vis = p->n_vis;
    a.scores = p->scores;  a.score_stride = p->score_stride;  a.status = p->status;
    a.wait_ns = g_wait_ns.load(std::memory_order_relaxed);
    a.dbg_drop_tile = g_drop_tile.load(std::memory_order_relaxed);
    static std::atomic<bool> done[kMaxDevices];
    e = ensure_smem(indexer_logits_kernel, kIdxSmemBytes, done);
    if (e != cudaSuccess) return int(e);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    indexer_logits_kernel<<<dim3(grid_x, p->B), kIdxThreads, kIdxSmemBytes, s>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return int(e);
    TopkArgs t{};
    t.rows = p->B * p->s_q;  t.k = p->k;  t.scores = p->scores;  t.stride = p->score_stride;  t.n_vis = p->n_vis;
    t.out = p->out_indices;  t.n_cap = p->max_pages * kIdxPageKeys;
    // With few rows a cluster pair shares each row, so that more SMs take part.  A copy of the
    // block's slice of the score row goes to shared memory when it fits next to the static 38 KB.
    const bool pair = t.rows * 2 <= sms;
    const int row_bytes = (pair ? (t.n_cap + 1) / 2 : t.n_cap) * int(sizeof(float));
    t.row_in_smem = row_bytes <= 180 * 1024 ? 1 : 0;
    static std::atomic<bool> done_topk[kMaxDevices], done_pair[kMaxDevices];
    e = pair ? ensure_smem(topk_select_pair_kernel, 180 * 1024, done_pair) : ensure_smem(topk_select_kernel, 180 * 1024, done_topk);
    if (e != cudaSuccess) return int(e);
    if (g_dbg.load(std::memory_order_relaxed) & 64) {
        if (pair) topk_select_pair_kernel<<<t.rows * 2, kTopkThreads, t.row_in_smem ? row_bytes : 0, s>>>(t);
        else topk_select_kernel<<<t.rows, kTopkThreads, t.row_in_smem ? row_bytes : 0, s>>>(t);
        return int(cudaGetLastError());
    }
    // as a programmatic dependent of the scoring kernel: resident (and waiting) when its last blocks finish
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pair ? t.rows * 2 : t.rows);
    cfg.blockDim = dim3(kTopkThreads);
    cfg.dynamicSmemBytes = t.row_in_smem ? row_bytes : 0;
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return int(pair ? cudaLaunchKernelEx(&cfg, topk_select_pair_kernel, t) : cudaLaunchKernelEx(&cfg, topk_select_kernel, t));
}

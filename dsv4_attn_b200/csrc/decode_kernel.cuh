// Decode attention over an FP8 latent KV cache on sm_100a tensor cores.
//
// One thread block handles (request-token row n, group of 128 heads, one half
// of the 512 value columns, one KV split).  Per 64-entry tile:
//   loader warps   gather the entries (index list -> block table -> 656-byte
//                  rows, or the dense / reference-layout equivalents) into
//                  registers, dequantise FP8 * scale -> BF16 and write the tile
//                  into shared memory in the 128-byte-swizzled operand layout;
//   MMA thread     S[128 heads x 64] = Q . K^T   (tcgen05.mma, BF16, K = 576
//                  or 512) into tensor memory, later O[128 x 256] += P . V with
//                  V read from the same tile as an MN-major operand;
//   softmax warps  read S from tensor memory (one head per thread), run the
//                  online softmax with a lazily updated reference maximum,
//                  write P (BF16) to shared memory, rescale O in tensor memory
//                  when the maximum moved, and finally normalise and store.
// All waits are bounded; a wait that gives up records where in `status` and the
// block leaves through the common exit, freeing its tensor memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <math_constants.h>
#include <stdint.h>
#include <type_traits>

#include "ptx.cuh"

namespace dsv4 {

constexpr int kTileN = 64;             // cache entries per tile (MMA N of S, K of PV)
constexpr int kHeadsPerCta = 128;      // MMA M
constexpr int kDvHalf = 256;           // value columns per block (MMA N of PV)
constexpr int kQChunkBytes = 128 * 128;   // 128 heads x 64 bf16
constexpr int kKvChunkBytes = kTileN * 128;  // 64 entries x 64 bf16
// Warp roles, four warpgroups of four warps.  Warps 0-3: softmax + epilogue.
// Warps 4-11: loaders.  Warp 12: issue of the S = Q.K^T MMAs and tensor-memory allocation;
// warp 13: issue of the O += P.V MMAs (its own thread, so that a ready P never waits for the
// other thread to finish issuing a group: an issuing thread is held while the tensor pipe's
// short queue is full); warps 14-15 only take part in the block-wide barriers.  All 16 warps start with 128
// registers (the whole register file); the last warpgroup gives most of its
// share back and the loaders take it, so that they can hold two tiles of cache
// entries in flight.  setmaxnreg.inc waits for registers without a time limit,
// so the matching .dec must be reached unconditionally, as it is here.
constexpr int kNumSoftmaxWarps = 4;
constexpr int kNumLoaderWarps = 8;
constexpr int kFirstLoaderWarp = 4;
constexpr int kMmaWarp = 12;
constexpr int kNumWarps = 16;
constexpr int kStageThreads = (kNumSoftmaxWarps + kNumLoaderWarps) * 32;   // threads that stage Q
constexpr int kLoaderRegs = 160;       // 8 x 32 x (160-128) = 8192 registers taken ...
constexpr int kIdleRegs = 64;          // ... from 4 x 32 x (128-64) = 8192 released
constexpr int kNumThreads = kNumWarps * 32;  // 512
constexpr int kNumKvGroups = 2;        // hand-overs per tile from the loaders to the MMA thread
constexpr int kQTmemChunks = 4;        // Q chunks (64 columns each) held in tensor memory as the A operand
constexpr int kTmemCols = 512;
constexpr int kTmemS = 0;              // two S accumulators of 64 columns; P (BF16) overwrites the first 32 of its S
constexpr int kTmemO = 128;            // O accumulator: 256 columns
constexpr int kTmemQ = 384;            // Q chunks 0..3 as packed BF16: 4 x 32 columns
constexpr uint64_t kWaitTimeoutNs = 2000000000ull;  // 2 s
constexpr float kRescaleThreshold = 8.0f;  // log2 units; O is rescaled only when the max grows by more

enum SourceKind : int {
    kSrcCsa = 0,   // index list + block table, packed 656-byte entries
    kSrcHca = 1,   // dense [0, kv_len) through the block table, then the window buffer
    kSrcRef = 2,   // reference layout: separate planes, 448 e4m3 + 7 UE8M0 + 64 bf16
    kSrcRefPaged = 3,   // the same bytes in packed pages: per page, page_size tokens of [448 e4m3 | 64 bf16]
                        // followed by page_size x 8 scale bytes (7 UE8M0 + 1 pad), behind block tables
};

// both kinds with the reference's quantisation (448 latent elements, one UE8M0 byte per 64)
__host__ __device__ constexpr bool is_ref_layout(int src) { return src == kSrcRef || src == kSrcRefPaged; }

// Operand format of the MMAs.  The packed 656-byte layout goes through FP16: FP8 -> FP16 is one
// exact conversion instruction per two elements and one packed multiply by the scale (the BF16
// route costs five integer/FP instructions per two elements, and that arithmetic is a third of
// the loaders' time), and FP16 keeps three more mantissa bits of fp8 x scale than BF16.  Q
// and P are converted to FP16 as well (exact for Q inside FP16's normal range; P <= 2^8).
// Limits: |q| below 65504; block scales above 146 (entries beyond +-65408) are clamped to 146 (the
// BF16 route's own limit on scales is 128).
// The reference layouts keep BF16: their power-of-two scales span BF16's exponent range.
__host__ __device__ constexpr bool use_f16(int src) { return !is_ref_layout(src); }

enum StatusCode : int {
    kStatusOk = 0,
    kStatusWaitKvFull = 1,
    kStatusWaitKvFree = 2,
    kStatusWaitSFull = 3,
    kStatusWaitPFull = 4,
    kStatusWaitOFull = 5,
    kStatusWaitQ = 6,
};

struct DecodeArgs {
    // TMA descriptor of Q viewed as [rows = B*s_q*H, cols = 64*NCHUNK] bf16, box 64 x 128, 128-byte swizzle
    alignas(64) CUtensorMap q_map;
    int B, s_q, H;
    int topk;            // CSA
    int max_pages;
    int win_cap;         // HCA
    int num_splits;
    float scale_log2;    // sm_scale * log2(e)
    const __nv_bfloat16* q;
    const uint8_t* kv_pool;
    const int32_t* block_table;
    const int32_t* indices;
    const int32_t* kv_len;
    const int32_t* topk_len;
    const uint8_t* win_pool;
    const int32_t* win_len;
    const float* attn_sink;
    __nv_bfloat16* out;
    float* lse;
    float* partial_o;
    float* partial_lse;
    int32_t* status;
    int partial_f32;             // split partials as FP32 (default: BF16 in the same workspace)
    int dbg;                     // profiling aid: bit1 no L2 prefetch
    unsigned long long* trace;   // optional profiling aid: block (0,0,0) records phase times here
    // reference layout planes (kSrcRef)
    const uint8_t* ref_kc;  const uint8_t* ref_kc_s;  const __nv_bfloat16* ref_kc_rope;
    const uint8_t* ref_ks;  const uint8_t* ref_ks_s;  const __nv_bfloat16* ref_ks_rope;
    int ref_m_cur, ref_swa_len;
    // packed pages (kSrcRefPaged): two pools (compressed cache, sliding window) with their block tables;
    // per-request lengths come through kv_len / win_len
    const uint8_t* pg_kv;  const uint8_t* pg_swa;
    const int32_t* pg_swa_table;
    int pg_swa_max_pages;
    int pg_page_shift;           // log2(page_size), page_size <= 64
    int64_t pg_page_bytes;       // page_size * 584
    int64_t pg_num_pages, pg_swa_num_pages;
};

template <int NCHUNK>
struct SmemLayout {
    static constexpr int kQSmemChunks = NCHUNK - kQTmemChunks;      // Q chunks kept in shared memory
    static constexpr int kQBytes = kQSmemChunks * kQChunkBytes;
    static constexpr int kKvStageBytes = NCHUNK * kKvChunkBytes;
    static constexpr int kQOff = 0;
    static constexpr int kKvOff = kQBytes;                          // two stages
    static constexpr int kMiscOff = kKvOff + 2 * kKvStageBytes;
    static constexpr int kMiscBytes = 512;
    static constexpr int kTotal = kMiscOff + kMiscBytes + 1024;     // + slack to align the base to 1024
    // the Q chunks bound for tensor memory are staged (as swizzled 16 KB chunks) in KV stage 1,
    // which the loaders do not touch before the copy to tensor memory has finished
    static constexpr int kQStageOff = kKvOff + kKvStageBytes;
    static_assert(kQTmemChunks * kQChunkBytes <= kKvStageBytes, "Q staging must fit in one KV stage");
};

struct SmemMisc {
    uint64_t bar_kv_full[2][10];   // [stage][chunk]: chunk written by all loader warps
    uint64_t bar_kv_free[2];
    uint64_t bar_s_full[2];
    uint64_t bar_p_full[2];
    uint64_t bar_o_full;
    uint64_t bar_q_full;      // Q tile landed in shared memory (TMA transaction count)
    uint64_t bar_q_ready;     // Q chunks copied to tensor memory, staging area released
    uint64_t valid_mask[2];   // per stage: bit t = entry t of the tile takes part in the softmax
    uint32_t tmem_base;
    uint32_t pad;
    // cluster-pair kernel: per stage, byte i = 4-bit mask of tile rows 4 i .. 4 i + 3 (written by the
    // loader warp that owns them, in either block of the pair)
    alignas(16) uint8_t valid_bytes[2][16];
    uint64_t bar_loc[2][4];   // [stage][span]: this block's loader warps have written their half of chunks 2 span, 2 span + 1 (span 3: and the RoPE tail)
};

__device__ __forceinline__ void report_timeout(int32_t* status, int code, int role, int tile) {
    if (status != nullptr) {
        if (atomicCAS(status, 0, code) == 0) {
            status[1] = int(blockIdx.x) | (int(blockIdx.y) << 8) | (int(blockIdx.z) << 20);
            status[2] = role;
            status[3] = tile;
        }
    }
}

// Profiling aid: block (0,0,0) stores %globaltimer values, 1024 slots per role
// (0 softmax, 1 MMA, 2 loader, 3 block phases).
__device__ __forceinline__ void trace_mark(const DecodeArgs& a, int role, int slot) {
    if (a.trace != nullptr && (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && slot < 1024)
        a.trace[role * 1024 + slot] = ptx::globaltimer_ns();
}

// Start (which = 0) and end (1) time of every block, in the last quarter of the trace buffer.
__device__ __forceinline__ void trace_block(const DecodeArgs& a, int which) {
    const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (a.trace != nullptr && lin < 240) a.trace[3 * 1024 + 512 + 2 * lin + which] = ptx::globaltimer_ns();
}

// Two FP8 e4m3 bytes sitting in bits [15:8] and [31:24] of `r` -> two BF16 bit
// patterns whose values are the FP8 values times 2^-120 (the e4m3 exponent and
// mantissa bits dropped into the BF16 exponent/mantissa fields; e4m3
// subnormals become BF16 subnormals, so one multiply fixes both).
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2_bits(uint32_t r) {
    return (r & 0x80008000u) | ((r >> 4) & 0x07F007F0u);
}

// Four FP8 e4m3 (one 32-bit word) times the block scale -> 4 BF16 (two packed
// words).  `scale2` holds scale * 2^120 in both halves; integer ALU plus one
// packed BF16 multiply per pair (no slow-rate conversion instructions).
__device__ __forceinline__ void dequant4(uint32_t w, __nv_bfloat162 scale2, uint32_t& lo, uint32_t& hi) {
    uint32_t r01 = e4m3x2_to_bf16x2_bits(__byte_perm(w, 0u, 0x1404u));
    uint32_t r23 = e4m3x2_to_bf16x2_bits(__byte_perm(w, 0u, 0x3424u));
    __nv_bfloat162 a = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&r01), scale2);
    __nv_bfloat162 b = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&r23), scale2);
    lo = *reinterpret_cast<uint32_t*>(&a);
    hi = *reinterpret_cast<uint32_t*>(&b);
}

// Four FP8 e4m3 (one 32-bit word) times the block scale -> 4 FP16 (two packed words).
__device__ __forceinline__ void dequant4_f16(uint32_t w, __half2 scale2, uint32_t& lo, uint32_t& hi) {
    const uint32_t a = ptx::e4m3x2_to_f16x2(w & 0xFFFFu), b = ptx::e4m3x2_to_f16x2(w >> 16);
    const __half2 x = __hmul2(*reinterpret_cast<const __half2*>(&a), scale2);
    const __half2 y = __hmul2(*reinterpret_cast<const __half2*>(&b), scale2);
    lo = *reinterpret_cast<const uint32_t*>(&x);
    hi = *reinterpret_cast<const uint32_t*>(&y);
}

// Registers one loader thread holds for one tile.  A loader warp owns 8
// consecutive entries of the tile, as two groups of 4: lane/8 picks the entry of
// a group and lane%8 one 16-byte piece of a 128-byte span (two 64-element latent
// chunks, or the RoPE tail).  One load instruction then covers 4 entries x 128
// contiguous bytes: measured on this part, an SM pulls records about 1.6 times
// faster in this shape than with 64 bytes per entry per instruction, and the
// record fetch is what the loader warps spend most of their time on.
//
// G = 2 groups (8 entries per warp) in the ordinary kernel; G = 1 (4 entries per warp) when the
// two blocks of a cluster pair share the work: each block then fetches and dequantises half of
// every tile and forwards it to the other block.
template <int SRC, int G = 2>
struct LoaderRegs {
    uint4 lat[G][4];         // [group][span j]: bytes [128 j + 16 (lane%8), +16) of the latent of entry 4 group + lane/8
    uint4 rope[G];           // [group]: RoPE 16-byte column lane%8 of that entry
    uint32_t sc[G][4];       // [group]: packed layout: the 4 FP32 scales; reference layout: the 7 UE8M0 bytes (2 words)
    uint32_t vmask;          // bit i = entry i of this warp takes part (same in all lanes)
};

// Where an entry lives: for the packed layouts the address of its 656-byte
// record; for the reference layout its row number in the plane, with bit 62 set
// for the sliding-window planes.  Lanes 0..7 of a loader warp resolve the warp's
// 8 entries one tile ahead of the data loads, so that the index -> block table
// -> row dependency chain is off the critical path.
template <int SRC>
__device__ __forceinline__ unsigned long long loader_resolve(const DecodeArgs& a, int b, int n, int v, int n_tok,
                                                             int kv_len_n, bool& valid) {
    valid = v < n_tok;
    unsigned long long key = 0;
    if constexpr (SRC == kSrcCsa) {
        int e = -1;
        if (valid) e = __ldg(a.indices + int64_t(n) * a.topk + v);
        valid = (e >= 0) && (e < kv_len_n);
        if (valid) {
            const int page = __ldg(a.block_table + int64_t(b) * a.max_pages + (e >> 6));
            key = reinterpret_cast<unsigned long long>(a.kv_pool + (int64_t(page) * 64 + (e & 63)) * 656);
        }
    } else if constexpr (SRC == kSrcHca) {
        if (valid) {
            if (v < kv_len_n) {
                const int page = __ldg(a.block_table + int64_t(b) * a.max_pages + (v >> 6));
                key = reinterpret_cast<unsigned long long>(a.kv_pool + (int64_t(page) * 64 + (v & 63)) * 656);
            } else {
                key = reinterpret_cast<unsigned long long>(a.win_pool + (int64_t(b) * a.win_cap + (v - kv_len_n)) * 656);
            }
        }
    } else if constexpr (SRC == kSrcRefPaged) {
        // key = address of the token's 576 data bytes (a multiple of 64) | slot of the token in its page
        // a token outside its block table, or a table value outside the pool, is left out of the
        // softmax instead of being read
        if (valid) {
            const int slot_mask = (1 << a.pg_page_shift) - 1;
            const bool swa = v >= kv_len_n;
            const int w = swa ? v - kv_len_n : v;
            const uint8_t* pool = swa ? a.pg_swa : a.pg_kv;
            const int32_t* table = swa ? a.pg_swa_table : a.block_table;
            const int cols = swa ? a.pg_swa_max_pages : a.max_pages;
            const int64_t pages = swa ? a.pg_swa_num_pages : a.pg_num_pages;
            valid = pool != nullptr && (w >> a.pg_page_shift) < cols;
            if (valid) {
                const int page = __ldg(table + int64_t(b) * cols + (w >> a.pg_page_shift));
                valid = page >= 0 && page < pages;
                if (valid)
                    key = reinterpret_cast<unsigned long long>(pool + int64_t(page) * a.pg_page_bytes + (w & slot_mask) * 576) |
                          (unsigned long long)(w & slot_mask);
            }
        }
    } else {
        if (valid) {
            key = (v < a.ref_m_cur) ? (unsigned long long)(int64_t(b) * a.ref_m_cur + v)
                                    : ((unsigned long long)(int64_t(b) * a.ref_swa_len + (v - a.ref_m_cur)) | (1ull << 62));
        }
    }
    return key;
}

// Two entries at once, with the two chains of dependent loads side by side.
template <int SRC>
__device__ __forceinline__ void loader_resolve2(const DecodeArgs& a, int b, int n, int va, int ntok_a, int vb, int ntok_b,
                                                int kv_len_n, unsigned long long& key_a, bool& valid_a,
                                                unsigned long long& key_b, bool& valid_b) {
    if constexpr (SRC == kSrcCsa) {
        valid_a = va < ntok_a;
        valid_b = vb < ntok_b;
        const int ea = valid_a ? __ldg(a.indices + int64_t(n) * a.topk + va) : -1;
        const int eb = valid_b ? __ldg(a.indices + int64_t(n) * a.topk + vb) : -1;
        valid_a = (ea >= 0) && (ea < kv_len_n);
        valid_b = (eb >= 0) && (eb < kv_len_n);
        const int pa = valid_a ? __ldg(a.block_table + int64_t(b) * a.max_pages + (ea >> 6)) : 0;
        const int pb = valid_b ? __ldg(a.block_table + int64_t(b) * a.max_pages + (eb >> 6)) : 0;
        key_a = valid_a ? reinterpret_cast<unsigned long long>(a.kv_pool + (int64_t(pa) * 64 + (ea & 63)) * 656) : 0ull;
        key_b = valid_b ? reinterpret_cast<unsigned long long>(a.kv_pool + (int64_t(pb) * 64 + (eb & 63)) * 656) : 0ull;
    } else {
        key_a = loader_resolve<SRC>(a, b, n, va, ntok_a, kv_len_n, valid_a);
        key_b = loader_resolve<SRC>(a, b, n, vb, ntok_b, kv_len_n, valid_b);
    }
}

// Warp-wide: resolve the 8 entries [v0, v0+8) (lanes 0..7), return the key in
// those lanes and the valid mask in all lanes.
template <int SRC, int E = 8>
__device__ __forceinline__ unsigned long long loader_resolve_warp(const DecodeArgs& a, int b, int n, int v0, int lane,
                                                                  int n_tok, int kv_len_n, uint32_t& vmask) {
    bool valid = false;
    unsigned long long key = 0;
    if (lane < E) key = loader_resolve<SRC>(a, b, n, v0 + lane, n_tok, kv_len_n, valid);
    vmask = __ballot_sync(0xFFFFFFFFu, valid) & 0xFFu;
    return key;
}

// Issue the loads of one tile for this lane's two entries (keys held by lanes 0..7).
template <int SRC, int G>
__device__ __forceinline__ void loader_fetch(const DecodeArgs& a, unsigned long long key, uint32_t vmask, int lane,
                                             LoaderRegs<SRC, G>& r) {
    r.vmask = vmask;
    const int piece = lane & 7;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int i = 4 * g + (lane >> 3);
        const unsigned long long k = __shfl_sync(0xFFFFFFFFu, key, i);
        if (!((vmask >> i) & 1u)) continue;
        if constexpr (!is_ref_layout(SRC)) {
            const uint8_t* row = reinterpret_cast<const uint8_t*>(k);
#pragma unroll
            for (int j = 0; j < 4; ++j) r.lat[g][j] = ptx::ldg_nc_v4(row + j * 128 + piece * 16);
            const uint4 s4 = ptx::ldg_nc_v4(row + 512);
            r.sc[g][0] = s4.x;  r.sc[g][1] = s4.y;  r.sc[g][2] = s4.z;  r.sc[g][3] = s4.w;
            r.rope[g] = ptx::ldg_nc_v4(row + 528 + piece * 16);
        } else if constexpr (SRC == kSrcRefPaged) {
            const int slot = int(k & 63ull);
            const uint8_t* lp = reinterpret_cast<const uint8_t*>(k & ~63ull);
            // the page's scale area starts after its page_size tokens: 8 bytes per token
            const uint8_t* sp = lp + int64_t((1 << a.pg_page_shift) - slot) * 576 + slot * 8;
#pragma unroll
            for (int j = 0; j < 3; ++j) r.lat[g][j] = ptx::ldg_nc_v4(lp + j * 128 + piece * 16);
            if (piece < 4) r.lat[g][3] = ptx::ldg_nc_v4(lp + 384 + piece * 16);
            const uint2 s2 = __ldg(reinterpret_cast<const uint2*>(sp));
            r.sc[g][0] = s2.x;  r.sc[g][1] = s2.y;
            r.rope[g] = ptx::ldg_nc_v4(lp + 448 + piece * 16);
        } else {
            const bool swa = (k >> 62) & 1ull;
            const int64_t e = int64_t(k & ~(1ull << 62));
            const uint8_t* lp = (swa ? a.ref_ks : a.ref_kc) + e * 448;
            const uint8_t* sp = (swa ? a.ref_ks_s : a.ref_kc_s) + e * 7;
            const uint8_t* rp = reinterpret_cast<const uint8_t*>(swa ? a.ref_ks_rope : a.ref_kc_rope) + e * 128;
#pragma unroll
            for (int j = 0; j < 3; ++j) r.lat[g][j] = ptx::ldg_nc_v4(lp + j * 128 + piece * 16);
            // the last span holds only chunk 6 (bytes 384..447 of the 448-byte row)
            if (piece < 4) r.lat[g][3] = ptx::ldg_nc_v4(lp + 384 + piece * 16);
            uint32_t s0 = 0, s1 = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) s0 |= uint32_t(__ldg(sp + j)) << (8 * j);
#pragma unroll
            for (int j = 0; j < 3; ++j) s1 |= uint32_t(__ldg(sp + 4 + j)) << (8 * j);
            r.sc[g][0] = s0;  r.sc[g][1] = s1;
            r.rope[g] = ptx::ldg_nc_v4(rp + piece * 16);
        }
    }
}

// Pull the 656-byte records of the warp's 8 entries (keys in lanes 0..7) into L2
// ahead of the loads: lane/4 picks the entry, lane%4 the 128-byte piece.
template <int SRC>
__device__ __forceinline__ void loader_prefetch_l2(unsigned long long key, uint32_t vmask, int lane) {
    if constexpr (!is_ref_layout(SRC)) {
        const int i = lane >> 2;
        const unsigned long long k = __shfl_sync(0xFFFFFFFFu, key, i);
        if ((vmask >> i) & 1u) {
            const uint8_t* row = reinterpret_cast<const uint8_t*>(k);
            ptx::prefetch_l2(row + (lane & 3) * 128);
            if ((lane & 3) < 2) ptx::prefetch_l2(row + 512 + (lane & 3) * 128);
        }
    } else if constexpr (SRC == kSrcRefPaged) {
        const int i = lane >> 2;
        const unsigned long long k = __shfl_sync(0xFFFFFFFFu, key, i);
        if ((vmask >> i) & 1u) {
            const uint8_t* lp = reinterpret_cast<const uint8_t*>(k & ~63ull);
            ptx::prefetch_l2(lp + (lane & 3) * 128);
            if ((lane & 3) == 0) ptx::prefetch_l2(lp + 512);
        }
    }
}

// Dequantise and write span j (latent chunks 2j and 2j+1) of this warp's 8 entries
// (tile rows t0 .. t0+7, t0 a multiple of 8) into the KV stage at kv_st.  Row t of a
// chunk is 128 bytes; 16-byte column c16 of row t lives at ((c16 ^ (t & 7)) << 4).
// One store instruction writes 4 rows x 2 chunks x 4 column positions, arranged
// (see the end of the function) so that it needs as few shared-memory wavefronts
// as 512 bytes can: four.
template <int NCHUNK, int SRC, int G>
__device__ __forceinline__ void loader_store_span(uint32_t kv_st, int t0, int lane, const LoaderRegs<SRC, G>& r, int j) {
    const uint32_t piece = uint32_t(lane & 7);
    const uint32_t c = 2u * uint32_t(j) + (piece >> 2);        // this lane's chunk
    const uint32_t p = piece & 3u;                             // 16 latent bytes -> 16-byte columns 2p, 2p+1
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int i = 4 * g + (lane >> 3);
        const int t = t0 + i;
        const bool valid = (r.vmask >> i) & 1u;
        const uint32_t base = kv_st + c * kKvChunkBytes + uint32_t(t) * 128u;
        const uint32_t sw = uint32_t(t & 7);
        if (is_ref_layout(SRC) && c >= uint32_t(NCHUNK - 1)) continue;   // reference layout: span 3 ends with chunk 6
        uint4 w0 = make_uint4(0, 0, 0, 0), w1 = make_uint4(0, 0, 0, 0);
        if (valid) {
            float s120;
            if constexpr (is_ref_layout(SRC)) {
                // one UE8M0 byte per 64 elements: 2^(byte-127) * 2^120; a zero byte means a zero
                // scale, as in the reference's dequantiser
                const uint32_t byte = ((c < 4u ? r.sc[g][0] >> (8u * c) : r.sc[g][1] >> (8u * (c - 4u))) & 0xFFu);
                s120 = byte ? __uint_as_float((byte + 120u) << 23) : 0.f;
            } else {
                s120 = __uint_as_float(r.sc[g][j]) * 1.329227995784916e36f;   // one FP32 scale per 128 elements; x 2^120
            }
            const uint4 x = r.lat[g][j];
            if constexpr (use_f16(SRC)) {
                // scales above 146 would take 448 x scale past FP16's largest finite value: such blocks saturate
                const __half2 scale2 = __float2half2_rn(fminf(__uint_as_float(r.sc[g][j]), 146.f));
                dequant4_f16(x.x, scale2, w0.x, w0.y);
                dequant4_f16(x.y, scale2, w0.z, w0.w);
                dequant4_f16(x.z, scale2, w1.x, w1.y);
                dequant4_f16(x.w, scale2, w1.z, w1.w);
            } else {
                const __nv_bfloat162 scale2 = __float2bfloat162_rn(s120);
                dequant4(x.x, scale2, w0.x, w0.y);
                dequant4(x.y, scale2, w0.z, w0.w);
                dequant4(x.z, scale2, w1.x, w1.y);
                dequant4(x.w, scale2, w1.z, w1.w);
            }
        }
        // A 16-byte store is served per quarter-warp: 8 lanes = one row, both chunks.  The two
        // chunks are 8 KB apart (same banks), so the lanes of the second chunk write their
        // odd column first and the even one second: every quarter-warp then covers all eight
        // 16-byte bank groups once per instruction.
        const uint32_t flip = piece >> 2;
        ptx::sts_v4(base + (((2u * p + flip) ^ sw) << 4), flip ? w1 : w0);
        ptx::sts_v4(base + (((2u * p + (flip ^ 1u)) ^ sw) << 4), flip ? w0 : w1);
    }
}

// The RoPE tail (chunk NCHUNK-1, a plain copy): 4 rows x 8 columns per store instruction.
template <int NCHUNK, int SRC, int G>
__device__ __forceinline__ void loader_store_rope(uint32_t kv_st, int t0, int lane, const LoaderRegs<SRC, G>& r) {
    const uint32_t piece = uint32_t(lane & 7);
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int i = 4 * g + (lane >> 3);
        const int t = t0 + i;
        const bool valid = (r.vmask >> i) & 1u;
        const uint32_t base = kv_st + uint32_t(NCHUNK - 1) * kKvChunkBytes + uint32_t(t) * 128u;
        uint4 w = valid ? r.rope[g] : make_uint4(0, 0, 0, 0);
        if constexpr (use_f16(SRC)) {
            w.x = ptx::bf16x2_to_f16x2(w.x);  w.y = ptx::bf16x2_to_f16x2(w.y);
            w.z = ptx::bf16x2_to_f16x2(w.z);  w.w = ptx::bf16x2_to_f16x2(w.w);
        }
        ptx::sts_v4(base + ((piece ^ uint32_t(t & 7)) << 4), w);
    }
}

// BF16 -> FP16 in place over the Q chunks that stay in shared memory, one share per thread of
// the softmax and loader warps (threads 0 .. kStageThreads-1), then the proxy fence that makes
// the result visible to the MMAs' reads.  Element-wise, so the swizzled layout is untouched.
template <int BYTES>
__device__ __forceinline__ void convert_q_smem(uint32_t q_base, int tid) {
    for (int i = tid; i < BYTES / 16; i += kStageThreads) {
        uint4 x = ptx::lds_v4(q_base + uint32_t(i) * 16u);
        x.x = ptx::bf16x2_to_f16x2(x.x);  x.y = ptx::bf16x2_to_f16x2(x.y);
        x.z = ptx::bf16x2_to_f16x2(x.z);  x.w = ptx::bf16x2_to_f16x2(x.w);
        ptx::sts_v4(q_base + uint32_t(i) * 16u, x);
    }
    ptx::fence_proxy_async_smem();
}

// Copy Q chunks [g0, g1) of the 32 head rows of lane quarter `warp % 4` from the staging area to
// tensor memory: head row = tensor-memory lane, two 16-bit values per 32-bit column, in K order
// (the A-operand layout of the MMA); converted to FP16 on the way when the kernel runs on FP16.
template <bool F16>
__device__ __forceinline__ void copy_q_chunks_to_tmem(uint32_t stage_base, uint32_t tmem, int warp, int lane, int g0, int g1) {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const uint32_t srow = stage_base + uint32_t(r) * 128u;
    const uint32_t sw = uint32_t(r & 7);
#pragma unroll 1
    for (int g = g0; g < g1; ++g) {
        uint32_t w32[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint4 x = ptx::lds_v4(srow + uint32_t(g) * kQChunkBytes + ((uint32_t(j) ^ sw) << 4));
            if constexpr (F16) {
                x.x = ptx::bf16x2_to_f16x2(x.x);  x.y = ptx::bf16x2_to_f16x2(x.y);
                x.z = ptx::bf16x2_to_f16x2(x.z);  x.w = ptx::bf16x2_to_f16x2(x.w);
            }
            w32[4 * j + 0] = x.x;  w32[4 * j + 1] = x.y;  w32[4 * j + 2] = x.z;  w32[4 * j + 3] = x.w;
        }
        ptx::tmem_st32(tmem + lane_addr + kTmemQ + g * 32, w32);
    }
}

// PAIR: launched as clusters of two blocks along x - the two blocks of a row and head group (the two
// halves of the value columns).  Both need the whole dequantised tile, so each fetches and
// dequantises half of its entries into its own stage, and a forwarder warp sends that half on to
// the same place in the other block's stage by bulk copies through distributed shared memory;
// everything after that is as in the ordinary kernel.  Bit-identical results; measured slower
// than the ordinary kernel (the copy sits in the two-stage ring), so it is a selectable variant.
template <int NCHUNK, int SRC, bool PAIR = false>
__global__ void __launch_bounds__(kNumThreads, 1) decode_mma_kernel(const __grid_constant__ DecodeArgs a) {
    static_assert(!PAIR || !is_ref_layout(SRC), "the cluster-pair variant is written for the packed layout");
    using L = SmemLayout<NCHUNK>;
    constexpr int G = PAIR ? 1 : 2;            // groups of 4 entries per loader warp and tile
    constexpr int E = 4 * G;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t q_base = smem_base + L::kQOff;
    const uint32_t kv_base = smem_base + L::kKvOff;
    SmemMisc* misc = reinterpret_cast<SmemMisc*>(smem_gen + L::kMiscOff);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int half = blockIdx.x & 1;
    const int hg = blockIdx.x >> 1;
    const int n = blockIdx.y;                // row = b * s_q + query token
    const int split = blockIdx.z;
    const int b = n / a.s_q;
    // the other block of the pair sees this block's shared memory at (address + peer_delta)
    const uint32_t peer_delta = PAIR ? ptx::mapa(smem_base, uint32_t(half ^ 1)) - smem_base : 0u;

    // The per-row lengths are requested here and used only after the set-up below: the Q load and the
    // barrier initialisation do not wait for them.
    int raw_len0 = 0, raw_len1 = 0;
    if constexpr (SRC == kSrcCsa) {
        raw_len0 = (a.topk_len != nullptr) ? __ldg(a.topk_len + n) : a.topk;
        raw_len1 = (a.kv_len != nullptr) ? __ldg(a.kv_len + n) : 0x7FFFFFFF;
    } else if constexpr (SRC == kSrcHca || SRC == kSrcRefPaged) {
        raw_len0 = __ldg(a.kv_len + n);
        raw_len1 = __ldg(a.win_len + n);
    }
    if (tid == 32) {
        // first link of the loaders' chains of dependent loads (index list -> block table -> entries): into L2 now
        if constexpr (SRC == kSrcCsa) {
            const int32_t* idx = a.indices + int64_t(n) * a.topk;
            const int lines = min((a.topk * 4 + 127) / 128, 8);
            for (int l = 0; l < lines; ++l) ptx::prefetch_l2(reinterpret_cast<const uint8_t*>(idx) + 128 * l);
        }
        if constexpr (SRC == kSrcCsa || SRC == kSrcHca || SRC == kSrcRefPaged)
            ptx::prefetch_l2(a.block_table + int64_t(b) * a.max_pages);
    }

    const uint32_t v_off = uint32_t(half ? 4 : 0) * kKvChunkBytes;   // this block's value columns inside a stage

    const uint32_t bar_kv_full = ptx::smem_u32(&misc->bar_kv_full[0][0]);   // [stage][chunk] at +80*stage + 8*chunk
    const uint32_t bar_kv_free = ptx::smem_u32(&misc->bar_kv_free[0]);
    const uint32_t bar_s_full = ptx::smem_u32(&misc->bar_s_full[0]);
    const uint32_t bar_p_full = ptx::smem_u32(&misc->bar_p_full[0]);
    const uint32_t bar_o_full = ptx::smem_u32(&misc->bar_o_full);
    const uint32_t bar_q_full = ptx::smem_u32(&misc->bar_q_full);
    const uint32_t bar_q_ready = ptx::smem_u32(&misc->bar_q_ready);

    // ── set-up ──
    if (tid == 0) {
        trace_mark(a, 3, 0);
        trace_block(a, 0);
        for (int st = 0; st < 2; ++st) {
            for (int g = 0; g < kNumKvGroups; ++g)
                ptx::mbar_init(bar_kv_full + 80 * st + 8 * g, kNumLoaderWarps + (PAIR ? 1 : 0));   // + the other block's forwarder
            for (int j = 0; j < 4; ++j) ptx::mbar_init(ptx::smem_u32(&misc->bar_loc[st][j]), kNumLoaderWarps);
            ptx::mbar_init(bar_kv_free + 8 * st, PAIR ? 2 : 1);     // PV commits of both blocks: a stage is refilled in both at once
            ptx::mbar_init(bar_s_full + 8 * st, 1);
            ptx::mbar_init(bar_p_full + 8 * st, kNumSoftmaxWarps);
        }
        ptx::mbar_init(bar_o_full, 1);
        ptx::mbar_init(bar_q_full, 1);
        ptx::mbar_init(bar_q_ready, (PAIR ? 2 : 1) * (kNumSoftmaxWarps + kNumLoaderWarps));
        ptx::fence_mbar_init();
        {
            // (issued whether or not this block has tiles: a block without tiles waits for it before it leaves)
            // Q tile [128 heads x NCHUNK*64] bf16 by TMA, one 64-column box per chunk, landing in
            // the swizzled operand layout: chunks >= kQTmemChunks at their final place, the others
            // in the staging area.  Rows past the end of Q read as zero; rows of a following
            // request (H < 128) are computed but never written out.
            ptx::mbar_arrive_expect_tx(bar_q_full, uint32_t(NCHUNK) * kQChunkBytes);
            const int row0 = n * a.H + hg * kHeadsPerCta;
#pragma unroll
            for (int c = 0; c < NCHUNK; ++c) {
                const uint32_t dst = (c < kQTmemChunks) ? smem_base + L::kQStageOff + uint32_t(c) * kQChunkBytes
                                                        : q_base + uint32_t(c - kQTmemChunks) * kQChunkBytes;
                ptx::tma_load_2d(dst, &a.q_map, c * 64, row0, bar_q_full);
            }
        }
        trace_mark(a, 3, 10);
    }

    // ── this block's tile range ──
    int n_tok, kv_len_n;
    if constexpr (SRC == kSrcCsa) {
        n_tok = min(max(raw_len0, 0), a.topk);
        kv_len_n = raw_len1;
    } else if constexpr (SRC == kSrcHca || SRC == kSrcRefPaged) {
        kv_len_n = max(raw_len0, 0);
        n_tok = kv_len_n + max(raw_len1, 0);
    } else {
        kv_len_n = a.ref_m_cur;
        n_tok = a.ref_m_cur + a.ref_swa_len;
    }
    const int tiles_total = (n_tok + kTileN - 1) / kTileN;
    const int tiles_per_split = (tiles_total + a.num_splits - 1) / a.num_splits;
    const int tile0 = min(split * tiles_per_split, tiles_total);
    const int tile1 = min(tile0 + tiles_per_split, tiles_total);
    const int ntiles = tile1 - tile0;

    // Block-wide rendezvous.  Every role runs the same number of them (one before the
    // main loops, one at the exit), each from its own branch.
    // (PAIR: a rendezvous of both blocks - nothing is written to, and no barrier is arrived on, in
    // the other block before its barriers are initialised.)
    auto block_sync = [&]() {
        ptx::tc_fence_before_sync();
        if constexpr (PAIR) ptx::cluster_sync(); else __syncthreads();
        ptx::tc_fence_after_sync();
    };
    // Q staging released / Q in tensor memory: in a pair the other block's loaders write into this
    // block's stage 1 as well, so they are told too.
    auto arrive_q_ready = [&]() {
        ptx::mbar_arrive(bar_q_ready);
        if constexpr (PAIR) ptx::mbar_arrive_cluster(bar_q_ready + peer_delta);
    };
    auto wait_q_ready = [&]() {
        return PAIR ? ptx::mbar_wait_cluster(bar_q_ready, 0u, kWaitTimeoutNs) : ptx::mbar_wait(bar_q_ready, 0u, kWaitTimeoutNs);
    };

    if (warp >= kFirstLoaderWarp && warp < kMmaWarp) {
        // ───────────── loader warps ─────────────
        // Two register sets, one per KV stage: while one tile is dequantised and stored, the
        // loads of the next one are in flight.  Keys run two tiles ahead of the loads, and the
        // records they name are pulled into L2 at that point.  The larger register allowance
        // holds for this branch only.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kLoaderRegs));
        const int lw = warp - kFirstLoaderWarp;
        const int row0 = PAIR ? 32 * half + 4 * lw : 8 * lw;      // this warp's E entries: tile rows row0 .. row0+E-1
        LoaderRegs<SRC, G> regs_a, regs_b;
        // keys of the tiles two and three ahead of the one being stored (records already
        // pulled into L2), and of the tile four ahead (resolved, not yet prefetched)
        unsigned long long key1 = 0, key2 = 0, key3 = 0, key4 = 0;
        uint32_t vm1 = 0, vm2 = 0, vm3 = 0, vm4 = 0;
        int e_ahead = -1;        // CSA: this lane's index-list value of the tile resolved next (lanes 0-7)
        if (lw == 0 && lane == 0) trace_mark(a, 3, 4);
        if (ntiles > 0) {
            // one round of dependent loads for the first four tiles: lanes 0-7, 8-15, 16-23, 24-31
            // (lanes 0-7 also resolve tile 4, as a second chain of loads in flight beside the first)
            bool valid = false, valid4 = false;
            const int which = lane >> 3;
            unsigned long long key, k4;
            loader_resolve2<SRC>(a, b, n, (tile0 + which) * kTileN + row0 + (lane & 7), (which < ntiles && (lane & 7) < E) ? n_tok : 0,
                                 (tile0 + 4) * kTileN + row0 + (lane & 7), (4 < ntiles && lane < E) ? n_tok : 0,
                                 kv_len_n, key, valid, k4, valid4);
            const uint32_t bal = __ballot_sync(0xFFFFFFFFu, valid);
            vm4 = __ballot_sync(0xFFFFFFFFu, valid4) & 0xFFu;
            key4 = k4;
            if constexpr (SRC == kSrcCsa) {
                // the index-list values of tile 5 (lanes 0-7), on their way one step before they are needed
                const int v5 = (tile0 + 5) * kTileN + row0 + lane;
                if (lane < E && 5 < ntiles && v5 < n_tok) e_ahead = __ldg(a.indices + int64_t(n) * a.topk + v5);
            }
            if (lw == 0 && lane == 0) trace_mark(a, 3, 5);
            vm2 = (bal >> 16) & 0xFFu;
            vm3 = (bal >> 24) & 0xFFu;
            key2 = __shfl_sync(0xFFFFFFFFu, key, (lane & 7) + 16);
            key3 = __shfl_sync(0xFFFFFFFFu, key, (lane & 7) + 24);
            // Only what the first tile needs goes out before the main loop: the number of loads
            // an SM keeps in flight is limited, and everything queued here delays tile 0.
            loader_fetch<SRC>(a, key, bal & 0xFFu, lane, regs_a);
            if (lw == 0 && lane == 0) trace_mark(a, 3, 6);
            key1 = __shfl_sync(0xFFFFFFFFu, key, (lane & 7) + 8);   // -> lanes 0..7
            vm1 = (bal >> 8) & 0xFFu;
        }
        if (lw == 0 && lane == 0) trace_mark(a, 3, 7);
        block_sync();
        if (lw == 0 && lane == 0) trace_mark(a, 3, 8);
        if (ntiles > 0) {
            bool lok = true;
            {
                // the loaders' share of the Q set-up, while their first loads are in flight: warps
                // 4-7 copy chunk 2 to tensor memory, warps 8-11 chunk 3, and (FP16 route) every
                // thread converts its part of the chunks that stay in shared memory
                const bool w = ptx::mbar_wait(bar_q_full, 0u, kWaitTimeoutNs);
                if (!__all_sync(0xFFFFFFFFu, w)) {
                    report_timeout(a.status, kStatusWaitQ, 2, tile0);
                    lok = false;
                } else {
                    const uint32_t tmem_q = misc->tmem_base;
                    const int g = 2 + (lw >> 2);
                    copy_q_chunks_to_tmem<use_f16(SRC)>(smem_base + L::kQStageOff, tmem_q, warp, lane, g, g + 1);
                    if constexpr (use_f16(SRC)) convert_q_smem<L::kQBytes>(q_base, tid);
                    ptx::tmem_wait_st();
                    ptx::tc_fence_before_sync();
                }
                __syncwarp();
                if (lane == 0) arrive_q_ready();     // also after a time-out, so that nobody waits for this warp
            }
            auto tile_step = [&](LoaderRegs<SRC, G>& regs, int it) {
                const int st = it & 1;
                if (it == 1) {
                    // stage 1 doubles as the Q staging area until the copy to tensor memory is done
                    const bool w = wait_q_ready();
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_timeout(a.status, kStatusWaitQ, 2, tile0 + it);
                        lok = false;
                        return;
                    }
                }
                if (it >= 2) {
                    // warp-uniform outcome: the warp-collective operations below need all lanes
                    const bool w = ptx::mbar_wait(bar_kv_free + 8 * st, uint32_t((it >> 1) - 1) & 1u, kWaitTimeoutNs);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_timeout(a.status, kStatusWaitKvFree, 2, tile0 + it);
                        lok = false;
                        return;
                    }
                }
                if (lw == 0 && lane == 0) trace_mark(a, 2, 2 * it);
                if (it != 0 && !(a.dbg & 2)) {
                    // the key resolved during the previous step has arrived by now: start pulling
                    // its records into L2 (using it earlier would stall on the block-table load)
                    loader_prefetch_l2<SRC>(key4, vm4, lane);
                }
                if constexpr (PAIR) {
                    if (lane == 0) reinterpret_cast<volatile uint8_t*>(&misc->valid_bytes[st][0])[8 * half + lw] = uint8_t(regs.vmask);
                } else {
                    if (lane == 0) reinterpret_cast<volatile uint8_t*>(&misc->valid_mask[st])[lw] = uint8_t(regs.vmask);
                }
                // in two groups (chunks 0-3, then the rest with the RoPE tail), so that the QK MMAs of this tile
                // start while it is still being written; one proxy fence and one arrival per group
                const uint32_t kv_st = kv_base + uint32_t(st) * L::kKvStageBytes;
                auto group_done = [&](int g) {
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::mbar_arrive(bar_kv_full + 80 * st + 8 * g);
                        if constexpr (PAIR) ptx::mbar_arrive(ptx::smem_u32(&misc->bar_loc[st][2 * g + 1]));   // the forwarder takes it from here
                    }
                };
                // (pair: the forwarder is told span by span, so that its copies run beside the stores)
                auto span_done = [&](int j) {
                    if constexpr (PAIR) {
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&misc->bar_loc[st][j]));
                    }
                };
                loader_store_span<NCHUNK, SRC, G>(kv_st, row0, lane, regs, 0);
                span_done(0);
                loader_store_span<NCHUNK, SRC, G>(kv_st, row0, lane, regs, 1);
                group_done(0);
                loader_store_span<NCHUNK, SRC, G>(kv_st, row0, lane, regs, 2);
                span_done(2);
                loader_store_span<NCHUNK, SRC, G>(kv_st, row0, lane, regs, 3);
                loader_store_rope<NCHUNK, SRC, G>(kv_st, row0, lane, regs);
                group_done(1);
                if (lw == 0 && lane == 0) trace_mark(a, 2, 2 * it + 1);
                if (it == 0) {
                    // Tile 0 is complete.  The loads of tile 1 and the records of tiles 2 and 3 are
                    // requested only here: queued earlier they would hold up the stores above (the
                    // load/store unit takes about a microsecond to accept a tile's worth of loads).
                    if (1 < ntiles) loader_fetch<SRC>(a, key1, vm1, lane, regs_b);
                    loader_prefetch_l2<SRC>(key2, vm2, lane);
                    loader_prefetch_l2<SRC>(key3, vm3, lane);
                }
                // this set is free again: loads of tile it+2, keys of tile it+5
                if (it + 2 < ntiles) loader_fetch<SRC>(a, key2, vm2, lane, regs);
                key2 = key3;  vm2 = vm3;
                key3 = key4;  vm3 = vm4;
                if constexpr (SRC == kSrcCsa) {
                    // Tile it+5: its index-list values were requested one step ago, so the ballot below
                    // does not wait for a load; the block-table load issued here is consumed a step
                    // later, and the index-list values of tile it+6 are requested now.
                    const bool valid = e_ahead >= 0 && e_ahead < kv_len_n;       // e_ahead is -1 past the list or the tiles
                    unsigned long long key = 0;
                    if (valid) {
                        const int page = __ldg(a.block_table + int64_t(b) * a.max_pages + (e_ahead >> 6));
                        key = reinterpret_cast<unsigned long long>(a.kv_pool + (int64_t(page) * 64 + (e_ahead & 63)) * 656);
                    }
                    vm4 = __ballot_sync(0xFFFFFFFFu, valid) & 0xFFu;
                    key4 = key;
                    const int v6 = (tile0 + it + 6) * kTileN + row0 + lane;
                    e_ahead = (lane < E && it + 6 < ntiles && v6 < n_tok) ? __ldg(a.indices + int64_t(n) * a.topk + v6) : -1;
                } else {
                    key4 = loader_resolve_warp<SRC, E>(a, b, n, (tile0 + it + 5) * kTileN + row0, lane,
                                                    (it + 5 < ntiles) ? n_tok : 0, kv_len_n, vm4);
                }
            };
            for (int it = 0; it < ntiles && lok; it += 2) {
                tile_step(regs_a, it);
                if (it + 1 < ntiles && lok) tile_step(regs_b, it + 1);
            }
        }
    } else if (warp >= kMmaWarp) {
        // ───────────── last warpgroup: MMA issue (one thread of warp 12), tensor-memory owner ─────────────
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kIdleRegs));
        if (warp == kMmaWarp) {
            ptx::tmem_alloc(ptx::smem_u32(&misc->tmem_base), kTmemCols);
            ptx::tmem_relinquish();
            if (lane == 0) trace_mark(a, 3, 9);
        }
        block_sync();
        const uint32_t tmem = misc->tmem_base;
        if (ntiles > 0 && warp == kMmaWarp) {
            if (lane == 0) {
                constexpr uint32_t idesc_qk = use_f16(SRC) ? ptx::make_idesc_f16(128, kTileN, false, false)
                                                            : ptx::make_idesc_bf16(128, kTileN, false, false);
                bool ok = true;
                // Q: shared-memory chunks landed (TMA) and tensor-memory chunks copied
                if (!ptx::mbar_wait(bar_q_full, 0u, kWaitTimeoutNs) || !wait_q_ready()) {
                    report_timeout(a.status, kStatusWaitQ, 1, tile0);
                    ok = false;
                }
                ptx::tc_fence_after_sync();
                // S(it) = Q . K(it)^T into S buffer it&1; one tile ahead of the PV MMAs so that
                // the softmax of tile it overlaps the QK MMAs of tile it+1.
                // Chunks [C0, C1) (4 MMAs each) of S(it) = Q . K(it)^T into S buffer it&1; the chunk
                // range is a compile-time constant so that the descriptors fold to immediates.
                constexpr uint32_t kDescHi = ptx::smem_desc_hi(1024);        // 8-row groups 1 KB apart
                const uint32_t q_lo = ptx::smem_desc_lo(q_base, 16);
                auto issue_qk_range = [&](int it, auto c0_tag, auto c1_tag) {
                    constexpr int C0 = decltype(c0_tag)::value, C1 = decltype(c1_tag)::value;
                    const int st = it & 1;
                    const uint32_t k_lo = ptx::smem_desc_lo(kv_base + uint32_t(st) * L::kKvStageBytes, 16);
                    const uint32_t d = tmem + kTmemS + uint32_t(st) * kTileN;
#pragma unroll
                    for (int c = C0; c < C1; ++c) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            // descriptor start addresses advance by constants (in 16-byte units)
                            const uint32_t b_lo = k_lo + uint32_t((c * kKvChunkBytes + k * 32) >> 4);
                            if (c < kQTmemChunks) {
                                // A = Q columns in tensor memory: 16 BF16 = 8 columns per K step
                                ptx::mma_bf16_ts2(d, tmem + kTmemQ + c * 32 + k * 8, b_lo, kDescHi, idesc_qk, (c | k) ? 1u : 0u);
                            } else {
                                const uint32_t a_lo = q_lo + uint32_t(((c - kQTmemChunks) * kQChunkBytes + k * 32) >> 4);
                                ptx::mma_bf16_ss2(d, a_lo, b_lo, kDescHi, idesc_qk, 1u);
                            }
                        }
                    }
                };
                // QK is issued group by group as the loaders deliver them; between groups a ready P
                // goes first.
                constexpr int kNumGroups = kNumKvGroups;
                static_assert(kNumGroups == 2, "group dispatch below is written for 2 groups");
                // the groups the loaders deliver: chunks 0-3, then the rest with the RoPE tail
                auto issue_qk_group = [&](int it, int g) {
                    if (g == 0) issue_qk_range(it, std::integral_constant<int, 0>{}, std::integral_constant<int, 4>{});
                    else issue_qk_range(it, std::integral_constant<int, 4>{}, std::integral_constant<int, NCHUNK>{});
                };
                // This thread issues only S = Q.K^T, group by group as the loaders deliver them; O += P.V is
                // issued by a thread of the next warp.  No order is needed between the two streams beyond
                // what the barriers already give: S(t+2) and the refill of stage t&1 both follow the
                // kv_free arrival of P(t).V(t), and P(t) follows S(t).  A P that becomes ready then never
                // waits for this thread to finish issuing a group.
                for (int it = 0; it < ntiles && ok; ++it) {
                    const int st = it & 1;
                    for (int g = 0; g < kNumGroups; ++g) {
                        const uint32_t bar = bar_kv_full + 80 * st + 8 * g, par = uint32_t(it >> 1) & 1u;
                        if (!(PAIR ? ptx::mbar_wait_cluster(bar, par, kWaitTimeoutNs) : ptx::mbar_wait(bar, par, kWaitTimeoutNs))) {
                            report_timeout(a.status, kStatusWaitKvFull, 1, tile0 + it);
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after_sync();
                        if (g == 0) trace_mark(a, 1, 2 * it);
                        issue_qk_group(it, g);
                    }
                    if (ok) ptx::mma_commit(bar_s_full + 8 * st);
                }
            }
            __syncwarp();
        } else if (ntiles > 0 && warp == kMmaWarp + 1) {
            // ───────────── O += P . V issue (one thread) ─────────────
            if (lane == 0) {
                constexpr uint32_t idesc_pv = use_f16(SRC) ? ptx::make_idesc_f16(128, kDvHalf, false, true)
                                                            : ptx::make_idesc_bf16(128, kDvHalf, false, true);
                constexpr uint32_t kDescHi = ptx::smem_desc_hi(1024);
                bool ok = true;
                for (int it = 0; it < ntiles; ++it) {
                    const int st = it & 1;
                    if (!ptx::mbar_wait(bar_p_full + 8 * st, uint32_t(it >> 1) & 1u, kWaitTimeoutNs)) {
                        report_timeout(a.status, kStatusWaitPFull, 1, tile0 + it);
                        ok = false;
                        break;
                    }
                    const uint32_t kv_st = kv_base + uint32_t(st) * L::kKvStageBytes;
                    ptx::tc_fence_after_sync();
                    trace_mark(a, 1, 2 * it + 1);
                    const uint32_t p_tmem = tmem + kTmemS + uint32_t(st) * kTileN;
                    // B = V[16 entries x 256 cols], MN-major: 64-col groups 8 KB apart (leading
                    // offset), 8-entry groups 1 KB apart; A = P in tensor memory, 8 columns per step
                    const uint32_t v_lo = ptx::smem_desc_lo(kv_st + v_off, kKvChunkBytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        ptx::mma_bf16_ts2(tmem + kTmemO, p_tmem + k * 8, v_lo + uint32_t((k * 2048) >> 4), kDescHi, idesc_pv,
                                          (it | k) ? 1u : 0u);
                    ptx::mma_commit(bar_kv_free + 8 * st);   // stage reusable, and O includes tile it
                    if constexpr (PAIR) ptx::mma_commit_cluster(bar_kv_free + 8 * st + peer_delta);   // the other block's forwarder copies into it
                    trace_mark(a, 1, 512 + 4 * it + 3);
                }
                if (ok) ptx::mma_commit(bar_o_full);
            }
            __syncwarp();
        } else if (PAIR && ntiles > 0 && warp == kMmaWarp + 2) {
            // ───────────── forwarder (cluster pair): this block's half of every group, once its loader
            // warps have written it, goes to the same place in the other block by bulk copies that
            // complete on the other block's kv_full barrier (no load/store-unit work, no registers)
            if (lane == 0) {
                constexpr uint32_t kHalfChunk = uint32_t(kKvChunkBytes) / 2;       // 32 rows x 128 bytes
                for (int it = 0; it < ntiles; ++it) {
                    const int st = it & 1;
                    const uint32_t kv_st = kv_base + uint32_t(st) * L::kKvStageBytes + uint32_t(half) * kHalfChunk;
                    bool fok = true;
                    for (int j = 0; j < 4 && fok; ++j) {
                        if (!ptx::mbar_wait(ptx::smem_u32(&misc->bar_loc[st][j]), uint32_t(it >> 1) & 1u, kWaitTimeoutNs)) {
                            report_timeout(a.status, kStatusWaitKvFull, 3, tile0 + it);
                            fok = false;
                            break;
                        }
                        const int g = j >> 1;
                        const uint32_t rbar = bar_kv_full + 80 * st + 8 * g + peer_delta;
                        if (j == 0) {
                            // this block's eight 4-bit validity masks of the tile
                            const unsigned long long vb = *reinterpret_cast<volatile unsigned long long*>(&misc->valid_bytes[st][8 * half]);
                            asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(ptx::smem_u32(&misc->valid_bytes[st][8 * half]) + peer_delta), "l"(vb) : "memory");
                        }
                        if ((j & 1) == 0) {
                            // one arrival per group, announcing all of the group's bytes
                            asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(rbar),
                                         "r"(uint32_t(g == 0 ? 4 : NCHUNK - 4) * kHalfChunk) : "memory");
                        }
                        const int c0 = 2 * j, c1 = j == 3 ? NCHUNK : 2 * j + 2;
                        for (int c = c0; c < c1; ++c) {
                            const uint32_t src = kv_st + uint32_t(c) * kKvChunkBytes;
                            asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(src + peer_delta),
                                         "r"(src), "r"(kHalfChunk), "r"(rbar) : "memory");
                        }
                    }
                    if (!fok) break;
                }
            }
            __syncwarp();
        }
    } else {
        // ───────────── softmax + epilogue warps ─────────────
        block_sync();
        const uint32_t tmem = misc->tmem_base;
        bool ok = true;
        if (ntiles > 0) {
            const bool w = ptx::mbar_wait(bar_q_full, 0u, kWaitTimeoutNs);
            if (!__all_sync(0xFFFFFFFFu, w)) {
                report_timeout(a.status, kStatusWaitQ, 0, tile0);
                ok = false;
            }
            if (tid == 0) trace_mark(a, 3, 11);
            if (ok) {
                // chunks 0-1 here, chunks 2 and 3 by the loader warps (each warp serves its lane quarter)
                static_assert(kQTmemChunks == 4, "the split of the copy below is written for four chunks");
                copy_q_chunks_to_tmem<use_f16(SRC)>(smem_base + L::kQStageOff, tmem, warp, lane, 0, 2);
                if constexpr (use_f16(SRC)) {
                    // the Q chunks that stay in shared memory: BF16 -> FP16 in place (element-wise, so
                    // the swizzled layout is untouched), then made visible to the MMAs' reads
                    // (shared with the loader warps: see convert_q_smem)
                    convert_q_smem<L::kQBytes>(q_base, tid);
                }
                ptx::tmem_wait_st();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) arrive_q_ready();
            }
        }
        if (tid == 0) trace_mark(a, 3, 1);
        if (ntiles > 0) {
            const int r = warp * 32 + lane;                // head row inside the group
            const uint32_t lane_addr = uint32_t(warp * 32) << 16;
            float m_ref = -CUDART_INF_F;                   // reference maximum used in exp2 (log2 units)
            float l_sum = 0.f;
            for (int it = 0; it < ntiles && ok; ++it) {
                const int st = it & 1;
                const uint32_t s_tmem = tmem + lane_addr + kTmemS + uint32_t(st) * kTileN;
                {
                    const bool w = ptx::mbar_wait(bar_s_full + 8 * st, uint32_t(it >> 1) & 1u, kWaitTimeoutNs);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_timeout(a.status, kStatusWaitSFull, 0, tile0 + it);
                        ok = false;  break;
                    }
                }
                ptx::tc_fence_after_sync();
                if (tid == 0) trace_mark(a, 0, 2 * it);
                uint32_t s0[32], s1[32];
                ptx::tmem_ld32(s_tmem, s0);
                ptx::tmem_ld32(s_tmem + 32, s1);
                ptx::tmem_wait_ld();
                uint64_t vmask;
                if constexpr (PAIR) {
                    // sixteen 4-bit masks, one per loader warp of the pair
                    const uint4 vb = ptx::lds_v4(ptx::smem_u32(&misc->valid_bytes[st][0]));
                    if ((vb.x & vb.y & vb.z & vb.w) == 0x0F0F0F0Fu) {
                        vmask = ~0ull;
                    } else {
                        auto nib = [](uint32_t w) { return (w & 0xFu) | ((w >> 4) & 0xF0u) | ((w >> 8) & 0xF00u) | ((w >> 12) & 0xF000u); };
                        vmask = uint64_t(nib(vb.x) | (nib(vb.y) << 16)) | (uint64_t(nib(vb.z) | (nib(vb.w) << 16)) << 32);
                    }
                } else {
                    vmask = *reinterpret_cast<volatile uint64_t*>(&misc->valid_mask[st]);
                }
                if (vmask != ~0ull) {
                    // entries that do not take part (padding, the end of the list): -inf before the scale
                    const uint32_t vm0 = uint32_t(vmask), vm1 = uint32_t(vmask >> 32);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (!((vm0 >> i) & 1u)) s0[i] = 0xFF800000u;
                        if (!((vm1 >> i) & 1u)) s1[i] = 0xFF800000u;
                    }
                }
                // maximum of the raw logits (the scale is positive), four chains
                float t4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        t4[k] = fmaxf(t4[k], fmaxf(__uint_as_float(s0[i + k]), __uint_as_float(s1[i + k])));
                }
                const float tmax = fmaxf(fmaxf(t4[0], t4[1]), fmaxf(t4[2], t4[3])) * a.scale_log2;
                // Lazy reference maximum: move it only when the true maximum exceeds it by
                // more than the threshold (exp2 of the excess stays <= 2^threshold).
                float alpha = 1.f;
                bool moved = false;
                if (tmax > m_ref + kRescaleThreshold) {   // also true for the first finite max
                    alpha = (m_ref == -CUDART_INF_F) ? 0.f : ptx::ex2(m_ref - tmax);
                    m_ref = tmax;
                    moved = true;
                }
                const float neg_m = (m_ref == -CUDART_INF_F) ? 0.f : -m_ref;
                // p = 2^(s * scale - m): one fused multiply-add and one exp2 per element
                float ps4[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = ptx::ex2(fmaf(__uint_as_float(s0[2 * i]), a.scale_log2, neg_m));
                    const float p1 = ptx::ex2(fmaf(__uint_as_float(s0[2 * i + 1]), a.scale_log2, neg_m));
                    ps4[i & 3] += p0 + p1;
                    pk[i] = use_f16(SRC) ? ptx::pack_f16x2(p0, p1) : ptx::pack_bf16x2(p0, p1);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = ptx::ex2(fmaf(__uint_as_float(s1[2 * i]), a.scale_log2, neg_m));
                    const float p1 = ptx::ex2(fmaf(__uint_as_float(s1[2 * i + 1]), a.scale_log2, neg_m));
                    ps4[i & 3] += p0 + p1;
                    pk[16 + i] = use_f16(SRC) ? ptx::pack_f16x2(p0, p1) : ptx::pack_bf16x2(p0, p1);
                }
                const float psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
                l_sum = l_sum * alpha + psum;
                // Rescale O where the reference maximum moved.  The PV MMAs of the previous
                // tile must have finished first (their commit is that stage's kv_free).
                if (it > 0 && __any_sync(0xFFFFFFFFu, moved)) {
                    const bool w = ptx::mbar_wait(bar_kv_free + 8 * ((it - 1) & 1), uint32_t((it - 1) >> 1) & 1u, kWaitTimeoutNs);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_timeout(a.status, kStatusWaitKvFree, 0, tile0 + it);
                        ok = false;  break;
                    }
                    ptx::tc_fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < kDvHalf / 32; ++c) {
                        uint32_t o[32];
                        ptx::tmem_ld32(tmem + lane_addr + kTmemO + c * 32, o);
                        ptx::tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        ptx::tmem_st32(tmem + lane_addr + kTmemO + c * 32, o);
                    }
                }
                // P (BF16, two entries per column) over the first 32 columns of this S buffer:
                // the A operand of the PV MMAs.  S has been read into registers above.
                ptx::tmem_st32(s_tmem, pk);
                ptx::tmem_wait_st();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_p_full + 8 * st);
                if (tid == 0) trace_mark(a, 0, 2 * it + 1);
            }
            // ── epilogue ──
            if (ok) {
                const bool w = ptx::mbar_wait(bar_o_full, 0u, kWaitTimeoutNs);
                if (!__all_sync(0xFFFFFFFFu, w)) {
                    report_timeout(a.status, kStatusWaitOFull, 0, tile1);
                    ok = false;
                }
            }
            if (ok) {
                ptx::tc_fence_after_sync();
                if (tid == 0) trace_mark(a, 3, 2);
                // A merge kernel launched as a programmatic dependent may be made resident once every block of
                // this grid is here (or gone): by then no block of this grid is waiting for an SM any more.
                if (tid == 0 && a.num_splits > 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
                const int h = hg * kHeadsPerCta + r;
                const bool write = h < a.H;
                const bool final_out = a.num_splits == 1;
                float denom = l_sum;
                if (final_out && a.attn_sink != nullptr && write) {
                    const float s2 = __ldg(a.attn_sink + h) * 1.4426950408889634f;
                    denom = (l_sum > 0.f) ? l_sum + ptx::ex2(s2 - m_ref) : 1.f;   // empty row: O is 0 anyway
                }
                const float inv = (l_sum > 0.f) ? 1.f / denom : 0.f;
                const float lse2 = (l_sum > 0.f) ? m_ref + log2f(l_sum) : -CUDART_INF_F;
                const int64_t row = int64_t(n) * a.H + h;
                // O leaves through shared memory (Q and the KV stages are free by now): each thread owns a
                // row in tensor memory, but rows are 1 KB apart in global memory, so the rows are first
                // laid down in shared memory (pitch = row + 16 bytes: conflict-free both ways) and then
                // written out 512 contiguous bytes per warp instruction.
                // (split partials are written as BF16 too: the merge reads them back at once, and at
                // eight splits their traffic exceeds the KV bytes; the FP32 form remains for a.partial_f32)
                const bool bf16_out = final_out || !a.partial_f32;
                const uint32_t row_bytes = bf16_out ? uint32_t(kDvHalf) * 2u : uint32_t(kDvHalf) * 4u;
                const uint32_t pitch = row_bytes + 16u;
                static_assert(4 * 32 * (kDvHalf * 4 + 16) <= L::kQBytes + 2 * L::kKvStageBytes, "epilogue staging must fit in the Q + KV area");
                const uint32_t stg = q_base + uint32_t(warp) * (32u * (uint32_t(kDvHalf) * 4u + 16u));
                const uint32_t my = stg + uint32_t(lane) * pitch;
#pragma unroll 1
                for (int c = 0; c < kDvHalf / 32; ++c) {
                    uint32_t o[32];
                    ptx::tmem_ld32(tmem + lane_addr + kTmemO + c * 32, o);
                    ptx::tmem_wait_ld();
                    if (bf16_out) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint4 w;
                            w.x = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                            w.y = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                            w.z = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                            w.w = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                            ptx::sts_v4(my + uint32_t(c) * 64u + uint32_t(v) * 16u, w);
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            uint4 w;
                            w.x = __float_as_uint(__uint_as_float(o[4 * v + 0]) * inv);
                            w.y = __float_as_uint(__uint_as_float(o[4 * v + 1]) * inv);
                            w.z = __float_as_uint(__uint_as_float(o[4 * v + 2]) * inv);
                            w.w = __float_as_uint(__uint_as_float(o[4 * v + 3]) * inv);
                            ptx::sts_v4(my + uint32_t(c) * 128u + uint32_t(v) * 16u, w);
                        }
                    }
                }
                __syncwarp();
                if (tid == 0) trace_mark(a, 3, 12);
                {
                    const uint32_t vecs_per_row = row_bytes / 16u;                  // 32 or 64
                    const int h0 = hg * kHeadsPerCta + warp * 32;                   // first head row of this warp
                    const int64_t prow = ((int64_t(split) * gridDim.y + n) * a.H) * 512 + half * kDvHalf;   // element index
                    uint8_t* gbase = final_out
                        ? reinterpret_cast<uint8_t*>(a.out + (int64_t(n) * a.H) * 512 + half * kDvHalf)
                        : (bf16_out ? reinterpret_cast<uint8_t*>(reinterpret_cast<__nv_bfloat16*>(a.partial_o) + prow)
                                    : reinterpret_cast<uint8_t*>(a.partial_o + prow));
                    const int64_t grow = bf16_out ? 512 * 2 : 512 * 4;              // bytes between head rows in global memory
#pragma unroll 4
                    for (uint32_t q = uint32_t(lane); q < 32u * vecs_per_row; q += 32u) {
                        const uint32_t rl = q / vecs_per_row, vc = q % vecs_per_row;
                        if (h0 + int(rl) < a.H) {
                            const uint4 w = ptx::lds_v4(stg + rl * pitch + vc * 16u);
                            *reinterpret_cast<uint4*>(gbase + int64_t(h0 + int(rl)) * grow + vc * 16u) = w;
                        }
                    }
                }
                if (tid == 0) trace_mark(a, 3, 13);
                if (write && half == 0) {
                    if (final_out) {
                        if (a.lse != nullptr) a.lse[row] = (l_sum > 0.f) ? lse2 * 0.6931471805599453f : -CUDART_INF_F;
                    } else {
                        a.partial_lse[int64_t(split) * gridDim.y * a.H + row] = lse2;
                    }
                }
            }
        }
    }
    if (ntiles <= 0) {
        // Nothing to attend to in this split: zero output, LSE = -inf.  The Q tile is on its way into
        // shared memory all the same and must have landed before the block leaves.
        if (tid == 0 && !ptx::mbar_wait(bar_q_full, 0u, kWaitTimeoutNs)) report_timeout(a.status, kStatusWaitQ, 3, tile0);
        const bool final_out = a.num_splits == 1;
        for (int i = tid; i < kHeadsPerCta * (kDvHalf / 8); i += kNumThreads) {
            const int r = i / (kDvHalf / 8), v = i % (kDvHalf / 8);
            const int h = hg * kHeadsPerCta + r;
            if (h >= a.H) continue;
            const int64_t row = int64_t(n) * a.H + h;
            const int col = half * kDvHalf + v * 8;
            if (final_out) {
                *reinterpret_cast<uint4*>(a.out + row * 512 + col) = make_uint4(0, 0, 0, 0);
            } else if (!a.partial_f32) {
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.partial_o) +
                                          (int64_t(split) * gridDim.y * a.H + row) * 512 + col) = make_uint4(0, 0, 0, 0);
            } else {
                float4* dst = reinterpret_cast<float4*>(a.partial_o + (int64_t(split) * gridDim.y * a.H + row) * 512 + col);
                dst[0] = make_float4(0.f, 0.f, 0.f, 0.f);
                dst[1] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        if (half == 0 && tid < kHeadsPerCta) {
            const int h = hg * kHeadsPerCta + tid;
            if (h < a.H) {
                const int64_t row = int64_t(n) * a.H + h;
                if (final_out) {
                    if (a.lse != nullptr) a.lse[row] = -CUDART_INF_F;
                } else {
                    a.partial_lse[int64_t(split) * gridDim.y * a.H + row] = -CUDART_INF_F;
                }
            }
        }
    }

    // ── common exit: every thread gets here, with or without an error ──
    // (PAIR: both blocks, so that neither leaves while the other may still arrive on its barriers)
    ptx::tc_fence_before_sync();
    if constexpr (PAIR) ptx::cluster_sync(); else __syncthreads();
    if (tid == 0) { trace_mark(a, 3, 3);  trace_block(a, 1); }
    if (warp == kMmaWarp) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(misc->tmem_base, kTmemCols);
    }
}

}  // namespace dsv4

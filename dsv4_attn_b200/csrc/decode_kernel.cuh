// Decode attention over an FP8 latent KV cache on sm_100a tensor cores.
//
// A thread block works through a list of work items.  An item is (query-token
// row n, group of 128 heads, a range of 64-entry tiles of that row); the block
// computes it for one half of the 512 value columns (the block with the other
// half runs the same list on the neighbouring SM).  The list is either the single
// item the block's grid position names (one launch = rows x head groups x splits
// blocks) or this block pair's slice of a schedule a planner kernel wrote (sched.cuh):
// the block then stays resident, keeps its tensor memory and barriers, and overlaps
// the set-up of the next item with the tail of the current one.
// Per 64-entry tile:
//   loader warps   gather the entries (index list -> block table -> 656-byte
//                  rows, or the dense / reference-layout equivalents) into
//                  registers, dequantise FP8 * scale -> FP16 (BF16 for the reference
//                  layouts) and write the tile into shared memory in the
//                  128-byte-swizzled operand layout;
//   MMA threads    S[128 heads x 64] = Q . K^T   (tcgen05.mma, K = 576 or 512) into
//                  tensor memory, later O[128 x 256] += P . V with V read from the
//                  same tile as an MN-major operand;
//   softmax warps  read S from tensor memory (one head per thread), run the
//                  online softmax with a lazily updated reference maximum,
//                  write P to tensor memory, rescale O in tensor memory
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
constexpr int kQChunkBytes = 128 * 128;   // 128 heads x 64 16-bit values
constexpr int kKvChunkBytes = kTileN * 128;  // 64 entries x 64 16-bit values
// Warp roles, four warpgroups of four warps.  Warps 0-3: softmax + epilogue.
// Warps 4-11: loaders (and the Q set-up).  Warp 12: issue of the S = Q.K^T MMAs, the Q load and the
// tensor-memory allocation; warp 13: issue of the O += P.V MMAs (its own thread, so that a ready P never
// waits for the other thread to finish issuing a group: an issuing thread is held while the tensor pipe's
// short queue is full); warp 14: walks the block's items and resolves, several tiles ahead, where every
// entry lives (index list -> block table -> record number), so that the loaders start from record numbers
// in shared memory; warp 15 only takes part in the block-wide barriers.  All 16 warps start with 128
// registers (the whole register file); the last warpgroup gives most of its
// share back and the loaders take it, so that they can hold two tiles of cache
// entries in flight.  setmaxnreg.inc waits for registers without a time limit,
// so the matching .dec must be reached unconditionally, as it is here.
constexpr int kNumSoftmaxWarps = 4;
constexpr int kNumLoaderWarps = 8;
constexpr int kFirstLoaderWarp = 4;
constexpr int kMmaWarp = 12;
constexpr int kNumWarps = 16;
constexpr int kLoaderThreads = kNumLoaderWarps * 32;
constexpr int kLoaderRegs = 160;       // 8 x 32 x (160-128) = 8192 registers taken ...
constexpr int kIdleRegs = 64;          // ... from 4 x 32 x (128-64) = 8192 released
constexpr int kNumThreads = kNumWarps * 32;  // 512
constexpr int kNumKvGroups = 2;        // hand-overs per tile from the loaders to the MMA thread
constexpr int kQTmemChunks = 4;        // Q chunks (64 columns each) held in tensor memory as the A operand
constexpr int kTmemCols = 512;
constexpr int kTmemS = 0;              // two S accumulators of 64 columns; P overwrites the first 32 of its S
constexpr int kTmemO = 128;            // O accumulator: 256 columns
constexpr int kTmemQ = 384;            // Q chunks 0..3 as packed 16-bit values: 4 x 32 columns
constexpr unsigned long long kDefaultWaitNs = 2000000000ull;  // 2 s
constexpr float kRescaleThreshold = 8.0f;  // log2 units; O is rescaled only when the max grows by more
constexpr int kItemWords = 8;          // int32 words per work item of a schedule
constexpr int kResolveWarp = 14;       // resolves the entries of the tiles ahead of the loaders
constexpr int kRing = 6;               // tiles the resolver may be ahead of the loaders' fetches

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
    kStatusBadIndex = 7,       // an index, length or block-table value pointed outside the cache: entry left out, not read
    kStatusWaitEpilogue = 8,
    kStatusWaitResolver = 9,
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
    long long num_pages; // pages in kv_pool: block-table values outside [0, num_pages) are not followed
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
    float* partial_o;            // split partials, stored as BF16 (the area is sized for FP32)
    float* partial_lse;
    int32_t* status;
    // schedule (sched.cuh): null = one item per block, named by the grid position
    const int32_t* sched_pair_begin;   // [pairs + 1]: first item of every block pair
    const int32_t* sched_items;        // [items][kItemWords]
#ifdef DSV4_TRACE
    unsigned long long* trace;         // development builds only: block 0 stores %globaltimer values here, 1024 slots per role
#endif
    unsigned long long wait_ns;        // limit of every bounded wait
    int dbg_drop_tile;                 // test aid (-1 = off): the loaders withhold the hand-over of the block's tile with this
                                       // running number, so that a bounded wait runs out and the error path can be checked
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

// One unit of work of a block: tiles [tile0, tile0 + ntiles) of row n for head group hg.
struct Item {
    int n, b, hg;
    int tile0, ntiles;
    int n_tok;        // entries of the row that take part (index-list slots in use, or kv_len + win_len)
    int kv_len_n;     // CSA: causal bound on index values; HCA: entries read through the block table
    int slot;         // < 0: the item is the whole row, write out / lse; else the partial slot to write
};

template <int NCHUNK>
struct SmemLayout {
    static constexpr int kQSmemChunks = NCHUNK - kQTmemChunks;      // Q chunks kept in shared memory
    static constexpr int kQBytes = kQSmemChunks * kQChunkBytes;
    static constexpr int kKvStageBytes = NCHUNK * kKvChunkBytes;
    static constexpr int kQOff = 0;
    static constexpr int kKvOff = kQBytes;                          // two stages
    static constexpr int kMiscOff = kKvOff + 2 * kKvStageBytes;
    static constexpr int kMiscBytes = 2048;
    static constexpr int kTotal = kMiscOff + kMiscBytes + 1024;     // + slack to align the base to 1024
    static_assert(kQTmemChunks * kQChunkBytes <= kKvStageBytes, "Q staging must fit in one KV stage");
    // epilogue staging inside one KV stage: per warp 32 rows of kEpiCols BF16 + 16 bytes; all 256 value columns at
    // once where the stage is large enough, else 128 at a time
    static constexpr int kEpiPasses = (kNumSoftmaxWarps * 32 * (kDvHalf * 2 + 16) <= kKvStageBytes) ? 1 : 2;
    static constexpr int kEpiCols = kDvHalf / kEpiPasses;
    static constexpr int kEpiPitch = kEpiCols * 2 + 16;
    static constexpr int kEpiWarpBytes = 32 * kEpiPitch;
    static_assert(kNumSoftmaxWarps * kEpiWarpBytes <= kKvStageBytes, "epilogue staging must fit in one KV stage");
};

// What the resolver hands the loaders for one tile.
struct TileSlot {
    uint32_t id[kTileN];      // per entry: bit 31 = takes part, bit 30 = second pool (window), low bits = record number
    uint64_t mask;            // bit t = entry t takes part
    uint32_t meta;            // row | head group << 16 | first tile of its item << 24 | last << 25 | bit 31: a tile at all
    uint32_t pad;
};

struct SmemMisc {
    TileSlot ring[kRing];
    uint64_t bar_res_full[kRing];    // slot written by the resolver
    uint64_t bar_res_empty[kRing];   // slot read by all loader warps
    uint64_t bar_kv_full[2][kNumKvGroups];   // [stage][group]: group written by all loader warps
    uint64_t bar_kv_free[2];
    uint64_t bar_s_full[2];
    uint64_t bar_p_full[2];
    uint64_t bar_o_full;      // per item: all P.V of the item have completed
    uint64_t bar_q_full;      // per item: Q chunks of the item landed in shared memory (TMA transaction count)
    uint64_t bar_q_ready;     // per item: Q in tensor memory, shared-memory chunks converted
    uint64_t bar_tmem;        // tensor memory allocated, its address in tmem_base
    uint64_t bar_q_copied;    // per item: every loader warp has copied its share of Q out of the staging area
    uint64_t valid_mask[2];   // per stage: bit t = entry t of the tile takes part in the softmax
    uint32_t tmem_base;
    uint32_t pad;
    volatile uint32_t epi_done[kNumSoftmaxWarps];   // items whose epilogue this softmax warp has finished (staging area free again)
};

__device__ __forceinline__ void report_status(int32_t* status, int code, int role, int tile) {
    if (status != nullptr) {
        if (atomicCAS(status, 0, code) == 0) {
            status[1] = int(blockIdx.x) | (int(blockIdx.y) << 8) | (int(blockIdx.z) << 20);
            status[2] = role;
            status[3] = tile;
        }
    }
}

// Development builds (-DDSV4_TRACE): block 0 records when its roles pass their pipeline points
// (role 0 softmax, 1 Q.K^T issue, 2 loader warp 0, 3 P.V issue).  Compiled out of the product.
#ifdef DSV4_TRACE
__device__ __forceinline__ void trace_mark(const DecodeArgs& a, int role, int slot) {
    if (a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && slot < 1024) {
        const long long c = clock64();                      // SM cycles: cheap to read, and one block = one SM
        a.trace[role * 1024 + slot] = c;
        a.trace[(4 + role) * 1024 + slot] = c;              // the trace buffer holds 12 x 1024 words
    }
}
#else
__device__ __forceinline__ void trace_mark(const DecodeArgs&, int, int) {}
#endif

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
    uint32_t a, b;
    ptx::e4m3x4_to_f16x4(w, a, b);
    const __half2 x = __hmul2(*reinterpret_cast<const __half2*>(&a), scale2);
    const __half2 y = __hmul2(*reinterpret_cast<const __half2*>(&b), scale2);
    lo = *reinterpret_cast<const uint32_t*>(&x);
    hi = *reinterpret_cast<const uint32_t*>(&y);
}

// Registers one loader thread holds for one tile.  A loader warp owns 8
// consecutive entries of the tile, as two groups of 4.  lane%8 picks one 16-byte piece of a 128-byte span
// (two 64-element latent chunks, or the RoPE tail); lane/8, with its lowest bit flipped in the lanes of
// the span's second chunk (loader_entry), picks the entry of a group.  One load instruction then covers
// 4 entries x 128 contiguous bytes: measured on this part, an SM pulls records about 1.6 times
// faster in this shape than with 64 bytes per entry per instruction.  The flip is for the stores: the 8
// lanes of a quarter-warp then write two neighbouring rows of the tile, whose swizzles differ in the lowest
// bit, and every store instruction covers all eight 16-byte bank groups without any lane-dependent choice
// of what to store.
__device__ __forceinline__ int loader_entry(int lane, int g) { return 4 * g + ((lane >> 3) ^ ((lane >> 2) & 1)); }

template <int SRC>
struct LoaderRegs {
    uint4 lat[2][4];         // [group][span j]: bytes [128 j + 16 (lane%8), +16) of the latent of entry loader_entry(lane, group)
    uint4 rope[2];           // [group]: RoPE 16-byte column lane%8 of that entry
    uint32_t sc[2][4];       // [group]: packed layout: the 4 FP32 scales; reference layout: the 7 UE8M0 bytes (2 words)
    uint32_t vmask;          // bit i = entry i of this warp takes part (same in all lanes)
    // An entry that does not take part holds zeros here (latent, RoPE and scales), so that the stores
    // need no validity test: a zero row stays finite under the MMA whatever its probability column holds.
};

// Where an entry lives, as a 32-bit record number with bit 31 = "takes part" and bit 30 = "second pool"
// (the window buffer / the sliding-window planes or pages): for the packed layout the number of its
// 656-byte record in the pool (page * 64 + slot) or in the window buffer (request * win_cap + row); for
// packed reference pages page << 6 | slot; for the reference planes the row number in the plane.  The
// resolver warp works these out several tiles ahead of the data loads, in stages, so that no stage uses
// the result of a load issued in the same step: the index -> block table -> record chain is off the
// critical path.
constexpr uint32_t kIdValid = 1u << 31, kIdSecond = 1u << 30, kIdNumber = (1u << 30) - 1u;

// What a tile's position in its row needs to be resolved (the same in all lanes of a warp).
struct TileCtx {
    int n, b;
    int n_tok, kv_len_n;
    int v0;              // first entry of the tile in its row
    uint32_t meta;       // row | head group << 16 | first tile of its item << 24 | last tile << 25 | bit 31: a tile at all
};
constexpr uint32_t kMetaFirst = 1u << 24, kMetaLast = 1u << 25, kMetaTile = 1u << 31;

// A resolution in flight: the block-table value requested (not yet looked at) and what is known already.
struct PendingId {
    int page;          // block-table value on its way; kNoPage: `id` is final
    uint32_t id;       // paged: kIdValid | second pool | slot in the page;  otherwise the final record number
};
constexpr int kNoPage = -2;

// Stage 1 (CSA only): the index-list value of entry `ent` of the tile, -1 where there is none.
__device__ __forceinline__ int resolve_index(const DecodeArgs& a, const TileCtx& c, int ent) {
    const int v = c.v0 + ent;
    if ((c.meta & kMetaTile) && v < c.n_tok) return __ldg(a.indices + int64_t(c.n) * a.topk + v);
    return -1;
}

// Stage 2: issue the block-table load (where there is one).  `e` is the index-list value (CSA).  An entry
// whose page slot lies outside the block table, or whose window row lies outside the window buffer, is
// reported and left out; nothing is read through it.
template <int SRC>
__device__ __forceinline__ PendingId resolve_issue(const DecodeArgs& a, const TileCtx& c, int e, int ent) {
    PendingId p{kNoPage, 0u};
    const int v = c.v0 + ent;
    const bool in_row = (c.meta & kMetaTile) && v < c.n_tok;
    if constexpr (SRC == kSrcCsa) {
        if (e >= 0 && e < c.kv_len_n) {
            if ((e >> 6) < a.max_pages) {
                p.page = __ldg(a.block_table + int64_t(c.b) * a.max_pages + (e >> 6));
                p.id = kIdValid | uint32_t(e & 63);
            } else {
                report_status(a.status, kStatusBadIndex, 4, e);
            }
        }
    } else if constexpr (SRC == kSrcHca) {
        if (in_row) {
            if (v < c.kv_len_n) {
                if ((v >> 6) < a.max_pages) {
                    p.page = __ldg(a.block_table + int64_t(c.b) * a.max_pages + (v >> 6));
                    p.id = kIdValid | uint32_t(v & 63);
                } else {
                    report_status(a.status, kStatusBadIndex, 4, v);
                }
            } else if (v - c.kv_len_n < a.win_cap) {
                p.id = kIdValid | kIdSecond | uint32_t(c.b * a.win_cap + (v - c.kv_len_n));
            } else {
                report_status(a.status, kStatusBadIndex, 4, v);
            }
        }
    } else if constexpr (SRC == kSrcRefPaged) {
        // a token outside its block table, or a table value outside the pool, is left out of the
        // softmax instead of being read
        if (in_row) {
            const int slot_mask = (1 << a.pg_page_shift) - 1;
            const bool swa = v >= c.kv_len_n;
            const int w = swa ? v - c.kv_len_n : v;
            const uint8_t* pool = swa ? a.pg_swa : a.pg_kv;
            const int32_t* table = swa ? a.pg_swa_table : a.block_table;
            const int cols = swa ? a.pg_swa_max_pages : a.max_pages;
            if (pool != nullptr && (w >> a.pg_page_shift) < cols) {
                p.page = __ldg(table + int64_t(c.b) * cols + (w >> a.pg_page_shift));
                p.id = kIdValid | (swa ? kIdSecond : 0u) | uint32_t(w & slot_mask);
            }
        }
    } else {
        if (in_row)
            p.id = kIdValid | ((v < a.ref_m_cur) ? uint32_t(c.b * a.ref_m_cur + v)
                                                 : (uint32_t(c.b * a.ref_swa_len + (v - a.ref_m_cur)) | kIdSecond));
    }
    return p;
}

// Stage 3 (a step later, when the block-table value has arrived): the record number.  A table value
// outside the pool is reported and the entry left out.
template <int SRC>
__device__ __forceinline__ uint32_t resolve_finish(const DecodeArgs& a, const PendingId& p) {
    if (p.page == kNoPage || !(p.id & kIdValid)) return p.id;
    if constexpr (SRC == kSrcRefPaged) {
        const int64_t pages = (p.id & kIdSecond) ? a.pg_swa_num_pages : a.pg_num_pages;
        if (p.page < 0 || p.page >= pages) return 0u;
        return (p.id & (kIdValid | kIdSecond)) | (uint32_t(p.page) << 6) | (p.id & 63u);
    } else {
        if (p.page < 0 || (long long)p.page >= a.num_pages) {
            report_status(a.status, kStatusBadIndex, 4, p.page);
            return 0u;
        }
        return kIdValid | (uint32_t(p.page) * 64u + (p.id & 63u));
    }
}

// Issue the loads of one tile for this lane's two entries (record numbers id[0], id[1]).
template <int SRC>
__device__ __forceinline__ void loader_fetch(const DecodeArgs& a, const uint32_t (&id)[2], uint32_t vmask, int lane,
                                             LoaderRegs<SRC>& r) {
    r.vmask = vmask;
    const int piece = lane & 7;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const int i = loader_entry(lane, g);
        if (!((vmask >> i) & 1u)) {
#pragma unroll
            for (int j = 0; j < 4; ++j) { r.lat[g][j] = make_uint4(0, 0, 0, 0);  r.sc[g][j] = 0u; }
            r.rope[g] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const uint32_t num = id[g] & kIdNumber;
        const bool second = (id[g] & kIdSecond) != 0u;
        if constexpr (!is_ref_layout(SRC)) {
            const uint8_t* row = (second ? a.win_pool : a.kv_pool) + int64_t(num) * 656;
#pragma unroll
            for (int j = 0; j < 4; ++j) r.lat[g][j] = ptx::ldg_nc_v4(row + j * 128 + piece * 16);
            const uint4 s4 = ptx::ldg_nc_v4(row + 512);
            r.sc[g][0] = s4.x;  r.sc[g][1] = s4.y;  r.sc[g][2] = s4.z;  r.sc[g][3] = s4.w;
            r.rope[g] = ptx::ldg_nc_v4(row + 528 + piece * 16);
        } else if constexpr (SRC == kSrcRefPaged) {
            const int slot = int(num & 63u);
            const uint8_t* lp = (second ? a.pg_swa : a.pg_kv) + int64_t(num >> 6) * a.pg_page_bytes + slot * 576;
            // the page's scale area starts after its page_size tokens: 8 bytes per token
            const uint8_t* sp = lp + int64_t((1 << a.pg_page_shift) - slot) * 576 + slot * 8;
#pragma unroll
            for (int j = 0; j < 3; ++j) r.lat[g][j] = ptx::ldg_nc_v4(lp + j * 128 + piece * 16);
            if (piece < 4) r.lat[g][3] = ptx::ldg_nc_v4(lp + 384 + piece * 16);
            const uint2 s2 = __ldg(reinterpret_cast<const uint2*>(sp));
            r.sc[g][0] = s2.x;  r.sc[g][1] = s2.y;
            r.rope[g] = ptx::ldg_nc_v4(lp + 448 + piece * 16);
        } else {
            const int64_t e = int64_t(num);
            const uint8_t* lp = (second ? a.ref_ks : a.ref_kc) + e * 448;
            const uint8_t* sp = (second ? a.ref_ks_s : a.ref_kc_s) + e * 7;
            const uint8_t* rp = reinterpret_cast<const uint8_t*>(second ? a.ref_ks_rope : a.ref_kc_rope) + e * 128;
#pragma unroll
            for (int j = 0; j < 3; ++j) r.lat[g][j] = ptx::ldg_nc_v4(lp + j * 128 + piece * 16);
            // the last span holds only chunk 6 (bytes 384..447 of the 448-byte row)
            if (piece < 4) r.lat[g][3] = ptx::ldg_nc_v4(lp + 384 + piece * 16);
            // this lane dequantises chunk 2 j + (lane / 4) % 2 of span j: only those scale bytes are fetched
            const int flip = (lane >> 2) & 1;
#pragma unroll
            for (int j = 0; j < 4; ++j) r.sc[g][j] = (2 * j + flip < 7) ? uint32_t(__ldg(sp + 2 * j + flip)) : 0u;
            r.rope[g] = ptx::ldg_nc_v4(rp + piece * 16);
        }
    }
}

// Pull the record of one entry into L2 ahead of the loads (the packed layouts: one contiguous record).
template <int SRC>
__device__ __forceinline__ void prefetch_record_l2(const DecodeArgs& a, uint32_t id) {
    if (!(id & kIdValid)) return;
    const uint32_t num = id & kIdNumber;
    const bool second = (id & kIdSecond) != 0u;
    if constexpr (!is_ref_layout(SRC)) {
        const uint8_t* row = (second ? a.win_pool : a.kv_pool) + int64_t(num) * 656;
#pragma unroll
        for (int j = 0; j < 6; ++j) ptx::prefetch_l2(row + j * 128);
    } else if constexpr (SRC == kSrcRefPaged) {
        const uint8_t* lp = (second ? a.pg_swa : a.pg_kv) + int64_t(num >> 6) * a.pg_page_bytes + int(num & 63u) * 576;
#pragma unroll
        for (int j = 0; j < 5; ++j) ptx::prefetch_l2(lp + j * 128);
    }
}

// Where this lane's stores of one tile go: for each of its two entries the shared-memory address of the first
// of the two 16-byte columns its 16 latent bytes of span 0 expand to (the second column is that address ^ 16;
// span j lies 2 j chunks further on), and the address of its RoPE column.  Row t of a chunk is 128 bytes;
// 16-byte column c16 of row t lives at ((c16 ^ (t & 7)) << 4).
struct LoaderAddr {
    uint32_t lat[2];
};
template <int NCHUNK>
__device__ __forceinline__ LoaderAddr loader_addresses(uint32_t kv_st, int t0, int lane) {
    LoaderAddr r;
    const uint32_t piece = uint32_t(lane & 7);
    const uint32_t flip = piece >> 2;                          // this lane's chunk within a span
    const uint32_t p = piece & 3u;                             // 16 latent bytes -> 16-byte columns 2p, 2p+1
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const uint32_t t = uint32_t(t0 + loader_entry(lane, g));
        const uint32_t row = kv_st + t * 128u;
        r.lat[g] = row + flip * kKvChunkBytes + (((2u * p) ^ (t & 7u)) << 4);
    }
    return r;
}

// Dequantise and write span j (latent chunks 2j and 2j+1) of this warp's 8 entries.  A 16-byte store is
// served per quarter-warp: its 8 lanes write the even columns of one row of chunk 2j and - one row further,
// where the swizzle turns them into the odd bank groups - the even columns of chunk 2j+1 (the chunks are
// 8 KB apart: same banks), then the odd ones: all eight 16-byte bank groups once per instruction, four
// shared-memory wavefronts per 512 bytes.
template <int NCHUNK, int SRC>
__device__ __forceinline__ void loader_store_span(const LoaderAddr& ad, int lane, const LoaderRegs<SRC>& r, int j) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const uint4 x = r.lat[g][j];
        uint4 w0, w1;
        if constexpr (use_f16(SRC)) {
            // scales above 146 would take 448 x scale past FP16's largest finite value: such blocks saturate
            const __half2 scale2 = __float2half2_rn(fminf(__uint_as_float(r.sc[g][j]), 146.f));
            dequant4_f16(x.x, scale2, w0.x, w0.y);
            dequant4_f16(x.y, scale2, w0.z, w0.w);
            dequant4_f16(x.z, scale2, w1.x, w1.y);
            dequant4_f16(x.w, scale2, w1.z, w1.w);
        } else {
            const uint32_t c = 2u * uint32_t(j) + (uint32_t(lane >> 2) & 1u);      // this lane's chunk
            if (c >= uint32_t(NCHUNK - 1)) continue;               // reference layout: span 3 ends with chunk 6
            // one UE8M0 byte per 64 elements: 2^(byte-127) * 2^120; a zero byte means a zero
            // scale, as in the reference's dequantiser
            const uint32_t byte = (SRC == kSrcRef) ? r.sc[g][j]
                                                   : ((c < 4u ? r.sc[g][0] >> (8u * c) : r.sc[g][1] >> (8u * (c - 4u))) & 0xFFu);
            const float s120 = byte ? __uint_as_float((byte + 120u) << 23) : 0.f;
            const __nv_bfloat162 scale2 = __float2bfloat162_rn(s120);
            dequant4(x.x, scale2, w0.x, w0.y);
            dequant4(x.y, scale2, w0.z, w0.w);
            dequant4(x.z, scale2, w1.x, w1.y);
            dequant4(x.w, scale2, w1.z, w1.w);
        }
        const uint32_t at = ad.lat[g] + uint32_t(j) * 2u * kKvChunkBytes;
        ptx::sts_v4(at, w0);
        ptx::sts_v4(at ^ 16u, w1);
    }
}

// The RoPE tail (chunk NCHUNK-1, a plain copy): 4 rows x 8 columns per store instruction.
template <int NCHUNK, int SRC>
__device__ __forceinline__ void loader_store_rope(const LoaderAddr& ad, int lane, const LoaderRegs<SRC>& r) {
    // the RoPE column of this lane from the address of its first latent column: same row, chunk NCHUNK-1,
    // column lane%8 instead of 2 (lane%4)   (both swizzled by the same row bits: the XOR of the two columns)
    const uint32_t piece = uint32_t(lane & 7), flip = piece >> 2;
    const uint32_t delta = (uint32_t(NCHUNK - 1) - flip) * kKvChunkBytes;
    const uint32_t colx = (piece ^ (2u * (piece & 3u))) << 4;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        uint4 w = r.rope[g];
        if constexpr (use_f16(SRC)) {
            w.x = ptx::bf16x2_to_f16x2(w.x);  w.y = ptx::bf16x2_to_f16x2(w.y);
            w.z = ptx::bf16x2_to_f16x2(w.z);  w.w = ptx::bf16x2_to_f16x2(w.w);
        }
        ptx::sts_v4((ad.lat[g] ^ colx) + delta, w);
    }
}

// BF16 -> FP16 in place over the Q chunks that stay in shared memory, one share per loader
// thread, then the proxy fence that makes the result visible to the MMAs' reads.
// Element-wise, so the swizzled layout is untouched.
template <int BYTES>
__device__ __forceinline__ void convert_q_smem(uint32_t q_base, int ltid) {
#pragma unroll 5
    for (int i = ltid; i < BYTES / 16; i += kLoaderThreads) {
        uint4 x = ptx::lds_v4(q_base + uint32_t(i) * 16u);
        x.x = ptx::bf16x2_to_f16x2(x.x);  x.y = ptx::bf16x2_to_f16x2(x.y);
        x.z = ptx::bf16x2_to_f16x2(x.z);  x.w = ptx::bf16x2_to_f16x2(x.w);
        ptx::sts_v4(q_base + uint32_t(i) * 16u, x);
    }
}

// Copy Q chunks g0 and g0 + 1 of the 32 head rows of lane quarter `lw % 4` from their staging area (the
// swizzled 16 KB chunks the TMA wrote) to tensor memory: head row = tensor-memory lane, two 16-bit values per
// 32-bit column, in K order (the A-operand layout of the MMA); converted to FP16 on the way when the kernel
// runs on FP16.
template <bool F16>
__device__ __forceinline__ void copy_q_chunks_to_tmem(uint32_t stage_base, uint32_t tmem, int lw, int lane) {
    const int quarter = lw & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const uint32_t srow = stage_base + uint32_t(r) * 128u;
    const uint32_t sw = uint32_t(r & 7);
    const int g0 = 2 * (lw >> 2);
#pragma unroll
    for (int g = g0; g < g0 + 2; ++g) {
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

// A loader warp's share of the Q set-up of an item: wait for the TMA,
// copy two of the staged chunks to tensor memory, convert this thread's part of the chunks that stay in shared
// memory.  Returns false when the wait ran out.
template <int NCHUNK, int SRC>
__device__ __forceinline__ bool loader_q_setup(uint32_t bar_q_full, uint32_t parity, unsigned long long wait_ns, uint32_t stage_base,
                                            uint32_t tmem, uint32_t q_base, int lw, int lane, int ltid) {
    const bool w = ptx::mbar_wait(bar_q_full, parity, wait_ns);
    if (!__all_sync(0xFFFFFFFFu, w)) return false;
    copy_q_chunks_to_tmem<use_f16(SRC)>(stage_base, tmem, lw, lane);
    if constexpr (use_f16(SRC)) convert_q_smem<SmemLayout<NCHUNK>::kQBytes>(q_base, ltid);
    ptx::fence_proxy_async_smem();
    ptx::tmem_wait_st();
    ptx::tc_fence_before_sync();
    return true;
}

// The Q rows of an item pulled into L2 ahead of their use: 128 rows x NCHUNK x 128 bytes, spread over the calling threads.
template <int NCHUNK>
__device__ __forceinline__ void prefetch_q_l2(const DecodeArgs& a, int n, int hg, int t, int nthreads) {
    const uint8_t* base = reinterpret_cast<const uint8_t*>(a.q + (int64_t(n) * a.H + hg * kHeadsPerCta) * (64 * NCHUNK));
    const int rows = min(kHeadsPerCta, a.H - hg * kHeadsPerCta);
    for (int l = t; l < rows * NCHUNK; l += nthreads) ptx::prefetch_l2(base + int64_t(l) * 128);
}

// The row lengths of an item, from the per-row length arrays.
template <int SRC>
__device__ __forceinline__ void row_lengths(const DecodeArgs& a, int n, int& n_tok, int& kv_len_n) {
    if constexpr (SRC == kSrcCsa) {
        const int raw = (a.topk_len != nullptr) ? __ldg(a.topk_len + n) : a.topk;
        n_tok = min(max(raw, 0), a.topk);
        kv_len_n = (a.kv_len != nullptr) ? __ldg(a.kv_len + n) : 0x7FFFFFFF;
    } else if constexpr (SRC == kSrcHca || SRC == kSrcRefPaged) {
        kv_len_n = max(__ldg(a.kv_len + n), 0);
        n_tok = kv_len_n + max(__ldg(a.win_len + n), 0);
    } else {
        kv_len_n = a.ref_m_cur;
        n_tok = a.ref_m_cur + a.ref_swa_len;
    }
}

template <int NCHUNK, int SRC>
__global__ void __launch_bounds__(kNumThreads, 1) decode_mma_kernel(const __grid_constant__ DecodeArgs a) {
    using L = SmemLayout<NCHUNK>;
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
    const bool sched = a.sched_pair_begin != nullptr;
    const int rows = a.B * a.s_q;
    const unsigned long long wait_ns = a.wait_ns;

    // ── this block's items ──
    int item_begin = 0, n_items = 1;
    if (sched) {
        const int pair = blockIdx.x >> 1;
        item_begin = __ldg(a.sched_pair_begin + pair);
        n_items = __ldg(a.sched_pair_begin + pair + 1) - item_begin;
    }
    auto get_item = [&](int k) -> Item {
        Item it;
        if (sched) {
            const int4* rec = reinterpret_cast<const int4*>(a.sched_items + int64_t(item_begin + k) * kItemWords);
            const int4 r0 = __ldg(rec), r1 = __ldg(rec + 1);
            it.n = r0.x;  it.hg = r0.y;  it.tile0 = r0.z;  it.ntiles = r0.w;
            it.slot = r1.x;  it.n_tok = r1.y;  it.kv_len_n = r1.z;
        } else {
            it.n = blockIdx.y;  it.hg = blockIdx.x >> 1;
            row_lengths<SRC>(a, it.n, it.n_tok, it.kv_len_n);
            const int split = blockIdx.z;
            const int tiles_total = (it.n_tok + kTileN - 1) / kTileN;
            const int tiles_per_split = (tiles_total + a.num_splits - 1) / a.num_splits;
            it.tile0 = min(split * tiles_per_split, tiles_total);
            it.ntiles = min(it.tile0 + tiles_per_split, tiles_total) - it.tile0;
            it.slot = a.num_splits > 1 ? split : -1;
        }
        it.b = it.n / a.s_q;
        return it;
    };
    // element index of head row 0 of the item's block of partial rows, and of its partial LSEs
    auto partial_row0 = [&](const Item& it) -> int64_t {
        return sched ? int64_t(it.slot) * kHeadsPerCta : (int64_t(it.slot) * rows + it.n) * a.H + it.hg * kHeadsPerCta;
    };

    const uint32_t v_off = uint32_t(half ? 4 : 0) * kKvChunkBytes;   // this block's value columns inside a stage

    const uint32_t bar_kv_full = ptx::smem_u32(&misc->bar_kv_full[0][0]);   // [stage][group] at +8*kNumKvGroups*stage + 8*group
    const uint32_t bar_kv_free = ptx::smem_u32(&misc->bar_kv_free[0]);
    const uint32_t bar_s_full = ptx::smem_u32(&misc->bar_s_full[0]);
    const uint32_t bar_p_full = ptx::smem_u32(&misc->bar_p_full[0]);
    const uint32_t bar_o_full = ptx::smem_u32(&misc->bar_o_full);
    const uint32_t bar_q_full = ptx::smem_u32(&misc->bar_q_full);
    const uint32_t bar_q_ready = ptx::smem_u32(&misc->bar_q_ready);
    const uint32_t bar_tmem = ptx::smem_u32(&misc->bar_tmem);
    const uint32_t bar_q_copied = ptx::smem_u32(&misc->bar_q_copied);
    constexpr uint32_t kKvFullStride = 8 * kNumKvGroups;
    const uint32_t bar_res_full = ptx::smem_u32(&misc->bar_res_full[0]);
    const uint32_t bar_res_empty = ptx::smem_u32(&misc->bar_res_empty[0]);

    // ── set-up ──
    if (tid == 0) {
        for (int st = 0; st < 2; ++st) {
            for (int g = 0; g < kNumKvGroups; ++g) ptx::mbar_init(bar_kv_full + kKvFullStride * st + 8 * g, kNumLoaderWarps);
            ptx::mbar_init(bar_kv_free + 8 * st, 1);
            ptx::mbar_init(bar_s_full + 8 * st, 1);
            ptx::mbar_init(bar_p_full + 8 * st, kNumSoftmaxWarps);
        }
        ptx::mbar_init(bar_o_full, 1);
        ptx::mbar_init(bar_q_full, 1);
        ptx::mbar_init(bar_q_ready, kNumLoaderWarps);
        ptx::mbar_init(bar_tmem, 1);
        ptx::mbar_init(bar_q_copied, kNumLoaderWarps);
        for (int i = 0; i < kRing; ++i) {
            ptx::mbar_init(bar_res_full + 8 * i, 1);
            ptx::mbar_init(bar_res_empty + 8 * i, kNumLoaderWarps);
        }
        for (int w = 0; w < kNumSoftmaxWarps; ++w) misc->epi_done[w] = 0u;
        ptx::fence_mbar_init();
    }

    // The barriers are initialised before any role starts.  The tensor-memory address is published through a
    // barrier of its own, so that the resolver and the loaders are at work while it is being allocated.
    __syncthreads();
    auto wait_tmem = [&]() -> bool {
        const bool w = ptx::mbar_wait(bar_tmem, 0u, wait_ns);
        ptx::tc_fence_after_sync();
        return w;
    };

    // Running counters, the same in every role: `gt` counts the tiles the block has gone through over all
    // its items (tile gt lives in stage gt & 1 and is the (gt >> 1)-th use of that stage's barriers), `qn`
    // the items that had tiles (the per-item barriers are in their qn-th phase).

    if (warp >= kFirstLoaderWarp && warp < kMmaWarp) {
        // ───────────── loader warps ─────────────
        // The tiles of all the block's items form one stream, described tile by tile by the resolver warp (record
        // numbers, validity mask, tag).  Two register sets: while one tile is dequantised and stored, the loads of
        // the next one are in flight - also across the boundary between two items.  The larger register allowance
        // holds for this branch only.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kLoaderRegs));
        const int lw = warp - kFirstLoaderWarp;
        const int ltid = tid - kFirstLoaderWarp * 32;
        const int row0 = 8 * lw;      // this warp's 8 entries: tile rows row0 .. row0+7
        LoaderRegs<SRC> regs_a, regs_b;
        uint32_t ma = 0, mb = 0;      // tags of the tiles in the two register sets
        uint32_t gt = 0, qn = 0;
        uint32_t pend0 = 0u, pend1 = 0u;     // per stage: the epilogue (by its running number) that must have released it before it is written again
        bool lok = true;

        // What the resolvers wrote for tile t of the stream, read into registers ahead of its loads: this lane's two
        // record numbers, this warp's validity bits, the tile's tag (0 past the end of the stream).
        struct TileInfo { uint32_t id[2]; uint32_t vmask; uint32_t meta; };
        auto peek_tile = [&](uint32_t t) -> TileInfo {
            TileInfo ti{{0u, 0u}, 0u, 0u};
            const uint32_t slot = t % kRing;
            const TileSlot& ts = misc->ring[slot];
            // The slot is normally long written (the resolver runs several tiles ahead): probe its barrier and read
            // the slot in one go, so that the two round trips through the shared-memory path overlap; only if the
            // probe fails, wait and read again.
            bool ready = ptx::mbar_test_wait(bar_res_full + 8 * slot, (t / kRing) & 1u);
            ti.meta = ts.meta;
            ti.id[0] = ts.id[row0 + loader_entry(lane, 0)];
            ti.id[1] = ts.id[row0 + loader_entry(lane, 1)];
            uint64_t mask = ts.mask;
            if (!__all_sync(0xFFFFFFFFu, ready)) {
                ready = ptx::mbar_wait(bar_res_full + 8 * slot, (t / kRing) & 1u, wait_ns);
                if (!__all_sync(0xFFFFFFFFu, ready)) {
                    report_status(a.status, kStatusWaitResolver, 2, int(t));
                    lok = false;
                    ti.meta = 0u;
                    return ti;
                }
                ti.meta = *reinterpret_cast<const volatile uint32_t*>(&ts.meta);
                ti.id[0] = *reinterpret_cast<const volatile uint32_t*>(&ts.id[row0 + loader_entry(lane, 0)]);
                ti.id[1] = *reinterpret_cast<const volatile uint32_t*>(&ts.id[row0 + loader_entry(lane, 1)]);
                mask = *reinterpret_cast<const volatile uint64_t*>(&ts.mask);
            }
            if (!(ti.meta & kMetaTile)) return ti;       // end of the stream (nothing to release: the resolver has stopped)
            ti.vmask = uint32_t(mask >> row0) & 0xFFu;
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_res_empty + 8 * slot);
            return ti;
        };
        // start the loads of that tile into `regs`; its tag goes to mt
        auto issue_tile = [&](const TileInfo& ti, LoaderRegs<SRC>& regs, uint32_t& mt) {
            mt = ti.meta;
            if (mt & kMetaTile) loader_fetch<SRC>(a, ti.id, ti.vmask, lane, regs);
        };
        auto fetch_tile = [&](uint32_t t, LoaderRegs<SRC>& regs, uint32_t& mt) {
            const TileInfo ti = peek_tile(t);
            issue_tile(ti, regs, mt);
        };
        // Only what the first tile needs goes out before the main loop: the number of loads an SM keeps in
        // flight is limited, and everything queued here delays tile 0.
        fetch_tile(0u, regs_a, ma);
        if (!__all_sync(0xFFFFFFFFu, wait_tmem())) {
            report_status(a.status, kStatusWaitQ, 2, -1);
            lok = false;
        }
        const uint32_t tmem = misc->tmem_base;

        // the stage of tile `g` must be free before it is written: the P.V of the tile two before it has completed, and
        // an output staged there (an item that ended with that tile) has been written out
        auto wait_stage_free = [&](uint32_t g) {
            const int st = int(g & 1u);
            if (g >= 2u) {
                // warp-uniform outcome: the warp-collective operations below need all lanes
                const bool w = ptx::mbar_wait(bar_kv_free + 8 * st, ((g >> 1) - 1u) & 1u, wait_ns);
                if (!__all_sync(0xFFFFFFFFu, w)) {
                    report_status(a.status, kStatusWaitKvFree, 2, int(g));
                    lok = false;
                    return;
                }
            }
            const uint32_t need = st ? pend1 : pend0;
            if (need != 0u) {
                const unsigned long long t0 = ptx::globaltimer_ns();
                bool free_now = false;
                while (true) {
                    free_now = misc->epi_done[0] >= need && misc->epi_done[1] >= need &&
                               misc->epi_done[2] >= need && misc->epi_done[3] >= need;
                    if (free_now || ptx::globaltimer_ns() - t0 > wait_ns) break;
                }
                if (!__all_sync(0xFFFFFFFFu, free_now)) {
                    report_status(a.status, kStatusWaitEpilogue, 2, int(g));
                    lok = false;
                    return;
                }
                __threadfence_block();
                if (st) pend1 = 0u; else pend0 = 0u;
            }
        };

        // one step: store the tile in `regs` (tag `mt`), then start the loads of the tile after next into the same set
        auto tile_step = [&](LoaderRegs<SRC>& regs, uint32_t& mt, auto first_tag) {
            constexpr bool kFirstStep = decltype(first_tag)::value;
            const uint32_t g = gt;
            const int st = int(g & 1u);
            if (lw == 0 && lane == 0) trace_mark(a, 2, 4 * int(g));
            if (mt & kMetaFirst) {
                // Q of the item that starts here has been sent for by the MMA thread (TMA, once the previous item's Q.K^T
                // had completed and this tile's stage was free): the chunks that stay in shared memory land at their
                // place and are converted there; the chunks that live in tensor memory land in this tile's stage,
                // which is written only after every loader warp has copied its share out of it.
                if (!loader_q_setup<NCHUNK, SRC>(bar_q_full, qn & 1u, wait_ns, kv_base + uint32_t(st) * L::kKvStageBytes, tmem, q_base,
                                                 lw, lane, ltid)) {
                    report_status(a.status, kStatusWaitQ, 2, int(g));
                    lok = false;
                }
                __syncwarp();
                if (lw == 0 && lane == 0) trace_mark(a, 2, 600 + 4 * int(qn) + 1);
                if (lane == 0) {
                    ptx::mbar_arrive(bar_q_ready);      // also after a time-out, so that nobody waits for this warp
                    ptx::mbar_arrive(bar_q_copied);
                }
                if (!lok) return;
                // the staging area is this tile's stage: no loader warp writes it before all have read it
                if (!__all_sync(0xFFFFFFFFu, ptx::mbar_wait(bar_q_copied, qn & 1u, wait_ns))) {
                    report_status(a.status, kStatusWaitQ, 2, int(g));
                    lok = false;
                    return;
                }
                if (lw == 0 && lane == 0) trace_mark(a, 2, 600 + 4 * int(qn) + 2);
            }
            wait_stage_free(g);
            if (!lok) return;
            if (lw == 0 && lane == 0) trace_mark(a, 2, 4 * int(g) + 1);
            if (lane == 0) reinterpret_cast<volatile uint8_t*>(&misc->valid_mask[st])[lw] = uint8_t(regs.vmask);
            // in two groups (chunks 0-3, then the rest with the RoPE tail), so that the QK MMAs of this tile
            // start while it is still being written; one proxy fence and one arrival per group
            const uint32_t kv_st = kv_base + uint32_t(st) * L::kKvStageBytes;
            const bool drop = a.dbg_drop_tile >= 0 && g == uint32_t(a.dbg_drop_tile);
            auto group_done = [&](int grp) {
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && !drop) ptx::mbar_arrive(bar_kv_full + kKvFullStride * st + 8 * grp);
            };
            const LoaderAddr ad = loader_addresses<NCHUNK>(kv_st, row0, lane);
            loader_store_span<NCHUNK, SRC>(ad, lane, regs, 0);
            loader_store_span<NCHUNK, SRC>(ad, lane, regs, 1);
            group_done(0);
            loader_store_span<NCHUNK, SRC>(ad, lane, regs, 2);
            loader_store_span<NCHUNK, SRC>(ad, lane, regs, 3);
            loader_store_rope<NCHUNK, SRC>(ad, lane, regs);
            group_done(1);
            if (lw == 0 && lane == 0) trace_mark(a, 2, 4 * int(g) + 2);
            if (mt & kMetaLast) {
                ++qn;
                if (st) pend1 = qn; else pend0 = qn;       // the item's output is staged in the stage of its last tile
            }
            ++gt;
            if constexpr (kFirstStep) {
                // The stream's first tile is complete.  The loads of the second are requested only here: queued
                // earlier they would hold up the stores above (the load/store unit takes about a microsecond to
                // accept a tile's worth of loads).
                fetch_tile(1u, regs_b, mb);
            }
            // this set is free again: loads of the tile after next
            if (lok) fetch_tile(g + 2u, regs, mt);
            if (lw == 0 && lane == 0) trace_mark(a, 2, 4 * int(g) + 3);
        };
        if (lok && (ma & kMetaTile)) tile_step(regs_a, ma, std::true_type{});
        while (lok && ((ma | mb) & kMetaTile)) {
            if (mb & kMetaTile) tile_step(regs_b, mb, std::false_type{});
            if (lok && (ma & kMetaTile)) tile_step(regs_a, ma, std::false_type{});
        }
    } else if (warp >= kMmaWarp) {
        // ───────────── last warpgroup: MMA issue (one thread each of warps 12 and 13), tensor-memory owner ─────────────
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kIdleRegs));
        if (warp == kMmaWarp) {
            ptx::tmem_alloc(ptx::smem_u32(&misc->tmem_base), kTmemCols);
            ptx::tmem_relinquish();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_tmem);
        }
        if (warp == kMmaWarp) {
            if (lane == 0) {
                const bool have_tmem = wait_tmem();
                const uint32_t tmem = misc->tmem_base;
                constexpr uint32_t idesc_qk = use_f16(SRC) ? ptx::make_idesc_f16(128, kTileN, false, false)
                                                            : ptx::make_idesc_bf16(128, kTileN, false, false);
                constexpr uint32_t kDescHi = ptx::smem_desc_hi(1024);        // 8-row groups 1 KB apart
                const uint32_t q_lo = ptx::smem_desc_lo(q_base, 16);
                // Chunks [C0, C1) (4 MMAs each) of S = Q . K^T of the tile in stage st into S buffer st; the chunk
                // range is a compile-time constant so that the descriptors fold to immediates.
                auto issue_qk_range = [&](int st, auto c0_tag, auto c1_tag) {
                    constexpr int C0 = decltype(c0_tag)::value, C1 = decltype(c1_tag)::value;
                    const uint32_t k_lo = ptx::smem_desc_lo(kv_base + uint32_t(st) * L::kKvStageBytes, 16);
                    const uint32_t d = tmem + kTmemS + uint32_t(st) * kTileN;
#pragma unroll
                    for (int c = C0; c < C1; ++c) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            // descriptor start addresses advance by constants (in 16-byte units)
                            const uint32_t b_lo = k_lo + uint32_t((c * kKvChunkBytes + k * 32) >> 4);
                            if (c < kQTmemChunks) {
                                // A = Q columns in tensor memory: 16 values = 8 columns per K step
                                ptx::mma_bf16_ts2(d, tmem + kTmemQ + c * 32 + k * 8, b_lo, kDescHi, idesc_qk, (c | k) ? 1u : 0u);
                            } else {
                                const uint32_t a_lo = q_lo + uint32_t(((c - kQTmemChunks) * kQChunkBytes + k * 32) >> 4);
                                ptx::mma_bf16_ss2(d, a_lo, b_lo, kDescHi, idesc_qk, 1u);
                            }
                        }
                    }
                };
                static_assert(kNumKvGroups == 2, "group dispatch below is written for 2 groups");
                // This thread issues only S = Q.K^T, group by group as the loaders deliver them; O += P.V is
                // issued by a thread of the next warp.  No order is needed between the two streams beyond
                // what the barriers already give: S(t+2) and the refill of stage t&1 both follow the
                // kv_free arrival of P(t).V(t), and P(t) follows S(t).
                bool ok = have_tmem;
                uint32_t gt = 0, qn = 0;
                uint32_t pend0 = 0u, pend1 = 0u;         // per stage: the epilogue (running number) whose output staging it holds
                Item cur = get_item(0);
                for (int k = 0; k < n_items && ok; ++k) {
                    const int ntiles = cur.ntiles;
                    if (ntiles > 0) {
                        // every Q.K^T of the previous item must have completed before its Q is replaced (its last
                        // tile's S commit is the last one this thread made) ...
                        if (gt > 0u) {
                            const uint32_t gl = gt - 1u;
                            if (!ptx::mbar_wait(bar_s_full + 8 * int(gl & 1u), (gl >> 1) & 1u, wait_ns)) {
                                report_status(a.status, kStatusWaitSFull, 1, int(gt));
                                ok = false;
                                break;
                            }
                        }
                        // ... and the stage of the item's first tile must be free: the chunks bound for tensor memory are
                        // staged there
                        const int st0 = int(gt & 1u);
                        if (gt >= 2u && !ptx::mbar_wait(bar_kv_free + 8 * st0, ((gt >> 1) - 1u) & 1u, wait_ns)) {
                            report_status(a.status, kStatusWaitKvFree, 1, int(gt));
                            ok = false;
                            break;
                        }
                        // (it may also still hold the output staging of the item before the previous one, when that one
                        // had a single tile)
                        {
                            const uint32_t need = st0 ? pend1 : pend0;
                            if (need != 0u) {
                                const unsigned long long t0 = ptx::globaltimer_ns();
                                bool free_now = false;
                                while (true) {
                                    free_now = misc->epi_done[0] >= need && misc->epi_done[1] >= need &&
                                               misc->epi_done[2] >= need && misc->epi_done[3] >= need;
                                    if (free_now || ptx::globaltimer_ns() - t0 > wait_ns) break;
                                }
                                if (!free_now) {
                                    report_status(a.status, kStatusWaitEpilogue, 1, int(gt));
                                    ok = false;
                                    break;
                                }
                                __threadfence_block();
                                if (st0) pend1 = 0u; else pend0 = 0u;
                            }
                        }
                        // Q tile [128 heads x NCHUNK*64] bf16 by TMA, one 64-column box per chunk, landing in the
                        // swizzled operand layout: chunks >= kQTmemChunks at their final place, the others in the
                        // staging area.  Rows past the end of Q read as zero; rows of a following request (H < 128)
                        // are computed but never written out.
                        trace_mark(a, 1, 600 + int(qn));
                        ptx::mbar_arrive_expect_tx(bar_q_full, uint32_t(NCHUNK) * kQChunkBytes);
                        const int qrow0 = cur.n * a.H + cur.hg * kHeadsPerCta;
#pragma unroll
                        for (int c = 0; c < NCHUNK; ++c) {
                            const uint32_t dst = (c < kQTmemChunks) ? kv_base + uint32_t(st0) * L::kKvStageBytes + uint32_t(c) * kQChunkBytes
                                                                    : q_base + uint32_t(c - kQTmemChunks) * kQChunkBytes;
                            ptx::tma_load_2d(dst, &a.q_map, c * 64, qrow0, bar_q_full);
                        }
                        if (!ptx::mbar_wait(bar_q_ready, qn & 1u, wait_ns)) {
                            report_status(a.status, kStatusWaitQ, 1, int(gt));
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after_sync();
                        for (int it = 0; it < ntiles && ok; ++it) {
                            const uint32_t g = gt + uint32_t(it);
                            const int st = int(g & 1u);
                            const uint32_t par = (g >> 1) & 1u;
                            for (int grp = 0; grp < kNumKvGroups; ++grp) {
                                if (!ptx::mbar_wait(bar_kv_full + kKvFullStride * st + 8 * grp, par, wait_ns)) {
                                    report_status(a.status, kStatusWaitKvFull, 1, int(g));
                                    ok = false;
                                    break;
                                }
                                ptx::tc_fence_after_sync();
                                trace_mark(a, 1, 4 * int(g) + grp);
                                if (grp == 0) issue_qk_range(st, std::integral_constant<int, 0>{}, std::integral_constant<int, 4>{});
                                else issue_qk_range(st, std::integral_constant<int, 4>{}, std::integral_constant<int, NCHUNK>{});
                            }
                            if (ok) {
                                trace_mark(a, 1, 4 * int(g) + 2);
                                ptx::mma_commit(bar_s_full + 8 * st);
                            }
                        }
                        gt += uint32_t(ntiles);
                        ++qn;
                        if ((gt - 1u) & 1u) pend1 = qn; else pend0 = qn;     // the item's output is staged in the stage of its last tile
                    }
                    if (k + 1 < n_items) cur = get_item(k + 1);
                }
            }
            __syncwarp();
        } else if (warp == kMmaWarp + 1) {
            // ───────────── O += P . V issue (one thread) ─────────────
            if (lane == 0) {
                bool ok = wait_tmem();
                if (!ok) report_status(a.status, kStatusWaitQ, 3, -1);
                const uint32_t tmem = misc->tmem_base;
                constexpr uint32_t idesc_pv = use_f16(SRC) ? ptx::make_idesc_f16(128, kDvHalf, false, true)
                                                            : ptx::make_idesc_bf16(128, kDvHalf, false, true);
                constexpr uint32_t kDescHi = ptx::smem_desc_hi(1024);
                uint32_t gt = 0;
                Item cur = get_item(0);
                for (int k = 0; k < n_items && ok; ++k) {
                    const int ntiles = cur.ntiles;
                    for (int it = 0; it < ntiles; ++it) {
                        const uint32_t g = gt + uint32_t(it);
                        const int st = int(g & 1u);
                        // (the first P of an item is written after the softmax warps have read the previous item's O out
                        // of tensor memory, so the overwrite below needs no barrier of its own)
                        if (!ptx::mbar_wait(bar_p_full + 8 * st, (g >> 1) & 1u, wait_ns)) {
                            report_status(a.status, kStatusWaitPFull, 3, int(g));
                            ok = false;
                            break;
                        }
                        const uint32_t kv_st = kv_base + uint32_t(st) * L::kKvStageBytes;
                        ptx::tc_fence_after_sync();
                        trace_mark(a, 3, 2 * int(g));
                        const uint32_t p_tmem = tmem + kTmemS + uint32_t(st) * kTileN;
                        // B = V[16 entries x 256 cols], MN-major: 64-col groups 8 KB apart (leading
                        // offset), 8-entry groups 1 KB apart; A = P in tensor memory, 8 columns per step
                        const uint32_t v_lo = ptx::smem_desc_lo(kv_st + v_off, kKvChunkBytes);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            ptx::mma_bf16_ts2(tmem + kTmemO, p_tmem + kk * 8, v_lo + uint32_t((kk * 2048) >> 4), kDescHi, idesc_pv,
                                              (it | kk) ? 1u : 0u);
                        ptx::mma_commit(bar_kv_free + 8 * st);   // stage reusable, and O includes tile it
                    }
                    if (ok && ntiles > 0) ptx::mma_commit(bar_o_full);
                    gt += uint32_t(ntiles);
                    if (k + 1 < n_items) cur = get_item(k + 1);
                }
            }
            __syncwarp();
        } else if (warp == kResolveWarp) {
            // ───────────── resolver: where does every entry of the next tiles live? ─────────────
            // Walks the block's items in order; for every tile it writes the 64 record numbers, the validity mask
            // and a tag into a ring in shared memory, up to kRing tiles ahead of the loaders.  A lane owns entries
            // lane and lane + 32 of a tile.  The dependent loads (index list -> block table) are issued one step
            // and looked at the next; the records and, at the start of an item, its Q rows are pulled into L2.
            int ck = 0, ct = 0;
            Item ci{};
            auto kc_seek = [&]() {        // the first item at or after ck that has tiles
                ct = 0;
                while (ck < n_items) {
                    ci = get_item(ck);
                    if (ci.ntiles > 0) break;
                    ++ck;
                }
            };
            auto kc_ctx = [&]() -> TileCtx {
                TileCtx c{};
                if (ck < n_items) {
                    c.n = ci.n;  c.b = ci.b;  c.n_tok = ci.n_tok;  c.kv_len_n = ci.kv_len_n;
                    c.v0 = (ci.tile0 + ct) * kTileN;
                    c.meta = kMetaTile | uint32_t(ci.n) | (uint32_t(ci.hg) << 16) | (ct == 0 ? kMetaFirst : 0u) |
                             (ct == ci.ntiles - 1 ? kMetaLast : 0u);
                }
                return c;
            };
            auto kc_advance = [&]() {
                if (ck >= n_items) return;
                if (++ct >= ci.ntiles) { ++ck;  kc_seek(); }
            };
            kc_seek();
            auto kc_next = [&]() -> TileCtx {
                const TileCtx c = kc_ctx();
                kc_advance();
                return c;
            };
            bool rok = true;
            uint32_t t = 0;            // the stream tile published next
            auto publish = [&](uint32_t meta, uint32_t id0, uint32_t id1) {
                const uint32_t slot = t % kRing;
                if (t >= uint32_t(kRing)) {
                    const bool w = ptx::mbar_wait(bar_res_empty + 8 * slot, ((t / kRing) - 1u) & 1u, wait_ns);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_status(a.status, kStatusWaitResolver, 4, int(t));
                        rok = false;
                        return;
                    }
                }
                TileSlot& ts = misc->ring[slot];
                ts.id[lane] = id0;
                ts.id[lane + 32] = id1;
                const uint32_t lo = __ballot_sync(0xFFFFFFFFu, (id0 & kIdValid) != 0u);
                const uint32_t hi = __ballot_sync(0xFFFFFFFFu, (id1 & kIdValid) != 0u);
                if (lane == 0) {
                    ts.mask = uint64_t(lo) | (uint64_t(hi) << 32);
                    ts.meta = meta;
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_res_full + 8 * slot);
                if (lane == 0) trace_mark(a, 3, 512 + int(t));
                ++t;
            };
            // three-stage pipeline over the stream: index values of the tile two ahead, block-table values of the
            // next tile, record numbers of this one
            TileCtx c0 = kc_next();
            TileCtx c1 = kc_next();
            int e1a = -1, e1b = -1;
            PendingId p0a, p0b;
            {
                int e0a = -1, e0b = -1;
                if constexpr (SRC == kSrcCsa) {
                    e0a = resolve_index(a, c0, lane);      e0b = resolve_index(a, c0, lane + 32);
                    e1a = resolve_index(a, c1, lane);      e1b = resolve_index(a, c1, lane + 32);
                }
                p0a = resolve_issue<SRC>(a, c0, e0a, lane);
                p0b = resolve_issue<SRC>(a, c0, e0b, lane + 32);
            }
            if ((c0.meta & (kMetaTile | kMetaFirst)) == (kMetaTile | kMetaFirst))
                prefetch_q_l2<NCHUNK>(a, c0.n, int((c0.meta >> 16) & 0xFFu), lane, 32);
            while (rok && (c0.meta & kMetaTile)) {
                // the next tile's block-table loads go out before this tile's are looked at
                const TileCtx c2 = kc_next();
                const PendingId p1a = resolve_issue<SRC>(a, c1, e1a, lane);
                const PendingId p1b = resolve_issue<SRC>(a, c1, e1b, lane + 32);
                if constexpr (SRC == kSrcCsa) {
                    e1a = resolve_index(a, c2, lane);      e1b = resolve_index(a, c2, lane + 32);
                }
                const uint32_t id0 = resolve_finish<SRC>(a, p0a), id1 = resolve_finish<SRC>(a, p0b);
                prefetch_record_l2<SRC>(a, id0);
                prefetch_record_l2<SRC>(a, id1);
                publish(c0.meta, id0, id1);
                if ((c1.meta & (kMetaTile | kMetaFirst)) == (kMetaTile | kMetaFirst))
                    prefetch_q_l2<NCHUNK>(a, c1.n, int((c1.meta >> 16) & 0xFFu), lane, 32);
                c0 = c1;  c1 = c2;
                p0a = p1a;  p0b = p1b;
            }
            // two end marks: the loaders look two tiles ahead
            if (rok) publish(0u, 0u, 0u);
            if (rok) publish(0u, 0u, 0u);
            __syncwarp();
        }
    } else {
        // ───────────── softmax + epilogue warps ─────────────
        bool ok = __all_sync(0xFFFFFFFFu, wait_tmem());
        if (!ok) report_status(a.status, kStatusWaitQ, 0, -1);
        const uint32_t tmem = misc->tmem_base;
        const int r = warp * 32 + lane;                // head row inside the group
        const uint32_t lane_addr = uint32_t(warp * 32) << 16;
        uint32_t gt = 0, qn = 0;
        Item cur = get_item(0);
        for (int k = 0; k < n_items && ok; ++k) {
            const int ntiles = cur.ntiles;
            const int n = cur.n, hg = cur.hg, slot = cur.slot, tile0 = cur.tile0;
            // destination of the item's head rows (this block's half of the value columns) and of their LSEs; worked
            // out where it is needed, so that nothing of it is held in registers through the tile loop
            auto destination = [&](int64_t& prow0) -> __nv_bfloat16* {
                Item it{};
                it.n = n;  it.hg = hg;  it.slot = slot;
                prow0 = slot < 0 ? 0 : partial_row0(it);
                return slot < 0 ? a.out + (int64_t(n) * a.H + hg * kHeadsPerCta) * 512 + half * kDvHalf
                                : reinterpret_cast<__nv_bfloat16*>(a.partial_o) + prow0 * 512 + half * kDvHalf;
            };
            if (ntiles <= 0) {
                // Nothing to attend to: zero output, LSE = -inf.
                const bool final_out = slot < 0;
                const int h = hg * kHeadsPerCta + r;
                const bool write = h < a.H;
                int64_t prow0;
                __nv_bfloat16* const out_rows = destination(prow0);
                for (int i = tid; i < kHeadsPerCta * (kDvHalf / 8); i += kNumSoftmaxWarps * 32) {
                    const int rr = i / (kDvHalf / 8), v = i % (kDvHalf / 8);
                    if (hg * kHeadsPerCta + rr < a.H)
                        *reinterpret_cast<uint4*>(out_rows + int64_t(rr) * 512 + v * 8) = make_uint4(0, 0, 0, 0);
                }
                if (half == 0 && write) {
                    if (final_out) {
                        if (a.lse != nullptr) a.lse[int64_t(n) * a.H + h] = -CUDART_INF_F;
                    } else {
                        a.partial_lse[prow0 + r] = -CUDART_INF_F;
                    }
                }
                if (k + 1 < n_items) cur = get_item(k + 1);
                continue;
            }
            float m_ref = -CUDART_INF_F;                   // reference maximum used in exp2 (log2 units)
            float l_sum = 0.f;
            for (int it = 0; it < ntiles && ok; ++it) {
                const uint32_t g = gt + uint32_t(it);
                const int st = int(g & 1u);
                const uint32_t s_tmem = tmem + lane_addr + kTmemS + uint32_t(st) * kTileN;
                {
                    const bool w = ptx::mbar_wait(bar_s_full + 8 * st, (g >> 1) & 1u, wait_ns);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_status(a.status, kStatusWaitSFull, 0, tile0 + it);
                        ok = false;  break;
                    }
                }
                ptx::tc_fence_after_sync();
                if (tid == 0) trace_mark(a, 0, 4 * int(g));
                uint32_t s0[32], s1[32];
                ptx::tmem_ld32(s_tmem, s0);
                ptx::tmem_ld32(s_tmem + 32, s1);
                ptx::tmem_wait_ld();
                const uint64_t vmask = *reinterpret_cast<volatile uint64_t*>(&misc->valid_mask[st]);
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
                    for (int kk = 0; kk < 4; ++kk)
                        t4[kk] = fmaxf(t4[kk], fmaxf(__uint_as_float(s0[i + kk]), __uint_as_float(s1[i + kk])));
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
                    const uint32_t gp = g - 1u;
                    const bool w = ptx::mbar_wait(bar_kv_free + 8 * int(gp & 1u), (gp >> 1) & 1u, wait_ns);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_status(a.status, kStatusWaitKvFree, 0, tile0 + it);
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
                // P (two entries per column) over the first 32 columns of this S buffer:
                // the A operand of the PV MMAs.  S has been read into registers above.
                ptx::tmem_st32(s_tmem, pk);
                ptx::tmem_wait_st();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_p_full + 8 * st);
                if (tid == 0) trace_mark(a, 0, 4 * int(g) + 1);
            }
            // ── epilogue ──
            const int tile_end = tile0 + ntiles;
            if (k + 1 < n_items) cur = get_item(k + 1);      // the next item's record arrives while this one is written out
            const bool final_out = slot < 0;
            const int h = hg * kHeadsPerCta + r;
            const bool write = h < a.H;
            int64_t prow0;
            __nv_bfloat16* const out_rows = destination(prow0);
            if (ok) {
                const bool w = ptx::mbar_wait(bar_o_full, qn & 1u, wait_ns);
                if (!__all_sync(0xFFFFFFFFu, w)) {
                    report_status(a.status, kStatusWaitOFull, 0, tile_end);
                    ok = false;
                }
            }
            if (ok) {
                ptx::tc_fence_after_sync();
                if (tid == 0) trace_mark(a, 0, 4 * int(gt + uint32_t(ntiles) - 1u) + 2);
                // A merge kernel launched as a programmatic dependent may be made resident once every block of
                // this grid is here (or gone): by then no block of this grid is waiting for an SM any more.
                if (tid == 0 && k == n_items - 1 && (sched || a.num_splits > 1)) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
                float denom = l_sum;
                if (final_out && a.attn_sink != nullptr && write) {
                    const float s2 = __ldg(a.attn_sink + h) * 1.4426950408889634f;
                    denom = (l_sum > 0.f) ? l_sum + ptx::ex2(s2 - m_ref) : 1.f;   // empty row: O is 0 anyway
                }
                const float inv = (l_sum > 0.f) ? 1.f / denom : 0.f;
                const float lse2 = (l_sum > 0.f) ? m_ref + log2f(l_sum) : -CUDART_INF_F;
                // O leaves through shared memory: each thread owns a row in tensor memory, but rows are 1 KB apart
                // in global memory, so 128 columns at a time are laid down in shared memory (pitch = 256 + 16
                // bytes: conflict-free both ways) and written out 2 x 256 contiguous bytes per warp instruction.
                // The staging area is the KV stage of the item's last tile, which nothing else uses until the
                // loaders have seen this warp's epi_done count (the other stage may already hold the next item's
                // first tile).  Split partials are BF16 as well: the merge reads them back at once, and at eight
                // splits their traffic would otherwise exceed the KV bytes.
                const uint32_t s_last = (gt + uint32_t(ntiles) - 1u) & 1u;
                const uint32_t stg = kv_base + s_last * L::kKvStageBytes + uint32_t(warp) * L::kEpiWarpBytes;
                const uint32_t my = stg + uint32_t(lane) * L::kEpiPitch;
                const int hw0 = hg * kHeadsPerCta + warp * 32;                   // first head row of this warp
                uint8_t* gbase = reinterpret_cast<uint8_t*>(out_rows + int64_t(warp) * 32 * 512);
#pragma unroll 1
                for (int pass = 0; pass < L::kEpiPasses; ++pass) {
#pragma unroll 1
                    for (int c = 0; c < L::kEpiCols / 32; ++c) {
                        uint32_t o[32];
                        ptx::tmem_ld32(tmem + lane_addr + kTmemO + pass * L::kEpiCols + c * 32, o);
                        ptx::tmem_wait_ld();
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint4 w;
                            w.x = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                            w.y = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                            w.z = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                            w.w = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                            ptx::sts_v4(my + uint32_t(c) * 64u + uint32_t(v) * 16u, w);
                        }
                    }
                    __syncwarp();
                    constexpr uint32_t kVecs = uint32_t(L::kEpiCols) / 8u;      // 16-byte pieces per staged row
#pragma unroll 4
                    for (uint32_t q = uint32_t(lane); q < 32u * kVecs; q += 32u) {
                        const uint32_t rl = q / kVecs, vc = q % kVecs;
                        if (hw0 + int(rl) < a.H) {
                            const uint4 w = ptx::lds_v4(stg + rl * L::kEpiPitch + vc * 16u);
                            *reinterpret_cast<uint4*>(gbase + int64_t(rl) * 1024 + pass * (L::kEpiCols * 2) + vc * 16u) = w;
                        }
                    }
                    __syncwarp();
                }
                if (lane == 0) {
                    __threadfence_block();
                    misc->epi_done[warp] = qn + 1u;
                }
                if (tid == 0) trace_mark(a, 0, 4 * int(gt + uint32_t(ntiles) - 1u) + 3);
                if (write && half == 0) {
                    if (final_out) {
                        if (a.lse != nullptr) a.lse[int64_t(n) * a.H + h] = (l_sum > 0.f) ? lse2 * 0.6931471805599453f : -CUDART_INF_F;
                    } else {
                        a.partial_lse[prow0 + r] = lse2;
                    }
                }
            }
            gt += uint32_t(ntiles);
            ++qn;
        }
    }

    // ── common exit: every thread gets here, with or without an error ──
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(misc->tmem_base, kTmemCols);
    }
}

}  // namespace dsv4

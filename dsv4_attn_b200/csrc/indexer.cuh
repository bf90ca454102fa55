// CSA indexer for decode: which compressed entries does each query token attend to?
//
//   score[t, s] = sum_h  w[t, h] * relu( q[t, h, :] . k[s, :] ) * kscale[s]
//   top-k over the s < n_vis[t] visible entries.
//
// Two kernels.
//  * indexer_logits_kernel: FP8 x FP8 -> FP32 on the tensor cores
//    (tcgen05.mma kind::f8f6f4).  The keys are the M side - 128 keys of two cache
//    pages per MMA, brought into shared memory by TMA straight from the paged
//    pool - and the 64 heads of each query token the N side, so that the head
//    reduction (ReLU, weight, sum) runs inside one thread of the epilogue: tensor
//    memory lane = key, columns = (token, head).  Warp roles: one TMA producer
//    lane, one MMA-issuing lane, four epilogue warps; a ring of key stages and two
//    accumulator buffers in tensor memory decouple the three.
//  * topk_select_kernel: per (request, token) row a radix select over the FP32
//    scores (four 8-bit rounds, histograms in shared memory), then a compaction
//    pass that writes the indices of the k best (unordered; -1 padded).
//
// Key page: 64 keys x 128 e4m3 bytes, then the 64 FP32 scales of those keys
// (8448 bytes = 66 rows of 128 bytes).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "ptx.cuh"
#include "decode_kernel.cuh"   // report_timeout, status codes, kDefaultWaitNs

namespace dsv4 {

constexpr int kIdxHeads = 64;
constexpr int kIdxDim = 128;
constexpr int kIdxPageKeys = 64;
constexpr int kIdxPageRows = 66;                        // 128-byte rows per page: 64 of keys, 2 of scales
constexpr int kIdxPageBytes = kIdxPageRows * 128;       // 8448
constexpr int kIdxTileKeys = 128;                       // keys per MMA tile (two pages)
constexpr int kIdxStages = 4;
constexpr int kIdxThreads = 192;                        // producer warp, MMA warp, four epilogue warps
constexpr int kIdxTmemCols = 256;                       // two accumulator buffers of up to 128 columns
constexpr int kStatusWaitIndexer = 32;

struct IndexerArgs {
    alignas(64) CUtensorMap key_map;     // pool as [num_pages*66, 128] bytes, box 64 rows, 128-byte swizzle
    alignas(64) CUtensorMap scale_map;   // same memory, box 2 rows, no swizzle
    alignas(64) CUtensorMap q_map;       // q as [B*s_q*64, 128] bytes, box s_q*64 rows, 128-byte swizzle
    int B, s_q, max_pages, tiles_per_cta;
    int64_t num_pages;
    const float* q_weight;               // [B, s_q, 64]
    const int32_t* block_table;          // [B, max_pages]
    const int32_t* n_vis;                // [B, s_q]
    float* scores;                       // [B*s_q, score_stride]
    int64_t score_stride;
    int32_t* status;
    unsigned long long wait_ns;          // limit of every barrier wait
    int dbg_drop_tile;                   // >= 0: the "accumulator full" signal of that tile of every block is left out (tests the limit)
};

struct IdxSmem {
    uint64_t full[kIdxStages];
    uint64_t empty[kIdxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t q_full;
    uint32_t tmem_base;
    uint32_t page_ok[kIdxStages];        // bit j: page j of the stage was loaded
    float weight[2 * kIdxHeads];
};

constexpr int kIdxQBytes = 2 * kIdxHeads * kIdxDim;                 // up to two query tokens
constexpr int kIdxStageKeyBytes = kIdxTileKeys * kIdxDim;           // 16 KB
constexpr int kIdxScaleBytes = 2 * 256;                             // two pages x 64 floats
constexpr int kIdxSmemBytes = 1024 + kIdxQBytes + kIdxStages * kIdxStageKeyBytes + kIdxStages * kIdxScaleBytes + 1024;

// Instruction descriptor for kind::f8f6f4 with e4m3 operands (format code 0), K-major, FP32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc_e4m3(int M, int N) {
    return (1u << 4) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(kIdxThreads, 2) indexer_logits_kernel(const __grid_constant__ IndexerArgs a) {
    extern __shared__ uint8_t idx_smem_raw[];
    const uint32_t base = (ptx::smem_u32(idx_smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = idx_smem_raw + (base - ptx::smem_u32(idx_smem_raw));
    const uint32_t q_smem = base;
    const uint32_t key_smem = base + kIdxQBytes;
    const uint32_t scale_smem = key_smem + kIdxStages * kIdxStageKeyBytes;
    const float* scale_gen = reinterpret_cast<const float*>(gen + kIdxQBytes + kIdxStages * kIdxStageKeyBytes);
    IdxSmem* sm = reinterpret_cast<IdxSmem*>(gen + kIdxQBytes + kIdxStages * kIdxStageKeyBytes + kIdxStages * kIdxScaleBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.y;
    const int N = a.s_q * kIdxHeads;

    int vis_max = 0;
    for (int t = 0; t < a.s_q; ++t) vis_max = max(vis_max, __ldg(a.n_vis + b * a.s_q + t));
    vis_max = min(vis_max, a.max_pages * kIdxPageKeys);
    const int tiles_total = (vis_max + kIdxTileKeys - 1) / kIdxTileKeys;
    const int tile0 = min(int(blockIdx.x) * a.tiles_per_cta, tiles_total);
    const int tile1 = min(tile0 + a.tiles_per_cta, tiles_total);
    const int ntiles = tile1 - tile0;
    if (ntiles <= 0) return;                                  // whole block, before any barrier or allocation

    const uint32_t bar_full = ptx::smem_u32(&sm->full[0]), bar_empty = ptx::smem_u32(&sm->empty[0]);
    const uint32_t bar_acc_full = ptx::smem_u32(&sm->acc_full[0]), bar_acc_empty = ptx::smem_u32(&sm->acc_empty[0]);
    const uint32_t bar_q = ptx::smem_u32(&sm->q_full);

    if (tid == 0) {
        for (int s = 0; s < kIdxStages; ++s) { ptx::mbar_init(bar_full + 8 * s, 1);  ptx::mbar_init(bar_empty + 8 * s, 1 + 4); }
        for (int d = 0; d < 2; ++d) { ptx::mbar_init(bar_acc_full + 8 * d, 1);  ptx::mbar_init(bar_acc_empty + 8 * d, 4); }
        ptx::mbar_init(bar_q, 1);
        ptx::fence_mbar_init();
    }
    if (tid < N) sm->weight[tid] = __ldg(a.q_weight + int64_t(b) * N + tid);
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(&sm->tmem_base), kIdxTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = sm->tmem_base;
    bool ok = true;

    if (warp == 0) {
        // ───────────── producer: Q once, then key pages and their scales, stage by stage ─────────────
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(bar_q, uint32_t(N) * kIdxDim);
            ptx::tma_load_2d(q_smem, &a.q_map, 0, b * N, bar_q);
            const int pages_vis = (vis_max + kIdxPageKeys - 1) / kIdxPageKeys;
            for (int i = 0; i < ntiles && ok; ++i) {
                const int st = i % kIdxStages;
                if (i >= kIdxStages && !ptx::mbar_wait(bar_empty + 8 * st, uint32_t(i / kIdxStages - 1) & 1u, a.wait_ns)) {
                    report_status(a.status, kStatusWaitIndexer, 0, tile0 + i);
                    ok = false;
                    break;
                }
                int page[2];
                uint32_t okmask = 0, bytes = 0;
                for (int j = 0; j < 2; ++j) {
                    const int lp = 2 * (tile0 + i) + j;            // logical page of the request
                    page[j] = (lp < pages_vis) ? __ldg(a.block_table + int64_t(b) * a.max_pages + lp) : -1;
                    if (page[j] >= 0 && page[j] < a.num_pages) { okmask |= 1u << j;  bytes += kIdxPageKeys * kIdxDim + 256; }
                }
                sm->page_ok[st] = okmask;
                ptx::mbar_arrive_expect_tx(bar_full + 8 * st, bytes);
                for (int j = 0; j < 2; ++j) {
                    if (!((okmask >> j) & 1u)) continue;
                    ptx::tma_load_2d(key_smem + st * kIdxStageKeyBytes + j * (kIdxPageKeys * kIdxDim), &a.key_map, 0,
                                     page[j] * kIdxPageRows, bar_full + 8 * st);
                    ptx::tma_load_2d(scale_smem + st * kIdxScaleBytes + j * 256, &a.scale_map, 0,
                                     page[j] * kIdxPageRows + kIdxPageKeys, bar_full + 8 * st);
                }
            }
        }
    } else if (warp == 1) {
        // ───────────── MMA issue: S^T[128 keys x N] = K[128 x 128] . Q[N x 128]^T, four K steps of 32 ─────────────
        if (lane == 0) {
            const uint32_t idesc = make_idesc_e4m3(kIdxTileKeys, N);
            if (!ptx::mbar_wait(bar_q, 0u, a.wait_ns)) { report_status(a.status, kStatusWaitIndexer, 1, -1);  ok = false; }
            for (int i = 0; i < ntiles && ok; ++i) {
                const int st = i % kIdxStages, d = i & 1;
                if (!ptx::mbar_wait(bar_full + 8 * st, uint32_t(i / kIdxStages) & 1u, a.wait_ns) ||
                    (i >= 2 && !ptx::mbar_wait(bar_acc_empty + 8 * d, uint32_t(i / 2 - 1) & 1u, a.wait_ns))) {
                    report_status(a.status, kStatusWaitIndexer, 1, tile0 + i);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int k = 0; k < kIdxDim / 32; ++k) {
                    const uint64_t ad = ptx::make_smem_desc(key_smem + st * kIdxStageKeyBytes + k * 32, 16, 1024);
                    const uint64_t bd = ptx::make_smem_desc(q_smem + k * 32, 16, 1024);
                    mma_f8_ss(tmem + d * 128, ad, bd, idesc, k ? 1u : 0u);
                }
                ptx::mma_commit(bar_empty + 8 * st);
                if (a.dbg_drop_tile < 0 || i != a.dbg_drop_tile) ptx::mma_commit(bar_acc_full + 8 * d);
            }
        }
    } else {
        // ───────────── epilogue: lane = key; ReLU, head weights, sum over heads, key scale ─────────────
        const int quarter = warp & 3;                                  // tensor-memory lanes 32*quarter .. +31
        const int r = quarter * 32 + lane;                             // key row inside the tile
        const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
        int vis[2];
        vis[0] = min(__ldg(a.n_vis + b * a.s_q), a.max_pages * kIdxPageKeys);
        vis[1] = (a.s_q > 1) ? min(__ldg(a.n_vis + b * a.s_q + 1), a.max_pages * kIdxPageKeys) : 0;
        for (int i = 0; i < ntiles && ok; ++i) {
            const int st = i % kIdxStages, d = i & 1;
            const bool w = ptx::mbar_wait(bar_acc_full + 8 * d, uint32_t(i / 2) & 1u, a.wait_ns) &&
                           ptx::mbar_wait(bar_full + 8 * st, uint32_t(i / kIdxStages) & 1u, a.wait_ns);
            if (!__all_sync(0xFFFFFFFFu, w)) {
                report_status(a.status, kStatusWaitIndexer, 2, tile0 + i);
                ok = false;
                break;
            }
            ptx::tc_fence_after_sync();
            const float kscale = scale_gen[st * (kIdxScaleBytes / 4) + r];
            const bool page_loaded = (sm->page_ok[st] >> (r >> 6)) & 1u;
            const int key = (tile0 + i) * kIdxTileKeys + r;
            for (int t = 0; t < a.s_q; ++t) {
                float acc = 0.f;
#pragma unroll
                for (int c = 0; c < kIdxHeads / 32; ++c) {
                    uint32_t v[32];
                    ptx::tmem_ld32(tmem + lane_addr + d * 128 + t * kIdxHeads + c * 32, v);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        acc = fmaf(fmaxf(__uint_as_float(v[j]), 0.f), sm->weight[t * kIdxHeads + c * 32 + j], acc);
                }
                if (key < vis[t])
                    a.scores[(int64_t(b) * a.s_q + t) * a.score_stride + key] = page_loaded ? acc * kscale : -CUDART_INF_F;
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(bar_acc_empty + 8 * d);
                ptx::mbar_arrive(bar_empty + 8 * st);
            }
        }
    }
    // common exit: every role arrives; the MMA warp frees tensor memory after all accumulator reads
    ptx::tc_fence_before_sync();
    __syncthreads();
    // the top-k kernel may be made resident as soon as every block of this grid is here or gone
    if (tid == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, kIdxTmemCols);
    }
}

// ───────────────────────── top-k ─────────────────────────

constexpr int kTopkThreads = 1024;
constexpr int kTopkBins = 1024;          // one bin per thread in the suffix scan
constexpr int kTopkCand = 4096;          // candidates of the threshold bin kept in shared memory

// order-preserving map float -> uint32 (larger float = larger key)
__device__ __forceinline__ uint32_t float_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct TopkArgs {
    int rows, k;
    const float* scores;        // [rows, stride]
    int64_t stride;
    const int32_t* n_vis;       // [rows]
    int32_t* out;               // [rows, k]
    int n_cap;                  // entries the score rows can hold
    int row_in_smem;            // the launch provides n_cap floats of dynamic shared memory for a copy of the row
};

struct TopkShared {
    uint32_t hist[kTopkBins];
    uint32_t cand_key[kTopkCand];
    int32_t cand_idx[kTopkCand];
    float red_lo[32], red_hi[32];
    uint32_t warp_sum[32];
    uint32_t radix[256];
    uint32_t t_bin, n_gt, need, n_cand, prefix, rneed, cnt_gt, cnt_eq;
};

// Exact selection of the `need` largest keys among the elements `src` enumerates
// (four 8-bit radix rounds, then a compaction), written to out[0 .. need).  Used on
// the few hundred candidates of the threshold bin, where contention is harmless.
// src(j, key, idx) returns false for positions that hold no element.
template <typename Src>
__device__ __forceinline__ void radix_select_emit(TopkShared& sh, int count, uint32_t need, int32_t* out, Src src) {
    const int tid = threadIdx.x;
    if (tid == 0) { sh.prefix = 0;  sh.rneed = need; }
    for (int round = 0; round < 4; ++round) {
        const int shift = 24 - 8 * round;
        if (tid < 256) sh.radix[tid] = 0;
        __syncthreads();
        const uint32_t prefix = sh.prefix;
        const uint32_t mask = (round == 0) ? 0u : (0xFFFFFFFFu << (shift + 8));
        for (int j = tid; j < count; j += kTopkThreads) {
            uint32_t key;  int32_t idx;
            if (src(j, key, idx) && (key & mask) == prefix) atomicAdd(&sh.radix[(key >> shift) & 0xFFu], 1u);
        }
        __syncthreads();
        if (tid < 32) {
            // the digit that holds the nd-th largest remaining key: lane l owns digits 8l .. 8l+7,
            // a suffix scan over the lanes finds the lane, a short loop the digit
            const uint32_t nd = sh.rneed;
            uint32_t c[8], sum = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { c[j] = sh.radix[8 * tid + j];  sum += c[j]; }
            uint32_t incl = sum;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t o = __shfl_down_sync(0xFFFFFFFFu, incl, d);
                if (tid + d < 32) incl += o;
            }
            const uint32_t higher = incl - sum;
            if (higher < nd && incl >= nd) {
                uint32_t rem = nd - higher, bin = 8u * tid;
#pragma unroll
                for (int j = 7; j >= 0; --j) {
                    if (c[j] >= rem) { bin = 8u * tid + uint32_t(j);  break; }
                    rem -= c[j];
                }
                sh.prefix = prefix | (bin << shift);
                sh.rneed = rem;
            }
        }
        __syncthreads();
    }
    const uint32_t kth = sh.prefix, need_eq = sh.rneed, above = need - need_eq;
    if (tid == 0) { sh.cnt_gt = 0;  sh.cnt_eq = 0; }
    __syncthreads();
    for (int j = tid; j < count; j += kTopkThreads) {
        uint32_t key;  int32_t idx;
        if (!src(j, key, idx)) continue;
        if (key > kth) {
            const uint32_t p = atomicAdd(&sh.cnt_gt, 1u);
            if (p < above) out[p] = idx;
        } else if (key == kth) {
            const uint32_t p = atomicAdd(&sh.cnt_eq, 1u);
            if (p < need_eq) out[above + p] = idx;
        }
    }
}

// One block - or, when there are few rows, a cluster pair of blocks that share a row - per
// (request, token).  The scores of a row share a handful of floating-point exponents, so a radix
// histogram over the raw bits would have every lane of a warp hit the same counter.  Instead:
// (A) minimum and maximum of the row; (B) a histogram over 1024 equal-width value bins - spread
// out, so the shared-memory atomics rarely collide; a block-wide suffix scan finds the bin that
// holds the k-th largest score; (C) everything in higher bins is part of the selection and is
// written out at once, the entries of the threshold bin (a few hundred) are collected in shared
// memory and the remaining places are filled from them by an exact radix select.  Binning is
// monotone in the score, so the result is the exact top-k (as a set).
//
// With a pair (C = 2) each block takes half of the row; range, histograms, output offsets and
// the candidate list are combined through distributed shared memory, with cluster barriers that
// both blocks reach unconditionally; block 0 of the pair does the final select.
template <int C>
__device__ __forceinline__ void topk_select_body(const TopkArgs& a, float* topk_row) {
    __shared__ TopkShared sh;
    __shared__ uint32_t sh_x[4];          // exchanged with the peer: own count above the threshold bin, own count in it
    const uint32_t rank = (C == 2) ? (blockIdx.x & 1u) : 0u;
    const uint32_t peer = rank ^ 1u;
    const int row = blockIdx.x / C;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = max(0, min(__ldg(a.n_vis + row), a.n_cap));
    const float* g = a.scores + int64_t(row) * a.stride;
    int32_t* out = a.out + int64_t(row) * a.k;
    if (n <= a.k) {                                          // same decision in both blocks of a pair
        if (rank == 0)
            for (int i = tid; i < a.k; i += kTopkThreads) out[i] = (i < n) ? i : -1;
        return;
    }
    // this block's slice of the row
    const int half = (C == 2) ? (n + 1) / 2 : n;
    const int s0 = int(rank) * half, s1 = min(n, s0 + half);
    // the passes read the slice from shared memory when it fits (copied during pass A)
    const float* s = a.row_in_smem ? topk_row - s0 : g;      // indexed by the global position i
    // (A) range of the finite scores
    float lo = CUDART_INF_F, hi = -CUDART_INF_F;
    for (int i0 = s0 + tid; i0 < s1; i0 += 8 * kTopkThreads) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {                        // eight loads in flight per thread
            const int i = i0 + u * kTopkThreads;
            v[u] = (i < s1) ? __ldg(g + i) : CUDART_NAN_F;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * kTopkThreads;
            if (a.row_in_smem && i < s1) topk_row[i - s0] = v[u];
            if (v[u] > -CUDART_INF_F && v[u] < CUDART_INF_F) { lo = fminf(lo, v[u]);  hi = fmaxf(hi, v[u]); }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, d));
        hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, d));
    }
    if (lane == 0) { sh.red_lo[warp] = lo;  sh.red_hi[warp] = hi; }
    sh.hist[tid] = 0;
    if (tid == 0) { sh.n_cand = 0;  sh.cnt_gt = 0; }
    __syncthreads();
    if (C == 2) ptx::cluster_sync();                        // the peer's partial ranges are written
    lo = sh.red_lo[lane];  hi = sh.red_hi[lane];
    if (C == 2) {
        lo = fminf(lo, __uint_as_float(ptx::lds_cluster_u32(ptx::mapa(ptx::smem_u32(&sh.red_lo[lane]), peer))));
        hi = fmaxf(hi, __uint_as_float(ptx::lds_cluster_u32(ptx::mapa(ptx::smem_u32(&sh.red_hi[lane]), peer))));
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, d));
        hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, d));
    }
    const float inv = (hi > lo) ? float(kTopkBins) / (hi - lo) : 0.f;
    // -inf and NaN go to bin 0, +inf to the last bin; monotone in v otherwise
    auto bin_of = [&](float v) -> int {
        if (!(v > -CUDART_INF_F)) return 0;
        const float x = (v - lo) * inv;
        return x >= float(kTopkBins - 1) ? kTopkBins - 1 : (x > 0.f ? int(x) : 0);
    };
    // (B) histogram of the slice, then for every bin the number of entries of the row in higher bins
    for (int i = s0 + tid; i < s1; i += kTopkThreads) atomicAdd(&sh.hist[bin_of(s[i])], 1u);
    __syncthreads();
    if (C == 2) ptx::cluster_sync();                        // both histograms complete
    const uint32_t own = sh.hist[tid];
    const uint32_t theirs = (C == 2) ? ptx::lds_cluster_u32(ptx::mapa(ptx::smem_u32(&sh.hist[tid]), peer)) : 0u;
    {
        // two suffix scans in one: low 32 bits the row's counts, high 32 bits this block's own
        unsigned long long incl = (unsigned long long)(own + theirs) | ((unsigned long long)own << 32);
        const unsigned long long mine = incl;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned long long o = __shfl_down_sync(0xFFFFFFFFu, incl, d);
            if (lane + d < 32) incl += o;
        }
        unsigned long long* wsum = reinterpret_cast<unsigned long long*>(sh.cand_key);   // free until pass C
        if (lane == 0) wsum[warp] = incl;
        __syncthreads();
        unsigned long long higher = 0;                      // entries in the warps above this one
        for (int w = warp + 1; w < 32; ++w) higher += wsum[w];
        incl += higher;
        const unsigned long long excl = incl - mine;
        const uint32_t incl_row = uint32_t(incl), excl_row = uint32_t(excl);
        if (excl_row < uint32_t(a.k) && incl_row >= uint32_t(a.k)) {
            sh.t_bin = uint32_t(tid);  sh.n_gt = excl_row;  sh.need = uint32_t(a.k) - excl_row;
            sh_x[0] = uint32_t(excl >> 32);                 // this block's entries above the threshold bin
            sh_x[1] = own;                                  // and inside it
        }
    }
    __syncthreads();
    if (C == 2) ptx::cluster_sync();                        // the peer's counts are written
    const int t_bin = int(sh.t_bin);
    const uint32_t n_gt = sh.n_gt, need = sh.need;
    // block 1 writes after block 0: offsets from block 0's counts
    const uint32_t base_out = (rank == 0) ? 0u : ptx::lds_cluster_u32(ptx::mapa(ptx::smem_u32(&sh_x[0]), 0));
    const uint32_t base_cand = (rank == 0) ? 0u : ptx::lds_cluster_u32(ptx::mapa(ptx::smem_u32(&sh_x[1]), 0));
    const uint32_t peer_cand = (C == 2) ? ptx::lds_cluster_u32(ptx::mapa(ptx::smem_u32(&sh_x[1]), peer)) : 0u;
    const uint32_t cand_key0 = (C == 2) ? ptx::mapa(ptx::smem_u32(&sh.cand_key[0]), 0) : 0u;
    const uint32_t cand_idx0 = (C == 2) ? ptx::mapa(ptx::smem_u32(&sh.cand_idx[0]), 0) : 0u;
    __syncthreads();                                        // the scan scratch (cand_key) is free again
    // (C) higher bins straight to the output, the threshold bin to block 0's candidate list
    for (int i0 = s0; i0 < s1; i0 += kTopkThreads) {
        const int i = i0 + tid;
        float v = 0.f;
        int bn = -1;
        if (i < s1) { v = s[i];  bn = bin_of(v); }
        const bool gt = bn > t_bin, eq = bn == t_bin;
        const uint32_t m_gt = __ballot_sync(0xFFFFFFFFu, gt), m_eq = __ballot_sync(0xFFFFFFFFu, eq);
        const uint32_t below = (1u << lane) - 1u;
        uint32_t base_gt = 0, base_eq = 0;
        if (lane == 0) {
            if (m_gt) base_gt = atomicAdd(&sh.cnt_gt, uint32_t(__popc(m_gt)));
            if (m_eq) base_eq = atomicAdd(&sh.n_cand, uint32_t(__popc(m_eq)));
        }
        base_gt = __shfl_sync(0xFFFFFFFFu, base_gt, 0);
        base_eq = __shfl_sync(0xFFFFFFFFu, base_eq, 0);
        if (gt) {
            out[base_out + base_gt + uint32_t(__popc(m_gt & below))] = i;   // exactly n_gt such entries in the row
        } else if (eq) {
            const uint32_t p = base_cand + base_eq + uint32_t(__popc(m_eq & below));
            if (p < uint32_t(kTopkCand)) {
                if (C == 2) {
                    ptx::sts_cluster_u32(cand_key0 + 4u * p, float_key(v));
                    ptx::sts_cluster_u32(cand_idx0 + 4u * p, uint32_t(i));
                } else {
                    sh.cand_key[p] = float_key(v);  sh.cand_idx[p] = i;
                }
            }
        }
    }
    __syncthreads();
    if (C == 2) ptx::cluster_sync();                        // the candidate list in block 0 is complete
    if (rank != 0) return;                                  // block 0 touches no memory of block 1 from here on
    const uint32_t n_cand = sh.n_cand + peer_cand;
    if (n_cand <= uint32_t(kTopkCand)) {
        radix_select_emit(sh, int(n_cand), need, out + n_gt, [&](int j, uint32_t& key, int32_t& idx) {
            key = sh.cand_key[j];  idx = sh.cand_idx[j];
            return true;
        });
    } else {
        // a threshold bin too crowded for the list (many equal scores): select among its entries in
        // place, over the whole row in global memory
        radix_select_emit(sh, n, need, out + n_gt, [&](int j, uint32_t& key, int32_t& idx) {
            const float v = g[j];
            key = float_key(v);  idx = j;
            return bin_of(v) == t_bin;
        });
    }
}

__global__ void __launch_bounds__(kTopkThreads) topk_select_kernel(const TopkArgs a) {
    extern __shared__ float topk_row[];
    asm volatile("griddepcontrol.wait;" ::: "memory");     // launched as a programmatic dependent of the scoring kernel
    topk_select_body<1>(a, topk_row);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTopkThreads) topk_select_pair_kernel(const TopkArgs a) {
    extern __shared__ float topk_row[];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    topk_select_body<2>(a, topk_row);
}

}  // namespace dsv4

// Decode attention over an FP8 latent KV cache, two thread blocks per row
// working as a cluster pair that splits the 576 (or 512) query/key columns.
//
// Block `half` of the pair owns four 64-column latent chunks (half 0: columns
// 0..255 and, in the packed layout, the RoPE tail; half 1: columns 256..511
// and, in the reference layout, the RoPE tail).  Those columns are at the same
// time its share of the QK reduction and its 256 value columns, so each block
// loads, dequantises and keeps only its own half of every cache entry:
//
//   S_half[128 heads x 64] = Q[:, own columns] . K[:, own columns]^T   (tcgen05.mma, BF16)
//   the two halves of S are exchanged through distributed shared memory and added,
//   both blocks run the same softmax on the full S,
//   O_half[128 x 256] += P . V[:, own columns]                         (tcgen05.mma, BF16)
//
// Compared with giving each block the full QK product, the pair does the QK
// MMAs and the FP8 -> BF16 conversion once instead of twice, and each block
// needs half the shared memory for Q and for a KV tile.
//
// Warp roles: warps 0-3 softmax + exchange + epilogue (one head row per thread =
// one tensor-memory lane), warps 4-11 loaders, warp 12 MMA issue and
// tensor-memory owner, warps 13-15 only take part in the block barriers.
// All waits on mbarriers are bounded; the cluster barriers at entry and exit are
// reached unconditionally by every thread of both blocks.
#pragma once

#include "decode_kernel.cuh"

namespace dsv4 {
namespace pair {

constexpr int kMaxOwn = 5;                       // chunks a block can own (4 latent + RoPE)
constexpr int kStageBytes = kMaxOwn * kKvChunkBytes;            // 40 KB
constexpr int kQBytes = kMaxOwn * kQChunkBytes;                 // 80 KB
constexpr int kXBytes = kHeadsPerCta * kTileN * 4;              // 32 KB: the partner's half of S, FP32
constexpr int kQOff = 0;
constexpr int kKvOff = kQBytes;                                 // two stages
constexpr int kXOff = kKvOff + 2 * kStageBytes;                 // two exchange buffers
constexpr int kMiscOff = kXOff + 2 * kXBytes;
constexpr int kMiscBytes = 512;
constexpr int kSmemTotal = kMiscOff + kMiscBytes + 1024;        // + slack to align the base to 1024
constexpr int kTmemS = 0;                                       // two S accumulators of 64 columns
constexpr int kTmemO = 128;                                     // O accumulator: 256 columns
constexpr int kTmemP = 384;                                     // two P buffers (BF16, 32 columns each)
constexpr int kTmemCols = 512;
constexpr int kStatusWaitX = 7;

struct Misc {
    uint64_t bar_kv_full[2];    // stage written by all loader warps
    uint64_t bar_kv_free[2];    // PV of the tile in this stage has finished
    uint64_t bar_s_full[2];     // own half of S complete in tensor memory
    uint64_t bar_p_full[2];     // P written to tensor memory
    uint64_t bar_s_free[2];     // S buffer read for the last time by the softmax warps
    uint64_t bar_x_full[2];     // the partner's half of S has landed in this block's exchange buffer
    uint64_t bar_x_free[2];     // the partner has read what this block sent into its buffer
    uint64_t bar_o_full;
    uint64_t bar_q_full;
    uint64_t valid_mask[2];
    uint32_t tmem_base;
    uint32_t pad;
};

// Which chunks a block owns.  Stage-local order: latent chunks first, RoPE last.
template <int NCHUNK>
struct Own {
    int lat0;        // first latent chunk (global chunk index)
    int n_lat;       // latent chunks owned (4, or 3 for half 1 of the reference layout)
    bool rope;       // owns the RoPE tail (global chunk NCHUNK-1)
    __device__ __forceinline__ int count() const { return n_lat + (rope ? 1 : 0); }
    __device__ __forceinline__ int global_chunk(int j) const { return j < n_lat ? lat0 + j : NCHUNK - 1; }
};
template <int NCHUNK>
__device__ __forceinline__ Own<NCHUNK> own_of(int half) {
    if constexpr (NCHUNK == 9) return half == 0 ? Own<NCHUNK>{0, 4, true} : Own<NCHUNK>{4, 4, false};
    else return half == 0 ? Own<NCHUNK>{0, 4, false} : Own<NCHUNK>{4, 3, true};
}

// Registers one loader thread holds for one tile: entry lane/4 of the warp's 8
// entries, 16-byte piece lane%4 of each owned 64-element chunk.
template <int SRC>
struct Regs {
    uint4 lat[4];
    uint4 rope[2];
    uint32_t sc[2];       // packed layout: the FP32 scales of the two owned 128-element blocks; reference: 4 UE8M0 bytes
    uint32_t vmask;
};

template <int NCHUNK, int SRC>
__device__ __forceinline__ void fetch(const DecodeArgs& a, const Own<NCHUNK>& own, unsigned long long key, uint32_t vmask,
                                      int lane, Regs<SRC>& r) {
    r.vmask = vmask;
    const int i = lane >> 2, piece = lane & 3;
    const unsigned long long k = __shfl_sync(0xFFFFFFFFu, key, i);
    if (!((vmask >> i) & 1u)) return;
    if constexpr (SRC != kSrcRef) {
        const uint8_t* row = reinterpret_cast<const uint8_t*>(k);
#pragma unroll
        for (int j = 0; j < 4; ++j) r.lat[j] = ptx::ldg_nc_v4(row + (own.lat0 + j) * 64 + piece * 16);
        const uint2 s2 = __ldg(reinterpret_cast<const uint2*>(row + 512 + own.lat0 * 2));   // scales lat0/2, lat0/2 + 1
        r.sc[0] = s2.x;  r.sc[1] = s2.y;
        if (own.rope) {
            r.rope[0] = ptx::ldg_nc_v4(row + 528 + piece * 16);
            r.rope[1] = ptx::ldg_nc_v4(row + 528 + (piece + 4) * 16);
        }
    } else {
        const bool swa = (k >> 62) & 1ull;
        const int64_t e = int64_t(k & ~(1ull << 62));
        const uint8_t* lp = (swa ? a.ref_ks : a.ref_kc) + e * 448;
        const uint8_t* sp = (swa ? a.ref_ks_s : a.ref_kc_s) + e * 7;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (j < own.n_lat) r.lat[j] = ptx::ldg_nc_v4(lp + (own.lat0 + j) * 64 + piece * 16);
        uint32_t s0 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (j < own.n_lat) s0 |= uint32_t(__ldg(sp + own.lat0 + j)) << (8 * j);
        r.sc[0] = s0;
        if (own.rope) {
            const uint8_t* rp = reinterpret_cast<const uint8_t*>(swa ? a.ref_ks_rope : a.ref_kc_rope) + e * 128;
            r.rope[0] = ptx::ldg_nc_v4(rp + piece * 16);
            r.rope[1] = ptx::ldg_nc_v4(rp + (piece + 4) * 16);
        }
    }
}

// Pull this block's part of the warp's 8 records into L2: lane/4 picks the
// entry, lane%4 one 128-byte piece of the 256 owned latent bytes or of the tail.
template <int NCHUNK, int SRC>
__device__ __forceinline__ void prefetch_l2(const Own<NCHUNK>& own, unsigned long long key, uint32_t vmask, int lane) {
    if constexpr (SRC != kSrcRef) {
        const int i = lane >> 2, part = lane & 3;
        const unsigned long long k = __shfl_sync(0xFFFFFFFFu, key, i);
        if ((vmask >> i) & 1u) {
            const uint8_t* row = reinterpret_cast<const uint8_t*>(k);
            if (part < 2) ptx::prefetch_l2(row + own.lat0 * 64 + part * 128);
            else if (part == 2) ptx::prefetch_l2(row + 512);
            else if (own.rope) ptx::prefetch_l2(row + 640);
        }
    }
}

// Dequantise and write stage-local chunk j of this warp's 8 entries (tile rows
// t0..t0+7).  Same shared-memory layout as the single-block kernel: row t of a
// chunk is 128 bytes, 16-byte column c16 at ((c16 ^ (t & 7)) << 4).
template <int NCHUNK, int SRC>
__device__ __forceinline__ void store_chunk(uint32_t stage_base, const Own<NCHUNK>& own, int t0, int lane,
                                            const Regs<SRC>& r, int j) {
    const int i = lane >> 2;
    const uint32_t piece = uint32_t(lane & 3);
    const int t = t0 + i;
    const bool valid = (r.vmask >> i) & 1u;
    const uint32_t base = stage_base + uint32_t(j) * kKvChunkBytes + uint32_t(t) * 128u;
    const uint32_t sw = uint32_t(t & 7);
    uint4 w0 = make_uint4(0, 0, 0, 0), w1 = make_uint4(0, 0, 0, 0);
    if (j >= own.n_lat) {                       // the RoPE tail: a plain copy
        if (valid) { w0 = r.rope[0];  w1 = r.rope[1]; }
        ptx::sts_v4(base + ((piece ^ sw) << 4), w0);
        ptx::sts_v4(base + (((piece + 4u) ^ sw) << 4), w1);
        return;
    }
    if (valid) {
        float s120;
        if constexpr (SRC == kSrcRef) {
            const uint32_t byte = (r.sc[0] >> (8 * j)) & 0xFFu;            // one UE8M0 byte per 64 elements
            s120 = byte ? __uint_as_float((byte + 120u) << 23) : 0.f;
        } else {
            s120 = __uint_as_float(r.sc[j >> 1]) * 1.329227995784916e36f;  // one FP32 scale per 128 elements; x 2^120
        }
        const __nv_bfloat162 scale2 = __float2bfloat162_rn(s120);
        const uint4 x = r.lat[j];
        dequant4(x.x, scale2, w0.x, w0.y);
        dequant4(x.y, scale2, w0.z, w0.w);
        dequant4(x.z, scale2, w1.x, w1.y);
        dequant4(x.w, scale2, w1.z, w1.w);
    }
    ptx::sts_v4(base + (((2u * piece) ^ sw) << 4), w0);
    ptx::sts_v4(base + (((2u * piece + 1u) ^ sw) << 4), w1);
}

template <int NCHUNK, int SRC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
decode_pair_kernel(const __grid_constant__ DecodeArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t q_base = smem_base + kQOff;
    const uint32_t kv_base = smem_base + kKvOff;
    const uint32_t x_base = smem_base + kXOff;
    Misc* misc = reinterpret_cast<Misc*>(smem_gen + kMiscOff);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int half = blockIdx.x & 1;            // = rank in the cluster pair
    const int hg = blockIdx.x >> 1;
    const int n = blockIdx.y;
    const int split = blockIdx.z;
    const int b = n / a.s_q;
    const Own<NCHUNK> own = own_of<NCHUNK>(half);
    const int n_own = own.count();

    int n_tok, kv_len_n;
    if constexpr (SRC == kSrcCsa) {
        n_tok = (a.topk_len != nullptr) ? min(max(__ldg(a.topk_len + n), 0), a.topk) : a.topk;
        kv_len_n = (a.kv_len != nullptr) ? __ldg(a.kv_len + n) : 0x7FFFFFFF;
    } else if constexpr (SRC == kSrcHca) {
        kv_len_n = max(__ldg(a.kv_len + n), 0);
        n_tok = kv_len_n + max(__ldg(a.win_len + n), 0);
    } else {
        kv_len_n = a.ref_m_cur;
        n_tok = a.ref_m_cur + a.ref_swa_len;
    }
    const int tiles_total = (n_tok + kTileN - 1) / kTileN;
    const int tiles_per_split = (tiles_total + a.num_splits - 1) / a.num_splits;
    const int tile0 = min(split * tiles_per_split, tiles_total);
    const int tile1 = min(tile0 + tiles_per_split, tiles_total);
    const int ntiles = tile1 - tile0;           // the same in both blocks of the pair

    const uint32_t bar_kv_full = ptx::smem_u32(&misc->bar_kv_full[0]);
    const uint32_t bar_kv_free = ptx::smem_u32(&misc->bar_kv_free[0]);
    const uint32_t bar_s_full = ptx::smem_u32(&misc->bar_s_full[0]);
    const uint32_t bar_p_full = ptx::smem_u32(&misc->bar_p_full[0]);
    const uint32_t bar_s_free = ptx::smem_u32(&misc->bar_s_free[0]);
    const uint32_t bar_x_full = ptx::smem_u32(&misc->bar_x_full[0]);
    const uint32_t bar_x_free = ptx::smem_u32(&misc->bar_x_free[0]);
    const uint32_t bar_o_full = ptx::smem_u32(&misc->bar_o_full);
    const uint32_t bar_q_full = ptx::smem_u32(&misc->bar_q_full);

    if (tid == 0) {
        trace_mark(a, 3, 0);
        for (int st = 0; st < 2; ++st) {
            ptx::mbar_init(bar_kv_full + 8 * st, kNumLoaderWarps);
            ptx::mbar_init(bar_kv_free + 8 * st, 1);
            ptx::mbar_init(bar_s_full + 8 * st, 1);
            ptx::mbar_init(bar_p_full + 8 * st, kNumSoftmaxWarps);
            ptx::mbar_init(bar_s_free + 8 * st, kNumSoftmaxWarps);
            ptx::mbar_init(bar_x_full + 8 * st, kNumSoftmaxWarps);        // one arrival per partner softmax warp
            ptx::mbar_init(bar_x_free + 8 * st, kNumSoftmaxWarps);
        }
        ptx::mbar_init(bar_o_full, 1);
        ptx::mbar_init(bar_q_full, 1);
        ptx::fence_mbar_init();
        if (ntiles > 0) {
            // own Q columns by TMA, one 64-column box per owned chunk, swizzled operand layout
            ptx::mbar_arrive_expect_tx(bar_q_full, uint32_t(n_own) * kQChunkBytes);
            const int row0 = n * a.H + hg * kHeadsPerCta;
            for (int j = 0; j < n_own; ++j)
                ptx::tma_load_2d(q_base + uint32_t(j) * kQChunkBytes, &a.q_map, own.global_chunk(j) * 64, row0, bar_q_full);
        }
    }
    if (warp == kMmaWarp) {
        ptx::tmem_alloc(ptx::smem_u32(&misc->tmem_base), kTmemCols);
        ptx::tmem_relinquish();
    }
    // Both blocks' barriers must exist before the partner arrives on them.
    ptx::tc_fence_before_sync();
    ptx::cluster_sync();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = misc->tmem_base;

    if (ntiles > 0) {
        if (warp >= kFirstLoaderWarp && warp < kMmaWarp) {
            // ───────────── loader warps ─────────────
            const int lw = warp - kFirstLoaderWarp;
            Regs<SRC> regs_a, regs_b;
            unsigned long long key2 = 0, key3 = 0, key4 = 0;
            uint32_t vm2 = 0, vm3 = 0, vm4 = 0;
            {
                bool valid = false;
                const int which = lane >> 3;
                const unsigned long long key = loader_resolve<SRC>(a, b, n, (tile0 + which) * kTileN + lw * 8 + (lane & 7),
                                                                   (which < ntiles) ? n_tok : 0, kv_len_n, valid);
                const uint32_t bal = __ballot_sync(0xFFFFFFFFu, valid);
                vm2 = (bal >> 16) & 0xFFu;
                vm3 = (bal >> 24) & 0xFFu;
                const unsigned long long key1 = __shfl_sync(0xFFFFFFFFu, key, (lane & 7) + 8);
                key2 = __shfl_sync(0xFFFFFFFFu, key, (lane & 7) + 16);
                key3 = __shfl_sync(0xFFFFFFFFu, key, (lane & 7) + 24);
                fetch<NCHUNK, SRC>(a, own, key, bal & 0xFFu, lane, regs_a);
                fetch<NCHUNK, SRC>(a, own, key1, (bal >> 8) & 0xFFu, lane, regs_b);
                prefetch_l2<NCHUNK, SRC>(own, key2, vm2, lane);
                prefetch_l2<NCHUNK, SRC>(own, key3, vm3, lane);
                key4 = loader_resolve_warp<SRC>(a, b, n, (tile0 + 4) * kTileN + lw * 8, lane, (4 < ntiles) ? n_tok : 0,
                                                kv_len_n, vm4);
            }
            bool lok = true;
            auto tile_step = [&](Regs<SRC>& regs, int it) {
                const int st = it & 1;
                if (it >= 2) {
                    const bool w = ptx::mbar_wait(bar_kv_free + 8 * st, uint32_t((it >> 1) - 1) & 1u, kWaitTimeoutNs);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_timeout(a.status, kStatusWaitKvFree, 2, tile0 + it);
                        lok = false;
                        return;
                    }
                }
                if (lw == 0 && lane == 0) trace_mark(a, 2, 2 * it);
                if (!(a.dbg & 2)) prefetch_l2<NCHUNK, SRC>(own, key4, vm4, lane);
                if (lane == 0) reinterpret_cast<volatile uint8_t*>(&misc->valid_mask[st])[lw] = uint8_t(regs.vmask);
                const uint32_t stage = kv_base + uint32_t(st) * kStageBytes;
#pragma unroll
                for (int j = 0; j < kMaxOwn; ++j)
                    if (j < n_own) store_chunk<NCHUNK, SRC>(stage, own, lw * 8, lane, regs, j);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_kv_full + 8 * st);
                if (lw == 0 && lane == 0) trace_mark(a, 2, 2 * it + 1);
                if (it + 2 < ntiles) fetch<NCHUNK, SRC>(a, own, key2, vm2, lane, regs);
                key2 = key3;  vm2 = vm3;
                key3 = key4;  vm3 = vm4;
                key4 = loader_resolve_warp<SRC>(a, b, n, (tile0 + it + 5) * kTileN + lw * 8, lane,
                                                (it + 5 < ntiles) ? n_tok : 0, kv_len_n, vm4);
            };
            for (int it = 0; it < ntiles && lok; it += 2) {
                tile_step(regs_a, it);
                if (it + 1 < ntiles && lok) tile_step(regs_b, it + 1);
            }
        } else if (warp == kMmaWarp) {
            // ───────────── MMA issue (one thread) ─────────────
            if (lane == 0) {
                constexpr uint32_t idesc_qk = ptx::make_idesc_bf16(128, kTileN, false, false);
                constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(128, kDvHalf, false, true);
                constexpr uint32_t kDescHi = ptx::smem_desc_hi(1024);
                bool ok = true;
                if (!ptx::mbar_wait(bar_q_full, 0u, kWaitTimeoutNs)) {
                    report_timeout(a.status, kStatusWaitQ, 1, tile0);
                    ok = false;
                }
                ptx::tc_fence_after_sync();
                const uint32_t q_lo = ptx::smem_desc_lo(q_base, 16);
                // own half of S(it): n_own chunks x 4 MMAs, all operands in shared memory
                auto issue_qk = [&](int it) {
                    const int st = it & 1;
                    const uint32_t k_lo = ptx::smem_desc_lo(kv_base + uint32_t(st) * kStageBytes, 16);
                    const uint32_t d = tmem + kTmemS + uint32_t(st) * kTileN;
                    ptx::tc_fence_after_sync();
                    trace_mark(a, 1, 2 * it);
#pragma unroll
                    for (int j = 0; j < kMaxOwn; ++j) {
                        if (j < n_own) {
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                ptx::mma_bf16_ss2(d, q_lo + uint32_t((j * kQChunkBytes + k * 32) >> 4),
                                                  k_lo + uint32_t((j * kKvChunkBytes + k * 32) >> 4), kDescHi, idesc_qk,
                                                  (j | k) ? 1u : 0u);
                        }
                    }
                    ptx::mma_commit(bar_s_full + 8 * st);
                };
                // O += P(it) . V(it): A = P in tensor memory, B = the four value chunks (stage chunks 0..3), MN-major
                auto issue_pv = [&](int it) {
                    const int st = it & 1;
                    ptx::tc_fence_after_sync();
                    trace_mark(a, 1, 2 * it + 1);
                    const uint32_t p_tmem = tmem + kTmemP + uint32_t(st) * 32;
                    const uint32_t v_lo = ptx::smem_desc_lo(kv_base + uint32_t(st) * kStageBytes, kKvChunkBytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        ptx::mma_bf16_ts2(tmem + kTmemO, p_tmem + k * 8, v_lo + uint32_t((k * 2048) >> 4), kDescHi, idesc_pv,
                                          (it | k) ? 1u : 0u);
                    ptx::mma_commit(bar_kv_free + 8 * st);
                };
                int qk_next = 0, pv_next = 0;
                uint64_t t_last = 0;
                uint32_t polls = 0;
                while (ok && pv_next < ntiles) {
                    bool progress = false;
                    if (pv_next < qk_next &&
                        ptx::mbar_test_wait(bar_p_full + 8 * (pv_next & 1), uint32_t(pv_next >> 1) & 1u)) {
                        issue_pv(pv_next);
                        ++pv_next;
                        progress = true;
                    } else if (qk_next < ntiles &&
                               (qk_next < 2 ||      // S buffer qk_next&1 was last read for tile qk_next-2
                                ptx::mbar_test_wait(bar_s_free + 8 * (qk_next & 1), uint32_t((qk_next >> 1) - 1) & 1u)) &&
                               ptx::mbar_test_wait(bar_kv_full + 8 * (qk_next & 1), uint32_t(qk_next >> 1) & 1u)) {
                        issue_qk(qk_next);
                        ++qk_next;
                        progress = true;
                    }
                    if (progress) {
                        polls = 0;
                    } else {
                        if (polls == 0) t_last = ptx::globaltimer_ns();
                        if ((++polls & 255u) != 0u || ptx::globaltimer_ns() - t_last <= kWaitTimeoutNs) continue;
                        report_timeout(a.status, (pv_next < qk_next) ? kStatusWaitPFull : kStatusWaitKvFull, 1, tile0 + pv_next);
                        ok = false;
                    }
                }
                if (ok) ptx::mma_commit(bar_o_full);
            }
            __syncwarp();
        } else if (warp < kNumSoftmaxWarps) {
            // ───────────── softmax + exchange + epilogue warps ─────────────
            const int r = warp * 32 + lane;
            const uint32_t lane_addr = uint32_t(warp * 32) << 16;
            const uint32_t peer = uint32_t(half ^ 1);
            // my row in the partner's exchange buffers, and the partner's barriers
            // exchange buffer layout [16-byte column v (16)][row (128)]: one warp instruction moves
            // 32 consecutive 16-byte pieces, both for the remote stores and for the local loads
            const uint32_t x_row_local = x_base + uint32_t(r) * 16u;
            const uint32_t x_row_peer = ptx::mapa(x_row_local, peer);
            const uint32_t bar_x_peer = ptx::mapa(bar_x_full, peer);
            const uint32_t bar_xfree_peer = ptx::mapa(bar_x_free, peer);
            float m_ref = -CUDART_INF_F;
            float l_sum = 0.f;
            bool ok = true;
            // Send this block's half of S(t) to the partner: wait for the QK MMAs, read the 64
            // columns, store them into the partner's exchange buffer t&1 and arrive on its barrier.
            // It runs one tile ahead of the softmax arithmetic, so that the transfer of tile t+1 is
            // in flight while tile t is being worked on.
            auto send_half = [&](int t) -> bool {
                const int st = t & 1;
                {
                    const bool w = ptx::mbar_wait(bar_s_full + 8 * st, uint32_t(t >> 1) & 1u, kWaitTimeoutNs);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_timeout(a.status, kStatusWaitSFull, 0, tile0 + t);
                        return false;
                    }
                }
                if (t >= 2) {
                    // the partner must have read tile t-2 out of that buffer
                    const bool w = ptx::mbar_wait_cluster(bar_x_free + 8 * st, uint32_t((t >> 1) - 1) & 1u, kWaitTimeoutNs);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_timeout(a.status, kStatusWaitX, 3, tile0 + t);
                        return false;
                    }
                }
                ptx::tc_fence_after_sync();
                if (tid == 0) trace_mark(a, 0, 2 * t);
                const uint32_t s_tmem = tmem + lane_addr + kTmemS + uint32_t(st) * kTileN;
                uint32_t h0[32], h1[32];
                ptx::tmem_ld32(s_tmem, h0);
                ptx::tmem_ld32(s_tmem + 32, h1);
                ptx::tmem_wait_ld();
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    ptx::sts_cluster_v4(x_row_peer + uint32_t(st) * kXBytes + uint32_t(v) * 2048u,
                                        make_uint4(h0[4 * v], h0[4 * v + 1], h0[4 * v + 2], h0[4 * v + 3]));
                    ptx::sts_cluster_v4(x_row_peer + uint32_t(st) * kXBytes + uint32_t(v + 8) * 2048u,
                                        make_uint4(h1[4 * v], h1[4 * v + 1], h1[4 * v + 2], h1[4 * v + 3]));
                }
                // one remote arrival per warp: every lane makes its stores visible at cluster scope
                // and lane 0 arrives for the warp
                ptx::fence_acq_rel_cluster();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(bar_x_peer + 8 * st);
                return true;
            };
            ok = send_half(0);
            for (int it = 0; it < ntiles && ok; ++it) {
                const int st = it & 1;
                const uint32_t s_tmem = tmem + lane_addr + kTmemS + uint32_t(st) * kTileN;
                if (it + 1 < ntiles) {
                    ok = send_half(it + 1);
                    if (!ok) break;
                }
                // the partner's half of S(it): every row of buffer st written (4 warp arrivals)
                {
                    const bool w = ptx::mbar_wait_cluster(bar_x_full + 8 * st, uint32_t(it >> 1) & 1u, kWaitTimeoutNs);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_timeout(a.status, kStatusWaitX, 0, tile0 + it);
                        ok = false;  break;
                    }
                }
                if (tid == 0) trace_mark(a, 0, 512 + it);
                uint32_t s0[32], s1[32];
                ptx::tmem_ld32(s_tmem, s0);             // own half again (still in tensor memory)
                ptx::tmem_ld32(s_tmem + 32, s1);
                ptx::tmem_wait_ld();
                // this S buffer may now be overwritten by the QK MMAs of tile it+2
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_s_free + 8 * st);
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    const uint4 p0 = ptx::lds_v4(x_row_local + uint32_t(st) * kXBytes + uint32_t(v) * 2048u);
                    const uint4 p1 = ptx::lds_v4(x_row_local + uint32_t(st) * kXBytes + uint32_t(v + 8) * 2048u);
                    s0[4 * v + 0] = __float_as_uint(__uint_as_float(s0[4 * v + 0]) + __uint_as_float(p0.x));
                    s0[4 * v + 1] = __float_as_uint(__uint_as_float(s0[4 * v + 1]) + __uint_as_float(p0.y));
                    s0[4 * v + 2] = __float_as_uint(__uint_as_float(s0[4 * v + 2]) + __uint_as_float(p0.z));
                    s0[4 * v + 3] = __float_as_uint(__uint_as_float(s0[4 * v + 3]) + __uint_as_float(p0.w));
                    s1[4 * v + 0] = __float_as_uint(__uint_as_float(s1[4 * v + 0]) + __uint_as_float(p1.x));
                    s1[4 * v + 1] = __float_as_uint(__uint_as_float(s1[4 * v + 1]) + __uint_as_float(p1.y));
                    s1[4 * v + 2] = __float_as_uint(__uint_as_float(s1[4 * v + 2]) + __uint_as_float(p1.z));
                    s1[4 * v + 3] = __float_as_uint(__uint_as_float(s1[4 * v + 3]) + __uint_as_float(p1.w));
                }
                // buffer st may be overwritten by the partner's tile it+2
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(bar_xfree_peer + 8 * st);
                const uint64_t vmask = *reinterpret_cast<volatile uint64_t*>(&misc->valid_mask[st]);
                const uint32_t vm0 = uint32_t(vmask), vm1 = uint32_t(vmask >> 32);
                float x0[32], x1[32];
                float tmax = -CUDART_INF_F;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    x0[i] = ((vm0 >> i) & 1u) ? __uint_as_float(s0[i]) * a.scale_log2 : -CUDART_INF_F;
                    x1[i] = ((vm1 >> i) & 1u) ? __uint_as_float(s1[i]) * a.scale_log2 : -CUDART_INF_F;
                    tmax = fmaxf(tmax, fmaxf(x0[i], x1[i]));
                }
                float alpha = 1.f;
                bool moved = false;
                if (tmax > m_ref + kRescaleThreshold) {
                    alpha = (m_ref == -CUDART_INF_F) ? 0.f : ptx::ex2(m_ref - tmax);
                    m_ref = tmax;
                    moved = true;
                }
                const float m_use = (m_ref == -CUDART_INF_F) ? 0.f : m_ref;
                float psum = 0.f;
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = ptx::ex2(x0[2 * i] - m_use), p1 = ptx::ex2(x0[2 * i + 1] - m_use);
                    psum += p0 + p1;
                    pk[i] = ptx::pack_bf16x2(p0, p1);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = ptx::ex2(x1[2 * i] - m_use), p1 = ptx::ex2(x1[2 * i + 1] - m_use);
                    psum += p0 + p1;
                    pk[16 + i] = ptx::pack_bf16x2(p0, p1);
                }
                l_sum = l_sum * alpha + psum;
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
                if (it >= 2) {
                    // P buffer st was the A operand of tile it-2's PV MMAs: they must have finished
                    const bool w = ptx::mbar_wait(bar_kv_free + 8 * st, uint32_t((it >> 1) - 1) & 1u, kWaitTimeoutNs);
                    if (!__all_sync(0xFFFFFFFFu, w)) {
                        report_timeout(a.status, kStatusWaitKvFree, 0, tile0 + it);
                        ok = false;  break;
                    }
                    ptx::tc_fence_after_sync();
                }
                ptx::tmem_st32(tmem + lane_addr + kTmemP + uint32_t(st) * 32, pk);
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
                const int h = hg * kHeadsPerCta + r;
                const bool write = h < a.H;
                const bool final_out = a.num_splits == 1;
                float denom = l_sum;
                if (final_out && a.attn_sink != nullptr && write) {
                    const float s2 = __ldg(a.attn_sink + h) * 1.4426950408889634f;
                    denom = (l_sum > 0.f) ? l_sum + ptx::ex2(s2 - m_ref) : 1.f;
                }
                const float inv = (l_sum > 0.f) ? 1.f / denom : 0.f;
                const float lse2 = (l_sum > 0.f) ? m_ref + log2f(l_sum) : -CUDART_INF_F;
                const int64_t row = int64_t(n) * a.H + h;
#pragma unroll 1
                for (int c = 0; c < kDvHalf / 32; ++c) {
                    uint32_t o[32];
                    ptx::tmem_ld32(tmem + lane_addr + kTmemO + c * 32, o);
                    ptx::tmem_wait_ld();
                    if (write) {
                        const int col = half * kDvHalf + c * 32;
                        if (final_out) {
                            uint4* dst = reinterpret_cast<uint4*>(a.out + row * 512 + col);
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                uint4 w;
                                w.x = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                                w.y = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                                w.z = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                                w.w = ptx::pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                                dst[v] = w;
                            }
                        } else {
                            float4* dst = reinterpret_cast<float4*>(
                                a.partial_o + (int64_t(split) * gridDim.y * a.H + row) * 512 + col);
#pragma unroll
                            for (int v = 0; v < 8; ++v)
                                dst[v] = make_float4(__uint_as_float(o[4 * v + 0]) * inv, __uint_as_float(o[4 * v + 1]) * inv,
                                                     __uint_as_float(o[4 * v + 2]) * inv, __uint_as_float(o[4 * v + 3]) * inv);
                        }
                    }
                }
                if (write && half == 0) {
                    if (final_out) {
                        if (a.lse != nullptr) a.lse[row] = (l_sum > 0.f) ? lse2 * 0.6931471805599453f : -CUDART_INF_F;
                    } else {
                        a.partial_lse[int64_t(split) * gridDim.y * a.H + row] = lse2;
                    }
                }
            }
        }
    } else {
        // Nothing to attend to in this split: zero output, LSE = -inf.
        const bool final_out = a.num_splits == 1;
        for (int i = tid; i < kHeadsPerCta * (kDvHalf / 8); i += kNumThreads) {
            const int r = i / (kDvHalf / 8), v = i % (kDvHalf / 8);
            const int h = hg * kHeadsPerCta + r;
            if (h >= a.H) continue;
            const int64_t row = int64_t(n) * a.H + h;
            const int col = half * kDvHalf + v * 8;
            if (final_out) {
                *reinterpret_cast<uint4*>(a.out + row * 512 + col) = make_uint4(0, 0, 0, 0);
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

    // ── common exit.  The partner may still be writing into this block's exchange buffers or
    // arriving on its barriers until it, too, has got here: leave together. ──
    ptx::tc_fence_before_sync();
    ptx::cluster_sync();
    if (tid == 0) trace_mark(a, 3, 3);
    if (warp == kMmaWarp) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(misc->tmem_base, kTmemCols);
    }
}

}  // namespace pair
}  // namespace dsv4

// Split-KV scheduler: a one-block planner kernel that turns the per-row lengths of a decode batch
// into a work list for the resident blocks of the decode kernel.
//
// A unit is (row, group of 128 heads); its work is its 64-entry tiles plus a fixed cost for the
// set-up and the write-out of an item.  Units are laid end to end on a cost axis and the axis is cut
// into equal parts, one per block pair (the two blocks of a pair compute the two halves of the value
// columns of the same items).  A unit that straddles a cut is split there: each piece becomes an item
// of its own with a partial-output slot, and the merge kernel adds the pieces up; a unit inside one
// part is a single item that writes the final output directly.  With `fixed_splits` >= 1 every unit is
// instead cut into that many equal pieces (the split count a caller asks for) and the pieces are dealt
// to the pairs in order; consecutive pieces of a unit that fall to the same pair run there as one item.
// The plan depends on the lengths only: one plan serves every layer of a step.
//
// Replaces the static "tile index = split index" bookkeeping of the reference
// (hca/sm100/helpers.h:831-869, hca/sm100/kernel.cu:99-102,248-257).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "decode_kernel.cuh"

namespace dsv4 {

constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxPairs = 1024;
// Costs in 1/32 of a tile's time (fine enough that the equal shares of many pairs do not round a few pairs away).
constexpr int kPlanTileCost = 32;
constexpr int kPlanFixedCost = 48;     // set-up and write-out of an item that the overlap with its neighbours does not hide
constexpr int kPlanMergeCost = 96;     // what cutting units costs a pair in partial traffic and merge time

struct PlanArgs {
    int kind;                    // SourceKind: where the lengths come from
    int rows, hgs;               // rows = B * s_q, hgs = groups of 128 heads
    int topk;                    // CSA
    const int32_t* topk_len;     // CSA, optional
    const int32_t* kv_len;       // CSA optional (passed through), HCA / packed pages required
    const int32_t* win_len;      // HCA / packed pages
    int ref_m_cur, ref_swa_len;  // reference planes
    int num_pairs;
    int fixed_splits;            // 0: balance over the pairs; >= 1: that many equal pieces per unit
    int item_cap, slot_cap;
    int32_t* pair_begin;         // out [num_pairs + 1]
    int32_t* items;              // out [item_cap][kItemWords]
    int32_t* unit_nsplits;       // out [rows * hgs]: pieces of the unit (1 = final output written by the decode kernel)
    int32_t* unit_slot;          // out [rows * hgs]: first partial slot of the unit (when split)
    long long* unit_prefix;      // scratch [rows * hgs]
    int32_t* info;               // out [4]: items, slots, 1 if a capacity was exceeded (plan then not usable), quota
};

__host__ __device__ __forceinline__ void plan_row_lengths(const PlanArgs& p, int row, int& n_tok, int& kv_len_n) {
    if (p.kind == kSrcCsa) {
        const int raw = (p.topk_len != nullptr) ? p.topk_len[row] : p.topk;
        n_tok = raw < 0 ? 0 : (raw > p.topk ? p.topk : raw);
        kv_len_n = (p.kv_len != nullptr) ? p.kv_len[row] : 0x7FFFFFFF;
    } else if (p.kind == kSrcHca || p.kind == kSrcRefPaged) {
        kv_len_n = p.kv_len[row] > 0 ? p.kv_len[row] : 0;
        n_tok = kv_len_n + (p.win_len[row] > 0 ? p.win_len[row] : 0);
    } else {
        kv_len_n = p.ref_m_cur;
        n_tok = p.ref_m_cur + p.ref_swa_len;
    }
}

__host__ __device__ __forceinline__ int plan_piece_cost(int tiles) { return tiles > 0 ? kPlanTileCost * tiles + kPlanFixedCost : 1; }

// Cost of a unit: one item, or its fixed_splits equal pieces.
__host__ __device__ __forceinline__ int plan_unit_cost(int tiles, int fixed_splits) {
    if (tiles <= 0 || fixed_splits <= 1) return plan_piece_cost(tiles);
    const int tps = (tiles + fixed_splits - 1) / fixed_splits;
    const int pieces = (tiles + tps - 1) / tps;
    return kPlanTileCost * tiles + pieces * kPlanFixedCost;
}

// Cutting units pays only when whole units cannot be dealt out evenly enough: compare the longest share
// whole units would give a pair with an equal share plus the cost of the cuts.
__host__ __device__ __forceinline__ bool plan_keep_whole(int n_units, int num_pairs, int max_cost, long long quota) {
    const long long t_whole = (n_units <= num_pairs) ? (long long)max_cost : quota + max_cost / 2;
    return t_whole <= quota + kPlanMergeCost;
}

// Walks the pieces of the unit that starts at C on the cost axis: next() yields (pair, first tile, tiles)
// of one piece after the other.
struct PieceWalk {
    long long C, quota, at;
    int cost, tiles, last_pair, fixed, tps, t, pr, p1;
    bool single, done;
    __host__ __device__ int pair_of(long long x) const {
        const long long q = x / quota;
        return int(q < last_pair ? q : last_pair);
    }
    __host__ __device__ PieceWalk(const PlanArgs& p, long long C_, int cost_, int tiles_, long long quota_, bool whole)
        : C(C_), quota(quota_), at(C_), cost(cost_), tiles(tiles_), last_pair(p.num_pairs - 1), fixed(p.fixed_splits), tps(1), t(0),
          pr(0), p1(0), single(false), done(false) {
        single = tiles <= 0 || (fixed <= 0 && whole) || fixed == 1;
        if (fixed > 1) tps = (tiles + fixed - 1) / fixed;
        pr = pair_of(C);
        p1 = pair_of(C + cost - 1);
    }
    __host__ __device__ bool next(int& pair, int& t0, int& nt) {
        if (done) return false;
        if (single) {
            pair = pair_of(C);  t0 = 0;  nt = tiles > 0 ? tiles : 0;
            done = true;
            return true;
        }
        if (fixed > 1) {
            if (t >= tiles) { done = true;  return false; }
            // consecutive pieces of the unit that fall to the same pair run as one item: their partial results
            // would only be added up again
            pair = pair_of(at);  t0 = t;  nt = 0;
            do {
                const int n = tps < tiles - t ? tps : tiles - t;
                nt += n;
                at += plan_piece_cost(n);
                t += n;
            } while (t < tiles && pair_of(at) == pair);
            return true;
        }
        const int p0 = pair_of(C);
        while (pr <= p1) {
            const long long lo = (pr == p0) ? 0 : (long long)pr * quota - C;
            const long long hi = (pr == p1) ? cost : (long long)(pr + 1) * quota - C;
            const int ta = int((lo * tiles + cost / 2) / cost), tb = int((hi * tiles + cost / 2) / cost);
            const int here = pr++;
            if (tb > ta) {
                pair = here;  t0 = ta;  nt = tb - ta;
                return true;
            }
        }
        done = true;
        return false;
    }
};

__global__ void __launch_bounds__(kPlanThreads) plan_kernel(const PlanArgs p) {
    __shared__ long long s_warp[32];
    __shared__ long long s_carry;
    __shared__ int s_max;
    __shared__ int s_count[kPlanMaxPairs];
    __shared__ int s_begin[kPlanMaxPairs + 1];
    __shared__ int s_slots, s_over;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int n_units = p.rows * p.hgs;
    if (tid == 0) { s_carry = 0;  s_max = 0;  s_slots = 0;  s_over = 0; }
    for (int i = tid; i < p.num_pairs; i += kPlanThreads) s_count[i] = 0;
    __syncthreads();

    // pass 1: cost of every unit and its start on the cost axis
    for (int base = 0; base < n_units; base += kPlanThreads) {
        const int u = base + tid;
        int cost = 0;
        if (u < n_units) {
            int n_tok, kv_len_n;
            plan_row_lengths(p, u / p.hgs, n_tok, kv_len_n);
            cost = plan_unit_cost((n_tok + kTileN - 1) / kTileN, p.fixed_splits);
            atomicMax(&s_max, cost);
        }
        long long incl = cost;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) s_warp[wid] = incl;
        __syncthreads();
        if (wid == 0) {
            long long w = s_warp[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const long long t = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += t;
            }
            s_warp[lane] = w;
        }
        __syncthreads();
        const long long before = s_carry + (wid > 0 ? s_warp[wid - 1] : 0) + incl - cost;
        if (u < n_units) p.unit_prefix[u] = before;
        __syncthreads();
        if (tid == kPlanThreads - 1) s_carry = before + cost;
        __syncthreads();
    }
    const long long total = s_carry;
    long long quota = (total + p.num_pairs - 1) / p.num_pairs;
    if (quota < 1) quota = 1;
    const bool whole = plan_keep_whole(n_units, p.num_pairs, s_max, quota);

    // pass 2: pieces per pair, pieces per unit, partial slots
    for (int u = tid; u < n_units; u += kPlanThreads) {
        int n_tok, kv_len_n;
        plan_row_lengths(p, u / p.hgs, n_tok, kv_len_n);
        const int tiles = (n_tok + kTileN - 1) / kTileN;
        const int cost = plan_unit_cost(tiles, p.fixed_splits);
        int pieces = 0;
        {
            PieceWalk w(p, p.unit_prefix[u], cost, tiles, quota, whole);
            int pr, t0, nt;
            while (w.next(pr, t0, nt)) { atomicAdd(&s_count[pr], 1);  ++pieces; }
        }
        int slot = -1;
        if (pieces > 1) {
            slot = atomicAdd(&s_slots, pieces);
            if (slot + pieces > p.slot_cap) { s_over = 1;  slot = -1; }
        }
        p.unit_nsplits[u] = pieces;
        p.unit_slot[u] = slot;
    }
    __syncthreads();

    // pass 3: first item of every pair
    if (tid == 0) {
        int acc = 0;
        for (int i = 0; i < p.num_pairs; ++i) { s_begin[i] = acc;  acc += s_count[i];  s_count[i] = 0; }
        s_begin[p.num_pairs] = acc;
        if (acc > p.item_cap) s_over = 1;
    }
    __syncthreads();
    const bool over = s_over != 0;
    // (pairs beyond num_pairs - a launch with more blocks than the plan was made for - find empty lists)
    for (int i = tid; i <= kPlanMaxPairs; i += kPlanThreads) p.pair_begin[i] = over ? 0 : s_begin[i < p.num_pairs ? i : p.num_pairs];
    if (tid == 0) {
        p.info[0] = s_begin[p.num_pairs];
        p.info[1] = s_slots;
        p.info[2] = over ? 1 : 0;
        p.info[3] = int(quota < 0x7FFFFFFF ? quota : 0x7FFFFFFF);
    }
    if (over) return;       // nothing is dealt out: every block finds an empty list (the host checks info[2] in its checked mode)

    // pass 4: the items
    for (int u = tid; u < n_units; u += kPlanThreads) {
        const int row = u / p.hgs, hg = u % p.hgs;
        int n_tok, kv_len_n;
        plan_row_lengths(p, row, n_tok, kv_len_n);
        const int tiles = (n_tok + kTileN - 1) / kTileN;
        const int cost = plan_unit_cost(tiles, p.fixed_splits);
        const int slot0 = p.unit_slot[u];
        PieceWalk w(p, p.unit_prefix[u], cost, tiles, quota, whole);
        int pr, t0, nt, j = 0;
        while (w.next(pr, t0, nt)) {
            const int at = s_begin[pr] + atomicAdd(&s_count[pr], 1);
            int4* rec = reinterpret_cast<int4*>(p.items + int64_t(at) * kItemWords);
            rec[0] = make_int4(row, hg, t0, nt);
            rec[1] = make_int4(slot0 >= 0 ? slot0 + j : -1, n_tok, kv_len_n, 0);
            ++j;
        }
    }
}

// The same plan computed serially on the host from length arrays in host memory (every pointer of `p`
// is then a host pointer).  For inspection and for tests of the planning arithmetic without a GPU; the
// order of the items inside a pair may differ from the kernel's (there it depends on the order of atomics).
inline void plan_host(const PlanArgs& p) {
    const int n_units = p.rows * p.hgs;
    long long total = 0;
    int max_cost = 0;
    for (int u = 0; u < n_units; ++u) {
        int n_tok, kv_len_n;
        plan_row_lengths(p, u / p.hgs, n_tok, kv_len_n);
        const int cost = plan_unit_cost((n_tok + kTileN - 1) / kTileN, p.fixed_splits);
        p.unit_prefix[u] = total;
        total += cost;
        if (cost > max_cost) max_cost = cost;
    }
    long long quota = (total + p.num_pairs - 1) / p.num_pairs;
    if (quota < 1) quota = 1;
    const bool whole = plan_keep_whole(n_units, p.num_pairs, max_cost, quota);
    for (int i = 0; i <= kPlanMaxPairs; ++i) p.pair_begin[i] = 0;
    int slots = 0, over = 0;
    for (int u = 0; u < n_units; ++u) {
        int n_tok, kv_len_n;
        plan_row_lengths(p, u / p.hgs, n_tok, kv_len_n);
        const int tiles = (n_tok + kTileN - 1) / kTileN;
        int pieces = 0;
        {
            PieceWalk w(p, p.unit_prefix[u], plan_unit_cost(tiles, p.fixed_splits), tiles, quota, whole);
            int pr, t0, nt;
            while (w.next(pr, t0, nt)) { ++p.pair_begin[pr + 1];  ++pieces; }
        }
        int slot = -1;
        if (pieces > 1) {
            slot = slots;
            slots += pieces;
            if (slots > p.slot_cap) over = 1;
        }
        p.unit_nsplits[u] = pieces;
        p.unit_slot[u] = slot;
    }
    for (int i = 0; i < kPlanMaxPairs; ++i) p.pair_begin[i + 1] += p.pair_begin[i];
    const int n_items = p.pair_begin[p.num_pairs];
    if (n_items > p.item_cap) over = 1;
    p.info[0] = n_items;  p.info[1] = slots;  p.info[2] = over;  p.info[3] = int(quota < 0x7FFFFFFF ? quota : 0x7FFFFFFF);
    if (over) {
        for (int i = 0; i <= kPlanMaxPairs; ++i) p.pair_begin[i] = 0;
        return;
    }
    int fill[kPlanMaxPairs] = {};
    for (int u = 0; u < n_units; ++u) {
        const int row = u / p.hgs, hg = u % p.hgs;
        int n_tok, kv_len_n;
        plan_row_lengths(p, row, n_tok, kv_len_n);
        const int tiles = (n_tok + kTileN - 1) / kTileN;
        const int slot0 = p.unit_slot[u];
        PieceWalk w(p, p.unit_prefix[u], plan_unit_cost(tiles, p.fixed_splits), tiles, quota, whole);
        int pr, t0, nt, j = 0;
        while (w.next(pr, t0, nt)) {
            int32_t* rec = p.items + int64_t(p.pair_begin[pr] + fill[pr]++) * kItemWords;
            rec[0] = row;  rec[1] = hg;  rec[2] = t0;  rec[3] = nt;
            rec[4] = slot0 >= 0 ? slot0 + j : -1;  rec[5] = n_tok;  rec[6] = kv_len_n;  rec[7] = 0;
            ++j;
        }
    }
}

}  // namespace dsv4

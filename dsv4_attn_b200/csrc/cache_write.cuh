// Cache-write side of the HCA path and of any path that appends rows to the
// paged FP8 cache.
//
//  * hca_compress_kernel: the one-branch compressor - each block of m rows
//    becomes one row, per channel a softmax over the m gating logits (plus a
//    per-position bias) weighting the m value rows - optionally fused with the
//    quantiser and the insert into the paged cache.
//  * kv_quantize_insert_kernel: BF16 rows [B, T, 576] -> 656-byte cache entries
//    (FP32 absmax/448 scale per 128 latent elements, e4m3, BF16 RoPE tail)
//    written at logical positions insert_pos[b] + t through the block table.
//
// Both stream their inputs once with 128-bit loads; the entry is produced in
// registers and written with 8/16-byte stores.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <math_constants.h>
#include <stdint.h>
#include <type_traits>

#include "ptx.cuh"
#include "compress_reduce.cuh"   // unpack8

namespace dsv4 {

constexpr int kStatusBadInsert = 16;   // status code: an insert position outside the block table / pool

struct CacheDest {
    uint8_t* kv_pool;             // [num_pages, 64, 656] or null
    const int32_t* block_table;   // [B, max_pages]
    const int32_t* insert_pos;    // [B] logical index of the first new entry
    int max_pages;
    int64_t num_pages;
    int32_t* status;              // optional
};

// Address of logical entry e of request b, or null (and a status code) when e is
// outside the block table or the table names a page outside the pool.
__device__ __forceinline__ uint8_t* entry_address(const CacheDest& d, int b, int64_t e) {
    if (e >= 0 && (e >> 6) < d.max_pages) {
        const int page = __ldg(d.block_table + int64_t(b) * d.max_pages + (e >> 6));
        if (page >= 0 && page < d.num_pages) return d.kv_pool + (int64_t(page) * 64 + (e & 63)) * 656;
    }
    if (d.status != nullptr && atomicCAS(d.status, 0, kStatusBadInsert) == 0) {
        d.status[1] = b;
        d.status[2] = int(e);
        d.status[3] = 0;
    }
    return nullptr;
}

__device__ __forceinline__ float bf16_round_f(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// scale of a 128-element block from its absolute maximum: absmax / 448, 1 for a block of zeros
__device__ __forceinline__ float block_scale(float absmax) {
    const float s = __fdiv_rn(absmax, 448.f);
    return s == 0.f ? 1.f : s;
}

// x / scale from the correctly rounded reciprocal r = RN(1 / scale): one multiply, the
// remainder by FMA, one corrective FMA (the classical FMA division step).  Three instructions
// instead of the dozen of a general division, whose range handling is not needed here: scale is
// a normal number and |x / scale| <= 448.  The step reproduced the IEEE quotient on every one of
// 8e7 random (x, scale) pairs checked on the CPU; a last-bit difference could change the e4m3
// byte only on an exact rounding boundary, and the GPU tests compare every byte written with
// the CPU restatement's.
__device__ __forceinline__ float div_by_scale(float x, float scale, float r) {
    const float q = x * r;
    const float rem = fmaf(-q, scale, x);
    return fmaf(rem, r, q);
}

__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d, float scale) {
    const float r = __frcp_rn(scale);
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(div_by_scale(a, scale, r), div_by_scale(b, scale, r)), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(div_by_scale(c, scale, r), div_by_scale(d, scale, r)), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// ───────────────────────── HCA compressor ─────────────────────────

struct HcaCompressArgs {
    int B, n, n_blocks, c, m;
    const __nv_bfloat16* C;  const __nv_bfloat16* Z;  const __nv_bfloat16* bias;
    int64_t stride_b, stride_n;                 // element strides of C and Z
    __nv_bfloat16* out;                         // [B, n/m, c] or null
    int64_t stride_out_b, stride_out_blk;
    CacheDest dst;                              // dst.kv_pool null: no insert (insert needs c == 576)
};

constexpr int kHcaVecsPerBlock = 72;            // 72 x 8 = 576 channels
constexpr int kHcaRowGroups = 4;
constexpr int kHcaCompressThreads = kHcaVecsPerBlock * kHcaRowGroups;   // 288
constexpr int kHcaBatch = 4;                    // rows per online-softmax step

// One block per (request, output row, 576-channel slab).  Thread t owns the 8
// channels of vector t % 72 and the rows of row group t / 72 (a quarter of the m
// rows), which it folds four at a time into an online softmax state (running
// maximum, denominator, weighted sum); the four states of a channel are merged
// through shared memory by row group 0, which rounds to BF16, writes the dense
// output and - for the cache insert - quantises: 16 consecutive threads hold one
// 128-channel scale block, so its absolute maximum is four shuffles away.
__global__ void __launch_bounds__(kHcaCompressThreads, 2) hca_compress_kernel(const HcaCompressArgs a) {
    __shared__ float sm_m[kHcaRowGroups - 1][kHcaVecsPerBlock][8];
    __shared__ float sm_l[kHcaRowGroups - 1][kHcaVecsPerBlock][8];
    __shared__ float sm_acc[kHcaRowGroups - 1][kHcaVecsPerBlock][8];
    constexpr float kLog2e = 1.4426950408889634f;
    const int t = threadIdx.x;
    const int vl = t % kHcaVecsPerBlock, rg = t / kHcaVecsPerBlock;
    const int v = blockIdx.y * kHcaVecsPerBlock + vl;
    const int b = blockIdx.x / a.n_blocks, blk = blockIdx.x % a.n_blocks;
    const bool active = v * 8 < a.c;
    const int ch = v * 8;
    const int rows_per = (a.m + kHcaRowGroups - 1) / kHcaRowGroups;
    const int r0 = rg * rows_per, r1 = min(r0 + rows_per, a.m);

    // The running maximum starts at a large negative finite value instead of -inf, so that the
    // update below needs no special cases: with it every difference stays finite, a logit of -inf
    // gets weight zero, and a block whose logits are all -inf ends with a zero denominator (NaN
    // out, as in the reference's softmax).
    constexpr float kLowest = -1e30f;
    float mx[8], l[8], acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { mx[k] = kLowest;  l[k] = 0.f;  acc[k] = 0.f; }
    if (active) {
        const int64_t base = int64_t(b) * a.stride_b + int64_t(blk) * a.m * a.stride_n + ch;
        // one step = kHcaBatch rows; FULL: all of them exist (no per-row predicates in the code)
        auto step = [&](int r, auto full_tag) {
            constexpr bool FULL = decltype(full_tag)::value;
            uint4 zv[kHcaBatch], cv[kHcaBatch], bv[kHcaBatch];
#pragma unroll
            for (int j = 0; j < kHcaBatch; ++j) {
                if (FULL || r + j < r1) {
                    zv[j] = ptx::ldg_nc_v4(a.Z + base + int64_t(r + j) * a.stride_n);
                    cv[j] = ptx::ldg_nc_v4(a.C + base + int64_t(r + j) * a.stride_n);
                    bv[j] = __ldg(reinterpret_cast<const uint4*>(a.bias + int64_t(r + j) * a.c + ch));
                }
            }
            // The reference maximum of the step is found in packed BF16 arithmetic (one add and
            // one max per two elements): any value close to the true maximum serves, as long as
            // the same one is used for every weight of the step.  Only the raw vectors stay in
            // registers; the logits themselves are formed in FP32 below.
            __nv_bfloat162 pm[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) pm[k] = __float2bfloat162_rn(kLowest);
#pragma unroll
            for (int j = 0; j < kHcaBatch; ++j) {
                if (FULL || r + j < r1) {
                    const __nv_bfloat162* z2 = reinterpret_cast<const __nv_bfloat162*>(&zv[j]);
                    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&bv[j]);
#pragma unroll
                    for (int k = 0; k < 4; ++k) pm[k] = __hmax2(pm[k], __hadd2(z2[k], u2[k]));
                }
            }
            float nref[8];                       // -(new reference maximum) * log2(e)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float r_lo = fmaxf(mx[2 * k], __low2float(pm[k])), r_hi = fmaxf(mx[2 * k + 1], __high2float(pm[k]));
                const float a_lo = ptx::ex2((mx[2 * k] - r_lo) * kLog2e), a_hi = ptx::ex2((mx[2 * k + 1] - r_hi) * kLog2e);
                l[2 * k] *= a_lo;      acc[2 * k] *= a_lo;      mx[2 * k] = r_lo;      nref[2 * k] = -r_lo * kLog2e;
                l[2 * k + 1] *= a_hi;  acc[2 * k + 1] *= a_hi;  mx[2 * k + 1] = r_hi;  nref[2 * k + 1] = -r_hi * kLog2e;
            }
#pragma unroll
            for (int j = 0; j < kHcaBatch; ++j) {
                if (FULL || r + j < r1) {
                    float z[8], u[8], cf[8];
                    unpack8(zv[j], z);
                    unpack8(bv[j], u);
                    unpack8(cv[j], cf);
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float e = ptx::ex2(fmaf(z[k] + u[k], kLog2e, nref[k]));
                        l[k] += e;
                        acc[k] = fmaf(e, cf[k], acc[k]);
                    }
                }
            }
        };
        const int r_full = r0 + ((r1 - r0) / kHcaBatch) * kHcaBatch;
        for (int r = r0; r < r_full; r += kHcaBatch) step(r, std::true_type{});
        if (r_full < r1) step(r_full, std::false_type{});
    }
    if (rg > 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) { sm_m[rg - 1][vl][k] = mx[k];  sm_l[rg - 1][vl][k] = l[k];  sm_acc[rg - 1][vl][k] = acc[k]; }
    }
    __syncthreads();
    if (rg != 0) return;

    float o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float mm = mx[k];
#pragma unroll
        for (int g = 0; g < kHcaRowGroups - 1; ++g) mm = fmaxf(mm, sm_m[g][vl][k]);
        const float ref = mm;
        float w = ptx::ex2((mx[k] - ref) * kLog2e);
        float ls = l[k] * w, as = acc[k] * w;
#pragma unroll
        for (int g = 0; g < kHcaRowGroups - 1; ++g) {
            w = ptx::ex2((sm_m[g][vl][k] - ref) * kLog2e);
            ls = fmaf(sm_l[g][vl][k], w, ls);
            as = fmaf(sm_acc[g][vl][k], w, as);
        }
        o[k] = bf16_round_f(as / ls);
    }
    if (active && a.out != nullptr) {
        uint4 w;
        w.x = ptx::pack_bf16x2(o[0], o[1]);  w.y = ptx::pack_bf16x2(o[2], o[3]);
        w.z = ptx::pack_bf16x2(o[4], o[5]);  w.w = ptx::pack_bf16x2(o[6], o[7]);
        *reinterpret_cast<uint4*>(a.out + int64_t(b) * a.stride_out_b + int64_t(blk) * a.stride_out_blk + ch) = w;
    }
    if (a.dst.kv_pool == nullptr) return;
    // cache insert (c == 576, one slab): threads 0..63 hold the latent, 64..71 the RoPE tail
    uint8_t* entry = nullptr;
    if ((t & 31) == 0 || t >= 64) entry = entry_address(a.dst, b, int64_t(__ldg(a.dst.insert_pos + b)) + blk);
    if (t < 64) {
        entry = reinterpret_cast<uint8_t*>(__shfl_sync(0xFFFFFFFFu, reinterpret_cast<unsigned long long>(entry), 0));
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(o[k]));
#pragma unroll
        for (int d = 1; d < 16; d <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
        const float scale = block_scale(amax);
        if (entry != nullptr) {
            uint2 q;
            q.x = quant4(o[0], o[1], o[2], o[3], scale);
            q.y = quant4(o[4], o[5], o[6], o[7], scale);
            *reinterpret_cast<uint2*>(entry + t * 8) = q;
            if ((t & 15) == 0) *reinterpret_cast<float*>(entry + 512 + 4 * (t >> 4)) = scale;
        }
    } else if (entry != nullptr) {
        uint4 w;
        w.x = ptx::pack_bf16x2(o[0], o[1]);  w.y = ptx::pack_bf16x2(o[2], o[3]);
        w.z = ptx::pack_bf16x2(o[4], o[5]);  w.w = ptx::pack_bf16x2(o[6], o[7]);
        *reinterpret_cast<uint4*>(entry + 528 + (t - 64) * 16) = w;
    }
}

// ───────────────────────── quantise + insert ─────────────────────────

struct KvInsertArgs {
    int B, T;
    const __nv_bfloat16* rows;      // [B, T, 576]
    int64_t stride_b, stride_t;     // element strides
    const int32_t* n_rows;          // optional [B]: rows of request b that are inserted (<= T)
    CacheDest dst;
};

constexpr int kInsertThreads = 256;

// One warp per row: lane l owns latent elements [16 l, 16 l + 16) and RoPE
// elements [2 l, 2 l + 2); 8 lanes make one 128-element scale block.
__global__ void __launch_bounds__(kInsertThreads) kv_quantize_insert_kernel(const KvInsertArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t total = int64_t(a.B) * a.T;
    for (int64_t row = int64_t(blockIdx.x) * (kInsertThreads / 32) + (threadIdx.x >> 5); row < total;
         row += int64_t(gridDim.x) * (kInsertThreads / 32)) {
        const int b = int(row / a.T), t = int(row % a.T);
        if (a.n_rows != nullptr && t >= __ldg(a.n_rows + b)) continue;
        const __nv_bfloat16* src = a.rows + int64_t(b) * a.stride_b + int64_t(t) * a.stride_t;
        const uint4 x0 = ptx::ldg_nc_v4(src + 16 * lane);
        const uint4 x1 = ptx::ldg_nc_v4(src + 16 * lane + 8);
        const uint32_t rope = __ldg(reinterpret_cast<const uint32_t*>(src + 512 + 2 * lane));
        uint8_t* entry = nullptr;
        if (lane == 0) entry = entry_address(a.dst, b, int64_t(__ldg(a.dst.insert_pos + b)) + t);
        entry = reinterpret_cast<uint8_t*>(__shfl_sync(0xFFFFFFFFu, reinterpret_cast<unsigned long long>(entry), 0));
        float f[16];
        {
            float lo[8], hi[8];
            unpack8(x0, lo);
            unpack8(x1, hi);
#pragma unroll
            for (int k = 0; k < 8; ++k) { f[k] = lo[k];  f[8 + k] = hi[k]; }
        }
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < 16; ++k) amax = fmaxf(amax, fabsf(f[k]));
#pragma unroll
        for (int d = 1; d < 8; d <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
        const float scale = block_scale(amax);
        if (entry == nullptr) continue;
        uint4 q;
        q.x = quant4(f[0], f[1], f[2], f[3], scale);
        q.y = quant4(f[4], f[5], f[6], f[7], scale);
        q.z = quant4(f[8], f[9], f[10], f[11], scale);
        q.w = quant4(f[12], f[13], f[14], f[15], scale);
        *reinterpret_cast<uint4*>(entry + 16 * lane) = q;
        if ((lane & 7) == 0) *reinterpret_cast<float*>(entry + 512 + 4 * (lane >> 3)) = scale;
        *reinterpret_cast<uint32_t*>(entry + 528 + 4 * lane) = rope;
    }
}

}  // namespace dsv4

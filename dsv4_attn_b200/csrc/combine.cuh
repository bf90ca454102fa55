// LSE-weighted merge of split-KV partial outputs.  One warp per (row, head):
// the per-split log2 LSEs are reduced with warp shuffles, each lane then owns
// 2 x 8 consecutive value columns, reads partials with 128-bit loads (two splits
// in flight per lane, issued without waiting for the weights) and writes BF16 with
// 128-bit stores.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <math_constants.h>
#include <stdint.h>

#include "ptx.cuh"

namespace dsv4 {

struct CombineArgs {
    int N, H, num_splits;
    const float* partial_o;
    const float* partial_lse;
    __nv_bfloat16* out;
    float* lse;
    const float* attn_sink;
    int64_t stride_po_split, stride_po_n, stride_po_h;
    int64_t stride_pl_split, stride_pl_n;
    int64_t stride_out_n, stride_out_h;
    int64_t stride_lse_n;
    int partial_bf16;          // partial_o holds BF16 (strides then count BF16 elements): the library's own split path
    // Scheduled decode (sched.cuh): the pieces of unit (row, head group) lie in partial slots
    // unit_slot[u] .. + unit_nsplits[u] - 1, a slot being 128 head rows of 512 BF16 (and 128 LSEs); a unit
    // with one piece was written out by the decode kernel itself and is skipped here.
    const int32_t* unit_nsplits;
    const int32_t* unit_slot;
    int hgs;
};

constexpr int kCombineWarps = 8;
constexpr int kCombineMaxSplits = 1024;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

__global__ void __launch_bounds__(kCombineWarps * 32) combine_kernel(const CombineArgs a) {
    // When launched as a programmatic dependent of the decode kernel (same call, same stream) the blocks may
    // be resident before that kernel has finished: nothing is read before it has completed and its
    // writes are visible.  Returns at once in an ordinary launch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t unit = int64_t(blockIdx.x) * kCombineWarps + warp;   // (row, head) flattened
    if (unit >= int64_t(a.N) * a.H) return;
    const int n = int(unit / a.H), h = int(unit % a.H);
    int S = a.num_splits;
    const float* pl;
    int64_t pl_stride, po_off, po_stride;      // po_*: element offsets into partial_o (FP32 or BF16 elements)
    if (a.unit_nsplits != nullptr) {
        const int u = n * a.hgs + (h >> 7);
        S = __ldg(a.unit_nsplits + u);
        if (S <= 1) return;
        const int64_t row = int64_t(__ldg(a.unit_slot + u)) * 128 + (h & 127);
        pl = a.partial_lse + row;
        pl_stride = 128;
        po_off = row * 512 + lane * 8;
        po_stride = 128 * 512;
    } else {
        pl = a.partial_lse + int64_t(n) * a.stride_pl_n + h;
        pl_stride = a.stride_pl_split;
        po_off = int64_t(n) * a.stride_po_n + int64_t(h) * a.stride_po_h + lane * 8;
        po_stride = a.stride_po_split;
    }

    // pass 1: maximum and sum over splits.  The first 32 LSEs are loaded once (one per lane) and serve the maximum,
    // the sum and the weights; only rows with more than 32 splits go back to memory.
    const float l_first = (lane < S) ? __ldg(pl + int64_t(lane) * pl_stride) : -CUDART_INF_F;
    float mx = l_first;
    for (int s = lane + 32; s < S; s += 32) mx = fmaxf(mx, __ldg(pl + int64_t(s) * pl_stride));
    mx = warp_max(mx);
    float sum = 0.f;
    if (mx != -CUDART_INF_F) {
        sum = exp2f(l_first - mx);
        for (int s = lane + 32; s < S; s += 32) sum += exp2f(__ldg(pl + int64_t(s) * pl_stride) - mx);
    }
    sum = warp_sum(sum);
    const bool has = sum != 0.f;
    const float glse = has ? log2f(sum) + mx : -CUDART_INF_F;
    if (lane == 0 && a.lse != nullptr)
        a.lse[int64_t(n) * a.stride_lse_n + h] = has ? glse * 0.6931471805599453f : -CUDART_INF_F;
    float denom = glse;
    if (a.attn_sink != nullptr) {
        const float s2 = __ldg(a.attn_sink + h) * 1.4426950408889634f;
        denom = has ? glse + log2f(1.f + exp2f(s2 - glse)) : s2;
    }

    float acc[2][8];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;

    for (int s0 = 0; s0 < S; s0 += 32) {
        // each lane computes the weight of one split of this group; broadcast by shuffle
        float w_mine = 0.f;
        if (s0 + lane < S) {
            const float l = (s0 == 0) ? l_first : __ldg(pl + int64_t(s0 + lane) * pl_stride);
            w_mine = (l == -CUDART_INF_F || denom == -CUDART_INF_F) ? 0.f : exp2f(l - denom);
        }
        const int cnt = min(32, S - s0);
        // two splits at a time: their loads are issued before the first is used
        for (int k0 = 0; k0 < cnt; k0 += 2) {
            float w[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float x = __shfl_sync(0xFFFFFFFFu, w_mine, (k0 + j) & 31);
                w[j] = (k0 + j < cnt) ? x : 0.f;      // an empty split has weight 0: what its partial holds is loaded but not used
            }
            if (a.partial_bf16) {
                const __nv_bfloat16* sb = reinterpret_cast<const __nv_bfloat16*>(a.partial_o) + po_off + int64_t(s0 + k0) * po_stride;
                uint4 v[2][2];
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                        v[j][i] = __ldg(reinterpret_cast<const uint4*>(sb + int64_t(k0 + j < cnt ? j : 0) * po_stride + i * 256));
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        if (w[j] == 0.f) v[j][i] = make_uint4(0, 0, 0, 0);      // whatever an empty split's slot holds is discarded
                        const uint32_t u[4] = {v[j][i].x, v[j][i].y, v[j][i].z, v[j][i].w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            acc[i][2 * q] = fmaf(w[j], __uint_as_float(u[q] << 16), acc[i][2 * q]);
                            acc[i][2 * q + 1] = fmaf(w[j], __uint_as_float(u[q] & 0xFFFF0000u), acc[i][2 * q + 1]);
                        }
                    }
            } else {
                const float* src = a.partial_o + po_off + int64_t(s0 + k0) * po_stride;
                float4 v[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        // not predicated on the weight: the loads go out before the weights are known; what an
                        // empty split's slot holds is discarded below
                        const float4* q = reinterpret_cast<const float4*>(src + int64_t(k0 + j < cnt ? j : 0) * po_stride + i * 256);
                        v[j][2 * i] = __ldg(q);
                        v[j][2 * i + 1] = __ldg(q + 1);
                    }
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const bool use = w[j] != 0.f;
                        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                        const float4 v0 = use ? v[j][2 * i] : z, v1 = use ? v[j][2 * i + 1] : z;
                        acc[i][0] = fmaf(w[j], v0.x, acc[i][0]);  acc[i][1] = fmaf(w[j], v0.y, acc[i][1]);
                        acc[i][2] = fmaf(w[j], v0.z, acc[i][2]);  acc[i][3] = fmaf(w[j], v0.w, acc[i][3]);
                        acc[i][4] = fmaf(w[j], v1.x, acc[i][4]);  acc[i][5] = fmaf(w[j], v1.y, acc[i][5]);
                        acc[i][6] = fmaf(w[j], v1.z, acc[i][6]);  acc[i][7] = fmaf(w[j], v1.w, acc[i][7]);
                    }
            }
        }
    }
    __nv_bfloat16* dst = a.out + int64_t(n) * a.stride_out_n + int64_t(h) * a.stride_out_h + lane * 8;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 w;
        w.x = ptx::pack_bf16x2(acc[i][0], acc[i][1]);
        w.y = ptx::pack_bf16x2(acc[i][2], acc[i][3]);
        w.z = ptx::pack_bf16x2(acc[i][4], acc[i][5]);
        w.w = ptx::pack_bf16x2(acc[i][6], acc[i][7]);
        *reinterpret_cast<uint4*>(dst + i * 256) = w;
    }
}

}  // namespace dsv4

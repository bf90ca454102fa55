// Pre- and post-pass of the attention path: partial RoPE on the last n_rope
// dimensions of a vector (split-halves pairing: element i rotates with element
// i + n_rope/2), optionally followed by an RMS norm over the whole vector.  One
// kernel covers the three uses: queries before decode (RoPE by +position, then
// norm), new cache rows before they are quantised (the same with one vector per
// position) and the attention output afterwards (RoPE by -position, no norm).
//
// One warp per vector.  The vector is read once (16-byte loads for the part that
// is only normalised, one rotated pair per lane), kept in registers, and written
// once.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "ptx.cuh"
#include "compress_reduce.cuh"   // unpack8

namespace dsv4 {

struct RopeNormArgs {
    int64_t n_rows;            // positions
    int vecs_per_row;          // vectors that share a position (heads)
    int c;                     // vector width; c - n_rope is a multiple of 8 and at most 512
    int n_rope;                // 64
    int inverse;               // rotate by -position
    float eps, theta;
    const __nv_bfloat16* x;
    __nv_bfloat16* out;        // may alias x
    const int32_t* positions;  // [n_rows]
    const __nv_bfloat16* weight;   // [c] or null: no norm
};

constexpr int kRopeNormThreads = 256;
constexpr int kRopeGroup = 4;           // vectors of one row handled by one warp

__global__ void __launch_bounds__(kRopeNormThreads) rope_norm_kernel(const RopeNormArgs a) {
    const int lane = threadIdx.x & 31;
    const int nope = a.c - a.n_rope;
    const int half = a.n_rope >> 1;        // 32: one rotated pair per lane
    // frequency of this lane's pair, 1 / theta^(2 i / n_rope): once per thread, not per vector
    const float freq = (lane < half) ? float(1.0 / pow(double(a.theta), double(2 * lane) / double(a.n_rope))) : 0.f;
    // A warp takes up to kRopeGroup vectors of one row in turn: they share the position, so the sine
    // and cosine are computed once for them.
    const int groups_per_row = (a.vecs_per_row + kRopeGroup - 1) / kRopeGroup;
    const int64_t n_items = a.n_rows * groups_per_row;
    for (int64_t item = int64_t(blockIdx.x) * (kRopeNormThreads / 32) + (threadIdx.x >> 5); item < n_items;
         item += int64_t(gridDim.x) * (kRopeNormThreads / 32)) {
      const int64_t row = item / groups_per_row;
      const int vec0 = int(item % groups_per_row) * kRopeGroup;
      float sn = 0.f, cs = 1.f;
      if (lane < half) {
          // the angle in FP32 as the reference forms it
          const float pos = float(__ldg(a.positions + row));
          sincosf((a.inverse ? -pos : pos) * freq, &sn, &cs);
      }
      for (int j = 0; j < kRopeGroup && vec0 + j < a.vecs_per_row; ++j) {
        const int64_t v = row * a.vecs_per_row + vec0 + j;
        const __nv_bfloat16* src = a.x + v * a.c;
        __nv_bfloat16* dst = a.out + v * a.c;
        // elements [16 lane, 16 lane + 16) of the part that is not rotated, in two 16-byte halves
        float f[16];
        bool have[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int e0 = 16 * lane + 8 * h;
            have[h] = e0 < nope;
            if (have[h]) {
                float t[8];
                unpack8(ptx::ldg_nc_v4(src + e0), t);
#pragma unroll
                for (int k = 0; k < 8; ++k) f[8 * h + k] = t[k];
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) f[8 * h + k] = 0.f;
            }
        }
        // the rotated pair (lane, lane + half)
        float x1 = 0.f, x2 = 0.f;
        if (lane < half) {
            x1 = __bfloat162float(src[nope + lane]);
            x2 = __bfloat162float(src[nope + half + lane]);
            const float r1 = x1 * cs - x2 * sn;
            const float r2 = x1 * sn + x2 * cs;
            x1 = r1;  x2 = r2;
        }
        if (a.weight != nullptr) {
            float ss = x1 * x1 + x2 * x2;
#pragma unroll
            for (int k = 0; k < 16; ++k) ss = fmaf(f[k], f[k], ss);
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, d);
            // x / rms * w as x * (1 / rms) * w: the difference is far below the BF16 rounding of the result
            const float inv_rms = 1.f / sqrtf(ss / float(a.c) + a.eps);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (have[h]) {
                    float w[8];
                    unpack8(__ldg(reinterpret_cast<const uint4*>(a.weight + 16 * lane + 8 * h)), w);
#pragma unroll
                    for (int k = 0; k < 8; ++k) f[8 * h + k] = f[8 * h + k] * inv_rms * w[k];
                }
            }
            if (lane < half) {
                x1 = x1 * inv_rms * __bfloat162float(a.weight[nope + lane]);
                x2 = x2 * inv_rms * __bfloat162float(a.weight[nope + half + lane]);
            }
        }
        // without a norm the part that is not rotated is unchanged: written only when out is another buffer
        if (a.weight != nullptr || dst != src) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (have[h]) {
                    uint4 w;
                    w.x = ptx::pack_bf16x2(f[8 * h + 0], f[8 * h + 1]);  w.y = ptx::pack_bf16x2(f[8 * h + 2], f[8 * h + 3]);
                    w.z = ptx::pack_bf16x2(f[8 * h + 4], f[8 * h + 5]);  w.w = ptx::pack_bf16x2(f[8 * h + 6], f[8 * h + 7]);
                    *reinterpret_cast<uint4*>(dst + 16 * lane + 8 * h) = w;
                }
            }
        }
        if (lane < half) {
            dst[nope + lane] = __float2bfloat16_rn(x1);
            dst[nope + half + lane] = __float2bfloat16_rn(x2);
        }
      }
    }
}

}  // namespace dsv4

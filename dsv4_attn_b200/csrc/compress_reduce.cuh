// CSA compressor, second pass: per output block and channel, a softmax over the
// 2m gating logits (m of the block's own rows on the a-side, m rows of the
// previous block on the b-side, each plus a per-position bias) weights the 2m
// value rows.  A pure streaming kernel: every input element is read once with
// vector loads, one thread owns 4 consecutive channels of one output block (8-byte loads: a
// thread then holds 16 vectors = 32 registers of raw data, four blocks fit an SM, and the 32
// resident warps hide each other's arithmetic phase; with 8 channels per thread and two blocks
// per SM the kernel was 7 % slower, with 2 channels and five blocks 30 % slower), and the grid
// is sized so that all SMs hold two waves of resident blocks.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <math_constants.h>
#include <stdint.h>

#include "ptx.cuh"

namespace dsv4 {

struct CompressReduceArgs {
    int B, n, n_blocks, c_out, m;
    const __nv_bfloat16* C_a;  const __nv_bfloat16* C_b;
    const __nv_bfloat16* Z_a;  const __nv_bfloat16* Z_b;
    const __nv_bfloat16* B_a;  const __nv_bfloat16* B_b;
    __nv_bfloat16* out;
    int64_t stride_c_b, stride_c_n;        // element strides of the four input streams
    int64_t stride_out_b, stride_out_blk;
};

constexpr int kCompressThreads = 256;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}

// Vector of VEC BF16 values and its FP32 unpacking: 16-byte vectors for VEC = 8, 8-byte for VEC = 4.
template <int VEC> struct BfVec;
template <> struct BfVec<8> {
    using T = uint4;
    static __device__ __forceinline__ T load_stream(const __nv_bfloat16* p) { return ptx::ldg_nc_v4(p); }
    static __device__ __forceinline__ void unpack(const T& v, float (&f)[8]) { unpack8(v, f); }
};
template <> struct BfVec<4> {
    using T = uint2;
    static __device__ __forceinline__ T load_stream(const __nv_bfloat16* p) {
        T v;
        asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
        return v;
    }
    static __device__ __forceinline__ void unpack(const T& v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x << 16);  f[1] = __uint_as_float(v.x & 0xFFFF0000u);
        f[2] = __uint_as_float(v.y << 16);  f[3] = __uint_as_float(v.y & 0xFFFF0000u);
    }
};

// VEC = 8 / 4: 16- / 8-byte vectors (c_out % VEC == 0 and rows aligned to the vector); VEC = 1: any c_out.
template <int M, int VEC>
__global__ void __launch_bounds__(kCompressThreads, VEC == 4 ? 4 : 2) compress_reduce_kernel(const CompressReduceArgs a) {
    const int vecs = a.c_out / VEC;
    const int64_t total = int64_t(a.B) * a.n_blocks * vecs;
    for (int64_t idx = int64_t(blockIdx.x) * kCompressThreads + threadIdx.x; idx < total;
         idx += int64_t(gridDim.x) * kCompressThreads) {
        const int v = int(idx % vecs);
        const int64_t bb = idx / vecs;
        const int blk = int(bb % a.n_blocks);
        const int b = int(bb / a.n_blocks);
        const int ch = v * VEC;
        const int64_t row_a = int64_t(b) * a.stride_c_b + int64_t(blk) * M * a.stride_c_n + ch;
        const int64_t row_b = row_a - int64_t(M) * a.stride_c_n;      // previous block (blk > 0 only)
        float o[VEC];
        if constexpr (VEC >= 4) {
            using V = typename BfVec<VEC>::T;
            // all 4m data vectors in flight first; the biases are small and cached, they are
            // re-read where needed so that the raw data can stay in registers
            V za[M], ca[M], zb[M], cb[M];
#pragma unroll
            for (int j = 0; j < M; ++j) {
                za[j] = BfVec<VEC>::load_stream(a.Z_a + row_a + j * a.stride_c_n);
                ca[j] = BfVec<VEC>::load_stream(a.C_a + row_a + j * a.stride_c_n);
            }
            const bool has_b = blk > 0;
            if (has_b) {
#pragma unroll
                for (int j = 0; j < M; ++j) {
                    zb[j] = BfVec<VEC>::load_stream(a.Z_b + row_b + j * a.stride_c_n);
                    cb[j] = BfVec<VEC>::load_stream(a.C_b + row_b + j * a.stride_c_n);
                }
            }
            auto logits = [&](int j, bool bside, float (&z)[VEC]) {
                float u[VEC];
                BfVec<VEC>::unpack(bside ? zb[j] : za[j], z);
                BfVec<VEC>::unpack(__ldg(reinterpret_cast<const V*>((bside ? a.B_b : a.B_a) + int64_t(j) * a.c_out + ch)), u);
#pragma unroll
                for (int k = 0; k < VEC; ++k) z[k] += u[k];
            };
            float zmax[VEC], sum[VEC], acc[VEC];
#pragma unroll
            for (int k = 0; k < VEC; ++k) { zmax[k] = -CUDART_INF_F;  sum[k] = 0.f;  acc[k] = 0.f; }
#pragma unroll
            for (int side = 0; side < 2; ++side) {
                if (side == 1 && !has_b) break;
#pragma unroll
                for (int j = 0; j < M; ++j) {
                    float z[VEC];
                    logits(j, side == 1, z);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) zmax[k] = fmaxf(zmax[k], z[k]);
                }
            }
#pragma unroll
            for (int k = 0; k < VEC; ++k)
                if (!(zmax[k] > -CUDART_INF_F) || !(zmax[k] < CUDART_INF_F)) zmax[k] = 0.f;   // all -inf (or NaN): avoid inf - inf
#pragma unroll
            for (int side = 0; side < 2; ++side) {
                if (side == 1 && !has_b) break;
#pragma unroll
                for (int j = 0; j < M; ++j) {
                    float z[VEC], c[VEC];
                    logits(j, side == 1, z);
                    BfVec<VEC>::unpack(side == 1 ? cb[j] : ca[j], c);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) {
                        const float e = ptx::ex2((z[k] - zmax[k]) * 1.4426950408889634f);
                        sum[k] += e;
                        acc[k] = fmaf(e, c[k], acc[k]);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < VEC; ++k) o[k] = acc[k] / sum[k];
        } else {
            float z[2 * M], c[2 * M];
#pragma unroll
            for (int j = 0; j < M; ++j) {
                z[j] = __bfloat162float(a.Z_a[row_a + j * a.stride_c_n]) + __bfloat162float(a.B_a[int64_t(j) * a.c_out + ch]);
                c[j] = __bfloat162float(a.C_a[row_a + j * a.stride_c_n]);
                if (blk > 0) {
                    z[M + j] = __bfloat162float(a.Z_b[row_b + j * a.stride_c_n]) + __bfloat162float(a.B_b[int64_t(j) * a.c_out + ch]);
                    c[M + j] = __bfloat162float(a.C_b[row_b + j * a.stride_c_n]);
                } else {
                    z[M + j] = -CUDART_INF_F;
                    c[M + j] = 0.f;
                }
            }
            float zmax = z[0];
#pragma unroll
            for (int j = 1; j < 2 * M; ++j) zmax = fmaxf(zmax, z[j]);
            if (!(zmax > -CUDART_INF_F) || !(zmax < CUDART_INF_F)) zmax = 0.f;
            float sum = 0.f, acc = 0.f;
#pragma unroll
            for (int j = 0; j < 2 * M; ++j) {
                const float e = ptx::ex2((z[j] - zmax) * 1.4426950408889634f);
                sum += e;
                acc = fmaf(e, c[j], acc);
            }
            o[0] = acc / sum;
        }
        __nv_bfloat16* dst = a.out + int64_t(b) * a.stride_out_b + int64_t(blk) * a.stride_out_blk + ch;
        if constexpr (VEC == 8) {
            uint4 w;
            w.x = ptx::pack_bf16x2(o[0], o[1]);  w.y = ptx::pack_bf16x2(o[2], o[3]);
            w.z = ptx::pack_bf16x2(o[4], o[5]);  w.w = ptx::pack_bf16x2(o[6], o[7]);
            *reinterpret_cast<uint4*>(dst) = w;
        } else if constexpr (VEC == 4) {
            uint2 w;
            w.x = ptx::pack_bf16x2(o[0], o[1]);  w.y = ptx::pack_bf16x2(o[2], o[3]);
            *reinterpret_cast<uint2*>(dst) = w;
        } else {
            dst[0] = __float2bfloat16_rn(o[0]);
        }
    }
}

}  // namespace dsv4

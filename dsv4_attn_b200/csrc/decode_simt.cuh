// Plain-SIMT validation kernel for decode attention: one thread block per
// (row, head), FP32 arithmetic, exact FP8 * scale dequantisation, no tensor
// cores and no splitting.  It exists to cross-check the tensor-core kernel on
// the device at sizes the CPU oracle cannot cover quickly; it is not a product
// path.
#pragma once

#include "decode_kernel.cuh"

namespace dsv4 {

constexpr int kSimtThreads = 128;

struct RowRef {
    const uint8_t* lat;       // FP8 latent
    const uint8_t* scale;     // 4 x float (packed layout) or 7 x UE8M0 (reference layout)
    const uint8_t* rope;      // 64 x bf16
    bool valid;
};

template <int SRC>
__device__ __forceinline__ RowRef resolve_row(const DecodeArgs& a, int b, int n, int v, int n_tok, int kv_len_n) {
    RowRef r{nullptr, nullptr, nullptr, false};
    if (v >= n_tok) return r;
    if constexpr (SRC == kSrcCsa) {
        const int e = a.indices[int64_t(n) * a.topk + v];
        if (e < 0 || e >= kv_len_n || (e >> 6) >= a.max_pages) return r;
        const int page = a.block_table[int64_t(b) * a.max_pages + (e >> 6)];
        if (page < 0 || (long long)page >= a.num_pages) return r;     // same rule as the tensor-core kernel: left out, not read
        const uint8_t* row = a.kv_pool + (int64_t(page) * 64 + (e & 63)) * 656;
        r = RowRef{row, row + 512, row + 528, true};
    } else if constexpr (SRC == kSrcHca) {
        const uint8_t* row;
        if (v < kv_len_n) {
            if ((v >> 6) >= a.max_pages) return r;
            const int page = a.block_table[int64_t(b) * a.max_pages + (v >> 6)];
            if (page < 0 || (long long)page >= a.num_pages) return r;
            row = a.kv_pool + (int64_t(page) * 64 + (v & 63)) * 656;
        } else {
            if (v - kv_len_n >= a.win_cap) return r;
            row = a.win_pool + (int64_t(b) * a.win_cap + (v - kv_len_n)) * 656;
        }
        r = RowRef{row, row + 512, row + 528, true};
    } else {
        if (v < a.ref_m_cur) {
            const int64_t e = int64_t(b) * a.ref_m_cur + v;
            r = RowRef{a.ref_kc + e * 448, a.ref_kc_s + e * 7,
                       reinterpret_cast<const uint8_t*>(a.ref_kc_rope + e * 64), true};
        } else {
            const int64_t e = int64_t(b) * a.ref_swa_len + (v - a.ref_m_cur);
            r = RowRef{a.ref_ks + e * 448, a.ref_ks_s + e * 7,
                       reinterpret_cast<const uint8_t*>(a.ref_ks_rope + e * 64), true};
        }
    }
    return r;
}

__device__ __forceinline__ float fp8_to_f32(uint8_t x) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(x), __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}

// Dequantised element d of a row; d in [0, latent + 64).
template <int SRC>
__device__ __forceinline__ float row_value(const RowRef& r, int d) {
    constexpr int kLat = (SRC == kSrcRef) ? 448 : 512;
    if (d < kLat) {
        float s;
        if constexpr (SRC == kSrcRef) s = __uint_as_float(uint32_t(r.scale[d >> 6]) << 23);
        else s = reinterpret_cast<const float*>(r.scale)[d >> 7];
        return fp8_to_f32(r.lat[d]) * s;
    }
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(r.rope)[d - kLat]);
}

template <int SRC>
__global__ void __launch_bounds__(kSimtThreads) decode_simt_kernel(const DecodeArgs a) {
    constexpr int kLat = (SRC == kSrcRef) ? 448 : 512;
    constexpr int kDqk = kLat + 64;
    extern __shared__ float simt_smem[];
    float* qs = simt_smem;              // [kDqk]
    float* red = qs + kDqk;             // [kSimtThreads]
    float* logit = red + kSimtThreads;  // [n_tok]
    const int n = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int b = n / a.s_q;
    int n_tok, kv_len_n;
    if constexpr (SRC == kSrcCsa) {
        n_tok = a.topk_len ? min(max(a.topk_len[n], 0), a.topk) : a.topk;
        kv_len_n = a.kv_len ? a.kv_len[n] : 0x7FFFFFFF;
    } else if constexpr (SRC == kSrcHca) {
        kv_len_n = max(a.kv_len[n], 0);
        n_tok = kv_len_n + max(a.win_len[n], 0);
    } else {
        kv_len_n = a.ref_m_cur;
        n_tok = a.ref_m_cur + a.ref_swa_len;
    }
    const __nv_bfloat16* q = a.q + (int64_t(n) * a.H + h) * kDqk;
    for (int d = tid; d < kDqk; d += kSimtThreads) qs[d] = __bfloat162float(q[d]);
    __syncthreads();

    float lmax = -CUDART_INF_F;
    for (int v = tid; v < n_tok; v += kSimtThreads) {
        const RowRef r = resolve_row<SRC>(a, b, n, v, n_tok, kv_len_n);
        float x = -CUDART_INF_F;
        if (r.valid) {
            float acc = 0.f;
            for (int d = 0; d < kDqk; ++d) acc = fmaf(qs[d], row_value<SRC>(r, d), acc);
            x = acc * a.scale_log2;
        }
        logit[v] = x;
        lmax = fmaxf(lmax, x);
    }
    red[tid] = lmax;
    __syncthreads();
    for (int s = kSimtThreads / 2; s > 0; s >>= 1) {
        if (tid < s) red[tid] = fmaxf(red[tid], red[tid + s]);
        __syncthreads();
    }
    lmax = red[0];
    __syncthreads();
    const float m_use = (lmax == -CUDART_INF_F) ? 0.f : lmax;
    float lsum = 0.f;
    for (int v = tid; v < n_tok; v += kSimtThreads) {
        const float p = exp2f(logit[v] - m_use);
        logit[v] = p;
        lsum += p;
    }
    red[tid] = lsum;
    __syncthreads();
    for (int s = kSimtThreads / 2; s > 0; s >>= 1) {
        if (tid < s) red[tid] += red[tid + s];
        __syncthreads();
    }
    lsum = red[0];

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int v = 0; v < n_tok; ++v) {
        const float p = logit[v];
        if (p == 0.f) continue;
        const RowRef r = resolve_row<SRC>(a, b, n, v, n_tok, kv_len_n);
        if (!r.valid) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = fmaf(p, row_value<SRC>(r, tid * 4 + i), acc[i]);
    }
    float denom = lsum;
    if (a.attn_sink != nullptr && lsum > 0.f) denom += exp2f(a.attn_sink[h] * 1.4426950408889634f - lmax);
    const float inv = lsum > 0.f ? 1.f / denom : 0.f;
    __nv_bfloat16* o = a.out + (int64_t(n) * a.H + h) * 512 + tid * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __float2bfloat16_rn(acc[i] * inv);
    if (tid == 0 && a.lse != nullptr)
        a.lse[int64_t(n) * a.H + h] = lsum > 0.f ? (lmax + log2f(lsum)) * 0.6931471805599453f : -CUDART_INF_F;
}

}  // namespace dsv4

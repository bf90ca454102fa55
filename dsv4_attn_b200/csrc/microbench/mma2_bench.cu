// Microbenchmark: tcgen05.mma.cta_group::2 (one instruction spanning the two SMs of a cluster
// pair) - cycles per instruction for the shapes a paired decode kernel would use.  Operands are
// zero-filled shared memory / tensor memory: only the timing is looked at.
#include <cstdio>
#include <cuda_runtime.h>
#include "../ptx.cuh"
using namespace dsv4;

__device__ __forceinline__ void tmem_alloc2(uint32_t dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma2_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t"
        "}\n" ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma2_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n\t"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma2_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct Mode { int M, N, ts, bmn; const char* name; };

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) k(int M, int N, int ts, int bmn, int iters, long long* out, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_base;
    const int warp = threadIdx.x >> 5;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    if (threadIdx.x == 0) { ptx::mbar_init(ptx::smem_u32(&bar), 1); ptx::fence_mbar_init(); }
    for (uint32_t i = threadIdx.x; i < 160 * 1024 / 16; i += 128) ptx::sts_v4(base + i * 16, make_uint4(0, 0, 0, 0));
    ptx::fence_proxy_async_smem();
    ptx::cluster_sync();
    if (warp == 0) { tmem_alloc2(ptx::smem_u32(&tmem_base), 512); tmem_relinquish2(); }
    ptx::tc_fence_before_sync();
    ptx::cluster_sync();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = tmem_base;
    if (rank == 0 && threadIdx.x == 0) {
        const uint32_t idesc = ptx::make_idesc_bf16(M, N, false, bmn != 0);
        const uint32_t hi = ptx::smem_desc_hi(1024);
        const uint32_t a_lo0 = ptx::smem_desc_lo(base, 16);
        // B per SM: N/2 rows (K-major) or N/2 columns (MN-major, 64-column chunks 8 KB apart at 64 K-rows)
        const uint32_t b_lo0 = bmn ? ptx::smem_desc_lo(base + 64 * 1024, 8192) : ptx::smem_desc_lo(base + 64 * 1024, 16);
        long long t0 = clock64();
        for (int i = 0; i < iters; i += 16) {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int k4 = u & 3, c = (u >> 2) & 3;
                const uint32_t a_lo = a_lo0 + ((c * 16384 + k4 * 32) >> 4);
                const uint32_t b_lo = bmn ? b_lo0 + ((k4 * 2048) >> 4) : b_lo0 + ((c * (64 * 128) + k4 * 32) >> 4);
                if (ts) mma2_ts(tmem, tmem + 256 + c * 32 + k4 * 8, b_lo, hi, idesc, (i | u) ? 1u : 0u);
                else mma2_ss(tmem, a_lo, b_lo, hi, idesc, (i | u) ? 1u : 0u);
            }
        }
        long long t1 = clock64();
        mma2_commit(ptx::smem_u32(&bar));
        if (!ptx::mbar_wait(ptx::smem_u32(&bar), 0, 2000000000ull)) *status = 1;
        long long t2 = clock64();
        if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
    }
    ptx::tc_fence_before_sync();
    ptx::cluster_sync();
    if (warp == 0) { ptx::tc_fence_after_sync(); tmem_dealloc2(tmem, 512); }
}

int main() {
    long long* out; int* status;
    cudaMallocManaged(&out, 16); cudaMallocManaged(&status, 4); *status = 0;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const Mode modes[] = {
        {128, 64, 0, 0, "M128 N64 ss"},   {128, 128, 0, 0, "M128 N128 ss"}, {128, 112, 0, 0, "M128 N112 ss"},
        {128, 128, 1, 0, "M128 N128 ts"}, {128, 256, 0, 1, "M128 N256 ss Bmn"}, {128, 256, 1, 1, "M128 N256 ts Bmn"},
        {256, 64, 0, 0, "M256 N64 ss"},   {256, 128, 0, 0, "M256 N128 ss"}, {256, 128, 1, 0, "M256 N128 ts"},
        {256, 256, 0, 1, "M256 N256 ss Bmn"}, {256, 256, 1, 1, "M256 N256 ts Bmn"},
    };
    for (const Mode& m : modes) {
        const int iters = 512;
        out[0] = out[1] = 0;
        k<<<148, 128, 200 * 1024>>>(m.M, m.N, m.ts, m.bmn, iters, out, status);
        cudaError_t e = cudaDeviceSynchronize();
        printf("2-SM %-18s issue %6.1f clk/mma  total %6.1f clk/mma  (err %d status %d)\n", m.name,
               double(out[0]) / iters, double(out[1]) / iters, int(e), *status);
        if (e != cudaSuccess) break;
    }
    return 0;
}

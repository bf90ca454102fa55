// Microbenchmark: tcgen05.mma throughput for the shapes the decode kernel uses.
#include <cstdio>
#include <cuda_runtime.h>
#include "../ptx.cuh"
using namespace dsv4;

// M = 128 or 64 rows.  mode: 0 = ss N=64, 1 = ts N=64, 2 = ss N=128, 3 = ts N=128, 4 = ss N=256 (B mn-major), 5 = ts N=256, 6 = ss N=256 k-major
__global__ void __launch_bounds__(128, 1) k(int mode, int iters, long long* out, int* status, int sep, int M) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_base;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) { ptx::mbar_init(ptx::smem_u32(&bar), 1); ptx::fence_mbar_init(); }
    if (warp == 0) { ptx::tmem_alloc(ptx::smem_u32(&tmem_base), 512); ptx::tmem_relinquish(); }
    // zero smem operands (160 KB)
    for (uint32_t i = threadIdx.x; i < 160 * 1024 / 16; i += 128) ptx::sts_v4(base + i * 16, make_uint4(0, 0, 0, 0));
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = tmem_base;
    if (threadIdx.x == 0) {
        const int N = (mode < 2) ? 64 : (mode < 4 ? 128 : 256);
        const bool ts = mode & 1;
        const bool bmn = (mode == 4 || mode == 5);
        const uint32_t idesc = ptx::make_idesc_bf16(M, N, false, bmn);
        const uint32_t hi = ptx::smem_desc_hi(1024);
        const uint32_t a_lo0 = ptx::smem_desc_lo(base, 16);
        const uint32_t b_lo0 = bmn ? ptx::smem_desc_lo(base + 64 * 1024, 8192) : ptx::smem_desc_lo(base + 64 * 1024, 16);
        long long t0 = clock64();
        for (int i = 0; i < iters; i += 16) {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int k4 = u & 3, c = (u >> 2) & 3;
                const uint32_t a_lo = a_lo0 + ((c * 16384 + k4 * 32) >> 4);
                const uint32_t b_lo = bmn ? b_lo0 + ((k4 * 2048) >> 4) : b_lo0 + ((c * (64 * 128) + k4 * 32) >> 4);
                if (ts) ptx::mma_bf16_ts2(tmem + (sep ? u * 16 : 0), tmem + 256 + c * 32 + k4 * 8, b_lo, hi, idesc, (i | u) ? 1u : 0u);
                else ptx::mma_bf16_ss2(tmem + (sep ? (u & 1) * 256 : 0), a_lo, b_lo, hi, idesc, (i | u) ? 1u : 0u);
            }
        }
        long long t1 = clock64();
        ptx::mma_commit(ptx::smem_u32(&bar));
        if (!ptx::mbar_wait(ptx::smem_u32(&bar), 0, 2000000000ull)) *status = 1;
        long long t2 = clock64();
        if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) { ptx::tc_fence_after_sync(); ptx::tmem_dealloc(tmem, 512); }
}

int main() {
    long long* out; int* status;
    cudaMallocManaged(&out, 16); cudaMallocManaged(&status, 4); *status = 0;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const char* names[] = {"ss N=64", "ts N=64", "ss N=128", "ts N=128", "ss N=256 Bmn", "ts N=256 Bmn", "ss N=256 Bk"};
    for (int M : {128, 64}) for (int sepv : {0, 1}) for (int grid : {148}) for (int mode = 0; mode < 7; ++mode) {
        if (sepv && mode >= 2) continue;
        const int iters = 512;
        k<<<grid, 128, 200 * 1024>>>(mode, iters, out, status, sepv, M);
        cudaError_t e = cudaDeviceSynchronize();
        printf("M %3d sep %d grid %3d %-14s issue %6.1f clk/mma  total %6.1f clk/mma  (err %d status %d)\n", M, sepv, grid, names[mode],
               double(out[0]) / iters, double(out[1]) / iters, int(e), *status);
    }
    return 0;
}

// Microbenchmark: exchange of 32 KB between the two blocks of a cluster pair.
#include <cstdio>
#include <cuda_runtime.h>
#include "../ptx.cuh"
using namespace dsv4;

// mode 0: 16 x st.shared::cluster.v4 per thread + per-thread release arrive
// mode 1: same stores + fence.acq_rel.cluster + warp arrive
// mode 2: st.async (complete_tx) 16 x 16 B per thread, receiver arms expect_tx
// mode 3: local st to staging + one cp.async.bulk (8 KB) per warp to the peer, complete_tx on peer barrier
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) k(int mode, int iters, long long* out, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    __shared__ uint64_t bar[2];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = blockIdx.x & 1, peer = rank ^ 1;
    const uint32_t xbuf = base;                // incoming [2][32 KB]
    const uint32_t stg = base + 65536;         // outgoing staging 32 KB
    if (tid == 0) {
        for (int b = 0; b < 2; ++b) ptx::mbar_init(ptx::smem_u32(&bar[b]), mode == 0 ? 128 : (mode == 1 ? 4 : 1));
        ptx::fence_mbar_init();
    }
    ptx::cluster_sync();
    const uint32_t my_row_peer = ptx::mapa(xbuf + tid * 16, peer);
    const uint32_t bar_peer = ptx::mapa(ptx::smem_u32(&bar[0]), peer);
    uint4 v = make_uint4(tid, 1, 2, 3);
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
        const int b = it & 1;
        const uint32_t par = (it >> 1) & 1;
        if (mode == 0 || mode == 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) ptx::sts_cluster_v4(my_row_peer + b * 32768 + j * 2048, v);
            if (mode == 0) ptx::mbar_arrive_cluster(bar_peer + 8 * b);
            else { ptx::fence_acq_rel_cluster(); __syncwarp(); if (lane == 0) ptx::mbar_arrive_cluster(bar_peer + 8 * b); }
        } else if (mode == 2) {
            if (tid == 0) ptx::mbar_arrive_expect_tx(ptx::smem_u32(&bar[b]), 32768);
#pragma unroll
            for (int j = 0; j < 16; ++j)
                asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                             :: "r"(my_row_peer + b * 32768 + j * 2048), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"(bar_peer + 8 * b) : "memory");
        } else {
            if (tid == 0) ptx::mbar_arrive_expect_tx(ptx::smem_u32(&bar[b]), 32768);
#pragma unroll
            for (int j = 0; j < 16; ++j) ptx::sts_v4(stg + warp * 8192 + j * 512 + lane * 16, v);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             :: "r"(ptx::mapa(xbuf + b * 32768 + warp * 8192, peer)), "r"(stg + warp * 8192), "r"(8192), "r"(bar_peer + 8 * b) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            }
            __syncwarp();
        }
        if (!ptx::mbar_wait_cluster(ptx::smem_u32(&bar[b]), par, 1000000000ull)) { *status = 1 + it; break; }
        uint4 r = ptx::lds_v4(xbuf + b * 32768 + tid * 16);
        v.x += r.x;
    }
    long long t1 = clock64();
    if (tid == 0 && blockIdx.x == 0) { out[0] = t1 - t0; out[1] = v.x; }
    ptx::cluster_sync();
}

int main() {
    long long* out; int* status;
    cudaMallocManaged(&out, 16); cudaMallocManaged(&status, 4);
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
    const char* names[] = {"st.cluster + 128 arrives", "st.cluster + fence + 4 arrives", "st.async complete_tx", "bulk copy per warp"};
    for (int mode = 0; mode < 4; ++mode) {
        *status = 0;
        const int iters = 200;
        k<<<2, 128, 120 * 1024>>>(mode, iters, out, status);
        cudaError_t e = cudaDeviceSynchronize();
        printf("%-32s %8.1f clk/exchange  (err %d status %d)\n", names[mode], double(out[0]) / iters, int(e), *status);
    }
    return 0;
}

// Microbenchmark: how fast one SM can pull 656-byte cache records into registers.
//
// Every block plays the loader warps of the decode kernel: per "tile" each warp
// reads RECS_PER_WARP records (one per lane group) with 16-byte loads, K loads per
// thread, all independent, then consumes them.  Reported per configuration:
//   issue    = cycles until the last load instruction has been issued
//   complete = cycles until all loaded values have been consumed
// for cold data (first touch after a flush of L2) and for data resident in L2.
//
// shape 0: lane/4 = record (8 per warp), lane%4 = 16-byte piece, load c at +64c   (64 B per record per load)
// shape 1: lane/8 = record (4 per warp), lane%8 = 16-byte piece, load c at +128c  (128 B per record per load)
// shape 2: one record per load instruction, lane = 16-byte piece of 512 contiguous bytes
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ long long clk() {
    long long c;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(c) :: "memory");
    return c;
}

template <int K, int SHAPE>
__global__ void __launch_bounds__(512, 1) gather(const uint8_t* pool, long long n_rec, int tiles, long long* out, uint32_t* sink) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    uint32_t acc = 0;
    long long issue = 0, complete = 0;
    for (int t = 0; t < tiles; ++t) {
        // records spread over the pool like pages behind a shuffled block table
        const long long slot = (long long)(blockIdx.x * tiles + t) * nwarps + warp;
        const uint8_t* p;
        if (SHAPE == 0) {
            const long long rec = (slot * 8 + (lane >> 2)) * 7919 % n_rec;
            p = pool + rec * 656 + (lane & 3) * 16;
        } else if (SHAPE == 1) {
            const long long rec = (slot * 4 + (lane >> 3)) * 7919 % n_rec;
            p = pool + rec * 656 + (lane & 7) * 16;
        } else {
            p = pool + (slot * 7919 % (n_rec - K)) * 656 + lane * 16;
        }
        __syncthreads();
        const long long t0 = clk();
        uint4 v[K];
#pragma unroll
        for (int c = 0; c < K; ++c) v[c] = ldg_nc_v4(p + (SHAPE == 0 ? 64 * c : SHAPE == 1 ? 128 * c : 656 * c));
        const long long t1 = clk();
#pragma unroll
        for (int c = 0; c < K; ++c) acc += v[c].x ^ v[c].y ^ v[c].z ^ v[c].w;
        asm volatile("" :: "r"(acc) : "memory");
        const long long t2 = clk();
        issue += t1 - t0;
        complete += t2 - t0;
    }
    if (acc == 0x12345678u) *sink = acc;
    if (threadIdx.x == 0) { out[2 * blockIdx.x] = issue / tiles;  out[2 * blockIdx.x + 1] = complete / tiles; }
}

template <int K, int SHAPE>
void run(const uint8_t* pool, long long n_rec, int threads, uint8_t* flush, size_t flush_bytes, long long* d_out, uint32_t* d_sink) {
    const int blocks = 128, tiles = 4;
    long long h[256];
    double res[2][2];
    for (int warm = 0; warm < 2; ++warm) {
        if (!warm) cudaMemset(flush, 1, flush_bytes);
        else gather<K, SHAPE><<<blocks, threads>>>(pool, n_rec, tiles, d_out, d_sink);   // leaves the records in L2
        gather<K, SHAPE><<<blocks, threads>>>(pool, n_rec, tiles, d_out, d_sink);
        cudaDeviceSynchronize();
        cudaMemcpy(h, d_out, sizeof(long long) * 2 * blocks, cudaMemcpyDeviceToHost);
        double a = 0, b = 0;
        for (int i = 0; i < blocks; ++i) { a += h[2 * i];  b += h[2 * i + 1]; }
        res[warm][0] = a / blocks;  res[warm][1] = b / blocks;
    }
    const double bytes = double(threads) * K * 16;
    printf("shape %d K %2d threads %3d bytes/tile %6.0f | cold issue %6.0f complete %6.0f (%.1f B/clk) | L2 issue %6.0f complete %6.0f (%.1f B/clk)\n",
           SHAPE, K, threads, bytes, res[0][0], res[0][1], bytes / res[0][1], res[1][0], res[1][1], bytes / res[1][1]);
}

int main() {
    const long long n_rec = 1 << 20;   // 688 MB of records
    uint8_t *pool, *flush;
    long long* d_out;
    uint32_t* d_sink;
    const size_t flush_bytes = 512ull << 20;
    cudaMalloc(&pool, n_rec * 656 + 65536);
    cudaMemset(pool, 3, n_rec * 656 + 65536);
    cudaMalloc(&flush, flush_bytes);
    cudaMalloc(&d_out, sizeof(long long) * 512);
    cudaMalloc(&d_sink, 4);
    for (int threads : {256, 512}) {
        run<2, 0>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<4, 0>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<6, 0>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<8, 0>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<11, 0>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<16, 0>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<3, 1>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<5, 1>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<10, 1>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<4, 2>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<8, 2>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
        run<16, 2>(pool, n_rec, threads, flush, flush_bytes, d_out, d_sink);
    }
    cudaError_t e = cudaDeviceSynchronize();
    printf("status %s\n", cudaGetErrorString(e));
    return e != cudaSuccess;
}

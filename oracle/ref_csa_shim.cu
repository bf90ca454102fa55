// TEST INFRASTRUCTURE ONLY.  A C entry point around the reference project's own
// CSA compressor reduce kernel (csa/sm100/kernel.cuh:25-112), so that the
// reference kernel itself can be run and timed beside this library's.  The
// reference reaches it through its torch extension (csa/interface.h:21-85); this
// shim fills the same parameter block (csa/params.h:12-39) the same way for
// contiguous tensors.  Compiled by oracle/build_ref.py against the reference
// sources where they lie; nothing of the reference is copied here.
#include "sm100/kernel.cuh"

extern "C" int ref_csa_compress_reduce(int B, int n, int c_out, int m,
                                       const void* C_a, const void* C_b, const void* Z_a, const void* Z_b,
                                       const void* B_a, const void* B_b, void* out, void* stream) {
    if (m != 4 || n % m != 0) return 1;
    dsv4::csa::CsaCompressReduceParams p{};
    p.B = B;  p.n = n;  p.n_blocks = n / m;  p.c_out = c_out;  p.m = m;
    p.C_a = static_cast<const __nv_bfloat16*>(C_a);  p.C_b = static_cast<const __nv_bfloat16*>(C_b);
    p.Z_a = static_cast<const __nv_bfloat16*>(Z_a);  p.Z_b = static_cast<const __nv_bfloat16*>(Z_b);
    p.B_a = static_cast<const __nv_bfloat16*>(B_a);  p.B_b = static_cast<const __nv_bfloat16*>(B_b);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.stride_C_b = n * c_out;  p.stride_C_n = c_out;
    p.stride_out_b = (n / m) * c_out;  p.stride_out_blk = c_out;
    dsv4::csa::sm100::launch_csa_compress_reduce<4>(p, static_cast<cudaStream_t>(stream));
    return int(cudaGetLastError());
}

// TEST INFRASTRUCTURE ONLY.  A C entry point around the reference project's
// own launch_hca_combine (hca/sm100/combine.h:31), so that the reference's
// merge kernel itself can be run beside this library's on the same partials.
// The reference reaches that function only through hca_decode_fwd
// (hca/sm100/kernel.cu:337-354); this shim fills the same fields the same way
// for contiguous tensors.  Compiled by oracle/build_ref.py against the
// reference sources where they lie; nothing of the reference is copied here.
#include "combine.h"

extern "C" int ref_hca_combine(int B, int H, int num_splits,
                               const float* partial_O, const float* partial_lse,
                               void* O, float* lse, const float* sink, void* stream) {
    dsv4::hca::sm100::HcaCombineParams cp{};
    cp.B = B;  cp.H = H;  cp.D = 512;  cp.num_splits = num_splits;
    cp.partial_O = partial_O;
    cp.partial_lse = partial_lse;
    cp.O = static_cast<__nv_bfloat16*>(O);
    cp.lse = lse;
    cp.attn_sink = sink;
    cp.stride_partial_O_split = int64_t(B) * H * 512;
    cp.stride_partial_O_b = int64_t(H) * 512;
    cp.stride_partial_O_h = 512;
    cp.stride_partial_lse_split = int64_t(B) * H;
    cp.stride_partial_lse_b = H;
    cp.stride_O_b = int64_t(H) * 512;
    cp.stride_O_h = 512;
    cp.stride_lse_b = H;
    dsv4::hca::sm100::launch_hca_combine(cp, static_cast<cudaStream_t>(stream));
    return int(cudaGetLastError());
}

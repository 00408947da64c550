// tcgen05 backward, flat tiling: the float16 instantiations (a translation unit of their own so that the build runs in parallel).
#include "na1d_tc_bwd_kernel.cuh"
#include "na1d_tc_bwd_flat.inl"

namespace na1d {

cudaError_t tc_bwd_flat_fp16(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k, const void* v,
                             const float* lse, const float* rpb, const int* valid_len, float* scratch, size_t scratch_floats,
                             const Geometry& gm, cudaStream_t st) {
    return run_flat<__half>(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, scratch_floats, gm, 1, st);
}
int tc_bwd_fp16_read_status() { return read_status_word(); }

}  // namespace na1d

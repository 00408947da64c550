// tcgen05 backward with attention dropout (flat tiling): the float16 instantiations.
#include "na1d_tc_bwd_kernel.cuh"
#include "na1d_tc_bwd_flat.inl"

namespace na1d {

cudaError_t tc_bwd_drop_fp16(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k, const void* v,
                             const float* lse, const float* rpb, const int* valid_len, float* scratch, size_t scratch_floats,
                             const Geometry& gm, const DropoutCfg& drop, cudaStream_t st) {
    return run_flat<__half, true>(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, scratch_floats, gm, 1, st, drop);
}
int tc_bwd_drop_fp16_read_status() { return read_status_word(); }

}  // namespace na1d

// tcgen05 backward with attention dropout (flat tiling): host entry point and the bfloat16 instantiations
// (the float16 ones are compiled in na1d_tc_bwd_drop_fp16.cu, in parallel).
#include "na1d_tc_bwd_kernel.cuh"
#include "na1d_tc_bwd_flat.inl"

namespace na1d {

cudaError_t tc_bwd_drop_fp16(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k, const void* v,
                             const float* lse, const float* rpb, const int* valid_len, float* scratch, size_t scratch_floats,
                             const Geometry& gm, const DropoutCfg& drop, cudaStream_t st);
int tc_bwd_drop_fp16_read_status();

cudaError_t tc_fused_bwd_dropout(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                                 const void* v, const float* lse, const float* rpb, const int* valid_len, float* scratch,
                                 size_t scratch_floats, const Geometry& gm, int dtype, const DropoutCfg& drop, cudaStream_t st) {
    if (!tc_bwd_supports(gm, rpb != nullptr, d_rpb != nullptr)) return cudaErrorInvalidValue;
    if (dtype != 0) return tc_bwd_drop_fp16(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, scratch_floats, gm, drop, st);
    return run_flat<__nv_bfloat16, true>(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, scratch_floats, gm, 0, st, drop);
}

int tc_bwd_drop_read_status() {
    const int a = read_status_word(), b = tc_bwd_drop_fp16_read_status();
    return (a > 0 || b > 0) ? (a > 0 ? a : b) : (a < 0 || b < 0) ? -1 : 0;
}

}  // namespace na1d

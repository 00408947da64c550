// tcgen05 backward, segmented tiling (any dilation, strided tensors): host entry points and the bfloat16 instantiations
// (the float16 ones are compiled in na1d_tc_bwd_seg_fp16.cu, in parallel).
#include "na1d_tc_bwd_kernel.cuh"
#include "na1d_tc_bwd_seg.inl"

namespace na1d {

cudaError_t tc_bwd_seg_fp16(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k, const void* v,
                            const float* lse, const float* rpb, const int* valid_len, float* scratch, size_t scratch_floats,
                            const Strides& sdq, const Strides& sdk, const Strides& sdv, const Strides& sdo, const Strides& sq,
                            const Strides& sk, const Strides& sv, const Geometry& gm, cudaStream_t st);
int tc_bwd_seg_fp16_read_status();

bool tc_bwd_seg_supports(const Geometry& gm, bool has_bias, bool wants_bias_grad) {
    return tc_seg_supports(gm) && bwd_smem_fits(gm, gm.win, has_bias, wants_bias_grad);
}

cudaError_t tc_fused_bwd_seg(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                             const void* v, const float* lse, const float* rpb, const int* valid_len, float* scratch,
                             size_t scratch_floats, const Strides& sdq, const Strides& sdk, const Strides& sdv, const Strides& sdo,
                             const Strides& sq, const Strides& sk, const Strides& sv, const Geometry& gm, int dtype, cudaStream_t st) {
    if (!tc_bwd_seg_supports(gm, rpb != nullptr, d_rpb != nullptr)) return cudaErrorInvalidValue;
    if (dtype != 0)
        return tc_bwd_seg_fp16(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, scratch_floats, sdq, sdk, sdv, sdo, sq, sk,
                               sv, gm, st);
    return run_seg<__nv_bfloat16>(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, scratch_floats, sdq, sdk, sdv, sdo, sq,
                                  sk, sv, gm, 0, st);
}

int tc_bwd_seg_read_status() {
    const int a = read_status_word(), b = tc_bwd_seg_fp16_read_status();
    return (a > 0 || b > 0) ? (a > 0 ? a : b) : (a < 0 || b < 0) ? -1 : 0;
}

}  // namespace na1d

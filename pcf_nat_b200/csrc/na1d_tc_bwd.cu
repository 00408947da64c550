// tcgen05 backward, flat tiling over the dense (N*T, C) matrix: host entry points and the bfloat16 instantiations
// (the float16 ones are compiled in na1d_tc_bwd_fp16.cu, in parallel).
#include "na1d_tc_bwd_kernel.cuh"

namespace na1d {

cudaError_t tc_bwd_flat_fp16(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k, const void* v,
                             const float* lse, const float* rpb, const int* valid_len, float* scratch, size_t scratch_floats,
                             const Geometry& gm, cudaStream_t st);
int tc_bwd_fp16_read_status();

}  // namespace na1d
#include "na1d_tc_bwd_flat.inl"

namespace na1d {

bool tc_bwd_supports(const Geometry& gm, bool has_bias, bool wants_bias_grad) {
    if (!(tc::pow2(gm.dil) && (gm.C == 64 || gm.C == 32 || gm.C == 16) && tc::eff_window(gm.win, gm.dil) <= 33 && gm.H <= 32 &&
          gm.T >= 32 && gm.T < (1 << 21)))
        return false;
    return bwd_smem_fits(gm, tc::eff_window(gm.win, gm.dil), has_bias, wants_bias_grad);
}

cudaError_t tc_fused_bwd(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                         const void* v, const float* lse, const float* rpb, const int* valid_len, float* scratch,
                         size_t scratch_floats, const Geometry& gm, int dtype, cudaStream_t st) {
    if (!tc_bwd_supports(gm, rpb != nullptr, d_rpb != nullptr)) return cudaErrorInvalidValue;
    if (dtype != 0) return tc_bwd_flat_fp16(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, scratch_floats, gm, st);
    return run_flat<__nv_bfloat16>(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, scratch_floats, gm, 0, st);
}

int tc_bwd_read_status() {
    const int a = read_status_word(), b = tc_bwd_fp16_read_status();
    return (a > 0 || b > 0) ? (a > 0 ? a : b) : (a < 0 || b < 0) ? -1 : 0;
}

}  // namespace na1d

// TEST INFRASTRUCTURE ONLY: C entry points around the REFERENCE's own CUDA launchers.
//
// This file contains no kernel code. It is compiled together with the reference's
// na1d_tensorcore/{bf16,fp16}_ana1d_kernel.cu, taken from where the reference project
// lies on disk (never copied into this repository), into oracle/_ref/libref_ana1d_<dtype>.so.
// The result lets the GPU tests hold the new kernels against the reference's kernels on
// identical device buffers, and lets the benchmark time the reference's kernels on the
// same GPU. The six entry points mirror the pybind shims of na1d_tensorcore/bf16_ana1d.cpp:8-104
// including their aliasing of six names onto three kernels and the C%16 dispatch.
//
// Build with -DREF_BF16 or -DREF_FP16 and -I<reference>/na1d_tensorcore.
#include <cuda_runtime.h>
#if defined(REF_BF16)
#include "bf16_ana1d.h"
typedef __nv_bfloat16 elem_t;
#define QK16 bf16_ana_qk_forward_C16
#define QK8 bf16_ana_qk_forward_C8
#define QB bf16_ana_q_backward
#define KB bf16_ana_k_backward
#elif defined(REF_FP16)
#include "fp16_ana1d.h"
typedef __half elem_t;
#define QK16 fp16_ana_qk_forward_C16
#define QK8 fp16_ana_qk_forward_C8
#define QB fp16_ana_q_backward
#define KB fp16_ana_k_backward
#else
#error "define REF_BF16 or REF_FP16"
#endif

extern "C" {

// band = Q.K^T over the window (also used for attn_gd = dO.V^T)
int ref_ana_qk_forward(float* attn, const void* q, const void* k, int N, int T, int C, int win, int left) {
    if (C % 16 == 0) QK16(attn, (const elem_t*)q, (const elem_t*)k, N, T, C, win, left);
    else             QK8(attn, (const elem_t*)q, (const elem_t*)k, N, T, C, win, left);
    return (int)cudaGetLastError();
}
// out = band . X (AV forward and dQ)
int ref_ana_band_x(void* out, const float* band, const void* x, int N, int T, int C, int win, int left) {
    QB((elem_t*)out, band, (const elem_t*)x, N, T, C, win, left);
    return (int)cudaGetLastError();
}
// out = band^T . X (dK and dV)
int ref_ana_bandT_x(void* out, const float* band, const void* x, int N, int T, int C, int win, int left) {
    KB((elem_t*)out, band, (const elem_t*)x, N, T, C, win, left);
    return (int)cudaGetLastError();
}

}  // extern "C"

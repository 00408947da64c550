// Internal C++ interface between the C ABI (na1d_api.cu) and the kernel families.
#pragma once
#include "na1d_common.cuh"

namespace na1d {

// ---- CUDA-core family (na1d_simt.cu)
bool simt_supports_channels(int C);
cudaError_t simt_qk(float* attn, const void* a, const void* b, const Geometry& gm, int dtype, cudaStream_t st);
cudaError_t simt_band_x(void* out, const float* band, const void* x, const Geometry& gm, int dtype, cudaStream_t st);
cudaError_t simt_bandT_x(void* out, const float* band, const void* x, const Geometry& gm, int dtype, cudaStream_t st);
cudaError_t simt_fused_fwd(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                           const int* valid_len, const Geometry& gm, int dtype, cudaStream_t st);
cudaError_t simt_delta(float* delta, const void* d_o, const void* o, int rows, int C, int dtype, cudaStream_t st);
cudaError_t simt_fused_bwd(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                           const void* v, const float* lse, const float* delta, const float* rpb, const int* valid_len,
                           const Geometry& gm, int dtype, cudaStream_t st);
cudaError_t window_index(int* j_out, unsigned char* inr, int T, int win, int left, int dil, cudaStream_t st);

// ---- tcgen05 / TMA family (na1d_tc_fwd.cu)
bool tc_fwd_supports(const Geometry& gm);  // shape limits of the tcgen05 forward
cudaError_t tc_fused_fwd(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                         const int* valid_len, const Geometry& gm, int dtype, cudaStream_t st);
// status words of the tcgen05 translation units (read and cleared; the call synchronises the device): 0 = no bounded
// wait expired, > 0 = a code naming the wait, < 0 = the read failed
int tc_read_status();
int tc_bwd_read_status();
int tc_seg_read_status();
int tc_bwd_seg_read_status();

// ---- tcgen05 / TMA family, segmented tiling (na1d_tc_fwd_seg.cu, na1d_tc_bwd_seg.cu): any dilation, strided tensors
SegGeom seg_geometry(const Geometry& gm, int step);
bool tc_seg_supports(const Geometry& gm);
bool tc_bwd_seg_supports(const Geometry& gm, bool has_bias = false, bool wants_bias_grad = false);
cudaError_t tc_fused_fwd_seg(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                             const int* valid_len, const Strides& sq, const Strides& sk, const Strides& sv, const Strides& so,
                             const Geometry& gm, int dtype, cudaStream_t st);
cudaError_t tc_fused_bwd_seg(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                             const void* v, const float* lse, const float* rpb, const int* valid_len, float* scratch,
                             size_t scratch_floats, const Strides& sdq, const Strides& sdk, const Strides& sdv, const Strides& sdo,
                             const Strides& sq, const Strides& sk, const Strides& sv, const Geometry& gm, int dtype, cudaStream_t st);
void tensor_map_cache_stats(long long* hits, long long* misses);

// ---- the unfused pair on the tcgen05 kernels (na1d_tc_unfused.cu): flat tiling, same shape limits as the fused forward
bool tc_unfused_supports(const Geometry& gm);
cudaError_t tc_qk(float* attn, const void* a, const void* b, const Geometry& gm, int dtype, cudaStream_t st);
cudaError_t tc_band_x(void* out, const float* band, const void* x, const Geometry& gm, int dtype, cudaStream_t st);
int tc_unfused_read_status();
bool tc_unfused_t_supports(const Geometry& gm);
cudaError_t tc_bandT_x(void* out, const float* band, const void* x, const Geometry& gm, int dtype, cudaStream_t st);
int tc_unfused_t_read_status();

// ---- fused pair with attention dropout (na1d_tc_fwd_drop.cu, na1d_tc_bwd_drop.cu): flat tiling of the tcgen05 kernels
cudaError_t tc_fused_fwd_dropout(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                                 const int* valid_len, const Geometry& gm, int dtype, const DropoutCfg& drop, cudaStream_t st);
cudaError_t tc_fused_bwd_dropout(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                                 const void* v, const float* lse, const float* rpb, const int* valid_len, float* scratch,
                                 size_t scratch_floats, const Geometry& gm, int dtype, const DropoutCfg& drop, cudaStream_t st);
int tc_drop_read_status();
int tc_bwd_drop_read_status();
// shape limits of the tcgen05 backward, including whether its shared memory fits with a bias table (has_bias) and the
// bias-gradient accumulators (wants_bias_grad)
bool tc_bwd_supports(const Geometry& gm, bool has_bias = false, bool wants_bias_grad = false);
cudaError_t tc_fused_bwd(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                         const void* v, const float* lse, const float* rpb, const int* valid_len, float* scratch,
                         size_t scratch_floats, const Geometry& gm, int dtype, cudaStream_t st);

}  // namespace na1d

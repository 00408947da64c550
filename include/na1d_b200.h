/*
 * na1d_b200.h -- C ABI of the B200 (sm_100a) 1-D neighbourhood-attention library.
 *
 * All pointers are DEVICE pointers unless a comment says otherwise; all tensors are dense and
 * row-major.  Every function is asynchronous on `stream` (a cudaStream_t passed as void*, NULL =
 * legacy default stream), allocates nothing unless stated, and returns 0 (NA1D_OK) or a negative
 * NA1D_ERR_* code after validating its arguments on the host; no argument error ever reaches
 * the device.  The library is re-entrant; the caller owns every buffer.
 *
 * Geometry shared by all entry points (reference: models/PCF_NATransformer.py:47-56, 153-171):
 *   N sequences (= batch*heads, head index fastest: n = b*heads + h), T tokens, C channels per
 *   head (multiple of 8), window `win` with `left` neighbours before the query, dilation `dil`.
 *   Neighbour kk of query t is key j = t + (kk-left)*dil; keys outside [0,T) read as zero rows.
 *
 * Each declaration cites the interface of the reference project (ChenNan1996/PCF-NAT) that it
 * replaces, as file:line inside that project.
 */
#ifndef NA1D_B200_H
#define NA1D_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element type of the 16-bit tensors */
#define NA1D_BF16 0 /* replaces the bf16_ana1d module, na1d_tensorcore/nattn.py:12-20 */
#define NA1D_FP16 1 /* replaces the fp16_ana1d module, na1d_tensorcore/nattn.py:21-29 */

/* status codes */
#define NA1D_OK 0
#define NA1D_ERR_NULL_POINTER (-1)   /* a required pointer is NULL */
#define NA1D_ERR_BAD_SHAPE (-2)      /* N,T,C <= 0, C % 8 != 0, C > 256, or a product overflows int32 */
#define NA1D_ERR_BAD_WINDOW (-3)     /* win <= 0, win > NA1D_MAX_WINDOW, left outside [0,win), dil <= 0 */
#define NA1D_ERR_BAD_DTYPE (-4)      /* dtype is neither NA1D_BF16 nor NA1D_FP16 */
#define NA1D_ERR_BAD_HEADS (-5)      /* heads <= 0 or N % heads != 0 */
#define NA1D_ERR_MISALIGNED (-6)     /* a 16-bit tensor pointer is not 16-byte aligned */
#define NA1D_ERR_CUDA (-7)           /* a CUDA runtime/driver call failed; see na1d_last_cuda_error() */
#define NA1D_ERR_DEVICE_TIMEOUT (-8) /* a bounded wait inside a kernel expired (reported by na1d_device_status) */
#define NA1D_ERR_TOO_LARGE (-9)      /* problem exceeds a fixed capacity of the entry point */
#define NA1D_ERR_UNSUPPORTED (-10)   /* the requested kernel family / tiling cannot run this shape */
#define NA1D_ERR_BAD_DROPOUT (-12)   /* dropout probability outside [0,1) */
#define NA1D_ERR_BAD_STRIDE (-11)    /* a stride is not a positive multiple of 8 elements, or the token stride is below C */

#define NA1D_MAX_WINDOW 128 /* the reference asserts win <= 80, models/PCF_NATransformer.py:53 */

/* Human-readable text for a status code (host pointer, static storage). */
const char* na1d_status_string(int status);
/* cudaError_t value of the most recent failing CUDA call on this host thread (0 if none). */
int na1d_last_cuda_error(void);
/* Library version, major*100+minor. */
int na1d_version(void);

/* ------------------------------------------------------------------------------------------
 * Unfused pair: the six entry points of the reference extension, same argument meaning.
 * `dil` extends them (the reference kernels support dil == 1 only, na1d_tensorcore/nattn.py:130).
 * ---------------------------------------------------------------------------------------- */

/* attn[n,t,kk] = sum_c q[n,t,c] * k[n,j,c]            attn: (N,T,win) fp32; q,k: (N,T,C) 16-bit.
 * Replaces torch_ana_qk_forward, na1d_tensorcore/bf16_ana1d.cpp:8-27 (kernels
 * bf16_ana1d_kernel.cu:42-282; fp16 twin fp16_ana1d.cpp:8-27). */
int na1d_qk_forward(float* attn, const void* q, const void* k, int64_t N, int64_t T, int64_t C,
                    int64_t win, int64_t left, int64_t dil, int dtype, void* stream);

/* q_gd[n,t,c] = sum_kk attn_gd[n,t,kk] * k[n,j,c]      q_gd: (N,T,C) 16-bit.
 * Replaces torch_ana_q_backward, na1d_tensorcore/bf16_ana1d.cpp:29-41 (kernel :285-391). */
int na1d_q_backward(void* q_gd, const float* attn_gd, const void* k, int64_t N, int64_t T, int64_t C,
                    int64_t win, int64_t left, int64_t dil, int dtype, void* stream);

/* k_gd[n,j,c] = sum_kk attn_gd[n,t,kk] * q[n,t,c] over all (t,kk) whose neighbour is j.
 * Replaces torch_ana_k_backward, na1d_tensorcore/bf16_ana1d.cpp:43-55 (kernel :394-492). */
int na1d_k_backward(void* k_gd, const float* attn_gd, const void* q, int64_t N, int64_t T, int64_t C,
                    int64_t win, int64_t left, int64_t dil, int dtype, void* stream);

/* result[n,t,c] = sum_kk attn[n,t,kk] * v[n,j,c].
 * Replaces torch_ana_av_forward, na1d_tensorcore/bf16_ana1d.cpp:57-69. */
int na1d_av_forward(void* result, const float* attn, const void* v, int64_t N, int64_t T, int64_t C,
                    int64_t win, int64_t left, int64_t dil, int dtype, void* stream);

/* attn_gd[n,t,kk] = sum_c result_gd[n,t,c] * v[n,j,c].
 * Replaces torch_ana_a_backward, na1d_tensorcore/bf16_ana1d.cpp:71-90. */
int na1d_a_backward(float* attn_gd, const void* result_gd, const void* v, int64_t N, int64_t T, int64_t C,
                    int64_t win, int64_t left, int64_t dil, int dtype, void* stream);

/* v_gd[n,j,c] = sum_kk attn[n,t,kk] * result_gd[n,t,c] over all (t,kk) whose neighbour is j.
 * Replaces torch_ana_v_backward, na1d_tensorcore/bf16_ana1d.cpp:92-104. */
int na1d_v_backward(void* v_gd, const float* attn, const void* result_gd, int64_t N, int64_t T, int64_t C,
                    int64_t win, int64_t left, int64_t dil, int dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused layer core: everything NAttention.forward does between the head split and the head
 * merge (models/PCF_NATransformer.py:141-150; MFA twin models/MFA_NATransformer.py:141-150):
 *   s[kk] = scale * q[t].k[j] + rpb[h,kk] + (masked ? -100 : 0);  p = softmax(s);  o = sum p[kk] v[j]
 *   masked = j outside [0,T)  or  j >= valid_len[b]  or  t >= valid_len[b]      (:87-116)
 * The fp32 (N,T,win) tensor of the unfused pair never exists in memory.
 * ---------------------------------------------------------------------------------------- */

/* o: (N,T,C) 16-bit; lse: (N,T) fp32 = log sum_kk exp(s[kk]) (kept for the backward pass; may be NULL);
 * rpb: (heads,win) fp32 or NULL; valid_len: (N/heads) int32 or NULL (= no padding). */
int na1d_fused_forward(void* o, float* lse, const void* q, const void* k, const void* v,
                       const float* rpb, const int32_t* valid_len, int64_t N, int64_t heads, int64_t T,
                       int64_t C, int64_t win, int64_t left, int64_t dil, float scale, int dtype,
                       void* stream);

/* Gradients of na1d_fused_forward. dq,dk,dv: (N,T,C) 16-bit. d_rpb: (heads,win) fp32, ACCUMULATED
 * into (caller zeroes it), or NULL. delta_ws: caller-provided scratch of N*T fp32. The CUDA-core
 * kernels keep the row sums of d_o*o there (written by a pre-pass, read by the main kernel); the
 * tcgen05 kernels need no such pre-pass: every CTA adds its partial d_rpb to the result with atomics at
 * its end (with NA1D_BIAS_GRAD_ROWS=1 in the environment: one partial row per CTA in delta_ws, summed in
 * a fixed order by a second small kernel).
 * Replaces the autograd chain AV.backward -> softmax backward -> QK.backward,
 * na1d_tensorcore/nattn.py:46-54 and :69-78. */
int na1d_fused_backward(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q,
                        const void* k, const void* v, const void* o, const float* lse, const float* rpb,
                        const int32_t* valid_len, float* delta_ws, int64_t N, int64_t heads, int64_t T,
                        int64_t C, int64_t win, int64_t left, int64_t dil, float scale, int dtype,
                        void* stream);

/* Backward pass for callers that must not allocate device memory and have no spare buffer to lend.
 * (No counterpart in the reference project: its Python layer allocates every tensor with torch.)
 *
 * Who needs it: a host that drives this library from a place where device allocation is forbidden or
 * simply unavailable -- a serving or training loop whose memory pool is frozen after start-up, a thread
 * that is between cudaStreamBeginCapture and cudaStreamEndCapture, or a plain C/C++ runtime that hands
 * a plug-in fixed input/output buffers and no allocator handle. na1d_fused_backward asks such a caller
 * for an N*T-float workspace (delta_ws) it cannot produce. This variant takes the same inputs and
 * outputs but keeps that workspace inside the library, in a fixed device array.
 *
 * Same results as na1d_fused_backward with the CUDA-core kernels (it always runs those: they are the
 * backward kernels that use the workspace). Limits and rules:
 *   - N*T <= NA1D_STATIC_SCRATCH_ROWS, otherwise NA1D_ERR_TOO_LARGE is returned and nothing is launched.
 *     The array (NA1D_STATIC_SCRATCH_ROWS floats = 4 MiB) exists once per GPU that loads the library and
 *     stays resident until the process exits.
 *   - It calls no cudaMalloc/cudaFree and no allocating library routine, on any call.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current). Make that first call outside any stream capture.
 *   - All calls on one device share the array. Every call overwrites the part it uses before reading
 *     it, so nothing has to be cleared between calls -- but two calls whose kernels can overlap on the
 *     GPU (different streams, no dependency) would race on it; order them on one stream or with events.
 *   - d_rpb, when given, is accumulated into exactly as in na1d_fused_backward (the caller zeroes it).
 */
#define NA1D_STATIC_SCRATCH_ROWS (1 << 20)
int na1d_fused_backward_static(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q,
                               const void* k, const void* v, const void* o, const float* lse,
                               const float* rpb, const int32_t* valid_len, int64_t N, int64_t heads,
                               int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil, float scale,
                               int dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Strided forms of the fused pair: q, k, v, o (and the gradients) may be views with arbitrary batch / head / token
 * strides, so that the head split and merge around the operator need no copies. Each `*_strides` argument is a HOST
 * pointer to three int64 element strides {batch, head, token} of a tensor addressed as [batch][head][token][channel]
 * (channel stride 1): a dense (N,T,C) tensor has {heads*T*C, T*C, C}; the q slice of a packed projection output
 * (batch, T, 3, heads, C) has {T*3*heads*C, C, 3*heads*C} and starts at the packed tensor's base (k: + heads*C
 * elements, v: + 2*heads*C); an output laid out (batch, T, heads, C) has {T*heads*C, C, heads*C}. Strides must be
 * positive multiples of 8 elements and pointers 16-byte aligned (NA1D_ERR_BAD_STRIDE / NA1D_ERR_MISALIGNED otherwise);
 * output views must not overlap themselves or each other. lse stays dense (N,T). These calls run the tcgen05 kernels on
 * the segmented tiling only (C in {16,32,64}, win <= 33, heads <= 32, T >= 2*dil; NA1D_ERR_UNSUPPORTED otherwise --
 * make dense copies and use the dense entry points then).
 * Replaces the head split of models/MFA_NATransformer.py:127-137 (and models/PCF_NATransformer.py:126-138), the head
 * merge of :151-152, and their autograd copies, together with the fused layer core above.
 * ---------------------------------------------------------------------------------------- */
/* 1 when the strided forward AND backward accept this shape (with a bias / with its gradient wanted), 0 when not,
 * negative for an invalid geometry. Host-only; lets a layer choose between the strided and the dense route up front. */
int na1d_fused_strided_supported(int64_t heads, int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil,
                                 int dtype, int has_bias, int wants_bias_grad);

int na1d_fused_forward_strided(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                               const int32_t* valid_len, const int64_t* o_strides, const int64_t* q_strides,
                               const int64_t* k_strides, const int64_t* v_strides, int64_t N, int64_t heads,
                               int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil, float scale, int dtype,
                               void* stream);

/* scratch: `scratch_floats` fp32 of device memory for the per-CTA partial rows of d_rpb (148 * heads * win is always
 * enough; with less, or NULL, the kernel adds to d_rpb with atomics). o is not needed. */
int na1d_fused_backward_strided(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q,
                                const void* k, const void* v, const float* lse, const float* rpb,
                                const int32_t* valid_len, float* scratch, int64_t scratch_floats,
                                const int64_t* dq_strides, const int64_t* dk_strides, const int64_t* dv_strides,
                                const int64_t* d_o_strides, const int64_t* q_strides, const int64_t* k_strides,
                                const int64_t* v_strides, int64_t N, int64_t heads, int64_t T, int64_t C, int64_t win,
                                int64_t left, int64_t dil, float scale, int dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused pair with attention dropout: p' = keep ? p / (1 - drop_p) : 0 on the normalised probabilities before the product
 * with v, as `self.attn_drop(attn)` between softmax and AV (models/PCF_NATransformer.py:149; the reference's configs set
 * the probability to 0). The keep decision of probability (row, kk) is a hash of (seed, dense row index n*T+t, kk) -- see
 * drop_hash in pcf_nat_b200/csrc/na1d_common.cuh; the backward re-derives the same mask from the same seed, nothing is
 * stored. lse is the log-sum-exp of the undropped logits. drop_p in [0,1); drop_p == 0 is the plain forward. Runs on the
 * tcgen05 kernels (flat tiling) only: NA1D_ERR_UNSUPPORTED for other shapes. `scratch` as in the strided backward.
 * ---------------------------------------------------------------------------------------- */
/* The keep decisions the dropout kernels derive, computed on the HOST into a HOST buffer of rows*win bytes
 * (keep_host[row*win + kk] = 1 if probability kk of dense row `row` = n*T+t is kept), for bit-exact checking of a
 * restatement of the hash. No device work. No counterpart in the reference (torch's dropout draws from the Philox stream). */
int na1d_dropout_keep_mask(uint8_t* keep_host, int64_t rows, int64_t win, float drop_p, uint64_t seed);

int na1d_fused_forward_dropout(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                               const int32_t* valid_len, int64_t N, int64_t heads, int64_t T, int64_t C, int64_t win,
                               int64_t left, int64_t dil, float scale, float drop_p, uint64_t seed, int dtype,
                               void* stream);
int na1d_fused_backward_dropout(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q,
                                const void* k, const void* v, const float* lse, const float* rpb,
                                const int32_t* valid_len, float* scratch, int64_t scratch_floats, int64_t N,
                                int64_t heads, int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil,
                                float scale, float drop_p, uint64_t seed, int dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Window index arithmetic as the kernels compute it, for bit-exact checking:
 * j_out[t,kk] = t + (kk-left)*dil (int32, (T,win)); in_range[t,kk] = 1 if 0 <= j < T else 0.
 * Restates the implicit pad+unfold indexing of models/PCF_NATransformer.py:158-165.
 * ---------------------------------------------------------------------------------------- */
int na1d_window_index(int32_t* j_out, uint8_t* in_range, int64_t T, int64_t win, int64_t left,
                      int64_t dil, void* stream);

/* Which kernel family the fused entry points would pick for a shape: 0 = CUDA-core kernels,
 * 1 = tcgen05/TMA kernels. Host-only query, no device work. The answer assumes one head, no bias and
 * no bias gradient: more than 32 heads, or 64-channel rows with an effective window above 17 together
 * with a bias of several heads or its gradient (no shared memory left for them), still move a call
 * to the CUDA-core kernels. */
int na1d_fused_kernel_family(int64_t N, int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil,
                             int dtype, int backward);

/* As na1d_fused_kernel_family, but tells the two tilings of the tcgen05 kernels apart: 0 = CUDA-core kernels,
 * 1 = tcgen05 on the flat tiling (tiles over the dense (N*T, C) matrix; dilation 1, or a power of two with
 * (win-1)*dil+1 <= 33), 2 = tcgen05 on the segmented tiling (tiles inside one residue class t = r mod dil of one
 * sequence: every dilation; also what the strided entry points run). Mirrors the tile heuristics of the reference's
 * launchers, na1d_tensorcore/bf16_ana1d_kernel.cu:495-580. */
int na1d_fused_kernel_tiling(int64_t N, int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil,
                             int dtype, int backward);

/* Force a kernel family for the fused entry points: -1 = automatic (default), 0 = CUDA-core,
 * 1 = tcgen05/TMA (the flat tiling wherever it can run, else the segmented one; for the unfused entry points: also
 * where the automatic choice would take a CUDA-core kernel), 2 = tcgen05/TMA on the segmented tiling. Process-wide;
 * meant for tests and benchmarks. Returns the previous setting. */
int na1d_set_kernel_family(int family);

/* Hits and misses of the library's cache of encoded TMA tensor maps since the process started (the cache is keyed by
 * pointer, extents, strides, box and element type; its only global state, behind a lock). Host-only.
 * No counterpart in the reference (its kernels take raw pointers). */
int na1d_tensor_map_cache_stats(int64_t* hits, int64_t* misses);

/* Synchronises the device, then returns and clears the device-side status word: 0 = every bounded
 * wait inside the tcgen05 kernels completed, otherwise NA1D_ERR_DEVICE_TIMEOUT. */
int na1d_device_status(void);

#ifdef __cplusplus
}
#endif
#endif /* NA1D_B200_H */

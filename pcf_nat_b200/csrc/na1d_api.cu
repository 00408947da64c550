// C ABI of the library: argument validation, kernel-family choice, launches. No torch types.
#include "../../include/na1d_b200.h"
#include "na1d_internal.h"

#include <atomic>
#include <climits>
#include <mutex>

namespace {

thread_local int g_last_cuda_error = 0;
std::atomic<int> g_family_override{-1};

int cuda_status(cudaError_t e) {
    if (e == cudaSuccess) return NA1D_OK;
    g_last_cuda_error = (int)e;
    return NA1D_ERR_CUDA;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_geometry(int64_t N, int64_t heads, int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil, int dtype,
                   float scale, na1d::Geometry& g) {
    if (dtype != NA1D_BF16 && dtype != NA1D_FP16) return NA1D_ERR_BAD_DTYPE;
    if (N <= 0 || T <= 0 || C <= 0 || C % 8 != 0 || C > 256) return NA1D_ERR_BAD_SHAPE;
    if (!na1d::simt_supports_channels((int)C)) return NA1D_ERR_BAD_SHAPE;
    if (win <= 0 || win > NA1D_MAX_WINDOW || left < 0 || left >= win || dil <= 0) return NA1D_ERR_BAD_WINDOW;
    if (heads <= 0 || N % heads != 0) return NA1D_ERR_BAD_HEADS;
    // every flat index used by the kernels must fit int32: rows, rows*win, window reach
    if (N * T > INT_MAX || N * T * win > INT_MAX || T * win > INT_MAX || win * dil > INT_MAX / 2 ||
        T + win * dil > INT_MAX / 2)
        return NA1D_ERR_BAD_SHAPE;
    g.N = (int)N; g.H = (int)heads; g.T = (int)T; g.C = (int)C; g.win = (int)win; g.left = (int)left; g.dil = (int)dil;
    g.scale = scale;
    return NA1D_OK;
}

// 32-byte rows with a window in the widest band bucket: the band-transposed mode of the tcgen05 backward kernel is bound by
// the fp32 band's gather there and loses to the CUDA-core kernel (measured at N=8192, T=150, C=16, win=27: 197 us against
// 121 us); the band-out and band-in modes win everywhere (94 against 174 us, 84 against 107 us) and are not affected.
bool narrow_rows_wide_window(const na1d::Geometry& g) { return g.C == 16 && (g.win - 1) * g.dil + 1 > 17; }

#define NA1D_REQUIRE_PTR(p) do { if ((p) == nullptr) return NA1D_ERR_NULL_POINTER; } while (0)
#define NA1D_REQUIRE_ALIGNED(p) do { if (!aligned16(p)) return NA1D_ERR_MISALIGNED; } while (0)

}  // namespace

extern "C" {

const char* na1d_status_string(int status) {
    switch (status) {
        case NA1D_OK: return "ok";
        case NA1D_ERR_NULL_POINTER: return "a required pointer is NULL";
        case NA1D_ERR_BAD_SHAPE: return "bad shape: need N,T,C > 0, C a supported multiple of 8 (<= 256), sizes within int32";
        case NA1D_ERR_BAD_WINDOW: return "bad window: need 0 < win <= 128, 0 <= left < win, dil >= 1";
        case NA1D_ERR_BAD_DTYPE: return "bad dtype: expected NA1D_BF16 or NA1D_FP16";
        case NA1D_ERR_BAD_HEADS: return "bad heads: need heads > 0 and N divisible by heads";
        case NA1D_ERR_MISALIGNED: return "a 16-bit tensor pointer is not 16-byte aligned";
        case NA1D_ERR_CUDA: return "a CUDA call failed (see na1d_last_cuda_error)";
        case NA1D_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel expired";
        case NA1D_ERR_TOO_LARGE: return "problem exceeds a fixed capacity of this entry point (e.g. N*T above NA1D_STATIC_SCRATCH_ROWS)";
        case NA1D_ERR_UNSUPPORTED: return "the requested kernel family or tiling does not support this shape";
        case NA1D_ERR_BAD_DROPOUT: return "bad dropout probability: need 0 <= p < 1";
        case NA1D_ERR_BAD_STRIDE: return "bad stride: element strides must be positive multiples of 8, the token stride >= C";
        default: return "unknown status";
    }
}
int na1d_last_cuda_error(void) { return g_last_cuda_error; }
int na1d_version(void) { return 100; }

int na1d_qk_forward(float* attn, const void* q, const void* k, int64_t N, int64_t T, int64_t C, int64_t win,
                    int64_t left, int64_t dil, int dtype, void* stream) {
    NA1D_REQUIRE_PTR(attn); NA1D_REQUIRE_PTR(q); NA1D_REQUIRE_PTR(k);
    NA1D_REQUIRE_ALIGNED(q); NA1D_REQUIRE_ALIGNED(k);
    na1d::Geometry g;
    if (int s = check_geometry(N, 1, T, C, win, left, dil, dtype, 1.f, g)) return s;
    if (g_family_override.load() != 0 && na1d::tc_unfused_supports(g) && aligned16(attn))   // the band goes out in 16-byte stores
        return cuda_status(na1d::tc_qk(attn, q, k, g, dtype, (cudaStream_t)stream));
    return cuda_status(na1d::simt_qk(attn, q, k, g, dtype, (cudaStream_t)stream));
}
int na1d_a_backward(float* attn_gd, const void* result_gd, const void* v, int64_t N, int64_t T, int64_t C, int64_t win,
                    int64_t left, int64_t dil, int dtype, void* stream) {
    return na1d_qk_forward(attn_gd, result_gd, v, N, T, C, win, left, dil, dtype, stream);
}
int na1d_q_backward(void* q_gd, const float* attn_gd, const void* k, int64_t N, int64_t T, int64_t C, int64_t win,
                    int64_t left, int64_t dil, int dtype, void* stream) {
    NA1D_REQUIRE_PTR(q_gd); NA1D_REQUIRE_PTR(attn_gd); NA1D_REQUIRE_PTR(k);
    NA1D_REQUIRE_ALIGNED(q_gd); NA1D_REQUIRE_ALIGNED(k);
    na1d::Geometry g;
    if (int s = check_geometry(N, 1, T, C, win, left, dil, dtype, 1.f, g)) return s;
    if (g_family_override.load() != 0 && na1d::tc_unfused_supports(g))
        return cuda_status(na1d::tc_band_x(q_gd, attn_gd, k, g, dtype, (cudaStream_t)stream));
    return cuda_status(na1d::simt_band_x(q_gd, attn_gd, k, g, dtype, (cudaStream_t)stream));
}
int na1d_av_forward(void* result, const float* attn, const void* v, int64_t N, int64_t T, int64_t C, int64_t win,
                    int64_t left, int64_t dil, int dtype, void* stream) {
    return na1d_q_backward(result, attn, v, N, T, C, win, left, dil, dtype, stream);
}
int na1d_k_backward(void* k_gd, const float* attn_gd, const void* q, int64_t N, int64_t T, int64_t C, int64_t win,
                    int64_t left, int64_t dil, int dtype, void* stream) {
    NA1D_REQUIRE_PTR(k_gd); NA1D_REQUIRE_PTR(attn_gd); NA1D_REQUIRE_PTR(q);
    NA1D_REQUIRE_ALIGNED(k_gd); NA1D_REQUIRE_ALIGNED(q);
    na1d::Geometry g;
    if (int s = check_geometry(N, 1, T, C, win, left, dil, dtype, 1.f, g)) return s;
    if (g_family_override.load() != 0 && na1d::tc_unfused_t_supports(g) && (!narrow_rows_wide_window(g) || g_family_override.load() == 1))
        return cuda_status(na1d::tc_bandT_x(k_gd, attn_gd, q, g, dtype, (cudaStream_t)stream));
    return cuda_status(na1d::simt_bandT_x(k_gd, attn_gd, q, g, dtype, (cudaStream_t)stream));
}
int na1d_v_backward(void* v_gd, const float* attn, const void* result_gd, int64_t N, int64_t T, int64_t C, int64_t win,
                    int64_t left, int64_t dil, int dtype, void* stream) {
    return na1d_k_backward(v_gd, attn, result_gd, N, T, C, win, left, dil, dtype, stream);
}

// 0 = CUDA-core kernels, 1 = tcgen05 kernels on the flat tiling, 2 = tcgen05 kernels on the segmented tiling.
// The flat tiling takes dilation 1 and those power-of-two dilations whose dilated window still fits the widest band bucket;
// the segmented tiling takes every dilation (each residue class of a sequence is a dilation-1 problem) at the price of
// partly empty last tiles. With a dilation both can run, the one with the cheaper band bucket per useful row wins.
static int pick_family(const na1d::Geometry& g, int backward, bool has_bias = false, bool wants_bias_grad = false) {
    const int forced = g_family_override.load();
    const bool flat_ok = backward ? na1d::tc_bwd_supports(g, has_bias, wants_bias_grad) : na1d::tc_fwd_supports(g);
    const bool seg_ok = backward ? na1d::tc_bwd_seg_supports(g, has_bias, wants_bias_grad) : na1d::tc_seg_supports(g);
    if (forced == 0) return 0;
    if (forced == 2) return seg_ok ? 2 : NA1D_ERR_UNSUPPORTED;
    if (forced == 1 && flat_ok) return 1;   // forced: the flat tiling wherever it can run (the choice below is for the automatic mode)
    int pick = 0;
    if (flat_ok && seg_ok && g.dil > 1) {
        // relative cost of a tile row in the window buckets 9 / 17 / 33 (measured at 64 utterances x 4 heads, 200 to 1000
        // tokens: the two narrow buckets cost about the same, the widest is bound by its compute warps, more so in the backward
        // with its two fragment sets per block), times the rows the
        // tiling processes per useful row, plus 10 % for the segmented tiling's shorter runs of tiles
        auto bucket_cost = [backward](int w) { return w <= 9 ? 1.0 : w <= 17 ? 1.05 : backward ? 2.0 : 1.5; };
        const int tp = (g.T + g.dil - 1) / g.dil;
        const int step = backward ? 128 - (g.win - 1) : 128;
        const double seg_rows = (double)((tp + step - 1) / step) * step / tp;
        const double flat = bucket_cost((g.win - 1) * g.dil + 1), seg = 1.1 * bucket_cost(g.win) * seg_rows;
        pick = seg < flat ? 2 : 1;
    } else if (flat_ok) {
        pick = 1;
    } else if (seg_ok) {
        pick = 2;
    }
    if (forced == 1 && pick == 0) return NA1D_ERR_UNSUPPORTED;
    return pick;
}

int na1d_fused_kernel_family(int64_t N, int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil, int dtype,
                             int backward) {
    na1d::Geometry g;
    if (int s = check_geometry(N, 1, T, C, win, left, dil, dtype, 1.f, g)) return s;
    const int fam = pick_family(g, backward);
    return fam == 2 ? 1 : fam;
}

int na1d_fused_kernel_tiling(int64_t N, int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil, int dtype,
                             int backward) {
    na1d::Geometry g;
    if (int s = check_geometry(N, 1, T, C, win, left, dil, dtype, 1.f, g)) return s;
    return pick_family(g, backward);
}

int na1d_set_kernel_family(int family) {
    if (family < -1 || family > 2) family = -1;
    return g_family_override.exchange(family);
}

int na1d_tensor_map_cache_stats(int64_t* hits, int64_t* misses) {
    NA1D_REQUIRE_PTR(hits); NA1D_REQUIRE_PTR(misses);
    long long h = 0, m = 0;
    na1d::tensor_map_cache_stats(&h, &m);
    *hits = h; *misses = m;
    return NA1D_OK;
}

int na1d_device_status(void) {
    // every word is read (and cleared) before anything is reported; an expired wait in any kernel wins over a failed read
    const int words[8] = {na1d::tc_read_status(), na1d::tc_bwd_read_status(), na1d::tc_seg_read_status(),
                          na1d::tc_bwd_seg_read_status(), na1d::tc_unfused_read_status(), na1d::tc_unfused_t_read_status(),
                          na1d::tc_drop_read_status(), na1d::tc_bwd_drop_read_status()};
    int v = 0, w = 0;
    for (int x : words) { if (x > 0) v = x; if (x < 0) w = x; }
    if (v > 0) return NA1D_ERR_DEVICE_TIMEOUT;
    if (w < 0) {
        const cudaError_t e = cudaGetLastError();
        return cuda_status(e == cudaSuccess ? cudaErrorUnknown : e);
    }
    return NA1D_OK;
}

int na1d_fused_forward(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                       const int32_t* valid_len, int64_t N, int64_t heads, int64_t T, int64_t C, int64_t win,
                       int64_t left, int64_t dil, float scale, int dtype, void* stream) {
    NA1D_REQUIRE_PTR(o); NA1D_REQUIRE_PTR(q); NA1D_REQUIRE_PTR(k); NA1D_REQUIRE_PTR(v);
    NA1D_REQUIRE_ALIGNED(o); NA1D_REQUIRE_ALIGNED(q); NA1D_REQUIRE_ALIGNED(k); NA1D_REQUIRE_ALIGNED(v);
    na1d::Geometry g;
    if (int s = check_geometry(N, heads, T, C, win, left, dil, dtype, scale, g)) return s;
    const int fam = pick_family(g, 0);
    if (fam < 0) return fam;
    if (fam == 1) return cuda_status(na1d::tc_fused_fwd(o, lse, q, k, v, rpb, valid_len, g, dtype, (cudaStream_t)stream));
    if (fam == 2) {
        const na1d::Strides d = na1d::dense_strides(g.H, g.T, g.C);
        return cuda_status(na1d::tc_fused_fwd_seg(o, lse, q, k, v, rpb, valid_len, d, d, d, d, g, dtype, (cudaStream_t)stream));
    }
    return cuda_status(na1d::simt_fused_fwd(o, lse, q, k, v, rpb, valid_len, g, dtype, (cudaStream_t)stream));
}

namespace {
// element strides (batch, head, token) given by the caller as three int64 on the host
int read_strides(const int64_t* p, int64_t batch, int64_t heads, int64_t T, int64_t C, na1d::Strides& out) {
    if (p == nullptr) return NA1D_ERR_NULL_POINTER;
    for (int i = 0; i < 3; ++i)
        if (p[i] <= 0 || p[i] % 8 != 0) return NA1D_ERR_BAD_STRIDE;
    if (p[2] < C) return NA1D_ERR_BAD_STRIDE;
    // the largest element offset must stay far inside int64 and inside what a tensor map can address (2^40 bytes per stride)
    const long double span = (long double)p[0] * (batch - 1) + (long double)p[1] * (heads - 1) + (long double)p[2] * (T - 1) + C;
    if (span > 4.0e12L || p[0] >= (1ll << 38) || p[1] >= (1ll << 38) || p[2] >= (1ll << 38)) return NA1D_ERR_BAD_STRIDE;
    out = na1d::Strides{(long long)p[0], (long long)p[1], (long long)p[2]};
    return NA1D_OK;
}
}  // namespace

int na1d_fused_strided_supported(int64_t heads, int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil, int dtype,
                                 int has_bias, int wants_bias_grad) {
    na1d::Geometry g;
    if (int s = check_geometry(heads, heads, T, C, win, left, dil, dtype, 1.f, g)) return s;
    return (na1d::tc_seg_supports(g) && na1d::tc_bwd_seg_supports(g, has_bias != 0, wants_bias_grad != 0)) ? 1 : 0;
}

int na1d_fused_forward_strided(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                               const int32_t* valid_len, const int64_t* o_strides, const int64_t* q_strides,
                               const int64_t* k_strides, const int64_t* v_strides, int64_t N, int64_t heads, int64_t T,
                               int64_t C, int64_t win, int64_t left, int64_t dil, float scale, int dtype, void* stream) {
    NA1D_REQUIRE_PTR(o); NA1D_REQUIRE_PTR(q); NA1D_REQUIRE_PTR(k); NA1D_REQUIRE_PTR(v);
    NA1D_REQUIRE_ALIGNED(o); NA1D_REQUIRE_ALIGNED(q); NA1D_REQUIRE_ALIGNED(k); NA1D_REQUIRE_ALIGNED(v);
    na1d::Geometry g;
    if (int s = check_geometry(N, heads, T, C, win, left, dil, dtype, scale, g)) return s;
    na1d::Strides so, sq, sk, sv;
    const int64_t batch = N / heads;
    if (int s = read_strides(o_strides, batch, heads, T, C, so)) return s;
    if (int s = read_strides(q_strides, batch, heads, T, C, sq)) return s;
    if (int s = read_strides(k_strides, batch, heads, T, C, sk)) return s;
    if (int s = read_strides(v_strides, batch, heads, T, C, sv)) return s;
    if (!na1d::tc_seg_supports(g)) return NA1D_ERR_UNSUPPORTED;
    return cuda_status(na1d::tc_fused_fwd_seg(o, lse, q, k, v, rpb, valid_len, sq, sk, sv, so, g, dtype, (cudaStream_t)stream));
}

int na1d_fused_backward_strided(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                                const void* v, const float* lse, const float* rpb, const int32_t* valid_len, float* scratch,
                                int64_t scratch_floats, const int64_t* dq_strides, const int64_t* dk_strides,
                                const int64_t* dv_strides, const int64_t* d_o_strides, const int64_t* q_strides,
                                const int64_t* k_strides, const int64_t* v_strides, int64_t N, int64_t heads, int64_t T,
                                int64_t C, int64_t win, int64_t left, int64_t dil, float scale, int dtype, void* stream) {
    NA1D_REQUIRE_PTR(dq); NA1D_REQUIRE_PTR(dk); NA1D_REQUIRE_PTR(dv); NA1D_REQUIRE_PTR(d_o); NA1D_REQUIRE_PTR(q);
    NA1D_REQUIRE_PTR(k); NA1D_REQUIRE_PTR(v); NA1D_REQUIRE_PTR(lse);
    NA1D_REQUIRE_ALIGNED(dq); NA1D_REQUIRE_ALIGNED(dk); NA1D_REQUIRE_ALIGNED(dv); NA1D_REQUIRE_ALIGNED(d_o);
    NA1D_REQUIRE_ALIGNED(q); NA1D_REQUIRE_ALIGNED(k); NA1D_REQUIRE_ALIGNED(v);
    na1d::Geometry g;
    if (int s = check_geometry(N, heads, T, C, win, left, dil, dtype, scale, g)) return s;
    if (d_rpb && heads * win * 4 > 48 * 1024) return NA1D_ERR_TOO_LARGE;
    if (scratch_floats < 0 || (scratch == nullptr && scratch_floats != 0)) return NA1D_ERR_NULL_POINTER;
    na1d::Strides s7[7];
    const int64_t* in[7] = {dq_strides, dk_strides, dv_strides, d_o_strides, q_strides, k_strides, v_strides};
    const int64_t batch = N / heads;
    for (int i = 0; i < 7; ++i)
        if (int s = read_strides(in[i], batch, heads, T, C, s7[i])) return s;
    if (!na1d::tc_bwd_seg_supports(g, rpb != nullptr, d_rpb != nullptr)) return NA1D_ERR_UNSUPPORTED;
    return cuda_status(na1d::tc_fused_bwd_seg(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, (size_t)scratch_floats,
                                              s7[0], s7[1], s7[2], s7[3], s7[4], s7[5], s7[6], g, dtype, (cudaStream_t)stream));
}

int na1d_fused_backward(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                        const void* v, const void* o, const float* lse, const float* rpb, const int32_t* valid_len,
                        float* delta_ws, int64_t N, int64_t heads, int64_t T, int64_t C, int64_t win, int64_t left,
                        int64_t dil, float scale, int dtype, void* stream) {
    NA1D_REQUIRE_PTR(dq); NA1D_REQUIRE_PTR(dk); NA1D_REQUIRE_PTR(dv); NA1D_REQUIRE_PTR(d_o); NA1D_REQUIRE_PTR(q);
    NA1D_REQUIRE_PTR(k); NA1D_REQUIRE_PTR(v); NA1D_REQUIRE_PTR(o); NA1D_REQUIRE_PTR(lse); NA1D_REQUIRE_PTR(delta_ws);
    NA1D_REQUIRE_ALIGNED(dq); NA1D_REQUIRE_ALIGNED(dk); NA1D_REQUIRE_ALIGNED(dv); NA1D_REQUIRE_ALIGNED(d_o);
    NA1D_REQUIRE_ALIGNED(q); NA1D_REQUIRE_ALIGNED(k); NA1D_REQUIRE_ALIGNED(v); NA1D_REQUIRE_ALIGNED(o);
    na1d::Geometry g;
    if (int s = check_geometry(N, heads, T, C, win, left, dil, dtype, scale, g)) return s;
    if (d_rpb && heads * win * 4 > 48 * 1024) return NA1D_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    const int fam = pick_family(g, 1, rpb != nullptr, d_rpb != nullptr);
    if (fam < 0) return fam;
    if (fam == 1)  // delta is recomputed inside the kernel from P and dP: o is not read; delta_ws (N*T floats) only holds the
                   // per-CTA partial sums of the bias gradient
        return cuda_status(na1d::tc_fused_bwd(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, delta_ws,
                                              (size_t)g.N * (size_t)g.T, g, dtype, st));
    if (fam == 2) {
        const na1d::Strides d = na1d::dense_strides(g.H, g.T, g.C);
        return cuda_status(na1d::tc_fused_bwd_seg(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, delta_ws,
                                                  (size_t)g.N * (size_t)g.T, d, d, d, d, d, d, d, g, dtype, st));
    }
    if (int s = cuda_status(na1d::simt_delta(delta_ws, d_o, o, g.N * g.T, g.C, dtype, st))) return s;
    return cuda_status(na1d::simt_fused_bwd(dq, dk, dv, d_rpb, d_o, q, k, v, lse, delta_ws, rpb, valid_len, g, dtype, st));
}

namespace {
int dropout_cfg(float drop_p, uint64_t seed, na1d::DropoutCfg& cfg) {
    if (!(drop_p >= 0.f) || drop_p >= 1.f) return NA1D_ERR_BAD_DROPOUT;
    const double th = (double)drop_p * 4294967296.0;
    cfg.threshold = th >= 4294967295.0 ? 4294967295u : (uint32_t)th;
    cfg.seed = (uint32_t)(seed ^ (seed >> 32));
    cfg.scale = 1.f / (1.f - drop_p);
    return NA1D_OK;
}
}  // namespace

int na1d_dropout_keep_mask(uint8_t* keep_host, int64_t rows, int64_t win, float drop_p, uint64_t seed) {
    NA1D_REQUIRE_PTR(keep_host);
    if (rows <= 0 || win <= 0 || rows > (int64_t)INT_MAX) return NA1D_ERR_BAD_SHAPE;
    na1d::DropoutCfg cfg;
    if (int s = dropout_cfg(drop_p, seed, cfg)) return s;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t kk = 0; kk < win; ++kk)
            keep_host[r * win + kk] = na1d::drop_hash((uint32_t)r, (uint32_t)kk, cfg.seed) >= cfg.threshold ? 1 : 0;
    return NA1D_OK;
}

int na1d_fused_forward_dropout(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                               const int32_t* valid_len, int64_t N, int64_t heads, int64_t T, int64_t C, int64_t win,
                               int64_t left, int64_t dil, float scale, float drop_p, uint64_t seed, int dtype, void* stream) {
    if (drop_p == 0.f) return na1d_fused_forward(o, lse, q, k, v, rpb, valid_len, N, heads, T, C, win, left, dil, scale, dtype, stream);
    NA1D_REQUIRE_PTR(o); NA1D_REQUIRE_PTR(q); NA1D_REQUIRE_PTR(k); NA1D_REQUIRE_PTR(v);
    NA1D_REQUIRE_ALIGNED(o); NA1D_REQUIRE_ALIGNED(q); NA1D_REQUIRE_ALIGNED(k); NA1D_REQUIRE_ALIGNED(v);
    na1d::Geometry g;
    if (int s = check_geometry(N, heads, T, C, win, left, dil, dtype, scale, g)) return s;
    na1d::DropoutCfg cfg;
    if (int s = dropout_cfg(drop_p, seed, cfg)) return s;
    if (!na1d::tc_fwd_supports(g)) return NA1D_ERR_UNSUPPORTED;
    return cuda_status(na1d::tc_fused_fwd_dropout(o, lse, q, k, v, rpb, valid_len, g, dtype, cfg, (cudaStream_t)stream));
}

int na1d_fused_backward_dropout(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                                const void* v, const float* lse, const float* rpb, const int32_t* valid_len, float* scratch,
                                int64_t scratch_floats, int64_t N, int64_t heads, int64_t T, int64_t C, int64_t win, int64_t left,
                                int64_t dil, float scale, float drop_p, uint64_t seed, int dtype, void* stream) {
    NA1D_REQUIRE_PTR(dq); NA1D_REQUIRE_PTR(dk); NA1D_REQUIRE_PTR(dv); NA1D_REQUIRE_PTR(d_o); NA1D_REQUIRE_PTR(q);
    NA1D_REQUIRE_PTR(k); NA1D_REQUIRE_PTR(v); NA1D_REQUIRE_PTR(lse);
    NA1D_REQUIRE_ALIGNED(dq); NA1D_REQUIRE_ALIGNED(dk); NA1D_REQUIRE_ALIGNED(dv); NA1D_REQUIRE_ALIGNED(d_o);
    NA1D_REQUIRE_ALIGNED(q); NA1D_REQUIRE_ALIGNED(k); NA1D_REQUIRE_ALIGNED(v);
    na1d::Geometry g;
    if (int s = check_geometry(N, heads, T, C, win, left, dil, dtype, scale, g)) return s;
    if (d_rpb && heads * win * 4 > 48 * 1024) return NA1D_ERR_TOO_LARGE;
    if (scratch_floats < 0 || (scratch == nullptr && scratch_floats != 0)) return NA1D_ERR_NULL_POINTER;
    na1d::DropoutCfg cfg;
    if (int s = dropout_cfg(drop_p, seed, cfg)) return s;
    if (!na1d::tc_bwd_supports(g, rpb != nullptr, d_rpb != nullptr)) return NA1D_ERR_UNSUPPORTED;
    return cuda_status(na1d::tc_fused_bwd_dropout(dq, dk, dv, d_rpb, d_o, q, k, v, lse, rpb, valid_len, scratch, (size_t)scratch_floats,
                                                  g, dtype, cfg, (cudaStream_t)stream));
}

int na1d_window_index(int32_t* j_out, uint8_t* in_range, int64_t T, int64_t win, int64_t left, int64_t dil,
                      void* stream) {
    NA1D_REQUIRE_PTR(j_out); NA1D_REQUIRE_PTR(in_range);
    na1d::Geometry g;
    if (int s = check_geometry(1, 1, T, 8, win, left, dil, NA1D_BF16, 1.f, g)) return s;
    return cuda_status(na1d::window_index(j_out, in_range, g.T, g.win, g.left, g.dil, (cudaStream_t)stream));
}

// ---------------------------------------------------------------------------------------------
// Backward pass without a caller-provided workspace (see the header for who needs this and why).
// The delta workspace of the CUDA-core backward lives in this file-scope device array. In host code
// the name below is only a handle for the runtime; the address a kernel can use is obtained once per
// device with cudaGetSymbolAddress and cached.
static __device__ __align__(256) float g_static_delta[NA1D_STATIC_SCRATCH_ROWS];

namespace {
std::mutex g_static_mutex;
float* g_static_delta_addr[64] = {nullptr};

// Device address of g_static_delta on the current device; looked up on the first call per device.
int static_delta_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e);
    if (dev < 0 || dev >= 64) return NA1D_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_delta_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_delta);  // needs `dev` current, which it is
        if (e != cudaSuccess) return cuda_status(e);
        if (p == nullptr) return NA1D_ERR_CUDA;
        g_static_delta_addr[dev] = static_cast<float*>(p);
    }
    *out = g_static_delta_addr[dev];
    return NA1D_OK;
}
}  // namespace

int na1d_fused_backward_static(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                               const void* v, const void* o, const float* lse, const float* rpb, const int32_t* valid_len,
                               int64_t N, int64_t heads, int64_t T, int64_t C, int64_t win, int64_t left, int64_t dil,
                               float scale, int dtype, void* stream) {
    NA1D_REQUIRE_PTR(dq); NA1D_REQUIRE_PTR(dk); NA1D_REQUIRE_PTR(dv); NA1D_REQUIRE_PTR(d_o); NA1D_REQUIRE_PTR(q);
    NA1D_REQUIRE_PTR(k); NA1D_REQUIRE_PTR(v); NA1D_REQUIRE_PTR(o); NA1D_REQUIRE_PTR(lse);
    NA1D_REQUIRE_ALIGNED(dq); NA1D_REQUIRE_ALIGNED(dk); NA1D_REQUIRE_ALIGNED(dv); NA1D_REQUIRE_ALIGNED(d_o);
    NA1D_REQUIRE_ALIGNED(q); NA1D_REQUIRE_ALIGNED(k); NA1D_REQUIRE_ALIGNED(v); NA1D_REQUIRE_ALIGNED(o);
    na1d::Geometry g;
    if (int s = check_geometry(N, heads, T, C, win, left, dil, dtype, scale, g)) return s;
    if (N * T > (int64_t)NA1D_STATIC_SCRATCH_ROWS) return NA1D_ERR_TOO_LARGE;  // the fixed workspace holds N*T floats
    if (d_rpb && heads * win * 4 > 48 * 1024) return NA1D_ERR_TOO_LARGE;
    float* delta = nullptr;
    if (int s = static_delta_address(&delta)) return s;
    cudaStream_t st = (cudaStream_t)stream;
    // The pre-pass writes delta[0 .. N*T) completely before the main kernel reads it, on the same stream:
    // leftovers of earlier calls are never observed.
    if (int s = cuda_status(na1d::simt_delta(delta, d_o, o, g.N * g.T, g.C, dtype, st))) return s;
    return cuda_status(na1d::simt_fused_bwd(dq, dk, dv, d_rpb, d_o, q, k, v, lse, delta, rpb, valid_len, g, dtype, st));
}

}  // extern "C"

// CUDA-core NA1D kernels: the general path (any window <= NA1D_MAX_WINDOW, any dilation, any
// channel count the ABI accepts, bf16/fp16). A group of G lanes owns one sequence row; each lane
// holds CHUNKS 16-byte chunks of the row, interleaved so a group reads a row as one coalesced
// segment. Dot products are reduced over the group with xor shuffles. All arithmetic is fp32.
//
// Replaces, for shapes the tensor-core kernels do not take: ana_qk_forward_kernel_C16/_C8
// (na1d_tensorcore/bf16_ana1d_kernel.cu:42-282), ana_q_backward_kernel (:285-391) and
// ana_k_backward_kernel (:394-492) of the reference, plus the eager softmax chain between them
// (models/PCF_NATransformer.py:141-150).
#include "na1d_internal.h"

namespace na1d {
namespace {

constexpr int kThreads = 128;

template <int G> __device__ __forceinline__ float group_sum(float x) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

template <typename E, int G, int CHUNKS>
__device__ __forceinline__ void load_row(const E* __restrict__ base, size_t row, int C, int g, float (&f)[CHUNKS][8]) {
    const uint4* p = reinterpret_cast<const uint4*>(base + row * (size_t)C);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) { uint4 u = __ldg(p + c * G + g); Cvt<E>::unpack(u, f[c]); }
}
template <typename E, int G, int CHUNKS>
__device__ __forceinline__ void store_row(E* __restrict__ base, size_t row, int C, int g, const float (&f)[CHUNKS][8]) {
    uint4* p = reinterpret_cast<uint4*>(base + row * (size_t)C);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) p[c * G + g] = Cvt<E>::pack(f[c]);
}
template <int CHUNKS> __device__ __forceinline__ float dot(const float (&a)[CHUNKS][8], const float (&b)[CHUNKS][8]) {
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) s = fmaf(a[c][i], b[c][i], s);
    return s;
}
template <int CHUNKS> __device__ __forceinline__ void axpy(float a, const float (&x)[CHUNKS][8], float (&y)[CHUNKS][8]) {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) y[c][i] = fmaf(a, x[c][i], y[c][i]);
}
template <int CHUNKS> __device__ __forceinline__ void zero(float (&y)[CHUNKS][8]) {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) y[c][i] = 0.f;
}

// ---------------------------------------------------------------- unfused pair
// attn[row,kk] = a[row] . b[n, j(t,kk)]   (QK forward, and dA = dO.V^T)
template <typename E, int G, int CHUNKS>
__global__ void __launch_bounds__(kThreads) qk_kernel(float* __restrict__ attn, const E* __restrict__ a,
                                                     const E* __restrict__ b, Geometry gm, int rows) {
    const int g = threadIdx.x % G;
    int row = blockIdx.x * (kThreads / G) + threadIdx.x / G;
    const bool live = row < rows;
    if (!live) row = rows - 1;
    const int n = row / gm.T, t = row - n * gm.T;
    float qa[CHUNKS][8], kb[CHUNKS][8];
    load_row<E, G, CHUNKS>(a, row, gm.C, g, qa);
    for (int kk = 0; kk < gm.win; ++kk) {
        const int j = neighbour(t, kk, gm.left, gm.dil);
        float s = 0.f;
        if (in_range(j, gm.T)) {
            load_row<E, G, CHUNKS>(b, (size_t)n * gm.T + j, gm.C, g, kb);
            s = dot<CHUNKS>(qa, kb);
        }
        s = group_sum<G>(s);
        if (live && g == (kk % G)) attn[(size_t)row * gm.win + kk] = s;
    }
}

// out[row] = sum_kk band[row,kk] * x[n, j(t,kk)]   (AV forward, dQ)
template <typename E, int G, int CHUNKS>
__global__ void __launch_bounds__(kThreads) band_x_kernel(E* __restrict__ out, const float* __restrict__ band,
                                                         const E* __restrict__ x, Geometry gm, int rows) {
    const int g = threadIdx.x % G;
    const int row = blockIdx.x * (kThreads / G) + threadIdx.x / G;
    if (row >= rows) return;
    const int n = row / gm.T, t = row - n * gm.T;
    float acc[CHUNKS][8], xr[CHUNKS][8];
    zero<CHUNKS>(acc);
    for (int kk = 0; kk < gm.win; ++kk) {
        const int j = neighbour(t, kk, gm.left, gm.dil);
        if (!in_range(j, gm.T)) continue;
        const float w = __ldg(band + (size_t)row * gm.win + kk);
        load_row<E, G, CHUNKS>(x, (size_t)n * gm.T + j, gm.C, g, xr);
        axpy<CHUNKS>(w, xr, acc);
    }
    store_row<E, G, CHUNKS>(out, row, gm.C, g, acc);
}

// out[n,j] = sum_kk band[(n,tq),kk] * x[n,tq],  tq = j - (kk-left)*dil in [0,T)   (dK, dV)
template <typename E, int G, int CHUNKS>
__global__ void __launch_bounds__(kThreads) bandT_x_kernel(E* __restrict__ out, const float* __restrict__ band,
                                                          const E* __restrict__ x, Geometry gm, int rows) {
    const int g = threadIdx.x % G;
    const int row = blockIdx.x * (kThreads / G) + threadIdx.x / G;
    if (row >= rows) return;
    const int n = row / gm.T, j = row - n * gm.T;
    float acc[CHUNKS][8], xr[CHUNKS][8];
    zero<CHUNKS>(acc);
    for (int kk = 0; kk < gm.win; ++kk) {
        const int tq = j - (kk - gm.left) * gm.dil;
        if (!in_range(tq, gm.T)) continue;
        const size_t r = (size_t)n * gm.T + tq;
        const float w = __ldg(band + r * gm.win + kk);
        load_row<E, G, CHUNKS>(x, r, gm.C, g, xr);
        axpy<CHUNKS>(w, xr, acc);
    }
    store_row<E, G, CHUNKS>(out, row, gm.C, g, acc);
}

// ---------------------------------------------------------------- fused forward
__device__ __forceinline__ float mask_term(int t, int j, int T, int vl) {
    return (j < 0 || j >= T || j >= vl || t >= vl) ? kMaskValue : 0.f;
}

template <typename E, int G, int CHUNKS>
__global__ void __launch_bounds__(kThreads) fused_fwd_kernel(E* __restrict__ o, float* __restrict__ lse,
                                                            const E* __restrict__ q, const E* __restrict__ k,
                                                            const E* __restrict__ v, const float* __restrict__ rpb,
                                                            const int* __restrict__ valid_len, Geometry gm, int rows) {
    const int g = threadIdx.x % G;
    int row = blockIdx.x * (kThreads / G) + threadIdx.x / G;
    const bool live = row < rows;
    if (!live) row = rows - 1;
    const int n = row / gm.T, t = row - n * gm.T;
    const int h = n % gm.H;
    const int vl = valid_len ? __ldg(valid_len + n / gm.H) : gm.T;
    float qf[CHUNKS][8], xr[CHUNKS][8], acc[CHUNKS][8];
    load_row<E, G, CHUNKS>(q, row, gm.C, g, qf);
    zero<CHUNKS>(acc);
    float m = -INFINITY, l = 0.f;  // running max / sum in the log2 domain
    const float sc = gm.scale * kLog2e;
    for (int kk = 0; kk < gm.win; ++kk) {
        const int j = neighbour(t, kk, gm.left, gm.dil);
        const bool inr = in_range(j, gm.T);
        const size_t r = (size_t)n * gm.T + (inr ? j : 0);
        float s = 0.f;
        if (inr) { load_row<E, G, CHUNKS>(k, r, gm.C, g, xr); s = dot<CHUNKS>(qf, xr); }
        s = group_sum<G>(s) * sc;
        const float b = (rpb ? __ldg(rpb + h * gm.win + kk) : 0.f) + mask_term(t, j, gm.T, vl);
        s = fmaf(b, kLog2e, s);
        const float mn = fmaxf(m, s);
        const float alpha = exp2f(m - mn), p = exp2f(s - mn);
        l = fmaf(l, alpha, p);
        m = mn;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[c][i] *= alpha;
        if (inr) { load_row<E, G, CHUNKS>(v, r, gm.C, g, xr); axpy<CHUNKS>(p, xr, acc); }
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[c][i] *= inv;
    if (live) {
        store_row<E, G, CHUNKS>(o, row, gm.C, g, acc);
        if (lse && g == 0) lse[row] = (m + log2f(l)) * kLn2;
    }
}

// ---------------------------------------------------------------- fused backward
// delta[row] = sum_c dO[row,c] * O[row,c]
template <typename E, int G, int CHUNKS>
__global__ void __launch_bounds__(kThreads) delta_kernel(float* __restrict__ delta, const E* __restrict__ d_o,
                                                        const E* __restrict__ o, int C, int rows) {
    const int g = threadIdx.x % G;
    int row = blockIdx.x * (kThreads / G) + threadIdx.x / G;
    const bool live = row < rows;
    if (!live) row = rows - 1;
    float a[CHUNKS][8], b[CHUNKS][8];
    load_row<E, G, CHUNKS>(d_o, row, C, g, a);
    load_row<E, G, CHUNKS>(o, row, C, g, b);
    const float s = group_sum<G>(dot<CHUNKS>(a, b));
    if (live && g == 0) delta[row] = s;
}

// One group owns row t twice: as a query (dQ[t], d_rpb) and as a key (dK[t], dV[t]); the band is
// recomputed from the saved log-sum-exp in both views, so no atomics on dK/dV are needed and the
// result is deterministic.
template <typename E, int G, int CHUNKS>
__global__ void __launch_bounds__(kThreads) fused_bwd_kernel(E* __restrict__ dq, E* __restrict__ dk, E* __restrict__ dv,
                                                            float* __restrict__ d_rpb, const E* __restrict__ d_o,
                                                            const E* __restrict__ q, const E* __restrict__ k,
                                                            const E* __restrict__ v, const float* __restrict__ lse,
                                                            const float* __restrict__ delta, const float* __restrict__ rpb,
                                                            const int* __restrict__ valid_len, Geometry gm, int rows) {
    extern __shared__ float s_drpb[];  // [H*win] when d_rpb != nullptr
    if (d_rpb) {
        for (int i = threadIdx.x; i < gm.H * gm.win; i += kThreads) s_drpb[i] = 0.f;
        __syncthreads();
    }
    const int g = threadIdx.x % G;
    int row = blockIdx.x * (kThreads / G) + threadIdx.x / G;
    const bool live = row < rows;
    if (!live) row = rows - 1;
    const int n = row / gm.T, t = row - n * gm.T;
    const int h = n % gm.H;
    const int vl = valid_len ? __ldg(valid_len + n / gm.H) : gm.T;
    const float sc = gm.scale * kLog2e;

    float own_a[CHUNKS][8], own_b[CHUNKS][8], xr[CHUNKS][8], yr[CHUNKS][8], acc[CHUNKS][8], acc2[CHUNKS][8];
    // ---- query view: dQ[t] = scale * sum_kk dS[kk] * k[j]
    {
        load_row<E, G, CHUNKS>(q, row, gm.C, g, own_a);
        load_row<E, G, CHUNKS>(d_o, row, gm.C, g, own_b);
        const float lse_t = __ldg(lse + row) * kLog2e, dl = __ldg(delta + row);
        zero<CHUNKS>(acc);
        for (int kk = 0; kk < gm.win; ++kk) {
            const int j = neighbour(t, kk, gm.left, gm.dil);
            const bool inr = in_range(j, gm.T);
            float s = 0.f, dp = 0.f;
            if (inr) {
                const size_t r = (size_t)n * gm.T + j;
                load_row<E, G, CHUNKS>(k, r, gm.C, g, xr);
                load_row<E, G, CHUNKS>(v, r, gm.C, g, yr);
                s = dot<CHUNKS>(own_a, xr);
                dp = dot<CHUNKS>(own_b, yr);
            }
            s = group_sum<G>(s) * sc;
            dp = group_sum<G>(dp);
            const float b = (rpb ? __ldg(rpb + h * gm.win + kk) : 0.f) + mask_term(t, j, gm.T, vl);
            const float p = exp2f(fmaf(b, kLog2e, s) - lse_t);
            const float ds = p * (dp - dl);
            if (inr) axpy<CHUNKS>(ds, xr, acc);
            if (d_rpb && live && g == 0) atomicAdd(&s_drpb[h * gm.win + kk], ds);
        }
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[c][i] *= gm.scale;
        if (live) store_row<E, G, CHUNKS>(dq, row, gm.C, g, acc);
    }
    // ---- key view: dK[t] = scale * sum dS * q[tq],  dV[t] = sum P * dO[tq]
    {
        load_row<E, G, CHUNKS>(k, row, gm.C, g, own_a);
        load_row<E, G, CHUNKS>(v, row, gm.C, g, own_b);
        zero<CHUNKS>(acc);
        zero<CHUNKS>(acc2);
        for (int kk = 0; kk < gm.win; ++kk) {
            const int tq = t - (kk - gm.left) * gm.dil;
            const bool inr = in_range(tq, gm.T);
            const size_t r = (size_t)n * gm.T + (inr ? tq : 0);
            float s = 0.f, dp = 0.f;
            if (inr) {
                load_row<E, G, CHUNKS>(q, r, gm.C, g, xr);
                load_row<E, G, CHUNKS>(d_o, r, gm.C, g, yr);
                s = dot<CHUNKS>(xr, own_a);
                dp = dot<CHUNKS>(yr, own_b);
            }
            s = group_sum<G>(s) * sc;
            dp = group_sum<G>(dp);
            if (inr) {
                const float b = (rpb ? __ldg(rpb + h * gm.win + kk) : 0.f) + mask_term(tq, t, gm.T, vl);
                const float p = exp2f(fmaf(b, kLog2e, s) - __ldg(lse + r) * kLog2e);
                const float ds = p * (dp - __ldg(delta + r));
                axpy<CHUNKS>(ds, xr, acc);
                axpy<CHUNKS>(p, yr, acc2);
            }
        }
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[c][i] *= gm.scale;
        if (live) {
            store_row<E, G, CHUNKS>(dk, row, gm.C, g, acc);
            store_row<E, G, CHUNKS>(dv, row, gm.C, g, acc2);
        }
    }
    if (d_rpb) {
        __syncthreads();
        for (int i = threadIdx.x; i < gm.H * gm.win; i += kThreads) {
            const float x = s_drpb[i];
            if (x != 0.f) atomicAdd(d_rpb + i, x);
        }
    }
}

__global__ void window_index_kernel(int* __restrict__ j_out, unsigned char* __restrict__ inr, int T, int win, int left,
                                    int dil) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * win) return;
    const int t = i / win, kk = i - t * win;
    const int j = neighbour(t, kk, left, dil);
    j_out[i] = j;
    inr[i] = in_range(j, T) ? 1 : 0;
}

// ---------------------------------------------------------------- dispatch on (dtype, G, CHUNKS)
struct Split { int G, chunks; };
inline bool split_channels(int C, Split& s) {
    int n = C / 8, G = 1;
    while (G < 8 && n % 2 == 0) { G *= 2; n /= 2; }
    s.G = G; s.chunks = n;
    return n >= 1 && n <= 4;
}

#define NA1D_DISPATCH_GC(E, sp, CALL)                                                     \
    switch ((sp).G * 8 + (sp).chunks) {                                                   \
        case 1 * 8 + 1: { constexpr int G = 1, CH = 1; CALL; } break;                     \
        case 1 * 8 + 3: { constexpr int G = 1, CH = 3; CALL; } break;                     \
        case 2 * 8 + 1: { constexpr int G = 2, CH = 1; CALL; } break;                     \
        case 2 * 8 + 3: { constexpr int G = 2, CH = 3; CALL; } break;                     \
        case 4 * 8 + 1: { constexpr int G = 4, CH = 1; CALL; } break;                     \
        case 4 * 8 + 3: { constexpr int G = 4, CH = 3; CALL; } break;                     \
        case 8 * 8 + 1: { constexpr int G = 8, CH = 1; CALL; } break;                     \
        case 8 * 8 + 2: { constexpr int G = 8, CH = 2; CALL; } break;                     \
        case 8 * 8 + 3: { constexpr int G = 8, CH = 3; CALL; } break;                     \
        case 8 * 8 + 4: { constexpr int G = 8, CH = 4; CALL; } break;                     \
        default: return cudaErrorInvalidValue;                                            \
    }

#define NA1D_DISPATCH(dtype, sp, CALL)                                                    \
    if ((dtype) == 0) { using E = __nv_bfloat16; NA1D_DISPATCH_GC(E, sp, CALL) }          \
    else { using E = __half; NA1D_DISPATCH_GC(E, sp, CALL) }

inline int grid_for(int rows, int G) { return (rows + kThreads / G - 1) / (kThreads / G); }

}  // namespace

bool simt_supports_channels(int C) { Split s; return C % 8 == 0 && split_channels(C, s); }

cudaError_t simt_qk(float* attn, const void* a, const void* b, const Geometry& gm, int dtype, cudaStream_t st) {
    Split sp; if (!split_channels(gm.C, sp)) return cudaErrorInvalidValue;
    const int rows = gm.N * gm.T;
    NA1D_DISPATCH(dtype, sp, (qk_kernel<E, G, CH><<<grid_for(rows, G), kThreads, 0, st>>>(attn, (const E*)a, (const E*)b, gm, rows)));
    return cudaGetLastError();
}
cudaError_t simt_band_x(void* out, const float* band, const void* x, const Geometry& gm, int dtype, cudaStream_t st) {
    Split sp; if (!split_channels(gm.C, sp)) return cudaErrorInvalidValue;
    const int rows = gm.N * gm.T;
    NA1D_DISPATCH(dtype, sp, (band_x_kernel<E, G, CH><<<grid_for(rows, G), kThreads, 0, st>>>((E*)out, band, (const E*)x, gm, rows)));
    return cudaGetLastError();
}
cudaError_t simt_bandT_x(void* out, const float* band, const void* x, const Geometry& gm, int dtype, cudaStream_t st) {
    Split sp; if (!split_channels(gm.C, sp)) return cudaErrorInvalidValue;
    const int rows = gm.N * gm.T;
    NA1D_DISPATCH(dtype, sp, (bandT_x_kernel<E, G, CH><<<grid_for(rows, G), kThreads, 0, st>>>((E*)out, band, (const E*)x, gm, rows)));
    return cudaGetLastError();
}
cudaError_t simt_fused_fwd(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                           const int* valid_len, const Geometry& gm, int dtype, cudaStream_t st) {
    Split sp; if (!split_channels(gm.C, sp)) return cudaErrorInvalidValue;
    const int rows = gm.N * gm.T;
    NA1D_DISPATCH(dtype, sp, (fused_fwd_kernel<E, G, CH><<<grid_for(rows, G), kThreads, 0, st>>>(
        (E*)o, lse, (const E*)q, (const E*)k, (const E*)v, rpb, valid_len, gm, rows)));
    return cudaGetLastError();
}
cudaError_t simt_delta(float* delta, const void* d_o, const void* o, int rows, int C, int dtype, cudaStream_t st) {
    Split sp; if (!split_channels(C, sp)) return cudaErrorInvalidValue;
    NA1D_DISPATCH(dtype, sp, (delta_kernel<E, G, CH><<<grid_for(rows, G), kThreads, 0, st>>>(delta, (const E*)d_o, (const E*)o, C, rows)));
    return cudaGetLastError();
}
cudaError_t simt_fused_bwd(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                           const void* v, const float* lse, const float* delta, const float* rpb, const int* valid_len,
                           const Geometry& gm, int dtype, cudaStream_t st) {
    Split sp; if (!split_channels(gm.C, sp)) return cudaErrorInvalidValue;
    const int rows = gm.N * gm.T;
    const size_t smem = d_rpb ? sizeof(float) * gm.H * gm.win : 0;
    NA1D_DISPATCH(dtype, sp, (fused_bwd_kernel<E, G, CH><<<grid_for(rows, G), kThreads, smem, st>>>(
        (E*)dq, (E*)dk, (E*)dv, d_rpb, (const E*)d_o, (const E*)q, (const E*)k, (const E*)v, lse, delta, rpb, valid_len, gm, rows)));
    return cudaGetLastError();
}
cudaError_t window_index(int* j_out, unsigned char* inr, int T, int win, int left, int dil, cudaStream_t st) {
    const int total = T * win;
    window_index_kernel<<<(total + 255) / 256, 256, 0, st>>>(j_out, inr, T, win, left, dil);
    return cudaGetLastError();
}

}  // namespace na1d

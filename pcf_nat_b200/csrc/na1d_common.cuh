// Shared device/host helpers for the NA1D kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace na1d {

// Additive logit for a masked neighbour. The reference adds -100 instead of excluding the
// neighbour (models/PCF_NATransformer.py:98), which keeps fully masked rows finite.
constexpr float kMaskValue = -100.0f;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// The single definition of the window index arithmetic used by every kernel:
// neighbour kk of query t is key t + (kk-left)*dil  (pad+unfold of
// models/PCF_NATransformer.py:158-165 made explicit).
__host__ __device__ __forceinline__ int neighbour(int t, int kk, int left, int dil) {
    return t + (kk - left) * dil;
}
__host__ __device__ __forceinline__ bool in_range(int j, int T) { return j >= 0 && j < T; }

struct Geometry {
    int N, H, T, C, win, left, dil;
    float scale;
};

// Element strides of a 16-bit tensor addressed as [batch][head][token][channel] (channel stride 1). A dense (N, T, C)
// tensor with n = batch * H + head has {H*T*C, T*C, C}; the q/k/v slices of a packed (batch, T, 3, H, C) projection
// output have {T*3*H*C, C, 3*H*C}.
struct Strides {
    long long batch, head, token;
};
__host__ __device__ inline Strides dense_strides(int H, int T, int C) {
    return Strides{(long long)H * T * C, (long long)T * C, (long long)C};
}

// Segmented tiling: the rows t = r (mod d) of one (batch, head) sequence form a residue sequence of Tp or Tp - 1 tokens
// on which a window of dilation d is an ordinary window of dilation 1; tiles never leave their residue sequence.
struct SegGeom {
    int d;     // residue classes per sequence (the dilation), >= 1
    int ra;    // residues r < ra have Tp tokens, the others Tp - 1 (ra = d when d divides T)
    int Tp;    // ceil(T / d)
    int tps;   // tiles per residue sequence
    int step;  // rows between the first rows of consecutive tiles of a sequence
};

// Attention dropout (models/PCF_NATransformer.py:149: nn.Dropout on the probabilities). The keep decision of probability
// (row, kk) is a pure function of a 32-bit seed, the dense row index n*T + t and the neighbour index kk, so the forward and
// the backward kernels (and the CPU oracle, which restates this function) derive the same mask without storing it:
// keep iff drop_hash(...) >= threshold, threshold = p * 2^32.
struct DropoutCfg {
    uint32_t threshold;   // 0 = no dropout
    uint32_t seed;
    float scale;          // 1 / (1 - p)
};
__host__ __device__ __forceinline__ uint32_t drop_hash(uint32_t row, uint32_t kk, uint32_t seed) {
    uint32_t x = row * 2654435761u + kk * 0x632BE5ABu + seed;
    x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
    return x;
}

// 8 consecutive 16-bit elements (one 16-byte chunk) <-> 8 floats
template <typename E> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        uint4 u; __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        return u;
    }
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t);
    }
    static __device__ __forceinline__ float from_bits(unsigned short raw) { return __uint_as_float((uint32_t)raw << 16); }
};
template <> struct Cvt<__half> {
    static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
        const __half2* p = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 t = __half22float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        uint4 u; __half2* p = reinterpret_cast<__half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        return u;
    }
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __half2 t = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&t);
    }
    static __device__ __forceinline__ float from_bits(unsigned short raw) { return __half2float(__ushort_as_half(raw)); }
};

}  // namespace na1d

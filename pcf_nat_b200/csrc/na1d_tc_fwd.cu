// Fused NA1D forward on the Blackwell tensor path (sm_100a): TMA-staged tiles, tcgen05 MMAs with
// accumulators in tensor memory, softmax on the band only.
//
// One CTA (128 threads, cluster size 1) owns one tile of 128 queries of one sequence:
//   1. thread 0 issues three plain (non-multicast) TMA tile loads: Q[128 x C], and K, V rows
//      [t0-left, t0-left+KT) with KT = round16(128 + win - 1). Rows outside [0,T) arrive as zeros
//      (TMA out-of-bounds fill), which is exactly the reference's zero padding of K and V
//      (na1d_tensorcore/bf16_ana1d_kernel.cu:99-112).
//   2. S = Q.K^T as C/16 tcgen05.mma steps (M=128, N=KT) into TMEM columns [0,KT).
//   3. each thread owns one query row (TMEM lane = row). Warp w reads columns [32w, 32w+31+win] of
//      its 32 lanes, every lane rotates its registers by its lane id (5-stage barrel shifter) so the
//      band sits at register 0..win-1, then scale, + rpb, + (-100) mask, softmax in fp32, and the
//      normalised probabilities go to shared memory as 16-bit values in the canonical K-major
//      core-matrix layout (zeros elsewhere) -- the reference rounds probabilities to 16 bits before
//      its A.V product too (bf16_ana1d_kernel.cu:301-306).
//   4. O = P.V as KT/16 tcgen05.mma steps (M=128, N=C) with V as an MN-major operand straight from
//      the TMA tile; O is read back from TMEM and stored.
// Every wait is bounded; on expiry the CTA records a code in a device status word and unwinds
// (TMEM is always released).
#include "na1d_internal.h"
#include "na1d_ptx.cuh"

namespace na1d {

__device__ int g_tc_status = 0;

namespace {

constexpr int kTileM = 128;
constexpr int kTmemCols = 256;
constexpr int kOCol = 192;  // O accumulator starts here; S uses [0, KT) with KT <= 192

template <int C> struct RowSwizzle;
template <> struct RowSwizzle<64> { static constexpr uint64_t umma = ptx::kSwizzle128B; };
template <> struct RowSwizzle<32> { static constexpr uint64_t umma = ptx::kSwizzle64B; };
template <> struct RowSwizzle<16> { static constexpr uint64_t umma = ptx::kSwizzle32B; };

template <typename E> struct Fmt;
template <> struct Fmt<__nv_bfloat16> { static constexpr uint32_t v = 1; };
template <> struct Fmt<__half> { static constexpr uint32_t v = 0; };

__host__ __device__ constexpr int round_up(int x, int m) { return (x + m - 1) / m * m; }

struct FwdSmemLayout {
    int q, k, v, p, misc, total;
};
__host__ __device__ inline FwdSmemLayout fwd_layout(int C, int KT) {
    FwdSmemLayout L;
    L.q = 0;
    L.k = L.q + round_up(kTileM * C * 2, 1024);
    L.v = L.k + round_up(KT * C * 2, 1024);
    L.p = L.v + round_up(KT * C * 2, 1024);
    L.misc = L.p + round_up(kTileM * KT * 2, 1024);
    L.total = L.misc + 1024 + 1024;  // + misc block + slack for manual 1024-byte alignment
    return L;
}

struct alignas(8) FwdMisc {
    uint64_t bar_full, bar_s, bar_o;
    uint32_t tmem_base;
    float rpb[64];
};

template <typename E, int C, int WB, bool PT>
__global__ void __launch_bounds__(128, 2)
tc_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, E* __restrict__ o, float* __restrict__ lse,
              const float* __restrict__ rpb, const int* __restrict__ valid_len, Geometry gm, int tiles_per_seq, int KT) {
    constexpr int LW = round_up(WB + 31, 16);  // TMEM columns each warp reads
    constexpr int kRowBytes = C * 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const FwdSmemLayout L = fwd_layout(C, KT);
    uint8_t* sQ = smem + L.q;
    uint8_t* sK = smem + L.k;
    uint8_t* sV = smem + L.v;
    uint8_t* sP = smem + L.p;
    FwdMisc* misc = reinterpret_cast<FwdMisc*>(smem + L.misc);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n = blockIdx.x / tiles_per_seq;
    const int t0 = (blockIdx.x - n * tiles_per_seq) * kTileM;
    const int h = n % gm.H;
    const int win = gm.win, left = gm.left, T = gm.T;

    if (tid == 0) {
        ptx::mbar_init(&misc->bar_full, 1);
        ptx::mbar_init(&misc->bar_s, 1);
        ptx::mbar_init(&misc->bar_o, 1);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tm_q);
        ptx::prefetch_tensormap(&tm_k);
        ptx::prefetch_tensormap(&tm_v);
    }
    if (warp == 0) {
        __syncwarp();
        ptx::tmem_alloc(&misc->tmem_base, kTmemCols);
        ptx::tmem_relinquish();
    }
    if constexpr (!PT) {   // P starts as zeros; only band entries are written later
        uint4* p4 = reinterpret_cast<uint4*>(sP);
        const int n16 = kTileM * KT * 2 / 16;
        for (int i = tid; i < n16; i += 128) p4[i] = make_uint4(0, 0, 0, 0);
    }
    if (tid < win) misc->rpb[tid] = rpb ? __ldg(rpb + h * win + tid) : 0.f;
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = misc->tmem_base;
    bool ok = true;

    // ---- loads and S = Q.K^T (one thread)
    if (tid == 0) {
        ptx::mbar_expect_tx(&misc->bar_full, (uint32_t)((kTileM + 2 * KT) * kRowBytes));
        ptx::tma_load_3d(sQ, &tm_q, &misc->bar_full, 0, t0, n);
        ptx::tma_load_3d(sK, &tm_k, &misc->bar_full, 0, t0 - left, n);
        ptx::tma_load_3d(sV, &tm_v, &misc->bar_full, 0, t0 - left, n);
        ok = ptx::mbar_wait(&misc->bar_full, 0);
        ptx::tc_fence_after_sync();
        if (ok) {
            const uint32_t idesc = ptx::instr_desc(Fmt<E>::v, 0, 0, kTileM, (uint32_t)KT);
            const uint32_t qa = ptx::smem_u32(sQ), ka = ptx::smem_u32(sK);
#pragma unroll
            for (int ks = 0; ks < C / 16; ++ks) {
                const uint64_t ad = ptx::smem_desc(qa + ks * 32, 16, 8 * kRowBytes, RowSwizzle<C>::umma);
                const uint64_t bd = ptx::smem_desc(ka + ks * 32, 16, 8 * kRowBytes, RowSwizzle<C>::umma);
                ptx::mma_ss(tmem, ad, bd, idesc, ks > 0 ? 1u : 0u);
            }
        } else {
            atomicExch(&g_tc_status, 1);
        }
        ptx::mma_commit(&misc->bar_s);
    }
    __syncwarp();

    // ---- softmax over the band: one thread per query row
    if (!ptx::mbar_wait(&misc->bar_s, 0)) { ok = false; atomicExch(&g_tc_status, 2); }
    ptx::tc_fence_after_sync();
    const int r = warp * 32 + lane;
    const int t = t0 + r;
    {
        float s[LW];
        const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(warp * 32);
#pragma unroll
        for (int c = 0; c < LW; c += 8) ptx::tmem_ld8(taddr + c, &s[c]);
        ptx::tmem_ld_wait();
        // rotate left by `lane`: afterwards s[kk] is the logit of neighbour kk of this row
#pragma unroll
        for (int b = 16; b >= 1; b >>= 1) {
            const bool on = (lane & b) != 0;
#pragma unroll
            for (int i = 0; i < WB + b - 1; ++i) s[i] = on ? s[i + b] : s[i];
        }
        const int vl = valid_len ? __ldg(valid_len + n / gm.H) : T;
        const float sc = gm.scale * kLog2e;
        float mx = -INFINITY;
#pragma unroll
        for (int kk = 0; kk < WB; ++kk) {
            if (kk < win) {
                const int j = neighbour(t, kk, left, 1);
                const bool masked = (j < 0) | (j >= T) | (j >= vl) | (t >= vl);
                const float x = fmaf(s[kk], sc, (misc->rpb[kk] + (masked ? kMaskValue : 0.f)) * kLog2e);
                s[kk] = x;
                mx = fmaxf(mx, x);
            }
        }
        float sum = 0.f;
#pragma unroll
        for (int kk = 0; kk < WB; ++kk) {
            if (kk < win) { const float p = exp2f(s[kk] - mx); s[kk] = p; sum += p; }
        }
        const float inv = 1.f / sum;
        if (t < T && lse) lse[(size_t)n * T + t] = (mx + log2f(sum)) * kLn2;
        if constexpr (!PT) {
            if (t < T) {
                // P[r][c], c = r + kk: K-major core matrices (8 rows x 16 bytes), K-adjacent matrices 2048 bytes apart
#pragma unroll
                for (int kk = 0; kk < WB; ++kk) {
                    if (kk < win) {
                        const int c = r + kk;
                        E* dst = reinterpret_cast<E*>(sP + (c >> 3) * 2048 + r * 16 + (c & 7) * 2);
                        *dst = (E)(s[kk] * inv);
                    }
                }
            }
        } else {
            // P goes to tensor memory over the S columns: rotate the band back to its diagonal position
            // (right by `lane`), pack pairs of 16-bit values per column, zero everything else in the row.
#pragma unroll
            for (int i = 0; i < LW; ++i) s[i] = (i < WB && i < win && t < T) ? s[i] * inv : 0.f;
#pragma unroll
            for (int b = 1; b <= 16; b <<= 1) {
                const bool on = (lane & b) != 0;
#pragma unroll
                for (int i = LW - 1; i >= 0; --i) {
                    const float from = (i >= b) ? s[i - b] : 0.f;
                    s[i] = on ? from : s[i];
                }
            }
            uint32_t w[LW / 2];
#pragma unroll
            for (int c = 0; c < LW / 2; ++c) w[c] = Cvt<E>::pack2(s[2 * c], s[2 * c + 1]);
            const uint32_t prow = tmem + ((uint32_t)(warp * 32) << 16);
            const uint32_t zeros[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int ci = 0; ci < KT / 16; ++ci)
                if (ci < 2 * warp || ci >= 2 * warp + LW / 16) ptx::tmem_st8(prow + ci * 8, zeros);
#pragma unroll
            for (int cj = 0; cj < LW / 16; ++cj) ptx::tmem_st8(prow + (2 * warp + cj) * 8, &w[cj * 8]);
            ptx::tmem_st_wait();
        }
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();

    // ---- O = P.V (one thread)
    if (tid == 0) {
        ptx::tc_fence_after_sync();
        if (ok) {
            const uint32_t idesc = ptx::instr_desc(Fmt<E>::v, 0, 1, kTileM, (uint32_t)C);
            const uint32_t pa = ptx::smem_u32(sP), va = ptx::smem_u32(sV);
            for (int ks = 0; ks < KT / 16; ++ks) {
                const uint64_t bd = ptx::smem_desc(va + ks * 16 * kRowBytes, 0, 8 * kRowBytes, RowSwizzle<C>::umma);
                if constexpr (PT) {
                    ptx::mma_ts(tmem + kOCol, tmem + ks * 8, bd, idesc, ks > 0 ? 1u : 0u);
                } else {
                    const uint64_t ad = ptx::smem_desc(pa + ks * 4096, 2048, 128, ptx::kSwizzleNone);
                    ptx::mma_ss(tmem + kOCol, ad, bd, idesc, ks > 0 ? 1u : 0u);
                }
            }
        }
        ptx::mma_commit(&misc->bar_o);
    }
    __syncwarp();
    if (!ptx::mbar_wait(&misc->bar_o, 0)) { ok = false; atomicExch(&g_tc_status, 3); }
    ptx::tc_fence_after_sync();
    {
        float acc[C];
        const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)kOCol;
#pragma unroll
        for (int c = 0; c < C; c += 8) ptx::tmem_ld8(taddr + c, &acc[c]);
        ptx::tmem_ld_wait();
        if (t < T && ok) {
            uint4* dst = reinterpret_cast<uint4*>(o + ((size_t)n * T + t) * C);
#pragma unroll
            for (int c = 0; c < C / 8; ++c) dst[c] = Cvt<E>::pack(&acc[c * 8]);
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        ptx::tmem_dealloc(tmem, kTmemCols);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
        if (qres != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

}  // namespace

// Tensor map over a dense (N, T, C) 16-bit tensor viewed as dims (C, T, N), box (C, rows, 1).
bool make_row_tile_map(CUtensorMap* map, const void* base, int dtype, int N, int T, int C, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)T, (cuuint64_t)N};
    const cuuint64_t strides[2] = {(cuuint64_t)C * 2, (cuuint64_t)T * C * 2};
    const cuuint32_t box[3] = {(cuuint32_t)C, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle sw = C == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : C == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    const CUtensorMapDataType dt = dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tc_fwd_supports(const Geometry& gm) {
    return gm.dil == 1 && (gm.C == 64 || gm.C == 32 || gm.C == 16) && gm.win <= 33;
}

template <typename E, int C, int WB, bool PT>
static cudaError_t launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* o, float* lse,
                              const float* rpb, const int* valid_len, const Geometry& gm, int tiles_per_seq, int KT,
                              cudaStream_t st) {
    const int smem = fwd_layout(C, KT).total;
    auto kern = tc_fwd_kernel<E, C, WB, PT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kern<<<gm.N * tiles_per_seq, 128, smem, st>>>(mq, mk, mv, (E*)o, lse, rpb, valid_len, gm, tiles_per_seq, KT);
    return cudaGetLastError();
}

cudaError_t tc_fused_fwd(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                         const int* valid_len, const Geometry& gm, int dtype, bool p_in_tmem, cudaStream_t st) {
    if (!tc_fwd_supports(gm)) return cudaErrorInvalidValue;
    const int KT = round_up(kTileM + gm.win - 1, 16);
    const int tiles_per_seq = (gm.T + kTileM - 1) / kTileM;
    CUtensorMap mq, mk, mv;
    if (!make_row_tile_map(&mq, q, dtype, gm.N, gm.T, gm.C, kTileM) || !make_row_tile_map(&mk, k, dtype, gm.N, gm.T, gm.C, KT) ||
        !make_row_tile_map(&mv, v, dtype, gm.N, gm.T, gm.C, KT))
        return cudaErrorInvalidValue;
#define NA1D_TC_FWD(E, C, WB)                                                                                   \
    return p_in_tmem ? launch_fwd<E, C, WB, true>(mq, mk, mv, o, lse, rpb, valid_len, gm, tiles_per_seq, KT, st) \
                     : launch_fwd<E, C, WB, false>(mq, mk, mv, o, lse, rpb, valid_len, gm, tiles_per_seq, KT, st)
#define NA1D_TC_FWD_W(E, C)                          \
    if (gm.win <= 9) { NA1D_TC_FWD(E, C, 9); }       \
    else if (gm.win <= 17) { NA1D_TC_FWD(E, C, 17); } \
    else { NA1D_TC_FWD(E, C, 33); }
#define NA1D_TC_FWD_C(E)                         \
    if (gm.C == 64) { NA1D_TC_FWD_W(E, 64) }     \
    else if (gm.C == 32) { NA1D_TC_FWD_W(E, 32) } \
    else { NA1D_TC_FWD_W(E, 16) }
    if (dtype == 0) { NA1D_TC_FWD_C(__nv_bfloat16) } else { NA1D_TC_FWD_C(__half) }
#undef NA1D_TC_FWD
#undef NA1D_TC_FWD_W
#undef NA1D_TC_FWD_C
}

// Reads and clears the device status word (synchronises the device). 0 = no bounded wait expired.
int tc_read_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
    return v;
}

}  // namespace na1d

// Fused NA1D backward on the Blackwell tensor path (sm_100a): persistent, warp-specialised.
//
// Tiling. A tile is a window W of 128 consecutive rows of one sequence; consecutive tiles start
// `stride = 128-(win-1)` rows apart, so they overlap by win-1 rows. All 128 rows act as queries
// (their band needs keys [w0-left, w0+127+right], staged as KT = round16(128+win-1) rows of K and V);
// a key row is "interior" when every query that attends it lies in W, which holds for
// rows [right, 128-left) of W -- exactly `stride` rows, and these are the rows whose dQ, dK and dV
// this tile stores. Every (query,key) pair of the band is thus seen with both rows inside one tile:
// no atomics, no second (key-owned) recomputation pass, deterministic results.
//
// Per tile (one CTA per SM, 192 threads):
//   warp 4  : TMA producer -- Q[W], dO[W], K[KT], V[KT] into a 2-stage ring (plain tile loads,
//             out-of-range rows arrive as zeros = the reference's zero padding).
//   warp 5  : MMA issuer  -- batch 1: S = Q.K^T, dP = dO.V^T (TMEM, N=KT);
//                            batch 2: dQ = dS.K (A from TMEM), dV = P^T.dO, dK = dS^T.Q (A from smem).
//   warps0-3: one thread per query row: reads its band of S and dP from TMEM, recomputes
//             P = exp(S - lse) from the saved log-sum-exp, delta = sum_k P.dP (equal to dot(dO,O), so
//             neither O nor a separate delta pass is needed), dS = P(dP - delta); writes dS back to
//             TMEM as a 16-bit A operand and P, dS transposed to shared memory; later reads
//             dQ/dK/dV from TMEM and stores the rows this tile owns.
// Replaces the four backward launches of the reference (na1d_tensorcore/nattn.py:46-54, 69-78) and
// the eager softmax backward between them.
#include "na1d_internal.h"
#include "na1d_ptx.cuh"

namespace na1d {

// Device status word of this translation unit (device symbols are per file without relocatable device code).
__device__ int g_tc_bwd_status = 0;

namespace {

constexpr int kTileM = 128;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kColDP = 160, kColDQ = 320, kColDK = 384, kColDV = 448;

template <int C> struct RowSwizzle;
template <> struct RowSwizzle<64> { static constexpr uint64_t umma = ptx::kSwizzle128B; };
template <> struct RowSwizzle<32> { static constexpr uint64_t umma = ptx::kSwizzle64B; };
template <> struct RowSwizzle<16> { static constexpr uint64_t umma = ptx::kSwizzle32B; };
template <typename E> struct Fmt;
template <> struct Fmt<__nv_bfloat16> { static constexpr uint32_t v = 1; };
template <> struct Fmt<__half> { static constexpr uint32_t v = 0; };

__host__ __device__ constexpr int round_up(int x, int m) { return (x + m - 1) / m * m; }

struct BwdSmemLayout {
    int stage_q, stage_do, stage_k, stage_v, stage_bytes;  // offsets inside one stage
    int pt, dst, misc, total;
};
__host__ __device__ inline BwdSmemLayout bwd_layout(int C, int KT) {
    BwdSmemLayout L;
    L.stage_q = 0;
    L.stage_do = L.stage_q + round_up(kTileM * C * 2, 1024);
    L.stage_k = L.stage_do + round_up(kTileM * C * 2, 1024);
    L.stage_v = L.stage_k + round_up(KT * C * 2, 1024);
    L.stage_bytes = L.stage_v + round_up(KT * C * 2, 1024);
    L.pt = 2 * L.stage_bytes;
    L.dst = L.pt + kTileM * kTileM * 2;
    L.misc = L.dst + kTileM * kTileM * 2;
    L.total = L.misc + 1024 + 1024;
    return L;
}

struct alignas(8) BwdMisc {
    uint64_t full[2], empty[2];
    uint64_t s_ready, p_ready, o_ready, o_free;
    uint32_t tmem_base;
    int abort;
    float rpb[64];
    float drpb[64];
};

template <typename E, int C, int WB>
__global__ void __launch_bounds__(kThreads, 1)
tc_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
              const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, E* __restrict__ dq,
              E* __restrict__ dk, E* __restrict__ dv, float* __restrict__ d_rpb, const float* __restrict__ lse,
              const float* __restrict__ rpb, const int* __restrict__ valid_len, Geometry gm, int tiles_per_seq, int stride,
              int KT, int total_tiles) {
    constexpr int LW = round_up(WB + 31, 16);
    constexpr int kRowBytes = C * 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const BwdSmemLayout L = bwd_layout(C, KT);
    uint8_t* sPT = smem + L.pt;
    uint8_t* sDST = smem + L.dst;
    BwdMisc* misc = reinterpret_cast<BwdMisc*>(smem + L.misc);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int win = gm.win, left = gm.left, right = gm.win - 1 - gm.left, T = gm.T;
    const int stage_tx = (2 * kTileM + 2 * KT) * kRowBytes;

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) { ptx::mbar_init(&misc->full[s], 1); ptx::mbar_init(&misc->empty[s], 1); }
        ptx::mbar_init(&misc->s_ready, 1);
        ptx::mbar_init(&misc->p_ready, 128);
        ptx::mbar_init(&misc->o_ready, 1);
        ptx::mbar_init(&misc->o_free, 128);
        misc->abort = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tm_q);
        ptx::prefetch_tensormap(&tm_do);
        ptx::prefetch_tensormap(&tm_k);
        ptx::prefetch_tensormap(&tm_v);
    }
    if (warp == 0) {
        __syncwarp();
        ptx::tmem_alloc(&misc->tmem_base, kTmemCols);
        ptx::tmem_relinquish();
    }
    {   // transposed operands start as zeros; the band positions are rewritten every tile
        uint4* z = reinterpret_cast<uint4*>(sPT);
        for (int i = tid; i < 2 * kTileM * kTileM * 2 / 16; i += kThreads) z[i] = make_uint4(0, 0, 0, 0);
    }
    if (tid < 64) misc->drpb[tid] = 0.f;
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = misc->tmem_base;
    volatile int* abort_flag = &misc->abort;

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1, k = it >> 1;
                if (!ptx::mbar_wait(&misc->empty[s], (k & 1) ^ 1) || *abort_flag) { atomicExch(&g_tc_bwd_status, 11); *abort_flag = 1; break; }
                const int n = tile / tiles_per_seq;
                const int w0 = (tile - n * tiles_per_seq) * stride - right;
                uint8_t* st = smem + s * L.stage_bytes;
                ptx::mbar_expect_tx(&misc->full[s], (uint32_t)stage_tx);
                ptx::tma_load_3d(st + L.stage_q, &tm_q, &misc->full[s], 0, w0, n);
                ptx::tma_load_3d(st + L.stage_do, &tm_do, &misc->full[s], 0, w0, n);
                ptx::tma_load_3d(st + L.stage_k, &tm_k, &misc->full[s], 0, w0 - left, n);
                ptx::tma_load_3d(st + L.stage_v, &tm_v, &misc->full[s], 0, w0 - left, n);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = ptx::instr_desc(Fmt<E>::v, 0, 0, kTileM, (uint32_t)KT);
            const uint32_t idesc_o = ptx::instr_desc(Fmt<E>::v, 0, 1, kTileM, (uint32_t)C);
            const uint32_t pt_a = ptx::smem_u32(sPT), dst_a = ptx::smem_u32(sDST);
            int it = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1, k = it >> 1;
                const uint32_t st = ptx::smem_u32(smem + s * L.stage_bytes);
                const uint32_t qa = st + L.stage_q, doa = st + L.stage_do, ka = st + L.stage_k, va = st + L.stage_v;
                if (!ptx::mbar_wait(&misc->full[s], k & 1) || *abort_flag) { atomicExch(&g_tc_bwd_status, 12); *abort_flag = 1; break; }
                ptx::tc_fence_after_sync();
                // batch 1: S = Q.K^T -> cols [0,KT), dP = dO.V^T -> cols [160,160+KT)
#pragma unroll
                for (int ks = 0; ks < C / 16; ++ks) {
                    const uint64_t ad = ptx::smem_desc(qa + ks * 32, 16, 8 * kRowBytes, RowSwizzle<C>::umma);
                    const uint64_t bd = ptx::smem_desc(ka + ks * 32, 16, 8 * kRowBytes, RowSwizzle<C>::umma);
                    ptx::mma_ss(tmem, ad, bd, idesc_s, ks > 0 ? 1u : 0u);
                }
#pragma unroll
                for (int ks = 0; ks < C / 16; ++ks) {
                    const uint64_t ad = ptx::smem_desc(doa + ks * 32, 16, 8 * kRowBytes, RowSwizzle<C>::umma);
                    const uint64_t bd = ptx::smem_desc(va + ks * 32, 16, 8 * kRowBytes, RowSwizzle<C>::umma);
                    ptx::mma_ss(tmem + kColDP, ad, bd, idesc_s, ks > 0 ? 1u : 0u);
                }
                ptx::mma_commit(&misc->s_ready);
                // operands from the compute warps, and the previous tile's outputs drained
                if (!ptx::mbar_wait(&misc->p_ready, it & 1) || !ptx::mbar_wait(&misc->o_free, (it & 1) ^ 1) || *abort_flag) {
                    atomicExch(&g_tc_bwd_status, 13); *abort_flag = 1; break;
                }
                ptx::tc_fence_after_sync();
                // batch 2: dQ = dS.K (A: TMEM cols [0,KT/2), 16-bit pairs), dV = P^T.dO, dK = dS^T.Q
                for (int ks = 0; ks < KT / 16; ++ks) {
                    const uint64_t bd = ptx::smem_desc(ka + ks * 16 * kRowBytes, 0, 8 * kRowBytes, RowSwizzle<C>::umma);
                    ptx::mma_ts(tmem + kColDQ, tmem + ks * 8, bd, idesc_o, ks > 0 ? 1u : 0u);
                }
#pragma unroll
                for (int ks = 0; ks < kTileM / 16; ++ks) {
                    const uint64_t ad = ptx::smem_desc(pt_a + ks * 4096, 2048, 128, ptx::kSwizzleNone);
                    const uint64_t bd = ptx::smem_desc(doa + ks * 16 * kRowBytes, 0, 8 * kRowBytes, RowSwizzle<C>::umma);
                    ptx::mma_ss(tmem + kColDV, ad, bd, idesc_o, ks > 0 ? 1u : 0u);
                }
#pragma unroll
                for (int ks = 0; ks < kTileM / 16; ++ks) {
                    const uint64_t ad = ptx::smem_desc(dst_a + ks * 4096, 2048, 128, ptx::kSwizzleNone);
                    const uint64_t bd = ptx::smem_desc(qa + ks * 16 * kRowBytes, 0, 8 * kRowBytes, RowSwizzle<C>::umma);
                    ptx::mma_ss(tmem + kColDK, ad, bd, idesc_o, ks > 0 ? 1u : 0u);
                }
                ptx::mma_commit(&misc->o_ready);
                ptx::mma_commit(&misc->empty[s]);
            }
        }
    } else {
        // ------------------------------------------------------------ compute warps: one thread per query row
        const int r = warp * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        const float sc = gm.scale * kLog2e;
        float drpb_acc[WB];
#pragma unroll
        for (int kk = 0; kk < WB; ++kk) drpb_acc[kk] = 0.f;
        int it = 0;
        int cached_h = -1;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            const int n = tile / tiles_per_seq;
            const int w0 = (tile - n * tiles_per_seq) * stride - right;
            const int t = w0 + r;
            const int h = n % gm.H;
            const bool valid_q = t >= 0 && t < T;
            const bool owned = valid_q && r >= right && r < kTileM - left;
            const int vl = valid_len ? __ldg(valid_len + n / gm.H) : T;
            const float lse2 = valid_q ? __ldg(lse + (size_t)n * T + t) * kLog2e : 0.f;
            if (h != cached_h) {
                // rpb row of this head (all compute threads agree on h; sync among the 4 compute warps only)
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (r < win) misc->rpb[r] = rpb ? __ldg(rpb + h * win + r) : 0.f;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                cached_h = h;
            }
            if (!ptx::mbar_wait(&misc->s_ready, it & 1) || *abort_flag) { atomicExch(&g_tc_bwd_status, 14); *abort_flag = 1; break; }
            ptx::tc_fence_after_sync();
            float s[LW], d[LW];
#pragma unroll
            for (int c = 0; c < LW; c += 8) ptx::tmem_ld8(lane_base + warp * 32 + c, &s[c]);
#pragma unroll
            for (int c = 0; c < LW; c += 8) ptx::tmem_ld8(lane_base + kColDP + warp * 32 + c, &d[c]);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int b = 16; b >= 1; b >>= 1) {
                const bool on = (lane & b) != 0;
#pragma unroll
                for (int i = 0; i < WB + b - 1; ++i) { s[i] = on ? s[i + b] : s[i]; d[i] = on ? d[i + b] : d[i]; }
            }
            // P, delta, dS on the band
            float delta = 0.f;
#pragma unroll
            for (int kk = 0; kk < WB; ++kk) {
                if (kk < win) {
                    const int j = neighbour(t, kk, left, 1);
                    const bool masked = (j < 0) | (j >= T) | (j >= vl) | (t >= vl);
                    const float x = fmaf(s[kk], sc, (misc->rpb[kk] + (masked ? kMaskValue : 0.f)) * kLog2e) - lse2;
                    const float p = valid_q ? exp2f(x) : 0.f;
                    s[kk] = p;
                    delta = fmaf(p, d[kk], delta);
                } else {
                    s[kk] = 0.f; d[kk] = 0.f;
                }
            }
#pragma unroll
            for (int kk = 0; kk < WB; ++kk) {
                const float ds = s[kk] * (d[kk] - delta);
                if (owned) drpb_acc[kk] += ds;
                d[kk] = ds * gm.scale;
            }
            // transposed operands: row m = key index inside W, column r = this query
#pragma unroll
            for (int kk = 0; kk < WB; ++kk) {
                if (kk < win) {
                    const int m = r + kk - left;
                    if (m >= 0 && m < kTileM) {
                        const int off = (r >> 3) * 2048 + m * 16 + (r & 7) * 2;
                        *reinterpret_cast<E*>(sPT + off) = (E)s[kk];
                        *reinterpret_cast<E*>(sDST + off) = (E)d[kk];
                    }
                }
            }
            // dS as a 16-bit A operand in TMEM over the S columns: rotate the band back to its diagonal
#pragma unroll
            for (int i = WB; i < LW; ++i) d[i] = 0.f;
#pragma unroll
            for (int b = 1; b <= 16; b <<= 1) {
                const bool on = (lane & b) != 0;
#pragma unroll
                for (int i = LW - 1; i >= 0; --i) {
                    const float from = (i >= b) ? d[i - b] : 0.f;
                    d[i] = on ? from : d[i];
                }
            }
            {
                uint32_t w[LW / 2];
#pragma unroll
                for (int c = 0; c < LW / 2; ++c) w[c] = Cvt<E>::pack2(d[2 * c], d[2 * c + 1]);
                const uint32_t zeros[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int ci = 0; ci < KT / 16; ++ci)
                    if (ci < 2 * warp || ci >= 2 * warp + LW / 16) ptx::tmem_st8(lane_base + ci * 8, zeros);
#pragma unroll
                for (int cj = 0; cj < LW / 16; ++cj) ptx::tmem_st8(lane_base + (2 * warp + cj) * 8, &w[cj * 8]);
                ptx::tmem_st_wait();
            }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&misc->p_ready);

            // epilogue: dQ, dK, dV rows owned by this tile
            if (!ptx::mbar_wait(&misc->o_ready, it & 1) || *abort_flag) { atomicExch(&g_tc_bwd_status, 15); *abort_flag = 1; break; }
            ptx::tc_fence_after_sync();
            const size_t row_off = ((size_t)n * T + (valid_q ? t : 0)) * C;
            {
                float acc[C];
#pragma unroll
                for (int c = 0; c < C; c += 8) ptx::tmem_ld8(lane_base + kColDQ + c, &acc[c]);
                ptx::tmem_ld_wait();
                if (owned) {
                    uint4* dst = reinterpret_cast<uint4*>(dq + row_off);
#pragma unroll
                    for (int c = 0; c < C / 8; ++c) dst[c] = Cvt<E>::pack(&acc[c * 8]);
                }
#pragma unroll
                for (int c = 0; c < C; c += 8) ptx::tmem_ld8(lane_base + kColDK + c, &acc[c]);
                ptx::tmem_ld_wait();
                if (owned) {
                    uint4* dst = reinterpret_cast<uint4*>(dk + row_off);
#pragma unroll
                    for (int c = 0; c < C / 8; ++c) dst[c] = Cvt<E>::pack(&acc[c * 8]);
                }
#pragma unroll
                for (int c = 0; c < C; c += 8) ptx::tmem_ld8(lane_base + kColDV + c, &acc[c]);
                ptx::tmem_ld_wait();
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(&misc->o_free);
                if (owned) {
                    uint4* dst = reinterpret_cast<uint4*>(dv + row_off);
#pragma unroll
                    for (int c = 0; c < C / 8; ++c) dst[c] = Cvt<E>::pack(&acc[c * 8]);
                }
            }
            // d_rpb changes head when the sequence changes: flush per tile (cheap: win shared atomics per warp)
            if (d_rpb) {
#pragma unroll
                for (int kk = 0; kk < WB; ++kk) {
                    if (kk < win) {
                        float x = drpb_acc[kk];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
                        if (lane == 0 && x != 0.f) atomicAdd(d_rpb + h * win + kk, x);
                    }
                    drpb_acc[kk] = 0.f;
                }
            }
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        ptx::tmem_dealloc(tmem, kTmemCols);
    }
}

template <typename E, int C, int WB>
cudaError_t launch_bwd(const CUtensorMap& mq, const CUtensorMap& mdo, const CUtensorMap& mk, const CUtensorMap& mv, void* dq,
                       void* dk, void* dv, float* d_rpb, const float* lse, const float* rpb, const int* valid_len,
                       const Geometry& gm, int tiles_per_seq, int stride, int KT, int sm_count, cudaStream_t st) {
    const int smem = bwd_layout(C, KT).total;
    auto kern = tc_bwd_kernel<E, C, WB>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const int total = gm.N * tiles_per_seq;
    const int grid = total < sm_count ? total : sm_count;
    kern<<<grid, kThreads, smem, st>>>(mq, mdo, mk, mv, (E*)dq, (E*)dk, (E*)dv, d_rpb, lse, rpb, valid_len, gm, tiles_per_seq,
                                       stride, KT, total);
    return cudaGetLastError();
}

}  // namespace

bool make_row_tile_map(CUtensorMap* map, const void* base, int dtype, int N, int T, int C, int box_rows);

bool tc_bwd_supports(const Geometry& gm) {
    return gm.dil == 1 && (gm.C == 64 || gm.C == 32 || gm.C == 16) && gm.win <= 33 && gm.H * gm.win <= 1 << 20;
}

int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Reads and clears the backward kernels' status word (synchronises the device).
int tc_bwd_read_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_bwd_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_tc_bwd_status, &zero, sizeof(int));
    return v;
}

cudaError_t tc_fused_bwd(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k,
                         const void* v, const float* lse, const float* rpb, const int* valid_len, const Geometry& gm, int dtype,
                         cudaStream_t st) {
    if (!tc_bwd_supports(gm)) return cudaErrorInvalidValue;
    const int KT = round_up(kTileM + gm.win - 1, 16);
    const int stride = kTileM - (gm.win - 1);
    const int tiles_per_seq = (gm.T + stride - 1) / stride;
    CUtensorMap mq, mdo, mk, mv;
    if (!make_row_tile_map(&mq, q, dtype, gm.N, gm.T, gm.C, kTileM) || !make_row_tile_map(&mdo, d_o, dtype, gm.N, gm.T, gm.C, kTileM) ||
        !make_row_tile_map(&mk, k, dtype, gm.N, gm.T, gm.C, KT) || !make_row_tile_map(&mv, v, dtype, gm.N, gm.T, gm.C, KT))
        return cudaErrorInvalidValue;
    const int sms = device_sm_count();
#define NA1D_TC_BWD(E, C, WB) \
    return launch_bwd<E, C, WB>(mq, mdo, mk, mv, dq, dk, dv, d_rpb, lse, rpb, valid_len, gm, tiles_per_seq, stride, KT, sms, st)
#define NA1D_TC_BWD_W(E, C)                          \
    if (gm.win <= 9) { NA1D_TC_BWD(E, C, 9); }       \
    else if (gm.win <= 17) { NA1D_TC_BWD(E, C, 17); } \
    else { NA1D_TC_BWD(E, C, 33); }
#define NA1D_TC_BWD_C(E)                         \
    if (gm.C == 64) { NA1D_TC_BWD_W(E, 64) }     \
    else if (gm.C == 32) { NA1D_TC_BWD_W(E, 32) } \
    else { NA1D_TC_BWD_W(E, 16) }
    if (dtype == 0) { NA1D_TC_BWD_C(__nv_bfloat16) } else { NA1D_TC_BWD_C(__half) }
#undef NA1D_TC_BWD
#undef NA1D_TC_BWD_W
#undef NA1D_TC_BWD_C
}

}  // namespace na1d

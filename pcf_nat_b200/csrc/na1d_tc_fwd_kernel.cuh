// Fused NA1D forward on the Blackwell tensor path (sm_100a): persistent, warp-specialised,
// TMA-staged tiles, tcgen05 MMAs with accumulators (and the probability operand) in tensor memory.
//
// Rows are tiled over the FLATTENED (sequence, token) axis: tile i is rows g0 = 128 i .. g0+127 of the (N*T, C) matrix,
// so every tile is full whatever T is. A tile may span several sequences; a neighbour outside the query's own sequence is
// what the reference reads as a zero-padded row (na1d_tensorcore/bf16_ana1d_kernel.cu:99-112): its logit is rpb - 100 and
// it contributes nothing to the output, which is enforced per element.
// Per tile (224 threads, up to two CTAs per SM):
//   warp 4  : TMA producer -- Q[128 x C] and K, V rows [g0-left, g0-left+KT), KT = round16(128+win-1),
//             into a 2-stage ring. Plain (non-multicast) tile loads; rows outside [0,T) arrive as
//             zeros, which is the reference's zero padding of K and V
//             (na1d_tensorcore/bf16_ana1d_kernel.cu:99-112).
//   warps 5,6: MMA issuers -- S = Q.K^T (C/16 steps, M=128, N=KT) into TMEM columns [0,KT);
//             O = P.V (KT/16 steps, N=C) with P read from TMEM and V as an MN-major operand straight
//             from the TMA tile. A tcgen05.mma costs its issuing thread ~120 cycles whatever its size, so
//             the key steps of P.V are split between two issuers with an accumulator each (even / odd
//             steps); the epilogue adds the two.
//   warps0-3: softmax on the band only. Warp w owns rows 32w..32w+31 as two 16-row accumulator
//             fragments (see na1d_tc_common.cuh): scale, + rpb, + (-100) mask, row max / sum with two
//             quad shuffles each, normalise, round to 16 bits -- the reference rounds probabilities to
//             16 bits before its A.V product too (bf16_ana1d_kernel.cu:301-306) -- and store P over the
//             S columns of TMEM (zeros outside the band). Later the same warps read O from TMEM, stage it
//             in the tile's idle V buffer and one thread issues a TMA tile store (rows >= T are clipped).
// Every wait is bounded; on expiry the CTA records a code in a device status word and unwinds
// (TMEM is always released).
//
// Segmented variant (template parameter SEG). Tiles lie inside one residue sequence -- the tokens t = r (mod d) of one
// (batch, head) sequence, d = dilation -- addressed through 5-D tensor maps (channel, token-in-residue, residue, head,
// batch) over tensors with arbitrary batch/head/token strides. On a residue sequence a window of dilation d is a plain
// window of dilation 1 (neighbour kk of token u is token u + kk - left of the same residue), so any dilation runs in the
// bucket of its own window size, and q, k, v, o may be strided views (the slices of a packed projection output, an
// output laid out as (batch, token, head, channel)). Rows outside the residue sequence are zero-filled by TMA on loads and
// clipped on stores; the last tile of a sequence is partly empty.
//
// This header is compiled into two translation units (flat and segmented instantiations); everything in it has
// internal linkage.
#pragma once
#include "na1d_internal.h"
#include <type_traits>
#include "na1d_tc_common.cuh"

namespace na1d {
namespace {

__device__ int g_tc_status = 0;

using tc::kTileM;
using tc::round_up;
using tc::RowSwizzle;
using tc::Fmt;
// Softmax warps per CTA: 8 -- warps w and w + 4 share tensor-memory lane quarter w & 3 and take one 16-row block of the tile
// each (the kernel is bound by the softmax warps' per-row chain at 16- and 32-channel rows, and the shorter chain still
// gains 2-12 % at 64 channels). Behind them: producer/store warp, two MMA issuer warps, and one idle warp that completes
// the last warp group. The code keeps the 4-warp form (two blocks per warp, 224 threads) behind the same constant.
__host__ __device__ constexpr int softmax_warps(int C, int mode) { return 8; }
__host__ __device__ constexpr int fwd_threads(int nsw) { return nsw == 8 ? 384 : 224; }
constexpr int kTmemCols = 256;
// Tensor-memory columns. P (16-bit pairs, KT/2 <= 80 columns) always starts at column 0. Two layouts:
//   shared  : S (fp32, KT <= 160 columns) at [0, KT) under P; O of the even key steps at [192, 192+C), O of the odd key
//             steps at [96, 96+C) inside the S columns (dead once softmax has read them). S overwrites the P area every
//             tile, so every tile re-zeroes the part of P outside the band.
//   separate: P at [0, KTmax/2), O (even) behind it, S at [256-KTmax, 256), O (odd) on the first S columns. Nothing but
//             the band stores ever writes the P columns: they are zeroed once, and the band chunks of a row block are the
//             same in every tile. Fits when KTmax/2 + C + KTmax <= 256 (16-channel rows; 32-channel rows below the
//             widest window bucket).
__host__ __device__ constexpr int kt_max(int WB) { return WB > 17 ? 160 : 144; }   // KT = round16(128 + win - 1)
__host__ __device__ constexpr bool separate_p(int C, int WB) { return kt_max(WB) / 2 + C + kt_max(WB) <= kTmemCols; }
__host__ __device__ constexpr int col_s(int C, int WB) { return separate_p(C, WB) ? kTmemCols - kt_max(WB) : 0; }
__host__ __device__ constexpr int col_o(int C, int WB) { return separate_p(C, WB) ? kt_max(WB) / 2 : 192; }
__host__ __device__ constexpr int col_ob(int C, int WB) { return separate_p(C, WB) ? col_s(C, WB) : 96; }
constexpr int kBiasPad = 16;

struct FwdSmemLayout {
    int q, ring, stage_k, stage_v, stage_bytes, misc, band_stage, total;  // q: the single Q buffer; ring: first K/V stage
};
// band_win > 0 (band-out mode with 8 softmax warps): room to stage a tile's fp32 band, 128 rows of band_win entries, for
// coalesced 16-byte stores
__host__ __device__ inline FwdSmemLayout fwd_layout(int C, int KT, int bias_heads, int band_win = 0) {
    FwdSmemLayout L;
    // Q is needed only by the S MMAs at the start of a tile, so one buffer serves both stages: it is refilled as soon as
    // those MMAs retire. K and V live in a 2-stage ring; the finished O is staged in the tile's V buffer (idle once the
    // P.V MMAs have retired). 16 KB less than a Q buffer per stage: two CTAs per SM also for the widest window bucket.
    L.q = 0;
    L.ring = round_up(kTileM * C * 2, 1024);
    L.stage_k = 0;
    L.stage_v = round_up(KT * C * 2, 1024);
    L.stage_bytes = 2 * round_up(KT * C * 2, 1024);
    L.misc = L.ring + 2 * L.stage_bytes;
    L.band_stage = L.misc + 256 + round_up(2 * bias_heads * (kBiasPad + 48) * 4, 256);
    L.total = L.band_stage + round_up(kTileM * band_win * 4, 256) + 1008;  // misc, two bias tables, band staging, alignment slack
    return L;
}

// rows of the additive-term table: one per head with a bias, one (0 inside the band, -inf outside) without, none in the band modes
__host__ __device__ constexpr int table_heads(bool has_bias, int H, int mode) { return mode != 0 ? 0 : has_bias ? H : 1; }

struct alignas(8) FwdMisc {
    uint64_t full[2], empty[2];  // K/V ring
    uint64_t full_q, empty_q;    // the single Q buffer
    uint64_t s_ready, p_ready, o_ready, o_free, o_staged;
    uint32_t tmem_base;
    int abort;
};
constexpr int kBiasRow = kBiasPad + 48;  // per-head table: log2e * rpb[h][kk] at index kk + kBiasPad, kk in [-16, 48)

// Tensor maps of one launch: one per tensor in the flat tiling, two in the segmented one (residues with Tp and with
// Tp - 1 tokens).
template <int NSETS> struct FwdMaps {
    CUtensorMap q[NSETS], k[NSETS], v[NSETS], o[NSETS];
};

// MODE selects what the kernel computes with the same tiles, rings and tensor-memory layout:
//   kFused  : o = softmax(scale q.k^T + rpb + mask) . v                        (reads q, k, v; writes o, lse)
//   kBandOut: band[t, kk] = q[t] . k[j(t, kk)], zero-padded keys                 (reads q, k; writes the fp32 band)
//             -- the unfused QK forward and dA = dO.V^T (na1d_tensorcore/bf16_ana1d_kernel.cu:42-282)
//   kBandIn : o[t] = sum_kk band[t, kk] v[j(t, kk)], zero-padded values          (reads the fp32 band and v; writes o)
//             -- the unfused AV forward and dQ = dS.K (na1d_tensorcore/bf16_ana1d_kernel.cu:285-391); the band is rounded
//             to 16 bits before the product, as the reference does (:301-306)
constexpr int kFused = 0, kBandOut = 1, kBandIn = 2;

template <typename E, int C, int WB, bool SEG, int MODE = kFused, bool DROP = false>
__global__ void __launch_bounds__(fwd_threads(softmax_warps(C, MODE)), 2)
tc_fwd_kernel(const __grid_constant__ FwdMaps<SEG ? 2 : 1> tm, float* __restrict__ lse, float* __restrict__ band,
              const float* __restrict__ rpb, const int* __restrict__ valid_len, Geometry gm, SegGeom sg, int KT, int total_tiles,
              DropoutCfg drop) {
    static_assert(MODE == kFused || !SEG, "the unfused modes run on the flat tiling");
    constexpr int NG = tc::band_groups(WB);
    constexpr int kRowBytes = C * 2;
    constexpr bool kSepP = separate_p(C, WB);
    constexpr int NSW = softmax_warps(C, MODE), NB = NSW == 8 ? 1 : 2;   // softmax warps; 16-row blocks per warp
    constexpr bool kStageBand = NSW == 8;   // band-out mode: the fp32 band goes out through shared memory (16-byte stores)
    constexpr int kProducerWarp = NSW, kIssuerA = NSW + 1, kIssuerB = NSW + 2;
    // registers per thread after the warp groups rebalance (NSW = 8: 384 threads, two CTAs per SM, 80 each at launch)
    constexpr int kRegsSoftmax = 104, kRegsOther = 32;
    constexpr int kSCol = col_s(C, WB), kOCol = col_o(C, WB), kOColB = col_ob(C, WB);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const FwdSmemLayout L = fwd_layout(C, KT, table_heads(rpb != nullptr, gm.H, MODE), (MODE == kBandOut && kStageBand) ? gm.win : 0);
    FwdMisc* misc = reinterpret_cast<FwdMisc*>(smem + L.misc);
    float* bias_tab = reinterpret_cast<float*>(smem + L.misc + 256);
    const int rows_total = gm.N * gm.T;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // flat tiling: the effective (dilated) window, neighbour kk of the reference is offset kk * dil of it;
    // segmented tiling: the dilation lives in the addressing, the window is the reference's own
    const int dil = SEG ? 1 : gm.dil, dmask = dil - 1, dshift = 31 - __clz(dil);
    const int win = tc::eff_window(gm.win, dil), left = gm.left * dil, T = gm.T;
    const int stage_tx = (MODE == kFused ? 2 : 1) * KT * kRowBytes;   // K and V, or only the one the mode reads
    tc::SegCursor pcur = {};  // position of the producer thread's next tile (segmented tiling)

    // Loads of tile `tile` (iteration `it` of this CTA): Q into the single Q buffer, K and V into ring stage it % 2.
    auto produce = [&](int tile, int it) -> bool {
        const int s = it & 1, k = it >> 1;
        const int g0 = tile * kTileM;
        const int set = SEG && pcur.r >= sg.ra ? 1 : 0, rc = pcur.r - (set ? sg.ra : 0), u0 = pcur.i * kTileM;
        if constexpr (MODE != kBandIn) {
            // Q: free once the S MMAs of the previous tile have retired
            if (!ptx::mbar_wait_relaxed(&misc->empty_q, (it & 1) ^ 1) || *(volatile int*)&misc->abort) return false;
            // At the start every CTA of the grid loads at once and DRAM is the limit: let the first tile land before the
            // second is requested, so that all CTAs start computing (and storing) early instead of at the end of the burst.
            if (it == 1 && !ptx::mbar_wait_relaxed(&misc->full[0], 0)) return false;
            ptx::mbar_expect_tx(&misc->full_q, (uint32_t)(kTileM * kRowBytes));
            if constexpr (SEG) ptx::tma_load_5d(smem + L.q, &tm.q[set], &misc->full_q, 0, u0, rc, pcur.h, pcur.b);
            else ptx::tma_load_3d(smem + L.q, &tm.q[0], &misc->full_q, 0, g0, 0);
        }
        // K, V: free once the tile two back has stored its output (staged in its V buffer)
        if (!ptx::mbar_wait_relaxed(&misc->empty[s], (k & 1) ^ 1) || *(volatile int*)&misc->abort) return false;
        uint8_t* st = smem + L.ring + s * L.stage_bytes;
        ptx::mbar_expect_tx(&misc->full[s], (uint32_t)stage_tx);
        if constexpr (SEG) {
            ptx::tma_load_5d(st + L.stage_k, &tm.k[set], &misc->full[s], 0, u0 - left, rc, pcur.h, pcur.b);
            ptx::tma_load_5d(st + L.stage_v, &tm.v[set], &misc->full[s], 0, u0 - left, rc, pcur.h, pcur.b);
            pcur.advance();
        } else {
            if constexpr (MODE != kBandIn) ptx::tma_load_3d(st + L.stage_k, &tm.k[0], &misc->full[s], 0, g0 - left, 0);
            if constexpr (MODE != kBandOut) ptx::tma_load_3d(st + L.stage_v, &tm.v[0], &misc->full[s], 0, g0 - left, 0);
        }
        return true;
    };
    bool first_ok = true;
    if (tid == kProducerWarp * 32) {
        // The producer thread sets up the barriers and requests the CTA's first tile at once: the loads are in flight
        // while the other warps allocate tensor memory and meet at the barrier below.
        for (int s = 0; s < 2; ++s) { ptx::mbar_init(&misc->full[s], 1); ptx::mbar_init(&misc->empty[s], 1); }
        ptx::mbar_init(&misc->full_q, 1);
        ptx::mbar_init(&misc->empty_q, 1);
        ptx::mbar_init(&misc->s_ready, 1);
        ptx::mbar_init(&misc->p_ready, NSW * 32);
        ptx::mbar_init(&misc->o_ready, 2);  // one commit per MMA issuer
        ptx::mbar_init(&misc->o_free, NSW * 32);
        ptx::mbar_init(&misc->o_staged, NSW * 32);
        misc->abort = 0;
        ptx::fence_mbar_init();
        for (int i = 0; i < (SEG ? 2 : 1); ++i) {
            ptx::prefetch_tensormap(&tm.q[i]);
            ptx::prefetch_tensormap(&tm.k[i]);
            ptx::prefetch_tensormap(&tm.v[i]);
            ptx::prefetch_tensormap(&tm.o[i]);
        }
        if constexpr (SEG) pcur.init((int)blockIdx.x, (int)gridDim.x, sg, gm.H);
        // global memory written by the predecessor kernel is read from here on
        ptx::grid_dependency_wait();
        first_ok = produce((int)blockIdx.x, 0);
    }
    if (warp == 0) {
        ptx::tmem_alloc(&misc->tmem_base, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = misc->tmem_base;
    volatile int* abort_flag = &misc->abort;
    // Outputs are written from here on: wait for the predecessor, and let the successor start its own set-up as this
    // grid drains.
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();

    if (warp >= NSW) {
    if constexpr (NSW == 8) ptx::warpgroup_regs_shrink<kRegsOther>();
    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int it = 1;
            bool ok = first_ok;
            for (int tile = blockIdx.x + gridDim.x; ok && tile < total_tiles; tile += gridDim.x, ++it) ok = produce(tile, it);
            if (!ok) { atomicExch(&g_tc_status, 1); *abort_flag = 1; }
        } else if (lane == 1 && MODE != kBandOut) {
            // ---------------------------------------------------------- output store thread: waits until the softmax warps
            // have staged a tile's O, issues the TMA store, and frees the stage once the store has read shared memory
            int it = 0;
            tc::SegCursor ocur = {};
            if constexpr (SEG) ocur.init((int)blockIdx.x, (int)gridDim.x, sg, gm.H);
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
                if (!ptx::mbar_wait_relaxed(&misc->o_staged, it & 1) || *abort_flag) { atomicExch(&g_tc_status, 6); *abort_flag = 1; break; }
                const uint8_t* staged = smem + L.ring + (it & 1) * L.stage_bytes + L.stage_v;
                if constexpr (SEG) {
                    const int set = ocur.r >= sg.ra ? 1 : 0;
                    ptx::tma_store_5d(&tm.o[set], staged, 0, ocur.i * kTileM, ocur.r - (set ? sg.ra : 0), ocur.h, ocur.b);
                    ocur.advance();
                } else {
                    ptx::tma_store_3d(&tm.o[0], staged, 0, tile * kTileM, 0);
                }
                ptx::tma_store_commit();
                ptx::tma_store_wait_read();
                ptx::mbar_arrive(&misc->empty[it & 1]);
            }
            ptx::tma_store_wait_all();
        }
    } else if (warp == kIssuerA) {
        // ------------------------------------------------------------ MMA issuer A: S, and the even key steps of P.V
        if (lane == 0) {
            const uint32_t idesc_s = ptx::instr_desc(Fmt<E>::v, 0, 0, kTileM, (uint32_t)KT);
            const uint32_t idesc_o = ptx::instr_desc(Fmt<E>::v, 0, 1, kTileM, (uint32_t)C);
            const int nks = KT / 16;
            int it = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1, k = it >> 1;
                const uint32_t st = ptx::smem_u32(smem + L.ring + s * L.stage_bytes);
                // S overwrites the columns that held the previous tile's P and odd-step accumulator: both must be drained
                if (!ptx::mbar_wait(&misc->full[s], k & 1) || (MODE != kBandIn && !ptx::mbar_wait(&misc->full_q, it & 1)) ||
                    !ptx::mbar_wait(&misc->o_free, (it & 1) ^ 1) || *abort_flag) {
                    atomicExch(&g_tc_status, 2); *abort_flag = 1; break;
                }
                ptx::tc_fence_after_sync();
                if constexpr (MODE != kBandIn) {
                    const uint64_t a0 = ptx::smem_desc(ptx::smem_u32(smem + L.q), 16, 8 * kRowBytes, RowSwizzle<C>::umma);
                    const uint64_t b0 = ptx::smem_desc(st + L.stage_k, 16, 8 * kRowBytes, RowSwizzle<C>::umma);
#pragma unroll
                    for (int ks = 0; ks < C / 16; ++ks)
                        ptx::mma_ss(tmem + kSCol, tc::desc_advance(a0, ks * 32), tc::desc_advance(b0, ks * 32), idesc_s, ks > 0 ? 1u : 0u);
                }
                if constexpr (MODE != kBandIn) {
                    ptx::mma_commit(&misc->empty_q);  // Q is read by nothing else
                    ptx::mma_commit(&misc->s_ready);
                }
                if constexpr (MODE == kBandOut) {
                    ptx::mma_commit(&misc->empty[s]);  // nothing else reads the K stage in this mode
                    continue;
                }
                if (!ptx::mbar_wait(&misc->p_ready, it & 1) || *abort_flag) { atomicExch(&g_tc_status, 3); *abort_flag = 1; break; }
                ptx::tc_fence_after_sync();
                {
                    const uint64_t b0 = ptx::smem_desc(st + L.stage_v, 0, 8 * kRowBytes, RowSwizzle<C>::umma);
#pragma unroll 1
                    for (int ks = 0; ks < nks; ks += 2)
                        ptx::mma_ts(tmem + kOCol, tmem + ks * 8, tc::desc_advance(b0, ks * 16 * kRowBytes), idesc_o, ks > 0 ? 1u : 0u);
                }
                ptx::mma_commit(&misc->o_ready);
            }
        }
    } else if (warp == kIssuerB) {
        // ------------------------------------------------------------ MMA issuer B: the odd key steps of P.V
        if (lane == 0 && MODE != kBandOut) {
            const uint32_t idesc_o = ptx::instr_desc(Fmt<E>::v, 0, 1, kTileM, (uint32_t)C);
            const int nks = KT / 16;
            int it = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1, k = it >> 1;
                const uint32_t st = ptx::smem_u32(smem + L.ring + s * L.stage_bytes);
                if (!ptx::mbar_wait(&misc->full[s], k & 1) || !ptx::mbar_wait(&misc->p_ready, it & 1) || *abort_flag) {
                    atomicExch(&g_tc_status, 7); *abort_flag = 1; break;
                }
                ptx::tc_fence_after_sync();
                const uint64_t b0 = ptx::smem_desc(st + L.stage_v, 0, 8 * kRowBytes, RowSwizzle<C>::umma);
#pragma unroll 1
                for (int ks = 1; ks < nks; ks += 2)
                    ptx::mma_ts(tmem + kOColB, tmem + ks * 8, tc::desc_advance(b0, ks * 16 * kRowBytes), idesc_o, ks > 1 ? 1u : 0u);
                ptx::mma_commit(&misc->o_ready);
            }
        }
    }
    } else {
        // ------------------------------------------------------------ softmax / epilogue warps
        if constexpr (NSW == 8) ptx::warpgroup_regs_grow<kRegsSoftmax>();
        const int cw = warp & 3;                          // quarter of the tensor-memory lanes (and tile rows)
        const int bo = NSW == 8 ? warp >> 2 : 0;          // first 16-row block of that quarter this warp takes
        const int rb = cw * 32 + 16 * bo;                 // tile row of that block
        const int r = cw * 32 + lane;                     // accumulator row this lane drains in the epilogue
        const int fr = lane >> 2, fc = 2 * (lane & 3);
        const int fa = fc - fr;
        const uint32_t lane_base = tmem + ((uint32_t)(cw * 32) << 16);
        const float sc = gm.scale * kLog2e;
        const float mask2 = kMaskValue * kLog2e;
        // which of the thread's fragment slots are neighbours: slot (g, hh, e) is window offset 8 (g - hh) + e + fa, the same
        // for every tile, so the band test is one bit of a per-thread constant (class c = 2 (g - hh + 1) + e)
        uint32_t band_bits = 0;
#pragma unroll
        for (int c = 0; c < 2 * (NG + 1); ++c) {
            const int kk = 8 * ((c >> 1) - 1) + (c & 1) + fa;
            if ((unsigned)kk < (unsigned)win && (kk & dmask) == 0) band_bits |= 1u << c;
        }
        const float inv_T = 1.f / (float)T, inv_H = 1.f / (float)gm.H;
        const int heads = table_heads(rpb != nullptr, gm.H, MODE);
        if constexpr (MODE == kFused) {
            // Table of every head's bias (one all-zero row without a bias), once per CTA (barrier among the softmax warps
            // only), with -inf at every offset that is not a neighbour (outside the window, between dilated neighbours): the
            // fragment slots take their additive term from it and need no band test of their own.
            // Two copies, the second shifted by one entry: a thread reads the terms of its two adjacent columns with one
            // 8-byte load whatever the parity of its first offset.
            for (int i = tid; i < 2 * heads * kBiasRow; i += NSW * 32) {
                const int copy = i / (heads * kBiasRow), j = i - copy * heads * kBiasRow;
                const int hh_ = j / kBiasRow, kk = j - hh_ * kBiasRow - kBiasPad + copy;
                const bool nb = kk >= 0 && kk < win && (kk & dmask) == 0;
                bias_tab[i] = !nb ? -INFINITY : rpb ? __ldg(rpb + hh_ * gm.win + (kk >> dshift)) * kLog2e : 0.f;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NSW * 32) : "memory");
        }
        if constexpr (kSepP && MODE != kBandOut) {
            // P columns of this warp's lanes: zero once, only the band chunks are ever written again
            const uint32_t zeros[4] = {0, 0, 0, 0};
#pragma unroll
            for (int b = 0; b < NB; ++b)
                for (int ci = 0; ci < KT / 16; ++ci) tc::st_pack2(lane_base + ((uint32_t)(16 * (bo + b)) << 16) + ci * 8, zeros);
            ptx::tmem_st_wait();
        }
        int it = 0;
        tc::RowCursor cur = {};
        tc::SegCursor scur = {};
        if constexpr (SEG) scur.init((int)blockIdx.x, (int)gridDim.x, sg, gm.H);
        else cur.init(blockIdx.x * kTileM, T, gm.H, gridDim.x * kTileM);
        const int batch = gm.N / gm.H;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            const int g0 = tile * kTileM;
            // tokens of the sequence the keys must lie in: the whole sequence, or the tile's residue sequence
            const int Trow = SEG ? scur.rows(sg) : T;
            // The four rows this thread sees in the fragments (block b, row half hh = local rows 32 warp + fr + 8k). Per row:
            //   jb  : key index inside the row's own sequence of neighbour kk is jb + (kk - fa); outside [0, T) it is the
            //         reference's zero-padded key row
            //   vle : keys >= vle are masked (0 when the query itself is padding)
            int jb[2][2], vle[2][2];
            const float* brow[2][2];
            bool need_mask = false;
            if constexpr (SEG) {
                // every row of the tile belongs to residue r of sequence (b, h); token u of it is token d u + r of the
                // sequence, valid while d u + r < valid_len[b], i.e. u < ceil((valid_len - r) / d)
                const int vl = valid_len ? min(T, __ldg(valid_len + scur.b)) : T;
                const int vl_seq = vl > scur.r ? (vl - scur.r + sg.d - 1) / sg.d : 0;
#pragma unroll
                for (int k = 0; k < 2 * NB; ++k) {
                    const int tq = scur.i * kTileM + rb + fr + 8 * k;
                    const int vlr = tq < Trow ? vl_seq : 0;
                    brow[k >> 1][k & 1] = bias_tab + ((fa & 1) ? heads * kBiasRow - 1 : 0) + (rpb ? scur.h : 0) * kBiasRow + kBiasPad + fa;
                    jb[k >> 1][k & 1] = tq - left + fa;
                    vle[k >> 1][k & 1] = tq >= vlr ? 0 : vlr;
                    need_mask |= tq < left || tq + (win - 1 - left) >= vlr;
                }
            } else {
                int tq, hq, bq;
                cur.row_at(rb + fr, inv_T, inv_H, tq, hq, bq);
#pragma unroll
                for (int k = 0; k < 2 * NB; ++k) {
                    const bool live = g0 + rb + fr + 8 * k < rows_total;
                    const int vlr = !live ? 0 : valid_len ? min(T, __ldg(valid_len + min(bq, batch - 1))) : T;
                    brow[k >> 1][k & 1] = bias_tab + ((fa & 1) ? heads * kBiasRow - 1 : 0) + (rpb ? hq : 0) * kBiasRow + kBiasPad + fa;
                    jb[k >> 1][k & 1] = tq - left + fa;
                    vle[k >> 1][k & 1] = tq >= vlr ? 0 : vlr;
                    need_mask |= tq < left || tq + (win - 1 - left) >= vlr;
                    tc::row_step8(T, gm.H, tq, hq, bq);
                }
            }
            // masks are needed only when one of the warp's rows touches a sequence end or a padded region
            need_mask = __any_sync(0xffffffffu, need_mask);
            float s[2][4 * NG];
            if constexpr (MODE != kBandIn) {
                if (!ptx::mbar_wait(&misc->s_ready, it & 1) || *abort_flag) { atomicExch(&g_tc_status, 4); *abort_flag = 1; break; }
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int b = 0; b < NB; ++b)
                    tc::ld_frag<NG>(lane_base + ((uint32_t)(16 * (bo + b)) << 16) + (uint32_t)(kSCol + rb + 16 * b), s[b]);
                ptx::tmem_ld_wait();
            }
            if constexpr (MODE == kBandOut) {
                // the dot products of the band go to the fp32 band tensor as they are (a key outside the query's own sequence
                // is the reference's zero-padded row: 0); the S columns are free for the next tile at once
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(&misc->o_free);
                // Staged in shared memory first: the band rows of the warp's 16 NB tile rows are one contiguous piece of the
                // band tensor (row r at r * win floats), 64-byte aligned because the first row is a multiple of 16, so the
                // warp writes it with full 16-byte stores instead of 20 scattered 4-byte stores per thread and row pair.
                float* stg = reinterpret_cast<float*>(smem + L.band_stage) + rb * gm.win;
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        // (the 4-warp form of the kernel, two blocks per warp, writes straight to global memory: the staging
                        // costs registers it does not have)
                        const int gq = g0 + rb + 16 * b + 8 * hh + fr;
                        if (!kStageBand && gq >= rows_total) continue;
                        float* dst = kStageBand ? stg + (16 * b + 8 * hh + fr) * gm.win : band + (size_t)gq * gm.win;
#pragma unroll
                        for (int g = 0; g < NG; ++g)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int kc = 8 * (g - hh) + e;
                                if (tc::dead_slot(g, hh, NG) || !((band_bits >> (2 * (g - hh + 1) + e)) & 1u)) continue;
                                const unsigned j = (unsigned)(jb[b][hh] + kc);
                                dst[(kc + fa) >> dshift] = j < (unsigned)Trow ? s[b][4 * g + 2 * hh + e] : 0.f;
                            }
                    }
                if constexpr (kStageBand) {
                    __syncwarp();
                    const int row0 = g0 + rb;
                    const int n = max(0, min(16 * NB, rows_total - row0)) * gm.win;   // floats of this warp's rows inside the tensor
                    float* out = band + (size_t)row0 * gm.win;
                    for (int i = lane; i < (n >> 2); i += 32) reinterpret_cast<float4*>(out)[i] = reinterpret_cast<const float4*>(stg)[i];
                    if (lane < (n & 3)) out[(n & ~3) + lane] = stg[(n & ~3) + lane];
                    __syncwarp();   // the next tile overwrites the staging rows
                }
                if constexpr (SEG) scur.advance(); else cur.advance();
                continue;
            }
            if constexpr (MODE == kBandIn) {
                // the probabilities come from the fp32 band tensor instead of a softmax: slot (g, hh, e) of row (b, hh) is
                // band[row, kk]; 0 outside the band, for rows past the tensor and for keys outside the row's own sequence
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int gq = g0 + rb + 16 * b + 8 * hh + fr;
                        // (read straight from global memory: the four lanes of a row share its cache lines, and staging the
                        // warp's rows through shared memory as the band-out mode does measured 15 % slower)
                        const float* src = band + (size_t)min(gq, rows_total - 1) * gm.win;
#pragma unroll
                        for (int g = 0; g < NG; ++g)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int kc = 8 * (g - hh) + e;
                                const bool on = !tc::dead_slot(g, hh, NG) && ((band_bits >> (2 * (g - hh + 1) + e)) & 1u) &&
                                                gq < rows_total && (unsigned)(jb[b][hh] + kc) < (unsigned)Trow;
                                s[b][4 * g + 2 * hh + e] = on ? __ldg(src + ((kc + fa) >> dshift)) : 0.f;
                            }
                    }
            }
            float sum[2][2] = {{1.f, 1.f}, {1.f, 1.f}};   // factor applied to s[] when it is packed: 1 / row sum (fused), 1 (band input)
            if constexpr (MODE == kFused) {
                sum[0][0] = sum[0][1] = sum[1][0] = sum[1][1] = 0.f;
                // logits on the band (log2 domain), everything else -inf; two straight-line copies, with and without masks
                float mx[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}};
                auto logits = [&](auto masked_tag) {
                    constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
                    for (int b = 0; b < NB; ++b)
#pragma unroll
                        for (int g = 0; g < NG; ++g)
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh) {
                                if (tc::dead_slot(g, hh, NG)) { s[b][4 * g + 2 * hh] = s[b][4 * g + 2 * hh + 1] = -INFINITY; continue; }
                                // additive terms of the thread's two adjacent columns of this group (-inf outside the band)
                                const float2 bias2 = *reinterpret_cast<const float2*>(brow[b][hh] + 8 * (g - hh));
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int idx = 4 * g + 2 * hh + e;
                                    const int kc = 8 * (g - hh) + e;  // window offset minus the lane constant fa
                                    float bias = e ? bias2.y : bias2.x;
                                    float dot = s[b][idx];
                                    if constexpr (kMasked) {
                                        const unsigned j = (unsigned)(jb[b][hh] + kc);
                                        if (j >= (unsigned)Trow) dot = 0.f;  // key outside the query's own sequence: the reference's zero row
                                        if (j >= (unsigned)vle[b][hh]) bias += mask2;
                                    }
                                    const float x = fmaf(dot, sc, bias);
                                    s[b][idx] = x;
                                    mx[b][hh] = fmaxf(mx[b][hh], x);
                                }
                            }
                };
                if (need_mask) logits(std::true_type{}); else logits(std::false_type{});
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) mx[b][hh] = tc::quad_max(mx[b][hh]);
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int g = 0; g < NG; ++g)
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int idx = 4 * g + 2 * hh + e;
                                if (tc::dead_slot(g, hh, NG)) { s[b][idx] = 0.f; continue; }
                                const float p = tc::fast_exp2(s[b][idx] - mx[b][hh]);  // exp2(-inf) = 0 outside the band
                                s[b][idx] = p;
                                sum[b][hh] += p;
                            }
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        sum[b][hh] = tc::quad_sum(sum[b][hh]);
                        if (lse && (lane & 3) == 0) {
                            const float val = (mx[b][hh] + tc::fast_log2(sum[b][hh])) * kLn2;
                            if constexpr (SEG) {
                                const int tq = scur.i * kTileM + rb + 16 * b + 8 * hh + fr;
                                if (tq < Trow) lse[(size_t)(scur.b * gm.H + scur.h) * T + (size_t)tq * sg.d + scur.r] = val;
                            } else {
                                const int gq = g0 + rb + 16 * b + 8 * hh + fr;
                                if (gq < rows_total) lse[gq] = val;
                            }
                        }
                        sum[b][hh] = tc::fast_rcp(sum[b][hh]);
                    }
            }
            // P. Per 16-lane block the band occupies NGP 8-key groups starting at the block's own first row; every other
            // 16-key chunk of the row range is zero: zeroed here when S shares the columns (the two sets are disjoint, so
            // one wait), once at the start otherwise.
            {
                constexpr int NGP = NG + (NG & 1);  // band groups padded to whole 16-key chunks
                const uint32_t zeros[4] = {0, 0, 0, 0};
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const uint32_t blk = lane_base + ((uint32_t)(16 * (bo + b)) << 16);
                    const int c0 = 2 * cw + bo + b;  // first band chunk (16 keys = 8 packed columns) of this block
                    if constexpr (!kSepP)
                        for (int ci = 0; ci < KT / 16; ++ci)
                            if (ci < c0 || ci >= c0 + NGP / 2) tc::st_pack2(blk + ci * 8, zeros);
                    uint32_t pk[2 * NGP];
#pragma unroll
                    for (int g = 0; g < NGP; ++g)
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            if (g >= NG || tc::dead_slot(g, hh, NG)) { pk[2 * g + hh] = 0u; continue; }
                            float p0 = s[b][4 * g + 2 * hh] * sum[b][hh], p1 = s[b][4 * g + 2 * hh + 1] * sum[b][hh];
                            if (need_mask) {
                                // a neighbour outside the query's sequence is a zero V row in the reference: it counts in the
                                // softmax denominator but must not pick up the other sequence's values
                                const int j0 = jb[b][hh] + 8 * (g - hh);
                                if ((unsigned)j0 >= (unsigned)Trow) p0 = 0.f;
                                if ((unsigned)(j0 + 1) >= (unsigned)Trow) p1 = 0.f;
                            }
                            if constexpr (DROP) {
                                // attention dropout on the normalised probabilities; the row's log-sum-exp is not affected
                                const int off = 8 * (g - hh) + fa;
                                const uint32_t row = SEG ? (uint32_t)((scur.b * gm.H + scur.h) * T + (scur.i * kTileM + rb + 16 * b + 8 * hh + fr) * sg.d + scur.r)
                                                         : (uint32_t)(g0 + rb + 16 * b + 8 * hh + fr);
                                p0 = drop_hash(row, (uint32_t)(off >> dshift), drop.seed) >= drop.threshold ? p0 * drop.scale : 0.f;
                                p1 = drop_hash(row, (uint32_t)((off + 1) >> dshift), drop.seed) >= drop.threshold ? p1 * drop.scale : 0.f;
                            }
                            pk[2 * g + hh] = Cvt<E>::pack2(p0, p1);
                        }
                    tc::st_pack<NGP>(blk + c0 * 8, pk);
                }
                ptx::tmem_st_wait();
            }
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&misc->p_ready);

            // epilogue: O -> 16 bits -> the tile's idle V buffer (same swizzle as the tensor map) -> TMA store
            if (!ptx::mbar_wait(&misc->o_ready, it & 1) || *abort_flag) { atomicExch(&g_tc_status, 5); *abort_flag = 1; break; }
            ptx::tc_fence_after_sync();
            {
                uint8_t* sO = smem + L.ring + (it & 1) * L.stage_bytes + L.stage_v;  // this tile's V buffer: P.V has retired
                // row r, 16-byte chunk c at r*rowbytes + ((c ^ swz(r)) * 16): the TMA swizzle of this row size
                const int swz = (C == 64) ? (r & 7) : (C == 32) ? ((r >> 1) & 3) : ((r >> 2) & 1);
                // columns per round: two rounds keep the register count down; with 8 softmax warps the two warps of a lane
                // quarter take one half of the columns each
                constexpr int HALF = (NSW == 8 || C >= 32) ? C / 2 : C;
#pragma unroll
                for (int c0 = (NSW == 8 ? bo * HALF : 0); c0 < (NSW == 8 ? (bo + 1) * HALF : C); c0 += HALF) {
                    float acc[HALF], accb[HALF];
#pragma unroll
                    for (int c = 0; c < HALF; c += 8) {
                        ptx::tmem_ld8(lane_base + kOCol + c0 + c, &acc[c]);
                        ptx::tmem_ld8(lane_base + kOColB + c0 + c, &accb[c]);
                    }
                    ptx::tmem_ld_wait();
                    if (NSW == 8 || c0 + HALF >= C) {
                        ptx::tc_fence_before_sync();
                        ptx::mbar_arrive(&misc->o_free);
                    }
#pragma unroll
                    for (int c = 0; c < HALF; ++c) acc[c] += accb[c];
#pragma unroll
                    for (int c = 0; c < HALF / 8; ++c)
                        *reinterpret_cast<uint4*>(sO + r * kRowBytes + (((c0 / 8 + c) ^ swz) * 16)) = Cvt<E>::pack(&acc[c * 8]);
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(&misc->o_staged);  // the store thread takes it from here
            }
            if constexpr (SEG) scur.advance(); else cur.advance();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        ptx::tmem_dealloc(tmem, kTmemCols);
    }
}

template <typename E, int C, int WB, bool SEG, int MODE, bool DROP>
cudaError_t launch_fwd(const FwdMaps<SEG ? 2 : 1>& maps, float* lse, float* band, const float* rpb, const int* valid_len,
                       const Geometry& gm, const SegGeom& sg, int KT, int total, int sm_count, bool pdl, const DropoutCfg& drop,
                       cudaStream_t st) {
    const int smem = fwd_layout(C, KT, table_heads(rpb != nullptr, gm.H, MODE), (MODE == kBandOut && softmax_warps(C, MODE) == 8) ? gm.win : 0).total;
    auto kern = tc_fwd_kernel<E, C, WB, SEG, MODE, DROP>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    if constexpr (softmax_warps(C, MODE) == 8) {
        // The warp groups of this variant trade registers among themselves (2 x 104 + 32 per thread): the CTA's pool must
        // hold 3 x 80, i.e. the kernel must have been compiled to 80 registers, or the softmax warps would wait for
        // registers that never come. Checked once per variant; a build that breaks it fails here, not on the GPU.
        static const int regs = [] {
            cudaFuncAttributes fa;
            return cudaFuncGetAttributes(&fa, tc_fwd_kernel<E, C, WB, SEG, MODE, DROP>) == cudaSuccess ? fa.numRegs : 0;
        }();
        if (regs < 80) return cudaErrorLaunchOutOfResources;
    }
    const int per_sm = (2 * (smem + 1024) <= 227 * 1024) ? 2 : 1;
    const int slots = sm_count * per_sm;
    const int grid = total < slots ? total : slots;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)fwd_threads(softmax_warps(C, MODE)));
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, maps, lse, band, rpb, valid_len, gm, sg, KT, total, drop);
}

// Picks the instantiation for (element type, channels, window bucket); `wb` is the window the band fragments must hold.
template <bool SEG, int MODE = kFused, bool DROP = false>
cudaError_t dispatch_fwd(const FwdMaps<SEG ? 2 : 1>& maps, float* lse, float* band, const float* rpb, const int* valid_len,
                         const Geometry& gm, const SegGeom& sg, int KT, int total, int wb, int dtype, cudaStream_t st,
                         const DropoutCfg& drop = DropoutCfg{0u, 0u, 1.f}) {
    const int sms = device_sm_count();
    const bool pdl = pdl_mode() == 1 || pdl_mode() == 2;
#define NA1D_TC_FWD(E, C, WB) return launch_fwd<E, C, WB, SEG, MODE, DROP>(maps, lse, band, rpb, valid_len, gm, sg, KT, total, sms, pdl, drop, st)
#define NA1D_TC_FWD_W(E, C)                        \
    if (wb <= 9) { NA1D_TC_FWD(E, C, 9); }         \
    else if (wb <= 17) { NA1D_TC_FWD(E, C, 17); }  \
    else { NA1D_TC_FWD(E, C, 33); }
#define NA1D_TC_FWD_C(E)                          \
    if (gm.C == 64) { NA1D_TC_FWD_W(E, 64) }      \
    else if (gm.C == 32) { NA1D_TC_FWD_W(E, 32) } \
    else { NA1D_TC_FWD_W(E, 16) }
    if (dtype == 0) { NA1D_TC_FWD_C(__nv_bfloat16) } else { NA1D_TC_FWD_C(__half) }
#undef NA1D_TC_FWD
#undef NA1D_TC_FWD_W
#undef NA1D_TC_FWD_C
}

// Reads and clears this translation unit's device status word (synchronises the device). 0 = no bounded wait expired.
int read_status_word() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
    return v;
}

}  // namespace
}  // namespace na1d

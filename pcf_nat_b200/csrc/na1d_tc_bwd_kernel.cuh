// Fused NA1D backward on the Blackwell tensor path (sm_100a): persistent, warp-specialised.
//
// Tiling. Rows are tiled over the FLATTENED (sequence, token) axis, so tiles are full whatever T is; a neighbour that
// falls outside the query's own sequence is the reference's zero-padded row and is excluded per element.
// A tile is a window W of 128 consecutive flattened rows; consecutive tiles start
// `stride = 128-(win-1)` rows apart, so they overlap by win-1 rows. All 128 rows act as queries
// (their band needs keys [w0-left, w0+127+right]; K and V are staged as KT = round16(128+win-1) rows
// starting at w0-left). A key row is "interior" when every query that attends it lies in W, which
// holds for rows [right, 128-left) of W -- exactly `stride` rows, and these are the rows whose dQ, dK
// and dV this tile stores. Every (query,key) pair of the
// band is thus seen with both rows inside one tile: no atomics, no second key-owned recomputation,
// deterministic results.
//
// Per tile (one CTA per SM, 384 threads):
//   warp 8  : TMA producer -- Q[W], dO[W], K[KT], V[KT] into a 2-stage ring (plain tile loads,
//             out-of-range rows arrive as zeros = the reference's zero padding).
//   warps 9-11: MMA issuers -- batch 1: S = Q.K^T, dP = dO.V^T (TMEM, N=KT);
//                            batch 2: dQ = dS.K, dV = P^T.dO, dK = dS^T.Q. One warp per accumulator chain.
//             Batch 1 of the NEXT tile is issued before batch 2 of the current one, so the compute warps
//             work on tile i+1 while the tensor pipe finishes tile i.
//   warps0-3: compute. Warp w owns query rows 32w..32w+31 (its TMEM lanes) as two 16-row blocks, read as
//             accumulator fragments (see na1d_tc_common.cuh). P = exp(S - lse) from the saved
//             log-sum-exp, delta = sum P.dP over the row (equal to dot(dO,O), so neither O nor a separate
//             delta pass is needed; two quad shuffles), dS = P(dP - delta). P and dS go to shared memory with
//             stmatrix as 16-bit row-major [query][key] matrices in 8x8 core-matrix order; the same bytes
//             serve as the K-major A operand of dQ = dS.K and as the MN-major A operand of
//             dK = dS^T.Q / dV = P^T.dO, so no transpose is ever materialised.
//   warps4-7: epilogue. Read dQ/dK/dV from TMEM (row m of dQ is query w0+m, row m of dK/dV is key
//             w0-left+m), round to 16 bits, stage the `stride` owned rows in the tile's idle Q/dO/K buffers
//             in the TMA swizzle and issue three TMA tile stores (rows >= T are clipped by the tensor map).
// Replaces the four backward launches of the reference (na1d_tensorcore/nattn.py:46-54, 69-78) and
// the eager softmax backward between them.
//
// Segmented variant (template parameter SEG): tiles lie inside one residue sequence (tokens t = r mod d of one (batch, head)
// sequence), addressed through 5-D tensor maps over tensors with arbitrary batch/head/token strides; see the forward
// kernel's header. Tile i of a residue sequence is the window of 128 tokens starting at token i * stride - right of it;
// tokens before 0 and from the sequence's length on are zero-filled on loads, inactive as queries and clipped on stores.
//
// This header is compiled into several translation units (flat / segmented, per element type); everything in it has
// internal linkage.
#pragma once
#include "na1d_internal.h"
#include <type_traits>
#include "na1d_tc_common.cuh"

namespace na1d {
namespace {

// Device status word of this translation unit (device symbols are per file without relocatable device code).
__device__ int g_tc_bwd_status = 0;

using tc::kTileM;
using tc::round_up;
using tc::RowSwizzle;
using tc::Fmt;
// Warp roles: NCW compute warps (0 .. NCW-1), four epilogue warps, the producer warp, three MMA-issuer warps.
// NCW = 4: compute warp w owns the 32 tensor-memory lanes of quarter w, two 16-row blocks one after the other or together.
// NCW = 8 (rows of at most 64 bytes, where registers allow 512 threads): warps w and w + 4 share quarter w & 3 and take one
// 16-row block each, so every scheduler has two compute warps to hide the latencies of the dependent chain
// TMEM load -> exp -> shuffle -> pack -> stmatrix behind one another.
__host__ __device__ constexpr int compute_warps(int C, int mode) { return (C <= 32 && mode == 0) ? 8 : 4; }
__host__ __device__ constexpr int bwd_threads(int ncw) { return (ncw + 8) * 32; }
constexpr int kQ = 0, kDO = 1, kK = 2, kV = 3;  // buffers of a stage
constexpr int kTmemCols = 512;
constexpr int kColDP = 160, kColDQ = 320, kColDK = 384, kColDV = 448;
constexpr int kBiasPad = 16;  // bias table index = kk + kBiasPad; fragment neighbour indices start at -15

struct BwdSmemLayout {
    int stage_q, stage_do, stage_k, stage_v, stage_bytes;  // offsets inside one stage
    int ds, p, out, misc, total;
    bool own_out;  // a dedicated 128-row staging buffer for the outputs fits next to everything else
    int out_bufs;  // how many of them: 3 (one per output: the three TMA stores of a tile go out together and are only waited
                   // for when the next tile needs the buffers), 1 (three rounds through one buffer) or 0
};
constexpr int kBiasRowB = 16 + 48;  // per-head table: log2e * rpb[h][kk] at index kk + 16, kk in [-16, 48)
// Depth of the operand ring: 64-channel tiles fill shared memory with two stages; narrower rows leave room for a third, which
// takes the TMA load latency (about 3 k cycles under load) out of the loop "batch 2 retires -> refill -> batch 1 -> compute".
__host__ __device__ constexpr int bwd_stages(int C) { return C == 64 ? 2 : 3; }
__host__ __device__ inline BwdSmemLayout bwd_layout(int C, int KT, int bias_heads, int acc_floats) {
    BwdSmemLayout L;
    L.stage_q = 0;
    L.stage_do = L.stage_q + round_up(kTileM * C * 2, 1024);
    L.stage_k = L.stage_do + round_up(kTileM * C * 2, 1024);
    L.stage_v = L.stage_k + round_up(KT * C * 2, 1024);
    L.stage_bytes = L.stage_v + round_up(KT * C * 2, 1024);
    L.ds = bwd_stages(C) * L.stage_bytes;  // dS [128 queries][KT keys]
    L.p = L.ds + kTileM * KT * 2;       // P  [128 queries][KT keys]
    L.out = L.p + kTileM * KT * 2;
    // misc block, bias table, bias-gradient accumulator, alignment slack
    const int tail = 512 + round_up(bias_heads * kBiasRowB * 4, 256) + round_up(acc_floats * 4, 256) + 1008;
    const int out_buf = round_up(kTileM * C * 2, 1024);
    L.out_bufs = L.out + 3 * out_buf + tail <= 227 * 1024 ? 3 : L.out + out_buf + tail <= 227 * 1024 ? 1 : 0;
    L.own_out = L.out_bufs > 0;
    L.misc = L.out + L.out_bufs * out_buf;
    L.total = L.misc + tail;
    return L;
}

// Bias gradient of neighbours outside the query's own sequence (rare: only padded query rows next to a sequence end have
// a non-zero probability there). Not inlined, to keep the many call sites of the unrolled loops small.
// row = this head's row of d_rpb, off = window offset of g0 (g1: off + 1); a non-zero gradient implies an offset that is a
// neighbour (a multiple of the dilation, 1 << dshift).
__device__ __noinline__ void bias_grad_outside(float* row, int off, int dshift, float g0, float g1) {
    if (g0 != 0.f) atomicAdd(row + (off >> dshift), g0);
    if (g1 != 0.f) atomicAdd(row + ((off + 1) >> dshift), g1);
}

// Bias gradient of one tile, one warp: sums of dS along the band's diagonals over the warp's owned query rows, read back
// from a 16-bit, scaled dS matrix in 8x8 core-matrix order (element (q, c) at (q/8) lboq + (c/8) 128 + (q%8) 16 + (c%8) 2): the
// dS operand of the tile, or the warp's private copy of its block (see the kernel). The warp's ROWS
// consecutive tile rows start at r0; lane l holds hr = the head of row r0 + l (-1: a row this tile does not own, and lanes
// past ROWS). A lane owns a WINDOW OFFSET, not a row: lane group rg = lane / NV walks the rows rg, rg + G, ... and adds up
// dS[row, row + i] for its offset i = lane % NV, so whether a row counts and for which head is the same for all lanes of
// a group at every step, nothing is exchanged until the G groups are added up (log2 G shuffles), and distinct lanes add
// to distinct accumulator entries (no atomics). ROWS rows span at most two sequences (T >= 32), hence two heads: two sums.
// (One lane per ROW with a shuffle butterfly over the 32 rows cost 3x the whole kernel's time at 33 offsets.) Offset NV
// exists only when the window fills its bucket. Not inlined: it keeps the tile loop short.
template <typename E, int NV, int ROWS, bool ATOMIC>
__device__ __noinline__ void bias_grad_tile(const uint8_t* ds, int lboq, int r0, int lane, int hr, int win, int ref_win,
                                            int dmask, int dshift, float inv_scale, float* acc) {
    const unsigned owned = __ballot_sync(0xffffffffu, hr >= 0);
    if (owned == 0) return;
    const int head_a = __shfl_sync(0xffffffffu, hr, __ffs(owned) - 1);
    const unsigned in_a = __ballot_sync(0xffffffffu, hr == head_a);
    const unsigned in_b = owned & ~in_a;
    const int head_b = __shfl_sync(0xffffffffu, hr, in_b ? __ffs(in_b) - 1 : 0);
    constexpr int G = 32 / NV, NR = ROWS / G;
    const int i = lane % NV, rg = lane / NV;
    const uint32_t base = ptx::smem_u32(ds);
    auto entry = [&](int row, int col) -> float {
        unsigned short raw;
        asm volatile("ld.shared.u16 %0, [%1];"
                     : "=h"(raw) : "r"(base + (uint32_t)((row >> 3) * lboq + (row & 7) * 16 + (col >> 3) * 128 + (col & 7) * 2)));
        return Cvt<E>::from_bits(raw);
    };
    auto add = [&](int head, int off, float x) {
        float* dst = acc + head * ref_win + (off >> dshift);
        if constexpr (ATOMIC) atomicAdd(dst, x * inv_scale); else *dst += x * inv_scale;
    };
    // all loads first (they are independent), then the sums; the second head only when the rows do cross a sequence end
    float v[NR];
#pragma unroll
    for (int k = 0; k < NR; ++k) v[k] = entry(r0 + k * G + rg, r0 + k * G + rg + i);
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int k = 0; k < NR; ++k) a += ((in_a >> (k * G + rg)) & 1u) ? v[k] : 0.f;
    if (in_b) {
#pragma unroll
        for (int k = 0; k < NR; ++k) b += ((in_b >> (k * G + rg)) & 1u) ? v[k] : 0.f;
    }
#pragma unroll
    for (int o = NV; o < 32; o <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    if (rg == 0 && i < win && (i & dmask) == 0) {
        add(head_a, i, a);
        if (in_b) add(head_b, i, b);
    }
    if (win > NV) {  // offset NV: one row per lane, then a sum over the lanes
        const int rl = lane < ROWS ? lane : 0;
        const float x = lane < ROWS ? entry(r0 + rl, r0 + rl + NV) : 0.f;
        float a2 = ((in_a >> rl) & 1u) ? x : 0.f, b2 = ((in_b >> rl) & 1u) ? x : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a2 += __shfl_xor_sync(0xffffffffu, a2, o);
            b2 += __shfl_xor_sync(0xffffffffu, b2, o);
        }
        if (lane == 0) {
            add(head_a, NV, a2);
            if (in_b) add(head_b, NV, b2);
        }
    }
}

// Bias gradient of one tile from a warp's private copy of its block's dS band (8 compute warps): 16 rows of PITCH 16-bit
// values, entry (row q, window offset kk) at q * PITCH + 8 + kk + (q & 1) -- the shift by the row's parity makes every
// thread's pair of adjacent offsets a 4-byte aligned store, the 8 leading cells and the overlap into the next row's
// leading cells take the fragment slots left and right of the band (always 0). Rows the tile does not own were stored as
// zeros, so lane i just adds up column i. The caller says (warp-uniform, from its row cursor -- no votes here) which rows
// [lo, hi) are owned and from which row `split` on they belong to the next sequence (head_b instead of head_a); only a
// warp whose owned rows do span two sequences separates the two sums. One shared reduction per lane and head.
template <typename E, int PITCH>
__device__ __forceinline__ void bias_grad_rows(const uint8_t* copy, int lane, int lo, int hi, int split, int head_a, int head_b,
                                            int win, int ref_win, int dmask, int dshift, float inv_scale, float* acc) {
    const uint32_t base = ptx::smem_u32(copy) + (uint32_t)(8 + lane) * 2u;
    float v[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) {
        unsigned short raw;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(raw) : "r"(base + (uint32_t)((q * PITCH + (q & 1)) * 2)));
        v[q] = Cvt<E>::from_bits(raw);
    }
    auto red = [&](int head, int off, float x) {
        asm volatile("red.shared.add.f32 [%0], %1;" ::"r"(ptx::smem_u32(acc + head * ref_win + (off >> dshift))), "f"(x * inv_scale) : "memory");
    };
    const float t = (((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]))) +
                    (((v[8] + v[9]) + (v[10] + v[11])) + ((v[12] + v[13]) + (v[14] + v[15])));
    const bool two = split > lo && split < hi;      // owned rows on both sides of a sequence end
    float b = 0.f;
    if (two) {
#pragma unroll
        for (int q = 0; q < 16; ++q) b += q >= split ? v[q] : 0.f;
    }
    if (lane < win && (lane & dmask) == 0) {
        red(split > lo ? head_a : head_b, lane, t - b);
        if (two) red(head_b, lane, b);
    }
    if (win > 32) {  // offset 32 (a window of 33): one row per lane, then a sum over the lanes
        float x = 0.f;
        if (lane < 16) {
            unsigned short raw;
            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(raw) : "r"(ptx::smem_u32(copy) + (uint32_t)((lane * PITCH + 8 + 32 + (lane & 1)) * 2)));
            x = Cvt<E>::from_bits(raw);
        }
        float b2 = (two && lane >= split) ? x : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            x += __shfl_xor_sync(0xffffffffu, x, o);
            b2 += __shfl_xor_sync(0xffffffffu, b2, o);
        }
        if (lane == 0) {
            red(split > lo ? head_a : head_b, 32, x - b2);
            if (two) red(head_b, 32, b2);
        }
    }
}

// The layout as both the launcher and the kernel compute it (one function, so they cannot disagree): bias table for every
// head when there is a bias, four per-warp (H, win) accumulators when its gradient is wanted.
// a warp's private copy of its block's dS band: 16 rows of (8 + window bucket + 1) 16-bit cells and the last row's overlap
__host__ __device__ constexpr int bias_copy_bytes(int KT) { return KT > 144 ? 1408 : 896; }
__host__ __device__ inline BwdSmemLayout bwd_layout_for(int C, int KT, const Geometry& gm, bool has_bias, bool wants_bias_grad,
                                                        int ncw = 0) {
    if (ncw == 0) ncw = compute_warps(C, 0);
    // bias gradient. 4 compute warps: one (H, win) accumulator per warp. 8 compute warps: one accumulator for the CTA and, per
    // warp, a private 16-bit copy of its block's dS band (16 rows x 8 NG columns in core-matrix order; NG <= 4 below the
    // widest bucket, 6 in it)
    const int acc = ncw == 8 ? round_up(gm.H * gm.win, 32) + 8 * bias_copy_bytes(KT) / 4 : ncw * gm.H * gm.win;
    return bwd_layout(C, KT, has_bias ? gm.H : 1, wants_bias_grad ? acc : 0);   // without a bias: one table row of 0 / -inf
}

struct alignas(8) BwdMisc {
    // ring barriers per stage and per buffer (kQ, kDO, kK, kV): each buffer is refilled as soon as its last reader retires
    uint64_t full[3][4], empty[3][4];
    uint64_t s_ready, s_free, p_ready, o_ready;
    uint64_t o_free[3];  // per accumulator (dQ, dV, dK): its MMA chain restarts as soon as the epilogue has drained it
    uint64_t acc_done;   // all compute threads have added their last tile to the bias-gradient accumulator
    uint32_t tmem_base;
    int abort;
};

// Tensor maps of one launch: one per tensor in the flat tiling, two in the segmented one (residues with Tp and with
// Tp - 1 tokens).
template <int NSETS> struct BwdMaps {
    CUtensorMap q[NSETS], d_o[NSETS], k[NSETS], v[NSETS], dq[NSETS], dk[NSETS], dv[NSETS];
};

// MODE selects what the kernel computes with the same tiles, rings and operand matrices:
//   kBwdFused : dq, dk, dv (and d_rpb) of the fused operator
//   kBandT    : out[j] = sum over the (t, kk) whose neighbour is j of band[t, kk] x[t] -- the unfused dK = dS^T.Q and
//               dV = P^T.dO (na1d_tensorcore/bf16_ana1d_kernel.cu:394-492): the fp32 band comes from global memory through
//               `lse`'s slot, x through the dO maps, out through the dV maps; only the dV chain of MMAs runs. The band is
//               rounded to 16 bits before the product, as the reference does (:409-415).
constexpr int kBwdFused = 0, kBandT = 1;

template <typename E, int C, int WB, bool OWN_OUT, bool SEG, int MODE = kBwdFused, bool DROP = false>
__global__ void __launch_bounds__(bwd_threads(compute_warps(C, MODE)), 1)
tc_bwd_kernel(const __grid_constant__ BwdMaps<SEG ? 2 : 1> tm, float* __restrict__ d_rpb, int drpb_direct,
              const float* __restrict__ lse,
              const float* __restrict__ rpb, const int* __restrict__ valid_len, Geometry gm, SegGeom sg, int stride, int KT,
              int total_tiles, DropoutCfg drop) {
    // With attention dropout (DROP) the forward used P' = P * keep / (1 - p): here dP = keep / (1 - p) * (dO.V^T), the P operand
    // of dV = P'^T.dO carries the same factor, and dS = P (dP - sum P dP) uses the undropped P; the keep decisions are
    // re-derived from (seed, dense row index, neighbour index), nothing was stored.
    constexpr int NG = tc::band_groups(WB);  // 8-column groups holding the band of a 16-row block
    constexpr int NS = bwd_stages(C);         // ring depth: tile `it` uses stage it % NS in ring round it / NS
    constexpr int NCW = compute_warps(C, MODE);
    constexpr int kThreads = bwd_threads(NCW), kProducerWarp = NCW + 4, kMmaWarp = NCW + 5, kEpiTid = NCW * 32;
    constexpr int kRegsCompute = 176, kRegsEpilogue = 104, kRegsIssue = 56;   // per thread, after the warp groups rebalance
    constexpr int kRowBytes = C * 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int n_bias = gm.H * gm.win;  // entries of the bias gradient
    const BwdSmemLayout L = bwd_layout_for(C, KT, gm, rpb != nullptr, d_rpb != nullptr, NCW);
    uint8_t* sDS = smem + L.ds;
    uint8_t* sP = smem + L.p;
    BwdMisc* misc = reinterpret_cast<BwdMisc*>(smem + L.misc);
    float* bias_tab = reinterpret_cast<float*>(smem + L.misc + 512);
    // accumulators of the bias gradient, one (H, win) array per compute warp: global atomics on the result -- one cache line
    // for the usual sizes -- serialise (5x the whole kernel's time when every tile issued them), so each warp adds up its
    // tiles here without atomics and the CTA hands over one row of partial sums at its end
    float* bias_acc = bias_tab + round_up((rpb ? gm.H : 1) * kBiasRowB, 64);
    // 8 compute warps: ONE accumulator for the CTA, and behind it every warp's private copy of its block's dS band. The
    // copy keeps the entries of neighbours outside the query's own sequence (they have a bias gradient but are zeroed in
    // the operand matrices) and is read back by its own warp right after the tile's stores, while batch 2 runs: the
    // read-back from the operand had to sit between "batch 2 retired" and "the next tile's stores", on the critical loop.
    constexpr bool kBiasCopy = NCW == 8;
    constexpr int kCopyPitch = 8 + WB + 1;   // 16-bit cells per row of a copy (even: WB is odd)
    uint8_t* bias_copy = reinterpret_cast<uint8_t*>(bias_acc + round_up(n_bias, 32));
    const int rows_total = gm.N * gm.T;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // flat tiling: the effective (dilated) window, neighbour kk of the reference is offset kk * dil of it;
    // segmented tiling: the dilation lives in the addressing, the window is the reference's own
    const int dil = SEG ? 1 : gm.dil, dmask = dil - 1, dshift = 31 - __clz(dil);
    const int win = tc::eff_window(gm.win, dil), left = gm.left * dil, right = (gm.win - 1 - gm.left) * dil, T = gm.T;
    const int lboq = KT * 16;  // bytes between 8-query groups of the dS matrix

    // Loads of tile `tile` (iteration `it` of this CTA) into ring stage it % NS, in the order in which the previous user of the
    // stage releases its buffers: V after batch 1, then K (dQ = dS.K is issued first in batch 2), dO (dV), Q (dK).
    tc::SegCursor pcur = {};  // position of the producer thread's next tile (segmented tiling)
    auto produce = [&](int tile, int it) -> bool {
        const int s = it % NS, k = it / NS;
        // first row of the window: on the flattened axis, or inside the tile's residue sequence
        const int g0 = (SEG ? pcur.i : tile) * stride - right;
        const int set = SEG && pcur.r >= sg.ra ? 1 : 0, rc = pcur.r - (set ? sg.ra : 0);
        uint8_t* st = smem + s * L.stage_bytes;
        bool ok = true;
        auto refill = [&](int buf, uint8_t* dst, const CUtensorMap* map, int rows, int row0) {
            if (!ok) return;
            if (!ptx::mbar_wait_relaxed(&misc->empty[s][buf], (k & 1) ^ 1) || *(volatile int*)&misc->abort) { ok = false; return; }
            ptx::mbar_expect_tx(&misc->full[s][buf], (uint32_t)(rows * kRowBytes));
            if constexpr (SEG) ptx::tma_load_5d(dst, map + set, &misc->full[s][buf], 0, row0, rc, pcur.h, pcur.b);
            else ptx::tma_load_3d(dst, map, &misc->full[s][buf], 0, row0, 0);
        };
        if constexpr (MODE == kBwdFused) {
            refill(kV, st + L.stage_v, tm.v, KT, g0 - left);
            refill(kK, st + L.stage_k, tm.k, KT, g0 - left);
        }
        refill(kDO, st + L.stage_do, tm.d_o, kTileM, g0);
        if constexpr (MODE == kBwdFused) refill(kQ, st + L.stage_q, tm.q, kTileM, g0);
        if constexpr (SEG) pcur.advance();
        return ok;
    };
    bool first_ok = true;
    if (tid == kProducerWarp * 32) {
        // The producer thread sets up the barriers and requests the CTA's first tile at once: the loads are in flight while
        // the other warps clear the operand matrices, allocate tensor memory and meet at the barrier below.
        for (int s = 0; s < NS; ++s)
            for (int b = 0; b < 4; ++b) { ptx::mbar_init(&misc->full[s][b], 1); ptx::mbar_init(&misc->empty[s][b], 1); }
        ptx::mbar_init(&misc->s_ready, 2);   // S chain and dP chain
        ptx::mbar_init(&misc->s_free, NCW * 32);
        ptx::mbar_init(&misc->p_ready, NCW * 32);
        ptx::mbar_init(&misc->o_ready, MODE == kBwdFused ? 3 : 1);   // dQ, dV, dK chains (only dV in the band-transpose mode)
        for (int i = 0; i < 3; ++i) ptx::mbar_init(&misc->o_free[i], 128);
        ptx::mbar_init(&misc->acc_done, NCW * 32);
        misc->abort = 0;
        ptx::fence_mbar_init();
        for (int i = 0; i < (SEG ? 2 : 1); ++i) {
            ptx::prefetch_tensormap(&tm.q[i]);
            ptx::prefetch_tensormap(&tm.d_o[i]);
            ptx::prefetch_tensormap(&tm.k[i]);
            ptx::prefetch_tensormap(&tm.v[i]);
            ptx::prefetch_tensormap(&tm.dq[i]);
            ptx::prefetch_tensormap(&tm.dk[i]);
            ptx::prefetch_tensormap(&tm.dv[i]);
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
    {   // operand matrices start as zeros; each warp rewrites the slab of its own rows every tile
        uint4* z = reinterpret_cast<uint4*>(sDS);
        const int n16 = 2 * kTileM * KT * 2 / 16;
        for (int i = tid; i < n16; i += kThreads) z[i] = make_uint4(0, 0, 0, 0);
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = misc->tmem_base;
    volatile int* abort_flag = &misc->abort;
    // Outputs are written from here on: wait for the predecessor, and let the successor start its own set-up as this
    // grid drains.
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();

    // 512 threads (NCW = 8) leave 128 registers each, which the compute warps' 16-row block does not fit in (spills in the
    // tile loop); the epilogue, producer and issuer warps need far fewer. Warp groups 0-1 (compute) take what groups 2
    // (epilogue) and 3 (producer, issuers) give back, each at the head of its own branch
    // (the register allocator then treats every branch with its own budget): 2 x 176 + 104 + 56 = 4 x 128.
    if (warp >= NCW + 4) {
    if constexpr (NCW == 8) ptx::warpgroup_regs_shrink<kRegsIssue>();
    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int it = 1;
            bool ok = first_ok;
            for (int tile = blockIdx.x + gridDim.x; ok && tile < total_tiles; tile += gridDim.x, ++it) ok = produce(tile, it);
            if (!ok) { atomicExch(&g_tc_bwd_status, 11); *abort_flag = 1; }
        }
    } else if (warp >= kMmaWarp) {
        // ------------------------------------------------------------ MMA issuers
        // One tcgen05.mma costs its issuing thread about 120 cycles whatever its size (measured), far more than the
        // tensor pipe needs for these small shapes, but issuers in different warps overlap. Three warps therefore issue
        // the MMAs of the three independent accumulator chains:  role 0: dQ (the longest chain),  role 1: dP and dV,
        // role 2: S and dK.
        const int role = warp - kMmaWarp;
        if (lane == 0) {
            const uint32_t idesc_s = ptx::instr_desc(Fmt<E>::v, 0, 0, kTileM, (uint32_t)KT);
            const uint32_t idesc_dq = ptx::instr_desc(Fmt<E>::v, 0, 1, kTileM, (uint32_t)C);   // A K-major, B MN-major
            const uint32_t idesc_dkv = ptx::instr_desc(Fmt<E>::v, 1, 1, kTileM, (uint32_t)C);  // A MN-major, B MN-major
            const uint32_t ds_a = ptx::smem_u32(sDS), p_a = ptx::smem_u32(sP);
            // key chunks of dQ = dS.K: the rows this tile owns end at 128 - left, their neighbours at column 127 + right
            const int nks = min(KT / 16, (kTileM + right + 15) / 16);
            // this role's part of batch 1 of tile `jt`: S = Q.K^T -> cols [0,KT) (role 2), dP = dO.V^T -> cols [160,160+KT) (role 1)
            auto batch1_ready = [&](int jt) -> bool {  // non-blocking: have this role's two operands of tile jt landed?
                const int s = jt % NS, k = jt / NS;
                return ptx::mbar_try_wait(&misc->full[s][role == 2 ? kK : kV], k & 1) &&
                       ptx::mbar_try_wait(&misc->full[s][role == 2 ? kQ : kDO], k & 1);
            };
            auto batch1 = [&](int jt) {
                const int s = jt % NS;
                const uint32_t st = ptx::smem_u32(smem + s * L.stage_bytes);
                ptx::tc_fence_after_sync();
                const uint64_t da0 = ptx::smem_desc(st + (role == 2 ? L.stage_q : L.stage_do), 16, 8 * kRowBytes, RowSwizzle<C>::umma);
                const uint64_t db0 = ptx::smem_desc(st + (role == 2 ? L.stage_k : L.stage_v), 16, 8 * kRowBytes, RowSwizzle<C>::umma);
                const uint32_t dcol = tmem + (role == 2 ? 0u : (uint32_t)kColDP);
#pragma unroll
                for (int ks = 0; ks < C / 16; ++ks)
                    ptx::mma_ss(dcol, tc::desc_advance(da0, ks * 32), tc::desc_advance(db0, ks * 32), idesc_s, ks > 0 ? 1u : 0u);
                if (role == 1) ptx::mma_commit(&misc->empty[s][kV]);  // nothing else reads V
                ptx::mma_commit(&misc->s_ready);
            };
            // Two job streams per issuer: batch 1 of iteration j (roles 1 and 2; needs the compute warps to have read S/dP of
            // iteration j-1 and the operands of tile j in shared memory) and batch 2 of iteration i (needs the compute warps'
            // operand matrices and the drained accumulator). Whichever is ready first is issued first, so a late TMA load never
            // holds back MMAs whose inputs are already there. Batch 1 runs at most one iteration ahead of batch 2.
            // band-transpose mode: no batch 1 at all, and only role 1 (the dV chain) has a batch 2
            const int n_it = (blockIdx.x < total_tiles && (MODE == kBwdFused || role == 1))
                                 ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
            int next_b1 = (role > 0 && MODE == kBwdFused) ? 0 : n_it, it = 0;
            uint32_t polls = 0;
            bool ok = true;
            while (it < n_it) {
                if (next_b1 < n_it && next_b1 <= it + 1 && (next_b1 == 0 || ptx::mbar_try_wait(&misc->s_free, (next_b1 - 1) & 1)) &&
                    batch1_ready(next_b1)) {
                    batch1(next_b1);
                    ++next_b1;
                    polls = 0;
                    continue;
                }
                if (!(ptx::mbar_try_wait(&misc->p_ready, it & 1) && ptx::mbar_try_wait(&misc->o_free[role], (it & 1) ^ 1) &&
                      (MODE == kBwdFused || ptx::mbar_try_wait(&misc->full[it % NS][kDO], (it / NS) & 1)))) {
                    if (++polls > (1u << 22) || *abort_flag) { ok = false; break; }
                    continue;
                }
                polls = 0;
                const int s = it % NS;
                const uint32_t st = ptx::smem_u32(smem + s * L.stage_bytes);
                ptx::tc_fence_after_sync();
                // batch 2. dS/P matrices: element (q, c) at (q/8)*lboq + (c/8)*128 + (q%8)*16 + (c%8)*2.
                if (role == 0) {
                    //   dQ = dS.K : A K-major (M = queries, K = KT keys): K-adjacent core matrices 128 B apart, 8-row groups lboq apart
                    const uint64_t a_dq = ptx::smem_desc(ds_a, 128, lboq, ptx::kSwizzleNone);
                    const uint64_t b_k = ptx::smem_desc(st + L.stage_k, 0, 8 * kRowBytes, RowSwizzle<C>::umma);
#pragma unroll 1
                    for (int ks = 0; ks < nks; ++ks)
                        ptx::mma_ss(tmem + kColDQ, tc::desc_advance(a_dq, ks * 256), tc::desc_advance(b_k, ks * 16 * kRowBytes), idesc_dq, ks > 0 ? 1u : 0u);
                    if constexpr (OWN_OUT) ptx::mma_commit(&misc->empty[s][kK]);   // K was read by S (long done) and dQ
                } else {
                    //   dV = P^T.dO (role 1), dK = dS^T.Q (role 2): the same matrices read MN-major (M = first 128 keys of the K
                    //   window, K = queries): 8-key groups 128 B apart, 8-query groups lboq apart
                    const uint64_t a_t = ptx::smem_desc(role == 1 ? p_a : ds_a, lboq, 128, ptx::kSwizzleNone);
                    const uint64_t b_t = ptx::smem_desc(st + (role == 1 ? L.stage_do : L.stage_q), 0, 8 * kRowBytes, RowSwizzle<C>::umma);
                    const uint32_t dcol = tmem + (role == 1 ? kColDV : kColDK);
#pragma unroll 1
                    for (int ks = 0; ks < kTileM / 16; ++ks)
                        ptx::mma_ss(dcol, tc::desc_advance(a_t, ks * 2 * lboq), tc::desc_advance(b_t, ks * 16 * kRowBytes), idesc_dkv, ks > 0 ? 1u : 0u);
                    if constexpr (OWN_OUT) ptx::mma_commit(&misc->empty[s][role == 1 ? kDO : kQ]);  // dO: dP and dV done; Q: S and dK done
                }
                ptx::mma_commit(&misc->o_ready);
                ++it;
            }
            if (!ok) { atomicExch(&g_tc_bwd_status, 12); *abort_flag = 1; }
        }
    }
    } else if (warp < NCW) {
        if constexpr (NCW == 8) ptx::warpgroup_regs_grow<kRegsCompute>();
        // ------------------------------------------------------------ compute warps
        const int cw = warp & 3;                        // quarter of the tensor-memory lanes (and tile rows) this warp works on
        const int bsel = warp >> 2;                     // NCW = 8: the 16-row block of that quarter this warp takes
        const int ct = warp * 32 + lane;                // index among the compute threads
        // row of the tile whose dS this lane reads back for the bias gradient: a warp reads back exactly the rows it is about
        // to overwrite (NCW = 8: its own 16-row block, on lanes 0-15)
        const int r = NCW == 8 ? cw * 32 + bsel * 16 + (lane & 15) : cw * 32 + lane;
        constexpr int kRowsPerWarp = NCW == 8 ? 16 : 32;
        const int r0w = cw * 32 + (NCW == 8 ? bsel * 16 : 0);   // first tile row of this warp
        const int fr = lane >> 2, fc = 2 * (lane & 3);  // fragment row / first column inside an 8x8 block
        const int fa = fc - fr;                         // neighbour index = 8(n-h) + e + fa
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
        const uint32_t ds_a = ptx::smem_u32(sDS), p_a = ptx::smem_u32(sP);
        if (d_rpb)
            for (int i = ct; i < (kBiasCopy ? 1 : NCW) * n_bias; i += NCW * 32) bias_acc[i] = 0.f;
        {
            // Table of every head's bias (one all-zero row without a bias), once per CTA, with -inf at every offset that is
            // not a neighbour (outside the window, between dilated neighbours): the fragment slots take their additive term
            // from it, and exp2 of it is the 0 of the slots outside the band -- no band test per slot. (Barrier among the
            // compute warps only.)
            const int heads = rpb ? gm.H : 1;
            for (int i = ct; i < heads * kBiasRowB; i += NCW * 32) {
                const int hh_ = i / kBiasRowB, kk = i - hh_ * kBiasRowB - kBiasPad;
                const bool nb = kk >= 0 && kk < win && (kk & dmask) == 0;
                bias_tab[i] = !nb ? -INFINITY : rpb ? __ldg(rpb + hh_ * gm.win + (kk >> dshift)) * kLog2e : 0.f;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        int it = 0;
        // log-sum-exp of the four fragment rows of a tile; loaded one tile ahead so the DRAM latency is hidden
        tc::RowCursor cur = {};  // flat tiling: row tile * stride = g0 + right
        tc::SegCursor scur = {};  // segmented tiling: the tile's residue sequence and its index in it
        if constexpr (SEG) scur.init((int)blockIdx.x, (int)gridDim.x, sg, gm.H);
        else cur.init(blockIdx.x * stride, T, gm.H, gridDim.x * stride);
        // one block per warp, flat tiling: a cursor of the thread's own first fragment row, so that the row facts of a tile
        // need no division
        constexpr bool kOwnCursor = !SEG && NCW == 8;
        tc::RowCursor mine = {};
        if constexpr (kOwnCursor) mine.init_signed((int)blockIdx.x * stride + cw * 32 + 16 * bsel + fr - right, T, gm.H, gridDim.x * stride);
        // fetches the log-sum-exp of tile `tile_`; in the segmented tiling `at` must stand on that tile
        auto load_lse = [&](int tile_, const tc::SegCursor& at, float (&dst)[2][2]) {
            const int g0_ = (SEG ? at.i : tile_) * stride - right;
            const int rows_ = SEG ? at.rows(sg) : rows_total;
            const float* base_ = SEG ? lse + (size_t)(at.b * gm.H + at.h) * T + at.r : lse;
            const int mul_ = SEG ? sg.d : 1;
            // one block per warp (NCW = 8): only that block's two rows, kept in dst[0]
#pragma unroll
            for (int b = 0; b < (NCW == 8 ? 1 : 2); ++b)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int gq = g0_ + cw * 32 + 16 * (NCW == 8 ? bsel : b) + 8 * hh + fr;
                    dst[b][hh] = (tile_ < total_tiles && gq >= 0 && gq < rows_) ? __ldg(base_ + (size_t)gq * mul_) : 0.f;
                }
        };
        float lse_next[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
        if constexpr (MODE == kBwdFused) load_lse(blockIdx.x, scur, lse_next);
        int prev_hr = -1;
        const int batch = gm.N / gm.H;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            // This tile's log-sum-exp was requested one tile ago; the next tile's is requested now, at the top, so that its
            // DRAM latency is over long before the values are used (requested at the end of the tile they stalled the
            // row facts of the next one for most of that latency).
            float lse_cur[2][2];
#pragma unroll
            for (int i = 0; i < 4; ++i) lse_cur[i >> 1][i & 1] = lse_next[i >> 1][i & 1];
            if constexpr (MODE == kBwdFused) {
                tc::SegCursor nxt = scur;
                if constexpr (SEG) nxt.advance();
                load_lse(tile + gridDim.x, nxt, lse_next);
            }
            // first row of the window: on the flattened axis, or inside the tile's residue sequence
            const int g0 = (SEG ? scur.i : tile) * stride - right;
            // tokens of the sequence the keys must lie in, and (segmented) the valid tokens of the residue sequence
            const int Trow = SEG ? scur.rows(sg) : T;
            int vl_seq = 0;
            if constexpr (SEG) {
                const int vl = valid_len ? min(T, __ldg(valid_len + scur.b)) : T;
                vl_seq = vl > scur.r ? (vl - scur.r + sg.d - 1) / sg.d : 0;
            }
            if constexpr (MODE == kBandT) {
                // the band of the tile's 128 query rows comes from global memory (fp32, `lse` points at it): slot (g, hh, e) of
                // row (b, hh) is band[row, kk]; 0 outside the band, for rows outside the tensor and for keys outside the row's
                // own sequence (they belong to another sequence's output rows)
                int jb[2][2];
                bool live4[2][2];
                {
                    int tq, hq, bq;
                    cur.row_at(cw * 32 + fr - right, inv_T, inv_H, tq, hq, bq);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int gq = g0 + cw * 32 + fr + 8 * k;
                        live4[k >> 1][k & 1] = gq >= 0 && gq < rows_total;
                        jb[k >> 1][k & 1] = tq - left + fa;
                        tc::row_step8(T, gm.H, tq, hq, bq);
                    }
                }
                uint32_t pk_p[2][2 * NG];
#pragma unroll
                for (int b = 0; b < 2; ++b)
#pragma unroll
                    for (int g = 0; g < NG; ++g)
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int gq = g0 + cw * 32 + 16 * b + 8 * hh + fr;
                            const float* src = lse + (size_t)min(max(gq, 0), rows_total - 1) * gm.win;
                            float p[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int kc = 8 * (g - hh) + e;
                                const bool on = !tc::dead_slot(g, hh, NG) && ((band_bits >> (2 * (g - hh + 1) + e)) & 1u) && live4[b][hh] &&
                                                (unsigned)(jb[b][hh] + kc) < (unsigned)T;
                                p[e] = on ? __ldg(src + ((kc + fa) >> dshift)) : 0.f;
                            }
                            pk_p[b][2 * g + hh] = Cvt<E>::pack2(p[0], p[1]);
                        }
                // the previous tile's MMAs must have finished reading the operand matrix before it is rewritten
                if (it > 0 && (!ptx::mbar_wait(&misc->o_ready, (it - 1) & 1) || *abort_flag)) { atomicExch(&g_tc_bwd_status, 16); *abort_flag = 1; break; }
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const uint32_t blk = (uint32_t)(4 * cw + 2 * b) * (uint32_t)lboq + (uint32_t)(4 * cw + 2 * b) * 128u;
                    tc::store_block_operand<NG>(p_a + blk, (uint32_t)lboq, pk_p[b], lane);
                }
                ptx::fence_proxy_async_smem();
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(&misc->p_ready);
                cur.advance();
                continue;
            } else if constexpr (WB == 33 || NCW == 8) {
                // Widest window bucket: the two 16-row blocks of the warp are processed one after the other in a ROLLED loop.
                // 48 fragment values of S and of dP per block and thread: holding both blocks at once spilled registers, and
                // the unrolled code of both did not fit the instruction cache (measured: 2-3x more cycles per tile).
                // the two rows of block b this thread sees (row half hh): see the comments of the unrolled path below
                float lse2[2];
                int jb[2], vle[2], hrow[2];
                bool ownr[2];                  // the tile owns the row (its band is complete here) and the row is in the tensor
                const float* btab[2];          // the rows' bias table entries of window offset fa
                uint32_t drow[2] = {0u, 0u};   // dense row index n*T + t of the two rows (dropout mask key)
                bool need_mask = false;
                auto row_facts = [&](int b) {
                        need_mask = false;
                        int tq = 0, hq = 0, bq = 0;
                        if constexpr (SEG) { tq = g0 + cw * 32 + 16 * b + fr; hq = scur.h; }
                        else if constexpr (kOwnCursor) { tq = mine.t; hq = mine.h; bq = mine.b; }
                        else cur.row_at(cw * 32 + 16 * b + fr - right, inv_T, inv_H, tq, hq, bq);
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int gq = g0 + cw * 32 + 16 * b + 8 * hh + fr;
                            const bool live = gq >= 0 && gq < (SEG ? Trow : rows_total);
                            const int vlr = !live ? 0 : SEG ? vl_seq : valid_len ? min(T, __ldg(valid_len + min(max(bq, 0), batch - 1))) : T;
                            hrow[hh] = hq;
                            ownr[hh] = live && cw * 32 + 16 * b + 8 * hh + fr >= right && cw * 32 + 16 * b + 8 * hh + fr < kTileM - left;
                            jb[hh] = tq - left + fa;
                            vle[hh] = !live ? -1 : tq >= vlr ? 0 : vlr;
                            need_mask |= tq < left || tq + right >= vlr;
                            lse2[hh] = !live ? INFINITY : (NCW != 8 && b ? lse_cur[1][hh] : lse_cur[0][hh]) * kLog2e;
                            btab[hh] = bias_tab + (rpb ? hq : 0) * kBiasRowB + kBiasPad + fa;
                            if constexpr (DROP) drow[hh] = SEG ? (uint32_t)((scur.b * gm.H + scur.h) * T + tq * sg.d + scur.r) : (uint32_t)gq;
                            if constexpr (SEG) tq += 8; else tc::row_step8(T, gm.H, tq, hq, bq);
                        }
                    need_mask = __any_sync(0xffffffffu, need_mask);
                };
                // one block per warp: its row facts do not depend on S, so they are worked out while the S chain still runs
                if constexpr (NCW == 8) row_facts(bsel);
                if (!ptx::mbar_wait(&misc->s_ready, it & 1) || *abort_flag) { atomicExch(&g_tc_bwd_status, 14); *abort_flag = 1; break; }
                ptx::tc_fence_after_sync();
                bool failed = false;
#pragma unroll 1
                for (int b = (NCW == 8 ? bsel : 0); b < (NCW == 8 ? bsel + 1 : 2); ++b) {
                    if constexpr (NCW != 8) row_facts(b);
                    float s1[4 * NG], d1[4 * NG];
                    const uint32_t a = lane_base + ((uint32_t)(16 * b) << 16) + (uint32_t)(cw * 32 + 16 * b);
                    tc::ld_frag<NG>(a, s1);
                    tc::ld_frag<NG>(a + kColDP, d1);
                    ptx::tmem_ld_wait();
                    if (b == 1 || NCW == 8) {  // S and dP of this tile (this warp's share of them) are out of tensor memory
                        ptx::tc_fence_before_sync();
                        ptx::mbar_arrive(&misc->s_free);
                    }
                    float delta[2] = {0.f, 0.f};
                    auto elements = [&](auto masked_tag) {
                        constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
                        for (int g = 0; g < NG; ++g)
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int idx = 4 * g + 2 * hh + e;
                                    if (tc::dead_slot(g, hh, NG)) { s1[idx] = 0.f; d1[idx] = 0.f; continue; }
                                    const int kc = 8 * (g - hh) + e;
                                    [[maybe_unused]] const int kk = kc + fa;
                                    float bias = btab[hh][kc];   // -inf outside the band
                                    float dot = s1[idx], dpv = d1[idx];
                                    if constexpr (kMasked) {
                                        const unsigned j = (unsigned)(jb[hh] + kc);
                                        if (j >= (unsigned)Trow) { dot = 0.f; dpv = 0.f; }
                                        if ((int)j >= vle[hh] || (int)j < 0) bias += mask2;
                                    }
                                    const float x = fmaf(dot, sc, bias) - lse2[hh];   // lse2 = +inf for rows outside the tensor
                                    float p = tc::fast_exp2(x);
                                    // A neighbour outside the query's sequence is a zero K/V row in the reference: its logit still
                                    // has a bias gradient, but neither P nor dS of it may reach the operand matrices. Without a
                                    // bias gradient nothing needs its probability: zero it here and the packing needs no masks.
                                    // With one (and 8 compute warps) the probability goes on NEGATED: its sign tells the packing
                                    // which entries go to the bias-gradient copy only (dpv is 0 there, so delta does not see it).
                                    if constexpr (kMasked)
                                        if ((unsigned)(jb[hh] + kc) >= (unsigned)Trow) p = !d_rpb ? 0.f : kBiasCopy ? -p : p;
                                    if constexpr (DROP)
                                        dpv = drop_hash(drow[hh], (uint32_t)(kk >> dshift), drop.seed) >= drop.threshold ? dpv * drop.scale : 0.f;
                                    s1[idx] = p;
                                    d1[idx] = dpv;
                                    delta[hh] = fmaf(p, dpv, delta[hh]);
                                }
                    };
                    if (need_mask) elements(std::true_type{}); else elements(std::false_type{});
                    delta[0] = tc::quad_sum(delta[0]);
                    delta[1] = tc::quad_sum(delta[1]);
                    uint32_t pk_p[2 * NG], pk_d[2 * NG], pk_b[kBiasCopy ? 2 * NG : 1];
#pragma unroll
                    for (int g = 0; g < NG; ++g)
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int idx = 4 * g + 2 * hh;
                            if (tc::dead_slot(g, hh, NG)) {
                                pk_d[2 * g + hh] = 0u; pk_p[2 * g + hh] = 0u;
                                if constexpr (kBiasCopy) pk_b[2 * g + hh] = 0u;
                                continue;
                            }
                            float p0 = s1[idx], p1 = s1[idx + 1];
                            const float t0 = (d1[idx] - delta[hh]) * gm.scale, t1 = (d1[idx + 1] - delta[hh]) * gm.scale;
                            if (kBiasCopy && need_mask && d_rpb) {
                                // negative = a neighbour outside the query's sequence: its dS goes to the bias-gradient copy, zeros
                                // go to the operand matrices
                                if constexpr (kBiasCopy) pk_b[2 * g + hh] = ownr[hh] ? Cvt<E>::pack2(fabsf(p0) * t0, fabsf(p1) * t1) : 0u;
                                p0 = fmaxf(p0, 0.f);
                                p1 = fmaxf(p1, 0.f);
                            }
                            float ds0 = p0 * t0, ds1 = p1 * t1;   // (scaled)
                            uint32_t dsp = Cvt<E>::pack2(ds0, ds1);
                            if constexpr (kBiasCopy)
                                if (!(need_mask && d_rpb)) pk_b[2 * g + hh] = ownr[hh] ? dsp : 0u;   // the bias gradient sees every band entry of an owned row
                            if (!kBiasCopy && need_mask && d_rpb) {
                                const int kc = 8 * (g - hh), kk0 = kc + fa;
                                const int j0 = jb[hh] + kc;
                                const int row = cw * 32 + 16 * b + 8 * hh + fr;
                                const bool own = d_rpb && row >= right && row < kTileM - left;
                                const bool out0 = (unsigned)j0 >= (unsigned)Trow, out1 = (unsigned)(j0 + 1) >= (unsigned)Trow;
                                if (out0 | out1) {
                                    // (ds is scaled here; the accumulators hold unscaled sums)
                                    if (own) bias_grad_outside(bias_acc + warp * n_bias + hrow[hh] * gm.win, kk0, dshift, out0 ? ds0 / gm.scale : 0.f, out1 ? ds1 / gm.scale : 0.f);
                                    if (out0) { ds0 = 0.f; p0 = 0.f; }
                                    if (out1) { ds1 = 0.f; p1 = 0.f; }
                                    dsp = Cvt<E>::pack2(ds0, ds1);
                                }
                            }
                            pk_d[2 * g + hh] = dsp;
                            if constexpr (DROP) {
                                const int off = 8 * (g - hh) + fa;
                                p0 = drop_hash(drow[hh], (uint32_t)(off >> dshift), drop.seed) >= drop.threshold ? p0 * drop.scale : 0.f;
                                p1 = drop_hash(drow[hh], (uint32_t)((off + 1) >> dshift), drop.seed) >= drop.threshold ? p1 * drop.scale : 0.f;
                            }
                            pk_p[2 * g + hh] = Cvt<E>::pack2(p0, p1);
                        }
                    if (b == 0 || NCW == 8) {
                        // Only the stores need the operand matrices: batch 2 of the previous tile must have finished reading
                        // them (everything above overlaps with it). The previous tile's bias gradient is read back from its
                        // dS operand first.
                        if (it > 0 && (!ptx::mbar_wait(&misc->o_ready, (it - 1) & 1) || *abort_flag)) { failed = true; break; }
                        if constexpr (!kBiasCopy)
                            if (d_rpb && it > 0)
                                bias_grad_tile<E, WB - 1, kRowsPerWarp, false>(sDS, lboq, r0w, lane, prev_hr, win, gm.win, dmask, dshift,
                                                                               1.f / gm.scale, bias_acc + warp * n_bias);
                    }
                    const uint32_t blk = (uint32_t)(4 * cw + 2 * b) * (uint32_t)lboq + (uint32_t)(4 * cw + 2 * b) * 128u;
                    tc::store_block_operand<NG>(ds_a + blk, (uint32_t)lboq, pk_d, lane);
                    tc::store_block_operand<NG>(p_a + blk, (uint32_t)lboq, pk_p, lane);
                    if constexpr (kBiasCopy)
                        if (d_rpb) {
                            // entry (row q, offset kk) at cell q * pitch + 8 + kk + (q & 1): the thread's pair (kk0, kk0 + 1), kk0
                            // of the row's parity, is one aligned 4-byte store
                            const uint32_t cp = ptx::smem_u32(bias_copy) + (uint32_t)(warp * bias_copy_bytes(KT)) +
                                                (uint32_t)((fr * kCopyPitch + 8 + fa + (fr & 1)) * 2);
#pragma unroll
                            for (int g = 0; g < NG; ++g)
#pragma unroll
                                for (int hh = 0; hh < 2; ++hh) {
                                    if (tc::dead_slot(g, hh, NG)) continue;
                                    asm volatile("st.shared.b32 [%0], %1;" ::"r"(cp + (uint32_t)((8 * hh * kCopyPitch + 8 * (g - hh)) * 2)), "r"(pk_b[2 * g + hh]) : "memory");
                                }
                        }
                }
                if (failed) { atomicExch(&g_tc_bwd_status, 16); *abort_flag = 1; break; }
            } else {
                // the four query rows this thread sees in the fragments: block b, row half hh (lse was fetched one tile ahead)
                // The four rows this thread sees in the fragments (local rows 32 warp + fr + 8k; lse was fetched one tile ahead):
                //   jb  : key index inside the row's own sequence of neighbour kk is jb + (kk - fa); outside [0, T) it is the
                //         reference's zero-padded K/V row
                //   vle : keys >= vle are masked (0 when the query itself is padding);  -1 marks a row outside the tensor
                float lse2[2][2];
                const float* btab[2][2];   // the rows' bias table entries of window offset fa
                int jb[2][2], vle[2][2], hrow[2][2];
                uint32_t drow[2][2] = {{0u, 0u}, {0u, 0u}};   // dense row index n*T + t of the four rows (dropout mask key)
                bool need_mask = false;
                {
                    int tq = 0, hq = 0, bq = 0;
                    if constexpr (SEG) { tq = g0 + cw * 32 + fr; hq = scur.h; }
                    else cur.row_at(cw * 32 + fr - right, inv_T, inv_H, tq, hq, bq);
    #pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int gq = g0 + cw * 32 + fr + 8 * k;
                        const bool live = gq >= 0 && gq < (SEG ? Trow : rows_total);
                        const int vlr = !live ? 0 : SEG ? vl_seq : valid_len ? min(T, __ldg(valid_len + min(max(bq, 0), batch - 1))) : T;
                        hrow[k >> 1][k & 1] = hq;
                        jb[k >> 1][k & 1] = tq - left + fa;
                        vle[k >> 1][k & 1] = !live ? -1 : tq >= vlr ? 0 : vlr;
                        need_mask |= tq < left || tq + right >= vlr;
                        lse2[k >> 1][k & 1] = !live ? INFINITY : lse_cur[k >> 1][k & 1] * kLog2e;
                        btab[k >> 1][k & 1] = bias_tab + (rpb ? hq : 0) * kBiasRowB + kBiasPad + fa;
                        if constexpr (DROP) drow[k >> 1][k & 1] = SEG ? (uint32_t)((scur.b * gm.H + scur.h) * T + tq * sg.d + scur.r) : (uint32_t)gq;
                        if constexpr (SEG) tq += 8; else tc::row_step8(T, gm.H, tq, hq, bq);
                    }
                }
                // masks are needed only when one of the warp's rows touches a sequence end or a padded region
                need_mask = __any_sync(0xffffffffu, need_mask);
                if (!ptx::mbar_wait(&misc->s_ready, it & 1) || *abort_flag) { atomicExch(&g_tc_bwd_status, 14); *abort_flag = 1; break; }
                ptx::tc_fence_after_sync();

                float s[2][4 * NG], d[2][4 * NG];
    #pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const uint32_t a = lane_base + ((uint32_t)(16 * b) << 16) + (uint32_t)(cw * 32 + 16 * b);
                    tc::ld_frag<NG>(a, s[b]);
                    tc::ld_frag<NG>(a + kColDP, d[b]);
                }
                ptx::tmem_ld_wait();
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(&misc->s_free);
                float delta[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
                // two straight-line copies of the element loop, with and without masks
                auto elements = [&](auto masked_tag) {
                    constexpr bool kMasked = decltype(masked_tag)::value;
    #pragma unroll
                    for (int b = 0; b < 2; ++b)
    #pragma unroll
                        for (int g = 0; g < NG; ++g)
    #pragma unroll
                            for (int hh = 0; hh < 2; ++hh)
    #pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int idx = 4 * g + 2 * hh + e;
                                    if (tc::dead_slot(g, hh, NG)) { s[b][idx] = 0.f; d[b][idx] = 0.f; continue; }
                                    const int kc = 8 * (g - hh) + e;
                                    [[maybe_unused]] const int kk = kc + fa;
                                    float bias = btab[b][hh][kc];   // -inf outside the band
                                    float dot = s[b][idx], dpv = d[b][idx];
                                    if constexpr (kMasked) {
                                        const unsigned j = (unsigned)(jb[b][hh] + kc);
                                        if (j >= (unsigned)Trow) { dot = 0.f; dpv = 0.f; }  // the reference's zero-padded K/V row
                                        if ((int)j >= vle[b][hh] || (int)j < 0) bias += mask2;
                                    }
                                    const float x = fmaf(dot, sc, bias) - lse2[b][hh];   // lse2 = +inf for rows outside the tensor
                                    float p = tc::fast_exp2(x);
                                    // without a bias gradient nothing needs the probability of a neighbour outside the query's
                                    // sequence: zero it here and the packing needs no masks
                                    if constexpr (kMasked) if (!d_rpb && (unsigned)(jb[b][hh] + kc) >= (unsigned)Trow) p = 0.f;
                                    if constexpr (DROP)
                                        dpv = drop_hash(drow[b][hh], (uint32_t)(kk >> dshift), drop.seed) >= drop.threshold ? dpv * drop.scale : 0.f;
                                    s[b][idx] = p;
                                    d[b][idx] = dpv;
                                    delta[b][hh] = fmaf(p, dpv, delta[b][hh]);
                                }
                };
                if (need_mask) elements(std::true_type{}); else elements(std::false_type{});
    #pragma unroll
                for (int b = 0; b < 2; ++b)
    #pragma unroll
                    for (int hh = 0; hh < 2; ++hh) delta[b][hh] = tc::quad_sum(delta[b][hh]);
                uint32_t pk_p[2][2 * NG], pk_d[2][2 * NG];
    #pragma unroll
                for (int b = 0; b < 2; ++b) {
    #pragma unroll
                    for (int g = 0; g < NG; ++g)
    #pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int idx = 4 * g + 2 * hh;
                            if (tc::dead_slot(g, hh, NG)) { pk_d[b][2 * g + hh] = 0u; pk_p[b][2 * g + hh] = 0u; continue; }
                            float ds0 = s[b][idx] * (d[b][idx] - delta[b][hh]);
                            float ds1 = s[b][idx + 1] * (d[b][idx + 1] - delta[b][hh]);
                            float p0 = s[b][idx], p1 = s[b][idx + 1];
                            if (need_mask && d_rpb) {   // (without a bias gradient these probabilities are already zero)
                                // a neighbour outside the query's sequence is a zero K/V row in the reference: its logit still has a
                                // bias gradient, but it must not reach the other sequence's dK/dV nor this query's dQ
                                const int kc = 8 * (g - hh), kk0 = kc + fa;
                                const int j0 = jb[b][hh] + kc;
                                const int row = cw * 32 + 16 * b + 8 * hh + fr;
                                const bool own = d_rpb && row >= right && row < kTileM - left;
                                const bool out0 = (unsigned)j0 >= (unsigned)Trow, out1 = (unsigned)(j0 + 1) >= (unsigned)Trow;
                                if (out0 | out1) {
                                    if (own) bias_grad_outside(bias_acc + warp * n_bias + hrow[b][hh] * gm.win, kk0, dshift, out0 ? ds0 : 0.f, out1 ? ds1 : 0.f);
                                    if (out0) { ds0 = 0.f; p0 = 0.f; }
                                    if (out1) { ds1 = 0.f; p1 = 0.f; }
                                }
                            }
                            pk_d[b][2 * g + hh] = Cvt<E>::pack2(ds0 * gm.scale, ds1 * gm.scale);
                            if constexpr (DROP) {
                                const int off = 8 * (g - hh) + fa;
                                p0 = drop_hash(drow[b][hh], (uint32_t)(off >> dshift), drop.seed) >= drop.threshold ? p0 * drop.scale : 0.f;
                                p1 = drop_hash(drow[b][hh], (uint32_t)((off + 1) >> dshift), drop.seed) >= drop.threshold ? p1 * drop.scale : 0.f;
                            }
                            pk_p[b][2 * g + hh] = Cvt<E>::pack2(p0, p1);
                        }
                }
                // Only the stores need the operand matrices: batch 2 of the previous tile must have finished reading them
                // (everything above overlaps with it).
                if (it > 0 && (!ptx::mbar_wait(&misc->o_ready, (it - 1) & 1) || *abort_flag)) { atomicExch(&g_tc_bwd_status, 16); *abort_flag = 1; break; }
                // Bias gradient of the PREVIOUS tile, read back from its dS operand now: while batch 2 runs its operand fetches own
                // the shared-memory bandwidth and the same read-back took thousands of cycles; here the tensor pipe is done with it.
                if (d_rpb && it > 0)
                    bias_grad_tile<E, WB - 1, kRowsPerWarp, false>(sDS, lboq, r0w, lane, prev_hr, win, gm.win, dmask, dshift, 1.f / gm.scale,
                                                                   bias_acc + warp * n_bias);
    #pragma unroll
                for (int b = 0; b < 2; ++b) {
                    // core matrix of the block's first row / first column: row group 4w+2b, column group 4w+2b
                    const uint32_t blk = (uint32_t)(4 * cw + 2 * b) * (uint32_t)lboq + (uint32_t)(4 * cw + 2 * b) * 128u;
                    tc::store_block_operand<NG>(ds_a + blk, (uint32_t)lboq, pk_d[b], lane);
                    tc::store_block_operand<NG>(p_a + blk, (uint32_t)lboq, pk_p[b], lane);
                }
            }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&misc->p_ready);
            if constexpr (kBiasCopy) {
                if (d_rpb) {
                    // This tile's share, from the warp's own copy (written by this warp just above: a warp-level barrier is all
                    // the ordering it needs), while the tensor pipe works on batch 2. Which of the warp's 16 rows the tile owns
                    // ([lo, hi): the same test as for the stored zeros) and where the next sequence starts (split) follow from
                    // the row cursor; the rows cross at most one sequence end.
                    int t0 = 0, h0 = SEG ? scur.h : 0;
                    if constexpr (kOwnCursor) { t0 = __shfl_sync(0xffffffffu, mine.t, 0); h0 = __shfl_sync(0xffffffffu, mine.h, 0); }
                    const int first = g0 + r0w;
                    const int lo = max(max(right - r0w, 0), -first);
                    const int hi = min(min(16, kTileM - left - r0w), (SEG ? Trow : rows_total) - first);
                    const int split = kOwnCursor ? T - t0 : 16;
                    __syncwarp();
                    if (hi > lo)
                        bias_grad_rows<E, kCopyPitch>(bias_copy + warp * bias_copy_bytes(KT), lane, lo, hi, split, h0, h0 + 1 == gm.H ? 0 : h0 + 1, win,
                                                      gm.win, dmask, dshift, 1.f / gm.scale, bias_acc);
                    __syncwarp();   // every lane has read the copy before any lane rewrites it in the next tile
                }
            } else if (d_rpb) {
                // head of the row this lane will read back (-1: a row this tile does not own)
                const int gr = g0 + r;
                prev_hr = -1;
                // (own cursor: lanes 0-3 stand on the warp's first row, and its 16 rows cross at most one sequence end)
                int t0 = 0, h0 = 0;
                if constexpr (kOwnCursor) { t0 = __shfl_sync(0xffffffffu, mine.t, 0); h0 = __shfl_sync(0xffffffffu, mine.h, 0); }
                if ((NCW == 4 || lane < 16) && r >= right && r < kTileM - left && gr >= 0 && gr < (SEG ? Trow : rows_total)) {
                    if constexpr (SEG) prev_hr = scur.h;
                    else if constexpr (kOwnCursor) prev_hr = t0 + (lane & 15) < T ? h0 : (h0 + 1 == gm.H ? 0 : h0 + 1);
                    else {
                        int tr, br;
                        cur.row_at(r - right, inv_T, inv_H, tr, prev_hr, br);
                    }
                }
            }
            if constexpr (SEG) scur.advance(); else cur.advance();
            if constexpr (kOwnCursor) mine.advance();
        }
        if constexpr (!kBiasCopy)
            if (d_rpb && it > 0 && ptx::mbar_wait(&misc->o_ready, (it - 1) & 1) && !*abort_flag)  // the last tile's share
                bias_grad_tile<E, WB - 1, kRowsPerWarp, false>(sDS, lboq, r0w, lane, prev_hr, win, gm.win, dmask, dshift, 1.f / gm.scale,
                                                               bias_acc + warp * n_bias);
        if (d_rpb) {
            // hand over this CTA's partial bias gradient: every compute thread arrives (also after an aborted loop), warp 0
            // waits for all of them and writes row blockIdx.x of the partial-sum matrix (or adds to the result directly when
            // the caller's scratch was too small for one row per CTA)
            ptx::mbar_arrive(&misc->acc_done);
            if (warp == 0 && ptx::mbar_wait(&misc->acc_done, 0)) {
                for (int i = lane; i < n_bias; i += 32) {
                    float x = bias_acc[i];   // 8 compute warps: the CTA's one accumulator
                    if constexpr (!kBiasCopy) x = (x + bias_acc[n_bias + i]) + (bias_acc[2 * n_bias + i] + bias_acc[3 * n_bias + i]);
                    if (drpb_direct) { if (x != 0.f) atomicAdd(d_rpb + i, x); }
                    else d_rpb[(size_t)blockIdx.x * n_bias + i] = x;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps (TMEM lanes 32 (warp - NCW) ..)
        if constexpr (NCW == 8) ptx::warpgroup_regs_shrink<kRegsEpilogue>();
        const int ew = warp - NCW;
        const int r = ew * 32 + lane;  // accumulator row m
        const uint32_t lane_base = tmem + ((uint32_t)(ew * 32) << 16);
        constexpr int CH = C / 8;
        int it = 0;
        tc::SegCursor ocur = {};
        if constexpr (SEG) ocur.init((int)blockIdx.x, (int)gridDim.x, sg, gm.H);
        // TMA store of `stride` staged rows to the rows this tile owns (dQ, dK and dV alike)
        auto store_rows = [&](const CUtensorMap* map, const uint8_t* src, int out_row) {
            if constexpr (SEG) {
                const int set = ocur.r >= sg.ra ? 1 : 0;
                ptx::tma_store_5d(map + set, src, 0, out_row, ocur.r - (set ? sg.ra : 0), ocur.h, ocur.b);
            } else {
                ptx::tma_store_3d(map, src, 0, out_row, 0);
            }
        };
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            // first row this tile stores: on the flattened axis, or inside the tile's residue sequence
            const int out_row = (SEG ? ocur.i : tile) * stride;
            uint8_t* st = smem + (it % NS) * L.stage_bytes;
            if (!ptx::mbar_wait_relaxed(&misc->o_ready, it & 1) || *abort_flag) { atomicExch(&g_tc_bwd_status, 15); *abort_flag = 1; break; }
            ptx::tc_fence_after_sync();
            // owned rows: dQ rows [right, right+stride), dK/dV rows [win-1, 128); both land on global rows
            // [out_row, out_row+stride) and are staged from row 0 of the (now idle) Q / dO / K buffers
            auto stage_rows = [&](uint8_t* buf, const float* acc, int m_first) {
                const int ms = r - m_first;  // staging row
                if (ms >= 0 && ms < stride) {
                    const int swz = (C == 64) ? (ms & 7) : (C == 32) ? ((ms >> 1) & 3) : ((ms >> 2) & 1);
#pragma unroll
                    for (int c = 0; c < CH; ++c)
                        *reinterpret_cast<uint4*>(buf + ms * kRowBytes + ((c ^ swz) * 16)) = Cvt<E>::pack(acc + c * 8);
                }
            };
            if constexpr (OWN_OUT) {
                // drain all three accumulators to 16-bit registers first so the MMA warp can reuse them, then
                // one staging buffer, three rounds: stage -> TMA store -> wait until the store has read it
                uint8_t* buf = smem + L.out;
                uint4 pk[3][CH];
#pragma unroll
                for (int which = 0; which < 3; ++which) {  // 0: dQ, 1: dV, 2: dK = the MMA roles
                    if (MODE == kBandT && which != 1) continue;
                    const uint32_t col = which == 0 ? kColDQ : which == 1 ? kColDV : kColDK;
                    float acc[C];
#pragma unroll
                    for (int c = 0; c < C; c += 8) ptx::tmem_ld8(lane_base + col + c, &acc[c]);
                    ptx::tmem_ld_wait();
                    ptx::tc_fence_before_sync();
                    ptx::mbar_arrive(&misc->o_free[which]);
#pragma unroll
                    for (int c = 0; c < CH; ++c) pk[which][c] = Cvt<E>::pack(acc + c * 8);
                }
                if (L.out_bufs == 3) {
                    // one buffer per output: wait (only now) until the previous tile's stores have read them, stage all three,
                    // issue the three stores together
                    if (tid == kEpiTid) ptx::tma_store_wait_read();
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    constexpr int kOutBuf = round_up(kTileM * C * 2, 1024);
#pragma unroll
                    for (int which = 0; which < 3; ++which) {
                        if (MODE == kBandT && which != 1) continue;
                        const int ms = r - (which == 0 ? right : win - 1);
                        if (ms >= 0 && ms < stride) {
                            const int swz = (C == 64) ? (ms & 7) : (C == 32) ? ((ms >> 1) & 3) : ((ms >> 2) & 1);
#pragma unroll
                            for (int c = 0; c < CH; ++c)
                                *reinterpret_cast<uint4*>(buf + which * kOutBuf + ms * kRowBytes + ((c ^ swz) * 16)) = pk[which][c];
                        }
                    }
                    ptx::fence_proxy_async_smem();
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    if (tid == kEpiTid) {
#pragma unroll
                        for (int which = 0; which < 3; ++which) {
                            if (MODE == kBandT && which != 1) continue;
                            store_rows(which == 0 ? tm.dq : which == 1 ? tm.dv : tm.dk, buf + which * kOutBuf, out_row);
                        }
                        ptx::tma_store_commit();
                    }
                    if constexpr (SEG) ocur.advance();
                    continue;
                }
#pragma unroll
                for (int which = 0; which < 3; ++which) {
                    if (MODE == kBandT && which != 1) continue;
                    if (which > 0 && MODE == kBwdFused) asm volatile("bar.sync 2, 128;" ::: "memory");  // previous store has read the buffer
                    const int ms = r - (which == 0 ? right : win - 1);
                    if (ms >= 0 && ms < stride) {
                        const int swz = (C == 64) ? (ms & 7) : (C == 32) ? ((ms >> 1) & 3) : ((ms >> 2) & 1);
#pragma unroll
                        for (int c = 0; c < CH; ++c) *reinterpret_cast<uint4*>(buf + ms * kRowBytes + ((c ^ swz) * 16)) = pk[which][c];
                    }
                    ptx::fence_proxy_async_smem();
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    if (tid == kEpiTid) {
                        store_rows(which == 0 ? tm.dq : which == 1 ? tm.dv : tm.dk, buf, out_row);
                        ptx::tma_store_commit();
                        ptx::tma_store_wait_read();
                    }
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
            } else {
                // no room for a staging buffer: use the tile's idle Q / dO / K buffers and release the stage afterwards
                float acc[C];
#pragma unroll
                for (int c = 0; c < C; c += 8) ptx::tmem_ld8(lane_base + kColDQ + c, &acc[c]);
                ptx::tmem_ld_wait();
                stage_rows(st + L.stage_q, acc, right);
#pragma unroll
                for (int c = 0; c < C; c += 8) ptx::tmem_ld8(lane_base + kColDK + c, &acc[c]);
                ptx::tmem_ld_wait();
                stage_rows(st + L.stage_do, acc, win - 1);
#pragma unroll
                for (int c = 0; c < C; c += 8) ptx::tmem_ld8(lane_base + kColDV + c, &acc[c]);
                ptx::tmem_ld_wait();
                ptx::tc_fence_before_sync();
                for (int i = 0; i < 3; ++i) ptx::mbar_arrive(&misc->o_free[i]);
                stage_rows(st + L.stage_k, acc, win - 1);
                ptx::fence_proxy_async_smem();
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (tid == kEpiTid) {
                    store_rows(tm.dq, st + L.stage_q, out_row);
                    store_rows(tm.dk, st + L.stage_do, out_row);
                    store_rows(tm.dv, st + L.stage_k, out_row);
                    ptx::tma_store_commit();
                    ptx::tma_store_wait_read();
                    // the staging used the tile's Q, dO and K buffers: only now may the producer refill them
                    ptx::mbar_arrive(&misc->empty[it % NS][kQ]);
                    ptx::mbar_arrive(&misc->empty[it % NS][kDO]);
                    ptx::mbar_arrive(&misc->empty[it % NS][kK]);
                }
            }
            if constexpr (SEG) ocur.advance();
        }
        if (tid == kEpiTid) ptx::tma_store_wait_all();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        ptx::tmem_dealloc(tmem, kTmemCols);
    }
}

// d_rpb[i] += sum over the CTAs' partial rows (column i of a (rows, n) matrix). One warp per entry: the lanes split the
// rows (a single thread walking 148 dependent-latency loads made this tiny kernel cost 20 us), then a shuffle reduction.
__global__ void bias_grad_reduce_kernel(float* __restrict__ d_rpb, const float* __restrict__ partial, int rows, int n) {
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (i >= n) return;
    float acc = 0.f;
    for (int r = lane; r < rows; r += 32) acc += partial[(size_t)r * n + i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) d_rpb[i] += acc;
}

template <typename E, int C, int WB, bool SEG, int MODE = kBwdFused, bool DROP = false>
cudaError_t launch_bwd(const BwdMaps<SEG ? 2 : 1>& maps, float* d_rpb, float* scratch, size_t scratch_floats,
                       const float* lse, const float* rpb, const int* valid_len, const Geometry& gm, const SegGeom& sg, int stride, int KT,
                       int total, int sm_count, bool pdl, const DropoutCfg& drop, cudaStream_t st) {
    const int n_bias = gm.H * gm.win;
    const BwdSmemLayout L = bwd_layout_for(C, KT, gm, rpb != nullptr, d_rpb != nullptr);
    const int smem = L.total;
    // only 64-channel rows can be too large for the dedicated output staging buffer
    if constexpr (C != 64) {
        if (!L.own_out) return cudaErrorInvalidValue;
    }
    if constexpr (MODE != kBwdFused) {
        if (!L.own_out) return cudaErrorInvalidValue;   // the band-transpose mode exists only with the dedicated staging buffer
    }
    auto kern = (MODE == kBwdFused && C == 64 && !L.own_out) ? tc_bwd_kernel<E, C, WB, C != 64 || MODE != kBwdFused, SEG, MODE, DROP>
                                                             : tc_bwd_kernel<E, C, WB, true, SEG, MODE, DROP>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    if constexpr (compute_warps(C, MODE) == 8) {
        // The warp groups of this variant trade registers among themselves (2 x 176 + 104 + 56 per thread): the CTA's pool
        // must hold 4 x 128, i.e. the kernel must have been compiled to 128 registers, or the compute warps would wait
        // for registers that never come. Checked once per variant; a build that breaks it fails here, not on the GPU.
        static const int regs = [] {
            cudaFuncAttributes fa;
            return cudaFuncGetAttributes(&fa, tc_bwd_kernel<E, C, WB, true, SEG, MODE, DROP>) == cudaSuccess ? fa.numRegs : 0;
        }();
        if (regs < 128) return cudaErrorLaunchOutOfResources;
    }
    const int grid = total < sm_count ? total : sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(bwd_threads(compute_warps(C, MODE)));
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // bias gradient: every CTA adds its partial sums to the result with atomics at its end; on request (and if the caller's
    // scratch holds one row per CTA) one partial row per CTA instead, summed in a fixed order by a second tiny kernel
    const bool partial_rows = bias_grad_partial_rows() && d_rpb && scratch && scratch_floats >= (size_t)grid * n_bias;
    float* bias_out = !d_rpb ? nullptr : partial_rows ? scratch : d_rpb;
    e = cudaLaunchKernelEx(&cfg, kern, maps, bias_out, partial_rows ? 0 : 1, lse, rpb, valid_len, gm, sg, stride, KT, total, drop);
    if (e != cudaSuccess || !partial_rows) return e;
    bias_grad_reduce_kernel<<<(n_bias + 7) / 8, 256, 0, st>>>(d_rpb, scratch, grid, n_bias);
    return cudaGetLastError();
}

// Picks the instantiation for (channels, window bucket) of element type E; `wb` is the window the band fragments must hold.
template <typename E, bool SEG, int MODE = kBwdFused, bool DROP = false>
cudaError_t dispatch_bwd(const BwdMaps<SEG ? 2 : 1>& maps, float* d_rpb, float* scratch, size_t scratch_floats, const float* lse,
                         const float* rpb, const int* valid_len, const Geometry& gm, const SegGeom& sg, int stride, int KT, int total,
                         int wb, cudaStream_t st, const DropoutCfg& drop = DropoutCfg{0u, 0u, 1.f}) {
    const int sms = device_sm_count();
    const bool pdl = pdl_mode() == 1 || pdl_mode() == 3;
#define NA1D_TC_BWD(C, WB) \
    return launch_bwd<E, C, WB, SEG, MODE, DROP>(maps, d_rpb, scratch, scratch_floats, lse, rpb, valid_len, gm, sg, stride, KT, total, sms, pdl, drop, st)
#define NA1D_TC_BWD_W(C)                       \
    if (wb <= 9) { NA1D_TC_BWD(C, 9); }        \
    else if (wb <= 17) { NA1D_TC_BWD(C, 17); } \
    else { NA1D_TC_BWD(C, 33); }
    if (gm.C == 64) { NA1D_TC_BWD_W(64) }
    else if (gm.C == 32) { NA1D_TC_BWD_W(32) }
    else { NA1D_TC_BWD_W(16) }
#undef NA1D_TC_BWD
#undef NA1D_TC_BWD_W
}

// shared-memory check common to both tilings: `weff` is the window the tile geometry is built on
bool bwd_smem_fits(const Geometry& gm, int weff, bool has_bias, bool wants_bias_grad) {
    // 64-channel rows with the widest window bucket leave 1.5 KB of shared memory: a bias table of more than 4 heads or the
    // bias-gradient accumulators do not fit there, and the call goes to the CUDA-core kernels
    const int KT = round_up(kTileM + weff - 1, 16);
    return bwd_layout_for(gm.C, KT, gm, has_bias, wants_bias_grad).total <= 227 * 1024;
}

// Reads and clears this translation unit's status word (synchronises the device).
int read_status_word() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_bwd_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_tc_bwd_status, &zero, sizeof(int));
    return v;
}

}  // namespace
}  // namespace na1d

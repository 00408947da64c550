// Pieces shared by the tcgen05 forward and backward kernels.
//
// Band access pattern. S = Q.K^T of a 128-query tile sits in tensor memory with lane = query row and
// column = key row of the staged K window. A warp may touch the 32 lanes 32w..32w+31; it reads them as
// two 16-row blocks with the 16x256b shape, which hands every thread the classic accumulator fragment
// (rows l/4 and l/4+8, two adjacent columns per 8-column group). For a 16-row block only
// NG = ceil((15+win)/8) column groups starting at the block's own first row hold band entries, so a
// thread sees 4*NG values per block, the band test is `0 <= column-row < win` on values known at
// compile time plus one per-thread constant, row reductions are two quad shuffles, and the 16-bit
// results are already in the register order that stmatrix (shared-memory operands) and the 16x128b
// TMEM store (tensor-memory operands) expect. Nothing is ever shifted between registers.
#pragma once
#include "na1d_common.cuh"
#include "na1d_ptx.cuh"

namespace na1d {
namespace tc {

constexpr int kTileM = 128;

template <int C> struct RowSwizzle;
template <> struct RowSwizzle<64> { static constexpr uint64_t umma = ptx::kSwizzle128B; };
template <> struct RowSwizzle<32> { static constexpr uint64_t umma = ptx::kSwizzle64B; };
template <> struct RowSwizzle<16> { static constexpr uint64_t umma = ptx::kSwizzle32B; };
template <typename E> struct Fmt;
template <> struct Fmt<__nv_bfloat16> { static constexpr uint32_t v = 1; };
template <> struct Fmt<__half> { static constexpr uint32_t v = 0; };

__host__ __device__ constexpr int round_up(int x, int m) { return (x + m - 1) / m * m; }
// column groups of 8 that can hold band entries of a 16-row block
__host__ __device__ constexpr int band_groups(int win_max) { return (15 + win_max + 7) / 8; }

// Fragment slot (g, hh, e) of a thread holds window offset 8 (g - hh) + e + fa with fa in [-7, 6]. The slots with
// g - hh == -1 (offsets below 0) and g - hh == NG - 1 (offsets of at least 8 NG - 15 >= the bucket's widest window) can
// never be band entries: a third of the slots in the narrowest bucket, a sixth in the widest. Loops over (g, hh) are fully
// unrolled, so this test is resolved at compile time and the arithmetic of those slots disappears.
__host__ __device__ constexpr bool dead_slot(int g, int hh, int ng) { return g - hh == -1 || g - hh == ng - 1; }

// Dilation d (a power of two) is handled as a window of (win-1) d + 1 consecutive keys of which every d-th is a neighbour:
// tiles, halos and masks use the effective window, the band test adds `offset % d == 0`.
__host__ __device__ constexpr int eff_window(int win, int dil) { return (win - 1) * dil + 1; }
__host__ __device__ constexpr bool pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }

// ---- tcgen05.ld 16x256b: x1 = 4 registers per thread: (row l/4: cols 2(l%4), +1), (row l/4+8: same cols)
__device__ __forceinline__ void ld_frag1(uint32_t taddr, float* f) {
    uint32_t r[4];
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x1.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void ld_frag2(uint32_t taddr, float* f) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[i]);
}
// NG column groups starting at the column in taddr; f[4n + 2h + e]: group n, row half h, column parity e
template <int NG> __device__ __forceinline__ void ld_frag(uint32_t taddr, float* f) {
#pragma unroll
    for (int n = 0; n + 1 < NG; n += 2) ld_frag2(taddr + 8 * n, f + 4 * n);
    if constexpr (NG % 2 == 1) ld_frag1(taddr + 8 * (NG - 1), f + 4 * (NG - 1));
}

// ---- tcgen05.st 16x128b: x1 = 2 registers per thread: (row l/4, 32-bit column l%4), (row l/4+8, same column).
// With two 16-bit values per column this is one 8-key group of a 16-bit A operand.
__device__ __forceinline__ void st_pack1(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.16x128b.x1.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(r[0]), "r"(r[1]) : "memory");
}
__device__ __forceinline__ void st_pack2(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1, %2, %3, %4};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}
template <int NG> __device__ __forceinline__ void st_pack(uint32_t taddr, const uint32_t* r) {
#pragma unroll
    for (int n = 0; n + 1 < NG; n += 2) st_pack2(taddr + 4 * n, r + 2 * n);
    if constexpr (NG % 2 == 1) st_pack1(taddr + 4 * (NG - 1), r + 2 * (NG - 1));
}

// ---- stmatrix: 8x8 matrices of 16-bit values, one 16-byte row per address
__device__ __forceinline__ void stmatrix_x4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
                 : "memory");
}
__device__ __forceinline__ void stmatrix_x2(uint32_t addr, uint32_t r0, uint32_t r1) {
    asm volatile("stmatrix.sync.aligned.m8n8.x2.shared.b16 [%0], {%1, %2};" ::"r"(addr), "r"(r0), "r"(r1) : "memory");
}

// Stores the 2*NG core matrices of one 16-row block (pk[2n+h]: column group n, row half h) into a
// row-major [query][key] operand matrix kept in 8x8 core-matrix order:
//   element (q, c) at (q/8)*group_stride + (c/8)*128 + (q%8)*16 + (c%8)*2.
// blk_addr = shared address of the core matrix (row group of the block's first row, column group of its first column).
template <int NG>
__device__ __forceinline__ void store_block_operand(uint32_t blk_addr, uint32_t group_stride, const uint32_t* pk, int lane) {
    const uint32_t lane_off = (uint32_t)((lane >> 3) & 1) * group_stride + (uint32_t)(lane >> 4) * 128u + (uint32_t)(lane & 7) * 16u;
#pragma unroll
    for (int n = 0; n + 1 < NG; n += 2)
        stmatrix_x4(blk_addr + n * 128 + lane_off, pk[2 * n], pk[2 * n + 1], pk[2 * n + 2], pk[2 * n + 3]);
    if constexpr (NG % 2 == 1) {
        // x2: lanes 0-15 supply the addresses (row half = lane/8)
        const uint32_t off2 = (uint32_t)((lane >> 3) & 1) * group_stride + (uint32_t)(lane & 7) * 16u;
        stmatrix_x2(blk_addr + (NG - 1) * 128 + off2, pk[2 * (NG - 1)], pk[2 * (NG - 1) + 1]);
    }
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Descriptor for the next K step: only the 14-bit start-address field (16-byte units) moves.
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (uint64_t)(bytes >> 4); }

// Warp-level store of 32 accumulator rows (this thread holds row `lane` as C floats) to global memory
// with full-line transactions: rows are converted to 16 bits, staged in a warp-private shared buffer
// (32 rows x C*2 bytes, 16-byte chunks XOR-swizzled by row so both phases are bank-conflict free),
// then every store instruction writes whole contiguous rows. row_ok(m) says whether local row m is
// written; dst_row0 points at local row 0 (rows are C elements apart).
template <typename E, int C, typename RowOk>
__device__ __forceinline__ void store_rows_coalesced(uint8_t* stage, const float* acc, E* dst_row0, int lane, RowOk row_ok) {
    constexpr int CH = C / 8;            // 16-byte chunks per row
    constexpr int RPI = 32 / CH;         // rows per store instruction
    __syncwarp();
#pragma unroll
    for (int c = 0; c < CH; ++c)
        *reinterpret_cast<uint4*>(stage + lane * (C * 2) + ((c ^ (lane % CH)) * 16)) = Cvt<E>::pack(acc + 8 * c);
    __syncwarp();
    const int chunk = lane % CH, sub = lane / CH;
#pragma unroll
    for (int k = 0; k < CH; ++k) {
        const int row = k * RPI + sub;
        const uint4 v = *reinterpret_cast<const uint4*>(stage + row * (C * 2) + ((chunk ^ (row % CH)) * 16));
        if (row_ok(row)) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dst_row0) + (size_t)row * (C * 2) + chunk * 16) = v;
    }
}

// floor(x / d) and the remainder for |x| < 2^22, 0 < d < 2^22, with inv_d = 1.f / d: the float quotient is off by at most
// one, which a single correction step repairs. Replaces the ~40-instruction integer division in per-row index math.
__device__ __forceinline__ int small_div(int x, int d, float inv_d, int* rem) {
    int q = __float2int_rd((float)x * inv_d);
    int r = x - q * d;
    if (r < 0) { --q; r += d; }
    else if (r >= d) { ++q; r -= d; }
    *rem = r;
    return q;
}

// Position of a tile's first row on the flattened (sequence, token) axis: token index t, head h, batch index b.
// One real division at the start; afterwards a persistent CTA moves from tile to tile with adds and compares only.
struct RowCursor {
    int t, h, b;
    int T, H, step_t, step_h, step_b;
    __device__ __forceinline__ void init(int row, int T_, int H_, int step_rows) {  // row >= 0
        T = T_; H = H_;
        const int n = row / T;
        t = row - n * T;
        b = n / H;
        h = n - b * H;
        const int sn = step_rows / T;
        step_t = step_rows - sn * T;
        step_b = sn / H;
        step_h = sn - step_b * H;
    }
    // the same for a row that may lie up to T - 1 rows before the tensor (a halo row of the first tile): it counts as a row
    // of sequence -1, which the caller treats as not live
    __device__ __forceinline__ void init_signed(int row, int T_, int H_, int step_rows) {  // row > -T
        init(row < 0 ? row + T_ : row, T_, H_, step_rows);
        if (row < 0) { h = H_ - 1; b = -1; }
    }
    __device__ __forceinline__ void advance() {
        t += step_t;
        const int carry = t >= T ? 1 : 0;
        t -= carry ? T : 0;
        h += step_h + carry;
        b += step_b;
        if (h >= H) { h -= H; ++b; }
        if (h >= H) { h -= H; ++b; }
    }
    // the row `off` rows away from the cursor, -T < off < 2^21
    __device__ __forceinline__ void row_at(int off, float inv_T, float inv_H, int& tq, int& hq, int& bq) const {
        const int dn = small_div(t + off, T, inv_T, &tq);
        const int db = small_div(h + dn, H, inv_H, &hq);
        bq = b + db;
    }
};
// eight rows further on; T >= 8
__device__ __forceinline__ void row_step8(int T, int H, int& tq, int& hq, int& bq) {
    tq += 8;
    if (tq >= T) {
        tq -= T;
        if (++hq >= H) { hq = 0; ++bq; }
    }
}

// Position of a tile in the segmented tiling as a mixed-radix counter (tile in sequence, residue, head, batch): two
// divisions at the start; afterwards a persistent CTA moves from tile to tile with adds and compares only.
struct SegCursor {
    int i, r, h, b;
    int si, sr, sh, sb;   // digits of the step between two tiles of this CTA
    int tps, d, H;
    __device__ __forceinline__ static void split(int x, int tps, int d, int H, int& i, int& r, int& h, int& b) {
        int s = x / tps;
        i = x - s * tps;
        int hv = s / d;
        r = s - hv * d;
        b = hv / H;
        h = hv - b * H;
    }
    __device__ __forceinline__ void init(int tile, int step_tiles, const SegGeom& g, int H_) {
        tps = g.tps; d = g.d; H = H_;
        split(tile, tps, d, H, i, r, h, b);
        split(step_tiles, tps, d, H, si, sr, sh, sb);
    }
    __device__ __forceinline__ void advance() {
        i += si;
        int c = i >= tps ? 1 : 0;
        i -= c ? tps : 0;
        r += sr + c;
        c = r >= d ? 1 : 0;
        r -= c ? d : 0;
        h += sh + c;
        c = h >= H ? 1 : 0;
        h -= c ? H : 0;
        b += sb + c;
    }
    // tokens of the tile's residue sequence
    __device__ __forceinline__ int rows(const SegGeom& g) const { return g.Tp - (r >= g.ra ? 1 : 0); }
};

__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    return x;
}
__device__ __forceinline__ float quad_max(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
    return x;
}

}  // namespace tc

// Tensor map over a dense (N, T, C) 16-bit tensor viewed as dims (C, T, N), box (C, rows, 1).
bool make_row_tile_map(CUtensorMap* map, const void* base, int dtype, int N, int T, int C, int box_rows);
// The pair of 5-D tensor maps (channel, token-in-residue, residue, head, batch) of the segmented tiling over a tensor with
// the given strides: maps[0] covers the residues r < ra (Tp tokens each), maps[1] the residues r >= ra (Tp - 1 tokens,
// residue coordinate r - ra); with ra == d the second is a copy of the first. Box (C, box_rows, 1, 1, 1).
bool make_seg_tile_maps(CUtensorMap* maps, const void* base, int dtype, int batch, int H, int T, int C, const Strides& st,
                        const SegGeom& sg, int box_rows);
int device_sm_count();
void bind_primary_context();
bool pdl_enabled();
int pdl_mode();
bool bias_grad_partial_rows();

}  // namespace na1d

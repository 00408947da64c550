// Host-side helpers shared by the tcgen05 kernels: TMA tensor maps and device properties.
#include "na1d_internal.h"
#include "na1d_tc_common.cuh"
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <unordered_map>

namespace na1d {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is fetched through the runtime so the library does not link against libcuda.
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

// ---- cache of encoded tensor maps ---------------------------------------------------------------------------------
// A CUtensorMap is a pure function of the arguments of cuTensorMapEncodeTiled, so the encoded 128 bytes are memoised under
// those arguments (pointer, data type, rank, extents, strides, box, swizzle, device): a loop that calls a layer with the
// same buffers every step pays the driver call once. One direct-mapped table per host thread (no lock on the hot path: the
// library stays re-entrant, and an autograd worker thread gets a table of its own); a colliding entry is overwritten.
namespace {

struct MapKey {
    uint64_t v[16];
};
struct MapSlot {
    MapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int kMapSlots = 512;
thread_local MapSlot* t_map_table = nullptr;   // allocated on a thread's first use, freed with the thread
thread_local struct MapTableOwner { ~MapTableOwner() { delete[] t_map_table; t_map_table = nullptr; } } t_map_owner;
thread_local int t_device = 0;                 // set by bind_primary_context() at the start of every entry point
std::atomic<long long> g_map_hits{0}, g_map_misses{0};

bool encode_cached(CUtensorMap* out, const void* base, int dtype, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                   const cuuint32_t* box, CUtensorMapSwizzle sw) {
    // NA1D_TENSOR_MAP_CACHE=0 (read once) turns the memoisation off, for measuring what it saves
    static const bool enabled = []() { const char* e = getenv("NA1D_TENSOR_MAP_CACHE"); return !(e && e[0] == '0'); }();
    MapKey key = {};
    MapSlot* slot = nullptr;
    if (enabled) {
        key.v[0] = reinterpret_cast<uint64_t>(base);
        key.v[1] = (uint64_t)dtype | ((uint64_t)rank << 8) | ((uint64_t)sw << 16) | ((uint64_t)t_device << 32);
        for (int i = 0; i < rank; ++i) key.v[2 + i] = dims[i];
        for (int i = 0; i + 1 < rank; ++i) key.v[7 + i] = strides[i];
        for (int i = 0; i < rank; ++i) key.v[11 + i] = box[i];
        uint64_t h = 1469598103934665603ull;
        for (uint64_t x : key.v) { h ^= x; h *= 1099511628211ull; }
        if (!t_map_table) { t_map_table = new MapSlot[kMapSlots](); (void)t_map_owner; }
        slot = &t_map_table[(h ^ (h >> 29)) % kMapSlots];
        if (slot->used && memcmp(slot->key.v, key.v, sizeof(key.v)) == 0) {
            *out = slot->map;
            g_map_hits.fetch_add(1, std::memory_order_relaxed);
            return true;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUtensorMapDataType dt = dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    g_map_misses.fetch_add(1, std::memory_order_relaxed);
    if (slot) { slot->key = key; slot->map = *out; slot->used = true; }
    return true;
}

CUtensorMapSwizzle row_swizzle(int C) {
    return C == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : C == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
}

}  // namespace

void tensor_map_cache_stats(long long* hits, long long* misses) {
    *hits = g_map_hits.load();
    *misses = g_map_misses.load();
}

// Tensor map over a dense (N, T, C) 16-bit tensor viewed as dims (C, T, N), box (C, box_rows, 1).
// The swizzle mode follows the row size (128/64/32 bytes) so that a staged tile is directly a
// canonical tcgen05 operand. Out-of-range rows read as zeros and are skipped on stores.
bool make_row_tile_map(CUtensorMap* map, const void* base, int dtype, int N, int T, int C, int box_rows) {
    const cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)T, (cuuint64_t)N};
    const cuuint64_t strides[2] = {(cuuint64_t)C * 2, (cuuint64_t)T * C * 2};
    const cuuint32_t box[3] = {(cuuint32_t)C, (cuuint32_t)box_rows, 1};
    return encode_cached(map, base, dtype, 3, dims, strides, box, row_swizzle(C));
}

bool make_seg_tile_maps(CUtensorMap* maps, const void* base, int dtype, int batch, int H, int T, int C, const Strides& st,
                        const SegGeom& sg, int box_rows) {
    // every global stride must be a multiple of 16 bytes (element strides a multiple of 8) and the base 16-byte aligned
    if ((st.token % 8) || (st.head % 8) || (st.batch % 8) || (reinterpret_cast<uintptr_t>(base) & 15u)) return false;
    const cuuint64_t strides[4] = {(cuuint64_t)st.token * sg.d * 2, (cuuint64_t)st.token * 2, (cuuint64_t)st.head * 2,
                                   (cuuint64_t)st.batch * 2};
    const cuuint32_t box[5] = {(cuuint32_t)C, (cuuint32_t)box_rows, 1, 1, 1};
    const cuuint64_t dims_a[5] = {(cuuint64_t)C, (cuuint64_t)sg.Tp, (cuuint64_t)sg.ra, (cuuint64_t)H, (cuuint64_t)batch};
    if (!encode_cached(&maps[0], base, dtype, 5, dims_a, strides, box, row_swizzle(C))) return false;
    if (sg.ra == sg.d) { maps[1] = maps[0]; return true; }
    if (sg.Tp < 2) return false;
    const cuuint64_t dims_b[5] = {(cuuint64_t)C, (cuuint64_t)(sg.Tp - 1), (cuuint64_t)(sg.d - sg.ra), (cuuint64_t)H, (cuuint64_t)batch};
    const uint8_t* base_b = static_cast<const uint8_t*>(base) + (size_t)sg.ra * st.token * 2;
    return encode_cached(&maps[1], base_b, dtype, 5, dims_b, strides, box, row_swizzle(C));
}

// Programmatic dependent launch is off unless NA1D_PDL (read once) says otherwise (measured: it shortens back-to-back
// launches of one kernel but not the alternating forward/backward sequence of a training step).
int pdl_mode() {  // 0 off, 1 both kernels, 2 forward only, 3 backward only; anything else counts as 0
    static const int m = []() {
        const char* e = getenv("NA1D_PDL");
        return (e && e[0] >= '1' && e[0] <= '3' && e[1] == '\0') ? (int)(e[0] - '0') : 0;
    }();
    return m;
}
bool pdl_enabled() { return pdl_mode() != 0; }

// How a backward launch hands over its CTAs' partial bias gradients. Default: every CTA adds its (heads, win) partial sum to
// d_rpb with atomics, once, at its end (148 adds per entry; 4 us cheaper than a second kernel, which is 15 % of a backward at
// the training shape). NA1D_BIAS_GRAD_ROWS=1 (read once): one row per CTA in the caller's scratch and a second small kernel
// that sums the rows in a fixed order -- the same bits from run to run for 64-channel rows.
bool bias_grad_partial_rows() {
    static const bool m = []() {
        const char* e = getenv("NA1D_BIAS_GRAD_ROWS");
        return e && e[0] == '1' && e[1] == '\0';
    }();
    return m;
}

// The tensor-map encoder is a DRIVER call and needs the device's primary context current on the calling thread. A thread that
// has made no runtime call yet (an autograd worker whose first CUDA work is this library) has none: bind it explicitly.
void bind_primary_context() {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) { cudaSetDevice(dev); t_device = dev; }
}

int device_sm_count() {
    static std::atomic<int> cached[64];  // zero-initialised; racing first calls store the same value
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

}  // namespace na1d

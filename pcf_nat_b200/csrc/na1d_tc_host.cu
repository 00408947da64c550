// Host-side helpers shared by the tcgen05 kernels: TMA tensor maps and device properties.
#include "na1d_internal.h"
#include "na1d_tc_common.cuh"
#include <atomic>
#include <cstdlib>

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

// Tensor map over a dense (N, T, C) 16-bit tensor viewed as dims (C, T, N), box (C, box_rows, 1).
// The swizzle mode follows the row size (128/64/32 bytes) so that a staged tile is directly a
// canonical tcgen05 operand. Out-of-range rows read as zeros and are skipped on stores.
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

// The tensor-map encoder is a DRIVER call and needs the device's primary context current on the calling thread. A thread that
// has made no runtime call yet (an autograd worker whose first CUDA work is this library) has none: bind it explicitly.
void bind_primary_context() {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
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

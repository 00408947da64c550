// tcgen05 forward, flat tiling over the dense (N*T, C) matrix: instantiations and host entry points.
#include "na1d_tc_fwd_kernel.cuh"

namespace na1d {

bool tc_fwd_supports(const Geometry& gm) {
    return tc::pow2(gm.dil) && (gm.C == 64 || gm.C == 32 || gm.C == 16) && tc::eff_window(gm.win, gm.dil) <= 33 && gm.H <= 32 &&
           gm.T >= 32 && gm.T < (1 << 21);
}

cudaError_t tc_fused_fwd(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                         const int* valid_len, const Geometry& gm, int dtype, cudaStream_t st) {
    if (!tc_fwd_supports(gm)) return cudaErrorInvalidValue;
    bind_primary_context();
    const int weff = tc::eff_window(gm.win, gm.dil);
    const int KT = tc::round_up(tc::kTileM + weff - 1, 16);
    const int rows = gm.N * gm.T;  // the tensors are tiled as one (N*T, C) matrix
    FwdMaps<1> maps;
    if (!make_row_tile_map(&maps.q[0], q, dtype, 1, rows, gm.C, tc::kTileM) || !make_row_tile_map(&maps.k[0], k, dtype, 1, rows, gm.C, KT) ||
        !make_row_tile_map(&maps.v[0], v, dtype, 1, rows, gm.C, KT) || !make_row_tile_map(&maps.o[0], o, dtype, 1, rows, gm.C, tc::kTileM))
        return cudaErrorInvalidValue;
    const int total = (rows + tc::kTileM - 1) / tc::kTileM;
    return dispatch_fwd<false>(maps, lse, nullptr, rpb, valid_len, gm, SegGeom{1, 1, gm.T, 0, tc::kTileM}, KT, total, weff, dtype, st);
}

int tc_read_status() { return read_status_word(); }

}  // namespace na1d

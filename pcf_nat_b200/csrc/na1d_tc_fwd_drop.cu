// tcgen05 forward with attention dropout (flat tiling): instantiations and host entry point.
#include "na1d_tc_fwd_kernel.cuh"

namespace na1d {

cudaError_t tc_fused_fwd_dropout(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                                 const int* valid_len, const Geometry& gm, int dtype, const DropoutCfg& drop, cudaStream_t st) {
    if (!tc_fwd_supports(gm)) return cudaErrorInvalidValue;
    bind_primary_context();
    const int weff = tc::eff_window(gm.win, gm.dil);
    const int KT = tc::round_up(tc::kTileM + weff - 1, 16);
    const int rows = gm.N * gm.T;
    FwdMaps<1> maps;
    if (!make_row_tile_map(&maps.q[0], q, dtype, 1, rows, gm.C, tc::kTileM) || !make_row_tile_map(&maps.k[0], k, dtype, 1, rows, gm.C, KT) ||
        !make_row_tile_map(&maps.v[0], v, dtype, 1, rows, gm.C, KT) || !make_row_tile_map(&maps.o[0], o, dtype, 1, rows, gm.C, tc::kTileM))
        return cudaErrorInvalidValue;
    const int total = (rows + tc::kTileM - 1) / tc::kTileM;
    return dispatch_fwd<false, kFused, true>(maps, lse, nullptr, rpb, valid_len, gm, SegGeom{1, 1, gm.T, 0, tc::kTileM}, KT, total, weff,
                                             dtype, st, drop);
}
int tc_drop_read_status() { return read_status_word(); }

}  // namespace na1d

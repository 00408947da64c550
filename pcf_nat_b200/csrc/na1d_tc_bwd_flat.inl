// Flat-tiling launch of the tcgen05 backward for one element type (included by the per-type translation units).
namespace na1d {
namespace {

template <typename E, bool DROP = false>
cudaError_t run_flat(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k, const void* v,
                     const float* lse, const float* rpb, const int* valid_len, float* scratch, size_t scratch_floats,
                     const Geometry& gm, int dtype, cudaStream_t st, const DropoutCfg& drop = DropoutCfg{0u, 0u, 1.f}) {
    bind_primary_context();
    const int weff = tc::eff_window(gm.win, gm.dil);
    const int KT = round_up(kTileM + weff - 1, 16);
    const int stride = kTileM - (weff - 1);
    const int rows = gm.N * gm.T;  // the tensors are tiled as one (N*T, C) matrix
    BwdMaps<1> m;
    if (!make_row_tile_map(&m.dq[0], dq, dtype, 1, rows, gm.C, stride) || !make_row_tile_map(&m.dk[0], dk, dtype, 1, rows, gm.C, stride) ||
        !make_row_tile_map(&m.dv[0], dv, dtype, 1, rows, gm.C, stride))
        return cudaErrorInvalidValue;
    if (!make_row_tile_map(&m.q[0], q, dtype, 1, rows, gm.C, kTileM) || !make_row_tile_map(&m.d_o[0], d_o, dtype, 1, rows, gm.C, kTileM) ||
        !make_row_tile_map(&m.k[0], k, dtype, 1, rows, gm.C, KT) || !make_row_tile_map(&m.v[0], v, dtype, 1, rows, gm.C, KT))
        return cudaErrorInvalidValue;
    const int total = (rows + stride - 1) / stride;
    return dispatch_bwd<E, false, kBwdFused, DROP>(m, d_rpb, scratch, scratch_floats, lse, rpb, valid_len, gm,
                                                   SegGeom{1, 1, gm.T, 0, stride}, stride, KT, total, weff, st, drop);
}

}  // namespace
}  // namespace na1d

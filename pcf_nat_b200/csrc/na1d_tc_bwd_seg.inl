// Segmented-tiling launch of the tcgen05 backward for one element type (included by the per-type translation units).
namespace na1d {
namespace {

template <typename E>
cudaError_t run_seg(void* dq, void* dk, void* dv, float* d_rpb, const void* d_o, const void* q, const void* k, const void* v,
                    const float* lse, const float* rpb, const int* valid_len, float* scratch, size_t scratch_floats,
                    const Strides& sdq, const Strides& sdk, const Strides& sdv, const Strides& sdo, const Strides& sq, const Strides& sk,
                    const Strides& sv, const Geometry& gm, int dtype, cudaStream_t st) {
    bind_primary_context();
    const int KT = round_up(kTileM + gm.win - 1, 16);
    const int stride = kTileM - (gm.win - 1);
    const SegGeom sg = seg_geometry(gm, stride);
    const int batch = gm.N / gm.H;
    BwdMaps<2> m;
    if (!make_seg_tile_maps(m.dq, dq, dtype, batch, gm.H, gm.T, gm.C, sdq, sg, stride) ||
        !make_seg_tile_maps(m.dk, dk, dtype, batch, gm.H, gm.T, gm.C, sdk, sg, stride) ||
        !make_seg_tile_maps(m.dv, dv, dtype, batch, gm.H, gm.T, gm.C, sdv, sg, stride) ||
        !make_seg_tile_maps(m.q, q, dtype, batch, gm.H, gm.T, gm.C, sq, sg, kTileM) ||
        !make_seg_tile_maps(m.d_o, d_o, dtype, batch, gm.H, gm.T, gm.C, sdo, sg, kTileM) ||
        !make_seg_tile_maps(m.k, k, dtype, batch, gm.H, gm.T, gm.C, sk, sg, KT) ||
        !make_seg_tile_maps(m.v, v, dtype, batch, gm.H, gm.T, gm.C, sv, sg, KT))
        return cudaErrorInvalidValue;
    const int total = gm.N * sg.d * sg.tps;
    return dispatch_bwd<E, true>(m, d_rpb, scratch, scratch_floats, lse, rpb, valid_len, gm, sg, stride, KT, total, gm.win, st);
}

}  // namespace
}  // namespace na1d

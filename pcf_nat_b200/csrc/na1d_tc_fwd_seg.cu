// tcgen05 forward, segmented tiling (any dilation, strided q/k/v/o): instantiations and host entry points.
#include "na1d_tc_fwd_kernel.cuh"

namespace na1d {

SegGeom seg_geometry(const Geometry& gm, int step) {
    SegGeom sg;
    sg.d = gm.dil;
    sg.Tp = (gm.T + gm.dil - 1) / gm.dil;
    sg.ra = gm.T % gm.dil == 0 ? gm.dil : gm.T % gm.dil;
    sg.step = step;
    sg.tps = (sg.Tp + step - 1) / step;
    return sg;
}

bool tc_seg_supports(const Geometry& gm) {
    // every residue sequence needs at least two tokens (the second tensor map has Tp - 1 rows), the window must fit the
    // widest bucket, and the tile count must fit an int
    const long long tiles = (long long)gm.N * gm.dil * (((gm.T + gm.dil - 1) / gm.dil + 63) / 64);
    return (gm.C == 64 || gm.C == 32 || gm.C == 16) && gm.win <= 33 && gm.H <= 32 && gm.T >= 2 * gm.dil && gm.T < (1 << 21) &&
           gm.dil <= 1024 && tiles < (1ll << 30);
}

cudaError_t tc_fused_fwd_seg(void* o, float* lse, const void* q, const void* k, const void* v, const float* rpb,
                             const int* valid_len, const Strides& sq, const Strides& sk, const Strides& sv, const Strides& so,
                             const Geometry& gm, int dtype, cudaStream_t st) {
    if (!tc_seg_supports(gm)) return cudaErrorInvalidValue;
    bind_primary_context();
    const int KT = tc::round_up(tc::kTileM + gm.win - 1, 16);
    const SegGeom sg = seg_geometry(gm, tc::kTileM);
    const int batch = gm.N / gm.H;
    FwdMaps<2> maps;
    if (!make_seg_tile_maps(maps.q, q, dtype, batch, gm.H, gm.T, gm.C, sq, sg, tc::kTileM) ||
        !make_seg_tile_maps(maps.k, k, dtype, batch, gm.H, gm.T, gm.C, sk, sg, KT) ||
        !make_seg_tile_maps(maps.v, v, dtype, batch, gm.H, gm.T, gm.C, sv, sg, KT) ||
        !make_seg_tile_maps(maps.o, o, dtype, batch, gm.H, gm.T, gm.C, so, sg, tc::kTileM))
        return cudaErrorInvalidValue;
    const int total = gm.N * sg.d * sg.tps;
    return dispatch_fwd<true>(maps, lse, nullptr, rpb, valid_len, gm, sg, KT, total, gm.win, dtype, st);
}

int tc_seg_read_status() { return read_status_word(); }

}  // namespace na1d

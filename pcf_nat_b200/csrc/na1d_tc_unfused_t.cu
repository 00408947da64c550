// The transposed half of the unfused pair on the tcgen05 kernels (flat tiling): out[j] = sum of band[t, kk] x[t] over the
// (t, kk) whose neighbour is j -- the backward kernel's overlapped tiles and operand matrix with everything but the
// P^T.dO chain taken out. Serves na1d_k_backward and na1d_v_backward (the reference's torch_ana_k_backward and
// torch_ana_v_backward; na1d_tensorcore/bf16_ana1d.cpp:43-55, 92-104).
#include "na1d_tc_bwd_kernel.cuh"

namespace na1d {

bool tc_unfused_t_supports(const Geometry& gm_in) {
    Geometry gm = gm_in;
    gm.H = 1;
    if (!(tc::pow2(gm.dil) && (gm.C == 64 || gm.C == 32 || gm.C == 16) && tc::eff_window(gm.win, gm.dil) <= 33 && gm.T >= 32 &&
          gm.T < (1 << 21)))
        return false;
    const int KT = round_up(kTileM + tc::eff_window(gm.win, gm.dil) - 1, 16);
    const BwdSmemLayout L = bwd_layout_for(gm.C, KT, gm, false, false);
    return L.own_out && L.total <= 227 * 1024;
}

namespace {
template <typename E>
cudaError_t run_band_t(void* out, const float* band, const void* x, const Geometry& gm_in, int dtype, cudaStream_t st) {
    Geometry gm = gm_in;
    gm.H = 1;
    gm.scale = 1.f;
    bind_primary_context();
    const int weff = tc::eff_window(gm.win, gm.dil);
    const int KT = round_up(kTileM + weff - 1, 16);
    const int stride = kTileM - (weff - 1);
    const int rows = gm.N * gm.T;
    BwdMaps<1> m;
    if (!make_row_tile_map(&m.dv[0], out, dtype, 1, rows, gm.C, stride) || !make_row_tile_map(&m.d_o[0], x, dtype, 1, rows, gm.C, kTileM))
        return cudaErrorInvalidValue;
    m.q[0] = m.k[0] = m.v[0] = m.d_o[0];   // never dereferenced in this mode
    m.dq[0] = m.dk[0] = m.dv[0];
    const int total = (rows + stride - 1) / stride;
    // the band pointer travels in the slot of the log-sum-exp
    return dispatch_bwd<E, false, kBandT>(m, nullptr, nullptr, 0, band, nullptr, nullptr, gm, SegGeom{1, 1, gm.T, 0, stride}, stride, KT,
                                          total, weff, st);
}
}  // namespace

cudaError_t tc_bandT_x(void* out, const float* band, const void* x, const Geometry& gm, int dtype, cudaStream_t st) {
    if (!tc_unfused_t_supports(gm)) return cudaErrorInvalidValue;
    return dtype == 0 ? run_band_t<__nv_bfloat16>(out, band, x, gm, 0, st) : run_band_t<__half>(out, band, x, gm, 1, st);
}
int tc_unfused_t_read_status() { return read_status_word(); }

}  // namespace na1d

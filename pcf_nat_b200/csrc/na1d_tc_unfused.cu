// The unfused pair on the tcgen05 kernels (flat tiling): banded Q.K^T with the fp32 band as output, and band . X with the
// fp32 band as input -- the forward kernel's tiles, rings and tensor-memory layout with the softmax taken out.
// Serves na1d_qk_forward / na1d_a_backward and na1d_av_forward / na1d_q_backward (the reference's torch_ana_qk_forward,
// _a_backward, _av_forward, _q_backward; na1d_tensorcore/bf16_ana1d.cpp:8-41, 57-90).
#include "na1d_tc_fwd_kernel.cuh"

namespace na1d {

bool tc_unfused_supports(const Geometry& gm) {
    return tc::pow2(gm.dil) && (gm.C == 64 || gm.C == 32 || gm.C == 16) && tc::eff_window(gm.win, gm.dil) <= 33 && gm.T >= 32 &&
           gm.T < (1 << 21);
}

namespace {
template <int MODE>
cudaError_t run_unfused(void* out, float* band, const void* a, const void* b, const Geometry& gm_in, int dtype, cudaStream_t st) {
    Geometry gm = gm_in;
    gm.H = 1;            // the unfused entry points know no heads: every sequence is its own "head"
    gm.scale = 1.f;
    if (!tc_unfused_supports(gm)) return cudaErrorInvalidValue;
    bind_primary_context();
    const int weff = tc::eff_window(gm.win, gm.dil);
    const int KT = tc::round_up(tc::kTileM + weff - 1, 16);
    const int rows = gm.N * gm.T;
    FwdMaps<1> maps;
    // band output: a = the row operand (q), b = the window operand (k). band input: b = the window operand (v), out = o.
    const void* row_op = MODE == kBandOut ? a : out;
    if (!make_row_tile_map(&maps.q[0], row_op, dtype, 1, rows, gm.C, tc::kTileM) || !make_row_tile_map(&maps.k[0], b, dtype, 1, rows, gm.C, KT))
        return cudaErrorInvalidValue;
    maps.v[0] = maps.k[0];
    maps.o[0] = maps.q[0];
    const int total = (rows + tc::kTileM - 1) / tc::kTileM;
    return dispatch_fwd<false, MODE>(maps, nullptr, band, nullptr, nullptr, gm, SegGeom{1, 1, gm.T, 0, tc::kTileM}, KT, total, weff, dtype, st);
}
}  // namespace

cudaError_t tc_qk(float* attn, const void* a, const void* b, const Geometry& gm, int dtype, cudaStream_t st) {
    return run_unfused<kBandOut>(nullptr, attn, a, b, gm, dtype, st);
}
cudaError_t tc_band_x(void* out, const float* band, const void* x, const Geometry& gm, int dtype, cudaStream_t st) {
    return run_unfused<kBandIn>(out, const_cast<float*>(band), nullptr, x, gm, dtype, st);
}
int tc_unfused_read_status() { return read_status_word(); }

}  // namespace na1d

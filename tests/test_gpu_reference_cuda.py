"""Hold the new kernels against the REFERENCE's own CUDA kernels on identical device buffers.

oracle/_ref/libref_ana1d_<dtype>.so is the reference's na1d_tensorcore/*_ana1d_kernel.cu compiled
as-is (see oracle/build_ref.py); it is prebuilt where the reference checkout exists and travels
with the tree. The reference kernels support dilation 1 only.

Shapes are restricted to those the reference launches as ONE tile per sequence (T <= 256 and within
its shared-memory heuristic): with more than one tile its dK/dV kernel stages
ceil((part+win-1)*win / threads) * threads band elements into a shared buffer sized for
(tile+win-1)*win (na1d_tensorcore/bf16_ana1d_kernel.cu:409-415 with the size from :571), guarded only
against the end of the global tensor, and that out-of-bounds shared-memory write raised a CUDA error
on a B200 at (N,T,C,win)=(4,300,64,15). Multi-tile shapes are therefore checked against the CPU oracle
only."""
import ctypes
import os

import pytest
import torch

from gpu_util import assert_close, randn16

pytestmark = pytest.mark.gpu
REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _ref(dtype):
    tag = "bf16" if dtype == torch.bfloat16 else "fp16"
    path = os.path.join(REF_DIR, "libref_ana1d_%s.so" % tag)
    if not os.path.exists(path):
        pytest.skip("reference CUDA library not built (%s)" % path)
    lib = ctypes.CDLL(path)
    for n in ("ref_ana_qk_forward", "ref_ana_band_x", "ref_ana_bandT_x"):
        getattr(lib, n).argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 5
        getattr(lib, n).restype = ctypes.c_int
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def reference_single_tile(T, win):
    """True when all three reference launchers (bf16_ana1d_kernel.cu:495-580) use one tile for T."""
    need = -(-T // 16)
    caps = [(12240 - win * 8) // (8 + win) // 16, (24584 - win * 8) // (8 + win) // 16,
            (24576 // (8 + win) - win + 1) // 16]
    return need <= 16 and all(need <= c for c in caps)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("N,T,C,win,left", [(8, 200, 32, 7, 3), (16, 150, 16, 27, 13), (4, 256, 64, 15, 7),
                                            (3, 77, 8, 6, 1), (2, 240, 64, 31, 15)])
def test_unfused_kernels_match_reference_cuda(N, T, C, win, left, dtype):
    from pcf_nat_b200 import ops
    ref = _ref(dtype)
    assert reference_single_tile(T, win), "multi-tile shapes must not be sent to the reference kernels"
    q, k, v, d_o = (randn16((N, T, C), dtype, 200 + i, scale=C ** -0.25).cuda() for i in range(4))
    torch.cuda.synchronize()
    # QK forward
    attn_ref = torch.empty(N, T, win, dtype=torch.float32, device="cuda")
    assert ref.ref_ana_qk_forward(_p(attn_ref), _p(q), _p(k), N, T, C, win, left) == 0
    torch.cuda.synchronize()
    attn = ops.qk_forward(q, k, win, left, 1)
    assert float((attn - attn_ref).abs().max()) < 1e-3 * max(1.0, float(attn_ref.abs().max()))
    # AV forward / dQ  (the reference rounds the band to 16 bits before its MMA)
    prob = torch.softmax(attn_ref, -1).contiguous()
    out_ref = torch.empty_like(v)
    assert ref.ref_ana_band_x(_p(out_ref), _p(prob), _p(v), N, T, C, win, left) == 0
    torch.cuda.synchronize()
    assert_close(ops.av_forward(prob, v, win, left, 1), out_ref.float(), dtype, "av vs reference CUDA")
    # dK / dV
    gd = torch.randn(N, T, win, device="cuda", generator=torch.Generator("cuda").manual_seed(5)) * 0.3
    kgd_ref = torch.empty_like(q)
    assert ref.ref_ana_bandT_x(_p(kgd_ref), _p(gd), _p(q), N, T, C, win, left) == 0
    torch.cuda.synchronize()
    assert_close(ops.k_backward(gd, q, win, left, 1), kgd_ref.float(), dtype, "k_gd vs reference CUDA")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_fused_forward_matches_reference_cuda_chain(dtype):
    """fused op == reference QK kernel -> softmax -> reference AV kernel (the chain the model runs)."""
    from pcf_nat_b200 import ops
    ref = _ref(dtype)
    N, T, C, win, left = 32, 200, 64, 7, 3
    assert reference_single_tile(T, win)
    q, k, v = (randn16((N, T, C), dtype, 300 + i, scale=C ** -0.25).cuda() for i in range(3))
    attn = torch.empty(N, T, win, dtype=torch.float32, device="cuda")
    assert ref.ref_ana_qk_forward(_p(attn), _p(q), _p(k), N, T, C, win, left) == 0
    torch.cuda.synchronize()
    j = torch.arange(T, device="cuda").unsqueeze(1) + torch.arange(win, device="cuda").unsqueeze(0) - left
    attn = attn + torch.where((j < 0) | (j >= T), -100.0, 0.0).unsqueeze(0)
    prob = torch.softmax(attn, -1).contiguous()
    out_ref = torch.empty_like(v)
    assert ref.ref_ana_band_x(_p(out_ref), _p(prob), _p(v), N, T, C, win, left) == 0
    torch.cuda.synchronize()
    o, _ = ops.fused_forward(q, k, v, win, left, 1, 1.0, None, None, 1)
    assert_close(o, out_ref.float(), dtype, "fused vs reference CUDA chain")

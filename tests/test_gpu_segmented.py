"""GPU parity of the tcgen05 kernels on the segmented tiling (tiles inside one residue class of one sequence), through
the C ABI: every dilation, wide dilated windows, lengths the dilation does not divide, and strided (layout-fused) tensors."""
import pytest
import torch

from gpu_util import assert_close, assert_close_strict, randn16
from oracle import na1d_oracle as orc

pytestmark = pytest.mark.gpu
DTYPES = [torch.bfloat16, torch.float16]


def _ops():
    from pcf_nat_b200 import ops
    return ops


# (N, H, T, C, win, left, dil): power-of-two and other dilations, T % dil != 0, windows whose dilated span exceeds the
# flat tiling's limit of 33, sequences shorter than a tile, several tiles per residue sequence, dilation 1
SEG_SHAPES = [
    (4, 2, 200, 64, 15, 7, 4), (4, 2, 200, 32, 31, 15, 2), (2, 1, 403, 64, 31, 15, 4), (6, 3, 150, 16, 27, 13, 1),
    (4, 2, 131, 32, 7, 3, 3), (2, 2, 257, 64, 7, 3, 5), (3, 1, 1000, 16, 15, 7, 4), (2, 1, 1001, 32, 31, 15, 4),
    (8, 4, 50, 64, 3, 1, 2), (2, 2, 300, 64, 7, 3, 1), (4, 2, 77, 32, 9, 0, 3), (4, 2, 77, 16, 9, 8, 6),
    (2, 1, 640, 64, 17, 8, 2), (2, 2, 129, 32, 33, 16, 2), (4, 4, 64, 16, 8, 3, 7),
    # residue sequences of two or three tokens, windows wider than a residue sequence
    (4, 2, 10, 32, 3, 1, 5), (4, 2, 11, 32, 9, 4, 5), (2, 1, 23, 16, 7, 3, 11), (64, 32, 40, 16, 5, 2, 3),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
def test_segmented_tiling_forward_backward(dtype):
    ops = _ops()
    old = ops.set_kernel_family(ops.FAMILY_TCGEN05_SEGMENTED)
    try:
        for idx, (N, H, T, C, win, left, dil) in enumerate(SEG_SHAPES):
            tag = "N=%d H=%d T=%d C=%d win=%d left=%d dil=%d " % (N, H, T, C, win, left, dil)
            assert ops.kernel_tiling(N, T, C, win, left, dil, dtype) == 2, tag
            sc = C ** -0.5
            q, k, v, d_o = (randn16((N, T, C), dtype, 7000 + 4 * idx + i) for i in range(4))
            rpb = 0.3 * torch.randn(H, win, generator=torch.Generator().manual_seed(idx))
            vl = [T] + [max(1, T - 5 - 3 * i) for i in range(N // H - 1)]
            o, lse = ops.fused_forward(q.cuda(), k.cuda(), v.cuda(), win, left, dil, sc, rpb.cuda(), vl, H)
            ops.device_status()
            o_r, dq_r, dk_r, dv_r, drpb_r = orc.na1d_fused_with_grads(q.float(), k.float(), v.float(), d_o.float(), win, left, dil,
                                                                      sc, rpb, vl, H)
            _, lse_r = orc.na1d_fused(q.float(), k.float(), v.float(), win, left, dil, sc, rpb, vl, H, return_lse=True)
            assert_close_strict(o, o_r, dtype, tag + "o")
            assert float((lse.cpu() - lse_r).abs().max()) < 1e-3 * max(1.0, float(lse_r.abs().max())), tag + "lse"
            bwd_args = (d_o.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, win, left, dil, sc, rpb.cuda(), vl, H)
            try:
                dq, dk, dv, drpb = ops.fused_backward(*bwd_args, need_d_rpb=True)
            except Exception as e:
                # 64-channel rows with the widest window bucket: no shared memory left for the bias tables of several heads
                assert getattr(e, "status", None) == -10 and C == 64 and win > 17 and H > 1, tag + repr(e)
                ops.set_kernel_family(ops.FAMILY_AUTO)
                dq, dk, dv, drpb = ops.fused_backward(*bwd_args, need_d_rpb=True)
                ops.set_kernel_family(ops.FAMILY_TCGEN05_SEGMENTED)
            ops.device_status()
            assert_close(dq, dq_r, dtype, tag + "dq")
            assert_close(dk, dk_r, dtype, tag + "dk")
            assert_close(dv, dv_r, dtype, tag + "dv")
            assert_close(drpb, drpb_r, dtype, tag + "drpb", factor=2.0)
    finally:
        ops.set_kernel_family(old)


def test_every_dilation_of_the_sweep_runs_on_tcgen05():
    """Automatic choice: every (window, dilation) of the sweep is taken by the tcgen05 kernels, forward and backward."""
    ops = _ops()
    for dtype in DTYPES:
        for win in (3, 7, 15, 31):
            for dil in (1, 2, 3, 4):
                for T in (200, 400, 1000, 1001):
                    for C in (32, 64):
                        for bw in (False, True):
                            t = ops.kernel_tiling(256, T, C, win, win - 1 - win // 2, dil, dtype, backward=bw)
                            assert t in (1, 2), (win, dil, T, C, bw, t)


@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
def test_packed_projection_layout_matches_dense_path(dtype):
    """q, k, v read from a packed (batch, T, 3, heads, C) projection output and o / gradients written in the layouts the
    neighbouring projections use: same values as the dense path with explicit head split / merge copies, and the oracle."""
    ops = _ops()
    for idx, (B, H, T, C, win, left, dil) in enumerate([(3, 4, 200, 64, 7, 3, 1), (2, 2, 150, 16, 27, 13, 1), (2, 4, 131, 32, 15, 7, 2),
                                                        (5, 2, 64, 32, 5, 2, 3)]):
        tag = "B=%d H=%d T=%d C=%d win=%d dil=%d " % (B, H, T, C, win, dil)
        sc = C ** -0.5
        g = torch.Generator().manual_seed(900 + idx)
        qkv = torch.randn(B, T, 3 * H * C, generator=g).to(dtype).cuda().requires_grad_(True)
        rpb = (0.3 * torch.randn(1, H, 1, win, generator=g)).cuda().requires_grad_(True)
        d_out = torch.randn(B, T, H * C, generator=g).to(dtype).cuda()
        vl = torch.tensor([T] + [max(1, T - 7 * i) for i in range(1, B)], dtype=torch.int32, device="cuda")
        assert ops.packed_supported(H, T, C, win, left, dil, dtype)
        out = ops.na1d_fused_packed(qkv, H, win, left, dil, sc, rpb, vl)
        out.backward(d_out)
        ops.device_status()
        # oracle on the explicitly split tensors
        p = qkv.detach().float().cpu().view(B, T, 3, H, C).permute(2, 0, 3, 1, 4).reshape(3, B * H, T, C)
        d_o = d_out.float().cpu().view(B, T, H, C).permute(0, 2, 1, 3).reshape(B * H, T, C)
        o_r, dq_r, dk_r, dv_r, drpb_r = orc.na1d_fused_with_grads(p[0], p[1], p[2], d_o, win, left, dil, sc,
                                                                  rpb.detach().cpu().reshape(H, win), vl.cpu().tolist(), H)
        merge = lambda x: x.view(B, H, T, C).permute(0, 2, 1, 3).reshape(B, T, H * C)
        assert_close_strict(out, merge(o_r), dtype, tag + "o")
        d_qkv_r = torch.stack([dq_r, dk_r, dv_r]).view(3, B, H, T, C).permute(1, 3, 0, 2, 4).reshape(B, T, 3 * H * C)
        assert_close(qkv.grad, d_qkv_r, dtype, tag + "d_qkv")
        assert_close(rpb.grad.reshape(H, win), drpb_r, dtype, tag + "drpb", factor=2.0)
        # and bit for bit the dense route on the segmented tiling (same kernels, same tiles, other addresses)
        old = ops.set_kernel_family(ops.FAMILY_TCGEN05_SEGMENTED)
        try:
            pd = qkv.detach().view(B, T, 3, H, C).permute(2, 0, 3, 1, 4).reshape(3, B * H, T, C).contiguous()
            o_d, lse_d = ops.fused_forward(pd[0], pd[1], pd[2], win, left, dil, sc, rpb.detach(), vl, H)
        finally:
            ops.set_kernel_family(old)
        assert torch.equal(out.detach(), o_d.view(B, H, T, C).permute(0, 2, 1, 3).reshape(B, T, H * C)), tag + "strided != dense"


def test_strided_entry_points_reject_bad_strides():
    import ctypes
    from pcf_nat_b200 import _lib
    L = _lib.lib()
    q = torch.zeros(2, 2, 64, 32, dtype=torch.bfloat16, device="cuda")
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    good = (ctypes.c_int64 * 3)(2 * 64 * 32, 64 * 32, 32)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for bad in ((0, 64 * 32, 32), (2 * 64 * 32, 64 * 32, 20), (2 * 64 * 32, 64 * 32 + 4, 32), (-8, 64 * 32, 32)):
        b = (ctypes.c_int64 * 3)(*bad)
        rc = L.na1d_fused_forward_strided(P(q), None, P(q), P(q), P(q), None, None, good, b, good, good, 4, 2, 64, 32, 7, 3, 1, 1.0, 0, st)
        assert rc == -11, (bad, rc)
    rc = L.na1d_fused_forward_strided(P(q), None, P(q), P(q), P(q), None, None, good, good, good, good, 4, 2, 64, 24, 7, 3, 1, 1.0, 0, st)
    assert rc in (-10, -11), rc   # 24 channels: not a tcgen05 shape
    rc = L.na1d_fused_forward_strided(P(q), None, P(q), P(q), P(q), None, None, good, good, good, good, 4, 2, 64, 32, 7, 3, 1, 1.0, 0, st)
    assert rc == 0
    torch.cuda.synchronize()
    _ops().device_status()


def test_tensor_map_cache_hits_on_repeated_buffers():
    ops = _ops()
    q, k, v = (randn16((8, 200, 64), torch.bfloat16, 31 + i).cuda() for i in range(3))
    ops.fused_forward(q, k, v, 7, 3)
    torch.cuda.synchronize()
    keep = []
    h0, m0 = ops.tensor_map_cache_stats()
    for _ in range(5):
        keep.append(ops.fused_forward(q, k, v, 7, 3))   # q, k, v maps hit; each new output buffer is one miss at most
    h1, m1 = ops.tensor_map_cache_stats()
    assert h1 - h0 >= 15 and m1 - m0 <= 5, (h0, m0, h1, m1)

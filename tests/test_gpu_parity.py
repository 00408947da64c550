"""GPU parity tests: every call goes through the C ABI (ctypes) of libna1d_b200.so and is
checked against the CPU oracle on the same seeded inputs, and against the committed vectors
that the reference's own CPU implementation produced."""
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs, win_left
from gpu_util import TOL, assert_close, assert_close_strict, randn16, rounded_inputs
from oracle import na1d_oracle as orc

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DTYPES = [torch.bfloat16, torch.float16]


def _ops():
    from pcf_nat_b200 import ops
    return ops


@pytest.fixture(params=["auto", "cuda_core"])
def family(request):
    """Runs a test once with the automatic kernel choice (tcgen05 kernels where they apply) and once
    with the CUDA-core kernels forced, so both families are held to the same oracle."""
    ops = _ops()
    old = ops.set_kernel_family(ops.FAMILY_CUDA_CORE if request.param == "cuda_core" else ops.FAMILY_AUTO)
    yield request.param
    ops.set_kernel_family(old)
    ops.device_status()


# ------------------------------------------------------------------ index math, bit exact
@pytest.mark.parametrize("T,win,left,dil", [(1, 3, 1, 1), (5, 9, 4, 1), (200, 7, 3, 1), (200, 8, 3, 1),
                                            (37, 7, 3, 2), (50, 15, 7, 4), (31, 6, 1, 1), (20, 5, 0, 1),
                                            (20, 5, 4, 3), (3000, 15, 7, 1), (1000, 31, 15, 4), (129, 80, 40, 1)])
def test_window_index_bit_exact(T, win, left, dil):
    j, inr = _ops().window_index(T, win, left, dil)
    jr, inr_r = orc.neighbour_index(T, win, left, dil)
    assert torch.equal(j.cpu().to(torch.int64), jr)
    assert torch.equal(inr.cpu(), inr_r)


# ------------------------------------------------------------------ fused forward / backward
@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
@pytest.mark.parametrize("name", list(CASES))
def test_fused_forward_matches_oracle_and_reference_vectors(name, dtype, family):
    c = CASES[name]
    win, left = win_left(c["win"])
    (q, k, v, _), (qf, kf, vf, _), rpb = rounded_inputs(name, dtype)
    o, lse = _ops().fused_forward(q, k, v, win, left, c["dil"], c["scale"], rpb.cuda(), c["valid_len"], c["H"])
    o_ref, lse_ref = orc.na1d_fused(qf, kf, vf, win, left, c["dil"], c["scale"], rpb, c["valid_len"], c["H"],
                                    return_lse=True)
    assert_close_strict(o, o_ref, dtype, name + " o")
    assert float((lse.cpu() - lse_ref).abs().max()) < 1e-3 * max(1.0, float(lse_ref.abs().max()))
    # vectors from the reference's CPU branch were computed on unrounded fp32 inputs: the gap
    # includes the 16-bit rounding of q/k/v themselves, hence the looser bound
    gold = torch.from_numpy(np.load(os.path.join(GOLD, name + ".npz"))["out"])
    assert_close(o, gold, dtype, name + " o vs reference vector", factor=4.0)


@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
@pytest.mark.parametrize("name", [n for n in CASES if CASES[n]["grads"]])
def test_fused_backward_matches_oracle(name, dtype, family):
    ops = _ops()
    c = CASES[name]
    win, left = win_left(c["win"])
    (q, k, v, d_o), (qf, kf, vf, dof), rpb = rounded_inputs(name, dtype)
    o, lse = ops.fused_forward(q, k, v, win, left, c["dil"], c["scale"], rpb.cuda(), c["valid_len"], c["H"])
    dq, dk, dv, drpb = ops.fused_backward(d_o, q, k, v, o, lse, win, left, c["dil"], c["scale"], rpb.cuda(),
                                          c["valid_len"], c["H"], need_d_rpb=True)
    _, dq_r, dk_r, dv_r, drpb_r = orc.na1d_fused_with_grads(qf, kf, vf, dof, win, left, c["dil"], c["scale"], rpb,
                                                            c["valid_len"], c["H"])
    assert_close(dq, dq_r, dtype, name + " dq")
    assert_close(dk, dk_r, dtype, name + " dk")
    assert_close(dv, dv_r, dtype, name + " dv")
    assert_close(drpb, drpb_r, dtype, name + " drpb", factor=2.0)


def test_fused_autograd_function_end_to_end():
    from pcf_nat_b200 import na1d_fused
    name, dtype = "mfa_w7_pad", torch.bfloat16
    c = CASES[name]
    win, left = win_left(c["win"])
    (q, k, v, d_o), (qf, kf, vf, dof), rpb = rounded_inputs(name, dtype)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    r = rpb.cuda().requires_grad_(True)
    o = na1d_fused(q, k, v, win, left, c["dil"], c["scale"], r, c["valid_len"], c["H"])
    o.backward(d_o)
    _, dq_r, dk_r, dv_r, drpb_r = orc.na1d_fused_with_grads(qf, kf, vf, dof, win, left, c["dil"], c["scale"], rpb,
                                                            c["valid_len"], c["H"])
    assert_close(q.grad, dq_r, dtype, "dq")
    assert_close(k.grad, dk_r, dtype, "dk")
    assert_close(v.grad, dv_r, dtype, "dv")
    assert_close(r.grad, drpb_r, dtype, "drpb", factor=2.0)


# ------------------------------------------------------------------ edge sweep (both ends of the sequence)
EDGE = [(T, win, left, dil, C)
        for T in (1, 6, 7, 15, 16, 17, 127, 128, 129, 200)
        for (win, left, dil, C) in ((7, 3, 1, 16), (8, 3, 1, 32), (6, 1, 1, 8), (7, 3, 2, 64), (15, 7, 4, 16),
                                    (31, 15, 1, 64), (5, 0, 1, 24), (5, 4, 1, 48))]


@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
def test_edge_sweep_forward_backward(dtype, family):
    ops = _ops()
    for idx, (T, win, left, dil, C) in enumerate(EDGE):
        N, H = 4, 2
        sc = C ** -0.5
        q, k, v, d_o = (randn16((N, T, C), dtype, 1000 + 4 * idx + i) for i in range(4))
        rpb = 0.3 * torch.randn(H, win, generator=torch.Generator().manual_seed(idx))
        vl = [T, max(1, T - 3)]
        o, lse = ops.fused_forward(q.cuda(), k.cuda(), v.cuda(), win, left, dil, sc, rpb.cuda(), vl, H)
        dq, dk, dv, drpb = ops.fused_backward(d_o.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, win, left, dil, sc,
                                              rpb.cuda(), vl, H, need_d_rpb=True)
        o_r, dq_r, dk_r, dv_r, drpb_r = orc.na1d_fused_with_grads(q.float(), k.float(), v.float(), d_o.float(), win,
                                                                  left, dil, sc, rpb, vl, H)
        tag = "T=%d win=%d left=%d dil=%d C=%d " % (T, win, left, dil, C)
        assert_close_strict(o, o_r, dtype, tag + "o")
        assert_close(dq, dq_r, dtype, tag + "dq")
        assert_close(dk, dk_r, dtype, tag + "dk")
        assert_close(dv, dv_r, dtype, tag + "dv")
        assert_close(drpb, drpb_r, dtype, tag + "drpb", factor=2.0)


# ------------------------------------------------------------------ unfused pair (reference API)
@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
@pytest.mark.parametrize("T,C,win,left,dil", [(200, 32, 7, 3, 1), (150, 16, 27, 13, 1), (33, 8, 8, 3, 1),
                                              (37, 64, 7, 3, 2), (129, 24, 15, 7, 4), (5, 8, 9, 4, 1),
                                              (300, 64, 15, 7, 1), (1000, 32, 31, 15, 1), (129, 16, 9, 4, 2), (64, 64, 8, 0, 4),
                                              (257, 32, 33, 32, 1)])
def test_unfused_pair_forward_and_gradients(T, C, win, left, dil, dtype):
    from pcf_nat_b200.nattn import getNA1dFunction
    QK, AV = getNA1dFunction(C, dil, dtype)
    N = 6
    q, k, v, d_o = (randn16((N, T, C), dtype, 50 + i, scale=C ** -0.25) for i in range(4))
    qg, kg, vg = (x.cuda().requires_grad_(True) for x in (q, k, v))
    attn = QK.apply(qg, kg, win, left, dil)
    assert attn.dtype == torch.float32 and attn.shape == (N, T, win)
    p = torch.softmax(attn, -1)
    out = AV.apply(p, vg, win, left, dil)
    assert out.dtype == dtype
    out.backward(d_o.cuda())
    qf, kf, vf = (x.float().requires_grad_(True) for x in (q, k, v))
    attn_r = orc.na1d_qk(qf, kf, win, left, dil)
    out_r = orc.na1d_av(torch.softmax(attn_r, -1), vf, win, left, dil)
    out_r.backward(d_o.float())
    assert float((attn.detach().cpu() - attn_r.detach()).abs().max()) < 1e-4 * max(1.0, float(attn_r.detach().abs().max()))
    assert_close_strict(out, out_r, dtype, "av")
    assert_close(qg.grad, qf.grad, dtype, "q_gd")
    assert_close(kg.grad, kf.grad, dtype, "k_gd")
    assert_close(vg.grad, vf.grad, dtype, "v_gd")


# ------------------------------------------------------------------ properties at the full benchmark shape
def test_full_size_training_shape_properties(family):
    """The PCF-NAT training shape: B=128, heads=4, L=200, head_dim=64, win=7, bf16."""
    ops = _ops()
    N, H, T, C, win, left = 512, 4, 200, 64, 7, 3
    dtype = torch.bfloat16
    q, k, v, d_o = (randn16((N, T, C), dtype, 1 + i).cuda() for i in range(4))
    sc = 1.0
    o, lse = ops.fused_forward(q, k, v, win, left, 1, sc, None, None, H)
    o2, lse2 = ops.fused_forward(q, k, v, win, left, 1, sc, None, None, H)
    assert torch.equal(o, o2) and torch.equal(lse, lse2), "forward is not deterministic"
    # full comparison (the oracle finishes this size in seconds)
    o_r, dq_r, dk_r, dv_r, _ = orc.na1d_fused_with_grads(q.float().cpu(), k.float().cpu(), v.float().cpu(),
                                                         d_o.float().cpu(), win, left, 1, sc, None, None, H)
    assert_close_strict(o, o_r, dtype, "training shape o")
    dq, dk, dv, _ = ops.fused_backward(d_o, q, k, v, o, lse, win, left, 1, sc, None, None, H)
    assert_close(dq, dq_r, dtype, "training shape dq")
    assert_close(dk, dk_r, dtype, "training shape dk")
    assert_close(dv, dv_r, dtype, "training shape dv")
    dq2, dk2, dv2, _ = ops.fused_backward(d_o, q, k, v, o, lse, win, left, 1, sc, None, None, H)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2), "backward is not deterministic"
    # probabilities sum to one: with V == 1 every interior row returns exactly 1
    ones = torch.ones_like(v)
    o1, _ = ops.fused_forward(q, k, ones, win, left, 1, sc, None, None, H)
    assert float((o1[:, left:T - (win - 1 - left)].float() - 1).abs().max()) < 1e-2
    # linearity in V
    v2 = randn16((N, T, C), dtype, 99).cuda()
    oa, _ = ops.fused_forward(q, k, v2, win, left, 1, sc, None, None, H)
    ob, _ = ops.fused_forward(q, k, (v.float() + v2.float()).to(dtype), win, left, 1, sc, None, None, H)
    assert float((ob.float() - (o.float() + oa.float())).abs().max()) < 6e-2


def test_batch_invariance_bitwise(family):
    """Row n of a batched call equals the same sequence run alone (the property the reference's
    own ad-hoc script looked at)."""
    ops = _ops()
    dtype = torch.bfloat16
    N, T, C, win, left = 512, 200, 16, 27, 13
    q, k, v = (randn16((N, T, C), dtype, 7 + i).cuda() for i in range(3))
    o, lse = ops.fused_forward(q, k, v, win, left, 1, 0.25, None, None, 1)
    for n in (0, 17, 511):
        o1, lse1 = ops.fused_forward(q[n:n + 1].contiguous(), k[n:n + 1].contiguous(), v[n:n + 1].contiguous(), win,
                                     left, 1, 0.25, None, None, 1)
        assert torch.equal(o[n:n + 1], o1) and torch.equal(lse[n:n + 1], lse1)


def test_outputs_stay_inside_their_buffers(family):
    """Sentinel margins around every output must survive (stands in for a memory checker)."""
    from pcf_nat_b200 import _lib
    import ctypes
    L = _lib.lib()
    dtype = torch.bfloat16
    for (N, T, C, win, left, dil) in ((3, 129, 64, 7, 3, 1), (2, 200, 32, 31, 15, 2), (5, 17, 16, 15, 7, 4)):
        q, k, v, d_o = (randn16((N, T, C), dtype, 3 + i).cuda() for i in range(4))
        M = 4096
        def guarded(numel, dt):
            buf = torch.full((numel + 2 * M,), 7.0, dtype=dt, device="cuda")
            return buf, buf[M:M + numel]
        bo, o = guarded(N * T * C, dtype)
        bl, lse = guarded(N * T, torch.float32)
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        s = L.na1d_fused_forward(p(o), p(lse), p(q), p(k), p(v), None, None, N, 1, T, C, win, left, dil, 0.125, 0, st)
        assert s == 0
        outs = [guarded(N * T * C, dtype) for _ in range(3)]
        bd, delta = guarded(N * T, torch.float32)
        s = L.na1d_fused_backward(p(outs[0][1]), p(outs[1][1]), p(outs[2][1]), None, p(d_o), p(q), p(k), p(v), p(o),
                                  p(lse), None, None, p(delta), N, 1, T, C, win, left, dil, 0.125, 0, st)
        assert s == 0
        torch.cuda.synchronize()
        for buf, view in [(bo, o), (bl, lse), (bd, delta)] + outs:
            n = view.numel()
            assert bool((buf[:M] == 7.0).all()) and bool((buf[M + n:] == 7.0).all()), "write outside the output"
            assert torch.isfinite(view.float()).all()


def test_bad_arguments_raise_without_touching_the_device():
    ops = _ops()
    from pcf_nat_b200._lib import Na1dError
    q = torch.zeros(2, 16, 16, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Na1dError):
        ops.fused_forward(q, q, q, 7, 7)            # left == win
    with pytest.raises(Na1dError):
        ops.fused_forward(q, q, q, 200, 3)          # window too large
    with pytest.raises(Na1dError):
        ops.fused_forward(q, q, q, 7, 3, heads=3)   # N % heads != 0
    with pytest.raises(TypeError):
        ops.fused_forward(q.float(), q.float(), q.float(), 7, 3)
    torch.cuda.synchronize()
    o, _ = ops.fused_forward(q, q, q, 7, 3)
    assert torch.isfinite(o.float()).all()


# ------------------------------------------------------------------ tcgen05 family: shapes it must take, and parity there
# (sequences, heads, tokens): tiles run over the flattened (sequence, token) axis, so short sequences of several heads
# share a tile and long ones straddle tiles
TC_SHAPES = [(N, H, T, C, win, left) for (N, H, T) in ((3, 1, 200), (2, 1, 128), (1, 1, 129), (2, 2, 32), (1, 1, 1000),
                                                        (2, 1, 383), (12, 4, 50), (6, 3, 150), (8, 2, 33))
             for (C, win, left) in ((64, 7, 3), (32, 7, 3), (16, 27, 13), (64, 15, 7), (64, 31, 15), (32, 33, 0),
                                    (16, 3, 2), (64, 8, 3), (32, 17, 16), (64, 9, 4), (16, 18, 9))]
# dilated windows (power-of-two dilation, (win - 1) * dil + 1 <= 33)
TC_SHAPES_DIL = [(N, H, T, C, win, left, dil) for (N, H, T) in ((3, 1, 200), (12, 4, 50), (2, 2, 129))
                 for (C, win, left, dil) in ((64, 7, 3, 2), (32, 7, 3, 4), (16, 15, 7, 2), (64, 3, 1, 8), (64, 9, 4, 4),
                                             (32, 5, 0, 8), (64, 3, 2, 16))]


@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
def test_tcgen05_forward_backward_shapes(dtype):
    ops = _ops()
    fam = ops.FAMILY_TCGEN05
    old = ops.set_kernel_family(fam)
    try:
        for idx, shape in enumerate([t + (1,) for t in TC_SHAPES] + TC_SHAPES_DIL):
            N, H, T, C, win, left, dil = shape
            assert ops.kernel_family(N, T, C, win, left, dil, dtype) == fam, "tcgen05 family should take this shape"
            sc = C ** -0.5
            q, k, v = (randn16((N, T, C), dtype, 500 + 3 * idx + i) for i in range(3))
            rpb = 0.3 * torch.randn(H, win, generator=torch.Generator().manual_seed(idx))
            vl = [T] + [max(1, T - 5)] * (N // H - 1)
            o, lse = ops.fused_forward(q.cuda(), k.cuda(), v.cuda(), win, left, dil, sc, rpb.cuda(), vl, H)
            ops.device_status()
            o_r, lse_r = orc.na1d_fused(q.float(), k.float(), v.float(), win, left, dil, sc, rpb, vl, H, return_lse=True)
            tag = "N=%d H=%d T=%d C=%d win=%d left=%d dil=%d " % (N, H, T, C, win, left, dil)
            assert_close_strict(o, o_r, dtype, tag + "o")
            assert float((lse.cpu() - lse_r).abs().max()) < 1e-3 * max(1.0, float(lse_r.abs().max())), tag + "lse"
            # backward through the tcgen05 family as well
            assert ops.kernel_family(N, T, C, win, left, dil, dtype, backward=True) == fam
            d_o = randn16((N, T, C), dtype, 900 + idx)
            bwd_args = (d_o.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, win, left, dil, sc, rpb.cuda(), vl, H)
            try:
                dq, dk, dv, drpb = ops.fused_backward(*bwd_args, need_d_rpb=True)
            except Exception as e:
                # 64-channel rows with the widest window bucket leave 1.5 KB of shared memory: with several heads the bias table
                # and the bias-gradient accumulators do not fit, the forced family refuses and the CUDA-core kernels take the call
                assert getattr(e, "status", None) == -10 and C == 64 and (win - 1) * dil + 1 > 17 and H > 1, tag
                ops.set_kernel_family(ops.FAMILY_AUTO)
                dq, dk, dv, drpb = ops.fused_backward(*bwd_args, need_d_rpb=True)
                ops.set_kernel_family(fam)
            ops.device_status()
            _, dq_r, dk_r, dv_r, drpb_r = orc.na1d_fused_with_grads(q.float(), k.float(), v.float(), d_o.float(), win,
                                                                    left, dil, sc, rpb, vl, H)
            assert_close(dq, dq_r, dtype, tag + "dq")
            assert_close(dk, dk_r, dtype, tag + "dk")
            assert_close(dv, dv_r, dtype, tag + "dv")
            assert_close(drpb, drpb_r, dtype, tag + "drpb", factor=2.0)
        # with the tcgen05 family forced: dilations and short sequences the flat tiling cannot take go to the segmented tiling,
        # channel counts outside {16, 32, 64} are refused (and taken by the CUDA-core kernels otherwise)
        assert ops.kernel_tiling(2, 64, 64, 7, 3, 3, dtype) == 2     # dilation not a power of two
        assert ops.kernel_tiling(2, 64, 64, 15, 7, 4, dtype) == 2    # dilated window wider than 33
        assert ops.kernel_tiling(2, 16, 64, 7, 3, 1, dtype) == 2     # sequences shorter than 32 tokens
        assert ops.kernel_tiling(2, 200, 64, 7, 3, 1, dtype) == 1
        assert ops.kernel_family(2, 64, 24, 7, 3, 1, dtype) == -10
        assert ops.kernel_family(2, 64, 64, 40, 20, 1, dtype) == -10  # window wider than the widest band bucket
    finally:
        ops.set_kernel_family(old)
    assert ops.kernel_family(2, 64, 24, 7, 3, 1, dtype) == 0
    assert ops.kernel_family(2, 64, 64, 40, 20, 1, dtype) == 0

"""GPU parity at the benchmark suite's own sizes, through the C ABI.

The oracle cannot run these shapes whole in seconds, so a sample of sequences (first, last, two in the middle -- each
(batch, head) sequence is independent) is compared in full, and the whole result is held to size-independent properties
(bitwise determinism, finite values). Inputs are generated on the device from a seed; the oracle is fed the very same
16-bit values.
"""
import pytest
import torch

from gpu_util import TOL, assert_close, assert_close_strict
from oracle import na1d_oracle as orc

pytestmark = pytest.mark.gpu
DTYPES = [torch.bfloat16, torch.float16]


def _ops():
    from pcf_nat_b200 import ops
    return ops


def _device_inputs(shape, dtype, seed, scale=1.0, n=4):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return [(torch.randn(shape, device="cuda", generator=g) * scale).to(dtype) for _ in range(n)]


def _sample(N):
    return sorted({0, N // 3, N // 2 + 1, N - 1})


def _compare_sampled(tag, dtype, q, k, v, d_o, o, lse, grads, win, left, dil, scale, heads=1, rpb=None, valid_len=None):
    """Oracle on whole utterances (all heads of the sampled batch entries), compared with the same rows of the GPU result."""
    N = q.shape[0]
    batch = N // heads
    for b in _sample(batch):
        sl = slice(b * heads, (b + 1) * heads)
        vl = None if valid_len is None else [int(valid_len[b])]
        f = lambda x: x[sl].float().cpu()
        if grads is None:
            o_r, lse_r = orc.na1d_fused(f(q), f(k), f(v), win, left, dil, scale, rpb, vl, heads, return_lse=True)
        else:
            o_r, dq_r, dk_r, dv_r, _ = orc.na1d_fused_with_grads(f(q), f(k), f(v), f(d_o), win, left, dil, scale, rpb, vl, heads)
            lse_r = None
        assert_close_strict(o[sl], o_r, dtype, "%s o[b=%d]" % (tag, b))
        if lse_r is not None:
            assert float((lse[sl].cpu() - lse_r).abs().max()) < 1e-3 * max(1.0, float(lse_r.abs().max())), tag + " lse"
        if grads is not None:
            for name, g, r in zip(("dq", "dk", "dv"), grads, (dq_r, dk_r, dv_r)):
                assert_close(g[sl], r, dtype, "%s %s[b=%d]" % (tag, name, b))


def test_long_utterance_forward_full_shape():
    """Long-utterance inference shape: B=16, heads=8, L=3000, head_dim=64, window 15, bf16, forward (and backward)."""
    ops = _ops()
    dtype = torch.bfloat16
    N, H, T, C, win, left = 128, 8, 3000, 64, 15, 7
    q, k, v, d_o = _device_inputs((N, T, C), dtype, 3)
    assert ops.kernel_family(N, T, C, win, left, 1, dtype) == ops.FAMILY_TCGEN05
    o, lse = ops.fused_forward(q, k, v, win, left, 1, 1.0, None, None, H)
    o2, lse2 = ops.fused_forward(q, k, v, win, left, 1, 1.0, None, None, H)
    ops.device_status()
    assert torch.equal(o, o2) and torch.equal(lse, lse2), "forward is not deterministic"
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    _compare_sampled("long utterance fwd", dtype, q, k, v, None, o, lse, None, win, left, 1, 1.0, H)
    dq, dk, dv, _ = ops.fused_backward(d_o, q, k, v, o, lse, win, left, 1, 1.0, None, None, H)
    dq2, dk2, dv2, _ = ops.fused_backward(d_o, q, k, v, o, lse, win, left, 1, 1.0, None, None, H)
    ops.device_status()
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2), "backward is not deterministic"
    _compare_sampled("long utterance bwd", dtype, q, k, v, d_o, o, lse, (dq, dk, dv), win, left, 1, 1.0, H)


# window / dilation / length / head-dim corners of the sweep (B=64, heads=4 -> 256 sequences, inputs scaled by D^-1/4)
SWEEP_CORNERS = [(L, D, win, dil) for L in (400, 1000) for D in (32, 64) for win in (3, 31) for dil in (1, 4)]
SWEEP_CORNERS += [(1000, 64, 15, 4), (400, 32, 31, 2), (200, 64, 7, 2), (1000, 32, 15, 2)]


@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
def test_sweep_corners_at_full_batch(dtype):
    ops = _ops()
    N, H = 256, 4
    for idx, (L, D, win, dil) in enumerate(SWEEP_CORNERS):
        left = win - 1 - win // 2
        q, k, v, d_o = _device_inputs((N, L, D), dtype, 20 + idx, scale=D ** -0.25)
        tag = "L=%d D=%d win=%d dil=%d" % (L, D, win, dil)
        o, lse = ops.fused_forward(q, k, v, win, left, dil, 1.0, None, None, H)
        dq, dk, dv, _ = ops.fused_backward(d_o, q, k, v, o, lse, win, left, dil, 1.0, None, None, H)
        ops.device_status()
        for t in (o, dq, dk, dv):
            assert torch.isfinite(t.float()).all(), tag
        _compare_sampled(tag, dtype, q, k, v, d_o, o, lse, (dq, dk, dv), win, left, dil, 1.0, H)


# Persistent CTAs with several tiles each, together with a bias, its gradient and padded utterances: more tiles than
# twice the number of SMs, so that the per-CTA accumulation of the bias gradient over tiles, the tile-to-tile row cursor
# and the padding masks across tiles are all compared with the oracle (whole tensors).
MULTI_TILE = [
    # N,   H,  T,   C,  win, dil
    (512,  4,  200, 64, 7,   1),
    (2048, 16, 150, 16, 27,  1),
    (512,  4,  200, 32, 7,   2),
    (768,  3,  130, 32, 15,  1),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
@pytest.mark.parametrize("shape", MULTI_TILE, ids=lambda s: "N%d_H%d_T%d_C%d_w%d_d%d" % s)
def test_many_tiles_per_cta_with_bias_and_padding(shape, dtype):
    ops = _ops()
    N, H, T, C, win, dil = shape
    left = win - 1 - win // 2
    batch = N // H
    sc = C ** -0.5
    q, k, v, d_o = _device_inputs((N, T, C), dtype, 77 + N)
    gen = torch.Generator().manual_seed(N + win)
    rpb = 0.3 * torch.randn(H, win, generator=gen)
    # a third of the utterances padded by up to half their length, one of them almost entirely
    vl = torch.full((batch,), T, dtype=torch.int64)
    pad_idx = torch.arange(0, batch, 3)
    vl[pad_idx] = torch.randint(T // 2, T, (pad_idx.numel(),), generator=gen)
    vl[batch // 2] = 2
    assert (N * T) // 128 > 2 * 148
    o, lse = ops.fused_forward(q, k, v, win, left, dil, sc, rpb.cuda(), vl.tolist(), H)
    dq, dk, dv, drpb = ops.fused_backward(d_o, q, k, v, o, lse, win, left, dil, sc, rpb.cuda(), vl.tolist(), H, need_d_rpb=True)
    ops.device_status()
    f = lambda x: x.float().cpu()
    o_r, dq_r, dk_r, dv_r, drpb_r = orc.na1d_fused_with_grads(f(q), f(k), f(v), f(d_o), win, left, dil, sc, rpb, vl.tolist(), H)
    tag = "N=%d H=%d T=%d C=%d win=%d dil=%d " % shape
    assert_close_strict(o, o_r, dtype, tag + "o")
    assert_close(dq, dq_r, dtype, tag + "dq")
    assert_close(dk, dk_r, dtype, tag + "dk")
    assert_close(dv, dv_r, dtype, tag + "dv")
    # the bias gradient is a sum over N*T/H rows: its bound is relative to its own magnitude
    assert_close(drpb, drpb_r, dtype, tag + "drpb", factor=2.0)
    # and twice the same bits
    dq2, dk2, dv2, drpb2 = ops.fused_backward(d_o, q, k, v, o, lse, win, left, dil, sc, rpb.cuda(), vl.tolist(), H, need_d_rpb=True)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


def test_first_config_forward_strict_and_against_unrounded_reference():
    """Forward-only case B=2, heads=4, L=200, head_dim=32, window 7: the strict bound against the oracle on the rounded
    inputs, and -- printed, with the looser bound that input rounding alone requires -- against the vector the reference's
    own CPU code produced from the unrounded fp32 inputs."""
    import os
    import numpy as np
    from cases import CASES, win_left
    from gpu_util import rounded_inputs
    ops = _ops()
    name = "cfg1_fwd"
    c = CASES[name]
    win, left = win_left(c["win"])
    gold = torch.from_numpy(np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))["out"])
    for dtype in DTYPES:
        (q, k, v, _), (qf, kf, vf, _), _ = rounded_inputs(name, dtype)
        o, _ = ops.fused_forward(q, k, v, win, left, c["dil"], c["scale"], None, None, c["H"])
        o_r = orc.na1d_fused(qf, kf, vf, win, left, c["dil"], c["scale"], None, None, c["H"])
        e_round = assert_close_strict(o, o_r, dtype, "first config o")
        e_gold = float((o.float().cpu() - gold).abs().max())
        e_inputs = float((o_r - gold).abs().max())   # what rounding q, k, v to 16 bits does to the fp32 result by itself
        print("first config %s: vs oracle on rounded inputs %.3e (bound %.0e); vs reference vector on unrounded fp32 "
              "inputs %.3e, of which input rounding alone %.3e" % (str(dtype).split(".")[-1], e_round, TOL[dtype], e_gold, e_inputs))
        assert e_gold <= e_inputs + TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("N,T,C,win,left,dil", [(2051, 150, 16, 27, 13, 1), (1027, 150, 32, 15, 7, 2), (515, 200, 64, 7, 3, 1)])
def test_unfused_entry_points_many_tiles_per_cta(N, T, C, win, left, dil, dtype):
    """The six unfused entry points with several tiles per CTA and a ragged last tile (N*T is no multiple of 128): the
    tcgen05 band modes against the CUDA-core kernels of the same library (both are held to the oracle at small sizes), and
    the band output through a pointer that is only 4-byte aligned (the 16-byte-store path must not be taken)."""
    from pcf_nat_b200 import ops
    g = torch.Generator().manual_seed(77)
    q, k, v, d_o = ((torch.randn(N, T, C, generator=g) * C ** -0.25).to(dtype).cuda() for _ in range(4))
    res = {}
    for fam in (ops.FAMILY_CUDA_CORE, ops.FAMILY_AUTO):
        old = ops.set_kernel_family(fam)
        try:
            attn = ops.qk_forward(q, k, win, left, dil)
            p = torch.softmax(attn, -1)
            res[fam] = (attn, ops.av_forward(p, v, win, left, dil), ops.a_backward(d_o, v, win, left, dil), ops.q_backward(p, k, win, left, dil),
                        ops.k_backward(p, q, win, left, dil), ops.v_backward(p, d_o, win, left, dil))
        finally:
            ops.set_kernel_family(old)
    ops.device_status()
    names = ("qk", "av", "a_gd", "q_gd", "k_gd", "v_gd")
    for nm, a, b in zip(names, res[ops.FAMILY_CUDA_CORE], res[ops.FAMILY_AUTO]):
        if a.dtype == torch.float32:
            assert float((a - b).abs().max()) < 1e-4 * max(1.0, float(a.abs().max())), nm
        else:
            assert_close(b, a, dtype, nm)
    # band output through a pointer that is 4-byte but not 16-byte aligned
    import ctypes
    from pcf_nat_b200 import _lib
    L = _lib.lib()
    buf = torch.full((N * T * win + 8,), float("nan"), dtype=torch.float32, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.na1d_qk_forward(ctypes.c_void_p(buf.data_ptr() + 4), ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()),
                           N, T, C, win, left, dil, 0 if dtype == torch.bfloat16 else 1, st)
    assert rc == 0
    torch.cuda.synchronize()
    got = buf[1:1 + N * T * win].view(N, T, win)
    ref = res[ops.FAMILY_CUDA_CORE][0]
    assert float((got - ref).abs().max()) < 1e-4 * max(1.0, float(ref.abs().max()))
    assert torch.isnan(buf[0]) and torch.isnan(buf[1 + N * T * win:]).all()


def test_bias_gradient_partial_rows_mode_in_a_fresh_process():
    """NA1D_BIAS_GRAD_ROWS=1 (read once per process): one partial row of d_rpb per CTA in the caller's scratch, summed by the
    second kernel in a fixed order -- same values as the oracle, and the same bits when the call is repeated (64-channel
    rows: per-warp accumulators, no atomics anywhere on the way)."""
    import os
    import subprocess
    import sys
    code = r'''
import sys, torch
sys.path[:0] = ["tests", "tests/golden"]
from gpu_util import assert_close
from oracle import na1d_oracle as orc
from pcf_nat_b200 import ops
N, H, T, C, win, left = 1200, 4, 200, 64, 7, 3
g = torch.Generator().manual_seed(5)
q, k, v, d_o = ((torch.randn(N, T, C, generator=g) * C ** -0.25).to(torch.bfloat16) for _ in range(4))
rpb = 0.3 * torch.randn(H, win, generator=g)
vl = [T - (i % 7) for i in range(N // H)]
sc = C ** -0.5
o, lse = ops.fused_forward(q.cuda(), k.cuda(), v.cuda(), win, left, 1, sc, rpb.cuda(), vl, H)
args = (d_o.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, win, left, 1, sc, rpb.cuda(), vl, H)
a = ops.fused_backward(*args, need_d_rpb=True)[3]
b = ops.fused_backward(*args, need_d_rpb=True)[3]
ops.device_status()
assert torch.equal(a, b), "partial rows summed in a fixed order must repeat bit for bit"
ref = orc.na1d_fused_with_grads(q.float(), k.float(), v.float(), d_o.float(), win, left, 1, sc, rpb, vl, H)[4]
assert_close(a, ref, torch.bfloat16, "drpb", factor=2.0)
print("ok")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NA1D_BIAS_GRAD_ROWS="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]

"""The backward entry point that allocates nothing (na1d_fused_backward_static).

Some hosts cannot give the backward pass its N*T-float workspace: their device memory pool is frozen,
or they sit inside a stream capture, or they are a bare C runtime with fixed buffers and no allocator.
For them the library keeps that workspace in a fixed device array. This file checks, through the C ABI,
that the variant returns what the regular entry point returns -- on two calls in a row, the second
smaller than the first so stale workspace contents would show -- and that it refuses problems larger
than the array instead of overrunning it. It is named to be collected last.
"""
import ctypes

import pytest
import torch

from gpu_util import assert_close, randn16



def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _run_both(L, ops, N, H, T, C, win, left, dil, dtype, seed, with_rpb):
    code = 0 if dtype == torch.bfloat16 else 1
    q, k, v, d_o = (randn16((N, T, C), dtype, seed + i).cuda() for i in range(4))
    rpb = (0.3 * torch.randn(H, win, generator=torch.Generator().manual_seed(seed))).cuda() if with_rpb else None
    sc = C ** -0.5
    o, lse = ops.fused_forward(q, k, v, win, left, dil, sc, rpb, None, H)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def outputs():
        return [torch.empty_like(q) for _ in range(3)] + [torch.zeros(H, win, device="cuda") if with_rpb else None]

    # existing entry point, CUDA-core kernels (the ones whose workspace the variant internalises)
    old = ops.set_kernel_family(ops.FAMILY_CUDA_CORE)
    try:
        ref = outputs()
        delta = torch.empty(N, T, device="cuda")
        assert L.na1d_fused_backward(_p(ref[0]), _p(ref[1]), _p(ref[2]), _p(ref[3]), _p(d_o), _p(q), _p(k), _p(v), _p(o),
                                     _p(lse), _p(rpb), None, _p(delta), N, H, T, C, win, left, dil, sc, code, st) == 0
    finally:
        ops.set_kernel_family(old)
    got = outputs()
    assert L.na1d_fused_backward_static(_p(got[0]), _p(got[1]), _p(got[2]), _p(got[3]), _p(d_o), _p(q), _p(k), _p(v),
                                        _p(o), _p(lse), _p(rpb), None, N, H, T, C, win, left, dil, sc, code, st) == 0
    torch.cuda.synchronize()
    for name, a, b in zip(("dq", "dk", "dv"), got, ref):
        assert_close(a, b.float(), dtype, "static " + name)
        assert torch.equal(a, b), name + ": same kernels, same inputs, must be bit-identical"
    if with_rpb:
        assert_close(got[3], ref[3], dtype, "static d_rpb", factor=2.0)
    # and against whatever the regular entry point picks on its own (the tcgen05 kernels where they apply)
    auto = ops.fused_backward(d_o, q, k, v, o, lse, win, left, dil, sc, rpb, None, H, need_d_rpb=with_rpb)
    for name, a, b in zip(("dq", "dk", "dv"), got, auto):
        assert_close(a, b.float(), dtype, "static vs automatic family " + name)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_static_backward_matches_regular_entry_point_twice_in_a_row(dtype):
    from pcf_nat_b200 import _lib, ops
    L = _lib.lib()
    _run_both(L, ops, 64, 4, 200, 64, 7, 3, 1, dtype, seed=700, with_rpb=True)
    _run_both(L, ops, 8, 2, 77, 32, 15, 7, 2, dtype, seed=710, with_rpb=False)   # smaller: old workspace contents remain behind it
    ops.device_status()


def test_static_backward_rejects_more_rows_than_the_workspace_holds():
    from pcf_nat_b200 import _lib
    L = _lib.lib()
    limit = 1 << 20             # NA1D_STATIC_SCRATCH_ROWS
    P = ctypes.c_void_p(4096)  # never dereferenced: the size check comes first
    N, T = 4096, 257            # N*T = 1052672 > 2**20
    assert N * T > limit
    s = L.na1d_fused_backward_static(P, P, P, None, P, P, P, P, P, P, None, None, N, 1, T, 64, 7, 3, 1, 1.0, 0, None)
    assert s == -9
    assert b"capacity" in L.na1d_status_string(s)
    # the check is host-side: no device is needed and nothing was launched


@pytest.mark.gpu
def test_static_backward_allocates_nothing_and_handles_padding():
    """Repeated calls leave the device's free memory unchanged, and a padded batch gives the regular entry point's bits."""
    from pcf_nat_b200 import _lib, ops
    L = _lib.lib()
    N, H, T, C, win, left = 8, 2, 77, 32, 7, 3
    dtype, code = torch.bfloat16, 0
    q, k, v, d_o = (randn16((N, T, C), dtype, 820 + i).cuda() for i in range(4))
    vl = torch.tensor([77, 40, 3, 60], dtype=torch.int32, device="cuda")
    o, lse = ops.fused_forward(q, k, v, win, left, 1, 0.2, None, vl, H)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    got = [torch.empty_like(q) for _ in range(3)]
    ref = [torch.empty_like(q) for _ in range(3)]
    delta = torch.empty(N, T, device="cuda")
    call = lambda out: L.na1d_fused_backward_static(_p(out[0]), _p(out[1]), _p(out[2]), None, _p(d_o), _p(q), _p(k), _p(v), _p(o),
                                                    _p(lse), None, _p(vl), N, H, T, C, win, left, 1, 0.2, code, st)
    assert call(got) == 0           # the first call on a device looks the array's address up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        assert call(got) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "the static entry point changed the device's free memory"
    old = ops.set_kernel_family(ops.FAMILY_CUDA_CORE)
    try:
        assert L.na1d_fused_backward(_p(ref[0]), _p(ref[1]), _p(ref[2]), None, _p(d_o), _p(q), _p(k), _p(v), _p(o), _p(lse), None,
                                     _p(vl), _p(delta), N, H, T, C, win, left, 1, 0.2, code, st) == 0
    finally:
        ops.set_kernel_family(old)
    torch.cuda.synchronize()
    for a, b in zip(got, ref):
        assert torch.equal(a, b)

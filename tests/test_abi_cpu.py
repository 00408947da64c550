"""CPU-side checks of the C ABI: the library loads, exports every declared symbol, and rejects
bad arguments on the host with status codes (no device work is attempted)."""
import ctypes

import pytest

from pcf_nat_b200 import _lib

L = _lib.lib()


def test_every_declared_symbol_is_exported():
    names = _lib.declared_symbols()
    assert "na1d_fused_forward" in names and "na1d_qk_forward" in names and len(names) >= 13
    for n in names:
        assert hasattr(L, n), "library does not export %s" % n


def test_status_strings():
    assert L.na1d_status_string(0) == b"ok"
    for s in range(-9, 0):
        assert len(L.na1d_status_string(s)) > 3
    assert L.na1d_version() >= 100


P = ctypes.c_void_p(4096)  # never dereferenced: validation fails first


@pytest.mark.parametrize("args,status", [
    ((None, P, P, 1, 8, 8, 3, 1, 1, 0, None), -1),
    ((P, P, P, 0, 8, 8, 3, 1, 1, 0, None), -2),
    ((P, P, P, 1, 8, 12, 3, 1, 1, 0, None), -2),      # C % 8 != 0
    ((P, P, P, 1, 8, 40, 3, 1, 1, 0, None), -2),      # unsupported channel split
    ((P, P, P, 1, 8, 8, 0, 0, 1, 0, None), -3),
    ((P, P, P, 1, 8, 8, 129, 0, 1, 0, None), -3),
    ((P, P, P, 1, 8, 8, 3, 3, 1, 0, None), -3),       # left == win
    ((P, P, P, 1, 8, 8, 3, 1, 0, 0, None), -3),       # dil == 0
    ((P, P, P, 1, 8, 8, 3, 1, 1, 7, None), -4),
    ((P, ctypes.c_void_p(4100), P, 1, 8, 8, 3, 1, 1, 0, None), -6),
    ((P, P, P, 1 << 20, 1 << 12, 8, 3, 1, 1, 0, None), -2),  # N*T overflows int32
])
def test_qk_forward_rejects_bad_arguments(args, status):
    assert L.na1d_qk_forward(*args) == status


def test_fused_rejects_bad_heads():
    a = (P, P, P, P, P, None, None, 6, 4, 8, 8, 3, 1, 1, 1.0, 0, None)
    assert L.na1d_fused_forward(*a) == -5


def test_ops_refuse_cpu_tensors():
    import torch
    from pcf_nat_b200 import ops
    q = torch.zeros(1, 4, 8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.fused_forward(q, q, q, 3, 1)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.qk_forward(q, q, 3, 1)


def test_compat_surface_matches_reference_names():
    import torch
    from pcf_nat_b200 import nattn
    qk, av = nattn.getNA1dFunction(16, 1, torch.bfloat16)
    assert qk.__name__ == "bf16_ANA1d_QK_Function" and av.__name__ == "bf16_ANA1d_AV_Function"
    qk, av = nattn.getNA1dFunction(16, 1, torch.float16)
    assert qk.__name__ == "fp16_ANA1d_QK_Function" and av.__name__ == "fp16_ANA1d_AV_Function"
    with pytest.raises(AssertionError):
        nattn.getNA1dFunction(12, 1, torch.bfloat16)
    with pytest.raises(AssertionError):
        nattn.getNA1dFunction(16, 1, torch.float32)
    nattn.install_as_na1d_tensorcore()
    from na1d_tensorcore.nattn import getNA1dFunction
    assert getNA1dFunction is nattn.getNA1dFunction


def test_strided_entry_points_validate_on_the_host():
    """Bad strides, dropout probabilities and shapes are refused before any device work (no GPU is needed here)."""
    good = (ctypes.c_int64 * 3)(2 * 64 * 32, 64 * 32, 32)
    common = (4, 2, 64, 32, 7, 3, 1, 1.0, 0, None)
    for bad in ((0, 2048, 32), (4096, 2048, 20), (4096, 2052, 32), (-8, 2048, 32), (4096, 2048, 24)):
        b = (ctypes.c_int64 * 3)(*bad)
        assert L.na1d_fused_forward_strided(P, None, P, P, P, None, None, good, b, good, good, *common) == -11, bad
    assert L.na1d_fused_forward_strided(P, None, P, P, P, None, None, good, None, good, good, *common) == -1
    assert L.na1d_fused_forward_strided(P, None, P, P, P, None, None, good, good, good, good, 4, 2, 64, 24, 7, 3, 1, 1.0, 0, None) in (-10, -11)
    # dropout probability outside [0, 1)
    args = (P, None, P, P, P, None, None, 4, 2, 64, 32, 7, 3, 1, 1.0)
    assert L.na1d_fused_forward_dropout(*args, 1.0, 5, 0, None) == -12
    assert L.na1d_fused_forward_dropout(*args, -0.1, 5, 0, None) == -12
    assert L.na1d_fused_forward_dropout(P, None, P, P, P, None, None, 4, 2, 64, 24, 7, 3, 1, 1.0, 0.1, 5, 0, None) == -10


def test_kernel_tiling_choice_is_a_host_side_query():
    """0 = CUDA cores, 1 = tcgen05 flat tiling, 2 = tcgen05 segmented tiling (no device work)."""
    t = lambda N, T, C, win, left, dil, bw=0: L.na1d_fused_kernel_tiling(N, T, C, win, left, dil, 0, bw)
    assert t(512, 200, 64, 7, 3, 1) == 1 and t(512, 200, 64, 7, 3, 1, 1) == 1
    assert t(128, 3000, 64, 15, 7, 1) == 1
    assert t(256, 1000, 64, 31, 15, 4) == 2 and t(256, 1000, 64, 31, 15, 4, 1) == 2   # dilated window beyond the flat limit
    assert t(256, 400, 32, 15, 7, 4) == 2
    assert t(256, 200, 64, 7, 3, 3) == 2                                             # dilation not a power of two
    assert t(256, 200, 64, 3, 1, 4) == 1                                             # narrow dilated window: flat tiling
    assert t(256, 1000, 64, 7, 3, 4) == 2 and t(256, 200, 64, 7, 3, 4) == 1          # bucket cost against tile utilisation
    assert t(4, 16, 64, 7, 3, 1) == 2                                                # shorter than 32 tokens
    assert t(4, 200, 24, 7, 3, 1) == 0 and t(4, 200, 64, 41, 20, 1) == 0 and t(4, 1, 64, 3, 1, 1) == 0
    assert L.na1d_fused_kernel_family(256, 1000, 64, 31, 15, 4, 0, 0) == 1
    assert L.na1d_fused_strided_supported(4, 300, 64, 7, 3, 1, 0, 1, 1) == 1
    assert L.na1d_fused_strided_supported(4, 300, 24, 7, 3, 1, 0, 1, 1) < 0 or L.na1d_fused_strided_supported(4, 300, 24, 7, 3, 1, 0, 1, 1) == 0
    assert L.na1d_fused_strided_supported(4, 300, 64, 31, 15, 1, 0, 1, 1) == 0        # no room for the bias tables of 4 heads

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

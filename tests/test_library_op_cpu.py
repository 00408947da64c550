"""torch.library registration of the fused operator: schemas and fake (meta) kernels, no GPU needed."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_ops_are_registered_with_schemas():
    import pcf_nat_b200  # noqa: F401
    fwd = torch.ops.pcf_nat_b200.na1d_fused_fwd.default
    bwd = torch.ops.pcf_nat_b200.na1d_fused_bwd.default
    assert "Tensor? rpb" in str(fwd._schema) and "-> (Tensor, Tensor)" in str(fwd._schema)
    assert "bool need_d_rpb" in str(bwd._schema)


def test_fake_kernels_propagate_shapes():
    import pcf_nat_b200
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        q = torch.empty(8, 200, 32, dtype=torch.bfloat16, device="cuda")
        rpb = torch.empty(1, 4, 1, 7, device="cuda")
        vl = torch.empty(2, dtype=torch.int32, device="cuda")
        o = pcf_nat_b200.na1d_fused(q, q, q, 7, 3, 1, 0.2, rpb, vl, 4)
        assert o.shape == q.shape and o.dtype == q.dtype and o.device.type == "cuda"
        o2, lse = torch.ops.pcf_nat_b200.na1d_fused_fwd(q, q, q, None, None, 7, 3, 1, 1.0, 4)
        assert lse.shape == (8, 200) and lse.dtype == torch.float32
        dq, dk, dv, d_rpb = torch.ops.pcf_nat_b200.na1d_fused_bwd(o, q, q, q, o, lse, rpb, vl, 7, 3, 1, 0.2, 4, True)
        assert dq.shape == q.shape and d_rpb.shape == (4, 7)
        *_, none_rpb = torch.ops.pcf_nat_b200.na1d_fused_bwd(o, q, q, q, o, lse, None, None, 7, 3, 1, 0.2, 4, True)
        assert none_rpb.numel() == 0


def test_fake_kernel_rejects_bad_arguments():
    import pcf_nat_b200  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        q = torch.empty(8, 200, 32, dtype=torch.float32, device="cuda")
        with pytest.raises(RuntimeError):
            torch.ops.pcf_nat_b200.na1d_fused_fwd(q, q, q, None, None, 7, 3, 1, 1.0, 4)   # fp32 is not supported
        h = q.to(torch.float16)
        with pytest.raises(RuntimeError):
            torch.ops.pcf_nat_b200.na1d_fused_fwd(h, h, h, None, None, 7, 7, 1, 1.0, 4)   # left >= win


def test_no_cpu_kernel():
    import pcf_nat_b200
    q = torch.zeros(2, 40, 16, dtype=torch.bfloat16)
    with pytest.raises(Exception):
        pcf_nat_b200.na1d_fused(q, q, q, 3, 1)

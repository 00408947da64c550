"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from cases import CASES, make_inputs, win_left
from oracle import na1d_oracle as orc

# BASELINE tolerances (max-abs against the fp32 oracle evaluated on the SAME 16-bit-rounded
# input values the kernel sees): 2e-2 for bf16, 5e-3 for fp16. For tensors whose magnitude
# exceeds 1 (gradients, unnormalised logits) the bound scales with max|reference|, since a
# 16-bit output cannot be closer than its own rounding step.
TOL = {torch.bfloat16: 2e-2, torch.float16: 5e-3}


def assert_close(got, ref, dtype, what="", factor=1.0):
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), what + ": non-finite values"
    err = float((got - ref).abs().max()) if got.numel() else 0.0
    bound = TOL[dtype] * factor * max(1.0, float(ref.abs().max()) if ref.numel() else 1.0)
    assert err <= bound, "%s: max-abs error %.4g > %.4g" % (what, err, bound)
    return err


def rounded_inputs(case, dtype, device="cuda"):
    """Seeded inputs rounded to `dtype`: (device 16-bit tensors, the same values as fp32 CPU tensors)."""
    arrs = make_inputs(case)
    q, k, v, d_out = (torch.from_numpy(a).to(dtype) for a in arrs[:4])
    rpb = torch.from_numpy(arrs[4])
    dev = tuple(x.to(device) for x in (q, k, v, d_out))
    cpu = tuple(x.float() for x in (q, k, v, d_out))
    return dev, cpu, rpb


def randn16(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)

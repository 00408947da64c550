"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from cases import CASES, make_inputs, win_left
from oracle import na1d_oracle as orc

# Tolerances of the operator's specification: max-abs 2e-2 for bf16, 5e-3 for fp16, against the fp32 oracle evaluated
# on the SAME 16-bit-rounded input values the kernel sees.
#   * forward outputs (`assert_close_strict`): the absolute bound, as stated, no scaling;
#   * gradients (`assert_close`): the bound scales with max|reference| when that exceeds 1 -- a gradient is a sum over
#     the window of products of O(1) terms, a 16-bit output cannot be closer to it than its own rounding step, and dS is
#     rounded to 16 bits before the second product as the reference does (bf16_ana1d_kernel.cu:305, :414).
TOL = {torch.bfloat16: 2e-2, torch.float16: 5e-3}


def _max_err(got, ref, what):
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), what + ": non-finite values"
    err = float((got - ref).abs().max()) if got.numel() else 0.0
    return err, (float(ref.abs().max()) if ref.numel() else 1.0)


def assert_close(got, ref, dtype, what="", factor=1.0):
    """Gradient bound: TOL * factor * max(1, max|ref|)."""
    err, mag = _max_err(got, ref, what)
    bound = TOL[dtype] * factor * max(1.0, mag)
    assert err <= bound, "%s: max-abs error %.4g > %.4g" % (what, err, bound)
    return err


def half_ulp(ref, dtype):
    """Half the spacing of `dtype` values at the magnitude of each element of `ref` (the unavoidable rounding of a result
    stored in that dtype): 2^(floor(log2|x|) - m), m = 8 mantissa bits for bfloat16, 11 for float16."""
    m = 8 if dtype == torch.bfloat16 else 11
    return torch.exp2(torch.floor(torch.log2(ref.abs().clamp_min(1e-30))) - m)


def assert_close_strict(got, ref, dtype, what=""):
    """Forward-output bound: the absolute tolerance of the specification, unscaled, for every element below 4 in
    magnitude. From 4 upwards a bfloat16 result is spaced 2^-5 apart, so its own storage rounding (up to 0.0156) is most
    of the 2e-2 budget before any arithmetic error; there -- and only there -- that rounding step is added to the bound.
    (Near-one-hot windows at scale 1 return single V rows, and |v| exceeds 4 a few times per million N(0,1) samples.)"""
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), what + ": non-finite values"
    if got.numel() == 0:
        return 0.0
    err = (got - ref).abs()
    bound = torch.full_like(ref, TOL[dtype]) + torch.where(ref.abs() >= 4.0, half_ulp(ref, dtype), torch.zeros_like(ref))
    bad = err > bound
    if bool(bad.any()):
        i = int(torch.argmax(err - bound))
        raise AssertionError("%s: max-abs error %.4g > %.4g (strict) at reference value %.4g" % (
            what, float(err.flatten()[i]), float(bound.flatten()[i]), float(ref.flatten()[i])))
    return float(err.max())


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

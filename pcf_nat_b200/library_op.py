"""The fused operator as ``torch.library`` custom ops, so that ``torch.compile`` / ``torch.export`` trace through it.

The reference's operators are opaque pybind calls inside ``torch.autograd.Function`` and break graphs
(``train_main.py:103-104`` sets ``suppress_errors`` for that reason). Here:

* ``pcf_nat_b200::na1d_fused_fwd(q, k, v, rpb?, valid_len?, win, left, dil, scale, heads) -> (o, lse)``
* ``pcf_nat_b200::na1d_fused_bwd(d_o, q, k, v, o, lse, rpb?, valid_len?, win, left, dil, scale, heads, need_d_rpb)
  -> (dq, dk, dv, d_rpb)``

with fake (meta) kernels for shape propagation and an autograd formula that saves ``(q, k, v, o, lse)``. Both are CUDA
only: there is no CPU kernel to fall back to.
"""
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import ops


@torch.library.custom_op("pcf_nat_b200::na1d_fused_fwd", mutates_args=(), device_types="cuda")
def na1d_fused_fwd(q: Tensor, k: Tensor, v: Tensor, rpb: Optional[Tensor], valid_len: Optional[Tensor], win: int, left: int,
                   dil: int, scale: float, heads: int) -> Tuple[Tensor, Tensor]:
    o, lse = ops.fused_forward(q, k, v, win, left, dil, scale, rpb, valid_len, heads)
    return o, lse


@na1d_fused_fwd.register_fake
def _(q, k, v, rpb, valid_len, win, left, dil, scale, heads):
    torch._check(q.dim() == 3 and q.shape == k.shape == v.shape, lambda: "q, k, v must be (N, T, C) of one shape")
    torch._check(q.dtype in (torch.bfloat16, torch.float16) and q.dtype == k.dtype == v.dtype, lambda: "bf16 or fp16 only")
    torch._check(0 <= left < win, lambda: "0 <= left < win")
    return torch.empty_like(q), q.new_empty((q.shape[0], q.shape[1]), dtype=torch.float32)


@torch.library.custom_op("pcf_nat_b200::na1d_fused_bwd", mutates_args=(), device_types="cuda")
def na1d_fused_bwd(d_o: Tensor, q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse: Tensor, rpb: Optional[Tensor],
                   valid_len: Optional[Tensor], win: int, left: int, dil: int, scale: float, heads: int,
                   need_d_rpb: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    dq, dk, dv, d_rpb = ops.fused_backward(d_o, q, k, v, o, lse, win, left, dil, scale, rpb, valid_len, heads,
                                           need_d_rpb=need_d_rpb and rpb is not None)
    if d_rpb is None:
        d_rpb = q.new_zeros((0,), dtype=torch.float32)
    return dq, dk, dv, d_rpb


@na1d_fused_bwd.register_fake
def _(d_o, q, k, v, o, lse, rpb, valid_len, win, left, dil, scale, heads, need_d_rpb):
    n = heads * win if (need_d_rpb and rpb is not None) else 0
    d_rpb = q.new_empty((heads, win) if n else (0,), dtype=torch.float32)
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), d_rpb


def _setup_context(ctx, inputs, output):
    q, k, v, rpb, valid_len, win, left, dil, scale, heads = inputs
    o, lse = output
    ctx.save_for_backward(q, k, v, o, lse, rpb, valid_len)
    ctx.cfg = (win, left, dil, scale, heads)


def _backward(ctx, d_o, d_lse):
    q, k, v, o, lse, rpb, valid_len = ctx.saved_tensors
    win, left, dil, scale, heads = ctx.cfg
    need = rpb is not None and ctx.needs_input_grad[3]
    dq, dk, dv, d_rpb = na1d_fused_bwd(d_o.contiguous(), q, k, v, o, lse, rpb, valid_len, win, left, dil, scale, heads, need)
    g_rpb = d_rpb.reshape(rpb.shape).to(rpb.dtype) if need else None
    return dq, dk, dv, g_rpb, None, None, None, None, None, None


torch.library.register_autograd("pcf_nat_b200::na1d_fused_fwd", _backward, setup_context=_setup_context)


def na1d_fused(q, k, v, win_size, left, dilation=1, scale=1.0, rpb=None, valid_len=None, heads=1, drop_p=0.0, seed=0):
    """``softmax(scale q.k^T + rpb + mask) . v`` over each query's window; (N*heads, T, C) in, same shape out.

    Under ``torch.compile`` / tracing (fake, functional or otherwise wrapped tensors) the call goes through the registered
    ``torch.library`` ops; on plain eager tensors through ``NA1dFusedFunction``.

    ``rpb``: ``(1, heads, 1, win)`` (or any shape with heads*win elements) fp32 parameter or None; ``valid_len``: int tensor
    or sequence of length N/heads (``T - padding``) or None. ``drop_p`` > 0 applies attention dropout (the reference's
    ``attn_drop``) with the mask that ``seed`` defines. Differentiable in q, k, v and rpb."""
    if drop_p and (type(q) is not Tensor or torch.compiler.is_compiling()):
        raise NotImplementedError("attention dropout is available on the eager route only")
    if type(q) is Tensor and not torch.compiler.is_compiling():
        # plain eager tensors: the autograd.Function route skips the dispatcher's generated backward (host time of a
        # forward+backward pair measured 5 to 35 % lower, depending on the host); same kernels, same saved tensors
        return ops.NA1dFusedFunction.apply(q, k, v, int(win_size), int(left), int(dilation), float(scale), rpb, valid_len,
                                           int(heads), float(drop_p), int(seed))
    if valid_len is not None and not isinstance(valid_len, Tensor):
        valid_len = torch.as_tensor(valid_len, dtype=torch.int32, device=q.device)
    o, _ = na1d_fused_fwd(q, k, v, rpb, valid_len, int(win_size), int(left), int(dilation), float(scale), int(heads))
    return o

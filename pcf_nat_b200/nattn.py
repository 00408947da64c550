"""Drop-in for the reference's ``na1d_tensorcore/nattn.py``: same names, arity and return types.

``getNA1dFunction(C, dilation, dtype)`` returns a ``(QK_Function, AV_Function)`` pair of
``torch.autograd.Function`` classes used as

    attn = QK.apply(q*scale, k, win_size, left, dilation)   # (N,T,win) fp32
    x    = AV.apply(attn, v, win_size, left, dilation)      # (N,T,C) in v's dtype

exactly like na1d_tensorcore/nattn.py:32-137, so models/PCF_NATransformer.py:85,141,150 and
models/MFA_NATransformer.py run unmodified. Differences: the kernels are the sm_100a ones of
this package, they launch on the current stream, and ``dilation > 1`` is honoured (the
reference accepts the argument and ignores it, nattn.py:34, and asserts ``dilation==1``, :130).
"""
import torch

from . import ops


def _make_pair(tag, dtype):
    class QK(torch.autograd.Function):
        @staticmethod
        def forward(ctx, q, k, win_size, left, dilation=1):
            assert q.is_contiguous() and k.is_contiguous()
            assert q.dtype == k.dtype == dtype
            ctx.save_for_backward(q, k)
            ctx.geom = (win_size, left, dilation)
            return ops.qk_forward(q, k, win_size, left, dilation)

        @staticmethod
        def backward(ctx, attn_gd):
            q, k = ctx.saved_tensors
            win_size, left, dilation = ctx.geom
            attn_gd = attn_gd.contiguous()
            q_gd = ops.q_backward(attn_gd, k, win_size, left, dilation)
            k_gd = ops.k_backward(attn_gd, q, win_size, left, dilation)
            return q_gd, k_gd, None, None, None

    class AV(torch.autograd.Function):
        @staticmethod
        def forward(ctx, attn, v, win_size, left, dilation=1):
            assert attn.is_contiguous() and v.is_contiguous()
            assert v.dtype == dtype
            ctx.save_for_backward(attn, v)
            ctx.geom = (win_size, left, dilation)
            return ops.av_forward(attn, v, win_size, left, dilation)

        @staticmethod
        def backward(ctx, result_gd):
            attn, v = ctx.saved_tensors
            win_size, left, dilation = ctx.geom
            result_gd = result_gd.contiguous()
            attn_gd = ops.a_backward(result_gd, v, win_size, left, dilation)
            v_gd = ops.v_backward(attn, result_gd, win_size, left, dilation)
            return attn_gd, v_gd, None, None, None

    QK.__name__ = QK.__qualname__ = "%s_ANA1d_QK_Function" % tag
    AV.__name__ = AV.__qualname__ = "%s_ANA1d_AV_Function" % tag
    return QK, AV


bf16_ANA1d_QK_Function, bf16_ANA1d_AV_Function = _make_pair("bf16", torch.bfloat16)
fp16_ANA1d_QK_Function, fp16_ANA1d_AV_Function = _make_pair("fp16", torch.float16)


def getNA1dFunction(C, dilation, dtype):
    assert C % 8 == 0
    assert dilation >= 1
    if dtype == torch.bfloat16:
        return bf16_ANA1d_QK_Function, bf16_ANA1d_AV_Function
    if dtype == torch.float16:
        return fp16_ANA1d_QK_Function, fp16_ANA1d_AV_Function
    assert False, "NA1D kernels exist for torch.bfloat16 and torch.float16 only"


def install_as_na1d_tensorcore():
    """Register this module as ``na1d_tensorcore.nattn`` so the reference's model files, which do
    ``from na1d_tensorcore.nattn import getNA1dFunction`` (models/PCF_NATransformer.py:22), import
    it without any edit and without the reference's JIT build."""
    import sys
    import types
    pkg = sys.modules.get("na1d_tensorcore") or types.ModuleType("na1d_tensorcore")
    pkg.nattn = sys.modules[__name__]
    sys.modules["na1d_tensorcore"] = pkg
    sys.modules["na1d_tensorcore.nattn"] = sys.modules[__name__]

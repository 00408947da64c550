"""Torch-facing wrappers over the C ABI: device memory and streams come from torch, the
arithmetic comes from libna1d_b200.so. CUDA tensors only -- there is no CPU fallback."""
import ctypes

import torch

from . import _lib
from ._lib import check

_L = _lib.lib()


def _dtype_code(t):
    if t.dtype == torch.bfloat16:
        return _lib.NA1D_BF16
    if t.dtype == torch.float16:
        return _lib.NA1D_FP16
    raise TypeError("NA1D kernels take bfloat16 or float16 tensors, got %s" % t.dtype)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("pcf_nat_b200 runs on CUDA devices only (no CPU fallback); got a %s tensor" % t.device)


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _shape3(x):
    if x.dim() != 3:
        raise ValueError("expected a (N,T,C) tensor, got shape %s" % (tuple(x.shape),))
    return x.shape


def _band_call(fn_name, out, a, b, N, T, C, win, left, dil, ref):
    with _on_device(ref.device):
        check(getattr(_L, fn_name)(_p(out), _p(a), _p(b), N, T, C, win, left, dil, _dtype_code(ref), _stream(ref)),
              fn_name)
    return out


# ------------------------------------------------------------------ unfused pair
def qk_forward(q, k, win, left, dil=1):
    """attn (N,T,win) fp32 = banded q.k^T (na1d_tensorcore/nattn.py:34-44 forward)."""
    _need_cuda(q, k)
    assert q.is_contiguous() and k.is_contiguous() and q.dtype == k.dtype and q.shape == k.shape
    N, T, C = _shape3(q)
    attn = torch.empty((N, T, win), dtype=torch.float32, device=q.device)
    return _band_call("na1d_qk_forward", attn, q, k, N, T, C, win, left, dil, q)


def q_backward(attn_gd, k, win, left, dil=1):
    _need_cuda(attn_gd, k)
    assert attn_gd.is_contiguous() and k.is_contiguous() and attn_gd.dtype == torch.float32
    N, T, C = _shape3(k)
    assert attn_gd.shape == (N, T, win)
    return _band_call("na1d_q_backward", torch.empty_like(k), attn_gd, k, N, T, C, win, left, dil, k)


def k_backward(attn_gd, q, win, left, dil=1):
    _need_cuda(attn_gd, q)
    assert attn_gd.is_contiguous() and q.is_contiguous() and attn_gd.dtype == torch.float32
    N, T, C = _shape3(q)
    assert attn_gd.shape == (N, T, win)
    return _band_call("na1d_k_backward", torch.empty_like(q), attn_gd, q, N, T, C, win, left, dil, q)


def av_forward(attn, v, win, left, dil=1):
    _need_cuda(attn, v)
    assert attn.is_contiguous() and v.is_contiguous() and attn.dtype == torch.float32
    N, T, C = _shape3(v)
    assert attn.shape == (N, T, win)
    return _band_call("na1d_av_forward", torch.empty_like(v), attn, v, N, T, C, win, left, dil, v)


def a_backward(result_gd, v, win, left, dil=1):
    _need_cuda(result_gd, v)
    assert result_gd.is_contiguous() and v.is_contiguous() and result_gd.dtype == v.dtype
    N, T, C = _shape3(v)
    attn_gd = torch.empty((N, T, win), dtype=torch.float32, device=v.device)
    return _band_call("na1d_a_backward", attn_gd, result_gd, v, N, T, C, win, left, dil, v)


def v_backward(attn, result_gd, win, left, dil=1):
    _need_cuda(attn, result_gd)
    assert attn.is_contiguous() and result_gd.is_contiguous() and attn.dtype == torch.float32
    N, T, C = _shape3(result_gd)
    assert attn.shape == (N, T, win)
    return _band_call("na1d_v_backward", torch.empty_like(result_gd), attn, result_gd, N, T, C, win, left, dil, result_gd)


# ------------------------------------------------------------------ fused layer core
def _prep_rpb(rpb, heads, win, dev):
    if rpb is None:
        return None
    r = rpb.detach()
    if r.dtype != torch.float32 or r.device != dev:
        r = r.to(device=dev, dtype=torch.float32)
    return r.reshape(heads, win).contiguous()


class _on_device:
    """``torch.cuda.device(dev)`` only when ``dev`` is not already current (the context manager costs ~10 us per call)."""

    def __init__(self, dev):
        self.ctx = None if dev.index == torch.cuda.current_device() else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)


def _prep_valid(valid_len, batch, dev):
    if valid_len is None:
        return None
    v = torch.as_tensor(valid_len, device=dev).to(torch.int32).reshape(batch).contiguous()
    return v


def fused_forward(q, k, v, win, left, dil=1, scale=1.0, rpb=None, valid_len=None, heads=1, need_lse=True, drop_p=0.0, seed=0):
    """(o, lse): o (N,T,C) in q's dtype, lse (N,T) fp32. ``drop_p`` > 0 applies attention dropout with the mask that
    ``seed`` defines (tcgen05 shapes only)."""
    _need_cuda(q, k, v)
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    assert q.dtype == k.dtype == v.dtype and q.shape == k.shape == v.shape
    N, T, C = _shape3(q)
    o = torch.empty_like(q)
    lse = torch.empty((N, T), dtype=torch.float32, device=q.device) if need_lse else None
    r = _prep_rpb(rpb, heads, win, q.device)
    vl = _prep_valid(valid_len, N // max(heads, 1), q.device)
    with _on_device(q.device):
        if drop_p:
            check(_L.na1d_fused_forward_dropout(_p(o), _p(lse), _p(q), _p(k), _p(v), _p(r), _p(vl), N, heads, T, C, win, left,
                                                dil, float(scale), float(drop_p), int(seed), _dtype_code(q), _stream(q)),
                  "na1d_fused_forward_dropout")
        else:
            check(_L.na1d_fused_forward(_p(o), _p(lse), _p(q), _p(k), _p(v), _p(r), _p(vl), N, heads, T, C, win, left,
                                        dil, float(scale), _dtype_code(q), _stream(q)), "na1d_fused_forward")
    return o, lse


def fused_backward(d_o, q, k, v, o, lse, win, left, dil=1, scale=1.0, rpb=None, valid_len=None, heads=1,
                   need_d_rpb=False, drop_p=0.0, seed=0):
    """(dq, dk, dv, d_rpb or None). ``drop_p`` / ``seed`` must be those of the forward call."""
    _need_cuda(d_o, q, k, v, o, lse)
    d_o = d_o.contiguous()
    N, T, C = _shape3(q)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty((N, T), dtype=torch.float32, device=q.device)
    r = _prep_rpb(rpb, heads, win, q.device)
    vl = _prep_valid(valid_len, N // max(heads, 1), q.device)
    d_rpb = torch.zeros((heads, win), dtype=torch.float32, device=q.device) if need_d_rpb else None
    with _on_device(q.device):
        if drop_p:
            check(_L.na1d_fused_backward_dropout(_p(dq), _p(dk), _p(dv), _p(d_rpb), _p(d_o), _p(q), _p(k), _p(v), _p(lse), _p(r),
                                                 _p(vl), _p(delta), N * T, N, heads, T, C, win, left, dil, float(scale),
                                                 float(drop_p), int(seed), _dtype_code(q), _stream(q)),
                  "na1d_fused_backward_dropout")
        else:
            check(_L.na1d_fused_backward(_p(dq), _p(dk), _p(dv), _p(d_rpb), _p(d_o), _p(q), _p(k), _p(v), _p(o), _p(lse),
                                         _p(r), _p(vl), _p(delta), N, heads, T, C, win, left, dil, float(scale),
                                         _dtype_code(q), _stream(q)), "na1d_fused_backward")
    return dq, dk, dv, d_rpb


# ------------------------------------------------------------------ strided (layout-fused) forms
def _strides3(t, C):
    """{batch, head, token} element strides of a 4-D view addressed [batch][head][token][channel]."""
    if t.dim() != 4 or t.stride(3) != 1 or t.shape[3] != C:
        raise ValueError("expected a (batch, heads, T, C) view with unit channel stride, got shape %s strides %s"
                         % (tuple(t.shape), t.stride()))
    return (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def fused_forward_strided(q, k, v, o, win, left, dil=1, scale=1.0, rpb=None, valid_len=None, need_lse=True):
    """Fused forward on strided views: q, k, v, o are (batch, heads, T, C) VIEWS (any batch/head/token strides that are
    multiples of 8 elements, channel stride 1), e.g. the slices of a packed projection output and an output buffer laid
    out (batch, T, heads, C). Writes o in place and returns lse (batch*heads, T) fp32. Raises ``Na1dError`` with status
    -10 when the tcgen05 kernels cannot take the shape (the caller then makes dense copies)."""
    _need_cuda(q, k, v, o)
    B, H, T, C = q.shape
    assert k.shape == q.shape and v.shape == q.shape and o.shape == q.shape and q.dtype == k.dtype == v.dtype == o.dtype
    lse = torch.empty((B * H, T), dtype=torch.float32, device=q.device) if need_lse else None
    r = _prep_rpb(rpb, H, win, q.device)
    vl = _prep_valid(valid_len, B, q.device)
    with _on_device(q.device):
        check(_L.na1d_fused_forward_strided(_p(o), _p(lse), _p(q), _p(k), _p(v), _p(r), _p(vl), _strides3(o, C), _strides3(q, C),
                                            _strides3(k, C), _strides3(v, C), B * H, H, T, C, win, left, dil, float(scale),
                                            _dtype_code(q), _stream(q)), "na1d_fused_forward_strided")
    return lse


def fused_backward_strided(d_o, q, k, v, lse, dq, dk, dv, win, left, dil=1, scale=1.0, rpb=None, valid_len=None,
                           need_d_rpb=False):
    """Gradients on strided views (all (batch, heads, T, C) views); writes dq, dk, dv in place, returns d_rpb or None."""
    _need_cuda(d_o, q, k, v, lse, dq, dk, dv)
    B, H, T, C = q.shape
    r = _prep_rpb(rpb, H, win, q.device)
    vl = _prep_valid(valid_len, B, q.device)
    d_rpb = scratch = None
    n_scratch = 0
    if need_d_rpb:
        d_rpb = torch.zeros((H, win), dtype=torch.float32, device=q.device)
        n_scratch = 160 * H * win          # one partial row per CTA (one CTA per SM)
        scratch = torch.empty(n_scratch, dtype=torch.float32, device=q.device)
    with _on_device(q.device):
        check(_L.na1d_fused_backward_strided(_p(dq), _p(dk), _p(dv), _p(d_rpb), _p(d_o), _p(q), _p(k), _p(v), _p(lse), _p(r),
                                             _p(vl), _p(scratch), n_scratch, _strides3(dq, C), _strides3(dk, C),
                                             _strides3(dv, C), _strides3(d_o, C), _strides3(q, C), _strides3(k, C),
                                             _strides3(v, C), B * H, H, T, C, win, left, dil, float(scale), _dtype_code(q),
                                             _stream(q)), "na1d_fused_backward_strided")
    return d_rpb


class NA1dFusedPackedFunction(torch.autograd.Function):
    """The fused layer core on a PACKED projection output: ``qkv`` is (batch, T, 3*heads*C) as the channels-last ``qkv``
    projection writes it (models/MFA_NATransformer.py:127: viewed as (batch, T, 3, heads, C)), the result is
    (batch, T, heads*C) as the output projection reads it (:151-152). The head split, the head merge and their autograd
    copies do not exist: the kernels address q, k, v, o, d_o, dq, dk, dv through strided tensor maps. Saves (qkv, lse) only
    -- the tcgen05 backward needs neither o nor the probabilities."""

    @staticmethod
    def forward(ctx, qkv, heads, win_size, left, dilation=1, scale=1.0, rpb=None, valid_len=None):
        B, T, C3 = qkv.shape
        C = C3 // (3 * heads)
        qkv = qkv.contiguous()
        p = qkv.view(B, T, 3, heads, C)
        q, k, v = (p[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        out = torch.empty((B, T, heads * C), dtype=qkv.dtype, device=qkv.device)
        lse = fused_forward_strided(q, k, v, out.view(B, T, heads, C).permute(0, 2, 1, 3), win_size, left, dilation, scale, rpb,
                                    valid_len)
        ctx.save_for_backward(qkv, lse, rpb if rpb is not None else torch.empty(0),
                              valid_len if isinstance(valid_len, torch.Tensor) else torch.empty(0))
        ctx.cfg = (heads, win_size, left, dilation, scale, rpb is not None,
                   valid_len if not isinstance(valid_len, torch.Tensor) else "tensor")
        return out

    @staticmethod
    def backward(ctx, d_out):
        qkv, lse, rpb, vl_t = ctx.saved_tensors
        heads, win, left, dil, scale, has_rpb, vl = ctx.cfg
        valid_len = vl_t if vl == "tensor" else vl
        B, T, C3 = qkv.shape
        C = C3 // (3 * heads)
        p = qkv.view(B, T, 3, heads, C)
        q, k, v = (p[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        d_qkv = torch.empty_like(qkv)
        g = d_qkv.view(B, T, 3, heads, C)
        dq, dk, dv = (g[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        d_o = d_out.contiguous().view(B, T, heads, C).permute(0, 2, 1, 3)
        need_rpb = has_rpb and ctx.needs_input_grad[6]
        d_rpb = fused_backward_strided(d_o, q, k, v, lse, dq, dk, dv, win, left, dil, scale, rpb if has_rpb else None, valid_len,
                                       need_d_rpb=need_rpb)
        if d_rpb is not None:
            d_rpb = d_rpb.reshape(rpb.shape).to(rpb.dtype)
        return d_qkv, None, None, None, None, None, d_rpb, None


def na1d_fused_packed(qkv, heads, win_size, left, dilation=1, scale=1.0, rpb=None, valid_len=None):
    """``(batch, T, 3*heads*C)`` packed projection output -> ``(batch, T, heads*C)`` attention output, no layout copies."""
    return NA1dFusedPackedFunction.apply(qkv, int(heads), int(win_size), int(left), int(dilation), float(scale), rpb, valid_len)


def packed_supported(heads, T, C, win, left, dil, dtype, has_bias=True, wants_bias_grad=True):
    """Whether ``na1d_fused_packed`` can take this shape, forward and backward (host-only query of the library)."""
    if dtype not in (torch.bfloat16, torch.float16):
        return False
    code = _lib.NA1D_BF16 if dtype == torch.bfloat16 else _lib.NA1D_FP16
    return _L.na1d_fused_strided_supported(heads, T, C, win, left, dil, code, int(has_bias), int(wants_bias_grad)) == 1


class NA1dFusedFunction(torch.autograd.Function):
    """o = softmax(scale*q.k^T + rpb + mask) . v over each query's window, as one op.

    Fuses models/PCF_NATransformer.py:141-150 (QK -> +bias -> +mask -> softmax -> AV); saves
    (q,k,v,o,lse) instead of the fp32 (N,T,win) probabilities the unfused pair keeps
    (na1d_tensorcore/nattn.py:41, :65).
    """

    @staticmethod
    def forward(ctx, q, k, v, win_size, left, dilation=1, scale=1.0, rpb=None, valid_len=None, heads=1, drop_p=0.0, seed=0):
        o, lse = fused_forward(q, k, v, win_size, left, dilation, scale, rpb, valid_len, heads, drop_p=drop_p, seed=seed)
        ctx.save_for_backward(q, k, v, o, lse, rpb if rpb is not None else torch.empty(0),
                              valid_len if isinstance(valid_len, torch.Tensor) else torch.empty(0))
        ctx.cfg = (win_size, left, dilation, scale, heads, rpb is not None,
                   valid_len if not isinstance(valid_len, torch.Tensor) else "tensor")
        ctx.drop = (drop_p, seed)
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse, rpb, vl_t = ctx.saved_tensors
        win, left, dil, scale, heads, has_rpb, vl = ctx.cfg
        valid_len = vl_t if vl == "tensor" else vl
        need_rpb = has_rpb and ctx.needs_input_grad[7]
        dq, dk, dv, d_rpb = fused_backward(d_o, q, k, v, o, lse, win, left, dil, scale, rpb if has_rpb else None,
                                           valid_len, heads, need_d_rpb=need_rpb, drop_p=ctx.drop[0], seed=ctx.drop[1])
        if d_rpb is not None:
            d_rpb = d_rpb.reshape(rpb.shape).to(rpb.dtype)
        return dq, dk, dv, None, None, None, None, d_rpb, None, None, None, None


def na1d_fused(q, k, v, win_size, left, dilation=1, scale=1.0, rpb=None, valid_len=None, heads=1, drop_p=0.0, seed=0):
    return NA1dFusedFunction.apply(q, k, v, win_size, left, dilation, scale, rpb, valid_len, heads, drop_p, seed)


def dropout_supported(heads, T, C, win, dil):
    """Whether the fused pair with attention dropout can take this shape (the tcgen05 kernels on the flat tiling, with room
    for a bias table and its gradient in the backward)."""
    weff = (win - 1) * dil + 1
    return C in (16, 32, 64) and dil & (dil - 1) == 0 and weff <= 33 and T >= 32 and heads <= 32 and not (C == 64 and weff > 17)


def dropout_keep_mask(rows, win, drop_p, seed):
    """The keep decisions of the dropout kernels as a (rows, win) bool tensor, computed on the host by the library."""
    import numpy as np
    buf = np.empty((rows, win), dtype=np.uint8)
    check(_L.na1d_dropout_keep_mask(buf.ctypes.data_as(ctypes.c_void_p), rows, win, float(drop_p), int(seed)), "na1d_dropout_keep_mask")
    return torch.from_numpy(buf.astype(bool))


def window_index(T, win, left, dil=1, device="cuda"):
    """(j, in_range) exactly as the kernels compute them: int32 (T,win) and bool (T,win)."""
    dev = torch.device(device)
    j = torch.empty((T, win), dtype=torch.int32, device=dev)
    inr = torch.empty((T, win), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        check(_L.na1d_window_index(_p(j), _p(inr), T, win, left, dil, _stream(j)), "na1d_window_index")
    return j, inr.bool()


FAMILY_AUTO, FAMILY_CUDA_CORE, FAMILY_TCGEN05, FAMILY_TCGEN05_SEGMENTED = -1, 0, 1, 2


def set_kernel_family(family):
    """Force the kernel family of the fused entry points (tests/benchmarks); returns the old setting."""
    return _L.na1d_set_kernel_family(int(family))


def kernel_family(N, T, C, win, left, dil, dtype, backward=False):
    """0 = CUDA-core kernels, 1 = tcgen05/TMA kernels, negative = status code (forced family unsupported)."""
    code = _lib.NA1D_BF16 if dtype == torch.bfloat16 else _lib.NA1D_FP16
    return _L.na1d_fused_kernel_family(N, T, C, win, left, dil, code, 1 if backward else 0)


def kernel_tiling(N, T, C, win, left, dil, dtype, backward=False):
    """0 = CUDA-core kernels, 1 = tcgen05 on the flat tiling, 2 = tcgen05 on the segmented tiling, negative = status code."""
    code = _lib.NA1D_BF16 if dtype == torch.bfloat16 else _lib.NA1D_FP16
    return _L.na1d_fused_kernel_tiling(N, T, C, win, left, dil, code, 1 if backward else 0)


def tensor_map_cache_stats():
    """(hits, misses) of the library's cache of encoded TMA tensor maps."""
    h, m = ctypes.c_int64(0), ctypes.c_int64(0)
    check(_L.na1d_tensor_map_cache_stats(ctypes.byref(h), ctypes.byref(m)), "na1d_tensor_map_cache_stats")
    return h.value, m.value


def device_status():
    """Synchronise and raise if a bounded wait inside a kernel expired."""
    check(_L.na1d_device_status(), "na1d_device_status")

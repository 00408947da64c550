"""The neighbourhood-attention layer as a packaged module on the fused operator.

``NAttention`` has the constructor, parameter names and state-dict layout of the reference's two layer classes

* ``models/PCF_NATransformer.py:44-178``  -- input ``(N, C, T)``, 1x1 ``Conv1d`` projections with ``groups``
  (``layout="channels_first"``),
* ``models/MFA_NATransformer.py:44-177``  -- input ``(N, T, C)``, ``Linear`` projections (``layout="channels_last"``),

so a checkpoint of either loads unchanged (keys ``qkv.*``, ``proj.*``, ``relative_position_bias``, ``attn_mask``).
Between the two projections the reference runs ``q*scale -> QK -> +rpb -> +mask -> softmax -> dropout -> AV`` as seven or
more kernels with an fp32 ``(N*heads, T, win)`` tensor in HBM (PCF_NATransformer.py:141-150); here that is one call of
``na1d_fused`` and the padding mask is computed inside the kernel from ``valid_len = T - padding``.

``fuse_nattention(model)`` rebinds ``forward`` of the reference's own layer objects inside an already built model to the
same fused path, for hosts that construct the unmodified reference model classes.
"""
import types

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .library_op import na1d_fused


def _window(win_size):
    """(win, left) from the reference's ``win_size`` argument: an int (``left = win-1-win//2``, so an even window has its
    extra key on the right) or ``[win, left]`` (PCF_NATransformer.py:47-54)."""
    if isinstance(win_size, int):
        if win_size <= 0:
            raise ValueError("win_size must be positive")
        return win_size, win_size - 1 - win_size // 2
    if isinstance(win_size, (list, tuple)) and len(win_size) == 2:
        win, left = int(win_size[0]), int(win_size[1])
        if not (0 <= left < win):
            raise ValueError("left must satisfy 0 <= left < win_size")
        return win, left
    raise ValueError("win_size must be an int or [win_size, left]")


def padding_mask(T, win, left, dilation=1, padding=None, dtype=torch.float32, device="cpu"):
    """The reference's additive mask (PCF_NATransformer.py:87-116): 0 where query t and key t+(kk-left)*dilation are both
    real frames of the utterance, -100 elsewhere; shape ``(N, 1, T, win)``. Only kept for state-dict compatibility
    (buffer ``attn_mask``) and for tests: the fused kernels derive the same mask from ``valid_len``."""
    if padding is None:
        padding = torch.zeros(1, dtype=torch.int, device=device)
    valid = (T - padding.to(torch.int64)).view(-1, 1, 1)                                   # (N,1,1)
    t = torch.arange(T, device=padding.device).view(1, T, 1)
    j = t + (torch.arange(win, device=padding.device).view(1, 1, win) - left) * dilation
    bad = (t >= valid) | (j < 0) | (j >= valid)
    mask = torch.zeros(bad.shape, dtype=dtype, device=padding.device).masked_fill(bad, -100.0)
    return mask.unsqueeze(1)


def _split_heads(x, layout, num_heads, groups):
    """Projection output -> q, k, v as ``(N*heads, T, head_dim)`` (the copies of PCF_NATransformer.py:126-138 and
    MFA_NATransformer.py:127-137)."""
    if layout == "channels_first":
        N, C3, T = x.shape
        C = C3 // 3
        hd = C // num_heads
        x = x.view(N, C // groups, groups, 3, T).transpose(1, 2).contiguous().view(N, num_heads, hd, 3, T)
        x = x.permute(3, 0, 1, 4, 2).contiguous().view(3, N * num_heads, T, hd)
    else:
        N, T, C3 = x.shape
        C = C3 // 3
        hd = C // num_heads
        x = x.view(N, T, 3, num_heads, hd).permute(2, 0, 3, 1, 4).contiguous().view(3, N * num_heads, T, hd)
    return x[0], x[1], x[2]


def _merge_heads(o, layout, N, num_heads):
    NH, T, hd = o.shape
    o = o.view(N, num_heads, T, hd)
    if layout == "channels_first":
        return o.transpose(2, 3).contiguous().view(N, num_heads * hd, T)
    return o.transpose(1, 2).contiguous().view(N, T, num_heads * hd)


def _dense_1x1(conv, groups):
    """The grouped 1x1 convolution's weight as a dense (out, in) matrix (block diagonal: group g maps input block g to
    output block g). At these sizes (256 channels) the tensor cores make the zeros free, and a dense matrix lets the
    channel shuffle of the head split be folded into a row permutation."""
    w = conv.weight.squeeze(-1)                                   # (out, in / groups)
    if groups == 1:
        return w
    return torch.block_diag(*w.view(groups, w.shape[0] // groups, w.shape[1]))


def _packed_row_order(C, num_heads, groups, device):
    """Row permutation that turns the qkv convolution's output channels into the packed (3, heads, head_dim) order.
    The reference views the 3C output channels as (C/groups, groups, 3), swaps the first two axes and reads the result as
    (heads, head_dim, 3) (PCF_NATransformer.py:127-129): output channel (c*groups + g)*3 + which is element
    g*(C/groups) + c = head*head_dim + d of tensor `which`."""
    P = C // groups
    f = torch.arange(C, device=device)
    ch = ((f % P) * groups + f // P) * 3                          # channel of q element f; k and v follow at +1, +2
    return torch.cat([ch, ch + 1, ch + 2])


def _fused_forward_channels_first_packed(self, x, valid_len):
    """The channels-first (PCF) layer on the packed route. The operator's operands need channel-contiguous rows, the network
    around the layer is (batch, C, T): the layout changes once on the C-channel input and once on the output; in between,
    both 1x1 convolutions are single GEMMs over all batch*T tokens (dense block-diagonal weights), the qkv rows permuted so
    that the result IS the packed (batch, T, 3, heads, head_dim) tensor the kernels read through strided tensor maps. The
    reference's copies of the 3C-channel projection output (channel shuffle, head split: PCF_NATransformer.py:127-138), of
    the merged heads (:151) and their autograd twins are gone, and so are the grouped convolutions. Measured at the
    reference's layer shape (512 x 150 frames, dim 256, 16 heads, window 27, groups 8; bf16 autocast, forward+backward):
    1.86 ms against 3.42 ms with convolutions and head split / merge copies around the dense operator (3.07 ms when the
    transposes are instead absorbed by batched GEMMs on strided views: 512 small GEMMs and a batch-sized weight gradient)."""
    N, C, T = x.shape
    g = getattr(self, "groups", 1)
    order = _packed_row_order(C, self.num_heads, g, x.device)
    xt = x.transpose(1, 2).contiguous()                            # (N, T, C)
    qkv = F.linear(xt, _dense_1x1(self.qkv, g)[order], None if self.qkv.bias is None else self.qkv.bias[order])
    o = ops.na1d_fused_packed(qkv, self.num_heads, self.win_size, self.left, self.dilation, float(self.scale),
                              self.relative_position_bias, valid_len)                           # (N, T, C)
    y = F.linear(o, _dense_1x1(self.proj, g), self.proj.bias)
    return self.proj_drop(y.transpose(1, 2).contiguous())


def _fused_forward(self, x, padding=None):
    layout = self._na1d_layout
    if layout == "channels_first":
        N, C, T = x.shape
    else:
        N, T, C = x.shape
    drop_p = float(self.attn_drop.p) if self.training else 0.0
    seed = 0
    if drop_p:
        # attention dropout (PCF_NATransformer.py:149) inside the fused kernels: the mask is a hash of a per-call seed drawn
        # from torch's CPU generator (reproducible under torch.manual_seed; no device synchronisation)
        if not ops.dropout_supported(self.num_heads, T, C // self.num_heads, self.win_size, self.dilation):
            raise NotImplementedError("attention dropout > 0 is fused for head dims 16/32/64, power-of-two dilation and a dilated "
                                      "window of at most 33 (17 at head dim 64) only")
        seed = int(torch.randint(0, 2 ** 62, (1,)).item())
    valid_len = None
    if not self.training and padding is not None:
        # eval: the mask follows the utterance's padding (PCF_NATransformer.py:131-134); training uses the constant mask
        valid_len = (T - padding.to(torch.int64)).clamp_(0, T).to(torch.int32).expand(N).contiguous()
    hd = C // self.num_heads
    if layout == "channels_first" and not drop_p and type(x) is torch.Tensor and x.is_cuda and not torch.compiler.is_compiling():
        # the dtype the projections will produce: the input's own 16-bit type, or autocast's
        dt = x.dtype if x.dtype in (torch.bfloat16, torch.float16) else (
            torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled() else None)
        if dt in (torch.bfloat16, torch.float16) and ops.packed_supported(self.num_heads, T, hd, self.win_size, self.left,
                                                                         self.dilation, dt):
            return _fused_forward_channels_first_packed(self, x, valid_len)
    qkv = self.qkv(x)
    if (layout == "channels_last" and not drop_p and type(qkv) is torch.Tensor and qkv.is_cuda and not torch.compiler.is_compiling() and
            ops.packed_supported(self.num_heads, T, hd, self.win_size, self.left, self.dilation, qkv.dtype)):
        # the kernels read q, k, v straight out of the packed projection output and write the output in the layout
        # `proj` consumes: no head split / merge copies (MFA_NATransformer.py:127-137, :151-152), forward or backward
        o = ops.na1d_fused_packed(qkv, self.num_heads, self.win_size, self.left, self.dilation, float(self.scale),
                                  self.relative_position_bias, valid_len)
        return self.proj_drop(self.proj(o))
    q, k, v = _split_heads(qkv, layout, self.num_heads, getattr(self, "groups", 1))
    o = na1d_fused(q, k, v, self.win_size, self.left, self.dilation, float(self.scale), self.relative_position_bias,
                   valid_len, self.num_heads, drop_p, seed)
    return self.proj_drop(self.proj(_merge_heads(o, layout, N, self.num_heads)))


class NAttention(nn.Module):
    """Drop-in for the reference's ``NAttention`` (same arguments; ``layout`` picks the PCF or the MFA variant)."""

    def __init__(self, frames, dim, num_heads, win_size, dilation=1, groups=1, proj_bias=True, qkv_bias=True, qk_scale=None,
                 attn_drop=0., proj_drop=0., dtype=torch.float32, layout="channels_first"):
        super().__init__()
        if layout not in ("channels_first", "channels_last"):
            raise ValueError("layout must be 'channels_first' (PCF) or 'channels_last' (MFA)")
        self.win_size, self.left = _window(win_size)
        if self.win_size > 80:
            raise ValueError("win_size <= 80 (PCF_NATransformer.py:53)")
        head_dim = dim // num_heads
        if dim % num_heads or head_dim % 8:
            raise ValueError("dim must split into heads of a multiple of 8 channels")
        self.dim, self.dilation, self.groups, self.num_heads = dim, dilation, groups, num_heads
        self.scale = qk_scale or head_dim ** -0.5
        self._na1d_layout = layout
        if layout == "channels_first":
            self.qkv = nn.Conv1d(dim, dim * 3, kernel_size=1, bias=qkv_bias, groups=groups)
            self.proj = nn.Conv1d(dim, dim, kernel_size=1, bias=proj_bias, groups=groups)
        else:
            if groups != 1:
                raise ValueError("groups is a channels_first (PCF) option")
            self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
            self.proj = nn.Linear(dim, dim, bias=proj_bias)
        self.relative_position_bias = nn.Parameter(torch.zeros((1, num_heads, 1, self.win_size)))
        nn.init.normal_(self.relative_position_bias, mean=0., std=.02)
        self.attn_drop = nn.Dropout(attn_drop)
        self.proj_drop = nn.Dropout(proj_drop)
        self.register_buffer("attn_mask", padding_mask(frames, self.win_size, self.left, dilation))

    forward = _fused_forward


def global_padding_mask(T, padding=None, dtype=torch.float32, device="cpu"):
    """The additive mask of the dense layers (PCF_NATransformer.py:406-414): -100 where the query or the key is a padded
    frame, 0 elsewhere; shape ``(N, 1, T, T)``."""
    if padding is None:
        padding = torch.zeros(1, dtype=torch.int, device=device)
    bad = torch.arange(T, device=padding.device).unsqueeze(0) >= (T - padding.unsqueeze(1))     # (N, T)
    both = bad.unsqueeze(-1) | bad.unsqueeze(-2)
    return torch.zeros(both.shape, device=padding.device, dtype=dtype).masked_fill(both, -100.0).unsqueeze(1)


def _global_forward(self, x, pos_emb, attn_mask=None):
    N, C, T = x.shape
    x = x + self.linear_pos(pos_emb)
    q, k, v = _split_heads(self.qkv(x), "channels_first", self.num_heads, self.groups)
    hd = C // self.num_heads
    q, k, v = (t.view(N, self.num_heads, T, hd) for t in (q, k, v))
    mask = None if attn_mask is None else attn_mask.to(q.dtype)
    drop = float(self.attn_drop.p) if self.training else 0.0
    o = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=drop, scale=float(self.scale))
    return self.proj_drop(self.proj(_merge_heads(o.reshape(N * self.num_heads, T, hd), "channels_first", N, self.num_heads)))


class GlobalAttention(nn.Module):
    """Drop-in for the reference's dense attention layer (``win_size == 0`` layers; PCF_NATransformer.py:181-225): same
    arguments, parameter names and state-dict layout (``linear_pos``, ``qkv``, ``proj``). The ``(N, heads, T, T)`` logits,
    their softmax and the dropout of the reference (:212-221) run as one fused attention call of the framework
    (``scaled_dot_product_attention``) instead of four kernels with a ``T x T`` fp32 tensor per head in HBM."""

    def __init__(self, dim, num_heads, groups=1, proj_bias=True, qkv_bias=True, qk_scale=None, attn_drop=0., proj_drop=0.):
        super().__init__()
        self.dim, self.num_heads, self.groups = dim, num_heads, groups
        self.scale = qk_scale or (dim // num_heads) ** -0.5
        self.linear_pos = nn.Conv1d(dim, dim, kernel_size=1, bias=False, groups=groups)
        self.qkv = nn.Conv1d(dim, dim * 3, kernel_size=1, bias=qkv_bias, groups=groups)
        self.attn_drop = nn.Dropout(attn_drop)
        self.proj = nn.Conv1d(dim, dim, kernel_size=1, bias=proj_bias, groups=groups)
        self.proj_drop = nn.Dropout(proj_drop)

    forward = _global_forward


def fuse_nattention(model, layout=None):
    """Rebind ``forward`` of every reference-style attention layer inside ``model`` to the fused path.

    A layer qualifies when it has ``qkv``, ``proj``, ``relative_position_bias``, ``win_size``, ``left``, ``num_heads`` and
    ``attn_drop``; its layout is taken from the type of ``qkv`` (``Conv1d`` -> channels_first) unless given.
    Returns the number of layers rebound."""
    n = 0
    for m in model.modules():
        if isinstance(m, (NAttention, GlobalAttention)):
            continue
        if all(hasattr(m, a) for a in ("qkv", "proj", "relative_position_bias", "win_size", "left", "num_heads", "attn_drop",
                                       "proj_drop", "scale", "dilation")):
            m._na1d_layout = layout or ("channels_first" if isinstance(m.qkv, nn.Conv1d) else "channels_last")
            m.forward = types.MethodType(_fused_forward, m)
            n += 1
        elif all(hasattr(m, a) for a in ("linear_pos", "qkv", "proj", "num_heads", "groups", "attn_drop", "proj_drop", "scale")):
            m.forward = types.MethodType(_global_forward, m)   # the reference's GlobalAttention
            n += 1
    return n

"""CPU oracle for 1-D neighbourhood attention (NA1D). TEST INFRASTRUCTURE ONLY.

This file restates, in plain fp32 PyTorch on the CPU, the arithmetic that the
reference executes for one neighbourhood-attention layer. It is the checker the
test-suite, the smoke test and the CPU-baseline leg of the benchmark compare the
CUDA kernels against; the product path never imports it.

Parity status: the reference ships no golden vectors or known-answer tests for this
path, so the oracle is pinned against outputs of the reference itself instead:
``tests/golden/make_golden.py`` imports the reference's own CPU branch of
``NAttention.forward`` (models/PCF_NATransformer.py:153-174 and
models/MFA_NATransformer.py:152-173), runs it on seeded inputs and commits the
results; ``tests/test_oracle_golden.py`` holds this file to those vectors.

Semantics restated here (reference file:line, paths inside the reference project):

* window geometry -- ``left = win-1-win//2`` for an integer window, or an explicit
  ``[win, left]`` pair (models/PCF_NATransformer.py:47-56); neighbour ``kk`` of query
  ``t`` is key ``j = t + (kk-left)*dilation`` (pad/unfold at :161-165, nn.Unfold with
  dilation at :158-159).
* keys/values outside ``[0,T)`` are read as zero rows (F.pad value=0 at :159,:161;
  CUDA: na1d_tensorcore/bf16_ana1d_kernel.cu:99-112).
* logits = (q*scale)·k + relative_position_bias[h,kk] + mask (:141-145 / :163-164),
  mask = -100 where the key is out of range, or key >= T-padding[b], or
  query >= T-padding[b] (get_attn_mask :87-99, get_attn_mask_dilation :101-116).
* softmax over the window in fp32 (:148 / :165), then probabilities · values
  (:150 / :171).
* the unfused pair the CUDA extension exposes (na1d_tensorcore/nattn.py:32-78):
  ``qk`` = banded Q·K^T with zero padded keys, ``av`` = banded A·V; their gradients
  follow from autograd through these same functions.
"""
from __future__ import annotations

import torch

__all__ = [
    "window_left",
    "neighbour_index",
    "attn_mask",
    "na1d_qk",
    "na1d_av",
    "na1d_logits",
    "na1d_fused",
    "na1d_fused_with_grads",
    "dropout_keep",
]


def window_left(win_size):
    """(win, left) from the reference's constructor argument.

    models/PCF_NATransformer.py:47-56: an int means a centred window with
    ``left = win-1-win//2``; a two-element list is ``[win, left]``.
    """
    if isinstance(win_size, int):
        win, left = win_size, win_size - 1 - win_size // 2
    else:
        win, left = int(win_size[0]), int(win_size[1])
    assert win > 0 and 0 <= left < win
    return win, left


def neighbour_index(T: int, win: int, left: int, dilation: int = 1):
    """Integer contract of the window: returns (j, in_range).

    ``j[t,kk] = t + (kk-left)*dilation`` (int64, shape (T,win)) and
    ``in_range = (0 <= j < T)``. This is the index arithmetic the pad+unfold of
    models/PCF_NATransformer.py:158-165 performs implicitly; the CUDA kernels must
    reproduce it bit for bit.
    """
    t = torch.arange(T, dtype=torch.int64).unsqueeze(1)
    kk = torch.arange(win, dtype=torch.int64).unsqueeze(0)
    j = t + (kk - left) * dilation
    return j, (j >= 0) & (j < T)


def _gather_rows(x: torch.Tensor, j: torch.Tensor, in_range: torch.Tensor) -> torch.Tensor:
    """x: (N,T,C) -> (N,T,win,C) with zero rows where the neighbour is out of range."""
    N, T, C = x.shape
    jc = j.clamp(0, T - 1)
    g = x[:, jc.reshape(-1), :].reshape(N, T, j.shape[1], C)
    return g * in_range.to(x.dtype).reshape(1, T, j.shape[1], 1)


def attn_mask(T: int, win: int, left: int, dilation: int, valid_len, batch: int) -> torch.Tensor:
    """Additive 0/-100 mask of shape (batch, T, win), fp32.

    Restates get_attn_mask / get_attn_mask_dilation
    (models/PCF_NATransformer.py:87-116) with ``valid_len = T - padding``.
    ``valid_len`` None means no padding (the training-time constant mask, :77-83).
    """
    j, inr = neighbour_index(T, win, left, dilation)
    if valid_len is None:
        vl = torch.full((batch,), T, dtype=torch.int64)
    else:
        vl = torch.as_tensor(valid_len, dtype=torch.int64).reshape(batch)
    t = torch.arange(T, dtype=torch.int64)
    row_bad = t.reshape(1, T, 1) >= vl.reshape(batch, 1, 1)
    col_bad = (~inr).unsqueeze(0) | (j.unsqueeze(0) >= vl.reshape(batch, 1, 1))
    bad = row_bad | col_bad
    return torch.zeros(batch, T, win, dtype=torch.float32).masked_fill(bad, -100.0)


def na1d_qk(q: torch.Tensor, k: torch.Tensor, win: int, left: int, dilation: int = 1) -> torch.Tensor:
    """Banded Q·K^T: attn[n,t,kk] = sum_c q[n,t,c]*k[n,j(t,kk),c], zero-padded keys.

    The forward of the reference's QK function (na1d_tensorcore/nattn.py:34-44,
    kernel bf16_ana1d_kernel.cu:42-163). fp32 in, fp32 out.
    """
    N, T, C = q.shape
    j, inr = neighbour_index(T, win, left, dilation)
    kg = _gather_rows(k, j, inr)
    return torch.einsum("ntc,ntwc->ntw", q, kg)


def na1d_av(attn: torch.Tensor, v: torch.Tensor, win: int, left: int, dilation: int = 1) -> torch.Tensor:
    """Banded A·V: out[n,t,c] = sum_kk attn[n,t,kk]*v[n,j(t,kk),c], zero-padded values.

    The forward of the reference's AV function (na1d_tensorcore/nattn.py:58-67,
    kernel bf16_ana1d_kernel.cu:285-391).
    """
    N, T, C = v.shape
    j, inr = neighbour_index(T, win, left, dilation)
    vg = _gather_rows(v, j, inr)
    return torch.einsum("ntw,ntwc->ntc", attn, vg)


def na1d_logits(q, k, win, left, dilation=1, scale=1.0, rpb=None, valid_len=None, heads=1):
    """Pre-softmax logits (N,T,win): scale*QK + rpb[h] + mask.

    ``N = batch*heads`` with the head index fastest (n = b*heads + h), as produced by
    the head split at models/PCF_NATransformer.py:137-138. ``rpb`` is (heads, win).
    """
    N, T, C = q.shape
    assert N % heads == 0
    batch = N // heads
    s = na1d_qk(q * scale, k, win, left, dilation)
    if rpb is not None:
        s = (s.reshape(batch, heads, T, win) + rpb.reshape(1, heads, 1, win)).reshape(N, T, win)
    m = attn_mask(T, win, left, dilation, valid_len, batch)
    s = (s.reshape(batch, heads, T, win) + m.reshape(batch, 1, T, win)).reshape(N, T, win)
    return s


def dropout_keep(rows: int, win: int, drop_p: float, seed: int) -> torch.Tensor:
    """Keep mask (rows, win), bool, of the attention dropout as the CUDA kernels derive it.

    The reference applies ``nn.Dropout`` to the probabilities (models/PCF_NATransformer.py:149), drawing from torch's
    random stream; a fused kernel cannot replay that stream, so the library defines the mask as a hash of
    (seed, dense row index n*T+t, neighbour index kk) -- restated here in 32-bit integer arithmetic: keep iff
    fmix32(row*2654435761 + kk*0x632BE5AB + seed32) >= floor(p * 2^32), with seed32 = low ^ high half of the 64-bit seed and
    fmix32 the usual xor-shift / multiply finaliser.
    """
    import numpy as np
    m = np.uint64(0xFFFFFFFF)
    seed32 = np.uint64((seed ^ (seed >> 32)) & 0xFFFFFFFF)
    row = np.arange(rows, dtype=np.uint64)[:, None]
    kk = np.arange(win, dtype=np.uint64)[None, :]
    x = (row * np.uint64(2654435761) + kk * np.uint64(0x632BE5AB) + seed32) & m
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(0x85EBCA6B)) & m
    x ^= x >> np.uint64(13)
    x = (x * np.uint64(0xC2B2AE35)) & m
    x ^= x >> np.uint64(16)
    th = min(int(float(np.float32(drop_p)) * 4294967296.0), 4294967295)
    return torch.from_numpy(x >= np.uint64(th))


def na1d_fused(q, k, v, win, left, dilation=1, scale=1.0, rpb=None, valid_len=None, heads=1,
               return_lse=False, drop_p=0.0, seed=0):
    """Whole layer core: logits -> softmax -> (dropout) -> weighted sum. fp32, (N,T,C) -> (N,T,C).

    Restates models/PCF_NATransformer.py:141-150 (CUDA branch) == :156-171 (CPU branch).
    """
    s = na1d_logits(q, k, win, left, dilation, scale, rpb, valid_len, heads)
    p = torch.softmax(s, dim=-1)
    if drop_p > 0:
        N, T, _ = q.shape
        keep = dropout_keep(N * T, win, drop_p, seed).reshape(N, T, win)
        p = p * keep.to(p.dtype) / (1.0 - float(torch.tensor(drop_p, dtype=torch.float32)))
    o = na1d_av(p, v, win, left, dilation)
    if return_lse:
        return o, torch.logsumexp(s, dim=-1)
    return o


def na1d_fused_with_grads(q, k, v, d_out, win, left, dilation=1, scale=1.0, rpb=None,
                          valid_len=None, heads=1, drop_p=0.0, seed=0):
    """Forward plus autograd gradients (dq, dk, dv, drpb-or-None) of ``na1d_fused``."""
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    r = None
    if rpb is not None:
        r = rpb.detach().clone().requires_grad_(True)
    o = na1d_fused(q, k, v, win, left, dilation, scale, r, valid_len, heads, drop_p=drop_p, seed=seed)
    o.backward(d_out)
    return o.detach(), q.grad, k.grad, v.grad, (r.grad if r is not None else None)

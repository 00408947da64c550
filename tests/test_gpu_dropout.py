"""GPU parity of the fused pair with attention dropout, through the C ABI: the kernels' mask is a hash the oracle restates
bit for bit, so outputs and gradients are compared exactly like the no-dropout path."""
import pytest
import torch

from gpu_util import assert_close, randn16
from oracle import na1d_oracle as orc

pytestmark = pytest.mark.gpu
DTYPES = [torch.bfloat16, torch.float16]

# (N, H, T, C, win, left, dil, p): all three window buckets, dilation, several tiles per CTA, padded utterances
DROP_SHAPES = [
    (8, 2, 200, 32, 7, 3, 1, 0.1), (6, 3, 150, 16, 27, 13, 1, 0.25), (4, 2, 129, 64, 7, 3, 2, 0.5), (4, 1, 300, 64, 15, 7, 1, 0.1),
    (512, 4, 200, 64, 7, 3, 1, 0.2), (12, 4, 50, 32, 5, 0, 4, 0.3),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "fp16"])
def test_dropout_forward_backward_match_oracle(dtype):
    from pcf_nat_b200 import ops
    for idx, (N, H, T, C, win, left, dil, p) in enumerate(DROP_SHAPES):
        tag = "N=%d H=%d T=%d C=%d win=%d dil=%d p=%.2f " % (N, H, T, C, win, dil, p)
        seed = 1000003 * (idx + 1) + (1 << 35)
        sc = C ** -0.5
        q, k, v, d_o = (randn16((N, T, C), dtype, 4000 + 4 * idx + i) for i in range(4))
        rpb = 0.3 * torch.randn(H, win, generator=torch.Generator().manual_seed(idx))
        vl = [T] + [max(1, T - 9)] * (N // H - 1)
        o, lse = ops.fused_forward(q.cuda(), k.cuda(), v.cuda(), win, left, dil, sc, rpb.cuda(), vl, H, drop_p=p, seed=seed)
        dq, dk, dv, drpb = ops.fused_backward(d_o.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, win, left, dil, sc, rpb.cuda(), vl, H,
                                              need_d_rpb=True, drop_p=p, seed=seed)
        ops.device_status()
        o_r, dq_r, dk_r, dv_r, drpb_r = orc.na1d_fused_with_grads(q.float(), k.float(), v.float(), d_o.float(), win, left, dil, sc,
                                                                  rpb, vl, H, drop_p=p, seed=seed)
        _, lse_r = orc.na1d_fused(q.float(), k.float(), v.float(), win, left, dil, sc, rpb, vl, H, return_lse=True)
        # the kept probabilities are scaled by 1/(1-p): outputs and gradients grow accordingly, and so does the tolerance
        f = 1.0 / (1.0 - p)
        assert_close(o, o_r, dtype, tag + "o", factor=f)
        assert float((lse.cpu() - lse_r).abs().max()) < 1e-3 * max(1.0, float(lse_r.abs().max())), tag + "lse is that of the undropped logits"
        assert_close(dq, dq_r, dtype, tag + "dq", factor=f)
        assert_close(dk, dk_r, dtype, tag + "dk", factor=f)
        assert_close(dv, dv_r, dtype, tag + "dv", factor=f)
        assert_close(drpb, drpb_r, dtype, tag + "drpb", factor=2.0 * f)
        # another seed gives another mask; the same seed the same bits
        o2, _ = ops.fused_forward(q.cuda(), k.cuda(), v.cuda(), win, left, dil, sc, rpb.cuda(), vl, H, drop_p=p, seed=seed)
        o3, _ = ops.fused_forward(q.cuda(), k.cuda(), v.cuda(), win, left, dil, sc, rpb.cuda(), vl, H, drop_p=p, seed=seed + 1)
        assert torch.equal(o, o2) and not torch.equal(o, o3), tag


def test_dropout_layer_trains_and_evaluates():
    """NAttention with attn_drop > 0: dropout in training mode (different calls differ, gradients flow), none in eval mode."""
    from pcf_nat_b200 import NAttention
    torch.manual_seed(5)
    layer = NAttention(64, 64, 2, 7, attn_drop=0.2, layout="channels_last").cuda()
    x = torch.randn(3, 64, 64, device="cuda", requires_grad=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        layer.train()
        a, b = layer(x), layer(x)
        a.float().sum().backward()
        layer.eval()
        c, d = layer(x), layer(x)
    assert not torch.equal(a, b) and torch.equal(c, d)
    assert torch.isfinite(x.grad).all() and float(x.grad.abs().sum()) > 0
    assert layer.relative_position_bias.grad is not None


def test_dropout_rejects_bad_probability_and_unsupported_shapes():
    from pcf_nat_b200 import ops
    from pcf_nat_b200._lib import Na1dError
    q = torch.zeros(2, 64, 32, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Na1dError) as e:
        ops.fused_forward(q, q, q, 7, 3, drop_p=1.0, seed=1)
    assert e.value.status == -12
    q24 = torch.zeros(2, 64, 24, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Na1dError) as e:
        ops.fused_forward(q24, q24, q24, 7, 3, drop_p=0.1, seed=1)
    assert e.value.status == -10

"""Pin the CPU oracle to vectors produced by the reference's own CPU implementation."""
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs, win_left
from oracle import na1d_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference_vectors(name):
    c = CASES[name]
    g = np.load(os.path.join(GOLD, name + ".npz"))
    q, k, v, d_out, rpb = (torch.from_numpy(a) for a in make_inputs(name))
    win, left = win_left(c["win"])
    o, dq, dk, dv, drpb = orc.na1d_fused_with_grads(
        q, k, v, d_out, win, left, c["dil"], c["scale"], rpb, c["valid_len"], c["H"])
    tol = dict(rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(o.numpy(), g["out"], **tol)
    if c["grads"]:
        np.testing.assert_allclose(dq.numpy(), g["dq"], rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(dk.numpy(), g["dk"], rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(dv.numpy(), g["dv"], rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(drpb.numpy(), g["drpb"], rtol=1e-4, atol=2e-5)


def test_window_left_rule():
    # models/PCF_NATransformer.py:47-56
    assert orc.window_left(7) == (7, 3)
    assert orc.window_left(8) == (8, 3)
    assert orc.window_left(27) == (27, 13)
    assert orc.window_left([6, 1]) == (6, 1)


def test_neighbour_index_contract():
    j, inr = orc.neighbour_index(5, 3, 1, 2)
    assert j.tolist() == [[-2, 0, 2], [-1, 1, 3], [0, 2, 4], [1, 3, 5], [2, 4, 6]]
    assert inr.tolist() == [[False, True, True], [False, True, True], [True, True, True],
                            [True, True, False], [True, True, False]]


def test_qk_av_equal_fused():
    torch.manual_seed(0)
    q, k, v = (torch.randn(3, 19, 8) for _ in range(3))
    s = orc.na1d_qk(q, k, 5, 2, 1)
    m = orc.attn_mask(19, 5, 2, 1, None, 3)
    o = orc.na1d_av(torch.softmax(s + m, -1), v, 5, 2, 1)
    torch.testing.assert_close(o, orc.na1d_fused(q, k, v, 5, 2))


def test_all_masked_row_is_plain_attention():
    # A query inside the padded region sees a uniform -100 shift that cancels in the
    # softmax (additive mask, models/PCF_NATransformer.py:87-99), so the row is finite.
    torch.manual_seed(1)
    q, k, v = (torch.randn(1, 12, 8) for _ in range(3))
    o = orc.na1d_fused(q, k, v, 3, 1, valid_len=[4])
    assert torch.isfinite(o).all()
    o_nopad = orc.na1d_fused(q, k, v, 3, 1)
    torch.testing.assert_close(o[:, 6:11], o_nopad[:, 6:11])


def test_dropout_mask_restatement_matches_the_library_bit_for_bit():
    """The oracle's numpy restatement of the dropout hash against the library's own host-side function, and the mask's
    statistics: keep rate 1 - p, no visible structure along rows or neighbours."""
    from pcf_nat_b200 import ops
    for p, seed in ((0.1, 12345), (0.5, 2 ** 40 + 7), (0.9, 0), (0.25, 2 ** 63 + 11)):
        mine = orc.dropout_keep(4000, 27, p, seed)
        theirs = ops.dropout_keep_mask(4000, 27, p, seed)
        assert torch.equal(mine, theirs)
        keep = mine.float()
        assert abs(float(keep.mean()) - (1 - p)) < 0.01
        assert float((keep.mean(0) - (1 - p)).abs().max()) < 0.04      # per neighbour index
        assert float((keep[:-1] * keep[1:]).mean() - (1 - p) ** 2) < 0.01  # adjacent rows are independent
    assert not torch.equal(orc.dropout_keep(100, 7, 0.5, 1), orc.dropout_keep(100, 7, 0.5, 2))


def test_oracle_dropout_is_a_rescaled_masked_softmax():
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(4, 20, 8, generator=g) for _ in range(3))
    keep = orc.dropout_keep(4 * 20, 5, 0.3, 99).reshape(4, 20, 5).float()
    p = torch.softmax(orc.na1d_logits(q, k, 5, 2), -1) * keep / (1 - float(torch.tensor(0.3)))
    torch.testing.assert_close(orc.na1d_fused(q, k, v, 5, 2, drop_p=0.3, seed=99), orc.na1d_av(p, v, 5, 2))

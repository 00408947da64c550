"""The packaged NAttention layer against whole-layer outputs of the reference (tests/golden/module_*.npz), on CPU:
state-dict layout, the padding mask, and the head split / merge copies, with the fused operator replaced by the oracle."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
from make_golden_module import MODULE_CASES  # noqa: E402
from oracle import na1d_oracle as orc  # noqa: E402

GOLD = os.path.join(ROOT, "tests", "golden")


def build(name):
    from pcf_nat_b200.nattention import NAttention
    model, N, T, dim, heads, win_size, dil, groups, padding = MODULE_CASES[name]
    g = np.load(os.path.join(GOLD, name + ".npz"))
    m = NAttention(frames=T, dim=dim, num_heads=heads, win_size=win_size, dilation=dil, groups=groups,
                   layout="channels_first" if model == "pcf" else "channels_last")
    return m, g


@pytest.mark.parametrize("name", list(MODULE_CASES))
def test_state_dict_matches_reference_layout(name):
    m, g = build(name)
    sd = m.state_dict()
    ref = {k[3:]: g[k] for k in g.files if k.startswith("sd_")}
    assert set(sd) == set(ref)
    for k in sd:
        assert tuple(sd[k].shape) == ref[k].shape, k
    # the constant training mask is bit-identical to the reference's buffer
    assert np.array_equal(sd["attn_mask"].numpy(), ref["attn_mask"])
    m.load_state_dict({k: torch.from_numpy(v) for k, v in ref.items()})


@pytest.mark.parametrize("name", list(MODULE_CASES))
def test_padding_mask_matches_reference(name):
    from pcf_nat_b200.nattention import padding_mask
    m, g = build(name)
    T = g["x"].shape[2] if m._na1d_layout == "channels_first" else g["x"].shape[1]
    mine = padding_mask(T, m.win_size, m.left, m.dilation, torch.from_numpy(g["padding"]))
    assert np.array_equal(mine.numpy(), g["mask_eval"])


@pytest.mark.parametrize("name", list(MODULE_CASES))
def test_layer_layout_with_oracle_operator(name, monkeypatch):
    """qkv -> head split -> operator -> head merge -> proj reproduces the reference's layer when the operator is the
    oracle: pins the layouts and the padding -> valid_len conversion without a GPU."""
    import pcf_nat_b200.nattention as mod
    m, g = build(name)
    m.load_state_dict({k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("sd_")})

    def oracle_op(q, k, v, win, left, dil, scale, rpb, valid_len, heads, drop_p=0.0, seed=0):
        vl = None if valid_len is None else [int(x) for x in valid_len]
        return orc.na1d_fused(q, k, v, win, left, dil, scale, rpb.reshape(heads, win), vl, heads, drop_p=drop_p, seed=seed)

    monkeypatch.setattr(mod, "na1d_fused", oracle_op)
    x = torch.from_numpy(g["x"])
    m.eval()
    y = m(x, torch.from_numpy(g["padding"]))
    assert float((y.detach() - torch.from_numpy(g["y_eval"])).abs().max()) < 2e-5
    m.train()
    y = m(x, None)
    assert float((y.detach() - torch.from_numpy(g["y_train"])).abs().max()) < 2e-5


def test_fuse_nattention_rebinds_reference_style_layers():
    import torch.nn as nn
    from pcf_nat_b200.nattention import NAttention, fuse_nattention

    class Foreign(nn.Module):  # has the attributes of the reference's layer, and its own forward
        def __init__(self):
            super().__init__()
            self.qkv = nn.Conv1d(16, 48, 1)
            self.proj = nn.Conv1d(16, 16, 1)
            self.relative_position_bias = nn.Parameter(torch.zeros(1, 2, 1, 3))
            self.win_size, self.left, self.num_heads, self.scale, self.dilation, self.groups = 3, 1, 2, 0.35, 1, 1
            self.attn_drop, self.proj_drop = nn.Dropout(0.0), nn.Dropout(0.0)

        def forward(self, x, padding=None):
            raise AssertionError("the original forward must not run after fusing")

    net = nn.Sequential(Foreign(), NAttention(8, 16, 2, 3))
    assert fuse_nattention(net) == 1
    assert net[0]._na1d_layout == "channels_first"
    assert net[0].forward.__func__.__name__ == "_fused_forward"


def test_argument_errors():
    from pcf_nat_b200.nattention import NAttention
    with pytest.raises(ValueError):
        NAttention(8, 16, 2, [3, 3])
    with pytest.raises(ValueError):
        NAttention(8, 20, 2, 3)          # head_dim 10 is not a multiple of 8
    with pytest.raises(ValueError):
        NAttention(8, 16, 2, 3, layout="channels_last", groups=2)


# ------------------------------------------------------------------ dense (global) attention layer
@pytest.mark.parametrize("name", ["module_global_h4", "module_global_g2"])
def test_global_attention_matches_reference_layer(name):
    """The packaged dense layer against outputs of the reference's GlobalAttention (make_golden_global.py)."""
    import numpy as np
    from pcf_nat_b200 import GlobalAttention
    from pcf_nat_b200.nattention import global_padding_mask
    z = np.load(os.path.join(GOLD, name + ".npz"))
    heads, groups = (4, 1) if name.endswith("h4") else (2, 2)
    sd = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("sd_")}
    m = GlobalAttention(z["x"].shape[1], heads, groups=groups).eval()
    assert set(m.state_dict()) == set(sd)
    m.load_state_dict(sd)
    x = torch.from_numpy(z["x"]).requires_grad_(True)
    mask = None
    if "padding" in z.files:
        mask = global_padding_mask(x.shape[-1], torch.from_numpy(z["padding"]))
        assert torch.equal(mask, torch.from_numpy(z["mask"]))
    y = m(x, torch.from_numpy(z["pos_emb"]), mask)
    torch.testing.assert_close(y, torch.from_numpy(z["y"]), rtol=1e-4, atol=1e-5)
    y.backward(torch.from_numpy(z["gy"]))
    torch.testing.assert_close(x.grad, torch.from_numpy(z["dx"]), rtol=1e-4, atol=1e-5)

"""The PCF-NAT-style extractor on CPU with the oracle standing in for the fused operator: wiring, shapes, gradients."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import na1d_oracle as orc  # noqa: E402


def test_extractor_wiring_with_oracle_operator(monkeypatch):
    import pcf_nat_b200.nattention as mod
    from pcf_nat_b200.model import PCFNATExtractor, model_flops_per_utterance

    def oracle_op(q, k, v, win, left, dil, scale, rpb, valid_len, heads, drop_p=0.0, seed=0):
        return orc.na1d_fused(q, k, v, win, left, dil, scale, rpb.reshape(heads, win), None, heads)

    monkeypatch.setattr(mod, "na1d_fused", oracle_op)
    torch.manual_seed(0)
    m = PCFNATExtractor(frames=40, feat=20, dim=32, heads=2, win=5, stages=3, blocks=2, emb=24, classes=50)
    assert len(m.fuse) == 2 and m.fuse[1].in_features == 3 * 32
    x = torch.randn(6, 20, 40)
    y = torch.randint(0, 50, (6,))
    emb = m.embedding(x)
    assert emb.shape == (6, 24)
    loss = m(x, y)
    loss.backward()
    assert torch.isfinite(loss)
    missing = [n for n, p in m.named_parameters() if p.grad is None]
    assert missing == [], missing
    # every attention layer's bias received a gradient through the operator
    assert all(float(b.attn.relative_position_bias.grad.abs().sum()) > 0 for st in m.stages for b in st)
    assert model_flops_per_utterance() > 3e10

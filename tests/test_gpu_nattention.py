"""The packaged NAttention layer on the GPU against whole-layer outputs of the reference (tests/golden/module_*.npz)."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
from make_golden_module import MODULE_CASES  # noqa: E402

pytestmark = pytest.mark.gpu
GOLD = os.path.join(ROOT, "tests", "golden")
# a whole layer in 16-bit arithmetic (two projections around the operator): looser than the operator's own bound
TOL = {torch.bfloat16: 4e-2, torch.float16: 8e-3}


def _layer(name, dtype):
    from pcf_nat_b200 import NAttention
    model, N, T, dim, heads, win_size, dil, groups, padding = MODULE_CASES[name]
    g = np.load(os.path.join(GOLD, name + ".npz"))
    m = NAttention(frames=T, dim=dim, num_heads=heads, win_size=win_size, dilation=dil, groups=groups,
                   layout="channels_first" if model == "pcf" else "channels_last")
    m.load_state_dict({k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("sd_")})
    return m.cuda().to(dtype), g


def _close(got, ref, dtype, what):
    ref = torch.from_numpy(ref)
    err = float((got.detach().float().cpu() - ref).abs().max())
    bound = TOL[dtype] * max(1.0, float(ref.abs().max()))
    assert err <= bound, "%s: max-abs error %.4g > %.4g" % (what, err, bound)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("name", list(MODULE_CASES))
def test_layer_matches_reference(name, dtype):
    m, g = _layer(name, dtype)
    x = torch.from_numpy(g["x"]).cuda().to(dtype)
    pad = torch.from_numpy(g["padding"]).cuda()
    m.eval()
    xe = x.clone().requires_grad_(True)
    y = m(xe, pad)
    _close(y, g["y_eval"], dtype, name + " y_eval")
    y.backward(torch.from_numpy(g["gy"]).cuda().to(dtype))
    _close(xe.grad, g["dx_eval"], dtype, name + " dx")
    _close(m.relative_position_bias.grad, g["drpb_eval"], dtype, name + " d_rpb")
    m.train()
    _close(m(x, None), g["y_train"], dtype, name + " y_train")


def test_fused_layer_on_foreign_module():
    """fuse_nattention() on an object that only has the reference layer's attributes gives the packaged layer's output."""
    import torch.nn as nn
    from pcf_nat_b200 import NAttention, fuse_nattention
    mine, g = _layer("module_pcf_w7", torch.bfloat16)

    class Foreign(nn.Module):
        def __init__(self, src):
            super().__init__()
            self.qkv, self.proj, self.relative_position_bias = src.qkv, src.proj, src.relative_position_bias
            self.win_size, self.left, self.num_heads, self.scale = src.win_size, src.left, src.num_heads, src.scale
            self.dilation, self.groups, self.attn_drop, self.proj_drop = src.dilation, src.groups, src.attn_drop, src.proj_drop

        def forward(self, x, padding=None):
            raise AssertionError("not fused")

    other = Foreign(mine).eval()
    assert fuse_nattention(other) == 1
    x = torch.from_numpy(g["x"]).cuda().to(torch.bfloat16)
    pad = torch.from_numpy(g["padding"]).cuda()
    mine.eval()
    assert torch.equal(other(x, pad), mine(x, pad))


def test_library_op_opcheck_and_compile():
    """The torch.library registration is consistent (schema, fake kernel, autograd) and traces without a graph break."""
    import pcf_nat_b200
    g = torch.Generator().manual_seed(5)
    q, k, v = ((torch.randn(8, 96, 32, generator=g) * 0.5).to(torch.bfloat16).cuda().requires_grad_(True) for _ in range(3))
    rpb = (0.2 * torch.randn(1, 4, 1, 7, generator=g)).cuda().requires_grad_(True)
    vl = torch.tensor([96, 80], dtype=torch.int32).cuda()
    torch.library.opcheck(torch.ops.pcf_nat_b200.na1d_fused_fwd.default, (q, k, v, rpb, vl, 7, 3, 1, 0.17, 4),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))

    def layer(q, k, v, rpb):
        return pcf_nat_b200.na1d_fused(q * 1.0, k, v, 7, 3, 1, 0.17, rpb, vl, 4).float().square().sum()

    eager = layer(q, k, v, rpb)
    ge = torch.autograd.grad(eager, (q, k, v, rpb))
    compiled = torch.compile(layer, backend="aot_eager", fullgraph=True)
    out = compiled(q, k, v, rpb)
    gc = torch.autograd.grad(out, (q, k, v, rpb))
    assert torch.equal(out, eager)
    for a, b in zip(ge, gc):
        assert torch.allclose(a.float(), b.float(), rtol=0, atol=1e-6 * max(1.0, float(a.float().abs().max())))


def test_extractor_fused_equals_unfused_chain():
    """A small PCF-NAT-style extractor: the fused layer and the reference's unfused operator chain (drop-in QK / AV functions
    around torch softmax) give the same loss and gradients."""
    from pcf_nat_b200.model import PCFNATExtractor
    kw = dict(frames=64, feat=24, dim=64, heads=4, win=7, stages=2, blocks=2, emb=32, classes=40)
    torch.manual_seed(1)
    a = PCFNATExtractor(attention="fused", **kw).cuda()
    b = PCFNATExtractor(attention="unfused", **kw).cuda()
    b.load_state_dict(a.state_dict())
    g = torch.Generator().manual_seed(2)
    x = torch.randn(8, 24, 64, generator=g).cuda()
    y = torch.randint(0, 40, (8,), generator=g).cuda()
    out = []
    for m in (a, b):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = m(x, y)
        loss.backward()
        out.append((float(loss.detach()), m.front.weight.grad.float().clone(), m.stages[0][0].attn.relative_position_bias.grad.clone()))
    assert abs(out[0][0] - out[1][0]) < 2e-2 * max(1.0, abs(out[1][0]))
    for i in (1, 2):
        ref = out[1][i]
        assert float((out[0][i] - ref).abs().max()) <= 5e-2 * max(1e-3, float(ref.abs().max()))


def test_backward_is_first_cuda_work_of_its_thread():
    """The autograd worker thread may reach the operator's backward before it has made any CUDA runtime call: the library
    binds the device's context itself before it encodes tensor maps (a driver call). Run in a fresh process so that the
    worker thread really is fresh."""
    import subprocess
    code = (
        "import sys, torch; sys.path.insert(0, %r); import pcf_nat_b200\n"
        "q, k, v = (torch.randn(8, 200, 32).to(torch.bfloat16).cuda().requires_grad_(True) for _ in range(3))\n"
        "o = pcf_nat_b200.na1d_fused(q, k, v, 7, 3, 1, 1.0, None, None, 4)\n"
        "o.backward(torch.ones_like(o)); torch.cuda.synchronize(); print('ok', float(q.grad.float().abs().sum()) > 0)\n" % ROOT)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "ok True" in out.stdout, out.stderr[-2000:]


@pytest.mark.parametrize("name", ["module_global_h4", "module_global_g2"])
def test_global_attention_layer_on_gpu(name):
    """The dense (win_size == 0) layer on the GPU in bf16 against the reference layer's fp32 output."""
    from pcf_nat_b200 import GlobalAttention
    from pcf_nat_b200.nattention import global_padding_mask
    z = np.load(os.path.join(GOLD, name + ".npz"))
    heads, groups = (4, 1) if name.endswith("h4") else (2, 2)
    m = GlobalAttention(z["x"].shape[1], heads, groups=groups).eval()
    m.load_state_dict({k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("sd_")})
    m = m.cuda()
    x = torch.from_numpy(z["x"]).cuda().requires_grad_(True)
    mask = global_padding_mask(x.shape[-1], torch.from_numpy(z["padding"]).cuda()) if "padding" in z.files else None
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(x, torch.from_numpy(z["pos_emb"]).cuda(), mask)
    y.float().backward(torch.from_numpy(z["gy"]).cuda())
    ref, dref = torch.from_numpy(z["y"]), torch.from_numpy(z["dx"])
    assert float((y.detach().float().cpu() - ref).abs().max()) <= 3e-2 * max(1.0, float(ref.abs().max()))
    assert float((x.grad.cpu() - dref).abs().max()) <= 3e-2 * max(1.0, float(dref.abs().max()))


@pytest.mark.parametrize("name", ["module_pcf_w7", "module_pcf_g2_asym", "module_mfa_w7"])
def test_layer_routes_make_no_layout_copies(name, monkeypatch):
    """Both layouts reach the kernels through strided tensor maps: the head split / merge copies are never made."""
    import pcf_nat_b200.nattention as mod

    def boom(*a, **k):
        raise AssertionError("a head split / merge copy was made")

    monkeypatch.setattr(mod, "_split_heads", boom)
    monkeypatch.setattr(mod, "_merge_heads", boom)
    m, g = _layer(name, torch.bfloat16)
    x = torch.from_numpy(g["x"]).cuda().to(torch.bfloat16).requires_grad_(True)
    y = m.eval()(x, torch.from_numpy(g["padding"]).cuda())
    y.backward(torch.from_numpy(g["gy"]).cuda().to(torch.bfloat16))
    _close(y, g["y_eval"], torch.bfloat16, name + " y_eval")
    _close(x.grad, g["dx_eval"], torch.bfloat16, name + " dx")
    # and under autocast with fp32 parameters and input, as a training script runs it
    m32, _ = _layer(name, torch.float32)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y32 = m32.eval()(torch.from_numpy(g["x"]).cuda(), torch.from_numpy(g["padding"]).cuda())
    _close(y32, g["y_eval"], torch.bfloat16, name + " y_eval under autocast")

"""Generate tests/golden/module_*.npz: whole-layer outputs of the REFERENCE's NAttention (CPU branch).

    python tests/golden/make_golden_module.py --reference /path/to/PCF-NAT

Unlike make_golden.py nothing is replaced inside the layer: the reference's own ``qkv`` / ``proj`` projections, head
split and merge copies, bias, mask and softmax all run (models/PCF_NATransformer.py:118-178,
models/MFA_NATransformer.py:118-177). Each file holds the layer's state dict, the input, the padding vector and the
output (eval mode with padding, and train mode), plus the gradient of the input for a seeded output gradient.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from make_golden import import_reference  # noqa: E402

MODULE_CASES = {
    # name: (model, N, T, dim, heads, win_size, dilation, groups, padding)
    "module_pcf_w7": ("pcf", 3, 48, 64, 4, 7, 1, 1, [0, 5, 17]),
    "module_pcf_g2_asym": ("pcf", 2, 40, 64, 2, [6, 1], 1, 2, [0, 9]),
    "module_pcf_dil2": ("pcf", 2, 56, 32, 2, 5, 2, 1, [3, 0]),
    "module_mfa_w7": ("mfa", 3, 48, 64, 4, 7, 1, 1, [0, 5, 17]),
    "module_mfa_w15_dil2": ("mfa", 2, 64, 64, 8, 15, 2, 1, [0, 20]),
}


def run(name, classes):
    model, N, T, dim, heads, win_size, dil, groups, padding = MODULE_CASES[name]
    torch.manual_seed(sum(ord(c) for c in name))
    kw = dict(frames=T, dim=dim, num_heads=heads, win_size=win_size, dilation=dil, dtype=torch.bfloat16)
    if model == "pcf":
        kw["groups"] = groups
    m = classes[model](**kw)
    with torch.no_grad():
        m.relative_position_bias.mul_(20.0)  # std 0.4 instead of 0.02 so the bias matters in the comparison
    x = torch.randn((N, dim, T) if model == "pcf" else (N, T, dim))
    pad = torch.tensor(padding, dtype=torch.int)
    res = {"sd_" + k: v.detach().numpy() for k, v in m.state_dict().items()}
    res["x"] = x.numpy()
    res["padding"] = pad.numpy()
    get_mask = m.get_attn_mask if dil == 1 else m.get_attn_mask_dilation
    res["mask_eval"] = get_mask(T, m.win_size, m.left, pad).numpy()
    m.eval()
    xe = x.clone().requires_grad_(True)
    ye = m(xe, pad)
    gy = torch.randn(ye.shape)
    ye.backward(gy)
    res.update(y_eval=ye.detach().numpy(), gy=gy.numpy(), dx_eval=xe.grad.numpy(),
               drpb_eval=m.relative_position_bias.grad.numpy().copy())
    m.zero_grad()
    m.train()
    res["y_train"] = m(x, None).detach().numpy()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    classes = import_reference(args.reference)
    for name in MODULE_CASES:
        res = run(name, classes)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **res)
        print(name, {k: v.shape for k, v in res.items() if not k.startswith("sd_")}, sorted(k for k in res if k.startswith("sd_")))


if __name__ == "__main__":
    main()

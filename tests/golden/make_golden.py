"""Generate tests/golden/*.npz from the REFERENCE's own CPU implementation.

Run where the reference project is checked out (it is not needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/PCF-NAT

The reference's ``NAttention.forward`` has a pure-PyTorch branch taken for CPU tensors
(models/PCF_NATransformer.py:153-174, models/MFA_NATransformer.py:152-173). Importing the
model files pulls in ``na1d_tensorcore.nattn``, which JIT-builds CUDA code at import
(na1d_tensorcore/nattn.py:12-29); a stub module is registered first so the import works
without a GPU. The stub is never called on the CPU branch.

To drive the layer with given q/k/v, the ``qkv`` projection is replaced by a module that
returns a pre-assembled tensor in the layout the layer expects, and ``proj`` by identity;
everything between them (scale, pad/unfold gather, bias, mask, softmax, weighted sum) is
the reference's code, unmodified. Gradients come from autograd through that code.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import CASES, make_inputs, win_left  # noqa: E402


def import_reference(path):
    stub = types.ModuleType("na1d_tensorcore.nattn")
    stub.getNA1dFunction = lambda C, dilation, dtype: (None, None)
    sys.modules["na1d_tensorcore"] = types.ModuleType("na1d_tensorcore")
    sys.modules["na1d_tensorcore.nattn"] = stub
    sys.path.insert(0, path)
    from models.MFA_NATransformer import NAttention as NA_mfa
    from models.PCF_NATransformer import NAttention as NA_pcf
    return {"mfa": NA_mfa, "pcf": NA_pcf}


class Inject(nn.Module):
    def __init__(self, t):
        super().__init__()
        self.t = t

    def forward(self, x):
        return self.t


def run_case(name, classes):
    c = CASES[name]
    B, H, T, D = c["B"], c["H"], c["T"], c["D"]
    win, left = win_left(c["win"])
    q, k, v, d_out, rpb = (torch.from_numpy(a) for a in make_inputs(name))
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    NA = classes[c["model"]]
    m = NA(frames=T, dim=H * D, num_heads=H, win_size=c["win"], dilation=c["dil"],
           qk_scale=c["scale"], dtype=torch.bfloat16).eval()
    assert (m.win_size, m.left) == (win, left)
    rp = rpb.clone().reshape(1, H, 1, win).requires_grad_(True)
    m.relative_position_bias = nn.Parameter(rp)
    qh, kh, vh = (a.reshape(B, H, T, D) for a in (q, k, v))
    if c["model"] == "mfa":
        # layer input (B,T,C); qkv output viewed as (B,T,3,H,D)
        packed = torch.stack([qh, kh, vh], 0).permute(1, 3, 0, 2, 4).reshape(B, T, 3 * H * D)
        x = torch.zeros(B, T, H * D)
    else:
        # layer input (B,C,T); qkv output viewed (groups=1) as (B,H,D,3,T)
        packed = torch.stack([qh, kh, vh], 0).permute(1, 2, 4, 0, 3).reshape(B, 3 * H * D, T)
        x = torch.zeros(B, H * D, T)
    m.qkv = Inject(packed)
    m.proj = nn.Identity()
    padding = None
    if c["valid_len"] is not None:
        padding = T - torch.tensor(c["valid_len"], dtype=torch.int)
    y = m(x, padding)
    if c["model"] == "mfa":
        out = y.reshape(B, T, H, D).permute(0, 2, 1, 3).reshape(B * H, T, D)
    else:
        out = y.reshape(B, H, D, T).permute(0, 1, 3, 2).reshape(B * H, T, D)
    res = {"out": out.detach().numpy()}
    if c["grads"]:
        out.backward(d_out)
        res.update(dq=q.grad.numpy(), dk=k.grad.numpy(), dv=v.grad.numpy(),
                   drpb=m.relative_position_bias.grad.reshape(H, win).numpy())
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    torch.set_grad_enabled(True)
    classes = import_reference(args.reference)
    for name in CASES:
        res = run_case(name, classes)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **res)
        print(name, {k_: v_.shape for k_, v_ in res.items()})


if __name__ == "__main__":
    main()

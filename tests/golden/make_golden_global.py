"""Generate tests/golden/module_global_*.npz: outputs of the REFERENCE's GlobalAttention layer (dense attention, the
``win_size == 0`` layers of the network; models/PCF_NATransformer.py:181-225) with the mask its network builds
(``get_attn_mask_global``, :406-414), on the CPU.

    python tests/golden/make_golden_global.py --reference /path/to/PCF-NAT

Each file holds the layer's state dict, the input, the positional embedding, the padding vector, the mask, the output and
the gradient of the input for a seeded output gradient.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from make_golden import import_reference  # noqa: E402

GLOBAL_CASES = {
    # name: (N, T, dim, heads, groups, padding or None)
    "module_global_h4": (3, 50, 64, 4, 1, [0, 7, 21]),
    "module_global_g2": (2, 37, 64, 2, 2, None),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    import_reference(args.reference)
    from models.PCF_NATransformer import GlobalAttention, PCF_NATransformer
    for name, (N, T, dim, heads, groups, padding) in GLOBAL_CASES.items():
        torch.manual_seed(sum(ord(c) for c in name))
        m = GlobalAttention(dim, heads, groups=groups).eval()
        x = torch.randn(N, dim, T, requires_grad=True)
        pos = torch.randn(1, dim, T)
        res = {"sd_" + k: v.detach().numpy() for k, v in m.state_dict().items()}
        mask = None
        if padding is not None:
            pad = torch.tensor(padding, dtype=torch.int)
            mask = PCF_NATransformer.get_attn_mask_global(None, T, padding=pad)
            res["padding"] = pad.numpy()
            res["mask"] = mask.numpy()
        y = m(x, pos, mask)
        gy = torch.randn(y.shape)
        y.backward(gy)
        res.update(x=x.detach().numpy(), pos_emb=pos.numpy(), y=y.detach().numpy(), gy=gy.numpy(), dx=x.grad.numpy())
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **res)
        print(name, {k: v.shape for k, v in res.items() if not k.startswith("sd_")})


if __name__ == "__main__":
    main()

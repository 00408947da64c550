"""Golden-vector cases for the NA1D path and the seeded input builder shared by the
generator (make_golden.py, run where the reference project is present) and the tests
(run anywhere). Inputs come from numpy's RandomState (MT19937), whose stream is stable
across numpy versions, so only the reference's OUTPUTS are stored in the .npz files.
"""
import numpy as np

# name -> dict(model, B, H, T, D, win, dil, valid_len, rpb, scale, grads, seed)
#   model: which reference caller produced the vector ("mfa" = models/MFA_NATransformer.py,
#          "pcf" = models/PCF_NATransformer.py)
#   win:   int (centred, left = win-1-win//2) or [win, left]
#   valid_len: None or list of B ints (= T - padding)
#   rpb:   True -> random relative position bias, False -> zeros
#   grads: also store dq/dk/dv/drpb from autograd through the reference
CASES = {
    # the forward-only parity configuration: B=2 heads=4 L=200 head_dim=32 win=7 dil=1, no bias
    "cfg1_fwd":        dict(model="mfa", B=2, H=4, T=200, D=32, win=7,      dil=1, valid_len=None,     rpb=False, scale=1.0,  grads=False, seed=0),
    "pcf_w7":          dict(model="pcf", B=2, H=2, T=48,  D=16, win=7,      dil=1, valid_len=None,     rpb=True,  scale=0.25, grads=True,  seed=11),
    "mfa_w7_pad":      dict(model="mfa", B=3, H=2, T=40,  D=16, win=7,      dil=1, valid_len=[40, 29, 3], rpb=True, scale=0.25, grads=True, seed=12),
    "mfa_w8_even":     dict(model="mfa", B=1, H=2, T=33,  D=8,  win=8,      dil=1, valid_len=None,     rpb=True,  scale=0.35, grads=True,  seed=13),
    "mfa_asym_6_1":    dict(model="mfa", B=2, H=1, T=31,  D=16, win=[6, 1], dil=1, valid_len=None,     rpb=True,  scale=0.25, grads=True,  seed=14),
    "mfa_left0":       dict(model="mfa", B=1, H=2, T=20,  D=8,  win=[5, 0], dil=1, valid_len=None,     rpb=False, scale=1.0,  grads=True,  seed=15),
    "mfa_leftmax":     dict(model="mfa", B=1, H=2, T=20,  D=8,  win=[5, 4], dil=1, valid_len=None,     rpb=False, scale=1.0,  grads=True,  seed=16),
    "mfa_w7_dil2":     dict(model="mfa", B=2, H=2, T=37,  D=16, win=7,      dil=2, valid_len=None,     rpb=True,  scale=0.25, grads=True,  seed=17),
    "pcf_w15_dil4_pad": dict(model="pcf", B=2, H=2, T=50, D=16, win=15,     dil=4, valid_len=[50, 33], rpb=True,  scale=0.25, grads=True,  seed=18),
    "mfa_w27_real":    dict(model="mfa", B=1, H=4, T=150, D=16, win=27,     dil=1, valid_len=None,     rpb=True,  scale=0.25, grads=False, seed=19),
    "mfa_win_gt_T":    dict(model="mfa", B=1, H=1, T=5,   D=8,  win=9,      dil=1, valid_len=None,     rpb=True,  scale=0.35, grads=True,  seed=20),
    "mfa_T1":          dict(model="mfa", B=2, H=1, T=1,   D=8,  win=3,      dil=1, valid_len=None,     rpb=True,  scale=0.35, grads=True,  seed=21),
    "mfa_w31_d64":     dict(model="mfa", B=1, H=2, T=70,  D=64, win=31,     dil=1, valid_len=None,     rpb=False, scale=0.125, grads=True, seed=22),
}


def win_left(win):
    if isinstance(win, int):
        return win, win - 1 - win // 2
    return int(win[0]), int(win[1])


def make_inputs(case):
    """Seeded fp32 inputs: q, k, v, d_out of shape (B*H, T, D) and rpb of shape (H, win)."""
    c = CASES[case] if isinstance(case, str) else case
    rs = np.random.RandomState(c["seed"])
    N = c["B"] * c["H"]
    shp = (N, c["T"], c["D"])
    q = rs.standard_normal(shp).astype(np.float32)
    k = rs.standard_normal(shp).astype(np.float32)
    v = rs.standard_normal(shp).astype(np.float32)
    d_out = rs.standard_normal(shp).astype(np.float32)
    win, _ = win_left(c["win"])
    if c["rpb"]:
        rpb = (0.5 * rs.standard_normal((c["H"], win))).astype(np.float32)
    else:
        rpb = np.zeros((c["H"], win), np.float32)
    return q, k, v, d_out, rpb

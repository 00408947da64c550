"""Shape sweep of the fused NA1D operator (BASELINE configs[2] and the other named shapes).

    python -m pcf_nat_b200.sweep [--quick] [--out FILE.md]

For every (dtype, win, dilation, L, head_dim) of the sweep it times forward and forward+backward through the C ABI
(CUDA events, one CUDA graph of rotating buffer sets larger than L2) and prints a markdown table with the kernel family
that ran, microseconds, queries/s and the fraction of the HBM roofline (algorithmic bytes / measured copy bandwidth).
"""
import argparse
import ctypes
import itertools
import json
import os
import sys

import torch

from . import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
L2_BYTES = 126 * 1024 * 1024


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    return float(json.load(open(p))["hbm_gbs"]) if os.path.exists(p) else 6650.0


def time_case(L, N, H, T, C, win, dil, dtype, reps=30):
    code = 0 if dtype == torch.bfloat16 else 1
    left = win - 1 - win // 2
    per_set = 9 * N * T * C * 2
    n_sets = max(2, min(8, (2 * L2_BYTES) // per_set + 2))
    g = torch.Generator(device="cuda").manual_seed(2)
    sets = []
    for _ in range(n_sets):
        q, k, v, d_o = ((torch.randn(N, T, C, device="cuda", generator=g) * C ** -0.25).to(dtype) for _ in range(4))
        sets.append(dict(q=q, k=k, v=v, d_o=d_o, o=torch.empty_like(q), dq=torch.empty_like(q), dk=torch.empty_like(q),
                         dv=torch.empty_like(q), lse=torch.empty(N, T, device="cuda"), delta=torch.empty(N, T, device="cuda")))
    P = lambda t: ctypes.c_void_p(t.data_ptr())

    def fwd(s, st):
        rc = L.na1d_fused_forward(P(s["o"]), P(s["lse"]), P(s["q"]), P(s["k"]), P(s["v"]), None, None, N, H, T, C, win, left, dil,
                                  1.0, code, st)
        assert rc == 0, rc

    def bwd(s, st):
        rc = L.na1d_fused_backward(P(s["dq"]), P(s["dk"]), P(s["dv"]), None, P(s["d_o"]), P(s["q"]), P(s["k"]), P(s["v"]),
                                   P(s["o"]), P(s["lse"]), None, None, P(s["delta"]), N, H, T, C, win, left, dil, 1.0, code, st)
        assert rc == 0, rc

    out = {}
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for name, fns in (("fwd", (fwd,)), ("fwd_bwd", (fwd, bwd))):
            st = ctypes.c_void_p(stream.cuda_stream)
            for s in sets:
                for f in fns:
                    f(s, st)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
                for i in range(reps):
                    for f in fns:
                        f(sets[i % n_sets], st)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            out[name] = 1e3 * e0.elapsed_time(e1) / reps
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="a 12-case subset")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the sweep needs a CUDA device")
    L = _lib.lib()
    peak = hbm_peak()
    B, H = 64, 4
    cases = list(itertools.product((torch.bfloat16, torch.float16), (3, 7, 15, 31), (1, 2, 4), (200, 400, 1000), (32, 64)))
    if args.quick:
        cases = [c for c in cases if c[0] == torch.bfloat16 and c[3] in (200, 1000) and c[4] == 64 and c[2] in (1, 4)
                 and c[1] in (7, 15, 31)]
    extra = [("train cfg2", torch.bfloat16, 7, 1, 200, 64, 128, 4), ("long cfg4 (fwd)", torch.bfloat16, 15, 1, 3000, 64, 16, 8),
             ("reference yaml", torch.bfloat16, 27, 1, 150, 16, 512, 16)]
    lines = ["| case | dtype | win | dil | L | D | N | family fwd/bwd | fwd us | fwd frac | fwd+bwd us | fwd+bwd Gq/s | fwd+bwd frac |",
             "|---|---|---|---|---|---|---|---|---|---|---|---|---|"]

    def row(tag, dtype, win, dil, T, C, b, h):
        N = b * h
        code = 0 if dtype == torch.bfloat16 else 1
        left = win - 1 - win // 2
        fam = "%s/%s" % tuple(["cuda-core", "tcgen05"][L.na1d_fused_kernel_family(N, T, C, win, left, dil, code, bw)] for bw in (0, 1))
        t = time_case(L, N, h, T, C, win, dil, dtype)
        fb, tb = 8 * N * T * C + 4 * N * T, 24 * N * T * C + 8 * N * T
        lines.append("| %s | %s | %d | %d | %d | %d | %d | %s | %.1f | %.2f | %.1f | %.2f | %.2f |" % (
            tag, "bf16" if code == 0 else "fp16", win, dil, T, C, N, fam, t["fwd"], fb / t["fwd"] / 1e3 / peak, t["fwd_bwd"],
            N * T / t["fwd_bwd"] / 1e3, tb / t["fwd_bwd"] / 1e3 / peak))
        print(lines[-1], flush=True)

    print("\n".join(lines[:2]))
    for tag, dtype, win, dil, T, C, b, h in extra:
        row(tag, dtype, win, dil, T, C, b, h)
    for dtype, win, dil, T, C in cases:
        row("sweep", dtype, win, dil, T, C, B, H)
    if args.out:
        with open(args.out, "w") as f:
            f.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    main()

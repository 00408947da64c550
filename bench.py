#!/usr/bin/env python
"""Benchmark of the NA1D hot path and of the model-level workloads built on it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--replays R]
    python bench.py --sweep OUT.md [--quick]          # the window/dilation/length/head-dim sweep as a markdown table

Operator workloads (default: the PCF-NAT training shape): one "step" is one forward+backward pass of the fused
neighbourhood-attention operator over one batch of synthetic inputs (seeded N(0,1) stand-ins for log-mel features).
The K steps are captured once in a CUDA graph over rotating buffer sets larger than L2; the graph is replayed R times,
every replay timed with CUDA events on the launching stream, and the MEDIAN replay gives `ms_per_step` (so
`ms_per_step * steps` is one replay of exactly K steps). N>1 is launched by torchrun, one rank per GPU; the operator has
no exchange step, so every rank runs the same per-GPU batch (weak scaling) and the only collectives are the timing
barrier and the max-over-ranks reduction of the elapsed time.

Model workloads (`cfg5_train`, `cfg5_embed`): the PCF-NAT-style extractor of `pcf_nat_b200.model`, batch-sharded over the
ranks with an NCCL gradient all-reduce (training) or an embedding all-gather (extraction); see `pcf_nat_b200.model_bench`.

Rank 0 prints one JSON line.
"""
import argparse
import ctypes
import itertools
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name -> batch, heads, T, C, win, dil, backward
WORKLOADS = {
    # the shape the headline metric is quoted on: 128 utterances x 4 heads, 200 frames, head dim 64, window 7
    "cfg2_train_B128_H4_L200_D64_w7": dict(B=128, H=4, T=200, C=64, win=7, dil=1, bwd=True),
    # long-utterance inference: 16 utterances x 8 heads, 3000 frames, window 15, forward only
    "cfg4_long_B16_H8_L3000_D64_w15": dict(B=16, H=8, T=3000, C=64, win=15, dil=1, bwd=False),
    # the shape the reference's own yaml trains (configs/pcf_nat4x4.yaml:16-17,50-53)
    "real_B512_H16_L150_D16_w27": dict(B=512, H=16, T=150, C=16, win=27, dil=1, bwd=True),
}
MODEL_WORKLOADS = ("cfg5_train", "cfg5_embed")
DEFAULT = "cfg2_train_B128_H4_L200_D64_w7"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel from an `ncu --set full` capture of this
# command; a constant taken from that capture, not something this run measures (writes still resident in L2 when the
# kernel ends are not in it)
NCU_TRAFFIC = {"cfg2_train_B128_H4_L200_D64_w7": 52.91e6 + 3.10e6, "real_B512_H16_L150_D16_w27": 162.33e6 + 83.05e6}
L2_BYTES = 126 * 1024 * 1024


def algorithmic_bytes(N, T, C, bwd):
    fwd = 8 * N * T * C + 4 * N * T          # read q,k,v; write o; write lse
    back = 16 * N * T * C + 4 * N * T        # read q,k,v,o,dO,lse; write dq,dk,dv
    return fwd, (back if bwd else 0)


def moved_bytes_bwd(N, T, C):
    """What the tcgen05 backward has to move: it never reads o (delta is recomputed from P and dP)."""
    return 14 * N * T * C + 4 * N * T


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.th.join(timeout=5)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for nm, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_host_inputs(w, seed=1, dtype=torch.bfloat16, scale=1.0):
    N = w["B"] * w["H"]
    g = torch.Generator().manual_seed(seed)
    shape = (N, w["T"], w["C"])
    return [(torch.randn(shape, generator=g) * scale).to(dtype) for _ in range(4)]  # q, k, v, dO


# ------------------------------------------------------------------------------------------ reference arm
def run_reference(args, w, name):
    """The reference's CPU implementation of the path (its eager pad/unfold/softmax branch,
    models/PCF_NATransformer.py:153-174), as restated by the oracle, on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import na1d_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    left = w["win"] - 1 - w["win"] // 2
    N = w["B"] * w["H"]
    host = make_host_inputs(w)

    def make_step(n_s):
        q, k, v, d_o = (x[:n_s].float() for x in host)

        def step():
            if w["bwd"]:
                orc.na1d_fused_with_grads(q, k, v, d_o, w["win"], left, w["dil"], 1.0, None, None, w["H"])
            else:
                orc.na1d_fused(q, k, v, w["win"], left, w["dil"], 1.0, None, None, w["H"])
        return step

    # size the per-step sample so that the whole run stays near args.ref_budget seconds
    probe_n = min(N, 32)
    probe = make_step(probe_n)
    probe()
    t0 = time.perf_counter()
    probe()
    per_seq = (time.perf_counter() - t0) / probe_n
    n_s = int(args.ref_budget / max(1, args.steps + args.warmup) / per_seq)
    n_s = max(1, min(N, n_s))
    step = make_step(n_s)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = args.steps * n_s * w["T"] / dt
    line = {
        "impl": "reference", "metric": "NA1D fwd+bwd queries/sec/GPU" if w["bwd"] else "NA1D fwd queries/sec/GPU",
        "value": val, "unit": "queries/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "N": N, "T": w["T"], "C": w["C"], "win": w["win"], "dil": w["dil"],
                   "sample": "%d of %d sequences per step" % (n_s, N)},
        "cpu_baseline": {"value": val, "unit": "queries/s", "cores": cores, "kind": "port",
                         "sample": "%d of %d sequences x %d steps, fp32 eager oracle" % (n_s, N, args.steps)},
        "e2e": {"value": val, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ operator timing
class OpBench:
    """Rotating device buffer sets of one operator shape and graph-replay timing through the C ABI."""

    def __init__(self, L, dev, N, H, T, C, win, dil, dtype, bwd, host=None, seed=2, scale=1.0, max_sets=8):
        self.L, self.dev = L, dev
        self.N, self.H, self.T, self.C, self.win, self.dil, self.bwd = N, H, T, C, win, dil, bwd
        self.left = win - 1 - win // 2
        self.code = 0 if dtype == torch.bfloat16 else 1
        self.per_set = (9 if bwd else 4) * N * T * C * 2
        # the other sets in the rotation exceed L2 several times over
        self.n_sets = int(max(4, min(max_sets, (3 * L2_BYTES) // self.per_set + 2)))
        g = torch.Generator(device=dev).manual_seed(seed)
        self.sets = []
        for _ in range(self.n_sets):
            if host is not None:
                q, k, v, d_o = (x.to(dev) for x in host)
            else:
                q, k, v, d_o = ((torch.randn(N, T, C, device=dev, generator=g) * scale).to(dtype) for _ in range(4))
            s = dict(q=q, k=k, v=v, d_o=d_o, o=torch.empty_like(q), lse=torch.empty(N, T, device=dev))
            if bwd:
                s.update(dq=torch.empty_like(q), dk=torch.empty_like(q), dv=torch.empty_like(q), delta=torch.empty(N, T, device=dev))
            self.sets.append(s)
        self.stream = torch.cuda.Stream(dev)

    def _fwd(self, s, st):
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        rc = self.L.na1d_fused_forward(P(s["o"]), P(s["lse"]), P(s["q"]), P(s["k"]), P(s["v"]), None, None, self.N, self.H,
                                       self.T, self.C, self.win, self.left, self.dil, 1.0, self.code, st)
        assert rc == 0, rc

    def _bwd(self, s, st):
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        rc = self.L.na1d_fused_backward(P(s["dq"]), P(s["dk"]), P(s["dv"]), None, P(s["d_o"]), P(s["q"]), P(s["k"]), P(s["v"]),
                                        P(s["o"]), P(s["lse"]), None, None, P(s["delta"]), self.N, self.H, self.T, self.C,
                                        self.win, self.left, self.dil, 1.0, self.code, st)
        assert rc == 0, rc

    def run_steps(self, n, what="both"):
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        for i in range(n):
            s = self.sets[i % self.n_sets]
            if what in ("both", "fwd"):
                self._fwd(s, st)
            if self.bwd and what in ("both", "bwd"):
                self._bwd(s, st)

    def timed(self, steps, what, replays, sync_ranks=None):
        """Median device time (ms) of one replay of a CUDA graph holding `steps` steps; every replay timed by events."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self.stream):
            self.run_steps(2, what)                      # lazy module load / first-use set-up outside capture
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=self.stream):
                self.run_steps(steps, what)
            g.replay()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
            torch.cuda.synchronize()
            if sync_ranks:
                sync_ranks()
            ev[0].record(self.stream)
            for i in range(replays):
                g.replay()
                ev[i + 1].record(self.stream)
            torch.cuda.synchronize()
            if sync_ranks:
                sync_ranks()
        ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(replays)]
        return statistics.median(ms), min(ms), max(ms)


def spot_check(ob, dtype):
    """A few sequences of buffer set 0 against the fp32 oracle (checker only; outside every timed region)."""
    from oracle import na1d_oracle as orc
    s = ob.sets[0]
    tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
    worst = 0.0
    for n0 in sorted({0, ob.N // 2, ob.N - 1}):
        f = lambda x: x[n0:n0 + 1].float().cpu()
        if ob.bwd:
            o_r, dq_r, dk_r, dv_r, _ = orc.na1d_fused_with_grads(f(s["q"]), f(s["k"]), f(s["v"]), f(s["d_o"]), ob.win, ob.left, ob.dil)
            pairs = [("o", s["o"], o_r, 1.0), ("dq", s["dq"], dq_r, None), ("dk", s["dk"], dk_r, None), ("dv", s["dv"], dv_r, None)]
        else:
            pairs = [("o", s["o"], orc.na1d_fused(f(s["q"]), f(s["k"]), f(s["v"]), ob.win, ob.left, ob.dil), 1.0)]
        for name, got, ref, mag in pairs:
            err = float((f(got) - ref).abs().max())
            bound = tol * (mag if mag is not None else max(1.0, float(ref.abs().max())))
            if not err <= bound:
                raise SystemExit("bench: %s of sequence %d differs from the oracle by %.3e (bound %.1e)" % (name, n0, err, bound))
            worst = max(worst, err / bound)
    return worst


def run_ours(args, w, name):
    import torch.distributed as dist
    from pcf_nat_b200 import _lib, na1d_fused, ops
    L = _lib.lib()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from pcf_nat_b200 import parallel

    N, H, T, C, win, dil = w["B"] * w["H"], w["H"], w["T"], w["C"], w["win"], w["dil"]
    left = win - 1 - win // 2
    fwd_b, bwd_b = algorithmic_bytes(N, T, C, w["bwd"])
    host = make_host_inputs(w, seed=1 + rank)
    ob = OpBench(L, dev, N, H, T, C, win, dil, torch.bfloat16, w["bwd"], host=host, max_sets=64)
    sync_ranks = dist.barrier if world > 1 else None

    with torch.cuda.stream(ob.stream):
        ob.run_steps(max(args.warmup, 3))
        torch.cuda.synchronize()
    ops.device_status()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    R = args.replays
    med_total, lo_total, hi_total = ob.timed(args.steps, "both", R, sync_ranks)
    med_fwd, _, _ = ob.timed(args.steps, "fwd", R, sync_ranks)
    med_bwd = ob.timed(args.steps, "bwd", R, sync_ranks)[0] if w["bwd"] else 0.0
    ops.device_status()   # an expired bounded wait would have ended kernels early: such a timing must not be reported
    ms_total = parallel.max_over_ranks(med_total, dev)
    ms_fwd = parallel.max_over_ranks(med_fwd, dev)
    ms_bwd = parallel.max_over_ranks(med_bwd, dev)
    checked = spot_check(ob, torch.bfloat16)

    # ---- end to end through the public torch API with HOST buffers: every step copies its q, k, v, dO from pinned host
    # memory and its o, dq, dk, dv back. Three streams and two buffer slots, as a training input pipeline would run it:
    # the upload of step i+1 and the download of step i-1 overlap the kernels of step i (PCIe is full duplex).
    pin = [x.pin_memory() for x in host]
    n_out = 4 if w["bwd"] else 1
    slots = 2
    dev_in = [[torch.empty_like(x, device=dev) for x in pin] for _ in range(slots)]
    host_out = [[torch.empty_like(pin[0]).pin_memory() for _ in range(n_out)] for _ in range(slots)]
    s_up, s_run, s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_up = [torch.cuda.Event() for _ in range(slots)]
    ev_run = [torch.cuda.Event() for _ in range(slots)]
    ev_down = [torch.cuda.Event() for _ in range(slots)]
    e2e_steps = max(4, min(args.steps, 20))

    def e2e_step(i):
        sl = i % slots
        with torch.cuda.stream(s_up):
            s_up.wait_event(ev_run[sl])                 # the kernels that read this slot two steps ago are done
            for dst, src in zip(dev_in[sl], pin):
                dst.copy_(src, non_blocking=True)
            ev_up[sl].record(s_up)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_up[sl])
            s_run.wait_event(ev_down[sl])               # the download of this slot's previous results is done
            q, k, v, d_o = (x.detach() for x in dev_in[sl])
            if w["bwd"]:
                q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
                o = na1d_fused(q, k, v, win, left, dil, 1.0, None, None, H)
                o.backward(d_o)
                outs = (o.detach(), q.grad, k.grad, v.grad)
            else:
                outs = (na1d_fused(q, k, v, win, left, dil, 1.0, None, None, H),)
            ev_run[sl].record(s_run)
        with torch.cuda.stream(s_down):
            s_down.wait_event(ev_run[sl])
            for dst, src in zip(host_out[sl], outs):
                src.record_stream(s_down)
                dst.copy_(src, non_blocking=True)
            ev_down[sl].record(s_down)

    for i in range(4):
        e2e_step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_up)
    for i in range(e2e_steps):
        e2e_step(i)
    s_down.wait_stream(s_run)
    s_down.wait_stream(s_up)
    e1.record(s_down)
    torch.cuda.synchronize()
    ms_e2e_rank = e0.elapsed_time(e1)
    ms_e2e = parallel.max_over_ranks(ms_e2e_rank, dev)
    ops.device_status()
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        peak, peak_kind = peaks()
        queries = N * T
        # dominant kernel: the fused backward main kernel when there is a backward, else the forward
        dom_ms = (ms_bwd if w["bwd"] else ms_fwd) / args.steps
        dom_bytes = bwd_b if w["bwd"] else fwd_b
        ach = dom_bytes / (dom_ms * 1e-3) / 1e9
        fam = L.na1d_fused_kernel_family(N, T, C, win, left, dil, 0, 1 if w["bwd"] else 0)
        h2d, d2h = 4 * N * T * C * 2, n_out * N * T * C * 2
        line = {
            "metric": "NA1D fwd+bwd queries/sec/GPU" if w["bwd"] else "NA1D fwd queries/sec/GPU",
            "value": world * queries * args.steps / (ms_total * 1e-3), "unit": "queries/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "N": N, "T": T, "C": C, "win": win, "dil": dil,
                       "l2": "rotating %d buffer sets of %.0f MB (> L2 between reuses)" % (ob.n_sets, ob.per_set / 1e6),
                       "launch": "one CUDA graph of the %d timed steps, replayed %d times; ms_per_step = median replay / steps "
                                 "(min %.4f, max %.4f ms per step on rank 0)" % (args.steps, R, lo_total / args.steps, hi_total / args.steps),
                       "kernel_family": ["cuda-core", "tcgen05"][fam],
                       "checked": "outputs of 3 sequences against the fp32 oracle after the timed region (worst error/bound %.2f); "
                                  "device status word clean" % checked},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "traffic": NCU_TRAFFIC.get(name),
                         "traffic_source": "ncu capture of this kernel at this workload, a constant (not measured by this run)",
                         "peak_kind": peak_kind,
                         "kernel": ("fused backward" if w["bwd"] else "fused forward") + (" (tcgen05)" if fam == 1 else " (cuda-core)"),
                         "algorithmic_bytes_per_launch": dom_bytes},
            "roofline_step": {"fwd_us": 1e3 * ms_fwd / args.steps, "bwd_us": 1e3 * ms_bwd / args.steps,
                              "fwd_frac": fwd_b / (ms_fwd / args.steps * 1e-3) / 1e9 / peak,
                              "step_frac": (fwd_b + bwd_b) / (ms_total / args.steps * 1e-3) / 1e9 / peak},
            "e2e": {"value": world * queries * e2e_steps / (ms_e2e * 1e-3), "unit": "queries/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "rank0_h2d_gbs": h2d * e2e_steps / (ms_e2e_rank * 1e-3) / 1e9,
                    "rank0_d2h_gbs": d2h * e2e_steps / (ms_e2e_rank * 1e-3) / 1e9,
                    "bound": "host<->device copies (uploads and downloads overlap each other and the kernels)"},
            "gpu_launches": args.steps * (2 if w["bwd"] else 1),
            "clocks": clocks,
        }
        if w["bwd"] and fam == 1:
            moved = moved_bytes_bwd(N, T, C)
            line["roofline"]["moved_bytes_per_launch"] = moved
            line["roofline"]["frac_moved_bytes"] = moved / (dom_ms * 1e-3) / 1e9 / peak
        line["cpu_baseline"] = cpu_baseline(w) if world == 1 and not args.no_cpu_baseline else None
        if world == 1:
            line["reference_cuda"] = reference_cuda_baseline(w, dev, host)
            line["compat_pair"] = compat_pair_timing(L, w, dev, host, line["reference_cuda"])
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _time_fn(fn, iters, stream=None):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return 1e3 * e0.elapsed_time(e1) / iters


def reference_cuda_baseline(w, dev, host, iters=30):
    """The reference's own sm_80-style CUDA kernels (oracle/_ref, compiled unmodified for sm_100a) on this GPU:
    the six launches of one forward+backward, alone and inside the unfused chain the model executes
    (QK -> +mask -> softmax -> AV, and its backward; models/PCF_NATransformer.py:141-150). Reported beside
    the product's number, never part of it. Only shapes the reference launches as one tile per sequence."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    so = os.path.join(ref_dir, "libref_ana1d_bf16.so")
    N, T, C, win = w["B"] * w["H"], w["T"], w["C"], w["win"]
    if not os.path.exists(so) or w["dil"] != 1 or T > 256 or not w["bwd"]:
        return None
    lib = ctypes.CDLL(so)
    for nm in ("ref_ana_qk_forward", "ref_ana_band_x", "ref_ana_bandT_x"):
        getattr(lib, nm).argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 5
        getattr(lib, nm).restype = ctypes.c_int
    left = win - 1 - win // 2
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    q, k, v, d_o = (x.to(dev) for x in host)
    attn = torch.empty(N, T, win, dtype=torch.float32, device=dev)
    attn_gd = torch.empty_like(attn)
    out, q_gd, k_gd, v_gd = (torch.empty_like(q) for _ in range(4))
    j = torch.arange(T, device=dev).unsqueeze(1) + torch.arange(win, device=dev).unsqueeze(0) - left
    mask = torch.where((j < 0) | (j >= T), -100.0, 0.0).unsqueeze(0)
    torch.cuda.synchronize()

    def kernels_only():
        lib.ref_ana_qk_forward(P(attn), P(q), P(k), N, T, C, win, left)
        lib.ref_ana_band_x(P(out), P(attn), P(v), N, T, C, win, left)
        lib.ref_ana_qk_forward(P(attn_gd), P(d_o), P(v), N, T, C, win, left)
        lib.ref_ana_bandT_x(P(v_gd), P(attn), P(d_o), N, T, C, win, left)
        lib.ref_ana_band_x(P(q_gd), P(attn_gd), P(k), N, T, C, win, left)
        lib.ref_ana_bandT_x(P(k_gd), P(attn_gd), P(q), N, T, C, win, left)

    def chain():
        lib.ref_ana_qk_forward(P(attn), P(q), P(k), N, T, C, win, left)
        p = torch.softmax(attn + mask, -1)
        lib.ref_ana_band_x(P(out), P(p), P(v), N, T, C, win, left)
        lib.ref_ana_qk_forward(P(attn_gd), P(d_o), P(v), N, T, C, win, left)
        lib.ref_ana_bandT_x(P(v_gd), P(p), P(d_o), N, T, C, win, left)
        ds = (p * (attn_gd - (p * attn_gd).sum(-1, keepdim=True))).contiguous()
        lib.ref_ana_band_x(P(q_gd), P(ds), P(k), N, T, C, win, left)
        lib.ref_ana_bandT_x(P(k_gd), P(ds), P(q), N, T, C, win, left)

    res = {}
    with torch.cuda.stream(torch.cuda.default_stream(dev)):   # the reference launches on the legacy default stream
        for name, fn in (("kernels_only", kernels_only), ("unfused_chain", chain)):
            us = _time_fn(fn, iters)
            res[name] = {"us_per_step": us, "queries_per_s": N * T / (us * 1e-6)}
    res["note"] = "reference na1d_tensorcore bf16 kernels compiled for sm_100a, same GPU, same shape, single buffer set (L2-warm)"
    return res


def compat_pair_timing(L, w, dev, host, ref, iters=30):
    """The unfused drop-in pair of this library (the six entry points an unmodified model file reaches through
    `getNA1dFunction`), timed like `reference_cuda_baseline`: the six launches alone and inside the unfused chain."""
    N, T, C, win, dil = w["B"] * w["H"], w["T"], w["C"], w["win"], w["dil"]
    if not w["bwd"]:
        return None
    left = win - 1 - win // 2
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    q, k, v, d_o = (x.to(dev) for x in host)
    attn = torch.empty(N, T, win, dtype=torch.float32, device=dev)
    attn_gd = torch.empty_like(attn)
    out, q_gd, k_gd, v_gd = (torch.empty_like(q) for _ in range(4))
    j = torch.arange(T, device=dev).unsqueeze(1) + (torch.arange(win, device=dev).unsqueeze(0) - left) * dil
    mask = torch.where((j < 0) | (j >= T), -100.0, 0.0).unsqueeze(0)
    stream = torch.cuda.Stream(dev)
    res = {}
    with torch.cuda.stream(stream):
        st = ctypes.c_void_p(stream.cuda_stream)

        def call(fn, a, b, c):
            rc = getattr(L, fn)(P(a), P(b), P(c), N, T, C, win, left, dil, 0, st)
            assert rc == 0, (fn, rc)

        def kernels_only():
            call("na1d_qk_forward", attn, q, k)
            call("na1d_av_forward", out, attn, v)
            call("na1d_a_backward", attn_gd, d_o, v)
            call("na1d_v_backward", v_gd, attn, d_o)
            call("na1d_q_backward", q_gd, attn_gd, k)
            call("na1d_k_backward", k_gd, attn_gd, q)

        def chain():
            call("na1d_qk_forward", attn, q, k)
            p = torch.softmax(attn + mask, -1)
            call("na1d_av_forward", out, p, v)
            call("na1d_a_backward", attn_gd, d_o, v)
            call("na1d_v_backward", v_gd, p, d_o)
            ds = (p * (attn_gd - (p * attn_gd).sum(-1, keepdim=True))).contiguous()
            call("na1d_q_backward", q_gd, ds, k)
            call("na1d_k_backward", k_gd, ds, q)

        for name, fn in (("kernels_only", kernels_only), ("unfused_chain", chain)):
            us = _time_fn(fn, iters, stream)
            res[name] = {"us_per_step": us, "queries_per_s": N * T / (us * 1e-6)}
            if ref and name in ref:
                res[name]["speedup_vs_reference_cuda"] = ref[name]["us_per_step"] / us
    res["note"] = "the six unfused entry points of this library, same shape and buffers as reference_cuda (single buffer set, L2-warm)"
    return res


def cpu_baseline(w, budget_s=12.0):
    """The fp32 oracle timed on the host cores on a bounded sample of the same workload."""
    from oracle import na1d_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    left = w["win"] - 1 - w["win"] // 2
    N = w["B"] * w["H"]
    n_s = min(N, 128)
    q, k, v, d_o = (x[:n_s].float() for x in make_host_inputs(w))

    def step():
        if w["bwd"]:
            orc.na1d_fused_with_grads(q, k, v, d_o, w["win"], left, w["dil"], 1.0, None, None, w["H"])
        else:
            orc.na1d_fused(q, k, v, w["win"], left, w["dil"], 1.0, None, None, w["H"])

    step()
    t0 = time.perf_counter()
    n = 0
    while time.perf_counter() - t0 < budget_s and n < 200:
        step()
        n += 1
    dt = time.perf_counter() - t0
    return {"value": n * n_s * w["T"] / dt, "unit": "queries/s", "cores": cores, "kind": "port",
            "sample": "%d of %d sequences x %d passes (%.1f s), fp32 eager oracle" % (n_s, N, n, dt)}


# ------------------------------------------------------------------------------------------ shape sweep
def run_sweep(args):
    """Forward and forward+backward time of every (dtype, window, dilation, length, head dim) of the sweep
    (64 utterances x 4 heads, inputs scaled by D^-1/4) plus the named shapes, as a markdown table."""
    from pcf_nat_b200 import _lib, ops
    if not torch.cuda.is_available():
        raise SystemExit("the sweep needs a CUDA device")
    L = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, peak_kind = peaks()
    cases = list(itertools.product((torch.bfloat16, torch.float16), (3, 7, 15, 31), (1, 2, 4), (200, 400, 1000), (32, 64)))
    if args.quick:
        cases = [c for c in cases if c[0] == torch.bfloat16 and c[3] in (200, 1000) and c[4] == 64 and c[1] in (7, 15, 31)]
    named = [("training shape", torch.bfloat16, 7, 1, 200, 64, 128, 4), ("long utterance", torch.bfloat16, 15, 1, 3000, 64, 16, 8),
             ("reference yaml", torch.bfloat16, 27, 1, 150, 16, 512, 16)]
    lines = ["fractions are of the %s copy bandwidth %.1f GB/s; graph of 20 steps, median of 11 replays" % (peak_kind, peak), "",
             "| case | dtype | win | dil | L | D | N | family fwd/bwd | fwd us | fwd frac | fwd+bwd us | fwd+bwd Gq/s | fwd+bwd frac |",
             "|---|---|---|---|---|---|---|---|---|---|---|---|---|"]
    print("\n".join(lines), flush=True)

    def row(tag, dtype, win, dil, T, C, b, h):
        N = b * h
        ob = OpBench(L, dev, N, h, T, C, win, dil, dtype, True, scale=C ** -0.25)
        fam = "%s/%s" % tuple(["cuda-core", "tcgen05"][L.na1d_fused_kernel_family(N, T, C, win, ob.left, dil, ob.code, bw)] for bw in (0, 1))
        t_f = 1e3 * ob.timed(20, "fwd", 11)[0] / 20
        t_b = 1e3 * ob.timed(20, "both", 11)[0] / 20
        ops.device_status()
        fb, tb = 8 * N * T * C + 4 * N * T, 24 * N * T * C + 8 * N * T
        lines.append("| %s | %s | %d | %d | %d | %d | %d | %s | %.1f | %.2f | %.1f | %.2f | %.2f |" % (
            tag, "bf16" if ob.code == 0 else "fp16", win, dil, T, C, N, fam, t_f, fb / t_f / 1e3 / peak, t_b,
            N * T / t_b / 1e3, tb / t_b / 1e3 / peak))
        print(lines[-1], flush=True)
        del ob
        torch.cuda.empty_cache()

    for tag, dtype, win, dil, T, C, b, h in named:
        row(tag, dtype, win, dil, T, C, b, h)
    for dtype, win, dil, T, C in cases:
        row("sweep", dtype, win, dil, T, C, 64, 4)
    with open(args.sweep, "w") as f:
        f.write("\n".join(lines) + "\n")


def run_host_cost(args):
    """Host time of one forward+backward pair of C-ABI calls at a small shape (32 sequences: the kernels take a few
    microseconds, the host side dominates), in a tight loop on reused buffers. Run once as is and once with
    NA1D_TENSOR_MAP_CACHE=0 in the environment to see what the tensor-map cache saves."""
    from pcf_nat_b200 import _lib, ops
    L = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    ob = OpBench(L, dev, 32, 4, 200, 64, 7, 1, torch.bfloat16, True)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    s = ob.sets[0]
    for _ in range(50):
        ob._fwd(s, st); ob._bwd(s, st)
    torch.cuda.synchronize()
    h0, m0 = ops.tensor_map_cache_stats()
    n = 2000
    t0 = time.perf_counter()
    for _ in range(n):
        ob._fwd(s, st); ob._bwd(s, st)
    host_us = (time.perf_counter() - t0) / n * 1e6
    torch.cuda.synchronize()
    wall_us = (time.perf_counter() - t0) / n * 1e6
    h1, m1 = ops.tensor_map_cache_stats()
    ops.device_status()
    print(json.dumps({"what": "host time of one na1d_fused_forward + na1d_fused_backward call pair, N=32 T=200 C=64 win=7",
                      "tensor_map_cache": os.environ.get("NA1D_TENSOR_MAP_CACHE", "1") != "0", "host_us_per_pair": host_us,
                      "wall_us_per_pair_incl_gpu": wall_us, "cache_hits": h1 - h0, "cache_misses": m1 - m0, "pairs": n}), flush=True)


def run_layer_cost(args):
    """Forward+backward time of one whole attention layer at the reference's own layer shape (512 utterances, 150 frames,
    dim 256, 16 heads, window 27, groups 8; models/PCF_NATransformer.py:44-178 and the MFA twin), bf16 autocast, for both
    layouts: through the strided tensor maps (no head split / merge copies) and with the copies around the dense operator."""
    import pcf_nat_b200.nattention as mod
    from pcf_nat_b200 import NAttention, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    N, T, dim, heads, win = 512, 150, 256, 16, 27
    out = {"what": "one NAttention layer forward+backward, N=512 T=150 dim=256 heads=16 win=27, bf16 autocast, us per call"}
    real_supported = ops.packed_supported
    for layout, groups in (("channels_first", 8), ("channels_last", 1)):
        torch.manual_seed(0)
        layer = NAttention(T, dim, heads, win, groups=groups, layout=layout).to(dev)
        x = torch.randn((N, dim, T) if layout == "channels_first" else (N, T, dim), device=dev, requires_grad=True)

        def step():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = layer(x)
            y.backward(torch.ones_like(y))
        for name, fn in (("strided", real_supported), ("copies", lambda *a, **k: False)):
            ops.packed_supported = fn
            mod.ops.packed_supported = fn
            g = torch.cuda.CUDAGraph()
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            with torch.cuda.graph(g):
                step()
            out["%s_%s" % (layout, name)] = _time_fn(g.replay, 50)
    ops.packed_supported = real_supported
    ops.device_status()
    print(json.dumps(out), flush=True)


def run_bias_cost(args):
    """What the layer's relative-position bias, its gradient and the padding masks cost in the fused kernels
    (models/PCF_NATransformer.py:141-150 adds all three; the operator workloads above time the bare kernels, as the
    reference's own kernels know none of them): forward and backward microseconds over rotating buffer sets, plain launches,
    CUDA events, at the training shape and at the reference's own shape."""
    import ctypes
    from pcf_nat_b200 import _lib, ops
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    out = {"what": "fused forward / backward us per launch (bf16): bare, + rpb, + rpb and d_rpb, + rpb, d_rpb and valid_len"}
    for name in ("cfg2_train_B128_H4_L200_D64_w7", "real_B512_H16_L150_D16_w27"):
        w = WORKLOADS[name]
        N, H, T, C, win = w["B"] * w["H"], w["H"], w["T"], w["C"], w["win"]
        left = win // 2
        g = torch.Generator(device=dev).manual_seed(0)
        sets = []
        for _ in range(4):
            q, k, v, do = (torch.randn(N, T, C, device=dev, generator=g).to(torch.bfloat16) for _ in range(4))
            sets.append((q, k, v, do) + tuple(torch.empty_like(q) for _ in range(4)) + (torch.empty(N, T, device=dev), torch.empty(N, T, device=dev)))
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rows = {}
        for label, use_rpb, use_drpb, use_vl in (("bare", 0, 0, 0), ("rpb", 1, 0, 0), ("rpb_drpb", 1, 1, 0), ("rpb_drpb_valid_len", 1, 1, 1)):
            rpb = 0.1 * torch.randn(H, win, device=dev, generator=g) if use_rpb else None
            drpb = torch.zeros(H, win, device=dev) if use_drpb else None
            vl = torch.full((N // H,), T - 5, dtype=torch.int32, device=dev) if use_vl else None
            i = [0]

            def fwd():
                q, k, v, do, o, dq, dk, dv, lse, ws = sets[i[0] % 4]
                assert lib.na1d_fused_forward(ptr(o), ptr(lse), ptr(q), ptr(k), ptr(v), ptr(rpb), ptr(vl), N, H, T, C, win, left, 1, C ** -0.5, 0, st) == 0

            def bwd():
                q, k, v, do, o, dq, dk, dv, lse, ws = sets[i[0] % 4]
                i[0] += 1
                assert lib.na1d_fused_backward(ptr(dq), ptr(dk), ptr(dv), ptr(drpb), ptr(do), ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), ptr(rpb), ptr(vl),
                                               ptr(ws), N, H, T, C, win, left, 1, C ** -0.5, 0, st) == 0
            for _ in range(4):
                fwd(); bwd()
            rows[label] = {"fwd_us": round(_time_fn(fwd, 20), 1), "bwd_us": round(_time_fn(bwd, 20), 1)}
        out[name] = rows
    ops.device_status()
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--replays", type=int, default=101, help="replays of the graph of --steps steps; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT, choices=list(WORKLOADS) + list(MODEL_WORKLOADS))
    ap.add_argument("--ref-budget", type=float, default=90.0, help="seconds of CPU work for --impl reference")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sweep", default=None, metavar="OUT.md", help="run the shape sweep and write the table to this file")
    ap.add_argument("--quick", action="store_true", help="with --sweep: a bf16, D=64 subset")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"], help="model workloads: split or replicate the batch")
    ap.add_argument("--attention", default="fused", choices=["fused", "unfused"], help="model workloads: operator variant")
    ap.add_argument("--precision", default="autocast", choices=["bf16", "autocast"],
                    help="model workloads: bf16 weights/activations with fp32 master weights, or bf16 autocast over fp32 parameters")
    ap.add_argument("--crop-batches", action="store_true",
                    help="cfg5_embed: cut every length-sorted batch to its own longest utterance (the reference's length-bucketed loader)")
    ap.add_argument("--layer-cost", action="store_true", help="whole attention layer, strided route against the copying route")
    ap.add_argument("--host-cost", action="store_true", help="host microseconds per forward+backward C-ABI call pair at a small shape")
    ap.add_argument("--bias-cost", action="store_true", help="fused kernels with the layer's bias, its gradient and padding masks")
    args = ap.parse_args()
    if args.host_cost:
        return run_host_cost(args)
    if args.bias_cost:
        return run_bias_cost(args)
    if args.layer_cost:
        return run_layer_cost(args)
    if args.sweep:
        return run_sweep(args)
    if args.workload in MODEL_WORKLOADS:
        from pcf_nat_b200 import model_bench
        return model_bench.run(args)
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w, args.workload)
    else:
        run_ours(args, w, args.workload)


if __name__ == "__main__":
    main()

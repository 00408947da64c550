"""Model-level workloads of the benchmark: the PCF-NAT-style extractor, batch-sharded over the GPUs of one box.

    python bench.py --workload cfg5_train [--gpus N] [--steps K] [--warmup W] [--scaling strong|weak] [--attention fused|unfused]
    python bench.py --workload cfg5_embed [--gpus N] ...
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench.py --workload cfg5_train --gpus N ...

One process per GPU. The operator itself never exchanges data; the only collectives are

* training: ONE all-reduce per step of the flattened fp32 gradients (every ``p.grad`` is a view into one buffer), between
  two CUDA-graph replays: graph A = zero gradients + forward + backward, graph B = the AdamW update. No NCCL call is ever
  inside a capture (a whole-step capture around DistributedDataParallel ran into the time limit here once and is not
  used); the step is launch-light on every rank count. Follows the step of the reference's ``train_main.py:53-95``
  (autocast forward, backward, optimizer) with synthetic log-mel features.
* extraction: ONE all-gather of the ``(utterances/ranks, 192)`` embeddings per pass. Follows ``evaluate_main.py:59-91``
  (``cal_emb``: batches of up to 512 utterances, mean normalisation over the valid frames, ``lens`` -> padding masks inside
  the attention layers, forward under ``no_grad`` + autocast).

Device time (CUDA events), barrier on both sides, max over ranks; rank 0 prints one JSON line.
"""
import datetime
import json
import os
import statistics

import torch

FRAMES, FEAT, CLASSES, EMB = 300, 80, 5994, 192


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d.get("bf16_tflops_sustained", 1371.6)), "measured"
    return 1400.0, "fallback"


def _setup():
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("the model workloads need a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # a short collective timeout: a rank that fails must end the job instead of leaving the others waiting
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    return world, rank, local, dev


def _timed_steps(step, n, dev, world):
    """Device time of n calls of step() in ms (barrier + synchronize on both sides), max over ranks."""
    from . import parallel
    torch.cuda.synchronize()
    parallel.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    torch.cuda.synchronize()
    parallel.barrier()
    return parallel.max_over_ranks(e0.elapsed_time(e1), dev)


def _bf16_body(model, dev):
    """Mixed precision without autocast: the body of the network (front end, attention stages, fusion, pooling) gets bf16
    weights that are views into ONE flat bf16 buffer, refreshed after every update from an fp32 master copy; the small tail
    (batch norm, embedding, loss) stays fp32 as views into the same master. Returns (master fp32 flat parameter, flat bf16
    body weights, number of body elements, body parameters, tail parameters)."""
    tail_mods = (model.bn, model.embed, model.loss)
    tail_ids = {id(p) for m in tail_mods for p in m.parameters()}
    body = [p for p in model.parameters() if id(p) not in tail_ids]
    tail = [p for p in model.parameters() if id(p) in tail_ids]
    master = torch.cat([p.detach().float().reshape(-1) for p in body + tail]).to(dev)
    nb = sum(p.numel() for p in body)
    flat_w = master[:nb].to(torch.bfloat16)
    off = 0
    for p in body:
        p.data = flat_w[off:off + p.numel()].view_as(p)
        off += p.numel()
    for p in tail:
        p.data = master[off:off + p.numel()].view_as(p)
        off += p.numel()
    return torch.nn.Parameter(master), flat_w, nb, body, tail


class TrainStep:
    """forward + backward + gradient all-reduce + AdamW of the extractor on one rank's share of the batch.

    precision "bf16" (default): bf16 weights and activations in the body with fp32 master weights, fp32 gradients for the
    all-reduce and the update (no autocast: no per-call weight and activation casts); "autocast": fp32 parameters under
    ``torch.autocast(bfloat16)`` as the reference's ``train_main.py`` runs."""

    def __init__(self, per_gpu, dev, world, rank, attention="fused", frames=FRAMES, use_graphs=True, precision="autocast"):
        import torch.distributed as dist
        from . import parallel
        from .model import PCFNATExtractor
        self.dist, self.world, self.dev, self.parallel, self.precision = dist, world, dev, parallel, precision
        torch.manual_seed(4)
        self.model = PCFNATExtractor(frames=frames, attention=attention).to(dev)
        g = torch.Generator(device=dev).manual_seed(4 + rank)
        self.fbank = torch.randn(per_gpu, FEAT, frames, device=dev, generator=g)
        self.labels = torch.randint(0, CLASSES, (per_gpu,), device=dev, generator=g)
        if precision == "bf16":
            self.master, self.flat_w, self.nb, body, tail = _bf16_body(self.model, dev)
            self.n_params = self.master.numel()
            # gradients: the body's arrive in bf16 (views into one buffer) and are widened into the fp32 buffer that is
            # all-reduced and handed to the optimizer; the tail's are views into that buffer directly
            self.flat = torch.zeros(self.n_params, dtype=torch.float32, device=dev)
            self.body_grad = torch.zeros(self.nb, dtype=torch.bfloat16, device=dev)
            off = 0
            for p in body:
                p.grad = self.body_grad[off:off + p.numel()].view_as(p)
                off += p.numel()
            for p in tail:
                p.grad = self.flat[off:off + p.numel()].view_as(p)
                off += p.numel()
            self.master.grad = self.flat
            self.opt = torch.optim.AdamW([self.master], lr=1e-4, fused=True, capturable=True)
        else:
            params = [p for p in self.model.parameters() if p.requires_grad]
            # every gradient is a view into one flat fp32 buffer: one all-reduce per step, no bucketing logic
            self.flat = parallel.flat_gradient_buffer(params)
            self.n_params = self.flat.numel()
            self.opt = torch.optim.AdamW(params, lr=1e-4, fused=True, capturable=True)
        self.loss = None
        self.graph_a = self.graph_b = None
        # eager warm-up on a side stream (cuBLAS workspaces, autotuning, AdamW state), then capture
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self._forward_backward()
                self._sync_gradients()
                self._update()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.launch = "eager"
        if use_graphs:
            self.graph_a = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph_a):
                self._forward_backward()
            self.graph_b = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph_b):
                self._update()
            self.launch = "graph A (zero grads, forward, backward) -> eager NCCL all-reduce -> graph B (AdamW)" if world > 1 else \
                "graph A (zero grads, forward, backward) -> graph B (AdamW)"

    def _forward_backward(self):
        self.flat.zero_()
        if self.precision == "bf16":
            self.body_grad.zero_()
            loss = self.model(self.fbank.to(torch.bfloat16), self.labels)
            loss.backward()
            self.flat[:self.nb].copy_(self.body_grad)
        else:
            with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=False):
                loss = self.model(self.fbank, self.labels)
            loss.backward()
        self.loss = loss.detach()

    def _sync_gradients(self):
        self.parallel.all_reduce_mean(self.flat)

    def _update(self):
        self.opt.step()
        if self.precision == "bf16":
            self.flat_w.copy_(self.master.detach()[:self.nb])

    def __call__(self):
        if self.graph_a is not None:
            self.graph_a.replay()
            self._sync_gradients()
            self.graph_b.replay()
        else:
            self._forward_backward()
            self._sync_gradients()
            self._update()
        return self.loss

    def allreduce_ms(self, n=10):
        """Time of the gradient all-reduce alone (ms per call), to name the collective's share of the step."""
        if self.world == 1:
            return 0.0
        scratch = torch.zeros_like(self.flat)
        for _ in range(3):
            self.dist.all_reduce(scratch, op=self.dist.ReduceOp.AVG)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            self.dist.all_reduce(scratch, op=self.dist.ReduceOp.AVG)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n


def run_train(args):
    from . import ops, parallel
    from .model import model_flops_per_utterance
    world, rank, local, dev = _setup()
    global_batch = 256
    lo, hi = parallel.shard_range(global_batch, world, rank) if args.scaling == "strong" else (0, global_batch)
    per_gpu = hi - lo
    ts = TrainStep(per_gpu, dev, world, rank, attention=args.attention, precision=args.precision)
    for _ in range(max(args.warmup, 3)):
        ts()
    ops.device_status()
    ms = _timed_steps(ts, args.steps, dev, world) / args.steps
    loss = float(ts.loss)
    ops.device_status()
    ar_ms = parallel.max_over_ranks(ts.allreduce_ms(), dev)

    # end to end: the features of every step come from pinned host memory, the loss goes back to the host
    host_fbank = ts.fbank.cpu().pin_memory()
    host_labels = ts.labels.cpu().pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        ts.fbank.copy_(host_fbank, non_blocking=True)
        ts.labels.copy_(host_labels, non_blocking=True)
        return float(ts())
    e2e_step()
    ms_e2e = _timed_steps(e2e_step, e2e_steps, dev, world) / e2e_steps

    total = per_gpu * world
    if rank == 0:
        peak, peak_kind = _peaks()
        tflops = model_flops_per_utterance(frames=FRAMES) * total / (ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "PCF-NAT utts/sec (training step)", "value": total / (ms * 1e-3), "unit": "utterances/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg5_train", "model": "conv 80->256, 6 stages x 4 NA blocks (dim 256, 4 heads, window 7, MLP x4), "
                       "progressive channel fusion, attentive statistics pooling, 192-d embedding, AAM-softmax over 5994 classes",
                       "global_batch": total, "per_gpu_batch": per_gpu, "frames": FRAMES, "attention": args.attention,
                       "parameters": ts.n_params, "launch": ts.launch, "parallelism": "dp%d" % world,
                       "batchnorm": "per-GPU statistics", "optimizer": "AdamW (fused)",
                       "precision": "bf16 weights and activations in the body, fp32 master weights, fp32 gradient all-reduce and update"
                       if args.precision == "bf16" else "bf16 autocast over fp32 parameters"},
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak * world, "unit": "TFLOP/s", "frac": tflops / (peak * world),
                         "traffic": None, "peak_kind": peak_kind + " sustained bf16 GEMM x ranks",
                         "note": "matmul FLOPs of the whole model (3x forward); the step is bound by PyTorch's elementwise, "
                                 "normalisation and copy kernels around the GEMMs, not by the tensor pipe"},
            "collective": {"op": "all_reduce(AVG) of the flat fp32 gradients", "bytes": ts.n_params * 4, "ms": ar_ms,
                           "share_of_step": ar_ms / ms if ms else None},
            "e2e": {"value": total / (ms_e2e * 1e-3), "unit": "utterances/s", "h2d_bytes_per_step": per_gpu * (FEAT * FRAMES * 4 + 8),
                    "d2h_bytes_per_step": 4, "steps": e2e_steps},
            "gpu_launches": None, "loss": loss}), flush=True)
    if world > 1:
        ts.dist.destroy_process_group()


class Extractor:
    """Embedding extraction of one rank's share of a set of utterances, in batches of up to `batch` utterances.

    `crop` follows the reference's length-bucketed loader (``evaluate_main.py:36-57, 118-123``: utterances sorted by length,
    every batch padded only to its own longest member): a batch is cut to its longest utterance, rounded up to 8 frames,
    before it enters the network, instead of carrying the padding of the longest utterance of the whole set."""

    def __init__(self, n_local, dev, rank, batch=512, frames=FRAMES, attention="fused", precision="autocast", crop=False):
        from .model import PCFNATExtractor
        torch.manual_seed(4)
        self.model = PCFNATExtractor(frames=frames, attention=attention).to(dev).eval()
        self.dev, self.frames, self.precision = dev, frames, precision
        if precision == "bf16":
            _bf16_body(self.model, dev)
        g = torch.Generator(device=dev).manual_seed(40 + rank)
        self.fbank = torch.randn(n_local, FEAT, frames, device=dev, generator=g)
        # utterance lengths: 2 to 3 s, sorted as the reference's length-bucketed loader delivers them
        self.lens = torch.sort(torch.randint(2 * frames // 3, frames + 1, (n_local,), device=dev, generator=g))[0]
        self.emb = torch.empty(n_local, EMB, device=dev)
        self.chunks = [(a, min(a + batch, n_local)) for a in range(0, n_local, batch)]
        # frames each batch is run at: its longest utterance (the lengths are sorted), or the whole padded length
        self.batch_frames = [min(frames, -(-int(self.lens[b - 1]) // 8) * 8) if crop else frames for a, b in self.chunks]
        self.static = {}   # (batch size, frames) -> (fbank buffer, lens buffer, output, graph)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for (a, b), tb in list(zip(self.chunks, self.batch_frames))[:1] + list(zip(self.chunks, self.batch_frames))[-1:]:
                self._embed(self.fbank[a:b, :, :tb], self.lens[a:b])
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for (a, b), tb in zip(self.chunks, self.batch_frames):
            key = (b - a, tb)
            if key in self.static:
                continue
            x, ln = self.fbank[a:b, :, :tb].clone(), self.lens[a:b].clone()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._embed(x, ln)
            self.static[key] = (x, ln, out, graph)

    def _embed(self, x, lens):
        with torch.no_grad():
            # mean normalisation over the valid frames (evaluate_main.py:78-82), then the network with padding masks
            frames = x.shape[-1]
            t = torch.arange(frames, device=x.device).view(1, 1, -1)
            mask = (t < lens.view(-1, 1, 1)).to(x.dtype)
            x = (x - (x * mask).sum(-1, keepdim=True) / lens.view(-1, 1, 1).to(x.dtype)) * mask   # padded frames are zeros
            if self.precision == "bf16":
                return self.model.embedding(x.to(torch.bfloat16), (frames - lens).to(torch.int32)).float()
            with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=False):
                return self.model.embedding(x, (frames - lens).to(torch.int32)).float()

    def run(self, source=None):
        """One pass over the local utterances; `source` = pinned host features to upload batch by batch (end to end)."""
        for (a, b), tb in zip(self.chunks, self.batch_frames):
            x, ln, out, graph = self.static[(b - a, tb)]
            x.copy_((self.fbank if source is None else source)[a:b, :, :tb], non_blocking=True)
            ln.copy_(self.lens[a:b], non_blocking=True)
            graph.replay()
            self.emb[a:b].copy_(out, non_blocking=True)
        return self.emb


def run_embed(args):
    import torch.distributed as dist
    from . import ops, parallel
    from .model import model_flops_per_utterance
    world, rank, local, dev = _setup()
    total = 4096
    if total % world:
        raise SystemExit("the utterance count %d must divide by the number of ranks" % total)
    n_local = total // world if args.scaling == "strong" else total
    ex = Extractor(n_local, dev, rank, attention=args.attention, precision=args.precision, crop=args.crop_batches)
    gathered = torch.empty(world * n_local, EMB, device=dev)

    def step(source=None):
        emb = ex.run(source)
        return parallel.all_gather_rows(emb, gathered)   # the one collective of the extraction path

    for _ in range(max(args.warmup, 3)):
        step()
    ops.device_status()
    ms = _timed_steps(step, args.steps, dev, world) / args.steps
    ops.device_status()
    finite = bool(torch.isfinite(gathered).all())
    host = ex.fbank.cpu().pin_memory()
    host_out = torch.empty(gathered.shape, dtype=gathered.dtype).pin_memory()
    e2e_steps = max(2, min(args.steps, 5))

    def e2e_step():
        out = step(host)
        if rank == 0:
            host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_step()
    ms_e2e = _timed_steps(e2e_step, e2e_steps, dev, world) / e2e_steps
    n_all = n_local * world
    if rank == 0:
        peak, peak_kind = _peaks()
        tflops = model_flops_per_utterance(frames=FRAMES) / 3 * n_all / (ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "PCF-NAT utts/sec (embedding extraction)", "value": n_all / (ms * 1e-3), "unit": "utterances/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg5_embed", "utterances": n_all, "per_gpu_utterances": n_local, "batch": 512, "frames": FRAMES,
                       "lengths": "2-3 s, sorted; padding masks inside the attention layers" +
                       ("; every batch cut to its own longest utterance" if args.crop_batches else ""), "attention": args.attention,
                       "launch": "one CUDA graph per batch size, then one all-gather of the (utterances/ranks, 192) embeddings",
                       "parallelism": "dp%d" % world, "finite": finite},
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak * world, "unit": "TFLOP/s", "frac": tflops / (peak * world),
                         "traffic": None, "peak_kind": peak_kind + " sustained bf16 GEMM x ranks"},
            "collective": {"op": "all_gather_into_tensor of the embeddings", "bytes": n_all * EMB * 4},
            "e2e": {"value": n_all / (ms_e2e * 1e-3), "unit": "utterances/s", "h2d_bytes_per_step": n_local * FEAT * FRAMES * 4,
                    "d2h_bytes_per_step": n_all * EMB * 4, "steps": e2e_steps},
            "gpu_launches": None}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run(args):
    if getattr(args, "impl", "ours") == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference's model needs its CUDA extension, data pipeline and "
                              "checkpoints; only the operator workloads have a CPU reference arm"}), flush=True)
        return
    if args.workload == "cfg5_train":
        run_train(args)
    else:
        run_embed(args)

"""Model-level benchmark: training steps of the PCF-NAT-style extractor, data-parallel over the GPUs of one box.

    python -m pcf_nat_b200.train_bench [--gpus N] [--steps K] [--warmup W] [--attention fused|unfused] [--scaling strong|weak]
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m pcf_nat_b200.train_bench --gpus N ...

One process per GPU; the batch is sharded by utterance (the operator itself never exchanges data), gradients are
all-reduced by DistributedDataParallel over NCCL. Synthetic log-mel features ~ N(0,1) stay resident on the GPU; a step is
forward + backward + all-reduce + AdamW update in bf16 autocast. Device time (CUDA events), barrier on both sides, max over
ranks; rank 0 prints one JSON line with utterances/s of the whole job.
"""
import argparse
import json
import os

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--global-batch", type=int, default=256)
    ap.add_argument("--frames", type=int, default=300)
    ap.add_argument("--attention", default="fused", choices=["fused", "unfused"])
    ap.add_argument("--launch", default="graph", choices=["graph", "eager"],
                    help="graph: the whole step (forward, backward, optimizer) is one CUDA graph replay; single GPU only -- "
                         "with more than one rank the step always runs eagerly (a captured NCCL all-reduce inside a "
                         "DistributedDataParallel step did not complete here)")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong: the global batch is split over the GPUs; weak: every GPU gets the whole global batch")
    args = ap.parse_args(argv)

    import torch.distributed as dist
    from . import parallel
    from .model import PCFNATExtractor, model_flops_per_utterance

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("the model benchmark needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        # a short collective timeout: a rank that fails must end the job instead of leaving the others waiting
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
        args.launch = "eager"
    lo, hi = parallel.shard_range(args.global_batch, world, rank) if args.scaling == "strong" else (0, args.global_batch)
    per_gpu = hi - lo

    torch.manual_seed(4)
    model = PCFNATExtractor(frames=args.frames, attention=args.attention).to(dev)
    n_params = sum(p.numel() for p in model.parameters())
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    fbank = torch.randn(per_gpu, 80, args.frames, device=dev, generator=g)
    labels = torch.randint(0, 5994, (per_gpu,), device=dev, generator=g)
    # DistributedDataParallel and the eager warm-up run on a side stream, as whole-step graph capture requires
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
        opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True, capturable=args.launch == "graph")

        def eager_step():
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=False):
                loss = net(fbank, labels)
            loss.backward()
            opt.step()
            return loss

        for _ in range(max(args.warmup, 3)):
            loss = eager_step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    launch = "eager"
    step = eager_step
    if args.launch == "graph":
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_loss = eager_step()
            launch = "graph"

            def step():
                graph.replay()
                return static_loss
        except Exception as e:  # capture is an optimisation of the launch path only: say so and time the eager step
            if rank == 0:
                print("whole-step graph capture failed (%s: %s); timing the eager step" % (type(e).__name__, e), flush=True)
            torch.cuda.synchronize()
    for _ in range(args.warmup):
        loss = step()
    torch.cuda.synchronize()
    parallel.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    parallel.barrier()
    ms = parallel.max_over_ranks(e0.elapsed_time(e1) / args.steps, dev)
    total_utts = per_gpu * world
    if rank == 0:
        flops = model_flops_per_utterance(frames=args.frames) * total_utts / (ms * 1e-3)
        print(json.dumps({
            "metric": "PCF-NAT-style extractor training utterances/sec", "value": total_utts / (ms * 1e-3), "unit": "utterances/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": args.scaling, "dtype": "bf16 autocast", "data": "synthetic",
            "config": {"workload": "cfg5_model_6x4_dim256_h4_w7", "global_batch": total_utts, "per_gpu_batch": per_gpu,
                       "frames": args.frames, "attention": args.attention, "parameters": n_params, "launch": launch,
                       "parallelism": "dp%d" % world},
            "model_tflops": flops / 1e12, "loss": float(loss.detach())}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Host-side logic of the multi-GPU path, run as two gloo ranks on the CPU."""
import json
import os
import subprocess
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from pcf_nat_b200 import parallel
    x = torch.arange(10 * 4 * 3 * 2, dtype=torch.float32).reshape(40, 3, 2)   # batch 10, heads 4
    (mine,) = parallel.shard_batch([x], heads=4, world=world, rank=rank)
    slowest = parallel.max_over_ranks(1.0 + rank)
    parallel.barrier()
    gathered = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, torch.tensor([mine.shape[0]]))
    if rank == 0:
        out.put((int(sum(g.item() for g in gathered)), slowest, mine.shape[0], float(mine[0, 0, 0])))
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_by_utterance_and_agree_on_slowest_rank():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    total, slowest, n0, first = out.get()
    assert total == 40 and n0 == 20 and first == 0.0
    assert slowest == 2.0


def _dp_worker(rank, world, port, out):
    """Data-parallel step of a small model on this rank's half of the batch: flat gradients, one mean all-reduce; and the
    embedding all-gather of the extraction path."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from pcf_nat_b200 import parallel
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
    x, y = torch.randn(8, 6), torch.randn(8, 3)
    flat = parallel.flat_gradient_buffer(net.parameters())
    lo, hi = parallel.shard_range(8, world, rank)
    for _ in range(2):   # the second pass checks that zeroing the flat buffer resets every view
        flat.zero_()
        torch.nn.functional.mse_loss(net(x[lo:hi]), y[lo:hi]).backward()
        assert all(p.grad.data_ptr() >= flat.data_ptr() for p in net.parameters()), "a gradient left the flat buffer"
        parallel.all_reduce_mean(flat)
    emb = net(x[lo:hi]).detach()
    rows = parallel.all_gather_rows(emb)
    if rank == 0:
        out.put((flat.clone(), rows.clone()))
    dist.destroy_process_group()


def test_two_gloo_ranks_flat_gradient_allreduce_and_embedding_gather():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    flat, rows = out.get()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    # single-process result on the whole batch: equal shards, mean-reduced losses -> the mean of the shard gradients
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
    x, y = torch.randn(8, 6), torch.randn(8, 3)
    torch.nn.functional.mse_loss(net(x), y).backward()
    ref = torch.cat([p.grad.reshape(-1) for p in net.parameters()])
    torch.testing.assert_close(flat, ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(rows, net(x).detach(), rtol=1e-5, atol=1e-6)


def test_shard_range_is_a_partition():
    from pcf_nat_b200.parallel import shard_range
    for total in (0, 1, 7, 128, 129):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_reference_arm_under_two_ranks_prints_one_line():
    """`bench.py --impl reference` launched as two ranks: rank 0 measures and prints, rank 1 exits 0 silently."""
    env = dict(os.environ, WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29999")
    outs = []
    for rank in (0, 1):
        e = dict(env, RANK=str(rank), LOCAL_RANK=str(rank))
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                            "--steps", "1", "--warmup", "0", "--ref-budget", "2"], env=e, capture_output=True, text=True,
                           timeout=300)
        assert r.returncode == 0, r.stderr
        outs.append(r.stdout.strip())
    assert outs[1] == ""
    line = json.loads(outs[0].splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0

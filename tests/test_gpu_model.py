"""The PCF-NAT-style extractor on the GPU: the fused layer (packed-projection route) against the reference's unfused
operator chain inside the same network, one training step through the benchmark's own step object, and the extraction loop."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _small(attention):
    from pcf_nat_b200.model import PCFNATExtractor
    torch.manual_seed(11)
    return PCFNATExtractor(frames=96, feat=24, dim=64, heads=2, win=7, stages=2, blocks=2, emb=32, classes=40, attention=attention).cuda()


def test_fused_and_unfused_networks_agree():
    fused, unfused = _small("fused"), _small("unfused")
    unfused.load_state_dict(fused.state_dict())
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(6, 24, 96, device="cuda", generator=g)
    y = torch.randint(0, 40, (6,), device="cuda", generator=g)
    losses, grads = [], []
    for m in (fused, unfused):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = m(x, y)
        loss.backward()
        losses.append(float(loss.detach()))
        grads.append(torch.cat([p.grad.reshape(-1).float() for p in m.parameters()]))
    assert abs(losses[0] - losses[1]) < 2e-2 * max(1.0, abs(losses[1])), losses
    rel = float((grads[0] - grads[1]).norm() / grads[1].norm())
    assert rel < 5e-2, rel
    from pcf_nat_b200 import ops
    ops.device_status()


def test_training_step_object_runs_and_learns():
    """The benchmark's step (graph A -> all-reduce -> graph B) on one GPU: finite loss that falls on a repeated batch."""
    from pcf_nat_b200 import model_bench, ops
    ts = model_bench.TrainStep(8, torch.device("cuda", 0), 1, 0, frames=96)
    first = float(ts())
    for _ in range(15):
        last = float(ts())
    assert first == first and last == last and last < first, (first, last)
    ops.device_status()


def test_extraction_loop_with_and_without_batch_cropping():
    """Padded frames must not change an utterance's embedding much: the batch cut to its longest utterance (the
    length-bucketed loader) gives the embeddings of the uncropped batch."""
    from pcf_nat_b200 import model_bench, ops
    dev = torch.device("cuda", 0)
    full = model_bench.Extractor(40, dev, 0, batch=16, frames=96)
    crop = model_bench.Extractor(40, dev, 0, batch=16, frames=96, crop=True)
    assert min(crop.batch_frames) < 96 and all(t % 8 == 0 for t in crop.batch_frames)
    a, b = full.run().clone(), crop.run().clone()
    torch.cuda.synchronize()
    assert torch.isfinite(a).all() and torch.isfinite(b).all()
    ops.device_status()
    # the attention layers mask the padding exactly; the convolutional front end and the pooling see it, so the two are
    # close, not equal
    rel = float((a - b).norm() / a.norm())
    assert rel < 0.5, rel

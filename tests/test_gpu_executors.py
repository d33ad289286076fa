"""The two executors around a layer: CapturedForward (CUDA-graph replay) and StreamingForward
(host-to-host pipeline over three streams). Both must give exactly what the eager forward gives
on the same tokens, for every batch and in submission order."""
import pytest
import torch

import fast_moe_b200 as fm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _layer(d=128, h=256, E=8):
    torch.manual_seed(7)
    return fm.SwiGLUFastMoELayer(d, h, d, E, dtype=torch.bfloat16).to(DEV)


def _batches(n, tokens, d, seed=3):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(1, tokens, d, generator=g) * (1 + i)).bfloat16().pin_memory() for i in range(n)]


def test_captured_forward_replays_match_eager():
    layer = _layer()
    xs = _batches(4, 300, 128)
    cap = fm.CapturedForward(layer, xs[0].to(DEV), 2)
    for x in xs:
        want = layer(x.to(DEV), 2)
        got = cap(x.to(DEV)).clone()
        assert torch.equal(got, want)
    # replay() reuses whatever sits in the static input
    assert torch.equal(cap.replay(), layer(xs[-1].to(DEV), 2))


@pytest.mark.parametrize("slots,capture", [(1, True), (2, True), (3, True), (2, False)])
def test_streaming_forward_matches_eager_for_every_batch(slots, capture):
    layer = _layer()
    xs = _batches(7, 257, 128)
    want = [layer(x.to(DEV), 2).cpu() for x in xs]
    pipe = fm.StreamingForward(layer, xs[0].to(DEV), 2, slots=slots, capture=capture)
    outs = [torch.empty(1, 257, 128, dtype=torch.bfloat16).pin_memory() for _ in xs]
    for x, y in zip(xs, outs):
        pipe.submit(x, y)
    pipe.drain()
    torch.cuda.synchronize()
    for i, (y, w) in enumerate(zip(outs, want)):
        assert torch.equal(y, w), f"batch {i}"
    # a second round through the same slots (buffers are reused)
    for x, y in zip(reversed(xs), outs):
        pipe.submit(x, y)
    pipe.synchronize()
    for i, (y, w) in enumerate(zip(outs, reversed(want))):
        assert torch.equal(y, w), f"second round, batch {i}"


def test_streaming_forward_refuses_cpu_example():
    layer = _layer()
    with pytest.raises(RuntimeError, match="CUDA"):
        fm.StreamingForward(layer, torch.zeros(1, 4, 128, dtype=torch.bfloat16), 2)


@pytest.mark.parametrize("slots", [1, 3])
def test_host_pipeline_matches_eager_for_every_batch(slots):
    """One graph launch per batch (copy-in, forward and copy-out of a slot captured together):
    every batch's result equals the eager forward, across several rounds through the slots."""
    layer = _layer()
    xs = _batches(7, 257, 128)
    want = [layer(x.to(DEV), 2).cpu() for x in xs]
    pipe = fm.HostPipeline(layer, xs[0].to(DEV), 2, slots=slots)
    for i, x in enumerate(xs):
        s = i % slots
        pipe.wait(s)                      # the slot's previous batch has been read out
        if i >= slots:
            assert torch.equal(pipe.host_out[s], want[i - slots]), f"batch {i - slots}"
        pipe.host_in[s].copy_(x)
        pipe.launch(s)
    pipe.synchronize()
    for i in range(max(0, len(xs) - slots), len(xs)):
        assert torch.equal(pipe.host_out[i % slots], want[i]), f"batch {i}"

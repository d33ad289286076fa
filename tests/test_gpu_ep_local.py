"""The peer-memory expert-parallel exchange on ONE GPU: W logical ranks live in one process, each
with its own tokens, its own expert shard and its own "peer" buffers (plain device tensors linked
by address), and the test drives the phases of all ranks in order - route, counts, plan +
dispatch, experts (the down projection stores into the owners' return buffers), combine. The
kernels, address arithmetic and layouts are exactly those of the multi-GPU layer; only the
transport differs (every "peer" address is local). Each rank's result must equal the CPU oracle
of the whole model on that rank's tokens. Kernels of different ranks never wait for one another
here: each phase is a separate launch that completes before the next phase starts."""
import pytest
import torch

import fast_moe_b200 as fm
from fast_moe_b200 import _lib
from fast_moe_b200.modules.expert_parallel import (ROUTE_SHIFT, ExpertParallelSwiGLUMoE, PeerBuffers,
                                                   peer_exchange_plan)
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _make_ranks(W, E, d, h, o, tokens_cap, k, seed=5):
    layers = [ExpertParallelSwiGLUMoE(d, h, o, E, dtype=torch.bfloat16, device=DEV, seed=seed, world_size=W, rank=r)
              for r in range(W)]
    for l in layers:
        l.setup_peer_buffers(tokens_cap, k, symmetric=False)
    PeerBuffers.link_local([l.peers for l in layers])
    return layers


def _full_model(layers):
    f = lambda name: torch.cat([getattr(l, name).detach() for l in layers]).float().cpu()
    return f("w_gate"), f("w_up"), f("w_down")


def _run_exchange(layers, xs, k):
    routed = [l.ep_route(x, k) for l, x in zip(layers, xs)]
    counts = torch.stack([meta.lengths for _, meta in routed])              # what the all-gather delivers
    for l, x, (_, meta) in zip(layers, xs, routed):
        l.ep_dispatch(x, meta, counts)
    for l in layers:
        l.ep_experts(rows_hint=max(1, xs[0].shape[0] * k))
    return [l.ep_combine(score, meta, k) for l, (score, meta) in zip(layers, routed)], counts, routed


@pytest.mark.parametrize("W,E,k,tokens", [(2, 8, 2, [300, 317]), (4, 16, 2, [64, 0, 200, 129]), (8, 64, 2, [150] * 8),
                                           (4, 8, 4, [100, 90, 80, 70]), (2, 4, 1, [33, 5])])
def test_peer_exchange_equals_oracle_on_every_rank(W, E, k, tokens):
    d, h, o = 128, 256, 128
    layers = _make_ranks(W, E, d, h, o, max(tokens), k)
    xs_cpu = [torch.randn(L, d, generator=torch.Generator().manual_seed(50 + r)).bfloat16() for r, L in enumerate(tokens)]
    xs = [x.to(DEV) for x in xs_cpu]
    for _ in range(2):                       # the second pass reuses every buffer the first one filled
        ys, counts, routed = _run_exchange(layers, xs, k)
    torch.cuda.synchronize()
    assert _lib.device_status(DEV) == 0
    wg, wu, wd = _full_model(layers)
    gate_w = layers[0].gate.weight.detach().float().cpu()
    gate_b = layers[0].gate.bias.detach().float().cpu()
    for r, (y, x) in enumerate(zip(ys, xs_cpu)):
        assert y.shape == (tokens[r], o)
        if tokens[r] == 0:
            continue
        ref = O.moe_layer_swiglu(x.float(), gate_w, gate_b, wg.permute(0, 2, 1), wu.permute(0, 2, 1),
                                 wd.permute(0, 2, 1), k)
        err = (y.float().cpu() - ref).abs()
        bad = (err > 1e-2 + 1e-2 * ref.abs()).any(dim=-1).float().mean().item()
        assert bad < 0.02, f"rank {r}: {bad:.2%} of tokens outside rtol/atol 1e-2 (max err {err.max().item():.3e})"
    # the plan kernel's outputs equal the tensor-arithmetic statement of the layout
    for r, l in enumerate(layers):
        dst_base, off_local = peer_exchange_plan(counts.cpu(), r)
        assert torch.equal(l._work["dst_base"].cpu(), dst_base)
        assert torch.equal(l._work["offsets_local"].cpu(), off_local)
        # every received row carries a valid return address: (source rank, row of that source)
        n = int(off_local[-1])
        route = l.peers.route[:n].cpu()
        src = route >> ROUTE_SHIFT
        row = route & ((1 << ROUTE_SHIFT) - 1)
        assert bool(((src >= 0) & (src < W)).all())
        assert bool((row < torch.tensor([t * k for t in tokens])[src]).all())
    # all return addresses together cover every rank's rows exactly once
    seen = torch.cat([l.peers.route[: int(l._work["offsets_local"][-1])].cpu() for l in layers])
    assert seen.unique().numel() == seen.numel() == sum(tokens) * k


def test_peer_exchange_equals_single_gpu_layer_bitwise_routing():
    """W = 1 of the same class and the W = 4 exchange see identical routing, and their outputs
    agree within the bf16 tolerance (different tile shapes / accumulation order only)."""
    W, E, k, d, h, o, L = 4, 8, 2, 256, 512, 256, 400
    layers = _make_ranks(W, E, d, h, o, L, k, seed=9)
    whole = ExpertParallelSwiGLUMoE(d, h, o, E, dtype=torch.bfloat16, device=DEV, seed=9, world_size=1)
    xs = [torch.randn(L, d, generator=torch.Generator().manual_seed(7 + r)).bfloat16().to(DEV) for r in range(W)]
    ys, _, routed = _run_exchange(layers, xs, k)
    for r in range(W):
        y1 = whole(xs[r].view(1, L, d), k).view(L, o)
        s1, m1 = whole.ep_route(xs[r], k)
        assert torch.equal(m1.gate_index, routed[r][1].gate_index) and torch.equal(s1, routed[r][0])
        torch.testing.assert_close(ys[r].float(), y1.float(), rtol=2e-2, atol=2e-2)
    assert _lib.device_status(DEV) == 0


def test_receive_capacity_overflow_is_reported_not_written():
    """A receive buffer too small for what arrives: the plan kernel records it in the status word
    and the dispatch kernel skips the rows that have no place (nothing is written out of bounds)."""
    W, E, k, d, h, o, L = 2, 4, 2, 128, 128, 128, 64
    layers = _make_ranks(W, E, d, h, o, L, k)
    # shrink rank 0's idea of everybody's capacity to below what will arrive
    for l in layers:
        l.peers.capacity = 8
    xs = [torch.randn(L, d, generator=torch.Generator().manual_seed(r)).bfloat16().to(DEV) for r in range(W)]
    routed = [l.ep_route(x, k) for l, x in zip(layers, xs)]
    counts = torch.stack([m.lengths for _, m in routed])
    for l in layers:
        l.peers.recv.fill_(3.0)
    canary = [l.peers.recv[8:].clone() for l in layers]
    for l, x, (_, m) in zip(layers, xs, routed):
        l.ep_dispatch(x, m, counts)
    torch.cuda.synchronize()
    assert _lib.device_status(DEV) == 1
    for l, c in zip(layers, canary):
        assert torch.equal(l.peers.recv[8:], c)

"""Host-side logic of the expert-parallel layer on CPU ranks (gloo, world size 2 and 4): the
exchange plan (split sizes, arrival-order -> expert-order permutation) is exercised with real
all_to_all_single calls, the expert arithmetic is done by the CPU oracle, and the result must equal
the single-process oracle on each rank's tokens. Failure injection is host-side only: a rank with
an inconsistent plan raises before any collective is entered."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fast_moe_b200.modules.expert_parallel import local_expert_plan, validate_plan
from oracle import moe_oracle as O


def test_local_expert_plan_small():
    rl = torch.tensor([[2, 0, 1], [1, 3, 0]])
    off, perm = local_expert_plan(rl)
    assert off.tolist() == [0, 3, 6, 7]
    assert perm.tolist() == [0, 1, 3, 4, 5, 6, 2]
    # empty experts and an empty source
    rl = torch.tensor([[0, 0], [0, 4], [0, 0]])
    off, perm = local_expert_plan(rl)
    assert off.tolist() == [0, 0, 4] and perm.tolist() == [0, 1, 2, 3]
    off, perm = local_expert_plan(torch.zeros(2, 3, dtype=torch.int64))
    assert off.tolist() == [0, 0, 0, 0] and perm.numel() == 0


def test_local_expert_plan_with_capacity_matches_exact_form():
    """The capacity form needs no row count from the host: its first n entries are the exact plan
    (empty segments, empty plans and a capacity equal to n included)."""
    g = torch.Generator().manual_seed(11)
    for trial in range(30):
        W, El = int(torch.randint(1, 6, (1,), generator=g)), int(torch.randint(1, 9, (1,), generator=g))
        rl = torch.randint(0, 7, (W, El), generator=g)
        if trial % 7 == 0:
            rl.zero_()
        n = int(rl.sum())
        off, perm = local_expert_plan(rl)
        for cap in (n, n + 1, n + 50):
            off2, padded = local_expert_plan(rl, capacity=cap)
            assert padded.numel() == cap
            assert torch.equal(off2, off)
            assert torch.equal(padded[:n], perm)


def test_local_expert_plan_random_is_a_grouping_permutation():
    g = torch.Generator().manual_seed(3)
    for _ in range(20):
        W, El = int(torch.randint(1, 6, (1,), generator=g)), int(torch.randint(1, 9, (1,), generator=g))
        rl = torch.randint(0, 7, (W, El), generator=g)
        off, perm = local_expert_plan(rl)
        n = int(rl.sum())
        assert sorted(perm.tolist()) == list(range(n))
        # expert id of every receive-buffer row, in arrival order (source-major, expert-minor)
        eid = torch.repeat_interleave(torch.arange(El).repeat(W), rl.reshape(-1))
        grouped = eid[perm]
        assert torch.equal(grouped, grouped.sort(stable=True).values)
        assert torch.equal(off[1:] - off[:-1], rl.sum(0))
        # within an expert rows keep arrival order
        for e in range(El):
            seg = perm[off[e]:off[e + 1]]
            assert torch.equal(seg, seg.sort().values)


def test_validate_plan_rejects_inconsistent_plans():
    rl = torch.tensor([[1, 2], [3, 4]])
    validate_plan([3, 7], [3, 7], rl, 2)
    with pytest.raises(ValueError):
        validate_plan([3, 7], [3, 6], rl, 2)
    with pytest.raises(ValueError):
        validate_plan([3], [3, 7], rl, 2)
    with pytest.raises(ValueError):
        validate_plan([3, -1], [3, 7], rl, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_worker(rank, world, port, E, k, d, h, o, L, fail_rank, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                       # shared model
        gate_w = torch.randn(E, d) * 0.3
        gate_b = torch.zeros(E)
        w_gate = torch.randn(E, d, h) * 0.1        # logical [E, K, N]
        w_up = torch.randn(E, d, h) * 0.1
        w_down = torch.randn(E, h, o) * 0.1
        x = torch.randn(L, d, generator=torch.Generator().manual_seed(100 + rank))
        El = E // world
        lo = rank * El
        # 1. local routing over all experts
        dense, idx = O.select_top_k(O.gating_scores(x, gate_w, gate_b), k)
        gate_index, token_index, scores_k, offsets, reverse, _ = O.routing_metadata(dense, idx)
        lengths = offsets[1:] - offsets[:-1]
        # 2. counts
        send_lengths = lengths.view(world, El).contiguous()
        recv_lengths = torch.empty_like(send_lengths)
        dist.all_to_all_single(recv_lengths.view(-1), send_lengths.view(-1))
        send_counts = send_lengths.sum(1).tolist()
        recv_counts = recv_lengths.sum(1).tolist()
        if rank == fail_rank:
            recv_counts[0] += 1                    # injected host-side fault: caught before the exchange
        validate_plan(send_counts, recv_counts, recv_lengths, world)
        # 3. dispatch
        send = x[token_index].contiguous()
        recv = torch.empty(sum(recv_counts), d)
        dist.all_to_all_single(recv, send, recv_counts, send_counts)
        # 4. local experts in expert-major order through the permutation
        off_local, perm = local_expert_plan(recv_lengths, sum(recv_counts))
        rows = recv[perm]
        ident = torch.arange(rows.shape[0]).view(-1, 1)
        hidden = O.index_select_jagged_bmm_swiglu(off_local, ident, rows, w_gate[lo:lo + El], None, w_up[lo:lo + El], None)
        y_rows = O.silu_jagged_bmm(off_local, hidden, w_down[lo:lo + El], None, has_silu=False)
        back_send = torch.empty_like(y_rows)
        back_send[perm] = y_rows                   # scatter back to arrival order
        # 5. return + combine
        back = torch.empty(L * k, o)
        dist.all_to_all_single(back, back_send, send_counts, recv_counts)
        y = O.mul_merge_k_add(token_index, back, k, scores_k, gate_index)
        ref = O.moe_layer_swiglu(x, gate_w, gate_b, w_gate, w_up, w_down, k)
        out_q.put((rank, "ok", float((y - ref).abs().max())))
    except ValueError as ex:
        out_q.put((rank, "ValueError", str(ex)))
    finally:
        dist.destroy_process_group()


def _run(world, fail_rank=-1, **kw):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    cfg = dict(E=8, k=2, d=16, h=24, o=12, L=37)
    cfg.update(kw)
    procs = [ctx.Process(target=_ep_worker, args=(r, world, port, cfg["E"], cfg["k"], cfg["d"], cfg["h"], cfg["o"],
                                                  cfg["L"], fail_rank, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    return sorted(res)


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_flow_matches_single_process_oracle(world):
    res = _run(world)
    for rank, status, err in res:
        assert status == "ok", (rank, status, err)
        assert err < 1e-5


def test_expert_parallel_skewed_routing_with_empty_experts():
    # 16 experts, top-1, few tokens: several experts (and possibly a whole rank) receive nothing
    res = _run(2, E=16, k=1, L=5)
    for rank, status, err in res:
        assert status == "ok" and err < 1e-5


def test_injected_plan_fault_raises_on_the_host_before_the_exchange():
    # every rank corrupts its own plan, so nobody enters the row exchange and nobody is left waiting
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker_all_fail, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert [r[1] for r in res] == ["ValueError", "ValueError"]


def _ep_worker_all_fail(rank, world, port, q):
    _ep_worker(rank, world, port, 8, 2, 16, 24, 12, 20, rank, q)

"""Host-side logic of the expert-parallel layer on CPU ranks (gloo, world size 2 and 4). Both
exchange forms are exercised with real collectives, the expert arithmetic is done by the CPU
oracle, and the result must equal the single-process oracle on each rank's tokens:
  - the library-collective form: split sizes, arrival-order -> expert-order permutation,
    all_to_all_single both ways;
  - the peer-memory form: all-gathered counts -> placement plan (expert-major receive buffers,
    return addresses); the stores into peer buffers are emulated by gathering every rank's rows
    and letting each owner place the ones addressed to it exactly where the plan says.
Failure injection is host-side only: a rank with an inconsistent plan raises before any
collective is entered, and - the counts being identical on all ranks - every rank raises."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fast_moe_b200.modules.expert_parallel import (ROUTE_SHIFT, local_expert_plan, peer_exchange_plan, validate_counts,
                                                   validate_plan)
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


# ------------------------------------------------------------------------- peer-memory exchange
def test_peer_exchange_plan_against_enumeration():
    g = torch.Generator().manual_seed(0)
    for W, E in [(2, 8), (4, 16), (8, 64), (1, 4)]:
        El = E // W
        counts = torch.randint(0, 5, (W, E), generator=g)
        if W == 4:
            counts[:, 5] = 0                      # an expert nobody routes to
            counts[2] = 0                         # a rank without tokens
        for r in range(W):
            dst_base, off_local = peer_exchange_plan(counts, r)
            for e in range(E):
                owner = e // El
                pos = sum(int(counts[:, f].sum()) for f in range(owner * El, e)) + int(counts[:r, e].sum())
                assert int(dst_base[e]) == pos
            want = [0]
            for le in range(El):
                want.append(want[-1] + int(counts[:, r * El + le].sum()))
            assert off_local.tolist() == want
        # the destination ranges of all (source, expert) pairs tile every owner's buffer exactly
        for owner in range(W):
            segs = []
            for s in range(W):
                db, _ = peer_exchange_plan(counts, s)
                segs += [(int(db[e]), int(db[e]) + int(counts[s, e])) for e in range(owner * El, owner * El + El)
                         if counts[s, e] > 0]
            segs.sort()
            assert all(a[1] == b[0] for a, b in zip(segs, segs[1:]))
            total = int(counts[:, owner * El:(owner + 1) * El].sum())
            assert (not segs and total == 0) or (segs[0][0] == 0 and segs[-1][1] == total)


def test_validate_counts_raises_the_same_on_every_rank():
    counts = torch.tensor([[2, 0, 1, 1], [1, 3, 0, 0]])
    validate_counts(counts, [2, 2], 2, capacity=8)
    with pytest.raises(ValueError):
        validate_counts(counts, [2, 3], 2, capacity=8)            # rank 1's counts do not add up
    with pytest.raises(ValueError):
        validate_counts(counts, [2, 2], 2, capacity=5)            # rank 0 would receive 6 rows
    bad = counts.clone()
    bad[0, 1] = -1
    with pytest.raises(ValueError):
        validate_counts(bad, [2, 2], 2, capacity=8)


def _peer_worker(rank, world, port, E, k, d, h, o, tokens, out_q):
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
        L = tokens[rank]
        x = torch.randn(L, d, generator=torch.Generator().manual_seed(100 + rank))
        El = E // world
        lo = rank * El
        dense, idx = O.select_top_k(O.gating_scores(x, gate_w, gate_b), k)
        gate_index, token_index, scores_k, offsets, reverse, _ = O.routing_metadata(dense, idx)
        lengths = (offsets[1:] - offsets[:-1]).contiguous()
        # counts of every rank (the one collective the plan needs)
        counts = torch.empty(world, E, dtype=torch.int64)
        dist.all_gather_into_tensor(counts.view(-1), lengths)
        capacity = world * max(tokens) * k
        validate_counts(counts, tokens, k, capacity)
        dst_base, off_local = peer_exchange_plan(counts, rank)
        # "peer stores": every rank publishes (owner, destination row, return address, row data);
        # each owner keeps what is addressed to it and places it where the sender computed
        A = L * k
        e_of_row = torch.searchsorted(offsets[1:].contiguous(), torch.arange(A), right=True)
        dest_row = dst_base[e_of_row] + (torch.arange(A) - offsets[e_of_row])
        owner = e_of_row // El
        ret = (rank << ROUTE_SHIFT) | torch.arange(A)
        amax = max(tokens) * k
        pack = torch.zeros(amax, d + 3)
        pack[:A, 0], pack[:A, 1], pack[:A, 2], pack[:A, 3:] = owner.float(), dest_row.float(), torch.arange(A).float(), x[token_index]
        pack[A:, 0] = -1
        allp = torch.empty(world, amax, d + 3)
        dist.all_gather_into_tensor(allp.view(-1), pack.view(-1))
        n_recv = int(off_local[-1])
        recv = torch.full((n_recv, d), float("nan"))
        route_src = torch.full((n_recv,), -1, dtype=torch.int64)
        route_row = torch.full((n_recv,), -1, dtype=torch.int64)
        for s in range(world):
            mine = allp[s][allp[s][:, 0] == rank]
            q = mine[:, 1].long()
            recv[q] = mine[:, 3:]
            route_src[q] = s
            route_row[q] = mine[:, 2].long()
        assert not torch.isnan(recv).any() and bool((route_src >= 0).all())
        # the receive buffer is expert-major: the experts run on it as it lies
        ident = torch.arange(n_recv).view(-1, 1)
        hidden = O.index_select_jagged_bmm_swiglu(off_local, ident, recv, w_gate[lo:lo + El], None, w_up[lo:lo + El], None)
        y_rows = O.silu_jagged_bmm(off_local, hidden, w_down[lo:lo + El], None, has_silu=False)
        # return: every result row goes to (source rank, row) - emulated by gathering all results
        outp = torch.zeros(capacity, o + 2)
        outp[:n_recv, 0], outp[:n_recv, 1], outp[:n_recv, 2:] = route_src.float(), route_row.float(), y_rows
        outp[n_recv:, 0] = -1
        allo = torch.empty(world, capacity, o + 2)
        dist.all_gather_into_tensor(allo.view(-1), outp.view(-1))
        back = torch.full((A, o), float("nan"))
        for s in range(world):
            mine = allo[s][allo[s][:, 0] == rank]
            back[mine[:, 1].long()] = mine[:, 2:]
        assert not torch.isnan(back).any()
        y = O.mul_merge_k_add(token_index, back, k, scores_k, gate_index) if L else torch.zeros(0, o)
        ref = O.moe_layer_swiglu(x, gate_w, gate_b, w_gate, w_up, w_down, k) if L else torch.zeros(0, o)
        out_q.put((rank, "ok", float((y - ref).abs().max()) if L else 0.0))
    except ValueError as ex:
        out_q.put((rank, "ValueError", str(ex)))
    finally:
        dist.destroy_process_group()


def _run_peer(world, tokens, E=8, k=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_peer_worker, args=(r, world, port, E, k, 16, 24, 12, tokens, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    return res


@pytest.mark.parametrize("world,tokens", [(2, [37, 21]), (4, [20, 0, 33, 5])])
def test_peer_exchange_flow_matches_single_process_oracle(world, tokens):
    """Includes ranks with different token counts, a rank without tokens, and (few tokens over
    8 experts) owners that receive nothing for some of their experts."""
    for rank, status, err in _run_peer(world, tokens):
        assert status == "ok", (rank, status, err)
        assert err < 1e-5


def test_peer_exchange_rank_that_receives_nothing():
    # top-1 over 16 experts with 3 + 2 tokens: most experts, possibly a whole rank, stay empty
    for rank, status, err in _run_peer(2, [3, 2], E=16, k=1):
        assert status == "ok" and err < 1e-5

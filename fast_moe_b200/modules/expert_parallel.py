"""Expert-parallel SwiGLU MoE layer: the experts are split in contiguous blocks over the ranks of
one node (one process per GPU), every rank keeps its own tokens, routes them over ALL experts, and
exchanges rows with the expert owners over NVLink.

The reference advertises an expert-parallel layer but ships none (README.md:100-113 names a file
that does not exist), so there is no reference behaviour to mirror: the contract here is that
the result equals the single-GPU SwiGLUFastMoELayer on the same tokens and weights.

Two exchange implementations:

``exchange="peer"`` (default) - the rows move through peer-mapped buffers (torch symmetric memory
gives every rank the addresses of every rank's buffers) and nothing in the forward waits for the
host:
  1. gate -> top-k -> counting sort over the global expert ids (rows sorted by expert are also
     sorted by owner rank).
  2. all-gather of the [E] row counts (a 512-byte collective; it also orders the reuse of the
     peer buffers between consecutive forwards).
  3. plan kernel: where this rank's rows for each expert start in the owner's receive buffer,
     and the jagged offsets of the local experts. Dispatch kernel: one warp per row stores the
     token row into the owner's receive buffer, which is laid out expert-major, and the row's
     return address into the owner's route table. A tiny all-reduce orders "rows have landed".
  4. up projection on the receive buffer (contiguous TMA tiles), down projection whose epilogue
     stores every result row at its return address in the token owner's buffer: the return
     transfer runs inside the GEMM. A tiny all-reduce orders "results have landed".
  5. gate-weighted combine where the tokens live.

``exchange="nccl"`` - variable-split ``all_to_all_single`` both ways with the split sizes read
back to the host (one synchronisation per forward), received rows consumed through a permutation
folded into the GEMMs. Kept as the library-collective baseline.
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _lib
from ..kernels import moe as ops
from .fast_moe_module import GateSplitCache, route_tokens

ROUTE_SHIFT = 40     # return address = (source rank << 40) | row in the source's expert-sorted order


def local_expert_plan(recv_lengths: torch.Tensor, total: Optional[int] = None,
                      capacity: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(``exchange="nccl"``) recv_lengths [W, E_local]: rows received from each source rank for each
    local expert, in the order they sit in the receive buffer (source-major, expert-minor).

    Returns (offsets [E_local + 1], perm [n]) where offsets are the jagged offsets of the local
    experts and perm[p] is the receive-buffer row that belongs at expert-major position p
    (within an expert: by source rank, then in arrival order). Pure index arithmetic on small
    tensors; runs on whatever device recv_lengths lives on.

    With ``capacity`` (an upper bound of the row count known without looking at the counts) the
    whole plan is computed without any host-side size: perm comes back with ``capacity`` entries
    of which the first n are the plan and the rest are padding, so the caller can queue this
    before it reads the counts back and slice afterwards.
    """
    W, El = recv_lengths.shape
    dev = recv_lengths.device
    flat = recv_lengths.reshape(-1)
    seg_start_recv = torch.cumsum(flat, 0) - flat                      # start of (src, e) in the buffer
    per_expert = recv_lengths.sum(0)
    offsets = torch.zeros(El + 1, dtype=torch.int64, device=dev)
    offsets[1:] = torch.cumsum(per_expert, 0)
    # destination order: expert-major, source-minor
    len_dst = recv_lengths.t().reshape(-1)
    start_src = seg_start_recv.view(W, El).t().reshape(-1)
    start_dst = torch.cumsum(len_dst, 0) - len_dst
    if capacity is not None:
        # row p belongs to the destination segment whose [start, end) contains it
        end_dst = torch.cumsum(len_dst, 0)
        p = torch.arange(capacity, device=dev)
        seg = torch.searchsorted(end_dst, p, right=True).clamp_(max=W * El - 1)
        return offsets, start_src[seg] + (p - start_dst[seg])
    if total is None:
        total = int(flat.sum().item())   # callers that already know the row count pass it and skip this sync
    seg_of_row = torch.repeat_interleave(torch.arange(W * El, device=dev), len_dst, output_size=total)
    perm = start_src[seg_of_row] + (torch.arange(total, device=dev) - start_dst[seg_of_row])
    return offsets, perm


def validate_plan(send_counts, recv_counts, recv_lengths, world: int) -> None:
    """(``exchange="nccl"``) Host-side consistency checks of an exchange plan; raises ValueError
    before anything is launched if the plan cannot be right (a mismatched split would otherwise
    surface as a hang or as garbage inside the collective)."""
    if len(send_counts) != world or len(recv_counts) != world:
        raise ValueError(f"split lists must have {world} entries, got {len(send_counts)} / {len(recv_counts)}")
    if any(c < 0 for c in send_counts) or any(c < 0 for c in recv_counts):
        raise ValueError("negative split size")
    if int(recv_lengths.sum()) != sum(recv_counts):
        raise ValueError("per-expert receive counts do not add up to the receive split sizes")
    if recv_lengths.shape[0] != world:
        raise ValueError("recv_lengths must have one row per source rank")


def peer_exchange_plan(counts: torch.Tensor, rank: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(``exchange="peer"``) What fmoe_ep_plan computes on the device, as plain tensor arithmetic
    (any device; used by the CPU tests and as the statement of the layout).

    counts [W, E]: counts[s, e] = rows rank s routes to global expert e; expert e lives on rank
    e // (E // W). An owner's receive buffer is expert-major: (local expert, source rank, the
    source's own row order). Returns
      dst_base [E]: row of the owner's receive buffer where rank ``rank``'s rows for expert e start
      offsets_local [E // W + 1]: jagged offsets of ``rank``'s local experts over the rows it receives.
    """
    W, E = counts.shape
    El = E // W
    tot = counts.sum(0)                                            # rows per expert over all sources
    start_in_owner = (torch.cumsum(tot.view(W, El), 1) - tot.view(W, El)).reshape(-1)
    before = counts[:rank].sum(0) if rank > 0 else torch.zeros_like(tot)
    dst_base = start_in_owner + before
    offsets_local = torch.zeros(El + 1, dtype=counts.dtype, device=counts.device)
    offsets_local[1:] = torch.cumsum(tot.view(W, El)[rank], 0)
    return dst_base, offsets_local


def validate_counts(counts: torch.Tensor, tokens_per_rank: List[int], k: int, capacity: int) -> None:
    """Host-side check of the all-gathered row counts (every rank holds the same tensor, so every
    rank raises or none does): each rank's counts add up to its rows, nothing is negative, and no
    owner receives more rows than its receive buffer holds."""
    W, E = counts.shape
    if bool((counts < 0).any()):
        raise ValueError("negative row count in the exchange plan")
    per_rank = counts.sum(1).tolist()
    for s, (have, want) in enumerate(zip(per_rank, tokens_per_rank)):
        if have != want * k:
            raise ValueError(f"rank {s} routes {have} rows but holds {want} tokens x top-{k}")
    recv = counts.view(W, W, E // W).sum(dim=(0, 2)).tolist()
    for r, n in enumerate(recv):
        if n > capacity:
            raise ValueError(f"rank {r} would receive {n} rows, more than its receive buffer of {capacity}")


class PeerBuffers:
    """One rank's peer-visible buffers - receive rows [capacity, d], route table [capacity] int64,
    return rows [back_rows, o] - plus, once linked, the device tables with every rank's addresses.

    Multi-process: one symmetric-memory allocation per rank carved into the three regions, the
    peers' base addresses come from the rendezvous. Single-process (tests that run several
    logical ranks on one GPU): plain tensors, linked by hand with ``link_local``."""

    def __init__(self, capacity: int, back_rows: int, d: int, o: int, dtype: torch.dtype, device: torch.device,
                 group=None, symmetric: bool = False) -> None:
        es = torch.empty((), dtype=dtype).element_size()
        self.capacity, self.back_rows, self.d, self.o, self.dtype, self.device = capacity, back_rows, d, o, dtype, device
        align = lambda n: (n + 255) // 256 * 256
        self._off_recv = 0
        self._off_route = align(capacity * d * es)
        self._off_back = self._off_route + align(capacity * 8)
        nbytes = self._off_back + align(back_rows * o * es)
        self.handle = None
        if symmetric:
            import torch.distributed._symmetric_memory as symm

            # plain peer mappings are all this layer needs: no NVLink multicast binding
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            pg = group if group is not None else dist.group.WORLD
            try:
                symm.enable_symm_mem_for_group(pg.group_name)
            except Exception:      # newer torch enables groups on demand
                pass
            self.blob = symm.empty(nbytes, dtype=torch.uint8, device=device)
            self.handle = symm.rendezvous(self.blob, pg.group_name)
            bases = [int(p) for p in self.handle.buffer_ptrs]
            self._make_tables(bases)
        else:
            self.blob = torch.empty(nbytes, dtype=torch.uint8, device=device)
        base = self.blob
        self.recv = base[self._off_recv:self._off_recv + capacity * d * es].view(dtype).view(capacity, d)
        self.route = base[self._off_route:self._off_route + capacity * 8].view(torch.int64)
        self.back = base[self._off_back:self._off_back + back_rows * o * es].view(dtype).view(back_rows, o)

    def _make_tables(self, bases: List[int]) -> None:
        i64 = dict(dtype=torch.int64, device=self.device)
        self.recv_ptrs = torch.tensor([b + self._off_recv for b in bases], **i64)
        self.route_ptrs = torch.tensor([b + self._off_route for b in bases], **i64)
        self.back_ptrs = torch.tensor([b + self._off_back for b in bases], **i64)

    @staticmethod
    def link_local(buffers: List["PeerBuffers"]) -> None:
        """Several logical ranks inside one process: everybody learns everybody's addresses."""
        bases = [b.blob.data_ptr() for b in buffers]
        for b in buffers:
            b._make_tables(bases)


class ExpertParallelSwiGLUMoE(nn.Module):
    """SwiGLU MoE layer whose experts are sharded over ``group`` (default: the world).

    Every rank holds the full gate and the weights of its E / W experts, stored with the
    reduction dimension contiguous: w_gate / w_up [E_local, h, d], w_down [E_local, o, h].
    Weight initialisation is seeded per GLOBAL expert id, so any sharding holds the same model.

    ``max_tokens_per_rank`` sizes the peer buffers (receive capacity = world x tokens x k rows:
    even if every token of every rank picks this rank's experts, nothing is dropped). Left at
    None it is agreed on at the first forward (an all-reduce of the token counts, the one time the
    layer waits for the host); a later, larger batch raises. All ranks must use the same top-k.
    """

    def __init__(self, input_dim: int, hidden_dim: int, output_dim: int, num_experts: int,
                 dtype: torch.dtype = torch.bfloat16, init_std: float = 0.02,
                 device: Optional[torch.device] = None, group: Optional[dist.ProcessGroup] = None,
                 seed: int = 0, world_size: Optional[int] = None, rank: Optional[int] = None,
                 exchange: str = "peer", max_tokens_per_rank: Optional[int] = None) -> None:
        super().__init__()
        if exchange not in ("peer", "nccl"):
            raise ValueError("exchange must be 'peer' or 'nccl'")
        self.group = group
        self.exchange = exchange
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._own_process_group = True
        if world_size is not None:
            if rank is not None:
                # a logical rank of a single-process job: the caller drives the phases itself
                self.world, self.rank, self._own_process_group = world_size, rank, False
            elif world_size == 1:
                # every expert on this process even inside a larger job
                self.world, self.rank = 1, 0
            elif world_size != self.world:
                raise ValueError(f"world_size={world_size} does not match the process group ({self.world} ranks)")
        if num_experts % self.world != 0:
            raise ValueError(f"{num_experts} experts cannot be split evenly over {self.world} ranks")
        self.input_dim, self.hidden_dim, self.output_dim = input_dim, hidden_dim, output_dim
        self.num_experts = num_experts
        self.experts_local = num_experts // self.world
        self.first_expert = self.rank * self.experts_local
        self.dtype = dtype
        self.max_tokens_per_rank = max_tokens_per_rank
        dev = device if device is not None else torch.device("cpu")
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        gate_w = torch.randn(num_experts, input_dim, generator=g, device=dev) * init_std
        self.gate = nn.Linear(input_dim, num_experts, device=dev)
        with torch.no_grad():
            self.gate.weight.copy_(gate_w)
            self.gate.bias.zero_()
        self._init = (seed, init_std, dev)

        def expert_weights(rows, cols, salt):
            out = torch.empty(self.experts_local, rows, cols, dtype=dtype, device=dev)
            for i in range(self.experts_local):
                out[i] = self._expert_matrix(self.first_expert + i, rows, cols, salt)
            return nn.Parameter(out)

        self._gate_split = GateSplitCache()
        self.w_gate = expert_weights(hidden_dim, input_dim, 1)
        self.w_up = expert_weights(hidden_dim, input_dim, 2)
        self.w_down = expert_weights(output_dim, hidden_dim, 3)
        self.peers: Optional[PeerBuffers] = None
        self._k: Optional[int] = None
        self._work = {}

    def _expert_matrix(self, expert: int, rows: int, cols: int, salt: int) -> torch.Tensor:
        seed, init_std, dev = self._init
        ge = torch.Generator(device=dev)
        ge.manual_seed(seed * 1000003 + expert * 7 + salt)
        return (torch.randn(rows, cols, generator=ge, device=dev) * init_std).to(self.dtype)

    def materialize_expert(self, expert: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """The initial (w_gate [h, d], w_up [h, d], w_down [o, h]) of GLOBAL expert id ``expert``,
        rebuilt from its seed on this rank's device whichever rank owns it: what a re-sharding, or
        a check of one rank's result against the whole model, needs without moving weights."""
        return (self._expert_matrix(expert, self.hidden_dim, self.input_dim, 1),
                self._expert_matrix(expert, self.hidden_dim, self.input_dim, 2),
                self._expert_matrix(expert, self.output_dim, self.hidden_dim, 3))

    # ------------------------------------------------------------------ peer buffers
    def setup_peer_buffers(self, tokens: int, k: int, symmetric: bool = True) -> PeerBuffers:
        """Allocates the peer-visible buffers for up to ``tokens`` tokens per rank and top-``k``.
        With ``symmetric`` this is a collective call (symmetric-memory rendezvous over the group)."""
        dev = self.gate.weight.device
        self.max_tokens_per_rank = tokens
        self._k = k
        capacity = self.world * tokens * k
        self.peers = PeerBuffers(capacity, tokens * k, self.input_dim, self.output_dim, self.dtype, dev,
                                 group=self.group, symmetric=symmetric)
        i64 = dict(dtype=torch.int64, device=dev)
        self._work = dict(
            counts=torch.zeros((self.world, self.num_experts), **i64),
            dst_base=torch.zeros(self.num_experts, **i64),
            offsets_local=torch.zeros(self.experts_local + 1, **i64),
            hidden=torch.empty((capacity, self.hidden_dim), dtype=self.dtype, device=dev),
            flag=torch.zeros(1, dtype=torch.float32, device=dev),
        )
        # route entries of rows that never arrive must not look like addresses
        self.peers.route.fill_(-1)
        return self.peers

    def _ensure_peer_buffers(self, L: int, k: int) -> None:
        if self.peers is not None:
            if L > self.max_tokens_per_rank or k != self._k:
                raise RuntimeError(
                    f"batch of {L} tokens / top-{k} does not fit the peer buffers sized for "
                    f"{self.max_tokens_per_rank} tokens / top-{self._k}; construct the layer with max_tokens_per_rank")
            return
        tokens = self.max_tokens_per_rank
        if tokens is None:
            t = torch.tensor([L], dtype=torch.int64, device=self.gate.weight.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            tokens = int(t.item())
        self.setup_peer_buffers(tokens, k, symmetric=True)

    # ------------------------------------------------------------------ phases of the peer exchange
    def ep_route(self, x_flat: torch.Tensor, k: int):
        return route_tokens(x_flat, self.gate, k, self.num_experts, self._gate_split)

    def ep_dispatch(self, x_flat: torch.Tensor, meta, counts: torch.Tensor) -> None:
        """Plan + dispatch: this rank's rows go into their owners' receive buffers."""
        lib = _lib.load()
        p, w = self.peers, self._work
        dev = x_flat.device
        xs = x_flat if x_flat.stride(1) == 1 else x_flat.contiguous()
        rows = meta.token_index.numel()
        with torch.cuda.device(dev):
            st = _lib.stream_ptr(dev)
            _lib.check(lib.fmoe_ep_plan(counts.data_ptr(), self.world, self.num_experts, self.rank, p.capacity,
                                        w["dst_base"].data_ptr(), w["offsets_local"].data_ptr(), st))
            _lib.check(lib.fmoe_ep_dispatch(
                xs.data_ptr(), _lib.dtype_code(xs.dtype), xs.shape[0], xs.stride(0), self.input_dim,
                meta.offsets.data_ptr(), meta.token_index.data_ptr(), rows, self.num_experts, self.world, self.rank,
                w["dst_base"].data_ptr(), p.recv_ptrs.data_ptr(), p.route_ptrs.data_ptr(), p.recv.stride(0), p.capacity, st))

    def ep_experts(self, rows_hint: int) -> None:
        """Local experts on the rows received; the down projection stores its rows in the token
        owners' return buffers."""
        lib = _lib.load()
        p, w = self.peers, self._work
        dev = p.device
        dt = _lib.dtype_code(self.dtype)
        wg, wu, wd = self.w_gate.detach(), self.w_up.detach(), self.w_down.detach()
        with torch.cuda.device(dev), _lib.stage("up"):
            st = _lib.stream_ptr(dev)
            _lib.check(lib.fmoe_ep_up_projection(
                w["offsets_local"].data_ptr(), p.capacity, rows_hint, p.recv.data_ptr(), dt, p.recv.stride(0),
                wg.data_ptr(), wu.data_ptr(), wg.stride(0), wg.stride(1), self.experts_local, self.input_dim,
                self.hidden_dim, w["hidden"].data_ptr(), w["hidden"].stride(0), st))
        with torch.cuda.device(dev), _lib.stage("down_return"):
            _lib.check(lib.fmoe_ep_down_projection(
                w["offsets_local"].data_ptr(), p.capacity, rows_hint, w["hidden"].data_ptr(), dt, w["hidden"].stride(0),
                wd.data_ptr(), wd.stride(0), wd.stride(1), self.experts_local, self.hidden_dim, self.output_dim,
                p.route.data_ptr(), p.back_ptrs.data_ptr(), self.world, p.back_rows, p.back.stride(0), st))

    def ep_combine(self, score: torch.Tensor, meta, k: int) -> torch.Tensor:
        rows = meta.token_index.numel()
        return ops.mul_merge_k_add(meta.token_index, meta.reverse_index, self.peers.back[:rows],
                                   weight=score.to(self.dtype), weight_index=meta.gate_index)

    def _sync_ranks(self) -> None:
        """Orders the peer stores of all ranks before what follows on this stream (a one-element
        all-reduce: every rank's kernels queued before it have completed when it completes)."""
        dist.all_reduce(self._work["flag"], group=self.group)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, num_experts_per_tok: int) -> torch.Tensor:
        shape = x.shape
        k = num_experts_per_tok
        W = self.world
        x_flat = x.reshape(-1, self.input_dim)
        if W == 1:
            score, meta = self.ep_route(x_flat, k)
            wg = self.w_gate.detach().permute(0, 2, 1)
            wu = self.w_up.detach().permute(0, 2, 1)
            wd = self.w_down.detach().permute(0, 2, 1)
            # every expert is local: the sorted order is already the GEMM order
            with _lib.stage("up"):
                hidden = ops.index_select_jagged_bmm_swiglu(0, meta.offsets, meta.gate_index.view(-1, k), x_flat,
                                                            wg, None, wu, None)
            with _lib.stage("down_combine"):
                y = ops.silu_jagged_bmm_combine(0, meta.offsets, hidden, wd, None, meta.token_index,
                                                meta.reverse_index, gating_scores=score,
                                                gates_index=meta.gate_index, has_silu=False, fused=k <= 2,
                                                round_scores=True)
            return y.view(*shape[:-1], self.output_dim)
        if not self._own_process_group:
            raise RuntimeError("a logical rank of a single-process job has no forward(): drive ep_route / "
                               "ep_dispatch / ep_experts / ep_combine of all ranks phase by phase")
        if x_flat.dtype != self.dtype:
            raise TypeError(f"tokens are {x_flat.dtype} but the layer (weights and exchange buffers) is {self.dtype}")
        if self.exchange == "nccl":
            return self._forward_nccl(x_flat, k).view(*shape[:-1], self.output_dim)
        self._ensure_peer_buffers(x_flat.shape[0], k)
        score, meta = self.ep_route(x_flat, k)
        with _lib.stage("plan"):
            counts = self._work["counts"]
            dist.all_gather_into_tensor(counts.view(-1), meta.lengths, group=self.group)
        with _lib.stage("dispatch"):
            self.ep_dispatch(x_flat, meta, counts)
        with _lib.stage("sync_dispatch"):
            self._sync_ranks()
        self.ep_experts(rows_hint=x_flat.shape[0] * k)
        with _lib.stage("sync_return"):
            self._sync_ranks()
        with _lib.stage("combine"):
            y = self.ep_combine(score, meta, k)
        return y.view(*shape[:-1], self.output_dim)

    def _forward_nccl(self, x_flat: torch.Tensor, k: int) -> torch.Tensor:
        W, El = self.world, self.experts_local
        dt = x_flat.dtype
        score, meta = self.ep_route(x_flat, k)
        wg = self.w_gate.detach().permute(0, 2, 1)
        wu = self.w_up.detach().permute(0, 2, 1)
        wd = self.w_down.detach().permute(0, 2, 1)
        with _lib.stage("plan"):
            send_lengths = meta.lengths.view(W, El)
            recv_lengths = torch.empty_like(send_lengths)
            dist.all_to_all_single(recv_lengths.view(-1), send_lengths.reshape(-1).contiguous(), group=self.group)
            # the pack kernel is queued before the host waits for the counts, so the GPU packs the
            # rows while the host reads the split sizes back
            send = ops.gather_rows(x_flat, meta.gate_index, k)
            counts = torch.stack([send_lengths.sum(1), recv_lengths.sum(1)]).cpu()   # the one host sync of this path
            send_counts, recv_counts = counts[0].tolist(), counts[1].tolist()
            validate_plan(send_counts, recv_counts, recv_lengths, W)
            n_recv = sum(recv_counts)
            # ranks may hold different numbers of tokens, so the plan is sized by what actually arrives
            offsets_local, perm = local_expert_plan(recv_lengths, total=n_recv)
        with _lib.stage("dispatch"):
            recv = torch.empty((n_recv, self.input_dim), dtype=dt, device=x_flat.device)
            dist.all_to_all_single(recv, send, recv_counts, send_counts, group=self.group)
        with _lib.stage("up"):
            hidden = ops.index_select_jagged_bmm_swiglu(0, offsets_local, perm.view(-1, 1), recv, wg, None, wu, None)
        with _lib.stage("down"):
            back_send = ops.silu_jagged_bmm(offsets_local, hidden, wd, None, has_silu=False, out_row_index=perm)
        with _lib.stage("return"):
            back = torch.empty((x_flat.shape[0] * k, self.output_dim), dtype=dt, device=x_flat.device)
            dist.all_to_all_single(back, back_send, send_counts, recv_counts, group=self.group)
        with _lib.stage("combine"):
            y = ops.mul_merge_k_add(meta.token_index, meta.reverse_index, back, weight=score.to(dt),
                                    weight_index=meta.gate_index)
        return y

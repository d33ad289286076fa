"""Expert-parallel SwiGLU MoE layer: the experts are split in contiguous blocks over the ranks of
one node (one process per GPU, torch.distributed / NCCL over NVLink), every rank keeps its own
tokens, routes them over ALL experts, and exchanges rows with the expert owners.

The reference advertises an expert-parallel layer but ships none (README.md:100-113 names a file
that does not exist), so there is no reference behaviour to mirror: the contract here is that
the result equals the single-GPU SwiGLUFastMoELayer on the same tokens and weights.

Per forward, on every rank:
  1. gate -> top-k -> counting sort over the global expert ids. Rows sorted by expert are also
     sorted by owner rank, so the rows bound for rank r are one contiguous slice.
  2. per-(rank, expert) row counts are exchanged (all_to_all_single on int64 [W * E_local]);
     the two split-size lists are read back to the host (the one synchronisation of the layer:
     NCCL needs the split sizes on the host).
  3. a row-gather kernel packs the token rows in sorted order; all_to_all_single moves them.
  4. received rows arrive ordered (source rank, local expert, token). The grouped GEMMs want them
     grouped by expert, so a permutation is handed to the up-projection kernel (which gathers
     through it while loading) and to the down-projection kernel (which scatters through it while
     storing): no separate reorder pass, and the results leave in arrival order.
  5. all_to_all_single returns the rows; the gate-weighted combine runs where the tokens live.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _lib
from ..kernels import moe as ops
from .fast_moe_module import GateSplitCache, route_tokens


def local_expert_plan(recv_lengths: torch.Tensor, total: Optional[int] = None,
                      capacity: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """recv_lengths [W, E_local]: rows received from each source rank for each local expert, in
    the order they sit in the receive buffer (source-major, expert-minor).

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
    """Host-side consistency checks of an exchange plan; raises ValueError before anything is
    launched if the plan cannot be right (a mismatched split would otherwise surface as a hang
    or as garbage inside the collective)."""
    if len(send_counts) != world or len(recv_counts) != world:
        raise ValueError(f"split lists must have {world} entries, got {len(send_counts)} / {len(recv_counts)}")
    if any(c < 0 for c in send_counts) or any(c < 0 for c in recv_counts):
        raise ValueError("negative split size")
    if int(recv_lengths.sum()) != sum(recv_counts):
        raise ValueError("per-expert receive counts do not add up to the receive split sizes")
    if recv_lengths.shape[0] != world:
        raise ValueError("recv_lengths must have one row per source rank")


class ExpertParallelSwiGLUMoE(nn.Module):
    """SwiGLU MoE layer whose experts are sharded over ``group`` (default: the world).

    Every rank holds the full gate and the weights of its E / W experts, stored with the
    reduction dimension contiguous: w_gate / w_up [E_local, h, d], w_down [E_local, o, h].
    Weight initialisation is seeded per GLOBAL expert id, so any sharding holds the same model.
    """

    def __init__(self, input_dim: int, hidden_dim: int, output_dim: int, num_experts: int,
                 dtype: torch.dtype = torch.bfloat16, init_std: float = 0.02,
                 device: Optional[torch.device] = None, group: Optional[dist.ProcessGroup] = None,
                 seed: int = 0, world_size: Optional[int] = None) -> None:
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if world_size is not None:
            # world_size=1 keeps every expert on this process even inside a larger job
            if world_size != 1 and world_size != self.world:
                raise ValueError(f"world_size={world_size} does not match the process group ({self.world} ranks)")
            if world_size == 1:
                self.world, self.rank = 1, 0
        if num_experts % self.world != 0:
            raise ValueError(f"{num_experts} experts cannot be split evenly over {self.world} ranks")
        self.input_dim, self.hidden_dim, self.output_dim = input_dim, hidden_dim, output_dim
        self.num_experts = num_experts
        self.experts_local = num_experts // self.world
        self.first_expert = self.rank * self.experts_local
        self.dtype = dtype
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

    @torch.no_grad()
    def forward(self, x: torch.Tensor, num_experts_per_tok: int) -> torch.Tensor:
        shape = x.shape
        k = num_experts_per_tok
        W, El = self.world, self.experts_local
        x_flat = x.reshape(-1, self.input_dim)
        dt = x.dtype
        score, meta = route_tokens(x_flat, self.gate, k, self.num_experts, self._gate_split)
        wg = self.w_gate.detach().permute(0, 2, 1)
        wu = self.w_up.detach().permute(0, 2, 1)
        wd = self.w_down.detach().permute(0, 2, 1)
        if W == 1:
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

        with _lib.stage("plan"):
            send_lengths = meta.lengths.view(W, El)
            recv_lengths = torch.empty_like(send_lengths)
            dist.all_to_all_single(recv_lengths.view(-1), send_lengths.reshape(-1).contiguous(), group=self.group)
            # the pack kernel is queued before the host waits for the counts, so the GPU packs the
            # rows while the host reads the split sizes back
            send = ops.gather_rows(x_flat, meta.gate_index, k)
            counts = torch.stack([send_lengths.sum(1), recv_lengths.sum(1)]).cpu()   # the layer's one host sync
            send_counts, recv_counts = counts[0].tolist(), counts[1].tolist()
            validate_plan(send_counts, recv_counts, recv_lengths, W)
            n_recv = sum(recv_counts)
            # ranks may hold different numbers of tokens, so the plan is sized by what actually arrives
            offsets_local, perm = local_expert_plan(recv_lengths, total=n_recv)
        with _lib.stage("dispatch"):
            recv = torch.empty((n_recv, self.input_dim), dtype=dt, device=x.device)
            dist.all_to_all_single(recv, send, recv_counts, send_counts, group=self.group)
        with _lib.stage("up"):
            hidden = ops.index_select_jagged_bmm_swiglu(0, offsets_local, perm.view(-1, 1), recv, wg, None, wu, None)
        with _lib.stage("down"):
            back_send = ops.silu_jagged_bmm(offsets_local, hidden, wd, None, has_silu=False, out_row_index=perm)
        with _lib.stage("return"):
            back = torch.empty((x_flat.shape[0] * k, self.output_dim), dtype=dt, device=x.device)
            dist.all_to_all_single(back, back_send, send_counts, recv_counts, group=self.group)
        with _lib.stage("combine"):
            y = ops.mul_merge_k_add(meta.token_index, meta.reverse_index, back, weight=score.to(dt),
                                    weight_index=meta.gate_index)
        return y.view(*shape[:-1], self.output_dim)

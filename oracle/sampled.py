"""Sampled-token form of the CPU oracle, for layers too large to restate in full on the host.

TEST INFRASTRUCTURE ONLY (imported by tests/ and by the parity leg of bench.py, never by the
fast_moe_b200 package). Nothing here adds arithmetic of its own: a token's output depends only on
that token's row, the gate, and the weights of the k experts it is routed to, so the oracle of a
SUBSET of tokens is the oracle layer (oracle/moe_oracle.py, pinned to the reference) run on those
rows with the experts they use. Experts are renumbered 0..U-1 in ascending order of their global
id, which keeps every ordering the reference defines (stable sort by expert, ascending-expert
combine order) unchanged.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence, Tuple

import torch

from . import moe_oracle as O

# e -> (w_gate [h, d], w_up [h, d], w_down [o, h]) as CPU tensors, reduction dimension contiguous
# (the storage layout of the layers' parameters)
ExpertWeights = Callable[[int], Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]


def route_full(x_rows: torch.Tensor, gate_w: torch.Tensor, gate_b: Optional[torch.Tensor], k: int):
    """Oracle routing of every token (cheap even at the largest sizes): returns
    (topk_idx [L, k], scores_k [L, k], gate_index, token_index, offsets, reverse_index, gap) where
    gap[t] is the distance between the k-th and (k+1)-th softmax scores of token t (tokens with a
    tiny gap may legitimately route differently under a different fp32 summation order)."""
    scores = O.gating_scores(x_rows.float(), gate_w.float(), None if gate_b is None else gate_b.float())
    dense, idx = O.select_top_k(scores, k)
    gate_index, token_index, scores_k, offsets, reverse, _ = O.routing_metadata(dense, idx)
    srt = torch.sort(scores, dim=1, descending=True).values
    gap = (srt[:, k - 1] - srt[:, k]) if scores.shape[1] > k else torch.full((scores.shape[0],), 1.0)
    return idx, scores_k, gate_index, token_index, offsets, reverse, gap


def pick_tokens(topk_idx: torch.Tensor, n: int, seed: int = 0, experts: Optional[Sequence[int]] = None,
                gap: Optional[torch.Tensor] = None, min_gap: float = 1e-6) -> torch.Tensor:
    """Seeded choice of up to n token ids. With ``experts`` only tokens whose k experts all lie in
    that set qualify (bounds how many experts' weights the host has to hold). Tokens whose routing
    is a near tie (gap < min_gap) are left out."""
    L = topk_idx.shape[0]
    ok = torch.ones(L, dtype=torch.bool)
    if experts is not None:
        ex = torch.as_tensor(list(experts), dtype=torch.int64)
        top = max(int(topk_idx.max()) if topk_idx.numel() else 0, int(ex.max()) if ex.numel() else 0)
        allowed = torch.zeros(top + 1, dtype=torch.bool)
        allowed[ex] = True
        ok &= allowed[topk_idx].all(dim=1)
    if gap is not None:
        ok &= gap >= min_gap
    cand = torch.nonzero(ok).view(-1)
    g = torch.Generator().manual_seed(seed)
    sel = cand[torch.randperm(cand.numel(), generator=g)[:n]]
    return torch.sort(sel).values


def _compact(x_rows, gate_w, gate_b, k):
    scores = O.gating_scores(x_rows.float(), gate_w.float(), None if gate_b is None else gate_b.float())
    dense, idx = O.select_top_k(scores, k)
    used = torch.unique(idx).tolist()
    remap = torch.full((dense.shape[1],), -1, dtype=torch.int64)
    remap[torch.as_tensor(used)] = torch.arange(len(used))
    idx_c = remap[idx]
    dense_c = dense[:, torch.as_tensor(used)]
    return used, idx, idx_c, dense_c


def swiglu_layer_on_tokens(x_rows: torch.Tensor, gate_w: torch.Tensor, gate_b: Optional[torch.Tensor], k: int,
                           expert_weights: ExpertWeights, with_operand_scale: bool = False):
    """moe_layer_swiglu (the reference's SwiGLU composition, kernels/pytorch/moe.py:306-391 behind
    FastMoELayer's routing) restricted to the given token rows. Returns (y [n, o] fp32, global
    topk_idx [n, k]) and, with ``with_operand_scale``, also S [n]: the largest magnitude among
    the gate-weighted expert rows that are summed into each token (the operands of the final
    k-way sum) - the scale a bf16 run's intermediate roundings are proportional to."""
    used, idx, idx_c, dense_c = _compact(x_rows, gate_w, gate_b, k)
    gate_index, token_index, scores_k, offsets, reverse, _ = O.routing_metadata(dense_c, idx_c)
    ws = [expert_weights(e) for e in used]
    wg = torch.stack([w[0].float() for w in ws]).permute(0, 2, 1)
    wu = torch.stack([w[1].float() for w in ws]).permute(0, 2, 1)
    wd = torch.stack([w[2].float() for w in ws]).permute(0, 2, 1)
    del ws
    # the three steps pytorch_fused_jagged_bmm_swiglu_combine composes (kernels/pytorch/moe.py:306-391)
    hidden = O.index_select_jagged_bmm_swiglu(offsets, gate_index.view(-1, k), x_rows.float(), wg, None, wu, None)
    y_rows = O.silu_jagged_bmm(offsets, hidden, wd, None, has_silu=False)
    y = O.mul_merge_k_add(token_index, y_rows, k, scores_k, gate_index)
    if not with_operand_scale:
        return y, idx
    weighted = (y_rows * scores_k.contiguous().view(-1)[gate_index].view(-1, 1)).abs().amax(dim=1)     # per sorted row
    S = torch.zeros(x_rows.shape[0]).scatter_reduce(0, token_index, weighted, reduce="amax", include_self=True)
    return y, idx, S


def swiglu_fp8_layer_on_tokens(x_rows: torch.Tensor, gate_w: torch.Tensor, gate_b: Optional[torch.Tensor], k: int,
                               expert_weights: ExpertWeights) -> Tuple[torch.Tensor, torch.Tensor]:
    """moe_layer_swiglu_fp8 (quantise -> e4m3 product -> descale, twice; rule of
    kernels/pytorch/quant_fp8.py:13-34 and GEMM definition of kernels/pytorch/moe_fp8.py:98-139)
    restricted to the given token rows, which keep their dtype (bf16 rows are rounded to bf16
    between the two products, as the layer does). Returns (y [n, o], global topk_idx)."""
    used, idx, idx_c, dense_c = _compact(x_rows, gate_w, gate_b, k)
    ws = [expert_weights(e) for e in used]
    wg = torch.stack([w[0] for w in ws])
    wu = torch.stack([w[1] for w in ws])
    wd = torch.stack([w[2] for w in ws])
    del ws
    y = _fp8_layer_with_routing(x_rows, dense_c, idx_c, wg, wu, wd, k)
    return y, idx


def _fp8_layer_with_routing(x_rows, dense_c, idx_c, w_gate_rows, w_up_rows, w_down_rows, k):
    """Body of moe_oracle.moe_layer_swiglu_fp8 with the routing decision passed in."""
    import torch.nn.functional as F

    dt = x_rows.dtype
    gate_index, token_index, scores_k, offsets, reverse, _ = O.routing_metadata(dense_c, idx_c)
    rows = x_rows[token_index]
    outs = []
    for e, r in enumerate(rows.split(O._segments(offsets))):
        if r.shape[0] == 0:
            outs.append(torch.zeros(0, w_down_rows.shape[1]))
            continue
        g = O._fp8_linear(r, w_gate_rows[e])
        u = O._fp8_linear(r, w_up_rows[e])
        hidden = (F.silu(g) * u).to(dt)
        outs.append(O._fp8_linear(hidden, w_down_rows[e]).to(dt).float())
    y_rows = torch.cat(outs, dim=0)
    return O.mul_merge_k_add(token_index, y_rows.to(dt), k, scores_k.to(dt), gate_index)


def compare_tokens(y_gpu_rows: torch.Tensor, y_ref_rows: torch.Tensor, rtol: float = 1e-2, atol: float = 1e-2,
                   operand_scale: Optional[torch.Tensor] = None) -> Dict[str, float]:
    """Per-token verdict of |gpu - ref| <= atol * max(1, S) + rtol * |ref| on every element.
    S (``operand_scale``, one value per token, default 1) is the magnitude of the operands of the
    token's final sum: a bf16 run rounds each expert row, and its product with the gate weight,
    to 8 significant bits BEFORE the k rows are added (F.linear and Tensor.mul return bf16 in the
    reference's own bf16 run), so where the rows are large and partly cancel, the error of the
    sum is a fraction of the operands' size, not of the result's. With outputs below 1 in
    magnitude S = 1 and this is plain rtol / atol. The count under the plain bar is reported too."""
    gpu, ref = y_gpu_rows.float(), y_ref_rows.float()
    err = (gpu - ref).abs()
    strict = (err > atol + rtol * ref.abs()).any(dim=1)
    scale = torch.ones(ref.shape[0]) if operand_scale is None else operand_scale.float().clamp_min(1.0)
    bad = (err > atol * scale.view(-1, 1) + rtol * ref.abs()).any(dim=1)
    return dict(tokens=int(ref.shape[0]), tokens_out_of_tolerance=int(bad.sum()),
                max_abs_err=float(err.max()) if err.numel() else 0.0, rtol=rtol, atol=atol,
                atol_scale="max(1, largest |gate-weighted expert row| of the token)" if operand_scale is not None else "1",
                max_operand_scale=float(scale.max()) if scale.numel() else 1.0,
                tokens_out_of_plain_rtol_atol=int(strict.sum()),
                elements_out_of_plain_rtol_atol=float((err > atol + rtol * ref.abs()).float().mean()) if err.numel() else 0.0)


def routing_exactness(idx_gpu: torch.Tensor, idx_ref: torch.Tensor, gap: torch.Tensor, min_gap: float = 1e-6
                      ) -> Dict[str, int]:
    """Expert sets per token, GPU against oracle (slot order aside). Tokens whose k-th and
    (k+1)-th scores are closer than min_gap are counted separately, not as mismatches."""
    a = torch.sort(idx_gpu.cpu(), dim=1).values
    b = torch.sort(idx_ref, dim=1).values
    diff = (a != b).any(dim=1)
    near = gap < min_gap
    return dict(tokens=int(a.shape[0]), mismatched=int((diff & ~near).sum()), near_ties=int(near.sum()),
                near_tie_mismatches=int((diff & near).sum()))

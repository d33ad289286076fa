"""Routing operators: gate -> softmax -> top-k, and the stable counting sort that produces the
jagged offsets and permutation tensors. They stand in for the eager ATen sequence in the
reference's FastMoELayer (modules/fast_moe_module.py:93-144)."""
from __future__ import annotations

from typing import NamedTuple, Optional, Tuple

import torch

from .. import _lib


class RoutingMetadata(NamedTuple):
    gate_index: torch.Tensor      # [L*k] int64: stable argsort of topk_idx.view(-1); value = token*k + slot
    token_index: torch.Tensor     # [L*k] int64: gate_index // k
    offsets: torch.Tensor         # [E+1] int64
    reverse_index: torch.Tensor   # [L, k] int64: stable argsort of token_index
    lengths: torch.Tensor         # [E] int64
    max_len: torch.Tensor         # [1] int64, on the device


def split_gate_weight(gate_weight: torch.Tensor) -> torch.Tensor:
    """Two-term bf16 expansion of the fp32 gate weights, hi = bf16(W), lo = bf16(W - hi), stacked
    as one [1, 2E, d] weight whose reduction dimension is contiguous. x @ hi + x @ lo reproduces
    x @ W to about 2^-17 relative per weight while running on the bf16 tensor cores; it is what
    ``gate_topk`` uses when a precomputed split is passed in (worth it once E * d is large)."""
    w = gate_weight.detach().to(torch.float32)
    hi = w.to(torch.bfloat16)
    lo = (w - hi.to(torch.float32)).to(torch.bfloat16)
    return torch.cat([hi, lo], dim=0).unsqueeze(0).contiguous()


def gate_topk(
    x: Optional[torch.Tensor],
    gate_weight: Optional[torch.Tensor],
    gate_bias: Optional[torch.Tensor],
    k: int,
    logits: Optional[torch.Tensor] = None,
    return_logits: bool = False,
    gate_split: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """softmax(x @ Wg^T + bg) -> top-k -> scores of the chosen experts renormalised to sum 1.

    x [L, d] (bf16 / f32), gate_weight [E, d], gate_bias [E] or None; the gate parameters are
    used in fp32. Alternatively pass ``logits`` [L, E] f32 and no x. With ``gate_split``
    (see ``split_gate_weight``) and bf16 x, the logits are computed by the tensor-core grouped
    GEMM instead of the CUDA-core loop. Returns
    (topk_idx [L, k] int64 with slots in descending score order, ties to the lower expert id;
    topk_score [L, k] f32; logits [L, E] f32 if requested).
    """
    lib = _lib.load()
    split = 0
    if logits is not None:
        dev = _lib.require_cuda(logits)
        lg = logits.to(torch.float32).contiguous()
        L, E = lg.shape
        ld_lg = E
        xx = gw = None
        gb = None
        d = 0
        x_dt = _lib.F32
        ldx = 0
    else:
        assert x is not None and gate_weight is not None
        dev = _lib.require_cuda(x, gate_weight, gate_bias)
        assert x.ndim == 2 and gate_weight.ndim == 2 and gate_weight.shape[1] == x.shape[1]
        xx = x if x.stride(1) == 1 else x.contiguous()
        gb = None if gate_bias is None else gate_bias.detach().to(torch.float32).contiguous()
        L, d = xx.shape
        E = gate_weight.shape[0]
        x_dt = _lib.dtype_code(xx.dtype)
        ldx = xx.stride(0)
        lg = None
        ld_lg = 0
        gw = None
        if gate_split is not None and xx.dtype == torch.bfloat16 and d % 8 == 0 and L > 0:
            from .moe import silu_jagged_bmm_raw

            off = torch.arange(2, dtype=torch.int64, device=dev) * L      # [0, L], built on the device
            lg = silu_jagged_bmm_raw(off, xx, gate_split.permute(0, 2, 1), out_dtype=torch.float32)   # [L, 2E]
            ld_lg = lg.stride(0)
            split = 1
            xx = None
        else:
            gw = gate_weight.detach().to(torch.float32).contiguous()
    idx = torch.empty((L, k), dtype=torch.int64, device=dev)
    score = torch.empty((L, k), dtype=torch.float32, device=dev)
    lout = torch.empty((L, E), dtype=torch.float32, device=dev) if return_logits else None
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_gate_topk(
                _lib.ptr(xx), x_dt, ldx, _lib.ptr(gw), _lib.ptr(gb), _lib.ptr(lg), ld_lg, split, L, d, E, k,
                _lib.ptr(lout), idx.data_ptr(), score.data_ptr(), _lib.stream_ptr(dev),
            )
        )
    return idx, score, lout


def route_metadata(topk_idx: torch.Tensor, num_experts: int) -> RoutingMetadata:
    """Stable counting sort of the (token, slot) pairs by expert id, on the device, with no
    host synchronisation."""
    lib = _lib.load()
    dev = _lib.require_cuda(topk_idx)
    assert topk_idx.ndim == 2
    idx = topk_idx.to(torch.int64).contiguous()
    L, k = idx.shape
    E = num_experts
    A = L * k
    i64 = dict(dtype=torch.int64, device=dev)
    lengths = torch.empty(E, **i64)
    offsets = torch.empty(E + 1, **i64)
    gate_index = torch.empty(A, **i64)
    token_index = torch.empty(A, **i64)
    reverse = torch.empty((L, k), **i64)
    max_len = torch.empty(1, **i64)
    ws_bytes = int(lib.fmoe_route_workspace_bytes(L, E, k))
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_route_metadata(
                idx.data_ptr(), L, E, k, lengths.data_ptr(), offsets.data_ptr(), gate_index.data_ptr(),
                token_index.data_ptr(), reverse.data_ptr(), max_len.data_ptr(), ws.data_ptr(), ws.numel(),
                _lib.stream_ptr(dev),
            )
        )
    return RoutingMetadata(gate_index, token_index, offsets, reverse, lengths, max_len)


def fused_routing_supported(x: torch.Tensor, gate_weight: torch.Tensor) -> bool:
    """True when ``route_tokens_fused`` can serve these tokens: bf16 rows that are 16-byte aligned,
    at most 32 experts, and a batch small enough for the single-launch placement."""
    if not x.is_cuda or x.ndim != 2 or x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[0] == 0:
        return False
    if gate_weight.dtype != torch.float32 or not gate_weight.is_contiguous():
        return False
    lib = _lib.load()
    return bool(lib.fmoe_gate_topk_counts_supported(x.data_ptr(), _lib.BF16, x.stride(0), gate_weight.data_ptr(),
                                                    x.shape[0], x.shape[1], gate_weight.shape[0]))


def route_tokens_fused(
    x: torch.Tensor,
    gate_weight: torch.Tensor,
    gate_bias: Optional[torch.Tensor],
    k: int,
    gather_rows: bool = False,
    zero_rows: Optional[Tuple[int, torch.dtype]] = None,
) -> Tuple[torch.Tensor, torch.Tensor, RoutingMetadata, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``gate_topk`` + ``route_metadata`` for small batches as two launches that read the expert
    choices once: the gate kernel also emits the rows per expert of every group of 16 tokens, and
    the placement kernel starts from those counts. The placement kernel can take two memory passes
    along that the layers would otherwise run as launches of their own:
      ``gather_rows``  returns x_sorted [L*k, d] with x_sorted[p] = x[token_index[p]] (the
                       index_select of the up projection; x is read once);
      ``zero_rows``    (cols, dtype): returns a cleared [L, cols] buffer (what a fused combine
                       accumulates into).
    Every tensor is bit-identical to what the separate operators produce. Returns
    (topk_idx, topk_score, RoutingMetadata, x_sorted or None, cleared buffer or None)."""
    lib = _lib.load()
    dev = _lib.require_cuda(x, gate_weight, gate_bias)
    L, d = x.shape
    E = gate_weight.shape[0]
    gb = None if gate_bias is None else gate_bias.detach().to(torch.float32).contiguous()
    gw = gate_weight.detach()
    i64 = dict(dtype=torch.int64, device=dev)
    idx = torch.empty((L, k), **i64)
    score = torch.empty((L, k), dtype=torch.float32, device=dev)
    counts = torch.empty(int(lib.fmoe_route_group_counts_bytes(L, E)) // 4, dtype=torch.int32, device=dev)
    A = L * k
    lengths = torch.empty(E, **i64)
    offsets = torch.empty(E + 1, **i64)
    gate_index = torch.empty(A, **i64)
    token_index = torch.empty(A, **i64)
    reverse = torch.empty((L, k), **i64)
    max_len = torch.empty(1, **i64)
    x_sorted = torch.empty((A, d), dtype=x.dtype, device=dev) if gather_rows else None
    zbuf = torch.empty((L, zero_rows[0]), dtype=zero_rows[1], device=dev) if zero_rows is not None else None
    with torch.cuda.device(dev):
        st = _lib.stream_ptr(dev)
        # the clear rides in the gate kernel: plain stores under its load latency
        in_gate = zbuf is not None
        zargs = (zbuf.data_ptr(), _lib.dtype_code(zbuf.dtype), zbuf.stride(0), zbuf.shape[1]) if zbuf is not None else (None, 0, 0, 0)
        none = (None, 0, 0, 0)
        _lib.check(lib.fmoe_gate_topk_counts(x.data_ptr(), _lib.BF16, x.stride(0), gw.data_ptr(), _lib.ptr(gb), L, d, E, k,
                                             None, idx.data_ptr(), score.data_ptr(), counts.data_ptr(),
                                             *(zargs if in_gate else none), st))
        _lib.check(lib.fmoe_route_metadata_gather(
            idx.data_ptr(), L, E, k, counts.data_ptr(), lengths.data_ptr(), offsets.data_ptr(), gate_index.data_ptr(),
            token_index.data_ptr(), reverse.data_ptr(), max_len.data_ptr(),
            x.data_ptr(), _lib.BF16, x.stride(0), d, _lib.ptr(x_sorted), d, *(none if in_gate else zargs), st))
    return idx, score, RoutingMetadata(gate_index, token_index, offsets, reverse, lengths, max_len), x_sorted, zbuf


def gate_topk_normalized(
    x: Optional[torch.Tensor],
    gate_weight: Optional[torch.Tensor],
    k: int,
    logits: Optional[torch.Tensor] = None,
    return_logits: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Router of the sparsely-gated layer (kernels/pytorch/mrn.py:236-252 of the reference):
    logits = x @ gate_weight^T divided by their L2 norm per token, softmax over all experts, the k
    largest probabilities in descending order (ties to the lower expert id), NOT renormalised.
    gate_weight is [E, d] (the reference keeps [d, E]); ``logits`` may be given instead of x.
    Returns (topk_idx [L, k] int64, gates [L, k] f32, un-normalised logits if requested)."""
    lib = _lib.load()
    if logits is not None:
        dev = _lib.require_cuda(logits)
        lg = logits.to(torch.float32).contiguous()
        L, E = lg.shape
        xx = gw = None
        d, x_dt, ldx, ld_lg = 0, _lib.F32, 0, E
    else:
        assert x is not None and gate_weight is not None
        dev = _lib.require_cuda(x, gate_weight)
        xx = x if x.stride(1) == 1 else x.contiguous()
        gw = gate_weight.detach().to(torch.float32).contiguous()
        L, d = xx.shape
        E = gw.shape[0]
        assert gw.shape[1] == d
        x_dt, ldx, lg, ld_lg = _lib.dtype_code(xx.dtype), xx.stride(0), None, 0
    idx = torch.empty((L, k), dtype=torch.int64, device=dev)
    score = torch.empty((L, k), dtype=torch.float32, device=dev)
    lout = torch.empty((L, E), dtype=torch.float32, device=dev) if return_logits else None
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_gate_topk_normalized(_lib.ptr(xx), x_dt, ldx, _lib.ptr(gw), None, _lib.ptr(lg), ld_lg, L, d, E, k,
                                                 _lib.ptr(lout), idx.data_ptr(), score.data_ptr(), _lib.stream_ptr(dev)))
    return idx, score, lout


def token_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float,
               group_norm: bool = False, num_groups: int = 1) -> torch.Tensor:
    """Layer norm of the rows of x [L, d], or (``group_norm``) F.group_norm of x viewed as
    [L, num_groups, d / num_groups] with one weight / bias per group; fp32 statistics, result in
    the dtype of x (kernels/pytorch/mrn.py:301-318 of the reference)."""
    lib = _lib.load()
    dev = _lib.require_cuda(x, weight, bias)
    assert x.ndim == 2
    xx = x if x.stride(1) == 1 else x.contiguous()
    L, d = xx.shape
    groups = num_groups if group_norm else 1
    w = None if weight is None else weight.detach().to(torch.float32).contiguous()
    b = None if bias is None else bias.detach().to(torch.float32).contiguous()
    want = groups if group_norm else d
    assert (w is None or w.numel() == want) and (b is None or b.numel() == want), "norm weight / bias size"
    out = torch.empty((L, d), dtype=xx.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_token_norm(xx.data_ptr(), _lib.dtype_code(xx.dtype), L, d, xx.stride(0) if L else d, groups,
                                       _lib.ptr(w), _lib.ptr(b), 1 if group_norm else 0, float(eps), out.data_ptr(), d,
                                       _lib.stream_ptr(dev)))
    return out


def sg_load_loss(meta: RoutingMetadata, score: torch.Tensor, num_experts: int, token_dtype: torch.dtype,
                 loss_coef: float, train: bool, smooth_load: Optional[torch.Tensor] = None
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """(loss scalar f32, load fractions [E] f32) of the sparsely-gated layer
    (kernels/pytorch/mrn.py:253-287): loss = coef * (cv2(importance) + cv2(load)) when training,
    0 otherwise; load fraction = rows of expert e / all rows. ``smooth_load`` [blocks, E]: the
    per-block sums of `noisy_gate`'s load estimate, which then replace the row counts in the loss."""
    lib = _lib.load()
    dev = _lib.require_cuda(score, meta.offsets, smooth_load)
    load = torch.empty(num_experts, dtype=torch.float32, device=dev)
    loss = torch.empty((), dtype=torch.float32, device=dev)
    sc = score.contiguous()
    gidx = meta.gate_index
    if sc.numel() == 0:      # an empty batch: its tensors have no storage; nothing is read through these
        sc = torch.zeros(1, dtype=torch.float32, device=dev)
        gidx = torch.zeros(1, dtype=torch.int64, device=dev)
    n_part = 0
    if smooth_load is not None:
        assert smooth_load.dtype == torch.float32 and smooth_load.is_contiguous() and smooth_load.shape[1] == num_experts
        n_part = smooth_load.shape[0]
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_sg_load_loss(meta.offsets.data_ptr(), gidx.data_ptr(), sc.data_ptr(), num_experts,
                                         1 if token_dtype == torch.bfloat16 else 0, float(loss_coef), 1 if train else 0,
                                         _lib.ptr(smooth_load), n_part, load.data_ptr(), loss.data_ptr(),
                                         _lib.stream_ptr(dev)))
    return loss, load


def noisy_gate(x: torch.Tensor, gate_noise_weight: torch.Tensor, k: int, noise: torch.Tensor, noise_eps: float = 1e-2
               ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Training-time router of the sparsely-gated layer with noisy gating
    (OrigSGMoEImpl._orig_noisy_gating and _prob_in_top_k, kernels/pytorch/mrn.py:191-252):
    x [L, d]; gate_noise_weight [2E, d] f32 = w_gate^T stacked on w_noise^T; noise [L, E] f32 (a
    standard-normal draw). Returns (topk_idx [L, k], gates [L, k] f32, per-block sums [blocks, E]
    of the smooth load for `sg_load_loss`, or None when k == E and every expert is picked)."""
    lib = _lib.load()
    dev = _lib.require_cuda(x, gate_noise_weight, noise)
    E2 = gate_noise_weight.shape[0]
    assert E2 % 2 == 0
    E = E2 // 2
    L = x.shape[0]
    assert noise.shape == (L, E) and noise.dtype == torch.float32
    if E2 > 256:
        raise ValueError(f"noisy gating supports up to 128 experts, got {E}")
    _, _, logits2 = gate_topk_normalized(x, gate_noise_weight, 1, return_logits=True)
    noisy = torch.empty((L, E), dtype=torch.float32, device=dev)
    stddev = torch.empty((L, E), dtype=torch.float32, device=dev)
    nz = noise.contiguous()
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_sg_noisy_logits(logits2.data_ptr(), E2, nz.data_ptr(), L, E, float(noise_eps), noisy.data_ptr(),
                                            stddev.data_ptr(), _lib.stream_ptr(dev)))
    idx, score, _ = gate_topk_normalized(None, None, k, logits=noisy)
    partials = None
    if k < E:
        blocks = max(1, min(148, (L + 7) // 8))
        partials = torch.empty((blocks, E), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.fmoe_sg_noisy_load(logits2.data_ptr(), E2, noisy.data_ptr(), stddev.data_ptr(), L, E, k,
                                              partials.data_ptr(), blocks, _lib.stream_ptr(dev)))
    return idx, score, partials

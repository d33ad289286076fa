"""CPU restatement of the reference's MoE forward path (meta-recsys/fast_moe, KernelType.PYTORCH).

TEST INFRASTRUCTURE ONLY. This module is the checker the CUDA kernels are compared against; it is
imported by tests/, by __graft_entry__.smoke() and by the CPU-baseline / reference legs of
bench.py, never by the fast_moe_b200 package. Parity status: PINNED - every function below is
compared with the reference's own code (imported through oracle/reference_shims.py) by
oracle/check_against_reference.py and by the golden fixtures under tests/golden/.

Floating-point work uses torch CPU ops in fp32 (the arithmetic the reference's PYTORCH path
performs); integer routing and the FP8 byte codec are plain numpy. Paths in the docstrings are
relative to the reference repository.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

FP8_MAX = 448.0
TWO_POW_127 = float(2.0**127)


# ------------------------------------------------------------------------------ routing
def gating_scores(x: torch.Tensor, gate_w: torch.Tensor, gate_b: Optional[torch.Tensor]) -> torch.Tensor:
    """softmax over experts of x @ gate_w^T + gate_b. x [..., d], gate_w [E, d].
    GatingNetwork.forward, modules/fast_moe_module.py:21-27."""
    return torch.softmax(F.linear(x, gate_w, gate_b), dim=-1)


def select_top_k(scores: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k experts per token and the dense score matrix with everything else zeroed and each
    row L1-normalised (eps 1e-12). FastMoELayer._select_top_k_experts,
    modules/fast_moe_module.py:93-105. Slot order: descending score, ties to the lower expert id
    (what torch.topk(sorted=False) returns on CPU for these sizes; the slot order only changes
    gate_index, never offsets / token_index / reverse_index)."""
    s = scores.reshape(-1, scores.shape[-1]).to(torch.float32).numpy()
    L, E = s.shape
    # stable argsort of -score gives descending score with ties to the lower index
    order = np.argsort(-s, axis=1, kind="stable")[:, :k]
    mask = np.zeros_like(s)
    np.put_along_axis(mask, order, 1.0, axis=1)
    kept = s * mask
    denom = np.maximum(np.abs(kept).sum(axis=1, keepdims=True), 1e-12)
    dense = (kept / denom).astype(np.float32)
    return torch.from_numpy(dense), torch.from_numpy(order.astype(np.int64))


def routing_metadata(dense_scores: torch.Tensor, topk_idx: torch.Tensor):
    """FastMoELayer._compute_routing_metadata, modules/fast_moe_module.py:107-144, including the
    fbgemm exclusive-cumsum-with-total (asynchronous_complete_cumsum, :131).
    Returns gate_index [A], token_index [A], gating_scores [L,k], offsets [E+1],
    reverse_token_index [L,k], max_seq_len (int); all index tensors int64."""
    idx = topk_idx.numpy().astype(np.int64)
    L, k = idx.shape
    dense = dense_scores.numpy()
    E = dense.shape[1]
    gate_index = np.argsort(idx.reshape(-1), kind="stable").astype(np.int64)
    token_index = gate_index // k
    lengths = (dense > 0).sum(axis=0).astype(np.int64)          # load = scores > 0 (:120,126)
    offsets = np.zeros(E + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    scores_k = np.take_along_axis(dense, idx, axis=1)
    reverse = np.argsort(token_index, kind="stable").astype(np.int64).reshape(L, k)
    max_seq_len = int(lengths.max()) if E > 0 else 0
    return (
        torch.from_numpy(gate_index),
        torch.from_numpy(token_index),
        torch.from_numpy(scores_k),
        torch.from_numpy(offsets),
        torch.from_numpy(reverse),
        max_seq_len,
    )


def histogram_lengths(topk_idx: torch.Tensor, E: int) -> torch.Tensor:
    """Rows per expert counted from the chosen indices (what the CUDA routing kernel computes).
    Equal to the reference's ``(scores > 0).sum(0)`` unless a chosen expert's softmax score
    underflowed to exactly 0."""
    return torch.from_numpy(np.bincount(topk_idx.numpy().reshape(-1), minlength=E).astype(np.int64))


# ------------------------------------------------------------------------------ expert GEMMs
def _segments(offsets: torch.Tensor) -> List[int]:
    o = offsets.tolist()
    return [o[i + 1] - o[i] for i in range(len(o) - 1)]


def _gather_rows(index: torch.Tensor, jagged: torch.Tensor) -> torch.Tensor:
    tok = index.reshape(-1) // index.shape[-1]
    return jagged[tok].contiguous()


def index_select_jagged_bmm(offsets, index, jagged, weight, bias) -> torch.Tensor:
    """Per expert e: rows gathered by index // A times weight[e] ([K, N]) plus bias[e].
    pytorch_index_select_jagged_bmm, kernels/pytorch/moe.py:40-84."""
    parts = _gather_rows(index, jagged).split(_segments(offsets))
    wt = weight.permute(0, 2, 1)
    outs = [F.linear(p, wt[e], None if bias is None else bias[e]) for e, p in enumerate(parts)]
    return torch.cat(outs, dim=0)


def index_select_jagged_bmm_3D(offsets, index, jagged, weight, bias) -> torch.Tensor:
    """jagged is [L, E, K]: the rows of expert e read slice e of their token, then weight[e] and
    bias[e] as in index_select_jagged_bmm. pytorch_index_select_jagged_bmm_3D,
    kernels/pytorch/moe.py:224-252."""
    tok = index.reshape(-1) // index.shape[-1]
    parts = jagged[tok].contiguous().split(_segments(offsets))
    wt = weight.permute(0, 2, 1)
    outs = [F.linear(p[:, e, :], wt[e], None if bias is None else bias[e]) for e, p in enumerate(parts)]
    return torch.cat(outs, dim=0)


def index_select_jagged_bmm_swiglu(offsets, index, jagged, weight, bias, weight_p, bias_p) -> torch.Tensor:
    """silu(x W + b) * (x Wp + bp) per expert. pytorch_index_select_jagged_bmm_swiglu,
    kernels/pytorch/moe.py:87-146."""
    parts = _gather_rows(index, jagged).split(_segments(offsets))
    wt, wpt = weight.permute(0, 2, 1), weight_p.permute(0, 2, 1)
    outs = []
    for e, p in enumerate(parts):
        g = F.linear(p, wt[e], None if bias is None else bias[e])
        u = F.linear(p, wpt[e], None if bias_p is None else bias_p[e])
        outs.append(F.silu(g) * u)
    return torch.cat(outs, dim=0)


def index_select_jagged_gating_bmm(offsets, index, jagged_a, jagged_b, weight_a, weight_b, bias_a, bias_b):
    """silu(A_g Wa + ba) * (B_g Wb + bb). pytorch_index_select_jagged_gating_bmm,
    kernels/pytorch/moe.py:149-221."""
    alpha = index_select_jagged_bmm(offsets, index, jagged_a, weight_a, bias_a)
    beta = index_select_jagged_bmm(offsets, index, jagged_b, weight_b, bias_b)
    return F.silu(alpha) * beta


def silu_jagged_bmm(offsets, jagged, weight, bias, has_silu: bool = True) -> torch.Tensor:
    """[silu](segment) @ weight[e] + bias[e]; weight is logical [E, K, N].
    pytorch_silu_jagged_bmm, kernels/pytorch/moe.py:255-275 (which receives the weight already
    permuted to [E, N, K] by its caller, :288-294)."""
    a = F.silu(jagged) if has_silu else jagged
    parts = a.split(_segments(offsets))
    wt = weight.permute(0, 2, 1)
    outs = [F.linear(p, wt[e], None if bias is None else bias[e]) for e, p in enumerate(parts)]
    return torch.cat(outs, dim=0)


def mul_merge_k_add(index, value, k: int, weight=None, weight_index=None) -> torch.Tensor:
    """value rows scaled by weight.view(-1)[weight_index], summed into their token row in fp32
    (ascending row order), cast back. pytorch_mul_merge_k_add, kernels/pytorch/moe.py:14-37."""
    if weight is not None:
        value = value * weight.contiguous().view(-1)[weight_index].view(-1, 1)
    acc = torch.zeros(index.shape[0] // k, value.shape[1], dtype=torch.float32)
    return acc.index_add(0, index, value.float()).to(value.dtype)


def silu_jagged_bmm_combine(offsets, jagged, weight, bias, index, k, gating_scores=None, gates_index=None,
                            has_silu: bool = True) -> torch.Tensor:
    """pytorch_silu_jagged_bmm_combine, kernels/pytorch/moe.py:278-303."""
    y = silu_jagged_bmm(offsets, jagged, weight, bias, has_silu)
    return mul_merge_k_add(index, y, k, gating_scores, gates_index)


def fused_jagged_bmm_swiglu_combine(offsets, index, jagged, weight, bias, weight_p, bias_p, weight_out, bias_out,
                                    k, gates=None, gates_index=None) -> torch.Tensor:
    """Whole SwiGLU expert FFN and combine in one call; ``index`` is the [L, k] gate_index
    tensor. pytorch_fused_jagged_bmm_swiglu_combine, kernels/pytorch/moe.py:306-391."""
    hidden = index_select_jagged_bmm_swiglu(offsets, index, jagged, weight, bias, weight_p, bias_p)
    y = silu_jagged_bmm(offsets, hidden, weight_out, bias_out, has_silu=False)
    tok = index.reshape(-1) // index.shape[-1]
    return mul_merge_k_add(tok, y, k, gates, gates_index)


# ------------------------------------------------------------------------------ layers
def moe_layer_mlp(x, gate_w, gate_b, w_hidden, b_hidden, w_out, b_out, k: int) -> torch.Tensor:
    """FastMoELayer.forward as shipped: fc1 + bias -> SiLU -> fc2 + bias -> weighted combine.
    modules/fast_moe_module.py:188-225. w_hidden is the parameter _experts_hidden_w [E, h, d],
    w_out is _experts_w [E, o, h] (the layer hands their permuted views to the operators,
    :167,177)."""
    shape = x.shape
    dense, idx = select_top_k(gating_scores(x, gate_w, gate_b), k)
    gate_index, token_index, scores_k, offsets, reverse, _ = routing_metadata(dense, idx)
    xf = x.reshape(-1, shape[-1])
    hidden = index_select_jagged_bmm(offsets, gate_index.view(-1, k), xf, w_hidden.permute(0, 2, 1), b_hidden)
    y = silu_jagged_bmm_combine(offsets, hidden, w_out.permute(0, 2, 1), b_out, token_index, k,
                                scores_k.to(x.dtype), gate_index, has_silu=True)
    return y.view(*shape[:-1], w_out.shape[1])


def moe_layer_swiglu(x, gate_w, gate_b, w_gate, w_up, w_down, k: int, b_gate=None, b_up=None,
                     b_down=None) -> torch.Tensor:
    """The SwiGLU layer the benchmark configurations describe: FastMoELayer routing, then
    index_select_jagged_bmm_swiglu and silu_jagged_bmm_combine(has_silu=False).
    Weights are logical [E, K, N]: w_gate / w_up [E, d, h], w_down [E, h, o]."""
    shape = x.shape
    dense, idx = select_top_k(gating_scores(x, gate_w, gate_b), k)
    gate_index, token_index, scores_k, offsets, reverse, _ = routing_metadata(dense, idx)
    xf = x.reshape(-1, shape[-1])
    y = fused_jagged_bmm_swiglu_combine(offsets, gate_index.view(-1, k), xf, w_gate, b_gate, w_up, b_up, w_down,
                                        b_down, k, scores_k.to(x.dtype), gate_index)
    return y.view(*shape[:-1], w_down.shape[2])


def moe_dense_reference(x, gate_w, gate_b, w_hidden, b_hidden, w_out, b_out, k: int) -> torch.Tensor:
    """Every expert applied to every token, mixed with the masked, renormalised gate scores:
    the ground truth the reference checks FastMoELayer against. MoeBase.forward,
    modules/moe_base.py:61-94 (with SiLU experts)."""
    shape = x.shape
    dense, _ = select_top_k(gating_scores(x, gate_w, gate_b), k)
    xf = x.reshape(-1, shape[-1])
    out = torch.zeros(xf.shape[0], w_out.shape[1], dtype=torch.float32)
    for e in range(w_hidden.shape[0]):
        h = F.silu(F.linear(xf, w_hidden[e], b_hidden[e]))
        out += dense[:, e : e + 1] * F.linear(h, w_out[e], b_out[e]).float()
    return out.to(x.dtype).view(*shape[:-1], w_out.shape[1])


# ------------------------------------------------------------------------------ FP8
def fp32_to_e4m3fn(v: np.ndarray) -> np.ndarray:
    """float32 -> float8_e4m3fn bytes, round to nearest even, no saturation (anything that would
    round past 448, and NaN, becomes 0x7F with the sign). This is the published conversion of
    c10::Float8_e4m3fn that Tensor.to(torch.float8_e4m3fn) performs
    (call site: kernels/pytorch/quant_fp8.py:33)."""
    f = np.ascontiguousarray(v, dtype=np.float32)
    flat = f.reshape(-1)
    out = np.empty(flat.shape, dtype=np.uint8)
    magic = np.float32(2.0 ** (141 - 127))
    step = 1 << 22                               # chunks keep the temporaries inside the cache
    for lo in range(0, flat.size, step):
        bits = flat[lo : lo + step].view(np.uint32)
        sign = ((bits >> np.uint32(24)) & np.uint32(0x80)).astype(np.uint8)
        mag = bits & np.uint32(0x7FFFFFFF)
        # normal range: re-bias the exponent, add half an e4m3 ulp (+1 when the kept bit is odd:
        # round to nearest even) and drop the 20 low mantissa bits; uint32 arithmetic wraps
        odd = (mag >> np.uint32(20)) & np.uint32(1)
        m_norm = (mag + np.uint32(((7 - 127) << 23) & 0xFFFFFFFF) + np.uint32(0x7FFFF) + odd) >> np.uint32(20)
        # below 2^-6 the value lands in the e4m3 subnormals: adding 2^14 lets the fp32 adder do
        # the round-to-nearest-even at the subnormal spacing 2^-9
        small = mag < np.uint32(121 << 23)
        fm = np.where(small, mag, np.uint32(0)).view(np.float32)
        m_small = (fm + magic).astype(np.float32).view(np.uint32) - np.uint32(141 << 23)
        over = mag >= np.uint32(1087 << 20)      # >= 480.0, inf, NaN
        code = np.where(over, np.uint32(0x7F), np.where(small, m_small, m_norm))
        out[lo : lo + step] = (code & np.uint32(0xFF)).astype(np.uint8) | sign
    return out.reshape(f.shape)


def _e4m3fn_table() -> np.ndarray:
    b = np.arange(256, dtype=np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0).astype(np.float32)
    exp = (b >> 3) & 0xF
    man = b & 0x7
    val = np.where(exp == 0, man * 2.0**-9, (1.0 + man / 8.0) * np.exp2(exp.astype(np.float32) - 7.0))
    val = np.where((exp == 15) & (man == 7), np.nan, val)
    return (sign * val).astype(np.float32)


_E4M3FN_TABLE = _e4m3fn_table()


def e4m3fn_to_fp32(b: np.ndarray) -> np.ndarray:
    """float8_e4m3fn bytes -> float32 (exact): sign, 4 exponent bits (bias 7), 3 mantissa bits,
    subnormals at exponent 0, 0x7F / 0xFF = NaN, no infinities. Table of the 256 codes."""
    return _E4M3FN_TABLE[np.asarray(b, dtype=np.uint8)]


def calculate_scale(a_max: torch.Tensor) -> torch.Tensor:
    """scale = 2^floor(log2(448 / amax)), 2^127 where that is inf or NaN. The division keeps the
    dtype of a_max (bf16 inputs divide in bf16) before widening to fp32.
    calculate_scale, kernels/pytorch/quant_fp8.py:13-23."""
    s = torch.div(FP8_MAX, a_max).to(torch.float32)
    s = torch.exp2(torch.floor(torch.log2(s)))
    bad = torch.isnan(s) | torch.isinf(s)
    return torch.where(bad, torch.full_like(s, TWO_POW_127), s)


def rowwise_quant_fp8(a: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(e4m3 bytes as uint8, fp32 scale per row of the last dim).
    pytorch_rowwise_quant_fp8, kernels/pytorch/quant_fp8.py:26-34."""
    a = a.contiguous()
    amax = a.abs().amax(dim=-1)
    scale = calculate_scale(amax)
    prod = (a * scale.unsqueeze(-1)).to(torch.float32)
    q = fp32_to_e4m3fn(prod.numpy())
    return torch.from_numpy(q), scale


def silu_jagged_fp8(jagged: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """silu in the input dtype, widened to fp32, rowwise quantised. Returns (bytes, scale); the
    reference returns only the quantised tensor. pytorch_silu_jagged_fp8,
    kernels/pytorch/moe_fp8.py:17-33."""
    s = F.silu(jagged).to(torch.float32)
    scale = calculate_scale(s.abs().amax(dim=1))
    q = fp32_to_e4m3fn((s * scale[:, None]).numpy())
    return torch.from_numpy(q), scale


def bmm_weight_rowwise_quant_fp8(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """weight [E, K, D]: absmax over K per (e, d). pytorch_bmm_weight_rowwise_quant_fp8,
    kernels/pytorch/moe_fp8.py:36-43."""
    amax = weight.abs().amax(dim=1)
    scale = calculate_scale(amax)
    q = fp32_to_e4m3fn((weight * scale[:, None, :]).to(torch.float32).numpy())
    return torch.from_numpy(q), scale


def index_select_jagged_bmm_fp8(offsets, index, jagged, weight, bias) -> torch.Tensor:
    """Quantise weight^T rows and token rows, multiply the quantised values (bf16 matmul of the
    exactly representable e4m3 values), divide by the scale product, cast, add bias.
    pytorch_index_select_jagged_bmm_fp8, kernels/pytorch/moe_fp8.py:98-139."""
    out_dtype = jagged.dtype
    wq, ws = rowwise_quant_fp8(weight.permute(0, 2, 1))      # [E, N, K], [E, N]
    xq, xs = rowwise_quant_fp8(jagged)                       # [L, K], [L]
    wv = torch.from_numpy(e4m3fn_to_fp32(wq.numpy())).to(torch.bfloat16)
    xv = torch.from_numpy(e4m3fn_to_fp32(xq.numpy())).to(torch.bfloat16)
    tok = index.reshape(-1) // index.shape[-1]
    seg = _segments(offsets)
    xparts = xv[tok].contiguous().split(seg)
    sparts = xs[tok].contiguous().split(seg)
    outs = []
    for e, (xp, sp) in enumerate(zip(xparts, sparts)):
        acc = torch.matmul(xp, wv[e].T)
        o = (acc / (sp[:, None] * ws[e][None, :])).to(out_dtype)
        outs.append(o + (bias[e] if bias is not None else 0))
    return torch.cat(outs, dim=0)


def silu_jagged_bmm_fp8(offsets, jagged, weight, bias, has_silu: bool = True) -> torch.Tensor:
    """FP8 down projection, [silu](jagged) @ weight[e] + bias[e] with e4m3 operands; weight is
    logical [E, K, N]. PARITY UNPINNED in the reference: the PYTORCH branch of silu_jagged_bmm_fp8
    (kernels/moe_fp8.py:98-124 -> kernels/pytorch/moe_fp8.py:46-75) quantises its operands, throws
    the result away and returns the unquantised product, and no reference test calls the
    operator. This restatement is therefore assembled from the pinned pieces, in the shape of the
    one FP8 GEMM the reference does define (pytorch_index_select_jagged_bmm_fp8,
    kernels/pytorch/moe_fp8.py:98-139): activations quantised per row after SiLU
    (pytorch_silu_jagged_fp8, :17-33, or the plain rowwise rule without SiLU), weight quantised
    per (expert, output column) over K, bf16 matmul of the e4m3 values, division by the scale
    product, cast to the activation type, bias added afterwards."""
    out_dtype = jagged.dtype
    xq, xs = silu_jagged_fp8(jagged) if has_silu else rowwise_quant_fp8(jagged)
    wq, ws = rowwise_quant_fp8(weight.permute(0, 2, 1))      # [E, N, K], [E, N]
    xv = torch.from_numpy(e4m3fn_to_fp32(xq.numpy())).to(torch.bfloat16)
    wv = torch.from_numpy(e4m3fn_to_fp32(wq.numpy())).to(torch.bfloat16)
    seg = _segments(offsets)
    outs = []
    for e, (xp, sp) in enumerate(zip(xv.split(seg), xs.split(seg))):
        acc = torch.matmul(xp, wv[e].T)
        o = (acc / (sp[:, None] * ws[e][None, :])).to(out_dtype)
        outs.append(o + (bias[e] if bias is not None else 0))
    return torch.cat(outs, dim=0)


def silu_jagged_bmm_combine_fp8(offsets, jagged, weight, bias, index, k, gating_scores=None, gates_index=None,
                                has_silu: bool = True) -> torch.Tensor:
    """silu_jagged_bmm_fp8 followed by the gate-weighted merge (pytorch_mul_merge_k_add,
    kernels/pytorch/moe.py:14-37): the quantised meaning of silu_jagged_bmm_combine_fp8
    (kernels/moe_fp8.py:127-182). PARITY UNPINNED in the reference for the same reason as
    silu_jagged_bmm_fp8: its PYTORCH branch falls back to the unquantised operator."""
    y = silu_jagged_bmm_fp8(offsets, jagged, weight, bias, has_silu)
    return mul_merge_k_add(index, y, k, gating_scores, gates_index)


def _fp8_linear(x: torch.Tensor, w_rows: torch.Tensor) -> torch.Tensor:
    """x [rows, K] @ w_rows[N, K]^T with both operands quantised rowwise to e4m3 (rule of
    kernels/pytorch/quant_fp8.py:13-34), exact products of the quantised values accumulated in
    fp32 and divided by the scale product - the arithmetic of
    pytorch_index_select_jagged_bmm_fp8 (kernels/pytorch/moe_fp8.py:98-139) without its
    intermediate bf16 rounding."""
    xq, xs = rowwise_quant_fp8(x)
    wq, ws = rowwise_quant_fp8(w_rows)
    xv = torch.from_numpy(e4m3fn_to_fp32(xq.numpy()))
    wv = torch.from_numpy(e4m3fn_to_fp32(wq.numpy()))
    return (xv @ wv.T) / (xs[:, None] * ws[None, :])


def moe_layer_swiglu_fp8(x, gate_w, gate_b, w_gate_rows, w_up_rows, w_down_rows, k: int) -> torch.Tensor:
    """FP8 SwiGLU layer, the composition the FP8 benchmark configuration describes: routing in
    fp32, tokens quantised per row, expert weights quantised per output row ([E, N, K] storage),
    hidden activations rounded to the activation type and quantised per row again before the down
    projection, fp32 combine. Built only from the reference's quantisation rule and its FP8 GEMM
    definition; there is no single reference function for the whole chain."""
    shape = x.shape
    dt = x.dtype
    dense, idx = select_top_k(gating_scores(x.float(), gate_w, gate_b), k)
    gate_index, token_index, scores_k, offsets, reverse, _ = routing_metadata(dense, idx)
    xf = x.reshape(-1, shape[-1])
    rows = xf[token_index]
    seg = _segments(offsets)
    outs = []
    for e, r in enumerate(rows.split(seg)):
        if r.shape[0] == 0:
            outs.append(torch.zeros(0, w_down_rows.shape[1]))
            continue
        g = _fp8_linear(r, w_gate_rows[e])
        u = _fp8_linear(r, w_up_rows[e])
        hidden = (F.silu(g) * u).to(dt)
        outs.append(_fp8_linear(hidden, w_down_rows[e]).to(dt).float())
    y_rows = torch.cat(outs, dim=0)
    y = mul_merge_k_add(token_index, y_rows.to(dt), k, scores_k.to(dt), gate_index)
    return y.view(*shape[:-1], w_down_rows.shape[1])

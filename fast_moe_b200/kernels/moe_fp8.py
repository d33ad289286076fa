"""FP8 (e4m3fn, rowwise power-of-two scales) operators with the reference's signatures
(kernels/moe_fp8.py:31-248, kernels/pytorch/quant_fp8.py:13-40), backed by libfmoe_b200."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from .moe import _gather_first, _index_i64, _prep_bias, gather_rows
from .utils import KernelType


def rowwise_quant_fp8(
    a: torch.Tensor, apply_silu: bool = False, reciprocal_scale: bool = False
) -> Tuple[torch.Tensor, torch.Tensor]:
    """(a * scale).to(float8_e4m3fn) with scale = 2^floor(log2(448 / max|row|)) per row of the
    last dimension; returns (quantised tensor, fp32 scale with the leading shape of ``a``).
    pytorch_rowwise_quant_fp8, kernels/pytorch/quant_fp8.py:26-34. ``apply_silu`` quantises
    silu(a) instead (pytorch_silu_jagged_fp8, kernels/pytorch/moe_fp8.py:17-33);
    ``reciprocal_scale`` returns 1/scale, the convention of the reference's fused
    quantisation kernel (kernels/triton/triton_quant_fp8.py:273-277)."""
    lib = _lib.load()
    dev = _lib.require_cuda(a)
    if a.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"rowwise_quant_fp8: float32 or bfloat16 expected, got {a.dtype}")
    a = a.contiguous()
    cols = a.shape[-1]
    a2 = a.view(-1, cols)
    rows = a2.shape[0]
    q = torch.empty(a.shape, dtype=torch.float8_e4m3fn, device=dev)
    scale = torch.empty(a.shape[:-1], dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_rowwise_quant_fp8(
                a2.data_ptr(), _lib.dtype_code(a.dtype), rows, cols, a2.stride(0) if rows > 0 else cols,
                1 if apply_silu else 0, 1 if reciprocal_scale else 0, q.data_ptr(), cols, scale.data_ptr(),
                _lib.stream_ptr(dev),
            )
        )
    return q, scale


def transpose_rowwise_quant_fp8(a: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantises along the second-to-last dimension (pytorch_transpose_rowwise_quant_fp8,
    kernels/pytorch/quant_fp8.py:37-40): returns tensors shaped like a.transpose(-2, -1)."""
    return rowwise_quant_fp8(a.transpose(-2, -1))


def silu_jagged_fp8(
    seq_offsets: torch.Tensor,
    Jagged: torch.Tensor,
    max_seq_len: int,
    K: int,
    Silu_Jagged: Optional[torch.Tensor],
    Silu_Jagged_fp8: Optional[torch.Tensor],
    Silu_Jagged_Scale: Optional[torch.Tensor],
    kernel: KernelType = KernelType.PYTORCH,
) -> torch.Tensor:
    """silu(Jagged) quantised rowwise to e4m3 (kernels/moe_fp8.py:31-74). As in both reference
    backends, the three output-buffer arguments are ignored and a new tensor is returned."""
    q, _ = rowwise_quant_fp8(Jagged, apply_silu=True)
    return q


def bmm_weight_rowwise_quant_fp8(weight: torch.Tensor, kernel: KernelType = KernelType.PYTORCH) -> torch.Tensor:
    """weight [E, D_in, D_out] -> e4m3 with one scale per (expert, output column), absmax taken
    over D_in (kernels/moe_fp8.py:77-95)."""
    q, _ = bmm_weight_quant_fp8(weight)
    return q


def bmm_weight_quant_fp8(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same as bmm_weight_rowwise_quant_fp8 but also returns the [E, D_out] scales."""
    lib = _lib.load()
    dev = _lib.require_cuda(weight)
    if weight.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"bmm_weight_rowwise_quant_fp8: float32 or bfloat16 expected, got {weight.dtype}")
    w = weight.contiguous()
    E, K, D = w.shape
    q = torch.empty(w.shape, dtype=torch.float8_e4m3fn, device=dev)
    scale = torch.empty((E, D), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_bmm_weight_quant_fp8(w.data_ptr(), _lib.dtype_code(w.dtype), E, K, D, q.data_ptr(),
                                          scale.data_ptr(), _lib.stream_ptr(dev))
        )
    return q, scale


def quantize_weight_kmajor(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantises a logical [E, K, N] weight per (expert, output column n) over K - the
    ``pytorch_rowwise_quant_fp8(weight.permute(0, 2, 1))`` step of the reference's FP8 up
    projection (kernels/pytorch/moe_fp8.py:112) - and returns (q [E, N, K] e4m3 with K
    contiguous, scale [E, N]). Meant to run once when weights are loaded."""
    return rowwise_quant_fp8(weight.permute(0, 2, 1))


def _pad16(t: torch.Tensor) -> torch.Tensor:
    K = t.shape[-1]
    kp = (K + 15) // 16 * 16
    if kp != K:
        t = torch.nn.functional.pad(t.view(torch.uint8), (0, kp - K)).view(torch.float8_e4m3fn)
    return t


def index_select_jagged_bmm_fp8_quantized(
    offsets: torch.Tensor,
    index: torch.Tensor,
    jagged_q: torch.Tensor,
    jagged_scale: torch.Tensor,
    weight_q: torch.Tensor,
    weight_scale: torch.Tensor,
    bias: Optional[torch.Tensor],
    out_dtype: torch.dtype = torch.bfloat16,
    weight_p_q: Optional[torch.Tensor] = None,
    weight_p_scale: Optional[torch.Tensor] = None,
    bias_p: Optional[torch.Tensor] = None,
    epilogue: int = _lib.EPI_NONE,
) -> torch.Tensor:
    """FP8 up projection on operands that are already quantised: jagged_q [L, K] e4m3 with
    jagged_scale [L]; weight_q [E, N, K] e4m3 (K contiguous) with weight_scale [E, N].
    out = (q_x . q_w) / (s_x * s_w) + bias, rows gathered by index // A (``index=None``: jagged_q
    and jagged_scale already hold the expert-sorted rows). With weight_p_q the SwiGLU form of the
    same product is computed."""
    lib = _lib.load()
    dev = _lib.require_cuda(offsets, index, jagged_q, jagged_scale, weight_q, weight_scale, bias)
    assert index is None or (index.ndim == 2 and index.shape[0] == jagged_q.shape[0])
    L, K = jagged_q.shape
    E, N, Kw = weight_q.shape
    assert Kw == K
    xq = _pad16(jagged_q.contiguous())
    wq = _pad16(weight_q.contiguous())
    wpq = None if weight_p_q is None else _pad16(weight_p_q.contiguous())
    kp = xq.shape[1]
    if weight_p_q is not None:
        epilogue = _lib.EPI_SWIGLU
    rows = index.numel() if index is not None else L
    out = torch.empty((rows, N), dtype=out_dtype, device=dev)
    b = _prep_bias(bias, out_dtype)
    bp = _prep_bias(bias_p, out_dtype)
    off = _index_i64(offsets)
    idx = None if index is None else _index_i64(index)
    xs = jagged_scale.to(torch.float32).contiguous()
    ws = weight_scale.to(torch.float32).contiguous()
    wps = None if weight_p_scale is None else weight_p_scale.to(torch.float32).contiguous()
    div = index.shape[1] if index is not None else 1
    if idx is not None and _gather_first(rows, N * (2 if weight_p_q is not None else 1)):
        # rows (and their scales) gathered once by the copy kernel; the GEMM reads contiguous tiles
        xq = gather_rows(xq, idx, div)
        xs = gather_rows(xs.view(-1, 1), idx, div).view(-1)
        idx, div, L = None, 1, rows
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_index_select_jagged_bmm_fp8(
                off.data_ptr(), _lib.ptr(idx), div, rows, xq.data_ptr(), xs.data_ptr(), L, xq.stride(0),
                wq.data_ptr(), ws.data_ptr(), _lib.ptr(wpq), _lib.ptr(wps), wq.stride(0), 1, wq.stride(1), N,
                _lib.ptr(b), _lib.ptr(bp), N, E, kp, N, epilogue, out.data_ptr(), _lib.dtype_code(out_dtype),
                out.stride(0), _lib.stream_ptr(dev),
            )
        )
    return out


def index_select_jagged_bmm(
    max_seq_len: int,
    offsets: torch.Tensor,
    index: torch.Tensor,
    jagged: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    kernel: KernelType = KernelType.PYTORCH,
    fp8: bool = False,
) -> torch.Tensor:
    """The reference's FP8-capable up projection (kernels/moe_fp8.py:185-248). With ``fp8``
    the weight (per output column) and the tokens (per row) are quantised on the fly - as the
    reference does on every call - and multiplied with e4m3 tensor-core math; without it the
    bf16 / tf32 operator runs."""
    if not fp8:
        from .moe import index_select_jagged_bmm as bmm

        return bmm(max_seq_len, offsets, index, jagged, weight, bias)
    assert jagged.dtype == weight.dtype and (bias is None or jagged.dtype == bias.dtype)
    wq, ws = quantize_weight_kmajor(weight)
    xq, xs = rowwise_quant_fp8(jagged)
    return index_select_jagged_bmm_fp8_quantized(offsets, index, xq, xs, wq, ws, bias, out_dtype=jagged.dtype)


def silu_jagged_bmm_fp8(
    seq_offsets: torch.Tensor,
    max_seq_len: int,
    jagged: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    kernel: KernelType = KernelType.PYTORCH,
) -> torch.Tensor:
    """silu(jagged) @ weight[e] + bias[e] with e4m3 operands (kernels/moe_fp8.py:98-124):
    silu and rowwise quantisation of the activations in one pass, weight [E, K, D_out]
    quantised per output column, FP8 grouped GEMM with the descale in the epilogue."""
    lib = _lib.load()
    dev = _lib.require_cuda(seq_offsets, jagged, weight, bias)
    rows, K = jagged.shape
    E, Kw, N = weight.shape
    assert Kw == K
    xq, xs = rowwise_quant_fp8(jagged, apply_silu=True)
    wq, ws = quantize_weight_kmajor(weight)
    xq, wq = _pad16(xq), _pad16(wq)
    out = torch.empty((rows, N), dtype=jagged.dtype, device=dev)
    b = _prep_bias(bias, jagged.dtype)
    off = _index_i64(seq_offsets)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_silu_jagged_bmm(
                off.data_ptr(), rows, xq.data_ptr(), _lib.E4M3, xq.stride(0), xs.data_ptr(), wq.data_ptr(),
                ws.data_ptr(), wq.stride(0), 1, wq.stride(1), N, _lib.ptr(b), N, E, xq.shape[1], N, 0, None, None, None,
                out.data_ptr(), _lib.dtype_code(out.dtype), out.stride(0), _lib.stream_ptr(dev),
            )
        )
    return out


def silu_jagged_bmm_combine_fp8(
    max_seq_len: int,
    offsets: torch.Tensor,
    jagged: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    index: torch.Tensor,
    reverse_index: torch.Tensor,
    gating_scores: Optional[torch.Tensor] = None,
    gates_index: Optional[torch.Tensor] = None,
    activation_checkpointing: bool = False,
    has_silu: bool = True,
    kernel: KernelType = KernelType.PYTORCH,
) -> torch.Tensor:
    """FP8 down projection followed by the gate-weighted combine (kernels/moe_fp8.py:127-182).
    weight is logical [E, D_in, D_out] (the layout of the reference's PYTORCH branch)."""
    from .moe import mul_merge_k_add

    if has_silu:
        y = silu_jagged_bmm_fp8(offsets, max_seq_len, jagged, weight, bias)
    else:
        xq, xs = rowwise_quant_fp8(jagged)
        wq, ws = quantize_weight_kmajor(weight)
        y = fp8_jagged_bmm_quantized(offsets, xq, xs, wq, ws, bias, out_dtype=jagged.dtype)
    return mul_merge_k_add(index, reverse_index, y, weight=gating_scores, weight_index=gates_index)


def fp8_jagged_bmm_quantized(
    offsets: torch.Tensor,
    jagged_q: torch.Tensor,
    jagged_scale: torch.Tensor,
    weight_q: torch.Tensor,
    weight_scale: torch.Tensor,
    bias: Optional[torch.Tensor],
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """Down projection on pre-quantised operands: jagged_q [rows, K] e4m3 + scale [rows],
    weight_q [E, N, K] e4m3 + scale [E, N]."""
    lib = _lib.load()
    dev = _lib.require_cuda(offsets, jagged_q, jagged_scale, weight_q, weight_scale, bias)
    rows, K = jagged_q.shape
    E, N, Kw = weight_q.shape
    assert Kw == K
    xq, wq = _pad16(jagged_q.contiguous()), _pad16(weight_q.contiguous())
    out = torch.empty((rows, N), dtype=out_dtype, device=dev)
    b = _prep_bias(bias, out_dtype)
    off = _index_i64(offsets)
    xs = jagged_scale.to(torch.float32).contiguous()
    ws = weight_scale.to(torch.float32).contiguous()
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_silu_jagged_bmm(
                off.data_ptr(), rows, xq.data_ptr(), _lib.E4M3, xq.stride(0), xs.data_ptr(), wq.data_ptr(),
                ws.data_ptr(), wq.stride(0), 1, wq.stride(1), N, _lib.ptr(b), N, E, xq.shape[1], N, 0, None, None, None,
                out.data_ptr(), _lib.dtype_code(out_dtype), out.stride(0), _lib.stream_ptr(dev),
            )
        )
    return out


def fp8_jagged_bmm_combine_quantized(
    offsets: torch.Tensor,
    jagged_q: torch.Tensor,
    jagged_scale: torch.Tensor,
    weight_q: torch.Tensor,
    weight_scale: torch.Tensor,
    bias: Optional[torch.Tensor],
    gating_scores: torch.Tensor,
    gates_index: torch.Tensor,
    num_tokens: int,
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """fp8_jagged_bmm_quantized followed by the gate-weighted combine, in one kernel: the GEMM
    epilogue descales, adds the bias, rounds to ``out_dtype``, multiplies by the gate weight
    (f32 scores are rounded to ``out_dtype`` first, as a cast of the scores would) and adds into
    the token rows. [rows = num_tokens * k, K] -> [num_tokens, N]. Bit-identical to the
    two-kernel form for k <= 2."""
    lib = _lib.load()
    dev = _lib.require_cuda(offsets, jagged_q, jagged_scale, weight_q, weight_scale, bias, gating_scores, gates_index)
    rows, K = jagged_q.shape
    E, N, Kw = weight_q.shape
    assert Kw == K and rows % max(num_tokens, 1) == 0 and gating_scores.numel() == rows == gates_index.numel()
    k = rows // num_tokens if num_tokens else 1
    xq, wq = _pad16(jagged_q.contiguous()), _pad16(weight_q.contiguous())
    out = torch.empty((num_tokens, N), dtype=out_dtype, device=dev)
    b = _prep_bias(bias, out_dtype)
    off = _index_i64(offsets)
    xs = jagged_scale.to(torch.float32).contiguous()
    ws = weight_scale.to(torch.float32).contiguous()
    g = gating_scores.contiguous().view(-1)
    if g.dtype not in (torch.float32, torch.bfloat16):
        g = g.to(torch.float32)
    gidx = _index_i64(gates_index)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_silu_jagged_bmm_combine_fused(
                off.data_ptr(), rows, xq.data_ptr(), _lib.E4M3, xq.stride(0), xs.data_ptr(), wq.data_ptr(),
                ws.data_ptr(), wq.stride(0), 1, wq.stride(1), N, _lib.ptr(b), N, g.data_ptr(), _lib.dtype_code(g.dtype),
                gidx.data_ptr(), num_tokens, k, E, xq.shape[1], N, 0, None, out.data_ptr(), _lib.dtype_code(out_dtype),
                out.stride(0), _lib.COMBINE_ROUND_GATE, _lib.stream_ptr(dev),
            )
        )
    return out

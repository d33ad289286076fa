"""Operators of the MoE forward path with the reference's signatures (kernels/moe.py:39-292),
backed by libfmoe_b200 (hand-written sm_100a kernels). An operator whose inputs require a gradient
runs as the matching autograd Function of kernels/autograd.py; otherwise nothing is recorded.

``kernel=`` / ``triton_option=`` are accepted and ignored: there is one implementation here.
Tensors must live on a CUDA device; outputs are freshly allocated on the same device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _lib
from .utils import KernelType


@dataclass
class IndexSelectJaggedBmmOption:
    """Backward-pass tuning knobs of the reference (kernels/triton/triton_moe.py:36-43);
    accepted for signature compatibility, unused by the forward kernels."""

    d_weight_optimization: bool = False
    d_weight_split_k_kernel: bool = False
    d_weight_split_k_kernel_tma: bool = False
    gemm_out_bf16: bool = False


@dataclass
class SiluJaggedBmmCombineOption:
    """See kernels/triton/triton_moe.py:3562-3567; unused by the forward kernels."""

    activation_checkpointing: bool = False
    d_weight_optimization: bool = False
    d_weight_split_k_kernel: bool = False
    d_weight_split_k_kernel_tma: bool = False


def _ag():
    from . import autograd

    return autograd


def _elem_align(dt: torch.dtype) -> int:
    """Elements per 16 bytes: TMA needs 16-byte aligned bases and row strides."""
    return 16 // torch.empty((), dtype=dt).element_size()


def _check_float(t: torch.Tensor, name: str) -> None:
    if t.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"{name}: float32 or bfloat16 expected, got {t.dtype}")


def prep_activation(jagged: torch.Tensor, k_pad: int) -> torch.Tensor:
    """Returns a [rows, >=K] view/copy whose last dim is contiguous, whose row stride and base
    are 16-byte aligned, zero-padded to k_pad columns when K itself is not aligned."""
    K = jagged.shape[1]
    a = _elem_align(jagged.dtype)
    if k_pad != K:
        return torch.nn.functional.pad(jagged, (0, k_pad - K))
    if jagged.stride(1) != 1 or jagged.stride(0) % a != 0 or jagged.data_ptr() % 16 != 0:
        return jagged.contiguous()
    return jagged


# A plain [E, K, N] weight (N contiguous) is read in place as an MN-major tensor-core operand
# where the hardware path exists (bf16, N a multiple of 64); False forces the transposed copy.
MN_MAJOR_WEIGHTS = True


def prep_weight(weight: torch.Tensor, k_pad: int) -> Tuple[torch.Tensor, int, int, int]:
    """weight is logical [E, K, N]. Returns (tensor whose data pointer the kernel takes, expert
    stride, K stride, N stride) in elements. The permuted view FastMoELayer passes
    (modules/fast_moe_module.py:167,177; storage [E, N, K], K contiguous) is used in place with
    strides (se, 1, sn). A plain contiguous [E, K, N] tensor - what the reference's operators are
    documented with (kernels/moe.py:39-68) - is used in place too when it is bf16 with N a
    multiple of 64 (strides (se, sk, 1)); otherwise it is transposed once (a copy)."""
    E, K, N = weight.shape
    a = _elem_align(weight.dtype)
    wt = weight.permute(0, 2, 1)  # [E, N, K]
    ok = (
        wt.stride(2) == 1
        and wt.stride(1) % a == 0
        and wt.stride(0) % a == 0
        and wt.data_ptr() % 16 == 0
        and k_pad == K
    )
    if ok:
        return wt, wt.stride(0), 1, wt.stride(1)
    if (MN_MAJOR_WEIGHTS and weight.dtype == torch.bfloat16 and weight.stride(2) == 1 and N % 64 == 0 and k_pad == K
            and K > 1 and weight.stride(1) % a == 0 and weight.stride(0) % a == 0 and weight.data_ptr() % 16 == 0):
        return weight, weight.stride(0), weight.stride(1), 1
    wt = wt.contiguous()
    if k_pad != K:
        wt = torch.nn.functional.pad(wt, (0, k_pad - K))
    return wt, wt.stride(0), 1, wt.stride(1)


def _pad_k(K: int, dt: torch.dtype) -> int:
    a = _elem_align(dt)
    return (K + a - 1) // a * a


def _prep_bias(bias: Optional[torch.Tensor], out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    if bias is None:
        return None
    b = bias.to(out_dtype)
    return b if b.is_contiguous() else b.contiguous()


def _index_i64(t: torch.Tensor) -> torch.Tensor:
    t = t if t.dtype == torch.int64 else t.to(torch.int64)
    return t if t.is_contiguous() else t.contiguous()


# ---------------------------------------------------------------------------- fp32 operands
# None: follow torch.backends.cuda.matmul.allow_tf32 at call time, as the reference's kernels do
# (kernels/triton/triton_moe.py:592; the default is False). "tf32" / "fp32" force either.
_FP32_MATMUL: Optional[str] = None


def set_fp32_matmul(mode: Optional[str]) -> None:
    """How float32 operands are multiplied: "tf32" (tensor cores round the operands to 10 mantissa
    bits), "fp32" (operands expanded into three bf16 terms each, one bf16 GEMM over a six times
    longer reduction: fp32 accuracy at about a third of the tf32 speed), or None to follow
    ``torch.backends.cuda.matmul.allow_tf32``."""
    global _FP32_MATMUL
    if mode not in (None, "tf32", "fp32"):
        raise ValueError("mode must be None, 'tf32' or 'fp32'")
    _FP32_MATMUL = mode


def fp32_uses_tf32() -> bool:
    if _FP32_MATMUL is not None:
        return _FP32_MATMUL == "tf32"
    return bool(torch.backends.cuda.matmul.allow_tf32)


def split_f32_rows(t: torch.Tensor, pattern: int, apply_silu: bool = False) -> torch.Tensor:
    """[rows, K] float32 -> [rows, 6 * Kp] bfloat16 (Kp = K padded to 4): the three-term expansion
    laid out for the left (pattern 0) or right (pattern 1) operand of the fp32-accurate product."""
    dev = _lib.require_cuda(t)
    lib = _lib.load()
    assert t.ndim == 2 and t.dtype == torch.float32
    src = t if t.stride(1) == 1 else t.contiguous()
    rows, K = src.shape
    kp = (K + 3) // 4 * 4
    out = torch.empty((rows, 6 * kp), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_split_f32_bf16x3(src.data_ptr(), rows, K, src.stride(0) if rows else K, kp, pattern,
                                             1 if apply_silu else 0, out.data_ptr(), 6 * kp, _lib.stream_ptr(dev)))
    return out


def split_f32_weight(weight: torch.Tensor) -> torch.Tensor:
    """Logical [E, K, N] float32 weight -> logical [E, 6 * Kp, N] bfloat16 weight whose reduction
    dimension is contiguous (the right-operand expansion of every output column's K vector)."""
    E, K, N = weight.shape
    wt = weight.permute(0, 2, 1)                      # [E, N, K]
    if not wt.is_contiguous():
        wt = wt.contiguous()
    w6 = split_f32_rows(wt.view(E * N, K), 1)
    return w6.view(E, N, -1).permute(0, 2, 1)


def _wants_fp32_split(*tensors: torch.Tensor) -> bool:
    return all(t.dtype == torch.float32 for t in tensors) and not fp32_uses_tf32()


# From this many output rows and columns on (both products of a gated GEMM counted), the rows are
# gathered once by the copy kernel and the GEMM reads them as contiguous TMA tiles. The in-kernel
# gather (16-byte cp.async by four warps) re-fetches a row tile for every column block and shares
# issue slots with the MMA thread: at 4096 x top-2 tokens, d=1024, h=4096 it costs 140 us against
# 8 + 111 us for copy + contiguous GEMM; with few column blocks the single pass of the fused form wins.
PREGATHER_MIN_ROWS = 1024
PREGATHER_MIN_COLS = 1024


def _gather_first(rows: int, total_cols: int) -> bool:
    return rows >= PREGATHER_MIN_ROWS and total_cols >= PREGATHER_MIN_COLS


def index_select_jagged_bmm(
    max_seq_len: int,
    offsets: torch.Tensor,
    index: torch.Tensor,
    jagged: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    kernel: KernelType = KernelType.PYTORCH,
    triton_option: Optional[IndexSelectJaggedBmmOption] = None,
    *,
    _epilogue: int = _lib.EPI_NONE,
    _rows_checked: bool = False,
    _out_dtype: Optional[torch.dtype] = None,
    _multiplier: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """out[r] = jagged[index.view(-1)[r] // A] @ weight[e] + bias[e] for the rows r of expert e.

    Same contract as the reference operator (kernels/moe.py:39-68): offsets [E+1], index [L, A],
    jagged [L, K], weight [E, K, N] (any strides), bias [E, N] or None -> [L*A, N].
    ``max_seq_len`` is accepted and not needed: the tile list is built on the device.
    float32 operands are multiplied in fp32 accuracy unless TF32 is allowed (``set_fp32_matmul``).
    ``index=None`` (not in the reference) means ``jagged`` already holds the expert-sorted rows.
    """
    assert index is None or (index.ndim == 2 and (_rows_checked or index.shape[0] == jagged.shape[0]))
    _check_float(jagged, "jagged")
    assert weight.dtype == jagged.dtype, f"{weight.dtype=} {jagged.dtype=}"
    if (index is not None and _epilogue == _lib.EPI_NONE and _out_dtype is None and _multiplier is None
            and _ag().needs_grad(jagged, weight, bias)):
        return _ag().IndexSelectJaggedBmmFn.apply(offsets, index, jagged, weight, bias)
    if _out_dtype is None and _wants_fp32_split(jagged, weight):
        return index_select_jagged_bmm(max_seq_len, offsets, index, split_f32_rows(jagged, 0), split_f32_weight(weight),
                                       bias, _epilogue=_epilogue, _rows_checked=_rows_checked,
                                       _out_dtype=torch.float32, _multiplier=_multiplier)
    od = _out_dtype or jagged.dtype
    dev = _lib.require_cuda(offsets, index, jagged, weight, bias)
    lib = _lib.load()
    L, K = jagged.shape
    E, Kw, N = weight.shape
    assert Kw == K, f"weight {tuple(weight.shape)} does not match jagged {tuple(jagged.shape)}"
    rows = index.numel() if index is not None else L
    kp = _pad_k(K, jagged.dtype)
    a = prep_activation(jagged, kp)
    w, w_se, w_sk, w_sn = prep_weight(weight, kp)
    b = _prep_bias(bias, od)
    off = _index_i64(offsets)
    idx = None if index is None else _index_i64(index)
    div = index.shape[1] if index is not None else 1
    if idx is not None and _gather_first(rows, N):
        a, idx, div, L = gather_rows(a, idx, div), None, 1, rows
    out = torch.empty((rows, N), dtype=od, device=dev)
    dt = _lib.dtype_code(jagged.dtype)
    if _multiplier is not None:
        m = _multiplier if (_multiplier.dtype == od and _multiplier.stride(1) == 1) else _multiplier.to(od).contiguous()
        assert tuple(m.shape) == (rows, N) and _epilogue == _lib.EPI_NONE
        with torch.cuda.device(dev):
            _lib.check(
                lib.fmoe_index_select_jagged_bmm_mul(
                    off.data_ptr(), _lib.ptr(idx), div, rows, a.data_ptr(), dt, L, a.stride(0),
                    w.data_ptr(), w_se, w_sk, w_sn, _lib.ptr(b), N, E, kp, N, m.data_ptr(), m.stride(0), out.data_ptr(),
                    _lib.dtype_code(od), out.stride(0), _lib.stream_ptr(dev),
                )
            )
        return out
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_index_select_jagged_bmm(
                off.data_ptr(), _lib.ptr(idx), div, rows, a.data_ptr(), dt, L, a.stride(0),
                w.data_ptr(), w_se, w_sk, w_sn, _lib.ptr(b), N, E, kp, N, _epilogue, out.data_ptr(), _lib.dtype_code(od),
                out.stride(0), _lib.stream_ptr(dev),
            )
        )
    return out


def index_select_jagged_bmm_3D(
    max_seq_len: int,
    offsets: torch.Tensor,
    index: torch.Tensor,
    jagged: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    kernel: KernelType = KernelType.PYTORCH,
) -> torch.Tensor:
    """index_select_jagged_bmm on a [L, E, K] input: the rows of expert e read slice e of their
    token (kernels/moe.py:118-153 -> kernels/pytorch/moe.py:224-252). Runs as the 2-D operator on
    the [L*E, K] view with the row index token * E + e; the expert of every sorted row comes
    from ``offsets`` on the device (no host synchronisation)."""
    assert index.ndim == 2 and index.shape[0] == jagged.shape[0] and jagged.ndim == 3
    _lib.require_cuda(offsets, index, jagged, weight, bias)
    L, E, K = jagged.shape
    assert weight.shape[0] == E and weight.shape[1] == K
    rows = index.numel()
    off = _index_i64(offsets)
    idx = _index_i64(index)
    flat_index = torch.empty((rows, 1), dtype=torch.int64, device=idx.device)
    lib = _lib.load()
    with torch.cuda.device(idx.device):
        _lib.check(lib.fmoe_expand_3d_index(off.data_ptr(), idx.data_ptr(), index.shape[1], E, rows, flat_index.data_ptr(),
                                            _lib.stream_ptr(idx.device)))
    x2d = jagged.reshape(L * E, K)
    return index_select_jagged_bmm(max_seq_len, off, flat_index, x2d, weight, bias, _rows_checked=True)


def index_select_jagged_bmm_swiglu(
    max_seq_len: int,
    offsets: torch.Tensor,
    index: torch.Tensor,
    jagged: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    weight_p: torch.Tensor,
    bias_p: Optional[torch.Tensor],
    kernel: KernelType = KernelType.PYTORCH,
    *,
    _out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """silu(x @ weight[e] + bias[e]) * (x @ weight_p[e] + bias_p[e]) on the gathered rows, one
    kernel, the activation row tile shared by both products (kernels/moe.py:156-189).
    ``index=None`` (not in the reference) means ``jagged`` already holds the expert-sorted rows."""
    assert index is None or (index.ndim == 2 and index.shape[0] == jagged.shape[0])
    _check_float(jagged, "jagged")
    assert weight.dtype == jagged.dtype and weight_p.dtype == jagged.dtype
    assert weight.shape == weight_p.shape
    if index is not None and _out_dtype is None and _ag().needs_grad(jagged, weight, bias, weight_p, bias_p):
        return _ag().IndexSelectJaggedBmmSwigluFn.apply(offsets, index, jagged, weight, bias, weight_p, bias_p)
    if _out_dtype is None and _wants_fp32_split(jagged, weight, weight_p):
        return index_select_jagged_bmm_swiglu(max_seq_len, offsets, index, split_f32_rows(jagged, 0),
                                              split_f32_weight(weight), bias, split_f32_weight(weight_p), bias_p,
                                              _out_dtype=torch.float32)
    od = _out_dtype or jagged.dtype
    dev = _lib.require_cuda(offsets, index, jagged, weight, weight_p, bias, bias_p)
    lib = _lib.load()
    L, K = jagged.shape
    E, Kw, N = weight.shape
    assert Kw == K
    rows = index.numel() if index is not None else L
    kp = _pad_k(K, jagged.dtype)
    a = prep_activation(jagged, kp)
    w, w_se, w_sk, w_sn = prep_weight(weight, kp)
    wp, wp_se, wp_sk, wp_sn = prep_weight(weight_p, kp)
    if (wp_se, wp_sk, wp_sn) != (w_se, w_sk, w_sn):
        # the kernel walks both weights with one set of strides: both as [E, N, K] copies
        w = weight.permute(0, 2, 1).contiguous()
        wp = weight_p.permute(0, 2, 1).contiguous()
        if kp != K:
            w = torch.nn.functional.pad(w, (0, kp - K))
            wp = torch.nn.functional.pad(wp, (0, kp - K))
        w_se, w_sk, w_sn = w.stride(0), 1, w.stride(1)
    b = _prep_bias(bias, od)
    bp = _prep_bias(bias_p, od)
    off = _index_i64(offsets)
    idx = None if index is None else _index_i64(index)
    div = index.shape[1] if index is not None else 1
    if idx is not None and _gather_first(rows, 2 * N):
        a, idx, div, L = gather_rows(a, idx, div), None, 1, rows
    out = torch.empty((rows, N), dtype=od, device=dev)
    dt = _lib.dtype_code(jagged.dtype)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_index_select_jagged_bmm_swiglu(
                off.data_ptr(), _lib.ptr(idx), div, rows, a.data_ptr(), dt, L, a.stride(0),
                w.data_ptr(), wp.data_ptr(), w_se, w_sk, w_sn, _lib.ptr(b), _lib.ptr(bp), N, E, kp, N,
                out.data_ptr(), _lib.dtype_code(od), out.stride(0), _lib.stream_ptr(dev),
            )
        )
    return out


def index_select_jagged_gating_bmm(
    max_seq_len: int,
    offsets: torch.Tensor,
    index: torch.Tensor,
    jagged_a: torch.Tensor,
    jagged_b: torch.Tensor,
    weight_a: torch.Tensor,
    bias_a: Optional[torch.Tensor],
    weight_b: torch.Tensor,
    bias_b: Optional[torch.Tensor],
    kernel: KernelType = KernelType.PYTORCH,
) -> torch.Tensor:
    """silu(A_g @ Wa + ba) * (B_g @ Wb + bb) (kernels/moe.py:192-233). With ``jagged_a is
    jagged_b`` this is the SwiGLU operator and runs as one kernel; two distinct inputs run as two
    grouped GEMMs: the first with the SiLU epilogue, the second multiplying its result by the
    first's in its epilogue."""
    assert (
        index.ndim == 2
        and index.shape[0] == jagged_a.shape[0] == jagged_b.shape[0]
        and jagged_a.shape == jagged_b.shape
        and weight_a.shape == weight_b.shape
    )
    if jagged_a is jagged_b:
        return index_select_jagged_bmm_swiglu(max_seq_len, offsets, index, jagged_a, weight_a, bias_a, weight_b, bias_b)
    if _ag().needs_grad(jagged_a, jagged_b, weight_a, weight_b, bias_a, bias_b):
        # with gradients: two differentiable products and the elementwise SwiGLU on top of them
        alpha = index_select_jagged_bmm(max_seq_len, offsets, index, jagged_a, weight_a, bias_a)
        beta = index_select_jagged_bmm(max_seq_len, offsets, index, jagged_b, weight_b, bias_b)
        return torch.nn.functional.silu(alpha) * beta
    alpha_silu = index_select_jagged_bmm(max_seq_len, offsets, index, jagged_a, weight_a, bias_a, _epilogue=_lib.EPI_SILU)
    # the second product multiplies its result by silu(first product) in its epilogue
    return index_select_jagged_bmm(max_seq_len, offsets, index, jagged_b, weight_b, bias_b, _multiplier=alpha_silu)


def mul_merge_k_add(
    index: torch.Tensor,
    reverse_index: torch.Tensor,
    value: torch.Tensor,
    stable_sorting: bool = False,
    weight: Optional[torch.Tensor] = None,
    weight_index: Optional[torch.Tensor] = None,
    kernel: KernelType = KernelType.PYTORCH,
    triton_cc_version: str = "",
) -> torch.Tensor:
    """out[t] = sum over the k rows p of token t of value[p] * weight.view(-1)[weight_index[p]]
    (kernels/moe.py:71-115). Uses the gather form (``reverse_index``), fp32 accumulation in
    ascending row order; ``index`` only takes part in the shape checks."""
    N = index.shape[0]
    L, K = reverse_index.shape
    _, D = value.shape
    assert index.ndim == 1 and reverse_index.ndim == 2
    assert N == L * K and N == value.shape[0]
    _check_float(value, "value")
    if _ag().needs_grad(value, weight):
        return _ag().MulMergeKAddFn.apply(index, reverse_index, value, weight, weight_index)
    dev = _lib.require_cuda(reverse_index, value, weight, weight_index)
    lib = _lib.load()
    w = None
    widx = None
    out_dtype = value.dtype
    if weight is not None:
        assert weight_index is not None
        assert weight.numel() == weight_index.numel() == value.shape[0], (
            f"{weight.shape=}, {weight_index.shape=}, {value.shape=}"
        )
        _check_float(weight, "weight")
        w = weight.contiguous().view(-1)
        widx = _index_i64(weight_index)
        out_dtype = torch.promote_types(value.dtype, weight.dtype)
    v = value if value.stride(1) == 1 else value.contiguous()
    rev = _index_i64(reverse_index)
    out = torch.empty((L, D), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_mul_merge_k_add(
                rev.data_ptr(), v.data_ptr(), _lib.dtype_code(v.dtype), v.stride(0), _lib.ptr(w),
                _lib.dtype_code(w.dtype) if w is not None else 0, _lib.ptr(widx), L, K, D, out.data_ptr(),
                _lib.dtype_code(out_dtype), out.stride(0), _lib.stream_ptr(dev),
            )
        )
    return out


def gather_rows(src: torch.Tensor, index: torch.Tensor, index_div: int = 1) -> torch.Tensor:
    """dst[r] = src[index[r] // index_div]: the index_select step of the up projection
    (kernels/pytorch/moe.py:69-73) as a kernel of its own. The expert-parallel layer uses it to
    pack the rows it sends in expert-sorted order."""
    dev = _lib.require_cuda(src, index)
    lib = _lib.load()
    s = src if src.stride(-1) == 1 else src.contiguous()
    idx = _index_i64(index.reshape(-1))
    rows, cols = idx.numel(), s.shape[1]
    out = torch.empty((rows, cols), dtype=s.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_gather_rows(s.data_ptr(), _lib.dtype_code(s.dtype), s.shape[0], s.stride(0), idx.data_ptr(),
                                 index_div, rows, cols, out.data_ptr(), out.stride(0), _lib.stream_ptr(dev))
        )
    return out


def silu_jagged_bmm(
    offsets: torch.Tensor,
    jagged: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    has_silu: bool = True,
    out_row_index: Optional[torch.Tensor] = None,
    *,
    _out_dtype: Optional[torch.dtype] = None,
    _act_scratch: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """[silu](jagged) @ weight[e] + bias[e] per expert segment; weight is logical [E, K, N]
    (the GEMM half of silu_jagged_bmm_combine, kernels/pytorch/moe.py:255-275).
    ``out_row_index`` (a permutation of the rows, not part of the reference operator) makes row r
    of the result land at out[out_row_index[r]]."""
    _check_float(jagged, "jagged")
    assert weight.dtype == jagged.dtype
    if _out_dtype is None and _act_scratch is None and _wants_fp32_split(jagged, weight):
        # SiLU is applied while the activations are expanded
        return silu_jagged_bmm(offsets, split_f32_rows(jagged, 0, apply_silu=has_silu), split_f32_weight(weight), bias,
                               has_silu=False, out_row_index=out_row_index, _out_dtype=torch.float32)
    od = _out_dtype or jagged.dtype
    dev = _lib.require_cuda(offsets, jagged, weight, bias)
    lib = _lib.load()
    rows, K = jagged.shape
    E, Kw, N = weight.shape
    assert Kw == K
    kp = _pad_k(K, jagged.dtype)
    a = prep_activation(jagged, kp)
    w, w_se, w_sk, w_sn = prep_weight(weight, kp)
    b = _prep_bias(bias, od)
    off = _index_i64(offsets)
    out = torch.empty((rows, N), dtype=od, device=dev)
    scratch = None
    if has_silu:
        # receives silu(jagged); a caller that wants to keep it (the backward pass) passes the buffer
        ok = _act_scratch is not None and kp == K and tuple(_act_scratch.shape) == (rows, K) and _act_scratch.is_contiguous()
        scratch = _act_scratch if ok else torch.empty((rows, kp), dtype=jagged.dtype, device=dev)
    oidx = None if out_row_index is None else _index_i64(out_row_index.reshape(-1))
    assert oidx is None or oidx.numel() == rows
    dt = _lib.dtype_code(jagged.dtype)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_silu_jagged_bmm(
                off.data_ptr(), rows, a.data_ptr(), dt, a.stride(0), None, w.data_ptr(), None, w_se, w_sk, w_sn, 0,
                _lib.ptr(b), N, E, kp, N, 1 if has_silu else 0, _lib.ptr(scratch), None, _lib.ptr(oidx), out.data_ptr(),
                _lib.dtype_code(od), out.stride(0),
                _lib.stream_ptr(dev),
            )
        )
    return out


def jagged_bmm_two_weights(offsets: torch.Tensor, jagged: torch.Tensor, weight0: torch.Tensor, weight1: torch.Tensor
                           ) -> Optional[torch.Tensor]:
    """rows[:, :K0] @ weight0[e] + rows[:, K0:] @ weight1[e] as one grouped product whose reduction
    walks the two weights (logical [E, K0, N] and [E, K1, N]). Returns None when the two weights
    cannot be read in place with one set of strides (the caller then concatenates)."""
    dev = _lib.require_cuda(offsets, jagged, weight0, weight1)
    lib = _lib.load()
    rows, K = jagged.shape
    E, K0, N = weight0.shape
    K1 = weight1.shape[1]
    if K0 + K1 != K or weight1.shape[0] != E or weight1.shape[2] != N or weight0.dtype != jagged.dtype:
        return None
    unit = 128 // jagged.element_size()
    if K0 % unit or _pad_k(K, jagged.dtype) != K or jagged.stride(1) != 1:
        return None
    w0, se0, sk0, sn0 = prep_weight(weight0, K0)
    w1, se1, sk1, sn1 = prep_weight(weight1, K1)
    if (se0, sk0, sn0) != (se1, sk1, sn1) or w0.data_ptr() != weight0.data_ptr() or w1.data_ptr() != weight1.data_ptr():
        return None
    a = prep_activation(jagged, K)
    out = torch.empty((rows, N), dtype=jagged.dtype, device=dev)
    off = _index_i64(offsets)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_jagged_bmm_two_weights(off.data_ptr(), rows, a.data_ptr(), _lib.dtype_code(jagged.dtype), a.stride(0),
                                                   w0.data_ptr(), w1.data_ptr(), K0, se0, sk0, sn0, E, K, N, out.data_ptr(),
                                                   _lib.dtype_code(out.dtype), out.stride(0), _lib.stream_ptr(dev)))
    return out


def silu_jagged_bmm_raw(offsets: torch.Tensor, jagged: torch.Tensor, weight: torch.Tensor,
                        out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Plain grouped product rows @ weight[e] with a chosen output type (bf16 operands may write
    f32): the building block the router uses for its logits. weight is logical [E, K, N]."""
    dev = _lib.require_cuda(offsets, jagged, weight)
    lib = _lib.load()
    rows, K = jagged.shape
    E, Kw, N = weight.shape
    assert Kw == K and weight.dtype == jagged.dtype
    kp = _pad_k(K, jagged.dtype)
    a = prep_activation(jagged, kp)
    w, w_se, w_sk, w_sn = prep_weight(weight, kp)
    od = out_dtype or jagged.dtype
    out = torch.empty((rows, N), dtype=od, device=dev)
    off = _index_i64(offsets)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_silu_jagged_bmm(
                off.data_ptr(), rows, a.data_ptr(), _lib.dtype_code(jagged.dtype), a.stride(0), None, w.data_ptr(),
                None, w_se, w_sk, w_sn, 0, None, 0, E, kp, N, 0, None, None, None, out.data_ptr(), _lib.dtype_code(od),
                out.stride(0), _lib.stream_ptr(dev),
            )
        )
    return out


def silu_jagged_bmm_combine(
    max_seq_len: int,
    offsets: torch.Tensor,
    jagged: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    index: torch.Tensor,
    reverse_index: torch.Tensor,
    gating_scores: Optional[torch.Tensor] = None,
    gates_index: Optional[torch.Tensor] = None,
    has_silu: bool = True,
    kernel: KernelType = KernelType.PYTORCH,
    triton_option: Optional[SiluJaggedBmmCombineOption] = None,
    *,
    fused: bool = False,
    out: Optional[torch.Tensor] = None,
    round_scores: bool = False,
) -> torch.Tensor:
    """Down projection of every expert segment followed by the gate-weighted merge of each
    token's k rows (kernels/moe.py:236-292): [L*k, D_in] -> [L, D_out].

    Default: GEMM into a [L*k, D_out] scratch, then the deterministic gather-reduce. With
    ``fused=True`` (needs gating_scores) the GEMM's epilogue multiplies by the gate weight and
    adds straight into the token rows: one kernel and no intermediate; bit-identical for k <= 2,
    last-bit order dependence for k > 2.

    ``round_scores=True`` treats gating_scores as if they had been cast to the activation type
    first, without a cast kernel. The reference has no such cast: its gate is an nn.Linear that
    runs in the dtype of x (modules/fast_moe_module.py:21-27), so with bf16 tokens the scores it
    hands to this operator are already bf16 and ``value * weight`` rounds to bf16
    (kernels/pytorch/moe.py:27). The layers here compute the router in fp32 (a deliberate
    deviation: exact top-k needs it) and use this flag to land on the same operand types.
    ``out`` (fused form only): an [L, D_out] tensor of the activation type that the rows are ADDED
    to - zeros prepared ahead of time, or a residual; it is returned."""
    N = index.shape[0]
    L, K = reverse_index.shape
    _, D_in = jagged.shape
    E, _, D_out = weight.shape
    assert index.ndim == 1 and reverse_index.ndim == 2
    assert N == L * K and N == jagged.shape[0], f"{N=}, {L=}, {K=}, {jagged.shape=}"
    if kernel == KernelType.TRITON_CC:
        raise NotImplementedError("TRITON_CC is not supported for silu_jagged_bmm_combine")
    _check_float(jagged, "jagged")
    assert weight.dtype == jagged.dtype
    if out is None and _ag().needs_grad(jagged, weight, bias, gating_scores):
        g_in = gating_scores
        if g_in is not None and round_scores:
            g_in = g_in.to(jagged.dtype)
        return _ag().SiluJaggedBmmCombineFn.apply(offsets, jagged, weight, bias, index, reverse_index, g_in, gates_index,
                                                  has_silu)
    if _wants_fp32_split(jagged, weight) and out is None:
        # fp32 accuracy: the GEMM on the expanded operands (f32 result rows), then the
        # deterministic fp32 merge; the operand types of the merge are those of the reference
        rows_f32 = silu_jagged_bmm(offsets, jagged, weight, bias, has_silu=has_silu)
        g32 = gating_scores
        if g32 is not None and round_scores:
            g32 = g32.to(jagged.dtype)
        return mul_merge_k_add(index, reverse_index, rows_f32, weight=g32, weight_index=gates_index)
    dev = _lib.require_cuda(offsets, jagged, weight, bias, reverse_index, gating_scores, gates_index)
    lib = _lib.load()
    kp = _pad_k(D_in, jagged.dtype)
    a = prep_activation(jagged, kp)
    w, w_se, w_sk, w_sn = prep_weight(weight, kp)
    b = _prep_bias(bias, jagged.dtype)
    off = _index_i64(offsets)
    rev = _index_i64(reverse_index)
    g = None
    gidx = None
    out_dtype = jagged.dtype
    if gating_scores is not None:
        assert gates_index is not None
        assert gating_scores.numel() == gates_index.numel() == N
        _check_float(gating_scores, "gating_scores")
        g = gating_scores.contiguous().view(-1)
        gidx = _index_i64(gates_index)
        if round_scores and not (fused and g.dtype == torch.float32):
            g = g.to(jagged.dtype)          # the two-kernel form takes the cast scores
        out_dtype = jagged.dtype if round_scores else torch.promote_types(jagged.dtype, g.dtype)
    act_scratch = torch.empty((N, kp), dtype=jagged.dtype, device=dev) if has_silu else None
    dt = _lib.dtype_code(jagged.dtype)
    use_fused = fused and g is not None and out_dtype == jagged.dtype
    accumulate = out is not None
    if out is not None:
        if not use_fused:
            raise ValueError("out= is only available with fused=True and gating scores of the activation type")
        _lib.require_cuda(out)
        if tuple(out.shape) != (L, D_out) or out.dtype != out_dtype or out.stride(1) != 1:
            raise ValueError(f"out must be [{L}, {D_out}] {out_dtype} with contiguous rows")
    else:
        out = torch.empty((L, D_out), dtype=out_dtype, device=dev)
    if use_fused:
        flags = (_lib.COMBINE_ACCUMULATE if accumulate else 0) | (_lib.COMBINE_ROUND_GATE if round_scores else 0)
        with torch.cuda.device(dev):
            _lib.check(
                lib.fmoe_silu_jagged_bmm_combine_fused(
                    off.data_ptr(), N, a.data_ptr(), dt, a.stride(0), None, w.data_ptr(), None, w_se, w_sk, w_sn, 0,
                    _lib.ptr(b), D_out, g.data_ptr(), _lib.dtype_code(g.dtype), gidx.data_ptr(), L, K, E, kp, D_out,
                    1 if has_silu else 0, _lib.ptr(act_scratch), out.data_ptr(), _lib.dtype_code(out_dtype),
                    out.stride(0), flags, _lib.stream_ptr(dev),
                )
            )
        return out
    bmm_scratch = torch.empty((N, D_out), dtype=jagged.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(
            lib.fmoe_silu_jagged_bmm_combine(
                off.data_ptr(), N, a.data_ptr(), dt, a.stride(0), w.data_ptr(), w_se, w_sk, w_sn, _lib.ptr(b), D_out,
                rev.data_ptr(), _lib.ptr(g), _lib.dtype_code(g.dtype) if g is not None else 0, _lib.ptr(gidx), L, K,
                E, kp, D_out, 1 if has_silu else 0, _lib.ptr(act_scratch), bmm_scratch.data_ptr(), out.data_ptr(),
                _lib.dtype_code(out_dtype), out.stride(0), _lib.stream_ptr(dev),
            )
        )
    return out

"""Backward pass of the MoE operators (forward + backward as torch.autograd.Functions).

The reference ships every operator as an autograd.Function whose backward is a set of Triton
kernels (kernels/triton/triton_moe.py:606-804 up projection, :1039-1100 combine, :2378-2511
SwiGLU, :3790-4027 down projection + combine). Here each matrix product of the backward pass is
the forward's grouped GEMM on differently laid out operands:

  d_x of a projection   rows of d_out times W[e]^T: the grouped GEMM on the transposed weight, then
                        the k rows of a token are summed by the combine kernel;
  d_W of a projection   dW[e] = X_e^T dOut_e, whose reduction runs over the rows of an expert: both
                        operands are transposed into [features, padded rows] and the grouped GEMM
                        runs in its reduction-over-rows mode;
  d_bias                column sums per expert;
  combine               d_rows[p] = d_out[token(p)] * gate[p], d_gate[p] = <d_out[token(p)], rows[p]>;
  SwiGLU                the two pre-activations are recomputed in the backward (two GEMMs) instead
                        of being stored by the forward, whose fused epilogue stays as it is.

The public operators in kernels/moe.py route here whenever an input requires a gradient. float32
operands use tf32 tensor-core math in the backward products.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib


def _ops():
    from . import moe

    return moe


# ------------------------------------------------------------------------------------ layouts
def transposed_weight(weight: torch.Tensor) -> torch.Tensor:
    """weight logical [E, K, N] -> logical [E, N, K] whose reduction dimension (N) is contiguous:
    the operand of d_x = d_out @ W[e]^T. A plain contiguous [E, K, N] weight already is that
    (a view); a weight stored [E, N, K] (the layers' layout) is transposed once."""
    E, K, N = weight.shape
    a = 16 // weight.element_size()
    if weight.stride(2) == 1 and weight.stride(1) % a == 0:
        return weight.permute(0, 2, 1)
    ops = _ops()
    if (ops.MN_MAJOR_WEIGHTS and weight.dtype == torch.bfloat16 and weight.stride(1) == 1 and K % 64 == 0 and N > 1
            and weight.stride(2) % a == 0 and weight.stride(0) % a == 0 and weight.data_ptr() % 16 == 0):
        # stored [E, N, K] (the layers' layout): as the operand of d_out @ W^T its output dimension K
        # is the contiguous one, which the grouped GEMM reads in place (MN-major operand)
        return weight.permute(0, 2, 1)
    lib = _lib.load()
    dev = weight.device
    wt = weight.permute(0, 2, 1)                      # [E, N, K]
    if wt.stride(2) != 1:
        wt = wt.contiguous()
    out = torch.empty((E, K, N), dtype=weight.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_batched_transpose(wt.data_ptr(), _lib.dtype_code(wt.dtype), E, wt.stride(0), wt.stride(1), N, K,
                                              out.data_ptr(), K * N, N, _lib.stream_ptr(dev)))
    return out.permute(0, 2, 1)


def transposed_weights_side_by_side(weight: torch.Tensor, weight_p: torch.Tensor) -> torch.Tensor:
    """The operand of d_x = [d_alpha | d_beta] @ [W ; Wp]^T as one product over 2N: logical
    [E, 2N, K] with storage [E, K, 2N] (2N contiguous). Each weight is transposed straight into its
    half of that storage; a weight that already has N contiguous is copied."""
    E, K, N = weight.shape
    dev = weight.device
    store = torch.empty((E, K, 2 * N), dtype=weight.dtype, device=dev)
    lib = _lib.load()
    for col0, w in ((0, weight), (N, weight_p)):
        half = store[:, :, col0:col0 + N]
        wt = w.permute(0, 2, 1)                       # [E, N, K]
        if w.stride(2) == 1 or wt.stride(2) != 1:
            half.copy_(w)                             # N already contiguous, or an arbitrary layout: plain copy
            continue
        with torch.cuda.device(dev):
            _lib.check(lib.fmoe_batched_transpose(wt.data_ptr(), _lib.dtype_code(wt.dtype), E, wt.stride(0), wt.stride(1), N, K,
                                                  half.data_ptr(), K * 2 * N, 2 * N, _lib.stream_ptr(dev)))
    return store.permute(0, 2, 1)


def _padded_reduction(offsets: torch.Tensor, E: int, dtype: torch.dtype, rows: int) -> Tuple[torch.Tensor, int]:
    lib = _lib.load()
    dev = offsets.device
    unit = 128 // torch.empty((), dtype=dtype).element_size()
    kseg = torch.empty(E + 1, dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_jagged_pad_offsets(offsets.data_ptr(), E, _lib.dtype_code(dtype), kseg.data_ptr(),
                                               _lib.stream_ptr(dev)))
    padded = (rows + E * unit + unit - 1) // unit * unit
    return kseg, padded


def _transpose_pad(src: torch.Tensor, offsets: torch.Tensor, kseg: torch.Tensor, padded: int, E: int, rows: int,
                   index: Optional[torch.Tensor] = None, index_div: int = 1) -> torch.Tensor:
    lib = _lib.load()
    dev = src.device
    s = src if src.stride(1) == 1 else src.contiguous()
    cols = s.shape[1]
    out = torch.empty((cols, padded), dtype=s.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_jagged_transpose_pad(s.data_ptr(), _lib.dtype_code(s.dtype), s.shape[0], s.stride(0),
                                                 _lib.ptr(index), index_div, offsets.data_ptr(), kseg.data_ptr(), E, rows, cols,
                                                 out.data_ptr(), padded, _lib.stream_ptr(dev)))
    return out


def grad_weight(offsets: torch.Tensor, d_out: torch.Tensor, x: torch.Tensor, E: int, out_dtype: torch.dtype,
                index: Optional[torch.Tensor] = None, index_div: int = 1, shared: Optional[dict] = None) -> torch.Tensor:
    """dW logical [E, K, N] with dW[e] = X_e^T dOut_e: d_out [rows, N] and x (rows named by
    ``index // index_div`` when given, else row r itself) [*, K], expert-sorted by ``offsets``.
    Computed in the storage layout [E, N, K] and returned as its permuted view. ``shared``: a dict
    two calls with the same offsets / x / index pass to transpose x once."""
    lib = _lib.load()
    dev = d_out.device
    rows, N = d_out.shape
    K = x.shape[1]
    dt = d_out.dtype
    assert x.dtype == dt
    if rows == 0:
        return torch.zeros((E, N, K), dtype=out_dtype, device=dev).permute(0, 2, 1)
    if shared is not None and "b_t" in shared:
        kseg, padded, b_t = shared["kseg"], shared["padded"], shared["b_t"]
    else:
        kseg, padded = _padded_reduction(offsets, E, dt, rows)
        b_t = _transpose_pad(x, offsets, kseg, padded, E, rows, index, index_div)
        if shared is not None:
            shared.update(kseg=kseg, padded=padded, b_t=b_t)
    a_t = _transpose_pad(d_out, offsets, kseg, padded, E, rows)
    group_off = torch.arange(E + 1, dtype=torch.int64, device=dev) * N
    out = torch.empty((E * N, K), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_jagged_jagged_bmm(group_off.data_ptr(), kseg.data_ptr(), padded, a_t.data_ptr(), padded,
                                              b_t.data_ptr(), padded, _lib.dtype_code(dt), E, N, K, out.data_ptr(),
                                              _lib.dtype_code(out_dtype), K, _lib.stream_ptr(dev)))
    return out.view(E, N, K).permute(0, 2, 1)


def grad_bias(offsets: torch.Tensor, d_out: torch.Tensor, E: int, out_dtype: torch.dtype) -> torch.Tensor:
    lib = _lib.load()
    dev = d_out.device
    d = d_out if d_out.stride(1) == 1 else d_out.contiguous()
    out = torch.empty((E, d.shape[1]), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_jagged_colsum(d.data_ptr(), _lib.dtype_code(d.dtype), d.stride(0) if d.shape[0] else d.shape[1],
                                          offsets.data_ptr(), E, d.shape[1], out.data_ptr(), _lib.dtype_code(out_dtype),
                                          _lib.stream_ptr(dev)))
    return out


def gather_scale_rows(src: torch.Tensor, index: torch.Tensor, index_div: int, weight: Optional[torch.Tensor],
                      weight_index: Optional[torch.Tensor]) -> torch.Tensor:
    """out[p] = src[index[p] // index_div] * weight.view(-1)[weight_index[p]]."""
    lib = _lib.load()
    dev = src.device
    s = src if src.stride(1) == 1 else src.contiguous()
    idx = index.reshape(-1).contiguous()
    rows, cols = idx.numel(), s.shape[1]
    w = None if weight is None else weight.contiguous().view(-1)
    widx = None if weight_index is None else weight_index.reshape(-1).contiguous()
    out = torch.empty((rows, cols), dtype=s.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_gather_scale_rows(s.data_ptr(), _lib.dtype_code(s.dtype), s.shape[0], s.stride(0), idx.data_ptr(),
                                              index_div, _lib.ptr(w), _lib.dtype_code(w.dtype) if w is not None else 0,
                                              _lib.ptr(widx), w.numel() if w is not None else 0, rows, cols, out.data_ptr(),
                                              cols, _lib.stream_ptr(dev)))
    return out


def row_dot(a: torch.Tensor, b: torch.Tensor, index: Optional[torch.Tensor], index_div: int = 1) -> torch.Tensor:
    """out[p] = <a[p], b[index[p] // index_div]> (fp32)."""
    lib = _lib.load()
    dev = a.device
    aa = a if a.stride(1) == 1 else a.contiguous()
    bb = b if b.stride(1) == 1 else b.contiguous()
    assert aa.dtype == bb.dtype and aa.shape[1] == bb.shape[1]
    idx = None if index is None else index.reshape(-1).contiguous()
    rows = aa.shape[0]
    out = torch.empty(rows, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_row_dot(aa.data_ptr(), aa.stride(0) if rows else aa.shape[1], bb.data_ptr(), bb.shape[0],
                                    bb.stride(0) if bb.shape[0] else bb.shape[1], _lib.dtype_code(aa.dtype), _lib.ptr(idx),
                                    index_div, rows, aa.shape[1], out.data_ptr(), _lib.stream_ptr(dev)))
    return out


def activation_backward(mode: int, d_out: torch.Tensor, alpha: torch.Tensor, beta: Optional[torch.Tensor],
                        d_alpha: torch.Tensor, d_beta: Optional[torch.Tensor]) -> None:
    lib = _lib.load()
    dev = d_out.device
    rows, cols = alpha.shape
    for t in (d_out, alpha, beta, d_alpha, d_beta):
        assert t is None or t.stride(1) == 1
    ld = lambda t: 0 if t is None else (t.stride(0) if rows else cols)
    with torch.cuda.device(dev):
        _lib.check(lib.fmoe_activation_backward(mode, d_out.data_ptr(), ld(d_out), alpha.data_ptr(), ld(alpha), _lib.ptr(beta),
                                                ld(beta), _lib.dtype_code(alpha.dtype), rows, cols, d_alpha.data_ptr(),
                                                ld(d_alpha), _lib.ptr(d_beta), ld(d_beta), _lib.stream_ptr(dev)))


def _inverse_rows(index: torch.Tensor) -> torch.Tensor:
    """index [L, A] holds, at every expert-sorted position p, the value token * A + slot. Returns
    [L, A]: for every token the sorted positions of its A rows (integer bookkeeping only)."""
    flat = index.reshape(-1)
    inv = torch.empty_like(flat)
    inv[flat] = torch.arange(flat.numel(), device=flat.device, dtype=flat.dtype)
    return inv.view(index.shape)


def _contig_rows(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


# ------------------------------------------------------------------------------------ functions
class IndexSelectJaggedBmmFn(torch.autograd.Function):
    """index_select_jagged_bmm (kernels/moe.py:39-68) with its backward
    (IndexSelectJaggedBmm.backward, kernels/triton/triton_moe.py:606-804)."""

    @staticmethod
    def forward(ctx, offsets, index, jagged, weight, bias):
        with torch.no_grad():
            out = _ops().index_select_jagged_bmm(0, offsets, index, jagged, weight, bias)
        ctx.save_for_backward(offsets, index, jagged, weight)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = None if bias is None else bias.dtype
        return out

    @staticmethod
    def backward(ctx, d_out):
        offsets, index, jagged, weight = ctx.saved_tensors
        ops = _ops()
        E = weight.shape[0]
        A = index.shape[1]
        d_out = _contig_rows(d_out)
        d_jagged = d_weight = d_bias = None
        with torch.no_grad():
            if ctx.needs_input_grad[2]:
                d_rows = ops.silu_jagged_bmm(offsets, d_out, transposed_weight(weight), None, has_silu=False)
                tok = index.reshape(-1) // A
                d_jagged = ops.mul_merge_k_add(tok, _inverse_rows(index), d_rows)
            if ctx.needs_input_grad[3]:
                d_weight = grad_weight(offsets, d_out, jagged, E, weight.dtype, index=index.reshape(-1).contiguous(), index_div=A)
            if ctx.has_bias and ctx.needs_input_grad[4]:
                d_bias = grad_bias(offsets, d_out, E, ctx.bias_dtype)
        return None, None, d_jagged, d_weight, d_bias


class IndexSelectJaggedBmmSwigluFn(torch.autograd.Function):
    """index_select_jagged_bmm_swiglu (kernels/moe.py:156-189) with its backward
    (kernels/triton/triton_moe.py:2378-2511, SwiGLU derivative :62-106). The forward is the fused
    kernel; the backward recomputes the two pre-activations."""

    @staticmethod
    def forward(ctx, offsets, index, jagged, weight, bias, weight_p, bias_p):
        with torch.no_grad():
            out = _ops().index_select_jagged_bmm_swiglu(0, offsets, index, jagged, weight, bias, weight_p, bias_p)
        ctx.save_for_backward(offsets, index, jagged, weight, weight_p, bias, bias_p)
        return out

    @staticmethod
    def backward(ctx, d_out):
        offsets, index, jagged, weight, weight_p, bias, bias_p = ctx.saved_tensors
        ops = _ops()
        E, K, N = weight.shape
        A = index.shape[1]
        d_out = _contig_rows(d_out)
        rows = d_out.shape[0]
        with torch.no_grad():
            alpha = ops.index_select_jagged_bmm(0, offsets, index, jagged, weight, bias)
            beta = ops.index_select_jagged_bmm(0, offsets, index, jagged, weight_p, bias_p)
            d_ab = torch.empty((rows, 2 * N), dtype=d_out.dtype, device=d_out.device)     # [d_alpha | d_beta]
            d_alpha, d_beta = d_ab[:, :N], d_ab[:, N:]
            activation_backward(1, d_out, alpha, beta, d_alpha, d_beta)
            d_jagged = d_w = d_wp = d_b = d_bp = None
            if ctx.needs_input_grad[2]:
                # d_rows = [d_alpha | d_beta] @ [W ; Wp]^T as one product over 2N
                # (the two transposed weights side by side: storage [E, K, 2N], 2N contiguous)
                # (one grouped product whose reduction walks both transposed weights where they lie;
                #  else the two are laid side by side first: storage [E, K, 2N], 2N contiguous)
                d_rows = ops.jagged_bmm_two_weights(offsets, d_ab, weight.permute(0, 2, 1), weight_p.permute(0, 2, 1))
                if d_rows is None:
                    w_cat = transposed_weights_side_by_side(weight, weight_p)                    # logical [E, 2N, K]
                    d_rows = ops.silu_jagged_bmm(offsets, d_ab, w_cat, None, has_silu=False)
                tok = index.reshape(-1) // A
                d_jagged = ops.mul_merge_k_add(tok, _inverse_rows(index), d_rows)
            flat = index.reshape(-1).contiguous()
            # two products, each written in its parameter's own storage layout (a gradient that
            # is a slice of a larger buffer would be copied by autograd); the token rows are
            # transposed once for both
            once: dict = {}
            if ctx.needs_input_grad[3]:
                d_w = grad_weight(offsets, d_alpha, jagged, E, weight.dtype, index=flat, index_div=A, shared=once)
            if ctx.needs_input_grad[5]:
                d_wp = grad_weight(offsets, d_beta, jagged, E, weight_p.dtype, index=flat, index_div=A, shared=once)
            if bias is not None and ctx.needs_input_grad[4]:
                d_b = grad_bias(offsets, d_alpha, E, bias.dtype)
            if bias_p is not None and ctx.needs_input_grad[6]:
                d_bp = grad_bias(offsets, d_beta, E, bias_p.dtype)
        return None, None, d_jagged, d_w, d_b, d_wp, d_bp


class MulMergeKAddFn(torch.autograd.Function):
    """mul_merge_k_add (kernels/moe.py:71-115) with its backward
    (MulMergeKAddFunction.backward, kernels/triton/triton_moe.py:1039-1100)."""

    @staticmethod
    def forward(ctx, index, reverse_index, value, weight, weight_index):
        with torch.no_grad():
            out = _ops().mul_merge_k_add(index, reverse_index, value, weight=weight, weight_index=weight_index)
        ctx.save_for_backward(index, value, weight, weight_index)
        return out

    @staticmethod
    def backward(ctx, d_out):
        index, value, weight, weight_index = ctx.saved_tensors
        d_out = _contig_rows(d_out)
        d_value = d_weight = None
        with torch.no_grad():
            g = d_out.to(value.dtype) if d_out.dtype != value.dtype else d_out
            if ctx.needs_input_grad[2]:
                d_value = gather_scale_rows(g, index, 1, weight, weight_index)
            if weight is not None and ctx.needs_input_grad[3]:
                dots = row_dot(value, g, index)
                d_flat = torch.zeros(weight.numel(), dtype=torch.float32, device=value.device)
                d_flat[weight_index.reshape(-1)] = dots
                d_weight = d_flat.view(weight.shape).to(weight.dtype)
        return None, None, d_value, d_weight, None


class SiluJaggedBmmCombineFn(torch.autograd.Function):
    """silu_jagged_bmm_combine (kernels/moe.py:236-292) with its backward
    (SiluJaggedBmmCombine.backward, kernels/triton/triton_moe.py:3790-4027)."""

    @staticmethod
    def forward(ctx, offsets, jagged, weight, bias, index, reverse_index, gating_scores, gates_index, has_silu):
        ops = _ops()
        with torch.no_grad():
            # silu(jagged), which the GEMM reads, is kept: the weight gradient needs it
            act = torch.empty_like(jagged, memory_format=torch.contiguous_format) if has_silu else None
            rows = ops.silu_jagged_bmm(offsets, jagged, weight, bias, has_silu=has_silu, _act_scratch=act)
            out = ops.mul_merge_k_add(index, reverse_index, rows, weight=gating_scores, weight_index=gates_index)
        ctx.save_for_backward(offsets, jagged, weight, index, gating_scores, gates_index, rows, act)
        ctx.has_silu = has_silu
        ctx.has_bias = bias is not None
        ctx.bias_dtype = None if bias is None else bias.dtype
        return out

    @staticmethod
    def backward(ctx, d_out):
        offsets, jagged, weight, index, gating_scores, gates_index, rows, act = ctx.saved_tensors
        ops = _ops()
        E = weight.shape[0]
        d_out = _contig_rows(d_out)
        d_jagged = d_weight = d_bias = d_gates = None
        with torch.no_grad():
            g = d_out.to(rows.dtype) if d_out.dtype != rows.dtype else d_out
            d_rows = gather_scale_rows(g, index, 1, gating_scores, gates_index)
            if gating_scores is not None and ctx.needs_input_grad[6]:
                dots = row_dot(rows, g, index)
                d_flat = torch.zeros(gating_scores.numel(), dtype=torch.float32, device=rows.device)
                d_flat[gates_index.reshape(-1)] = dots
                d_gates = d_flat.view(gating_scores.shape).to(gating_scores.dtype)
            if ctx.needs_input_grad[1]:
                d_act = ops.silu_jagged_bmm(offsets, d_rows, transposed_weight(weight), None, has_silu=False)
                if ctx.has_silu:
                    d_jagged = torch.empty_like(d_act)
                    activation_backward(0, d_act, _contig_rows(jagged), None, d_jagged, None)
                else:
                    d_jagged = d_act
            if ctx.needs_input_grad[2]:
                d_weight = grad_weight(offsets, d_rows, act if ctx.has_silu else jagged, E, weight.dtype)
            if ctx.has_bias and ctx.needs_input_grad[3]:
                d_bias = grad_bias(offsets, d_rows, E, ctx.bias_dtype)
        return None, d_jagged, d_weight, d_bias, None, None, d_gates, None, None


class RouterFn(torch.autograd.Function):
    """gate Linear -> softmax -> top-k -> renormalised scores (fmoe_gate_topk) with the backward the
    reference gets from autograd through its eager routing code (modules/fast_moe_module.py:21-27,
    :93-135). Returns (topk_idx [L, k] int64, not differentiable; scores [L, k] f32)."""

    @staticmethod
    def forward(ctx, x, gate_weight, gate_bias, k):
        from .routing import gate_topk

        with torch.no_grad():
            idx, score, _ = gate_topk(x, gate_weight, gate_bias, k)
        ctx.save_for_backward(x, gate_weight, idx, score)
        ctx.has_bias = gate_bias is not None
        ctx.mark_non_differentiable(idx)
        return idx, score

    @staticmethod
    def backward(ctx, _d_idx, d_score):
        x, gate_weight, idx, score = ctx.saved_tensors
        lib = _lib.load()
        dev = x.device
        L, d = x.shape
        E = gate_weight.shape[0]
        k = idx.shape[1]
        with torch.no_grad():
            dy = d_score.to(torch.float32).contiguous()
            d_logits = torch.empty((L, E), dtype=torch.float32, device=dev)
            gw = gate_weight.detach().to(torch.float32).contiguous()
            xx = x if x.stride(1) == 1 else x.contiguous()
            d_x = torch.empty_like(xx) if ctx.needs_input_grad[0] else None
            d_w = torch.empty((E, d), dtype=torch.float32, device=dev) if ctx.needs_input_grad[1] else None
            d_b = torch.empty(E, dtype=torch.float32, device=dev) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
            with torch.cuda.device(dev):
                st = _lib.stream_ptr(dev)
                _lib.check(lib.fmoe_router_backward(idx.data_ptr(), score.data_ptr(), dy.data_ptr(), L, E, k,
                                                    d_logits.data_ptr(), st))
                _lib.check(lib.fmoe_gate_linear_backward(d_logits.data_ptr(), xx.data_ptr(), _lib.dtype_code(xx.dtype),
                                                         xx.stride(0) if L else d, gw.data_ptr(), L, d, E, _lib.ptr(d_x),
                                                         d, _lib.ptr(d_w), _lib.ptr(d_b), st))
            if d_w is not None and d_w.dtype != gate_weight.dtype:
                d_w = d_w.to(gate_weight.dtype)
        return d_x, d_w, d_b, None


class TokenNormFn(torch.autograd.Function):
    """fmoe_token_norm (layer norm, or group norm with one weight / bias per group;
    kernels/pytorch/mrn.py:301-318) with its backward: d_x and the gradients of weight and bias."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, group_norm, num_groups):
        from .routing import token_norm

        with torch.no_grad():
            out = token_norm(x, weight, bias, eps, group_norm=group_norm, num_groups=num_groups)
        ctx.save_for_backward(x, weight)
        ctx.cfg = (float(eps), bool(group_norm), int(num_groups) if group_norm else 1, bias is not None,
                   None if bias is None else bias.dtype)
        return out

    @staticmethod
    def backward(ctx, d_out):
        x, weight = ctx.saved_tensors
        eps, group_norm, groups, has_bias, bias_dtype = ctx.cfg
        lib = _lib.load()
        dev = x.device
        L, d = x.shape
        with torch.no_grad():
            xx = x if x.stride(1) == 1 else x.contiguous()
            g = _contig_rows(d_out.to(xx.dtype) if d_out.dtype != xx.dtype else d_out)
            w32 = None if weight is None else weight.detach().to(torch.float32).contiguous()
            n_params = groups if group_norm else d
            want_w = weight is not None and ctx.needs_input_grad[1]
            want_b = has_bias and ctx.needs_input_grad[2]
            d_x = torch.empty((L, d), dtype=xx.dtype, device=dev)
            chunks = max(1, min(64, (L + 63) // 64))
            stats = torch.empty(max(1, L * groups * 2), dtype=torch.float32, device=dev)
            partial = torch.empty(chunks * 2 * d, dtype=torch.float32, device=dev) if (want_w or want_b) else None
            d_w = torch.empty(n_params, dtype=torch.float32, device=dev) if want_w else None
            d_b = torch.empty(n_params, dtype=torch.float32, device=dev) if want_b else None
            with torch.cuda.device(dev):
                _lib.check(lib.fmoe_token_norm_backward(
                    xx.data_ptr(), g.data_ptr(), _lib.dtype_code(xx.dtype), L, d, xx.stride(0) if L else d,
                    g.stride(0) if L else d, groups, _lib.ptr(w32), 1 if group_norm else 0, eps, d_x.data_ptr(), d,
                    stats.data_ptr(), _lib.ptr(partial), chunks, _lib.ptr(d_w), _lib.ptr(d_b), _lib.stream_ptr(dev)))
            if d_w is not None and d_w.dtype != weight.dtype:
                d_w = d_w.to(weight.dtype)
            if d_b is not None and d_b.dtype != bias_dtype:
                d_b = d_b.to(bias_dtype)
        return (d_x if ctx.needs_input_grad[0] else None), d_w, d_b, None, None, None


class SGRouterFn(torch.autograd.Function):
    """Router of the sparsely-gated layer (fmoe_gate_topk_normalized; kernels/pytorch/mrn.py:236-252)
    with the backward the reference gets from autograd: softmax over all experts of the
    L2-normalised logits, then the gate product. ``gate_weight`` is the parameter as the reference
    stores it, [d, E]. Returns (topk_idx, not differentiable; gates [L, k] f32)."""

    @staticmethod
    def forward(ctx, x, gate_weight, k):
        from .routing import gate_topk_normalized

        with torch.no_grad():
            rows = gate_weight.detach().to(torch.float32).t().contiguous()        # [E, d]
            idx, score, logits = gate_topk_normalized(x, rows, k, return_logits=True)
        ctx.save_for_backward(x, rows, idx, logits)
        ctx.w_dtype = gate_weight.dtype
        ctx.mark_non_differentiable(idx)
        return idx, score

    @staticmethod
    def backward(ctx, _d_idx, d_score):
        x, rows, idx, logits = ctx.saved_tensors
        lib = _lib.load()
        dev = x.device
        L, d = x.shape
        E = rows.shape[0]
        k = idx.shape[1]
        with torch.no_grad():
            dy = d_score.to(torch.float32).contiguous()
            d_logits = torch.empty((L, E), dtype=torch.float32, device=dev)
            xx = x if x.stride(1) == 1 else x.contiguous()
            d_x = torch.empty_like(xx) if ctx.needs_input_grad[0] else None
            d_w = torch.empty((E, d), dtype=torch.float32, device=dev) if ctx.needs_input_grad[1] else None
            with torch.cuda.device(dev):
                st = _lib.stream_ptr(dev)
                _lib.check(lib.fmoe_sg_router_backward(logits.data_ptr(), idx.data_ptr(), dy.data_ptr(), L, E, k,
                                                       d_logits.data_ptr(), st))
                _lib.check(lib.fmoe_gate_linear_backward(d_logits.data_ptr(), xx.data_ptr(), _lib.dtype_code(xx.dtype),
                                                         xx.stride(0) if L else d, rows.data_ptr(), L, d, E, _lib.ptr(d_x),
                                                         d, _lib.ptr(d_w), None, st))
            if d_w is not None:
                d_w = d_w.t().to(ctx.w_dtype)          # back to the parameter's [d, E]
        return d_x, d_w, None


class SGNoisyRouterFn(torch.autograd.Function):
    """Router of the sparsely-gated layer with noisy gating (training): noise * (softplus(x @ w_noise)
    + eps) on the logits, routing on the noisy logits, and the smooth load estimate
    (kernels/pytorch/mrn.py:191-252). ``gate_weight`` / ``noise_weight`` are the parameters [d, E];
    ``noise`` [L, E] f32 is the standard-normal draw. Returns (topk_idx, not differentiable; gates
    [L, k] f32; per-block sums of the smooth load [blocks, E], differentiable, or an empty tensor
    when k == E)."""

    @staticmethod
    def forward(ctx, x, gate_weight, noise_weight, k, noise, noise_eps=1e-2):
        from .routing import gate_topk_normalized

        lib = _lib.load()
        dev = x.device
        L = x.shape[0]
        E = gate_weight.shape[1]
        if 2 * E > 256:
            raise ValueError(f"noisy gating supports up to 128 experts, got {E}")
        with torch.no_grad():
            both = torch.cat([gate_weight.detach().to(torch.float32).t(), noise_weight.detach().to(torch.float32).t()],
                             dim=0).contiguous()                                     # [2E, d]
            _, _, logits2 = gate_topk_normalized(x, both, 1, return_logits=True)
            nz = noise.detach().to(torch.float32).contiguous()
            noisy = torch.empty((L, E), dtype=torch.float32, device=dev)
            stddev = torch.empty((L, E), dtype=torch.float32, device=dev)
            with torch.cuda.device(dev):
                _lib.check(lib.fmoe_sg_noisy_logits(logits2.data_ptr(), 2 * E, nz.data_ptr(), L, E, float(noise_eps),
                                                    noisy.data_ptr(), stddev.data_ptr(), _lib.stream_ptr(dev)))
            idx, score, _ = gate_topk_normalized(None, None, k, logits=noisy)
            if k < E:
                blocks = max(1, min(148, (L + 7) // 8))
                partials = torch.empty((blocks, E), dtype=torch.float32, device=dev)
                with torch.cuda.device(dev):
                    _lib.check(lib.fmoe_sg_noisy_load(logits2.data_ptr(), 2 * E, noisy.data_ptr(), stddev.data_ptr(), L, E,
                                                      k, partials.data_ptr(), blocks, _lib.stream_ptr(dev)))
            else:
                partials = torch.empty((0, E), dtype=torch.float32, device=dev)
        ctx.save_for_backward(x, both, idx, logits2, nz, noisy, stddev)
        ctx.dtypes = (gate_weight.dtype, noise_weight.dtype)
        ctx.mark_non_differentiable(idx)
        return idx, score, partials

    @staticmethod
    def backward(ctx, _d_idx, d_score, d_partials):
        x, both, idx, logits2, nz, noisy, stddev = ctx.saved_tensors
        lib = _lib.load()
        dev = x.device
        L, d = x.shape
        E = both.shape[0] // 2
        k = idx.shape[1]
        with torch.no_grad():
            dy = d_score.to(torch.float32).contiguous()
            # every per-block row carries the same d loss / d load
            d_load = d_partials[0].to(torch.float32).contiguous() if (d_partials is not None and d_partials.shape[0] > 0) else None
            d_logits2 = torch.empty((L, 2 * E), dtype=torch.float32, device=dev)
            xx = x if x.stride(1) == 1 else x.contiguous()
            d_x = torch.empty_like(xx) if ctx.needs_input_grad[0] else None
            want_w = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
            d_both = torch.empty((2 * E, d), dtype=torch.float32, device=dev) if want_w else None
            with torch.cuda.device(dev):
                st = _lib.stream_ptr(dev)
                _lib.check(lib.fmoe_sg_noisy_router_backward(logits2.data_ptr(), 2 * E, nz.data_ptr(), noisy.data_ptr(),
                                                             stddev.data_ptr(), idx.data_ptr(), dy.data_ptr(), _lib.ptr(d_load),
                                                             L, E, k, d_logits2.data_ptr(), 2 * E, st))
                _lib.check(lib.fmoe_gate_linear_backward(d_logits2.data_ptr(), xx.data_ptr(), _lib.dtype_code(xx.dtype),
                                                         xx.stride(0) if L else d, both.data_ptr(), L, d, 2 * E, _lib.ptr(d_x),
                                                         d, _lib.ptr(d_both), None, st))
            d_wg = d_wn = None
            if d_both is not None:
                if ctx.needs_input_grad[1]:
                    d_wg = d_both[:E].t().to(ctx.dtypes[0])
                if ctx.needs_input_grad[2]:
                    d_wn = d_both[E:].t().to(ctx.dtypes[1])
        return d_x, d_wg, d_wn, None, None, None


class SGLossFn(torch.autograd.Function):
    """Training loss and load fractions of the sparsely-gated layer (fmoe_sg_load_loss;
    kernels/pytorch/mrn.py:186-189, :253-277). The loss differentiates with respect to the gates
    through the importance; the load is a count. Returns (loss, load fractions)."""

    @staticmethod
    def forward(ctx, score, offsets, gate_index, num_experts, round_bf16, loss_coef, smooth_load=None):
        lib = _lib.load()
        dev = score.device
        load = torch.empty(num_experts, dtype=torch.float32, device=dev)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        sc = score.detach().contiguous()
        part = None if smooth_load is None else smooth_load.detach().contiguous()
        ctx.part = part
        ctx.empty = sc.numel() == 0
        if ctx.empty:        # an empty batch: its tensors have no storage; nothing is read through these
            sc = torch.zeros(1, dtype=torch.float32, device=dev)
            gate_index = torch.zeros(1, dtype=torch.int64, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.fmoe_sg_load_loss(offsets.data_ptr(), gate_index.data_ptr(), sc.data_ptr(), num_experts,
                                             1 if round_bf16 else 0, float(loss_coef), 1, _lib.ptr(part),
                                             0 if part is None else part.shape[0], load.data_ptr(), loss.data_ptr(),
                                             _lib.stream_ptr(dev)))
        ctx.save_for_backward(sc, offsets, gate_index)
        ctx.score_shape = tuple(score.shape)
        ctx.cfg = (int(num_experts), bool(round_bf16), float(loss_coef))
        ctx.mark_non_differentiable(load)
        return loss, load

    @staticmethod
    def backward(ctx, d_loss, _d_load):
        sc, offsets, gate_index = ctx.saved_tensors
        E, round_bf16, coef = ctx.cfg
        lib = _lib.load()
        dev = sc.device
        part = ctx.part
        if ctx.empty:
            d_part = None if part is None else torch.zeros_like(part)
            return (torch.zeros((0, 0), dtype=torch.float32, device=dev).reshape(ctx.score_shape), None, None, None, None,
                    None, d_part)
        with torch.no_grad():
            d_score = torch.zeros_like(sc)
            dl = d_loss.to(torch.float32).contiguous()
            d_load = None if part is None else torch.empty(E, dtype=torch.float32, device=dev)
            with torch.cuda.device(dev):
                _lib.check(lib.fmoe_sg_loss_backward(offsets.data_ptr(), gate_index.data_ptr(), sc.data_ptr(), E,
                                                     1 if round_bf16 else 0, coef, dl.data_ptr(), d_score.data_ptr(),
                                                     _lib.ptr(part), 0 if part is None else part.shape[0], _lib.ptr(d_load),
                                                     _lib.stream_ptr(dev)))
            # load[e] is the sum of the per-block rows: every row receives d loss / d load
            d_part = None if part is None else d_load.unsqueeze(0).expand_as(part).contiguous()
        return d_score, None, None, None, None, None, d_part


def needs_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)

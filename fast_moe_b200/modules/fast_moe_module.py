"""MoE layers on the sm_100a kernels.

``FastMoELayer`` keeps the constructor, parameter names and forward signature of the reference
layer (modules/fast_moe_module.py:45-225): gate Linear + softmax, top-k, fc1 + bias -> SiLU ->
fc2 + bias per expert, gate-weighted combine. ``SwiGLUFastMoELayer`` is the same routing around
a SwiGLU expert (index_select_jagged_bmm_swiglu + silu_jagged_bmm_combine(has_silu=False),
kernels/moe.py:156-189, :236-292), optionally with e4m3 operands and rowwise scales.
Tensors must be on a CUDA device. The default is the fused inference path; ``layer.autograd = True``
sends the bf16 / fp32 layers through the differentiable operators (kernels/autograd.py).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
from torch.autograd.profiler import record_function

from .. import _lib
from ..kernels import moe as ops
from ..kernels import moe_fp8 as ops_fp8
from ..kernels.routing import (RoutingMetadata, fused_routing_supported, gate_topk, route_metadata,
                               route_tokens_fused, split_gate_weight)
from ..kernels.utils import KernelType


class GatingNetwork(nn.Module):
    """Linear(d -> E); same parameter names as the reference (modules/fast_moe_module.py:21-27).
    ``forward`` returns the dense softmax scores through PyTorch for callers that want them; the
    layers below use the fused gate/top-k kernel instead."""

    def __init__(self, input_dim: int, num_experts: int) -> None:
        super().__init__()
        self.gate = nn.Linear(input_dim, num_experts)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.softmax(self.gate(x), dim=2)


def _xavier_stack(num: int, rows: int, cols: int) -> torch.Tensor:
    """[num, rows, cols], each matrix Xavier-uniform (what utils/utils.py:38-42 produces)."""
    bound = math.sqrt(6.0 / (rows + cols))
    return torch.empty(num, rows, cols).uniform_(-bound, bound)


class _CastCache:
    """Per-dtype copies of parameters, refreshed when the parameter changes in place. The
    reference re-casts every weight on every forward (modules/fast_moe_module.py:167-168,
    :177-178); here the cast happens once per weight update."""

    def __init__(self) -> None:
        self._store: Dict[Tuple[str, torch.dtype], Tuple[int, int, torch.Tensor]] = {}

    def get(self, name: str, p: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        if p.dtype == dtype:
            return p.detach()
        key = (name, dtype)
        hit = self._store.get(key)
        if hit is not None and hit[0] == p._version and hit[1] == p.data_ptr():
            return hit[2]
        t = p.detach().to(dtype)
        self._store[key] = (p._version, p.data_ptr(), t)
        return t


class _SplitCache:
    """Three-term bf16 expansions of float32 weights (ops.split_f32_weight), recomputed when the
    parameter changes in place or moves: what a float32 forward multiplies with when TF32 is not
    allowed. Done once per weight update instead of once per forward."""

    def __init__(self) -> None:
        self._store: Dict[str, Tuple[int, int, torch.Tensor]] = {}

    def get(self, name: str, p: torch.Tensor) -> torch.Tensor:
        """p: parameter stored [E, N, K] float32 -> logical [E, 6 * Kp, N] bf16 weight."""
        hit = self._store.get(name)
        if hit is not None and hit[0] == p._version and hit[1] == p.data_ptr():
            return hit[2]
        t = ops.split_f32_weight(p.detach().to(torch.float32).permute(0, 2, 1))
        self._store[name] = (p._version, p.data_ptr(), t)
        return t


def _training_graph(x: torch.Tensor, module: nn.Module) -> bool:
    """True when this forward has to record an autograd graph: the layer was switched to
    ``autograd = True`` (the default, False, keeps every call on the fused inference path without
    the caller having to wrap it in ``torch.no_grad()``), autograd is recording, and x or a
    parameter requires a gradient."""
    return (getattr(module, "autograd", False) and torch.is_grad_enabled()
            and (x.requires_grad or any(p.requires_grad for p in module.parameters())))


def _fp32_exact(dt: torch.dtype) -> bool:
    return dt == torch.float32 and not ops.fp32_uses_tf32()


def _combine_rows_f32(rows: torch.Tensor, meta: RoutingMetadata, score: torch.Tensor) -> torch.Tensor:
    return ops.mul_merge_k_add(meta.token_index, meta.reverse_index, rows, weight=score.to(rows.dtype),
                               weight_index=meta.gate_index)


# Above this many multiply-adds the gate logits go through the tensor cores (two-term bf16
# expansion of the fp32 gate weights); below it the CUDA-core kernel is as fast and exact in fp32.
GATE_TENSOR_CORE_MACS = 1 << 28


class GateSplitCache:
    """split_gate_weight(weight), recomputed when the weight changes in place or moves."""

    def __init__(self) -> None:
        self._key = None
        self._val: Optional[torch.Tensor] = None

    def get(self, w: torch.Tensor) -> torch.Tensor:
        key = (w._version, w.data_ptr(), w.device)
        if key != self._key:
            self._val = split_gate_weight(w)
            self._key = key
        assert self._val is not None
        return self._val


def route_tokens_with_passes(x_flat: torch.Tensor, gate: nn.Linear, k: int, num_experts: int, cache: GateSplitCache,
                             gather_rows: bool = False, zero_rows: Optional[Tuple[int, torch.dtype]] = None):
    """route_tokens that, for small bf16 batches, runs as the two-launch fused form and lets the
    placement kernel also gather the token rows into expert order and / or clear the buffer the
    fused combine accumulates into. Returns (score, meta, x_sorted or None, cleared buffer or None);
    the last two are None whenever the fused form does not apply (the caller then runs those
    passes the usual way)."""
    L, d = x_flat.shape
    tensor_core_logits = x_flat.dtype == torch.bfloat16 and d % 8 == 0 and L * d * num_experts >= GATE_TENSOR_CORE_MACS
    w = gate.weight.detach()
    if not tensor_core_logits and w.dtype == torch.float32 and fused_routing_supported(x_flat, w):
        with _lib.stage("route"):
            _, score, meta, xs, zbuf = route_tokens_fused(
                x_flat, w, None if gate.bias is None else gate.bias.detach(), k, gather_rows=gather_rows,
                zero_rows=zero_rows)
        return score, meta, xs, zbuf
    score, meta = route_tokens(x_flat, gate, k, num_experts, cache)
    return score, meta, None, None


def route_tokens(x_flat: torch.Tensor, gate: nn.Linear, k: int, num_experts: int,
                 cache: GateSplitCache) -> Tuple[torch.Tensor, RoutingMetadata]:
    """Gate, top-k and routing metadata for one batch of tokens (shared by all layers here)."""
    with _lib.stage("route"):
        L, d = x_flat.shape
        split = None
        if x_flat.dtype == torch.bfloat16 and d % 8 == 0 and L * d * num_experts >= GATE_TENSOR_CORE_MACS:
            split = cache.get(gate.weight)
        idx, score, _ = gate_topk(x_flat, gate.weight.detach(), None if gate.bias is None else gate.bias.detach(), k,
                                  gate_split=split)
        meta = route_metadata(idx, num_experts)
    return score, meta


class _MoEBase(nn.Module):
    num_experts: int
    # False: forward only (the fused inference path, whatever torch's grad mode says). True: when
    # autograd is recording and x or a parameter requires a gradient, the forward runs as autograd
    # Functions (router, projections, combine) and backward() works as it does on the reference.
    autograd = False
    # Fold the gate-weighted combine into the down-projection GEMM (atomic adds into the token
    # rows). "auto": only when k <= 2, where two commutative additions keep the result
    # bit-reproducible; True / False force it on / off.
    fused_combine = "auto"

    def _use_fused_combine(self, k: int) -> bool:
        return k <= 2 if self.fused_combine == "auto" else bool(self.fused_combine)

    def _route(self, x_flat: torch.Tensor, k: int) -> Tuple[torch.Tensor, RoutingMetadata]:
        if not hasattr(self, "_gate_split"):
            self._gate_split = GateSplitCache()
        return route_tokens(x_flat, self.gate.gate, k, self.num_experts, self._gate_split)  # type: ignore[attr-defined]

    def _route_with_passes(self, x_flat: torch.Tensor, k: int, up_cols: int, out_cols: int, fused: bool):
        """Routing plus, when the fused small-batch form applies, the expert-sorted copy of the
        token rows (if the up projection would gather them first anyway) and the cleared
        accumulation buffer of the fused combine."""
        if not hasattr(self, "_gate_split"):
            self._gate_split = GateSplitCache()
        gather = ops._gather_first(x_flat.shape[0] * k, up_cols)
        zero = (out_cols, x_flat.dtype) if fused and x_flat.dtype == torch.bfloat16 else None
        return route_tokens_with_passes(x_flat, self.gate.gate, k, self.num_experts, self._gate_split,  # type: ignore[attr-defined]
                                        gather_rows=gather, zero_rows=zero)


class FastMoELayer(_MoEBase):
    def __init__(
        self,
        input_dim: int,
        hidden_dim: int,
        output_dim: int,
        num_experts: int,
        kernel: KernelType = KernelType.PYTORCH,
        dtype: torch.dtype = torch.bfloat16,
    ) -> None:
        super().__init__()
        self.input_dim = input_dim
        self.hidden_dim = hidden_dim
        self.output_dim = output_dim
        self.num_experts = num_experts
        self.kernel = kernel   # kept for interface compatibility; one implementation exists
        self.dtype = dtype
        self.gate = GatingNetwork(input_dim, num_experts)
        # stored [E, out, in]: the operators receive the permuted [E, in, out] view, whose
        # reduction dimension is contiguous - the layout the tensor core reads directly
        self._experts_hidden_w = nn.Parameter(_xavier_stack(num_experts, hidden_dim, input_dim).to(dtype))
        self._experts_hidden_bias = nn.Parameter(torch.zeros(num_experts, hidden_dim, dtype=dtype))
        self._experts_w = nn.Parameter(_xavier_stack(num_experts, output_dim, hidden_dim).to(dtype))
        self._experts_bias = nn.Parameter(torch.zeros(num_experts, output_dim, dtype=dtype))
        self._cast = _CastCache()
        self._split = _SplitCache()

    def forward(self, x: torch.Tensor, num_experts_per_tok: int) -> torch.Tensor:
        """Forward pass. When a gradient is needed (x or any parameter requires one and autograd
        is recording) the operators run as autograd Functions - the reference's own composition:
        index_select_jagged_bmm, then silu_jagged_bmm_combine(has_silu=True)
        (modules/fast_moe_module.py:146-186) - otherwise as the fused inference path."""
        if _training_graph(x, self):
            return self._forward_with_grad(x, num_experts_per_tok)
        with torch.no_grad():
            return self._forward_inference(x, num_experts_per_tok)

    def _forward_with_grad(self, x: torch.Tensor, k: int) -> torch.Tensor:
        from ..kernels.autograd import RouterFn

        shape = x.shape
        _lib.require_cuda(x)
        x_flat = x.reshape(-1, self.input_dim)
        dt = x.dtype
        idx, score = RouterFn.apply(x_flat, self.gate.gate.weight, self.gate.gate.bias, k)
        meta = route_metadata(idx, self.num_experts)
        with record_function("## expert_forward##"):
            cast = lambda p: p if p.dtype == dt else p.to(dt)
            hidden = ops.index_select_jagged_bmm(0, meta.offsets, meta.gate_index.view(-1, k), x_flat,
                                                 cast(self._experts_hidden_w).permute(0, 2, 1), cast(self._experts_hidden_bias))
            y = ops.silu_jagged_bmm_combine(0, meta.offsets, hidden, cast(self._experts_w).permute(0, 2, 1),
                                            cast(self._experts_bias), meta.token_index, meta.reverse_index,
                                            gating_scores=score, gates_index=meta.gate_index, has_silu=True,
                                            round_scores=True)
        return y.view(*shape[:-1], self.output_dim)

    def _forward_inference(self, x: torch.Tensor, num_experts_per_tok: int) -> torch.Tensor:
        shape = x.shape
        k = num_experts_per_tok
        x_flat = x.reshape(-1, self.input_dim)
        _lib.require_cuda(x)
        fused = self._use_fused_combine(k)
        if _fp32_exact(x.dtype):
            score, meta = self._route(x_flat, k)
            # float32 without TF32: operands expanded into bf16 terms (weights once per update)
            with record_function("## expert_forward##"):
                b1 = self._cast.get("b1", self._experts_hidden_bias, x.dtype)
                b2 = self._cast.get("b2", self._experts_bias, x.dtype)
                with _lib.stage("up"):
                    hidden = ops.index_select_jagged_bmm(
                        0, meta.offsets, meta.gate_index.view(-1, k), ops.split_f32_rows(x_flat, 0),
                        self._split.get("w1", self._experts_hidden_w), b1, _epilogue=_lib.EPI_SILU,
                        _out_dtype=torch.float32)
                with _lib.stage("down"):
                    rows = ops.silu_jagged_bmm(meta.offsets, ops.split_f32_rows(hidden, 0),
                                               self._split.get("w2", self._experts_w), b2, has_silu=False,
                                               _out_dtype=torch.float32)
                with _lib.stage("combine"):
                    y = _combine_rows_f32(rows, meta, score)
            return y.view(*shape[:-1], self.output_dim)
        score, meta, x_sorted, y_buf = self._route_with_passes(x_flat, k, self.hidden_dim, self.output_dim, fused)
        with record_function("## expert_forward##"):
            dt = x.dtype
            w1 = self._cast.get("w1", self._experts_hidden_w, dt).permute(0, 2, 1)
            b1 = self._cast.get("b1", self._experts_hidden_bias, dt)
            w2 = self._cast.get("w2", self._experts_w, dt).permute(0, 2, 1)
            b2 = self._cast.get("b2", self._experts_bias, dt)
            # SiLU is applied in the first GEMM's epilogue rather than on the second GEMM's input
            with _lib.stage("up"):
                if x_sorted is not None:
                    hidden = ops.index_select_jagged_bmm(0, meta.offsets, None, x_sorted, w1, b1, _epilogue=_lib.EPI_SILU)
                else:
                    hidden = ops.index_select_jagged_bmm(
                        0, meta.offsets, meta.gate_index.view(-1, k), x_flat, w1, b1, _epilogue=_lib.EPI_SILU
                    )
            with _lib.stage("down_combine"):
                y = ops.silu_jagged_bmm_combine(
                    0, meta.offsets, hidden, w2, b2, meta.token_index, meta.reverse_index,
                    gating_scores=score, gates_index=meta.gate_index, has_silu=False,
                    fused=fused, round_scores=True, out=y_buf,
                )
        return y.view(*shape[:-1], self.output_dim)


class SwiGLUFastMoELayer(_MoEBase):
    """Top-k routed SwiGLU experts: y = sum_j g_j * W_down[e_j] (silu(x W_gate[e_j]) * (x W_up[e_j])).

    Parameters are stored with the reduction dimension contiguous: w_gate / w_up [E, h, d],
    w_down [E, o, h]. With ``fp8=True`` the weights are quantised once (per output row, rule of
    kernels/pytorch/quant_fp8.py:13-34) by ``quantize_weights()`` and the forward quantises x
    and the hidden activations per row before each e4m3 GEMM.
    """

    def __init__(
        self,
        input_dim: int,
        hidden_dim: int,
        output_dim: int,
        num_experts: int,
        dtype: torch.dtype = torch.bfloat16,
        init_std: float = 0.02,
        fp8: bool = False,
    ) -> None:
        super().__init__()
        self.input_dim = input_dim
        self.hidden_dim = hidden_dim
        self.output_dim = output_dim
        self.num_experts = num_experts
        self.dtype = dtype
        self.fp8 = fp8
        self.gate = GatingNetwork(input_dim, num_experts)
        self.w_gate = nn.Parameter((torch.randn(num_experts, hidden_dim, input_dim) * init_std).to(dtype))
        self.w_up = nn.Parameter((torch.randn(num_experts, hidden_dim, input_dim) * init_std).to(dtype))
        self.w_down = nn.Parameter((torch.randn(num_experts, output_dim, hidden_dim) * init_std).to(dtype))
        self._cast = _CastCache()
        self._split = _SplitCache()
        self._q: Optional[Dict[str, Tuple[torch.Tensor, torch.Tensor]]] = None

    @torch.no_grad()
    def quantize_weights(self) -> None:
        """(Re)builds the e4m3 copies of the three weight tensors and their [E, rows] scales."""
        self._q = {
            name: ops_fp8.rowwise_quant_fp8(getattr(self, name).detach())
            for name in ("w_gate", "w_up", "w_down")
        }

    def forward(self, x: torch.Tensor, num_experts_per_tok: int) -> torch.Tensor:
        """Forward pass; with a gradient needed (and no FP8) the operators run as autograd
        Functions: index_select_jagged_bmm_swiglu, then silu_jagged_bmm_combine(has_silu=False)."""
        if not self.fp8 and _training_graph(x, self):
            return self._forward_with_grad(x, num_experts_per_tok)
        with torch.no_grad():
            return self._forward_inference(x, num_experts_per_tok)

    def _forward_with_grad(self, x: torch.Tensor, k: int) -> torch.Tensor:
        from ..kernels.autograd import RouterFn

        shape = x.shape
        _lib.require_cuda(x)
        x_flat = x.reshape(-1, self.input_dim)
        dt = x.dtype
        idx, score = RouterFn.apply(x_flat, self.gate.gate.weight, self.gate.gate.bias, k)
        meta = route_metadata(idx, self.num_experts)
        cast = lambda p: p if p.dtype == dt else p.to(dt)
        hidden = ops.index_select_jagged_bmm_swiglu(0, meta.offsets, meta.gate_index.view(-1, k), x_flat,
                                                    cast(self.w_gate).permute(0, 2, 1), None,
                                                    cast(self.w_up).permute(0, 2, 1), None)
        y = ops.silu_jagged_bmm_combine(0, meta.offsets, hidden, cast(self.w_down).permute(0, 2, 1), None,
                                        meta.token_index, meta.reverse_index, gating_scores=score,
                                        gates_index=meta.gate_index, has_silu=False, round_scores=True)
        return y.view(*shape[:-1], self.output_dim)

    def _forward_inference(self, x: torch.Tensor, num_experts_per_tok: int) -> torch.Tensor:
        shape = x.shape
        k = num_experts_per_tok
        x_flat = x.reshape(-1, self.input_dim)
        _lib.require_cuda(x)
        fused = self._use_fused_combine(k)
        dt = x.dtype
        x_sorted = y_buf = None
        if self.fp8 or _fp32_exact(dt):
            score, meta = self._route(x_flat, k)
        else:
            score, meta, x_sorted, y_buf = self._route_with_passes(x_flat, k, 2 * self.hidden_dim, self.output_dim, fused)
        index = meta.gate_index.view(-1, k)
        with record_function("## expert_forward##"):
            if self.fp8:
                if self._q is None:
                    self.quantize_weights()
                assert self._q is not None
                (wg, sg), (wu, su), (wd, sd) = self._q["w_gate"], self._q["w_up"], self._q["w_down"]
                with _lib.stage("quant_x"):
                    xq, xs = ops_fp8.rowwise_quant_fp8(x_flat)
                with _lib.stage("up"):
                    hidden = ops_fp8.index_select_jagged_bmm_fp8_quantized(
                        meta.offsets, index, xq, xs, wg, sg, None, out_dtype=dt, weight_p_q=wu, weight_p_scale=su
                    )
                with _lib.stage("quant_hidden"):
                    hq, hs = ops_fp8.rowwise_quant_fp8(hidden)
                if fused and dt == torch.bfloat16:
                    with _lib.stage("down_combine"):
                        y = ops_fp8.fp8_jagged_bmm_combine_quantized(
                            meta.offsets, hq, hs, wd, sd, None, score, meta.gate_index, x_flat.shape[0], out_dtype=dt
                        )
                else:
                    with _lib.stage("down"):
                        y_rows = ops_fp8.fp8_jagged_bmm_quantized(meta.offsets, hq, hs, wd, sd, None, out_dtype=dt)
                    with _lib.stage("combine"):
                        y = ops.mul_merge_k_add(
                            meta.token_index, meta.reverse_index, y_rows, weight=score.to(dt),
                            weight_index=meta.gate_index,
                        )
            elif _fp32_exact(dt):
                with _lib.stage("up"):
                    hidden = ops.index_select_jagged_bmm_swiglu(
                        0, meta.offsets, index, ops.split_f32_rows(x_flat, 0), self._split.get("wg", self.w_gate), None,
                        self._split.get("wu", self.w_up), None, _out_dtype=torch.float32)
                with _lib.stage("down"):
                    rows = ops.silu_jagged_bmm(meta.offsets, ops.split_f32_rows(hidden, 0),
                                               self._split.get("wd", self.w_down), None, has_silu=False,
                                               _out_dtype=torch.float32)
                with _lib.stage("combine"):
                    y = _combine_rows_f32(rows, meta, score)
            else:
                wg = self._cast.get("wg", self.w_gate, dt).permute(0, 2, 1)
                wu = self._cast.get("wu", self.w_up, dt).permute(0, 2, 1)
                wd = self._cast.get("wd", self.w_down, dt).permute(0, 2, 1)
                with _lib.stage("up"):
                    if x_sorted is not None:
                        hidden = ops.index_select_jagged_bmm_swiglu(0, meta.offsets, None, x_sorted, wg, None, wu, None)
                    else:
                        hidden = ops.index_select_jagged_bmm_swiglu(0, meta.offsets, index, x_flat, wg, None, wu, None)
                with _lib.stage("down_combine"):
                    y = ops.silu_jagged_bmm_combine(
                        0, meta.offsets, hidden, wd, None, meta.token_index, meta.reverse_index,
                        gating_scores=score, gates_index=meta.gate_index, has_silu=False,
                        fused=fused, round_scores=True, out=y_buf,
                    )
        return y.view(*shape[:-1], self.output_dim)


class CapturedForward:
    """One forward of a layer recorded as a CUDA graph and replayed with a single launch.

    The layer's kernels are tiny next to their launch cost at small token counts (eight launches
    per forward); replaying a captured graph removes the host work between them. Input and output
    live in static buffers: ``__call__`` copies the new tokens in, replays, and returns the
    static output tensor (overwritten by the next call). Shapes, dtype and ``k`` are fixed at
    capture time; weights are read in place, so in-place weight updates are seen by later replays.
    """

    def __init__(self, layer: nn.Module, example: torch.Tensor, num_experts_per_tok: int, warmup: int = 3) -> None:
        if not example.is_cuda:
            raise RuntimeError("CapturedForward needs a CUDA tensor")
        if _lib._stage_timer is not None:
            raise RuntimeError("stage timing records events and cannot be captured; disable it first")
        self.k = num_experts_per_tok
        self.x = example.clone()
        side = torch.cuda.Stream(device=example.device)
        side.wait_stream(torch.cuda.current_stream(example.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):      # first calls resolve symbols and set kernel attributes
                layer(self.x, self.k)
        torch.cuda.current_stream(example.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.y = layer(self.x, self.k)

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.y

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        self.x.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.y


class CapturedTrainStep:
    """Forward and backward of a layer (``layer.autograd = True``) recorded as one CUDA graph.

    A training step of a layer at small token counts is some fifty launches and as many Python
    calls of autograd bookkeeping; replayed as a graph it costs one launch. ``step(x, d_out)``
    copies the tokens and the output gradient into static buffers, replays, and leaves
    ``self.y`` (the output), ``self.d_x`` and every parameter's ``.grad`` (static tensors,
    overwritten by the next step; an optimizer reads them in place). The backward seeds from
    ``d_out``; ``forward_fn(layer, x)`` may replace the default call ``layer(x, k)`` and must
    return the tensor to differentiate. Shapes, dtype and routing width are fixed at capture time;
    the routing itself is data dependent and runs inside the graph."""

    def __init__(self, layer: nn.Module, example: torch.Tensor, num_experts_per_tok: int, warmup: int = 3,
                 forward_fn=None) -> None:
        if not example.is_cuda:
            raise RuntimeError("CapturedTrainStep needs a CUDA tensor")
        if not getattr(layer, "autograd", False):
            raise RuntimeError("CapturedTrainStep needs layer.autograd = True")
        if _lib._stage_timer is not None:
            raise RuntimeError("stage timing records events and cannot be captured; disable it first")
        self.layer = layer
        k = num_experts_per_tok
        self._fwd = forward_fn if forward_fn is not None else (lambda m, t: m(t, k))
        dev = example.device
        self.x = example.detach().clone().requires_grad_(True)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            y = self._fwd(layer, self.x)
            self.d_out = torch.zeros_like(y)
            y.backward(self.d_out)
            for _ in range(max(0, warmup - 1)):
                self._clear_grads()
                self._fwd(layer, self.x).backward(self.d_out)
        torch.cuda.current_stream(dev).wait_stream(side)
        self._clear_grads()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.y = self._fwd(layer, self.x)
            self.y.backward(self.d_out)
        self.d_x = self.x.grad

    def _clear_grads(self) -> None:
        self.x.grad = None
        for p in self.layer.parameters():
            p.grad = None

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.y

    def step(self, x: torch.Tensor, d_out: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            self.x.copy_(x, non_blocking=True)
            self.d_out.copy_(d_out, non_blocking=True)
        self.graph.replay()
        return self.y


class StreamingForward:
    """Host-to-host forward over a stream of batches: tokens come from pinned host memory and the
    result goes back to pinned host memory, with the three legs of consecutive batches overlapped.

    Each of ``slots`` slots owns a device input buffer and (single-process layers) a CUDA graph of
    the forward with its own output buffer. ``submit`` queues, without blocking the host, the
    host-to-device copy on a copy-in stream, the forward on a compute stream and the
    device-to-host copy on a copy-out stream; events order the legs of one batch and keep a slot's
    buffers from being overwritten while an earlier batch still uses them. With two or more slots
    the copy of batch i+1 and the read-back of batch i-1 run while batch i computes, so the
    steady-state cost of a batch is the slowest leg instead of their sum. ``drain`` makes the
    caller's stream wait for everything queued so far. Batches complete in submission order.

    ``capture=False`` runs the layer eagerly on the compute stream (needed for layers that
    synchronise with the host inside the forward, like the expert-parallel one).
    """

    def __init__(self, layer: nn.Module, example: torch.Tensor, num_experts_per_tok: int, slots: int = 2,
                 capture: bool = True) -> None:
        if not example.is_cuda:
            raise RuntimeError("StreamingForward needs a CUDA example tensor (shape and dtype of one batch)")
        if slots < 1:
            raise ValueError("slots must be >= 1")
        dev = example.device
        self.layer = layer
        self.k = num_experts_per_tok
        self.device = dev
        self.s_in = torch.cuda.Stream(device=dev)
        self.s_run = torch.cuda.Stream(device=dev)
        self.s_out = torch.cuda.Stream(device=dev)
        self.graphs = [CapturedForward(layer, example, num_experts_per_tok) for _ in range(slots)] if capture else None
        self.x = [g.x for g in self.graphs] if capture else [torch.empty_like(example) for _ in range(slots)]
        self.y = [None] * slots
        ev = lambda: torch.cuda.Event(enable_timing=True)
        self.in_start = [ev() for _ in range(slots)]
        self.run_start = [ev() for _ in range(slots)]
        self.out_start = [ev() for _ in range(slots)]
        self.in_ready = [ev() for _ in range(slots)]
        self.run_done = [ev() for _ in range(slots)]
        self.out_done = [ev() for _ in range(slots)]
        self.used = [False] * slots
        self.count = 0
        cur = torch.cuda.current_stream(dev)
        for st in (self.s_in, self.s_run, self.s_out):
            st.wait_stream(cur)

    def submit(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        """Queue one batch: x_host (pinned) -> device -> forward -> y_host (pinned)."""
        s = self.count % len(self.x)
        self.count += 1
        with torch.cuda.stream(self.s_in):
            if self.used[s]:
                self.s_in.wait_event(self.run_done[s])      # the slot's previous batch has been consumed
            self.in_start[s].record(self.s_in)
            self.x[s].copy_(x_host, non_blocking=True)
            self.in_ready[s].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.in_ready[s])
            if self.used[s]:
                self.s_run.wait_event(self.out_done[s])     # the slot's previous result has left the device
            self.run_start[s].record(self.s_run)
            if self.graphs is not None:
                y = self.graphs[s].replay()
            else:
                y = self.layer(self.x[s], self.k)
                y.record_stream(self.s_out)
            self.y[s] = y
            self.run_done[s].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.run_done[s])
            self.out_start[s].record(self.s_out)
            y_host.copy_(y.view(y_host.shape), non_blocking=True)
            self.out_done[s].record(self.s_out)
        self.used[s] = True

    def drain(self) -> None:
        """Make the current stream wait for every batch submitted so far (no host block)."""
        cur = torch.cuda.current_stream(self.device)
        for st in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(st)

    def synchronize(self) -> None:
        for st in (self.s_in, self.s_run, self.s_out):
            st.synchronize()

    def leg_times_ms(self) -> Dict[str, float]:
        """Device time of the three legs of the most recent batch of every slot (host-to-device
        copy, forward, device-to-host copy), averaged over the slots in use: shows which leg a
        pipeline that is slower than its forward is waiting for. Synchronises."""
        self.synchronize()
        used = [s for s in range(len(self.x)) if self.used[s]]
        if not used:
            return {}
        avg = lambda a, b: sum(a[s].elapsed_time(b[s]) for s in used) / len(used)
        return dict(h2d=avg(self.in_start, self.in_ready), forward=avg(self.run_start, self.run_done),
                    d2h=avg(self.out_start, self.out_done))


class HostPipeline:
    """Host-to-host forward with ONE launch per batch: every slot owns a pinned input buffer, a
    pinned output buffer, a stream and a CUDA graph that holds the slot's host-to-device copy, the
    forward and the device-to-host copy. ``launch(s)`` replays slot s's graph on its stream;
    consecutive batches go to different slots, so the copies of one batch overlap the forward of
    another (copy engines and SMs work side by side) while the host issues a single call per batch
    - at small batch sizes the per-batch host work of ``StreamingForward`` (stream switches, event
    records and waits) is otherwise the slowest part of the pipeline.

    The caller writes a batch into ``host_in[s]`` (pinned: fill it in place), calls ``launch(s)``,
    and reads ``host_out[s]`` after ``wait(s)``. Shapes, dtype and ``k`` are fixed at construction;
    the layer must not synchronise with the host inside its forward."""

    def __init__(self, layer: nn.Module, example: torch.Tensor, num_experts_per_tok: int, slots: int = 3,
                 out_shape: Optional[Tuple[int, ...]] = None) -> None:
        if not example.is_cuda:
            raise RuntimeError("HostPipeline needs a CUDA example tensor (shape and dtype of one batch)")
        if _lib._stage_timer is not None:
            raise RuntimeError("stage timing records events and cannot be captured; disable it first")
        dev = example.device
        self.device = dev
        self.k = num_experts_per_tok
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(slots)]
        self.host_in = [torch.empty(example.shape, dtype=example.dtype).pin_memory() for _ in range(slots)]
        self.x = [torch.empty_like(example) for _ in range(slots)]
        self.graphs, self.y, self.host_out = [], [], []
        cur = torch.cuda.current_stream(dev)
        for s in range(slots):
            st = self.streams[s]
            st.wait_stream(cur)
            with torch.cuda.stream(st):
                self.x[s].copy_(example)
                for _ in range(2):
                    y = layer(self.x[s], self.k)
                st.synchronize()
                self.host_out.append(torch.empty(y.shape, dtype=y.dtype).pin_memory())
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    self.x[s].copy_(self.host_in[s], non_blocking=True)
                    y = layer(self.x[s], self.k)
                    self.host_out[s].copy_(y, non_blocking=True)
                self.graphs.append(g)
                self.y.append(y)
        for st in self.streams:
            st.synchronize()

    def launch(self, slot: int) -> None:
        """Queue slot's batch: host_in[slot] -> device -> forward -> host_out[slot]."""
        with torch.cuda.stream(self.streams[slot]):
            self.graphs[slot].replay()

    def wait(self, slot: int) -> None:
        self.streams[slot].synchronize()

    def drain(self) -> None:
        """Make the current stream wait for every batch queued so far (no host block)."""
        cur = torch.cuda.current_stream(self.device)
        for st in self.streams:
            cur.wait_stream(st)

    def synchronize(self) -> None:
        for st in self.streams:
            st.synchronize()

"""The sparsely-gated ("MRN" / SGMoE) layer on the sm_100a kernels: constructor, parameter names and
forward signature of the reference's OrigSGMoEImpl (kernels/pytorch/mrn.py:93-333).

  x -> layer norm or group norm -> router (L2-normalised logits, softmax over all experts, the k
  largest probabilities kept as they are) -> fc1 + bias -> SiLU -> fc2 + bias per expert ->
  gate-weighted sum per token -> + x @ output_weight (a dense map of the un-normalised tokens)
  -> MRNOutput(y, loss, load fractions)

The experts, the combine and the dense map are the grouped GEMMs of the FastMoELayer path; the
router is the gate kernel in its normalised-logit mode; normalisation and the load / loss summary
are small kernels of their own. ``layer.autograd = True`` switches the forward to a chain of
differentiable operators (backward of the norm, the router, the experts, the shared map and the
loss); the default is the fused inference path under any grad mode. With noisy gating a layer in training mode adds
softplus-scaled standard-normal noise to the logits before routing and uses the smooth load
estimate in its loss; in evaluation mode it routes on the clean logits (as the reference does).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import NamedTuple, Optional

import torch
import torch.nn as nn

from .. import _lib
from ..kernels import moe as ops
from ..kernels.routing import gate_topk_normalized, noisy_gate, route_metadata, sg_load_loss, token_norm
from .fast_moe_module import _CastCache, _SplitCache, _fp32_exact, _xavier_stack


class MRNOutput(NamedTuple):
    x: torch.Tensor
    loss: Optional[torch.Tensor]
    load: Optional[torch.Tensor]


@dataclass
class SGConfig:
    """kernels/pytorch/mrn.py:26-41 of the reference."""

    model_d: int
    num_experts: int
    num_activated_experts: int
    loss_coef: float = 1e-2
    use_input_dtype: bool = True
    activation_checkpointing: bool = False
    enable_noisy_gating: bool = False


class SGMoELayer(nn.Module):
    def __init__(self, input_size: int, output_size: int, config: SGConfig, custom_kernel: bool = True,
                 is_train: bool = True) -> None:
        super().__init__()
        self.num_experts = config.num_experts
        self.k = config.num_activated_experts
        self.loss_coef = config.loss_coef
        self.model_d = config.model_d
        self.output_size = output_size
        self.input_size = input_size
        self.custom_kernel = custom_kernel       # kept for interface compatibility; one implementation exists
        self.is_train = is_train
        self.use_input_dtype = config.use_input_dtype
        self.enable_noisy_gating = config.enable_noisy_gating
        assert self.k <= self.num_experts
        E = self.num_experts
        self._experts_hidden_w = nn.Parameter(_xavier_stack(E, self.model_d, input_size))
        self._experts_hidden_bias = nn.Parameter(torch.zeros(E, self.model_d))
        self._experts_w = nn.Parameter(_xavier_stack(E, output_size, self.model_d))
        self._experts_bias = nn.Parameter(torch.zeros(E, output_size))
        if self.enable_noisy_gating:
            self._w_gate = nn.Parameter(torch.zeros(input_size, E))
            self._w_noise = nn.Parameter(torch.zeros(input_size, E))
        else:
            self._w_gate = nn.Parameter(nn.init.xavier_uniform_(torch.empty(input_size, E)))
        self.register_buffer("mean", torch.tensor([0.0]))
        self.register_buffer("std", torch.tensor([1.0]))
        self._output_weight = nn.Parameter(nn.init.xavier_uniform_(torch.empty(input_size, output_size)))
        self._k_plus = min(self.k + 1, E)
        self._cast = _CastCache()
        self._split = _SplitCache()
        self._gate_t = None          # (version, data_ptr, [E, d] f32 copy of _w_gate)
        self._gate_noise_t = None    # (versions, data_ptrs, [2E, d] f32: _w_gate^T stacked on _w_noise^T)
        self._noise = None           # standard-normal draw for the next noisy forward (set_noise)
        self.autograd = False        # True: forward through the differentiable operators (training)
        self._out_t = {}             # dtype -> (version, data_ptr, [1, o, d] copy of _output_weight)
        self._ident = {}

    # ------------------------------------------------------------------ cached layouts
    def _gate_weight_rows(self) -> torch.Tensor:
        p = self._w_gate
        hit = self._gate_t
        if hit is None or hit[0] != p._version or hit[1] != p.data_ptr():
            self._gate_t = hit = (p._version, p.data_ptr(), p.detach().to(torch.float32).t().contiguous())
        return hit[2]

    def _gate_noise_rows(self) -> torch.Tensor:
        g, n = self._w_gate, self._w_noise
        key = (g._version, n._version, g.data_ptr(), n.data_ptr())
        hit = self._gate_noise_t
        if hit is None or hit[0] != key:
            both = torch.cat([g.detach().to(torch.float32).t(), n.detach().to(torch.float32).t()], dim=0).contiguous()
            self._gate_noise_t = hit = (key, both)
        return hit[1]

    def set_noise(self, noise: Optional[torch.Tensor]) -> None:
        """Noise [L, num_experts] (f32, standard normal) for the next noisy-gating forward instead of
        a fresh torch.randn draw: reproducible runs and tests. Used once."""
        self._noise = noise

    def _shared_weight(self, dtype: torch.dtype) -> torch.Tensor:
        """_output_weight [d, o] as a one-expert weight with the reduction dimension contiguous:
        storage [1, o, d], handed to the operators as its logical [1, d, o] view."""
        p = self._output_weight
        hit = self._out_t.get(dtype)
        if hit is None or hit[0] != p._version or hit[1] != p.data_ptr():
            self._out_t[dtype] = hit = (p._version, p.data_ptr(), p.detach().to(dtype).t().contiguous().unsqueeze(0))
        return hit[2].permute(0, 2, 1)

    def _identity_routing(self, L: int, dtype: torch.dtype, dev: torch.device):
        key = (L, dtype, dev)
        if key not in self._ident:
            ar = torch.arange(L, dtype=torch.int64, device=dev)
            self._ident = {key: (torch.tensor([0, L], dtype=torch.int64, device=dev), ar, ar.view(L, 1),
                                 torch.ones((L, 1), dtype=dtype, device=dev))}
        return self._ident[key]

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, x_offsets: Optional[torch.Tensor], max_seq_len: int, group_norm: bool,
                num_groups: int, linear_dim: int, norm_weight: Optional[torch.Tensor],
                norm_bias: Optional[torch.Tensor], norm_eps: float) -> MRNOutput:
        """x [L, input_size] (jagged batch, already flattened; ``x_offsets`` / ``max_seq_len`` are
        accepted and unused, as in the reference) -> MRNOutput(y [L, output_size], loss, load).
        With ``self.autograd = True`` (and torch's grad mode on) the call records a backward for x,
        the norm's weight / bias and every parameter; otherwise it is the fused inference path."""
        if self.autograd and torch.is_grad_enabled():
            return self._forward_with_grad(x, group_norm, num_groups, linear_dim, norm_weight, norm_bias, norm_eps)
        with torch.no_grad():
            return self._forward_inference(x, group_norm, num_groups, linear_dim, norm_weight, norm_bias, norm_eps)

    def _forward_with_grad(self, x, group_norm, num_groups, linear_dim, norm_weight, norm_bias, norm_eps) -> MRNOutput:
        """The same layer as a chain of differentiable operators: token norm, router, the two
        expert products with SiLU between them and the gate-weighted combine, the dense map of the
        un-normalised tokens, and the loss (with noisy gating: noise on the logits and the smooth load,
        both differentiated with respect to the two gate matrices)."""
        from ..kernels.autograd import SGLossFn, SGNoisyRouterFn, SGRouterFn, TokenNormFn

        dev = _lib.require_cuda(x)
        assert x.ndim == 2 and x.shape[1] == self.input_size
        L, k, E, dt = x.shape[0], self.k, self.num_experts, x.dtype
        cast = lambda p: p if p.dtype == dt else p.to(dt)
        x_norm = TokenNormFn.apply(x, norm_weight, norm_bias, norm_eps, bool(group_norm), num_groups)
        smooth_load = None
        if self.training and self.enable_noisy_gating:
            noise, self._noise = self._noise, None
            if noise is None:
                noise = torch.randn((L, E), dtype=torch.float32, device=dev)
            idx, score, smooth_load = SGNoisyRouterFn.apply(x_norm, self._w_gate, self._w_noise, k, noise.to(dev))
            if smooth_load.shape[0] == 0:
                smooth_load = None
        else:
            idx, score = SGRouterFn.apply(x_norm, self._w_gate, k)
        meta = route_metadata(idx, E)
        hidden = ops.index_select_jagged_bmm(0, meta.offsets, meta.gate_index.view(-1, k), x_norm,
                                             cast(self._experts_hidden_w).permute(0, 2, 1), cast(self._experts_hidden_bias))
        moe = ops.silu_jagged_bmm_combine(0, meta.offsets, hidden, cast(self._experts_w).permute(0, 2, 1),
                                          cast(self._experts_bias), meta.token_index, meta.reverse_index,
                                          gating_scores=score, gates_index=meta.gate_index, has_silu=True, round_scores=True)
        off1, ar, ar2, _ = self._identity_routing(L, dt, dev)
        shared = ops.index_select_jagged_bmm(0, off1, ar2, x, cast(self._output_weight).unsqueeze(0), None)
        y = moe + shared
        if self.training:
            loss, load = SGLossFn.apply(score, meta.offsets, meta.gate_index, E, dt == torch.bfloat16, self.loss_coef,
                                        smooth_load)
        else:
            loss, load = sg_load_loss(meta, score.detach(), E, dt, self.loss_coef, False)
        return MRNOutput(y, loss, load)

    def _forward_inference(self, x: torch.Tensor, group_norm: bool, num_groups: int, linear_dim: int,
                           norm_weight: Optional[torch.Tensor], norm_bias: Optional[torch.Tensor],
                           norm_eps: float) -> MRNOutput:
        dev = _lib.require_cuda(x)
        assert x.ndim == 2 and x.shape[1] == self.input_size
        if group_norm:
            assert num_groups * linear_dim == self.input_size
        L, k, E, dt = x.shape[0], self.k, self.num_experts, x.dtype
        with _lib.stage("norm"):
            x_norm = token_norm(x, norm_weight, norm_bias, norm_eps, group_norm=group_norm, num_groups=num_groups)
        smooth_load = None
        with _lib.stage("route"):
            if self.training and self.enable_noisy_gating:
                noise, self._noise = self._noise, None
                if noise is None:
                    noise = torch.randn((L, E), dtype=torch.float32, device=dev)
                idx, score, smooth_load = noisy_gate(x_norm, self._gate_noise_rows(), k, noise.to(dev, torch.float32))
            else:
                idx, score, _ = gate_topk_normalized(x_norm, self._gate_weight_rows(), k)
            meta = route_metadata(idx, E)
        index = meta.gate_index.view(-1, k)
        b1 = self._cast.get("b1", self._experts_hidden_bias, dt)
        b2 = self._cast.get("b2", self._experts_bias, dt)
        if _fp32_exact(dt):
            with _lib.stage("up"):
                hidden = ops.index_select_jagged_bmm(0, meta.offsets, index, ops.split_f32_rows(x_norm, 0),
                                                     self._split.get("w1", self._experts_hidden_w), b1,
                                                     _epilogue=_lib.EPI_SILU, _out_dtype=torch.float32)
            with _lib.stage("down"):
                rows = ops.silu_jagged_bmm(meta.offsets, ops.split_f32_rows(hidden, 0),
                                           self._split.get("w2", self._experts_w), b2, has_silu=False,
                                           _out_dtype=torch.float32)
            with _lib.stage("combine"):
                moe = ops.mul_merge_k_add(meta.token_index, meta.reverse_index, rows, weight=score, weight_index=meta.gate_index)
            with _lib.stage("shared"):
                off1, _, _, _ = self._identity_routing(L, dt, dev)
                shared = ops.silu_jagged_bmm(off1, x, self._shared_weight(torch.float32), None, has_silu=False)
                y = moe.add_(shared)      # the one elementwise step left to torch, in the fp32-accuracy mode only
        else:
            w1 = self._cast.get("w1", self._experts_hidden_w, dt).permute(0, 2, 1)
            w2 = self._cast.get("w2", self._experts_w, dt).permute(0, 2, 1)
            with _lib.stage("up"):
                hidden = ops.index_select_jagged_bmm(0, meta.offsets, index, x_norm, w1, b1, _epilogue=_lib.EPI_SILU)
            with _lib.stage("down_combine"):
                moe = ops.silu_jagged_bmm_combine(0, meta.offsets, hidden, w2, b2, meta.token_index, meta.reverse_index,
                                                  gating_scores=score, gates_index=meta.gate_index, has_silu=False,
                                                  fused=k <= 2, round_scores=True)
            with _lib.stage("shared"):
                # y = moe + x @ output_weight: the dense map runs as a one-expert grouped GEMM whose
                # epilogue adds its rows to what `moe` holds (identity routing, gate weight 1)
                off1, ar, ar2, ones = self._identity_routing(L, dt, dev)
                y = ops.silu_jagged_bmm_combine(0, off1, x, self._shared_weight(dt), None, ar, ar2, gating_scores=ones,
                                                gates_index=ar, has_silu=False, fused=True, out=moe) if L else moe
        with _lib.stage("loss"):
            loss, load = sg_load_loss(meta, score, E, dt, self.loss_coef, self.training, smooth_load)
        return MRNOutput(y, loss, load)

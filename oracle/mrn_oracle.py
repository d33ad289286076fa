"""CPU restatement of the reference's sparsely-gated ("MRN" / SGMoE) layer forward:
OrigSGMoEImpl in kernels/pytorch/mrn.py of meta-recsys/fast_moe (paths below are relative to the
reference repository).

TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared against; imported by tests/ only.
Parity status: PINNED - tests/golden/make_golden.py runs the unmodified reference class on seeded
inputs (group "mrn") and tests/test_oracle_golden.py holds these functions to the recorded outputs.

Differences from the FastMoELayer router (modules/fast_moe_module.py:93-105) that this file pins:
logits are L2-normalised per token before the softmax, the softmax runs over ALL experts and the
k largest probabilities are used as they are (no renormalisation), experts are ordered by a
stable descending sort, the tokens are normalised (layer / group norm) before routing and before
the experts, and a dense "shared" linear map of the un-normalised tokens is added to the result.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from . import moe_oracle as O


def normalise_tokens(x, group_norm: bool, num_groups: int, linear_dim: int, weight, bias, eps: float):
    """Layer norm over the feature dimension, or group norm of x viewed as [L, num_groups,
    linear_dim] (one weight / bias per group). OrigSGMoEImpl.forward, kernels/pytorch/mrn.py:301-318."""
    if group_norm:
        return F.group_norm(x.view(-1, num_groups, linear_dim), num_groups=num_groups, weight=weight, bias=bias,
                            eps=eps).view(x.shape[0], -1)
    return F.layer_norm(x, normalized_shape=(x.shape[-1],), weight=weight, bias=bias, eps=eps)


def cv_squared(v: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Squared coefficient of variation, var / (mean^2 + eps), zero for a single value.
    OrigSGMoEImpl._cv_squared, kernels/pytorch/mrn.py:186-189."""
    if v.shape[0] == 1:
        return torch.zeros(())
    v = v.float()
    return v.var() / (v.mean() ** 2 + eps)


def gating(x_norm, w_gate, k: int, train: bool, w_noise=None, noise=None, noise_eps: float = 1e-2,
           post_softmax: bool = False):
    """OrigSGMoEImpl._orig_noisy_gating, kernels/pytorch/mrn.py:221-277 (the noise tensor that the
    reference draws with randn_like is an argument here). Returns (dense gates [L, E], top-k
    indices [L, k] in descending-logit order with ties to the lower expert id, top-k gate values
    [L, k], loss before the coefficient)."""
    E = w_gate.shape[1]
    k_plus = min(k + 1, E)
    clean = x_norm @ w_gate
    noisy = w_noise is not None and train
    if noisy:
        stddev = F.softplus(x_norm @ w_noise) + noise_eps
        logits_raw = clean + noise * stddev
    else:
        logits_raw = clean
    logits = F.normalize(logits_raw, dim=1)
    ln = logits.float().numpy()
    order = np.argsort(-ln, axis=1, kind="stable")                 # stable descending sort
    sorted_logits = torch.from_numpy(np.take_along_axis(ln, order, axis=1))
    idx = torch.from_numpy(order[:, :k].astype(np.int64))
    if post_softmax and k > 1:
        top_k_gates = F.softmax(sorted_logits[:, :k], dim=1)
    else:
        top_k_gates = F.softmax(sorted_logits, dim=1)[:, :k]
    top_k_gates = top_k_gates.to(x_norm.dtype)
    gates = torch.zeros(logits.shape, dtype=top_k_gates.dtype).scatter(1, idx, top_k_gates)
    if not train:
        return gates, idx, top_k_gates, torch.zeros(())
    if k < E and noisy:
        # probability of each expert being in the top k under a fresh noise draw (:191-219)
        top = sorted_logits[:, :k_plus]
        thr_in = top[:, k:k + 1]
        thr_out = top[:, k - 1:k]
        normal = torch.distributions.normal.Normal(torch.tensor([0.0]), torch.tensor([1.0]), validate_args=False)
        is_in = logits_raw > thr_in
        prob = torch.where(is_in, normal.cdf((clean - thr_in) / stddev), normal.cdf((clean - thr_out) / stddev))
        load = prob.sum(0)
    else:
        load = (gates > 0).sum(0)
    loss = cv_squared(gates.sum(0)) + cv_squared(load)
    return gates, idx, top_k_gates, loss


def sg_moe_forward(x, norm_weight, norm_bias, norm_eps: float, w_gate, w_hidden, b_hidden, w_out, b_out,
                   output_weight, k: int, train: bool = False, loss_coef: float = 1e-2, group_norm: bool = False,
                   num_groups: int = 1, linear_dim: Optional[int] = None, w_noise=None, noise=None
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """OrigSGMoEImpl.forward, kernels/pytorch/mrn.py:289-333 with router_forward (:279-287):
    x [L, d]; w_hidden [E, m, d], w_out [E, o, m] (F.linear layout), w_gate [d, E],
    output_weight [d, o]. Returns (y [L, o], loss, load fractions [E])."""
    linear_dim = linear_dim or x.shape[-1] // num_groups
    x_norm = normalise_tokens(x, group_norm, num_groups, linear_dim, norm_weight, norm_bias, norm_eps).to(x.dtype)
    gates, idx, top_k_gates, loss = gating(x_norm, w_gate, k, train, w_noise, noise)
    loss = loss * loss_coef
    # dispatch / experts / combine: the expert MLP of FastMoELayer on the normalised tokens, rows in
    # ascending expert order, gate-weighted sum per token in fp32 (OrigDispatcherImpl, :50-90)
    E = w_gate.shape[1]
    dense_for_sort = torch.zeros(x.shape[0], E).scatter(1, idx, 1.0)
    gate_index, token_index, _, offsets, reverse, _ = O.routing_metadata(dense_for_sort, idx)
    hidden = O.index_select_jagged_bmm(offsets, gate_index.view(-1, k), x_norm, w_hidden.permute(0, 2, 1), b_hidden)
    moe = O.silu_jagged_bmm_combine(offsets, hidden, w_out.permute(0, 2, 1), b_out, token_index, k, top_k_gates,
                                    gate_index, has_silu=True)
    y = torch.addmm(moe, x, output_weight)
    load = (gates > 0).sum(0) / (gates > 0).sum()
    return y, loss, load

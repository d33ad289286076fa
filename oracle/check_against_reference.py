"""Runs the CPU oracle side by side with the UNMODIFIED reference (imported through
oracle/reference_shims.py) on fresh seeded inputs and reports the largest difference per function.
TEST INFRASTRUCTURE ONLY; needs a checkout of the reference (its path in the environment variable
FAST_MOE_REFERENCE). The committed fixtures under tests/golden/ are the portable record of the
same comparison.

    python oracle/check_against_reference.py
"""
from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oracle import moe_oracle as O  # noqa: E402
from oracle import reference_shims  # noqa: E402


def main() -> int:
    ref = reference_shims.modules()
    KT = ref.utils.KernelType
    torch.manual_seed(123)
    worst = {}

    def rec(name, a, b, exact=False):
        d = float((a.double() - b.double()).abs().max()) if a.numel() else 0.0
        worst[name] = max(worst.get(name, 0.0), d)
        if exact:
            assert torch.equal(a, b), name

    for (B, T, d, h, o, E, k) in [(4, 16, 16, 32, 16, 8, 2), (2, 40, 64, 96, 48, 4, 1), (3, 33, 32, 64, 32, 16, 4)]:
        layer = ref.layer.FastMoELayer(d, h, o, E, KT.PYTORCH, torch.float32)
        with torch.no_grad():
            layer._experts_hidden_bias.normal_(0, 0.1)
            layer._experts_bias.normal_(0, 0.1)
        x = torch.randn(B, T, d)
        with torch.no_grad():
            scores, topk = layer._select_top_k_experts(x, k)
            gi, ti, gs, off, rev, msl = layer._compute_routing_metadata(x, scores, topk, k)
            y = layer(x, k)
        gw, gb = layer.gate.gate.weight.detach(), layer.gate.gate.bias.detach()
        dense, idx = O.select_top_k(O.gating_scores(x, gw, gb), k)
        rec("topk experts (as sets)", idx.sort(1).values, topk.view(-1, k).sort(1).values, exact=True)
        ogi, oti, ogs, ooff, orev, omsl = O.routing_metadata(dense, topk.view(-1, k))
        rec("gate_index", ogi, gi, exact=True)
        rec("token_index", oti, ti, exact=True)
        rec("offsets", ooff, off, exact=True)
        rec("reverse_index", orev, rev, exact=True)
        assert omsl == msl
        rec("gating_scores", ogs, gs)
        wh, bh = layer._experts_hidden_w.detach(), layer._experts_hidden_bias.detach()
        wo, bo = layer._experts_w.detach(), layer._experts_bias.detach()
        rec("FastMoELayer.forward", O.moe_layer_mlp(x, gw, gb, wh, bh, wo, bo, k), y)
        wu = torch.randn(E, d, h) * 0.05
        with torch.no_grad():
            fused = ref.pt_moe.pytorch_fused_jagged_bmm_swiglu_combine(
                off, gi.view(-1, k), x.view(-1, d), wh.permute(0, 2, 1), bh, wu, None, wo.permute(0, 2, 1), bo, k, gs, gi)
        mine = O.fused_jagged_bmm_swiglu_combine(off, gi.view(-1, k), x.view(-1, d), wh.permute(0, 2, 1), bh, wu, None,
                                                 wo.permute(0, 2, 1), bo, k, gs, gi)
        rec("fused_jagged_bmm_swiglu_combine", mine, fused)
    # FP8
    for dt in (torch.float32, torch.bfloat16):
        a = (torch.randn(64, 48) * 10 ** torch.randint(-3, 3, (64, 1)).float()).to(dt)
        q, s = ref.pt_quant.pytorch_rowwise_quant_fp8(a)
        oq, os_ = O.rowwise_quant_fp8(a)
        rec(f"rowwise_quant scale {dt}", os_, s, exact=True)
        rec(f"rowwise_quant payload {dt}", oq, q.view(torch.uint8), exact=True)
    for name, v in worst.items():
        print(f"{name:40s} max |diff| = {v:.3e}")
    bad = [n for n, v in worst.items() if v > 1e-5]
    print("OK" if not bad else f"MISMATCH: {bad}")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())

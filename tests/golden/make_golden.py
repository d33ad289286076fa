"""Generates the golden fixtures in this directory by running the UNMODIFIED reference
(meta-recsys/fast_moe, KernelType.PYTORCH, CPU) on seeded inputs.

    python tests/golden/make_golden.py [--reference /path/to/fast_moe]

The reference ships no fixture files (all its expectations are computed at test time), so these
vectors are the pinned record of what its code returns: inputs and outputs are stored together,
and tests compare both the CPU oracle (oracle/moe_oracle.py) and the CUDA kernels against them.
bfloat16 tensors are stored as uint16 bit patterns under a "::bf16" key suffix, float8 tensors
as uint8 under "::e4m3".
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import reference_shims  # noqa: E402


def pack(d):
    out = {}
    for k, v in d.items():
        if isinstance(v, torch.Tensor):
            v = v.detach()
            if v.dtype == torch.bfloat16:
                out[k + "::bf16"] = v.contiguous().view(torch.int16).numpy().view(np.uint16)
            elif v.dtype == torch.float8_e4m3fn:
                out[k + "::e4m3"] = v.contiguous().view(torch.uint8).numpy()
            else:
                out[k] = v.contiguous().numpy()
        else:
            out[k] = np.asarray(v)
    return out


def save(name, d):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **pack(d))
    print(f"{name}.npz  {os.path.getsize(path) / 1024:.1f} KiB")


def routing_case(ref, L, E, k, seed):
    """Routing tensors the way the reference's operator tests build them
    (kernels/tests/moe_test.py:191-197, :241)."""
    g = torch.Generator().manual_seed(seed)
    idx = torch.randn(L, E, generator=g).topk(k, dim=1).indices
    flat = idx.reshape(-1)
    _, gate_index = flat.sort(stable=True)
    lengths = torch.zeros(E, dtype=torch.int64).scatter_add_(0, flat, torch.ones_like(flat))
    offsets = torch.ops.fbgemm.asynchronous_complete_cumsum(lengths)
    token_index = gate_index // k
    reverse = token_index.sort(stable=True)[1].view(L, k)
    return idx, gate_index, token_index, offsets, reverse


def layer_cases(ref):
    KT = ref.utils.KernelType
    cases = [
        # (B, T, d, h, o, E, k, seed)
        (4, 8, 16, 32, 16, 4, 1, 1),
        (4, 16, 16, 32, 32, 8, 2, 2),
        (2, 48, 64, 128, 64, 8, 2, 3),
        (2, 33, 32, 48, 40, 16, 4, 4),
    ]
    for ci, (B, T, d, h, o, E, k, seed) in enumerate(cases):
        torch.manual_seed(seed)
        layer = ref.layer.FastMoELayer(d, h, o, E, KT.PYTORCH, torch.float32)
        with torch.no_grad():
            layer._experts_hidden_bias.normal_(0, 0.1)
            layer._experts_bias.normal_(0, 0.1)
        x = torch.randn(B, T, d)
        with torch.no_grad():
            scores, topk = layer._select_top_k_experts(x, k)
            gi, ti, gs, off, rev, msl = layer._compute_routing_metadata(x, scores, topk, k)
            y = layer(x, k)
            logits = layer.gate.gate(x)
            # SwiGLU composition on the same routing: second weight drawn here
            w_up = torch.randn(E, d, h) * 0.05
            w_gate = layer._experts_hidden_w.permute(0, 2, 1)
            w_down = layer._experts_w.permute(0, 2, 1)
            hidden_sw = ref.moe.index_select_jagged_bmm_swiglu(
                msl, off, gi.view(-1, k), x.view(-1, d), w_gate, layer._experts_hidden_bias, w_up, None)
            y_sw = ref.moe.silu_jagged_bmm_combine(
                msl, off, hidden_sw, w_down, layer._experts_bias, ti, rev, gs, gi, has_silu=False)
            y_sw_fused = ref.pt_moe.pytorch_fused_jagged_bmm_swiglu_combine(
                off, gi.view(-1, k), x.view(-1, d), w_gate, layer._experts_hidden_bias, w_up, None, w_down,
                layer._experts_bias, k, gs, gi)
        assert torch.allclose(y_sw, y_sw_fused, atol=1e-6), "reference SwiGLU composition != fused reference"
        save(f"layer_{ci}", dict(
            k=k, x=x, gate_w=layer.gate.gate.weight, gate_b=layer.gate.gate.bias,
            w_hidden=layer._experts_hidden_w, b_hidden=layer._experts_hidden_bias,
            w_out=layer._experts_w, b_out=layer._experts_bias, w_up=w_up,
            logits=logits, dense_scores=scores.view(-1, E), topk_idx=topk.view(-1, k),
            gate_index=gi, token_index=ti, gating_scores=gs, offsets=off, reverse_index=rev, max_seq_len=msl,
            y_mlp=y, hidden_swiglu=hidden_sw, y_swiglu=y_sw,
        ))


def op_cases(ref):
    cases = [
        # (L, E, k, K, N, dtype, kmajor, bias, seed)
        (16, 4, 2, 12, 32, torch.float32, False, True, 10),
        (100, 8, 4, 64, 72, torch.float32, True, False, 11),
        (300, 16, 2, 32, 64, torch.bfloat16, True, True, 12),
        (32, 4, 2, 64, 32, torch.bfloat16, False, True, 13),
        (150, 64, 8, 64, 40, torch.bfloat16, True, True, 14),   # E > rows of some experts: empty segments
    ]
    for ci, (L, E, k, K, N, dtype, kmajor, use_bias, seed) in enumerate(cases):
        torch.manual_seed(seed)
        idx, gi, ti, off, rev = routing_case(ref, L, E, k, seed)

        def mkw(rows, cols):
            # logical [E, rows, cols]; "kmajor" stores [E, cols, rows] and hands out the permuted view
            if kmajor:
                return torch.empty(E, cols, rows).uniform_(-1, 1).to(dtype).permute(0, 2, 1)
            return torch.empty(E, rows, cols).uniform_(-1, 1).to(dtype)

        x = torch.empty(L, K).uniform_(-1, 1).to(dtype)
        x2 = torch.empty(L, K).uniform_(-1, 1).to(dtype)
        w, wp = mkw(K, N), mkw(K, N)
        b = torch.empty(E, N).uniform_(-1, 1).to(dtype) if use_bias else None
        bp = torch.empty(E, N).uniform_(-1, 1).to(dtype) if use_bias else None
        w2 = mkw(N, K)
        b2 = torch.empty(E, K).uniform_(-1, 1).to(dtype) if use_bias else None
        gates = torch.rand(L, k).to(dtype)
        f32 = lambda t: None if t is None else t.float()
        index = gi.view(-1, k)
        msl = int((off[1:] - off[:-1]).max())
        # the reference's tests run the PYTORCH kernel on fp32 copies (kernels/utils.py:28-33)
        up = ref.moe.index_select_jagged_bmm(msl, off, index, f32(x), f32(w), f32(b))
        sw = ref.moe.index_select_jagged_bmm_swiglu(msl, off, index, f32(x), f32(w), f32(b), f32(wp), f32(bp))
        gt = ref.moe.index_select_jagged_gating_bmm(msl, off, index, f32(x), f32(x2), f32(w), f32(b), f32(wp), f32(bp))
        hid = torch.empty(L * k, N).uniform_(-1, 1).to(dtype)
        dn_silu = ref.moe.silu_jagged_bmm_combine(msl, off, f32(hid), f32(w2), f32(b2), ti, rev, f32(gates), gi, has_silu=True)
        dn_lin = ref.moe.silu_jagged_bmm_combine(msl, off, f32(hid), f32(w2), f32(b2), ti, rev, f32(gates), gi, has_silu=False)
        d = dict(k=k, E=E, kmajor=int(kmajor), x=x, x2=x2, w=w.contiguous() if not kmajor else w.permute(0, 2, 1).contiguous(),
                 wp=wp.contiguous() if not kmajor else wp.permute(0, 2, 1).contiguous(),
                 w2=w2.contiguous() if not kmajor else w2.permute(0, 2, 1).contiguous(),
                 hid=hid, gates=gates, topk_idx=idx, gate_index=gi, token_index=ti, offsets=off, reverse_index=rev,
                 up=up, swiglu=sw, gating=gt, down_silu=dn_silu, down_lin=dn_lin)
        if use_bias:
            d.update(b=b, bp=bp, b2=b2)
        save(f"ops_{ci}", d)


def combine_cases(ref):
    """mul_merge_k_add with strided gate weights and a random weight_index, as in
    kernels/tests/moe_test.py:326-400; outputs in the operand dtype (bit-exact target)."""
    for ci, (N, K, D, dtype, seed) in enumerate([
        (2, 4, 128, torch.float32, 20), (33, 16, 256, torch.bfloat16, 21), (100, 4, 128, torch.bfloat16, 22),
        (200, 2, 72, torch.float32, 23),
    ]):
        torch.manual_seed(seed)
        value = torch.empty(N * K, D).uniform_(-1, 1).to(dtype)
        w_full = torch.empty(N, K * 2).uniform_(-1, 1).to(dtype)
        w = w_full[:, :K]
        w_index = torch.randperm(w.numel())
        perm = torch.randperm(N * K)
        o2i = torch.arange(N).repeat(K).view(-1)[perm]
        i2o = o2i.sort(stable=True)[1].view(-1, K)
        out = ref.moe.mul_merge_k_add(index=o2i, reverse_index=i2o, value=value, weight=w, weight_index=w_index)
        out_now = ref.moe.mul_merge_k_add(index=o2i, reverse_index=i2o, value=value)
        save(f"combine_{ci}", dict(K=K, value=value, w_full=w_full, w_index=w_index, index=o2i, reverse_index=i2o,
                                   out=out, out_noweight=out_now))


def fp8_cases(ref):
    q = ref.pt_quant
    # 1. scale rule on every finite positive bf16 amax, and on fp32 values around the 448 / 2^k edges
    bits = torch.arange(0, 0x7F80, dtype=torch.int32).to(torch.int16)
    amax_bf16 = bits.view(torch.bfloat16)
    scale_bf16 = q.calculate_scale(amax_bf16)
    edge = []
    for e in range(-20, 21):
        c = 448.0 / 2.0**e
        edge += [np.nextafter(np.float32(c), np.float32(0)), np.float32(c), np.nextafter(np.float32(c), np.float32(1e30))]
    amax_f32 = torch.tensor(np.array(edge + [0.0, 1e-45, 1e-38, 3e38, np.inf, np.nan, 1.0, 3.0, 1e-30], dtype=np.float32))
    scale_f32 = q.calculate_scale(amax_f32)
    # 2. the cast itself: every e4m3 value, every midpoint between neighbours, and their fp32 neighbours
    vals = torch.arange(0, 256, dtype=torch.int32).to(torch.uint8).view(torch.float8_e4m3fn).float()
    finite = vals[~vals.isnan()].unique().numpy().astype(np.float64)
    pts = [finite]
    mids = (finite[1:] + finite[:-1]) / 2
    for arr in (finite, mids):
        a32 = arr.astype(np.float32)
        pts += [a32, np.nextafter(a32, np.float32(-1e30)), np.nextafter(a32, np.float32(1e30))]
    extra = np.array([449, 463.9, 464, 464.1, 479.9, 480, 1e9, np.inf, -np.inf, np.nan, 1e-12, -1e-12, 2**-10, 2**-9 * 0.5,
                      -464, -465], dtype=np.float32)
    cast_in = torch.tensor(np.unique(np.concatenate([np.asarray(p, dtype=np.float32) for p in pts] + [extra])))
    cast_in = torch.cat([cast_in, torch.tensor([float("nan")])])
    cast_out = cast_in.to(torch.float8_e4m3fn)
    d = dict(amax_bf16=amax_bf16, scale_bf16=scale_bf16, amax_f32=amax_f32, scale_f32=scale_f32, cast_in=cast_in,
             cast_out=cast_out)
    # 3. rowwise quant on the shapes of kernels/tests/quant_fp8_test.py:22-83
    torch.manual_seed(30)
    for si, shape in enumerate([(32, 16), (32, 8, 16), (7, 9, 13), (51, 5), (64, 1100)]):
        for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            a = (torch.randn(*shape) * (10.0 ** torch.randint(-3, 3, shape[:-1] + (1,)).float())).to(dt)
            if si == 0:
                a[3] = 0          # all-zero row -> scale 2^127
                a[5, 2] = 1e30 if dt == torch.float32 else 3e38
            aq, s = q.pytorch_rowwise_quant_fp8(a)
            d[f"rq{si}_{tag}_in"] = a
            d[f"rq{si}_{tag}_q"] = aq
            d[f"rq{si}_{tag}_scale"] = s
            if len(shape) >= 2:
                tq, ts = q.pytorch_transpose_rowwise_quant_fp8(a)
                d[f"rq{si}_{tag}_tq"] = tq
                d[f"rq{si}_{tag}_tscale"] = ts
    # 4. silu + quant, weight column quant (kernels/tests/moe_fp8_test.py:27-193)
    for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        j = (torch.randn(70, 64) * 3).to(dt)
        d[f"sj_{tag}_in"] = j
        d[f"sj_{tag}_q"] = ref.moe_fp8.silu_jagged_fp8(None, j, 0, 64, None, None, None)
        w = torch.randn(4, 32, 48).to(dt)
        d[f"wq_{tag}_in"] = w
        d[f"wq_{tag}_q"] = ref.moe_fp8.bmm_weight_rowwise_quant_fp8(w)
    save("fp8_quant", d)
    # 5. fp8 up projection (kernels/tests/moe_fp8_test.py:337-370)
    for ci, (L, E, k, K, N, seed) in enumerate([(100, 8, 2, 64, 32, 40), (300, 4, 4, 128, 16, 41), (64, 16, 2, 32, 32, 42)]):
        torch.manual_seed(seed)
        idx, gi, ti, off, rev = routing_case(ref, L, E, k, seed)
        x = torch.empty(L, K).uniform_(-1, 1).bfloat16()
        w = torch.empty(E, N, K).uniform_(-1, 1).bfloat16().permute(0, 2, 1)
        b = torch.empty(E, N).uniform_(-1, 1).bfloat16()
        out = ref.moe_fp8.index_select_jagged_bmm(0, off, gi.view(-1, k), x, w, b, fp8=True)
        raw = ref.moe_fp8.index_select_jagged_bmm(0, off, gi.view(-1, k), x.float(), w.float(), b.float(), fp8=False)
        save(f"fp8_bmm_{ci}", dict(k=k, x=x, w=w.permute(0, 2, 1).contiguous(), b=b, gate_index=gi, offsets=off,
                                   out=out, out_unquantised=raw))


def op3d_cases(ref):
    """index_select_jagged_bmm_3D (kernels/moe.py:118-153): jagged is [L, E, K], the rows of expert
    e read slice e of their token."""
    cases = [
        # (L, E, k, K, N, dtype, kmajor, bias, seed)
        (24, 4, 2, 16, 32, torch.float32, False, True, 30),
        (200, 8, 2, 64, 48, torch.bfloat16, True, True, 31),
        (90, 16, 4, 32, 24, torch.bfloat16, True, False, 32),    # some experts empty
    ]
    for ci, (L, E, k, K, N, dtype, kmajor, use_bias, seed) in enumerate(cases):
        torch.manual_seed(seed)
        idx, gi, ti, off, rev = routing_case(ref, L, E, k, seed)
        x = torch.empty(L, E, K).uniform_(-1, 1).to(dtype)
        if kmajor:
            w = torch.empty(E, N, K).uniform_(-1, 1).to(dtype).permute(0, 2, 1)
        else:
            w = torch.empty(E, K, N).uniform_(-1, 1).to(dtype)
        b = torch.empty(E, N).uniform_(-1, 1).to(dtype) if use_bias else None
        f32 = lambda t: None if t is None else t.float()
        msl = int((off[1:] - off[:-1]).max())
        out = ref.moe.index_select_jagged_bmm_3D(msl, off, gi.view(-1, k), f32(x), f32(w), f32(b))
        d = dict(k=k, E=E, kmajor=int(kmajor), x=x, w=w.contiguous() if not kmajor else w.permute(0, 2, 1).contiguous(),
                 topk_idx=idx, gate_index=gi, offsets=off, out=out)
        if use_bias:
            d.update(b=b)
        save(f"ops3d_{ci}", d)


def mrn_cases(ref):
    """The sparsely-gated layer of kernels/pytorch/mrn.py (OrigSGMoEImpl.forward): token norm,
    L2-normalised logits, softmax over all experts, top-k without renormalisation, MLP experts,
    shared linear map, load fractions and the training loss. Shapes follow
    kernels/tests/mrn_test.py:660-862 (d = model_d = 64, E in {4, 8}, k in {1, 2}) plus a group-norm
    case, a k = E case and one with noisy gating (the noise the reference draws is recorded)."""
    import importlib

    mrn = importlib.import_module("fast_moe.kernels.pytorch.mrn")
    cases = [
        # (L, d, m, o, E, k, group_norm, groups, train, noisy, seed)
        (50, 64, 64, 64, 4, 1, False, 1, False, False, 0),
        (477, 64, 64, 64, 8, 2, False, 1, True, False, 1),
        (60, 32, 48, 32, 8, 2, True, 2, True, False, 2),
        (40, 32, 32, 32, 4, 2, False, 1, True, True, 3),
        (33, 16, 24, 16, 8, 8, False, 1, True, False, 4),
    ]
    for ci, (L, d, m, o, E, k, gn, groups, train, noisy, seed) in enumerate(cases):
        torch.manual_seed(seed)
        cfg = mrn.SGConfig(model_d=m, num_experts=E, num_activated_experts=k, enable_noisy_gating=noisy)
        layer = mrn.OrigSGMoEImpl(d, o, cfg)
        with torch.no_grad():
            layer._experts_hidden_bias.normal_(0, 0.1)
            layer._experts_bias.normal_(0, 0.1)
            if noisy:
                layer._w_gate.normal_(0, 0.3)
                layer._w_noise.normal_(0, 0.3)
        layer.train(train)
        x = torch.randn(L, d)
        ns = groups if gn else d
        nw = torch.randn(ns) * 0.2 + 1
        nb = torch.randn(ns) * 0.1
        torch.manual_seed(100 + seed)
        noise = torch.randn(L, E) if (noisy and train) else None
        torch.manual_seed(100 + seed)          # the layer's randn_like draws the recorded noise
        with torch.no_grad():
            out = layer(x, None, 0, gn, groups, d // groups, nw, nb, 1e-5)
            x_norm = (torch.nn.functional.group_norm(x.view(-1, groups, d // groups), groups, nw, nb, 1e-5).view(L, d)
                      if gn else torch.nn.functional.layer_norm(x, (d,), nw, nb, 1e-5))
            gates, _ = layer._orig_noisy_gating(x_norm, train) if not noisy else (None, None)
        rec = dict(k=k, group_norm=int(gn), num_groups=groups, train=int(train), loss_coef=cfg.loss_coef, norm_eps=1e-5,
                   x=x, norm_weight=nw, norm_bias=nb, x_norm=x_norm, w_gate=layer._w_gate, w_hidden=layer._experts_hidden_w,
                   b_hidden=layer._experts_hidden_bias, w_out=layer._experts_w, b_out=layer._experts_bias,
                   output_weight=layer._output_weight, y=out.x, loss=out.loss.reshape(-1), load=out.load)
        if gates is not None:
            rec["gates"] = gates
        if noisy:
            rec.update(w_noise=layer._w_noise, noise=noise)
        save(f"mrn_{ci}", rec)


def grad_cases(ref):
    """Gradients of the operators: torch autograd through the reference's PYTORCH functions on CPU
    in fp32 (what its own tests use as the reference for the Triton backward,
    kernels/tests/moe_test.py:35-129, :299-400, :729-949, :951-1133), with the same generators:
    U(-1, 1) data, dout = randn * 0.01."""
    cases = [
        # (L, E, k, D_in, D_hidden, D_out, bias, has_silu, seed)
        (100, 4, 2, 32, 64, 32, True, True, 40),
        (200, 8, 4, 32, 48, 40, True, False, 41),
        (37, 16, 2, 12, 32, 24, False, True, 42),       # K = 12 (padding), empty experts likely
        (130, 4, 2, 64, 128, 64, True, True, 43),
    ]
    for ci, (L, E, k, d, h, o, use_bias, has_silu, seed) in enumerate(cases):
        torch.manual_seed(seed)
        idx, gi, ti, off, rev = routing_case(ref, L, E, k, seed)
        msl = int((off[1:] - off[:-1]).max())
        u = lambda *shape: torch.empty(*shape).uniform_(-1, 1)
        x = u(L, d).requires_grad_()
        w1 = u(E, d, h).requires_grad_()
        w1p = u(E, d, h).requires_grad_()
        b1 = u(E, h).requires_grad_() if use_bias else None
        b1p = u(E, h).requires_grad_() if use_bias else None
        w2 = u(E, h, o).requires_grad_()
        b2 = u(E, o).requires_grad_() if use_bias else None
        gates = torch.rand(L, k).requires_grad_()
        rec = dict(k=k, E=E, has_silu=int(has_silu), topk_idx=idx, gate_index=gi, token_index=ti, offsets=off, reverse_index=rev,
                   x=x, w1=w1, w1p=w1p, w2=w2, gates=gates)
        if use_bias:
            rec.update(b1=b1, b1p=b1p, b2=b2)

        def grads(out, dout, named):
            ts = [t for _, t in named if t is not None]
            gs = torch.autograd.grad(out, ts, dout, allow_unused=False)
            return {n: g for (n, t), g in zip([(n, t) for n, t in named if t is not None], gs)}

        # up projection
        up = ref.moe.index_select_jagged_bmm(msl, off, gi.view(-1, k), x, w1, b1)
        d_up = torch.randn_like(up) * 0.01
        for n, g in grads(up, d_up, [("x", x), ("w1", w1), ("b1", b1)]).items():
            rec["up_d_" + n] = g
        rec.update(up_out=up, up_dout=d_up)
        # SwiGLU up projection
        sw = ref.moe.index_select_jagged_bmm_swiglu(msl, off, gi.view(-1, k), x, w1, b1, w1p, b1p)
        d_sw = torch.randn_like(sw) * 0.01
        for n, g in grads(sw, d_sw, [("x", x), ("w1", w1), ("b1", b1), ("w1p", w1p), ("b1p", b1p)]).items():
            rec["sw_d_" + n] = g
        rec.update(sw_out=sw, sw_dout=d_sw)
        # down projection + combine on a fresh hidden tensor
        hid = u(L * k, h).requires_grad_()
        y = ref.moe.silu_jagged_bmm_combine(msl, off, hid, w2, b2, ti, rev, gates, gi, has_silu=has_silu)
        d_y = torch.randn_like(y) * 0.01
        for n, g in grads(y, d_y, [("hid", hid), ("w2", w2), ("b2", b2), ("gates", gates)]).items():
            rec["down_d_" + n] = g
        rec.update(hid=hid, down_out=y, down_dout=d_y)
        # combine alone
        val = u(L * k, o).requires_grad_()
        z = ref.moe.mul_merge_k_add(ti, rev, val, weight=gates, weight_index=gi)
        d_z = torch.randn_like(z) * 0.01
        for n, g in grads(z, d_z, [("val", val), ("gates", gates)]).items():
            rec["comb_d_" + n] = g
        rec.update(val=val, comb_out=z, comb_dout=d_z)
        save(f"grad_{ci}", rec)


def layer_grad_cases(ref):
    """Gradients through the whole reference layer (FastMoELayer, PYTORCH kernels, fp32, CPU):
    x, the gate Linear and the four expert parameters, for d(sum(y * dout))."""
    KT = ref.utils.KernelType
    for ci, (B, T, d, h, o, E, k, seed) in enumerate([(2, 24, 32, 64, 32, 4, 2, 50), (3, 17, 48, 40, 24, 8, 2, 51)]):
        torch.manual_seed(seed)
        layer = ref.layer.FastMoELayer(d, h, o, E, KT.PYTORCH, torch.float32)
        with torch.no_grad():
            layer._experts_hidden_bias.normal_(0, 0.1)
            layer._experts_bias.normal_(0, 0.1)
        x = torch.randn(B, T, d).requires_grad_()
        y = layer(x, k)
        dout = torch.randn_like(y) * 0.01
        y.backward(dout)
        sd = {n: p.detach().clone() for n, p in layer.state_dict().items()}
        rec = dict(k=k, x=x.detach(), y=y.detach(), dout=dout, d_x=x.grad)
        for n, p in layer.named_parameters():
            rec["p::" + n] = p.detach()
            rec["g::" + n] = p.grad
        save(f"lgrad_{ci}", rec)


NOISY_SEED = 31      # chosen like the others: no near tie of the k-th / (k+1)-th noisy gate in fp32 or bf16


def mrn_grad_cases(ref):
    """Gradients of the sparsely-gated layer: OrigSGMoEImpl (kernels/pytorch/mrn.py) in training
    mode on CPU in fp32, backward of sum(y * dout) + loss - what kernels/tests/mrn_test.py:816-860
    compares between its two implementations (x, every parameter, the norm's weight and bias),
    plus the training loss's own path into the router."""
    import importlib

    mrn = importlib.import_module("fast_moe.kernels.pytorch.mrn")
    cases = [
        # (L, d, m, o, E, k, group_norm, groups, seed)
        # seeds chosen so that no token's k-th and (k+1)-th gate probabilities come closer than
        # 5e-4, with the tokens in fp32 and rounded to bf16 alike: both dtypes route identically
        (96, 64, 64, 64, 8, 2, False, 1, 23, False),
        (70, 32, 48, 24, 4, 1, False, 1, 22, False),
        (64, 32, 40, 32, 8, 3, True, 2, 22, False),
        # noisy gating: the noise the reference draws is recorded; the loss then holds the smooth load
        (80, 32, 32, 32, 8, 2, False, 1, NOISY_SEED, True),
    ]
    for ci, (L, d, m, o, E, k, gn, groups, seed, noisy) in enumerate(cases):
        torch.manual_seed(seed)
        cfg = mrn.SGConfig(model_d=m, num_experts=E, num_activated_experts=k, loss_coef=0.5, enable_noisy_gating=noisy)
        layer = mrn.OrigSGMoEImpl(d, o, cfg)
        with torch.no_grad():
            layer._experts_hidden_bias.normal_(0, 0.1)
            layer._experts_bias.normal_(0, 0.1)
            if noisy:
                layer._w_gate.normal_(0, 0.3)
                layer._w_noise.normal_(0, 0.3)
        layer.train(True)
        x = torch.randn(L, d, requires_grad=True)
        ns = groups if gn else d
        nw = (torch.randn(ns) * 0.2 + 1).requires_grad_()
        nb = (torch.randn(ns) * 0.1).requires_grad_()
        torch.manual_seed(200 + seed)
        noise = torch.randn(L, E) if noisy else None
        torch.manual_seed(200 + seed)          # the layer's randn_like draws the recorded noise
        out = layer(x, None, 0, gn, groups, d // groups, nw, nb, 1e-5)
        dout = torch.randn_like(out.x) * 0.01
        ((out.x * dout).sum() + out.loss).backward()
        rec = dict(k=k, group_norm=int(gn), num_groups=groups, loss_coef=cfg.loss_coef, norm_eps=1e-5, x=x.detach(),
                   norm_weight=nw.detach(), norm_bias=nb.detach(), y=out.x.detach(), loss=out.loss.detach().reshape(-1),
                   dout=dout, d_x=x.grad, d_norm_weight=nw.grad, d_norm_bias=nb.grad)
        if noisy:
            rec["noise"] = noise
        for n, p_ in layer.named_parameters():
            rec["p::" + n] = p_.detach()
            rec["g::" + n] = p_.grad
        save(f"mgrad_{ci}", rec)


GROUPS = {"mgrad": mrn_grad_cases, "lgrad": layer_grad_cases, "grad": grad_cases, "layer": layer_cases, "ops": op_cases, "combine": combine_cases, "fp8": fp8_cases, "ops3d": op3d_cases,
          "mrn": mrn_cases}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None,
                    help="checkout of meta-recsys/fast_moe (default: the FAST_MOE_REFERENCE environment variable)")
    ap.add_argument("--only", default=None, choices=sorted(GROUPS), help="regenerate one group of fixtures")
    a = ap.parse_args()
    torch.set_num_threads(1)   # one thread: summation order of the CPU BLAS is then fixed
    ref = reference_shims.modules(a.reference)
    for name, fn in GROUPS.items():
        if a.only in (None, name):
            fn(ref)


if __name__ == "__main__":
    main()

"""Layer-level parity at the sizes and routing distributions of the benchmark configurations,
against the CPU oracle on the same seeded inputs, plus size-independent properties of the routing
tensors (permutation, sortedness, inverse relations) at full size.

Every benchmark configuration is checked at its real size: the GPU layer runs on the whole batch,
routing tensors are compared bit for bit on the whole batch, and outputs on a seeded sample of
tokens (the oracle then needs only those rows and the weights of the experts they use).

Bars: bf16 outputs rtol 1e-2 / atol 1e-2 (tokens whose k-th / (k+1)-th gate scores nearly tie may
route differently and are counted, not asserted); FP8: per-row scales exact, payload exact,
outputs within 4e-2 of the row maximum of the oracle's emulation of the same chain and within
6e-2 relative per quantised GEMM of the unquantised fp32 oracle."""
import pytest
import torch

import fast_moe_b200 as fm
from fast_moe_b200 import _lib
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cpu(p):
    return p.detach().float().cpu()


def _oracle_swiglu(layer, x, k):
    return O.moe_layer_swiglu(x.float().cpu(), _cpu(layer.gate.gate.weight), _cpu(layer.gate.gate.bias),
                              _cpu(layer.w_gate).permute(0, 2, 1), _cpu(layer.w_up).permute(0, 2, 1),
                              _cpu(layer.w_down).permute(0, 2, 1), k)


def _routing_properties(idx, meta, E, k):
    L = idx.shape[0]
    A = L * k
    gi, ti, off, rev = meta.gate_index, meta.token_index, meta.offsets, meta.reverse_index
    assert int(off[0]) == 0 and int(off[-1]) == A
    assert bool((off[1:] >= off[:-1]).all())
    # gate_index is a permutation of 0..A-1
    assert torch.equal(gi.sort().values, torch.arange(A, device=gi.device))
    # rows are grouped by expert, ascending; inside an expert ascending (token, slot): stable sort
    experts_sorted = idx.reshape(-1)[gi]
    assert bool((experts_sorted[1:] >= experts_sorted[:-1]).all())
    same = experts_sorted[1:] == experts_sorted[:-1]
    assert bool((gi[1:][same] > gi[:-1][same]).all())
    assert torch.equal(ti, gi // k)
    # histogram
    assert torch.equal(off[1:] - off[:-1], torch.bincount(idx.reshape(-1), minlength=E))
    # reverse_index lists each token's rows, ascending position
    assert torch.equal(ti[rev.reshape(-1)], torch.arange(L, device=gi.device).repeat_interleave(k))
    assert bool((rev[:, 1:] > rev[:, :-1]).all()) if k > 1 else True
    assert int(meta.max_len) == int((off[1:] - off[:-1]).max())


def test_c2_full_size_swiglu_layer_bf16():
    torch.manual_seed(0)
    B, T, d, h, o, E, k = 8, 512, 1024, 4096, 1024, 8, 2
    layer = fm.SwiGLUFastMoELayer(d, h, o, E, dtype=torch.bfloat16)
    with torch.no_grad():
        layer.gate.gate.weight.normal_(0, 0.02)
        layer.gate.gate.bias.zero_()
    layer.to(DEV)
    x = torch.randn(B, T, d).bfloat16()
    y = layer(x.to(DEV), k)
    assert _lib.device_status(torch.device(DEV)) == 0
    ref = _oracle_swiglu(layer, x, k)
    err = (y.float().cpu() - ref).abs()
    bad_tokens = (err > 1e-2 + 1e-2 * ref.abs()).view(-1, o).any(dim=1).float().mean().item()
    assert bad_tokens < 5e-3, f"{bad_tokens:.3%} of tokens outside tolerance"
    # routing at full size
    idx, score, _ = fm.gate_topk(x.view(-1, d).to(DEV), layer.gate.gate.weight, layer.gate.gate.bias, k)
    meta = fm.route_metadata(idx, E)
    _routing_properties(idx, meta, E, k)
    lengths = (meta.offsets[1:] - meta.offsets[:-1]).float()
    assert lengths.min() > 0.5 * lengths.mean(), "N(0, 0.02) gate should give roughly uniform loads"


def _bench():
    import bench

    return bench


def _assert_parity(par, score_tol=1e-5):
    assert par["routing"]["mismatched"] == 0, par["routing"]
    assert par["routing"]["metadata_bit_exact"], par["routing"]
    assert par["routing"]["max_score_diff"] < score_tol, par["routing"]
    assert par["sample"]["tokens"] >= 16, par["sample"]
    assert par["outputs"]["tokens_out_of_tolerance"] == 0, par["outputs"]
    assert par["ok"], par


def test_c4_true_size_zipf_routing_with_empty_experts():
    """The skewed-routing benchmark configuration at its real size: 8192 tokens, d=2048, h=8192,
    64 experts, top-8, router biased to a Zipf(1.2) load. Some experts get no tokens; the most
    loaded ones sit at the cap of one row per token (1/8 of the assignments - with top-8 an expert
    cannot receive more). Routing tensors bit exact on the whole batch; outputs of a seeded sample
    of tokens within rtol / atol 1e-2 of the fp32 oracle."""
    B = _bench()
    c = B.CONFIGS["c4"]
    L, d, E, k = c["tokens"], c["d"], c["E"], c["k"]
    layer = B.build_layer(c, torch.device(DEV))
    x = B.make_inputs(c, 0)
    idx, score, _ = fm.gate_topk(x.view(-1, d).to(DEV), layer.gate.gate.weight, layer.gate.gate.bias, k)
    meta = fm.route_metadata(idx, E)
    _routing_properties(idx, meta, E, k)
    lengths = meta.offsets[1:] - meta.offsets[:-1]
    assert int((lengths == 0).sum()) >= 1, "expected at least one empty expert"
    assert lengths.max().item() >= 0.10 * L * k, "the most loaded expert should be near the 1/8 cap"
    assert lengths[lengths > 0].min().item() < 0.01 * L * k, "expected a long tail of lightly loaded experts"
    y = layer(x.to(DEV), k)
    assert _lib.device_status(torch.device(DEV)) == 0
    par = B.parity_block(layer, c, x, y, B.layer_expert_weights(layer), layer.gate.gate, n_sample=256, max_experts=24)
    _assert_parity(par)
    # the lightly loaded experts too: tokens routed to the least loaded non-empty experts
    load = lengths.cpu()
    tail = torch.argsort(torch.where(load > 0, load, torch.full_like(load, 1 << 40)))[:6].tolist()
    top = torch.argsort(load, descending=True)[:18].tolist()
    from oracle import sampled as S

    idx_ref, _, _, _, _, _, gap = S.route_full(x.view(-1, d), layer.gate.gate.weight.detach().float().cpu(),
                                               layer.gate.gate.bias.detach().float().cpu(), k)
    allowed = set(tail + top)
    hits = [t for t in range(L) if set(idx_ref[t].tolist()) <= allowed and set(idx_ref[t].tolist()) & set(tail)
            and gap[t] > 1e-6][:24]
    if hits:
        sel = torch.tensor(hits)
        y_ref, _ = S.swiglu_layer_on_tokens(x.view(-1, d)[sel], layer.gate.gate.weight.detach().float().cpu(),
                                            layer.gate.gate.bias.detach().float().cpu(), k,
                                            B.layer_expert_weights(layer))
        got = S.compare_tokens(y.view(-1, c["o"])[sel.to(DEV)].float().cpu(), y_ref)
        assert got["tokens_out_of_tolerance"] == 0, got


def test_c3_true_size_fp8_layer_with_outlier_rows():
    """The FP8 benchmark configuration at its real size: 16384 tokens, d=4096, h=14336, 8 experts,
    top-2; x ~ N(0,1) with 1 % of the rows scaled by 50; weights e4m3 with per-row fp32 scales.
    Per-row scales exact on every token and every weight row, payload exact on samples; outputs of
    a seeded sample of tokens within 4e-2 (of the row's largest magnitude) of the oracle's
    quantise -> e4m3 product -> descale chain, and within 6e-2 relative per quantised GEMM of the
    unquantised fp32 oracle."""
    B = _bench()
    from fast_moe_b200.kernels import moe_fp8

    c = B.CONFIGS["c3"]
    d, k = c["d"], c["k"]
    layer = B.build_layer(c, torch.device(DEV))
    x = B.make_inputs(c, 0)
    xr = x.view(-1, d)
    xq, xs = moe_fp8.rowwise_quant_fp8(xr.to(DEV))
    # scales: every row, by the reference rule (torch ops on the host)
    assert torch.equal(xs.cpu(), O.calculate_scale(xr.abs().amax(dim=-1)))
    rows = torch.randperm(xr.shape[0], generator=torch.Generator().manual_seed(1))[:1024]
    oq, os_ = O.rowwise_quant_fp8(xr[rows])
    assert torch.equal(xq.cpu().view(torch.uint8)[rows], oq) and torch.equal(xs.cpu()[rows], os_)
    for name in ("w_gate", "w_up", "w_down"):
        wq, ws = layer._q[name]
        w = getattr(layer, name).detach()
        assert torch.equal(ws.cpu(), O.calculate_scale(w.abs().amax(dim=-1).cpu())), name
        oq, _ = O.rowwise_quant_fp8(w[3, 100:612].cpu())
        assert torch.equal(wq[3, 100:612].cpu().view(torch.uint8), oq), name
    y = layer(x.to(DEV), k)
    assert y.dtype == torch.bfloat16
    assert _lib.device_status(torch.device(DEV)) == 0
    par = B.parity_block(layer, c, x, y, B.layer_expert_weights(layer), layer.gate.gate, n_sample=256, max_experts=3)
    # the outlier rows carry logits 50 times larger than the rest, and an fp32 sum of 4096 products
    # taken in another order differs by about 1e-6 of the logit's size: the scores of those rows
    # agree to 1e-4 rather than 1e-5 (the expert choice itself is compared exactly)
    _assert_parity(par, score_tol=2e-4)
    assert par["outputs"]["rel_err_vs_fp32_median"] < 2 * 6e-2, par["outputs"]
    assert par["outputs"]["rel_err_vs_fp32_median"] <= par["outputs"]["fp8_oracle_rel_err_vs_fp32_median"] * 1.1 + 1e-3


def test_c5_dims_on_one_gpu_all_experts_local():
    """The per-rank workload of the expert-parallel benchmark with all 64 experts on this GPU:
    8192 tokens, d=4096, h=14336, top-2, bf16 (22.5 GB of weights)."""
    B = _bench()
    from fast_moe_b200.modules.expert_parallel import ExpertParallelSwiGLUMoE

    c = B.CONFIGS["c5"]
    dev = torch.device(DEV)
    layer = ExpertParallelSwiGLUMoE(c["d"], c["h"], c["o"], c["E"], dtype=torch.bfloat16, device=dev, world_size=1)
    # the rebuilt initial weights are the parameters themselves
    wg, wu, wd = layer.materialize_expert(37)
    assert torch.equal(wg, layer.w_gate[37]) and torch.equal(wu, layer.w_up[37]) and torch.equal(wd, layer.w_down[37])
    x = B.make_inputs(c, 0)
    y = layer(x.to(dev), c["k"])
    assert _lib.device_status(dev) == 0
    par = B.parity_block(layer, c, x, y, lambda e: tuple(t.cpu() for t in layer.materialize_expert(e)), layer.gate,
                         n_sample=256, max_experts=8)
    _assert_parity(par)
    del layer
    torch.cuda.empty_cache()


def test_mlp_layer_medium_size_matches_oracle():
    """FastMoELayer as shipped (fc1 + bias -> SiLU -> fc2 + bias) at a mid size, bf16."""
    torch.manual_seed(3)
    B, T, d, h, o, E, k = 4, 512, 512, 1024, 384, 8, 2
    layer = fm.FastMoELayer(d, h, o, E, dtype=torch.bfloat16)
    with torch.no_grad():
        layer._experts_hidden_bias.normal_(0, 0.1)
        layer._experts_bias.normal_(0, 0.1)
    layer.to(DEV)
    x = torch.randn(B, T, d).bfloat16()
    y = layer(x.to(DEV), k)
    ref = O.moe_layer_mlp(x.float(), _cpu(layer.gate.gate.weight), _cpu(layer.gate.gate.bias),
                          _cpu(layer._experts_hidden_w), _cpu(layer._experts_hidden_bias),
                          _cpu(layer._experts_w), _cpu(layer._experts_bias), k)
    err = (y.float().cpu() - ref).abs()
    bad_tokens = (err > 1e-2 + 1e-2 * ref.abs()).view(-1, o).any(dim=1).float().mean().item()
    assert bad_tokens < 5e-3, f"{bad_tokens:.3%} of tokens outside tolerance"
    assert _lib.device_status(torch.device(DEV)) == 0

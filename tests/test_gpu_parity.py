"""Parity of the CUDA path (through the C ABI) with the golden vectors recorded from the
reference and with the CPU oracle on seeded inputs.

Bars: routing indices, offsets, permutations, FP8 payload and scales, and the combine in its
operand type are bit exact; bf16 outputs rtol 1e-2 / atol 1e-2 against the fp32 reference on the
same bf16-rounded inputs; fp32 inputs run with tf32 tensor-core math and use the same bound.
"""
import numpy as np
import pytest
import torch

import fast_moe_b200 as fm
from fast_moe_b200 import _lib
from fast_moe_b200.kernels import moe, moe_fp8
from oracle import moe_oracle as O
from tests import golden_io as G

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = dict(rtol=1e-2, atol=1e-2)


def cu(t):
    return None if t is None else t.to(DEV)


def clean_status():
    assert _lib.device_status(torch.device(DEV)) == 0


# ------------------------------------------------------------------------------- routing
@pytest.mark.parametrize("name", G.names("layer_"))
def test_gate_topk_against_golden(name):
    g = G.load(name)
    k = g["k"]
    x = g["x"].reshape(-1, g["x"].shape[-1])
    idx, score, logits = fm.gate_topk(cu(x), cu(g["gate_w"]), cu(g["gate_b"]), k, return_logits=True)
    torch.testing.assert_close(logits.cpu(), g["logits"].reshape(logits.shape), atol=1e-5, rtol=1e-5)
    # expert choice bit exact as a set per token (slot order of torch.topk(sorted=False) is
    # implementation-defined); tokens whose k-th / (k+1)-th scores are closer than 1e-6 are
    # reported, not asserted
    dense = g["dense_scores"]
    full = torch.softmax(g["logits"].reshape(-1, dense.shape[1]), dim=1)
    srt = full.sort(dim=1, descending=True).values
    safe = torch.ones(full.shape[0], dtype=torch.bool) if k == full.shape[1] else (srt[:, k - 1] - srt[:, k]) > 1e-6
    got = idx.cpu().sort(dim=1).values
    want = g["topk_idx"].sort(dim=1).values
    assert torch.equal(got[safe], want[safe]), f"{(~safe).sum().item()} near-tie tokens excluded"
    # renormalised scores per (token, expert)
    got_dense = torch.zeros_like(dense).scatter_(1, idx.cpu(), score.cpu())
    torch.testing.assert_close(got_dense[safe], dense[safe], atol=1e-6, rtol=1e-5)
    # logits given directly: same routing
    idx2, score2, _ = fm.gate_topk(None, None, None, k, logits=logits)
    assert torch.equal(idx2, idx) and torch.equal(score2, score)
    clean_status()


@pytest.mark.parametrize("name", G.names("layer_") + G.names("ops_"))
def test_route_metadata_bit_exact_against_golden(name):
    g = G.load(name)
    E = g["gate_w"].shape[0] if "gate_w" in g else g["E"]
    m = fm.route_metadata(cu(g["topk_idx"]), E)
    assert torch.equal(m.gate_index.cpu(), g["gate_index"])
    assert torch.equal(m.token_index.cpu(), g["token_index"])
    assert torch.equal(m.offsets.cpu(), g["offsets"])
    assert torch.equal(m.reverse_index.cpu(), g["reverse_index"])
    lengths = g["offsets"][1:] - g["offsets"][:-1]
    assert torch.equal(m.lengths.cpu(), lengths)
    assert m.max_len.item() == lengths.max().item()
    clean_status()


@pytest.mark.parametrize("L,E,k,skew", [(1, 4, 1, 0.0), (255, 8, 2, 0.0), (257, 8, 8, 0.0), (1000, 64, 8, 3.0),
                                        (4096, 8, 2, 0.0), (8192, 64, 8, 2.0), (5000, 256, 4, 1.0), (0, 4, 2, 0.0),
                                        # either side of the single-block / three-pass switch
                                        (8192, 32, 4, 0.5), (8193, 8, 2, 0.0), (33, 300, 3, 0.0)])
def test_route_metadata_against_oracle(L, E, k, skew):
    g = torch.Generator().manual_seed(L * 131 + E)
    logits = torch.randn(L, E, generator=g) - skew * torch.arange(E).float().log1p()
    idx = logits.topk(k, dim=1).indices if L > 0 else torch.zeros(0, k, dtype=torch.int64)
    dense = torch.zeros(L, E).scatter_(1, idx, 1.0)
    gi, ti, _, off, rev, msl = O.routing_metadata(dense, idx)
    m = fm.route_metadata(cu(idx), E)
    assert torch.equal(m.offsets.cpu(), off)
    assert torch.equal(m.gate_index.cpu(), gi)
    assert torch.equal(m.token_index.cpu(), ti)
    assert torch.equal(m.reverse_index.cpu(), rev)
    assert m.max_len.item() == msl
    if skew >= 2.0:
        assert (m.lengths == 0).any(), "the skewed case is meant to leave some experts empty"
    clean_status()


def test_gate_topk_against_oracle_bf16():
    torch.manual_seed(5)
    L, d, E, k = 777, 512, 64, 8
    x = torch.randn(L, d).bfloat16()
    gw = (torch.randn(E, d) * 0.05)
    gb = torch.randn(E) * 0.1
    idx, score, logits = fm.gate_topk(cu(x), cu(gw), cu(gb), k, return_logits=True)
    ref_logits = torch.nn.functional.linear(x.float(), gw, gb)
    torch.testing.assert_close(logits.cpu(), ref_logits, atol=1e-4, rtol=1e-4)
    # shared logits -> identical choice, descending slots, ties to the lower id
    dense, oidx = O.select_top_k(torch.softmax(logits.cpu(), dim=1), k)
    srt = torch.softmax(logits.cpu(), dim=1).sort(dim=1, descending=True).values
    safe = (srt[:, :k] - srt[:, 1 : k + 1]).min(dim=1).values > 1e-7
    assert safe.float().mean() > 0.9
    assert torch.equal(idx.cpu()[safe], oidx[safe])
    torch.testing.assert_close(score.cpu()[safe], dense.gather(1, oidx)[safe], atol=1e-6, rtol=1e-5)
    clean_status()


@pytest.mark.parametrize("L,d,E,k", [(4096, 1024, 8, 2), (1000, 200, 8, 2), (77, 64, 5, 3), (513, 2048, 16, 4),
                                     (300, 512, 24, 8), (31, 8, 32, 1)])
def test_gate_topk_few_experts_warp_mma_path(L, d, E, k):
    """bf16 tokens with E <= 32 take the mma.sync kernel (three-term bf16 expansion of the fp32 gate
    weights): logits within fp32 rounding of the fp32 product, the same choice as the oracle away
    from near-ties, and bit-identical scores to the kernel that is handed those logits."""
    g = torch.Generator().manual_seed(L * 7 + E)
    x = torch.randn(L, d, generator=g).bfloat16()
    gw = torch.randn(E, d, generator=g) * 0.05
    gb = torch.randn(E, generator=g) * 0.1
    idx, score, logits = fm.gate_topk(cu(x), cu(gw), cu(gb), k, return_logits=True)
    ref_logits = torch.nn.functional.linear(x.double(), gw.double(), gb.double()).float()
    torch.testing.assert_close(logits.cpu(), ref_logits, atol=2e-6 * max(1.0, d ** 0.5 / 8), rtol=1e-5)
    dense, oidx = O.select_top_k(torch.softmax(logits.cpu(), dim=1), k)
    srt = torch.softmax(logits.cpu(), dim=1).sort(dim=1, descending=True).values
    safe = (srt[:, :k] - srt[:, 1 : k + 1]).min(dim=1).values > 1e-7 if k < E else torch.ones(L, dtype=torch.bool)
    assert torch.equal(idx.cpu()[safe], oidx[safe])
    torch.testing.assert_close(score.cpu()[safe], dense.gather(1, oidx)[safe], atol=1e-6, rtol=1e-5)
    idx2, score2, _ = fm.gate_topk(None, None, None, k, logits=logits)
    assert torch.equal(idx2, idx) and torch.equal(score2, score)
    # rows of a strided view (row stride > d)
    wide = torch.zeros(L, d + 8, dtype=torch.bfloat16)
    wide[:, :d] = x
    idx3, score3, _ = fm.gate_topk(cu(wide)[:, :d], cu(gw), cu(gb), k)
    assert torch.equal(idx3, idx) and torch.equal(score3, score)
    clean_status()


@pytest.mark.parametrize("L,d,E,k", [(1, 64, 4, 1), (15, 64, 8, 2), (16, 128, 8, 8), (17, 64, 5, 3), (33, 256, 16, 4),
                                     (1000, 200, 32, 8), (4096, 1024, 8, 2), (5000, 512, 32, 2)])
def test_fused_small_batch_routing_is_bit_identical(L, d, E, k):
    """gate kernel that also emits per-group counts + single-launch placement that also gathers
    the token rows and clears the combine buffer, against the separate operators: every tensor
    must be equal bit for bit."""
    from fast_moe_b200.kernels.routing import fused_routing_supported, route_tokens_fused

    g = torch.Generator().manual_seed(L * 7 + E)
    x = cu(torch.randn(L, d, generator=g).bfloat16())
    gw = cu(torch.randn(E, d, generator=g) * 0.3)
    gb = cu(torch.randn(E, generator=g) * 0.1)
    assert fused_routing_supported(x, gw)
    idx0, score0, _ = fm.gate_topk(x, gw, gb, k)
    meta0 = fm.route_metadata(idx0, E)
    rows0 = moe.gather_rows(x, meta0.gate_index, k)
    idx, score, meta, xs, zbuf = route_tokens_fused(x, gw, gb, k, gather_rows=True, zero_rows=(264, torch.bfloat16))
    assert torch.equal(idx, idx0) and torch.equal(score, score0)
    for name in ("gate_index", "token_index", "offsets", "reverse_index", "lengths", "max_len"):
        assert torch.equal(getattr(meta, name), getattr(meta0, name)), name
    assert torch.equal(xs, rows0)
    assert zbuf.shape == (L, 264) and int((zbuf != 0).sum()) == 0
    # without the optional passes
    _, _, meta2, xs2, z2 = route_tokens_fused(x, gw, None, k)
    assert xs2 is None and z2 is None
    idx1, _, _ = fm.gate_topk(x, gw, None, k)
    assert torch.equal(meta2.gate_index, fm.route_metadata(idx1, E).gate_index)
    clean_status()


def test_layers_with_and_without_fused_routing_agree_bitwise(monkeypatch):
    import fast_moe_b200.modules.fast_moe_module as M

    torch.manual_seed(4)
    d, h, o, E, k = 256, 1024, 256, 8, 2
    x = cu(torch.randn(3, 400, d).bfloat16())            # 1200 tokens: rows are gathered first
    for layer in (fm.SwiGLUFastMoELayer(d, h, o, E, dtype=torch.bfloat16).to(DEV),
                  fm.FastMoELayer(d, h, o, E, dtype=torch.bfloat16).to(DEV)):
        y_fused = layer(x, k)
        with monkeypatch.context() as mp:
            mp.setattr(M, "fused_routing_supported", lambda *a, **kw: False)
            y_plain = layer(x, k)
        assert torch.equal(y_fused, y_plain)
        y8 = layer(x[:, :40], k)                          # small batch: in-kernel gather, fused routing still on
        with monkeypatch.context() as mp:
            mp.setattr(M, "fused_routing_supported", lambda *a, **kw: False)
            assert torch.equal(y8, layer(x[:, :40], k))
    clean_status()


def test_gate_topk_tensor_core_logits_match_fp32_path():
    """bf16 hi/lo expansion of the gate weights on the tensor cores: logits agree with the fp32
    CUDA-core path to ~1e-5 and route identically wherever the k-th / (k+1)-th gap is not tiny."""
    from fast_moe_b200.kernels.routing import split_gate_weight

    torch.manual_seed(9)
    L, d, E, k = 3000, 1024, 64, 8
    x = torch.randn(L, d).bfloat16().to(DEV)
    gw = (torch.randn(E, d) * 0.05).to(DEV)
    gb = (torch.randn(E) * 0.1).to(DEV)
    idx0, sc0, lg0 = fm.gate_topk(x, gw, gb, k, return_logits=True)
    idx1, sc1, lg1 = fm.gate_topk(x, gw, gb, k, return_logits=True, gate_split=split_gate_weight(gw))
    torch.testing.assert_close(lg1, lg0, atol=2e-4, rtol=1e-4)
    srt = torch.softmax(lg0, dim=1).sort(dim=1, descending=True).values
    safe = (srt[:, :k] - srt[:, 1 : k + 1]).min(dim=1).values > 1e-5
    assert safe.float().mean() > 0.95
    assert torch.equal(idx0[safe], idx1[safe])
    torch.testing.assert_close(sc1[safe], sc0[safe], atol=1e-5, rtol=1e-3)
    clean_status()


# ------------------------------------------------------------------------------- operators
def _logical(g, key, dev=True):
    w = g[key]
    w = w.permute(0, 2, 1) if g["kmajor"] else w
    return cu(w) if dev else w


@pytest.mark.parametrize("name", G.names("ops_"))
def test_up_projection_operators_against_golden(name):
    g = G.load(name)
    k = g["k"]
    index = cu(g["gate_index"]).view(-1, k)
    off = cu(g["offsets"])
    x, x2 = cu(g["x"]), cu(g["x2"])
    w, wp = _logical(g, "w"), _logical(g, "wp")
    b, bp = cu(g.get("b")), cu(g.get("bp"))
    up = fm.index_select_jagged_bmm(0, off, index, x, w, b)
    assert up.dtype == x.dtype and up.shape == g["up"].shape
    torch.testing.assert_close(up.float().cpu(), g["up"], **TOL)
    sw = fm.index_select_jagged_bmm_swiglu(0, off, index, x, w, b, wp, bp)
    torch.testing.assert_close(sw.float().cpu(), g["swiglu"], rtol=2e-2, atol=2e-2)
    gt = fm.index_select_jagged_gating_bmm(0, off, index, x, x2, w, b, wp, bp)
    torch.testing.assert_close(gt.float().cpu(), g["gating"], rtol=2e-2, atol=2e-2)
    gt_same = fm.index_select_jagged_gating_bmm(0, off, index, x, x, w, b, wp, bp)
    assert torch.equal(gt_same, sw)
    clean_status()


@pytest.mark.parametrize("name", G.names("ops3d_"))
def test_index_select_jagged_bmm_3d_against_golden(name):
    """[L, E, K] input: rows of expert e read slice e of their token (kernels/moe.py:118-153)."""
    g = G.load(name)
    k = g["k"]
    x = cu(g["x"])
    out = fm.index_select_jagged_bmm_3D(0, cu(g["offsets"]), cu(g["gate_index"]).view(-1, k), x, _logical(g, "w"),
                                        cu(g.get("b")))
    assert out.dtype == x.dtype and out.shape == g["out"].shape
    torch.testing.assert_close(out.float().cpu(), g["out"], **TOL)
    # a non-contiguous [L, E, K] view gives the same rows
    wide = torch.zeros(x.shape[0], x.shape[1], x.shape[2] + 8, dtype=x.dtype, device=x.device)
    wide[..., : x.shape[2]] = x
    out2 = fm.index_select_jagged_bmm_3D(0, cu(g["offsets"]), cu(g["gate_index"]).view(-1, k), wide[..., : x.shape[2]],
                                         _logical(g, "w"), cu(g.get("b")))
    assert torch.equal(out2, out)
    clean_status()


@pytest.mark.parametrize("name", G.names("ops_"))
def test_down_projection_combine_against_golden(name):
    g = G.load(name)
    k = g["k"]
    off = cu(g["offsets"])
    w2 = _logical(g, "w2")
    for has_silu, key in ((True, "down_silu"), (False, "down_lin")):
        y = fm.silu_jagged_bmm_combine(0, off, cu(g["hid"]), w2, cu(g.get("b2")), cu(g["token_index"]),
                                       cu(g["reverse_index"]), cu(g["gates"]), cu(g["gate_index"]), has_silu=has_silu)
        assert y.dtype == g["hid"].dtype
        # The golden values are fp32. In bf16 the per-row GEMM result is rounded to bf16 before the
        # gate multiply, exactly as F.linear rounds it in the reference's bf16 run, so the absolute
        # error scales with the magnitude of those rows (U(-1,1) data): atol follows the tensor's scale.
        ref = g[key]
        torch.testing.assert_close(y.float().cpu(), ref, rtol=2e-2, atol=1e-2 * max(1.0, ref.abs().max().item()))
    clean_status()


@pytest.mark.parametrize("name", G.names("combine_"))
def test_mul_merge_k_add_bit_exact_against_golden(name):
    g = G.load(name)
    K = g["K"]
    w = cu(g["w_full"])[:, :K]          # strided gate weights, as the reference test passes them
    out = fm.mul_merge_k_add(cu(g["index"]), cu(g["reverse_index"]), cu(g["value"]), weight=w,
                             weight_index=cu(g["w_index"]))
    assert out.dtype == g["out"].dtype
    assert torch.equal(out.cpu(), g["out"])
    out2 = fm.mul_merge_k_add(cu(g["index"]), cu(g["reverse_index"]), cu(g["value"]))
    assert torch.equal(out2.cpu(), g["out_noweight"])
    clean_status()


# ------------------------------------------------------------------------------- FP8
def test_fp8_rowwise_quant_bit_exact_against_golden():
    g = G.load("fp8_quant")
    for si in range(5):
        for tag in ("f32", "bf16"):
            a = g[f"rq{si}_{tag}_in"]
            q, s = moe_fp8.rowwise_quant_fp8(cu(a))
            assert q.dtype == torch.float8_e4m3fn and q.shape == a.shape and s.shape == a.shape[:-1]
            assert torch.equal(s.cpu().view(torch.int32), g[f"rq{si}_{tag}_scale"].view(torch.int32)), (si, tag)
            assert torch.equal(q.cpu().view(torch.uint8), g[f"rq{si}_{tag}_q"]), (si, tag)
            tq, ts = moe_fp8.transpose_rowwise_quant_fp8(cu(a))
            assert torch.equal(ts.cpu(), g[f"rq{si}_{tag}_tscale"])
            assert torch.equal(tq.cpu().view(torch.uint8), g[f"rq{si}_{tag}_tq"])
            _, r = moe_fp8.rowwise_quant_fp8(cu(a), reciprocal_scale=True)
            torch.testing.assert_close(r.cpu(), 1.0 / g[f"rq{si}_{tag}_scale"], rtol=0, atol=0)
    clean_status()


def test_fp8_scale_rule_every_bf16_amax_and_cast_table():
    g = G.load("fp8_quant")
    # one row per bf16 amax value: the row is [amax, 0, 0, ...]
    amax = g["amax_bf16"]
    a = torch.zeros(amax.numel(), 16, dtype=torch.bfloat16)
    a[:, 3] = amax
    _, s = moe_fp8.rowwise_quant_fp8(cu(a))
    assert torch.equal(s.cpu().view(torch.int32), g["scale_bf16"].view(torch.int32))
    a32 = torch.zeros(g["amax_f32"].numel(), 8)
    a32[:, 1] = g["amax_f32"]
    _, s32 = moe_fp8.rowwise_quant_fp8(cu(a32))
    assert torch.equal(s32.cpu().view(torch.int32), g["scale_f32"].view(torch.int32))
    # the cast: a row whose amax is 448 has scale 1, so the payload is the cast of the input
    vals = g["cast_in"]
    ok = vals.abs() <= 448
    row = torch.cat([vals[ok], torch.tensor([448.0])])
    q, s1 = moe_fp8.rowwise_quant_fp8(cu(row.view(1, -1)))
    assert s1.item() == 1.0
    assert torch.equal(q.cpu().view(torch.uint8)[0, :-1], g["cast_out"][ok])
    clean_status()


def test_fp8_silu_and_weight_quant_against_golden():
    g = G.load("fp8_quant")
    for tag in ("f32", "bf16"):
        j = g[f"sj_{tag}_in"]
        q = moe_fp8.silu_jagged_fp8(None, cu(j), 0, j.shape[1], None, None, None)
        got, want = q.cpu().view(torch.uint8), g[f"sj_{tag}_q"]
        # SiLU uses the device exp: the payload may differ by one code where silu(x) sits on a
        # rounding boundary; everything else must match exactly
        diff = (got.to(torch.int16) - want.to(torch.int16)).abs()
        assert diff.max().item() <= 1 and (diff > 0).float().mean().item() < 2e-3
        w = g[f"wq_{tag}_in"]
        wq = moe_fp8.bmm_weight_rowwise_quant_fp8(cu(w))
        assert torch.equal(wq.cpu().view(torch.uint8), g[f"wq_{tag}_q"])
    clean_status()


@pytest.mark.parametrize("name", G.names("fp8_bmm_"))
def test_fp8_up_projection_against_golden(name):
    g = G.load(name)
    k = g["k"]
    w = cu(g["w"]).permute(0, 2, 1)
    out = moe_fp8.index_select_jagged_bmm(0, cu(g["offsets"]), cu(g["gate_index"]).view(-1, k), cu(g["x"]), w,
                                          cu(g["b"]), fp8=True)
    assert out.dtype == torch.bfloat16
    # bound of the reference's fp8-vs-emulation test (kernels/tests/moe_fp8_test.py:337-370)
    torch.testing.assert_close(out.float().cpu(), g["out"].float(), rtol=1e-2, atol=1e-2)
    # against the unquantised product: the reference's own bound for these small-K, U(-1,1) shapes
    # (kernels/tests/moe_fp8_test.py:302-335); the quantisation error must not exceed what the
    # reference's emulation itself shows on the same data
    ref = g["out_unquantised"]
    torch.testing.assert_close(out.float().cpu(), ref, rtol=1e-1, atol=4e-1)
    rel = (out.float().cpu() - ref).abs().amax(dim=1) / ref.abs().amax(dim=1).clamp_min(1e-6)
    rel_golden = (g["out"].float() - ref).abs().amax(dim=1) / ref.abs().amax(dim=1).clamp_min(1e-6)
    assert rel.max().item() <= rel_golden.max().item() * 1.1 + 1e-3
    clean_status()


@pytest.mark.parametrize("L,E,k,K,N,dt,bias,has_silu", [
    (300, 4, 2, 256, 192, torch.bfloat16, True, True),
    (64, 8, 1, 128, 64, torch.bfloat16, False, True),
    (500, 8, 4, 512, 320, torch.bfloat16, True, False),
    (200, 16, 2, 64, 128, torch.float32, True, True),
])
def test_fp8_down_projection_operators_against_oracle(L, E, k, K, N, dt, bias, has_silu):
    """moe_fp8.silu_jagged_bmm_fp8 and silu_jagged_bmm_combine_fp8 (kernels/moe_fp8.py:98-182)
    against the oracle's "quantise -> e4m3 product -> descale (-> combine)" chain built from the
    reference's quantisation rule and its one defined FP8 GEMM. The reference itself leaves these
    two operators unpinned (its PYTORCH branch returns the unquantised product and no test calls
    them), so the bars are the ones its FP8 up-projection test uses: rtol / atol 1e-2 against the
    emulation (kernels/tests/moe_fp8_test.py:337-370), and no further from the unquantised
    product than the emulation itself is."""
    g = torch.Generator().manual_seed(L + 31 * k + N)
    idx = torch.randn(L, E, generator=g).topk(k, dim=1).indices
    meta = fm.route_metadata(cu(idx), E)
    hid = (torch.rand(L * k, K, generator=g) * 2 - 1).to(dt)            # U(-1, 1), as the reference's tests
    w = ((torch.rand(E, K, N, generator=g) * 2 - 1) * 0.2).to(dt)       # logical [E, K, N], plain contiguous
    b = ((torch.rand(E, N, generator=g) * 2 - 1) * 0.1).to(dt) if bias else None
    score = torch.rand(L, k, generator=g).to(dt)
    off = meta.offsets.cpu()
    if has_silu:
        rows = moe_fp8.silu_jagged_bmm_fp8(meta.offsets, 0, cu(hid), cu(w), cu(b))
        want_rows = O.silu_jagged_bmm_fp8(off, hid, w, b, has_silu=True)
        raw = O.silu_jagged_bmm(off, hid.float(), w.float(), None if b is None else b.float(), has_silu=True)
        assert rows.dtype == dt and rows.shape == (L * k, N)
        scale = max(1.0, raw.abs().max().item())
        torch.testing.assert_close(rows.float().cpu(), want_rows.float(), rtol=1e-2, atol=1e-2 * scale)
        err = (rows.float().cpu() - raw).abs().amax(dim=1) / raw.abs().amax(dim=1).clamp_min(1e-6)
        err_emu = (want_rows.float() - raw).abs().amax(dim=1) / raw.abs().amax(dim=1).clamp_min(1e-6)
        assert err.max().item() <= err_emu.max().item() * 1.1 + 1e-2
    got = moe_fp8.silu_jagged_bmm_combine_fp8(0, meta.offsets, cu(hid), cu(w), cu(b), meta.token_index,
                                              meta.reverse_index, gating_scores=cu(score),
                                              gates_index=meta.gate_index, has_silu=has_silu)
    want = O.silu_jagged_bmm_combine_fp8(off, hid, w, b, meta.token_index.cpu(), k, score, meta.gate_index.cpu(),
                                         has_silu=has_silu)
    unq = O.silu_jagged_bmm_combine(off, hid.float(), w.float(), None if b is None else b.float(),
                                    meta.token_index.cpu(), k, score.float(), meta.gate_index.cpu(), has_silu=has_silu)
    assert got.dtype == dt and got.shape == (L, N)
    scale = max(1.0, unq.abs().max().item())
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=1e-2 * scale)
    # within the 6e-2 relative bound of one quantised GEMM against the unquantised operator
    rel = (got.float().cpu() - unq).norm(dim=1) / unq.norm(dim=1).clamp_min(1e-6)
    assert rel.quantile(0.99).item() < 6e-2, rel.quantile(0.99).item()
    clean_status()


# ------------------------------------------------------------------------------- layers
def _near_tie_mask(g):
    E = g["gate_w"].shape[0]
    k = g["k"]
    full = torch.softmax(g["logits"].reshape(-1, E), dim=1)
    if k == E:
        return torch.ones(full.shape[0], dtype=torch.bool)
    srt = full.sort(dim=1, descending=True).values
    return (srt[:, k - 1] - srt[:, k]) > 1e-6


@pytest.mark.parametrize("name", G.names("layer_"))
def test_layers_against_golden(name):
    g = G.load(name)
    k = g["k"]
    x = g["x"]
    B, T, d = x.shape
    E, h, _ = g["w_hidden"].shape
    o = g["w_out"].shape[1]
    layer = fm.FastMoELayer(d, h, o, E, fm.KernelType.PYTORCH, torch.float32)
    layer.load_state_dict({
        "gate.gate.weight": g["gate_w"], "gate.gate.bias": g["gate_b"], "_experts_hidden_w": g["w_hidden"],
        "_experts_hidden_bias": g["b_hidden"], "_experts_w": g["w_out"], "_experts_bias": g["b_out"]})
    layer.to(DEV)
    y = layer(cu(x), k)
    assert y.shape == (B, T, o)
    safe = _near_tie_mask(g)
    torch.testing.assert_close(y.cpu().view(-1, o)[safe], g["y_mlp"].view(-1, o)[safe], **TOL)
    # bf16 run of the same layer against the same fp32 reference output
    yb = layer.to(torch.bfloat16)(cu(x).bfloat16(), k)
    assert yb.dtype == torch.bfloat16
    ref_b = O.moe_layer_mlp(x.bfloat16().float(), g["gate_w"].bfloat16().float(), g["gate_b"].bfloat16().float(),
                            g["w_hidden"].bfloat16().float(), g["b_hidden"].bfloat16().float(),
                            g["w_out"].bfloat16().float(), g["b_out"].bfloat16().float(), k)
    bad = (yb.float().cpu().view(-1, o) - ref_b.view(-1, o)).abs() > (2e-2 + 2e-2 * ref_b.view(-1, o).abs())
    # bf16 gate logits can flip a near-tie: allow a few tokens to differ, none of the others
    assert bad.any(dim=1).float().mean().item() < 0.05
    # SwiGLU composition
    sw = fm.SwiGLUFastMoELayer(d, h, o, E, dtype=torch.float32)
    with torch.no_grad():
        sw.gate.gate.weight.copy_(g["gate_w"]); sw.gate.gate.bias.copy_(g["gate_b"])
        sw.w_gate.copy_(g["w_hidden"]); sw.w_up.copy_(g["w_up"].permute(0, 2, 1)); sw.w_down.copy_(g["w_out"])
    sw.to(DEV)
    ref = O.moe_layer_swiglu(x, g["gate_w"], g["gate_b"], g["w_hidden"].permute(0, 2, 1), g["w_up"],
                             g["w_out"].permute(0, 2, 1), k)
    ysw = sw(cu(x), k)
    torch.testing.assert_close(ysw.cpu().view(-1, o)[safe], ref.view(-1, o)[safe], **TOL)
    clean_status()


@pytest.mark.parametrize("name", G.names("layer_"))
def test_fp32_layers_at_the_reference_fp32_tolerance(name):
    """float32 tokens and weights with TF32 not allowed - the default of
    torch.backends.cuda.matmul.allow_tf32, which the reference's kernels follow
    (kernels/triton/triton_moe.py:592) - must hold the tolerance of the reference's own fp32
    end-to-end parity test, atol 1e-4 (modules/tests/test_kernel_parity.py:29-90). Operands are
    expanded into three bf16 terms and multiplied by one bf16 tensor-core GEMM over a six times
    longer reduction. With TF32 allowed the same call runs the tf32 kernels at the 1e-2 bound."""
    g = G.load(name)
    k = g["k"]
    x = g["x"]
    B, T, d = x.shape
    E, h, _ = g["w_hidden"].shape
    o = g["w_out"].shape[1]
    layer = fm.FastMoELayer(d, h, o, E, fm.KernelType.PYTORCH, torch.float32)
    layer.load_state_dict({
        "gate.gate.weight": g["gate_w"], "gate.gate.bias": g["gate_b"], "_experts_hidden_w": g["w_hidden"],
        "_experts_hidden_bias": g["b_hidden"], "_experts_w": g["w_out"], "_experts_bias": g["b_out"]})
    layer.to(DEV)
    sw = fm.SwiGLUFastMoELayer(d, h, o, E, dtype=torch.float32)
    with torch.no_grad():
        sw.gate.gate.weight.copy_(g["gate_w"]); sw.gate.gate.bias.copy_(g["gate_b"])
        sw.w_gate.copy_(g["w_hidden"]); sw.w_up.copy_(g["w_up"].permute(0, 2, 1)); sw.w_down.copy_(g["w_out"])
    sw.to(DEV)
    ref_sw = O.moe_layer_swiglu(x, g["gate_w"], g["gate_b"], g["w_hidden"].permute(0, 2, 1), g["w_up"],
                                g["w_out"].permute(0, 2, 1), k)
    safe = _near_tie_mask(g)
    assert torch.backends.cuda.matmul.allow_tf32 is False and not fm.fp32_uses_tf32()
    try:
        y = layer(cu(x), k)
        assert y.dtype == torch.float32
        torch.testing.assert_close(y.cpu().view(-1, o)[safe], g["y_mlp"].view(-1, o)[safe], rtol=1e-5, atol=1e-4)
        ysw = sw(cu(x), k)
        torch.testing.assert_close(ysw.cpu().view(-1, o)[safe], ref_sw.view(-1, o)[safe], rtol=1e-5, atol=1e-4)
        # the cached expansion follows in-place weight updates
        with torch.no_grad():
            layer._experts_w.mul_(0.5)
            layer._experts_bias.mul_(0.5)
        y_half = layer(cu(x), k)
        torch.testing.assert_close(y_half.cpu().view(-1, o)[safe], 0.5 * g["y_mlp"].view(-1, o)[safe], rtol=1e-5, atol=1e-4)
        # operators on float32 tensors take the same path
        off, gi = cu(g["offsets"]), cu(g["gate_index"])
        xf = cu(x.reshape(-1, d))
        w1 = cu(g["w_hidden"]).permute(0, 2, 1)
        up = fm.index_select_jagged_bmm(0, off, gi.view(-1, k), xf, w1, cu(g["b_hidden"]))
        want = O.index_select_jagged_bmm(g["offsets"], g["gate_index"].view(-1, k), x.reshape(-1, d),
                                         g["w_hidden"].permute(0, 2, 1), g["b_hidden"])
        torch.testing.assert_close(up.cpu(), want, rtol=1e-5, atol=1e-4)
        # TF32 allowed: the tf32 kernels, at their own bound; visibly less accurate than the above
        fm.set_fp32_matmul("tf32")
        assert fm.fp32_uses_tf32()
        with torch.no_grad():
            layer._experts_w.mul_(2.0)
            layer._experts_bias.mul_(2.0)
        y_tf32 = layer(cu(x), k)
        torch.testing.assert_close(y_tf32.cpu().view(-1, o)[safe], g["y_mlp"].view(-1, o)[safe], **TOL)
    finally:
        fm.set_fp32_matmul(None)
    clean_status()


@pytest.mark.parametrize("name", G.names("ops_"))
def test_fused_combine_epilogue_against_two_kernel_form(name):
    """silu_jagged_bmm_combine(fused=True): the GEMM epilogue scales by the gate weight and adds
    into the token rows. Same roundings as the two-kernel form; k <= 2 must match it bit for bit
    in bf16, larger k within one bf16 ulp of accumulation order."""
    g = G.load(name)
    k = g["k"]
    off = cu(g["offsets"])
    w2 = _logical(g, "w2")
    args = (0, off, cu(g["hid"]), w2, cu(g.get("b2")), cu(g["token_index"]), cu(g["reverse_index"]),
            cu(g["gates"]), cu(g["gate_index"]))
    for has_silu in (False, True):
        two = fm.silu_jagged_bmm_combine(*args, has_silu=has_silu)
        one = fm.silu_jagged_bmm_combine(*args, has_silu=has_silu, fused=True)
        assert one.dtype == two.dtype and one.shape == two.shape
        if k <= 2 and g["hid"].dtype == torch.bfloat16:
            assert torch.equal(one, two)
        else:
            scale = max(1.0, two.float().abs().max().item())
            torch.testing.assert_close(one.float(), two.float(), rtol=1e-2, atol=1e-2 * scale)
    clean_status()


@pytest.mark.parametrize("name", G.names("ops_"))
def test_fused_combine_flags_round_scores_and_accumulate(name):
    """round_scores=True with f32 scores equals casting the scores to the activation type first
    (the reference's gate runs in the layer's dtype, modules/fast_moe_module.py:21-27, so its scores arrive in that type), in both forms; out= adds the
    combined rows to what the buffer already holds (a residual) and returns that buffer."""
    g = G.load(name)
    k = g["k"]
    hid = cu(g["hid"])
    dt = hid.dtype
    off = cu(g["offsets"])
    w2 = _logical(g, "w2")
    gates32 = cu(g["gates"]).float() * 0.731 + 0.013       # values that do not survive a bf16 round trip
    common = (0, off, hid, w2, cu(g.get("b2")), cu(g["token_index"]), cu(g["reverse_index"]))
    idx = cu(g["gate_index"])
    for fused in (False, True):
        cast_first = fm.silu_jagged_bmm_combine(*common, gates32.to(dt), idx, has_silu=False, fused=fused)
        in_kernel = fm.silu_jagged_bmm_combine(*common, gates32, idx, has_silu=False, fused=fused, round_scores=True)
        assert in_kernel.dtype == dt
        if k <= 2 or not fused:
            assert torch.equal(in_kernel, cast_first)
        else:
            scale = max(1.0, cast_first.float().abs().max().item())
            torch.testing.assert_close(in_kernel.float(), cast_first.float(), rtol=1e-2, atol=1e-2 * scale)
    # accumulate into a residual
    base = fm.silu_jagged_bmm_combine(*common, gates32, idx, has_silu=False, fused=True, round_scores=True)
    resid = torch.randn_like(base.float()).to(dt)
    buf = resid.clone()
    got = fm.silu_jagged_bmm_combine(*common, gates32, idx, has_silu=False, fused=True, round_scores=True, out=buf)
    assert got.data_ptr() == buf.data_ptr()
    scale = max(1.0, base.float().abs().max().item())
    torch.testing.assert_close(got.float(), resid.float() + base.float(), rtol=1e-2, atol=1.6e-2 * scale)
    with pytest.raises(ValueError):
        fm.silu_jagged_bmm_combine(*common, gates32, idx, has_silu=False, fused=False, out=buf)
    with pytest.raises(ValueError):
        fm.silu_jagged_bmm_combine(*common, gates32, idx, has_silu=False, fused=True, round_scores=True,
                                   out=buf[:, :-1])
    clean_status()


@pytest.mark.parametrize("L,E,k,K,N", [(300, 4, 2, 256, 192), (64, 8, 1, 128, 64), (500, 8, 4, 512, 320)])
def test_fp8_down_projection_with_fused_combine(L, E, k, K, N):
    """e4m3 down projection with the combine in the epilogue against the two-kernel form on the
    same quantised operands: bit-identical for k <= 2, accumulation order only for larger k."""
    from fast_moe_b200.kernels import moe_fp8

    g = torch.Generator().manual_seed(L + 17 * k)
    logits = torch.randn(L, E, generator=g)
    idx = logits.topk(k, dim=1).indices
    meta = fm.route_metadata(cu(idx), E)
    hid = cu((torch.randn(L * k, K, generator=g) * 2).bfloat16())
    w = cu((torch.randn(E, N, K, generator=g) * 0.05).bfloat16())          # [E, N, K]: K contiguous
    bias = cu((torch.randn(E, N, generator=g) * 0.1).bfloat16())
    score = cu(torch.rand(L, k, generator=g))                               # f32, not bf16-representable
    hq, hs = moe_fp8.rowwise_quant_fp8(hid)
    wq, ws = moe_fp8.rowwise_quant_fp8(w)
    rows = moe_fp8.fp8_jagged_bmm_quantized(meta.offsets, hq, hs, wq, ws, bias, out_dtype=torch.bfloat16)
    two = fm.mul_merge_k_add(meta.token_index, meta.reverse_index, rows, weight=score.to(torch.bfloat16),
                             weight_index=meta.gate_index)
    one = moe_fp8.fp8_jagged_bmm_combine_quantized(meta.offsets, hq, hs, wq, ws, bias, score, meta.gate_index, L)
    assert one.shape == two.shape and one.dtype == two.dtype
    if k <= 2:
        assert torch.equal(one, two)
    else:
        scale = max(1.0, two.float().abs().max().item())
        torch.testing.assert_close(one.float(), two.float(), rtol=1e-2, atol=1e-2 * scale)
    clean_status()


@pytest.mark.parametrize("cols", [1032, 4096, 14336, 16384])
@pytest.mark.parametrize("apply_silu", [False, True])
def test_rowwise_quant_single_pass_kernel_matches_generic_kernel_and_oracle(cols, apply_silu):
    """Wide 16-byte-aligned bf16 rows take the register-resident single-pass kernel; a view that
    starts 2 bytes later takes the generic two-pass kernel. Payload and scales must be identical,
    and equal to the CPU oracle's."""
    from fast_moe_b200.kernels import moe_fp8

    g = torch.Generator().manual_seed(cols + int(apply_silu))
    rows = 37
    big = torch.randn(rows, cols + 8, generator=g) * torch.logspace(-3, 3, rows).view(-1, 1)
    big[3, 5] = float("nan")
    big[4] = 0.0
    big[5, 7] = float("inf")
    big = big.bfloat16()
    a = big[:, :cols].contiguous()
    fast_q, fast_s = moe_fp8.rowwise_quant_fp8(cu(a), apply_silu=apply_silu)
    # same values at an odd element offset: the generic kernel
    shifted = torch.empty(rows * cols + 1, dtype=torch.bfloat16, device=DEV)
    shifted[1:] = cu(a).view(-1)
    lib = _lib.load()
    q2 = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=DEV)
    s2 = torch.empty(rows, dtype=torch.float32, device=DEV)
    _lib.check(lib.fmoe_rowwise_quant_fp8(shifted.data_ptr() + 2, _lib.BF16, rows, cols, cols, int(apply_silu), 0,
                                          q2.data_ptr(), cols, s2.data_ptr(), None))
    torch.cuda.synchronize()
    assert torch.equal(fast_s.cpu().view(torch.int32), s2.cpu().view(torch.int32))
    assert torch.equal(fast_q.view(torch.uint8), q2.view(torch.uint8))
    if not apply_silu:
        oq, os_ = O.rowwise_quant_fp8(a[6:])        # the rows without NaN / inf / all-zero specials
        assert torch.equal(fast_s.cpu()[6:].view(torch.int32), os_.view(torch.int32))
        assert torch.equal(fast_q.cpu()[6:].view(torch.uint8), oq.view(torch.uint8))
    clean_status()


@pytest.mark.parametrize("L,k,D,dt,wdt", [(300, 2, 1024, torch.bfloat16, torch.bfloat16), (77, 8, 64, torch.bfloat16, torch.bfloat16),
                                          (513, 1, 8, torch.bfloat16, torch.float32), (40, 33, 256, torch.bfloat16, torch.bfloat16),
                                          (129, 4, 1000, torch.float32, torch.float32), (64, 3, 1001, torch.bfloat16, torch.bfloat16),
                                          (2000, 8, 2048, torch.bfloat16, torch.bfloat16)])
def test_mul_merge_k_add_both_kernels_bit_exact_against_oracle(L, k, D, dt, wdt):
    """Aligned rows with k <= 32 take the warp-per-token kernel, everything else the generic one
    (k = 33, D = 1001 here); both must reproduce the oracle's fp32 ascending-order sum bit for bit,
    with and without gate weights."""
    g = torch.Generator().manual_seed(L * 3 + k)
    E = max(k, 8)
    idx = torch.rand(L, E, generator=g).topk(k, dim=1).indices
    meta = fm.route_metadata(cu(idx), E)
    value = torch.randn(L * k, D, generator=g).to(dt)
    weight = torch.rand(L, k, generator=g).to(wdt)
    ti, gi = meta.token_index.cpu(), meta.gate_index.cpu()
    want = O.mul_merge_k_add(ti, value, k, weight, gi)
    got = fm.mul_merge_k_add(meta.token_index, meta.reverse_index, cu(value), weight=cu(weight), weight_index=meta.gate_index)
    assert got.dtype == want.dtype
    assert torch.equal(got.cpu(), want)
    want2 = O.mul_merge_k_add(ti, value, k)
    got2 = fm.mul_merge_k_add(meta.token_index, meta.reverse_index, cu(value))
    assert torch.equal(got2.cpu(), want2)
    clean_status()


@pytest.mark.parametrize("src_rows,rows,cols,dt,div", [(300, 1000, 256, torch.bfloat16, 1), (64, 500, 1000, torch.bfloat16, 2),
                                                       (100, 257, 64, torch.bfloat16, 1), (50, 99, 7, torch.float32, 3),
                                                       (128, 4096, 1024, torch.float32, 1), (77, 300, 4096, torch.float8_e4m3fn, 1)])
def test_gather_rows_all_kernel_forms(src_rows, rows, cols, dt, div):
    """Row gather: warp-per-row form (16-byte-aligned rows of 512 bytes or more), 16-byte piece
    form and byte form against torch indexing; an index outside the source is reported and its
    row reads as zeros."""
    g = torch.Generator().manual_seed(rows + cols)
    if dt == torch.float8_e4m3fn:
        src = torch.randint(0, 255, (src_rows, cols), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
    else:
        src = torch.randn(src_rows, cols, generator=g).to(dt)
    index = torch.randint(0, src_rows * div, (rows,), generator=g)
    as_bytes = lambda t: t.contiguous().view(torch.uint8)
    want = as_bytes(src)[index // div]
    got = fm.kernels.moe.gather_rows(cu(src), cu(index), div)
    assert got.dtype == src.dtype and tuple(got.shape) == (rows, cols)
    assert torch.equal(as_bytes(got.cpu()), want)
    clean_status()
    bad = index.clone()
    bad[3] = src_rows * div + 5
    got = as_bytes(fm.kernels.moe.gather_rows(cu(src), cu(bad), div).cpu())
    assert _lib.device_status(DEV) == 1
    assert int(got[3].count_nonzero()) == 0
    keep = torch.ones(rows, dtype=torch.bool)
    keep[3] = False
    assert torch.equal(got[keep], want[keep])
    clean_status()


@pytest.mark.parametrize("L,E,k,K,N", [(512, 4, 2, 128, 256), (4096, 2, 2, 200, 192), (300, 8, 3, 64, 64),
                                       (8192, 4, 1, 1024, 1024)])
def test_plain_weight_layout_is_read_in_place(L, E, k, K, N):
    """A plain contiguous [E, K, N] bf16 weight (N contiguous; N a multiple of 64) is read in place
    as an MN-major tensor-core operand: same bits as the transposed-copy path, for the plain, SiLU,
    gated and combine operators, lone CTAs and CTA pairs, ragged K and N tiles."""
    from fast_moe_b200.kernels import moe as ops

    torch.manual_seed(L + K)
    dev = torch.device(DEV)
    idx = torch.rand(L, E, device=dev).topk(k, dim=1).indices
    meta = fm.route_metadata(idx, E)
    index = meta.gate_index.view(-1, k)
    x = torch.randn(L, K, device=dev).bfloat16()
    w = (torch.randn(E, K, N, device=dev) * 0.1).bfloat16()
    wp = (torch.randn(E, K, N, device=dev) * 0.1).bfloat16()
    b = (torch.randn(E, N, device=dev) * 0.1).bfloat16()
    hid = torch.randn(L * k, K, device=dev).bfloat16()
    score = torch.rand(L, k, device=dev)

    def run():
        return (
            fm.index_select_jagged_bmm(0, meta.offsets, index, x, w, b),
            fm.index_select_jagged_bmm_swiglu(0, meta.offsets, index, x, w, None, wp, None),
            ops.silu_jagged_bmm(meta.offsets, hid, w, b, has_silu=True),
            fm.silu_jagged_bmm_combine(0, meta.offsets, hid, w, None, meta.token_index, meta.reverse_index,
                                       gating_scores=score, gates_index=meta.gate_index, has_silu=False),
        )

    assert ops.prep_weight(w, K)[2] == N and ops.prep_weight(w, K)[3] == 1       # taken in place, N contiguous
    got = run()
    ops.MN_MAJOR_WEIGHTS = False
    try:
        assert ops.prep_weight(w, K)[2] == 1
        want = run()
    finally:
        ops.MN_MAJOR_WEIGHTS = True
    for g_, w_ in zip(got, want):
        assert torch.equal(g_, w_)
    assert _lib.device_status(dev) == 0

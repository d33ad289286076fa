"""Backward pass of the operators on the GPU against gradients recorded from the reference:
torch autograd through its PYTORCH functions on CPU in fp32 (tests/golden/make_golden.py, group
"grad"), the same reference and the same generators (U(-1, 1) data, dout = randn * 0.01) its own
backward tests use (kernels/tests/moe_test.py:35-129, :299-400, :951-1133).

Bars: float32 operands run the forward in fp32 accuracy and the backward products d_x likewise;
the weight-gradient product uses tf32 tensor-core math, so float32 gradients are held to rtol 1e-2
of the tensor's largest magnitude; bfloat16 to the reference's own bf16 bound for gradients
(rtol 1e-2 with atol scaled by the tensor's magnitude, kernels/tests/moe_test.py:60-66)."""
import pytest
import torch

import fast_moe_b200 as fm
from fast_moe_b200 import _lib
from fast_moe_b200.kernels import autograd as AG
from tests import golden_io as G

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def leaf(t, dt):
    return None if t is None else t.to(dt).to(DEV).requires_grad_()


def close(got, want, dt, what, bf16_tol=2.5e-2):
    want = want.float()
    scale = max(float(want.abs().max()), 1e-6)
    tol = 1e-2 if dt == torch.float32 else bf16_tol
    err = float((got.detach().float().cpu() - want).abs().max())
    assert err <= tol * scale, f"{what}: max err {err:.3e} vs {tol:.0e} x {scale:.3e}"


@pytest.mark.parametrize("name", G.names("grad_"))
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kmajor", [False, True])
def test_operator_gradients_against_reference_autograd(name, dt, kmajor):
    g = G.load(name)
    k, E = g["k"], g["E"]
    off, gi = g["offsets"].to(DEV), g["gate_index"].to(DEV)
    ti, rev = g["token_index"].to(DEV), g["reverse_index"].to(DEV)
    index = gi.view(-1, k)

    def weight_leaf(w):
        # both weight layouts of the reference's tests: plain [E, K, N], and stored [E, N, K]
        w = w.to(dt).to(DEV)
        if kmajor:
            w = w.permute(0, 2, 1).contiguous().permute(0, 2, 1)
        return w.detach().requires_grad_()

    # ---- up projection
    x, w1, b1 = leaf(g["x"], dt), weight_leaf(g["w1"]), leaf(g.get("b1"), dt)
    out = fm.index_select_jagged_bmm(0, off, index, x, w1, b1)
    assert out.requires_grad
    close(out, g["up_out"], dt, "up forward")
    out.backward(g["up_dout"].to(dt).to(DEV))
    close(x.grad, g["up_d_x"], dt, "up d_x")
    close(w1.grad, g["up_d_w1"], dt, "up d_w")
    if b1 is not None:
        close(b1.grad, g["up_d_b1"], dt, "up d_bias")
    # ---- SwiGLU up projection
    x, w1, w1p = leaf(g["x"], dt), weight_leaf(g["w1"]), weight_leaf(g["w1p"])
    b1, b1p = leaf(g.get("b1"), dt), leaf(g.get("b1p"), dt)
    out = fm.index_select_jagged_bmm_swiglu(0, off, index, x, w1, b1, w1p, b1p)
    close(out, g["sw_out"], dt, "swiglu forward")
    out.backward(g["sw_dout"].to(dt).to(DEV))
    close(x.grad, g["sw_d_x"], dt, "swiglu d_x")
    close(w1.grad, g["sw_d_w1"], dt, "swiglu d_w")
    close(w1p.grad, g["sw_d_w1p"], dt, "swiglu d_wp")
    if b1 is not None:
        close(b1.grad, g["sw_d_b1"], dt, "swiglu d_bias")
        close(b1p.grad, g["sw_d_b1p"], dt, "swiglu d_bias_p")
    # ---- down projection + combine
    hid, w2, b2, gates = leaf(g["hid"], dt), weight_leaf(g["w2"]), leaf(g.get("b2"), dt), leaf(g["gates"], dt)
    y = fm.silu_jagged_bmm_combine(0, off, hid, w2, b2, ti, rev, gates, gi, has_silu=bool(g["has_silu"]))
    close(y, g["down_out"], dt, "down forward")
    y.backward(g["down_dout"].to(dt).to(DEV))
    close(hid.grad, g["down_d_hid"], dt, "down d_jagged")
    close(w2.grad, g["down_d_w2"], dt, "down d_w")
    close(gates.grad, g["down_d_gates"], dt, "down d_gates")
    if b2 is not None:
        close(b2.grad, g["down_d_b2"], dt, "down d_bias")
    # ---- combine alone
    val, gates = leaf(g["val"], dt), leaf(g["gates"], dt)
    z = fm.mul_merge_k_add(ti, rev, val, weight=gates, weight_index=gi)
    close(z, g["comb_out"], dt, "combine forward")
    z.backward(g["comb_dout"].to(dt).to(DEV))
    close(val.grad, g["comb_d_val"], dt, "combine d_value")
    close(gates.grad, g["comb_d_gates"], dt, "combine d_weight")
    assert _lib.device_status(torch.device(DEV)) == 0


def test_weight_gradient_product_with_empty_and_ragged_experts():
    """dW[e] = X_e^T dOut_e through the transposed, padded operands and the grouped GEMM's
    reduction-over-rows mode, against per-expert matmuls: experts with 0, 1, 63, 64, 65 and 1000
    rows (K steps are 64 bf16 rows), output dims that are not tile multiples."""
    lens = [0, 1, 63, 64, 65, 0, 1000, 7]
    E, N, K = len(lens), 200, 72
    off = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    rows = int(off[-1])
    gen = torch.Generator().manual_seed(3)
    d_out = torch.randn(rows, N, generator=gen).bfloat16()
    x = torch.randn(rows, K, generator=gen).bfloat16()
    got = AG.grad_weight(off.to(DEV), d_out.to(DEV), x.to(DEV), E, torch.float32)
    assert got.shape == (E, K, N)
    for e in range(E):
        a, b = int(off[e]), int(off[e + 1])
        want = x[a:b].float().t() @ d_out[a:b].float()
        torch.testing.assert_close(got[e].cpu(), want, rtol=1e-3, atol=1e-3 * max(1.0, float(want.abs().max())))
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_weight_gradient_product_large_outputs_take_cta_pairs(dt):
    """1024 output rows per expert and more: the reduction-over-rows mode on CTA pairs (256-row
    tiles, the K loop of every tile as long as its expert's padded row range)."""
    lens = [700, 0, 1500, 333]
    E, N, K = len(lens), 1280, 384
    off = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    rows = int(off[-1])
    gen = torch.Generator().manual_seed(5)
    d_out = (torch.randn(rows, N, generator=gen) * 0.1).to(dt)
    x = torch.randn(rows, K, generator=gen).to(dt)
    got = AG.grad_weight(off.to(DEV), d_out.to(DEV), x.to(DEV), E, torch.float32)
    for e in range(E):
        a, b = int(off[e]), int(off[e + 1])
        want = x[a:b].float().t() @ d_out[a:b].float()
        tol = 1e-3 if dt == torch.bfloat16 else 3e-3          # f32 operands: tf32 products
        torch.testing.assert_close(got[e].cpu(), want, rtol=tol, atol=tol * max(1.0, float(want.abs().max())))
    assert _lib.device_status(torch.device(DEV)) == 0


def test_no_grad_calls_take_the_forward_only_path():
    g = G.load(G.names("grad_")[0])
    k = g["k"]
    x = g["x"].bfloat16().to(DEV).requires_grad_()
    w = g["w1"].bfloat16().to(DEV).requires_grad_()
    with torch.no_grad():
        out = fm.index_select_jagged_bmm(0, g["offsets"].to(DEV), g["gate_index"].to(DEV).view(-1, k), x, w, None)
    assert not out.requires_grad


@pytest.mark.parametrize("name", G.names("lgrad_"))
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_layer_gradients_against_reference_layer(name, dt):
    """FastMoELayer with ``autograd = True``: y.backward(dout) gives the gradients of x, the gate
    Linear and the expert parameters that the reference layer (PYTORCH kernels, fp32, CPU) gives on
    the same inputs. The router's gradient flows through the renormalised top-k scores."""
    g = G.load(name)
    k = g["k"]
    x0 = g["x"]
    B, T, d = x0.shape
    E, h, _ = g["p::_experts_hidden_w"].shape
    o = g["p::_experts_w"].shape[1]
    layer = fm.FastMoELayer(d, h, o, E, fm.KernelType.PYTORCH, dt)
    layer.load_state_dict({n[3:]: g[n] for n in g if n.startswith("p::")})
    layer.to(DEV)
    layer.autograd = True
    x = x0.to(dt).to(DEV).requires_grad_()
    y = layer(x, k)
    assert y.requires_grad
    close(y, g["y"], dt, "layer forward")
    y.backward(g["dout"].to(dt).to(DEV))
    close(x.grad, g["d_x"], dt, "d_x")
    for n, p in layer.named_parameters():
        assert p.grad is not None, n
        # the gate's gradients are sums over all tokens of small, partly cancelling score
        # gradients: in bf16 (scores, expert rows and dout all rounded to 8 bits) they carry more
        # relative noise than the expert parameters' gradients
        close(p.grad, g["g::" + n], dt, "d " + n, bf16_tol=6e-2 if n.startswith("gate.") else 2.5e-2)
    # switched off (the default) the same call records nothing
    layer.autograd = False
    assert not layer(x, k).requires_grad
    assert _lib.device_status(torch.device(DEV)) == 0


def test_swiglu_layer_gradients_against_oracle_autograd():
    """SwiGLUFastMoELayer with ``autograd = True`` against torch autograd through the CPU oracle's
    SwiGLU composition (the oracle's expert math is plain differentiable torch code; routing is
    taken from the GPU so that both sides differentiate the same selection)."""
    from oracle import moe_oracle as O

    torch.manual_seed(11)
    d, h, o, E, k, L = 64, 96, 48, 8, 2, 150
    layer = fm.SwiGLUFastMoELayer(d, h, o, E, dtype=torch.float32).to(DEV)
    layer.autograd = True
    x = torch.randn(1, L, d)
    xg = x.to(DEV).requires_grad_()
    y = layer(xg, k)
    dout = torch.randn_like(y) * 0.01
    y.backward(dout)
    # reference: same routing, differentiable scores recomputed on the CPU
    xc = x.clone().requires_grad_()
    gw = layer.gate.gate.weight.detach().cpu().requires_grad_()
    gb = layer.gate.gate.bias.detach().cpu().requires_grad_()
    wg = layer.w_gate.detach().cpu().requires_grad_()
    wu = layer.w_up.detach().cpu().requires_grad_()
    wd = layer.w_down.detach().cpu().requires_grad_()
    idx, _, _ = fm.gate_topk(x.view(-1, d).to(DEV), layer.gate.gate.weight, layer.gate.gate.bias, k)
    idx = idx.cpu()
    probs = torch.softmax(torch.nn.functional.linear(xc.view(-1, d), gw, gb), dim=1)
    sel = probs.gather(1, idx)
    scores = sel / sel.sum(dim=1, keepdim=True).clamp_min(1e-12)
    dense = torch.zeros(L, E).scatter(1, idx, 1.0)
    gi, ti, _, off, rev, _ = O.routing_metadata(dense, idx)
    ref = O.fused_jagged_bmm_swiglu_combine(off, gi.view(-1, k), xc.view(-1, d), wg.permute(0, 2, 1), None,
                                            wu.permute(0, 2, 1), None, wd.permute(0, 2, 1), None, k, scores, gi)
    ref.backward(dout.cpu().view(-1, o))
    close(y.view(-1, o), ref.detach(), torch.float32, "forward")
    close(xg.grad, xc.grad, torch.float32, "d_x")
    close(layer.gate.gate.weight.grad, gw.grad, torch.float32, "d gate weight")
    close(layer.gate.gate.bias.grad, gb.grad, torch.float32, "d gate bias")
    close(layer.w_gate.grad, wg.grad, torch.float32, "d w_gate")
    close(layer.w_up.grad, wu.grad, torch.float32, "d w_up")
    close(layer.w_down.grad, wd.grad, torch.float32, "d w_down")
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("swiglu", [False, True])
def test_captured_train_step_matches_eager(swiglu):
    """Forward + backward replayed as one CUDA graph: output, d_x and every parameter gradient equal
    the eager autograd run bit for bit where no atomics are involved (the gate weight gradient is
    summed with atomics: 1e-5), also after new tokens are copied in."""
    torch.manual_seed(3)
    d, h, o, E, k, L = 64, 128, 64, 8, 2, 256
    cls = fm.SwiGLUFastMoELayer if swiglu else fm.FastMoELayer
    layer = cls(d, h, o, E, dtype=torch.bfloat16).to(DEV)
    layer.autograd = True
    x0 = torch.randn(1, L, d, device=DEV).bfloat16()
    step = fm.CapturedTrainStep(layer, x0, k)
    for seed in (4, 5):
        torch.manual_seed(seed)
        x = torch.randn(1, L, d, device=DEV).bfloat16()
        dout = (torch.randn(1, L, o, device=DEV) * 0.01).bfloat16()
        y = step.step(x, dout).clone()
        got = {n: p.grad.clone() for n, p in layer.named_parameters()}
        got_dx = step.d_x.clone()
        # eager reference on fresh leaves
        for p in layer.parameters():
            p.grad = None
        xe = x.clone().requires_grad_()
        ye = layer(xe, k)
        ye.backward(dout)
        assert torch.equal(y, ye)
        assert torch.equal(got_dx, xe.grad)
        for n, p in layer.named_parameters():
            if n.startswith("gate."):
                torch.testing.assert_close(got[n], p.grad, atol=1e-5, rtol=1e-4)
            else:
                assert torch.equal(got[n], p.grad), n
        # hand the static gradient tensors back to the graph
        for n, p in layer.named_parameters():
            p.grad = None
        step = fm.CapturedTrainStep(layer, x0, k)
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("stored_kmajor", [True, False])
@pytest.mark.parametrize("rows_per_expert", [96, 1500])
def test_reduction_over_two_weights_matches_concatenation(stored_kmajor, rows_per_expert):
    """jagged_bmm_two_weights (d_x of the gated up projection: d_alpha @ W^T + d_beta @ Wp^T as one
    product) gives the bits of the product with the two transposed weights laid side by side, for
    weights stored [E, N, K] (read as MN-major operands) and plain [E, K, N] ones."""
    from fast_moe_b200.kernels import moe as ops

    torch.manual_seed(rows_per_expert)
    E, K, N = 4, 128, 192          # the up projection's K (tokens) and N (hidden); d_ab is [rows, 2N]
    lens = torch.tensor([rows_per_expert, 0, rows_per_expert + 37, 5])
    off = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)]).to(DEV)
    rows = int(lens.sum())
    d_ab = torch.randn(rows, 2 * N, device=DEV).bfloat16()

    def make():
        w = (torch.randn(E, K, N, device=DEV) * 0.1).bfloat16()
        return w.permute(0, 2, 1).contiguous().permute(0, 2, 1) if stored_kmajor else w

    w, wp = make(), make()
    got = ops.jagged_bmm_two_weights(off, d_ab, w.permute(0, 2, 1), wp.permute(0, 2, 1))
    assert got is not None
    w_cat = AG.transposed_weights_side_by_side(w, wp)
    want = ops.silu_jagged_bmm(off, d_ab, w_cat, None, has_silu=False)
    assert torch.equal(got, want)
    ref = torch.zeros(rows, K)
    for e in range(E):
        a, b = int(off[e]), int(off[e + 1])
        ref[a:b] = d_ab[a:b, :N].float().cpu() @ w[e].float().cpu().t() + d_ab[a:b, N:].float().cpu() @ wp[e].float().cpu().t()
    close(got, ref, torch.bfloat16, "two-weight product")
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("swiglu", [False, True])
def test_partial_gradients_frozen_experts_or_constant_input(swiglu):
    """Only what requires a gradient gets one: frozen expert weights stay without .grad while x and
    the gate still receive theirs (equal to the all-trainable run), and a constant input with
    trainable parameters works as well."""
    torch.manual_seed(8)
    d, h, o, E, k, L = 64, 128, 64, 4, 2, 200
    cls = fm.SwiGLUFastMoELayer if swiglu else fm.FastMoELayer
    layer = cls(d, h, o, E, dtype=torch.bfloat16).to(DEV)
    layer.autograd = True
    x = torch.randn(1, L, d, device=DEV).bfloat16()
    dout = (torch.randn(1, L, o, device=DEV) * 0.01).bfloat16()
    xa = x.clone().requires_grad_()
    layer(xa, k).backward(dout)
    full = {n: p.grad.clone() for n, p in layer.named_parameters()}
    for n, p in layer.named_parameters():
        p.grad = None
        if not n.startswith("gate."):
            p.requires_grad_(False)
    xb = x.clone().requires_grad_()
    layer(xb, k).backward(dout)
    assert torch.equal(xb.grad, xa.grad)
    for n, p in layer.named_parameters():
        if n.startswith("gate."):
            torch.testing.assert_close(p.grad, full[n], atol=1e-5, rtol=1e-4)
        else:
            assert p.grad is None, n
    # constant input, trainable experts
    for n, p in layer.named_parameters():
        p.requires_grad_(True)
        p.grad = None
    y = layer(x, k)
    assert y.requires_grad
    y.backward(dout)
    for n, p in layer.named_parameters():
        if not n.startswith("gate."):
            assert torch.equal(p.grad, full[n]), n
    assert _lib.device_status(torch.device(DEV)) == 0

"""The sparsely-gated ("MRN" / SGMoE) layer on the GPU against fixtures recorded from the reference's
OrigSGMoEImpl (kernels/pytorch/mrn.py, run unmodified on CPU by tests/golden/make_golden.py) and
against the CPU oracle (oracle/mrn_oracle.py) at the shapes of the reference's own test
(kernels/tests/mrn_test.py:660-862: d = model_d = 64, E in {4, 8}, k in {1, 2}, bf16, rtol = atol =
1e-2). float32 tokens run in fp32 accuracy and are held to 1e-4."""
import pytest
import torch

import fast_moe_b200 as fm
from fast_moe_b200 import _lib
from oracle import mrn_oracle as M
from tests import golden_io as G

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def cu(t):
    return None if t is None else t.to(DEV)


def _layer_from_golden(g, dtype=torch.float32):
    L, d = g["x"].shape
    E, m, _ = g["w_hidden"].shape
    o = g["w_out"].shape[1]
    cfg = fm.SGConfig(model_d=m, num_experts=E, num_activated_experts=g["k"], loss_coef=g["loss_coef"],
                      enable_noisy_gating="w_noise" in g)
    layer = fm.SGMoELayer(d, o, cfg)
    with torch.no_grad():
        layer._experts_hidden_w.copy_(g["w_hidden"]); layer._experts_hidden_bias.copy_(g["b_hidden"])
        layer._experts_w.copy_(g["w_out"]); layer._experts_bias.copy_(g["b_out"])
        layer._w_gate.copy_(g["w_gate"]); layer._output_weight.copy_(g["output_weight"])
        if "w_noise" in g:
            layer._w_noise.copy_(g["w_noise"])
    return layer.to(DEV)


def _safe_tokens(g, min_gap=1e-6):
    """Tokens whose k-th and (k+1)-th gate probabilities are not a near tie."""
    x_norm = g["x_norm"]
    raw = x_norm @ g["w_gate"]
    if "w_noise" in g and g["train"]:
        raw = raw + g["noise"] * (torch.nn.functional.softplus(x_norm @ g["w_noise"]) + 1e-2)
    logits = torch.nn.functional.normalize(raw, dim=1)
    p = torch.softmax(logits, dim=1).sort(dim=1, descending=True).values
    k = g["k"]
    if k >= p.shape[1]:
        return torch.ones(p.shape[0], dtype=torch.bool)
    return (p[:, k - 1] - p[:, k]) > min_gap


@pytest.mark.parametrize("name", G.names("mrn_"))
def test_token_norm_and_router_against_golden(name):
    g = G.load(name)
    d = g["x"].shape[1]
    groups = g["num_groups"]
    gn = bool(g["group_norm"])
    x_norm = fm.token_norm(cu(g["x"]), cu(g["norm_weight"]), cu(g["norm_bias"]), g["norm_eps"], group_norm=gn,
                           num_groups=groups)
    torch.testing.assert_close(x_norm.cpu(), g["x_norm"], atol=2e-6, rtol=1e-5)
    if "gates" not in g:
        return
    k = g["k"]
    idx, score, logits = fm.gate_topk_normalized(cu(g["x_norm"]), cu(g["w_gate"].t().contiguous()), k, return_logits=True)
    torch.testing.assert_close(logits.cpu(), g["x_norm"] @ g["w_gate"], atol=1e-5, rtol=1e-5)
    safe = _safe_tokens(g)
    dense = torch.zeros_like(g["gates"]).scatter_(1, idx.cpu(), score.cpu())
    assert torch.equal((dense > 0)[safe], (g["gates"] > 0)[safe])
    torch.testing.assert_close(dense[safe], g["gates"][safe], atol=1e-6, rtol=1e-5)
    # slots in descending probability, ties to the lower expert id; precomputed logits route the same
    assert bool((score[:, :-1] >= score[:, 1:]).all())
    idx2, score2, _ = fm.gate_topk_normalized(None, None, k, logits=logits)
    assert torch.equal(idx2, idx) and torch.equal(score2, score)
    assert _lib.device_status(torch.device(DEV)) == 0


def _check_noisy_layer(g):
    """Noisy gating while training (kernels/pytorch/mrn.py:191-237): with the noise the reference
    drew, the layer reproduces its output, its load fractions and its loss (which uses the smooth
    load estimate); the same noise twice gives the same bits; a fresh draw and evaluation mode run."""
    d = g["x"].shape[1]
    args = (None, 0, False, 1, d, cu(g["norm_weight"]), cu(g["norm_bias"]), g["norm_eps"])
    layer = _layer_from_golden(g)
    layer.train(True)
    safe = _safe_tokens(g)
    layer.set_noise(cu(g["noise"]))
    out = layer(cu(g["x"]), *args)
    torch.testing.assert_close(out.x.cpu()[safe], g["y"][safe], atol=1e-4, rtol=1e-4)
    if bool(safe.all()):
        torch.testing.assert_close(out.load.cpu(), g["load"], atol=1e-7, rtol=1e-6)
        torch.testing.assert_close(out.loss.cpu().reshape(-1), g["loss"], atol=1e-6, rtol=1e-4)
    layer.set_noise(cu(g["noise"]))
    again = layer(cu(g["x"]), *args)
    assert torch.equal(again.x, out.x) and torch.equal(again.loss, out.loss)
    fresh = layer(cu(g["x"]), *args)                      # the layer's own draw
    assert torch.isfinite(fresh.x).all() and torch.isfinite(fresh.loss)
    # evaluation: clean logits, no loss
    layer.train(False)
    ev = layer(cu(g["x"]), *args)
    ref, _, ref_load = M.sg_moe_forward(g["x"], g["norm_weight"], g["norm_bias"], g["norm_eps"], g["w_gate"], g["w_hidden"],
                                        g["b_hidden"], g["w_out"], g["b_out"], g["output_weight"], g["k"], train=False)
    logits = torch.nn.functional.normalize(g["x_norm"] @ g["w_gate"], dim=1)
    p = torch.softmax(logits, dim=1).sort(dim=1, descending=True).values
    clean_safe = (p[:, g["k"] - 1] - p[:, g["k"]]) > 1e-6
    torch.testing.assert_close(ev.x.cpu()[clean_safe], ref[clean_safe], atol=1e-4, rtol=1e-4)
    assert float(ev.loss) == 0.0
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("L,d,E,k", [(1000, 64, 64, 4), (333, 48, 8, 2), (64, 32, 128, 7), (5, 16, 4, 3), (40, 32, 4, 4)])
def test_noisy_router_against_oracle(L, d, E, k):
    """noisy_gate against the CPU restatement of _orig_noisy_gating / _prob_in_top_k on the same
    noise: picks and gate values on tokens without a near tie, the smooth load per expert and the
    loss built on it (fp32 sums in a different order: 1e-5 relative)."""
    from fast_moe_b200.kernels.routing import noisy_gate, route_metadata, sg_load_loss

    torch.manual_seed(L + E)
    x = torch.randn(L, d)
    wg = torch.randn(d, E) * 0.3
    wn = torch.randn(d, E) * 0.3
    noise = torch.randn(L, E)
    gates, idx_ref, topk_ref, loss_ref = M.gating(x, wg, k, True, wn, noise)
    both = torch.cat([wg.t(), wn.t()], dim=0).contiguous()
    idx, score, partials = noisy_gate(cu(x), cu(both), k, cu(noise))
    raw = x @ wg + noise * (torch.nn.functional.softplus(x @ wn) + 1e-2)
    p = torch.softmax(torch.nn.functional.normalize(raw, dim=1), dim=1).sort(dim=1, descending=True).values
    safe = (p[:, k - 1] - p[:, k]) > 1e-6 if k < E else torch.ones(L, dtype=torch.bool)
    assert torch.equal(idx.cpu()[safe], idx_ref[safe])
    torch.testing.assert_close(score.cpu()[safe], topk_ref[safe], atol=1e-6, rtol=1e-5)
    meta = route_metadata(idx, E)
    loss, load = sg_load_loss(meta, score, E, torch.float32, 1.0, True, partials)
    if k < E:
        assert partials is not None
        # the oracle's smooth load, recomputed here from its definition
        stddev = torch.nn.functional.softplus(x @ wn) + 1e-2
        srt = torch.nn.functional.normalize(raw, dim=1).sort(dim=1, descending=True).values
        thr_in, thr_out = srt[:, k:k + 1], srt[:, k - 1:k]
        nrm = torch.distributions.normal.Normal(torch.tensor([0.0]), torch.tensor([1.0]), validate_args=False)
        prob = torch.where(raw > thr_in, nrm.cdf((x @ wg - thr_in) / stddev), nrm.cdf((x @ wg - thr_out) / stddev))
        torch.testing.assert_close(partials.sum(0).cpu(), prob.sum(0), atol=1e-4, rtol=2e-5)
    else:
        assert partials is None
    if bool(safe.all()):
        torch.testing.assert_close(loss.cpu(), loss_ref.float(), atol=1e-6, rtol=1e-4)
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("name", G.names("mrn_"))
def test_sg_moe_layer_against_golden(name):
    g = G.load(name)
    if "w_noise" in g:
        _check_noisy_layer(g)
        return
    d = g["x"].shape[1]
    groups = g["num_groups"]
    gn = bool(g["group_norm"])
    args = (None, 0, gn, groups, d // groups, cu(g["norm_weight"]), cu(g["norm_bias"]), g["norm_eps"])
    layer = _layer_from_golden(g)
    layer.train(bool(g["train"]))
    safe = _safe_tokens(g)
    out = layer(cu(g["x"]), *args)
    assert isinstance(out, fm.MRNOutput) and out.x.dtype == torch.float32
    torch.testing.assert_close(out.x.cpu()[safe], g["y"][safe], atol=1e-4, rtol=1e-4)
    if bool(safe.all()):
        torch.testing.assert_close(out.load.cpu(), g["load"], atol=1e-7, rtol=1e-6)
        torch.testing.assert_close(out.loss.cpu().reshape(-1), g["loss"], atol=1e-6, rtol=1e-4)
    # TF32 allowed: same call on the tf32 kernels, at the bf16-class bound
    fm.set_fp32_matmul("tf32")
    try:
        out_tf32 = layer(cu(g["x"]), *args)
        torch.testing.assert_close(out_tf32.x.cpu()[safe], g["y"][safe], atol=2e-2, rtol=2e-2)
    finally:
        fm.set_fp32_matmul(None)
    # bf16 tokens: the reference test's own bound against the fp32 reference on the rounded inputs
    xb = g["x"].bfloat16()
    ref, ref_loss, ref_load = M.sg_moe_forward(
        xb.float(), g["norm_weight"], g["norm_bias"], g["norm_eps"], g["w_gate"], g["w_hidden"].bfloat16().float(),
        g["b_hidden"].bfloat16().float(), g["w_out"].bfloat16().float(), g["b_out"].bfloat16().float(),
        g["output_weight"].bfloat16().float(), g["k"], train=bool(g["train"]), loss_coef=g["loss_coef"], group_norm=gn,
        num_groups=groups, linear_dim=d // groups)
    outb = layer(cu(xb), *args)
    assert outb.x.dtype == torch.bfloat16
    err = (outb.x.float().cpu() - ref).abs()
    bad = (err > 2e-2 + 2e-2 * ref.abs()).any(dim=1).float().mean().item()
    # the experts see bf16(x_norm): a token whose gate probabilities nearly tie may route differently
    assert bad < 0.05, f"{bad:.2%} of tokens outside tolerance, max err {err.max().item():.3e}"
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("B,max_seq_len,E,k", [(16, 32, 4, 1), (32, 64, 8, 2), (16, 128, 8, 2)])
def test_sg_moe_layer_at_the_reference_test_shapes(B, max_seq_len, E, k):
    """kernels/tests/mrn_test.py:660-862: jagged batch of B sequences, input_d = model_d = 64, bf16,
    rtol = atol = 1e-2, training mode without noisy gating; checked against the CPU oracle."""
    d = 64
    g = torch.Generator().manual_seed(B + E + k)
    lengths = torch.randint(1, max_seq_len + 1, (B,), generator=g)
    L = int(lengths.sum())
    torch.manual_seed(0)
    layer = fm.SGMoELayer(d, d, fm.SGConfig(model_d=d, num_experts=E, num_activated_experts=k)).to(DEV)
    layer.train(True)
    x = torch.randn(L, d, generator=g).bfloat16()
    nw, nb = torch.ones(d), torch.zeros(d)
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)])
    out = layer(cu(x), cu(offsets), max_seq_len, False, 1, d, cu(nw), cu(nb), 1e-5)
    f = lambda p: p.detach().float().cpu()
    rb = lambda p: p.detach().to(torch.bfloat16).float().cpu()
    ref, ref_loss, ref_load = M.sg_moe_forward(
        x.float(), nw, nb, 1e-5, f(layer._w_gate), rb(layer._experts_hidden_w), rb(layer._experts_hidden_bias),
        rb(layer._experts_w), rb(layer._experts_bias), rb(layer._output_weight), k, train=True, loss_coef=layer.loss_coef)
    err = (out.x.float().cpu() - ref).abs()
    bad = (err > 1e-2 + 1e-2 * ref.abs()).any(dim=1).float().mean().item()
    assert bad < 0.03, f"{bad:.2%} of tokens outside rtol/atol 1e-2, max err {err.max().item():.3e}"
    torch.testing.assert_close(out.load.cpu(), ref_load, atol=2e-2, rtol=0)
    torch.testing.assert_close(out.loss.cpu(), ref_loss, atol=1e-3, rtol=5e-2)
    assert _lib.device_status(torch.device(DEV)) == 0


def _close(got, want, dt, what, bf16_tol=2.5e-2):
    want = want.float()
    scale = max(float(want.abs().max()), 1e-6)
    tol = 1e-2 if dt == torch.float32 else bf16_tol
    err = float((got.detach().float().cpu() - want).abs().max())
    assert err <= tol * scale, f"{what}: max err {err:.3e} vs {tol:.0e} x {scale:.3e}"


@pytest.mark.parametrize("name", G.names("mgrad_"))
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_sg_moe_layer_gradients_against_reference(name, dt):
    """``autograd = True``: backward of sum(y * dout) + loss gives the gradients the reference's
    OrigSGMoEImpl gives on CPU in fp32 for x, the norm's weight and bias and every parameter
    (what kernels/tests/mrn_test.py:816-860 compares), the loss's own path into the router
    included; one fixture trains with noisy gating (recorded noise; both gate matrices get gradients
    through the noise scale and the smooth load). Bars as for the FastMoELayer gradients: 1e-2 of a tensor's largest magnitude in fp32
    (tf32 weight-gradient products), the reference's bf16 bound otherwise."""
    g = G.load(name)
    d = g["x"].shape[1]
    E, m, _ = g["p::_experts_hidden_w"].shape
    o = g["p::_experts_w"].shape[1]
    groups, gn = g["num_groups"], bool(g["group_norm"])
    noisy = "noise" in g
    cfg = fm.SGConfig(model_d=m, num_experts=E, num_activated_experts=g["k"], loss_coef=g["loss_coef"],
                      enable_noisy_gating=noisy)
    layer = fm.SGMoELayer(d, o, cfg)
    with torch.no_grad():
        for n, p in layer.named_parameters():
            p.copy_(g["p::" + n])
    layer.to(DEV)
    layer.train(True)
    layer.autograd = True
    if noisy:
        layer.set_noise(g["noise"].to(DEV))
    x = g["x"].to(dt).to(DEV).requires_grad_()
    nw = g["norm_weight"].to(DEV).requires_grad_()
    nb = g["norm_bias"].to(DEV).requires_grad_()
    out = layer(x, None, 0, gn, groups, d // groups, nw, nb, g["norm_eps"])
    assert out.x.requires_grad and out.loss.requires_grad and not out.load.requires_grad
    _close(out.x, g["y"], dt, "forward")
    _close(out.loss.reshape(-1), g["loss"], dt, "loss")
    ((out.x.float() * g["dout"].to(DEV)).sum() + out.loss).backward()
    # With noisy gating the loss differentiates Phi((clean - threshold) / stddev), whose slope in
    # clean is z * pdf(z) / stddev^2 with stddev down to 0.1 here: bf16 tokens (8 bits) move clean by
    # ~1e-2 and with it the router's share of the gradients of x, the norm and the two gate matrices
    # by 10-20 % of their largest value. Those are held to the reference in fp32 only (and, piece by
    # piece, against torch autograd in test_noisy_router_backward_against_torch_autograd); in bf16
    # they must be finite, and the expert parameters hold the usual bound.
    through_router = noisy and dt == torch.bfloat16
    for name, got, want in (("d_x", x.grad, g["d_x"]), ("d norm weight", nw.grad, g["d_norm_weight"]),
                            ("d norm bias", nb.grad, g["d_norm_bias"])):
        if through_router:
            assert torch.isfinite(got).all(), name
        else:
            _close(got, want, dt, name)
    for n, p in layer.named_parameters():
        assert p.grad is not None, n
        if n in ("_w_gate", "_w_noise"):
            if through_router:
                assert torch.isfinite(p.grad).all(), n
            else:
                _close(p.grad, g["g::" + n], dt, "d " + n, bf16_tol=6e-2)
        else:
            _close(p.grad, g["g::" + n], dt, "d " + n)
    # switched off (the default) nothing is recorded
    layer.autograd = False
    assert not layer(x, None, 0, gn, groups, d // groups, nw, nb, g["norm_eps"]).x.requires_grad
    assert _lib.device_status(torch.device(DEV)) == 0


def test_sg_moe_pieces_against_torch_autograd():
    """The layer's own backward kernels one at a time against torch autograd on the CPU: token norm
    (layer and group form, with parameter gradients), the normalised-logit router, the loss."""
    from fast_moe_b200.kernels.autograd import SGLossFn, SGRouterFn, TokenNormFn
    import torch.nn.functional as F

    torch.manual_seed(5)
    L, d, E, k = 300, 96, 16, 3
    # ---- token norm
    for gn, groups in ((False, 1), (True, 4)):
        x = torch.randn(L, d)
        ns = groups if gn else d
        w = torch.randn(ns) * 0.3 + 1
        b = torch.randn(ns) * 0.1
        dy = torch.randn(L, d)
        xc, wc, bc = x.clone().requires_grad_(), w.clone().requires_grad_(), b.clone().requires_grad_()
        ref = (F.group_norm(xc.view(-1, groups, d // groups), groups, wc, bc, 1e-5).view(L, d) if gn
               else F.layer_norm(xc, (d,), wc, bc, 1e-5))
        ref.backward(dy)
        xg, wg, bg = cu(x).requires_grad_(), cu(w).requires_grad_(), cu(b).requires_grad_()
        out = TokenNormFn.apply(xg, wg, bg, 1e-5, gn, groups)
        out.backward(cu(dy))
        torch.testing.assert_close(out.detach().cpu(), ref.detach(), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(xg.grad.cpu(), xc.grad, atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(wg.grad.cpu(), wc.grad, atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(bg.grad.cpu(), bc.grad, atol=1e-4, rtol=1e-4)
    # ---- router: softmax over all experts of the L2-normalised logits, k largest kept
    x = torch.randn(L, d)
    wgt = torch.randn(d, E) * 0.2
    dsc = torch.randn(L, k)
    xg, wg = cu(x).requires_grad_(), cu(wgt).requires_grad_()
    idx, score = SGRouterFn.apply(xg, wg, k)
    score.backward(cu(dsc))
    xc, wc = x.clone().requires_grad_(), wgt.clone().requires_grad_()
    p = torch.softmax(F.normalize(xc @ wc, dim=1), dim=1)
    sel = p.gather(1, idx.cpu())
    torch.testing.assert_close(score.detach().cpu(), sel.detach(), atol=1e-6, rtol=1e-5)
    sel.backward(dsc)
    torch.testing.assert_close(xg.grad.cpu(), xc.grad, atol=1e-5, rtol=1e-3)
    torch.testing.assert_close(wg.grad.cpu(), wc.grad, atol=1e-4, rtol=1e-3)
    # ---- loss through the importance
    meta = fm.route_metadata(idx, E)
    sg = score.detach().clone().requires_grad_()
    loss, load = SGLossFn.apply(sg, meta.offsets, meta.gate_index, E, False, 0.7)
    (loss * 3.0).backward()
    sc = score.detach().cpu().clone().requires_grad_()
    gates = torch.zeros(L, E).scatter(1, idx.cpu(), sc)
    ref_loss = 0.7 * (M.cv_squared(gates.sum(0)) + M.cv_squared((gates > 0).sum(0)))
    (ref_loss * 3.0).backward()
    torch.testing.assert_close(loss.detach().cpu(), ref_loss.detach(), atol=1e-6, rtol=1e-4)
    torch.testing.assert_close(sg.grad.cpu(), sc.grad, atol=1e-6, rtol=1e-3)
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("L,d,E,k", [(257, 48, 8, 2), (64, 32, 16, 5), (50, 16, 4, 4)])
def test_noisy_router_backward_against_torch_autograd(L, d, E, k):
    """SGNoisyRouterFn + SGLossFn against torch autograd on the CPU through the same definition
    (noise * (softplus(x w_noise) + eps) on the logits, L2 normalisation, softmax over all experts,
    k largest kept; smooth load = sum of Phi((clean - threshold) / stddev) with the thresholds
    taken from the sorted normalised logits): gradients of x and of both gate matrices for
    sum(scores * r) + loss."""
    from fast_moe_b200.kernels.autograd import SGLossFn, SGNoisyRouterFn
    import torch.nn.functional as F

    torch.manual_seed(L + E)
    x = torch.randn(L, d)
    wg = torch.randn(d, E) * 0.3
    wn = torch.randn(d, E) * 0.3
    noise = torch.randn(L, E)
    r = torch.randn(L, k)
    coef = 0.7
    # ---- GPU
    xg, wgg, wng = cu(x).requires_grad_(), cu(wg).requires_grad_(), cu(wn).requires_grad_()
    idx, score, part = SGNoisyRouterFn.apply(xg, wgg, wng, k, cu(noise))
    meta = fm.route_metadata(idx, E)
    loss, _ = SGLossFn.apply(score, meta.offsets, meta.gate_index, E, False, coef, part if part.shape[0] else None)
    ((score * cu(r)).sum() + loss).backward()
    # ---- CPU reference with the GPU's selection
    xc, wgc, wnc = x.clone().requires_grad_(), wg.clone().requires_grad_(), wn.clone().requires_grad_()
    clean = xc @ wgc
    sd = F.softplus(xc @ wnc) + 1e-2
    noisy = clean + noise * sd
    n = F.normalize(noisy, dim=1)
    srt, order = n.sort(dim=1, descending=True, stable=True)
    p = torch.softmax(srt, dim=1)[:, :k]
    assert torch.equal(order[:, :k], idx.cpu()), "routing differs (near tie): pick another seed"
    gates = torch.zeros(L, E).scatter(1, order[:, :k], p)
    if k < E:
        thr_in, thr_out = srt[:, k:k + 1], srt[:, k - 1:k]
        nrm = torch.distributions.normal.Normal(torch.tensor([0.0]), torch.tensor([1.0]), validate_args=False)
        prob = torch.where(noisy > thr_in, nrm.cdf((clean - thr_in) / sd), nrm.cdf((clean - thr_out) / sd))
        load = prob.sum(0)
    else:
        load = (gates > 0).sum(0)
    ref_loss = coef * (M.cv_squared(gates.sum(0)) + M.cv_squared(load))
    ((p * r).sum() + ref_loss).backward()
    torch.testing.assert_close(score.detach().cpu(), p.detach(), atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(loss.detach().cpu(), ref_loss.detach().float(), atol=1e-6, rtol=1e-4)
    torch.testing.assert_close(xg.grad.cpu(), xc.grad, atol=2e-5, rtol=2e-3)
    torch.testing.assert_close(wgg.grad.cpu(), wgc.grad, atol=2e-4, rtol=2e-3)
    torch.testing.assert_close(wng.grad.cpu(), wnc.grad, atol=2e-4, rtol=2e-3)
    assert _lib.device_status(torch.device(DEV)) == 0

"""Edge cases of the C-ABI entry points on a GPU: empty batches (zero rows are valid input, an
empty tensor's data pointer is NULL), an out-of-range gate index in the fused combine (recorded
and skipped, nothing written), and the layers' per-dtype weight caches."""
import pytest
import torch

import fast_moe_b200 as fm
from fast_moe_b200 import _lib
from fast_moe_b200.kernels import moe, moe_fp8

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _empty_routing(E, k):
    idx = torch.empty((0, k), dtype=torch.int64, device=DEV)
    return fm.route_metadata(idx, E)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_operators_accept_zero_rows(dt):
    E, k, K, N = 4, 2, 64, 96
    meta = _empty_routing(E, k)
    assert meta.offsets.tolist() == [0] * (E + 1)
    x = torch.empty((0, K), dtype=dt, device=DEV)
    w = torch.randn(E, N, K, device=DEV).to(dt).permute(0, 2, 1)
    b = torch.zeros(E, N, device=DEV, dtype=dt)
    index = meta.gate_index.view(-1, k)
    assert moe.index_select_jagged_bmm(0, meta.offsets, index, x, w, b).shape == (0, N)
    assert moe.index_select_jagged_bmm_swiglu(0, meta.offsets, index, x, w, b, w, b).shape == (0, N)
    hid = torch.empty((0, N), dtype=dt, device=DEV)
    w2 = torch.randn(E, K, N, device=DEV).to(dt).permute(0, 2, 1)
    score = torch.empty((0, k), dtype=dt, device=DEV)
    for fused in (False, True):
        y = moe.silu_jagged_bmm_combine(0, meta.offsets, hid, w2, None, meta.token_index, meta.reverse_index,
                                        gating_scores=score, gates_index=meta.gate_index, has_silu=False, fused=fused)
        assert y.shape == (0, K)
    assert moe.silu_jagged_bmm(meta.offsets, hid, w2, None, has_silu=False).shape == (0, K)
    assert moe.mul_merge_k_add(meta.token_index, meta.reverse_index, torch.empty((0, K), dtype=dt, device=DEV),
                               weight=score, weight_index=meta.gate_index).shape == (0, K)
    assert moe.gather_rows(torch.randn(5, K, device=DEV).to(dt), meta.gate_index, k).shape == (0, K)
    if dt == torch.bfloat16:
        q, s = moe_fp8.rowwise_quant_fp8(x)
        assert q.shape == (0, K) and s.shape == (0,)
    assert _lib.device_status(torch.device(DEV)) == 0


def test_layers_accept_an_empty_batch():
    layer = fm.SwiGLUFastMoELayer(64, 128, 64, 4, dtype=torch.bfloat16).to(DEV)
    y = layer(torch.empty((2, 0, 64), dtype=torch.bfloat16, device=DEV), 2)
    assert y.shape == (2, 0, 64)
    mlp = fm.FastMoELayer(64, 128, 64, 4, dtype=torch.bfloat16).to(DEV)
    assert mlp(torch.empty((0, 3, 64), dtype=torch.bfloat16, device=DEV), 2).shape == (0, 3, 64)
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("N", [256, 200])     # vector stores / scalar tail path
def test_fused_combine_skips_a_row_whose_gate_index_is_out_of_range(N):
    """One entry of gates_index points past the end. The kernel must record FMOE_DEV_BAD_INDEX and
    write nothing for that row: the token rows equal the clean result minus that row's share, and
    the canary rows behind the output stay untouched."""
    L, E, k, K = 300, 4, 2, 128
    g = torch.Generator().manual_seed(N)
    idx = torch.randn(L, E, generator=g).topk(k, dim=1).indices.to(DEV)
    meta = fm.route_metadata(idx, E)
    hid = (torch.randn(L * k, K, generator=g)).bfloat16().to(DEV)
    w2 = (torch.randn(E, N, K, generator=g) * 0.1).bfloat16().to(DEV).permute(0, 2, 1)
    score = torch.rand(L, k, generator=g).bfloat16().to(DEV)
    args = (0, meta.offsets, hid, w2, None, meta.token_index, meta.reverse_index)
    clean = moe.silu_jagged_bmm_combine(*args, gating_scores=score, gates_index=meta.gate_index, has_silu=False, fused=True)
    rows = moe.silu_jagged_bmm(meta.offsets, hid, w2, None, has_silu=False)
    assert _lib.device_status(torch.device(DEV)) == 0
    bad_row = 123
    bad_index = meta.gate_index.clone()
    victim = int(bad_index[bad_row])
    bad_index[bad_row] = L * k + 5                      # would land k rows past the end of `out`
    canary = torch.full((L + 8, N), 7.0, dtype=torch.bfloat16, device=DEV)
    out = canary[:L]
    out.zero_()
    got = moe.silu_jagged_bmm_combine(*args, gating_scores=score, gates_index=bad_index, has_silu=False, fused=True,
                                      out=out)
    torch.cuda.synchronize()
    assert _lib.device_status(torch.device(DEV)) == 1      # FMOE_DEV_BAD_INDEX, cleared by the read
    assert bool((canary[L:] == 7.0).all()), "rows behind the output were written"
    token = victim // k
    share = (rows[bad_row].float() * score.view(-1)[victim].float())
    expect = clean.float().clone()
    expect[token] -= share
    torch.testing.assert_close(got.float(), expect, rtol=2e-2, atol=2e-2 * max(1.0, float(clean.abs().max())))
    others = torch.ones(L, dtype=torch.bool, device=DEV)
    others[token] = False
    assert torch.equal(got[others], clean[others])


def test_cast_cache_follows_dtype_mismatch_and_in_place_updates():
    """Parameters kept in fp32, tokens in bf16: the layer casts each weight once and reuses the
    copy; an in-place update of the parameter (an optimiser step) or a move invalidates it."""
    torch.manual_seed(0)
    d, h, o, E, k = 64, 128, 64, 4, 2
    layer = fm.SwiGLUFastMoELayer(d, h, o, E, dtype=torch.float32).to(DEV)
    twin = fm.SwiGLUFastMoELayer(d, h, o, E, dtype=torch.bfloat16).to(DEV)
    x = torch.randn(2, 50, d, device=DEV).bfloat16()

    def sync_twin():
        with torch.no_grad():
            for n in ("w_gate", "w_up", "w_down"):
                getattr(twin, n).copy_(getattr(layer, n).to(torch.bfloat16))
            twin.gate.gate.weight.copy_(layer.gate.gate.weight)
            twin.gate.gate.bias.copy_(layer.gate.gate.bias)

    sync_twin()
    y1 = layer(x, k)
    assert y1.dtype == torch.bfloat16 and torch.equal(y1, twin(x, k))
    cached = layer._cast.get("wg", layer.w_gate, torch.bfloat16)
    assert cached.dtype == torch.bfloat16
    assert layer._cast.get("wg", layer.w_gate, torch.bfloat16) is cached          # second use: no new cast
    with torch.no_grad():
        layer.w_gate.mul_(1.5)                                                     # in-place update
        layer.w_down.add_(0.01)
    fresh = layer._cast.get("wg", layer.w_gate, torch.bfloat16)
    assert fresh is not cached and torch.equal(fresh, layer.w_gate.detach().to(torch.bfloat16))
    sync_twin()
    y2 = layer(x, k)
    assert torch.equal(y2, twin(x, k)) and not torch.equal(y1, y2)
    # same dtype: the parameter itself is used, nothing is cached
    assert twin._cast.get("wg", twin.w_gate, torch.bfloat16).data_ptr() == twin.w_gate.data_ptr()
    # the MLP layer's caches behave the same way
    mlp = fm.FastMoELayer(d, h, o, E, dtype=torch.float32).to(DEV)
    ya = mlp(x, k)
    with torch.no_grad():
        mlp._experts_w.mul_(0.5)
        mlp._experts_bias.add_(1.0)
    yb = mlp(x, k)
    assert not torch.equal(ya, yb)
    ref = fm.FastMoELayer(d, h, o, E, dtype=torch.bfloat16).to(DEV)
    with torch.no_grad():
        for n in ("_experts_hidden_w", "_experts_hidden_bias", "_experts_w", "_experts_bias"):
            getattr(ref, n).copy_(getattr(mlp, n).to(torch.bfloat16))
        ref.gate.gate.weight.copy_(mlp.gate.gate.weight)
        ref.gate.gate.bias.copy_(mlp.gate.gate.bias)
    assert torch.equal(yb, ref(x, k))
    assert _lib.device_status(torch.device(DEV)) == 0


def test_quantized_weights_are_persistent_until_requantized():
    torch.manual_seed(1)
    layer = fm.SwiGLUFastMoELayer(64, 128, 64, 4, dtype=torch.bfloat16, fp8=True).to(DEV)
    x = torch.randn(1, 40, 64, device=DEV).bfloat16()
    y1 = layer(x, 2)
    q1 = layer._q["w_gate"][0]
    y1b = layer(x, 2)
    assert layer._q["w_gate"][0] is q1 and torch.equal(y1, y1b)     # no re-quantisation per forward
    with torch.no_grad():
        layer.w_gate.mul_(2.0)
    layer.quantize_weights()
    assert layer._q["w_gate"][0] is not q1
    assert not torch.equal(layer(x, 2), y1)
    assert _lib.device_status(torch.device(DEV)) == 0


def test_training_and_sparsely_gated_paths_accept_an_empty_batch():
    """Zero tokens through the differentiable paths and the sparsely-gated layer (inference, noisy
    gating, training with backward): shapes come back right, gradients are zeros, no status."""
    d, h, o, E, k = 64, 128, 64, 4, 2
    layer = fm.SwiGLUFastMoELayer(d, h, o, E, dtype=torch.bfloat16).to(DEV)
    layer.autograd = True
    x = torch.empty((1, 0, d), dtype=torch.bfloat16, device=DEV, requires_grad=True)
    y = layer(x, k)
    assert y.shape == (1, 0, o)
    y.sum().backward()
    assert x.grad.shape == x.shape
    for p in layer.parameters():
        assert p.grad is not None and float(p.grad.abs().sum()) == 0.0
    mlp = fm.FastMoELayer(d, h, o, E, dtype=torch.bfloat16).to(DEV)        # SiLU experts with biases
    mlp.autograd = True
    xm = torch.empty((1, 0, d), dtype=torch.bfloat16, device=DEV, requires_grad=True)
    mlp(xm, k).sum().backward()
    assert xm.grad.shape == xm.shape and all(p.grad is not None for p in mlp.parameters())
    nw, nb = torch.ones(d, device=DEV), torch.zeros(d, device=DEV)
    x2 = torch.empty((0, d), dtype=torch.bfloat16, device=DEV)
    for noisy in (False, True):
        sg = fm.SGMoELayer(d, o, fm.SGConfig(model_d=h, num_experts=E, num_activated_experts=k, enable_noisy_gating=noisy)).to(DEV)
        for train in (False, True):
            sg.train(train)
            out = sg(x2, None, 0, False, 1, d, nw, nb, 1e-5)
            assert out.x.shape == (0, o) and torch.isfinite(out.loss)
    sg = fm.SGMoELayer(d, o, fm.SGConfig(model_d=h, num_experts=E, num_activated_experts=k)).to(DEV)
    sg.train(True)
    sg.autograd = True
    xg = x2.clone().requires_grad_()
    out = sg(xg, None, 0, False, 1, d, nw, nb, 1e-5)
    (out.x.float().sum() + out.loss).backward()
    assert xg.grad.shape == (0, d)
    assert _lib.device_status(torch.device(DEV)) == 0


def test_two_weight_product_and_in_place_weights_at_the_small_end():
    """One expert, N = 64 (a single 64-column atom), a handful of rows; and zero rows."""
    E, K, N = 1, 64, 64
    off = torch.tensor([0, 5], dtype=torch.int64, device=DEV)
    x = torch.randn(5, K, device=DEV).bfloat16()
    w = (torch.randn(E, K, N, device=DEV) * 0.1).bfloat16()          # plain layout: N contiguous
    assert moe.prep_weight(w, K)[3] == 1
    got = moe.silu_jagged_bmm(off, x, w, None, has_silu=False)
    torch.testing.assert_close(got.float(), x.float() @ w[0].float(), atol=2e-2, rtol=2e-2)
    a = torch.randn(5, 2 * K, device=DEV).bfloat16()
    w1 = (torch.randn(E, K, N, device=DEV) * 0.1).bfloat16()
    two = moe.jagged_bmm_two_weights(off, a, w, w1)
    assert two is not None
    torch.testing.assert_close(two.float(), a[:, :K].float() @ w[0].float() + a[:, K:].float() @ w1[0].float(), atol=3e-2, rtol=2e-2)
    off0 = torch.zeros(2, dtype=torch.int64, device=DEV)
    empty = moe.jagged_bmm_two_weights(off0, torch.empty((0, 2 * K), dtype=torch.bfloat16, device=DEV), w, w1)
    assert empty is not None and empty.shape == (0, N)
    assert _lib.device_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("L,d,h,o,E,k", [
    (1, 8, 8, 8, 1, 1),          # one token, one expert, the smallest aligned sizes
    (17, 64, 96, 32, 4, 4),      # k == E: every expert for every token
    (255, 72, 200, 40, 3, 2),    # sizes that are multiples of 8 only; ragged tiles everywhere
    (257, 128, 64, 128, 32, 1),  # top-1 over many experts: most segments a handful of rows
    (33, 16, 24, 16, 5, 3),
])
@pytest.mark.parametrize("swiglu", [False, True])
def test_layers_at_degenerate_shapes_against_oracle(L, d, h, o, E, k, swiglu):
    """Both layers at the corners of their shape space, bf16, against the CPU oracle on the same
    inputs (rtol / atol 2e-2; tokens whose k-th / (k+1)-th gate scores nearly tie are counted)."""
    from oracle import moe_oracle as O

    torch.manual_seed(L * 7 + E)
    f = lambda p: p.detach().float().cpu()
    x = torch.randn(1, L, d).bfloat16()
    if swiglu:
        layer = fm.SwiGLUFastMoELayer(d, h, o, E, dtype=torch.bfloat16).to(DEV)
        y = layer(x.to(DEV), k)
        ref = O.moe_layer_swiglu(x.float(), f(layer.gate.gate.weight), f(layer.gate.gate.bias),
                                 f(layer.w_gate).permute(0, 2, 1), f(layer.w_up).permute(0, 2, 1),
                                 f(layer.w_down).permute(0, 2, 1), k)
    else:
        layer = fm.FastMoELayer(d, h, o, E, dtype=torch.bfloat16).to(DEV)
        with torch.no_grad():
            layer._experts_hidden_bias.normal_(0, 0.1)
            layer._experts_bias.normal_(0, 0.1)
        y = layer(x.to(DEV), k)
        ref = O.moe_layer_mlp(x.float(), f(layer.gate.gate.weight), f(layer.gate.gate.bias),
                                  f(layer._experts_hidden_w), f(layer._experts_hidden_bias),
                                  f(layer._experts_w), f(layer._experts_bias), k)
    assert y.shape == (1, L, o)
    err = (y.float().cpu() - ref).abs()
    bad = (err > 2e-2 + 2e-2 * ref.abs()).view(L, o).any(dim=1).float().mean().item()
    allowed = 0.0 if L < 50 else 0.02       # a near tie may route a token differently in a large batch
    assert bad <= allowed, f"{bad:.2%} of tokens out of tolerance, max err {err.max():.3e}"
    assert _lib.device_status(torch.device(DEV)) == 0

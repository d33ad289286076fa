"""Host-side layout decisions of the Python mirror (no GPU): which weight tensors the kernels read
in place and with which strides, and the row padding of the weight-gradient reduction."""
import torch

from fast_moe_b200.kernels import moe


def test_prep_weight_reads_both_reference_layouts_in_place():
    E, K, N = 3, 128, 192
    # FastMoELayer's view: storage [E, N, K], handed over as its permuted [E, K, N] view
    stored = torch.zeros(E, N, K, dtype=torch.bfloat16)
    w, se, sk, sn = moe.prep_weight(stored.permute(0, 2, 1), K)
    assert w.data_ptr() == stored.data_ptr() and (se, sk, sn) == (N * K, 1, K)
    # a plain contiguous [E, K, N] bf16 tensor with N a multiple of 64: in place, N contiguous
    plain = torch.zeros(E, K, N, dtype=torch.bfloat16)
    w, se, sk, sn = moe.prep_weight(plain, K)
    assert w.data_ptr() == plain.data_ptr() and (se, sk, sn) == (K * N, N, 1)
    # the same in float32, or with N not a multiple of 64, or switched off: transposed once
    for t in (torch.zeros(E, K, N), torch.zeros(E, K, 100, dtype=torch.bfloat16)):
        w, se, sk, sn = moe.prep_weight(t, K)
        assert w.data_ptr() != t.data_ptr() and sk == 1 and w.shape == (E, t.shape[2], K)
    moe.MN_MAJOR_WEIGHTS = False
    try:
        w, se, sk, sn = moe.prep_weight(plain, K)
        assert w.data_ptr() != plain.data_ptr() and sk == 1
    finally:
        moe.MN_MAJOR_WEIGHTS = True
    # K that needs padding to a 16-byte multiple: a padded K-contiguous copy either way
    odd = torch.zeros(E, 100, N, dtype=torch.bfloat16)
    w, se, sk, sn = moe.prep_weight(odd, 104)
    assert w.shape == (E, N, 104) and sk == 1


def test_prep_activation_pads_and_aligns():
    x = torch.zeros(5, 100, dtype=torch.bfloat16)
    assert moe.prep_activation(x, 104).shape == (5, 104)
    y = torch.zeros(5, 128, dtype=torch.bfloat16)
    assert moe.prep_activation(y, 128).data_ptr() == y.data_ptr()
    assert moe.prep_activation(y.t().contiguous().t(), 128).stride(1) == 1      # made row-contiguous

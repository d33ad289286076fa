"""The failure path of the kernels, exercised without faulting the GPU: a wait that can never be
satisfied runs into its (short) limit, the kernel records a status code and returns, the host
reads the code, and the same context then runs a normal operator correctly. Bad indices are
skipped and reported the same way."""
import time

import pytest
import torch

import fast_moe_b200 as fm
from fast_moe_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def test_bounded_wait_gives_up_and_reports():
    lib = _lib.load()
    torch.cuda.set_device(0)
    assert _lib.device_status(DEV) == 0
    t0 = time.perf_counter()
    _lib.check(lib.fmoe_selftest_bounded_wait(20000, torch.cuda.current_stream(DEV).cuda_stream))   # 20 ms limit
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert dt < 5.0, "the wait must end by itself"
    code = _lib.device_status(DEV)          # reads and clears
    assert code == 2, f"expected FMOE_DEV_WAIT_PRODUCER (2), got {code}"
    assert _lib.device_status(DEV) == 0
    with pytest.raises(_lib.FmoeError):
        _lib.check(lib.fmoe_selftest_bounded_wait(0, None))
    # the context is intact: a normal operator still gives the right answer
    idx = torch.tensor([[0, 1], [1, 0], [1, 2]], device=DEV)
    m = fm.route_metadata(idx, 3)
    assert m.offsets.tolist() == [0, 2, 5, 6]


def test_out_of_range_indices_are_skipped_and_reported():
    torch.cuda.set_device(0)
    E, k = 4, 2
    idx = torch.tensor([[0, 1], [7, 2], [3, -1]], device=DEV)      # 7 and -1 are not experts
    m = fm.route_metadata(idx, E)
    torch.cuda.synchronize()
    assert _lib.device_status(DEV) == 1                              # FMOE_DEV_BAD_INDEX
    assert m.lengths.tolist() == [1, 1, 1, 1]                        # the four valid picks were counted
    # a gather index beyond the token matrix: the GEMM reads row 0 instead and reports
    x = torch.randn(8, 64, device=DEV).bfloat16()
    w = torch.randn(1, 64, 64, device=DEV).bfloat16().permute(0, 2, 1)
    off = torch.tensor([0, 4], device=DEV)
    index = torch.tensor([[0], [1], [999], [3]], device=DEV)
    with pytest.raises(AssertionError):
        fm.index_select_jagged_bmm(0, off, index, x, w, None)        # the reference's shape assert still holds
    index = torch.tensor([0, 1, 999, 3, 0, 0, 0, 0], device=DEV).view(8, 1)
    out = fm.index_select_jagged_bmm(0, off, index, x, w, None)
    torch.cuda.synchronize()
    assert _lib.device_status(DEV) == 1
    assert torch.isfinite(out[:4].float()).all()

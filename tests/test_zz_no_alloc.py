"""The allocation-free routing entry point (fmoe_route_metadata_static).

Who needs it: callers that may not call cudaMalloc - code running inside a framework's
pre-planned memory region, plugins that are handed only their input and output buffers, services
with a fixed device-memory budget. They cannot supply the scratch table fmoe_route_metadata asks
for, so this variant keeps it inside the library. The test calls it through the C ABI on buffers
the caller owns and checks, twice in a row and on different inputs, that every output equals what
the workspace-taking entry point produces (integer results: equal bit for bit), and that a problem
beyond the built-in table is refused with a clear message rather than overrunning it.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import pytest
import torch

from fast_moe_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _route(entry, idx, E, with_workspace):
    lib = _lib.load()
    L, k = idx.shape
    i64 = dict(dtype=torch.int64, device=DEV)
    # poison the outputs so stale values cannot pass for results
    out = dict(lengths=torch.full((E,), -7, **i64), offsets=torch.full((E + 1,), -7, **i64),
               gate_index=torch.full((L * k,), -7, **i64), token_index=torch.full((L * k,), -7, **i64),
               reverse_index=torch.full((L, k), -7, **i64), max_len=torch.full((1,), -7, **i64))
    args = [idx.data_ptr(), L, E, k, out["lengths"].data_ptr(), out["offsets"].data_ptr(),
            out["gate_index"].data_ptr(), out["token_index"].data_ptr(), out["reverse_index"].data_ptr(),
            out["max_len"].data_ptr()]
    stream = torch.cuda.current_stream(torch.device(DEV)).cuda_stream
    if with_workspace:
        nbytes = int(lib.fmoe_route_workspace_bytes(L, E, k))
        ws = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=DEV)
        rc = getattr(lib, entry)(*args, ws.data_ptr(), ws.numel(), stream)
    else:
        rc = getattr(lib, entry)(*args, stream)
    return rc, out


def test_static_scratch_routing_equals_workspace_routing_twice():
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(11)
    # every call reuses the table the previous one filled; the third case (157 blocks x 256 experts
    # = 40192 entries) is past the size the single-launch placement handles and takes the
    # count -> scan -> place path on the built-in table
    cases = [(3000, 64, 8), (777, 8, 2), (40000, 256, 2), (1000, 16, 4)]
    for L, E, k in cases:
        idx = torch.randn(L, E, generator=g).topk(k, dim=1).indices.to(DEV)
        rc_ref, ref = _route("fmoe_route_metadata", idx, E, True)
        rc, got = _route("fmoe_route_metadata_static", idx, E, False)
        torch.cuda.synchronize()
        assert rc_ref == 0 and rc == 0, _lib.load().fmoe_last_error()
        for name in ref:
            assert torch.equal(got[name], ref[name]), f"{name} differs for L={L} E={E} k={k}"
        assert int(got["offsets"][-1]) == L * k
    assert _lib.device_status(torch.device(DEV)) == 0


def test_static_scratch_rejects_sizes_beyond_the_built_in_table():
    torch.cuda.set_device(0)
    lib = _lib.load()
    L, E, k = 70000, 256, 1                         # ceil(70000/256) * 256 = 70144 > 65536 entries
    idx = torch.zeros((L, k), dtype=torch.int64, device=DEV)
    rc, _ = _route("fmoe_route_metadata_static", idx, E, False)
    assert rc == _lib.FMOE_ERR_UNSUPPORTED
    msg = lib.fmoe_last_error().decode()
    assert "65536" in msg and "fmoe_route_metadata" in msg
    # the workspace-taking entry point still serves that size
    rc, out = _route("fmoe_route_metadata", idx, E, True)
    torch.cuda.synchronize()
    assert rc == 0 and int(out["offsets"][-1]) == L * k and int(out["lengths"][0]) == L

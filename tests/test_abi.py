"""CPU-side checks of the drop-in boundary: the shared library builds, loads and exports every
symbol include/fmoe_b200.h declares, the ctypes table agrees with the header, argument
validation answers with error codes (no GPU needed for those), and the Python operators keep
the reference's signatures and refuse CPU tensors instead of falling back."""
import ctypes
import inspect
import os
import re

import pytest
import torch

import fast_moe_b200 as fm
from fast_moe_b200 import _lib
from fast_moe_b200.kernels import moe, moe_fp8

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fmoe_b200.h")


def _header_decls():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    decls = {}
    for m in re.finditer(r"\b(?:int|size_t|long long|const char\*)\s+(fmoe_\w+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        args = m.group(2).strip()
        n = 0 if args in ("", "void") else len(args.split(","))
        decls[m.group(1)] = n
    return decls


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    decls = _header_decls()
    assert len(decls) >= 15
    for name, nargs in decls.items():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
        assert len(_lib.SIGNATURES[name][1]) == nargs, f"{name}: ctypes table has the wrong argument count"
    assert set(_lib.SIGNATURES) == set(decls)
    assert lib.fmoe_version() >= 100


def test_argument_validation_returns_status_not_crash():
    lib = _lib.load()
    # k > E
    rc = lib.fmoe_gate_topk(None, _lib.F32, 0, None, None, None, 0, 0, 4, 8, 4, 5, None, None, None, None)
    assert rc == _lib.FMOE_ERR_BAD_ARG
    assert b"k=5" in lib.fmoe_last_error()
    # missing workspace
    rc = lib.fmoe_route_metadata(None, 16, 4, 2, None, ctypes.c_void_p(16), None, None, None, None, None, 0, None)
    assert rc == _lib.FMOE_ERR_BAD_ARG
    # a weight with neither K nor N contiguous is refused, never silently transposed (so is an
    # N-contiguous one outside bf16 with N a multiple of 64)
    rc = lib.fmoe_index_select_jagged_bmm(ctypes.c_void_p(16), ctypes.c_void_p(16), 2, 8, ctypes.c_void_p(16),
                                          _lib.BF16, 4, 64, ctypes.c_void_p(16), 64 * 128, 128, 2, None, 0, 2, 64, 64,
                                          0, ctypes.c_void_p(16), _lib.BF16, 64, None)
    assert rc == _lib.FMOE_ERR_UNSUPPORTED
    rc = lib.fmoe_index_select_jagged_bmm(ctypes.c_void_p(16), ctypes.c_void_p(16), 2, 8, ctypes.c_void_p(16),
                                          _lib.F32, 4, 64, ctypes.c_void_p(16), 64 * 64, 64, 1, None, 0, 2, 64, 64,
                                          0, ctypes.c_void_p(16), _lib.F32, 64, None)
    assert rc == _lib.FMOE_ERR_UNSUPPORTED
    assert b"contiguous" in lib.fmoe_last_error()
    with pytest.raises(_lib.FmoeError):
        _lib.check(rc)
    assert lib.fmoe_route_workspace_bytes(1000, 8, 2) == 4 * 8 * 4


REFERENCE_SIGNATURES = {
    # kernels/moe.py:39-48, :71-80, :156-166, :192-203, :236-249
    moe.index_select_jagged_bmm: ["max_seq_len", "offsets", "index", "jagged", "weight", "bias", "kernel", "triton_option"],
    moe.index_select_jagged_bmm_3D: ["max_seq_len", "offsets", "index", "jagged", "weight", "bias", "kernel"],   # :118-126
    moe.mul_merge_k_add: ["index", "reverse_index", "value", "stable_sorting", "weight", "weight_index", "kernel",
                          "triton_cc_version"],
    moe.index_select_jagged_bmm_swiglu: ["max_seq_len", "offsets", "index", "jagged", "weight", "bias", "weight_p",
                                         "bias_p", "kernel"],
    moe.index_select_jagged_gating_bmm: ["max_seq_len", "offsets", "index", "jagged_a", "jagged_b", "weight_a", "bias_a",
                                         "weight_b", "bias_b", "kernel"],
    moe.silu_jagged_bmm_combine: ["max_seq_len", "offsets", "jagged", "weight", "bias", "index", "reverse_index",
                                  "gating_scores", "gates_index", "has_silu", "kernel", "triton_option"],
    # kernels/moe_fp8.py:31-40, :77-80, :98-105, :127-140, :185-194
    moe_fp8.silu_jagged_fp8: ["seq_offsets", "Jagged", "max_seq_len", "K", "Silu_Jagged", "Silu_Jagged_fp8",
                              "Silu_Jagged_Scale", "kernel"],
    moe_fp8.bmm_weight_rowwise_quant_fp8: ["weight", "kernel"],
    moe_fp8.silu_jagged_bmm_fp8: ["seq_offsets", "max_seq_len", "jagged", "weight", "bias", "kernel"],
    moe_fp8.silu_jagged_bmm_combine_fp8: ["max_seq_len", "offsets", "jagged", "weight", "bias", "index", "reverse_index",
                                          "gating_scores", "gates_index", "activation_checkpointing", "has_silu",
                                          "kernel"],
    moe_fp8.index_select_jagged_bmm: ["max_seq_len", "offsets", "index", "jagged", "weight", "bias", "kernel", "fp8"],
}


def test_operator_signatures_match_reference():
    for fn, names in REFERENCE_SIGNATURES.items():
        params = [p.name for p in inspect.signature(fn).parameters.values() if p.kind != p.KEYWORD_ONLY]
        assert params == names, fn.__name__


@pytest.mark.skipif(not os.environ.get("FAST_MOE_REFERENCE"), reason="FAST_MOE_REFERENCE (a reference checkout) is not set")
def test_operator_signatures_match_the_live_reference():
    """With a checkout of the reference at hand, the hand-written table above is checked against
    inspect.signature of the reference's own callables (imported unmodified through the shims)."""
    from oracle import reference_shims

    ref = reference_shims.modules()
    pairs = [
        (moe.index_select_jagged_bmm, ref.moe.index_select_jagged_bmm),
        (moe.mul_merge_k_add, ref.moe.mul_merge_k_add),
        (moe.index_select_jagged_bmm_3D, ref.moe.index_select_jagged_bmm_3D),
        (moe.index_select_jagged_bmm_swiglu, ref.moe.index_select_jagged_bmm_swiglu),
        (moe.index_select_jagged_gating_bmm, ref.moe.index_select_jagged_gating_bmm),
        (moe.silu_jagged_bmm_combine, ref.moe.silu_jagged_bmm_combine),
        (moe_fp8.silu_jagged_fp8, ref.moe_fp8.silu_jagged_fp8),
        (moe_fp8.bmm_weight_rowwise_quant_fp8, ref.moe_fp8.bmm_weight_rowwise_quant_fp8),
        (moe_fp8.silu_jagged_bmm_fp8, ref.moe_fp8.silu_jagged_bmm_fp8),
        (moe_fp8.silu_jagged_bmm_combine_fp8, ref.moe_fp8.silu_jagged_bmm_combine_fp8),
        (moe_fp8.index_select_jagged_bmm, ref.moe_fp8.index_select_jagged_bmm),
    ]
    for ours, theirs in pairs:
        mine = [(p.name, p.default if p.default is inspect.Parameter.empty or not hasattr(p.default, "name") else p.default.name)
                for p in inspect.signature(ours).parameters.values() if p.kind != p.KEYWORD_ONLY]
        want = [(p.name, p.default if p.default is inspect.Parameter.empty or not hasattr(p.default, "name") else p.default.name)
                for p in inspect.signature(theirs).parameters.values()]
        assert mine == want, ours.__name__
    rl, ol = ref.layer.FastMoELayer, fm.FastMoELayer
    assert list(inspect.signature(ol.__init__).parameters) == list(inspect.signature(rl.__init__).parameters)
    assert list(inspect.signature(ol.forward).parameters) == list(inspect.signature(rl.forward).parameters)
    torch.manual_seed(0)
    assert sorted(ol(8, 16, 8, 2).state_dict()) == sorted(rl(8, 16, 8, 2).state_dict())


def test_layer_keeps_reference_parameter_names_and_signature():
    layer = fm.FastMoELayer(16, 32, 24, 4, fm.KernelType.PYTORCH, torch.float32)
    assert sorted(layer.state_dict()) == ["_experts_bias", "_experts_hidden_bias", "_experts_hidden_w", "_experts_w",
                                          "gate.gate.bias", "gate.gate.weight"]
    assert tuple(layer._experts_hidden_w.shape) == (4, 32, 16)
    assert tuple(layer._experts_w.shape) == (4, 24, 32)
    assert list(inspect.signature(fm.FastMoELayer.__init__).parameters)[1:] == [
        "input_dim", "hidden_dim", "output_dim", "num_experts", "kernel", "dtype"]
    assert list(inspect.signature(fm.FastMoELayer.forward).parameters)[1:] == ["x", "num_experts_per_tok"]


def test_no_cpu_fallback():
    layer = fm.FastMoELayer(16, 32, 16, 4, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        layer(torch.randn(2, 4, 16), 2)
    off = torch.tensor([0, 4, 8])
    idx = torch.arange(8).view(4, 2)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        moe.index_select_jagged_bmm(4, off, idx, torch.randn(4, 16), torch.randn(2, 16, 8), None)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        moe_fp8.rowwise_quant_fp8(torch.randn(4, 16))


def test_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "fast_moe_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"

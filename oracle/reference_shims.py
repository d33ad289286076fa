"""Imports the UNMODIFIED reference (meta-recsys/fast_moe) from a checkout so that its
KernelType.PYTORCH path can run on CPU. TEST INFRASTRUCTURE ONLY: used by
oracle/check_against_reference.py and tests/golden/make_golden.py on a machine that has the
reference checkout; nothing that runs on a GPU box imports this file.

The reference cannot be imported as shipped outside its home monorepo:
  * its root __init__ pulls in the Triton backend, which needs the absent ``mslk`` package and a
    Triton fork (kernels/triton/grouped_gemm.py:14,47-59);
  * kernels/moe.py:35-36 calls torch.ops.load_library on Buck targets ("//deeplearning/...");
  * modules/fast_moe_module.py:131 needs torch.ops.fbgemm.asynchronous_complete_cumsum;
  * the checkout directory is not named ``fast_moe``.
The shims below are harness-side only; no reference file is touched or copied.
"""
from __future__ import annotations

import importlib
import os
import sys
import types
from dataclasses import dataclass

import torch


def reference_root(root=None) -> str:
    """The reference checkout to import from: the argument, else the FAST_MOE_REFERENCE environment
    variable. There is no built-in default: the location is the caller's to state."""
    root = root or os.environ.get("FAST_MOE_REFERENCE")
    if not root:
        raise FileNotFoundError(
            "no reference checkout given: pass its path (--reference) or set FAST_MOE_REFERENCE to a clone of "
            "meta-recsys/fast_moe")
    return root


_installed = False
_fbgemm_lib = None


def _namespace(name: str, path: str) -> types.ModuleType:
    m = types.ModuleType(name)
    m.__path__ = [path]  # type: ignore[attr-defined]
    m.__package__ = name
    sys.modules[name] = m
    return m


def install(root=None) -> None:
    """Registers ``fast_moe`` and its sub-packages as namespace modules pointing into `root`
    (so the root __init__ never runs) and stubs what the PYTORCH path does not need."""
    global _installed, _fbgemm_lib
    if _installed:
        return
    root = reference_root(root)
    if not os.path.isdir(root):
        raise FileNotFoundError(f"reference checkout not found at {root}")
    _namespace("fast_moe", root)
    for sub in ("kernels", "kernels/pytorch", "kernels/triton", "modules", "utils"):
        _namespace("fast_moe." + sub.replace("/", "."), os.path.join(root, sub))

    def _unavailable(*_a, **_k):
        raise NotImplementedError("the reference's Triton backend is not runnable here")

    # names kernels/moe.py:21-30 imports from the Triton backend
    @dataclass
    class IndexSelectJaggedBmmOption:
        d_weight_optimization: bool = False

    @dataclass
    class SiluJaggedBmmCombineOption:
        activation_checkpointing: bool = False
        d_weight_optimization: bool = False
        d_weight_split_k_kernel: bool = False
        d_weight_split_k_kernel_tma: bool = False

    tm = types.ModuleType("fast_moe.kernels.triton.triton_moe")
    tm.IndexSelectJaggedBmmOption = IndexSelectJaggedBmmOption
    tm.SiluJaggedBmmCombineOption = SiluJaggedBmmCombineOption
    for n in (
        "triton_index_select_jagged_bmm_3D_wrapper",
        "triton_index_select_jagged_bmm_swiglu_wrapper",
        "triton_index_select_jagged_bmm_wrapper",
        "triton_index_select_jagged_gating_bmm_wrapper",
        "triton_mul_merge_k_add_wrapper",
        "triton_silu_jagged_bmm_combine_wrapper",
    ):
        setattr(tm, n, _unavailable)
    sys.modules[tm.__name__] = tm
    # names kernels/moe_fp8.py:21-27 imports
    tf = types.ModuleType("fast_moe.kernels.triton.triton_moe_fp8")
    for n in (
        "triton_bmm_weight_rowwise_quant_fp8",
        "triton_index_select_jagged_bmm_fp8",
        "triton_silu_jagged_bmm_combine_fp8",
        "triton_silu_jagged_bmm_fp8",
        "triton_silu_jagged_fp8",
    ):
        setattr(tf, n, _unavailable)
    sys.modules[tf.__name__] = tf

    real_load = torch.ops.load_library

    def load_library(path):
        if isinstance(path, str) and path.startswith("//"):
            return None
        return real_load(path)

    torch.ops.load_library = load_library  # type: ignore[assignment]

    # fbgemm's exclusive cumsum with the total appended (integer arithmetic)
    if not hasattr(torch.ops, "fbgemm") or not hasattr(torch.ops.fbgemm, "asynchronous_complete_cumsum"):
        _fbgemm_lib = torch.library.Library("fbgemm", "DEF")
        _fbgemm_lib.define("asynchronous_complete_cumsum(Tensor t) -> Tensor")

        def _cumsum(t):
            return torch.cat([t.new_zeros(1), t.cumsum(0)])

        _fbgemm_lib.impl("asynchronous_complete_cumsum", _cumsum, "CompositeExplicitAutograd")
    _installed = True


def modules(root=None):
    """Returns the reference modules on the MoE forward path, imported in place."""
    install(root)
    names = {
        "moe": "fast_moe.kernels.moe",
        "moe_fp8": "fast_moe.kernels.moe_fp8",
        "pt_moe": "fast_moe.kernels.pytorch.moe",
        "pt_moe_fp8": "fast_moe.kernels.pytorch.moe_fp8",
        "pt_quant": "fast_moe.kernels.pytorch.quant_fp8",
        "layer": "fast_moe.modules.fast_moe_module",
        "dense": "fast_moe.modules.moe_base",
        "utils": "fast_moe.kernels.utils",
    }
    return types.SimpleNamespace(**{k: importlib.import_module(v) for k, v in names.items()})

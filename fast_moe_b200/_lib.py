"""ctypes binding of libfmoe_b200.so (the C ABI declared in include/fmoe_b200.h).

There is no CPU or PyTorch fallback: if the library is missing and cannot be built, or a call
returns an error status, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_longlong, c_size_t, c_void_p
from pathlib import Path
from typing import Optional

import torch

FMOE_OK = 0
FMOE_ERR_BAD_ARG = -1
FMOE_ERR_UNSUPPORTED = -2
FMOE_ERR_CUDA = -3
FMOE_ERR_DEVICE = -4

F32, BF16, E4M3 = 0, 1, 3
EPI_NONE, EPI_SILU, EPI_SWIGLU = 0, 1, 2
COMBINE_ACCUMULATE, COMBINE_ROUND_GATE = 1, 2      # flags of fmoe_silu_jagged_bmm_combine_fused

DEV_STATUS_NAMES = {
    0: "ok",
    1: "an index or expert id outside its range was skipped",
    2: "producer wait ran out",
    3: "MMA wait ran out",
    4: "epilogue wait ran out",
}

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfmoe_b200.so"
_lib: Optional[ctypes.CDLL] = None


class FmoeError(RuntimeError):
    """A call into libfmoe_b200 returned a non-zero status."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"libfmoe_b200 status {code}: {msg}")
        self.code = code


# name -> (restype, argtypes); must list every symbol include/fmoe_b200.h declares.
P = c_void_p
I64 = c_int64
SIGNATURES = {
    "fmoe_version": (c_int, []),
    "fmoe_last_error": (c_char_p, []),
    "fmoe_device_status": (c_int, [P, c_int, P]),
    "fmoe_kernel_launch_count": (c_longlong, []),
    "fmoe_selftest_bounded_wait": (c_int, [I64, P]),
    "fmoe_gate_topk": (c_int, [P, c_int, I64, P, P, P, I64, c_int, I64, c_int, c_int, c_int, P, P, P, P]),
    "fmoe_gate_topk_counts_supported": (c_int, [P, c_int, I64, P, I64, c_int, c_int]),
    "fmoe_route_group_counts_bytes": (c_size_t, [I64, c_int]),
    "fmoe_gate_topk_counts": (c_int, [P, c_int, I64, P, P, I64, c_int, c_int, c_int, P, P, P, P, P, c_int, I64, c_int, P]),
    "fmoe_route_metadata_gather": (c_int, [P, I64, c_int, c_int, P, P, P, P, P, P, P, P, c_int, I64, c_int, P, I64, P,
                                           c_int, I64, c_int, P]),
    "fmoe_gate_topk_normalized": (c_int, [P, c_int, I64, P, P, P, I64, I64, c_int, c_int, c_int, P, P, P, P]),
    "fmoe_token_norm": (c_int, [P, c_int, I64, c_int, I64, c_int, P, P, c_int, c_float, P, I64, P]),
    "fmoe_sg_load_loss": (c_int, [P, P, P, c_int, c_int, c_float, c_int, P, c_int, P, P, P]),
    "fmoe_token_norm_backward": (c_int, [P, P, c_int, I64, c_int, I64, I64, c_int, P, c_int, c_float, P, I64, P, P, c_int, P, P, P]),
    "fmoe_sg_router_backward": (c_int, [P, P, P, I64, c_int, c_int, P, P]),
    "fmoe_sg_loss_backward": (c_int, [P, P, P, c_int, c_int, c_float, P, P, P, c_int, P, P]),
    "fmoe_sg_noisy_router_backward": (c_int, [P, I64, P, P, P, P, P, P, I64, c_int, c_int, P, I64, P]),
    "fmoe_jagged_bmm_two_weights": (c_int, [P, I64, P, c_int, I64, P, P, c_int, I64, I64, I64, c_int, c_int, c_int, P, c_int, I64, P]),
    "fmoe_sg_noisy_logits": (c_int, [P, I64, P, I64, c_int, c_float, P, P, P]),
    "fmoe_sg_noisy_load": (c_int, [P, I64, P, P, I64, c_int, c_int, P, c_int, P]),
    "fmoe_route_workspace_bytes": (c_size_t, [I64, c_int, c_int]),
    "fmoe_route_metadata": (c_int, [P, I64, c_int, c_int, P, P, P, P, P, P, P, c_size_t, P]),
    "fmoe_route_metadata_static": (c_int, [P, I64, c_int, c_int, P, P, P, P, P, P, P]),
    "fmoe_index_select_jagged_bmm": (
        c_int,
        [P, P, c_int, I64, P, c_int, I64, I64, P, I64, I64, I64, P, I64, c_int, c_int, c_int, c_int, P, c_int, I64, P],
    ),
    "fmoe_index_select_jagged_bmm_mul": (
        c_int,
        [P, P, c_int, I64, P, c_int, I64, I64, P, I64, I64, I64, P, I64, c_int, c_int, c_int, P, I64, P, c_int, I64, P],
    ),
    "fmoe_index_select_jagged_bmm_swiglu": (
        c_int,
        [P, P, c_int, I64, P, c_int, I64, I64, P, P, I64, I64, I64, P, P, I64, c_int, c_int, c_int, P, c_int, I64, P],
    ),
    "fmoe_index_select_jagged_bmm_fp8": (
        c_int,
        [P, P, c_int, I64, P, P, I64, I64, P, P, P, P, I64, I64, I64, I64, P, P, I64, c_int, c_int, c_int, c_int, P,
         c_int, I64, P],
    ),
    "fmoe_silu_jagged_bmm": (
        c_int,
        [P, I64, P, c_int, I64, P, P, P, I64, I64, I64, I64, P, I64, c_int, c_int, c_int, c_int, P, P, P, P, c_int,
         I64, P],
    ),
    "fmoe_expand_3d_index": (c_int, [P, P, c_int, c_int, I64, P, P]),
    "fmoe_split_f32_bf16x3": (c_int, [P, I64, c_int, I64, c_int, c_int, c_int, P, I64, P]),
    "fmoe_gather_rows": (c_int, [P, c_int, I64, I64, P, c_int, I64, c_int, P, I64, P]),
    "fmoe_mul_merge_k_add": (c_int, [P, P, c_int, I64, P, c_int, P, I64, c_int, c_int, P, c_int, I64, P]),
    "fmoe_silu_jagged_bmm_combine": (
        c_int,
        [P, I64, P, c_int, I64, P, I64, I64, I64, P, I64, P, P, c_int, P, I64, c_int, c_int, c_int, c_int, c_int, P,
         P, P, c_int, I64, P],
    ),
    "fmoe_silu_jagged_bmm_combine_fused": (
        c_int,
        [P, I64, P, c_int, I64, P, P, P, I64, I64, I64, I64, P, I64, P, c_int, P, I64, c_int, c_int, c_int, c_int,
         c_int, P, P, c_int, I64, c_int, P],
    ),
    "fmoe_ep_plan": (c_int, [P, c_int, c_int, c_int, I64, P, P, P]),
    "fmoe_ep_dispatch": (c_int, [P, c_int, I64, I64, c_int, P, P, I64, c_int, c_int, c_int, P, P, P, I64, I64, P]),
    "fmoe_ep_up_projection": (c_int, [P, I64, I64, P, c_int, I64, P, P, I64, I64, c_int, c_int, c_int, P, I64, P]),
    "fmoe_ep_down_projection": (c_int, [P, I64, I64, P, c_int, I64, P, I64, I64, c_int, c_int, c_int, P, P, c_int, I64,
                                        I64, P]),
    "fmoe_router_backward": (c_int, [P, P, P, I64, c_int, c_int, P, P]),
    "fmoe_gate_linear_backward": (c_int, [P, P, c_int, I64, P, I64, c_int, c_int, P, I64, P, P, P]),
    "fmoe_batched_transpose": (c_int, [P, c_int, c_int, I64, I64, c_int, c_int, P, I64, I64, P]),
    "fmoe_jagged_pad_offsets": (c_int, [P, c_int, c_int, P, P]),
    "fmoe_jagged_transpose_pad": (c_int, [P, c_int, I64, I64, P, c_int, P, P, c_int, I64, c_int, P, I64, P]),
    "fmoe_jagged_jagged_bmm": (c_int, [P, P, I64, P, I64, P, I64, c_int, c_int, c_int, c_int, P, c_int, I64, P]),
    "fmoe_jagged_colsum": (c_int, [P, c_int, I64, P, c_int, c_int, P, c_int, P]),
    "fmoe_gather_scale_rows": (c_int, [P, c_int, I64, I64, P, c_int, P, c_int, P, I64, I64, c_int, P, I64, P]),
    "fmoe_row_dot": (c_int, [P, I64, P, I64, I64, c_int, P, c_int, I64, c_int, P, P]),
    "fmoe_activation_backward": (c_int, [c_int, P, I64, P, I64, P, I64, c_int, I64, c_int, P, I64, P, I64, P]),
    "fmoe_rowwise_quant_fp8": (c_int, [P, c_int, I64, c_int, I64, c_int, c_int, P, I64, P, P]),
    "fmoe_bmm_weight_quant_fp8": (c_int, [P, c_int, c_int, c_int, c_int, P, P, P]),
}


def lib_path() -> Path:
    return _LIB_PATH


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Loads the shared library, compiling it first when it is absent and nvcc is available."""
    global _lib
    if _lib is not None:
        return _lib
    from .build import build_library, library_is_current

    if not library_is_current():
        # missing, or built from other sources than the ones next to it: never run a stale library
        if not build_if_missing:
            raise FileNotFoundError(
                f"{_LIB_PATH} is missing or was not built from the sources beside it; run `python -m fast_moe_b200.build`")
        build_library()
    lib = ctypes.CDLL(os.fspath(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the export is missing: fail loudly
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != FMOE_OK:
        msg = load().fmoe_last_error()
        raise FmoeError(rc, msg.decode() if msg else "")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    if dt == torch.float8_e4m3fn or dt == torch.uint8:
        return E4M3
    raise TypeError(f"fast_moe_b200 kernels take float32, bfloat16 or float8_e4m3fn tensors, got {dt}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "fast_moe_b200 runs on CUDA tensors only (there is no CPU path); got a tensor on " + str(t.device)
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    assert dev is not None
    return dev


def device_status(device: Optional[torch.device] = None, reset: bool = True) -> int:
    """Reads (and by default clears) the status word kernels write when they skip bad input or
    give up a bounded wait. Synchronises the current stream."""
    lib = load()
    device = device or torch.device("cuda", torch.cuda.current_device())
    out = c_int(0)
    with torch.cuda.device(device):
        check(lib.fmoe_device_status(ctypes.byref(out), 1 if reset else 0, stream_ptr(device)))
    return out.value


def raise_on_device_status(device: Optional[torch.device] = None) -> None:
    code = device_status(device)
    if code != 0:
        raise FmoeError(FMOE_ERR_DEVICE, DEV_STATUS_NAMES.get(code, f"device status {code}"))


def kernel_launch_count() -> int:
    return int(load().fmoe_kernel_launch_count())


# ---------------------------------------------------------------------------- stage timing
class StageTimer:
    """Optional CUDA-event timing of the stages of a layer forward ("route", "up", "down",
    "combine", ...). Disabled unless a caller installs one with ``set_stage_timer``; events are
    recorded on the current stream, so they time exactly the kernels launched in between."""

    def __init__(self) -> None:
        self.pairs = {}

    def stage(self, name: str):
        return _Stage(self, name)

    def totals_ms(self):
        torch.cuda.synchronize()
        return {k: (sum(a.elapsed_time(b) for a, b in v), len(v)) for k, v in self.pairs.items()}


class _Stage:
    def __init__(self, timer: "StageTimer", name: str) -> None:
        self.timer, self.name = timer, name

    def __enter__(self):
        self.a = torch.cuda.Event(enable_timing=True)
        self.b = torch.cuda.Event(enable_timing=True)
        self.a.record()
        return self

    def __exit__(self, *exc):
        self.b.record()
        self.timer.pairs.setdefault(self.name, []).append((self.a, self.b))
        return False


class _NoStage:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_STAGE = _NoStage()
_stage_timer: Optional[StageTimer] = None


def set_stage_timer(t: Optional[StageTimer]) -> None:
    global _stage_timer
    _stage_timer = t


def stage(name: str):
    return _NO_STAGE if _stage_timer is None else _stage_timer.stage(name)

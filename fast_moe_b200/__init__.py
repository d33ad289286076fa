"""fast_moe_b200: the FastMoE mixture-of-experts forward path on hand-written sm_100a CUDA
kernels (tcgen05 grouped GEMMs fed by TMA, routing / combine / FP8-quantisation kernels) behind
the operator and module signatures of meta-recsys/fast_moe. The kernels live in
``lib/libfmoe_b200.so`` (C ABI: include/fmoe_b200.h); there is no CPU or PyTorch fallback."""
from .kernels.moe import (
    IndexSelectJaggedBmmOption,
    SiluJaggedBmmCombineOption,
    index_select_jagged_bmm,
    index_select_jagged_bmm_swiglu,
    index_select_jagged_bmm_3D,
    index_select_jagged_gating_bmm,
    fp32_uses_tf32,
    mul_merge_k_add,
    set_fp32_matmul,
    silu_jagged_bmm,
    silu_jagged_bmm_combine,
)
from .kernels.routing import RoutingMetadata, gate_topk, gate_topk_normalized, route_metadata, token_norm
from .kernels.utils import KernelType
from .modules.fast_moe_module import (CapturedForward, CapturedTrainStep, FastMoELayer, GatingNetwork, HostPipeline, StreamingForward,
                                      SwiGLUFastMoELayer)
from .modules.sg_moe import MRNOutput, SGConfig, SGMoELayer

__all__ = [
    "FastMoELayer",
    "GatingNetwork",
    "SwiGLUFastMoELayer",
    "CapturedForward",
    "CapturedTrainStep",
    "StreamingForward",
    "HostPipeline",
    "KernelType",
    "IndexSelectJaggedBmmOption",
    "SiluJaggedBmmCombineOption",
    "index_select_jagged_bmm",
    "index_select_jagged_bmm_3D",
    "index_select_jagged_bmm_swiglu",
    "index_select_jagged_gating_bmm",
    "mul_merge_k_add",
    "silu_jagged_bmm",
    "silu_jagged_bmm_combine",
    "set_fp32_matmul",
    "fp32_uses_tf32",
    "SGMoELayer",
    "SGConfig",
    "MRNOutput",
    "gate_topk_normalized",
    "token_norm",
    "gate_topk",
    "route_metadata",
    "RoutingMetadata",
]

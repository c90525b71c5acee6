"""B200-native (sm_100a) fused Mixture-of-Experts path behind the FlagGems-vllm
operator names: ``grouped_topk``, ``moe_align_block_size`` and
``fused_experts_impl`` with their companions.  All compute runs in hand-written
CUDA kernels reached through the C ABI of ``libmoe_sm100.so``."""

from ._lib import MoeKernelError, read_status  # noqa: F401
from .activation import silu_and_mul, silu_and_mul_out  # noqa: F401
from .align import (  # noqa: F401
    moe_align_block_size,
    moe_align_block_size_no_tle,
    moe_align_block_size_triton,
)
from .fused_moe import (  # noqa: F401
    fused_experts_impl,
    inplace_fused_experts,
    outplace_fused_experts,
)
from .quant import SUPPORTED_FP8_DTYPE, moe_sum, per_token_group_quant_fp8  # noqa: F401
from .router_gemm import (  # noqa: F401
    fp32_router_gemm,
    router_gemm,
    router_gemm_grouped_topk,
    supports_fp32_router_gemm,
)
from .routing import grouped_topk, topk_sigmoid, topk_softmax  # noqa: F401

# compatibility alias kept by the reference (src/flaggems_vllm/__init__.py:40-49)
ops_experts_impl = fused_experts_impl

device = "cuda"
vendor_name = "nvidia"
__version__ = "0.1.0"

__all__ = [
    "grouped_topk", "moe_align_block_size", "moe_align_block_size_triton", "moe_align_block_size_no_tle",
    "fused_experts_impl", "inplace_fused_experts", "outplace_fused_experts", "ops_experts_impl", "moe_sum",
    "per_token_group_quant_fp8", "SUPPORTED_FP8_DTYPE", "read_status", "MoeKernelError", "topk_softmax",
    "topk_sigmoid", "router_gemm", "fp32_router_gemm", "supports_fp32_router_gemm", "router_gemm_grouped_topk",
    "silu_and_mul", "silu_and_mul_out",
]

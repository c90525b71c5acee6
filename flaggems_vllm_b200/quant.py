"""per_token_group_quant_fp8 and moe_sum: thin host wrappers.

Signatures follow src/flaggems_vllm/ops/per_token_group_quant_fp8.py:226-233
and src/flaggems_vllm/ops/moe_sum.py:250-253."""

from __future__ import annotations

import logging
from typing import Optional, Tuple

import torch

from . import _lib

logger = logging.getLogger(__name__)

SUPPORTED_FP8_DTYPE = torch.float8_e4m3fn


def per_token_group_quant_fp8(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    dtype: Optional[torch.dtype] = None,
    column_major_scales: bool = False,
    scale_ue8m0: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """1 x group_size e4m3 quantisation of the last dimension.

    Returns (x_q, x_s) with x_s of shape x.shape[:-1] + (cols / group_size,),
    column-major in memory when ``column_major_scales``."""
    logger.debug("GEMS PER TOKEN GROUP QUANT FP8")
    fp8_dtype = SUPPORTED_FP8_DTYPE if dtype is None else dtype
    assert x.shape[-1] % group_size == 0, (
        f"the last dimension of `x` {x.shape[-1]} must be divisible by `group_size` {group_size}"
    )
    assert x.stride(-1) == 1, "`x` groups must be contiguous"
    _lib.require_cuda(x, "per_token_group_quant_fp8")
    if fp8_dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise NotImplementedError(f"8-bit float format {fp8_dtype} is not implemented (e4m3fn and e5m2 are)")
    xc = x if x.is_contiguous() else x.contiguous()
    cols = xc.shape[-1]
    rows = xc.numel() // cols if cols else 0
    x_q = torch.empty(xc.shape, device=x.device, dtype=fp8_dtype)
    groups = cols // group_size
    lead = rows
    if column_major_scales:
        if xc.ndim != 2:
            raise ValueError("column-major scales need a 2-D input (the reference's (-1, -2) permutation of a "
                             "[groups, rows] buffer)")
        # the reference lays the scales out as [groups, *leading dims] and returns the (-1, -2) permutation
        x_s = torch.empty((groups,) + tuple(xc.shape[:-1]), device=x.device, dtype=torch.float32)
    else:
        x_s = torch.empty(tuple(xc.shape[:-1]) + (groups,), device=x.device, dtype=torch.float32)
    flags = int(column_major_scales) | (2 if scale_ue8m0 else 0)
    if group_size == 128 and fp8_dtype == torch.float8_e4m3fn and abs(eps - 1e-10) <= 1e-16:
        rc = _lib.lib().moe_per_token_group_quant_fp8(
            xc.data_ptr(), _lib.dtype_code(xc.dtype), rows, cols, group_size, x_q.data_ptr(), x_s.data_ptr(), flags,
            lead, _lib.stream_of(x))
    else:
        rc = _lib.lib().moe_per_token_group_quant_fp8_ex(
            xc.data_ptr(), _lib.dtype_code(xc.dtype), rows, cols, group_size, float(eps),
            int(fp8_dtype == torch.float8_e5m2), x_q.data_ptr(), x_s.data_ptr(), flags, lead, _lib.stream_of(x))
    _lib.check(rc)
    if column_major_scales:
        x_s = x_s.permute(-1, -2)
    return x_q, x_s


def moe_sum(input: torch.Tensor, output: torch.Tensor):
    """output[m, :] = sum over the top-k axis of input[m, :, :] (fp32 accumulate)."""
    logger.debug("GEMS MOE SUM")
    if input.ndim != 3 or output.ndim != 2:
        raise ValueError("moe_sum expects input [M, topk, H] and output [M, H]")
    M, topk, H = input.shape
    if output.shape != (M, H) or output.dtype != input.dtype or output.device != input.device:
        raise ValueError("moe_sum: output must be [M, H] with the dtype and device of input")
    _lib.require_cuda(input, "moe_sum")
    src = input if input.is_contiguous() else input.contiguous()
    # rows of the output may be any number of elements apart (a window of a wider tensor); only
    # non-contiguous columns go through a temporary
    direct = M == 0 or H == 1 or output.stride(1) == 1
    dst = output if direct else torch.empty_like(output, memory_format=torch.contiguous_format)
    rc = _lib.lib().moe_sum_ld(src.data_ptr(), dst.data_ptr(), dst.stride(0) if M > 0 and dst.stride(0) >= H else H,
                               _lib.dtype_code(src.dtype), M, topk, H, None, 0, 0, None, None, _lib.stream_of(input))
    _lib.check(rc)
    if dst is not output:
        output.copy_(dst)

"""grouped_topk: host side of the warp-per-token routing kernel.

Signature, argument checks and error types mirror the reference function
(src/flaggems_vllm/ops/grouped_topk.py:1674-1739)."""

from __future__ import annotations

import logging
from typing import Optional

import torch

from . import _lib

logger = logging.getLogger(__name__)


def _validate_padding(scores, bias, is_padding, n_group, topk_group, topk):
    # mirrors src/flaggems_vllm/ops/grouped_topk.py:1638-1671
    rows, experts = scores.shape
    if (
        is_padding.dtype != torch.bool
        or is_padding.shape != (rows,)
        or is_padding.device != scores.device
        or not is_padding.is_contiguous()
    ):
        raise ValueError("is_padding must be contiguous bool [num_tokens] on the scores device")
    if (
        bias.shape != (experts,)
        or bias.device != scores.device
        or not bias.is_contiguous()
        or scores.stride(1) != 1
        or scores.stride(0) < experts
    ):
        raise ValueError("masked grouped_topk needs row-major scores and contiguous same-device bias")
    if not 1 <= topk_group <= n_group <= 32 or not 1 <= topk <= 32:
        raise ValueError("expected valid group counts and topk in [1, 32]")
    if experts // n_group < 2 or experts > 4096 or topk > (experts // n_group) * topk_group:
        raise ValueError(
            "masked grouped_topk needs at least 2 experts per group, at most 4096 "
            "experts, and at least topk candidates after group selection"
        )


def grouped_topk(
    scores: torch.Tensor,
    n_group: int,
    topk_group: int,
    topk: int,
    renormalize: bool,
    routed_scaling_factor: float,
    bias: torch.Tensor,
    scoring_func: int = 0,
    is_padding: Optional[torch.Tensor] = None,
):
    """Route scores; optional padding rows emit zero weights and -1 ids.

    Returns (topk_weights fp32 [M, topk], topk_ids int32 [M, topk])."""
    logger.debug("GEMS GROUPED TOPK")
    if scores.ndim != 2:
        raise ValueError("scores must be a 2D Tensor")
    num_tokens, num_experts = scores.shape
    if is_padding is not None:
        _validate_padding(scores, bias, is_padding, n_group, topk_group, topk)
    if num_experts % n_group != 0:
        raise ValueError("num_experts must be divisible by n_group")
    if n_group > 32:
        raise ValueError("n_group should be smaller than or equal to 32")
    if topk > 32:
        raise ValueError("topk should be smaller than or equal to 32 for now")
    if scoring_func not in (0, 1):
        raise ValueError("scoring_func must be 0 (none) or 1 (sigmoid)")
    if bias.ndim != 1:
        bias = bias.flatten()
    if len(bias) != num_experts:
        raise ValueError(f"bias length ({len(bias)}) must match num_experts ({num_experts})")
    sdt = _lib.dtype_code(scores.dtype)  # ValueError("Unsupported dtype") like the reference
    if bias.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        bias = bias.float()
    if not bias.is_contiguous():
        bias = bias.contiguous()
    if bias.device != scores.device:
        raise ValueError("bias must be on the scores device")

    _lib.require_cuda(scores, "grouped_topk")
    weights = torch.empty((num_tokens, topk), device=scores.device, dtype=torch.float32)
    ids = torch.empty((num_tokens, topk), device=scores.device, dtype=torch.int32)
    if num_tokens == 0:
        return weights, ids
    pad = is_padding.view(torch.uint8) if is_padding is not None else None
    rc = _lib.lib().moe_grouped_topk(
        scores.data_ptr(), sdt, scores.stride(0), scores.stride(1), bias.data_ptr(),
        _lib.dtype_code(bias.dtype), _lib.ptr(pad), num_tokens, num_experts, n_group, topk_group, topk,
        int(bool(renormalize)), float(routed_scaling_factor), int(scoring_func), weights.data_ptr(),
        ids.data_ptr(), _lib.stream_of(scores))
    _lib.check(rc)
    return weights, ids


def _launch_topk_route(topk_weights, topk_indices, token_expert_indices, gating_output, renormalize,
                       e_score_correction_bias, is_padding, *, sigmoid: bool, scale: float) -> None:
    # argument contract of the reference (src/flaggems_vllm/ops/topk_sigmoid.py:86-126)
    assert gating_output.ndim == 2 and topk_weights.ndim == 2
    if gating_output.device.type != "cuda":
        raise NotImplementedError("Extended top-k routing requires a CUDA device")
    m, e = gating_output.shape
    k = topk_weights.shape[1]
    assert gating_output.is_contiguous()
    assert gating_output.dtype in (torch.float32, torch.float16, torch.bfloat16)
    assert topk_weights.dtype == torch.float32 and topk_weights.shape == (m, k)
    kinds = {torch.int32: 0, torch.int64: 1}
    if not sigmoid:
        kinds[torch.uint32] = 2
    if topk_indices.dtype not in kinds:
        raise TypeError("topk_indices must be int32/int64/uint32")
    assert token_expert_indices.dtype == torch.int32
    assert topk_indices.shape == token_expert_indices.shape == (m, k)
    assert all(t.is_contiguous() and t.device == gating_output.device
               for t in (topk_weights, topk_indices, token_expert_indices))
    assert 0 < k <= min(32, e)
    if e > 1024:
        raise NotImplementedError("Top-k routing supports at most 1024 experts")
    if e_score_correction_bias is not None:
        assert e_score_correction_bias.shape == (e,)
        assert e_score_correction_bias.dtype == torch.float32
        assert e_score_correction_bias.is_contiguous()
        assert e_score_correction_bias.device == gating_output.device
    if is_padding is not None:
        assert is_padding.shape == (m,) and is_padding.dtype == torch.bool
        assert is_padding.is_contiguous() and is_padding.device == gating_output.device
    if not m:
        return
    pad = is_padding.view(torch.uint8) if is_padding is not None else None
    rc = _lib.lib().moe_topk_route(
        gating_output.data_ptr(), _lib.dtype_code(gating_output.dtype), _lib.ptr(e_score_correction_bias),
        _lib.ptr(pad), m, e, k, int(sigmoid), int(bool(renormalize)), float(scale), topk_weights.data_ptr(),
        topk_indices.data_ptr(), kinds[topk_indices.dtype], token_expert_indices.data_ptr(),
        _lib.stream_of(gating_output))
    _lib.check(rc)


def topk_softmax(
    topk_weights: torch.Tensor,
    topk_indices: torch.Tensor,
    token_expert_indices: torch.Tensor,
    gating_output: torch.Tensor,
    renormalize: bool = False,
    e_score_correction_bias: torch.Tensor | None = None,
    is_padding: torch.Tensor | None = None,
) -> None:
    """Route with softmax scores, optionally using bias for expert selection.

    Returned weights are unbiased.  Padded rows have zero weights and expert
    id -1, with valid expanded token row indices.  Outputs are written in place
    (src/flaggems_vllm/ops/topk_softmax.py:126-140)."""
    logger.debug("GEMS TOPK SOFTMAX")
    _launch_topk_route(topk_weights, topk_indices, token_expert_indices, gating_output, renormalize,
                       e_score_correction_bias, is_padding, sigmoid=False, scale=1.0)


def topk_sigmoid(
    topk_weights: torch.Tensor,
    topk_indices: torch.Tensor,
    token_expert_indices: torch.Tensor,
    gating_output: torch.Tensor,
    renormalize: bool = False,
    e_score_correction_bias: torch.Tensor | None = None,
    routed_scaling_factor: float = 1.0,
    is_padding: torch.Tensor | None = None,
) -> None:
    """Route with sigmoid scores, then scale the optionally normalised weights.

    Bias affects expert selection only (src/flaggems_vllm/ops/topk_sigmoid.py:203-226)."""
    logger.debug("GEMS TOPK SIGMOID")
    _launch_topk_route(topk_weights, topk_indices, token_expert_indices, gating_output, renormalize,
                       e_score_correction_bias, is_padding, sigmoid=True, scale=routed_scaling_factor)

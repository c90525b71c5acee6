"""moe_align_block_size: host side of the single-launch stable counting sort.

Buffer sizes, names and the expert_map handling mirror
src/flaggems_vllm/ops/moe_align_block_size.py:843-927.  The reference's
function names are kept (``moe_align_block_size_triton`` writes caller-owned
buffers) so existing call sites keep working; nothing here uses Triton."""

from __future__ import annotations

import logging
from typing import Optional

import torch

from . import _lib

logger = logging.getLogger(__name__)


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def round_up(a: int, b: int) -> int:
    return ceil_div(a, b) * b


def moe_align_block_size_triton(
    topk_ids: torch.Tensor,
    num_experts: int,
    block_size: int,
    sorted_token_ids: torch.Tensor,
    expert_ids: torch.Tensor,
    num_tokens_post_pad: torch.Tensor,
) -> None:
    """Fill the three caller-owned int32 buffers (all entries are written)."""
    logger.debug("GEMS MOE ALIGN BLOCK SIZE")
    _lib.require_cuda(topk_ids, "moe_align_block_size")
    if topk_ids.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"topk_ids must be int32 or int64, got {topk_ids.dtype}")
    for t in (sorted_token_ids, expert_ids, num_tokens_post_pad):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise ValueError("output buffers must be contiguous int32 tensors")
    ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
    rc = _lib.lib().moe_align_block_size(
        ids.data_ptr(), int(ids.dtype == torch.int64), ids.numel(), int(num_experts), int(block_size),
        sorted_token_ids.data_ptr(), sorted_token_ids.numel(), expert_ids.data_ptr(), expert_ids.numel(),
        num_tokens_post_pad.data_ptr(), _lib.status_word(ids.device).data_ptr(), _lib.stream_of(ids))
    _lib.check(rc)


def _alloc(topk_ids, max_num_tokens_padded, block_size):
    dev = topk_ids.device
    sorted_ids = torch.empty((max_num_tokens_padded,), dtype=torch.int32, device=dev)
    expert_ids = torch.empty((ceil_div(max_num_tokens_padded, block_size),), dtype=torch.int32, device=dev)
    num_tokens_post_pad = torch.empty((1), dtype=torch.int32, device=dev)
    return sorted_ids, expert_ids, num_tokens_post_pad


def moe_align_block_size(
    topk_ids: torch.Tensor,
    block_size: int,
    num_experts: int,
    expert_map: Optional[torch.Tensor] = None,
    pad_sorted_ids: bool = False,
) -> "tuple[torch.Tensor, torch.Tensor, torch.Tensor]":
    """Returns (sorted_ids, expert_ids, num_tokens_post_pad), int32.

    sorted_ids holds flat route indices (token * topk + slot) grouped by expert,
    each expert's run padded with ``topk_ids.numel()`` to a multiple of
    ``block_size``; inside a run the indices ascend."""
    max_num_tokens_padded = topk_ids.numel() + num_experts * (block_size - 1)
    if pad_sorted_ids:
        max_num_tokens_padded = round_up(max_num_tokens_padded, block_size)
    sorted_ids, expert_ids, num_tokens_post_pad = _alloc(topk_ids, max_num_tokens_padded, block_size)
    moe_align_block_size_triton(topk_ids, num_experts, block_size, sorted_ids, expert_ids, num_tokens_post_pad)
    if expert_map is not None:
        expert_ids = expert_map[expert_ids]
    return sorted_ids, expert_ids, num_tokens_post_pad


def moe_align_block_size_no_tle(
    topk_ids: torch.Tensor,
    block_size: int,
    num_experts: int,
    expert_map: Optional[torch.Tensor] = None,
    pad_sorted_ids: bool = False,
    workspace=None,
) -> "tuple[torch.Tensor, torch.Tensor, torch.Tensor]":
    """Same as :func:`moe_align_block_size` with the small-batch bound
    ``numel * block_size`` on the buffer sizes.  ``workspace`` is accepted and
    ignored: the kernel keeps its counters in shared memory."""
    del workspace
    max_num_tokens_padded = topk_ids.numel() + num_experts * (block_size - 1)
    if pad_sorted_ids:
        max_num_tokens_padded = round_up(max_num_tokens_padded, block_size)
    if topk_ids.numel() < num_experts:
        max_num_tokens_padded = min(topk_ids.numel() * block_size, max_num_tokens_padded)
    sorted_ids, expert_ids, num_tokens_post_pad = _alloc(topk_ids, max_num_tokens_padded, block_size)
    moe_align_block_size_triton(topk_ids, num_experts, block_size, sorted_ids, expert_ids, num_tokens_post_pad)
    if expert_map is not None:
        expert_ids = expert_map[expert_ids]
    return sorted_ids, expert_ids, num_tokens_post_pad

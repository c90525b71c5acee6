"""Expert-parallel MoE layer for 2/4/8 GPUs of one node.

Experts are partitioned across ranks (rank r owns experts
[r*E/R, (r+1)*E/R)); tokens are data-parallel.  Every rank routes its own
tokens with the full score matrix, then

    dispatch   all-to-all of the routed rows to the rank that owns the expert
               (FP8 mode: the e4m3 row and its 1x128 scales travel, half the
               bytes of the bf16 row; plus local expert id and route weight)
    compute    align -> GEMM1 -> GEMM2 over the received rows (top-k = 1); the
               GEMM2 epilogue applies the route weight and writes rows in
               receive order, which IS the combine send order: no pack kernel
    combine    all-to-all of the bf16 rows back to their source rank
    sum        fixed-order fp32 sum over each token's k routes, reading the
               returned rows through an index (no un-permute pass)

Collectives are NCCL ``all_to_all_single`` over NVLink/NVSwitch; every payload
lands in the rank's own HBM before a kernel touches it.  The reference's own
expert-parallel hook is ``expert_map`` with replicated tokens and a caller-side
all-reduce (src/flaggems_vllm/ops/fused_moe.py:2553-2560, 2668-2669); that mode
is served by ``fused_experts_impl(expert_map=...)``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from .fused_moe import combine_routes, quantize_rows, route_pipeline


def partition_routes(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """Host-side plan of the dispatch: routes ordered by destination rank
    (stable), and how many go to each rank.  Works on CPU tensors too."""
    dest = torch.div(topk_ids.reshape(-1), experts_per_rank, rounding_mode="floor").clamp_(0, world - 1)
    order = torch.sort(dest, stable=True)[1]
    counts = torch.bincount(dest, minlength=world)[:world]
    return order, counts


class ExpertParallelMoE:
    """Holds this rank's expert shard and runs the dispatch/compute/combine step."""

    def __init__(self, w1, w2, w1_scale, w2_scale, num_experts_global: int, group=None, *,
                 mode: int = _lib.MODE_FP8_BLOCK, compute_fn=None, combine_fn=None):
        """``compute_fn(a_rows, a_scales_t, route_weight, local_ids) -> y`` and
        ``combine_fn(y_back, out, topk_ids, row_index)`` replace the CUDA steps;
        the CPU (gloo) tests of the dispatch/combine plumbing inject them."""
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.E = num_experts_global
        assert self.E % self.world == 0, "experts must divide evenly over ranks"
        self.E_local = self.E // self.world
        assert w1.shape[0] == self.E_local and w2.shape[0] == self.E_local
        self.w1, self.w2, self.s1, self.s2 = w1, w2, w1_scale, w2_scale
        self.mode = mode
        self.last_counts = None
        self.compute_fn = compute_fn or self._compute_cuda
        self.combine_fn = combine_fn or self._combine_cuda

    def _compute_cuda(self, a_rows, a_scales_t, route_weight, local_ids, act_dtype):
        return route_pipeline(a_rows, a_scales_t, self.w1, self.w2, route_weight, local_ids, mode=self.mode,
                              act_dtype=act_dtype, w1_scale=self.s1, w2_scale=self.s2,
                              global_num_experts=self.E_local, expert_map=None,
                              apply_router_weight_on_input=False)

    def _combine_cuda(self, y_back, out, topk_ids, row_index):
        combine_routes(y_back, out, topk_ids, self.E, None, row_index=row_index)

    def _a2a(self, out, inp, out_splits, in_splits):
        dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits,
                               group=self.group)

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        M, H = x.shape
        k = topk_ids.shape[1]
        dev = x.device
        fp8 = self.mode == _lib.MODE_FP8_BLOCK

        # ---- plan: routes by destination rank, counts to/from every rank
        order, send_counts = partition_routes(topk_ids, self.E_local, self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        counts = torch.stack([send_counts, recv_counts]).tolist()  # the one host sync of the step
        send_splits, recv_splits = counts[0], counts[1]
        n_send, n_recv = sum(send_splits), sum(recv_splits)
        self.last_counts = (send_splits, recv_splits)

        # ---- dispatch payload, in send order
        src_tok = torch.div(order, k, rounding_mode="floor")
        flat_ids = topk_ids.reshape(-1)[order]
        meta_send = torch.stack([(flat_ids % self.E_local).float(),
                                 topk_weights.reshape(-1)[order].float()], dim=1).contiguous()
        meta_recv = torch.empty((n_recv, 2), dtype=torch.float32, device=dev)
        self._a2a(meta_recv, meta_send, recv_splits, send_splits)
        if fp8:
            xq, xs_t = quantize_rows(x)
            rows_send = xq.view(torch.uint8)[src_tok]
            sc_send = xs_t.t()[src_tok].contiguous()
            rows_recv = torch.empty((n_recv, H), dtype=torch.uint8, device=dev)
            sc_recv = torch.empty((n_recv, H // 128), dtype=torch.float32, device=dev)
            self._a2a(rows_recv, rows_send, recv_splits, send_splits)
            self._a2a(sc_recv, sc_send, recv_splits, send_splits)
            a_rows = rows_recv.view(torch.float8_e4m3fn)
            a_scales_t = sc_recv.t().contiguous()
        else:
            rows_send = x[src_tok]
            rows_recv = torch.empty((n_recv, H), dtype=x.dtype, device=dev)
            self._a2a(rows_recv, rows_send, recv_splits, send_splits)
            a_rows, a_scales_t = rows_recv, None

        # ---- local experts over the received rows (top-k = 1)
        if n_recv > 0:
            local_ids = meta_recv[:, 0].to(torch.int32).view(n_recv, 1)
            y = self.compute_fn(a_rows, a_scales_t, meta_recv[:, 1].contiguous(), local_ids, x.dtype)
        else:
            y = torch.empty((0, H), dtype=x.dtype, device=dev)

        # ---- combine: rows return in send order; sum through the inverse permutation
        y_back = torch.empty((n_send, H), dtype=x.dtype, device=dev)
        self._a2a(y_back, y, send_splits, recv_splits)
        inverse = torch.empty_like(order, dtype=torch.int32)
        inverse[order] = torch.arange(order.numel(), device=dev, dtype=torch.int32)
        out = torch.empty_like(x)
        self.combine_fn(y_back, out, topk_ids, inverse)
        return out

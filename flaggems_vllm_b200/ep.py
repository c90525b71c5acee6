"""Expert-parallel MoE layer for 2/4/8 GPUs of one node.

Experts are partitioned across ranks (rank r owns experts
[r*E/R, (r+1)*E/R)); tokens are data-parallel.  Every rank routes its own
tokens with the full score matrix.  The unit that travels is a
(token, destination rank) pair, not a route: a token whose k experts live on
fewer than k ranks is sent once per rank (DeepSeek-V3's group-limited routing
keeps a token's 8 experts inside 4 of 8 groups, so with one group per rank
dispatch and combine move half the rows a per-route exchange would).

    plan       which ranks each token visits (a [M, R] mask), counts all-to-all
    dispatch   all-to-all of the rows (FP8 mode: e4m3, half the bytes of a bf16
               row) and of one fp32 side row per pair (the token's k expert ids
               and weights, plus its 1x128 scales in FP8 mode); the receiver
               marks the slots that belong to other ranks with -1
    compute    align -> GEMM1 -> GEMM2 over the received rows with their k
               slots, then the fixed-order sum of each row's local routes: the
               result is already the per-(token, rank) partial output, in
               receive order, which IS the combine send order
    combine    all-to-all of those bf16 rows back to their source rank
    sum        fixed-order fp32 sum over the ranks each token visited, reading
               the returned rows through an index

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
from . import fused_moe as _fm
from .fused_moe import combine_routes, route_pipeline
from .quant import per_token_group_quant_fp8


def plan_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """Which (token, rank) pairs exist.  Returns
    ``tok`` [P] token of each pair, ``dst`` [P] its rank (pairs ordered by rank,
    then token), ``counts`` [R] pairs per rank, ``index`` [M, R] position of the
    pair of (token, rank) in that order or -1.  Works on CPU tensors too."""
    M = topk_ids.shape[0]
    ids = topk_ids.long()
    valid = ids >= 0
    dest = torch.div(ids.clamp_min(0), experts_per_rank, rounding_mode="floor").clamp_(max=world - 1)
    # a rank is visited when ANY route goes there (a plain scatter of the validity flags would let
    # a padded route, which also maps to rank 0, overwrite a real one)
    visits = torch.zeros((M, world), dtype=torch.int32, device=topk_ids.device)
    visits.scatter_add_(1, dest, valid.to(torch.int32))
    visits = visits > 0
    counts = visits.sum(0)
    pairs = visits.t().nonzero(as_tuple=False)  # sorted by rank, then token
    dst, tok = pairs[:, 0], pairs[:, 1]
    index = torch.full((M, world), -1, dtype=torch.int32, device=topk_ids.device)
    index[tok, dst] = torch.arange(pairs.shape[0], device=topk_ids.device, dtype=torch.int32)
    return tok, dst, counts, index, dest


class ExpertParallelMoE:
    """Holds this rank's expert shard and runs the dispatch/compute/combine step."""

    def __init__(self, w1, w2, w1_scale, w2_scale, num_experts_global: int, group=None, *,
                 mode: int = _lib.MODE_FP8_BLOCK, compute_fn=None, combine_fn=None, chunks: int = 1,
                 overlap_combine: bool = False, free_sms: int = 16):
        """``compute_fn(a_rows, a_scales_t, slot_weights, slot_ids, act_dtype) -> rows``
        and ``combine_fn(rows_back, out, index)`` replace the CUDA steps; the CPU
        (gloo) tests of the dispatch/combine plumbing inject them."""
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
        self.last_bytes = None
        self._host_counts = {}  # (device, stream) -> (pinned [2, R] int32, event): the host's view of the pair counts
        self.compute_fn = compute_fn or self._compute_cuda
        self.combine_fn = combine_fn or self._combine_cuda
        # Token chunks run as independent dispatch/compute/combine steps on their own streams and
        # their own communicators, so one chunk's all-to-alls travel under the other chunk's GEMMs
        # (collectives of one communicator run in issue order, which would chain the chunks).
        self.chunks = max(1, int(chunks))
        self._lanes = None
        # The combine in two column halves: GEMM 2 runs once per half of the hidden columns, and the
        # first half's local sum and all-to-all travel (on a side stream) while the second half's
        # GEMM 2 runs on all but `free_sms` SMs.  Every rank takes the same decision (it depends on
        # the layer only), so the ranks issue the same collectives; bitwise the same result.
        self.overlap_combine = bool(overlap_combine)
        self.free_sms = int(free_sms)
        self._side = {}

    def _chunk_lanes(self, device):
        if self._lanes is None:
            ranks = dist.get_process_group_ranks(self.group)
            self._lanes = [(torch.cuda.Stream(device=device), self.group if c == 0 else dist.new_group(ranks))
                           for c in range(self.chunks)]
        return self._lanes

    def _compute_cuda(self, a_rows, a_scales_t, slot_weights, slot_ids, act_dtype):
        y, row_index = route_pipeline(a_rows, a_scales_t, self.w1, self.w2, slot_weights, slot_ids, mode=self.mode,
                                      act_dtype=act_dtype, w1_scale=self.s1, w2_scale=self.s2,
                                      global_num_experts=self.E_local, expert_map=None,
                                      apply_router_weight_on_input=False)
        rows = torch.empty((a_rows.shape[0], y.shape[1]), dtype=act_dtype, device=y.device)
        combine_routes(y, rows, slot_ids, self.E_local, row_index=row_index)  # slots of other ranks (-1) are skipped
        return rows

    def _combine_cuda(self, rows_back, out, index):
        # one slot per rank; ranks the token did not visit have index -1
        combine_routes(rows_back, out, None, 0, None, row_index=index)

    def _a2a(self, out, inp, out_splits, in_splits, group=None):
        dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits,
                               group=group if group is not None else self.group)

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and self.compute_fn == self._compute_cuda:
            if self.chunks > 1 and x.shape[0] >= 2 * self.chunks:
                return self._forward_chunked(x, topk_weights, topk_ids)
            return self._forward_cuda(x, topk_weights, topk_ids, self.group)
        return self._forward_torch(x, topk_weights, topk_ids)

    def _forward_chunked(self, x, topk_weights, topk_ids):
        """Every rank cuts its tokens into the same number of chunks; chunk c of all ranks forms one
        dispatch/compute/combine step on lane c (stream + communicator).  Results land in one
        output tensor; the caller's stream waits for every lane."""
        M = x.shape[0]
        main = torch.cuda.current_stream(x.device)
        lanes = self._chunk_lanes(x.device)
        out = torch.empty_like(x)
        bounds = [M * c // self.chunks for c in range(self.chunks + 1)]
        for c, (stream, group) in enumerate(lanes):
            lo, hi = bounds[c], bounds[c + 1]
            stream.wait_stream(main)
            with torch.cuda.stream(stream):
                part = self._forward_cuda(x[lo:hi], topk_weights[lo:hi], topk_ids[lo:hi], group, out=out[lo:hi])
                part.record_stream(stream)
        for stream, _ in lanes:
            main.wait_stream(stream)
        return out

    def _forward_cuda(self, x, topk_weights, topk_ids, group=None, out=None):
        """The same step with the bookkeeping done by three kernels (plan, pack, unpack) instead
        of some thirty small tensor operations; one host read (the pair counts) remains."""
        M, H = x.shape
        k = topk_ids.shape[1]
        dev = x.device
        L, st = _lib.lib(), _lib.stream_of(x)
        fp8 = self.mode == _lib.MODE_FP8_BLOCK
        R = self.world
        ids = topk_ids if topk_ids.dtype == torch.int32 and topk_ids.is_contiguous() else topk_ids.to(torch.int32).contiguous()
        tw = topk_weights if topk_weights.dtype == torch.float32 and topk_weights.is_contiguous() \
            else topk_weights.float().contiguous()
        index = torch.empty((M, R), dtype=torch.int32, device=dev)
        both = torch.empty((2, R), dtype=torch.int32, device=dev)  # [send counts; receive counts]
        tok = torch.empty((max(M * R, 1),), dtype=torch.int32, device=dev)
        _lib.check(L.moe_ep_plan(ids.data_ptr(), M, k, self.E_local, R, index.data_ptr(), both[0].data_ptr(),
                                 tok.data_ptr(), st))
        group = group if group is not None else self.group
        mark = _fm.STAGE_HOOK or _fm._no_mark  # the timing hook of the single-GPU pipeline also sees these stages
        mark("ep_plan")
        dist.all_to_all_single(both[1], both[0], group=group)
        # The one host read of the step (NCCL takes the split sizes from the host).  The counts are
        # copied to pinned memory and the host waits for that copy only; the quantiser, which does
        # not need them, is enqueued first, so the GPU has work while the host waits and then
        # enqueues the rest of the step.
        cur = torch.cuda.current_stream(dev)
        key = (dev.index, cur.cuda_stream)
        slot = self._host_counts.get(key)
        if slot is None or slot[0].shape[1] != R:
            slot = (torch.empty((2, R), dtype=torch.int32).pin_memory(), torch.cuda.Event())
            self._host_counts[key] = slot
        host_counts, copied = slot
        host_counts.copy_(both, non_blocking=True)
        copied.record(cur)

        g = H // 128 if fp8 else 0
        if fp8:
            xq, xs = per_token_group_quant_fp8(x, 128)
            rows_src, row_bytes, rows_dtype = xq, H, torch.float8_e4m3fn
        else:
            xs = None
            rows_src, row_bytes, rows_dtype = x if x.is_contiguous() else x.contiguous(), H * x.element_size(), x.dtype
        copied.synchronize()
        counts = host_counts.tolist()
        send_splits, recv_splits = counts[0], counts[1]
        n_send, n_recv = sum(send_splits), sum(recv_splits)
        self.last_counts = (send_splits, recv_splits)
        mark("ep_counts")
        rows_send = torch.empty((n_send, H), dtype=rows_dtype, device=dev)
        side_send = torch.empty((n_send, g + 2 * k), dtype=torch.float32, device=dev)
        _lib.check(L.moe_ep_pack(rows_src.data_ptr(), row_bytes, _lib.ptr(xs), g, ids.data_ptr(), tw.data_ptr(), k,
                                 tok.data_ptr(), n_send, rows_send.data_ptr(), side_send.data_ptr(), st))
        side_recv = torch.empty((n_recv, g + 2 * k), dtype=torch.float32, device=dev)
        a_rows = torch.empty((n_recv, H), dtype=rows_dtype, device=dev)
        # bytes that leave this GPU (pairs whose destination is another rank), per direction of the step
        off_rank = n_send - send_splits[self.rank]
        self.last_bytes = {"dispatch": off_rank * (row_bytes + (g + 2 * k) * 4),
                           "combine_in": off_rank * H * x.element_size(),
                           "combine": (n_recv - recv_splits[self.rank]) * H * x.element_size()}
        mark("ep_pack")
        # the fp8 rows travel as bytes (NCCL has no e4m3 all-to-all on every version)
        self._a2a(side_recv, side_send, recv_splits, send_splits, group)
        self._a2a(a_rows.view(torch.uint8) if fp8 else a_rows, rows_send.view(torch.uint8) if fp8 else rows_send,
                  recv_splits, send_splits, group)
        mark("ep_dispatch")
        a_scales_t = torch.empty((g, n_recv), dtype=torch.float32, device=dev) if fp8 else None
        slot_ids = torch.empty((n_recv, k), dtype=torch.int32, device=dev)
        slot_w = torch.empty((n_recv, k), dtype=torch.float32, device=dev)
        _lib.check(L.moe_ep_unpack(side_recv.data_ptr(), n_recv, g, k, self.rank, self.E_local, _lib.ptr(a_scales_t),
                                   slot_ids.data_ptr(), slot_w.data_ptr(), st))
        mark("ep_unpack")
        if out is None:
            out = torch.empty_like(x)
        if self.overlap_combine and H % 512 == 0 and self.compute_fn == self._compute_cuda:
            self._combine_in_halves(a_rows, a_scales_t, slot_w, slot_ids, x.dtype, send_splits, recv_splits, group,
                                    out, index, mark)
            return out
        if n_recv > 0:
            rows = self.compute_fn(a_rows, a_scales_t, slot_w, slot_ids, x.dtype)
        else:
            rows = torch.empty((0, H), dtype=x.dtype, device=dev)
        rows_back = torch.empty((n_send, H), dtype=x.dtype, device=dev)
        mark("ep_local_sum")
        self._a2a(rows_back, rows, send_splits, recv_splits, group)
        mark("ep_combine")
        self.combine_fn(rows_back, out, index)
        mark("ep_sum")
        return out

    def _combine_in_halves(self, a_rows, a_scales_t, slot_w, slot_ids, act_dtype, send_splits, recv_splits, group,
                           out, index, mark):
        """Local experts, then the combine as two all-to-alls of half-width rows.  When GEMM 2 can
        produce the column halves one after the other, the first half's all-to-all runs beside the
        second half's GEMM 2; otherwise the finished rows are cut in two.  Either way every rank
        issues the same two collectives."""
        dev = out.device
        H = out.shape[1]
        n_recv, n_send = a_rows.shape[0], sum(send_splits)
        h0 = (H // 2) // 256 * 256
        main = torch.cuda.current_stream(dev)
        side = self._side.get(dev.index)
        if side is None:
            side = self._side[dev.index] = torch.cuda.Stream(device=dev)
        sent = []  # (first column, returned rows, event after the all-to-all)

        def send_half(c0, rows_h):
            ready = torch.cuda.Event()
            ready.record(main)
            rows_back_h = torch.empty((n_send, rows_h.shape[1]), dtype=act_dtype, device=dev)
            side.wait_event(ready)
            with torch.cuda.stream(side):
                self._a2a(rows_back_h, rows_h, send_splits, recv_splits, group)
                done = torch.cuda.Event()
                done.record(side)
            rows_h.record_stream(side)
            rows_back_h.record_stream(side)
            sent.append((c0, rows_back_h, done))

        def after_gemm2(half, c0, y_w, row_index):
            rows_h = torch.empty((n_recv, y_w.shape[1]), dtype=act_dtype, device=dev)
            combine_routes(y_w, rows_h, slot_ids, self.E_local, row_index=row_index)
            mark("ep_local_sum")
            send_half(c0, rows_h)

        rows = None
        if n_recv > 0:
            y, row_index = route_pipeline(a_rows, a_scales_t, self.w1, self.w2, slot_w, slot_ids, mode=self.mode,
                                          act_dtype=act_dtype, w1_scale=self.s1, w2_scale=self.s2,
                                          global_num_experts=self.E_local, expert_map=None,
                                          apply_router_weight_on_input=False,
                                          column_halves=(after_gemm2, self.free_sms))
            if y is not None:  # GEMM 2 wrote whole rows (few rows per expert): sum them, then cut
                rows = torch.empty((n_recv, H), dtype=act_dtype, device=dev)
                combine_routes(y, rows, slot_ids, self.E_local, row_index=row_index)
        else:
            rows = torch.empty((0, H), dtype=act_dtype, device=dev)
        if rows is not None:
            mark("ep_local_sum")
            send_half(0, rows[:, :h0].contiguous())
            send_half(h0, rows[:, h0:].contiguous())
        for c0, rows_back_h, done in sent:
            main.wait_event(done)
            self.combine_fn(rows_back_h, out[:, c0:c0 + rows_back_h.shape[1]], index)  # into the column window
        mark("ep_sum")

    def _forward_torch(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        M, H = x.shape
        k = topk_ids.shape[1]
        dev = x.device
        fp8 = self.mode == _lib.MODE_FP8_BLOCK

        # ---- plan and counts
        tok, dst, send_counts, index, dest = plan_dispatch(topk_ids, self.E_local, self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        counts = torch.stack([send_counts, recv_counts]).tolist()  # the one host sync of the step
        send_splits, recv_splits = counts[0], counts[1]
        n_send, n_recv = sum(send_splits), sum(recv_splits)
        self.last_counts = (send_splits, recv_splits)

        # ---- side data of each pair: the token's k global expert ids and weights (and, in FP8 mode,
        # its 1x128 scales) travel as one fp32 row; the receiver keeps the ids it owns
        g = H // 128 if fp8 else 0
        if fp8:
            xq, xs = per_token_group_quant_fp8(x, 128)
            side_send = torch.cat([xs[tok], topk_ids[tok].float(), topk_weights[tok].float()], dim=1)
            rows_send = xq.view(torch.uint8)[tok]
        else:
            side_send = torch.cat([topk_ids[tok].float(), topk_weights[tok].float()], dim=1)  # ids < 2^24: exact
            rows_send = x[tok]
        side_recv = torch.empty((n_recv, g + 2 * k), dtype=torch.float32, device=dev)
        self._a2a(side_recv, side_send, recv_splits, send_splits)
        a_rows = torch.empty((n_recv, H), dtype=rows_send.dtype, device=dev)
        self._a2a(a_rows, rows_send, recv_splits, send_splits)
        if fp8:
            a_rows = a_rows.view(torch.float8_e4m3fn)
            a_scales_t = side_recv[:, :g].t().contiguous()
        else:
            a_scales_t = None
        local = side_recv[:, g:g + k].to(torch.int32) - self.rank * self.E_local
        slot_ids = torch.where((local >= 0) & (local < self.E_local), local, -1)  # -1: another rank's route
        slot_w = side_recv[:, g + k:].contiguous()

        # ---- local experts over the received rows
        if n_recv > 0:
            rows = self.compute_fn(a_rows, a_scales_t, slot_w, slot_ids, x.dtype)
        else:
            rows = torch.empty((0, H), dtype=x.dtype, device=dev)

        # ---- combine
        rows_back = torch.empty((n_send, H), dtype=x.dtype, device=dev)
        self._a2a(rows_back, rows, send_splits, recv_splits)
        out = torch.empty_like(x)
        self.combine_fn(rows_back, out, index)
        return out

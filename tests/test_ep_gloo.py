"""Expert-parallel plumbing on CPU: two gloo ranks run the dispatch / combine
of ExpertParallelMoE with the per-route expert computation supplied by the CPU
oracle, and the result must equal the single-process layer."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flaggems_vllm_b200 import _lib
from flaggems_vllm_b200.ep import ExpertParallelMoE, partition_routes
from oracle import moe_oracle as O


def test_partition_routes_orders_by_destination_rank():
    ids = torch.tensor([[5, 0], [2, 7], [4, 1]], dtype=torch.int32)
    order, counts = partition_routes(ids, 4, 2)
    assert counts.tolist() == [3, 3]
    assert order.tolist() == [1, 2, 5, 0, 3, 4]  # stable inside a destination


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, E, H, I, k, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        w1 = (torch.randn(E, 2 * I, H, generator=g) * H**-0.5).to(torch.bfloat16)
        w2 = (torch.randn(E, H, I, generator=g) * I**-0.5).to(torch.bfloat16)
        xs = torch.randn(world, M, H, generator=g).to(torch.bfloat16)
        logits = torch.randn(world, M, E, generator=g)
        tw, ti = O.softmax_topk_oracle(logits[rank], k, torch.float32)
        El = E // world
        lw1, lw2 = w1[rank * El:(rank + 1) * El], w2[rank * El:(rank + 1) * El]

        def compute(a_rows, a_scales_t, route_weight, local_ids, act_dtype):
            # one route per received row
            y = O.fused_moe_half_oracle(a_rows, lw1, lw2, route_weight.view(-1, 1), local_ids)
            return y.to(act_dtype)

        def combine(y_back, out, topk_ids, row_index):
            Mloc, kk = topk_ids.shape
            out.copy_(y_back.float()[row_index.long()].view(Mloc, kk, out.shape[1]).sum(1).to(out.dtype))

        layer = ExpertParallelMoE(lw1, lw2, None, None, E, mode=_lib.MODE_HALF, compute_fn=compute,
                                  combine_fn=combine)
        out = layer.forward(xs[rank], tw, ti)
        ref = O.fused_moe_half_oracle(xs[rank], w1, w2, tw, ti)
        ret[rank] = (O.rel_l2(out.float(), ref), O.cosine(out.float(), ref), layer.last_counts)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [0, 5, 33])
def test_two_rank_dispatch_combine_matches_single_process(M):
    world, E, H, I, k = 2, 8, 64, 128, 2
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, M, E, H, I, k, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        rl2, cs, counts = ret[rank]
        assert sum(counts[0]) == M * k
        if M:
            assert rl2 < 1e-2 and cs > 0.9999, f"rank {rank}: rel_l2={rl2} cos={cs}"
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0
    assert ret[0][2][0][1] == ret[1][2][1][0] and ret[1][2][0][0] == ret[0][2][1][1]

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
from flaggems_vllm_b200.ep import ExpertParallelMoE, plan_dispatch
from oracle import moe_oracle as O


def test_plan_dispatch_sends_a_token_once_per_rank():
    ids = torch.tensor([[5, 0], [2, 3], [4, 1], [-1, 6]], dtype=torch.int32)
    tok, dst, counts, index, dest = plan_dispatch(ids, 4, 2)
    assert counts.tolist() == [3, 3]                      # token 1 visits rank 0 once although both routes go there
    assert dst.tolist() == [0, 0, 0, 1, 1, 1] and tok.tolist() == [0, 1, 2, 0, 2, 3]
    assert index.tolist() == [[0, 3], [1, -1], [2, 4], [-1, 5]]


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

        def compute(a_rows, a_scales_t, slot_w, slot_ids, act_dtype):
            # slots with id -1 belong to other ranks: route them to expert 0 with weight 0
            ids = slot_ids.clamp_min(0)
            w = torch.where(slot_ids >= 0, slot_w, torch.zeros(()))
            return O.fused_moe_half_oracle(a_rows, lw1, lw2, w, ids).to(act_dtype)

        def combine(rows_back, out, index):
            padded = torch.cat([rows_back.float(), torch.zeros(1, out.shape[1])])
            out.copy_(padded[index.long()].sum(1).to(out.dtype))  # index -1 picks the zero row

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
        assert sum(counts[0]) <= M * k
        if M:
            assert rl2 < 1e-2 and cs > 0.9999, f"rank {rank}: rel_l2={rl2} cos={cs}"
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0
    assert ret[0][2][0][1] == ret[1][2][1][0] and ret[1][2][0][0] == ret[0][2][1][1]


def _fault_worker(rank, world, port, fault, ret):
    """Rank 1 fails on the host between steps (it raises, or it never joins the step); rank 0
    must leave its next collective with an error inside the process group's time limit instead of
    waiting for ever, and must still be able to tear the group down."""
    import datetime
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    E, H, I, k, M = 4, 32, 64, 2, 6
    g = torch.Generator().manual_seed(3)
    w1 = torch.randn(E // world, 2 * I, H, generator=g).to(torch.bfloat16)
    w2 = torch.randn(E // world, H, I, generator=g).to(torch.bfloat16)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16)
    tw, ti = O.softmax_topk_oracle(torch.randn(M, E, generator=g), k, torch.float32)

    def compute(a_rows, a_scales_t, slot_w, slot_ids, act_dtype):
        w = torch.where(slot_ids >= 0, slot_w, torch.zeros(()))
        return O.fused_moe_half_oracle(a_rows, w1, w2, w, slot_ids.clamp_min(0)).to(act_dtype)

    def combine(rows_back, out, index):
        padded = torch.cat([rows_back.float(), torch.zeros(1, out.shape[1])])
        out.copy_(padded[index.long()].sum(1).to(out.dtype))

    layer = ExpertParallelMoE(w1, w2, None, None, E, mode=_lib.MODE_HALF, compute_fn=compute, combine_fn=combine)
    layer.forward(x, tw, ti)  # one good step first: the failure happens between steps
    dist.barrier()
    t0 = time.time()
    try:
        if rank == 1:
            if fault == "raises":
                raise ValueError("injected host failure on rank 1")
            time.sleep(8.0)  # "never joins": stays alive past rank 0's time limit, issues nothing
            ret[rank] = ("idle", time.time() - t0)
            return
        layer.forward(x, tw, ti)
        ret[rank] = ("completed", time.time() - t0)
    except ValueError as exc:
        ret[rank] = ("raised", str(exc))
    except Exception as exc:  # gloo reports a lost or silent peer as RuntimeError / DistBackendError
        ret[rank] = ("collective_error", time.time() - t0, type(exc).__name__)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("fault", ["raises", "never_joins"])
def test_peer_failure_between_steps_ends_the_next_collective_with_an_error(fault):
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_fault_worker, args=(world, port, fault, ret), nprocs=world, join=True)
    assert ret[1][0] == ("raised" if fault == "raises" else "idle")
    kind, seconds = ret[0][0], ret[0][1]
    assert kind == "collective_error", f"rank 0 {kind} although its peer was gone"
    assert seconds < 7.5, f"rank 0 needed {seconds:.1f} s to notice"

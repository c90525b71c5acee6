"""Worker for the multi-GPU expert-parallel parity test (run under torchrun).

Every rank builds the same seeded global layer, keeps its expert shard, runs the
expert-parallel step on its own tokens and compares with the single-GPU layer
computed locally from the full weights."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import flaggems_vllm_b200 as fg  # noqa: E402
from flaggems_vllm_b200 import _lib, ep  # noqa: E402
from flaggems_vllm_b200 import testing as T  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    for mode, (M, E, H, I, k) in (("fp8", (96, 32, 512, 256, 8)), ("half", (64, 16, 256, 256, 4)),
                                  ("fp8", (1, 32, 512, 256, 8)), ("fp8", (2048, 32, 512, 256, 8)),
                                  ("half", (1024, 16, 512, 256, 4))):
        x = T.make_activations(M, H, dev, seed=50 + rank)
        logits, bias = T.make_router_inputs(M, E, dev, seed=60 + rank)
        El = E // world
        if mode == "fp8":
            w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, dev, seed=1, std=H**-0.5)
            w2, s2 = T.make_fp8_block_weights(E, H, I, dev, seed=2, std=I**-0.5)
            tw, ti = fg.grouped_topk(logits, 8, 4, k, True, 2.5, torch.zeros_like(bias), 1)
            full = fg.fused_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2,
                                         block_shape=[128, 128])
            sl = slice(rank * El, (rank + 1) * El)
            layer = ep.ExpertParallelMoE(w1[sl].contiguous(), w2[sl].contiguous(), s1[sl].contiguous(),
                                         s2[sl].contiguous(), E, mode=_lib.MODE_FP8_BLOCK)
        else:
            w1 = T.make_half_weights(E, 2 * I, H, dev, seed=1, std=H**-0.5)
            w2 = T.make_half_weights(E, H, I, dev, seed=2, std=I**-0.5)
            tw, ti = fg.grouped_topk(torch.softmax(logits, -1), 1, 1, k, True, 1.0, torch.zeros_like(bias), 0)
            full = fg.fused_experts_impl(x, w1, w2, tw, ti)
            sl = slice(rank * El, (rank + 1) * El)
            layer = ep.ExpertParallelMoE(w1[sl].contiguous(), w2[sl].contiguous(), None, None, E,
                                         mode=_lib.MODE_HALF)
        out = layer.forward(x, tw, ti)
        torch.cuda.synchronize()
        if M >= 8:
            # the same step cut into two token chunks on two streams / communicators: identical rows
            layer.chunks = 2
            out2 = layer.forward(x, tw, ti)
            torch.cuda.synchronize()
            layer.chunks = 1
            assert torch.equal(out2, out), "chunked expert-parallel step differs from the unchunked one"
        # the combine in two column halves (the first half's all-to-all beside the second half's GEMM 2
        # when there are enough rows per expert, otherwise the finished rows cut in two): identical rows
        layer.overlap_combine = True
        out3 = layer.forward(x, tw, ti)
        torch.cuda.synchronize()
        layer.overlap_combine = False
        assert torch.equal(out3, out), "combine in column halves differs from the one-piece combine"
        a, b = out.float(), full.float()
        rl2 = ((a - b).norm() / b.norm().clamp_min(1e-20)).item()
        st = fg.read_status(dev)
        # the per-rank partial sums are rounded to the activation dtype before the final sum,
        # one rounding more than the single-GPU layer: allow 5e-3 (the layer tolerance is 1e-2)
        good = rl2 < 5e-3 and st == 0
        ok = ok and good
        print(f"rank {rank} {mode} M={M}: rel_l2 vs single-GPU layer {rl2:.2e} status {st} {'OK' if good else 'FAIL'}",
              flush=True)
    flag = torch.tensor([0 if ok else 1], device=dev)
    dist.all_reduce(flag)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 0 else 1)


if __name__ == "__main__":
    main()

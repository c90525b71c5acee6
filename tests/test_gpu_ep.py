"""Expert-parallel parity on real GPUs: launched as torchrun child processes
when the box has at least two GPUs."""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_matches_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "ep_worker.py")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:]
    assert "FAIL" not in r.stdout and r.stdout.count(" OK") == 5 * world, r.stdout[-4000:]  # five cases per rank


@pytest.mark.gpu
@pytest.mark.parametrize("M,R", [(0, 2), (1, 8), (77, 2), (1000, 4), (8192, 8)])
def test_plan_pack_unpack_kernels_match_the_tensor_formulation(M, R):
    """moe_ep_plan / moe_ep_pack / moe_ep_unpack against plan_dispatch and plain indexing."""
    import torch

    from flaggems_vllm_b200 import _lib
    from flaggems_vllm_b200.ep import plan_dispatch

    dev = torch.device("cuda", 0)
    E, k, H, g = 64, 8, 256, 2
    epr = E // R
    gen = torch.Generator(device="cpu").manual_seed(M + R)
    ids = torch.randint(0, E, (M, k), generator=gen, dtype=torch.int32)
    if M > 3:
        ids[3, :4] = -1  # padded routes
    ids = ids.to(dev)
    tw = torch.rand((M, k), generator=gen).to(dev)
    rows = torch.randint(0, 255, (M, H), generator=gen, dtype=torch.uint8).to(dev)
    scales = torch.rand((M, g), generator=gen).to(dev)
    L, st = _lib.lib(), _lib.stream_of(ids)

    index = torch.empty((M, R), dtype=torch.int32, device=dev)
    counts = torch.empty((R,), dtype=torch.int32, device=dev)
    tok = torch.full((max(M * R, 1),), -5, dtype=torch.int32, device=dev)
    _lib.check(L.moe_ep_plan(ids.data_ptr(), M, k, epr, R, index.data_ptr(), counts.data_ptr(), tok.data_ptr(), st))
    rtok, rdst, rcounts, rindex, _ = plan_dispatch(ids, epr, R)
    P = int(rcounts.sum())
    assert counts.tolist() == rcounts.tolist()
    assert torch.equal(index, rindex) and torch.equal(tok[:P].long(), rtok)

    rows_out = torch.empty((P, H), dtype=torch.uint8, device=dev)
    side = torch.empty((P, g + 2 * k), dtype=torch.float32, device=dev)
    _lib.check(L.moe_ep_pack(rows.data_ptr(), H, scales.data_ptr(), g, ids.data_ptr(), tw.data_ptr(), k, tok.data_ptr(), P,
                             rows_out.data_ptr(), side.data_ptr(), st))
    assert torch.equal(rows_out, rows[rtok])
    assert torch.equal(side, torch.cat([scales[rtok], ids[rtok].float(), tw[rtok]], dim=1))

    rank = R - 1
    scales_t = torch.empty((g, P), dtype=torch.float32, device=dev)
    slot_ids = torch.empty((P, k), dtype=torch.int32, device=dev)
    slot_w = torch.empty((P, k), dtype=torch.float32, device=dev)
    _lib.check(L.moe_ep_unpack(side.data_ptr(), P, g, k, rank, epr, scales_t.data_ptr(), slot_ids.data_ptr(),
                               slot_w.data_ptr(), st))
    local = ids[rtok] - rank * epr
    assert torch.equal(slot_ids, torch.where((local >= 0) & (local < epr) & (ids[rtok] >= 0), local, -1))
    assert torch.equal(slot_w, tw[rtok]) and torch.equal(scales_t, scales[rtok].t().contiguous())

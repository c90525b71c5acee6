"""Failure handling on a real GPU without faulting or hanging it: a bounded wait that is made
to run out sets the status bit and the context stays usable."""

import pytest
import torch

import flaggems_vllm_b200 as fg
from flaggems_vllm_b200 import _lib
from flaggems_vllm_b200 import testing as T

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_a_wait_that_runs_out_sets_the_status_bit_and_the_gpu_still_answers():
    L = _lib.lib()
    dev = torch.device(DEV)
    status = _lib.status_word(dev)
    assert fg.read_status(dev) == 0
    gave_up = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    # one warp waits 1 ms on a barrier nobody arrives at
    _lib.check(L.moe_debug_wait_timeout(status.data_ptr(), 1_000_000, gave_up.data_ptr(), st))
    torch.cuda.synchronize()
    assert int(gave_up.item()) == 1
    assert fg.read_status(dev) & _lib.ST_WAIT_TIMEOUT
    assert fg.read_status(dev) == 0  # reading cleared it
    # the context is alive: a layer runs and reports nothing
    M, E, H, I, k = 8, 8, 256, 256, 2
    x = T.make_activations(M, H, DEV)
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    logits, _ = T.make_router_inputs(M, E, DEV)
    tw, ti = fg.grouped_topk(torch.softmax(logits, -1), 1, 1, k, True, 1.0, torch.zeros(E, device=DEV), 0)
    out = fg.fused_experts_impl(x, w1, w2, tw.to(torch.bfloat16), ti)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all() and fg.read_status(dev) == 0


def test_wait_limit_setter_round_trip():
    L = _lib.lib()
    old = L.moe_set_wait_limit_ns(0)
    assert old > 0
    assert L.moe_set_wait_limit_ns(5_000_000) == old
    assert L.moe_set_wait_limit_ns(old) == 5_000_000
    assert L.moe_set_wait_limit_ns(0) == old


def test_status_check_mode_raises(monkeypatch):
    """FLAGGEMS_B200_CHECK_STATUS=1: the layer reads the status word and raises when a kernel reported a problem."""
    monkeypatch.setenv("FLAGGEMS_B200_CHECK_STATUS", "1")
    M, E, H, I, k = 8, 8, 256, 256, 2
    x = T.make_activations(M, H, DEV)
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    logits, _ = T.make_router_inputs(M, E, DEV)
    tw, ti = fg.grouped_topk(torch.softmax(logits, -1), 1, 1, k, True, 1.0, torch.zeros(E, device=DEV), 0)
    fg.fused_experts_impl(x, w1, w2, tw.to(torch.bfloat16), ti)  # clean: no exception
    bad = ti.clone()
    bad[0, 0] = E + 3  # an expert id outside the table: skipped by align, reported in the status word
    with pytest.raises(fg.MoeKernelError, match="status word"):
        fg.fused_experts_impl(x, w1, w2, tw.to(torch.bfloat16), bad)
    assert fg.read_status() == 0

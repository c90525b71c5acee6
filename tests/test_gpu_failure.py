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


class _GuardedAllocator:
    """Stands in for torch.empty inside the layer: every workspace sits between two guard bands
    filled with a byte pattern, so a kernel that writes outside its buffer is caught."""

    GUARD = 4096  # bytes on either side (keeps the 16-byte / 1024-byte alignments the kernels ask for)
    PATTERN = 0xA5

    def __init__(self):
        self.real_empty = torch.empty
        self.blocks = []

    def __call__(self, *size, dtype=None, device=None, **kw):
        if len(size) == 1 and not isinstance(size[0], int):
            size = tuple(size[0])
        dtype = dtype or torch.get_default_dtype()
        if device is None or torch.device(device).type != "cuda" or kw:
            return self.real_empty(tuple(size), dtype=dtype, device=device, **kw)
        n = 1
        for s in size:
            n *= int(s)
        nbytes = n * self.real_empty((), dtype=dtype).element_size()
        padded = (nbytes + 255) // 256 * 256
        whole = torch.full((padded + 2 * self.GUARD,), self.PATTERN, dtype=torch.uint8, device=device)
        self.blocks.append((whole, padded))
        return whole[self.GUARD:self.GUARD + nbytes].view(dtype).view(size)

    def check(self):
        assert self.blocks, "no workspace was allocated through the guarded allocator"
        for whole, padded in self.blocks:
            lo, hi = whole[:self.GUARD], whole[self.GUARD + padded:]
            assert bool((lo == self.PATTERN).all()) and bool((hi == self.PATTERN).all()), \
                f"a kernel wrote outside a {padded}-byte workspace"
        return len(self.blocks)


@pytest.mark.parametrize("mode", ["bf16", "fp8", "w8a16"])
@pytest.mark.parametrize("M", [1, 5, 200, 1500])
def test_guard_bands_around_every_workspace_stay_intact(monkeypatch, mode, M):
    """All internal buffers of the layer (sorted ids, expert ids, quantised rows and scales, the
    sorted copies, the intermediate, y, the row index, split-K partial sums) are allocated with guard
    bands on both sides; after the layer every band still holds its pattern.  The sizes cover the
    small-batch schedule, the 128-row kernels with row stores and the staged TMA output."""
    E, H, I, k = 8, 512, 512, 2
    x = T.make_activations(M, H, DEV, seed=M)
    logits, _ = T.make_router_inputs(M, E, DEV, seed=M + 1)
    tw, ti = fg.grouped_topk(torch.softmax(logits, -1), 1, 1, k, True, 1.0, torch.zeros(E, device=DEV), 0)
    kw = {}
    if mode == "bf16":
        w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
        w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    elif mode == "fp8":
        w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1)
        w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2)
        kw = dict(use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2, block_shape=[128, 128])
    else:
        w1, s1 = T.make_int8_channel_weights(E, 2 * I, H, DEV, seed=1)
        w2, s2 = T.make_int8_channel_weights(E, H, I, DEV, seed=2)
        kw = dict(use_int8_w8a16=True, per_channel_quant=True, w1_scale=s1, w2_scale=s2)
    ref = fg.fused_experts_impl(x, w1, w2, tw, ti, **kw)
    guard = _GuardedAllocator()
    monkeypatch.setattr(torch, "empty", guard)
    try:
        out = fg.fused_experts_impl(x, w1, w2, tw, ti, **kw)
        torch.cuda.synchronize()
    finally:
        monkeypatch.undo()
    assert guard.check() >= 4
    assert torch.equal(out, ref) and fg.read_status(torch.device(DEV)) == 0

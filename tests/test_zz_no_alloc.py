"""The allocation-free GEMM 2 of the small-batch schedule against the ordinary entry point.

Some hosts of this library cannot allocate device memory when a layer runs: a serving
engine gives all free memory to its own pools at start-up, and a decode loop must not run
cudaMalloc / cudaFree between kernels because both stall the device.  For them
``moe_small_m_gemm2_static`` keeps its scratch (route rows, split-K partial sums, counter
tables) in a fixed array inside the library.  This test drives it through the C ABI and
checks the layer output against ``moe_small_m_gemm`` on the same inputs, twice in a row
with different batches, so that what the first call left in the shared array is shown not
to leak into the second.  It is collected last on purpose: a run that stops at the first
failure has then already run every other test."""

import ctypes

import pytest
import torch

from flaggems_vllm_b200 import _lib
from flaggems_vllm_b200 import testing as T
from flaggems_vllm_b200.align import round_up
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_L2, COS = 1e-2, 0.9999  # the layer tolerance of the other GPU tests


def _plan(L, mode, K, N, rows_cap, M, hint):
    sizes = (ctypes.c_int64 * 3)()
    base = ctypes.addressof(sizes)
    _lib.check(L.moe_small_m_plan(0, mode, K, N, rows_cap, M, hint, base, base + 8, base + 16))
    return int(sizes[0]), int(sizes[1]), int(sizes[2])


def _both_gemm2(M, seed, mode=_lib.MODE_HALF, hint=3):
    """Runs align and GEMM 1 through the ordinary entry points, then GEMM 2 through both."""
    L = _lib.lib()
    E, H, I, k = 16, 512, 1024, 4
    dev = torch.device(DEV)
    st = torch.cuda.current_stream().cuda_stream
    status = _lib.status_word(dev)
    x = T.make_activations(M, H, DEV, seed=seed)
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    logits, _ = T.make_router_inputs(M, E, DEV, seed=seed)
    tw, ti = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    tw, ti = (tw / tw.sum(-1, keepdim=True)).float().contiguous(), ti.to(torch.int32).contiguous()
    numel, bm = M * k, 8
    rows_cap = round_up(numel + min(numel, E) * (bm - 1), bm)
    sorted_ids = torch.empty(rows_cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(rows_cap // bm, dtype=torch.int32, device=dev)
    npp = torch.empty(1, dtype=torch.int32, device=dev)
    _lib.check(L.moe_align_block_size(ti.data_ptr(), 0, numel, E, bm, sorted_ids.data_ptr(), rows_cap,
                                      expert_ids.data_ptr(), expert_ids.numel(), npp.data_ptr(), status.data_ptr(), st))
    bf16 = _lib.dtype_code(torch.bfloat16)
    act = torch.empty((rows_cap, I), dtype=torch.bfloat16, device=dev)
    c1 = torch.zeros(rows_cap // bm * (I // 64) * 8, dtype=torch.int32, device=dev)
    _lib.check(L.moe_small_m_gemm(1, mode, bf16, x.data_ptr(), M, k, w1.data_ptr(), None, expert_ids.data_ptr(),
                                  sorted_ids.data_ptr(), npp.data_ptr(), None, E, tw.data_ptr(), 0, ti.data_ptr(), 0,
                                  rows_cap, E, H, I, act.data_ptr(), None, 1, None, c1.data_ptr(), None,
                                  status.data_ptr(), st))
    # ordinary entry point: the caller owns the scratch
    part, uc, tc = _plan(L, mode, I, H, rows_cap, M, hint)
    counters = torch.zeros(uc + tc, dtype=torch.int32, device=dev)
    partial = torch.empty(max(part, 1), dtype=torch.float32, device=dev)
    y = torch.empty((numel, H), dtype=torch.bfloat16, device=dev)
    ref = torch.full((M, H), float("nan"), dtype=torch.bfloat16, device=dev)
    _lib.check(L.moe_small_m_gemm(0, mode, bf16, act.data_ptr(), M, k, w2.data_ptr(), None, expert_ids.data_ptr(),
                                  sorted_ids.data_ptr(), npp.data_ptr(), None, E, tw.data_ptr(), 1, ti.data_ptr(), 0,
                                  rows_cap, E, I, H, y.data_ptr(), ref.data_ptr(), hint, partial.data_ptr(),
                                  counters.data_ptr(), counters.data_ptr() + 4 * uc, status.data_ptr(), st))
    # allocation-free entry point: inputs and the output only
    out = torch.full((M, H), float("nan"), dtype=torch.bfloat16, device=dev)
    _lib.check(L.moe_small_m_gemm2_static(mode, bf16, act.data_ptr(), M, k, w2.data_ptr(), None, expert_ids.data_ptr(),
                                          sorted_ids.data_ptr(), npp.data_ptr(), None, E, tw.data_ptr(), 1,
                                          ti.data_ptr(), 0, rows_cap, E, I, H, out.data_ptr(), hint,
                                          status.data_ptr(), st))
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 0
    oracle = O.fused_moe_half_oracle(x, w1, w2, tw, ti)
    return out, ref, oracle


def test_static_scratch_gemm2_matches_the_ordinary_entry_point_twice_in_a_row():
    for M, seed in ((24, 11), (5, 12)):  # the second batch is smaller: stale rows of the first stay in the array
        out, ref, oracle = _both_gemm2(M, seed)
        assert torch.isfinite(out.float()).all()
        rl2, cs = O.rel_l2(out.float(), ref.float()), O.cosine(out.float(), ref.float())
        assert rl2 <= REL_L2 and cs >= COS, f"M={M}: static-scratch GEMM2 vs ordinary: rel_l2={rl2:.3e} cos={cs:.6f}"
        rl2, cs = O.rel_l2(out.float(), oracle), O.cosine(out.float(), oracle)
        assert rl2 <= REL_L2 and cs >= COS, f"M={M}: static-scratch layer vs oracle: rel_l2={rl2:.3e} cos={cs:.6f}"


def test_static_scratch_gemm2_rejects_what_does_not_fit():
    L = _lib.lib()
    dev = torch.device(DEV)
    dummy = torch.zeros(64, dtype=torch.int32, device=dev)
    # 4096 tokens x 8 routes x 7168 columns of bf16 rows alone are 470 MB: far beyond the fixed array
    rc = L.moe_small_m_gemm2_static(_lib.MODE_HALF, _lib.dtype_code(torch.bfloat16), dummy.data_ptr(), 4096, 8,
                                    dummy.data_ptr(), None, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None,
                                    256, dummy.data_ptr(), 1, dummy.data_ptr(), 0, 8 * (4096 * 8 + 256 * 7) // 8, 256,
                                    2048, 7168, dummy.data_ptr(), 1, None, torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    assert b"fixed array holds" in L.moe_last_error()

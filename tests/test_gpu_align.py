"""GPU parity of moe_align_block_size: all three outputs byte-equal to the CPU
oracle (full buffers, sentinels included) and to the reference-made vectors."""

import numpy as np
import pytest
import torch

import flaggems_vllm_b200 as fg
from conftest import golden_files, load_golden
from flaggems_vllm_b200 import testing as T
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check(ids, bs, E, expert_map=None, pad_sorted_ids=False):
    s, e, n = fg.moe_align_block_size(ids, bs, E, expert_map, pad_sorted_ids)
    os_, oe, on = O.moe_align_block_size_oracle(ids, bs, E, expert_map, pad_sorted_ids)
    assert s.dtype == e.dtype == n.dtype == torch.int32
    assert np.array_equal(s.cpu().numpy(), os_)
    assert np.array_equal(e.cpu().numpy(), oe)
    assert np.array_equal(n.cpu().numpy(), on)
    return s, e, n


@pytest.mark.parametrize("name", golden_files("align_"))
def test_golden_vectors(name):
    g = load_golden(name)
    E, bs = [int(v) for v in g["params"]]
    s, e, n = fg.moe_align_block_size(g["topk_ids"].to(DEV), bs, E)
    ge = g["expert_ids"].numpy()
    assert np.array_equal(s.cpu().numpy(), g["sorted_ids"].numpy())
    assert np.array_equal(n.cpu().numpy(), g["num_post_pad"].numpy())
    assert np.array_equal(e.cpu().numpy()[: ge.size], ge) and np.all(e.cpu().numpy()[ge.size:] == -1)


@pytest.mark.parametrize("M", [1, 128, 2048, 8192])
@pytest.mark.parametrize("skewed", [False, True])
@pytest.mark.parametrize("bs", [64, 128])
def test_config5_bit_exact(M, skewed, bs):
    ids = T.make_align_ids(M, 8, 256, DEV, skewed=skewed, seed=M)
    _check(ids, bs, 256)


@pytest.mark.parametrize("M,k,E,bs", [(1, 1, 10, 16), (3, 2, 8, 16), (7, 8, 250, 32), (16384, 10, 512, 64),
                                      (32768, 8, 256, 128), (1000, 6, 128, 16), (4096, 4, 1024, 32),
                                      (513, 3, 4096, 16), (9, 8, 3, 7)])
def test_other_shapes(M, k, E, bs):
    ids = T.make_align_ids(M, k, E, DEV, seed=E + M)
    _check(ids, bs, E)
    _check(ids.long(), bs, E)


def test_empty_input():
    ids = torch.zeros((0, 8), dtype=torch.int32, device=DEV)
    s, e, n = _check(ids, 64, 256)
    assert int(n.item()) == 0


def test_invalid_ids_are_skipped_and_flagged():
    fg.read_status()
    ids = torch.tensor([[-1, 2], [9, 2], [3, 300]], dtype=torch.int32, device=DEV)
    _check(ids, 4, 8)
    assert fg.read_status() & 1  # MOE_ST_BAD_EXPERT_ID
    assert fg.read_status() == 0


def test_expert_map_and_pad_sorted_ids():
    ids = T.make_align_ids(77, 4, 16, DEV, seed=1)
    emap = torch.full((16,), -1, dtype=torch.int32, device=DEV)
    emap[4:8] = torch.arange(4, dtype=torch.int32, device=DEV)
    _check(ids, 16, 16, expert_map=emap)
    s, _, _ = _check(ids, 16, 16, pad_sorted_ids=True)
    assert s.numel() % 16 == 0


def test_no_tle_variant_uses_tight_bound():
    ids = T.make_align_ids(2, 2, 256, DEV, seed=2)
    s, e, n = fg.moe_align_block_size_no_tle(ids, 64, 256)
    assert s.numel() == 4 * 64 and e.numel() == 4
    os_, oe, on = O.moe_align_block_size_oracle(ids, 64, 256)
    assert np.array_equal(s.cpu().numpy(), os_[: s.numel()])
    assert np.array_equal(e.cpu().numpy(), oe[:4]) and int(n.item()) == int(on[0])


def test_caller_owned_buffers_and_determinism():
    ids = T.make_align_ids(8192, 8, 256, DEV, skewed=True, seed=11)
    cap = ids.numel() + 256 * 63
    first = None
    for _ in range(100):
        s = torch.full((cap,), -7, dtype=torch.int32, device=DEV)
        e = torch.full(((cap + 63) // 64,), -7, dtype=torch.int32, device=DEV)
        n = torch.full((1,), -7, dtype=torch.int32, device=DEV)
        fg.moe_align_block_size_triton(ids, 256, 64, s, e, n)
        cur = (s.clone(), e.clone(), n.clone())
        if first is None:
            first = cur
        else:
            assert all(torch.equal(a, b) for a, b in zip(first, cur))
    os_, oe, on = O.moe_align_block_size_oracle(ids, 64, 256)
    assert np.array_equal(first[0].cpu().numpy(), os_) and np.array_equal(first[1].cpu().numpy(), oe)


def test_sortedness_property_at_chunk_size():
    # size-independent properties at the largest chunk the layer ever aligns
    M, k, E, bs = 32768, 8, 256, 128
    ids = T.make_align_ids(M, k, E, DEV, seed=4)
    s, e, n = fg.moe_align_block_size(ids, bs, E)
    n = int(n.item())
    flat = ids.view(-1)
    sv = s[:n]
    valid = sv < flat.numel()
    assert int(valid.sum()) == flat.numel()                          # a permutation of all routes
    assert torch.equal(torch.sort(sv[valid])[0], torch.arange(flat.numel(), device=DEV, dtype=torch.int32))
    blk_e = e[: n // bs].repeat_interleave(bs)
    assert torch.equal(flat[sv[valid].long()], blk_e[valid])          # every route sits in its expert's block
    assert torch.all(blk_e[1:] >= blk_e[:-1])                         # experts ascend
    pos = torch.arange(n, device=DEV)
    same = (blk_e[1:] == blk_e[:-1]) & valid[1:] & valid[:-1]
    assert torch.all(sv[1:][same] > sv[:-1][same])                    # stable inside an expert
    assert torch.all(s[n:] == flat.numel()) and torch.all(e[n // bs:] == -1)
    del pos


def test_cuda_graph_capture_of_empty_and_nonempty():
    ids = T.make_align_ids(64, 8, 256, DEV, seed=8)
    static = ids.clone()
    fg.moe_align_block_size(static, 64, 256)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        s, e, n = fg.moe_align_block_size(static, 64, 256)
    for seed in (9, 10):
        fresh = T.make_align_ids(64, 8, 256, DEV, seed=seed)
        static.copy_(fresh)
        graph.replay()
        torch.cuda.synchronize()
        os_, oe, on = O.moe_align_block_size_oracle(fresh, 64, 256)
        assert np.array_equal(s.cpu().numpy(), os_) and np.array_equal(e.cpu().numpy(), oe)
        assert int(n.item()) == int(on[0])

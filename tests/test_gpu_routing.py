"""GPU parity of grouped_topk against the CPU oracle and the reference-made
golden vectors: ids bit-exact (ties toward the lower expert id), weights within
2e-6 (the tolerance of the reference's own eager-oracle tests,
tests/test_grouped_topk.py:737)."""

import pytest
import torch

import flaggems_vllm_b200 as fg
from conftest import golden_files, load_golden
from flaggems_vllm_b200 import testing as T
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}


def _check(scores, G, keep, k, ren, scale, bias, sf, pad=None):
    w, ids = fg.grouped_topk(scores, G, keep, k, ren, scale, bias, sf, pad)
    ow, oi = O.grouped_topk_oracle(scores, G, keep, k, ren, scale, bias, sf, pad)
    assert w.dtype == torch.float32 and ids.dtype == torch.int32
    assert w.shape == ids.shape == (scores.shape[0], k)
    assert torch.equal(ids.cpu(), oi)
    torch.testing.assert_close(w.cpu(), ow, rtol=2e-6, atol=2e-6)
    return w, ids


@pytest.mark.parametrize("name", golden_files("routing_"))
def test_golden_vectors(name):
    g = load_golden(name)
    E, G, keep, k, ren, sf = [int(v) for v in g["params"]]
    scores = g["scores"].to(DT[g["score_dtype"]]).to(DEV)
    w, ids = fg.grouped_topk(scores, G, keep, k, bool(ren), float(g["scale"][0]), g["bias"].to(DEV), sf)
    assert torch.equal(ids.cpu(), g["ids"])
    torch.testing.assert_close(w.cpu(), g["weights"], rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("M", [1, 32, 128, 1024, 8192])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_deepseek_v3_routing(M, dtype):
    logits, bias = T.make_router_inputs(M, 256, DEV, seed=M)
    _check(logits.to(dtype), 8, 4, 8, True, 2.5, bias, 1)


@pytest.mark.parametrize("E,k,M", [(8, 2, 64), (8, 2, 4096), (128, 8, 512), (128, 8, 4096)])
def test_softmax_routing_single_group(E, k, M):
    logits, _ = T.make_router_inputs(M, E, DEV, seed=E + M)
    scores = torch.softmax(logits, dim=-1)
    _check(scores, 1, 1, k, True, 1.0, torch.zeros(E, device=DEV), 0)


@pytest.mark.parametrize("E,G,keep,k", [(16, 4, 2, 2), (64, 4, 2, 6), (384, 3, 2, 4), (512, 1, 1, 16),
                                        (1024, 32, 4, 32), (24, 2, 1, 3)])
@pytest.mark.parametrize("sf", [0, 1])
def test_other_shapes(E, G, keep, k, sf):
    logits, bias = T.make_router_inputs(37, E, DEV, seed=E)
    for ren in (True, False):
        _check(logits, G, keep, k, ren, 1.5, bias, sf)
        _check(logits.half(), G, keep, k, ren, 1.5, bias.half(), sf)


@pytest.mark.parametrize("E,G,keep,k", [(2048, 8, 4, 8), (4096, 1, 1, 32), (1536, 16, 3, 6), (1280, 32, 32, 1),
                                        (4096, 32, 2, 32)])
@pytest.mark.parametrize("sf", [0, 1])
def test_wide_routers_beyond_one_warp_of_registers(E, G, keep, k, sf):
    """More than 1024 experts: the one-CTA-per-token kernel, same ordering rules (the reference
    serves such widths through its generic path)."""
    logits, bias = T.make_router_inputs(19, E, DEV, seed=E + G)
    pad = torch.zeros(19, dtype=torch.bool, device=DEV)
    pad[3] = True
    for ren in (True, False):
        _check(logits, G, keep, k, ren, 1.5, bias, sf)
        _check(logits.to(torch.bfloat16), G, keep, k, ren, 1.5, bias, sf)
    w, ids = fg.grouped_topk(logits, G, keep, k, True, 1.0, bias, sf, pad)
    assert torch.all(ids[3] == -1) and torch.all(w[3] == 0)
    # ties: equal scores are ranked by the lower expert id
    w, ids = fg.grouped_topk(torch.ones((2, E), device=DEV), 1, 1, k, True, 1.0, torch.zeros(E, device=DEV), 0)
    assert torch.equal(ids.cpu(), torch.arange(k, dtype=torch.int32).expand(2, k))


@pytest.mark.parametrize("groups,keep", [(1, 1), (8, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("separate", [False, True])
def test_known_answer_ties_and_tiny_bias(groups, keep, dtype, separate):
    scores = torch.ones((3, 256), device=DEV, dtype=dtype)
    bias = torch.arange(256, device=DEV, dtype=torch.float32) * (2**-20 if separate else 0.0)
    w, ids = fg.grouped_topk(scores, groups, keep, 8, True, 2.5, bias, 0)
    exp = torch.arange(255, 247, -1) if separate else torch.arange(8)
    assert torch.equal(ids.cpu(), exp.expand(3, -1).int())
    torch.testing.assert_close(w, torch.full_like(w, 2.5 / 8))


@pytest.mark.parametrize("experts,topk", [(8, 3), (17, 5), (63, 7), (129, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_known_answer_strided_ties(experts, topk, dtype):
    backing = torch.ones((5, experts + 11), device=DEV, dtype=dtype)
    scores = backing[:, :experts]
    w, ids = fg.grouped_topk(scores, 1, 1, topk, True, 1.0, torch.zeros(experts, device=DEV), 0)
    assert torch.equal(ids.cpu(), torch.arange(topk, dtype=torch.int32).expand(5, -1))
    torch.testing.assert_close(w, torch.full_like(w, 1.0 / topk))


@pytest.mark.parametrize("groups,keep", [(1, 1), (8, 4)])
def test_known_answer_inf_and_signed_zero(groups, keep):
    scores = torch.ones((2, 256), device=DEV)
    scores[:, [1, 253]] = float("inf")
    bias = torch.zeros(256, device=DEV)
    w, ids = fg.grouped_topk(scores, groups, keep, 8, False, 1.0, bias, 0)
    assert torch.equal(ids.cpu(), torch.tensor([1, 253, 0, 2, 3, 4, 5, 6]).int().expand(2, -1))
    assert torch.isposinf(w[:, :2]).all()
    torch.testing.assert_close(w[:, 2:], torch.ones_like(w[:, 2:]))
    scores.zero_()
    scores[:, ::2] = -0.0
    w, ids = fg.grouped_topk(scores, groups, keep, 8, False, 1.0, bias, 0)
    assert torch.equal(ids.cpu(), torch.arange(8).int().expand(2, -1))
    assert torch.equal(torch.signbit(w), torch.signbit(scores[:, :8]))


@pytest.mark.parametrize("mode", ["mixed", "all", "none"])
def test_padding_rows(mode):
    rows, E = 9, 256
    score = torch.linspace(-2.0, 2.0, E, device=DEV)
    scores = torch.stack([score.roll(i * 17) for i in range(rows)])
    bias = torch.linspace(-0.30, 0.30, E, device=DEV)
    if mode == "mixed":
        mask = torch.arange(rows, device=DEV) % 3 == 1
    else:
        mask = torch.full((rows,), mode == "all", device=DEV, dtype=torch.bool)
    w, ids = _check(scores, 8, 4, 8, True, 3.998, bias, 1, mask)
    assert torch.all(w[mask] == 0) and torch.all(ids[mask] == -1)


def test_empty_and_2d_bias():
    w, ids = fg.grouped_topk(torch.zeros((0, 256), device=DEV), 8, 4, 8, True, 2.5, torch.zeros(256, device=DEV), 1)
    assert w.shape == (0, 8) and ids.shape == (0, 8)
    logits, bias = T.make_router_inputs(5, 64, DEV)
    _check(logits, 4, 2, 4, True, 1.0, bias.view(1, 64), 1)


def test_cuda_graph_replay_with_new_scores():
    logits, bias = T.make_router_inputs(64, 256, DEV, seed=5)
    static = logits.clone()
    fg.grouped_topk(static, 8, 4, 8, True, 2.5, bias, 1)  # warm-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        w, ids = fg.grouped_topk(static, 8, 4, 8, True, 2.5, bias, 1)
    for seed in (6, 7):
        fresh, _ = T.make_router_inputs(64, 256, DEV, seed=seed)
        static.copy_(fresh)
        graph.replay()
        torch.cuda.synchronize()
        ow, oi = O.grouped_topk_oracle(fresh, 8, 4, 8, True, 2.5, bias, 1)
        assert torch.equal(ids.cpu(), oi)
        torch.testing.assert_close(w.cpu(), ow, rtol=2e-6, atol=2e-6)


# ---------------------------------------------------------------- non-grouped routers
def _route_outputs(m, k, index_dtype=torch.int32):
    return (torch.empty((m, k), device=DEV), torch.empty((m, k), device=DEV, dtype=index_dtype),
            torch.empty((m, k), device=DEV, dtype=torch.int32))


@pytest.mark.parametrize("name", golden_files("topk_sigmoid_"))
def test_topk_sigmoid_golden_vectors(name):
    g = load_golden(name)
    k, ren, bias_on = [int(v) for v in g["params"]]
    logits = g["logits"].to(DEV)
    w, ids, src = _route_outputs(logits.shape[0], k)
    fg.topk_sigmoid(w, ids, src, logits, bool(ren), g["bias"].to(DEV) if bias_on else None)
    assert torch.equal(ids.cpu(), g["ids"]) and torch.equal(src.cpu(), g["source"])
    torch.testing.assert_close(w.cpu(), g["weights"], atol=2e-7, rtol=2e-6)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(0, 32, 4), (1, 64, 8), (7, 128, 8), (64, 256, 4), (4096, 128, 8), (33, 1000, 32)])
@pytest.mark.parametrize("renormalize", [False, True])
@pytest.mark.parametrize("bias_on", [False, True])
@pytest.mark.parametrize("sigmoid", [False, True])
def test_topk_routers_match_oracle(dtype, shape, renormalize, bias_on, sigmoid):
    m, e, k = shape
    logits = (torch.randn((m, e), generator=torch.Generator().manual_seed(31)) * 2).to(dtype).to(DEV)
    bias = (torch.randn((e,), generator=torch.Generator().manual_seed(5)) * 0.1).to(DEV) if bias_on else None
    for idt in (torch.int32, torch.int64):
        w, ids, src = _route_outputs(m, k, idt)
        if sigmoid:
            fg.topk_sigmoid(w, ids, src, logits, renormalize, bias, 2.5)
        else:
            fg.topk_softmax(w, ids, src, logits, renormalize, bias)
        ow, oi, osrc = O.topk_route_oracle(logits, bias, k, renormalize, sigmoid, 2.5 if sigmoid else 1.0)
        assert torch.equal(ids.cpu().long(), oi) and torch.equal(src.cpu(), osrc)
        torch.testing.assert_close(w.cpu(), ow, atol=2e-7, rtol=2e-6)


@pytest.mark.parametrize("normalize", [False, True])
@pytest.mark.parametrize("expert_count", [5, 256, 257, 512])
@pytest.mark.parametrize("sigmoid", [False, True])
def test_topk_routers_bias_padding_and_nonfinite(normalize, expert_count, sigmoid):
    # the fixture of tests/test_topk_softmax.py:121-164 in the reference
    logits = torch.tensor([[2, 1, 0, 1, 4], [4, 3, 2, 1, 0], [1, 3, 2, 3, 0], [float("nan"), 1, 2, 3, 4],
                           [float("inf"), 1, 2, 3, 4], [float("-inf")] * 5], device=DEV)
    bias = torch.tensor([0.0, 0.75, 0.0, 0.75, -0.5], device=DEV)
    if expert_count > 5:
        extra = torch.arange(expert_count - 5, device=DEV)
        logits = torch.cat((logits, (extra.remainder(13).float() / 5 - 2).expand(6, -1)), dim=1).contiguous()
        bias = torch.cat((bias, (extra.remainder(7).float() - 3) * 0.03125))
    padding = torch.tensor([False, True, False, False, False, False], device=DEV)
    w, ids, src = _route_outputs(6, 3, torch.int64)
    if sigmoid:
        fg.topk_sigmoid(w, ids, src, logits, normalize, bias, 1.0, padding)
    else:
        fg.topk_softmax(w, ids, src, logits, normalize, bias, padding)
    ow, oi, osrc = O.topk_route_oracle(logits, bias, 3, normalize, sigmoid, is_padding=padding)
    assert torch.equal(ids.cpu(), oi) and torch.equal(src.cpu(), osrc)
    torch.testing.assert_close(w.cpu(), ow, atol=2e-7, rtol=2e-6)
    assert torch.all(w[1] == 0) and torch.all(ids[1] == -1)


def test_topk_sigmoid_ties_nan_and_graph_replay():
    logits = torch.zeros((3, 128), device=DEV)
    logits[1] = float("nan")
    logits[2] = -float("inf")
    w, ids, src = _route_outputs(3, 8)
    fg.topk_sigmoid(w, ids, src, logits, True)
    ow, oi, _ = O.topk_route_oracle(logits, None, 8, True, True)
    assert torch.equal(ids.cpu().long(), oi)
    torch.testing.assert_close(w.cpu(), ow)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fg.topk_sigmoid(w, ids, src, logits, True)
    logits.copy_(torch.randn_like(logits))
    graph.replay()
    torch.cuda.synchronize()
    ow, oi, _ = O.topk_route_oracle(logits, None, 8, True, True)
    assert torch.equal(ids.cpu().long(), oi)
    torch.testing.assert_close(w.cpu(), ow, atol=2e-7, rtol=2e-6)


# ---------------------------------------------------------------- router GEMMs
# shapes of the reference's tests/test_router_gemm.py:22-37 plus prefill sizes served by the tensor-core kernel
@pytest.mark.parametrize("shape", [(1, 256, 7168), (8, 256, 7168), (16, 256, 7168), (32, 256, 7168), (128, 256, 7168),
                                   (1, 64, 4096), (16, 128, 4096), (64, 384, 7168), (0, 256, 7168),
                                   (1000, 256, 7168), (8192, 256, 7168), (65, 200, 4096), (300, 8, 512)])
def test_router_gemm_matches_oracle(shape):
    M, N, K = shape
    g = torch.Generator(device="cpu").manual_seed(M + N)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn((N, K), generator=g).to(torch.bfloat16).to(DEV)
    out = fg.router_gemm(x, w)
    assert out.shape == (M, N) and out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), O.router_gemm_oracle(x, w), rtol=1e-4, atol=2e-3)
    if M > 0:  # both kernels reduce in a fixed order: bitwise repeatable
        assert torch.equal(out, fg.router_gemm(x, w))
    if M > 64:  # f16 takes the tensor-core kernel too; f32 operands the row-streaming kernel at any M
        outh = fg.router_gemm(x.half(), w.half())
        torch.testing.assert_close(outh.cpu(), O.router_gemm_oracle(x.half(), w.half()), rtol=1e-4, atol=2e-3)
        if M <= 1000:
            outf = fg.router_gemm(x.float(), w.float())
            torch.testing.assert_close(outf.cpu(), O.router_gemm_oracle(x, w), rtol=1e-4, atol=2e-3)


@pytest.mark.parametrize("M", [1, 7, 32, 64, 130])
@pytest.mark.parametrize("cfg", [(256, 7168, 8, 4, 8, 1), (128, 2048, 1, 1, 8, 0), (64, 4096, 4, 2, 6, 1)])
def test_router_gemm_fused_with_grouped_topk(M, cfg):
    """One launch from hidden states to (weights, ids): bit for bit the two separate ops, and the ids are those
    the oracle picks from the kernel's own logits."""
    E, K, n_group, topk_group, k, scoring = cfg
    g = torch.Generator(device="cpu").manual_seed(M + E)
    x = (torch.randn((M, K), generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn((E, K), generator=g) * K**-0.5).to(torch.bfloat16).to(DEV)
    bias = (torch.randn((E,), generator=g) * 0.1).to(DEV)
    tw, ti, logits = fg.router_gemm_grouped_topk(x, w, n_group, topk_group, k, True, 2.5, bias, scoring,
                                                 return_logits=True)
    sep_logits = fg.router_gemm(x, w) if M <= 64 else None
    if sep_logits is not None:
        assert torch.equal(logits, sep_logits)
    rw, ri = fg.grouped_topk(logits, n_group, topk_group, k, True, 2.5, bias, scoring)
    assert torch.equal(ti, ri) and torch.equal(tw, rw)
    ow, oi = O.grouped_topk_oracle(logits, n_group, topk_group, k, True, 2.5, bias, scoring)
    assert torch.equal(ti.cpu(), oi)
    torch.testing.assert_close(tw.cpu(), ow, atol=2e-6, rtol=2e-6)
    torch.testing.assert_close(logits.cpu(), O.router_gemm_oracle(x, w), rtol=1e-4, atol=2e-3)
    tw2, ti2 = fg.router_gemm_grouped_topk(x, w, n_group, topk_group, k, True, 2.5, bias, scoring)
    assert torch.equal(ti2, ti) and torch.equal(tw2, tw)


# tests/test_fp32_router_gemm.py:14-38 (same sizes, value scales, strides and tolerances)
@pytest.mark.parametrize("m", [0, 1, 3, 4, 8, 16, 32])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("strided", [False, True])
def test_fp32_router_gemm_matches_oracle(m, dtype, strided):
    g = torch.Generator(device="cpu").manual_seed(29)
    cols = 12288 if strided else 6144
    x = torch.randn((m, cols), generator=g).to(dtype).to(DEV)
    w = (torch.randn((128, cols), generator=g) * 0.01).to(DEV)
    if strided:
        x, w = x[:, ::2], w[:, ::2]
    out = fg.fp32_router_gemm(x, w)
    assert out.shape == (m, 128) and out.dtype == torch.float32
    expected = torch.mm(x.cpu().double(), w.cpu().double().t()).float()  # correctly rounded fp32 logits
    torch.testing.assert_close(out.cpu(), expected, atol=3e-6, rtol=2e-5)
    torch.testing.assert_close(out.cpu(), O.router_gemm_oracle(x, w), atol=3e-6, rtol=2e-5)
    if m:
        assert torch.equal(out.cpu().argmax(-1), expected.argmax(-1))
        assert torch.equal(out, fg.fp32_router_gemm(x, w))
    with pytest.raises(NotImplementedError):
        fg.fp32_router_gemm(torch.zeros((33, 6144), device=DEV, dtype=dtype), w)
    with pytest.raises(NotImplementedError):
        fg.fp32_router_gemm(torch.zeros((2, 7168), device=DEV, dtype=dtype), torch.zeros((128, 7168), device=DEV))


def test_fp32_router_gemm_under_graph_replay():
    x = torch.randn((4, 6144), device=DEV, dtype=torch.bfloat16)
    w = torch.randn((128, 6144), device=DEV) * 0.01
    fg.fp32_router_gemm(x, w)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fg.fp32_router_gemm(x, w)
    x.mul_(-1)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, fg.fp32_router_gemm(x, w))

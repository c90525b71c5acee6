"""Pins the CPU oracle against vectors produced by the reference's own golden
functions (tests/golden/*.npz, see tests/golden/make_golden.py) and against the
known-answer cases the reference tests spell out."""

import numpy as np
import pytest
import torch

from conftest import golden_files, load_golden
from oracle import moe_oracle as O

DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16,
      "torch.float16": torch.float16}


@pytest.mark.parametrize("name", golden_files("routing_"))
def test_routing_matches_reference_golden(name):
    g = load_golden(name)
    E, G, keep, k, ren, sf = [int(v) for v in g["params"]]
    scale = float(g["scale"][0])
    scores = g["scores"].to(DT[g["score_dtype"]])
    w, ids = O.grouped_topk_oracle(scores, G, keep, k, bool(ren), scale, g["bias"], sf)
    assert torch.equal(ids, g["ids"])
    torch.testing.assert_close(w, g["weights"], rtol=2e-6, atol=2e-6)
    if "ids_packed" in g:  # the second, independent golden of the reference agrees too
        assert torch.equal(ids, g["ids_packed"])
        torch.testing.assert_close(w, g["weights_packed"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("groups,keep", [(1, 1), (8, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("separate", [False, True])
def test_routing_known_answer_ties_and_tiny_bias(groups, keep, dtype, separate):
    # reference: tests/test_grouped_topk.py:811-830
    scores = torch.ones((3, 256), dtype=dtype)
    bias = torch.arange(256, dtype=torch.float32) * (2**-20 if separate else 0.0)
    w, ids = O.grouped_topk_oracle(scores, groups, keep, 8, True, 2.5, bias, 0)
    exp = torch.arange(255, 247, -1) if separate else torch.arange(8)
    assert torch.equal(ids, exp.expand(3, -1).int())
    torch.testing.assert_close(w, torch.full_like(w, 2.5 / 8))


@pytest.mark.parametrize("groups,keep", [(1, 1), (8, 4)])
def test_routing_known_answer_inf_and_signed_zero(groups, keep):
    # reference: tests/test_grouped_topk.py:846-867
    scores = torch.ones((2, 256))
    scores[:, [1, 253]] = float("inf")
    bias = torch.zeros(256)
    w, ids = O.grouped_topk_oracle(scores, groups, keep, 8, False, 1.0, bias, 0)
    exp = torch.tensor([1, 253, 0, 2, 3, 4, 5, 6]).int()
    assert torch.equal(ids, exp.expand(2, -1))
    assert torch.isposinf(w[:, :2]).all()
    scores.zero_()
    scores[:, ::2] = -0.0
    w, ids = O.grouped_topk_oracle(scores, groups, keep, 8, False, 1.0, bias, 0)
    assert torch.equal(ids, torch.arange(8).int().expand(2, -1))
    assert torch.equal(torch.signbit(w), torch.signbit(scores[:, :8]))


@pytest.mark.parametrize("experts,topk", [(8, 3), (17, 5), (63, 7), (129, 8)])
def test_routing_known_answer_strided_ties(experts, topk):
    # reference: tests/test_grouped_topk.py:833-843
    backing = torch.ones((5, experts + 11))
    scores = backing[:, :experts]
    w, ids = O.grouped_topk_oracle(scores, 1, 1, topk, True, 1.0, torch.zeros(experts), 0)
    assert torch.equal(ids, torch.arange(topk, dtype=torch.int32).expand(5, -1))
    torch.testing.assert_close(w, torch.full_like(w, 1.0 / topk))


def test_routing_padding_rows():
    scores = torch.randn(9, 256)
    mask = torch.arange(9) % 3 == 1
    w, ids = O.grouped_topk_oracle(scores, 8, 4, 8, True, 2.5, torch.zeros(256), 1, is_padding=mask)
    assert torch.all(w[mask] == 0) and torch.all(ids[mask] == -1)
    assert torch.all(ids[~mask] >= 0)


@pytest.mark.parametrize("name", golden_files("align_"))
def test_align_matches_reference_golden(name):
    g = load_golden(name)
    E, bs = [int(v) for v in g["params"]]
    s, e, n = O.moe_align_block_size_oracle(g["topk_ids"], bs, E)
    gs, ge, gn = g["sorted_ids"].numpy(), g["expert_ids"].numpy(), g["num_post_pad"].numpy()
    assert np.array_equal(s, gs)
    assert np.array_equal(n, gn)
    # the golden sizes expert_ids with floor division, the public function
    # with ceil: compare the common prefix, the extra tail must be -1
    assert np.array_equal(e[: ge.size], ge)
    assert np.all(e[ge.size:] == -1)


def test_align_known_answer_tiny_orders():
    # reference: tests/test_moe_align_block_size.py:605-646
    s, e, n = O.moe_align_block_size_oracle(torch.tensor([[1, 3]], dtype=torch.int32), 8, 8)
    assert n[0] == 16 and list(e[:2]) == [1, 3]
    assert s[0] == 0 and s[8] == 1 and np.all(s[1:8] == 2) and np.all(s[9:16] == 2)
    ids = torch.tensor([[0, 1], [1, 2], [2, 3], [3, 0]], dtype=torch.int32)
    s, e, n = O.moe_align_block_size_oracle(ids, 8, 8)
    assert n[0] == 32 and list(e[:4]) == [0, 1, 2, 3]
    assert list(s[0:2]) == [0, 7] and list(s[8:10]) == [1, 2]
    assert list(s[16:18]) == [3, 4] and list(s[24:26]) == [5, 6]


def test_align_empty_and_invalid_ids():
    s, e, n = O.moe_align_block_size_oracle(torch.zeros((0, 8), dtype=torch.int32), 16, 8)
    assert n[0] == 0 and np.all(e == -1) and np.all(s == 0)
    ids = torch.tensor([[-1, 2], [9, 2]], dtype=torch.int32)
    s, e, n = O.moe_align_block_size_oracle(ids, 4, 8)
    assert n[0] == 4 and list(s[:4]) == [1, 3, 4, 4] and e[0] == 2


def test_align_expert_map_and_pad_sorted():
    ids = torch.tensor([[0, 3], [3, 1]], dtype=torch.int32)
    emap = torch.tensor([-1, 0, -1, 1], dtype=torch.int32)
    s, e, n = O.moe_align_block_size_oracle(ids, 4, 4, expert_map=emap, pad_sorted_ids=True)
    assert s.size % 4 == 0 and n[0] == 12
    assert list(e[:3]) == [-1, 0, 1]
    # unused blocks hold -1 before the lookup, which indexes the LAST map entry
    assert np.all(e[3:] == 1)


def test_quant_fp8_matches_reference_golden():
    g = load_golden("quant_fp8_0.npz")
    q, s = O.per_token_group_quant_fp8_oracle(g["x"], 128, reciprocal=True)
    nz = g["x"].float().reshape(-1, 128).abs().amax(dim=1).reshape(s.shape) > 0
    assert torch.equal(s[nz], g["s"][nz])
    # all-zero groups: the golden clamps eps in bf16, the kernel (and the oracle) in fp32
    torch.testing.assert_close(s[~nz], g["s"][~nz], rtol=1e-3, atol=0)
    assert torch.equal(q.view(torch.uint8), g["q"].view(torch.uint8))


@pytest.mark.parametrize("name", golden_files("quant_fp8_group_"))
def test_quant_fp8_other_group_sizes_match_reference_golden(name):
    g = load_golden(name)
    group, eps = int(g["params"][0]), float(g["params"][1])
    q, s = O.per_token_group_quant_fp8_oracle(g["x"], group, eps=eps, reciprocal=True)
    # the golden clamps in bf16 (the input dtype), the kernel and the oracle in fp32: groups whose
    # amax is below the clamp may differ in the last bits of the scale
    big = g["x"].float().reshape(-1, group).abs().amax(dim=1).reshape(s.shape) > eps
    assert torch.equal(s[big], g["s"][big])
    torch.testing.assert_close(s[~big], g["s"][~big], rtol=1e-2, atol=0)
    rows_big = big.repeat_interleave(group, dim=-1)
    assert torch.equal(q.view(torch.uint8)[rows_big], g["q"].view(torch.uint8)[rows_big])


@pytest.mark.parametrize("name", golden_files("quant_int8_"))
def test_int8_per_token_quant_and_swigluoai_match_reference_literals(name):
    g = load_golden(name)
    dt = {"torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}[g["dtype"]]
    x = g["x"].to(dt)
    q, s = O.int8_per_token_quant_oracle(x)
    # amax * fp32(1/127) (the kernel, which the oracle follows) against amax / 127 (the literal): the same
    # fp32 value or its neighbour; where they differ, a quotient that sits on a half-way point (26 / (52/127)
    # = 63.5) may round to either side
    torch.testing.assert_close(s, g["s"], rtol=2e-7, atol=0)
    same = (s == g["s"]).expand_as(q)
    assert torch.equal(q[same], g["q"][same])
    assert (q.int() - g["q"].int()).abs().max() <= 1 and same.float().mean() > 0.7
    out = O.swigluoai_oracle(g["packed"].to(dt)).to(dt)
    assert torch.equal(out.float(), g["oai"].to(dt).float())


@pytest.mark.parametrize("name", golden_files("layer_w8a8_int8_"))
def test_int8_w8a8_layer_oracle_matches_reference_literal_loop(name):
    g = load_golden(name)
    dt = {"torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}[g["dtype"]]
    out = O.fused_moe_row_scaled_oracle(g["x"].to(dt), g["w1"], g["w2"], g["w1_scale"], g["w2_scale"],
                                        g["topk_weights"], g["topk_ids"], fmt="int8", per_token=True,
                                        activation="swigluoai_uninterleave")
    ref = g["out"]
    # the literal rounds the sum of the routes to the activation dtype; the oracle returns fp32
    torch.testing.assert_close(out.to(dt).float(), ref, rtol=1.6e-2 if dt == torch.bfloat16 else 3e-3,
                               atol=4e-3 if dt == torch.bfloat16 else 5e-4)
    assert O.rel_l2(out, ref) < 4e-3


def test_quant_fp8_power_of_two_scales_match_reference_golden():
    g = load_golden("quant_fp8_ue8m0_0.npz")
    q, s = O.per_token_group_quant_fp8_oracle(g["x"], 128, reciprocal=True, scale_ue8m0=True)
    nz = g["x"].float().reshape(-1, 128).abs().amax(dim=1).reshape(s.shape) > 0
    assert torch.equal(s[nz], g["s"][nz])
    assert torch.equal(torch.exp2(torch.round(torch.log2(s))), s)  # powers of two
    assert torch.equal(q.view(torch.uint8), g["q"].view(torch.uint8))


@pytest.mark.parametrize("name", golden_files("layer_half_"))
def test_layer_half_matches_reference_golden(name):
    g = load_golden(name)
    dt = DT[g["dtype"]]
    x, w1, w2 = g["x"].to(dt), g["w1"].to(dt), g["w2"].to(dt)
    tw, ti = O.softmax_topk_oracle(g["gating"], g["topk_ids"].shape[1], dt)
    assert torch.equal(ti, g["topk_ids"])
    torch.testing.assert_close(tw.float(), g["topk_weights"])
    out = O.fused_moe_half_oracle(x, w1, w2, tw, ti)
    # the golden accumulates the k routes in the activation dtype; the oracle
    # keeps fp32, so they agree to activation-dtype rounding
    assert O.rel_l2(out, g["out"]) < 6e-3
    assert O.cosine(out, g["out"]) > 0.9999


@pytest.mark.parametrize("name", golden_files("layer_fp8_"))
def test_layer_fp8_matches_reference_golden(name):
    g = load_golden(name)
    x = g["x"]
    xq, xs = O.per_token_group_quant_fp8_oracle(x, 128, reciprocal=False)
    assert torch.equal(xs, g["xs"])
    assert torch.equal(xq.view(torch.uint8), g["xq"].view(torch.uint8))
    out = O.fused_moe_fp8_block_oracle(
        x, g["w1"], g["w2"], g["w1_scale"], g["w2_scale"],
        g["topk_weights"].to(x.dtype), g["topk_ids"], faithful=True, reciprocal=False)
    assert O.rel_l2(out, g["out"]) < 1e-2
    assert O.cosine(out, g["out"]) > 0.9999


@pytest.mark.parametrize("name", golden_files("layer_w8a16_"))
def test_layer_w8a16_matches_reference_golden(name):
    g = load_golden(name)
    x = g["x"]
    out = O.fused_moe_w8a16_oracle(x, g["w1"], g["w2"], g["w1_scale"], g["w2_scale"],
                                   g["topk_weights"].to(x.dtype), g["topk_ids"])
    assert O.rel_l2(out, g["out"]) < 6e-3
    assert O.cosine(out, g["out"]) > 0.9999


def test_block_matmul_oracle_against_plain_dequant():
    torch.manual_seed(3)
    a = torch.randn(5, 256)
    b = torch.randn(384, 256) * 0.05
    aq, as_ = O.per_token_group_quant_fp8_oracle(a, 128)
    bq, bs = O.quantize_weight_fp8_block(b[None])
    c = O.block_scaled_matmul_oracle(aq, as_, bq[0], bs[0], 128, 128)
    ad = aq.float() * as_.repeat_interleave(128, dim=1)
    bd = bq[0].float() * bs[0].repeat_interleave(128, 0).repeat_interleave(128, 1)
    torch.testing.assert_close(c, ad @ bd.t(), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("name", golden_files("topk_sigmoid_"))
def test_topk_sigmoid_matches_reference_golden(name):
    g = load_golden(name)
    k, ren, bias_on = [int(v) for v in g["params"]]
    w, ids, src = O.topk_route_oracle(g["logits"], g["bias"] if bias_on else None, k, bool(ren), True)
    assert torch.equal(ids.int(), g["ids"]) and torch.equal(src, g["source"])
    torch.testing.assert_close(w, g["weights"], atol=2e-7, rtol=2e-6)


def test_topk_softmax_known_answer_bias_padding_nonfinite():
    # reference: tests/test_topk_softmax.py:121-164
    logits = torch.tensor([[2, 1, 0, 1, 4], [4, 3, 2, 1, 0], [1, 3, 2, 3, 0], [float("nan"), 1, 2, 3, 4],
                           [float("inf"), 1, 2, 3, 4], [float("-inf")] * 5])
    bias = torch.tensor([0.0, 0.75, 0.0, 0.75, -0.5])
    padding = torch.tensor([False, True, False, False, False, False])
    for ren in (False, True):
        w, ids, src = O.topk_route_oracle(logits, bias, 3, ren, False, is_padding=padding)
        probabilities = torch.softmax(logits.float(), dim=-1).nan_to_num()
        exp_ids = torch.argsort(probabilities + bias, dim=-1, descending=True, stable=True)[:, :3]
        exp_w = probabilities.gather(1, exp_ids)
        if ren:
            den = exp_w.sum(-1, keepdim=True)
            exp_w = exp_w / torch.where(den > 0, den, torch.ones_like(den))
        assert torch.equal(ids, exp_ids.masked_fill(padding[:, None], -1))
        torch.testing.assert_close(w, exp_w.masked_fill(padding[:, None], 0))
        assert torch.equal(src, (torch.arange(3)[None, :] * 6 + torch.arange(6)[:, None]).int())


def test_silu_and_mul_oracle_known_answers():
    """tests/test_silu_and_mul.py of the reference states the golden as torch.mul(silu(a), b)."""
    import math

    a = torch.tensor([0.0, 1.0, -1.0, 20.0, -20.0], dtype=torch.float32)
    b = torch.tensor([3.0, 2.0, 2.0, 0.5, 1.0], dtype=torch.float32)
    out = O.silu_and_mul_oracle(a, b)
    sig = lambda v: 1.0 / (1.0 + math.exp(-v))
    want = torch.tensor([0.0, 2.0 * sig(1.0), -2.0 * sig(-1.0), 10.0 * sig(20.0), -20.0 * sig(-20.0)], dtype=torch.float64)
    torch.testing.assert_close(out, want, rtol=1e-12, atol=1e-15)

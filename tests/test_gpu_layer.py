"""GPU parity of fused_experts_impl against the CPU oracle.

Tolerance (stated by the task's parity definition): relative L2 <= 1e-2 and
cosine >= 0.9999 against the oracle's fp32-accumulate result on the same
seeded inputs; the reference's own assert_close tolerances are checked too."""

import os

import pytest
import torch

import flaggems_vllm_b200 as fg
from conftest import golden_files, load_golden
from flaggems_vllm_b200 import _lib, fused_moe
from flaggems_vllm_b200 import testing as T
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_L2, COS = 1e-2, 0.9999
DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}


def _assert_parity(out, ref, what=""):
    rl2, cs = O.rel_l2(out.float(), ref), O.cosine(out.float(), ref)
    assert fg.read_status() == 0, f"{what}: kernel status word set"
    assert rl2 <= REL_L2 and cs >= COS, f"{what}: rel_l2={rl2:.3e} cos={cs:.6f}"
    return rl2, cs


def _route(M, E, k, dtype, seed=0):
    logits, _ = T.make_router_inputs(M, E, DEV, seed=seed)
    w, ids = fg.grouped_topk(torch.softmax(logits, -1), 1, 1, k, True, 1.0, torch.zeros(E, device=DEV), 0)
    return w.to(dtype), ids


def _both_kernels(run):
    """Runs ``run()`` with each GEMM kernel: the generic one, the tensor-core
    kernel with one CTA per 128-row block, and the CTA-pair (cta_group::2) one.
    MOE_TEST_KERNELS = generic | tensor | widen | pair | wide | pairwide | presort | presortwide | both
    (default: all)."""
    outs = {}
    which = os.environ.get("MOE_TEST_KERNELS", "both")
    off = {"FLAGGEMS_B200_GENERIC_GEMM": "0", "FLAGGEMS_B200_TC_PAIR": "0", "FLAGGEMS_B200_TC_WIDE": "0",
           "FLAGGEMS_B200_TC_PAIR_WIDE": "0", "FLAGGEMS_B200_W8_WIDEN": "0", "FLAGGEMS_B200_PRESORT": "0"}
    variants = (("generic", dict(off, FLAGGEMS_B200_GENERIC_GEMM="1")),
                ("tensor", off),
                ("widen", dict(off, FLAGGEMS_B200_W8_WIDEN="1")),  # weight-only int8: widening pass + half kernels
                ("pair", dict(off, FLAGGEMS_B200_TC_PAIR="1")),
                ("wide", dict(off, FLAGGEMS_B200_TC_WIDE="1")),  # half precision only; FP8 falls back to "tensor"
                ("pairwide", dict(off, FLAGGEMS_B200_TC_PAIR_WIDE="1")),  # half precision only
                ("presort", dict(off, FLAGGEMS_B200_PRESORT="1")),  # half precision: GEMM1 reads a sorted copy
                ("presortwide", dict(off, FLAGGEMS_B200_PRESORT="1", FLAGGEMS_B200_TC_WIDE="1")))
    for name, env in variants:
        if which not in ("both", name):
            continue
        saved = {k: os.environ.get(k) for k in env}
        os.environ.update(env)
        try:
            outs[name] = run()
        finally:
            for k, v in saved.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
    return outs


# ---------------------------------------------------------------- golden vectors
@pytest.mark.parametrize("name", golden_files("layer_half_"))
def test_golden_half(name):
    g = load_golden(name)
    dt = DT[g["dtype"]]
    x, w1, w2 = (g[n].to(dt).to(DEV) for n in ("x", "w1", "w2"))
    tw, ti = g["topk_weights"].to(dt).to(DEV), g["topk_ids"].to(DEV)
    for name_, out in _both_kernels(lambda: fg.ops_experts_impl(x, w1, w2, tw, ti)).items():
        _assert_parity(out, O.fused_moe_half_oracle(x, w1, w2, tw, ti), name_)
        ref = g["out"]
        torch.testing.assert_close(out.float().cpu(), ref, rtol=1e-1, atol=max(1e-2, ref.abs().max().item() * 1e-5))


@pytest.mark.parametrize("name", golden_files("layer_fp8_"))
def test_golden_fp8(name):
    g = load_golden(name)
    x, w1, w2, s1, s2 = (g[n].to(DEV) for n in ("x", "w1", "w2", "w1_scale", "w2_scale"))
    tw, ti = g["topk_weights"].to(x.dtype).to(DEV), g["topk_ids"].to(DEV)
    run = lambda: fg.ops_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2,
                                      block_shape=[128, 128])
    for name_, out in _both_kernels(run).items():
        _assert_parity(out, O.fused_moe_fp8_block_oracle(x, w1, w2, s1, s2, tw, ti), name_)
        ref = g["out"]
        torch.testing.assert_close(out.float().cpu(), ref, rtol=2e-1, atol=max(5e-2, ref.abs().max().item() * 5e-2))


@pytest.mark.parametrize("name", golden_files("layer_w8a16_"))
def test_golden_w8a16(name):
    g = load_golden(name)
    x, w1, w2, s1, s2 = (g[n].to(DEV) for n in ("x", "w1", "w2", "w1_scale", "w2_scale"))
    tw, ti = g["topk_weights"].to(x.dtype).to(DEV), g["topk_ids"].to(DEV)
    run = lambda: fg.ops_experts_impl(x, w1, w2, tw, ti, use_int8_w8a16=True, per_channel_quant=True, w1_scale=s1,
                                      w2_scale=s2)
    for name_, out in _both_kernels(run).items():
        _assert_parity(out, O.fused_moe_w8a16_oracle(x, w1, w2, s1, s2, tw, ti), name_)
        ref = g["out"]
        torch.testing.assert_close(out.float().cpu(), ref, rtol=2e-1, atol=max(5e-2, ref.abs().max().item() * 2e-2))


# ---------------------------------------------------------------- reference test shapes
HALF_SHAPES = [(1, 8, 128, 256, 2), (4, 8, 128, 256, 2), (8, 4, 64, 128, 2), (16, 8, 256, 512, 2),
               (32, 8, 128, 256, 4), (64, 8, 256, 512, 2), (128, 16, 128, 256, 4), (4, 16, 512, 1024, 2),
               (10, 256, 2048, 128, 8), (256, 256, 2048, 128, 8)]


@pytest.mark.parametrize("cfg", HALF_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_half_shapes(cfg, dtype):
    M, E, H, I, k = cfg
    x = T.make_activations(M, H, DEV, dtype=dtype)
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, dtype=dtype, std=H**-0.5)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2, dtype=dtype, std=I**-0.5)
    tw, ti = _route(M, E, k, dtype)
    ref = O.fused_moe_half_oracle(x, w1, w2, tw, ti)
    for name, out in _both_kernels(lambda: fg.fused_experts_impl(x, w1, w2, tw, ti)).items():
        _assert_parity(out, ref, name)


QUANT_SHAPES = [(1, 8, 128, 256, 2), (4, 8, 128, 256, 2), (16, 8, 256, 512, 2), (32, 8, 128, 256, 4),
                (64, 8, 256, 512, 2), (128, 16, 128, 256, 4), (300, 16, 512, 384, 4)]


@pytest.mark.parametrize("cfg", QUANT_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fp8_block_shapes(cfg, dtype):
    M, E, H, I, k = cfg
    x = T.make_activations(M, H, DEV, dtype=dtype)
    w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    tw, ti = _route(M, E, k, dtype)
    ref = O.fused_moe_fp8_block_oracle(x, w1, w2, s1, s2, tw, ti)
    run = lambda: fg.fused_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2,
                                        block_shape=[128, 128])
    for name, out in _both_kernels(run).items():
        _assert_parity(out, ref, name)


@pytest.mark.parametrize("cfg", QUANT_SHAPES + [(64, 128, 2048, 768, 8), (700, 4, 320, 640, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_w8a16_shapes(cfg, dtype):
    M, E, H, I, k = cfg
    x = T.make_activations(M, H, DEV, dtype=dtype)
    w1, s1 = T.make_int8_channel_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2, s2 = T.make_int8_channel_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    w1[0, 0, :8] = torch.tensor([-128, 127, 0, -1, 1, -127, 64, -64], dtype=torch.int8, device=DEV)  # range ends
    tw, ti = _route(M, E, k, dtype)
    ref = O.fused_moe_w8a16_oracle(x, w1, w2, s1, s2, tw, ti)
    run = lambda: fg.fused_experts_impl(x, w1, w2, tw, ti, use_int8_w8a16=True, per_channel_quant=True,
                                        w1_scale=s1, w2_scale=s2)
    for name, out in _both_kernels(run).items():
        _assert_parity(out, ref, name)


# ---------------------------------------------------------------- benchmark configurations
def test_config1_small_bf16_layer():
    M, E, H, I, k = 64, 8, 1024, 2048, 2
    x = T.make_activations(M, H, DEV)
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2)
    tw, ti = _route(M, E, k, torch.bfloat16)
    s, e, n = fg.moe_align_block_size(ti, 16, E)
    os_, oe, on = O.moe_align_block_size_oracle(ti, 16, E)
    assert torch.equal(s.cpu(), torch.from_numpy(os_)) and torch.equal(e.cpu(), torch.from_numpy(oe))
    out = fg.fused_experts_impl(x, w1, w2, tw, ti)
    _assert_parity(out, O.fused_moe_half_oracle(x, w1, w2, tw, ti))


def test_config3_deepseek_shape_reduced_expert_count():
    # full H and I, 32 experts so the CPU oracle finishes in seconds
    M, E, H, I, k = 256, 32, 7168, 2048, 8
    x = T.make_activations(M, H, DEV)
    w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1)
    w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2)
    logits, bias = T.make_router_inputs(M, E, DEV)
    tw, ti = fg.grouped_topk(logits, 8, 4, k, True, 2.5, bias, 1)
    out = fg.fused_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2,
                                block_shape=[128, 128])
    _assert_parity(out, O.fused_moe_fp8_block_oracle(x, w1, w2, s1, s2, tw, ti))


def _sample_tokens(ti, E, n=64, seed=0):
    """At most ``n`` distinct tokens that include the first and the last expert-sorted row of the
    fullest and of the emptiest expert in use (rows inside an expert are ordered by flat route
    index), filled up with a seeded random choice."""
    M, k = ti.shape
    flat = ti.reshape(-1).long().cpu()
    counts = torch.bincount(flat, minlength=E)
    used = torch.nonzero(counts).flatten()
    fullest = int(used[counts[used].argmax()])
    emptiest = int(used[counts[used].argmin()])
    picked = []
    for e in (fullest, emptiest):
        routes = torch.nonzero(flat == e).flatten()
        picked += [int(routes[0]) // k, int(routes[-1]) // k]
    extra = torch.randperm(M, generator=torch.Generator().manual_seed(seed))[:n].tolist()
    rows = list(dict.fromkeys(picked + extra))[: min(M, n)]
    return torch.tensor(sorted(rows), device=ti.device)


def _sampled_oracle_fp8(x, w1, s1, w2, s2, tw, ti, rows):
    """Oracle on a sample of tokens: only the experts those tokens use are copied to the host."""
    xs, tws, tis = x[rows].cpu(), tw[rows].cpu(), ti[rows].cpu()
    used = torch.unique(tis).tolist()
    remap = {e: i for i, e in enumerate(used)}
    idx = torch.tensor(used, device=x.device)
    lw1, ls1, lw2, ls2 = w1[idx].cpu(), s1[idx].cpu(), w2[idx].cpu(), s2[idx].cpu()
    lti = torch.tensor([[remap[int(e)] for e in r] for r in tis], dtype=torch.int32)
    return O.fused_moe_fp8_block_oracle(xs, lw1, lw2, ls1, ls2, tws, lti)


@pytest.mark.parametrize("M", [1, 32, 128, 1024, 8192])
@pytest.mark.parametrize("pair", ["0", "1"])
def test_config3_full_size_sampled_parity_and_properties(M, pair, monkeypatch):
    if os.environ.get("MOE_TEST_KERNELS", "both") not in ("both", "pair" if pair == "1" else "tensor"):
        pytest.skip("kernel variant not selected")
    monkeypatch.setenv("FLAGGEMS_B200_TC_PAIR", pair)
    E, H, I, k = 256, 7168, 2048, 8
    x = T.make_activations(M, H, DEV)
    w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1)
    w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2)
    logits, bias = T.make_router_inputs(M, E, DEV)
    tw, ti = fg.grouped_topk(logits, 8, 4, k, True, 2.5, bias, 1)
    kw = dict(use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2, block_shape=[128, 128])
    out = fg.fused_experts_impl(x, w1, w2, tw, ti, **kw)
    rows = _sample_tokens(ti, E, 64 if pair == "0" else 16)
    _assert_parity(out[rows], _sampled_oracle_fp8(x, w1, s1, w2, s2, tw, ti, rows), f"M={M}")
    # run-to-run determinism (bitwise)
    assert torch.equal(out, fg.fused_experts_impl(x, w1, w2, tw, ti, **kw))
    # token permutation commutes with the layer (bitwise: rows are independent)
    perm = torch.randperm(M, device=DEV)
    assert torch.equal(fg.fused_experts_impl(x[perm].contiguous(), w1, w2, tw[perm].contiguous(),
                                             ti[perm].contiguous(), **kw), out[perm])
    # linear in the route weights
    out2 = fg.fused_experts_impl(x, w1, w2, tw * 2.0, ti, **kw)
    assert O.rel_l2(out2.float(), out.float() * 2.0) < 5e-3


@pytest.fixture(scope="module")
def mixtral_weights():
    E, H, I = 8, 4096, 14336
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, chunk=1)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2, chunk=1)
    yield w1, w2
    del w1, w2
    torch.cuda.empty_cache()


@pytest.mark.parametrize("M", [1, 16, 64, 256, 1024, 4096, 16384])
def test_config2_mixtral_shape_sampled(M, mixtral_weights):
    """Every token count of the Mixtral-shape sweep with the kernel the layer picks for it
    (small-batch schedule, 128-row tiles, 256-row tiles with pre-sorted rows)."""
    E, H, I, k = 8, 4096, 14336, 2
    w1, w2 = mixtral_weights
    x = T.make_activations(M, H, DEV)
    tw, ti = _route(M, E, k, torch.bfloat16)
    out = fg.fused_experts_impl(x, w1, w2, tw, ti)
    rows = _sample_tokens(ti, E, 64)
    ref = O.fused_moe_half_oracle(x[rows], w1, w2, tw[rows], ti[rows])
    _assert_parity(out[rows], ref, f"M={M}")
    assert torch.equal(out, fg.fused_experts_impl(x, w1, w2, tw, ti))  # bitwise run-to-run


@pytest.mark.parametrize("M", [1, 64, 512, 4096])
def test_config4_qwen3_shape(M):
    E, H, I, k = 128, 2048, 768, 8
    x = T.make_activations(M, H, DEV)
    w1, s1 = T.make_int8_channel_weights(E, 2 * I, H, DEV, seed=1)
    w2, s2 = T.make_int8_channel_weights(E, H, I, DEV, seed=2)
    tw, ti = _route(M, E, k, torch.bfloat16)
    kw = dict(use_int8_w8a16=True, per_channel_quant=True, w1_scale=s1, w2_scale=s2)
    out = fg.fused_experts_impl(x, w1, w2, tw, ti, **kw)
    rows = _sample_tokens(ti, E, 64)
    _assert_parity(out[rows], O.fused_moe_w8a16_oracle(x[rows], w1, w2, s1, s2, tw[rows], ti[rows]), f"M={M}")
    assert torch.equal(out, fg.fused_experts_impl(x, w1, w2, tw, ti, **kw))


# ---------------------------------------------------------------- row-scaled W8A8 modes and swigluoai
@pytest.mark.parametrize("name", golden_files("quant_int8_"))
def test_rowwise_int8_quant_matches_oracle_and_reference_vectors(name):
    g = load_golden(name)
    dt = DT[g["dtype"]]
    x = g["x"].to(dt).to(DEV)
    L = _lib.lib()
    q = torch.empty(x.shape, dtype=torch.int8, device=DEV)
    sc = torch.empty(x.shape[0], dtype=torch.float32, device=DEV)
    _lib.check(L.moe_rowwise_quant(x.data_ptr(), _lib.dtype_code(dt), x.shape[0], x.shape[1], 0, None, None, 0,
                                   q.data_ptr(), sc.data_ptr(), _lib.stream_of(x)))
    oq, os_ = O.int8_per_token_quant_oracle(g["x"].to(dt))
    assert torch.equal(q.cpu(), oq) and torch.equal(sc.cpu().reshape(-1, 1), os_)
    same = (os_ == g["s"]).expand_as(oq)  # rows where the kernel's amax * (1/127) equals the literal's amax / 127
    assert torch.equal(q.cpu()[same], g["q"][same])


def _rowwise(x, kind, static=None, row_ids=None, valid_below=0):
    L = _lib.lib()
    q = torch.empty(x.shape, dtype=torch.uint8, device=DEV)
    sc = torch.empty(x.shape[0] if kind in (0, 1) else 1, dtype=torch.float32, device=DEV)
    _lib.check(L.moe_rowwise_quant(x.data_ptr(), _lib.dtype_code(x.dtype), x.shape[0], x.shape[1], kind,
                                   _lib.ptr(static), _lib.ptr(row_ids), valid_below, q.data_ptr(), sc.data_ptr(),
                                   _lib.stream_of(x)))
    return q.cpu(), sc.cpu()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rowwise_fp8_quant_kinds(dtype):
    x = (torch.randn(19, 320, device=DEV) * 4).to(dtype)
    x[3] = 0
    q, sc = _rowwise(x, 1)
    oq, os_ = O.fp8_per_token_quant_oracle(x)
    assert torch.equal(q, oq.view(torch.uint8)) and torch.equal(sc.reshape(-1, 1), os_)
    static = torch.tensor([0.037], device=DEV)
    q, sc = _rowwise(x, 2, static)
    oq, _ = O.fp8_per_tensor_quant_oracle(x, static)
    assert torch.equal(q, oq.view(torch.uint8)) and float(sc) == float(static)
    q, sc = _rowwise(x, 3)
    oq, os_ = O.fp8_per_tensor_quant_oracle(x)
    assert torch.equal(sc, os_) and torch.equal(q, oq.view(torch.uint8))
    # dynamic per-tensor scale over a subset of rows (padding rows of the sorted intermediate are skipped)
    ids = torch.arange(19, dtype=torch.int32, device=DEV)
    ids[5:] += 100
    x2 = x.clone()
    x2[10] = 1000.0  # a skipped row must not move the scale
    q2, sc2 = _rowwise(x2, 3, None, ids, 50)
    oq2, os2 = O.fp8_per_tensor_quant_oracle(x2[:5])
    assert torch.equal(sc2, os2) and torch.equal(q2[:5], oq2.view(torch.uint8))


@pytest.mark.parametrize("name", golden_files("layer_w8a8_int8_"))
def test_golden_int8_w8a8_swigluoai(name):
    g = load_golden(name)
    dt = DT[g["dtype"]]
    x, w1, w2 = g["x"].to(dt).to(DEV), g["w1"].to(DEV), g["w2"].to(DEV)
    s1, s2 = g["w1_scale"].to(DEV), g["w2_scale"].to(DEV)
    tw, ti = g["topk_weights"].to(DEV), g["topk_ids"].to(DEV)
    kw = dict(activation="swigluoai_uninterleave", use_int8_w8a8=True, per_channel_quant=True, w1_scale=s1, w2_scale=s2,
              gemm1_alpha=1.702, gemm1_beta=1.0, gemm1_clamp_limit=7.0)
    out = fg.fused_experts_impl(x, w1, w2, tw, ti, **kw)
    ref = O.fused_moe_row_scaled_oracle(x, w1, w2, s1, s2, tw, ti, fmt="int8", per_token=True,
                                        activation="swigluoai_uninterleave")
    _assert_parity(out, ref, name)
    # the reference test's own tolerance against its literal loop (tests/test_fused_moe.py:161-166)
    torch.testing.assert_close(out.float().cpu(), g["out"], atol=0.0005 if dt == torch.float16 else 0.004,
                               rtol=0.003 if dt == torch.float16 else 0.016)
    buf = x.clone()
    assert fg.inplace_fused_experts(buf, w1, w2, tw, ti, **kw) is None and torch.equal(buf, out)


@pytest.mark.parametrize("variant", ["tensor_dynamic", "tensor_static", "token_channel"])
def test_fp8_per_tensor_and_per_token_layers(variant):
    M, E, H, I, k = 33, 8, 256, 384, 2
    x = T.make_activations(M, H, DEV)
    w1f = torch.randn(E, 2 * I, H, device=DEV) * H**-0.5
    w2f = torch.randn(E, H, I, device=DEV) * I**-0.5
    tw, ti = _route(M, E, k, torch.bfloat16)
    if variant == "token_channel":
        s1 = w1f.abs().amax(-1) / 448.0
        s2 = w2f.abs().amax(-1) / 448.0
        w1, w2 = (w1f / s1[..., None]).to(torch.float8_e4m3fn), (w2f / s2[..., None]).to(torch.float8_e4m3fn)
        out = fg.fused_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, per_channel_quant=True, w1_scale=s1, w2_scale=s2)
        ref = O.fused_moe_row_scaled_oracle(x, w1, w2, s1, s2, tw, ti, fmt="fp8", per_token=True)
    else:
        s1 = w1f.abs().amax(dim=(1, 2)) / 448.0
        s2 = w2f.abs().amax(dim=(1, 2)) / 448.0
        w1 = (w1f / s1[:, None, None]).to(torch.float8_e4m3fn)
        w2 = (w2f / s2[:, None, None]).to(torch.float8_e4m3fn)
        a1 = a2 = None
        if variant == "tensor_static":
            a1, a2 = torch.tensor([0.02], device=DEV), torch.tensor([0.004], device=DEV)
        out = fg.fused_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2, a1_scale=a1,
                                    a2_scale=a2)
        ref = O.fused_moe_row_scaled_oracle(x, w1, w2, s1[:, None].expand(E, 2 * I), s2[:, None].expand(E, H), tw, ti,
                                            fmt="fp8", per_token=False, a1_scale=a1, a2_scale=a2)
    _assert_parity(out, ref, variant)


@pytest.mark.parametrize("fmt", ["half", "w8a16", "fp8"])
def test_swigluoai_activation_on_the_other_weight_formats(fmt):
    M, E, H, I, k = 21, 8, 256, 256, 2
    x = T.make_activations(M, H, DEV)
    tw, ti = _route(M, E, k, torch.bfloat16)
    act = lambda z: O.swigluoai_oracle(z, 1.5, 0.5, 3.0)
    kw = dict(activation="swigluoai_uninterleave", gemm1_alpha=1.5, gemm1_beta=0.5, gemm1_clamp_limit=3.0)
    if fmt == "half":
        w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
        w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
        out = fg.fused_experts_impl(x, w1, w2, tw, ti, **kw)
        ref = O.fused_moe_half_oracle(x, w1, w2, tw, ti, act_fn=act)
    elif fmt == "w8a16":
        w1, s1 = T.make_int8_channel_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
        w2, s2 = T.make_int8_channel_weights(E, H, I, DEV, seed=2, std=I**-0.5)
        out = fg.fused_experts_impl(x, w1, w2, tw, ti, use_int8_w8a16=True, per_channel_quant=True, w1_scale=s1,
                                    w2_scale=s2, **kw)
        wd1 = (w1.float() * s1[..., None]).to(torch.bfloat16)
        wd2 = (w2.float() * s2[..., None]).to(torch.bfloat16)
        ref = O.fused_moe_half_oracle(x, wd1.float(), wd2.float(), tw, ti, act_fn=act)
    else:
        w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
        w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2, std=I**-0.5)
        out = fg.fused_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2,
                                    block_shape=[128, 128], **kw)
        # same layer with SiLU swapped for the other activation: compare with the half oracle on the dequantised
        # weights and activations is too loose; check against the structure instead: the SiLU result must differ
        silu = fg.fused_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2,
                                     block_shape=[128, 128])
        assert O.rel_l2(out.float(), silu.float()) > 1e-2
        wd1 = (w1.float().view(E, 2 * I // 128, 128, H // 128, 128) * s1[:, :, None, :, None]).view(E, 2 * I, H)
        wd2 = (w2.float().view(E, H // 128, 128, I // 128, 128) * s2[:, :, None, :, None]).view(E, H, I)
        ref = O.fused_moe_half_oracle(x, wd1, wd2, tw, ti, act_fn=act)
        assert O.rel_l2(out.float(), ref) < 6e-2 and O.cosine(out.float(), ref) > 0.998  # two e4m3 quantisations apart
        return
    _assert_parity(out, ref, fmt)


# ---------------------------------------------------------------- small-batch schedule
@pytest.mark.parametrize("M", [1, 2, 7, 16, 32, 64])
@pytest.mark.parametrize("fmt", ["half", "fp8", "w8a16"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_small_batch_schedule_matches_the_oracle(M, fmt, dtype, monkeypatch):
    """The weight-streaming split-K kernels, forced on: H = 2304 needs two K slices in GEMM 1
    (three with the slice hint), so the ordered partial-sum reduction runs; k = 4 routes per
    token exercise the in-kernel top-k combine."""
    monkeypatch.setenv("FLAGGEMS_B200_SMALL_M", "1")
    E, H, I, k = 16, 2304, 384, 4
    x = T.make_activations(M, H, DEV, dtype=dtype)
    tw, ti = _route(M, E, k, dtype)
    if fmt == "half":
        w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, dtype=dtype, std=H**-0.5)
        w2 = T.make_half_weights(E, H, I, DEV, seed=2, dtype=dtype, std=I**-0.5)
        kw = {}
        ref = O.fused_moe_half_oracle(x, w1, w2, tw, ti)
    elif fmt == "fp8":
        w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
        w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2, std=I**-0.5)
        kw = dict(use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2, block_shape=[128, 128])
        ref = O.fused_moe_fp8_block_oracle(x, w1, w2, s1, s2, tw, ti)
    else:
        w1, s1 = T.make_int8_channel_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
        w2, s2 = T.make_int8_channel_weights(E, H, I, DEV, seed=2, std=I**-0.5)
        kw = dict(use_int8_w8a16=True, per_channel_quant=True, w1_scale=s1, w2_scale=s2)
        ref = O.fused_moe_w8a16_oracle(x, w1, w2, s1, s2, tw, ti)
    keep = {}
    out = torch.empty_like(x)
    mode = {"half": _lib.MODE_HALF, "fp8": _lib.MODE_FP8_BLOCK, "w8a16": _lib.MODE_W8A16}[fmt]
    fused_moe.run_chunk(x, w1, w2, tw, ti, out, mode=mode, w1_scale=kw.get("w1_scale"), w2_scale=kw.get("w2_scale"),
                        global_num_experts=E, expert_map=None, apply_router_weight_on_input=False, keep=keep)
    assert keep["kernel"] == "small"
    _assert_parity(out, ref, f"{fmt} M={M}")
    again = fg.fused_experts_impl(x, w1, w2, tw, ti, **kw)
    assert torch.equal(out, again)                      # bitwise run to run, and the counters were left clean
    perm = torch.randperm(M, device=DEV)
    assert torch.equal(fg.fused_experts_impl(x[perm].contiguous(), w1, w2, tw[perm].contiguous(),
                                             ti[perm].contiguous(), **kw), out[perm])
    buf = x.clone()
    fg.fused_experts_impl(buf, w1, w2, tw, ti, inplace=True, **kw)
    assert torch.equal(buf, out)


def test_small_batch_schedule_expert_map_and_weight_on_input(monkeypatch):
    monkeypatch.setenv("FLAGGEMS_B200_SMALL_M", "1")
    M, E, H, I, k = 12, 16, 256, 256, 4
    x = T.make_activations(M, H, DEV)
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    tw, ti = _route(M, E, k, torch.bfloat16)
    full = fg.fused_experts_impl(x, w1, w2, tw, ti)
    total = torch.zeros_like(full, dtype=torch.float32)
    for r in range(2):
        lo, hi = r * 8, (r + 1) * 8
        emap = torch.full((E,), -1, dtype=torch.int32, device=DEV)
        emap[lo:hi] = torch.arange(8, dtype=torch.int32, device=DEV)
        part = fg.fused_experts_impl(x, w1[lo:hi].contiguous(), w2[lo:hi].contiguous(), tw, ti,
                                     global_num_experts=E, expert_map=emap)
        total += part.float()
    assert O.rel_l2(total, full.float()) < 5e-3
    # a token whose routes all belong to the other rank gets a zero row
    ti2 = ti.clone()
    ti2[0] = torch.tensor([8, 9, 10, 11], dtype=ti.dtype, device=DEV)
    emap = torch.full((E,), -1, dtype=torch.int32, device=DEV)
    emap[:8] = torch.arange(8, dtype=torch.int32, device=DEV)
    part = fg.fused_experts_impl(x, w1[:8].contiguous(), w2[:8].contiguous(), tw, ti2, global_num_experts=E,
                                 expert_map=emap)
    assert torch.all(part[0] == 0)
    xw = T.make_activations(M, H, DEV, seed=9)
    tw1, ti1 = _route(M, E, 1, torch.bfloat16)
    out = fg.fused_experts_impl(xw, w1, w2, tw1, ti1, apply_router_weight_on_input=True)
    _assert_parity(out, O.fused_moe_half_oracle(xw, w1, w2, tw1, ti1, apply_router_weight_on_input=True))
    assert fg.read_status() == 0


# ---------------------------------------------------------------- API behaviour
def _small_half(dtype=torch.bfloat16, M=16, E=8, H=256, I=512, k=2):
    x = T.make_activations(M, H, DEV, dtype=dtype)
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, dtype=dtype, std=H**-0.5)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2, dtype=dtype, std=I**-0.5)
    tw, ti = _route(M, E, k, dtype)
    return x, w1, w2, tw, ti


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_inplace_outplace_bitwise(dtype):
    x, w1, w2, tw, ti = _small_half(dtype)
    ref = fg.fused_experts_impl(x.clone(), w1, w2, tw, ti, inplace=False)
    buf = x.clone()
    res = fg.fused_experts_impl(buf, w1, w2, tw, ti, inplace=True)
    assert res.data_ptr() == buf.data_ptr()
    assert torch.equal(res, ref)
    buf2 = x.clone()
    assert fg.inplace_fused_experts(buf2, w1, w2, tw, ti) is None
    assert torch.equal(buf2, ref)
    keep = x.clone()
    out = fg.outplace_fused_experts(x, w1, w2, tw, ti)
    assert torch.equal(x, keep) and torch.equal(out, ref) and out.data_ptr() != x.data_ptr()


def test_router_weight_on_input():
    x, w1, w2, tw, ti = _small_half()
    out = fg.fused_experts_impl(x, w1, w2, tw, ti, apply_router_weight_on_input=True)
    ref = O.fused_moe_half_oracle(x, w1, w2, tw, ti, apply_router_weight_on_input=True)
    _assert_parity(out, ref)


def test_int64_ids_and_fp32_activations():
    x, w1, w2, tw, ti = _small_half()
    a = fg.fused_experts_impl(x, w1, w2, tw, ti)
    b = fg.fused_experts_impl(x, w1, w2, tw, ti.long())
    assert torch.equal(a, b)
    xf, w1f, w2f = x.float(), w1.float(), w2.float()
    c = fg.fused_experts_impl(xf, w1f, w2f, tw.float(), ti)
    _assert_parity(c, O.fused_moe_half_oracle(xf, w1f, w2f, tw.float(), ti))


def test_expert_parallel_halves_sum_to_the_full_layer():
    M, E, H, I, k = 64, 16, 256, 256, 4
    x = T.make_activations(M, H, DEV)
    w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    tw, ti = _route(M, E, k, torch.bfloat16)
    kw = dict(use_fp8_w8a8=True, block_shape=[128, 128])
    full = fg.fused_experts_impl(x, w1, w2, tw, ti, w1_scale=s1, w2_scale=s2, **kw)
    total = torch.zeros_like(full, dtype=torch.float32)
    for r in range(2):
        lo, hi = r * 8, (r + 1) * 8
        emap = torch.full((E,), -1, dtype=torch.int32, device=DEV)
        emap[lo:hi] = torch.arange(8, dtype=torch.int32, device=DEV)
        part = fg.fused_experts_impl(x, w1[lo:hi].contiguous(), w2[lo:hi].contiguous(), tw, ti,
                                     global_num_experts=E, expert_map=emap, w1_scale=s1[lo:hi].contiguous(),
                                     w2_scale=s2[lo:hi].contiguous(), **kw)
        total += part.float()
    assert O.rel_l2(total, full.float()) < 5e-3
    assert fg.read_status() == 0


def test_more_tokens_than_one_chunk():
    M, E, H, I, k = 32768 + 100, 8, 128, 128, 2
    x = T.make_activations(M, H, DEV)
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    tw, ti = _route(M, E, k, torch.bfloat16)
    out = fg.fused_experts_impl(x, w1, w2, tw, ti)
    rows = torch.cat([torch.arange(0, 64), torch.arange(32768 - 8, 32768 + 100)]).to(DEV)
    _assert_parity(out[rows], O.fused_moe_half_oracle(x[rows], w1, w2, tw[rows], ti[rows]))


def test_intermediates_follow_the_documented_layout():
    M, E, H, I, k = 40, 8, 256, 256, 2
    x = T.make_activations(M, H, DEV)
    w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    tw, ti = _route(M, E, k, torch.bfloat16)
    keep = {}
    out = torch.empty_like(x)
    fused_moe.run_chunk(x, w1, w2, tw, ti, out, mode=_lib.MODE_FP8_BLOCK, w1_scale=s1, w2_scale=s2,
                        global_num_experts=E, expert_map=None, apply_router_weight_on_input=False, keep=keep)
    torch.cuda.synchronize()
    assert keep["used_tensor_cores"] and keep["block_m"] in (128, 256)
    bm = keep["block_m"]
    xq, xs = O.per_token_group_quant_fp8_oracle(x, 128)
    assert torch.equal(keep["a_rows"].cpu().view(torch.uint8), xq.view(torch.uint8))
    assert torch.equal(keep["a_scales_t"].cpu().t(), xs)
    # the intermediate is in sorted order: row p belongs to route sorted_ids[p]
    n = int(keep["num_post_pad"].item())
    sid = keep["sorted_ids"][:n].cpu()
    valid = sid < M * k
    os_, oe, on = O.moe_align_block_size_oracle(ti, bm, E, pad_sorted_ids=True)
    assert n == int(on[0]) and torch.equal(sid, torch.from_numpy(os_[:n]))
    act = keep["act"][:n].cpu().float() * keep["act_scales_t"][:, :n].cpu().t().repeat_interleave(128, dim=1)
    assert torch.isfinite(act[valid]).all()


@pytest.mark.parametrize("mode", ["fp8", "bf16"])
def test_gemm2_in_two_column_windows_equals_the_one_piece_gemm2(mode):
    """GEMM 2 over the two halves of the hidden columns (the second on fewer SMs) writes exactly the
    columns the one-piece GEMM 2 writes, and the sum into a column window of a wider tensor equals
    the sum into a tensor of its own."""
    M, E, H, I, k = 1500, 8, 1024, 256, 2
    x = T.make_activations(M, H, DEV)
    tw, ti = _route(M, E, k, torch.bfloat16)
    if mode == "fp8":
        w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
        w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2, std=I**-0.5)
        a_rows, a_scales = fused_moe.quantize_rows(x)
        m = _lib.MODE_FP8_BLOCK
    else:
        w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
        w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
        s1 = s2 = None
        a_rows, a_scales = x, None
        m = _lib.MODE_HALF
    kw = dict(mode=m, act_dtype=x.dtype, w1_scale=s1, w2_scale=s2, global_num_experts=E, expert_map=None,
              apply_router_weight_on_input=False, use_tensor_cores=fused_moe.KERNEL_TC)
    y, row_index = fused_moe.route_pipeline(a_rows, a_scales, w1, w2, tw, ti, **kw)
    assert row_index is not None, "this size is meant to take the sorted-output GEMM 2"
    windows = []
    y2, row_index2 = fused_moe.route_pipeline(a_rows, a_scales, w1, w2, tw, ti, **kw,
                                              column_halves=(lambda h, c0, yw, ri: windows.append((c0, yw)), 24))
    torch.cuda.synchronize()
    assert y2 is None and len(windows) == 2 and torch.equal(row_index2, row_index)
    n = int(row_index.max().item()) + 1
    valid = torch.zeros(y.shape[0], dtype=torch.bool, device=DEV)
    valid[row_index.flatten().long()] = True
    for c0, yw in windows:
        assert torch.equal(yw[valid], y[valid][:, c0:c0 + yw.shape[1]])
    out = torch.empty((M, H), dtype=x.dtype, device=DEV)
    fused_moe.combine_routes(y, out, ti, E, row_index=row_index)
    out_w = torch.zeros((M, H), dtype=x.dtype, device=DEV)
    for c0, yw in windows:
        fused_moe.combine_routes(yw, out_w[:, c0:c0 + yw.shape[1]], ti, E, row_index=row_index)
    assert torch.equal(out_w, out) and n <= y.shape[0] and fg.read_status(torch.device(DEV)) == 0


# shapes and dtypes of the reference's tests/test_silu_and_mul.py (accuracy_utils.POINTWISE_SHAPES, FLOAT_DTYPES)
@pytest.mark.parametrize("shape", [(), (1,), (1024, 1024), (20, 320, 15), (16, 128, 64, 60), (16, 7, 57, 32, 29)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
def test_silu_and_mul_and_its_gradients(shape, dtype):
    g = torch.Generator(device="cpu").manual_seed(len(shape) + 7)
    a = torch.randn(shape, generator=g).to(dtype).to(DEV).requires_grad_(True)
    b = torch.randn(shape, generator=g).to(dtype).to(DEV).requires_grad_(True)
    # one rounding to the dtype: within half an ulp of the float64 value (plus fp32 evaluation error)
    tol = {torch.float32: dict(rtol=2e-6, atol=1e-6), torch.float16: dict(rtol=1e-3, atol=1e-4),
           torch.bfloat16: dict(rtol=8e-3, atol=1e-4)}[dtype]
    out = fg.silu_and_mul(a, b)
    assert out.shape == tuple(shape) and out.dtype == dtype
    ref = O.silu_and_mul_oracle(a.detach(), b.detach())
    torch.testing.assert_close(out.detach().double().cpu(), ref, **tol)
    buf = torch.empty_like(a.detach())
    assert fg.silu_and_mul_out(a.detach(), b.detach(), buf) is buf and torch.equal(buf, out.detach())
    grad = torch.randn(shape, generator=g).to(dtype).to(DEV)
    da, db = torch.autograd.grad(out, (a, b), grad)
    ad, bd = a.detach().double().cpu().requires_grad_(True), b.detach().double().cpu().requires_grad_(True)
    rda, rdb = torch.autograd.grad(torch.mul(torch.nn.functional.silu(ad), bd), (ad, bd), grad.double().cpu())
    torch.testing.assert_close(da.double().cpu(), rda, **tol)
    torch.testing.assert_close(db.double().cpu(), rdb, **tol)


def test_silu_and_mul_broadcasts_and_promotes():
    a = torch.randn(4, 1, 8, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(5, 8, device=DEV, dtype=torch.float32)
    out = fg.silu_and_mul(a, b)
    assert out.shape == (4, 5, 8) and out.dtype == torch.float32
    torch.testing.assert_close(out.double().cpu(), O.silu_and_mul_oracle(a, b).expand(4, 5, 8), rtol=2e-6, atol=1e-6)


def test_quant_and_sum_wrappers():
    x = torch.randn(33, 512, device=DEV, dtype=torch.bfloat16) * 3
    x[0, :128] = 0
    q, s = fg.per_token_group_quant_fp8(x, 128)
    oq, os_ = O.per_token_group_quant_fp8_oracle(x, 128)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8)) and torch.equal(s.cpu(), os_)
    q2, s2 = fg.per_token_group_quant_fp8(x, 128, column_major_scales=True)
    assert s2.shape == s.shape and s2.stride(0) == 1 and torch.equal(s2.contiguous(), s) and torch.equal(
        q2.view(torch.uint8), q.view(torch.uint8))
    # power-of-two scales: the same expression as the oracle; log2 of a value a few ulps above a
    # power of two may round either way, so a scale may differ by exactly one binade, rarely
    xb = torch.randn(257, 1024, device=DEV, dtype=torch.bfloat16) * 5
    q3, s3 = fg.per_token_group_quant_fp8(xb, 128, scale_ue8m0=True)
    oq3, os3 = O.per_token_group_quant_fp8_oracle(xb, 128, scale_ue8m0=True)
    s3c = s3.cpu()
    assert torch.equal(torch.exp2(torch.round(torch.log2(s3c))), s3c)
    same = s3c == os3
    assert same.float().mean() > 0.999 and torch.all((s3c[~same] == 2 * os3[~same]) | (2 * s3c[~same] == os3[~same]))
    rows_same = same.repeat_interleave(128, dim=1)
    assert torch.equal(q3.cpu().view(torch.uint8)[rows_same], oq3.view(torch.uint8)[rows_same])
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        for (m, k, h) in [(1, 2, 128), (33, 6, 511), (222, 2, 1024)]:
            inp = torch.randn(m, k, h, device=DEV, dtype=dt)
            o = torch.empty(m, h, device=DEV, dtype=dt)
            fg.moe_sum(inp, o)
            torch.testing.assert_close(o.float().cpu(), O.moe_sum_oracle(inp).to(dt).float(),
                                       rtol=1.6e-2 if dt != torch.float32 else 1.3e-6, atol=1e-4 * k)


@pytest.mark.parametrize("name", golden_files("quant_fp8_group_"))
def test_quant_other_group_sizes_and_clamps(name):
    """Any group size and eps, bit for bit against the oracle (which the reference-made vectors pin)."""
    g = load_golden(name)
    group, eps = int(g["params"][0]), float(g["params"][1])
    x = g["x"].to(DEV)
    q, s = fg.per_token_group_quant_fp8(x, group, eps=eps)
    oq, os_ = O.per_token_group_quant_fp8_oracle(g["x"], group, eps=eps)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8)) and torch.equal(s.cpu(), os_)
    q2, s2 = fg.per_token_group_quant_fp8(x, group, eps=eps, column_major_scales=True)
    assert s2.stride(0) == 1 and torch.equal(s2.contiguous(), s) and torch.equal(q2.view(torch.uint8), q.view(torch.uint8))
    for dt in (torch.float32, torch.float16):
        xx = (torch.randn(17, 4 * group, device=DEV) * 3).to(dt)
        qq, ss = fg.per_token_group_quant_fp8(xx, group, eps=eps)
        oq, os_ = O.per_token_group_quant_fp8_oracle(xx, group, eps=eps)
        assert torch.equal(qq.cpu().view(torch.uint8), oq.view(torch.uint8)) and torch.equal(ss.cpu(), os_)


def test_quant_e5m2_output():
    x = torch.randn(9, 512, device=DEV, dtype=torch.bfloat16) * 4
    q, s = fg.per_token_group_quant_fp8(x, 128, dtype=torch.float8_e5m2)
    assert q.dtype == torch.float8_e5m2
    xr = x.float().cpu().reshape(-1, 128)
    sc = xr.abs().amax(dim=1, keepdim=True).clamp(min=1e-10) * torch.tensor(1.0 / 57344.0)
    ref = (xr / sc).clamp(-57344.0, 57344.0).to(torch.float8_e5m2)
    assert torch.equal(s.cpu().reshape(-1, 1), sc)
    assert torch.equal(q.cpu().view(torch.uint8).reshape(-1, 128), ref.view(torch.uint8))


def test_moe_sum_accepts_strided_tensors():
    # the reference's general kernel is stride-aware (src/flaggems_vllm/ops/moe_sum.py:295-310)
    big = torch.randn(40, 6, 512, device=DEV, dtype=torch.bfloat16)
    inp = big[::2, 1:5, ::2]                      # non-contiguous in every dimension
    out_big = torch.zeros(20, 512, device=DEV, dtype=torch.bfloat16)
    out = out_big[:, ::2]
    fg.moe_sum(inp, out)
    torch.testing.assert_close(out.float().cpu(), O.moe_sum_oracle(inp.contiguous()).to(torch.bfloat16).float(),
                               rtol=1.6e-2, atol=1e-3)
    assert torch.all(out_big[:, 1::2] == 0)       # the gaps of the strided output stay untouched
    # rows apart, columns contiguous: written in place (a column window of a wider tensor)
    wide = torch.full((20, 1024), -3.0, device=DEV, dtype=torch.bfloat16)
    cont = torch.randn(20, 4, 256, device=DEV, dtype=torch.bfloat16)
    fg.moe_sum(cont, wide[:, 512:768])
    assert torch.equal(wide[:, 512:768].float().cpu(), O.moe_sum_oracle(cont).to(torch.bfloat16).float())
    assert torch.all(wide[:, :512] == -3.0) and torch.all(wide[:, 768:] == -3.0)


def test_gather_rows_matches_index_select():
    from flaggems_vllm_b200 import _lib
    M, k, E, H, bm = 77, 4, 16, 256, 128
    x = T.make_activations(M, H, DEV)
    ids = T.make_align_ids(M, k, E, DEV)
    sorted_ids, expert_ids, npp = fg.moe_align_block_size(ids, bm, E)
    rows_cap = sorted_ids.numel()
    out = torch.full((rows_cap, H), -7.0, device=DEV, dtype=x.dtype)
    _lib.check(_lib.lib().moe_gather_rows(x.data_ptr(), M, k, H * 2, sorted_ids.data_ptr(), npp.data_ptr(), rows_cap,
                                          out.data_ptr(), _lib.stream_of(x)))
    n = int(npp.item())
    sid = sorted_ids[:n].long()
    valid = sid < M * k
    assert torch.equal(out[:n][valid], x[sid[valid] // k])
    assert torch.all(out[:n][~valid] == -7.0) and torch.all(out[n:] == -7.0)  # padding and tail untouched


def test_layer_under_cuda_graph_replay_with_new_inputs():
    M, E, H, I, k = 32, 32, 512, 256, 4
    w1, s1 = T.make_fp8_block_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2, s2 = T.make_fp8_block_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    x = T.make_activations(M, H, DEV, seed=3)
    logits, bias = T.make_router_inputs(M, E, DEV, seed=4)

    def step():
        tw, ti = fg.grouped_topk(logits, 8, 4, k, True, 2.5, bias, 1)
        return tw, ti, fg.fused_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2,
                                             block_shape=[128, 128])

    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        tw, ti, out = step()
    for seed in (5, 6):
        x.copy_(T.make_activations(M, H, DEV, seed=seed))
        logits.copy_(T.make_router_inputs(M, E, DEV, seed=seed)[0])
        graph.replay()
        torch.cuda.synchronize()
        ow, oi = O.grouped_topk_oracle(logits, 8, 4, k, True, 2.5, bias, 1)
        assert torch.equal(ti.cpu(), oi)
        _assert_parity(out, O.fused_moe_fp8_block_oracle(x, w1, w2, s1, s2, ow, oi), f"replay {seed}")


@pytest.mark.parametrize("case", ["bf16_small_batch", "w8a16_small_batch", "bf16_sorted_output"])
def test_other_paths_under_cuda_graph_replay_with_new_inputs(case):
    """The small-batch schedule (its counters clean themselves, its scratch is reused) and the
    staged-output GEMM 2 replay correctly from a CUDA graph when the inputs change."""
    E, H, I, k = 8, 512, 256, 2
    M = {"bf16_small_batch": 2, "w8a16_small_batch": 1, "bf16_sorted_output": 700}[case]
    if case == "w8a16_small_batch":
        w1, s1 = T.make_int8_channel_weights(E, 2 * I, H, DEV, seed=1)
        w2, s2 = T.make_int8_channel_weights(E, H, I, DEV, seed=2)
        kw = dict(use_int8_w8a16=True, per_channel_quant=True, w1_scale=s1, w2_scale=s2)
        oracle = lambda x, tw, ti: O.fused_moe_w8a16_oracle(x, w1, w2, s1, s2, tw, ti)
    else:
        w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
        w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
        kw = {}
        oracle = lambda x, tw, ti: O.fused_moe_half_oracle(x, w1, w2, tw, ti)
    x = T.make_activations(M, H, DEV, seed=3)
    logits, _ = T.make_router_inputs(M, E, DEV, seed=4)
    zero_bias = torch.zeros(E, device=DEV)

    def step():
        tw, ti = fg.grouped_topk(torch.softmax(logits, -1), 1, 1, k, True, 1.0, zero_bias, 0)
        return tw, ti, fg.fused_experts_impl(x, w1, w2, tw, ti, **kw)

    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        tw, ti, out = step()
    for seed in (5, 6, 7):
        x.copy_(T.make_activations(M, H, DEV, seed=seed))
        logits.copy_(T.make_router_inputs(M, E, DEV, seed=seed)[0])
        graph.replay()
        torch.cuda.synchronize()
        _assert_parity(out, oracle(x, tw, ti), f"{case} replay {seed}")


def test_empty_batch_and_single_token():
    E, H, I, k = 8, 128, 256, 2
    w1 = T.make_half_weights(E, 2 * I, H, DEV, seed=1, std=H**-0.5)
    w2 = T.make_half_weights(E, H, I, DEV, seed=2, std=I**-0.5)
    x0 = torch.empty((0, H), device=DEV, dtype=torch.bfloat16)
    out0 = fg.fused_experts_impl(x0, w1, w2, torch.empty((0, k), device=DEV), torch.empty((0, k), device=DEV,
                                                                                           dtype=torch.int32))
    assert out0.shape == (0, H)
    x1 = T.make_activations(1, H, DEV)
    tw, ti = _route(1, E, k, torch.bfloat16)
    _assert_parity(fg.fused_experts_impl(x1, w1, w2, tw, ti), O.fused_moe_half_oracle(x1, w1, w2, tw, ti))

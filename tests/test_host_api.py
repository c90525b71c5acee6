"""CPU-only checks: the C-ABI library loads and exports every declared symbol,
the Python entry points keep the reference's signatures, argument validation
raises the reference's error types before any device work."""

import ctypes
import inspect
import os
import re

import pytest
import torch

import flaggems_vllm
import flaggems_vllm_b200 as fg
from flaggems_vllm_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    handle = ctypes.CDLL(path)
    header = open(os.path.join(ROOT, "include", "moe_sm100.h")).read()
    declared = set(re.findall(r"^(?:int|unsigned long long|const char\*)\s+(moe_[a-z0-9_]+)\s*\(", header, flags=re.M))
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SYMBOLS), "ctypes table and header disagree"
    assert handle.moe_abi_version() >= 1


def _sig(fn):
    return [(n, p.kind, p.default) for n, p in inspect.signature(fn).parameters.items()]


def test_signatures_match_reference():
    # names, order, kinds and defaults of src/flaggems_vllm/ops/grouped_topk.py:1674-1684
    assert _sig(fg.grouped_topk) == [
        ("scores", inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect._empty),
        ("n_group", inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect._empty),
        ("topk_group", inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect._empty),
        ("topk", inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect._empty),
        ("renormalize", inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect._empty),
        ("routed_scaling_factor", inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect._empty),
        ("bias", inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect._empty),
        ("scoring_func", inspect.Parameter.POSITIONAL_OR_KEYWORD, 0),
        ("is_padding", inspect.Parameter.POSITIONAL_OR_KEYWORD, None),
    ]
    # src/flaggems_vllm/ops/moe_align_block_size.py:896-902
    assert [(n, d) for n, _, d in _sig(fg.moe_align_block_size)] == [
        ("topk_ids", inspect._empty), ("block_size", inspect._empty), ("num_experts", inspect._empty),
        ("expert_map", None), ("pad_sorted_ids", False)]
    # src/flaggems_vllm/ops/fused_moe.py:2314-2344
    names = [n for n, _, _ in _sig(fg.fused_experts_impl)]
    assert names == [
        "hidden_states", "w1", "w2", "topk_weights", "topk_ids", "inplace", "activation",
        "apply_router_weight_on_input", "use_fp8_w8a8", "use_int8_w8a8", "use_int8_w8a16", "use_int4_w4a16",
        "ocp_mx_scheme", "per_channel_quant", "global_num_experts", "expert_map", "w1_scale", "w2_scale",
        "w1_zp", "w2_zp", "a1_scale", "a2_scale", "block_shape", "w1_bias", "w2_bias", "gemm1_alpha",
        "gemm1_beta", "gemm1_clamp_limit"]
    kinds = [k for _, k, _ in _sig(fg.fused_experts_impl)]
    assert kinds[:25] == [inspect.Parameter.POSITIONAL_OR_KEYWORD] * 25
    assert kinds[25:] == [inspect.Parameter.KEYWORD_ONLY] * 3
    assert inspect.signature(fg.fused_experts_impl).parameters["global_num_experts"].default == -1
    assert fg.ops_experts_impl is fg.fused_experts_impl
    assert flaggems_vllm.grouped_topk is fg.grouped_topk
    assert flaggems_vllm.ops_experts_impl is fg.fused_experts_impl
    assert "inplace" not in inspect.signature(fg.inplace_fused_experts).parameters
    # src/flaggems_vllm/ops/router_gemm.py:207, src/flaggems_vllm/ops/fp32_router_gemm.py:17,143
    assert [n for n, _, _ in _sig(fg.router_gemm)] == ["x", "weight"]
    assert [n for n, _, _ in _sig(fg.fp32_router_gemm)] == ["input", "router_weight"]
    assert [n for n, _, _ in _sig(fg.supports_fp32_router_gemm)] == [
        "hidden_size", "num_experts", "input_dtype", "weight_dtype"]
    assert flaggems_vllm.router_gemm is fg.router_gemm


_KIND = {inspect.Parameter.POSITIONAL_OR_KEYWORD: "positional", inspect.Parameter.POSITIONAL_ONLY: "positional",
         inspect.Parameter.KEYWORD_ONLY: "keyword_only", inspect.Parameter.VAR_POSITIONAL: "var_positional",
         inspect.Parameter.VAR_KEYWORD: "var_keyword"}


def test_signatures_match_the_reference_source():
    """Names, order, kinds and defaults of every public function of the path, against
    tests/golden/signatures.json, which tests/golden/make_signatures.py reads from the
    reference's source with ast."""
    import json

    with open(os.path.join(ROOT, "tests", "golden", "signatures.json")) as fh:
        ref = json.load(fh)
    assert len(ref) >= 14
    for name, info in ref.items():
        ours = [[n, _KIND[p.kind], None if p.default is inspect._empty else repr(p.default)]
                for n, p in inspect.signature(getattr(fg, name)).parameters.items()]
        assert ours == info["params"], f"{name} differs from {info['source']}"
        assert getattr(flaggems_vllm, name) is getattr(fg, name)


def test_grouped_topk_validation_errors():
    s = torch.zeros(4, 16)
    b = torch.zeros(16)
    with pytest.raises(ValueError, match="2D"):
        fg.grouped_topk(torch.zeros(16), 1, 1, 2, True, 1.0, b)
    with pytest.raises(ValueError, match="divisible"):
        fg.grouped_topk(s, 3, 1, 2, True, 1.0, b)
    with pytest.raises(ValueError, match="n_group"):
        fg.grouped_topk(torch.zeros(4, 64), 64, 1, 2, True, 1.0, torch.zeros(64))
    with pytest.raises(ValueError, match="topk"):
        fg.grouped_topk(torch.zeros(4, 64), 1, 1, 33, True, 1.0, torch.zeros(64))
    with pytest.raises(ValueError, match="scoring_func"):
        fg.grouped_topk(s, 1, 1, 2, True, 1.0, b, 2)
    with pytest.raises(ValueError, match="bias length"):
        fg.grouped_topk(s, 1, 1, 2, True, 1.0, torch.zeros(8))
    with pytest.raises(ValueError, match="Unsupported dtype"):
        fg.grouped_topk(s.double(), 1, 1, 2, True, 1.0, b)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fg.grouped_topk(s, 1, 1, 2, True, 1.0, b)  # valid arguments, CPU tensors


def test_fused_experts_validation_errors():
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    w1 = torch.zeros(2, 256, 64, dtype=torch.bfloat16)
    w2 = torch.zeros(2, 64, 128, dtype=torch.bfloat16)
    tw = torch.zeros(4, 2)
    ti = torch.zeros(4, 2, dtype=torch.int32)
    with pytest.raises(ValueError, match="Unknown MoE activation"):
        fg.fused_experts_impl(x, w1, w2, tw, ti, activation="tanh")
    with pytest.raises(ValueError, match="Only 'silu'"):
        fg.fused_experts_impl(x, w1, w2, tw, ti, activation="gelu")
    with pytest.raises(ValueError, match="require swigluoai"):
        fg.fused_experts_impl(x, w1, w2, tw, ti, gemm1_alpha=1.0)
    with pytest.raises(NotImplementedError):
        fg.fused_experts_impl(x, w1, w2, tw, ti, ocp_mx_scheme="w_bogus")
    with pytest.raises(AssertionError, match="Hidden size mismatch"):
        fg.fused_experts_impl(torch.zeros(4, 32, dtype=torch.bfloat16), w1, w2, tw, ti)
    with pytest.raises(AssertionError, match="topk shape"):
        fg.fused_experts_impl(x, w1, w2, torch.zeros(4, 3), ti)
    with pytest.raises(AssertionError, match="contiguous"):
        fg.fused_experts_impl(torch.zeros(64, 4, dtype=torch.bfloat16).t(), w1, w2, tw, ti)
    with pytest.raises(AssertionError, match="weights expected"):
        fg.fused_experts_impl(x, w1, w2, tw, ti, use_int8_w8a8=True)  # bf16 weights are not int8 weights
    with pytest.raises(NotImplementedError, match="block-quantised INT8"):
        fg.fused_experts_impl(x, w1.to(torch.int8), w2.to(torch.int8), tw, ti, use_int8_w8a8=True, block_shape=[128, 128])
    with pytest.raises(NotImplementedError, match="block_shape"):
        fg.fused_experts_impl(x, w1, w2, tw, ti, use_fp8_w8a8=True, block_shape=[64, 64])
    with pytest.raises(ValueError, match="finite scalar gemm1_alpha"):
        fg.fused_experts_impl(x, w1, w2, tw, ti, activation="swigluoai_uninterleave")
    with pytest.raises(ValueError, match="gemm1_clamp_limit >= 0"):
        fg.fused_experts_impl(x, w1, w2, tw, ti, activation="swigluoai_uninterleave", gemm1_alpha=1.702,
                              gemm1_beta=1.0, gemm1_clamp_limit=-1.0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fg.fused_experts_impl(x, w1, w2, tw, ti)


def test_router_gemm_validation_errors():
    x, w = torch.zeros(2, 16, dtype=torch.bfloat16), torch.zeros(4, 16, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="2D"):
        fg.router_gemm(x[0], w)
    with pytest.raises(ValueError, match="shape"):
        fg.router_gemm(x, w[:, :8])
    with pytest.raises(ValueError, match="CUDA device"):
        fg.fp32_router_gemm(x, w.float())
    assert fg.supports_fp32_router_gemm(6144, 128, torch.bfloat16, torch.float32)
    assert not fg.supports_fp32_router_gemm(7168, 256, torch.bfloat16, torch.float32)
    assert not fg.supports_fp32_router_gemm(6144, 128, torch.bfloat16, torch.bfloat16)


def test_align_rejects_cpu_tensors_and_bad_dtypes():
    with pytest.raises(RuntimeError, match="no CPU path"):
        fg.moe_align_block_size(torch.zeros(4, 2, dtype=torch.int32), 16, 8)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or Triton fallback"):
        _lib.lib()


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "flaggems_vllm_b200")
    for fn in os.listdir(pkg):
        if fn.endswith(".py"):
            src = open(os.path.join(pkg, fn)).read()
            assert "oracle" not in src, f"{fn} mentions the oracle"


def test_small_batch_slice_count_model():
    """The K-slice count asked of the small-batch GEMMs: never below what one unit can hold, never
    above 16, and the choices the measurements were taken with."""
    from flaggems_vllm_b200 import fused_moe

    H, I = 4096, 14336  # one token of the Mixtral shape: two experts
    assert fused_moe.small_k_slices(_lib.MODE_HALF, True, H, I, 2, 148) == 2      # 896 units, 7 per CTA at most
    assert fused_moe.small_k_slices(_lib.MODE_HALF, False, I, H, 2, 148) == 9     # 576 units: four full waves
    assert fused_moe.small_k_slices(_lib.MODE_W8A16, True, 2048, 768, 8, 148) == 1  # 96 units fit one wave
    for mode in (_lib.MODE_HALF, _lib.MODE_FP8_BLOCK, _lib.MODE_W8A16):
        for K in (128, 512, 2048, 7168, 14336):
            for blocks in (1, 2, 8, 64):
                for gemm1 in (True, False):
                    S = fused_moe.small_k_slices(mode, gemm1, K, 1024, blocks, 148)
                    chunks = K // (64 if mode == _lib.MODE_HALF else 128)
                    need = -(-chunks // (16 if mode == _lib.MODE_W8A16 else 32))
                    assert 1 <= S <= 16 and (S >= need or need > 16) and S <= max(chunks, 1)


def test_kernel_choice_at_the_benchmark_configurations(monkeypatch):
    """Host policy (no device work): which schedule serves the configurations of the benchmark plan."""
    from flaggems_vllm_b200 import fused_moe as fm

    for var in ("FLAGGEMS_B200_GENERIC_GEMM", "FLAGGEMS_B200_TC_WIDE", "FLAGGEMS_B200_TC_PAIR", "FLAGGEMS_B200_TC_PAIR_WIDE",
                "FLAGGEMS_B200_PRESORT", "FLAGGEMS_B200_TMA_OUT", "FLAGGEMS_B200_SMALL_M"):
        monkeypatch.delenv(var, raising=False)
    bf16 = torch.bfloat16
    # DeepSeek-V3 shape, FP8 block scales: always the 128-row tcgen05 kernel, never the small-batch schedule
    for M in (1, 32, 128, 1024, 8192):
        numel = M * 8
        assert fm._choose_kernel(_lib.MODE_FP8_BLOCK, bf16, 7168, 2048, numel, 256) == fm.KERNEL_TC
        assert not fm._use_small_path(_lib.MODE_FP8_BLOCK, bf16, 7168, 2048, numel, 8)
        assert fm._presort_rows(_lib.MODE_FP8_BLOCK, fm.KERNEL_TC, numel, 256) == (M >= 4096)
        assert fm._sorted_output(_lib.MODE_FP8_BLOCK, fm.KERNEL_TC, numel, 256) == (M >= 2048)
    # Mixtral shape, bf16: small-batch schedule up to 8 routes, the 256x256 tile from 256 rows per expert on
    assert fm._use_small_path(_lib.MODE_HALF, bf16, 4096, 14336, 2, 2)
    assert not fm._use_small_path(_lib.MODE_HALF, bf16, 4096, 14336, 32, 2)
    assert fm._choose_kernel(_lib.MODE_HALF, bf16, 4096, 14336, 512, 8) == fm.KERNEL_TC
    assert fm._choose_kernel(_lib.MODE_HALF, bf16, 4096, 14336, 2048, 8) == fm.KERNEL_TC_WIDE
    assert not fm._sorted_output(_lib.MODE_HALF, fm.KERNEL_TC_WIDE, 8192, 8)
    # Qwen3 shape, weight-only int8: small-batch schedule up to 16 routes, the converter kernel beyond
    assert fm._use_small_path(_lib.MODE_W8A16, bf16, 2048, 768, 8, 8)
    assert not fm._use_small_path(_lib.MODE_W8A16, bf16, 2048, 768, 512, 8)
    assert fm._choose_kernel(_lib.MODE_W8A16, bf16, 2048, 768, 32768, 128) == fm.KERNEL_TC
    # shapes the tensor-core kernels do not serve fall to the generic kernel; the switches override
    assert fm._choose_kernel(_lib.MODE_HALF, torch.float32, 4096, 14336, 2048, 8) == fm.KERNEL_GENERIC
    assert fm._choose_kernel(_lib.MODE_FP8_BLOCK, bf16, 7168 + 64, 2048, 64, 256) == fm.KERNEL_GENERIC
    monkeypatch.setenv("FLAGGEMS_B200_TC_PAIR", "1")
    assert fm._choose_kernel(_lib.MODE_FP8_BLOCK, bf16, 7168, 2048, 65536, 256) == fm.KERNEL_TC_PAIR
    monkeypatch.setenv("FLAGGEMS_B200_GENERIC_GEMM", "1")
    assert fm._choose_kernel(_lib.MODE_FP8_BLOCK, bf16, 7168, 2048, 65536, 256) == fm.KERNEL_GENERIC

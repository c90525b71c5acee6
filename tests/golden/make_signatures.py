"""Write tests/golden/signatures.json: the parameter lists of the reference's public functions
on the fused-MoE path, read from its source with ``ast`` (nothing is imported or executed).

    python tests/golden/make_signatures.py /path/to/FlagGems-vllm

Each entry is a list of [name, kind, default] with kind one of "positional", "keyword_only",
"var_positional", "var_keyword" and default the source text of the default (null: none).
tests/test_host_api.py compares the signatures of this package with the file."""

from __future__ import annotations

import ast
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
WANTED = {
    "grouped_topk.py": ["grouped_topk"],
    "moe_align_block_size.py": ["moe_align_block_size", "moe_align_block_size_triton", "moe_align_block_size_no_tle"],
    "fused_moe.py": ["fused_experts_impl", "inplace_fused_experts", "outplace_fused_experts"],
    "moe_sum.py": ["moe_sum"],
    "per_token_group_quant_fp8.py": ["per_token_group_quant_fp8"],
    "topk_softmax.py": ["topk_softmax"],
    "topk_sigmoid.py": ["topk_sigmoid"],
    "router_gemm.py": ["router_gemm"],
    "fp32_router_gemm.py": ["fp32_router_gemm", "supports_fp32_router_gemm"],
    "silu_and_mul.py": ["silu_and_mul", "silu_and_mul_out"],
}


def params_of(fn: ast.FunctionDef):
    a = fn.args
    out = []
    pos = list(a.posonlyargs) + list(a.args)
    defaults = [None] * (len(pos) - len(a.defaults)) + list(a.defaults)
    for arg, d in zip(pos, defaults):
        out.append([arg.arg, "positional", None if d is None else ast.unparse(d)])
    if a.vararg:
        out.append([a.vararg.arg, "var_positional", None])
    for arg, d in zip(a.kwonlyargs, a.kw_defaults):
        out.append([arg.arg, "keyword_only", None if d is None else ast.unparse(d)])
    if a.kwarg:
        out.append([a.kwarg.arg, "var_keyword", None])
    return out


def main(ref_root: str) -> None:
    ops = os.path.join(ref_root, "src", "flaggems_vllm", "ops")
    sigs = {}
    for fname, names in WANTED.items():
        path = os.path.join(ops, fname)
        with open(path, encoding="utf-8") as fh:
            tree = ast.parse(fh.read(), filename=path)
        for node in tree.body:
            if isinstance(node, ast.FunctionDef) and node.name in names:
                sigs[node.name] = {"source": f"src/flaggems_vllm/ops/{fname}:{node.lineno}", "params": params_of(node)}
        missing = [n for n in names if n not in sigs]
        if missing:
            raise RuntimeError(f"{path}: not found: {missing}")
    with open(os.path.join(HERE, "signatures.json"), "w") as fh:
        json.dump(sigs, fh, indent=1, sort_keys=True)
    print(f"wrote {len(sigs)} signatures")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_signatures.py /path/to/FlagGems-vllm")
    main(sys.argv[1])

"""Generate the golden vectors under tests/golden/ by EXECUTING the reference
project's own golden functions.

The reference package itself cannot be imported on a GPU-less machine, and its
test modules import it at the top, so this script lifts the individual golden
function definitions (and the few module constants they use) out of the
reference's test files with ``ast`` and executes them unchanged on the CPU.
Nothing of the reference is copied into this repository: only the inputs and
the outputs of those functions are stored, as compressed ``.npz`` files.

Run (only where the reference checkout is available):

    python tests/golden/make_golden.py /path/to/reference

The committed ``.npz`` files are what the tests read; this script is kept so
the vectors can be regenerated and audited.
"""

from __future__ import annotations

import ast
import os
import sys
from math import ceil

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def lift(path: str, names: list[str], extra_globals: dict) -> dict:
    """Execute the top-level definitions called ``names`` from ``path``."""
    with open(path, "r", encoding="utf-8") as fh:
        tree = ast.parse(fh.read(), filename=path)
    picked = []
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef,)) and node.name in names:
            picked.append(node)
        elif isinstance(node, ast.Assign):
            tg = [t.id for t in node.targets if isinstance(t, ast.Name)]
            if any(t in names for t in tg):
                picked.append(node)
    found = set()
    for node in picked:
        if isinstance(node, ast.FunctionDef):
            found.add(node.name)
        else:
            found.update(t.id for t in node.targets if isinstance(t, ast.Name))
    missing = set(names) - found
    if missing:
        raise RuntimeError(f"{path}: not found: {sorted(missing)}")
    mod = ast.Module(body=picked, type_ignores=[])
    ns = dict(extra_globals)
    exec(compile(mod, path, "exec"), ns)
    return ns


def t2n(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def save(name: str, **arrays):
    out = {k: (t2n(v) if torch.is_tensor(v) else np.asarray(v)) for k, v in arrays.items()}
    np.savez_compressed(os.path.join(HERE, name), **out)
    print("wrote", name, {k: v.shape for k, v in out.items()})


def main(ref_root: str):
    tests = os.path.join(ref_root, "tests")
    base = {"torch": torch, "device": "cpu", "vendor_name": "nvidia", "ceil": ceil}

    # ------------------------------------------------------------ routing
    rt = lift(
        os.path.join(tests, "test_grouped_topk.py"),
        ["MAX_IDX", "SIGN_MASK_INT32", "SIGN_MASK_INT64", "_pack_val_idx_fp32",
         "_unpack_val_idx_fp32", "torch_grouped_topk", "_torch_padding_routing_reference"],
        base,
    )
    eager = rt["_torch_padding_routing_reference"]
    packed = rt["torch_grouped_topk"]
    g = torch.Generator().manual_seed(1234)
    cases = []
    # (experts, groups, keep, topk, renorm, scale, scoring, score dtype, rows)
    specs = [
        (256, 8, 4, 8, True, 2.5, 1, torch.float32, 24),
        (256, 8, 4, 8, True, 2.5, 1, torch.bfloat16, 24),
        (256, 8, 4, 8, False, 1.0, 0, torch.float32, 9),
        (256, 1, 1, 8, True, 1.0, 0, torch.float32, 9),
        (128, 1, 1, 8, True, 1.0, 0, torch.float32, 17),
        (8, 1, 1, 2, True, 1.0, 0, torch.float32, 33),
        (64, 4, 2, 6, True, 1.5, 1, torch.float16, 11),
        (16, 4, 2, 2, False, 1.0, 1, torch.float32, 8),
    ]
    for i, (E, G, keep, k, ren, scale, sf, dt, rows) in enumerate(specs):
        scores = torch.randn(rows, E, generator=g, dtype=torch.float32)
        if sf == 0:
            scores = torch.softmax(scores, dim=-1)
        scores = scores.to(dt)
        bias = torch.randn(E, generator=g, dtype=torch.float32) * 0.1
        if G == 1:
            bias = torch.zeros(E)
        w, ids = eager(scores, G, keep, k, ren, scale, bias, sf)
        w2, ids2 = packed(scores, G, keep, k, ren, scale, bias, sf)
        cases.append(i)
        save(
            f"routing_{i}.npz",
            scores=scores.float(), score_dtype=str(dt), bias=bias,
            params=np.array([E, G, keep, k, int(ren), sf]), scale=np.array([scale]),
            weights=w.float(), ids=ids.int(), weights_packed=w2.float(), ids_packed=ids2.int(),
        )
    # the margin-heavy linspace/roll fixture of the reference's padding test
    for j, (E, G, keep, k) in enumerate([(256, 1, 1, 8), (256, 8, 4, 8)]):
        rows = 9
        score = torch.linspace(-2.0, 2.0, E)
        scores = torch.stack([score.roll(i * 17) for i in range(rows)])
        bias = torch.linspace(-0.30, 0.30, E)
        w, ids = eager(scores, G, keep, k, True, 3.998, bias, 1)
        save(
            f"routing_linspace_{j}.npz", scores=scores, score_dtype="torch.float32", bias=bias,
            params=np.array([E, G, keep, k, 1, 1]), scale=np.array([3.998]),
            weights=w.float(), ids=ids.int(),
        )

    # ------------------------------------------------------------ align
    al = lift(os.path.join(tests, "test_moe_align_block_size.py"),
              ["torch_moe_align_block_size"], base)
    golden_align = al["torch_moe_align_block_size"]
    g = torch.Generator().manual_seed(99)
    aspecs = [(1, 2, 8, 8), (4, 2, 8, 8), (33, 8, 256, 64), (128, 8, 256, 128), (77, 10, 250, 16),
              (300, 4, 10, 32), (64, 6, 128, 16), (5, 8, 512, 64)]
    for i, (M, k, E, bs) in enumerate(aspecs):
        ids = torch.randint(0, E, (M, k), generator=g, dtype=torch.int32)
        if i == 0:
            ids = torch.tensor([[1, 3]], dtype=torch.int32)
        if i == 1:
            ids = torch.tensor([[0, 1], [1, 2], [2, 3], [3, 0]], dtype=torch.int32)
        max_pad = ids.numel() + E * (bs - 1)
        s = torch.empty(max_pad, dtype=torch.int32)
        e = torch.empty(max_pad // bs, dtype=torch.int32)
        n = torch.empty(1, dtype=torch.int32)
        golden_align(ids, E, bs, s, e, n)
        save(f"align_{i}.npz", topk_ids=ids, params=np.array([E, bs]),
             sorted_ids=s, expert_ids=e, num_post_pad=n)
    # ------------------------------------------------------------ layers
    ly = lift(
        os.path.join(tests, "test_fused_experts_impl.py"),
        ["make_topk_routing", "torch_fused_moe_reference", "torch_w8a8_block_matmul",
         "torch_per_token_group_quant_fp8", "torch_w8a8_block_fp8_moe",
         "torch_fused_moe_weight_only_reference"],
        base,
    )
    for i, (M, E, H, I, k, dt) in enumerate(
        [(8, 4, 64, 128, 2, torch.bfloat16), (16, 4, 128, 128, 2, torch.float16),
         (5, 4, 128, 128, 3, torch.bfloat16)]
    ):
        torch.manual_seed(i)
        x = torch.randn(M, H, dtype=dt)
        w1 = torch.randn(E, 2 * I, H, dtype=dt) * (1.0 / H**0.5)
        w2 = torch.randn(E, H, I, dtype=dt) * (1.0 / I**0.5)
        gating = torch.randn(M, E, dtype=torch.float32)
        tw, ti = ly["make_topk_routing"](gating, k, dt)
        ref = ly["torch_fused_moe_reference"](x, w1, w2, tw, ti)
        save(f"layer_half_{i}.npz", dtype=str(dt), x=x, w1=w1, w2=w2,
             gating=gating, topk_weights=tw.float(), topk_ids=ti, out=ref.float())
    for i, (M, E, H, I, k) in enumerate([(6, 4, 128, 128, 2), (16, 4, 256, 256, 2)]):
        torch.manual_seed(10 + i)
        dt = torch.bfloat16
        x = torch.randn(M, H, dtype=dt)
        w1 = (torch.randn(E, 2 * I, H) * (1.0 / H**0.5)).to(torch.float8_e4m3fn)
        w2 = (torch.randn(E, H, I) * (1.0 / I**0.5)).to(torch.float8_e4m3fn)
        w1s = torch.randn(E, ceil(2 * I / 128), ceil(H / 128))
        w2s = torch.randn(E, ceil(H / 128), ceil(I / 128))
        gating = torch.randn(M, E)
        tw, ti = ly["make_topk_routing"](gating, k, dt)
        ref = ly["torch_w8a8_block_fp8_moe"](x, w1, w2, w1s, w2s, tw, ti, [128, 128])
        xq, xs = ly["torch_per_token_group_quant_fp8"](x, 128)
        save(f"layer_fp8_{i}.npz", x=x, w1=w1, w2=w2, w1_scale=w1s, w2_scale=w2s,
             topk_weights=tw.float(), topk_ids=ti, out=ref.float(), xq=xq, xs=xs)
    for i, (M, E, H, I, k) in enumerate([(7, 4, 128, 128, 2)]):
        torch.manual_seed(20 + i)
        dt = torch.bfloat16
        x = torch.randn(M, H, dtype=dt)
        w1f = torch.randn(E, 2 * I, H) * (1.0 / H**0.5)
        w2f = torch.randn(E, H, I) * (1.0 / I**0.5)
        s1 = w1f.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10) / 127.0
        s2 = w2f.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10) / 127.0
        w1 = (w1f / s1).round().clamp(-128, 127).to(torch.int8)
        w2 = (w2f / s2).round().clamp(-128, 127).to(torch.int8)
        gating = torch.randn(M, E)
        tw, ti = ly["make_topk_routing"](gating, k, dt)
        ref = ly["torch_fused_moe_weight_only_reference"](
            x, w1, w2, s1.squeeze(-1), s2.squeeze(-1), tw, ti)
        save(f"layer_w8a16_{i}.npz", x=x, w1=w1, w2=w2, w1_scale=s1.squeeze(-1),
             w2_scale=s2.squeeze(-1), topk_weights=tw.float(), topk_ids=ti, out=ref.float())

    # ------------------------------------------------------------ non-grouped routers
    ts = lift(os.path.join(tests, "test_topk_sigmoid.py"), ["reference"], base)
    g = torch.Generator().manual_seed(31)
    for i, (m, e, k, ren, bias_on) in enumerate([(7, 128, 8, True, True), (64, 256, 4, False, False),
                                                 (5, 64, 8, True, False)]):
        logits = torch.randn((m, e), generator=g)
        bias = torch.randn((e,), generator=g) * 0.1 if bias_on else None
        w, ids, src = ts["reference"](logits, bias, k, ren)
        save(f"topk_sigmoid_{i}.npz", logits=logits, bias=bias if bias is not None else torch.zeros(0),
             params=np.array([k, int(ren), int(bias_on)]), weights=w, ids=ids.int(), source=src)

    # ------------------------------------------------------------ fp8 quant
    qt = lift(os.path.join(tests, "test_per_token_group_quant_fp8.py"),
              ["native_per_token_group_quant_fp8"], base)
    torch.manual_seed(7)
    x = torch.randn(9, 384, dtype=torch.bfloat16) * 3.0
    x[0, :128] = 0
    q, s = qt["native_per_token_group_quant_fp8"](x, 128, dtype=torch.float8_e4m3fn)
    save("quant_fp8_0.npz", x=x, q=q, s=s)
    q, s = qt["native_per_token_group_quant_fp8"](x, 128, dtype=torch.float8_e4m3fn, scale_ue8m0=True)
    save("quant_fp8_ue8m0_0.npz", x=x, q=q, s=s)
    # other group sizes and a larger clamp (a group of zeros then takes the clamp as its amax)
    for i, (group, eps) in enumerate([(64, 1e-10), (256, 1e-10), (32, 1e-4), (384, 1e-2)]):
        torch.manual_seed(70 + i)
        xg = torch.randn(5, 768, dtype=torch.bfloat16) * 2.0
        xg[1, :group] = 0
        q, s = qt["native_per_token_group_quant_fp8"](xg, group, eps=eps, dtype=torch.float8_e4m3fn)
        save(f"quant_fp8_group_{i}.npz", x=xg, q=q, s=s, params=np.array([group, eps]))

    # ------------------------------------------------------------ INT8 W8A8 with the swigluoai activation
    fm = lift(os.path.join(tests, "test_fused_moe.py"), ["literal_oai", "literal_quant"], base)
    for i, (dt, shape) in enumerate([(torch.bfloat16, (7, 384)), (torch.float16, (32, 768)), (torch.bfloat16, (1, 127))]):
        torch.manual_seed(43 + i)
        x = torch.randn(shape, dtype=dt) * 8
        if i == 0:  # the half-way and all-zero rows the reference tests spell out
            x[0, :4] = torch.tensor([127.0, 0.5, 1.5, 2.5], dtype=dt)
            x[0, 4:] = 0
            x[1] = 0
            x[2, :4] = torch.tensor([52.0, 26.0, 13.0, 0.0], dtype=dt)
        q, sc = fm["literal_quant"](x)
        packed = torch.randn((shape[0], 2 * shape[1]), dtype=dt) * 8
        save(f"quant_int8_{i}.npz", dtype=str(dt), x=x, q=q, s=sc, packed=packed, oai=fm["literal_oai"](packed))
    for i, (dt, m, inter) in enumerate([(torch.bfloat16, 7, 384), (torch.float16, 5, 256)]):
        # the literal loop of tests/test_fused_moe.py:143-160, with that file's own quantiser and activation
        torch.manual_seed(47 + i)
        e, h, k = 4, 128, 2
        x = torch.randn((m, h), dtype=dt)
        w1 = torch.randint(-64, 64, (e, 2 * inter, h), dtype=torch.int8)
        w2 = torch.randint(-64, 64, (e, h, inter), dtype=torch.int8)
        s1 = torch.rand((e, 2 * inter)) * 0.001 + 0.001
        s2 = torch.rand((e, h)) * 0.001 + 0.001
        ids = (torch.arange(m * k).view(m, k) % e).int()
        weights = torch.rand((m, k))
        weights /= weights.sum(-1, keepdim=True)
        qx, sx = fm["literal_quant"](x)
        contributions = []
        for t in range(m):
            row = []
            for rank in range(k):
                ex = int(ids[t, rank])
                up = (qx[t:t + 1].float() @ w1[ex].float().t()) * sx[t] * s1[ex]
                activated = fm["literal_oai"](up.to(dt))
                qa, sa = fm["literal_quant"](activated)
                down = (qa.float() @ w2[ex].float().t()) * sa * s2[ex]
                row.append((down * weights[t, rank]).to(dt))
            contributions.append(torch.stack(row).float().sum(0).to(dt))
        save(f"layer_w8a8_int8_{i}.npz", dtype=str(dt), x=x, w1=w1, w2=w2, w1_scale=s1, w2_scale=s2,
             topk_weights=weights, topk_ids=ids, out=torch.cat(contributions).float())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/FlagGems-vllm")
    main(sys.argv[1])

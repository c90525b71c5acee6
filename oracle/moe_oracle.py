"""CPU oracle for the fused-MoE hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU and in plain torch/numpy, the algorithms that
the reference project's own tests use as goldens for the path

    grouped_topk -> moe_align_block_size -> fused_experts_impl

It exists to check the CUDA kernels and to provide the timed CPU baseline.  It
is never imported by the product package: only ``tests/``, the smoke check of
``__graft_entry__`` and, in ``bench.py``, the ``cpu_baseline`` / ``--impl reference`` legs and
the expert-parallel parity check (as the checker of sampled tokens, outside every timed region)
may use it.

Parity is PINNED: ``tests/golden/`` holds vectors produced by executing the
reference's own golden functions (extracted from its test files by
``tests/golden/make_golden.py``), and ``tests/test_oracle_golden.py`` checks
every function below against them, plus the known-answer cases the reference
tests spell out (tie order, +-inf, signed zeros, tiny exact-order align cases).

Reference locations each function follows (paths inside the reference tree):

* routing      tests/test_grouped_topk.py:673-708 (``_torch_padding_routing_reference``)
               cross-checked with tests/test_grouped_topk.py:82-155 (``torch_grouped_topk``)
* softmax top-k tests/test_fused_experts_impl.py:142-146 (``make_topk_routing``)
* align        tests/test_moe_align_block_size.py:293-388 (``torch_moe_align_block_size``)
               with the output sizes of src/flaggems_vllm/ops/moe_align_block_size.py:896-927
* fp8 quant    tests/test_per_token_group_quant_fp8.py:70-104 and
               tests/test_fused_experts_impl.py:551-570
* block matmul tests/test_fused_experts_impl.py:500-548
* layers       tests/test_fused_experts_impl.py:149-191 (half), :573-631 (fp8 block),
               :817-852 (int8 weight-only)
* moe_sum      tests/test_moe_sum.py:27-42
"""

from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


# ----------------------------------------------------------------------------
# Routing
# ----------------------------------------------------------------------------
def _sigmoid_f32(x: torch.Tensor) -> torch.Tensor:
    """fp32 sigmoid defined as the double-precision value rounded once to
    fp32 (i.e. correctly rounded).  torch's fp32 sigmoid and the reference
    kernel's ``1/(1+exp2(-x*log2e))`` (src/flaggems_vllm/ops/grouped_topk.py:304-307)
    are both within an ulp or two of this value; fixing the definition makes
    the ranking reproducible bit for bit on any device."""
    return torch.sigmoid(x.double()).float()


def grouped_topk_oracle(
    scores: torch.Tensor,
    n_group: int,
    topk_group: int,
    topk: int,
    renormalize: bool,
    routed_scaling_factor: float,
    bias: torch.Tensor,
    scoring_func: int = 0,
    is_padding: Optional[torch.Tensor] = None,
):
    """Group-limited top-k, all arithmetic in fp32.

    Follows the fast branch of ``_torch_padding_routing_reference``
    (tests/test_grouped_topk.py:673-708): unbiased = sigmoid(scores) or scores;
    ranked = unbiased + bias; a group's score is the sum of its two largest
    ranked values; the ``topk_group`` best groups survive (stable descending
    order, so ties keep the lower group id); the ``topk`` best ranked values
    among surviving groups are selected (ties keep the lower expert id, output
    order is descending); weights are the *unbiased* values, divided by
    (sum + 1e-20) when renormalising, then multiplied by the scaling factor.
    Padded rows produce weight 0 and id -1 (tests/test_grouped_topk.py:739-742).
    """
    s = scores.detach().to("cpu")
    b = bias.detach().to("cpu").flatten().float()
    rows, experts = s.shape
    per_group = experts // n_group
    u = s.float()
    unbiased = _sigmoid_f32(u) if scoring_func == 1 else u
    ranked = unbiased + b
    if per_group >= 2:
        group_score = ranked.view(rows, n_group, per_group).topk(2, dim=-1)[0].sum(-1)
    else:
        # One expert per group: the kernel's second extraction sees an empty
        # group and adds -inf is avoided by defining the score as the value.
        group_score = ranked.view(rows, n_group, per_group)[..., 0]
    group_ids = group_score.argsort(descending=True, stable=True)[:, :topk_group]
    enabled = torch.zeros_like(group_score, dtype=torch.bool)
    enabled.scatter_(1, group_ids, True)
    selected = enabled.unsqueeze(-1).expand(-1, -1, per_group).reshape(rows, experts)
    masked = ranked.masked_fill(~selected, float("-inf"))
    ids = masked.argsort(descending=True, stable=True)[:, :topk]
    weights = unbiased.gather(1, ids)
    if renormalize:
        weights = weights / (weights.sum(-1, keepdim=True) + 1e-20)
    weights = weights * routed_scaling_factor
    ids = ids.to(torch.int32)
    if is_padding is not None:
        pad = is_padding.detach().to("cpu").bool()
        weights = weights.masked_fill(pad[:, None], 0.0)
        ids = ids.masked_fill(pad[:, None], -1)
    return weights.float(), ids


def routing_margin_ulps(
    scores, n_group, topk_group, topk, bias, scoring_func=0
) -> torch.Tensor:
    """Per-row smallest gap, in fp32 ulps of the larger value, between
    neighbouring candidates that decide the result: the ``topk+1`` largest
    ranked values among surviving groups and the ``topk_group+1`` largest
    group scores.  A row whose margin is below a few ulps can legitimately
    change under a 1-ulp difference in how sigmoid is evaluated; tests use
    this to separate such rows from real mismatches."""
    s = scores.detach().to("cpu").float()
    b = bias.detach().to("cpu").flatten().float()
    rows, experts = s.shape
    per_group = experts // n_group
    unbiased = _sigmoid_f32(s) if scoring_func == 1 else s
    ranked = unbiased + b
    if per_group >= 2:
        top2 = ranked.view(rows, n_group, per_group).topk(2, dim=-1)[0]
        group_score = top2.sum(-1)
    else:
        group_score = ranked.view(rows, n_group)
    gs, gi = group_score.sort(descending=True, stable=True)
    enabled = torch.zeros_like(group_score, dtype=torch.bool)
    enabled.scatter_(1, gi[:, :topk_group], True)
    selected = enabled.unsqueeze(-1).expand(-1, -1, per_group).reshape(rows, experts)
    masked = ranked.masked_fill(~selected, float("-inf"))
    vs = masked.sort(descending=True, stable=True)[0][:, : min(topk + 1, experts)]

    def gaps(v):
        if v.shape[1] < 2:
            return torch.full((rows,), float("inf"))
        d = (v[:, :-1] - v[:, 1:]).double()
        ulp = torch.maximum(v[:, :-1].abs(), v[:, 1:].abs()).double() * 2.0**-23
        ulp = ulp.clamp_min(2.0**-149)
        g = torch.where(torch.isfinite(d), d / ulp, torch.full_like(d, float("inf")))
        return g.min(dim=1)[0]

    m = gaps(vs)
    if n_group > topk_group:
        m = torch.minimum(m, gaps(gs[:, : topk_group + 1]))
    if n_group > 1:
        # the top-2 sum itself may round differently only if sigmoid differs;
        # that is already covered by the ranked-value gaps above.
        pass
    return m


def topk_route_oracle(logits, bias, k, renormalize, sigmoid, scale=1.0, is_padding=None):
    """Non-grouped routers (tests/test_topk_sigmoid.py:11-24, tests/test_topk_softmax.py:146-164):
    p = sigmoid or softmax of the logits with NaN -> 0 (a softmax row holding NaN or +inf
    is all zeros), choice = p + bias, stable descending top-k of choice, weights = p
    gathered, divided by their sum when renormalising (if positive), times ``scale``;
    padded rows give weight 0 and id -1; source[m, j] = j * M + m.  Scores are the
    double-precision values rounded once to fp32 (see ``_sigmoid_f32``)."""
    x = logits.detach().cpu().double()
    p = (torch.sigmoid(x) if sigmoid else torch.softmax(x, dim=-1)).float()
    p = torch.nan_to_num(p, nan=0.0)
    choice = p if bias is None else p + bias.detach().cpu().float()
    ids = torch.argsort(choice, dim=-1, descending=True, stable=True)[:, :k]
    w = p.gather(1, ids)
    if renormalize:
        den = w.sum(-1, keepdim=True)
        w = w / torch.where(den > 0, den, torch.ones_like(den))
    w = w * scale
    m = x.shape[0]
    source = (torch.arange(k)[None, :] * m + torch.arange(m)[:, None]).int()
    if is_padding is not None:
        pad = is_padding.detach().cpu().bool()
        w = w.masked_fill(pad[:, None], 0.0)
        ids = ids.masked_fill(pad[:, None], -1)
    return w, ids, source


def softmax_topk_oracle(gating: torch.Tensor, topk: int, dtype: torch.dtype):
    """softmax -> top-k -> renormalise, ids int32
    (tests/test_fused_experts_impl.py:142-146)."""
    w, ids = torch.topk(torch.softmax(gating.cpu(), dim=-1), topk, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return w.to(dtype), ids.to(torch.int32)


# ----------------------------------------------------------------------------
# Align
# ----------------------------------------------------------------------------
def moe_align_block_size_oracle(
    topk_ids,
    block_size: int,
    num_experts: int,
    expert_map=None,
    pad_sorted_ids: bool = False,
):
    """Counting sort of the flat id array by expert, each non-empty expert's
    run padded to a multiple of ``block_size``.

    Ordering and sentinels follow ``torch_moe_align_block_size``
    (tests/test_moe_align_block_size.py:293-388): stable order inside an
    expert (ascending flat index), pad value ``numel``, unused block ids -1,
    ids outside ``[0, num_experts)`` are ignored.  Buffer sizes follow the
    public function (src/flaggems_vllm/ops/moe_align_block_size.py:896-927):
    ``numel + E*(bs-1)`` sorted slots (rounded up to a block multiple when
    ``pad_sorted_ids``), ``ceil`` of that over ``bs`` block ids, and the
    ``expert_map`` lookup is applied to the finished block-id array with torch
    indexing semantics (so -1 picks the last map entry).

    Returns numpy int32 arrays (sorted_ids, expert_ids, num_tokens_post_pad).
    """
    ids = np.asarray(
        topk_ids.detach().cpu().numpy() if torch.is_tensor(topk_ids) else topk_ids
    ).reshape(-1).astype(np.int64)
    numel = ids.size
    max_pad = numel + num_experts * (block_size - 1)
    if pad_sorted_ids:
        max_pad = -(-max_pad // block_size) * block_size
    n_blocks = -(-max_pad // block_size)
    sorted_ids = np.full(max_pad, numel, dtype=np.int32)
    expert_ids = np.full(n_blocks, -1, dtype=np.int32)
    valid = (ids >= 0) & (ids < num_experts)
    order = np.argsort(np.where(valid, ids, num_experts), kind="stable")
    counts = np.bincount(ids[valid], minlength=num_experts)[:num_experts]
    pos = 0
    blk = 0
    start = 0
    for e in range(num_experts):
        c = int(counts[e])
        if c > 0:
            sorted_ids[pos : pos + c] = order[start : start + c].astype(np.int32)
            nb = -(-c // block_size)
            expert_ids[blk : blk + nb] = e
            pos += nb * block_size
            blk += nb
        start += c
    total = np.array([pos], dtype=np.int32)
    if expert_map is not None:
        em = np.asarray(
            expert_map.detach().cpu().numpy() if torch.is_tensor(expert_map) else expert_map
        )
        expert_ids = em[expert_ids].astype(np.int32)
    return sorted_ids, expert_ids, total


# ----------------------------------------------------------------------------
# Quantisation helpers
# ----------------------------------------------------------------------------
def per_token_group_quant_fp8_oracle(x: torch.Tensor, group_size: int = 128, eps: float = 1e-10,
                                     reciprocal: bool = True, scale_ue8m0: bool = False):
    """1 x ``group_size`` e4m3 quantisation of the last dimension.

    ``reciprocal=True`` multiplies amax by fp32(1/448) like the reference kernel
    and ``native_per_token_group_quant_fp8`` (tests/test_per_token_group_quant_fp8.py:70-104);
    ``reciprocal=False`` divides by 448 like ``torch_per_token_group_quant_fp8``
    (tests/test_fused_experts_impl.py:551-570).  The two differ by at most one
    ulp of the scale.
    """
    assert x.shape[-1] % group_size == 0
    x = x.detach().cpu().contiguous()
    xr = x.reshape(-1, group_size)
    # eps is applied in fp32 like the reference kernel does
    # (src/flaggems_vllm/ops/per_token_group_quant_fp8.py:150-151); the torch
    # goldens clamp in the input dtype, which only differs for all-zero groups.
    amax = xr.float().abs().max(dim=-1, keepdim=True)[0].clamp(min=eps)
    if reciprocal:
        s = amax * torch.tensor(1.0 / FP8_MAX, dtype=torch.float32)
    else:
        s = amax / FP8_MAX
    if scale_ue8m0:
        # power-of-two scales, the expression of the reference kernel and of its golden
        # (per_token_group_quant_fp8.py:153-154, tests/test_per_token_group_quant_fp8.py:88-91)
        s = torch.exp2(torch.ceil(torch.log2(torch.maximum(s.abs(), torch.tensor(1e-10)))))
    q = (xr.float() / s).clamp(min=-FP8_MAX, max=FP8_MAX).to(FP8)
    return q.reshape(x.shape), s.reshape(x.shape[:-1] + (x.shape[-1] // group_size,))


def router_gemm_oracle(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """fp32 logits ``x @ weight.T`` with both operands upcast first, the reference the
    project's own tests compare against (tests/test_router_gemm.py:46-50,
    tests/test_fp32_router_gemm.py)."""
    return torch.mm(x.detach().cpu().float(), weight.detach().cpu().float().t())


def block_scaled_matmul_oracle(a_q, a_s, b_q, b_s, block_n: int, block_k: int):
    """``C = sum_kb (A_kb @ B_kb^T) * a_s[:, kb] * b_s[nb, kb]`` in fp32
    (tests/test_fused_experts_impl.py:500-548), vectorised over blocks."""
    a = a_q.float()
    b = b_q.float()
    m, k = a.shape
    n = b.shape[0]
    kt = -(-k // block_k)
    nt = -(-n // block_n)
    c = torch.zeros(m, n, dtype=torch.float32)
    for i in range(kt):
        ks = slice(i * block_k, min((i + 1) * block_k, k))
        part = a[:, ks] @ b[:, ks].t()
        col_scale = b_s[:, i].float().repeat_interleave(block_n)[:n]
        c += part * a_s[:, i : i + 1].float() * col_scale[None, :]
    del nt
    return c


def _silu_mul(z: torch.Tensor) -> torch.Tensor:
    d = z.shape[-1] // 2
    g = z[..., :d]
    return (g * torch.sigmoid(g)) * z[..., d:]


# ----------------------------------------------------------------------------
# Layers.  All are per-expert batched restatements of per-(token, route) loops.
# ----------------------------------------------------------------------------
def _expert_rows(topk_ids: torch.Tensor, e: int):
    flat = topk_ids.reshape(-1)
    idx = torch.nonzero(flat == e, as_tuple=False).flatten()
    return idx


def fused_moe_half_oracle(hidden, w1, w2, topk_weights, topk_ids, *,
                          faithful: bool = False, apply_router_weight_on_input: bool = False, act_fn=None):
    """bf16/fp16 layer with fp32 math (tests/test_fused_experts_impl.py:149-191):
    ``out[m] = sum_j w[m,j] * W2[e] (SiLU(G) * U)``, ``[G;U] = W1[e] x[m]``.

    ``faithful=True`` additionally rounds the activation output and each
    weighted route output to the activation dtype, which is what the reference
    kernels store between launches (src/flaggems_vllm/ops/fused_moe.py:1969).
    The result is returned in fp32 so callers can measure error precisely.
    """
    hidden = hidden.cpu()
    dt = hidden.dtype
    M, H = hidden.shape
    k = topk_ids.shape[1]
    ids = topk_ids.cpu().long()
    wts = topk_weights.cpu().float().reshape(-1)
    x = hidden.float()
    per_route = torch.zeros(M * k, H, dtype=torch.float32)
    for e in range(w1.shape[0]):
        rows = _expert_rows(ids, e)
        if rows.numel() == 0:
            continue
        tok = rows // k
        xin = x[tok]
        if apply_router_weight_on_input:
            z = (xin @ w1[e].cpu().float().t()) * wts[rows, None]
        else:
            z = xin @ w1[e].cpu().float().t()
        # an unfused activation (``act_fn``) reads GEMM 1's output after it was stored in the activation dtype
        s = _silu_mul(z) if act_fn is None else act_fn(z.to(dt))
        if faithful or act_fn is not None:
            s = s.to(dt).float()
        r = s @ w2[e].cpu().float().t()
        if not apply_router_weight_on_input:
            r = r * wts[rows, None]
        if faithful:
            r = r.to(dt).float()
        per_route[rows] = r
    return per_route.view(M, k, H).sum(dim=1)


def fused_moe_fp8_block_oracle(hidden, w1_q, w2_q, w1_s, w2_s, topk_weights, topk_ids,
                               block_shape=(128, 128), *, faithful: bool = False,
                               reciprocal: bool = True):
    """FP8 e4m3 layer with 128x128 weight block scales and 1x128 activation
    groups (tests/test_fused_experts_impl.py:573-631).  The golden rounds the
    first GEMM's output and the second GEMM's output to the activation dtype;
    ``faithful=True`` keeps those roundings, ``faithful=False`` keeps only the
    one before re-quantisation (which every real kernel needs, since the
    re-quantisation input is defined in the activation dtype)."""
    hidden = hidden.cpu()
    dt = hidden.dtype
    bn, bk = block_shape
    M, H = hidden.shape
    k = topk_ids.shape[1]
    ids = topk_ids.cpu().long()
    wts = topk_weights.cpu().float().reshape(-1)
    xq, xs = per_token_group_quant_fp8_oracle(hidden, bk, reciprocal=reciprocal)
    per_route = torch.zeros(M * k, H, dtype=torch.float32)
    for e in range(w1_q.shape[0]):
        rows = _expert_rows(ids, e)
        if rows.numel() == 0:
            continue
        tok = rows // k
        inter = block_scaled_matmul_oracle(xq[tok], xs[tok], w1_q[e].cpu(), w1_s[e].cpu(), bn, bk)
        if faithful:
            # the golden rounds GEMM1 to the activation dtype and evaluates
            # SiLU and the product in that dtype
            inter = inter.to(dt)
            d = inter.shape[-1] // 2
            act = torch.nn.functional.silu(inter[..., :d]) * inter[..., d:]
        else:
            act = _silu_mul(inter).to(dt)
        aq, asc = per_token_group_quant_fp8_oracle(act, bk, reciprocal=reciprocal)
        r = block_scaled_matmul_oracle(aq, asc, w2_q[e].cpu(), w2_s[e].cpu(), bn, bk)
        if faithful:
            r = r.to(dt).float()
        else:
            r = r * wts[rows, None]
        per_route[rows] = r
    if faithful:
        wdt = topk_weights.cpu().reshape(M, k, 1).to(dt)
        return (per_route.view(M, k, H).to(dt) * wdt).sum(dim=1).float()
    return per_route.view(M, k, H).sum(dim=1)


def fused_moe_w8a16_oracle(hidden, w1_i8, w2_i8, w1_s, w2_s, topk_weights, topk_ids):
    """INT8 weight-only layer (tests/test_fused_experts_impl.py:817-852):
    weights are ``int8 * per-output-channel fp32 scale``, everything else as in
    the half layer, fp32 math."""
    hidden = hidden.cpu()
    M, H = hidden.shape
    k = topk_ids.shape[1]
    ids = topk_ids.cpu().long()
    wts = topk_weights.cpu().float().reshape(-1)
    x = hidden.float()
    per_route = torch.zeros(M * k, H, dtype=torch.float32)
    for e in range(w1_i8.shape[0]):
        rows = _expert_rows(ids, e)
        if rows.numel() == 0:
            continue
        tok = rows // k
        w1d = w1_i8[e].cpu().float() * w1_s[e].cpu().float().unsqueeze(-1)
        w2d = w2_i8[e].cpu().float() * w2_s[e].cpu().float().unsqueeze(-1)
        s = _silu_mul(x[tok] @ w1d.t())
        per_route[rows] = (s @ w2d.t()) * wts[rows, None]
    return per_route.view(M, k, H).sum(dim=1)


def int8_per_token_quant_oracle(x: torch.Tensor):
    """Per-row dynamic INT8 quantisation (tests/test_fused_moe.py:22-25, ``literal_quant``; kernel
    src/flaggems_vllm/ops/fused_moe.py:994-1010): amax clamped at 1e-10 IN THE INPUT DTYPE, scale =
    amax * fp32(1/127) as the kernel forms it (the literal divides by 127: the same value except
    for one ulp on rare rows), q = round-half-even(x / scale) clamped to [-128, 127]."""
    x = x.detach().cpu()
    amax = x.abs().amax(-1, keepdim=True).clamp(min=1e-10).float()
    scale = amax * torch.tensor(1.0 / 127.0, dtype=torch.float32)
    q = (x.float() / scale).round().clamp(-128, 127)
    q = torch.where(torch.isnan(q), torch.zeros_like(q), q).to(torch.int8)
    return q, scale


def fp8_per_token_quant_oracle(x: torch.Tensor):
    """Per-row dynamic e4m3 quantisation (src/flaggems_vllm/ops/fused_moe.py:899-911)."""
    x = x.detach().cpu()
    amax = x.abs().amax(-1, keepdim=True).clamp(min=1e-10).float()
    scale = (amax / FP8_MAX).clamp(min=1.0 / (FP8_MAX * 512.0))
    q = (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q, scale


def fp8_per_tensor_quant_oracle(x: torch.Tensor, scale: torch.Tensor | None = None):
    """Per-tensor e4m3 quantisation, static (``scale`` given: x / scale) or dynamic (amax / 448,
    multiplied by the reciprocal) -- src/flaggems_vllm/ops/fused_moe.py:913-922."""
    x = x.detach().cpu()
    if scale is not None:
        sc = scale.detach().cpu().float().reshape(1, 1)
        return (x.float() / sc).clamp(-FP8_MAX, FP8_MAX).to(FP8), sc.reshape(1)
    amax = x.abs().amax().clamp(min=1e-10).float()
    sc = amax / FP8_MAX
    q = (x.float() * (1.0 / sc)).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q, sc.reshape(1)


def swigluoai_oracle(z: torch.Tensor, alpha: float = 1.702, beta: float = 1.0, limit: float = 7.0) -> torch.Tensor:
    """gate|up halves: min(gate, limit) * sigmoid(alpha * gate) * (clamp(up, -limit, limit) + beta), fp32
    (tests/test_fused_moe.py:15-19 ``literal_oai``; kernel src/flaggems_vllm/ops/fused_moe.py:733-773)."""
    gate, up = z.float().chunk(2, dim=-1)
    gate = gate.clamp(max=limit)
    up = up.clamp(-limit, limit)
    return gate * torch.sigmoid(alpha * gate) * (up + beta)


def fused_moe_row_scaled_oracle(hidden, w1_q, w2_q, w1_s, w2_s, topk_weights, topk_ids, *, fmt: str,
                                per_token: bool = True, a1_scale=None, a2_scale=None, activation: str = "silu",
                                alpha: float = 1.702, beta: float = 1.0, limit: float = 7.0):
    """W8A8 layers whose scales multiply the finished dot product: INT8 (``fmt="int8"``) or e4m3
    (``fmt="fp8"``) activations with one scale per row (``per_token``) or per tensor, weights with one
    scale per output channel ``[E, N]`` (a per-tensor weight scale is that vector filled with one
    value).  Restates the literal loop of tests/test_fused_moe.py:143-160 per expert:
    ``up = (qx @ W1^T) * sx * s1`` rounded to the activation dtype, activation in fp32 rounded to the
    activation dtype, re-quantised, ``down = (qa @ W2^T) * sa * s2``, times the route weight, rounded to
    the activation dtype, summed over the routes in fp32."""
    hidden = hidden.detach().cpu()
    dt = hidden.dtype
    M, H = hidden.shape
    k = topk_ids.shape[1]
    ids = topk_ids.cpu().long()
    wts = topk_weights.cpu().float().reshape(-1)

    def quant(t, static):
        if fmt == "int8":
            if per_token:
                return int8_per_token_quant_oracle(t)
            sc = static.detach().cpu().float().reshape(1, 1)
            return (t.float() / sc).round().clamp(-128, 127).to(torch.int8), sc.expand(t.shape[0], 1)
        if per_token:
            return fp8_per_token_quant_oracle(t)
        q, sc = fp8_per_tensor_quant_oracle(t, static)
        return q, sc.reshape(1, 1).expand(t.shape[0], 1)

    # both activations are evaluated in fp32 on the stored (activation-dtype) output of GEMM 1
    act_fn = (lambda z: swigluoai_oracle(z, alpha, beta, limit)) if activation == "swigluoai_uninterleave" \
        else (lambda z: _silu_mul(z.float()))
    xq, xs = quant(hidden, a1_scale)
    rows_all = [(_expert_rows(ids, e), e) for e in range(w1_q.shape[0])]
    inter = torch.zeros(M * k, w1_q.shape[1] // 2, dtype=dt)
    for rows, e in rows_all:
        if rows.numel():
            tok = rows // k
            up = (xq[tok].float() @ w1_q[e].cpu().float().t()) * xs[tok] * w1_s[e].cpu().float().reshape(1, -1)
            inter[rows] = act_fn(up.to(dt)).to(dt)
    # the per-tensor dynamic scale of the intermediate is taken over all routes at once, as the reference does
    aq, as_ = quant(inter, a2_scale)
    per_route = torch.zeros(M * k, H, dtype=torch.float32)
    for rows, e in rows_all:
        if rows.numel():
            down = (aq[rows].float() @ w2_q[e].cpu().float().t()) * as_[rows] * w2_s[e].cpu().float().reshape(1, -1)
            per_route[rows] = (down * wts[rows, None]).to(dt).float()
    return per_route.view(M, k, H).sum(dim=1)


def moe_sum_oracle(inp: torch.Tensor) -> torch.Tensor:
    """fp32 sum over the top-k axis (tests/test_moe_sum.py:27-42)."""
    return inp.cpu().float().sum(dim=1)


# ----------------------------------------------------------------------------
# Parity metrics
# ----------------------------------------------------------------------------
def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().cpu().double()
    b = b.detach().cpu().double()
    den = b.norm().item()
    return (a - b).norm().item() / (den if den > 0 else 1.0)


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().cpu().double().flatten()
    b = b.detach().cpu().double().flatten()
    den = a.norm().item() * b.norm().item()
    return float((a @ b).item() / den) if den > 0 else 1.0


# ----------------------------------------------------------------------------
# Seeded synthetic inputs of the benchmark configurations
# ----------------------------------------------------------------------------
def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def quantize_weight_fp8_block(w: torch.Tensor, bn: int = 128, bk: int = 128):
    """fp32 [E,N,K] -> (e4m3 [E,N,K], fp32 scale [E,ceil(N/bn),ceil(K/bk)]),
    scale = amax(block)/448."""
    E, N, K = w.shape
    nt, kt = -(-N // bn), -(-K // bk)
    wp = torch.zeros(E, nt * bn, kt * bk, dtype=torch.float32)
    wp[:, :N, :K] = w
    blocks = wp.view(E, nt, bn, kt, bk)
    amax = blocks.abs().amax(dim=(2, 4)).clamp(min=1e-10)
    scale = amax / FP8_MAX
    q = (blocks / scale[:, :, None, :, None]).clamp(-FP8_MAX, FP8_MAX)
    q = q.reshape(E, nt * bn, kt * bk)[:, :N, :K].contiguous().to(FP8)
    return q, scale.contiguous()


def quantize_weight_int8_channel(w: torch.Tensor):
    """fp32 [E,N,K] -> (int8, fp32 scale [E,N]); symmetric, scale = amax/127
    (tests/test_fused_experts_impl.py:877-887)."""
    amax = w.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10)
    scale = amax / 127.0
    q = (w / scale).round().clamp(-128, 127).to(torch.int8)
    return q, scale.squeeze(-1).contiguous()


def make_layer_inputs(M, E, H, I, seed=0, dtype=torch.bfloat16, w_std=0.02):
    g = _gen(seed)
    x = torch.randn(M, H, generator=g, dtype=torch.float32).to(dtype)
    w1 = torch.randn(E, 2 * I, H, generator=g, dtype=torch.float32) * w_std
    w2 = torch.randn(E, H, I, generator=g, dtype=torch.float32) * w_std
    logits = torch.randn(M, E, generator=g, dtype=torch.float32)
    return x, w1, w2, logits


def make_align_ids(M, topk=8, E=256, skewed=False, seed=0):
    """Config-5 ids: uniform on [0,E), or with probability 0.5 one of the four
    hot experts {0,1,2,3}."""
    g = _gen(seed)
    ids = torch.randint(0, E, (M, topk), generator=g, dtype=torch.int64)
    if skewed:
        hot = torch.randint(0, 4, (M, topk), generator=g, dtype=torch.int64)
        pick = torch.rand(M, topk, generator=g) < 0.5
        ids = torch.where(pick, hot, ids)
    return ids.to(torch.int32)


def expected_distinct_experts(M, topk, E):
    return E * (1.0 - math.pow(1.0 - 1.0 / E, M * topk))


def silu_and_mul_oracle(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """SiLU(a) * b as the reference's test states it (tests/test_silu_and_mul.py:35,63:
    ``torch.mul(torch.nn.functional.silu(a), b)`` on upcast operands), in float64."""
    return torch.mul(torch.nn.functional.silu(a.double().cpu()), b.double().cpu())

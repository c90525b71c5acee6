"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (weights ~N(0, 0.02), activations ~N(0, 1), router
logits ~N(0, 1), routing bias ~N(0, 0.1)).  Used by the tests and by bench.py;
weights are generated and quantised on the device a few experts at a time so
that an 11 GB FP8 layer never needs an fp32 copy of itself."""

from __future__ import annotations

import torch

FP8_MAX = 448.0


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def make_half_weights(E, N, K, device, seed=0, dtype=torch.bfloat16, std=0.02, chunk=8):
    g = _gen(device, seed)
    w = torch.empty((E, N, K), dtype=dtype, device=device)
    for e0 in range(0, E, chunk):
        e1 = min(E, e0 + chunk)
        w[e0:e1] = (torch.randn((e1 - e0, N, K), generator=g, device=device, dtype=torch.float32) * std).to(dtype)
    return w


def make_fp8_block_weights(E, N, K, device, seed=0, std=0.02, block=128, chunk=8):
    """e4m3 weights [E, N, K] with fp32 scales [E, N/block, K/block], scale = amax/448."""
    assert N % block == 0 and K % block == 0
    g = _gen(device, seed)
    q = torch.empty((E, N, K), dtype=torch.float8_e4m3fn, device=device)
    s = torch.empty((E, N // block, K // block), dtype=torch.float32, device=device)
    for e0 in range(0, E, chunk):
        e1 = min(E, e0 + chunk)
        w = torch.randn((e1 - e0, N, K), generator=g, device=device, dtype=torch.float32) * std
        blocks = w.view(e1 - e0, N // block, block, K // block, block)
        amax = blocks.abs().amax(dim=(2, 4)).clamp(min=1e-10)
        sc = amax / FP8_MAX
        q[e0:e1] = (blocks / sc[:, :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(e1 - e0, N, K).to(
            torch.float8_e4m3fn)
        s[e0:e1] = sc
    return q, s


def make_int8_channel_weights(E, N, K, device, seed=0, std=0.02, chunk=16):
    """int8 weights [E, N, K], fp32 scale [E, N] = amax(row)/127 (symmetric)."""
    g = _gen(device, seed)
    q = torch.empty((E, N, K), dtype=torch.int8, device=device)
    s = torch.empty((E, N), dtype=torch.float32, device=device)
    for e0 in range(0, E, chunk):
        e1 = min(E, e0 + chunk)
        w = torch.randn((e1 - e0, N, K), generator=g, device=device, dtype=torch.float32) * std
        sc = w.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10) / 127.0
        q[e0:e1] = (w / sc).round().clamp(-128, 127).to(torch.int8)
        s[e0:e1] = sc.squeeze(-1)
    return q, s


def make_activations(M, H, device, seed=1, dtype=torch.bfloat16):
    return torch.randn((M, H), generator=_gen(device, seed), device=device, dtype=torch.float32).to(dtype)


def make_router_inputs(M, E, device, seed=2, bias_std=0.1):
    g = _gen(device, seed)
    logits = torch.randn((M, E), generator=g, device=device, dtype=torch.float32)
    bias = torch.randn((E,), generator=g, device=device, dtype=torch.float32) * bias_std
    return logits, bias


def make_align_ids(M, topk, E, device, skewed=False, seed=3):
    """Uniform ids, or (skewed) each assignment goes to one of the hot experts
    {0,1,2,3} with probability 0.5."""
    g = _gen(device, seed)
    ids = torch.randint(0, E, (M, topk), generator=g, device=device, dtype=torch.int32)
    if skewed:
        hot = torch.randint(0, 4, (M, topk), generator=g, device=device, dtype=torch.int32)
        pick = torch.rand((M, topk), generator=g, device=device) < 0.5
        ids = torch.where(pick, hot, ids)
    return ids

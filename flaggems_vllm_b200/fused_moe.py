"""fused_experts_impl: the MoE layer on expert-sorted rows.

Pipeline per chunk of at most 32768 tokens (the reference's chunk size,
src/flaggems_vllm/ops/fused_moe.py:2399-2400):

    moe_align_block_size          stable sort of routes by expert, 1 launch
    per_token_group_quant_fp8     FP8 mode only: activations -> e4m3 + 1x128 scales, once per token
    gemm1                         gathers token rows; SiLU(x Wg^T) * (x Wu^T)   (+ 1x128 re-quant, FP8)
    gemm2                         (act W2^T) * route weight -> y[route, H]
    moe_sum                       fixed-order fp32 sum over the top-k routes

The signature, accepted arguments and error types are those of the reference
function (src/flaggems_vllm/ops/fused_moe.py:2314-2390).  Modes served:
f16/bf16/f32 weights, FP8 e4m3 with 128x128 block scales, INT8/INT4-in-INT8
weight-only with per-channel scales.  Every other mode raises
NotImplementedError: there is no fallback path.
"""

from __future__ import annotations

import ctypes
import logging
import os
from typing import Optional

import torch

from . import _lib
from .align import ceil_div, round_up

logger = logging.getLogger(__name__)

CHUNK_SIZE = 32 * 1024
TC_BLOCK_M = 128
TC_PAIR_BLOCK_M = 256
TC_PAIR_WIDE_BLOCK_M = 512
GENERIC_BLOCK_M = 16
# kernel selector passed to moe_gemm1 / moe_gemm2
KERNEL_GENERIC, KERNEL_TC, KERNEL_TC_PAIR, KERNEL_TC_WIDE, KERNEL_TC_PAIR_WIDE = 0, 1, 2, 3, 4

_SUPPORTED_ACTIVATIONS = ("silu", "swigluoai_uninterleave")
_ALL_ACTIVATIONS = ("silu", "gelu", "relu2", "swigluoai", "swigluoai_uninterleave", "swiglustep",
                    "silu_no_mul", "gelu_no_mul", "relu2_no_mul")


# bench.py sets this to a callable(name) to time the stages of a step
STAGE_HOOK = None


def _no_mark(_name):
    return None


def _force_generic() -> bool:
    return os.environ.get("FLAGGEMS_B200_GENERIC_GEMM", "0").lower() in ("1", "true", "yes", "on")


def _policy(var: str) -> str:
    """Environment switch: 0 / off, 1 / on, anything else = auto."""
    v = os.environ.get(var, "auto").lower()
    return {"0": "off", "off": "off", "1": "on", "on": "on"}.get(v, "auto")


def _choose_kernel(mode, act_dtype, H, I, numel, num_experts):
    """Which GEMM kernel serves the call.  FLAGGEMS_B200_GENERIC_GEMM=1 forces the generic
    kernel, FLAGGEMS_B200_TC_WIDE / FLAGGEMS_B200_TC_PAIR = 0/1 force the 256-row variants
    off/on (tests and experiments); otherwise:

    * FP8 block scales: one CTA per 128-row block.  (The cta_group::2 pair loses there: the
      per-K-block accumulator hand-off would cross two SMs; GEMM1 3.6 -> 4.2 ms at M=8192.)
    * weight-only int8: the kernel that widens the weights in shared memory.
    * half precision with >= 256 rows per expert: the 256x256 single-CTA tile,
      which fetches each weight tile once per 256 rows.
    """
    if _force_generic() or not _tc_eligible(mode, act_dtype, H, I):
        return KERNEL_GENERIC
    wide, pair = _policy("FLAGGEMS_B200_TC_WIDE"), _policy("FLAGGEMS_B200_TC_PAIR")
    pair_wide = _policy("FLAGGEMS_B200_TC_PAIR_WIDE")
    if mode == _lib.MODE_W8A16:
        return KERNEL_TC  # int8 weights widened in shared memory, one CTA per 128-row block
    if pair_wide == "on" and mode == _lib.MODE_HALF:
        return KERNEL_TC_PAIR_WIDE
    if wide == "on" and mode == _lib.MODE_HALF:
        return KERNEL_TC_WIDE
    if pair == "on":
        return KERNEL_TC_PAIR
    if mode == _lib.MODE_HALF and numel >= 256 * num_experts and wide != "off":
        return KERNEL_TC_WIDE
    return KERNEL_TC


def _presort_rows(mode, kernel, numel, num_experts) -> bool:
    """GEMM1 reads a sorted copy of the token rows (TMA) instead of gathering them itself:
    half precision on the single-CTA tensor-core kernels with >= 256 rows per expert, FP8
    (e4m3 rows and their transposed scales) on the 128-row kernel with >= 128 rows per expert.
    FLAGGEMS_B200_PRESORT = 0/1 forces it off/on."""
    if mode == _lib.MODE_FP8_BLOCK:
        if kernel not in (KERNEL_TC, KERNEL_TC_PAIR):
            return False
    elif mode != _lib.MODE_HALF or kernel not in (KERNEL_TC, KERNEL_TC_WIDE):
        return False
    force = _policy("FLAGGEMS_B200_PRESORT")
    if force != "auto":
        return force == "on"
    return numel >= (128 if mode == _lib.MODE_FP8_BLOCK else 256) * num_experts


def _sorted_output(mode, kernel, numel, num_experts) -> bool:
    """GEMM2 of the 128-row tensor-core kernel writes its rows in sorted order through a staged tile and
    TMA stores (FP8 block scales and half precision) when experts own enough rows for the epilogue to
    matter: from 64 rows per expert on.  FLAGGEMS_B200_TMA_OUT = 0/1 forces it off/on."""
    if kernel != KERNEL_TC or mode not in (_lib.MODE_FP8_BLOCK, _lib.MODE_HALF):
        return False
    force = _policy("FLAGGEMS_B200_TMA_OUT")
    if force != "auto":
        return force == "on"
    return numel >= 64 * num_experts


def _tc_eligible(mode: int, act_dtype: torch.dtype, H: int, I: int) -> bool:
    if act_dtype not in (torch.bfloat16, torch.float16):
        return False
    if mode == _lib.MODE_FP8_BLOCK:
        return H % 128 == 0 and I % 128 == 0
    if mode in (_lib.MODE_HALF, _lib.MODE_W8A16):
        return H % 64 == 0 and I % 128 == 0
    return False


def _check_activation(activation, gemm1_alpha, gemm1_beta, gemm1_clamp_limit):
    if activation not in _ALL_ACTIVATIONS:
        raise ValueError(f"Unknown MoE activation: {activation!r}. Valid activations: {list(_ALL_ACTIVATIONS)}")
    if activation == "swigluoai_uninterleave":
        # the reference's parameter checks (src/flaggems_vllm/ops/fused_moe.py:688-730): finite scalars, limit >= 0
        vals = []
        for name, value in (("gemm1_alpha", gemm1_alpha), ("gemm1_beta", gemm1_beta),
                            ("gemm1_clamp_limit", gemm1_clamp_limit)):
            if value is None or isinstance(value, bool) or not isinstance(value, (int, float)) \
                    or value != value or value in (float("inf"), float("-inf")):
                raise ValueError(f"swigluoai_uninterleave requires a finite scalar {name}, got {value!r}")
            vals.append(float(value))
        if vals[2] < 0:
            raise ValueError("swigluoai_uninterleave requires gemm1_clamp_limit >= 0")
        return (_lib.ACT_SWIGLUOAI, vals[0], vals[1], vals[2])
    if activation == "silu":
        if any(v is not None for v in (gemm1_alpha, gemm1_beta, gemm1_clamp_limit)):
            raise ValueError("gemm1_alpha/beta/clamp_limit require swigluoai_uninterleave")
        return (_lib.ACT_SILU, 0.0, 0.0, 0.0)
    raise ValueError(
        f"Only 'silu' and 'swigluoai_uninterleave' activations are supported, got {activation!r}")


SMALL_BLOCK_M = 8
_small_scratch = {}


def _small_eligible(mode, act_dtype, H, I, k) -> bool:
    if act_dtype not in (torch.bfloat16, torch.float16) or k > 32:
        return False
    if mode == _lib.MODE_HALF:
        return H % 128 == 0 and I % 64 == 0
    return H % 128 == 0 and I % 128 == 0


def _use_small_path(mode, act_dtype, H, I, numel, k) -> bool:
    """The weight-streaming split-K schedule serves the smallest decode batches.  Measured under
    CUDA-graph replay it beats the 128-row tensor-core tiles for half precision up to 8 routes
    per call (Mixtral shape, one token: 0.162 against 0.193 ms) and for weight-only int8 up to
    16 routes (Qwen3 shape, one token: 0.049 against 0.054 ms); for FP8 block scales the tile
    kernels stay ahead even at one token (0.103 against 0.135 ms), so FP8 uses it only when
    forced.  FLAGGEMS_B200_SMALL_M = 0/1 forces it off/on."""
    if numel == 0 or not _small_eligible(mode, act_dtype, H, I, k) or _force_generic():
        return False
    force = _policy("FLAGGEMS_B200_SMALL_M")
    if force != "auto":
        return force == "on" and numel <= 4096
    if mode == _lib.MODE_HALF:
        return numel <= 8
    if mode == _lib.MODE_W8A16:
        return numel <= 16
    return False


_sm_counts = {}


def _sm_count(dev) -> int:
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _sm_counts:
        _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_counts[idx]


def _small_counters(dev, n):
    """Zeroed int32 words the small-batch kernels count arrivals in.  Every launch leaves them
    zero, so one buffer per (device, stream) is zeroed once and reused."""
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    buf = _small_scratch.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=dev)
        _small_scratch[key] = buf
    return buf


def small_k_slices(mode, gemm1, K, N, blocks, sms) -> int:
    """K slices per tile of the small-batch schedule.  Every CTA takes a contiguous share of the
    (tile, slice) units, so a GEMM lasts ceil(units / SMs) units of (128-byte chunks per slice + a
    fixed cost); the slice count that minimises that product is asked for.  ``blocks`` = align
    blocks of 8 routes (one per routed expert for decode)."""
    chunk_elems = 64 if mode == _lib.MODE_HALF else 128   # K elements in 128 bytes of weights
    max_chunks = 16 if mode == _lib.MODE_W8A16 else 32    # what one unit holds of the activation rows
    unit_overhead = 4                                     # staging + epilogue of a unit, in chunk times
    nt = N // 64 if gemm1 else N // 128
    chunks = max(1, K // chunk_elems)
    best, hint = None, 1
    for S in range(-(-chunks // max_chunks), min(16, chunks) + 1):
        cps = -(-chunks // S)
        units = blocks * nt * -(-chunks // cps)
        cost = -(-units // sms) * (cps + unit_overhead)
        if best is None or cost < best:
            best, hint = cost, S
    return hint


def run_chunk_small(x, w1, w2, topk_weights, topk_ids, out, *, mode, w1_scale, w2_scale, global_num_experts,
                    expert_map, apply_router_weight_on_input, keep=None, mark=None):
    """One chunk on the small-batch schedule: align (blocks of 8 routes) -> GEMM1 -> GEMM2 with
    the top-k combine inside.  Three launches, no quantiser and no moe_sum pass."""
    if mark is None:
        mark = STAGE_HOOK or _no_mark
    L = _lib.lib()
    dev = x.device
    st = _lib.stream_of(x)
    status = _lib.status_word(dev)
    M, H = x.shape
    k = topk_ids.shape[1]
    E_local, N2, _ = w1.shape
    I = N2 // 2
    numel = M * k
    act_code = _lib.dtype_code(x.dtype)
    bm = SMALL_BLOCK_M
    rows_cap = round_up(numel + min(numel, global_num_experts) * (bm - 1), bm)
    sorted_ids = torch.empty(rows_cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(rows_cap // bm, dtype=torch.int32, device=dev)
    npp = torch.empty(1, dtype=torch.int32, device=dev)
    ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
    ids64 = int(ids.dtype == torch.int64)
    _lib.check(L.moe_align_block_size(ids.data_ptr(), ids64, numel, global_num_experts, bm, sorted_ids.data_ptr(),
                                      rows_cap, expert_ids.data_ptr(), expert_ids.numel(), npp.data_ptr(),
                                      status.data_ptr(), st))
    mark("align")
    emap = None
    if expert_map is not None:
        emap = expert_map if expert_map.dtype == torch.int32 else expert_map.to(torch.int32)
        emap = emap.contiguous()
    rw = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
    rw = rw if rw.is_contiguous() else rw.contiguous()
    blocks = max(1, min(numel, global_num_experts))  # exact for one token, an upper bound otherwise
    sms = _sm_count(dev)

    def plan(gemm1, K, N):
        hint = small_k_slices(mode, gemm1, K, N, blocks, sms)
        sizes = (ctypes.c_int64 * 3)()
        _lib.check(L.moe_small_m_plan(int(gemm1), mode, K, N, rows_cap, M, hint, ctypes.addressof(sizes),
                                      ctypes.addressof(sizes) + 8, ctypes.addressof(sizes) + 16))
        return hint, int(sizes[0]), int(sizes[1]), int(sizes[2])

    h1, part1, uc1, _ = plan(True, H, I)
    h2, part2, uc2, tc2 = plan(False, I, H)
    counters = _small_counters(dev, uc1 + uc2 + tc2)
    partial = torch.empty(max(part1, part2, 1), dtype=torch.float32, device=dev)
    act = torch.empty((rows_cap, I), dtype=x.dtype, device=dev)
    y = torch.empty((numel, H), dtype=x.dtype, device=dev)
    cptr = counters.data_ptr()
    _lib.check(L.moe_small_m_gemm(1, mode, act_code, x.data_ptr(), M, k, w1.data_ptr(), _lib.ptr(w1_scale),
                                  expert_ids.data_ptr(), sorted_ids.data_ptr(), npp.data_ptr(), _lib.ptr(emap),
                                  global_num_experts, rw.data_ptr(), int(apply_router_weight_on_input), ids.data_ptr(),
                                  ids64, rows_cap, E_local, H, I, act.data_ptr(), None, h1, partial.data_ptr(), cptr,
                                  None, status.data_ptr(), st))
    mark("gemm1")
    _lib.check(L.moe_small_m_gemm(0, mode, act_code, act.data_ptr(), M, k, w2.data_ptr(), _lib.ptr(w2_scale),
                                  expert_ids.data_ptr(), sorted_ids.data_ptr(), npp.data_ptr(), _lib.ptr(emap),
                                  global_num_experts, rw.data_ptr(), int(not apply_router_weight_on_input),
                                  ids.data_ptr(), ids64, rows_cap, E_local, I, H, y.data_ptr(), out.data_ptr(), h2,
                                  partial.data_ptr(), cptr + 4 * uc1, cptr + 4 * (uc1 + uc2), status.data_ptr(), st))
    mark("gemm2")
    if keep is not None:
        keep.update(sorted_ids=sorted_ids, expert_ids=expert_ids, num_post_pad=npp, act=act, y=y, block_m=bm,
                    rows_cap=rows_cap, used_tensor_cores=True, kernel="small")


def _widen_int8(w, dtype):
    out = torch.empty(w.shape, dtype=dtype, device=w.device)
    _lib.check(_lib.lib().moe_widen_int8(w.data_ptr(), out.data_ptr(), _lib.dtype_code(dtype), w.numel(),
                                         _lib.stream_of(w)))
    return out


def quantize_rows(x, mark=None):
    """FP8 mode: e4m3 rows [M, H] plus transposed 1x128 scales [H/128, M]."""
    M, H = x.shape
    q = torch.empty((M, H), dtype=torch.float8_e4m3fn, device=x.device)
    s_t = torch.empty((H // 128, M), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().moe_per_token_group_quant_fp8(x.data_ptr(), _lib.dtype_code(x.dtype), M, H, 128,
                                                        q.data_ptr(), s_t.data_ptr(), 1, M, _lib.stream_of(x)))
    return q, s_t


def route_pipeline(a_rows, a_scales_t, w1, w2, route_weight, topk_ids, *, mode, act_dtype, w1_scale, w2_scale,
                   global_num_experts, expert_map, apply_router_weight_on_input, use_tensor_cores=None,
                   keep=None, mark=None, act_fn=(0, 0.0, 0.0, 0.0), row_quant=None, column_halves=None):
    """align -> GEMM1 -> GEMM2 for ``a_rows`` [tokens, H] (activation dtype, or
    e4m3 with ``a_scales_t`` [H/128, tokens] in FP8 mode) and ``topk_ids``
    [tokens, k].  Returns ``(y, row_index)``: y holds one row per route in ``act_dtype``, already
    multiplied by the route weight (unless the weight was applied on the input).  With
    ``row_index`` None, y is [tokens * k, H] and row = flat route index; otherwise y is in
    sorted order [rows_cap, H] and ``row_index`` [tokens, k] names the row of every route.  Rows
    (and index entries) of routes whose expert is not local are left unwritten.  ``act_fn`` = (activation code, alpha, beta, limit).  Row-scaled W8A8 modes:
    ``a_rows`` is e4m3 / int8 with ``a_scales_t`` [tokens]; ``row_quant`` = (kind, static scale or
    None) says how the intermediate is quantised between the two GEMMs.
    ``column_halves`` = (callback, SMs to leave free): when GEMM2 writes sorted rows and H splits
    into two windows of whole 256-column tiles, GEMM2 runs once per window and
    ``callback(half, col0, y_window, row_index)`` is called after each launch (the second launch
    keeps off the given number of SMs); the function then returns ``(None, row_index)``."""
    if mark is None:
        mark = STAGE_HOOK or _no_mark
    L = _lib.lib()
    dev = a_rows.device
    st = _lib.stream_of(a_rows)
    status = _lib.status_word(dev)
    M, H = a_rows.shape
    k = topk_ids.shape[1]
    E_local, N2, _ = w1.shape
    I = N2 // 2
    numel = M * k
    act_code = _lib.dtype_code(act_dtype)
    if use_tensor_cores is None:
        kernel = _choose_kernel(mode, act_dtype, H, I, numel, global_num_experts)
        if act_fn[0] != _lib.ACT_SILU or mode in (_lib.MODE_FP8_ROW, _lib.MODE_INT8_ROW):
            # activations other than SiLU and the row-scaled W8A8 modes run on the generic kernel
            kernel = KERNEL_GENERIC
    else:
        kernel = int(use_tensor_cores)
    block_m = {KERNEL_GENERIC: GENERIC_BLOCK_M, KERNEL_TC: TC_BLOCK_M, KERNEL_TC_PAIR: TC_PAIR_BLOCK_M,
               KERNEL_TC_WIDE: TC_PAIR_BLOCK_M, KERNEL_TC_PAIR_WIDE: TC_PAIR_WIDE_BLOCK_M}[kernel]

    # every expert that owns at least one route pads by < block_m
    rows_cap = round_up(numel + min(numel, global_num_experts) * (block_m - 1), block_m)
    sorted_ids = torch.empty(rows_cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(rows_cap // block_m, dtype=torch.int32, device=dev)
    npp = torch.empty(1, dtype=torch.int32, device=dev)
    ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
    _lib.check(L.moe_align_block_size(ids.data_ptr(), int(ids.dtype == torch.int64), numel, global_num_experts,
                                      block_m, sorted_ids.data_ptr(), rows_cap, expert_ids.data_ptr(),
                                      expert_ids.numel(), npp.data_ptr(), status.data_ptr(), st))
    mark("align")
    if expert_map is not None:
        # same post-hoc lookup as the reference (moe_align_block_size.py:924-925);
        # unused blocks (-1) lie beyond num_tokens_post_padded and are never visited
        emap = expert_map if expert_map.dtype == torch.int32 else expert_map.to(torch.int32)
        _lib.check(L.moe_map_expert_ids(expert_ids.data_ptr(), expert_ids.numel(), emap.data_ptr(),
                                        emap.numel(), st))

    fp8 = mode == _lib.MODE_FP8_BLOCK
    row_scaled = mode in (_lib.MODE_FP8_ROW, _lib.MODE_INT8_ROW)
    if fp8:
        act = torch.empty((rows_cap, I), dtype=torch.float8_e4m3fn, device=dev)
        act_scales = torch.empty((I // 128, rows_cap), dtype=torch.float32, device=dev)
    else:
        act = torch.empty((rows_cap, I), dtype=act_dtype, device=dev)
        act_scales = None
    rw = route_weight if route_weight.dtype == torch.float32 else route_weight.float()
    rw = rw if rw.is_contiguous() else rw.contiguous()
    tc = kernel
    a_in, a_sorted, a_scales_in = a_rows, 0, a_scales_t
    if _presort_rows(mode, kernel, numel, global_num_experts):
        # many rows per expert: copy the token rows into sorted order once and let GEMM1 read
        # them with TMA boxes instead of gathering them inside the kernel
        a_in = torch.empty((rows_cap, H), dtype=a_rows.dtype, device=dev)
        _lib.check(L.moe_gather_rows(a_rows.data_ptr(), M, k, H * a_rows.element_size(), sorted_ids.data_ptr(),
                                     npp.data_ptr(), rows_cap, a_in.data_ptr(), st))
        if fp8:
            sc_in = torch.empty((H // 128, rows_cap), dtype=torch.float32, device=dev)
            _lib.check(L.moe_gather_scales_t(a_scales_t.data_ptr(), H // 128, M, k, sorted_ids.data_ptr(),
                                             npp.data_ptr(), rows_cap, sc_in.data_ptr(), st))
            a_scales_in = sc_in
        a_sorted = 1
        mark("gather")
    _lib.check(L.moe_gemm1_ex(mode, act_code, a_in.data_ptr(), a_sorted, _lib.ptr(a_scales_in), M, k, w1.data_ptr(),
                              _lib.ptr(w1_scale), expert_ids.data_ptr(), sorted_ids.data_ptr(), npp.data_ptr(),
                              rw.data_ptr(), int(apply_router_weight_on_input), rows_cap, block_m, E_local, H, I,
                              act.data_ptr(), _lib.ptr(act_scales), tc, act_fn[0], act_fn[1], act_fn[2], act_fn[3],
                              status.data_ptr(), st))
    mark("gemm1")
    act_in = act
    if row_scaled:
        # quantise the intermediate (sorted rows) the way the mode says: one scale per row, or one for
        # the whole tensor (dynamic: over the occupied rows only; padding rows hold stale bytes)
        kind, static = row_quant
        act_in = torch.empty((rows_cap, I), dtype=torch.int8 if mode == _lib.MODE_INT8_ROW else torch.float8_e4m3fn,
                             device=dev)
        per_row = kind in (0, 1)
        sc = torch.empty(rows_cap if per_row else 1, dtype=torch.float32, device=dev)
        _lib.check(L.moe_rowwise_quant(act.data_ptr(), act_code, rows_cap, I, kind, _lib.ptr(static),
                                       sorted_ids.data_ptr() if kind == 3 else None, numel, act_in.data_ptr(),
                                       sc.data_ptr(), st))
        act_scales = sc if per_row else sc.expand(rows_cap).contiguous()
        mark("quant2")
    row_index = None
    if _sorted_output(mode, kernel, numel, global_num_experts):
        # the 128-row kernel stages its output tile and writes whole tiles (TMA) in sorted row order;
        # the combine finds a route's row through `row_index`
        row_index = torch.empty((M, k), dtype=torch.int32, device=dev)
        if column_halves is not None and H % 512 == 0 and not (mode == _lib.MODE_HALF and w2_scale is not None):
            callback, free_sms = column_halves
            h0 = (H // 2) // 256 * 256
            for half, (c0, nc) in enumerate(((0, h0), (h0, H - h0))):
                y_w = torch.empty((rows_cap, nc), dtype=act_dtype, device=dev)
                limit = max(1, _sm_count(dev) - free_sms) if half == 1 and free_sms > 0 else 0
                _lib.check(L.moe_gemm2_sorted_cols(mode, act_code, act_in.data_ptr(), _lib.ptr(act_scales), w2.data_ptr(),
                                                   _lib.ptr(w2_scale), expert_ids.data_ptr(), sorted_ids.data_ptr(),
                                                   npp.data_ptr(), rw.data_ptr(), int(not apply_router_weight_on_input),
                                                   numel, rows_cap, block_m, E_local, H, I, c0, nc, y_w.data_ptr(),
                                                   row_index.data_ptr(), limit, status.data_ptr(), st))
                mark("gemm2")
                callback(half, c0, y_w, row_index)
            return None, row_index
        y = torch.empty((rows_cap, H), dtype=act_dtype, device=dev)
        _lib.check(L.moe_gemm2_sorted(mode, act_code, act_in.data_ptr(), _lib.ptr(act_scales), w2.data_ptr(),
                                      _lib.ptr(w2_scale), expert_ids.data_ptr(), sorted_ids.data_ptr(), npp.data_ptr(),
                                      rw.data_ptr(), int(not apply_router_weight_on_input), numel, rows_cap, block_m,
                                      E_local, H, I, y.data_ptr(), row_index.data_ptr(), status.data_ptr(), st))
    else:
        y = torch.empty((numel, H), dtype=act_dtype, device=dev)
        _lib.check(L.moe_gemm2(mode, act_code, act_in.data_ptr(), _lib.ptr(act_scales), w2.data_ptr(),
                               _lib.ptr(w2_scale), expert_ids.data_ptr(), sorted_ids.data_ptr(), npp.data_ptr(),
                               rw.data_ptr(), int(not apply_router_weight_on_input), numel, rows_cap, block_m, E_local,
                               H, I, y.data_ptr(), tc, status.data_ptr(), st))
    mark("gemm2")
    if keep is not None:
        keep.update(sorted_ids=sorted_ids, expert_ids=expert_ids, num_post_pad=npp, a_rows=a_rows,
                    a_scales_t=a_scales_t, act=act, act_scales_t=act_scales, y=y, block_m=block_m,
                    rows_cap=rows_cap, used_tensor_cores=kernel != KERNEL_GENERIC, kernel=kernel, row_index=row_index)
    return y, row_index


def combine_routes(y, out, topk_ids, global_num_experts, expert_map=None, row_index=None):
    """out[m] = fp32 sum, in fixed slot order, of the rows of token m.

    With ``topk_ids`` [M, k]: slot (m, j) is row m*k + j of ``y`` (or
    ``row_index[m, j]``), skipped when its expert id is negative, >= the expert
    count, or not local under ``expert_map``.  With ``topk_ids=None``:
    ``row_index`` [M, S] alone names the rows; negative entries are skipped.  ``out`` may be a
    column window of a wider tensor (rows ``out.stride(0)`` elements apart, columns contiguous)."""
    M, H = out.shape
    assert out.stride(1) == 1 or H == 1, "the columns of the output must be contiguous"
    ids = None
    if topk_ids is not None:
        k = topk_ids.shape[1]
        ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
    else:
        k = row_index.shape[1]
    emap = None
    if expert_map is not None:
        emap = expert_map if expert_map.dtype == torch.int32 else expert_map.to(torch.int32)
        emap = emap.contiguous()
    if row_index is not None:
        row_index = row_index.contiguous()
    _lib.check(_lib.lib().moe_sum_ld(y.data_ptr(), out.data_ptr(), out.stride(0) if M > 0 else H,
                                     _lib.dtype_code(out.dtype), M, k, H, _lib.ptr(ids),
                                     int(ids is not None and ids.dtype == torch.int64), global_num_experts,
                                     _lib.ptr(emap), _lib.ptr(row_index), _lib.stream_of(out)))


def run_chunk(x, w1, w2, topk_weights, topk_ids, out, *, mode, w1_scale, w2_scale, global_num_experts,
              expert_map, apply_router_weight_on_input, use_tensor_cores=None, keep=None, mark=None,
              act_fn=(0, 0.0, 0.0, 0.0), row_quant=None):
    """One chunk of the layer.  ``keep`` (a dict) receives the intermediates for
    tests; ``mark(name)`` is called after each stage has been enqueued (bench.py
    records CUDA events there)."""
    if mark is None:
        mark = STAGE_HOOK or _no_mark
    # (half-precision weights with per-channel scales -- the widened int8 experiment -- stay on the tile kernels)
    if use_tensor_cores is None and act_fn[0] == _lib.ACT_SILU and not (
            mode == _lib.MODE_HALF and w1_scale is not None) and _use_small_path(
            mode, x.dtype, x.shape[1], w1.shape[1] // 2, x.shape[0] * topk_ids.shape[1], topk_ids.shape[1]):
        run_chunk_small(x, w1, w2, topk_weights, topk_ids, out, mode=mode, w1_scale=w1_scale, w2_scale=w2_scale,
                        global_num_experts=global_num_experts, expert_map=expert_map,
                        apply_router_weight_on_input=apply_router_weight_on_input, keep=keep, mark=mark)
        return
    row_quant2 = None
    if mode == _lib.MODE_FP8_BLOCK:
        # activations are quantised once per token; the GEMM gathers rows by token
        a_rows, a_scales = quantize_rows(x)
    elif mode in (_lib.MODE_FP8_ROW, _lib.MODE_INT8_ROW):
        # row_quant = ((kind, static scale) of the input, (kind, static scale) of the intermediate)
        (kind, static), row_quant2 = row_quant
        M = x.shape[0]
        a_rows = torch.empty(x.shape, dtype=torch.int8 if mode == _lib.MODE_INT8_ROW else torch.float8_e4m3fn,
                             device=x.device)
        per_row = kind in (0, 1)
        sc = torch.empty(M if per_row else 1, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().moe_rowwise_quant(x.data_ptr(), _lib.dtype_code(x.dtype), M, x.shape[1], kind,
                                                _lib.ptr(static), None, 0, a_rows.data_ptr(), sc.data_ptr(),
                                                _lib.stream_of(x)))
        a_scales = sc if per_row else sc.expand(M).contiguous()
    else:
        a_rows, a_scales = x, None
    mark("quant")
    y, row_index = route_pipeline(a_rows, a_scales, w1, w2, topk_weights, topk_ids, mode=mode, act_dtype=x.dtype,
                       w1_scale=w1_scale, w2_scale=w2_scale, global_num_experts=global_num_experts,
                       expert_map=expert_map, apply_router_weight_on_input=apply_router_weight_on_input,
                       use_tensor_cores=use_tensor_cores, keep=keep, mark=mark, act_fn=act_fn, row_quant=row_quant2)
    combine_routes(y, out, topk_ids, global_num_experts, expert_map, row_index=row_index)
    mark("sum")


def fused_experts_impl(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    inplace: bool = False,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    use_int8_w8a8: bool = False,
    use_int8_w8a16: bool = False,
    use_int4_w4a16: bool = False,
    ocp_mx_scheme: str | None = None,
    per_channel_quant: bool = False,
    global_num_experts: int = -1,
    expert_map: torch.Tensor | None = None,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    w1_zp: torch.Tensor | None = None,
    w2_zp: torch.Tensor | None = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[list[int]] = None,
    w1_bias: Optional[torch.Tensor] = None,
    w2_bias: Optional[torch.Tensor] = None,
    *,
    gemm1_alpha: float | None = None,
    gemm1_beta: float | None = None,
    gemm1_clamp_limit: float | None = None,
) -> torch.Tensor:
    logger.debug("GEMS FUSED MOE")
    act = _check_activation(activation, gemm1_alpha, gemm1_beta, gemm1_clamp_limit)

    if ocp_mx_scheme is not None:
        if not (ocp_mx_scheme.startswith("w_mxfp4") or ocp_mx_scheme.startswith("w_mxfp6")):
            raise NotImplementedError(f"Unsupported ocp_mx_scheme={ocp_mx_scheme}")
        raise NotImplementedError("OCP MX weight formats are not implemented by the B200 kernels")
    assert hidden_states.size(1) == w1.size(2), f"Hidden size mismatch {hidden_states.size(1)} != {w1.size(2)}"
    assert topk_weights.size() == topk_ids.size(), "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.stride(-1) == 1, "Stride of last dimension must be 1"
    assert w2.stride(-1) == 1, "Stride of last dimension must be 1"
    assert hidden_states.dtype in [torch.float32, torch.float16, torch.bfloat16]

    if w1_zp is not None or w2_zp is not None:
        raise NotImplementedError("zero points are not implemented by the B200 kernels")
    if w1_bias is not None or w2_bias is not None:
        raise NotImplementedError("expert biases are not implemented by the B200 kernels")

    num_tokens = hidden_states.size(0)
    E, N, _ = w1.size()
    K = w2.size(1)
    assert N % 2 == 0 and w2.size(2) == N // 2 and w2.size(0) == E and K == hidden_states.size(1), \
        "w1/w2 shapes do not describe a gated MoE layer"
    if global_num_experts == -1:
        global_num_experts = E

    row_quant = None
    if use_fp8_w8a8 and block_shape is not None:
        if list(block_shape) != [128, 128]:
            raise NotImplementedError("FP8 block quantisation is implemented for block_shape=[128, 128] only")
        if per_channel_quant:
            raise NotImplementedError("per-token activation scales cannot be combined with block_shape")
        if a1_scale is not None or a2_scale is not None:
            raise NotImplementedError("static activation scales are not used with block_shape")
        assert w1.dtype == torch.float8_e4m3fn and w2.dtype == torch.float8_e4m3fn, "FP8 weights expected"
        assert w1_scale is not None and w2_scale is not None, "FP8 block scales expected"
        assert hidden_states.dtype != torch.float32, "FP8 path needs f16/bf16 activations"
        assert K % 128 == 0 and (N // 2) % 128 == 0, "FP8 block quantisation needs sizes divisible by 128"
        assert tuple(w1_scale.shape) == (E, ceil_div(N, 128), K // 128), "w1_scale shape"
        assert tuple(w2_scale.shape) == (E, K // 128, (N // 2) // 128), "w2_scale shape"
        mode = _lib.MODE_FP8_BLOCK
    elif use_fp8_w8a8 or use_int8_w8a8:
        # per-tensor or per-token/per-channel W8A8 (src/flaggems_vllm/ops/fused_moe.py:853-1010): the scales
        # multiply the finished dot products
        if use_int8_w8a8 and block_shape is not None:
            raise NotImplementedError("block-quantised INT8 W8A8 is not implemented")
        wdt = torch.float8_e4m3fn if use_fp8_w8a8 else torch.int8
        assert w1.dtype == wdt and w2.dtype == wdt, f"{wdt} weights expected"
        assert w1_scale is not None and w2_scale is not None, "weight scales expected"
        assert hidden_states.dtype != torch.float32, "W8A8 paths need f16/bf16 activations"
        mode = _lib.MODE_FP8_ROW if use_fp8_w8a8 else _lib.MODE_INT8_ROW
        if per_channel_quant:
            kinds = (1, 1) if use_fp8_w8a8 else (0, 0)
            statics = (None, None)
        elif use_fp8_w8a8:
            kinds = (2 if a1_scale is not None else 3, 2 if a2_scale is not None else 3)
            statics = (a1_scale, a2_scale)
        else:
            assert a1_scale is not None and a2_scale is not None, "int8 per-tensor requires A_scale"
            kinds, statics = (4, 4), (a1_scale, a2_scale)
        statics = tuple(None if t is None else t.to(torch.float32).reshape(-1)[:1].contiguous() for t in statics)
        row_quant = ((kinds[0], statics[0]), (kinds[1], statics[1]))
    elif use_int8_w8a16 or use_int4_w4a16:
        if block_shape is not None and len(block_shape) == 2 and block_shape[1] > 0:
            raise NotImplementedError("group-quantised weight-only formats are not implemented")
        assert w1.dtype == torch.int8 and w2.dtype == torch.int8, "INT8 weight containers expected"
        assert w1_scale is not None and w2_scale is not None, "per-channel weight scales expected"
        assert w1_scale.numel() == E * N and w2_scale.numel() == E * K, "per-channel scale shape"
        mode = _lib.MODE_W8A16
    else:
        assert w1.dtype == hidden_states.dtype and w2.dtype == hidden_states.dtype, \
            "weights must have the activation dtype"
        mode = _lib.MODE_HALF

    _lib.require_cuda(hidden_states, "fused_experts_impl")
    w1c = w1 if w1.is_contiguous() else w1.contiguous()
    w2c = w2 if w2.is_contiguous() else w2.contiguous()
    s1 = s2 = None
    if mode in (_lib.MODE_FP8_ROW, _lib.MODE_INT8_ROW):
        # one scale per output channel; a per-tensor scale ([E], [E, 1] or [E, 1, 1]) is that vector filled
        def per_channel(ws, rows):
            ws = ws.to(torch.float32).reshape(E, -1)
            assert ws.shape[1] in (1, rows), "weight scales must be per tensor or per output channel"
            return ws.expand(E, rows).contiguous()

        s1, s2 = per_channel(w1_scale, N), per_channel(w2_scale, K)
    elif mode != _lib.MODE_HALF:
        s1 = w1_scale.to(torch.float32).contiguous()
        s2 = w2_scale.to(torch.float32).contiguous()

    if (mode == _lib.MODE_W8A16 and os.environ.get("FLAGGEMS_B200_W8_WIDEN", "0") == "1" and not _force_generic()
            and _tc_eligible(_lib.MODE_HALF, hidden_states.dtype, K, N // 2)):
        # experiment switch: widen the int8 weights to the activation dtype in global memory
        # first (one extra pass over them per call) and run the half-precision kernels; the
        # default is the kernel that widens them in shared memory
        w1c, w2c = _widen_int8(w1c, hidden_states.dtype), _widen_int8(w2c, hidden_states.dtype)
        mode = _lib.MODE_HALF

    out_hidden_states = hidden_states if inplace else torch.empty_like(hidden_states)
    for chunk in range((num_tokens // CHUNK_SIZE) + 1):
        begin, end = chunk * CHUNK_SIZE, min((chunk + 1) * CHUNK_SIZE, num_tokens)
        if end - begin <= 0:
            break
        run_chunk(hidden_states[begin:end], w1c, w2c, topk_weights[begin:end], topk_ids[begin:end],
                  out_hidden_states[begin:end], mode=mode, w1_scale=s1, w2_scale=s2,
                  global_num_experts=global_num_experts, expert_map=expert_map,
                  apply_router_weight_on_input=apply_router_weight_on_input, act_fn=act, row_quant=row_quant)
    if os.environ.get("FLAGGEMS_B200_CHECK_STATUS", "0") == "1":
        # debugging aid (one device synchronisation per call): a kernel that gave up on a wait or met
        # corrupt routing data leaves the output undefined; say so instead of returning it
        st = _lib.read_status(hidden_states.device)
        if st != 0:
            raise _lib.MoeKernelError(f"fused_experts_impl: kernel status word = {st} "
                                      "(1 bad expert id, 2 wait timed out, 4 bad sorted row)")
    return out_hidden_states


def inplace_fused_experts(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    use_int8_w8a8: bool = False,
    use_int8_w8a16: bool = False,
    use_int4_w4a16: bool = False,
    per_channel_quant: bool = False,
    global_num_experts: int = -1,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[list[int]] = None,
    w1_bias: Optional[torch.Tensor] = None,
    w2_bias: Optional[torch.Tensor] = None,
    *,
    gemm1_alpha: float | None = None,
    gemm1_beta: float | None = None,
    gemm1_clamp_limit: float | None = None,
) -> None:
    """Writes the layer output into ``hidden_states``; returns None."""
    fused_experts_impl(
        hidden_states, w1, w2, topk_weights, topk_ids, inplace=True, activation=activation,
        apply_router_weight_on_input=apply_router_weight_on_input, use_fp8_w8a8=use_fp8_w8a8,
        use_int8_w8a8=use_int8_w8a8, use_int8_w8a16=use_int8_w8a16, use_int4_w4a16=use_int4_w4a16,
        per_channel_quant=per_channel_quant, global_num_experts=global_num_experts, w1_scale=w1_scale,
        w2_scale=w2_scale, a1_scale=a1_scale, a2_scale=a2_scale, block_shape=block_shape, w1_bias=w1_bias,
        w2_bias=w2_bias, gemm1_alpha=gemm1_alpha, gemm1_beta=gemm1_beta, gemm1_clamp_limit=gemm1_clamp_limit)


def outplace_fused_experts(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    use_int8_w8a8: bool = False,
    use_int8_w8a16: bool = False,
    use_int4_w4a16: bool = False,
    per_channel_quant: bool = False,
    global_num_experts: int = -1,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[list[int]] = None,
    w1_bias: Optional[torch.Tensor] = None,
    w2_bias: Optional[torch.Tensor] = None,
    *,
    gemm1_alpha: float | None = None,
    gemm1_beta: float | None = None,
    gemm1_clamp_limit: float | None = None,
) -> torch.Tensor:
    """Allocates and returns the layer output; ``hidden_states`` is left untouched."""
    return fused_experts_impl(
        hidden_states, w1, w2, topk_weights, topk_ids, inplace=False, activation=activation,
        apply_router_weight_on_input=apply_router_weight_on_input, use_fp8_w8a8=use_fp8_w8a8,
        use_int8_w8a8=use_int8_w8a8, use_int8_w8a16=use_int8_w8a16, use_int4_w4a16=use_int4_w4a16,
        per_channel_quant=per_channel_quant, global_num_experts=global_num_experts, w1_scale=w1_scale,
        w2_scale=w2_scale, a1_scale=a1_scale, a2_scale=a2_scale, block_shape=block_shape, w1_bias=w1_bias,
        w2_bias=w2_bias, gemm1_alpha=gemm1_alpha, gemm1_beta=gemm1_beta, gemm1_clamp_limit=gemm1_clamp_limit)

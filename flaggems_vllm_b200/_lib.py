"""ctypes binding of libmoe_sm100.so (the C ABI declared in include/moe_sm100.h).

There is no fallback: if the library is missing or a call is rejected, the
caller gets an exception."""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_uint64, c_void_p

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmoe_sm100.so")

MOE_F32, MOE_F16, MOE_BF16, MOE_FP8E4M3, MOE_INT8 = 0, 1, 2, 3, 4
MODE_HALF, MODE_FP8_BLOCK, MODE_W8A16, MODE_FP8_ROW, MODE_INT8_ROW = 0, 1, 2, 3, 4
ACT_SILU, ACT_SWIGLUOAI = 0, 1
ST_BAD_EXPERT_ID, ST_WAIT_TIMEOUT, ST_BAD_ROW = 1, 2, 4

_DTYPE_CODE = {torch.float32: MOE_F32, torch.float16: MOE_F16, torch.bfloat16: MOE_BF16}

SYMBOLS = {
    "moe_abi_version": (c_int, []),
    "moe_last_error": (c_char_p, []),
    "moe_set_wait_limit_ns": (c_uint64, [c_uint64]),
    "moe_debug_wait_timeout": (c_int, [c_void_p, c_uint64, c_void_p, c_void_p]),
    "moe_grouped_topk": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_void_p, c_int64, c_int,
                                 c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "moe_topk_route": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_float,
                               c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "moe_map_expert_ids": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p]),
    "moe_align_block_size": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p,
                                     c_int64, c_void_p, c_void_p, c_void_p]),
    "moe_per_token_group_quant_fp8": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p,
                                              c_int, c_int64, c_void_p]),
    "moe_per_token_group_quant_fp8_ex": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_float, c_int, c_void_p,
                                                 c_void_p, c_int, c_int64, c_void_p]),
    "moe_widen_int8": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p]),
    "moe_ep_plan": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "moe_ep_pack": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int64,
                            c_void_p, c_void_p, c_void_p]),
    "moe_ep_unpack": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                              c_void_p]),
    "moe_router_gemm": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "moe_router_gemm_grouped_topk": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p, c_int64, c_int, c_int,
                                             c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p]),
    "moe_gather_rows": (c_int, [c_void_p, c_int64, c_int, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "moe_gather_scales_t": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "moe_gemm1": (c_int, [c_int, c_int, c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p,
                          c_void_p, c_int, c_void_p, c_void_p]),
    "moe_gemm1_ex": (c_int, [c_int, c_int, c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p,
                             c_void_p, c_int, c_int, c_float, c_float, c_float, c_void_p, c_void_p]),
    "moe_rowwise_quant": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p,
                                  c_void_p, c_void_p]),
    "moe_gemm2": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int,
                          c_void_p, c_void_p]),
    "moe_small_m_plan": (c_int, [c_int, c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "moe_small_m_gemm": (c_int, [c_int, c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int64, c_int, c_int,
                                 c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "moe_small_m_gemm2_static": (c_int, [c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int64, c_int,
                                         c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "moe_gemm2_sorted_cols": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int,
                                      c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "moe_gemm2_sorted": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                 c_void_p, c_void_p]),
    "moe_sum": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int64, c_void_p, c_int, c_int, c_void_p,
                        c_void_p, c_void_p]),
    "moe_silu_and_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p]),
    "moe_silu_and_mul_grad": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p]),
    "moe_sum_ld": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int, c_int64, c_void_p, c_int, c_int, c_void_p,
                           c_void_p, c_void_p]),
}

_lib = None
_status = {}
# calls of entry points that enqueue a kernel (bench.py reports the count of its timed region)
LAUNCHES = 0
_NO_KERNEL = ("moe_abi_version", "moe_last_error", "moe_small_m_plan", "moe_set_wait_limit_ns")


class _Counted:
    """The library handle with a call counter in front of every kernel-launching entry point."""

    def __init__(self, handle):
        for name in SYMBOLS:
            fn = getattr(handle, name)
            setattr(self, name, fn if name in _NO_KERNEL else self._wrap(fn))

    @staticmethod
    def _wrap(fn):
        def call(*args):
            global LAUNCHES
            LAUNCHES += 1
            return fn(*args)

        return call


class MoeKernelError(RuntimeError):
    """A launch was rejected or failed; the message is the library's text."""


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA kernels have not been built "
                "(run `python -m flaggems_vllm_b200.build`). There is no CPU or Triton fallback."
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = _Counted(handle)
    return _lib


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise ValueError(f"Unsupported dtype: {dt}") from None


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(t: torch.Tensor, who: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{who}: tensors must live on a CUDA device (there is no CPU path)")


def status_word(device) -> torch.Tensor:
    """Per-device int32 word the kernels OR failure bits into."""
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status[key]


def read_status(device=None, clear: bool = True) -> int:
    """Synchronising read of the status word (0 = no kernel reported a problem)."""
    if device is None:
        device = torch.cuda.current_device()
    w = status_word(device)
    v = int(w.item())
    if clear and v:
        w.zero_()
    return v


def check(rc: int, exc=MoeKernelError) -> None:
    if rc != 0:
        msg = lib().moe_last_error().decode("utf-8", "replace")
        if rc in (-1, -2, -3, -5):
            raise ValueError(f"{msg} (code {rc})")
        raise exc(f"{msg} (code {rc})")

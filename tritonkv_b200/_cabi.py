"""ctypes binding of ``libtritonkv_b200.so`` (the C ABI declared in
``include/tritonkv_b200.h``).

The library is the only compute path of this package.  If it is missing or does
not load, every operation raises ``RuntimeError``: there is no fallback.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p, POINTER

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtritonkv_b200.so")

TKV_OK = 0
TKV_ERR_INVALID = 1
TKV_ERR_UNSUPPORTED = 2
TKV_ERR_CUDA = 3
TKV_ERR_ALIGN = 4

DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 0, 1, 2
FLAG_PARTIALS_ONLY = 1
FLAG_COMBINE = 2
FLAG_K_PER_CHANNEL = 4
KERNEL_FUSED_SPLIT, KERNEL_FP16_SPLIT = 0, 1
KERNEL_FUSED_SPLIT_KCHAN = 4

_TORCH_DTYPE = {torch.float16: DTYPE_F16, torch.bfloat16: DTYPE_BF16, torch.float32: DTYPE_F32}

# Every symbol include/tritonkv_b200.h declares: (restype, argtypes).
SIGNATURES = {
    "tkv_version": (c_int, []),
    "tkv_last_error": (c_char_p, []),
    "tkv_device_info": (c_int, [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "tkv_kernel_attrs": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int),
                                 POINTER(c_int), POINTER(c_int)]),
    "tkv_pack_codes": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "tkv_unpack_codes": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "tkv_quantize_pack": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                  c_int, c_int, c_void_p]),
    "tkv_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
                               c_int, c_void_p]),
    "tkv_fused_decode": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                 c_void_p, c_int, c_void_p]),
    "tkv_fp16_decode": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                c_int, c_void_p, c_int, c_void_p]),
    "tkv_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                            c_int, c_int, c_int, c_void_p]),
    "tkv_combine_strided": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int64, c_int, c_int, c_int64, c_int64, c_int64, c_int64,
                                    c_void_p]),
    "tkv_wave_programs": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_int)]),
    "tkv_decode_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_int, POINTER(c_int), POINTER(c_int)]),
    "tkv_device_status": (c_int, [POINTER(c_int)]),
    "tkv_device_status_clear": (c_int, []),
    "tkv_quantize_append": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                    c_int64, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "tkv_combine_push": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_int64,
                                 c_int64, c_int64, POINTER(c_void_p), c_void_p, c_int, c_int, c_int,
                                 c_void_p]),
    "tkv_merge_wait": (c_int, [c_void_p, c_int64, c_int, POINTER(c_void_p), c_void_p, c_int, c_int,
                               c_int, c_void_p]),
    "tkv_quantize_keys_per_channel": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                              c_int64, c_int64, c_int, c_int, c_void_p]),
    "tkv_combine_exchange": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                     c_int64, c_int64, c_int64, c_int64, POINTER(c_void_p), c_void_p,
                                     c_int, c_int, c_int, c_void_p]),
    "tkv_fused_decode_static": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_float, c_void_p]),
}

_lib = None
_load_error: Exception | None = None


def load():
    """Return the loaded library, or raise ``RuntimeError`` (never falls back)."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if _load_error is None:
        try:
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
            return _lib
        except Exception as exc:  # missing file, missing symbol, loader error
            _load_error = exc
    raise RuntimeError(
        f"tritonkv_b200: CUDA library {LIB_PATH} is not available ({_load_error!r}); "
        "build it with `python -m tritonkv_b200.build`. There is no CPU or PyTorch fallback."
    )


_available_ok: tuple[bool, str] | None = None


def available() -> tuple[bool, str]:
    """(usable, why): the library loads and a CUDA device is present."""
    global _available_ok
    if _available_ok is not None:
        return _available_ok
    r = _available()
    if r[0]:
        _available_ok = r  # a positive answer does not change during the process
    return r


def _available() -> tuple[bool, str]:
    try:
        lib = load()
    except RuntimeError as exc:
        return False, str(exc)
    if not torch.cuda.is_available():
        return False, "torch.cuda.is_available() is False"
    return True, f"tritonkv_b200 {lib.tkv_version()} (CUDA sm_100a, C ABI)"


def last_error() -> str:
    return load().tkv_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Map a C-ABI status to the exception type the reference raises."""
    if status == TKV_OK:
        return
    msg = last_error()
    if status in (TKV_ERR_INVALID, TKV_ERR_UNSUPPORTED, TKV_ERR_ALIGN):
        raise ValueError(msg)
    raise RuntimeError(msg)


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _TORCH_DTYPE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float16, bfloat16 or float32") from None


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"tritonkv_b200: {what} must be a CUDA tensor (got device {t.device}); "
            "this package has no CPU path"
        )


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device: torch.device) -> int:
    """Handle of torch's current stream on ``device`` (the raw getter when torch has it:
    the Stream object costs microseconds per call)."""
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


_current_device = getattr(torch._C, "_cuda_getDevice", None) or torch.cuda.current_device


class on_device:
    """``with on_device(dev):`` makes ``dev`` current for the C-ABI calls inside; when it
    already is (the common case) this costs one integer compare instead of a device switch."""

    __slots__ = ("idx", "prev")

    def __init__(self, device: torch.device):
        self.idx = device.index if device.index is not None else _current_device()
        self.prev = -1

    def __enter__(self):
        cur = _current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def device_info(device: int | None = None) -> dict:
    lib = load()
    if device is None:
        device = torch.cuda.current_device()
    vals = [c_int(0) for _ in range(4)]
    check(lib.tkv_device_info(device, *[ctypes.byref(v) for v in vals]))
    return {"sm_count": vals[0].value, "l2_bytes": vals[1].value,
            "cc": (vals[2].value, vals[3].value)}


def kernel_attrs(kernel_id: int, nbits: int, D: int, gs: int) -> dict:
    lib = load()
    vals = [c_int(0) for _ in range(4)]
    check(lib.tkv_kernel_attrs(kernel_id, nbits, D, gs, *[ctypes.byref(v) for v in vals]))
    return {"regs": vals[0].value, "smem_bytes": vals[1].value, "local_bytes": vals[2].value,
            "ctas_per_sm": vals[3].value}


def device_status_clear() -> None:
    check(load().tkv_device_status_clear())


def device_status() -> int:
    """0 = ok; bit 0 = a bounded wait inside a decode kernel gave up, bit 1 = a bounded wait
    for a peer's data in the cross-GPU merge gave up (synchronises)."""
    v = c_int(0)
    check(load().tkv_device_status(ctypes.byref(v)))
    return v.value


_plan_cache: dict = {}


def decode_plan(kernel_id: int, nbits: int, D: int, gs: int, B: int, HQ: int, HKV: int, S: int,
                num_splits: int, split_size: int, ragged: bool) -> tuple[int, int]:
    """(nslots, grid): partial slots per (batch, head) and CTAs of the split kernel."""
    key = (kernel_id, nbits, D, gs, B, HQ, HKV, S, num_splits, split_size, ragged,
           _current_device())
    r = _plan_cache.get(key)
    if r is None:
        ns, grid = c_int(0), c_int(0)
        check(load().tkv_decode_plan(kernel_id, nbits, D, gs, B, HQ, HKV, S, num_splits, split_size,
                                     1 if ragged else 0, ctypes.byref(ns), ctypes.byref(grid)))
        r = (ns.value, grid.value)
        if len(_plan_cache) < 4096:
            _plan_cache[key] = r
    return r


_wave_cache: dict = {}


def wave_programs(kernel_id: int, nbits: int, D: int, gs: int) -> int:
    key = (kernel_id, nbits, D, gs, torch.cuda.current_device())
    if key not in _wave_cache:
        v = c_int(0)
        check(load().tkv_wave_programs(kernel_id, nbits, D, gs, ctypes.byref(v)))
        _wave_cache[key] = v.value
    return _wave_cache[key]

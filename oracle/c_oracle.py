"""ctypes wrapper of ``libtkv_oracle.so`` (built from ``tkv_oracle.c`` by the
Makefile beside it).  TEST INFRASTRUCTURE ONLY: the C twin of ``tkv_oracle.py``,
used for parity cases too large for numpy and as the timed CPU baseline."""

from __future__ import annotations

import ctypes
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libtkv_oracle.so")
_lib = None


def load():
    global _lib
    if _lib is None:
        src = os.path.join(_HERE, "tkv_oracle.c")
        if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
            subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)
        lib = ctypes.CDLL(_LIB)
        lib.tkvo_num_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def num_threads() -> int:
    return load().tkvo_num_threads()


def use_all_cores() -> int:
    """Use every host core the process may run on, whatever OMP_NUM_THREADS says."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    load().tkvo_set_num_threads(n)
    return num_threads()


def pack_codes(codes, nbits):
    codes = np.ascontiguousarray(codes, np.uint8)
    D = codes.shape[-1]
    out = np.empty(codes.shape[:-1] + (D * nbits // 8,), np.uint8)
    load().tkvo_pack_codes(_p(codes), _p(out), ctypes.c_int64(codes.size // D), D, nbits)
    return out


def unpack_codes(packed, nbits, D):
    packed = np.ascontiguousarray(packed, np.uint8)
    out = np.empty(packed.shape[:-1] + (D,), np.uint8)
    load().tkvo_unpack_codes(_p(packed), _p(out), ctypes.c_int64(out.size // D), D, nbits)
    return out


def quantize_groupwise(x, nbits, gs):
    x = np.ascontiguousarray(x, np.float32)
    D = x.shape[-1]
    rows = x.size // D
    packed = np.empty(x.shape[:-1] + (D * nbits // 8,), np.uint8)
    scale = np.empty(x.shape[:-1] + (D // gs,), np.uint16)
    zero = np.empty_like(scale)
    load().tkvo_quantize_groupwise(_p(x), _p(packed), _p(scale), _p(zero), ctypes.c_int64(rows), D,
                                   nbits, gs)
    return packed, scale, zero


def dequantize_groupwise(packed, scale, zero, nbits, gs, D):
    packed = np.ascontiguousarray(packed, np.uint8)
    scale = np.ascontiguousarray(scale).view(np.uint16)
    zero = np.ascontiguousarray(zero).view(np.uint16)
    out = np.empty(packed.shape[:-1] + (D,), np.float32)
    load().tkvo_dequantize_groupwise(_p(packed), _p(scale), _p(zero), _p(out),
                                     ctypes.c_int64(out.size // D), D, nbits, gs)
    return out


class DecodeStep:
    """Preallocated work buffers for repeated timing of one decode step."""

    def __init__(self, B, HQ, HKV, S, D, nbits, gs):
        self.dims = (B, HQ, HKV, S, D, nbits, gs)
        self.work = np.empty(2 * B * HKV * S * D + B * HQ * S, np.float32)
        self.out = np.empty((B, HQ, D), np.float32)

    def __call__(self, q, kp, ks, kz, vp, vs, vz, sm_scale=None, seq_lens=None):
        B, HQ, HKV, S, D, nbits, gs = self.dims
        sm_scale = 1.0 / math.sqrt(D) if sm_scale is None else sm_scale
        sl = None if seq_lens is None else _p(np.ascontiguousarray(seq_lens, np.int32))
        load().tkvo_decode_step(_p(q), _p(kp), _p(ks), _p(kz), _p(vp), _p(vs), _p(vz), _p(self.out),
                                _p(self.work), B, HQ, HKV, S, D, nbits, gs,
                                ctypes.c_float(sm_scale), sl)
        return self.out


def decode_step(q, kp, ks, kz, vp, vs, vz, nbits, gs, sm_scale=None, seq_lens=None):
    q = np.ascontiguousarray(q, np.float32)
    B, HQ, D = q.shape
    _, HKV, S, _ = kp.shape
    arrs = [np.ascontiguousarray(a) for a in (kp, ks, kz, vp, vs, vz)]
    arrs = [a if a.dtype == np.uint8 else a.view(np.uint16) for a in arrs]
    return DecodeStep(B, HQ, HKV, S, D, nbits, gs)(q, *arrs, sm_scale=sm_scale,
                                                   seq_lens=seq_lens).copy()

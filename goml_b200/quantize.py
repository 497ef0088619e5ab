"""Host binding of libfp8quant.so (per-tensor FP32 -> e4m3 quantiser).

``QuantizeF32ToF8E4M3(src, dst, scale, amax, n)`` and
``QuantizeF32ToF8E4M3Unit(...)`` carry the names and argument order of the calls
goml's attention chain makes (internal/abjexam/battle_a_llm.go:476-494): raw
device pointers for the FP32 source, the code buffer, one-float scale and amax
buffers, and the element count.  The first uses ``scale = amax/448``
(libs1/fp8_quantize_v2.cu:91), the second ``scale = amax``.
"""
from __future__ import annotations

import ctypes as C
import threading

from . import loader

AMAX_OVER_448 = 0
UNIT = 1

_lock = threading.Lock()
_lib = None


class QuantizeError(RuntimeError):
    pass


def _init():
    global _lib
    with _lock:
        if _lib is None:
            lib = loader.dlopen(loader.resolve_lib("libfp8quant.so"))
            lib.fp8_quantize_f32.restype = C.c_int
            lib.fp8_quantize_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
            lib.fp8_dequantize_to_fp16.restype = C.c_int
            lib.fp8_dequantize_to_fp16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
            lib.fp8_quantize_fp16.restype = C.c_int
            lib.fp8_quantize_fp16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
            lib.cuda_device_sync2.restype = C.c_int
            lib.fp8_quantize_mx_f32.restype = C.c_int
            lib.fp8_quantize_mx_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
            _lib = lib
    return _lib


def QuantizeF32ToF8E4M3(src: int, dst: int, scale: int, amax: int, n: int, stream: int = 0) -> None:
    rc = _init().fp8_quantize_f32(src, dst, scale, amax, n, AMAX_OVER_448, stream or None)
    if rc != 0:
        raise QuantizeError(f"fp8_quantize_f32: CUDA error {rc}")


def QuantizeF32ToF8E4M3Unit(src: int, dst: int, scale: int, amax: int, n: int, stream: int = 0) -> None:
    rc = _init().fp8_quantize_f32(src, dst, scale, amax, n, UNIT, stream or None)
    if rc != 0:
        raise QuantizeError(f"fp8_quantize_f32: CUDA error {rc}")


def DequantizeToFP16(src: int, dst: int, scale: int, n: int) -> None:
    rc = _init().fp8_dequantize_to_fp16(src, dst, scale, n)
    if rc != 0:
        raise QuantizeError(f"fp8_dequantize_to_fp16: CUDA error {rc}")


def QuantizeFP16(src: int, dst: int, scale: int, n: int) -> None:
    """fp8_quantize_fp16 of libs1/fp8_quantize_v2.cu:176-204: FP16 source, scale = amax/448, default stream."""
    rc = _init().fp8_quantize_fp16(src, dst, scale, n)
    if rc != 0:
        raise QuantizeError(f"fp8_quantize_fp16: CUDA error {rc}")


def DeviceSync2() -> None:
    rc = _init().cuda_device_sync2()
    if rc != 0:
        raise QuantizeError(f"cuda_device_sync2: CUDA error {rc}")


def mx_scale_bytes(rows: int, K: int) -> int:
    """Size of the tiled ue8m0 scale array of a [rows, K] block-scaled tensor (one scale per 32 elements along K)."""
    return ((rows + 127) // 128) * ((K + 127) // 128) * 512


def QuantizeMXF32(src: int, codes: int, scales: int, rows: int, K: int, stream: int = 0) -> None:
    """[rows, K] fp32 -> e4m3 codes + ue8m0 block scales (fp8_quantize_mx_f32), the operand format of FP8GEMMMX."""
    rc = _init().fp8_quantize_mx_f32(src, codes, scales, rows, K, stream or None)
    if rc != 0:
        raise QuantizeError(f"fp8_quantize_mx_f32: CUDA error {rc}")

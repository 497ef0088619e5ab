"""Host binding of libfp8gemm.so, mirroring goml's backend/cuda/fp8_gemm.go.

``FP8GEMM(M, N, K, A, B, C, mode, stream)`` has the argument meaning of
``cuda.FP8GEMM`` (backend/cuda/fp8_gemm.go:52-62): raw device pointers as
integers, ``mode`` 0/1, ``stream`` a CUDA stream handle or 0, and a non-zero
return code raised as ``"fp8_gemm: CUDA error %d"``.  ``FP8GEMMScaled`` binds
the additive extension (dequantising alpha, BF16 output).
"""
from __future__ import annotations

import ctypes as C
import threading

from . import loader

ModeOriginal = 0
ModeSinglesync = 1
OutFP16 = 0
OutBF16 = 1


class FP8GEMMError(RuntimeError):
    pass


_state = {"lib": None, "err": None}
_once = threading.Lock()


def _init():
    """sync.Once-style load of libfp8gemm.so (backend/cuda/fp8_gemm.go:27-41)."""
    with _once:
        if _state["lib"] is None and _state["err"] is None:
            try:
                lib = loader.dlopen(loader.resolve_lib("libfp8gemm.so"), global_symbols=True)
                i, p, f = C.c_int, C.c_void_p, C.c_float
                lib.fp8_gemm.restype = i
                lib.fp8_gemm.argtypes = [i, i, i, p, p, p, i, p]
                for name in ("fp8_gemm_original", "fp8_gemm_singlesync"):
                    fn = getattr(lib, name)
                    fn.restype = i
                    fn.argtypes = [i, i, i, p, p, p, p]
                lib.fp8_gemm_scaled.restype = i
                lib.fp8_gemm_scaled.argtypes = [i, i, i, p, p, p, f, p, p, i, p]
                lib.fp8_gemm_accumulate_f32.restype = i
                lib.fp8_gemm_accumulate_f32.argtypes = [i, i, i, p, p, p, f, p, p, p]
                lib.fp8_gemm_swiglu.restype = i
                lib.fp8_gemm_swiglu.argtypes = [i, i, i, p, p, p, f, p, p, p, p]
                lib.fp8_gemm_fp8out.restype = i
                lib.fp8_gemm_fp8out.argtypes = [i, i, i, p, p, p, f, p, p, p, p, p]
                lib.fp8_gemm_device_status.restype = i
                lib.fp8_gemm_mx.restype = i
                lib.fp8_gemm_mx.argtypes = [i, i, i, p, p, p, p, p, f, i, p]
                lib.fp8_mx_scale_bytes.restype = C.c_size_t
                lib.fp8_mx_scale_bytes.argtypes = [i, i]
                lib.fp8_gemm_mx_device_status.restype = i
                lib.fp8_gemm_selftest_wait_expiry.restype = i
                lib.fp8_gemm_selftest_wait_expiry.argtypes = [p]
                lib.fp8_gemm_set_tile_pairs.restype = i
                lib.fp8_gemm_set_tile_pairs.argtypes = [i]
                lib.fp8_gemm_version.restype = C.c_char_p
                _state["lib"] = lib
            except OSError as e:
                _state["err"] = e
    if _state["err"] is not None:
        raise _state["err"]
    return _state["lib"]


def FP8GEMM(M: int, N: int, K: int, A: int, B: int, Cptr: int, mode: int = ModeSinglesync, stream: int = 0) -> None:
    """C[M,N] (fp16) = A[M,K] x B[N,K]^T on e4m3 device buffers."""
    rc = _init().fp8_gemm(M, N, K, A, B, Cptr, mode, stream)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm: CUDA error {rc}")


def FP8GEMMOriginal(M, N, K, A, B, Cptr, stream=0) -> None:
    rc = _init().fp8_gemm_original(M, N, K, A, B, Cptr, stream)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm: CUDA error {rc}")


def FP8GEMMSinglesync(M, N, K, A, B, Cptr, stream=0) -> None:
    rc = _init().fp8_gemm_singlesync(M, N, K, A, B, Cptr, stream)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm: CUDA error {rc}")


def FP8GEMMScaled(M, N, K, A, B, Cptr, alpha=1.0, scale_a=0, scale_b=0, out_dtype=OutBF16, stream=0) -> None:
    """C = alpha * (*scale_a) * (*scale_b) * A x B^T; scale pointers are device pointers or 0."""
    rc = _init().fp8_gemm_scaled(M, N, K, A, B, Cptr, alpha, scale_a or None, scale_b or None, out_dtype, stream)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm_scaled: CUDA error {rc}")


def FP8GEMMAccumulateF32(M, N, K, A, B, X, alpha=1.0, scale_a=0, scale_b=0, stream=0) -> None:
    """X (fp32 [M, N]) += alpha * (*scale_a) * (*scale_b) * A x B^T: the residual update in the GEMM epilogue."""
    rc = _init().fp8_gemm_accumulate_f32(M, N, K, A, B, X, alpha, scale_a or None, scale_b or None, stream or None)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm_accumulate_f32: CUDA error {rc}")


def FP8GEMMSwiGLU(M, F, K, A, B_interleaved, H, alpha=1.0, scale_a=0, scale_b=0, amax_out=0, stream=0) -> None:
    """H (bf16 [M, F]) = silu(g) * u with [g | u] = alpha * sa * sb * A x B_interleaved^T; max|H| -> *amax_out."""
    rc = _init().fp8_gemm_swiglu(M, F, K, A, B_interleaved, H, alpha, scale_a or None, scale_b or None, amax_out, stream or None)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm_swiglu: CUDA error {rc}")


def FP8GEMMFP8Out(M, N, K, A, B, D, alpha=1.0, scale_a=0, scale_b=0, scale_d=0, amax_d=0, stream=0) -> None:
    """D (e4m3 [M, N]) = e4m3((*scale_d) * v), v = alpha * sa * sb * A x B^T; max|v| -> *amax_d (0 = not wanted).
    The delayed-scaling epilogue of fp8_matmul_fp8out (libs1/cublas_lt_wrapper_v3.c:220-229)."""
    rc = _init().fp8_gemm_fp8out(M, N, K, A, B, D, alpha, scale_a or None, scale_b or None, scale_d or None,
                                 amax_d or None, stream or None)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm_fp8out: CUDA error {rc}")


def interleave_gate_up(w_gate_up, F: int):
    """[2F, K] (gate rows first) -> the [2*Fp, K] layout fp8_gemm_swiglu reads (Fp = F rounded up to 32): per 32
    feed-forward columns, the 32 gate rows followed by the 32 up rows; rows past F are zero.  Works on torch tensors
    and numpy arrays."""
    Fp = (F + 31) // 32 * 32
    K = w_gate_up.shape[1]
    gate, up = w_gate_up[:F], w_gate_up[F:2 * F]
    if hasattr(w_gate_up, "new_zeros"):
        out = w_gate_up.new_zeros((Fp // 32, 2, 32, K))
    else:
        out = __import__("numpy").zeros((Fp // 32, 2, 32, K), w_gate_up.dtype)
    full = F // 32
    if full:
        out[:full, 0] = gate[:32 * full].reshape(full, 32, K)
        out[:full, 1] = up[:32 * full].reshape(full, 32, K)
    if F % 32:
        out[full, 0, :F % 32] = gate[32 * full:]
        out[full, 1, :F % 32] = up[32 * full:]
    return out.reshape(2 * Fp, K)


def SetTilePairs(mode: int) -> None:
    """-1 = tile pairs chosen per problem (default), 0 = single tiles only; results are bit-identical."""
    rc = _init().fp8_gemm_set_tile_pairs(mode)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm_set_tile_pairs: CUDA error {rc}")


def FP8GEMMMX(M, N, K, A, scale_a, B, scale_b, Cptr, alpha=1.0, out_dtype=OutBF16, stream=0) -> None:
    """Block-scaled GEMM: e4m3 codes with one ue8m0 scale per 32 K elements of every row of A and of B (the arrays
    fp8_quantize_mx_f32 writes); C = alpha * sum_kb 2^(ea+eb) A_kb . B_kb, fp32 accumulation, fp16/bf16 out."""
    rc = _init().fp8_gemm_mx(M, N, K, A, scale_a, B, scale_b, Cptr, alpha, out_dtype, stream or None)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm_mx: CUDA error {rc}")


def mx_device_status() -> int:
    return _init().fp8_gemm_mx_device_status()


def SelftestWaitExpiry(stream: int = 0) -> None:
    """Launch the one-warp kernel whose bounded wait runs out; the next device_status() then returns 0x1F0."""
    rc = _init().fp8_gemm_selftest_wait_expiry(stream or None)
    if rc != 0:
        raise FP8GEMMError(f"fp8_gemm_selftest_wait_expiry: CUDA error {rc}")


def device_status() -> int:
    return _init().fp8_gemm_device_status()


def version() -> str:
    return _init().fp8_gemm_version().decode()

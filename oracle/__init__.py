"""CPU oracle for the FP8 attention-forward / FP8 GEMM / FP8 quantiser path.

TEST INFRASTRUCTURE ONLY.  This package is the checker (and the timed CPU
baseline); the product package never imports it.  It wraps

* ``liboracle.so`` — the C restatement in ``oracle.c`` (each function there
  cites the reference file:line it follows), and
* ``_ref/libref_*.so`` — the reference's own host CPU code compiled from the
  reference tree by ``oracle/Makefile`` (present only where that tree was
  available at build time).
"""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)


def reference_root() -> str:
    """Where the reference tree lies, or "" when it is not on this machine: $GOML_REFERENCE, else the
    ``reference_path`` entry of BASELINE.json at the repository root."""
    cand = os.environ.get("GOML_REFERENCE", "")
    if not cand:
        try:
            import json
            with open(os.path.join(os.path.dirname(_HERE), "BASELINE.json")) as f:
                cand = json.load(f).get("reference_path", "")
        except (OSError, ValueError):
            cand = ""
    return cand if cand and os.path.isdir(os.path.join(cand, "libs")) else ""


def build(ref: bool = True) -> None:
    """Compile liboracle.so (and oracle/_ref when the reference tree is there)."""
    root = reference_root() if ref else ""
    target = "all" if root else os.path.join(_HERE, "liboracle.so")
    cmd = ["make", "-C", _HERE, target] + ([f"REF={root}"] if root else [])
    subprocess.run(cmd, check=True, capture_output=True)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build(ref=False)
        L = C.CDLL(path)
        L.oracle_e4m3_decode.restype = C.c_float
        L.oracle_e4m3_decode.argtypes = [C.c_uint8]
        L.oracle_e4m3_encode.restype = C.c_uint8
        L.oracle_e4m3_encode.argtypes = [C.c_float]
        L.oracle_e4m3_decode_n.argtypes = [_u8p, _f32p, C.c_size_t]
        L.oracle_e4m3_encode_n.argtypes = [_f32p, _u8p, C.c_size_t]
        L.oracle_quantize_f32.argtypes = [_f32p, _u8p, _f32p, _f32p, C.c_size_t, C.c_int]
        L.oracle_attention_f64.argtypes = [_u8p, _u8p, _u8p, _f64p, _f64p] + [C.c_int] * 5 + [C.c_double] * 2
        L.oracle_attention_f64_rows.argtypes = [_u8p, _u8p, _u8p, _f64p, _f64p] + [C.c_int] * 5 + [C.c_double] * 2 + [C.c_int] * 2
        L.oracle_attention_f32.argtypes = [_u8p, _u8p, _u8p, _f32p] + [C.c_int] * 5 + [C.c_float, C.c_int]
        L.oracle_gemm_f64.argtypes = [_u8p, _u8p, _f64p, C.c_int, C.c_int, C.c_int, C.c_double]
        L.oracle_gemm_f32.argtypes = [_u8p, _u8p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.oracle_harness_attention_inputs.argtypes = [_u8p, _u8p, _u8p, C.c_size_t]
        L.oracle_harness_gemm_inputs.argtypes = [_u8p, C.c_size_t, _u8p, C.c_size_t]
        L.oracle_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint8)
    return a


# ----------------------------------------------------------------------- e4m3

def e4m3_decode(codes) -> np.ndarray:
    codes = _u8(codes)
    out = np.empty(codes.shape, np.float32)
    lib().oracle_e4m3_decode_n(_p(codes, _u8p), _p(out, _f32p), codes.size)
    return out


def e4m3_encode(x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint8)
    lib().oracle_e4m3_encode_n(_p(x, _f32p), _p(out, _u8p), x.size)
    return out


def quantize_f32(x, convention: int = 0):
    """Per-tensor quantiser. Returns (codes u8, scale f32, amax f32).

    convention 0: scale = amax/448 (reference quantiser); 1: scale = amax.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.empty(x.shape, np.uint8)
    scale = C.c_float()
    amax = C.c_float()
    lib().oracle_quantize_f32(_p(x, _f32p), _p(q, _u8p), C.byref(scale), C.byref(amax), x.size, convention)
    return q, np.float32(scale.value), np.float32(amax.value)


# ------------------------------------------------------------------ attention

def attention_f64(q, k, v, causal=0, window=0, scale=None, v_descale=1.0, want_lse=True):
    """FP64 attention on e4m3 codes [bh, sl, hd] -> (O f64, LSE f64 or None)."""
    q, k, v = _u8(q), _u8(k), _u8(v)
    bh, sl, hd = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(hd)
    o = np.empty((bh, sl, hd), np.float64)
    lse = np.empty((bh, sl), np.float64) if want_lse else None
    lib().oracle_attention_f64(_p(q, _u8p), _p(k, _u8p), _p(v, _u8p), _p(o, _f64p),
                               _p(lse, _f64p) if want_lse else None,
                               bh, sl, hd, int(causal), int(window), float(scale), float(v_descale))
    return o, lse


def attention_f64_rows(q, k, v, q_begin, q_end, causal=0, window=0, scale=None, v_descale=1.0):
    """FP64 attention for query rows [q_begin, q_end) of every head."""
    q, k, v = _u8(q), _u8(k), _u8(v)
    bh, sl, hd = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(hd)
    nq = q_end - q_begin
    o = np.empty((bh, nq, hd), np.float64)
    lse = np.empty((bh, nq), np.float64)
    lib().oracle_attention_f64_rows(_p(q, _u8p), _p(k, _u8p), _p(v, _u8p), _p(o, _f64p), _p(lse, _f64p),
                                    bh, sl, hd, int(causal), int(window), float(scale), float(v_descale),
                                    int(q_begin), int(q_end))
    return o, lse


def attention_f32(q, k, v, causal=0, window=0, scale=None, parallel=False):
    """FP32 attention with the arithmetic of the reference's CPU loops."""
    q, k, v = _u8(q), _u8(k), _u8(v)
    bh, sl, hd = q.shape
    if scale is None:
        scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    o = np.empty((bh, sl, hd), np.float32)
    lib().oracle_attention_f32(_p(q, _u8p), _p(k, _u8p), _p(v, _u8p), _p(o, _f32p),
                               bh, sl, hd, int(causal), int(window), float(scale), int(parallel))
    return o


# ----------------------------------------------------------------------- GEMM

def gemm_f64(a, b, alpha=1.0) -> np.ndarray:
    """alpha * A[M,K] . B[N,K]^T on e4m3 codes, FP64 accumulate."""
    a, b = _u8(a), _u8(b)
    M, K = a.shape
    N, K2 = b.shape
    assert K == K2
    c = np.empty((M, N), np.float64)
    lib().oracle_gemm_f64(_p(a, _u8p), _p(b, _u8p), _p(c, _f64p), M, N, K, float(alpha))
    return c


def gemm_f32(a, b, parallel=False) -> np.ndarray:
    a, b = _u8(a), _u8(b)
    M, K = a.shape
    N, _ = b.shape
    c = np.empty((M, N), np.float32)
    lib().oracle_gemm_f32(_p(a, _u8p), _p(b, _u8p), _p(c, _f32p), M, N, K, int(parallel))
    return c


# --------------------------------------------------------------- harness data

def harness_attention_inputs(bh, sl, hd):
    n = bh * sl * hd
    q, k, v = (np.empty(n, np.uint8) for _ in range(3))
    lib().oracle_harness_attention_inputs(_p(q, _u8p), _p(k, _u8p), _p(v, _u8p), n)
    return q.reshape(bh, sl, hd), k.reshape(bh, sl, hd), v.reshape(bh, sl, hd)


def harness_gemm_inputs(M, N, K):
    a = np.empty(M * K, np.uint8)
    b = np.empty(N * K, np.uint8)
    lib().oracle_harness_gemm_inputs(_p(a, _u8p), a.size, _p(b, _u8p), b.size)
    return a.reshape(M, K), b.reshape(N, K)


def num_threads() -> int:
    return lib().oracle_num_threads()


# ----------------------------------------------------- rounding of the outputs

def round_fp16(x) -> np.ndarray:
    return np.asarray(x, np.float64).astype(np.float16)


def round_bf16(x) -> np.ndarray:
    """Round to bf16 (RNE), returned as float32 holding bf16 values."""
    f = np.asarray(x, np.float64).astype(np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32).copy()
    out[np.isnan(f)] = np.nan
    return out


# ------------------------------------------------------ seeded synthetic data

def seeded_normal(name: str, shape, std: float = 1.0, config: str = "") -> np.ndarray:
    """i.i.d. N(0, std) fp32 tensor from a fixed 64-bit seed derived from
    (config id, tensor name), so GPU and CPU sides draw identical values."""
    import hashlib
    h = hashlib.sha256(f"{config}/{name}".encode()).digest()
    seed = int.from_bytes(h[:8], "little")
    rng = np.random.Generator(np.random.Philox(seed))
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


def error_stats(got, ref):
    """(max-abs error, mean relative error = mean|x-ref| / mean|ref|)."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    d = np.abs(got - ref)
    return float(d.max()), float(d.mean() / max(np.abs(ref).mean(), 1e-300))


# ----------------------------------------- the reference's own compiled CPU code

class Ref:
    """ctypes view of oracle/_ref (the reference's own host code)."""

    def __init__(self):
        d = os.path.join(_HERE, "_ref")
        self.fa128 = self._open(os.path.join(d, "libref_fa_hd128.so"))
        self.fa64 = self._open(os.path.join(d, "libref_fa_hd64.so"))
        self.gemm = self._open(os.path.join(d, "libref_gemm.so"))
        # the reference's quantiser kernels (libs1/fp8_quantize_v2.cu:159-217), compiled for this GPU as they stand:
        # GPU code, used by the -m gpu tests to pin e4m3 codes to the reference's own output
        self.quant = self._open(os.path.join(d, "libref_quant.so"))
        if self.quant is not None:
            self.quant.fp8_quantize_fp16.restype = C.c_int
            self.quant.fp8_quantize_fp16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
            self.quant.cuda_device_sync2.restype = C.c_int
        for L in (self.fa128, self.fa64):
            if L is not None:
                L.ref_cpu_attention_fp8.argtypes = [_u8p, _u8p, _u8p, _f32p] + [C.c_int] * 5
                L.ref_float_to_e4m3.restype = C.c_uint8
                L.ref_float_to_e4m3.argtypes = [C.c_float]
                L.ref_e4m3_to_float.restype = C.c_float
                L.ref_e4m3_to_float.argtypes = [C.c_uint8]
        if self.gemm is not None:
            G = self.gemm
            G.ref_gemm_float_to_e4m3.restype = C.c_uint8
            G.ref_gemm_float_to_e4m3.argtypes = [C.c_float]
            G.ref_gemm_e4m3_to_float.restype = C.c_float
            G.ref_gemm_e4m3_to_float.argtypes = [C.c_uint8]
            G.ref_gemm_cpu_loop.argtypes = [_u8p, _u8p, _f32p, C.c_int, C.c_int, C.c_int]
            G.ref_fp8_gemm.restype = C.c_int
            G.ref_fp8_gemm.argtypes = [C.c_int] * 3 + [C.c_void_p] * 3 + [C.c_int, C.c_void_p]

    @staticmethod
    def _open(path):
        return C.CDLL(path) if os.path.exists(path) else None

    @property
    def available(self) -> bool:
        return self.fa128 is not None and self.gemm is not None

    def cpu_attention_fp8(self, q, k, v, causal=0, window=0):
        q, k, v = _u8(q), _u8(k), _u8(v)
        bh, sl, hd = q.shape
        L = self.fa128 if hd == 128 else self.fa64
        o = np.empty((bh, sl, hd), np.float32)
        L.ref_cpu_attention_fp8(_p(q, _u8p), _p(k, _u8p), _p(v, _u8p), _p(o, _f32p), bh, sl, hd, int(causal), int(window))
        return o

    def gemm_cpu_loop(self, a, b):
        a, b = _u8(a), _u8(b)
        M, K = a.shape
        N, _ = b.shape
        c = np.empty((M, N), np.float32)
        self.gemm.ref_gemm_cpu_loop(_p(a, _u8p), _p(b, _u8p), _p(c, _f32p), M, N, K)
        return c


_ref = None


def ref() -> Ref:
    global _ref
    if _ref is None:
        _ref = Ref()
    return _ref

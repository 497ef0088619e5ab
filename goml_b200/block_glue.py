"""Host binding of libfp8block.so: the decoder block's row-local glue fused with the per-tensor e4m3
quantiser (RMSNorm (+ residual), half-split RoPE + head permute of Q/K/V, head permute of the attention
output, SwiGLU, residual add).

These take the place of goml's libtransformer.so calls (rmsnorm_forward / swiglu_forward / rope_forward,
libs/transformer_kernels.cu:384-438) followed by separate quantiser launches and host round trips
(internal/abjexam/battle_a_llm.go:380-494).  Arguments are raw device pointers and sizes, like every
other binding of this package; each call is asynchronous on `stream`.
"""
from __future__ import annotations

import ctypes as C
import threading

from . import loader

_lock = threading.Lock()
_lib = None


class BlockGlueError(RuntimeError):
    pass


def _init():
    global _lib
    with _lock:
        if _lib is None:
            lib = loader.dlopen(loader.resolve_lib("libfp8block.so"))
            p, i, f, z = C.c_void_p, C.c_int, C.c_float, C.c_size_t
            for name, args in {
                "fp8_rope_table": [p, p, i, i, f, p],
                "fp8_rmsnorm_quantize": [p, p, p, p, p, p, p, p, i, i, f, p],
                "fp8_rope_quantize_qkv": [p, p, p, p, p, p, p, p, i, i, i, i, p],
                "fp8_permute_quantize_heads": [p, p, p, p, i, i, i, i, p],
                "fp8_swiglu_quantize": [p, p, p, p, i, i, p],
                "fp8_quantize_bf16": [p, p, p, p, z, p],
                "fp8_residual_add": [p, p, z, p],
            }.items():
                fn = getattr(lib, name)
                fn.restype = C.c_int
                fn.argtypes = args
            _lib = lib
    return _lib


def _check(name: str, rc: int) -> None:
    if rc != 0:
        raise BlockGlueError(f"{name}: CUDA error {rc}")


def RopeTable(cos: int, sin: int, seq_len: int, head_dim: int, theta: float, stream: int = 0) -> None:
    _check("fp8_rope_table", _init().fp8_rope_table(cos, sin, seq_len, head_dim, theta, stream or None))


def RMSNormQuantize(x: int, residual_bf16: int, h_out: int, gamma: int, q: int, scale: int, amax: int, rstd_ws: int,
                    rows: int, hidden: int, eps: float, stream: int = 0) -> None:
    _check("fp8_rmsnorm_quantize", _init().fp8_rmsnorm_quantize(x, residual_bf16 or None, h_out or None, gamma, q, scale, amax, rstd_ws,
                                                                rows, hidden, eps, stream or None))


def RopeQuantizeQKV(qkv_bf16: int, cos: int, sin: int, q: int, k: int, v: int, scales: int, amaxes: int,
                    batch: int, seq_len: int, heads: int, head_dim: int, stream: int = 0) -> None:
    _check("fp8_rope_quantize_qkv", _init().fp8_rope_quantize_qkv(qkv_bf16, cos, sin, q, k, v, scales, amaxes, batch, seq_len, heads,
                                                                  head_dim, stream or None))


def PermuteQuantizeHeads(o_fp16: int, q: int, scale: int, amax: int, batch: int, seq_len: int, heads: int, head_dim: int,
                         stream: int = 0) -> None:
    _check("fp8_permute_quantize_heads", _init().fp8_permute_quantize_heads(o_fp16, q, scale, amax, batch, seq_len, heads, head_dim,
                                                                            stream or None))


def SwiGLUQuantize(gate_up_bf16: int, q: int, scale: int, amax: int, rows: int, ffn_hidden: int, stream: int = 0) -> None:
    _check("fp8_swiglu_quantize", _init().fp8_swiglu_quantize(gate_up_bf16, q, scale, amax, rows, ffn_hidden, stream or None))


def QuantizeBF16(x_bf16: int, q: int, scale: int, amax_in: int, n: int, stream: int = 0) -> None:
    _check("fp8_quantize_bf16", _init().fp8_quantize_bf16(x_bf16, q, scale, amax_in, n, stream or None))


def ResidualAdd(x: int, y_bf16: int, n: int, stream: int = 0) -> None:
    _check("fp8_residual_add", _init().fp8_residual_add(x, y_bf16, n, stream or None))

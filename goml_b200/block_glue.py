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


class DecodeAppendArgs(C.Structure):
    """fp8_decode_append_args_t (include/fp8_block.h)."""
    _fields_ = [
        ("qkv_bf16", C.c_void_p), ("cos_tab", C.c_void_p), ("sin_tab", C.c_void_p), ("positions", C.c_void_p),
        ("q_out", C.c_void_p), ("q_scale_out", C.c_void_p), ("q_amax_out", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("seq_lens_out", C.c_void_p), ("block_table", C.c_void_p),
        ("batch", C.c_int32), ("q_heads", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("s_max", C.c_int32), ("rope_rows", C.c_int32),
        ("page_size", C.c_int32), ("max_pages_per_seq", C.c_int32), ("num_pages", C.c_int32), ("reserved", C.c_int32),
        ("stream", C.c_void_p),
    ]


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
                "fp8_decode_rope_append": [C.POINTER(DecodeAppendArgs)],
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


def DecodeRopeAppend(qkv_bf16, cos_tab, sin_tab, positions, q_out, q_scale_out, q_amax_out, k_cache, v_cache, k_scale, v_scale,
                     batch, q_heads, kv_heads, head_dim, s_max, rope_rows, seq_lens_out=0, block_table=0, page_size=0,
                     max_pages_per_seq=0, num_pages=0, stream=0) -> None:
    """Decode step: RoPE at positions[b] on the new token's Q and K, Q codes with a fresh per-tensor scale, K and V
    codes (cache scales *k_scale, *v_scale) written at positions[b] of the contiguous or paged FP8 KV cache."""
    a = DecodeAppendArgs(qkv_bf16, cos_tab, sin_tab, positions, q_out, q_scale_out, q_amax_out, k_cache, v_cache, k_scale, v_scale,
                         seq_lens_out or None, block_table or None, batch, q_heads, kv_heads, head_dim, s_max, rope_rows,
                         page_size, max_pages_per_seq, num_pages, 0, stream or None)
    _check("fp8_decode_rope_append", _init().fp8_decode_rope_append(C.byref(a)))

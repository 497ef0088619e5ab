"""Host binding of libfa_sm120.so, mirroring goml's backend/cuda/fa_forward.go.

Names and behaviour follow that file: ``FALoad`` (one-time dlopen with the
search order of fa_forward.go:74-115: ``$GOML_FA_LIB``, then
``libs/fa_sm120/libfa_sm120.so``, ``./libfa_sm120.so``,
``/usr/local/lib/libfa_sm120.so`` — this package's own ``libs`` directory is
tried right after the environment override), ``FACreate`` (fa_forward.go:123-142,
including "context returned together with an error is read for its message and
destroyed"), ``FAContext.ForwardTrain`` (fa_forward.go:161-183) and
``FAVersion``.  ``FAContext.Forward`` binds ``fa_forward`` (which the Go file
leaves unbound) and ``FAContext.ForwardEx`` binds the additive struct-pointer
entry.  Pointers are raw device addresses (ints); errors are raised as
``FAError("<entry>: <status text> (<context message>)")``.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

from . import loader

FA_OK = 0
FA_ERR_INVALID_ARG = 1
FA_ERR_UNSUPPORTED_ARCH = 2
FA_ERR_UNSUPPORTED_HD = 3
FA_ERR_UNSUPPORTED_SHAPE = 4
FA_ERR_CUDA = 5
FA_ERR_OOM = 6
FA_ERR_INTERNAL = 7

FA_KERNEL_NONE = -1
FA_KERNEL_V121R, FA_KERNEL_V121, FA_KERNEL_V118 = 100, 101, 102
FA_KERNEL_V122, FA_KERNEL_V117B, FA_KERNEL_V96B = 103, 104, 105
FA_KERNEL_V89, FA_KERNEL_V80B = 200, 201


class FAError(RuntimeError):
    def __init__(self, entry: str, status: int, msg: str = ""):
        self.status = status
        self.msg = msg
        text = FAStatusString(status)
        super().__init__(f"{entry}: {text} ({msg})" if msg else f"{entry}: {text}")


class ForwardArgs(C.Structure):
    """fa_forward_args_t of include/fa_sm120.h."""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("l_out", C.c_void_p),
        ("batch_heads", C.c_int), ("seq_len", C.c_int), ("head_dim", C.c_int),
        ("causal", C.c_int), ("window", C.c_int),
        ("scale", C.c_float), ("v_descale", C.c_float),
        ("scale_q_dev", C.c_void_p), ("scale_k_dev", C.c_void_p), ("scale_v_dev", C.c_void_p),
        ("stream", C.c_void_p),
    ]


class DecodeArgs(C.Structure):
    """fa_decode_args_t (include/fa_sm120.h)."""
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("o", C.c_void_p), ("l_out", C.c_void_p),
        ("seq_lens", C.c_void_p),
        ("batch", C.c_int), ("q_heads", C.c_int), ("kv_heads", C.c_int), ("head_dim", C.c_int),
        ("s_max", C.c_int), ("seq_len", C.c_int),
        ("scale", C.c_float), ("v_descale", C.c_float),
        ("scale_q_dev", C.c_void_p), ("scale_k_dev", C.c_void_p), ("scale_v_dev", C.c_void_p),
        ("stream", C.c_void_p),
        ("block_table", C.c_void_p), ("page_size", C.c_int), ("max_pages_per_seq", C.c_int), ("num_pages", C.c_int),
    ]


_lock = threading.Lock()
_lib = None
_lib_err = None


def _candidates():
    env = os.environ.get("GOML_FA_LIB", "")
    if env:
        yield env
    yield loader.resolve_lib("libfa_sm120.so")
    yield os.path.join("libs", "fa_sm120", "libfa_sm120.so")
    yield os.path.join(".", "libfa_sm120.so")
    yield "/usr/local/lib/libfa_sm120.so"


def FALoad():
    """One-time dlopen of libfa_sm120.so and symbol registration."""
    global _lib, _lib_err
    with _lock:
        if _lib is None and _lib_err is None:
            last = None
            for path in _candidates():
                if os.path.sep in path and not os.path.exists(path):
                    continue
                try:
                    lib = loader.dlopen(path)
                except OSError as e:
                    last = e
                    continue
                i, p, f = C.c_int, C.c_void_p, C.c_float
                lib.fa_create.restype = i
                lib.fa_create.argtypes = [C.POINTER(p)]
                lib.fa_destroy.restype = i
                lib.fa_destroy.argtypes = [p]
                lib.fa_version.restype = C.c_char_p
                lib.fa_status_str.restype = C.c_char_p
                lib.fa_status_str.argtypes = [i]
                lib.fa_last_cuda_error.restype = C.c_char_p
                lib.fa_last_cuda_error.argtypes = [p]
                lib.fa_forward.restype = i
                lib.fa_forward.argtypes = [p, p, p, p, p, i, i, i, i, i, f, p]
                lib.fa_forward_train.restype = i
                lib.fa_forward_train.argtypes = [p, p, p, p, p, p, i, i, i, i, i, f, p]
                lib.fa_dispatch_select.restype = i
                lib.fa_dispatch_select.argtypes = [i] * 5
                lib.fa_kernel_name.restype = C.c_char_p
                lib.fa_kernel_name.argtypes = [i]
                lib.fa_forward_ex.restype = i
                lib.fa_forward_ex.argtypes = [p, C.POINTER(ForwardArgs)]
                lib.fa_forward_noalloc.restype = i
                lib.fa_forward_noalloc.argtypes = [C.POINTER(ForwardArgs), C.c_char_p, i]
                lib.fa_decode.restype = i
                lib.fa_decode.argtypes = [p, C.POINTER(DecodeArgs)]
                lib.fa_device_status.restype = i
                lib.fa_device_status.argtypes = [p]
                lib.fa_noalloc_device_status.restype = i
                lib.fa_noalloc_device_status.argtypes = []
                lib.fa_selftest_wait_expiry.restype = i
                lib.fa_selftest_wait_expiry.argtypes = [p, p]
                _lib = lib
                break
            if _lib is None:
                _lib_err = loader.LibraryNotFound(
                    f"fa: dlopen libfa_sm120.so failed ({last}); set GOML_FA_LIB or build with "
                    f"`python -m goml_b200.build`")
    if _lib_err is not None:
        raise _lib_err
    return _lib


def FAStatusString(status: int) -> str:
    try:
        return FALoad().fa_status_str(int(status)).decode()
    except OSError:
        return f"unknown({status})"


def FAVersion() -> str:
    return FALoad().fa_version().decode()


def FADispatchSelect(bh: int, sl: int, hd: int, causal: int, window: int) -> int:
    return FALoad().fa_dispatch_select(bh, sl, hd, causal, window)


def FAKernelName(kid: int) -> str:
    return FALoad().fa_kernel_name(kid).decode()


class FAContext:
    """Opaque handle; one per GPU (the device current when it was created)."""

    def __init__(self, ptr: int):
        self.ptr = ptr

    def _msg(self) -> str:
        return FALoad().fa_last_cuda_error(self.ptr).decode(errors="replace") if self.ptr else ""

    def Destroy(self) -> None:
        if self.ptr:
            FALoad().fa_destroy(self.ptr)
            self.ptr = 0

    def ForwardTrain(self, q, k, v, o, lOut, bh, sl, hd, causal, window, scale, stream=0) -> None:
        if not self.ptr:
            raise FAError("FAContext.ForwardTrain: nil ctx", FA_ERR_INVALID_ARG)
        st = FALoad().fa_forward_train(self.ptr, q, k, v, o, lOut or None, bh, sl, hd, causal, window, scale, stream or None)
        if st != FA_OK:
            raise FAError("fa_forward_train", st, self._msg())

    def Forward(self, q, k, v, o, bh, sl, hd, causal, window, scale, stream=0) -> None:
        if not self.ptr:
            raise FAError("FAContext.Forward: nil ctx", FA_ERR_INVALID_ARG)
        st = FALoad().fa_forward(self.ptr, q, k, v, o, bh, sl, hd, causal, window, scale, stream or None)
        if st != FA_OK:
            raise FAError("fa_forward", st, self._msg())

    def ForwardEx(self, q, k, v, o, lOut, bh, sl, hd, causal, window, scale, v_descale=1.0,
                  scale_q_dev=0, scale_k_dev=0, scale_v_dev=0, stream=0) -> None:
        if not self.ptr:
            raise FAError("FAContext.ForwardEx: nil ctx", FA_ERR_INVALID_ARG)
        a = ForwardArgs(q, k, v, o, lOut or None, bh, sl, hd, causal, window, scale, v_descale,
                        scale_q_dev or None, scale_k_dev or None, scale_v_dev or None, stream or None)
        st = FALoad().fa_forward_ex(self.ptr, C.byref(a))
        if st != FA_OK:
            raise FAError("fa_forward_ex", st, self._msg())

    def Decode(self, q, k_cache, v_cache, o, lOut, seq_lens, batch, q_heads, kv_heads, hd, s_max, seq_len, scale, v_descale=1.0,
               scale_q_dev=0, scale_k_dev=0, scale_v_dev=0, stream=0, block_table=0, page_size=0, max_pages_per_seq=0,
               num_pages=0) -> None:
        """One new token per sequence against an e4m3 KV cache [batch, kv_heads, s_max, hd], grouped-query heads;
        seq_lens: device pointer to batch int32 lengths, or 0 to use seq_len for every sequence.  With block_table
        (device pointer to int32 [batch, max_pages_per_seq]) the caches are page pools [num_pages, kv_heads, page_size,
        hd] and s_max is ignored."""
        if not self.ptr:
            raise FAError("FAContext.Decode: nil ctx", FA_ERR_INVALID_ARG)
        a = DecodeArgs(q, k_cache, v_cache, o, lOut or None, seq_lens or None, batch, q_heads, kv_heads, hd, s_max, seq_len,
                       scale, v_descale, scale_q_dev or None, scale_k_dev or None, scale_v_dev or None, stream or None,
                       block_table or None, page_size, max_pages_per_seq, num_pages)
        st = FALoad().fa_decode(self.ptr, C.byref(a))
        if st != FA_OK:
            raise FAError("fa_decode", st, self._msg())

    def DeviceStatus(self) -> None:
        st = FALoad().fa_device_status(self.ptr)
        if st != FA_OK:
            raise FAError("fa_device_status", st, self._msg())

    def SelftestWaitExpiry(self, stream=0) -> None:
        """Launch the one-warp kernel whose bounded wait runs out; the next DeviceStatus() then raises FA_ERR_INTERNAL."""
        st = FALoad().fa_selftest_wait_expiry(self.ptr, stream or None)
        if st != FA_OK:
            raise FAError("fa_selftest_wait_expiry", st, self._msg())

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.Destroy()


NOALLOC_MAX_ELEMS = 16 << 20


def FAForwardNoAlloc(q, k, v, o, lOut, bh, sl, hd, causal, window, scale, v_descale=1.0,
                     scale_q_dev=0, scale_k_dev=0, scale_v_dev=0, stream=0) -> None:
    """Attention forward for callers that may not allocate (frameworks that reserved the whole
    GPU, frozen-memory-map processes): scratch is a fixed 32 MiB array inside the library, so
    bh*sl*hd must not exceed NOALLOC_MAX_ELEMS.  No context is needed.  Calls that overlap on
    the GPU share (and race on) that array; make the first call on a device before any capture."""
    a = ForwardArgs(q, k, v, o, lOut or None, bh, sl, hd, causal, window, scale, v_descale,
                    scale_q_dev or None, scale_k_dev or None, scale_v_dev or None, stream or None)
    buf = C.create_string_buffer(256)
    st = FALoad().fa_forward_noalloc(C.byref(a), buf, len(buf))
    if st != FA_OK:
        raise FAError("fa_forward_noalloc", st, buf.value.decode(errors="replace"))


def FANoAllocDeviceStatus() -> int:
    """fa_device_status without a context (for users of FAForwardNoAlloc): 0, a kernel's wait-expiry code, or
    a negated CUDA error."""
    return FALoad().fa_noalloc_device_status()


def FACreate() -> FAContext:
    """Create an FA context on the current device (fa_forward.go:123-142)."""
    lib = FALoad()
    ptr = C.c_void_p()
    st = lib.fa_create(C.byref(ptr))
    if st != FA_OK:
        if ptr.value:
            msg = lib.fa_last_cuda_error(ptr).decode(errors="replace")
            lib.fa_destroy(ptr)
            raise FAError("fa_create", st, msg)
        raise FAError("fa_create", st)
    return FAContext(ptr.value)

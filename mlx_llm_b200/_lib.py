"""ctypes binding of libb200llm.so (the C ABI declared in include/b200llm.h).

The library is the product; this module only loads it.  There is no fallback: if the shared
library is missing, or no CUDA device is present when a context is created, the call raises.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200llm.so")

B2_OK = 0
ERRORS = {
    -1: "B2_ERR_CUDA", -2: "B2_ERR_MISSING_TENSOR", -3: "B2_ERR_IO", -4: "B2_ERR_CONFIG", -5: "B2_ERR_UNSUPPORTED",
    -6: "B2_ERR_CANCELED", -7: "B2_ERR_MSG", -8: "B2_ERR_OOM_PAGES", -9: "B2_ERR_TIMEOUT",
}


class B2Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"{ERRORS.get(code, code)}: {msg}")
        self.code = code


_lib = None


def load():
    """Load libb200llm.so; raises if it has not been built (python -m mlx_llm_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m mlx_llm_b200.build` (needs nvcc); "
                              "there is no CPU fallback")
        _lib = C.CDLL(LIB_PATH)
        _lib.b2_last_error.restype = C.c_char_p
    return _lib


def check(rc):
    if rc != B2_OK:
        raise B2Error(rc, load().b2_last_error().decode(errors="replace"))
    return rc


def ptr(a):
    """Device pointer (int / DevBuf) or host numpy array -> c_void_p."""
    if a is None:
        return None
    if isinstance(a, DevBuf):
        return C.c_void_p(a.ptr)
    if isinstance(a, np.ndarray):
        return a.ctypes.data_as(C.c_void_p)
    return C.c_void_p(int(a))


class DevBuf:
    """A device allocation made through b2_malloc, with numpy upload/download helpers."""

    def __init__(self, ctx, nbytes):
        self.ctx = ctx
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(load().b2_malloc(ctx.h, C.c_size_t(self.nbytes), C.byref(p)))
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, ctx, arr):
        arr = np.ascontiguousarray(arr)
        b = cls(ctx, arr.nbytes)
        b.upload(arr)
        b.shape, b.dtype = arr.shape, arr.dtype
        return b

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes <= self.nbytes
        check(load().b2_memcpy_h2d(self.ctx.h, C.c_void_p(self.ptr), arr.ctypes.data_as(C.c_void_p), C.c_size_t(arr.nbytes)))

    def download(self, shape=None, dtype=None):
        shape = shape if shape is not None else self.shape
        dtype = dtype if dtype is not None else self.dtype
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        check(load().b2_memcpy_d2h(self.ctx.h, out.ctypes.data_as(C.c_void_p), C.c_void_p(self.ptr), C.c_size_t(out.nbytes)))
        return out

    def free(self):
        if self.ptr:
            load().b2_free(self.ctx.h, C.c_void_p(self.ptr))
            self.ptr = 0


class Context:
    """One context = one GPU = one host thread (b2_ctx_create)."""

    def __init__(self, device=0):
        self.h = C.c_void_p()
        check(load().b2_ctx_create(int(device), C.byref(self.h)))
        self.device = device

    def sync(self):
        check(load().b2_ctx_sync(self.h))

    def timer_start(self):
        check(load().b2_timer_start(self.h))

    def timer_stop_ms(self):
        ms = C.c_float(0)
        check(load().b2_timer_stop_ms(self.h, C.byref(ms)))
        return ms.value

    def flush_l2(self):
        check(load().b2_flush_l2(self.h))

    def profiler_range(self, on):
        check(load().b2_profiler_range(self.h, C.c_int32(1 if on else 0)))

    def nvtx(self, on):
        """NVTX ranges per kernel class around every step's launches (b2_nvtx_enable)."""
        check(load().b2_nvtx_enable(self.h, C.c_int32(1 if on else 0)))

    def mem_info(self):
        f, t = C.c_size_t(0), C.c_size_t(0)
        check(load().b2_mem_info(self.h, C.byref(f), C.byref(t)))
        return f.value, t.value

    def launch_count(self):
        n = C.c_int64(0)
        check(load().b2_launch_count(self.h, C.byref(n)))
        return n.value

    def buf(self, arr):
        return DevBuf.from_numpy(self, arr)

    def empty(self, shape, dtype):
        b = DevBuf(self, int(np.prod(shape)) * np.dtype(dtype).itemsize)
        b.shape, b.dtype = tuple(shape), np.dtype(dtype)
        return b

    def close(self):
        if self.h:
            load().b2_ctx_free(self.h)
            self.h = C.c_void_p()


def device_count():
    n = C.c_int32(0)
    rc = load().b2_device_count(C.byref(n))
    return n.value if rc == 0 else 0

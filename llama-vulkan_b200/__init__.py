"""B200-native decode path for aodenis/llama-vulkan: ctypes bindings.

The native code lives in ``liblv_b200.so`` (sm_100a kernels behind the C ABI
declared in ``include/lv_b200.h``) and ``libllava_host.so`` (the C++ host
surface: ggml_file, llava_session, ... with the C wrappers declared in
``include/llava_host.h``).  This module only loads them and declares
argument types; there is no Python or CPU fallback for any kernel: if the
libraries are missing, ``load_kernels()`` / ``load_host()`` raise.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
KERNEL_LIB = os.path.join(HERE, "liblv_b200.so")
HOST_LIB = os.path.join(HERE, "libllava_host.so")

LV_OK = 0
LV_ERR_NOK = 1
LV_ERR_BAD_ARGUMENTS = 7
LV_ERR_CUDA = 100
LV_ERR_DEVICE_WAIT = 101
LV_ERR_TIMEOUT = 102
LV_ERR_COMM = 103

TYPE_F32, TYPE_F16, TYPE_Q4_0, TYPE_Q8_0 = 0, 1, 2, 8

_p = C.c_void_p
_u32 = C.c_uint32
_sz = C.c_size_t
_int = C.c_int

# name -> (restype, argtypes); mirrors include/lv_b200.h
KERNEL_API = {
    "lv_device_count": (_int, [C.POINTER(_int)]),
    "lv_ctx_create": (_int, [_int, C.POINTER(_p)]),
    "lv_ctx_destroy": (_int, [_p]),
    "lv_last_error_string": (C.c_char_p, []),
    "lv_ctx_stream": (_p, [_p]),
    "lv_ctx_sm_count": (_int, [_p]),
    "lv_arena_create": (_int, [_p, _sz, C.POINTER(_p)]),
    "lv_arena_free": (_int, [_p, _p]),
    "lv_host_alloc": (_int, [_p, _sz, C.POINTER(_p)]),
    "lv_host_free": (_int, [_p, _p]),
    "lv_upload": (_int, [_p, _p, _p, _sz]),
    "lv_download": (_int, [_p, _p, _p, _sz]),
    "lv_upload_async": (_int, [_p, _p, _p, _sz]),
    "lv_download_async": (_int, [_p, _p, _p, _sz]),
    "lv_memset": (_int, [_p, _p, _int, _sz]),
    "lv_copy_d2d": (_int, [_p, _p, _p, _sz]),
    "lv_graph_begin_capture": (_int, [_p]),
    "lv_graph_end_capture": (_int, [_p, C.POINTER(_p)]),
    "lv_graph_launch": (_int, [_p, _p]),
    "lv_graph_destroy": (_int, [_p]),
    "lv_stream_sync": (_int, [_p, _int]),
    "lv_norm_f32": (_int, [_p, _p, _p, _p, _u32, _u32]),
    "lv_gemv": (_int, [_p, _p, _p, _int, _p, _u32, _u32, _u32, _int]),
    "lv_gemv_silu": (_int, [_p, _p, _p, _p, _int, _p, _u32, _u32, _u32]),
    "lv_kv_append_f16": (_int, [_p, _p, _p, _p, _u32, _u32, _u32]),
    "lv_rope_table_build": (_int, [_p, _p, _u32, _u32]),
    "lv_attn_scores_rope": (_int, [_p, _p, _p, _p, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_softmax_masked": (_int, [_p, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_attn_values": (_int, [_p, _p, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_copy_f32": (_int, [_p, _p, _p, _sz]),
    "lv_add_f32": (_int, [_p, _p, _p, _sz]),
    "lv_dequant_rows": (_int, [_p, _p, _p, _int, _p, _u32, _u32]),
    "lv_argmax_f32": (_int, [_p, _p, _p, _u32]),
    "lv_norm_qkv_kvappend": (_int, [_p, _p, _p, _p, _p, _p, _p, _int, _p, _p, _p, _u32, _u32, _u32]),
    "lv_attention_scratch_bytes": (_sz, [_u32, _u32, _u32, _u32]),
    "lv_attention_fused": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_norm_gate_up_silu": (_int, [_p, _p, _p, _p, _int, _p, _p, _u32, _u32, _u32]),
    "lv_norm_gemv": (_int, [_p, _p, _p, _int, _p, _p, _u32, _u32, _u32]),
}

_kernels = None
_host = None


class LvError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"lv error {code}: {message}")
        self.code = code


def _declare(lib, table):
    for name, (res, args) in table.items():
        fn = getattr(lib, name)      # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args


def load_kernels():
    """Loads liblv_b200.so; raises if it has not been built."""
    global _kernels
    if _kernels is None:
        if not os.path.exists(KERNEL_LIB):
            raise RuntimeError(f"{KERNEL_LIB} is missing: run `python llama-vulkan_b200/build.py` "
                               "(there is no fallback path)")
        lib = C.CDLL(KERNEL_LIB, mode=C.RTLD_GLOBAL)
        _declare(lib, KERNEL_API)
        _kernels = lib
    return _kernels


def check(code):
    """Raises LvError for a non-zero status of an lv_* call."""
    if code != LV_OK:
        msg = load_kernels().lv_last_error_string()
        raise LvError(code, msg.decode("utf-8", "replace") if msg else "")
    return code


class Context:
    """One GPU + one stream (lv_ctx) with small helpers for tests and benches."""

    def __init__(self, device=0):
        self.lib = load_kernels()
        self.handle = _p()
        check(self.lib.lv_ctx_create(device, C.byref(self.handle)))
        self._arenas = []

    def close(self):
        if self.handle:
            for a in self._arenas:
                self.lib.lv_arena_free(self.handle, a)
            self._arenas = []
            self.lib.lv_ctx_destroy(self.handle)
            self.handle = _p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def alloc(self, nbytes):
        d = _p()
        check(self.lib.lv_arena_create(self.handle, max(int(nbytes), 16), C.byref(d)))
        self._arenas.append(d)
        return d

    def free(self, d):
        self._arenas = [a for a in self._arenas if a.value != d.value]
        check(self.lib.lv_arena_free(self.handle, d))

    def upload(self, array):
        """numpy array -> new device buffer (returned as c_void_p)."""
        import numpy as np
        a = np.ascontiguousarray(array)
        d = self.alloc(a.nbytes)
        if a.nbytes:
            check(self.lib.lv_upload(self.handle, d, a.ctypes.data_as(_p), a.nbytes))
        return d

    def download(self, d, dtype, count):
        import numpy as np
        out = np.empty(count, dtype=dtype)
        if out.nbytes:
            check(self.lib.lv_download(self.handle, out.ctypes.data_as(_p), d, out.nbytes))
        return out

    def zeros(self, nbytes):
        d = self.alloc(nbytes)
        check(self.lib.lv_memset(self.handle, d, 0, int(nbytes)))
        return d

    def sync(self, timeout_ms=0):
        check(self.lib.lv_stream_sync(self.handle, timeout_ms))


def offset(ptr, nbytes):
    """c_void_p arithmetic."""
    return _p(ptr.value + int(nbytes))

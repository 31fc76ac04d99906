"""ctypes bindings of the CPU oracle (oracle/llava_oracle.h) for the tests.

The oracle is the checker, never the product: only tests, the smoke check and
the bench's cpu_baseline leg load it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB = os.path.join(ORACLE_DIR, "_build", "liboracle.so")
REF_LIB = os.path.join(ORACLE_DIR, "_ref", "libref_ggml.so")

_p, _u32, _u16, _f = C.c_void_p, C.c_uint32, C.c_uint16, C.c_float
_fp = C.POINTER(C.c_float)


class ModelInfo(C.Structure):
    _fields_ = [(n, _u32) for n in ("file_version", "vocab_size", "dim", "multiple_of", "n_heads", "n_layers",
                                    "rot", "ftype", "ff_size", "wtype", "n_tensors")]


def build():
    src = [os.path.join(ORACLE_DIR, f) for f in ("llava_oracle.c", "llava_oracle.h")]
    if (not os.path.exists(LIB)) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in src):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "_build/liboracle.so"], stdout=subprocess.DEVNULL,
                              stderr=subprocess.DEVNULL)
    return LIB


_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    lib = C.CDLL(build())
    sig = {
        "orc_half_to_float": (_f, [_u16]),
        "orc_float_to_half": (_u16, [_f]),
        "orc_row_bytes": (C.c_size_t, [C.c_int, C.c_int, _u32]),
        "orc_dequant": (C.c_int, [_p, C.c_int, C.c_int, _p, _u32]),
        "orc_norm": (None, [_p, _p, _p, _u32, _u32]),
        "orc_gemv": (C.c_int, [_p, _p, C.c_int, C.c_int, _p, _u32, _u32, _u32, C.c_int]),
        "orc_gemv_silu": (C.c_int, [_p, _p, _p, C.c_int, C.c_int, _p, _u32, _u32, _u32]),
        "orc_kv_append": (None, [_p, _p, _u32, _u32]),
        "orc_mhsa": (None, [_p, _p, _p, _u32, _u32, _u32, _u32]),
        "orc_softmax": (None, [_p, _u32, _u32, _u32, _u32]),
        "orc_kqv": (None, [_p, _p, _p, _u32, _u32, _u32]),
        "orc_argmax": (_u32, [_p, _u32]),
        "orc_sampler_candidates": (_u32, [_p, _u32, _p, _u32, _f, _p, _p, _fp]),
        "orc_sampler_mu_update": (_f, [_f, _f, _f]),
        "orc_model_open": (_p, [C.c_char_p]),
        "orc_model_close": (None, [_p]),
        "orc_model_get_info": (None, [_p, C.POINTER(ModelInfo)]),
        "orc_model_tensor": (C.c_int, [_p, _u32, C.c_char_p, C.c_size_t, C.POINTER(_u32), C.POINTER(C.c_uint64),
                                       C.POINTER(_u32), C.POINTER(_u32), C.POINTER(C.c_uint64)]),
        "orc_model_tensor_data": (_p, [_p, C.c_char_p]),
        "orc_model_token": (_p, [_p, _u32, C.POINTER(_u32), _fp]),
        "orc_session_create": (_p, [_p, _u32]),
        "orc_session_destroy": (None, [_p]),
        "orc_session_push_token": (C.c_int, [_p, _u32]),
        "orc_session_rewind": (None, [_p, _u32]),
        "orc_session_token_count": (_u32, [_p]),
        "orc_session_backlog": (_u32, [_p]),
        "orc_session_eval": (C.c_int, [_p, _p]),
        "orc_session_k_cache": (_p, [_p, _u32]),
        "orc_session_v_cache": (_p, [_p, _u32]),
        "orc_session_residual": (_p, [_p]),
        "orc_session_layer_outputs": (_p, [_p]),
        "orc_set_threads": (None, [C.c_int]),
        "orc_get_threads": (C.c_int, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def ptr(a):
    return a.ctypes.data_as(_p)


# ---- numpy-facing wrappers -------------------------------------------------
def dequant(raw, wtype, count, version=3):
    out = np.empty(count, np.float32)
    assert load().orc_dequant(ptr(raw), wtype, version, ptr(out), count) == 0
    return out


def norm(x, w, wgs=1024):
    out = np.empty_like(x)
    load().orc_norm(ptr(out), ptr(x), ptr(w), x.size, wgs)
    return out


def gemv(W, wtype, x, rows, cols, workers, out=None, version=3):
    add = out is not None
    o = out.copy() if add else np.empty(rows, np.float32)
    assert load().orc_gemv(ptr(o), ptr(W), wtype, version, ptr(x), rows, cols, workers, int(add)) == 0
    return o


def gemv_silu(w3, w1, wtype, x, rows, cols, workers, version=3):
    o = np.empty(rows, np.float32)
    assert load().orc_gemv_silu(ptr(o), ptr(w3), ptr(w1), wtype, version, ptr(x), rows, cols, workers) == 0
    return o


def mhsa(k_cache, q, pos, heads, rot):
    scores = np.zeros(((pos + 1), heads), np.float32)
    load().orc_mhsa(ptr(scores), ptr(k_cache), ptr(q), pos, pos + 1, heads, rot)
    return scores


def softmax(scores_filled, pos, backlog, heads, rot):
    s = np.zeros((backlog, heads), np.float32)
    s[: pos + 1] = scores_filled
    load().orc_softmax(ptr(s), pos, backlog, heads, rot)
    return s


def kqv(v_cache, probs, backlog, heads, rot):
    out = np.empty(heads * rot, np.float32)
    load().orc_kqv(ptr(out), ptr(v_cache), ptr(probs), backlog, heads, rot)
    return out


def attention(k_cache, v_cache, q, pos, backlog, heads, rot):
    """mhsa -> softmax -> kqv_matching, as llava_layer.cpp:59-62 chains them."""
    return kqv(v_cache, softmax(mhsa(k_cache, q, pos, heads, rot), pos, backlog, heads, rot), backlog, heads, rot)


def f32_to_f16_bits(x):
    lib = load()
    return np.array([lib.orc_float_to_half(float(v)) for v in np.asarray(x, np.float32).ravel()], np.uint16).reshape(np.shape(x))

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
import struct

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
TYPE_Q4_0_V1 = 258

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
    "lv_graph_kernel_nodes": (_int, [_p, _p]),
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
    "lv_dequant_rows": (_int, [_p, _p, _p, _int, _p, _p, _u32, _u32, _u32]),
    "lv_argmax_f32": (_int, [_p, _p, _p, _u32]),
    "lv_decode_advance": (_int, [_p, _p, _p, _p, _u32, _u32]),
    "lv_tp_arm_push": (_int, [_p, _int, _u32]),
    "lv_tp_arm_pull": (_int, [_p, _int, _u32, _u32, _p]),
    "lv_argmax_advance": (_int, [_p, _p, _u32, _p, _p, _u32, _u32, _p, _p]),
    "lv_norm_qkv_kvappend": (_int, [_p, _p, _p, _p, _p, _p, _p, _int, _p, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_comm_unique_id": (_int, [_p]),
    "lv_comm_init_rank": (_int, [_p, _p, _int, _int]),
    "lv_allreduce_f32": (_int, [_p, _p, _sz]),
    "lv_allreduce_add_f32": (_int, [_p, _p, _p, _sz]),
    "lv_peer_window_bytes": (_sz, [_int, _u32]),
    "lv_peer_window_create": (_int, [_p, _int, _u32, _p]),
    "lv_peer_connect": (_int, [_p, _int, _p]),
    "lv_peer_destroy": (_int, [_p]),
    "lv_comm_status": (_int, [_p]),
    "lv_comm_abort": (_int, [_p]),
    "lv_comm_destroy": (_int, [_p]),
    "lv_attention_scratch_bytes": (_sz, [_u32, _u32, _u32, _u32]),
    "lv_attention_fused": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_attention_static_scratch_limit": (_sz, []),
    "lv_attention_fused_static": (_int, [_p, _p, _p, _p, _p, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_act_split_bytes": (_sz, [_u32, _u32]),
    "lv_act_split_f16": (_int, [_p, _p, _p, _p, _u32, _u32]),
    "lv_act_split_f16_padded": (_int, [_p, _p, _p, _p, _u32, _u32, _u32]),
    "lv_dequant_rows_group": (_int, [_p, _p, _p, _int, _p, _u32, _u32, _u32]),
    "lv_gemm_tc_qkv_kvappend_group": (_int, [_p, _p, _p, _p, _p, _int, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_attention_fused_group": (_int, [_p, _p, _p, _p, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_argmax_advance_group": (_int, [_p, _p, _u32, _p, _u32, _u32, _p, _p]),
    "lv_gemm_tc_set_exact": (_int, [_p, _int]),
    "lv_gemm_tc": (_int, [_p, _p, _p, _int, _p, _u32, _u32, _u32, _int]),
    "lv_gemm_tc_silu": (_int, [_p, _p, _p, _p, _int, _p, _u32, _u32, _u32]),
    "lv_gemm_tc_qkv_kvappend": (_int, [_p, _p, _p, _p, _p, _p, _p, _int, _p, _p, _u32, _u32, _u32, _u32]),
    "lv_norm_gate_up_silu": (_int, [_p, _p, _p, _p, _int, _p, _p, _u32, _u32, _u32]),
    "lv_norm_gemv": (_int, [_p, _p, _p, _int, _p, _p, _u32, _u32, _u32]),
    "lv_sample_mirostat": (_int, [_p, _p, _u32, _p, _p, _p, C.c_float, _p, _u32, _p, _p, _p]),
    "lv_step_plan_create": (_int, [_p, _p, C.POINTER(_p)]),
    "lv_step_plan_destroy": (_int, [_p]),
    "lv_step_plan_set_trace": (_int, [_p, _int]),
    "lv_step_plan_read_trace": (_int, [_p, _p, _sz, _p, _p, _p]),
    "lv_decode_step": (_int, [_p, _p, _p, _p, _u32, _p, _p, _p, _int]),
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
        lib = C.CDLL(KERNEL_LIB)
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


# ---- libllava_host.so: the C++ host surface --------------------------------------------
_u64 = C.c_uint64
_f32p = C.POINTER(C.c_float)
_u32p = C.POINTER(C.c_uint32)

# name -> (restype, argtypes); mirrors include/llava_host.h
HOST_API = {
    "llava_synth_write": (_int, [C.c_char_p, _u32, _u32, _u32, _u32, _u32, _int, _u64, _u32]),
    "llava_synth_write_ex": (_int, [C.c_char_p, _u32, _u32, _u32, _u32, _u32, _int, _u64, _u32, _u32, _int]),
    "llava_synth_quantize_v1": (None, [_p, _sz, _p]),
    "llava_synth_file_size": (_u64, [_u32, _u32, _u32, _u32, _u32, _int]),
    "llava_synth_normal": (C.c_float, [_u64, _u32, _u64]),
    "llava_synth_quantize": (None, [_p, _sz, _int, _p]),
    "ggml_file_open": (_p, [C.c_char_p]),
    "ggml_file_close": (None, [_p]),
    "ggml_file_header": (None, [_p, _u32p]),
    "ggml_file_n_tensors": (_u32, [_p]),
    "ggml_file_tensor": (_int, [_p, _u32, C.c_char_p, _sz, _u32p, C.POINTER(_u64), _u32p, _u32p, C.POINTER(_u64)]),
    "ggml_file_find": (_int, [_p, C.c_char_p, C.POINTER(_u64)]),
    "ggml_file_tokenize": (_u32, [_p, C.c_char_p, _sz, _int, _p, _u32]),
    "ggml_file_tokens_to_text": (_u32, [_p, _p, _u32, C.c_char_p, _u32]),
    "ggml_file_token": (_u32, [_p, _u32, C.c_char_p, _u32, _f32p]),
    "llava_dequantize": (_int, [_p, _int, _u32, _p, _u32]),
    "llava_context_open": (_p, [C.c_char_p, _int]),
    "llava_context_open_model_only": (_p, [C.c_char_p]),
    "llava_context_open_sharded": (_p, [C.c_char_p, _int, _u32, _u32, _p]),
    "llava_context_peer_window_create": (_int, [_p, _p]),
    "llava_context_peer_connect": (_int, [_p, _p]),
    "llava_tp_shape": (_int, [_int, _u32, _u32, _u32, _u32, _u32, _u32p, _u32p, _u32p, C.POINTER(_u64)]),
    "llava_tp_pack": (_int, [_p, _int, _u32, _u32, _u32, _u32, _u32, _p]),
    "llava_context_close": (None, [_p]),
    "llava_context_lv": (_p, [_p]),
    "llava_context_run": (_int, [_int, C.POINTER(C.c_char_p)]),
    "llava_session_create": (_p, [_p]),
    "llava_session_destroy": (None, [_p]),
    "llava_session_set_text": (_int, [_p, C.c_char_p, _sz]),
    "llava_session_add_text": (_int, [_p, C.c_char_p, _sz]),
    "llava_session_push_token": (_int, [_p, _u32]),
    "llava_session_predict_next_token": (_u32, [_p]),
    "llava_session_start_next_token_prediction": (_int, [_p]),
    "llava_session_finish_next_token_prediction": (_u32, [_p]),
    "llava_session_rewind": (None, [_p, _u32]),
    "llava_session_set_options": (_u32, [_p, _u32]),
    "llava_session_save_frame": (_u32, [_p, C.c_char_p]),
    "llava_session_snapshot": (_u32, [_p, C.c_char_p]),
    "llava_session_restore": (_u32, [_p, C.c_char_p]),
    "llava_session_get_token_count": (_u32, [_p]),
    "llava_session_get_tokens": (_u32, [_p, _p, _u32]),
    "llava_session_set_deterministic": (None, [_p, _int]),
    "llava_session_set_seed": (None, [_p, _u32]),
    "llava_session_set_host_sampler": (None, [_p, _int]),
    "llava_session_get_mirostat_mu": (C.c_float, [_p]),
    "llava_session_set_max_batch": (_int, [_p, _u32]),
    "llava_session_generate_greedy_on_device": (_int, [_p, _u32, _p]),
    "llava_session_enqueue_greedy_on_device": (_int, [_p, _u32]),
    "llava_session_collect_greedy_on_device": (_int, [_p, _p, _u32]),
    "llava_session_get_logits": (_int, [_p, _p, _u32]),
    "llava_session_get_backlog_size": (_u32, [_p]),
    "llava_session_get_tokens_in_gpu": (_u32, [_p]),
    "llava_session_step_kernel_launches": (_u32, [_p]),
    "llava_session_set_step_trace": (_int, [_p, _int]),
    "llava_session_read_step_trace": (_u64, [_p, _p, _u64, _p]),
    "llava_session_read_kv": (_int, [_p, _u32, _int, _u32, _u32, _p]),
    "llava_tp_snapshot_slice_offset": (_u64, [_u32, _u32, _u32, _u32, _u32, _u32, _u32]),
    "llava_tp_snapshot_file_size": (_u64, [_u32, _u32, _u32]),
    "llava_wrapper_owner_create": (_p, [_p]),
    "llava_wrapper_owner_destroy": (None, [_p]),
    "llava_wrapper_owner_dead_sessions": (_u32, [_p]),
    "llava_wrapper_owner_pop": (_int, [_p, _int, _u32p, _u32p, _u32p, _u32p, _p, _u32, _u32p]),
    "llava_wrapper_create": (_p, [_p, _int]),
    "llava_wrapper_session_id": (_u32, [_p]),
    "llava_wrapper_start": (None, [_p]),
    "llava_wrapper_push_order": (None, [_p, _u32, _u32, _u32, _u32, C.c_char_p, _sz]),
    "llava_wrapper_join": (None, [_p]),
    "llava_wrapper_destroy": (None, [_p]),
    "llava_session_group_create": (_p, [_p, C.POINTER(_p), _u32]),
    "llava_session_group_destroy": (None, [_p]),
    "llava_session_group_step": (_int, [_p, _u32p]),
    "llava_session_group_generate_greedy_on_device": (_int, [_p, _u32, _u32p]),
    "llava_session_group_get_logits": (_int, [_p, _u32, _p, _u32]),
    "llava_session_group_kernel_launches": (_u32, [_p]),
    "llava_server_create": (_p, [_p, _u32, C.c_char_p, _int]),
    "llava_server_port": (_u32, [_p]),
    "llava_server_grouped_steps": (_u64, [_p]),
    "llava_server_grouped_tokens": (_u64, [_p]),
    "llava_server_steps_ahead": (_u64, [_p]),
    "llava_server_scheduler_collect_us": (_u64, [_p]),
    "llava_server_scheduler_device_us": (_u64, [_p]),
    "llava_server_start": (None, [_p]),
    "llava_server_stop": (None, [_p]),
    "llava_server_destroy": (None, [_p]),
}

NO_TOKEN = 0xFFFFFFFF
GEOMETRY = {   # dim, n_heads, ff_size, full depth
    "7b": (4096, 32, 11008, 32),
    "13b": (5120, 40, 13824, 40),
}


def load_host():
    """Loads libllava_host.so (and liblv_b200.so, which it links); raises if not built."""
    global _host
    if _host is None:
        load_kernels()
        if not os.path.exists(HOST_LIB):
            raise RuntimeError(f"{HOST_LIB} is missing: run `python llama-vulkan_b200/build.py`")
        lib = C.CDLL(HOST_LIB)
        _declare(lib, HOST_API)
        _host = lib
    return _host


def write_synthetic_model(path, geometry="7b", n_layers=None, wtype=TYPE_Q4_0, vocab=32000, seed=1234, threads=0, file_version=3,
                          f32_embeddings=False):
    """Writes a seeded synthetic ggjt model file (version 3, or 1 for the old q4_0 block layout) and returns its size in bytes."""
    dim, heads, ff, depth = GEOMETRY[geometry]
    n_layers = depth if n_layers is None else n_layers
    if not load_host().llava_synth_write_ex(os.fsencode(path), dim, heads, n_layers, ff, vocab, wtype, seed, threads, file_version,
                                            int(f32_embeddings)):
        raise RuntimeError(f"cannot write synthetic model {path}")
    return os.path.getsize(path)


class ModelFile:
    """ggml_file: header, tensor table, tokenizer (no GPU needed)."""

    def __init__(self, path):
        self.lib = load_host()
        self.handle = self.lib.ggml_file_open(os.fsencode(path))
        if not self.handle:
            raise RuntimeError(f"cannot open model {path}")
        h = (_u32 * 10)()
        self.lib.ggml_file_header(self.handle, h)
        (self.magic, self.file_version, self.vocab_size, self.dim, self.multiple_of, self.n_heads, self.n_layers,
         self.rot, self.ftype, self.ff_size) = list(h)

    def close(self):
        if self.handle:
            self.lib.ggml_file_close(self.handle)
            self.handle = None

    def tensors(self):
        out = []
        name = C.create_string_buffer(256)
        t, s1, s2 = _u32(), _u32(), _u32()
        off, size = _u64(), _u64()
        for i in range(self.lib.ggml_file_n_tensors(self.handle)):
            self.lib.ggml_file_tensor(self.handle, i, name, 256, C.byref(t), C.byref(off), C.byref(s1), C.byref(s2), C.byref(size))
            out.append((name.value.decode(), t.value, off.value, s1.value, s2.value, size.value))
        return out

    def tokenize(self, text, bos=True):
        data = text if isinstance(text, bytes) else text.encode("utf-8")
        cap = len(data) + 2
        buf = (_u32 * cap)()
        n = self.lib.ggml_file_tokenize(self.handle, data, len(data), int(bos), buf, cap)
        return list(buf[:n])

    def tokens_to_text(self, tokens):
        arr = (_u32 * len(tokens))(*tokens)
        n = self.lib.ggml_file_tokens_to_text(self.handle, arr, len(tokens), None, 0)
        out = C.create_string_buffer(n + 1)
        self.lib.ggml_file_tokens_to_text(self.handle, arr, len(tokens), out, n)
        return out.raw[:n]

    def token(self, i):
        score = C.c_float()
        n = self.lib.ggml_file_token(self.handle, i, None, 0, C.byref(score))
        out = C.create_string_buffer(n + 1)
        self.lib.ggml_file_token(self.handle, i, out, n, C.byref(score))
        return out.raw[:n], score.value


class HostContext:
    """llava_context: model + device + uploaded layers."""

    def __init__(self, model_path, device=0, rank=0, n_ranks=1, nccl_id=None):
        self.lib = load_host()
        if device is None:            # the model file only: no device context, no sessions
            self.handle = self.lib.llava_context_open_model_only(os.fsencode(model_path))
        elif n_ranks == 1:
            self.handle = self.lib.llava_context_open(os.fsencode(model_path), device)
        else:
            buf = (C.c_uint8 * 128).from_buffer_copy(bytes(nccl_id))
            self.handle = self.lib.llava_context_open_sharded(os.fsencode(model_path), device, rank, n_ranks, buf)
        if not self.handle:
            raise RuntimeError(f"llava_context::open({model_path}) failed: "
                               + (load_kernels().lv_last_error_string() or b"").decode("utf-8", "replace"))

    def close(self):
        if self.handle:
            self.lib.llava_context_close(self.handle)
            self.handle = None

    def peer_window_handle(self):
        """Creates this rank's peer window; returns its 64-byte CUDA IPC handle."""
        buf = (C.c_uint8 * 64)()
        if not self.lib.llava_context_peer_window_create(self.handle, buf):
            raise RuntimeError("peer window creation failed")
        return bytes(buf)

    def peer_connect(self, handles):
        """handles: the 64-byte handles of all ranks, in rank order."""
        blob = b"".join(handles)
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        if not self.lib.llava_context_peer_connect(self.handle, buf):
            raise RuntimeError("peer connect failed: " + (load_kernels().lv_last_error_string() or b"").decode("utf-8", "replace"))

    def session(self):
        return Session(self)

    def set_exact_batched_products(self, on):
        """Batched (prompt) q4_0 products with the exact hi/lo weight planes instead of one fp16 plane (lv_gemm_tc_set_exact).
        Takes effect for steps recorded afterwards: set it before the session evaluates its first batch."""
        check(load_kernels().lv_gemm_tc_set_exact(_p(self.lib.llava_context_lv(self.handle)), int(bool(on))))


class Session:
    """llava_session."""

    def __init__(self, ctx):
        self.lib = ctx.lib
        self.ctx = ctx
        self.handle = self.lib.llava_session_create(ctx.handle)

    def close(self):
        if self.handle:
            self.lib.llava_session_destroy(self.handle)
            self.handle = None

    def push_token(self, t):
        return bool(self.lib.llava_session_push_token(self.handle, t))

    def set_text(self, text):
        data = text if isinstance(text, bytes) else text.encode("utf-8")
        return bool(self.lib.llava_session_set_text(self.handle, data, len(data)))

    def add_text(self, text):
        data = text if isinstance(text, bytes) else text.encode("utf-8")
        return bool(self.lib.llava_session_add_text(self.handle, data, len(data)))

    def predict_next_token(self):
        return self.lib.llava_session_predict_next_token(self.handle)

    def start_next_token_prediction(self):
        return bool(self.lib.llava_session_start_next_token_prediction(self.handle))

    def finish_next_token_prediction(self):
        return self.lib.llava_session_finish_next_token_prediction(self.handle)

    def rewind(self, n):
        self.lib.llava_session_rewind(self.handle, n)

    def set_options(self, o):
        return self.lib.llava_session_set_options(self.handle, o)

    def save_frame(self, path):
        return self.lib.llava_session_save_frame(self.handle, os.fsencode(path))

    def snapshot(self, path):
        return self.lib.llava_session_snapshot(self.handle, os.fsencode(path))

    def restore(self, path):
        return self.lib.llava_session_restore(self.handle, os.fsencode(path))

    def tokens(self):
        n = self.lib.llava_session_get_token_count(self.handle)
        buf = (_u32 * max(n, 1))()
        self.lib.llava_session_get_tokens(self.handle, buf, n)
        return list(buf[:n])

    def set_deterministic(self, on=True):
        self.lib.llava_session_set_deterministic(self.handle, int(on))

    def set_seed(self, seed):
        self.lib.llava_session_set_seed(self.handle, seed)

    def set_host_sampler(self, on=True):
        """Non-greedy tokens from the host sampler (std::discrete_distribution, as the reference) instead of the device one."""
        self.lib.llava_session_set_host_sampler(self.handle, int(on))

    def mirostat_mu(self):
        return self.lib.llava_session_get_mirostat_mu(self.handle)

    def set_max_batch(self, n):
        return bool(self.lib.llava_session_set_max_batch(self.handle, n))

    def generate_greedy_on_device(self, n):
        buf = (_u32 * n)()
        if not self.lib.llava_session_generate_greedy_on_device(self.handle, n, buf):
            raise RuntimeError("generate_greedy_on_device failed")
        return list(buf)

    def enqueue_greedy_on_device(self, n):
        if not self.lib.llava_session_enqueue_greedy_on_device(self.handle, n):
            raise RuntimeError("enqueue_greedy_on_device failed")
        self._enqueued = n

    def collect_greedy_on_device(self):
        n = self._enqueued
        buf = (_u32 * n)()
        if not self.lib.llava_session_collect_greedy_on_device(self.handle, buf, n):
            raise RuntimeError("collect_greedy_on_device failed")
        return list(buf)

    def logits(self, vocab):
        import numpy as np
        out = np.empty(vocab, np.float32)
        if not self.lib.llava_session_get_logits(self.handle, out.ctypes.data_as(_p), vocab):
            raise RuntimeError("get_logits failed")
        return out

    def backlog_size(self):
        return self.lib.llava_session_get_backlog_size(self.handle)

    def tokens_in_gpu(self):
        return self.lib.llava_session_get_tokens_in_gpu(self.handle)

    def step_kernel_launches(self):
        """Kernel launches of one replay of the step evaluated last."""
        return self.lib.llava_session_step_kernel_launches(self.handle)

    def set_step_trace(self, on=True):
        return bool(self.lib.llava_session_set_step_trace(self.handle, int(on)))

    def read_step_trace(self):
        """[operation][CTA][point] nanosecond stamps of the last traced one-launch step, or None."""
        import numpy as np
        buf = np.zeros(1 << 21, np.uint64)
        dims = (_u32 * 3)()
        n = self.lib.llava_session_read_step_trace(self.handle, buf.ctypes.data_as(_p), buf.size, dims)
        return buf[:n].reshape(dims[0], dims[1], dims[2]).copy() if n else None

    def read_kv(self, layer, which, row0, nrows, dim):
        import numpy as np
        out = np.empty((nrows, dim), np.uint16)
        if not self.lib.llava_session_read_kv(self.handle, layer, which, row0, nrows, out.ctypes.data_as(_p)):
            raise RuntimeError("read_kv failed")
        return out


class SessionGroup:
    """llava_session_group: one greedy decoding step for several sessions with one pass over the weights."""

    def __init__(self, ctx, sessions):
        self.lib = ctx.lib
        self.sessions = list(sessions)
        arr = (_p * len(self.sessions))(*[s.handle for s in self.sessions])
        self.handle = self.lib.llava_session_group_create(ctx.handle, arr, len(self.sessions))
        if not self.handle:
            raise RuntimeError("these sessions cannot form a group")

    def close(self):
        if self.handle:
            self.lib.llava_session_group_destroy(self.handle)
            self.handle = None

    def step(self):
        """-> the greedy next token of every member (not pushed), or None on failure."""
        out = (_u32 * len(self.sessions))()
        return list(out) if self.lib.llava_session_group_step(self.handle, out) else None

    def generate_greedy_on_device(self, n):
        """n steps with the tokens fed back on the device -> per member its n tokens (appended to the members' buffers)."""
        k = len(self.sessions)
        out = (_u32 * (k * n))()
        if not self.lib.llava_session_group_generate_greedy_on_device(self.handle, n, out):
            return None
        return [list(out[i * n:(i + 1) * n]) for i in range(k)]

    def logits(self, member, vocab):
        import numpy as np
        v = np.empty(vocab, np.float32)
        if not self.lib.llava_session_group_get_logits(self.handle, member, v.ctypes.data_as(_p), vocab):
            raise RuntimeError("no logits")
        return v

    def kernel_launches(self):
        return self.lib.llava_session_group_kernel_launches(self.handle)


class Server:
    """lsrv::tlv_server on a thread of its own: the TCP front end of the session protocol
    (reference server/server.cpp:44-331).  `port` 0 binds any free port; read it back from `.port`."""

    def __init__(self, ctx, port=0, address="127.0.0.1", deterministic=False):
        self.lib = ctx.lib
        self.handle = self.lib.llava_server_create(ctx.handle, port, address.encode(), int(deterministic))
        if not self.handle:
            raise RuntimeError(f"cannot listen on {address}:{port}")
        self.port = self.lib.llava_server_port(self.handle)
        self.lib.llava_server_start(self.handle)

    def grouped(self):
        """-> (rounds that stepped two or more sessions together, tokens those rounds produced)."""
        return self.lib.llava_server_grouped_steps(self.handle), self.lib.llava_server_grouped_tokens(self.handle)

    def scheduler_times(self):
        """-> (microseconds the scheduler's rounds waited for their callers, microseconds they waited for the device)."""
        return self.lib.llava_server_scheduler_collect_us(self.handle), self.lib.llava_server_scheduler_device_us(self.handle)

    def steps_ahead(self):
        """Grouped steps that were already queued on the device when their sessions asked for them."""
        return self.lib.llava_server_steps_ahead(self.handle)

    def close(self):
        if self.handle:
            self.lib.llava_server_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class Client:
    """A blocking client of the session protocol: frames of {u32 command, u32 request id, u32 length, payload}
    out, {u32 reply opcode, u32 request id (0 = broadcast), u32 size, payload} back
    (reference server/client.cpp:116-144 and 302-313)."""

    # requests (server/types.h:50-71) and replies (server/types.h:73-84)
    GET_TOKEN_MAP, NEW_SESSION, LIST_SESSIONS = 0, 1, 2
    GET_SESSION_TOKENS, SUBSCRIBE, UNSUBSCRIBE, KILL_SESSION, START, STOP, TICK, GET_STATUS = 16, 17, 18, 19, 20, 21, 22, 23
    REWIND, ADD_TOKEN, ADD_TEXT, SET_OPTIONS, SAVE_FRAME, SNAPSHOT, RESTORE = 32, 33, 34, 35, 36, 37, 38
    NEW_TOKEN, BUFFER, TOKEN_MAP, SESSION_CREATED, SESSION_LIST, DROPPED_SESSION, ACK, STATUS = range(8)

    def __init__(self, port, address="127.0.0.1", timeout=30.0):
        import socket
        self.sock = socket.create_connection((address, port), timeout=timeout)
        self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self._request = 0

    def close(self):
        self.sock.close()

    def send(self, command, payload=b"", request_id=None):
        """Sends one request; returns its request id."""
        if request_id is None:
            self._request += 1
            request_id = self._request
        self.sock.sendall(struct.pack("<III", command, request_id, len(payload)) + payload)
        return request_id

    def _exactly(self, n):
        parts = []
        while n:
            b = self.sock.recv(n)
            if not b:
                raise ConnectionError("server closed the connection")
            parts.append(b)
            n -= len(b)
        return b"".join(parts)

    def recv(self):
        """-> (reply opcode, request id, payload) of the next packet."""
        op, request_id, size = struct.unpack("<III", self._exactly(12))
        return op, request_id, self._exactly(size)

    def call(self, command, payload=b""):
        """Sends a request and returns (opcode, payload) of the reply that carries its id; packets that arrive
        in between (broadcasts, other replies) are collected in `.others`."""
        rid = self.send(command, payload)
        self.others = []
        while True:
            op, got, data = self.recv()
            if got == rid:
                return op, data
            self.others.append((op, got, data))

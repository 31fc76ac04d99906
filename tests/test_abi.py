"""The C-ABI library loads and exports every symbol include/lv_b200.h declares (CPU only: no compute calls)."""
import os
import re

from conftest import ROOT, load_pkg


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lv_[a-z0-9_]+|llava_[a-z0-9_]+|ggml_[a-z0-9_]+)\s*\(", text)))


def test_kernel_library_exports_every_declared_symbol():
    pkg = load_pkg()
    lib = pkg.load_kernels()
    names = [n for n in _declared("lv_b200.h") if n.startswith("lv_")]
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/lv_b200.h but not exported"
        assert n in pkg.KERNEL_API, f"{n} has no ctypes signature"


def test_status_codes_match_the_header():
    pkg = load_pkg()
    text = open(os.path.join(ROOT, "include", "lv_b200.h")).read()
    for name in ("LV_OK", "LV_ERR_NOK", "LV_ERR_BAD_ARGUMENTS", "LV_ERR_CUDA", "LV_ERR_DEVICE_WAIT", "LV_ERR_TIMEOUT", "LV_ERR_COMM"):
        m = re.search(name + r"\s*=\s*(\d+)", text)
        assert m and int(m.group(1)) == getattr(pkg, name)


def test_calls_without_a_gpu_fail_with_a_status_not_a_crash():
    pkg = load_pkg()
    lib = pkg.load_kernels()
    import ctypes as C
    n = C.c_int(-1)
    rc = lib.lv_device_count(C.byref(n))
    if rc == pkg.LV_OK and n.value > 0:
        return                                    # a GPU is present: covered by the gpu tests
    h = C.c_void_p()
    assert lib.lv_ctx_create(0, C.byref(h)) != pkg.LV_OK
    assert lib.lv_last_error_string()

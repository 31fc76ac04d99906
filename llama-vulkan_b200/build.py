"""Builds the native libraries of this package in-tree with nvcc / g++.

    python llama-vulkan_b200/build.py [--force]

Outputs (next to this file): liblv_b200.so (sm_100a kernels + C ABI),
libllava_host.so (C++ host surface) and the vulkan_llama command-line tool.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math=false", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found")
    return nvcc


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def _glob(d, exts):
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(exts))


def build_kernels(force=False, verbose_ptxas=False):
    """Compiles every .cu file to an object of its own (in parallel, only the stale ones) and links them."""
    from concurrent.futures import ThreadPoolExecutor
    cu = _glob(CSRC, (".cu",))
    headers = _glob(CSRC, (".cuh", ".h")) + [os.path.join(ROOT, "include", "lv_b200.h")]
    out = os.path.join(HERE, "liblv_b200.so")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    if verbose_ptxas:
        flags += ["-Xptxas", "-v"]
    objs, stale = [], []
    for src in cu:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or verbose_ptxas or _newer(obj, [src] + headers):
            stale.append((src, obj))
    with ThreadPoolExecutor(max_workers=max(1, min(len(stale), os.cpu_count() or 1))) as pool:
        list(pool.map(lambda so: _run([_nvcc(), "-c", "-o", so[1]] + flags + [so[0]]), stale))
    if stale or not os.path.exists(out):
        _run([_nvcc(), "-shared", "-o", out, "-gencode", "arch=compute_100a,code=sm_100a"] + objs + ["-lcudart", "-ldl"])
    return out


def build_host(force=False):
    if not os.path.isdir(HOST):
        return None
    cpp = [f for f in _glob(HOST, (".cpp",)) if not f.endswith("main.cpp")] + _glob(os.path.join(HOST, "server"), (".cpp",))
    if not cpp:
        return None
    deps = cpp + _glob(HOST, (".h",)) + _glob(os.path.join(HOST, "server"), (".h",)) + [os.path.join(ROOT, "include", "lv_b200.h"), os.path.join(ROOT, "include", "llava_host.h")]
    deps = [d for d in deps if os.path.exists(d)]
    out = os.path.join(HERE, "libllava_host.so")
    cxx = shutil.which("g++") or "g++"
    if force or _newer(out, deps):
        _run([cxx, "-std=c++20", "-O2", "-fPIC", "-shared", "-pthread", "-Wall", "-o", out] + cpp +
             ["-L" + HERE, "-llv_b200", "-Wl,-rpath,$ORIGIN", "-Wl,-Bsymbolic"])
    main = os.path.join(HOST, "main.cpp")
    exe = os.path.join(HERE, "vulkan_llama")
    if os.path.exists(main) and (force or _newer(exe, [main, out])):
        _run([cxx, "-std=c++20", "-O2", "-pthread", "-o", exe, main, "-L" + HERE, "-lllava_host", "-llv_b200",
              "-Wl,-rpath,$ORIGIN"])
    return out


def build_all(force=False):
    k = build_kernels(force)
    h = build_host(force)
    return k, h


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)

#!/usr/bin/env python
"""Kernel microbenchmark of the quantised GEMV family (seeded N(0, 0.02)
weights, N(0, 1) activations), one line of JSON per shape:

    python microbench.py [--shape NAME ...] [--wtype q4_0|q8_0] [--batch Z] [--tc] [--iters N]

With --tc the plain / add / silu shapes run on the tensor cores (lv_gemm_tc*, batch 1..64,
q4_0), otherwise the GEMV reads the matrix once per token of the batch; TFLOP/s =
2 * rows * cols * batch / time is reported beside GB/s.

Every timed launch reads a different copy of the matrix from a ring of copies
larger than the 126 MB L2, so the figure is HBM bandwidth, not L2 bandwidth.
GB/s = quantised matrix bytes / time.
"""
import argparse
import ctypes as C
import importlib.util
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
HERE = os.path.join(ROOT, "llama-vulkan_b200")
sys.path.insert(0, os.path.join(ROOT, "tests"))

SHAPES = {                      # rows, cols, kind
    "wq": (4096, 4096, "plain"),
    "gate_up": (11008, 4096, "silu"),
    "w2": (4096, 11008, "add"),
    "w2_13b": (5120, 13824, "add"),
    "head": (32000, 4096, "plain"),
    "tiny": (592, 4096, "plain"),        # one row group per SM: the fixed cost of a launch
    "tiny_ff": (592, 11008, "plain"),
    "tiny_norm": (592, 4096, "norm"),
    "qkv": (4096, 4096, "qkv"),          # norm + wk, wq, wv (3 x 4096 rows) + cache append
    "attn": (4096, 4096, "attn"),        # fused attention, 32 heads, --pos rows in the cache
}


def load_pkg():
    name = "llama_vulkan_b200"
    if name not in sys.modules:
        spec = importlib.util.spec_from_file_location(name, os.path.join(HERE, "__init__.py"), submodule_search_locations=[HERE])
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return sys.modules[name]


def group_steps(args):
    """K sessions, each with its own 32-token prompt, then args.iters shared steps (one pass over the weights per step)."""
    import time
    import numpy as np
    pkg = load_pkg()
    wt = 2 if args.wtype == "q4_0" else 8
    path = os.path.join(os.environ.get("LV_MODEL_DIR", "/tmp/lv_models"), f"7b_L{args.layers}_t{wt}_seed1234.ggjt")
    os.makedirs(os.path.dirname(path), exist_ok=True)
    if not os.path.exists(path):
        pkg.write_synthetic_model(path, "7b", n_layers=args.layers, wtype=wt)
    ctx = pkg.HostContext(path, 0)
    sessions = []
    for i in range(args.sessions):
        s = ctx.session()
        s.set_deterministic(True)
        assert s.set_max_batch(64)
        for t in np.random.default_rng(1000 + i).integers(3, 32000, 32):
            assert s.push_token(int(t))
        tok = s.predict_next_token()
        assert tok != pkg.NO_TOKEN and s.push_token(tok)
        sessions.append(s)
    group = pkg.SessionGroup(ctx, sessions)
    assert group.generate_greedy_on_device(2) is not None          # records the step
    t0 = time.perf_counter()
    assert group.generate_greedy_on_device(args.iters) is not None
    sec = time.perf_counter() - t0
    print(json.dumps({"sessions": args.sessions, "layers": args.layers, "wtype": args.wtype, "steps": args.iters,
                      "ms_per_step": sec * 1e3 / args.iters, "tokens_per_s": args.sessions * args.iters / sec,
                      "launches_per_step": group.kernel_launches()}), flush=True)
    group.close()
    for s in sessions:
        s.close()
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", nargs="*", default=sorted(SHAPES))
    ap.add_argument("--wtype", default="q4_0", choices=["q4_0", "q8_0"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--tc", action="store_true", help="batched product on the tensor cores instead of one GEMV per token")
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--ring-mb", type=int, default=400)
    ap.add_argument("--pos", type=int, default=200, help="cache rows already filled, for the attn shape")
    ap.add_argument("--copies", type=int, default=0,
                    help="override the ring length; 1 keeps the matrix resident in L2 and shows the kernel's compute ceiling")
    ap.add_argument("--sessions", type=int, default=0,
                    help="instead of single products: K sessions of the 7B model (--layers, --wtype) decoding together through "
                         "llava_session_group, --iters steps fed back on the device; prints the time per shared step")
    ap.add_argument("--layers", type=int, default=32)
    args = ap.parse_args()
    if args.sessions:
        return group_steps(args)

    import numpy as np
    import torch
    import quant_np as qn
    pkg = load_pkg()
    wtype = qn.Q4_0 if args.wtype == "q4_0" else qn.Q8_0
    peak = 6520.5
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = float(json.load(open(p))["hbm_gbs"])
    with pkg.Context(0) as gpu:
        lib, h = gpu.lib, gpu.handle
        stream = torch.cuda.ExternalStream(lib.lv_ctx_stream(h), device=0)
        rng = np.random.default_rng(99)
        for name in args.shape:
            rows, cols, kind = SHAPES[name]
            nmat = {"silu": 2, "qkv": 3}.get(kind, 1)
            rb = qn.row_bytes(wtype, cols)
            slab_rows = 256
            slab = qn.quantize((rng.standard_normal((slab_rows, cols)) * 0.02).astype(np.float32), wtype)
            host = np.tile(slab, -(-rows // slab_rows))[: rows * rb]
            mat_bytes = rows * rb
            copies = args.copies if args.copies > 0 else max(3, int(args.ring_mb * 1e6 // (nmat * mat_bytes)) + 1)
            ring = gpu.alloc(copies * nmat * mat_bytes)
            for i in range(copies * nmat):
                pkg.check(lib.lv_upload(h, pkg.offset(ring, i * mat_bytes), host.ctypes.data_as(C.c_void_p), mat_bytes))
            x = gpu.upload(rng.standard_normal((args.batch, cols)).astype(np.float32))
            out = gpu.zeros(args.batch * rows * 4)

            if kind in ("norm", "silu"):
                nw = gpu.upload((1 + 0.01 * rng.standard_normal(cols)).astype(np.float32))
            if kind in ("qkv", "attn"):
                ctx_rows = 2048
                kc, vc = gpu.zeros(ctx_rows * rows * 2), gpu.zeros(ctx_rows * rows * 2)
                if kind == "attn":
                    fill = (rng.standard_normal((args.pos + 1, rows)) * 0.5).astype(np.float16)
                    for c in (kc, vc):
                        pkg.check(lib.lv_upload(h, c, fill.ctypes.data_as(C.c_void_p), fill.nbytes))
                nw = gpu.upload((1 + 0.01 * rng.standard_normal(cols)).astype(np.float32))
                dpos = gpu.upload(np.array([args.pos] * 4, np.uint32))
                table = gpu.alloc(ctx_rows * 128 * 4)
                pkg.check(lib.lv_rope_table_build(h, table, ctx_rows, 128))
                backlog = 128
                while backlog <= args.pos:
                    backlog *= 2
                scratch = gpu.zeros(lib.lv_attention_scratch_bytes(rows // 128, 128, ctx_rows, 1))

            if args.tc:
                xh = gpu.alloc(lib.lv_act_split_bytes(cols, args.batch))
                pkg.check(lib.lv_act_split_f16(h, xh, x, None, cols, args.batch))

            def launch(i):
                w = pkg.offset(ring, (i % copies) * nmat * mat_bytes)
                if args.tc and kind in ("plain", "add", "norm"):
                    pkg.check(lib.lv_gemm_tc(h, out, w, wtype, xh, rows, cols, args.batch, 1 if kind == "add" else 0))
                elif args.tc and kind == "silu":
                    pkg.check(lib.lv_gemm_tc_silu(h, out, w, pkg.offset(w, mat_bytes), wtype, xh, rows, cols, args.batch))
                elif kind == "qkv":
                    pkg.check(lib.lv_norm_qkv_kvappend(h, out, kc, vc, w, pkg.offset(w, mat_bytes), pkg.offset(w, 2 * mat_bytes), wtype,
                                                       x, nw, dpos, rows, cols, 1, ctx_rows))
                elif kind == "attn":
                    pkg.check(lib.lv_attention_fused(h, out, x, kc, vc, dpos, table, scratch, rows // 128, 128, backlog, 1))
                elif kind == "norm":
                    pkg.check(lib.lv_norm_gemv(h, out, w, wtype, x, nw, rows, cols, args.batch))
                elif kind == "silu":
                    pkg.check(lib.lv_norm_gate_up_silu(h, out, w, pkg.offset(w, mat_bytes), wtype, x, nw, rows, cols, args.batch))   # as the decode step calls it
                else:
                    pkg.check(lib.lv_gemv(h, out, w, wtype, x, rows, cols, args.batch, 1 if kind == "add" else 0))

            for i in range(min(copies, 8)):
                launch(i)
            gpu.sync()
            # the launches are recorded into one CUDA graph so that the host's launch rate does
            # not limit the figure
            graph = C.c_void_p()
            pkg.check(lib.lv_graph_begin_capture(h))
            for i in range(args.iters):
                launch(i)
            pkg.check(lib.lv_graph_end_capture(h, C.byref(graph)))
            pkg.check(lib.lv_graph_launch(h, graph))
            gpu.sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            pkg.check(lib.lv_graph_launch(h, graph))
            e1.record(stream)
            gpu.sync()
            pkg.check(lib.lv_graph_destroy(graph))
            sec = e0.elapsed_time(e1) * 1e-3 / args.iters
            nbytes = nmat * mat_bytes if kind != "attn" else 2 * (args.pos + 1) * rows * 2
            gbs = nbytes / sec / 1e9
            print(json.dumps({"shape": name, "rows": rows, "cols": cols, "kind": kind, "wtype": args.wtype, "batch": args.batch,
                              "path": "tcgen05" if args.tc else "gemv", "us_per_launch": sec * 1e6, "bytes": nbytes, "GB/s": gbs,
                              "frac_of_measured_hbm": gbs / peak, "TFLOP/s": 2.0 * nmat * rows * cols * args.batch / sec / 1e12,
                              "ring_copies": copies}), flush=True)
            for d in (ring, x, out):
                gpu.free(d)


if __name__ == "__main__":
    main()

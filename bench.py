#!/usr/bin/env python
"""Decode-throughput benchmark of the B200 path (and, with --impl reference, of
the CPU restatement of the reference's path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one decoded token: one pass of the per-token hot path (embedding
row, 32 x {norm+QKV+cache append, attention, wo+residual, norm+gate/up+SiLU,
w2+residual}, final norm, output head, argmax).  The default workload is
LLaMA-7B q4_0 with seeded synthetic weights: a 64-token seeded prompt is
ingested (untimed), then W warm-up tokens and exactly K timed greedy tokens.
Prints one JSON line on rank 0.
"""
import argparse
import ctypes as C
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "tests"))

WORKLOADS = {
    # name: geometry, layers (None = full depth), type code, prompt tokens, BASELINE.json config index
    "7b-q4_0": dict(geometry="7b", n_layers=None, wtype=2, prompt=64, config=1),
    "7b-q8_0": dict(geometry="7b", n_layers=None, wtype=8, prompt=1024, config=2),
    "13b-q4_0": dict(geometry="13b", n_layers=None, wtype=2, prompt=128, config=3),
    "tiny-q4_0": dict(geometry="7b", n_layers=2, wtype=2, prompt=16, config=0),
}
PROMPT_SEED = 4321
MODEL_DIR = os.environ.get("LV_MODEL_DIR", "/tmp/lv_models")


def load_pkg():
    name = "llama_vulkan_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(ROOT, "llama-vulkan_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def model_geometry(pkg, w):
    dim, heads, ff, depth = pkg.GEOMETRY[w["geometry"]]
    return dim, heads, ff, (depth if w["n_layers"] is None else w["n_layers"])


def weight_bytes_per_token(dim, ff, n_layers, vocab, wtype):
    """Bytes of weights one decoded token streams: every layer matrix and norm
    vector, the final norm, the output head and one embedding row."""
    bpb = 18 if wtype == 2 else 34
    per_layer = (4 * dim * dim + 3 * ff * dim) * bpb // 32 + 2 * dim * 4
    return n_layers * per_layer + vocab * dim * bpb // 32 + dim * 4 + dim * bpb // 32


def kv_bytes_per_token(dim, n_layers, pos):
    """f16 K and V rows read (pos + 1 each) and written (one each) per layer."""
    return n_layers * (2 * (pos + 1) * dim * 2 + 2 * dim * 2)


def ensure_model(pkg, name, w, rank, world):
    os.makedirs(MODEL_DIR, exist_ok=True)
    dim, heads, ff, n_layers = model_geometry(pkg, w)
    path = os.path.join(MODEL_DIR, f"{w['geometry']}_L{n_layers}_t{w['wtype']}_seed1234.ggjt")
    want = pkg.load_host().llava_synth_file_size(dim, heads, n_layers, ff, 32000, w["wtype"])
    done = path + ".done"
    if rank == 0:
        if not (os.path.exists(done) and os.path.exists(path) and os.path.getsize(path) == want):
            t0 = time.time()
            pkg.write_synthetic_model(path, w["geometry"], n_layers=n_layers, wtype=w["wtype"])
            open(done, "w").write("ok")
            print(f"[bench] wrote {path} ({want / 1e9:.2f} GB) in {time.time() - t0:.1f} s", file=sys.stderr)
    else:
        while not (os.path.exists(done) and os.path.getsize(path) == want):
            time.sleep(0.5)
    return path


def prompt_tokens(n):
    import numpy as np
    return [int(t) for t in np.random.default_rng(PROMPT_SEED).integers(3, 32000, n)]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.rows, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def time_dominant_kernel(pkg, ctx_handle_lv, dim, ff, wtype, stream, torch):
    """Average duration of the gate/up SiLU GEMV (the kernel that moves the most
    bytes per launch), launched back to back on a ring of matrix copies larger
    than L2.  Returns (seconds per launch, algorithmic bytes per launch)."""
    import numpy as np
    import quant_np as qn
    lib = pkg.load_kernels()
    rng = np.random.default_rng(99)
    rows_sample = 512                                   # quantise a slab once, tile it to the full matrix
    slab = qn.quantize((rng.standard_normal((rows_sample, dim)) * 0.02).astype(np.float32), wtype)
    rb = qn.row_bytes(wtype, dim)
    mat_bytes = ff * rb
    reps = -(-ff // rows_sample)
    host = np.tile(slab, reps)[:mat_bytes]
    copies = max(3, int(400e6 // (2 * mat_bytes)) + 1)  # > 400 MB in the ring, well over the 126 MB L2
    d = C.c_void_p()
    pkg.check(lib.lv_arena_create(ctx_handle_lv, copies * 2 * mat_bytes + ff * 4 + 2 * dim * 4, C.byref(d)))
    for i in range(copies * 2):
        pkg.check(lib.lv_upload(ctx_handle_lv, C.c_void_p(d.value + i * mat_bytes), host.ctypes.data_as(C.c_void_p), mat_bytes))
    x = rng.standard_normal(dim).astype(np.float32)
    dx = C.c_void_p(d.value + copies * 2 * mat_bytes)
    dnorm = C.c_void_p(dx.value + dim * 4)
    dout = C.c_void_p(dnorm.value + dim * 4)
    norm_w = (1.0 + 0.01 * rng.standard_normal(dim)).astype(np.float32)
    pkg.check(lib.lv_upload(ctx_handle_lv, dx, x.ctypes.data_as(C.c_void_p), dim * 4))
    pkg.check(lib.lv_upload(ctx_handle_lv, dnorm, norm_w.ctypes.data_as(C.c_void_p), dim * 4))
    def launch(i):
        w3 = C.c_void_p(d.value + (2 * (i % copies)) * mat_bytes)
        w1 = C.c_void_p(w3.value + mat_bytes)
        pkg.check(lib.lv_norm_gate_up_silu(ctx_handle_lv, dout, w3, w1, wtype, dx, dnorm, ff, dim, 1))   # as the decode step calls it
    for i in range(copies):
        launch(i)
    pkg.check(lib.lv_stream_sync(ctx_handle_lv, 0))
    n = 20 * copies
    graph = C.c_void_p()                      # one graph of n launches: the host's launch rate stays out of the figure
    pkg.check(lib.lv_graph_begin_capture(ctx_handle_lv))
    for i in range(n):
        launch(i)
    pkg.check(lib.lv_graph_end_capture(ctx_handle_lv, C.byref(graph)))
    pkg.check(lib.lv_graph_launch(ctx_handle_lv, graph))
    pkg.check(lib.lv_stream_sync(ctx_handle_lv, 0))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    pkg.check(lib.lv_graph_launch(ctx_handle_lv, graph))
    e1.record(stream)
    pkg.check(lib.lv_stream_sync(ctx_handle_lv, 0))
    pkg.check(lib.lv_graph_destroy(graph))
    sec = e0.elapsed_time(e1) * 1e-3 / n
    pkg.check(lib.lv_arena_free(ctx_handle_lv, d))
    return sec, 2 * mat_bytes


def cpu_oracle_tokens_per_s(path, n_tokens, budget_s, threads=0):
    """Times the CPU oracle (full depth, all host threads) on the first tokens of
    the prompt; stops early once budget_s is used.  Returns (tokens/s, tokens timed, threads)."""
    import numpy as np
    import oracle_bind as ob
    lib = ob.load()
    if threads:
        lib.orc_set_threads(threads)
    model = lib.orc_model_open(os.fsencode(path))
    sess = lib.orc_session_create(model, 1024)
    info = ob.ModelInfo()
    lib.orc_model_get_info(model, C.byref(info))
    logits = np.empty(info.vocab_size, np.float32)
    toks = prompt_tokens(max(n_tokens, 1) + 1)
    lib.orc_session_push_token(sess, toks[0])
    lib.orc_session_eval(sess, ob.ptr(logits))         # warm the page cache / thread pool
    done, t0 = 0, time.perf_counter()
    while done < n_tokens:
        lib.orc_session_push_token(sess, toks[done + 1])
        lib.orc_session_eval(sess, ob.ptr(logits))
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    nthreads = lib.orc_get_threads()
    lib.orc_session_destroy(sess)
    lib.orc_model_close(model)
    return done / dt, done, nthreads


def run_reference(args, rank, world):
    """The reference arm: the reference's path restated for the CPU (oracle/),
    since its own implementation needs Vulkan, which does not exist on this box."""
    if rank != 0:
        return
    pkg = load_pkg()
    w = WORKLOADS[args.workload]
    path = ensure_model(pkg, args.workload, w, 0, 1)
    # bounded sample: whole-depth tokens, at most ~150 s in total
    for _ in range(min(args.warmup, 1)):
        cpu_oracle_tokens_per_s(path, 1, 30)
    tps, timed, threads = cpu_oracle_tokens_per_s(path, args.steps, 150.0)
    dim, heads, ff, n_layers = model_geometry(pkg, w)
    line = {
        "impl": "reference", "metric": "decode tokens/s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / tps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"LLaMA-{w['geometry'].upper()} {'q4_0' if w['wtype'] == 2 else 'q8_0'} decode, {n_layers} layers, "
                               "seeded synthetic ggjt-v3 weights, host cores only", "baseline_config_index": w["config"]},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{timed} whole-depth decode tokens at context 1..{timed + 1} (CPU restatement of the "
                                   "reference shaders; the reference's own Vulkan path is unavailable on this box)"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="7b-q4_0", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"],
                    help="N > 1: one-kernel all-reduce over NVLink peer memory (default) or NCCL + add")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch
    pkg = load_pkg()
    w = WORKLOADS[args.workload]
    dim, heads, ff, n_layers = model_geometry(pkg, w)
    n_prompt = w["prompt"]
    if n_prompt + args.warmup + args.steps + 1 > 2048:
        raise SystemExit("prompt + warm-up + steps exceeds the 2048-token context of the reference")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (launch with torch.distributed.run); got WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dist = None
    nccl_id = None
    klib = pkg.load_kernels()
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            pkg.check(klib.lv_comm_unique_id(buf))
            ident = torch.tensor(list(buf), dtype=torch.uint8, device="cuda")
        dist.broadcast(ident, 0)
        nccl_id = bytes(ident.cpu().tolist())

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(seconds):
        if dist is None:
            return seconds
        t = torch.tensor([seconds], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    path = ensure_model(pkg, args.workload, w, rank, world)
    barrier()
    t0 = time.time()
    ctx = pkg.HostContext(path, local_rank, rank, world, nccl_id)
    print(f"[bench] rank {rank}: model on device in {time.time() - t0:.1f} s", file=sys.stderr)
    if world > 1 and args.allreduce == "peer":
        mine = torch.tensor(list(ctx.peer_window_handle()), dtype=torch.uint8, device="cuda")
        gathered = [torch.zeros(64, dtype=torch.uint8, device="cuda") for _ in range(world)]
        dist.all_gather(gathered, mine)
        ctx.peer_connect([bytes(g.cpu().tolist()) for g in gathered])
        barrier()
    lv = C.c_void_p(ctx.lib.llava_context_lv(ctx.handle))
    stream = torch.cuda.ExternalStream(klib.lv_ctx_stream(lv), device=local_rank)

    prompt_eval = {}

    def fresh_session():
        s = ctx.session()
        s.set_deterministic(True)
        if world == 1:
            assert s.set_max_batch(64)          # prompt in steps of up to 64 tokens (tensor-core path for q4_0)
        for t in prompt_tokens(n_prompt):
            assert s.push_token(t)
        t0 = time.perf_counter()
        first = s.predict_next_token()          # ingests the prompt (records its steps on first use)
        prompt_eval.update(tokens=n_prompt, seconds=time.perf_counter() - t0, max_batch=64 if world == 1 else 1)
        assert first != pkg.NO_TOKEN
        assert s.push_token(first)
        return s

    # ---- device-resident loop: inputs in HBM, no host round trip per token -------------------
    s = fresh_session()
    s.generate_greedy_on_device(args.warmup)
    sampler = ClockSampler(local_rank)
    sampler.start()
    pkg.check(klib.lv_stream_sync(lv, 0))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    s.enqueue_greedy_on_device(args.steps)
    e1.record(stream)
    toks_dev = s.collect_greedy_on_device()
    pkg.check(klib.lv_stream_sync(lv, 0))
    barrier()
    sec_dev = max_over_ranks(e0.elapsed_time(e1) * 1e-3)
    s.close()

    # ---- end to end through the session API: token id in, argmax out, host in the loop -------
    s = fresh_session()
    for _ in range(args.warmup):
        s.push_token(s.predict_next_token())
    pkg.check(klib.lv_stream_sync(lv, 0))
    barrier()
    toks_e2e = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        assert s.start_next_token_prediction()          # H2D: the pushed token id (pinned, 4 B)
        tok = s.finish_next_token_prediction()          # D2H: the argmax (pinned, 4 B)
        toks_e2e.append(tok)
        s.push_token(tok)
    sec_e2e = max_over_ranks(time.perf_counter() - t0)
    barrier()
    clocks = sampler.stop()
    s.close()
    if toks_e2e != toks_dev:
        raise SystemExit("device-resident and host-driven decoding disagree on the greedy tokens")

    # ---- roofline of the dominant kernel ---------------------------------------------------
    peak, peak_kind = measured_peaks()
    k_sec, k_bytes = time_dominant_kernel(pkg, lv, dim, ff // world, w["wtype"], stream, torch)
    first_pos = n_prompt + 1 + args.warmup               # cache rows already filled when the timed steps start
    mean_pos = first_pos + (args.steps - 1) / 2
    bytes_per_token = weight_bytes_per_token(dim, ff, n_layers, 32000, w["wtype"]) + kv_bytes_per_token(dim, n_layers, mean_pos)
    tps = args.steps / sec_dev
    achieved = k_bytes / k_sec / 1e9
    peak_all = peak * world                               # aggregate bandwidth of the N GPUs for the whole step
    roofline = {"bound": "hbm", "kernel": f"lv_qrow_stream_kernel<{'q4_0' if w['wtype'] == 2 else 'q8_0'}, SILU> (norm + gate/up + SiLU, "
                                          f"{ff // world}x{dim} pair)", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": f"of {peak_kind}",
                # dram__bytes_read + dram__bytes_write of one launch of this kernel at this shape (ncu capture summarised
                # in profiles/gemv_silu_q4_0_11008x4096.md); no capture exists for the other shapes
                "traffic": 50810368 if (w["wtype"] == 2 and dim == 4096 and world == 1) else None,
                "algorithmic_bytes_per_launch": k_bytes,
                "whole_step": {"bytes_per_token": bytes_per_token, "achieved": bytes_per_token * tps / 1e9,
                               "aggregate_peak": peak_all, "frac": bytes_per_token * tps / 1e9 / peak_all}}

    cpu = None
    if rank != 0:
        ctx.close()
        barrier()
        dist.destroy_process_group()
        return
    if not args.no_cpu_baseline and world == 1:
        ctx.close()
        ctx = None
        v, timed, threads = cpu_oracle_tokens_per_s(path, 12, 20.0)
        cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{timed} whole-depth decode tokens at context 1..{timed + 1} of the same model file"}
    if ctx is not None:
        ctx.close()

    # embedding row, 5 kernels per layer (7 with the two all-reduce + residual kernels of a sharded layer), norm + head, argmax + advance
    launches_per_token = 1 + (5 if world == 1 else 7) * n_layers + 2
    line = {
        "metric": "decode tokens/s", "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec_dev * 1e3 / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"LLaMA-{w['geometry'].upper()} {'q4_0' if w['wtype'] == 2 else 'q8_0'} single-stream greedy decode, "
                               f"{n_layers} layers, {n_prompt}-token seeded prompt, f16 KV cache, context {first_pos}..{first_pos + args.steps}",
                   "baseline_config_index": w["config"], "cache": "weights per token (GBs) exceed the 126 MB L2; no flush needed",
                   "parallelism": f"tp{world}" + (f" ({args.allreduce} all-reduce)" if world > 1 else "")},
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": args.steps / sec_e2e, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
        "gpu_launches": launches_per_token * args.steps, "clocks": clocks,
        # not part of the metric: wall time of the prompt's evaluation, first use (records the steps) included
        "prompt_eval": dict(prompt_eval, tokens_per_s=prompt_eval["tokens"] / prompt_eval["seconds"]) if prompt_eval else None,
    }
    print(json.dumps(line), flush=True)
    barrier()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

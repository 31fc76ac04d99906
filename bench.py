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
RESULT_OUT = None    # where the JSON line goes (main() keeps the original stdout here)


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


def prompt_tokens(n, seed=PROMPT_SEED):
    import numpy as np
    return [int(t) for t in np.random.default_rng(seed).integers(3, 32000, n)]


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


def oracle_threads():
    """Host threads the CPU oracle may use: the cores this process is allowed on.  Set explicitly, because
    launchers such as torch.distributed.run export OMP_NUM_THREADS=1 to their children."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_oracle_tokens_per_s(path, n_prompt, n_warmup, n_tokens, budget_s):
    """Times the CPU oracle (full depth, all host threads): evaluates n_prompt prompt tokens and n_warmup greedy
    tokens untimed, then times up to n_tokens greedy tokens, stopping early once budget_s is used.
    Returns (tokens/s, tokens timed, threads, first timed context length)."""
    import numpy as np
    import oracle_bind as ob
    lib = ob.load()
    lib.orc_set_threads(oracle_threads())
    model = lib.orc_model_open(os.fsencode(path))
    sess = lib.orc_session_create(model, 2048)
    info = ob.ModelInfo()
    lib.orc_model_get_info(model, C.byref(info))
    logits = np.empty(info.vocab_size, np.float32)
    for t in prompt_tokens(max(n_prompt, 1)):
        lib.orc_session_push_token(sess, t)

    def step():
        lib.orc_session_eval(sess, ob.ptr(logits))          # evaluates every token pushed since the last call
        lib.orc_session_push_token(sess, int(lib.orc_argmax(ob.ptr(logits), logits.size)))

    for _ in range(1 + n_warmup):                           # the first call ingests the prompt
        step()
    first_ctx = lib.orc_session_token_count(sess)
    done, t0 = 0, time.perf_counter()
    while done < n_tokens:
        step()
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    nthreads = lib.orc_get_threads()
    lib.orc_session_destroy(sess)
    lib.orc_model_close(model)
    return done / dt, done, nthreads, first_ctx


def workload_config(pkg, name, args, world):
    """The `config` object of the JSON line; both arms print the same one for the same arguments."""
    w = WORKLOADS[name]
    dim, heads, ff, n_layers = model_geometry(pkg, w)
    first_pos = w["prompt"] + 1 + args.warmup               # cache rows already filled when the timed steps start
    return {"workload": f"LLaMA-{w['geometry'].upper()} {'q4_0' if w['wtype'] == 2 else 'q8_0'} single-stream greedy decode, "
                        f"{n_layers} layers, {w['prompt']}-token seeded prompt, f16 KV cache, context {first_pos}..{first_pos + args.steps}",
            "baseline_config_index": w["config"], "cache": "weights per token (GBs) exceed the 126 MB L2; no flush needed",
            "parallelism": f"tp{world}" + (f" ({args.allreduce} all-reduce)" if world > 1 else "")}


def model_path_for(pkg, w):
    dim, heads, ff, n_layers = model_geometry(pkg, w)
    return os.path.join(MODEL_DIR, f"{w['geometry']}_L{n_layers}_t{w['wtype']}_seed1234.ggjt")


def run_reference(args, rank, world):
    """The reference arm: the reference's path restated for the CPU (oracle/), since its own implementation
    needs Vulkan, which does not exist on this box.  Same model file, prompt, warm-up and step count as the GPU
    arm (the timed part stops early after ~150 s)."""
    if rank != 0:
        return
    pkg = load_pkg()                 # ctypes declarations only; the native product libraries are loaded on demand
    w = WORKLOADS[args.workload]
    path = model_path_for(pkg, w)
    if not (os.path.exists(path + ".done") and os.path.exists(path)):
        path = ensure_model(pkg, args.workload, w, 0, 1)       # first run on this box: the synthetic file has to be written
    tps, timed, threads, first_ctx = cpu_oracle_tokens_per_s(path, w["prompt"], args.warmup, args.steps, 150.0)
    line = {
        "impl": "reference", "metric": "decode tokens/s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / tps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(pkg, args.workload, args, args.gpus),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{timed} whole-depth greedy decode tokens from context {first_ctx} on, after the same "
                                   f"{w['prompt']}-token prompt and {args.warmup} warm-up tokens (CPU restatement of the "
                                   "reference shaders; the reference's own Vulkan path is unavailable on this box)"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=RESULT_OUT or sys.stdout, flush=True)


PARITY_MODELS = (("7b", 2, 2), ("13b", 2, 2))        # geometry, layers, type: BASELINE config 0 and its 13B-geometry twin
PARITY_PROMPT, PARITY_DECODE = 16, 32
PARITY_MAX_ABS, PARITY_REL_L2 = 1e-2, 1e-3


def oracle_trajectory(path, prompt, n_decode):
    """Greedy decoding on the CPU oracle: the logits of every step and the tokens chosen."""
    import numpy as np
    import oracle_bind as ob
    lib = ob.load()
    lib.orc_set_threads(oracle_threads())
    model = lib.orc_model_open(os.fsencode(path))
    sess = lib.orc_session_create(model, 1024)
    logits = np.empty(32000, np.float32)
    for t in prompt:
        lib.orc_session_push_token(sess, t)
    all_logits, tokens = [], []
    for _ in range(n_decode):
        lib.orc_session_eval(sess, ob.ptr(logits))
        all_logits.append(logits.copy())
        tokens.append(int(lib.orc_argmax(ob.ptr(logits), logits.size)))
        lib.orc_session_push_token(sess, tokens[-1])
    lib.orc_session_destroy(sess)
    lib.orc_model_close(model)
    return all_logits, tokens


class Rig:
    """Process-wide plumbing: rank, torch.distributed, context creation with the peer windows connected."""

    def __init__(self, args):
        import torch
        self.torch = torch
        self.args = args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.pkg = load_pkg()
        self.klib = self.pkg.load_kernels()
        torch.cuda.set_device(self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, seconds):
        if self.dist is None:
            return seconds
        t = self.torch.tensor([seconds], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def agree(self, ok):
        """True only if every rank says ok."""
        if self.dist is None:
            return ok
        t = self.torch.tensor([1 if ok else 0], dtype=self.torch.int32, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def open_context(self, path):
        torch, dist, pkg = self.torch, self.dist, self.pkg
        nccl_id = None
        if self.world > 1:
            ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
            if self.rank == 0:
                buf = (C.c_uint8 * 128)()
                pkg.check(self.klib.lv_comm_unique_id(buf))
                ident = torch.tensor(list(buf), dtype=torch.uint8, device="cuda")
            dist.broadcast(ident, 0)
            nccl_id = bytes(ident.cpu().tolist())
        ctx = pkg.HostContext(path, self.local_rank, self.rank, self.world, nccl_id)
        if self.world > 1 and self.args.allreduce == "peer":
            mine = torch.tensor(list(ctx.peer_window_handle()), dtype=torch.uint8, device="cuda")
            gathered = [torch.zeros(64, dtype=torch.uint8, device="cuda") for _ in range(self.world)]
            dist.all_gather(gathered, mine)
            ctx.peer_connect([bytes(g.cpu().tolist()) for g in gathered])
            self.barrier()
        return ctx


def parity_check(rig):
    """Before anything is timed: the two-layer 7B-geometry model of BASELINE config 0 and a two-layer
    13B-geometry model, 16 seeded prompt tokens + 32 greedy tokens on the N ranks, every step's logits and
    token compared on rank 0 with the CPU oracle.  Returns the worst distances; raises SystemExit on a miss."""
    import numpy as np
    pkg = rig.pkg
    out = {"max_abs_tolerance": PARITY_MAX_ABS, "rel_l2_tolerance": PARITY_REL_L2, "tokens_per_model": PARITY_DECODE, "models": {}}
    prompt = prompt_tokens(PARITY_PROMPT)
    for geometry, n_layers, wtype in PARITY_MODELS:
        w = dict(geometry=geometry, n_layers=n_layers, wtype=wtype, prompt=PARITY_PROMPT, config=0)
        path = ensure_model(pkg, f"parity-{geometry}", w, rig.rank, rig.world)
        rig.barrier()
        want_logits, want_tokens = oracle_trajectory(path, prompt, PARITY_DECODE) if rig.rank == 0 else (None, None)
        ctx = rig.open_context(path)
        s = ctx.session()
        s.set_deterministic(True)
        for t in prompt:
            assert s.push_token(t)
        worst_abs = worst_rel = 0.0
        ok, why = True, ""
        for step in range(PARITY_DECODE):
            tok = s.predict_next_token()
            if tok == pkg.NO_TOKEN:
                ok, why = False, f"step {step}: evaluation failed"
                break
            if rig.rank == 0:
                got = s.logits(32000).astype(np.float64)
                want = want_logits[step].astype(np.float64)
                worst_abs = max(worst_abs, float(np.abs(got - want).max()))
                worst_rel = max(worst_rel, float(np.linalg.norm(got - want) / np.linalg.norm(want)))
                if tok != want_tokens[step]:
                    ok, why = False, f"step {step}: token {tok}, oracle {want_tokens[step]}"
                if not (worst_abs <= PARITY_MAX_ABS and worst_rel <= PARITY_REL_L2):
                    ok, why = False, f"step {step}: logits max-abs {worst_abs:.3e} rel-L2 {worst_rel:.3e}"
            if not rig.agree(ok):
                ok = False
                break
            s.push_token(tok)
        s.close()
        ctx.close()
        rig.barrier()
        out["models"][f"{geometry}-geometry, {n_layers} layers, q4_0"] = {"logits_max_abs": worst_abs, "logits_rel_l2": worst_rel,
                                                                        "greedy_tokens_identical": ok}
        if not ok:
            if rig.rank == 0:
                print(json.dumps({"parity": out, "failed": why}), file=RESULT_OUT or sys.stdout, flush=True)
            raise SystemExit(f"parity check against the CPU oracle failed on {rig.world} GPU(s): {why}")
    out["against"] = "CPU oracle (oracle/llava_oracle.c), rank 0"
    return out


def median_spread(values):
    v = sorted(values)
    return v[len(v) // 2], {"min": v[0], "max": v[-1], "repeats": len(v)}


def measure_decode(rig, ctx, name, args, repeats):
    """Decode throughput of one workload on an open context: `repeats` timed regions of args.steps greedy tokens
    each over the same context window (the session is rewound in between), device-resident and host-driven.
    Returns a dict; tokens/s figures are medians over the repeats of the max over ranks."""
    torch, pkg, klib = rig.torch, rig.pkg, rig.klib
    w = WORKLOADS[name]
    n_prompt, world = w["prompt"], rig.world
    lv = C.c_void_p(ctx.lib.llava_context_lv(ctx.handle))
    stream = torch.cuda.ExternalStream(klib.lv_ctx_stream(lv), device=rig.local_rank)
    prompt_eval = {}

    s = ctx.session()
    s.set_deterministic(True)
    # prompt in steps of up to 64 tokens (tensor-core path); a sharded session whose shard shapes do not fit the tiles
    # (7B at 8 ranks: 1376 rows of w3 / w1 per rank) refuses and goes token by token
    batched = bool(s.set_max_batch(64))
    assert batched or world > 1
    for t in prompt_tokens(n_prompt):
        assert s.push_token(t)
    t0 = time.perf_counter()
    first = s.predict_next_token()          # ingests the prompt (records its steps on first use)
    if world > 1 and batched and not rig.agree(first != pkg.NO_TOKEN):
        # the batched steps of a sharded session failed on some rank (a bounded device wait ran out; stderr has the code):
        # say so in the line and measure the decode loop with the prompt evaluated token by token
        print(f"[bench] rank {rig.rank}: batched prompt evaluation failed at {world} ranks, falling back to single tokens", file=sys.stderr, flush=True)
        prompt_eval["batched_prompt_failed"] = True
        batched = False
        s.close()
        klib.lv_stream_sync(lv, 0)             # reports and clears the device error word
        rig.barrier()
        s = ctx.session()
        s.set_deterministic(True)
        for t in prompt_tokens(n_prompt):
            assert s.push_token(t)
        t0 = time.perf_counter()
        first = s.predict_next_token()
    prompt_eval.update(tokens=n_prompt, seconds=time.perf_counter() - t0, max_batch=64 if batched else 1)
    assert first != pkg.NO_TOKEN
    assert s.push_token(first)
    warm = s.generate_greedy_on_device(args.warmup)
    base = s.tokens()                        # prompt, first token, warm-up tokens; the last one is not evaluated yet
    assert len(base) == n_prompt + 1 + args.warmup and warm == base[-args.warmup:]

    def restart():
        """Back to the state right after the warm-up: every token but the last evaluated."""
        s.rewind(len(base) - 1)
        assert s.push_token(base[-1])

    # ---- device-resident loop: inputs in HBM, no host round trip per token -------------------
    dev_times, toks_dev = [], None
    for r in range(repeats):
        restart()
        pkg.check(klib.lv_stream_sync(lv, 0))
        rig.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        s.enqueue_greedy_on_device(args.steps)
        e1.record(stream)
        toks = s.collect_greedy_on_device()
        pkg.check(klib.lv_stream_sync(lv, 0))
        rig.barrier()
        dev_times.append(rig.max_over_ranks(e0.elapsed_time(e1) * 1e-3))
        if toks_dev is not None and toks != toks_dev:
            raise SystemExit("two device-resident runs over the same context disagree on the greedy tokens")
        toks_dev = toks
    launches = s.step_kernel_launches()

    # ---- end to end through the session API: token id in, argmax out, host in the loop -------
    e2e_times = []
    for r in range(repeats):
        restart()
        pkg.check(klib.lv_stream_sync(lv, 0))
        rig.barrier()
        toks_e2e = []
        t0 = time.perf_counter()
        for _ in range(args.steps):
            assert s.start_next_token_prediction()          # H2D: the pushed token id (pinned, 4 B)
            tok = s.finish_next_token_prediction()          # D2H: the argmax (pinned, 4 B)
            toks_e2e.append(tok)
            s.push_token(tok)
        e2e_times.append(rig.max_over_ranks(time.perf_counter() - t0))
        rig.barrier()
        if toks_e2e != toks_dev:
            raise SystemExit("device-resident and host-driven decoding disagree on the greedy tokens")
    # ---- the same loop with the reference's sampler (its CLI never decodes greedily): token drawn on the device ----
    s.set_deterministic(False)
    s.set_seed(1)
    sampled_times = []
    for r in range(min(repeats, 3)):
        restart()
        pkg.check(klib.lv_stream_sync(lv, 0))
        rig.barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            assert s.start_next_token_prediction()
            tok = s.finish_next_token_prediction()
            assert tok != pkg.NO_TOKEN
            s.push_token(tok)
        sampled_times.append(rig.max_over_ranks(time.perf_counter() - t0))
        rig.barrier()
    s.close()
    # ---- a long prompt through the batched (tensor-core) steps, second pass so that the steps are already recorded ----
    if batched:
        long_n = 1024
        sp = ctx.session()
        sp.set_deterministic(True)
        assert sp.set_max_batch(64)
        long_secs, long_ok = [], True
        for r in range(3):
            sp.rewind(0)
            for t in prompt_tokens(long_n):
                assert sp.push_token(t)
            klib.lv_stream_sync(lv, 0)
            rig.barrier()
            t0 = time.perf_counter()
            long_ok = rig.agree(sp.predict_next_token() != pkg.NO_TOKEN)
            long_secs.append(rig.max_over_ranks(time.perf_counter() - t0))
            if not long_ok:
                break
        sp.close()
        klib.lv_stream_sync(lv, 0)
        if long_ok:
            prompt_eval["long_prompt"] = {"tokens": long_n, "max_batch": 64, "first_pass_seconds": long_secs[0],
                                          "seconds": min(long_secs[1:]), "tokens_per_s": long_n / min(long_secs[1:])}
        else:
            prompt_eval["long_prompt"] = {"tokens": long_n, "max_batch": 64, "failed": True}
    sec_dev, dev_spread = median_spread(dev_times)
    sec_e2e, e2e_spread = median_spread(e2e_times)
    dim, heads, ff, n_layers = model_geometry(pkg, w)
    first_pos = n_prompt + 1 + args.warmup
    mean_pos = first_pos + (args.steps - 1) / 2
    bytes_per_token = weight_bytes_per_token(dim, ff, n_layers, 32000, w["wtype"]) + kv_bytes_per_token(dim, n_layers, mean_pos)
    tps = args.steps / sec_dev
    return {"tokens_per_s": tps, "ms_per_step": sec_dev * 1e3 / args.steps,
            "spread_tokens_per_s": {"min": args.steps / dev_spread["max"], "max": args.steps / dev_spread["min"], "repeats": repeats},
            "e2e_tokens_per_s": args.steps / sec_e2e,
            "e2e_spread_tokens_per_s": {"min": args.steps / e2e_spread["max"], "max": args.steps / e2e_spread["min"], "repeats": repeats},
            "sampled_e2e_tokens_per_s": args.steps / median_spread(sampled_times)[0],
            "bytes_per_token": bytes_per_token, "launches_per_token": launches, "tokens_digest": int(sum((i + 1) * t for i, t in enumerate(toks_dev)) % (1 << 31)),
            "prompt_eval": dict(prompt_eval, tokens_per_s=prompt_eval["tokens"] / prompt_eval["seconds"])}


def measure_concurrent_sessions(rig, ctx, name, args, counts=(4, 16, 64)):
    """Aggregate greedy decode tokens/s of k sessions stepped together by llava_session_group (one pass over the weights
    per step for all of them): every session has its own seeded 32-token prompt; args.steps steps with the tokens fed
    back on the device, timed on the host around the queued steps and their completion (second run, steps recorded)."""
    pkg = rig.pkg
    out = {}
    for k in counts:
        sessions = []
        for i in range(k):
            s = ctx.session()
            s.set_deterministic(True)
            assert s.set_max_batch(64)
            for t in prompt_tokens(32, seed=PROMPT_SEED + 1 + i):
                assert s.push_token(t)
            tok = s.predict_next_token()
            assert tok != pkg.NO_TOKEN and s.push_token(tok)
            sessions.append(s)
        group = pkg.SessionGroup(ctx, sessions)
        assert group.generate_greedy_on_device(args.warmup) is not None          # records the step
        secs = []
        for r in range(3):
            t0 = time.perf_counter()
            toks = group.generate_greedy_on_device(args.steps)
            secs.append(time.perf_counter() - t0)
            assert toks is not None
        sec = sorted(secs)[1]
        out[str(k)] = {"tokens_per_s": k * args.steps / sec, "ms_per_step": sec * 1e3 / args.steps, "launches_per_step": group.kernel_launches()}
        group.close()
        for s in sessions:
            s.close()
    return out


def measure_server_sessions(rig, ctx, args, counts=(1, 4, 16), seconds=1.5):
    """Tokens/s that clients of the TCP front end receive when k sessions generate at once (greedy, 32-token seeded prompts):
    the server's scheduler steps the running sessions together.  Counted from the newToken broadcasts that arrive on one
    subscribed client connection over `seconds`, from the moment every session has delivered four tokens."""
    import struct
    pkg = rig.pkg
    out = {}
    with pkg.Server(ctx, deterministic=True) as server:
        for k in counts:
            c = pkg.Client(server.port, timeout=120.0)
            sids = []
            for i in range(k):
                op, sid = c.call(c.NEW_SESSION)
                assert op == c.SESSION_CREATED
                for t in prompt_tokens(32, seed=PROMPT_SEED + 100 + i):
                    assert c.call(c.ADD_TOKEN, sid + struct.pack("<I", t))[0] == c.ACK
                assert c.call(c.SUBSCRIBE, sid)[0] == c.ACK
                sids.append(sid)
            for sid in sids:
                c.send(c.START, sid)
            # the window opens once every session has produced a few tokens (its prompt is ingested, the group has formed)
            seen = {sid: 0 for sid in sids}
            t0, n = None, 0
            while True:
                op, rid, data = c.recv()
                if op != c.NEW_TOKEN or rid != 0:
                    continue
                if t0 is None:
                    seen[data[:4]] += 1
                    if min(seen.values()) >= 4:
                        t0 = time.perf_counter()
                        g0, a0, t0s = server.grouped(), server.steps_ahead(), server.scheduler_times()
                    continue
                n += 1
                if time.perf_counter() - t0 >= seconds:
                    break
            elapsed = time.perf_counter() - t0
            g1, a1, t1s = server.grouped(), server.steps_ahead(), server.scheduler_times()
            for sid in sids:
                c.call(c.KILL_SESSION, sid)
            c.close()
            steps, toks = g1[0] - g0[0], g1[1] - g0[1]
            out[str(k)] = {"tokens_per_s": n / elapsed, "sessions_per_shared_step": (toks / steps) if steps else 1.0,
                           "shared_steps_queued_ahead": ((a1 - a0) / steps) if steps else 0.0,
                           "ms_per_round_waiting_for_sessions": ((t1s[0] - t0s[0]) / 1e3 / steps) if steps else None,
                           "ms_per_round_waiting_for_device": ((t1s[1] - t0s[1]) / 1e3 / steps) if steps else None}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="7b-q4_0", choices=sorted(WORKLOADS))
    ap.add_argument("--repeats", type=int, default=5, help="timed regions per figure; the median is reported")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison that precedes the timed runs")
    ap.add_argument("--no-13b", action="store_true", help="skip the second measurement on LLaMA-13B q4_0 (BASELINE config 3)")
    ap.add_argument("--no-sessions", action="store_true", help="skip the aggregate throughput of 4 / 16 / 64 sessions stepped together")
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"],
                    help="N > 1: exchanges over NVLink peer memory (default) or NCCL + add")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    # stdout carries the one JSON line and nothing else: libraries that write to descriptor 1 (NCCL's version banner)
    # get stderr instead, and the line goes to the descriptor kept aside here
    global RESULT_OUT
    sys.stdout.flush()
    RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        return run_reference(args, rank, world)

    pkg = load_pkg()
    w = WORKLOADS[args.workload]
    dim, heads, ff, n_layers = model_geometry(pkg, w)
    n_prompt = w["prompt"]
    if n_prompt + args.warmup + args.steps + 1 > 2048:
        raise SystemExit("prompt + warm-up + steps exceeds the 2048-token context of the reference")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (launch with torch.distributed.run); got WORLD_SIZE={world}")
    rig = Rig(args)
    torch, klib = rig.torch, rig.klib

    parity = None if args.no_parity else parity_check(rig)

    path = ensure_model(pkg, args.workload, w, rank, world)
    rig.barrier()
    t0 = time.time()
    ctx = rig.open_context(path)
    print(f"[bench] rank {rank}: model on device in {time.time() - t0:.1f} s", file=sys.stderr)
    lv = C.c_void_p(ctx.lib.llava_context_lv(ctx.handle))
    stream = torch.cuda.ExternalStream(klib.lv_ctx_stream(lv), device=rig.local_rank)

    sampler = ClockSampler(rig.local_rank)
    sampler.start()
    m = measure_decode(rig, ctx, args.workload, args, args.repeats)
    clocks = sampler.stop()

    # ---- roofline of the dominant kernel ---------------------------------------------------
    peak, peak_kind = measured_peaks()
    k_sec, k_bytes = time_dominant_kernel(pkg, lv, dim, ff // world, w["wtype"], stream, torch)
    achieved = k_bytes / k_sec / 1e9
    peak_all = peak * world                               # aggregate bandwidth of the N GPUs for the whole step
    tps = m["tokens_per_s"]
    roofline = {"bound": "hbm", "kernel": f"lv_qrow_stream_kernel<{'q4_0' if w['wtype'] == 2 else 'q8_0'}, SILU> (norm + gate/up + SiLU, "
                                          f"{ff // world}x{dim} pair)", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": f"of {peak_kind}",
                # dram__bytes_read + dram__bytes_write of one launch of this kernel at this shape (ncu capture summarised
                # in profiles/gemv_silu_q4_0_11008x4096.md); no capture exists for the other shapes
                "traffic": 50810368 if (w["wtype"] == 2 and dim == 4096 and world == 1) else None,
                "algorithmic_bytes_per_launch": k_bytes,
                "whole_step": {"bytes_per_token": m["bytes_per_token"], "achieved": m["bytes_per_token"] * tps / 1e9,
                               "aggregate_peak": peak_all, "frac": m["bytes_per_token"] * tps / 1e9 / peak_all}}
    sessions = None
    if world == 1 and not args.no_sessions and w["wtype"] == 2:
        sessions = measure_concurrent_sessions(rig, ctx, args.workload, args)
        sessions["through_the_server"] = measure_server_sessions(rig, ctx, args)
    ctx.close()
    rig.barrier()

    # ---- BASELINE config 3 (LLaMA-13B q4_0), the model the multi-GPU target is stated on -------
    config3 = None
    if not args.no_13b and args.workload != "13b-q4_0":
        w13 = WORKLOADS["13b-q4_0"]
        path13 = ensure_model(pkg, "13b-q4_0", w13, rank, world)
        rig.barrier()
        ctx13 = rig.open_context(path13)
        m13 = measure_decode(rig, ctx13, "13b-q4_0", args, max(3, args.repeats // 2))
        ctx13.close()
        rig.barrier()
        config3 = {"workload": workload_config(pkg, "13b-q4_0", args, world)["workload"], "tokens_per_s": m13["tokens_per_s"],
                   "ms_per_step": m13["ms_per_step"], "spread_tokens_per_s": m13["spread_tokens_per_s"],
                   "e2e_tokens_per_s": m13["e2e_tokens_per_s"], "bytes_per_token": m13["bytes_per_token"],
                   "whole_step_frac": m13["bytes_per_token"] * m13["tokens_per_s"] / 1e9 / peak_all,
                   "prompt_eval_tokens_per_s": m13["prompt_eval"]["tokens_per_s"]}

    if rank != 0:
        rig.dist.destroy_process_group()
        return
    cpu = None
    if not args.no_cpu_baseline and world == 1:
        v, timed, threads, first_ctx = cpu_oracle_tokens_per_s(path, 1, 0, 12, 20.0)
        cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{timed} whole-depth decode tokens from context {first_ctx} on, same model file"}

    line = {
        "metric": "decode tokens/s", "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32 accumulate; weights q4_0/q8_0 blocks as stored; activations 22-bit fixed point per 32-block (exact int32 dot products)",
        "data": "synthetic", "config": workload_config(pkg, args.workload, args, world),
        "spread": dict(m["spread_tokens_per_s"], unit="tokens/s", value_is="median"),
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": m["e2e_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4,
                "spread": m["e2e_spread_tokens_per_s"],
                # same loop, token drawn by the reference's sampler (temperature 0.8, mirostat-style cut) on the device
                "sampled_tokens_per_s": m["sampled_e2e_tokens_per_s"]},
        "gpu_launches": m["launches_per_token"] * args.steps, "clocks": clocks,
        "parity": parity, "tokens_digest": m["tokens_digest"], "config3_13b": config3,
        "concurrent_sessions": sessions,
        # not part of the metric: wall time of the prompt's evaluation, first use (records the steps) included
        "prompt_eval": m["prompt_eval"],
    }
    print(json.dumps(line), file=RESULT_OUT or sys.stdout, flush=True)
    if rig.dist is not None:
        rig.dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Tensor-parallel decoding on 2 GPUs (one process per GPU, NCCL all-reduce after
wo and w2) against the single-GPU path on the same 2-layer model: logits within
the end-to-end tolerance, greedy tokens identical.  Skipped on a 1-GPU box."""
import ctypes as C
import os
import queue

import numpy as np
import pytest

from conftest import load_pkg

pytestmark = pytest.mark.gpu

N_PROMPT, N_DECODE = 8, 12


def _device_count():
    pkg = load_pkg()
    n = C.c_int(0)
    pkg.load_kernels().lv_device_count(C.byref(n))
    return n.value


def _prompt():
    return [int(t) for t in np.random.default_rng(4321).integers(3, 32000, N_PROMPT)]


def _decode(ctx):
    s = ctx.session()
    s.set_deterministic(True)
    for t in _prompt():
        assert s.push_token(t)
    toks, logits = [], []
    for _ in range(N_DECODE):
        tok = s.predict_next_token()
        assert tok != 0xFFFFFFFF
        toks.append(tok)
        logits.append(s.logits(32000))
        s.push_token(tok)
    assert not s.set_max_batch(4) or ctx_is_single(ctx)
    s.close()
    return toks, logits


def _decode_batched(ctx, n_prompt=40, max_batch=16, n_decode=4):
    """A prompt in tensor-core batches (16 + 16 + 8), then a few single tokens."""
    s = ctx.session()
    s.set_deterministic(True)
    assert s.set_max_batch(max_batch)
    for t in [int(t) for t in np.random.default_rng(99).integers(3, 32000, n_prompt)]:
        assert s.push_token(t)
    toks, logits = [], []
    for _ in range(n_decode):
        tok = s.predict_next_token()
        assert tok != 0xFFFFFFFF
        toks.append(tok)
        logits.append(s.logits(32000))
        s.push_token(tok)
    s.close()
    return toks, logits


def ctx_is_single(ctx):
    return getattr(ctx, "n_ranks", 1) == 1


def _worker(rank, world, path, id_q, out_q, peer_q=None, one_launch=False, batched=False):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    if one_launch:
        os.environ["LV_DECODE_STEP"] = "1"          # read when a session is created: every token as one persistent kernel
    pkg = load_pkg()
    klib = pkg.load_kernels()
    if rank == 0:
        buf = (C.c_uint8 * 128)()
        pkg.check(klib.lv_comm_unique_id(buf))
        for _ in range(world - 1):
            id_q.put(bytes(buf))
        ident = bytes(buf)
    else:
        ident = id_q.get(timeout=120)
    ctx = pkg.HostContext(path, rank, rank, world, ident)
    ctx.n_ranks = world
    if peer_q is not None:                      # one-kernel all-reduce over peer memory instead of NCCL + add
        mine = ctx.peer_window_handle()
        for r in range(world):
            peer_q[r].put((rank, mine))
        got = dict(peer_q[rank].get(timeout=120) for _ in range(world))
        ctx.peer_connect([got[r] for r in range(world)])
    toks, logits = _decode_batched(ctx) if batched else _decode(ctx)
    ctx.close()
    out_q.put((rank, toks, [l.tobytes() for l in logits]))


@pytest.mark.parametrize("exchange", ["nccl", "peer", "peer-one-launch"])
def test_two_gpu_tensor_parallel_matches_one_gpu(pkg, tmp_path, exchange):
    if _device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    path = str(tmp_path / "tiny.bin")
    pkg.write_synthetic_model(path, "7b", n_layers=2)
    ctx = pkg.HostContext(path, 0)
    want_toks, want_logits = _decode(ctx)
    ctx.close()
    mpc = mp.get_context("spawn")
    id_q, out_q = mpc.Queue(), mpc.Queue()
    peer_q = [mpc.Queue() for _ in range(2)] if exchange != "nccl" else None
    procs = [mpc.Process(target=_worker, args=(r, 2, path, id_q, out_q, peer_q, exchange == "peer-one-launch")) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(2):
        try:
            r, toks, logits = out_q.get(timeout=300)
        except queue.Empty:
            for p in procs:
                p.kill()
            raise AssertionError("a rank did not finish")
        results[r] = (toks, [np.frombuffer(b, np.float32) for b in logits])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[0][0] == results[1][0] == want_toks
    for step in range(N_DECODE):
        for r in (0, 1):
            got, want = results[r][1][step].astype(np.float64), want_logits[step].astype(np.float64)
            assert np.abs(got - want).max() <= 1e-2
            assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3
        assert np.array_equal(results[0][1][step], results[1][1][step])      # every rank holds the same logits


@pytest.mark.parametrize("exchange", ["nccl", "peer"])
def test_two_gpu_prompt_batches_on_the_tensor_cores(pkg, tmp_path, exchange):
    """A sharded session evaluates a prompt in batches: row shards of wq / wk / wv / w3 / w1 and padded column shards of
    wo / w2 on the tcgen05 path, one exchange per sub-block for the whole batch.  Against the same batches on one GPU."""
    if _device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    path = str(tmp_path / "tiny.bin")
    pkg.write_synthetic_model(path, "7b", n_layers=2)
    ctx = pkg.HostContext(path, 0)
    want_toks, want_logits = _decode_batched(ctx)
    ctx.close()
    mpc = mp.get_context("spawn")
    id_q, out_q = mpc.Queue(), mpc.Queue()
    peer_q = [mpc.Queue() for _ in range(2)] if exchange != "nccl" else None
    procs = [mpc.Process(target=_worker, args=(r, 2, path, id_q, out_q, peer_q, False, True)) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(2):
        try:
            r, toks, logits = out_q.get(timeout=300)
        except queue.Empty:
            for p in procs:
                p.kill()
            raise AssertionError("a rank did not finish")
        results[r] = (toks, [np.frombuffer(b, np.float32) for b in logits])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[0][0] == results[1][0] == want_toks
    for step in range(len(want_toks)):
        for r in (0, 1):
            got, want = results[r][1][step].astype(np.float64), want_logits[step].astype(np.float64)
            assert np.abs(got - want).max() <= 1e-2
            assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3
        assert np.array_equal(results[0][1][step], results[1][1][step])


def _snapshot_worker(rank, world, path, id_q, out_q, peer_q, snap_in, snap_out, n_first, n_more):
    """Restores snap_in (if given), or feeds the prompt and decodes n_first tokens; decodes n_more tokens; writes snap_out."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    pkg = load_pkg()
    klib = pkg.load_kernels()
    if rank == 0:
        buf = (C.c_uint8 * 128)()
        pkg.check(klib.lv_comm_unique_id(buf))
        for _ in range(world - 1):
            id_q.put(bytes(buf))
        ident = bytes(buf)
    else:
        ident = id_q.get(timeout=120)
    ctx = pkg.HostContext(path, rank, rank, world, ident)
    mine = ctx.peer_window_handle()
    for r in range(world):
        peer_q[r].put((rank, mine))
    got = dict(peer_q[rank].get(timeout=120) for _ in range(world))
    ctx.peer_connect([got[r] for r in range(world)])
    s = ctx.session()
    s.set_deterministic(True)
    toks = []
    if snap_in:
        assert s.restore(snap_in) == 0
        before = s.tokens()
    else:
        for t in _prompt():
            assert s.push_token(t)
        for _ in range(n_first):
            toks.append(s.predict_next_token())
            s.push_token(toks[-1])
        before = None
    if snap_out:
        s.predict_next_token()                 # evaluate the last pushed token too, so that it is part of the snapshot
        assert s.snapshot(snap_out) == 0
    more = []
    if snap_in and n_more:
        # the snapshot holds evaluated tokens only; the token that followed them is the next greedy choice of the
        # uninterrupted run, which the test passes in n_first
        s.push_token(n_first)
        for _ in range(n_more):
            more.append(s.predict_next_token())
            s.push_token(more[-1])
    out_q.put((rank, toks, before, more))
    s.close()
    ctx.close()


def _run_ranks(target, args_of_rank, world=2):
    import torch.multiprocessing as mp
    mpc = mp.get_context("spawn")
    id_q, out_q = mpc.Queue(), mpc.Queue()
    peer_q = [mpc.Queue() for _ in range(world)]
    procs = [mpc.Process(target=target, args=(r, world) + args_of_rank(r, id_q, out_q, peer_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        try:
            res = out_q.get(timeout=300)
        except queue.Empty:
            for p in procs:
                p.kill()
            raise AssertionError("a rank did not finish")
        results[res[0]] = res[1:]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return results


def test_snapshot_written_by_two_ranks_restores_on_one_gpu_and_back(pkg, tmp_path):
    """llava_session::snapshot on a sharded session gathers every rank's head slice into the reference's file layout:
    the file written by 2 ranks is byte-identical in size to a 1-GPU one and a 1-GPU session restored from it continues
    with the tokens of an uninterrupted run; a 1-GPU snapshot restores on 2 ranks likewise."""
    if _device_count() < 2:
        pytest.skip("needs 2 GPUs")
    path = str(tmp_path / "tiny.bin")
    pkg.write_synthetic_model(path, "7b", n_layers=2)
    ctx = pkg.HostContext(path, 0)
    want_toks, _ = _decode(ctx)                                   # uninterrupted: prompt + N_DECODE greedy tokens
    n_first = 5
    # --- 2 ranks write, 1 GPU restores ---
    snap2 = str(tmp_path / "snap_2ranks.bin")
    res = _run_ranks(_snapshot_worker, lambda r, id_q, out_q, peer_q: (path, id_q, out_q, peer_q, None, snap2, n_first, 0))
    assert res[0][0] == res[1][0] == want_toks[:n_first]
    n_eval = N_PROMPT + n_first
    assert os.path.getsize(snap2) == 4 + 4 * n_eval + 2 * 2 * n_eval * 4096 * 2
    s = ctx.session()
    s.set_deterministic(True)
    assert s.restore(snap2) == 0
    assert s.tokens() == _prompt() + want_toks[:n_first]
    # the next greedy token is known from the uninterrupted run; push it and go on
    cont = []
    s.push_token(want_toks[n_first])
    for _ in range(n_first + 1, N_DECODE):
        cont.append(s.predict_next_token())
        s.push_token(cont[-1])
    assert cont == want_toks[n_first + 1:]
    # --- 1 GPU writes, 2 ranks restore ---
    snap1 = str(tmp_path / "snap_1gpu.bin")
    s.rewind(0)
    for t in _prompt() + want_toks[:n_first]:
        s.push_token(t)
    s.predict_next_token()
    assert s.snapshot(snap1) == 0
    s.close()
    ctx.close()
    a, b = np.fromfile(snap1, np.uint8), np.fromfile(snap2, np.uint8)
    assert a.size == b.size and np.array_equal(a[:4 + 4 * n_eval], b[:4 + 4 * n_eval])
    # cache rows: the same numbers up to neighbouring halves (the sharded exchange sums in another order)
    ha, hb = a[4 + 4 * n_eval:].view(np.float16).astype(np.float32), b[4 + 4 * n_eval:].view(np.float16).astype(np.float32)
    assert np.abs(ha - hb).max() <= 2e-3 * np.abs(ha).max()
    n_more = N_DECODE - n_first - 1
    res = _run_ranks(_snapshot_worker, lambda r, id_q, out_q, peer_q: (path, id_q, out_q, peer_q, snap1, None, want_toks[n_first], n_more))
    assert res[0][1] == res[1][1] == _prompt() + want_toks[:n_first]
    assert res[0][2] == res[1][2] == want_toks[n_first + 1:]                  # the sharded session continues the same trajectory

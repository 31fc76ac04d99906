"""Tensor-parallel sharding (host logic) on the CPU: shard geometry, packing with
padding, and a world_size-2 gloo run in which every rank evaluates its shard with
the oracle and the partial products are all-reduced, as the GPU path does with NCCL."""
import ctypes as C
import os
import socket

import numpy as np
import pytest

import oracle_bind as ob
import quant_np as qn
from conftest import load_pkg

ROWS, COLS = 1, 2


def shape(lib, wtype, rows, cols, how, rank, n):
    r, c, u, b = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint64()
    ok = lib.llava_tp_shape(wtype, rows, cols, how, rank, n, C.byref(r), C.byref(c), C.byref(u), C.byref(b))
    return (r.value, c.value, u.value, b.value) if ok else None


def pack(lib, raw, wtype, rows, cols, how, rank, n):
    r, c, u, b = shape(lib, wtype, rows, cols, how, rank, n)
    out = np.empty(b, np.uint8)
    assert lib.llava_tp_pack(raw.ctypes.data_as(C.c_void_p), wtype, rows, cols, how, rank, n, out.ctypes.data_as(C.c_void_p)) == 1
    return out, r, c, u


def test_shard_geometry_of_the_7b_and_13b_matrices(pkg):
    lib = pkg.load_host()
    # 7B wo at 8 ranks: 16 blocks per rank, already a multiple of 8; w2: 43 blocks -> padded to 48
    assert shape(lib, qn.Q4_0, 4096, 4096, COLS, 3, 8) == (4096, 512, 512, 4096 * 16 * 18)
    assert shape(lib, qn.Q4_0, 4096, 11008, COLS, 0, 8) == (4096, 1536, 1376, 4096 * 48 * 18)
    # 13B wo at 8 ranks: 20 blocks -> 24; rows of 24 * 18 = 432 bytes start on 16-byte boundaries
    r, c, u, b = shape(lib, qn.Q4_0, 5120, 5120, COLS, 7, 8)
    assert (r, c, u) == (5120, 768, 640) and (b // r) % 16 == 0
    assert shape(lib, qn.Q8_0, 5120, 13824, COLS, 1, 4) == (5120, 3584, 3456, 5120 * 112 * 34)
    assert shape(lib, qn.Q4_0, 11008, 4096, ROWS, 5, 8) == (1376, 4096, 4096, 1376 * 128 * 18)
    assert shape(lib, qn.Q4_0, 4096, 4096, ROWS, 0, 3) is None          # 4096 rows do not divide by 3
    assert shape(lib, qn.Q4_0, 4096, 4096, COLS, 0, 3) is None          # nor do 128 blocks
    assert shape(lib, qn.Q4_0, 4096, 4096, COLS, 2, 2) is None          # rank out of range


@pytest.mark.parametrize("dim,ff", [(4096, 11008), (5120, 13824)], ids=["7b", "13b"])
@pytest.mark.parametrize("n", [2, 4, 8])
def test_shard_shapes_fit_the_batched_products(pkg, dim, ff, n):
    """What lets a sharded session ingest prompts in batches (llava_session::tensor_core_shapes_ok and the argument
    checks of lv_gemm_tc*): row shards of a multiple of 32 rows (a last row tile may be ragged), column shards padded
    to a multiple of 256 columns, activations to pad in multiples of 8."""
    lib = pkg.load_host()
    for rows, cols in ((dim, dim), (ff, dim)):                           # wq/wk/wv and w1/w3
        r, c, u, _ = shape(lib, qn.Q4_0, rows, cols, ROWS, n - 1, n)
        assert r % 32 == 0 and c == u == cols and c % 256 == 0
    for rows, cols in ((dim, dim), (dim, ff)):                           # wo and w2
        r, c, u, _ = shape(lib, qn.Q4_0, rows, cols, COLS, n - 1, n)
        assert r % 128 == 0 and c % 256 == 0 and u % 8 == 0 and 0 <= c - u < 256


@pytest.mark.parametrize("wtype", [qn.Q4_0, qn.Q8_0])
@pytest.mark.parametrize("n", [2, 4, 8])
def test_shards_reassemble_and_partial_products_add_up(pkg, wtype, n):
    lib = pkg.load_host()
    rng = np.random.default_rng(n + wtype)
    rows, cols = 64, 1280                      # 40 blocks: 5 per rank at 8 ranks -> padded to 8
    W = qn.quantize((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32), wtype)
    x = rng.standard_normal(cols).astype(np.float32)
    full = ob.gemv(W, wtype, x, rows, cols, 128)
    bb = 18 if wtype == qn.Q4_0 else 34
    # row shards are contiguous slices of the tensor
    got_rows = []
    for r in range(n):
        sh, lr, lc, _ = pack(lib, W, wtype, rows, cols, ROWS, r, n)
        assert np.array_equal(sh, W[r * lr * (cols // 32) * bb:(r + 1) * lr * (cols // 32) * bb])
        got_rows.append(ob.gemv(sh, wtype, x, lr, lc, 128))
    np.testing.assert_array_equal(np.concatenate(got_rows), full)
    # column shards: padded rows, zero blocks at the end, partial products sum to the whole
    total = np.zeros(rows, np.float64)
    for r in range(n):
        sh, lr, lc, used = pack(lib, W, wtype, rows, cols, COLS, r, n)
        assert lc % 256 == 0 and used == cols // n
        xs = np.zeros(lc, np.float32)
        xs[:used] = x[r * used:(r + 1) * used]
        deq = ob.dequant(sh, wtype, lr * lc).reshape(lr, lc)
        assert not deq[:, used:].any()
        np.testing.assert_array_equal(deq[:, :used], ob.dequant(W, wtype, rows * cols).reshape(rows, cols)[:, r * used:(r + 1) * used])
        total += ob.gemv(sh, wtype, xs, lr, lc, 128)
    np.testing.assert_allclose(total, full, rtol=0, atol=2e-5 * np.abs(full).max())


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _tp_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = load_pkg().load_host()
    rng = np.random.default_rng(2024)                     # same weights on every rank
    dim, ff = 512, 1280
    w13 = [qn.quantize_q4_0((rng.standard_normal((ff, dim)) * 0.05).astype(np.float32)) for _ in range(2)]
    w2 = qn.quantize_q4_0((rng.standard_normal((dim, ff)) * 0.05).astype(np.float32))
    x = rng.standard_normal(dim).astype(np.float32)
    residual = rng.standard_normal(dim).astype(np.float32)
    # this rank: rows of w3 / w1, columns of w2 (the FFN block of llava_layer.cpp:68-73, sharded)
    s3, lr, lc, _ = pack(lib, w13[0], qn.Q4_0, ff, dim, ROWS, rank, world)
    s1, _, _, _ = pack(lib, w13[1], qn.Q4_0, ff, dim, ROWS, rank, world)
    s2, r2, c2, used = pack(lib, w2, qn.Q4_0, dim, ff, COLS, rank, world)
    assert used == lr
    h = np.zeros(c2, np.float32)
    h[:lr] = ob.gemv_silu(s3, s1, qn.Q4_0, x, lr, lc, 128)
    partial = torch.from_numpy(ob.gemv(s2, qn.Q4_0, h, r2, c2, 128))
    dist.all_reduce(partial)                              # the exchange step
    out = residual + partial.numpy()
    if rank == 0:
        want = ob.gemv(w2, qn.Q4_0, ob.gemv_silu(w13[0], w13[1], qn.Q4_0, x, ff, dim, 128), dim, ff, 128, out=residual)
        q.put(float(np.abs(out - want).max() / np.abs(want).max()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_ffn_block_matches_the_unsharded_block():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    err = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err < 2e-5


def _snapshot_worker(rank, world, port, path, q):
    """Every rank writes its column slices of seeded cache rows where llava_session::snapshot would put them; after a
    barrier rank 0 compares the file with the single-GPU layout {n, tokens, per layer K [n][dim], V [n][dim]}."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = load_pkg().load_host()
    n, dim, layers = 7, 256, 3
    rng = np.random.default_rng(99)                       # the same "caches" on every rank; each keeps its columns
    tokens = rng.integers(0, 32000, n).astype(np.uint32)
    caches = rng.integers(0, 65536, (layers, 2, n, dim)).astype(np.uint16)
    width = dim // world
    fd = os.open(path, os.O_WRONLY | os.O_CREAT, 0o644)
    os.ftruncate(fd, lib.llava_tp_snapshot_file_size(n, dim, layers))
    os.pwrite(fd, np.uint32(n).tobytes() + tokens.tobytes(), 0)
    for layer in range(layers):
        for which in range(2):
            for row in range(n):
                mine = caches[layer, which, row, rank * width:(rank + 1) * width]
                os.pwrite(fd, mine.tobytes(), lib.llava_tp_snapshot_slice_offset(n, dim, layer, which, row, rank, world))
    os.close(fd)
    dist.barrier()
    if rank == 0:
        want = np.uint32(n).tobytes() + tokens.tobytes() + caches.tobytes()
        q.put(open(path, "rb").read() == want)
        # and back: the slices a rank would read on restore
        raw = np.frombuffer(want, np.uint8)
        ok = True
        for r in range(world):
            at = lib.llava_tp_snapshot_slice_offset(n, dim, 2, 1, 5, r, world)
            ok = ok and raw[at:at + 2 * width].tobytes() == caches[2, 1, 5, r * width:(r + 1) * width].tobytes()
        q.put(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_snapshot_slices_assemble_the_single_gpu_file(tmp_path):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    path = str(tmp_path / "snap.bin")
    procs = [ctx.Process(target=_snapshot_worker, args=(r, 2, port, path, q)) for r in range(2)]
    for p in procs:
        p.start()
    assert q.get(timeout=120) and q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0

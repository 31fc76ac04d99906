"""Parity of every kernel entry point with the CPU oracle, through the C ABI.

Bit-exact for integer/byte work (dequantisation, f16 cache rows, argmax);
fp32 results differ from the oracle only by summation order, so they are held
to a relative-L2 of 1e-5 and a max-abs of 1e-4 of the largest output -- two
orders tighter than the end-to-end logits tolerance (max-abs 1e-2, rel-L2 1e-3).
"""
import ctypes as C

import numpy as np
import pytest

import oracle_bind as ob
import quant_np as qn

pytestmark = pytest.mark.gpu

HEADS, ROT = 32, 128
DIM = HEADS * ROT


def close(got, want, rel_l2=1e-5, max_abs_frac=1e-4):
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    assert got.shape == want.shape
    assert np.all(np.isfinite(got))
    denom = np.linalg.norm(want) or 1.0
    l2 = np.linalg.norm(got - want) / denom
    mx = np.abs(got - want).max()
    assert l2 <= rel_l2, f"rel-L2 {l2:.3e}"
    assert mx <= max_abs_frac * (np.abs(want).max() or 1.0), f"max-abs {mx:.3e}"


def workers_for(cols):
    return 32 if cols == 5120 else 128      # llava_session.cpp:357-371


def u32_dev(gpu, value):
    return gpu.upload(np.array([value, value, value, value], np.uint32))   # config_buffer: token_count x4


@pytest.mark.parametrize("wtype", [qn.Q4_0, qn.Q8_0])
def test_dequant_rows_bit_exact(gpu, pkg, wtype):
    rng = np.random.default_rng(20)
    vocab, cols = 64, 4096
    table = qn.quantize((rng.standard_normal((vocab, cols)) * 0.02).astype(np.float32), wtype)
    ids = np.array([0, 63, 17, 17, 5], np.uint32)
    d_out = gpu.alloc(ids.size * cols * 4)
    pkg.check(gpu.lib.lv_dequant_rows(gpu.handle, d_out, gpu.upload(table), wtype, gpu.upload(ids), None, cols, vocab, ids.size))
    gpu.sync()
    got = gpu.download(d_out, np.float32, ids.size * cols).reshape(ids.size, cols)
    rb = qn.row_bytes(wtype, cols)
    for z, t in enumerate(ids):
        want = ob.dequant(table[t * rb:(t + 1) * rb], wtype, cols)
        assert np.array_equal(got[z].view(np.uint32), want.view(np.uint32))
    # ids taken from a device-resident token log at a device-resident position
    pkg.check(gpu.lib.lv_dequant_rows(gpu.handle, d_out, gpu.upload(table), wtype, gpu.upload(ids), u32_dev(gpu, 2), cols, vocab, 2))
    gpu.sync()
    got = gpu.download(d_out, np.float32, 2 * cols).reshape(2, cols)
    for z, t in enumerate(ids[2:4]):
        assert np.array_equal(got[z], ob.dequant(table[t * rb:(t + 1) * rb], wtype, cols))


@pytest.mark.parametrize("dim,batch", [(4096, 1), (5120, 3)])
def test_norm(gpu, pkg, dim, batch):
    rng = np.random.default_rng(21)
    x = (rng.standard_normal((batch, dim)) * 3 + 0.2).astype(np.float32)
    w = (1 + 0.01 * rng.standard_normal(dim)).astype(np.float32)
    d_out = gpu.alloc(x.nbytes)
    pkg.check(gpu.lib.lv_norm_f32(gpu.handle, d_out, gpu.upload(x), gpu.upload(w), dim, batch))
    gpu.sync()
    got = gpu.download(d_out, np.float32, x.size).reshape(batch, dim)
    for z in range(batch):
        close(got[z], ob.norm(x[z], w), rel_l2=2e-6, max_abs_frac=2e-6)


GEMV_SHAPES = [
    (qn.Q4_0, 4096, 4096), (qn.Q4_0, 4096, 11008), (qn.Q4_0, 5120, 13824), (qn.Q4_0, 5120, 5120),
    (qn.Q4_0, 32000, 4096), (qn.Q8_0, 4096, 4096), (qn.Q8_0, 4096, 11008), (qn.Q8_0, 1024, 5120),
    (qn.Q4_0, 4, 256), (qn.Q8_0, 8, 512),
]


@pytest.mark.parametrize("wtype,rows,cols", GEMV_SHAPES)
def test_gemv_and_residual_add(gpu, pkg, wtype, rows, cols):
    rng = np.random.default_rng(rows + cols)
    W = qn.quantize((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32), wtype)
    x = rng.standard_normal(cols).astype(np.float32)
    base = rng.standard_normal(rows).astype(np.float32)
    dW, dx = gpu.upload(W), gpu.upload(x)
    d_out = gpu.upload(base)
    pkg.check(gpu.lib.lv_gemv(gpu.handle, d_out, dW, wtype, dx, rows, cols, 1, 0))
    gpu.sync()
    want = ob.gemv(W, wtype, x, rows, cols, workers_for(cols))
    close(gpu.download(d_out, np.float32, rows), want)
    pkg.check(gpu.lib.lv_upload(gpu.handle, d_out, base.ctypes.data_as(C.c_void_p), base.nbytes))
    pkg.check(gpu.lib.lv_gemv(gpu.handle, d_out, dW, wtype, dx, rows, cols, 1, 1))      # matmul_add_*
    gpu.sync()
    close(gpu.download(d_out, np.float32, rows), base + want)
    for d in (dW, dx, d_out):
        gpu.free(d)


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (4096, 11008), (5120, 13824), (8, 512)])
def test_gemv_on_version_1_blocks(gpu, pkg, rows, cols):
    """q4_0 as ggjt version 1 files store it (f32 scale, byte j = elements 2j and 2j+1; matmul_dim.comp / matmul_ff.comp
    without the _fp16 suffix, llava_buffer.cpp:193-224): plain, add-in-place, with a norm in front, and the SiLU pair."""
    rng = np.random.default_rng(rows * 3 + cols)
    W = qn.quantize_q4_0_v1((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    x = rng.standard_normal(cols).astype(np.float32)
    base = rng.standard_normal(rows).astype(np.float32)
    dW, dx, d_out = gpu.upload(W), gpu.upload(x), gpu.upload(base)
    want = ob.gemv(W, qn.Q4_0, x, rows, cols, workers_for(cols), version=1)
    pkg.check(gpu.lib.lv_gemv(gpu.handle, d_out, dW, qn.Q4_0_V1, dx, rows, cols, 1, 1))
    gpu.sync()
    close(gpu.download(d_out, np.float32, rows), base + want)
    nw = (1 + 0.01 * rng.standard_normal(cols)).astype(np.float32)
    pkg.check(gpu.lib.lv_norm_gemv(gpu.handle, d_out, dW, qn.Q4_0_V1, dx, gpu.upload(nw), rows, cols, 1))
    gpu.sync()
    close(gpu.download(d_out, np.float32, rows), ob.gemv(W, qn.Q4_0, ob.norm(x, nw), rows, cols, workers_for(cols), version=1))
    if rows % 2 == 0 and rows >= 4096:
        half = rows // 2
        d_g = gpu.alloc(half * 4)
        rb = cols // 32 * 20
        pkg.check(gpu.lib.lv_gemv_silu(gpu.handle, d_g, dW, pkg.offset(dW, half * rb), qn.Q4_0_V1, dx, half, cols, 1))
        gpu.sync()
        close(gpu.download(d_g, np.float32, half), ob.gemv_silu(W[:half * rb], W[half * rb:], qn.Q4_0, x, half, cols, workers_for(cols), version=1))
        gpu.free(d_g)
    for d in (dW, dx, d_out):
        gpu.free(d)


def test_dequant_rows_of_version_1_blocks_bit_exact(gpu, pkg):
    rng = np.random.default_rng(41)
    vocab, cols = 64, 4096
    table = qn.quantize_q4_0_v1((rng.standard_normal((vocab, cols)) * 0.02).astype(np.float32))
    ids = np.array([5, 0, 63, 17], np.uint32)
    d_out = gpu.alloc(ids.size * cols * 4)
    pkg.check(gpu.lib.lv_dequant_rows(gpu.handle, d_out, gpu.upload(table), qn.Q4_0_V1, gpu.upload(ids), None, cols, vocab, ids.size))
    gpu.sync()
    got = gpu.download(d_out, np.float32, ids.size * cols).reshape(ids.size, cols)
    rb = cols // 32 * 20
    for z, t in enumerate(ids):
        assert np.array_equal(got[z].view(np.uint32), ob.dequant(table[t * rb:(t + 1) * rb], qn.Q4_0, cols, version=1).view(np.uint32))


def _outlier_activations(rng, cols):
    """Activations as a trained LLaMA's residual stream has them: a few channels two to three orders of
    magnitude above the rest -- alone in a 32-block, several in one block, in many blocks -- plus an
    all-zero block and a block of denormals.  The GEMV stores each block of activations as fixed point
    relative to the block's largest magnitude, so these are the inputs that stress it most."""
    x = rng.standard_normal(cols).astype(np.float32)
    x[5] *= 1000.0                                   # one outlier alone in its block
    x[64:96:7] *= 300.0                              # several in one block
    x[3 * 32 + 1] = -850.0
    x[np.arange(7, cols, 416)] *= 120.0              # spread over many blocks
    x[10 * 32:11 * 32] = 0.0                         # an all-zero block
    x[12 * 32:13 * 32] = (rng.standard_normal(32) * 1e-41).astype(np.float32)    # denormals only
    x[14 * 32:15 * 32] = 0.0
    x[14 * 32 + 9] = 512.0                           # a block that is one outlier and nothing else
    return x


@pytest.mark.parametrize("wtype,rows,cols", [(qn.Q4_0, 4096, 4096), (qn.Q4_0, 4096, 11008), (qn.Q8_0, 4096, 4096), (qn.Q8_0, 1024, 11008)])
def test_gemv_with_outlier_activations(gpu, pkg, wtype, rows, cols):
    rng = np.random.default_rng(77 + rows + cols + wtype)
    W = qn.quantize((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32), wtype)
    x = _outlier_activations(rng, cols)
    dW, dx = gpu.upload(W), gpu.upload(x)
    d_out = gpu.alloc(rows * 4)
    pkg.check(gpu.lib.lv_gemv(gpu.handle, d_out, dW, wtype, dx, rows, cols, 1, 0))
    gpu.sync()
    close(gpu.download(d_out, np.float32, rows), ob.gemv(W, wtype, x, rows, cols, workers_for(cols)))
    for d in (dW, dx, d_out):
        gpu.free(d)


def test_norm_gate_up_silu_with_outlier_activations(gpu, pkg):
    rng = np.random.default_rng(78)
    ff, dim = 11008, 4096
    w3 = qn.quantize_q4_0((rng.standard_normal((ff, dim)) * 0.02).astype(np.float32))
    w1 = qn.quantize_q4_0((rng.standard_normal((ff, dim)) * 0.02).astype(np.float32))
    x = _outlier_activations(rng, dim)
    nw = (1 + 0.01 * rng.standard_normal(dim)).astype(np.float32)
    d_out = gpu.alloc(ff * 4)
    pkg.check(gpu.lib.lv_norm_gate_up_silu(gpu.handle, d_out, gpu.upload(w3), gpu.upload(w1), qn.Q4_0, gpu.upload(x), gpu.upload(nw), ff, dim, 1))
    gpu.sync()
    close(gpu.download(d_out, np.float32, ff), ob.gemv_silu(w3, w1, qn.Q4_0, ob.norm(x, nw), ff, dim, 128))


@pytest.mark.parametrize("wtype,ff,dim", [(qn.Q4_0, 11008, 4096), (qn.Q8_0, 11008, 4096), (qn.Q4_0, 13824, 5120)])
def test_gemv_silu(gpu, pkg, wtype, ff, dim):
    rng = np.random.default_rng(ff)
    w3 = qn.quantize((rng.standard_normal((ff, dim)) * 0.02).astype(np.float32), wtype)
    w1 = qn.quantize((rng.standard_normal((ff, dim)) * 0.02).astype(np.float32), wtype)
    x = rng.standard_normal(dim).astype(np.float32)
    d3, d1, dx = gpu.upload(w3), gpu.upload(w1), gpu.upload(x)
    d_out = gpu.alloc(ff * 4)
    pkg.check(gpu.lib.lv_gemv_silu(gpu.handle, d_out, d3, d1, wtype, dx, ff, dim, 1))
    gpu.sync()
    close(gpu.download(d_out, np.float32, ff), ob.gemv_silu(w3, w1, wtype, x, ff, dim, workers_for(dim)))
    for d in (d3, d1, dx, d_out):
        gpu.free(d)


def test_gemv_batch_rows_are_independent(gpu, pkg):
    rng = np.random.default_rng(22)
    rows, cols, batch = 512, 4096, 3
    W = qn.quantize_q4_0((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    d_out = gpu.alloc(batch * rows * 4)
    pkg.check(gpu.lib.lv_gemv(gpu.handle, d_out, gpu.upload(W), qn.Q4_0, gpu.upload(x), rows, cols, batch, 0))
    gpu.sync()
    got = gpu.download(d_out, np.float32, batch * rows).reshape(batch, rows)
    for z in range(batch):
        close(got[z], ob.gemv(W, qn.Q4_0, x[z], rows, cols, 128))


def test_norm_fused_gemv_matches_norm_then_gemv(gpu, pkg):
    rng = np.random.default_rng(23)
    rows, cols = 1024, 4096
    W = qn.quantize_q4_0((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    x = (rng.standard_normal(cols) * 2).astype(np.float32)
    nw = (1 + 0.01 * rng.standard_normal(cols)).astype(np.float32)
    d_out = gpu.alloc(rows * 4)
    pkg.check(gpu.lib.lv_norm_gemv(gpu.handle, d_out, gpu.upload(W), qn.Q4_0, gpu.upload(x), gpu.upload(nw), rows, cols, 1))
    gpu.sync()
    close(gpu.download(d_out, np.float32, rows), ob.gemv(W, qn.Q4_0, ob.norm(x, nw), rows, cols, 128))


def test_gemv_rejects_bad_arguments(gpu, pkg):
    lib = gpu.lib
    d = gpu.alloc(4096)
    assert lib.lv_gemv(gpu.handle, d, d, 3, d, 4, 256, 1, 0) == pkg.LV_ERR_BAD_ARGUMENTS        # q4_1 unsupported
    assert lib.lv_gemv(gpu.handle, d, d, qn.Q4_0, d, 4, 96, 1, 0) == pkg.LV_ERR_BAD_ARGUMENTS   # cols % 256
    assert lib.lv_gemv(gpu.handle, d, d, qn.Q4_0, d, 6, 256, 1, 0) == pkg.LV_ERR_BAD_ARGUMENTS  # rows % 4
    assert lib.lv_gemv(gpu.handle, d, pkg.offset(d, 2), qn.Q4_0, d, 4, 256, 1, 0) == pkg.LV_ERR_BAD_ARGUMENTS
    assert lib.lv_gemv(None, d, d, qn.Q4_0, d, 4, 256, 1, 0) == pkg.LV_ERR_BAD_ARGUMENTS
    assert b"" != lib.lv_last_error_string()


def test_kv_append_bit_exact(gpu, pkg):
    rng = np.random.default_rng(24)
    batch, ctx_rows, pos = 3, 16, 5
    x = np.concatenate([rng.standard_normal((batch, DIM - 6)) * 2, np.tile([1e-7, 65519.0, 7e4, -0.0, 6.1e-5, 1.0009766], (batch, 1))], 1).astype(np.float32)
    cache = gpu.zeros(ctx_rows * DIM * 2)
    pkg.check(gpu.lib.lv_kv_append_f16(gpu.handle, cache, gpu.upload(x), u32_dev(gpu, pos), DIM, batch, ctx_rows))
    gpu.sync()
    got = gpu.download(cache, np.uint16, ctx_rows * DIM).reshape(ctx_rows, DIM)
    want = np.zeros((ctx_rows, DIM), np.uint16)
    with np.errstate(over="ignore"):
        want[pos:pos + batch] = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)
    assert np.array_equal(want[pos], ob.f32_to_f16_bits(x[0]))
    # a row outside the cache is refused and reported, never written
    pkg.check(gpu.lib.lv_kv_append_f16(gpu.handle, cache, gpu.upload(x), u32_dev(gpu, ctx_rows - 1), DIM, batch, ctx_rows))
    with pytest.raises(pkg.LvError) as e:
        gpu.sync()
    assert e.value.code == pkg.LV_ERR_DEVICE_WAIT
    gpu.sync()      # the error word was cleared


def _caches(rng, n, rows):
    k = np.zeros((rows, DIM), np.float16)
    v = np.zeros((rows, DIM), np.float16)
    k[:n] = (rng.standard_normal((n, DIM)) * 0.7).astype(np.float16)
    v[:n] = (rng.standard_normal((n, DIM)) * 0.7).astype(np.float16)
    return k.view(np.uint16), v.view(np.uint16)


@pytest.fixture(scope="module")
def rope_table(gpu, pkg):
    t = gpu.alloc(2048 * ROT * 4)
    pkg.check(gpu.lib.lv_rope_table_build(gpu.handle, t, 2048, ROT))
    return t


@pytest.mark.parametrize("pos,backlog", [(0, 128), (1, 128), (63, 128), (64, 128), (127, 128), (300, 512)])
def test_three_attention_ops_match_reference_shaders(gpu, pkg, rope_table, pos, backlog):
    rng = np.random.default_rng(100 + pos)
    k, v = _caches(rng, pos + 1, backlog)
    q = rng.standard_normal(DIM).astype(np.float32)
    lib, h = gpu.lib, gpu.handle
    dk, dv, dq, dpos = gpu.upload(k), gpu.upload(v), gpu.upload(q), u32_dev(gpu, pos)
    d_scores = gpu.alloc(backlog * HEADS * 4)
    d_out = gpu.alloc(DIM * 4)
    pkg.check(lib.lv_attn_scores_rope(h, d_scores, dk, dq, dpos, rope_table, backlog, HEADS, ROT, 1))
    gpu.sync()
    scores = gpu.download(d_scores, np.float32, backlog * HEADS).reshape(backlog, HEADS)
    want_scores = ob.mhsa(k, q, pos, HEADS, ROT)
    close(scores[: pos + 1], want_scores, rel_l2=2e-6, max_abs_frac=1e-5)
    assert np.all(scores[pos + 1:] == 0)
    pkg.check(lib.lv_softmax_masked(h, d_scores, dpos, backlog, HEADS, ROT, 1))
    gpu.sync()
    probs = gpu.download(d_scores, np.float32, backlog * HEADS).reshape(backlog, HEADS)
    want_probs = ob.softmax(want_scores, pos, backlog, HEADS, ROT)
    close(probs, want_probs, rel_l2=5e-6, max_abs_frac=1e-5)
    assert np.all(probs[pos + 1:] == 0)
    pkg.check(lib.lv_attn_values(h, d_out, dv, d_scores, backlog, HEADS, ROT, 1))
    gpu.sync()
    close(gpu.download(d_out, np.float32, DIM), ob.kqv(v, want_probs, backlog, HEADS, ROT), rel_l2=5e-6, max_abs_frac=2e-5)
    for d in (dk, dv, dq, d_scores, d_out):
        gpu.free(d)


@pytest.mark.parametrize("grid", ["whole-cache", "backlog"])
@pytest.mark.parametrize("pos", [0, 1, 31, 32, 63, 64, 65, 127, 128, 255, 256, 300, 511, 1023, 1500, 2047])
def test_fused_attention(gpu, pkg, rope_table, pos, grid):
    """grid "whole-cache": one CTA per 256 rows of the 2048-row cache (more CTAs than SMs: the variant with
    the compact rotation table); "backlog": only the current backlog, as a session launches it (at most
    one CTA per SM up to a backlog of 1024: exact table rows staged)."""
    rng = np.random.default_rng(200 + pos)
    backlog = 128
    while backlog <= pos:
        backlog *= 2
    max_ctx = 2048 if grid == "whole-cache" else backlog
    k, v = _caches(rng, pos + 1, max_ctx)
    q = rng.standard_normal(DIM).astype(np.float32)
    nbytes = gpu.lib.lv_attention_scratch_bytes(HEADS, ROT, max_ctx, 1)
    assert nbytes > 0
    scratch = gpu.zeros(nbytes)
    dk, dv, dq = gpu.upload(k), gpu.upload(v), gpu.upload(q)
    d_out = gpu.alloc(DIM * 4)
    want = ob.attention(k, v, q, pos, backlog, HEADS, ROT)
    for _ in range(2):       # the second launch proves the arrival counters were reset
        pkg.check(gpu.lib.lv_memset(gpu.handle, d_out, 0xFF, DIM * 4))
        pkg.check(gpu.lib.lv_attention_fused(gpu.handle, d_out, dq, dk, dv, u32_dev(gpu, pos), rope_table, scratch,
                                             HEADS, ROT, max_ctx, 1))
        gpu.sync()
        # grids with more CTAs than SMs (here: the 2048-row cache) form cos/sin of a distance from two table
        # rows; a few units in the last place per rotation add up over two thousand rows
        close(gpu.download(d_out, np.float32, DIM), want, rel_l2=5e-6 if max_ctx < 2048 else 1e-5, max_abs_frac=2e-5)
    for d in (dk, dv, dq, d_out, scratch):
        gpu.free(d)


def test_fused_attention_refuses_a_position_outside_the_cache(gpu, pkg, rope_table):
    """A position word at or beyond max_ctx would index past the caches and the rotation table: the kernel
    reports it through the error word and writes nothing (like lv_kv_append_f16), and the arrival counters
    stay clear, so the next call with a valid position is unaffected."""
    rng = np.random.default_rng(32)
    for batch, max_ctx in ((1, 256), (6, 512)):         # one CTA per SM / the two-CTAs-per-SM variant
        k, v = _caches(rng, max_ctx, max_ctx)
        q = rng.standard_normal((batch, DIM)).astype(np.float32)
        scratch = gpu.zeros(gpu.lib.lv_attention_scratch_bytes(HEADS, ROT, max_ctx, batch))
        dk, dv, dq = gpu.upload(k), gpu.upload(v), gpu.upload(q)
        d_out = gpu.alloc(batch * DIM * 4)
        pkg.check(gpu.lib.lv_memset(gpu.handle, d_out, 0xA5, batch * DIM * 4))
        pkg.check(gpu.lib.lv_attention_fused(gpu.handle, d_out, dq, dk, dv, u32_dev(gpu, max_ctx), rope_table, scratch, HEADS, ROT, max_ctx, batch))
        with pytest.raises(pkg.LvError) as e:
            gpu.sync()
        assert e.value.code == pkg.LV_ERR_DEVICE_WAIT
        assert np.all(gpu.download(d_out, np.uint8, batch * DIM * 4) == 0xA5)
        # the refused call left no trace: the next one, with every row of the batch inside the cache, is correct
        pos = max_ctx - batch
        pkg.check(gpu.lib.lv_attention_fused(gpu.handle, d_out, dq, dk, dv, u32_dev(gpu, pos), rope_table, scratch, HEADS, ROT, max_ctx, batch))
        gpu.sync()
        got = gpu.download(d_out, np.float32, batch * DIM).reshape(batch, DIM)
        for z in range(batch):
            close(got[z], ob.attention(k, v, q[z], pos + z, max_ctx, HEADS, ROT), rel_l2=1e-5, max_abs_frac=2e-5)
        for d in (dk, dv, dq, d_out, scratch):
            gpu.free(d)


def test_fused_attention_batch_is_causal(gpu, pkg, rope_table):
    rng = np.random.default_rng(31)
    batch, pos, max_ctx = 4, 70, 256
    k, v = _caches(rng, pos + batch, max_ctx)
    q = rng.standard_normal((batch, DIM)).astype(np.float32)
    scratch = gpu.zeros(gpu.lib.lv_attention_scratch_bytes(HEADS, ROT, max_ctx, batch))
    d_out = gpu.alloc(batch * DIM * 4)
    pkg.check(gpu.lib.lv_attention_fused(gpu.handle, d_out, gpu.upload(q), gpu.upload(k), gpu.upload(v), u32_dev(gpu, pos),
                                         rope_table, scratch, HEADS, ROT, max_ctx, batch))
    gpu.sync()
    got = gpu.download(d_out, np.float32, batch * DIM).reshape(batch, DIM)
    for z in range(batch):       # row z sees cache rows 0 .. pos + z (softmax.comp:35)
        close(got[z], ob.attention(k, v, q[z], pos + z, 128, HEADS, ROT), rel_l2=5e-6, max_abs_frac=2e-5)


def test_qkv_fused_writes_cache_rows_and_query(gpu, pkg):
    rng = np.random.default_rng(32)
    ctx_rows, pos, batch = 8, 3, 2
    ws = [qn.quantize_q4_0((rng.standard_normal((DIM, DIM)) * 0.02).astype(np.float32)) for _ in range(3)]
    wq, wk, wv = ws
    x = (rng.standard_normal((batch, DIM)) * 2).astype(np.float32)
    nw = (1 + 0.01 * rng.standard_normal(DIM)).astype(np.float32)
    dkc, dvc = gpu.zeros(ctx_rows * DIM * 2), gpu.zeros(ctx_rows * DIM * 2)
    dq = gpu.alloc(batch * DIM * 4)
    pkg.check(gpu.lib.lv_norm_qkv_kvappend(gpu.handle, dq, dkc, dvc, gpu.upload(wq), gpu.upload(wk), gpu.upload(wv), qn.Q4_0,
                                           gpu.upload(x), gpu.upload(nw), u32_dev(gpu, pos), DIM, DIM, batch, ctx_rows))
    gpu.sync()
    gq = gpu.download(dq, np.float32, batch * DIM).reshape(batch, DIM)
    gk = gpu.download(dkc, np.uint16, ctx_rows * DIM).reshape(ctx_rows, DIM).view(np.float16).astype(np.float32)
    gv = gpu.download(dvc, np.uint16, ctx_rows * DIM).reshape(ctx_rows, DIM).view(np.float16).astype(np.float32)
    for z in range(batch):
        h = ob.norm(x[z], nw)
        close(gq[z], ob.gemv(wq, qn.Q4_0, h, DIM, DIM, 128))
        # f16 rounding of a value that differs in the last fp32 bits may land on the neighbouring half
        close(gk[pos + z], ob.gemv(wk, qn.Q4_0, h, DIM, DIM, 128), rel_l2=6e-4, max_abs_frac=1e-3)
        close(gv[pos + z], ob.gemv(wv, qn.Q4_0, h, DIM, DIM, 128), rel_l2=6e-4, max_abs_frac=1e-3)
    assert not gk[:pos].any() and not gk[pos + batch:].any()


def test_argmax_copy_add(gpu, pkg):
    rng = np.random.default_rng(33)
    lib, h = gpu.lib, gpu.handle
    d_idx = gpu.alloc(16)
    for case in range(4):
        v = rng.standard_normal(32000).astype(np.float32)
        if case == 1:
            v[[31999, 777, 12345]] = v.max() + 1        # ties: lowest index wins
        if case == 2:
            v[5] = np.nan
        if case == 3:
            v[0] = np.nan
        pkg.check(lib.lv_argmax_f32(h, d_idx, gpu.upload(v), v.size))
        gpu.sync()
        assert gpu.download(d_idx, np.uint32, 1)[0] == ob.load().orc_argmax(ob.ptr(v), v.size)
    a, b = rng.standard_normal(5000).astype(np.float32), rng.standard_normal(5000).astype(np.float32)
    da, db, dc = gpu.upload(a), gpu.upload(b), gpu.alloc(a.nbytes)
    pkg.check(lib.lv_copy_f32(h, dc, da, a.size))
    pkg.check(lib.lv_add_f32(h, da, db, a.size))
    gpu.sync()
    assert np.array_equal(gpu.download(dc, np.float32, a.size), a)
    assert np.array_equal(gpu.download(da, np.float32, a.size), a + b)


def test_argmax_odd_sizes_and_unaligned_start(gpu, pkg):
    rng = np.random.default_rng(35)
    lib, h = gpu.lib, gpu.handle
    d_idx = gpu.alloc(16)
    big = rng.standard_normal(40000).astype(np.float32)
    big[[3, 20001, 39999]] = 9.0                        # equal maxima at both ends of the vector paths
    d_big = gpu.upload(big)
    for first, n in ((0, 1), (0, 3), (1, 4097), (0, 32769), (2, 39998), (3, 37), (4, 36001)):
        pkg.check(lib.lv_argmax_f32(h, d_idx, C.c_void_p(d_big.value + 4 * first), n))
        gpu.sync()
        v = np.ascontiguousarray(big[first:first + n])
        assert gpu.download(d_idx, np.uint32, 1)[0] == ob.load().orc_argmax(ob.ptr(v), n), (first, n)


def test_argmax_advance_logs_the_token_and_moves_the_position(gpu, pkg):
    """One launch = lv_argmax_f32 + lv_decode_advance, plus the token in mapped host memory."""
    rng = np.random.default_rng(36)
    lib, h = gpu.lib, gpu.handle
    host = C.c_void_p()
    pkg.check(lib.lv_host_alloc(h, 64, C.byref(host)))
    word = (C.c_uint32 * 16).from_address(host.value)
    try:
        for case, batch in ((0, 1), (1, 3), (2, 1)):
            v = rng.standard_normal(32000).astype(np.float32)
            if case == 1:
                v[[31000, 42]] = v.max() + 2
            if case == 2:
                v[0] = np.nan
            want = ob.load().orc_argmax(ob.ptr(v), v.size)
            cfg, log, am = u32_dev(gpu, 7), gpu.upload(np.full(32, 0xFFFFFFFF, np.uint32)), gpu.zeros(4)
            word[5] = 0xDEADBEEF
            pkg.check(lib.lv_argmax_advance(h, gpu.upload(v), v.size, cfg, log, batch, 32, am, C.c_void_p(host.value + 20)))
            gpu.sync()
            assert word[5] == want
            assert gpu.download(am, np.uint32, 1)[0] == want
            got_log = gpu.download(log, np.uint32, 32)
            assert got_log[7 + batch] == want and (np.delete(got_log, 7 + batch) == 0xFFFFFFFF).all()
            assert (gpu.download(cfg, np.uint32, 4) == 7 + batch).all()
        # a log index outside the log is reported, not written
        cfg, log = u32_dev(gpu, 31), gpu.upload(np.full(32, 0xFFFFFFFF, np.uint32))
        pkg.check(lib.lv_argmax_advance(h, gpu.upload(np.ones(64, np.float32)), 64, cfg, log, 1, 32, None, None))
        assert lib.lv_stream_sync(h, 10000) == pkg.LV_ERR_DEVICE_WAIT
        assert (gpu.download(log, np.uint32, 32) == 0xFFFFFFFF).all()
    finally:
        pkg.check(lib.lv_host_free(h, host))


def test_graph_capture_replays_with_a_new_position(gpu, pkg, rope_table):
    """The recorded step reads the position from device memory, so one graph serves every token."""
    rng = np.random.default_rng(34)
    ctx_rows = 16
    x = rng.standard_normal((1, DIM)).astype(np.float32)
    cache = gpu.zeros(ctx_rows * DIM * 2)
    dpos, dx = u32_dev(gpu, 2), gpu.upload(x)
    g = C.c_void_p()
    pkg.check(gpu.lib.lv_graph_begin_capture(gpu.handle))
    pkg.check(gpu.lib.lv_kv_append_f16(gpu.handle, cache, dx, dpos, DIM, 1, ctx_rows))
    pkg.check(gpu.lib.lv_graph_end_capture(gpu.handle, C.byref(g)))
    for pos in (2, 9):
        p = np.array([pos] * 4, np.uint32)
        pkg.check(gpu.lib.lv_upload(gpu.handle, dpos, p.ctypes.data_as(C.c_void_p), 16))
        pkg.check(gpu.lib.lv_graph_launch(gpu.handle, g))
        gpu.sync()
    got = gpu.download(cache, np.uint16, ctx_rows * DIM).reshape(ctx_rows, DIM)
    want = x.astype(np.float16).view(np.uint16)[0]
    assert np.array_equal(got[2], want) and np.array_equal(got[9], want)
    assert not got[[0, 1, 3, 8, 10]].any()
    pkg.check(gpu.lib.lv_graph_destroy(g))


@pytest.mark.parametrize("two_phase", ["0", "1"], ids=["sum-per-cta", "sum-per-gpu"])
def test_exchange_fused_into_the_gemvs_on_one_rank(pkg, two_phase, monkeypatch):
    """lv_tp_arm_push / lv_tp_arm_pull with a single-rank window: the pushed rows of one GEMV come
    back as `x + rows` in the input of the next normalising GEMV, which also stores that sum.  Both
    ways of forming the sum (in every CTA; one slice per CTA, then shared through local flags)."""
    monkeypatch.setenv("LV_TP_TWO_PHASE", two_phase)
    rng = np.random.default_rng(60)
    K, rows_out, steps = 1024, 512, 3
    Wa = qn.quantize_q4_0((rng.standard_normal((K, 512)) * 0.05).astype(np.float32))      # K rows of 512 columns
    Wb = qn.quantize_q4_0((rng.standard_normal((rows_out, K)) * 0.05).astype(np.float32))
    nw = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    with pkg.Context(0) as g:
        lib, h = g.lib, g.handle
        handle = (C.c_uint8 * 64)()
        pkg.check(lib.lv_peer_window_create(h, 1, K, handle))
        pkg.check(lib.lv_peer_connect(h, 0, handle))
        cfg, dWa, dWb, dnw = u32_dev(g, 0), g.upload(Wa), g.upload(Wb), g.upload(nw)
        for step in range(steps):                       # a new step number (flag epoch) every round
            v = rng.standard_normal(512).astype(np.float32)
            x = rng.standard_normal(K).astype(np.float32)
            dx, dxo, dout, dummy = g.upload(x), g.zeros(K * 4), g.zeros(rows_out * 4), g.zeros(K * 4)
            for exchange in (0, 1):                     # both slot sets
                pkg.check(lib.lv_tp_arm_push(h, exchange, 2))
                pkg.check(lib.lv_gemv(h, dummy, dWa, qn.Q4_0, g.upload(v), K, 512, 1, 0))
                pkg.check(lib.lv_tp_arm_pull(h, exchange, 2, K, dxo))
                pkg.check(lib.lv_norm_gemv(h, dout, dWb, qn.Q4_0, dx, dnw, rows_out, K, 1))
                g.sync()
                partial = ob.gemv(Wa, qn.Q4_0, v, K, 512, 128)
                close(g.download(dxo, np.float32, K), x + partial, rel_l2=2e-6, max_abs_frac=2e-6)
                close(g.download(dout, np.float32, rows_out), ob.gemv(Wb, qn.Q4_0, ob.norm(x + partial, nw), rows_out, K, 128))
                assert not g.download(dummy, np.float32, K).any()          # a pushing GEMV does not write its `out`
            pkg.check(lib.lv_decode_advance(h, cfg, None, None, 1, 0))      # ends the step: the next epochs differ
        # an armed role without connected windows is refused, as is an exchange index outside the step
        assert lib.lv_tp_arm_push(h, 2, 2) == pkg.LV_ERR_BAD_ARGUMENTS
        pkg.check(lib.lv_peer_destroy(h))
        assert lib.lv_tp_arm_push(h, 0, 2) == pkg.LV_ERR_BAD_ARGUMENTS

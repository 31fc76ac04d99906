"""Batched products on the tensor cores (lv_gemm_tc*) against the CPU oracle's per-token GEMV.

The oracle (matmul.glsl restated) is evaluated token by token.  The products that enter the tensor
cores are exact; their fp32 accumulator truncates instead of rounding, which over K = 4096..11008
leaves a relative error of about 1e-5, so the tolerances here are rel-L2 <= 3e-5 and max-abs <=
1e-4 of the largest output (the GEMV tests hold 1e-5), the f16 cache rows up to a neighbouring half.

Every test runs in both forms of the q4_0 weight tiles.  "exact" (hi/lo fp16 pair) is held to the tolerances above.
"fast" (one fp16 plane: each weight rounded to 11 significant bits, the default of the library) is held to the same
tight tolerances against the product with fp16-rounded weights -- the kernel does what it says -- and to rel-L2 <=
5e-4 / max-abs <= 2e-3 of the largest output against the oracle (observed: 1.5e-4 for one product, 3.1e-4 for the gated
pair): what the rounding of the weights costs.  Both forms exist for q4_0 and q8_0 matrices.
"""
import ctypes as C

import numpy as np
import pytest

import oracle_bind as ob
import quant_np as qn

pytestmark = pytest.mark.gpu

FAST_REL_L2, FAST_MAX_ABS_FRAC = 5e-4, 2e-3


@pytest.fixture(autouse=True, params=["exact", "fast"])
def form(request, gpu, pkg):
    pkg.check(gpu.lib.lv_gemm_tc_set_exact(gpu.handle, int(request.param == "exact")))
    yield request.param
    pkg.check(gpu.lib.lv_gemm_tc_set_exact(gpu.handle, 0))


def loose(form, wtype, rel_l2=3e-5, max_abs_frac=1e-4):
    """Tolerances against the oracle for this form and weight type."""
    if form == "fast":
        return dict(rel_l2=max(rel_l2, FAST_REL_L2), max_abs_frac=max(max_abs_frac, FAST_MAX_ABS_FRAC))
    return dict(rel_l2=rel_l2, max_abs_frac=max_abs_frac)


def rounded_weights_product(W, x, rows, cols, wtype=qn.Q4_0):
    """x @ fp16(w)^T in float64: what the fast form computes, up to the accumulation order."""
    w16 = qn.dequantize_np(W, wtype).reshape(rows, cols).astype(np.float16).astype(np.float64)
    return x.astype(np.float64) @ w16.T


def close(got, want, rel_l2=3e-5, max_abs_frac=1e-4):
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    assert got.shape == want.shape
    assert np.all(np.isfinite(got))
    l2 = np.linalg.norm(got - want) / (np.linalg.norm(want) or 1.0)
    mx = np.abs(got - want).max()
    assert l2 <= rel_l2, f"rel-L2 {l2:.3e}"
    assert mx <= max_abs_frac * (np.abs(want).max() or 1.0), f"max-abs {mx:.3e}"


def workers_for(cols):
    return 32 if cols == 5120 else 128


def split(gpu, pkg, x, norm_w=None):
    batch, cols = x.shape
    xh = gpu.alloc(gpu.lib.lv_act_split_bytes(cols, batch))
    pkg.check(gpu.lib.lv_act_split_f16(gpu.handle, xh, gpu.upload(x), None if norm_w is None else gpu.upload(norm_w), cols, batch))
    return xh


def matrix(rng, rows, cols, scale=0.02, wtype=qn.Q4_0):
    return qn.quantize((rng.standard_normal((rows, cols)) * scale).astype(np.float32), wtype)


def planes_of(raw, zpad, cols):
    """Undo the tile layout of lv_act_split_f16: [cols/64][2 zpad rows][8 units ^ (row & 7)][8] -> (hi, lo) as [zpad][cols]."""
    t = raw.reshape(cols // 64, 2 * zpad, 8, 8)
    out = np.empty_like(t)
    for r in range(2 * zpad):
        for u in range(8):
            out[:, r, u] = t[:, r, u ^ (r & 7)]
    rows = out.reshape(cols // 64, 2 * zpad, 64).transpose(1, 0, 2).reshape(2 * zpad, cols)
    return rows[:zpad].astype(np.float64), rows[zpad:].astype(np.float64)


def test_act_split_planes_add_up_to_the_input(gpu, pkg):
    rng = np.random.default_rng(50)
    batch, cols = 5, 512
    x = (rng.standard_normal((batch, cols)) * np.exp(rng.uniform(-6, 6, (batch, cols)))).astype(np.float32)
    x = np.clip(x, -6e4, 6e4)
    xh = split(gpu, pkg, x)
    gpu.sync()
    hi, lo = planes_of(gpu.download(xh, np.float16, 2 * 16 * cols), 16, cols)
    assert not hi[batch:].any() and not lo[batch:].any()                  # padding tokens are zero
    err = np.abs(hi[:batch] + lo[:batch] - x)
    assert (err <= np.maximum(np.abs(x) * 2.0 ** -21, 2.0 ** -24)).all()
    assert np.array_equal(hi[:batch].astype(np.float16), x.astype(np.float16))
    # with a norm: same as the oracle's normalisation
    w = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    xs = rng.standard_normal((batch, cols)).astype(np.float32)
    xh = split(gpu, pkg, xs, w)
    gpu.sync()
    hi, lo = planes_of(gpu.download(xh, np.float16, 2 * 16 * cols), 16, cols)
    for z in range(batch):
        close(hi[z] + lo[z], ob.norm(xs[z], w), rel_l2=2e-6, max_abs_frac=2e-6)


@pytest.mark.parametrize("wtype", [qn.Q4_0, qn.Q8_0], ids=["q4_0", "q8_0"])
@pytest.mark.parametrize("rows,cols,batch", [(128, 256, 16), (256, 4096, 5), (4096, 4096, 64), (384, 11008, 33), (640, 5120, 17),
                                             (160, 512, 16), (4000, 1024, 9)])       # the last two end in a ragged row tile
def test_gemm_tc_store_and_add(gpu, pkg, rows, cols, batch, wtype, form):
    rng = np.random.default_rng(51)
    W = matrix(rng, rows, cols, wtype=wtype)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    xh = split(gpu, pkg, x)
    want = np.stack([ob.gemv(W, wtype, x[z], rows, cols, workers_for(cols)) for z in range(batch)])
    dW = gpu.upload(W)
    out = gpu.upload(np.full((batch + 1, rows), 7.0, np.float32))
    pkg.check(gpu.lib.lv_gemm_tc(gpu.handle, out, dW, wtype, xh, rows, cols, batch, 0))
    gpu.sync()
    got = gpu.download(out, np.float32, (batch + 1) * rows).reshape(batch + 1, rows)
    close(got[:batch], want, **loose(form, wtype))
    if form == "fast":
        close(got[:batch], rounded_weights_product(W, x, rows, cols, wtype))
    assert (got[batch] == 7.0).all()                                     # nothing written past the batch
    base = rng.standard_normal((batch, rows)).astype(np.float32)
    out = gpu.upload(base)
    pkg.check(gpu.lib.lv_gemm_tc(gpu.handle, out, dW, wtype, xh, rows, cols, batch, 1))
    gpu.sync()
    close(gpu.download(out, np.float32, batch * rows).reshape(batch, rows), base + want, **loose(form, wtype))


def test_gemm_tc_extreme_scales_are_exact_products(gpu, pkg, form):
    """Blocks whose scale is tiny, huge or negative: hi + lo reproduces (q - 8) * d exactly; the single plane of the
    fast form reproduces fp16((q - 8) * d), subnormal products included."""
    rng = np.random.default_rng(52)
    rows, cols, batch = 128, 256, 16
    W = matrix(rng, rows, cols).reshape(rows, cols // 32, 18).copy()
    scales = np.array([6.1e-5, 3.0e-6, 1.0, -0.37, 1000.0, 0.0999, 2.0 ** -20, 7.77], np.float16).view(np.uint8).reshape(8, 2)
    W[:, :, 0:2] = scales[None, :, :]
    W = W.reshape(-1)
    x = (rng.integers(-8, 9, (batch, cols)) / 8.0).astype(np.float32)    # exactly representable inputs: the result is exact in fp32 order-free
    xh = split(gpu, pkg, x)
    out = gpu.zeros(batch * rows * 4)
    pkg.check(gpu.lib.lv_gemm_tc(gpu.handle, out, gpu.upload(W), qn.Q4_0, xh, rows, cols, batch, 0))
    gpu.sync()
    want = x.astype(np.float64) @ qn.dequantize_np(W, qn.Q4_0).reshape(rows, cols).astype(np.float64).T
    if form == "fast":
        want = rounded_weights_product(W, x, rows, cols)
    close(gpu.download(out, np.float32, batch * rows).reshape(batch, rows), want, rel_l2=2e-6, max_abs_frac=2e-6)


@pytest.mark.parametrize("wtype", [qn.Q4_0, qn.Q8_0], ids=["q4_0", "q8_0"])
@pytest.mark.parametrize("ff,dim,batch", [(192, 512, 16), (256, 4096, 24), (11008, 4096, 20)])     # the middle one is split along K
def test_gemm_tc_silu_pair(gpu, pkg, ff, dim, batch, wtype, form):
    rng = np.random.default_rng(53)
    w3, w1 = matrix(rng, ff, dim, wtype=wtype), matrix(rng, ff, dim, wtype=wtype)
    x = rng.standard_normal((batch, dim)).astype(np.float32)
    nw = (1 + 0.05 * rng.standard_normal(dim)).astype(np.float32)
    xh = split(gpu, pkg, x, nw)
    out = gpu.zeros(batch * ff * 4)
    pkg.check(gpu.lib.lv_gemm_tc_silu(gpu.handle, out, gpu.upload(w3), gpu.upload(w1), wtype, xh, ff, dim, batch))
    gpu.sync()
    got = gpu.download(out, np.float32, batch * ff).reshape(batch, ff)
    for z in range(0, batch, 7):
        close(got[z], ob.gemv_silu(w3, w1, wtype, ob.norm(x[z], nw), ff, dim, workers_for(dim)), **loose(form, wtype))


@pytest.mark.parametrize("dim", [512, 1024])             # 1024: two CTAs per row tile, each with half of K
def test_gemm_tc_qkv_writes_cache_rows_at_the_position(gpu, pkg, dim, form):
    rng = np.random.default_rng(54)
    batch, ctx_rows, pos = 18, 64, 9
    wq, wk, wv = (matrix(rng, dim, dim, 0.05) for _ in range(3))
    x = rng.standard_normal((batch, dim)).astype(np.float32)
    xh = split(gpu, pkg, x)
    q = gpu.zeros(batch * dim * 4)
    kc, vc = gpu.zeros(ctx_rows * dim * 2), gpu.zeros(ctx_rows * dim * 2)
    dpos = gpu.upload(np.array([pos] * 4, np.uint32))
    pkg.check(gpu.lib.lv_gemm_tc_qkv_kvappend(gpu.handle, q, kc, vc, gpu.upload(wq), gpu.upload(wk), gpu.upload(wv), qn.Q4_0, xh,
                                              dpos, dim, dim, batch, ctx_rows))
    gpu.sync()
    gq = gpu.download(q, np.float32, batch * dim).reshape(batch, dim)
    gk = gpu.download(kc, np.float16, ctx_rows * dim).reshape(ctx_rows, dim)
    gv = gpu.download(vc, np.float16, ctx_rows * dim).reshape(ctx_rows, dim)
    for z in range(batch):
        close(gq[z], ob.gemv(wq, qn.Q4_0, x[z], dim, dim, 128), **loose(form, qn.Q4_0, rel_l2=1e-5))
        close(gk[pos + z], ob.gemv(wk, qn.Q4_0, x[z], dim, dim, 128), rel_l2=6e-4, max_abs_frac=1e-3)
        close(gv[pos + z], ob.gemv(wv, qn.Q4_0, x[z], dim, dim, 128), rel_l2=6e-4, max_abs_frac=1e-3)
    assert not gk[:pos].any() and not gk[pos + batch:].any()


def test_gemm_tc_refuses_what_it_cannot_do(gpu, pkg):
    lib, h = gpu.lib, gpu.handle
    d = gpu.zeros(1 << 16)
    assert lib.lv_gemm_tc(h, d, d, 0, d, 128, 256, 16, 0) == pkg.LV_ERR_BAD_ARGUMENTS            # f32 matrices are not taken
    assert lib.lv_gemm_tc(h, d, d, qn.Q4_0, d, 100, 256, 16, 0) == pkg.LV_ERR_BAD_ARGUMENTS      # rows not a multiple of 32
    assert lib.lv_gemm_tc(h, d, d, qn.Q4_0, d, 128, 96, 16, 0) == pkg.LV_ERR_BAD_ARGUMENTS       # cols not a multiple of 256
    assert lib.lv_gemm_tc(h, d, d, qn.Q4_0, d, 128, 256, 65, 0) == pkg.LV_ERR_BAD_ARGUMENTS      # batch above 64
    assert lib.lv_gemm_tc(h, d, d, qn.Q4_0, None, 128, 256, 16, 0) == pkg.LV_ERR_BAD_ARGUMENTS


def test_gemm_tc_split_along_k_is_reproducible(gpu, pkg, form):
    """Tiles shared by several CTAs are summed in a fixed order: two launches give the same bits, and a launch right
    after another one (the arrival counters must be back at zero) is as good as the first."""
    rng = np.random.default_rng(55)
    rows, cols, batch = 512, 4096, 40
    W = matrix(rng, rows, cols)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    xh, dW = split(gpu, pkg, x), gpu.upload(W)
    outs = []
    for _ in range(3):
        out = gpu.zeros(batch * rows * 4)
        pkg.check(gpu.lib.lv_gemm_tc(gpu.handle, out, dW, qn.Q4_0, xh, rows, cols, batch, 0))
        outs.append(out)
    gpu.sync()
    got = [gpu.download(o, np.float32, batch * rows) for o in outs]
    assert np.array_equal(got[0], got[1]) and np.array_equal(got[0], got[2])
    want = np.stack([ob.gemv(W, qn.Q4_0, x[z], rows, cols, 128) for z in range(batch)])
    close(got[0].reshape(batch, rows), want, **loose(form, qn.Q4_0))


def test_shared_memory_form_of_the_fast_tiles_in_a_child_process():
    """LV_GEMM_TC_SMEM_TILES=1 (read once per process) keeps the fast weight tile in shared memory instead of tensor memory:
    the product and pair tests of this file must hold for that kernel too."""
    import os
    import subprocess
    import sys
    if os.environ.get("LV_GEMM_TC_SMEM_TILES") == "1":
        pytest.skip("already the child")
    env = dict(os.environ, LV_GEMM_TC_SMEM_TILES="1")
    r = subprocess.run([sys.executable, "-m", "pytest", __file__, "-q", "-m", "gpu", "-k", "fast and (store_and_add or silu_pair or reproducible)"],
                       env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=900)
    tail = r.stdout.decode(errors="replace")[-600:]
    assert r.returncode == 0 and " passed" in tail, tail


def test_act_split_padded_pads_the_shard_columns_with_zeros(gpu, pkg):
    """lv_act_split_f16_padded: dense rows of cols_used values against a matrix of cols >= cols_used columns (the padded
    column shard of wo / w2 on a tensor-parallel rank)."""
    rng = np.random.default_rng(60)
    batch, used, cols = 7, 640, 768                        # a 13B head slice at 8 ranks: 20 blocks padded to 24
    x = rng.standard_normal((batch, used)).astype(np.float32)
    xh = gpu.alloc(gpu.lib.lv_act_split_bytes(cols, batch))
    pkg.check(gpu.lib.lv_act_split_f16_padded(gpu.handle, xh, gpu.upload(x), None, used, cols, batch))
    gpu.sync()
    hi, lo = planes_of(gpu.download(xh, np.float16, 2 * 16 * cols), 16, cols)
    assert np.array_equal(hi[:batch, :used].astype(np.float16), x.astype(np.float16))
    assert np.abs(hi[:batch, :used] + lo[:batch, :used] - x).max() <= 2.0 ** -21 * np.abs(x).max()
    assert not hi[:, used:].any() and not lo[:, used:].any() and not hi[batch:].any()
    assert gpu.lib.lv_act_split_f16_padded(gpu.handle, xh, gpu.upload(x), None, 644, cols, batch) == pkg.LV_ERR_BAD_ARGUMENTS
    assert gpu.lib.lv_act_split_f16_padded(gpu.handle, xh, gpu.upload(x), None, 800, cols, batch) == pkg.LV_ERR_BAD_ARGUMENTS


@pytest.mark.parametrize("rows,cols,used,batch", [(5120, 768, 640, 64), (5120, 1792, 1728, 40), (4096, 1536, 1376, 16), (640, 5120, 5120, 64)],
                         ids=["13b-wo-shard-of-8", "13b-w2-shard-of-8", "7b-w2-shard-of-8", "13b-wq-shard-of-8"])
def test_gemm_tc_on_the_shard_shapes_of_eight_ranks(gpu, pkg, rows, cols, used, batch, form):
    """The matrices a rank of 8 holds (few groups of K, padded columns): the product with the padded activation split
    against the oracle on the unpadded data."""
    rng = np.random.default_rng(61)
    W_used = (rng.standard_normal((rows, used)) * 0.02).astype(np.float32)
    W = np.zeros((rows, cols), np.float32)
    W[:, :used] = W_used
    Wq = qn.quantize(W, qn.Q4_0)
    x = rng.standard_normal((batch, used)).astype(np.float32)
    xh = gpu.alloc(gpu.lib.lv_act_split_bytes(cols, batch))
    pkg.check(gpu.lib.lv_act_split_f16_padded(gpu.handle, xh, gpu.upload(x), None, used, cols, batch))
    out = gpu.zeros(batch * rows * 4)
    pkg.check(gpu.lib.lv_gemm_tc(gpu.handle, out, gpu.upload(Wq), qn.Q4_0, xh, rows, cols, batch, 0))
    gpu.sync()
    xp = np.zeros((batch, cols), np.float32)
    xp[:, :used] = x
    want = np.stack([ob.gemv(Wq, qn.Q4_0, xp[z], rows, cols, 128) for z in range(0, batch, 5)])
    close(gpu.download(out, np.float32, batch * rows).reshape(batch, rows)[::5], want, **loose(form, qn.Q4_0))


@pytest.mark.parametrize("ff,dim,batch", [(1728, 5120, 64), (1376, 4096, 64), (96, 512, 7)], ids=["13b", "7b-ragged-last-tile", "small-ragged"])
def test_gemm_tc_silu_pair_on_the_shards_of_eight_ranks(gpu, pkg, ff, dim, batch, form):
    """11008 / 8 = 1376 rows are 21 tiles of 64 and one of 32: the last CTA's missing rows read as zero blocks and are
    not stored."""
    rng = np.random.default_rng(62)
    w3, w1 = matrix(rng, ff, dim), matrix(rng, ff, dim)
    x = rng.standard_normal((batch, dim)).astype(np.float32)
    nw = (1 + 0.05 * rng.standard_normal(dim)).astype(np.float32)
    xh = split(gpu, pkg, x, nw)
    out = gpu.upload(np.full((batch + 1, ff), 7.0, np.float32))
    pkg.check(gpu.lib.lv_gemm_tc_silu(gpu.handle, out, gpu.upload(w3), gpu.upload(w1), qn.Q4_0, xh, ff, dim, batch))
    gpu.sync()
    got = gpu.download(out, np.float32, (batch + 1) * ff).reshape(batch + 1, ff)
    for z in list(range(0, batch, 13)) + [batch - 1]:
        close(got[z], ob.gemv_silu(w3, w1, qn.Q4_0, ob.norm(x[z], nw), ff, dim, workers_for(dim)), **loose(form, qn.Q4_0))
    assert (got[batch] == 7.0).all()                                     # the ragged tile wrote nothing past the matrix

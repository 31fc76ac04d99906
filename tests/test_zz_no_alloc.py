"""lv_attention_fused_static: attention for callers that cannot allocate device
memory where they need it (inside a capture, behind a fixed memory budget, as a
plug-in that only receives its inputs and outputs).  Its scratch is built into
the library, so it must give the results of lv_attention_fused -- which takes
the scratch from the caller -- call after call, whatever the shared buffer
still holds from earlier calls.  Collected last on purpose.
"""
import numpy as np
import pytest

import quant_np  # noqa: F401  (keeps the tests directory on the import path consistent)

pytestmark = pytest.mark.gpu

HEADS, ROT = 32, 128
DIM = HEADS * ROT


def _case(gpu, pkg, rng, pos, max_ctx):
    k = np.zeros((max_ctx, DIM), np.float16)
    v = np.zeros((max_ctx, DIM), np.float16)
    k[: pos + 1] = (rng.standard_normal((pos + 1, DIM)) * 0.7).astype(np.float16)
    v[: pos + 1] = (rng.standard_normal((pos + 1, DIM)) * 0.7).astype(np.float16)
    q = rng.standard_normal(DIM).astype(np.float32)
    return gpu.upload(k.view(np.uint16)), gpu.upload(v.view(np.uint16)), gpu.upload(q), gpu.upload(np.array([pos] * 4, np.uint32))


def test_static_scratch_variant_matches_caller_scratch_variant_twice_in_a_row(gpu, pkg):
    lib, h = gpu.lib, gpu.handle
    max_ctx = 2048
    assert lib.lv_attention_static_scratch_limit() == 1 << 20
    assert lib.lv_attention_scratch_bytes(HEADS, ROT, max_ctx, 1) <= lib.lv_attention_static_scratch_limit()
    table = gpu.alloc(max_ctx * ROT * 4)
    pkg.check(lib.lv_rope_table_build(h, table, max_ctx, ROT))
    scratch = gpu.zeros(lib.lv_attention_scratch_bytes(HEADS, ROT, max_ctx, 1))
    rng = np.random.default_rng(77)
    for pos in (700, 130):            # second call: fewer chunks than the first left behind in the shared buffer
        dk, dv, dq, dpos = _case(gpu, pkg, rng, pos, max_ctx)
        want_d, got_d = gpu.alloc(DIM * 4), gpu.alloc(DIM * 4)
        pkg.check(lib.lv_memset(h, got_d, 0xFF, DIM * 4))
        pkg.check(lib.lv_attention_fused(h, want_d, dq, dk, dv, dpos, table, scratch, HEADS, ROT, max_ctx, 1))
        pkg.check(lib.lv_attention_fused_static(h, got_d, dq, dk, dv, dpos, table, HEADS, ROT, max_ctx, 1))
        gpu.sync()
        want = gpu.download(want_d, np.float32, DIM).astype(np.float64)
        got = gpu.download(got_d, np.float32, DIM).astype(np.float64)
        assert np.all(np.isfinite(got))
        assert np.linalg.norm(got - want) <= 5e-6 * np.linalg.norm(want)
        assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
        for d in (dk, dv, dq, dpos, want_d, got_d):
            gpu.free(d)


def test_shapes_beyond_the_built_in_buffer_are_refused(gpu, pkg):
    lib, h = gpu.lib, gpu.handle
    d = gpu.alloc(4096)
    assert lib.lv_attention_scratch_bytes(HEADS, ROT, 2048, 6) <= lib.lv_attention_static_scratch_limit()
    assert lib.lv_attention_scratch_bytes(HEADS, ROT, 2048, 16) > lib.lv_attention_static_scratch_limit()
    rc = lib.lv_attention_fused_static(h, d, d, d, d, d, d, HEADS, ROT, 2048, 16)
    assert rc == pkg.LV_ERR_BAD_ARGUMENTS
    assert b"built-in buffer" in lib.lv_last_error_string()
    gpu.sync()

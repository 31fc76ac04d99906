"""lv_attention_fused_static: attention for callers that cannot allocate device
memory where they need it (inside a capture, behind a fixed memory budget, as a
plug-in that only receives its inputs and outputs).  Its scratch is built into
the library, so it must give the results of lv_attention_fused -- which takes
the scratch from the caller -- and of the CPU oracle's mhsa / softmax /
kqv_matching chain, call after call, whatever the shared buffer still holds
from earlier calls.  Collected last on purpose.
"""
import numpy as np
import pytest

import oracle_bind as ob

pytestmark = pytest.mark.gpu

HEADS, ROT = 32, 128
DIM = HEADS * ROT


def _case(gpu, rng, pos, max_ctx, batch):
    """Caches filled up to the last row the batch can see, one query per token of the batch."""
    n = pos + batch
    k = np.zeros((max_ctx, DIM), np.float16)
    v = np.zeros((max_ctx, DIM), np.float16)
    k[:n] = (rng.standard_normal((n, DIM)) * 0.7).astype(np.float16)
    v[:n] = (rng.standard_normal((n, DIM)) * 0.7).astype(np.float16)
    q = rng.standard_normal((batch, DIM)).astype(np.float32)
    return k.view(np.uint16), v.view(np.uint16), q


@pytest.mark.parametrize("batch,positions", [(1, (700, 130)), (6, (2042, 300))], ids=["batch1", "batch6-at-the-limit"])
def test_static_scratch_variant_matches_the_oracle_and_the_caller_scratch_variant_twice_in_a_row(gpu, pkg, batch, positions):
    lib, h = gpu.lib, gpu.handle
    max_ctx = 2048
    assert lib.lv_attention_static_scratch_limit() == 1 << 20
    assert lib.lv_attention_scratch_bytes(HEADS, ROT, max_ctx, batch) <= lib.lv_attention_static_scratch_limit()
    table = gpu.alloc(max_ctx * ROT * 4)
    pkg.check(lib.lv_rope_table_build(h, table, max_ctx, ROT))
    scratch = gpu.zeros(lib.lv_attention_scratch_bytes(HEADS, ROT, max_ctx, batch))
    rng = np.random.default_rng(77 + batch)
    for pos in positions:            # second call: fewer chunks than the first left behind in the shared buffer
        k, v, q = _case(gpu, rng, pos, max_ctx, batch)
        dk, dv, dq, dpos = gpu.upload(k), gpu.upload(v), gpu.upload(q), gpu.upload(np.array([pos] * 4, np.uint32))
        want_d, got_d = gpu.alloc(batch * DIM * 4), gpu.alloc(batch * DIM * 4)
        pkg.check(lib.lv_memset(h, got_d, 0xFF, batch * DIM * 4))
        pkg.check(lib.lv_attention_fused(h, want_d, dq, dk, dv, dpos, table, scratch, HEADS, ROT, max_ctx, batch))
        pkg.check(lib.lv_attention_fused_static(h, got_d, dq, dk, dv, dpos, table, HEADS, ROT, max_ctx, batch))
        gpu.sync()
        sibling = gpu.download(want_d, np.float32, batch * DIM).astype(np.float64).reshape(batch, DIM)
        got = gpu.download(got_d, np.float32, batch * DIM).astype(np.float64).reshape(batch, DIM)
        assert np.all(np.isfinite(got))
        for z in range(batch):
            # the same kernel with other scratch memory: equal up to the order in which chunks arrive
            assert np.linalg.norm(got[z] - sibling[z]) <= 5e-6 * np.linalg.norm(sibling[z])
            assert np.abs(got[z] - sibling[z]).max() <= 2e-5 * np.abs(sibling[z]).max()
            # the reference's three shaders restated on the CPU, tolerances of the fused-attention test at 2048 rows
            want = ob.attention(k, v, q[z], pos + z, max_ctx, HEADS, ROT).astype(np.float64)
            assert np.linalg.norm(got[z] - want) <= 1e-5 * np.linalg.norm(want)
            assert np.abs(got[z] - want).max() <= 2e-5 * np.abs(want).max()
        for d in (dk, dv, dq, dpos, want_d, got_d):
            gpu.free(d)
    gpu.free(scratch)
    gpu.free(table)


def test_shapes_beyond_the_built_in_buffer_are_refused(gpu, pkg):
    lib, h = gpu.lib, gpu.handle
    d = gpu.alloc(4096)
    assert lib.lv_attention_scratch_bytes(HEADS, ROT, 2048, 6) <= lib.lv_attention_static_scratch_limit()
    assert lib.lv_attention_scratch_bytes(HEADS, ROT, 2048, 16) > lib.lv_attention_static_scratch_limit()
    rc = lib.lv_attention_fused_static(h, d, d, d, d, d, d, HEADS, ROT, 2048, 16)
    assert rc == pkg.LV_ERR_BAD_ARGUMENTS
    assert b"built-in buffer" in lib.lv_last_error_string()
    gpu.sync()

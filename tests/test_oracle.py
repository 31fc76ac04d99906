"""Known-answer tests of the CPU oracle (CPU only).

The reference ships no golden vectors for this path, so the oracle is pinned by
hand-built cases whose answers follow from the reference's formulas, and by an
independent numpy restatement in float64.
"""
import numpy as np
import pytest

import oracle_bind as ob
import quant_np as qn


@pytest.fixture(scope="module")
def lib():
    return ob.load()


def test_half_to_float_all_bit_patterns(lib):
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([lib.orc_half_to_float(int(b)) for b in bits], np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_float_to_half_round_to_nearest_even(lib):
    rng = np.random.default_rng(1)
    vals = np.concatenate([
        rng.standard_normal(20000).astype(np.float32),
        (rng.standard_normal(5000) * 1e-6).astype(np.float32),          # subnormal halves
        (rng.standard_normal(5000) * 3e4).astype(np.float32),           # near overflow
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 1.5 * 2.0 ** -25,
                  1.00048828125, 1.0009765625 + 2.0 ** -12, np.inf, -np.inf], np.float32),
    ])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([lib.orc_float_to_half(float(v)) for v in vals], np.uint16)
    assert np.array_equal(got, want)


def _block_q4(scale_bits, nibbles32):
    b = np.zeros(18, np.uint8)
    b[0], b[1] = scale_bits & 0xFF, scale_bits >> 8
    n = np.asarray(nibbles32, np.uint8)
    b[2:] = n[:16] | (n[16:] << 4)
    return b


@pytest.mark.parametrize("scale_bits", [0x3C00, 0x2E66, 0x0001, 0x03FF, 0xBC00])   # 1.0, ~0.1, subnormals, -1.0
def test_dequant_q4_0_known_answers(scale_bits):
    # element j carries nibble j % 16 (+ offset), so every nibble value appears in both halves
    nib = np.array([(j * 7 + 3) % 16 for j in range(32)], np.uint8)
    got = ob.dequant(_block_q4(scale_bits, nib), qn.Q4_0, 32)
    d = np.array([scale_bits], np.uint16).view(np.float16).astype(np.float32)[0]
    want = (nib.astype(np.int32) - 8).astype(np.float32) * d
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_q4_0_v1_interleaved_order():
    # ggjt v1: f32 scale, byte j holds elements 2j (low) and 2j+1 (high)  (llava_buffer.cpp:350-359)
    blk = np.zeros(20, np.uint8)
    blk[:4] = np.array([0.5], np.float32).view(np.uint8)
    nib = np.arange(32, dtype=np.uint8) % 16
    blk[4:] = nib[0::2] | (nib[1::2] << 4)
    got = ob.dequant(blk, qn.Q4_0, 32, version=1)
    assert np.array_equal(got, (nib.astype(np.float32) - 8) * 0.5)


def test_dequant_q8_0_known_answers():
    blk = np.zeros(34, np.uint8)
    blk[:2] = np.array([0.25], np.float16).view(np.uint8)
    vals = np.array([-128, -127, -1, 0, 1, 127] + list(range(-13, 13)), np.int8)
    blk[2:] = vals.view(np.uint8)
    got = ob.dequant(blk, qn.Q8_0, 32)
    assert np.array_equal(got, vals.astype(np.float32) * 0.25)


@pytest.mark.parametrize("wtype", [qn.Q4_0, qn.Q8_0])
def test_dequant_matches_numpy_restatement(wtype):
    rng = np.random.default_rng(2)
    w = (rng.standard_normal(4096 * 8) * 0.02).astype(np.float32)
    raw = qn.quantize(w, wtype)
    got = ob.dequant(raw, wtype, w.size)
    want = qn.dequantize_np(raw, wtype)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    step = np.abs(w).reshape(-1, 32).max(axis=1) / (8 if wtype == qn.Q4_0 else 127)
    # quantisation error is bounded by (slightly more than) half a step, one full step at the clamped end of q4_0
    assert np.all(np.abs(got - w).reshape(-1, 32) <= step[:, None] * 1.01 + 1e-9)


@pytest.mark.parametrize("dim", [4096, 5120])
def test_norm_against_float64(dim):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(dim) * 2 + 0.3).astype(np.float32)
    w = (1 + 0.01 * rng.standard_normal(dim)).astype(np.float32)
    got = ob.norm(x, w)
    x64 = x.astype(np.float64)
    want = x64 * w * (1.0 / np.sqrt(np.mean((x64 - x64.mean()) ** 2)))
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=0)


def test_norm_constant_plus_ramp_has_no_epsilon_and_keeps_the_mean_in_the_numerator():
    dim = 4096
    x = (5.0 + np.arange(dim) / dim).astype(np.float32)
    w = np.ones(dim, np.float32)
    got = ob.norm(x, w)
    var = np.mean((x.astype(np.float64) - x.astype(np.float64).mean()) ** 2)      # ~1/12
    np.testing.assert_allclose(got, x / np.sqrt(var), rtol=1e-4)
    assert got.mean() > 15            # not centred: a textbook layer norm would give mean 0


@pytest.mark.parametrize("wtype,rows,cols,workers", [(qn.Q4_0, 64, 4096, 128), (qn.Q4_0, 32, 11008, 128),
                                                      (qn.Q8_0, 64, 4096, 128), (qn.Q4_0, 32, 5120, 32),
                                                      (qn.Q8_0, 16, 13824, 128)])
def test_gemv_against_float64(wtype, rows, cols, workers):
    rng = np.random.default_rng(4)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    raw = qn.quantize(w, wtype)
    got = ob.gemv(raw, wtype, x, rows, cols, workers)
    want = qn.dequantize_np(raw, wtype).reshape(rows, cols).astype(np.float64) @ x.astype(np.float64)
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-5 * np.abs(want).max())
    base = rng.standard_normal(rows).astype(np.float32)
    got_add = ob.gemv(raw, wtype, x, rows, cols, workers, out=base)
    np.testing.assert_array_equal(got_add, base + got)


def test_gemv_silu_formula():
    rng = np.random.default_rng(5)
    rows, cols = 64, 4096
    w3 = qn.quantize_q4_0((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    w1 = qn.quantize_q4_0((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    x = rng.standard_normal(cols).astype(np.float32)
    r1 = ob.gemv(w3, qn.Q4_0, x, rows, cols, 128)
    r2 = ob.gemv(w1, qn.Q4_0, x, rows, cols, 128)
    got = ob.gemv_silu(w3, w1, qn.Q4_0, x, rows, cols, 128)
    want = r1 * r2 / (np.exp(-r2.astype(np.float32)) + np.float32(1))
    np.testing.assert_allclose(got, want, rtol=1e-6)


HEADS, ROT = 32, 128
DIM = HEADS * ROT


def _rand_cache(rng, n, backlog):
    c = np.zeros((backlog, DIM), np.float16)
    c[:n] = (rng.standard_normal((n, DIM)) * 0.5).astype(np.float16)
    return c.view(np.uint16)


def test_attention_first_token_returns_the_cached_value(lib):
    rng = np.random.default_rng(6)
    k, v = _rand_cache(rng, 1, 128), _rand_cache(rng, 1, 128)
    q = rng.standard_normal(DIM).astype(np.float32)
    out = ob.attention(k, v, q, 0, 128, HEADS, ROT)
    np.testing.assert_array_equal(out, v[0].view(np.float16).astype(np.float32))


def test_rope_distance_zero_is_the_identity():
    rng = np.random.default_rng(7)
    pos = 5
    k = _rand_cache(rng, pos + 1, 128)
    q = rng.standard_normal(DIM).astype(np.float32)
    s = ob.mhsa(k, q, pos, HEADS, ROT)
    kf = k.view(np.float16).astype(np.float64)[pos].reshape(HEADS, ROT)
    want = (kf * q.astype(np.float64).reshape(HEADS, ROT)).sum(axis=1)
    np.testing.assert_allclose(s[pos], want, rtol=0, atol=1e-4)


def test_mhsa_equals_textbook_rope_in_float64():
    rng = np.random.default_rng(8)
    pos = 37
    k = _rand_cache(rng, pos + 1, 128)
    q = rng.standard_normal(DIM).astype(np.float32)
    s = ob.mhsa(k, q, pos, HEADS, ROT)
    theta = 10000.0 ** (-np.arange(ROT // 2) / (ROT // 2))
    def rot(vec, p):        # textbook: rotate adjacent pairs by +p*theta
        v = vec.reshape(-1, HEADS, ROT // 2, 2).astype(np.float64)
        a = p * theta
        return np.stack([v[..., 0] * np.cos(a) - v[..., 1] * np.sin(a), v[..., 0] * np.sin(a) + v[..., 1] * np.cos(a)], -1)
    kf = k.view(np.float16).astype(np.float64)
    qr = rot(q, pos)[0]
    want = np.stack([(rot(kf[p], p)[0] * qr).sum(axis=(1, 2)) for p in range(pos + 1)])
    np.testing.assert_allclose(s, want, rtol=0, atol=2e-4)


@pytest.mark.parametrize("pos,backlog", [(0, 128), (17, 128), (127, 128), (200, 256)])
def test_softmax_rows_sum_to_one_and_masked_slots_are_zero(pos, backlog):
    rng = np.random.default_rng(9)
    scores = (rng.standard_normal((pos + 1, HEADS)) * 10).astype(np.float32)
    pr = ob.softmax(scores, pos, backlog, HEADS, ROT)
    np.testing.assert_allclose(pr.sum(axis=0), 1.0, rtol=1e-5)
    assert np.all(pr[pos + 1:] == 0)
    e = np.exp(scores.astype(np.float64) / np.sqrt(ROT))
    np.testing.assert_allclose(pr[: pos + 1], e / e.sum(axis=0), rtol=1e-5)


def test_kqv_against_float64():
    rng = np.random.default_rng(10)
    pos, backlog = 50, 128
    v = _rand_cache(rng, pos + 1, backlog)
    pr = np.zeros((backlog, HEADS), np.float32)
    pr[: pos + 1] = rng.random((pos + 1, HEADS)).astype(np.float32)
    out = ob.kqv(v, pr, backlog, HEADS, ROT)
    want = np.einsum("pd,pd->d", v.view(np.float16).astype(np.float64), np.repeat(pr.astype(np.float64), ROT, axis=1))
    np.testing.assert_allclose(out, want, rtol=0, atol=1e-4)


def test_argmax_first_maximum_and_nan_rules(lib):
    v = np.array([1, 5, 3, 5, 2], np.float32)
    assert lib.orc_argmax(ob.ptr(v), v.size) == 1
    v = np.array([np.nan, 5, 3], np.float32)
    assert lib.orc_argmax(ob.ptr(v), v.size) == 0        # nothing compares greater than NaN
    v = np.array([1, np.nan, 3], np.float32)
    assert lib.orc_argmax(ob.ptr(v), v.size) == 2


def test_sampler_candidates_penalise_only_token_13(lib):
    rng = np.random.default_rng(11)
    n = 1000
    logits = rng.standard_normal(n).astype(np.float32) * 3
    logits[13] = 4.0
    toks = np.array([13, 7, 13, 9], np.uint32)
    probs, ids, kept = np.empty(n, np.float32), np.empty(n, np.uint32), C_float()
    k = lib.orc_sampler_candidates(ob.ptr(logits), n, ob.ptr(toks), toks.size, 10.0, ob.ptr(probs), ob.ptr(ids), kept)
    l2 = logits.astype(np.float64).copy()
    l2[13] = l2[13] / 1.1 - 0.1 * 2
    p = np.exp(l2 / 0.8)
    p /= p.sum()
    keep = np.nonzero(p >= 0.5 ** 10)[0]
    assert k == keep.size and np.array_equal(ids[:k], keep)
    np.testing.assert_allclose(probs[:k], p[keep], rtol=2e-4)
    np.testing.assert_allclose(kept.value, p[keep].sum(), rtol=2e-4)
    mu = lib.orc_sampler_mu_update(10.0, float(probs[0]), kept.value)
    np.testing.assert_allclose(mu, 10.0 + 0.1 * (5.0 + np.log2(probs[0] / kept.value)), rtol=1e-6)


def C_float():
    import ctypes
    return ctypes.c_float()

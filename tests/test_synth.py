"""Synthetic ggjt writer: value generator, quantiser, determinism.  CPU only."""
import ctypes as C
import os

import numpy as np

import oracle_bind as ob
import quant_np as qn


def test_normal_generator_is_deterministic_and_standard(pkg):
    lib = pkg.load_host()
    a = np.array([lib.llava_synth_normal(1234, 3, i) for i in range(40000)], np.float64)
    b = np.array([lib.llava_synth_normal(1234, 3, i) for i in range(2000)], np.float64)
    assert np.array_equal(a[:2000], b)
    assert abs(a.mean()) < 0.02 and abs(a.std() - 1) < 0.02
    assert abs(np.mean(a ** 3)) < 0.05 and abs(np.mean(a ** 4) - 3) < 0.15
    other = np.array([lib.llava_synth_normal(1234, 4, i) for i in range(2000)], np.float64)
    assert abs(np.corrcoef(a[:2000], other)[0, 1]) < 0.08
    assert abs(np.corrcoef(a[0::2][:10000], a[1::2][:10000])[0, 1]) < 0.03      # the two halves of a pair


def test_quantiser_matches_the_numpy_restatement(pkg):
    lib = pkg.load_host()
    rng = np.random.default_rng(5)
    w = (rng.standard_normal(32 * 500) * 0.02).astype(np.float32)
    w[:32] = 0                                     # an all-zero block: scale 0, values at the offset
    w[32:64] = np.float32(0.02)                    # constant block
    for wtype, bb in ((qn.Q4_0, 18), (qn.Q8_0, 34)):
        out = np.empty(w.size // 32 * bb, np.uint8)
        lib.llava_synth_quantize(w.ctypes.data_as(C.c_void_p), w.size, wtype, out.ctypes.data_as(C.c_void_p))
        assert np.array_equal(out, qn.quantize(w, wtype))
        deq = ob.dequant(out, wtype, w.size)
        step = np.abs(w).reshape(-1, 32).max(axis=1) / (8 if wtype == qn.Q4_0 else 127)
        assert np.all(np.abs(deq - w).reshape(-1, 32) <= step[:, None] * 1.01 + 1e-9)
        host = np.empty(w.size, np.float32)
        assert lib.llava_dequantize(out.ctypes.data_as(C.c_void_p), wtype, 3, host.ctypes.data_as(C.c_void_p), w.size) == 1
        assert np.array_equal(host.view(np.uint32), deq.view(np.uint32))    # host dequant == oracle, bit for bit


def test_file_is_reproducible_and_weights_follow_the_generator(pkg, tmp_path):
    lib = pkg.load_host()
    a, b = str(tmp_path / "a.bin"), str(tmp_path / "b.bin")
    for p, threads in ((a, 1), (b, 5)):
        assert lib.llava_synth_write(os.fsencode(p), 256, 2, 2, 512, 1000, qn.Q8_0, 77, threads) == 1
    ra, rb = open(a, "rb").read(), open(b, "rb").read()
    assert ra == rb                                       # independent of the thread count
    assert len(ra) == lib.llava_synth_file_size(256, 2, 2, 512, 1000, qn.Q8_0)
    m = pkg.ModelFile(a)
    tensors = m.tensors()
    # tensor 3 = layers.0.attention.wq: rows of N(0, 0.02) values quantised to q8_0
    name, t, off, rows, cols, size = tensors[3]
    assert name == "layers.0.attention.wq.weight" and t == qn.Q8_0 and (rows, cols) == (256, 256)
    want = np.array([0.02 * lib.llava_synth_normal(77, 3, i) for i in range(2 * cols)], np.float32)
    got = np.frombuffer(ra, np.uint8, 2 * qn.row_bytes(qn.Q8_0, cols), off)
    assert np.array_equal(got, qn.quantize_q8_0(want))
    name, t, off, rows, cols, size = tensors[1]
    assert name == "norm.weight" and t == 0 and cols == 1
    norm = np.frombuffer(ra, np.float32, rows, off)
    assert abs(norm.mean() - 1) < 0.005 and 0.005 < norm.std() < 0.02
    m.close()
    assert lib.llava_synth_write(os.fsencode(a), 250, 2, 2, 512, 1000, qn.Q8_0, 77, 1) == 0      # dim % 32
    assert lib.llava_synth_write(os.fsencode(a), 256, 2, 2, 512, 1000, 3, 77, 1) == 0            # q4_1

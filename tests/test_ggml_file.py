"""Loader and tokenizer against the golden answers recorded from the reference's
own ggml_file.cpp (tests/golden/make_golden.py), and the oracle's parser against
the same answers.  CPU only."""
import ctypes as C
import hashlib
import json
import os

import pytest

import oracle_bind as ob
from conftest import ROOT

GOLDEN = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def small_model(pkg, tmp_path_factory):
    cfg = json.load(open(os.path.join(GOLDEN, "tensor_table.json")))["config"]
    path = str(tmp_path_factory.mktemp("model") / "small.bin")
    ok = pkg.load_host().llava_synth_write(os.fsencode(path), cfg["dim"], cfg["n_heads"], cfg["n_layers"], cfg["ff_size"],
                                           cfg["vocab"], cfg["wtype"], cfg["seed"], 0)
    assert ok
    return path


def test_synthetic_file_has_the_layout_the_fixtures_were_made_from(small_model):
    g = json.load(open(os.path.join(GOLDEN, "tensor_table.json")))
    raw = open(small_model, "rb").read()
    assert len(raw) == g["file_size"]
    first = min(t[2] for t in g["tensors"])
    assert hashlib.sha256(raw[:first - 64]).hexdigest() == g["sha256_before_first_tensor"]


def test_tensor_table_matches_reference_parser(pkg, small_model):
    g = json.load(open(os.path.join(GOLDEN, "tensor_table.json")))
    m = pkg.ModelFile(small_model)
    hdr = [m.magic, m.file_version, m.vocab_size, m.dim, m.multiple_of, m.n_heads, m.n_layers, m.rot, m.ftype, m.ff_size]
    assert hdr == g["header"]
    assert [list(t) for t in m.tensors()] == g["tensors"]
    # name lookup falls back to name + ".weight" (ggml_file.cpp:337-344)
    off = C.c_uint64()
    assert m.lib.ggml_file_find(m.handle, b"layers.0.attention.wq", C.byref(off)) == 1
    assert off.value == dict((t[0], t[2]) for t in g["tensors"])["layers.0.attention.wq.weight"]
    assert m.lib.ggml_file_find(m.handle, b"layers.0.attention.nope", C.byref(off)) == 0
    m.close()


def test_oracle_parser_matches_reference_parser(small_model):
    g = json.load(open(os.path.join(GOLDEN, "tensor_table.json")))
    lib = ob.load()
    h = lib.orc_model_open(os.fsencode(small_model))
    assert h
    info = ob.ModelInfo()
    lib.orc_model_get_info(h, C.byref(info))
    assert [info.file_version, info.vocab_size, info.dim, info.multiple_of, info.n_heads, info.n_layers, info.rot,
            info.ftype, info.ff_size] == g["header"][1:]
    name = C.create_string_buffer(256)
    t, s1, s2, off, size = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint64(), C.c_uint64()
    rows = []
    for i in range(info.n_tensors):
        assert lib.orc_model_tensor(h, i, name, 256, C.byref(t), C.byref(off), C.byref(s1), C.byref(s2), C.byref(size)) == 0
        rows.append([name.value.decode(), t.value, off.value, s1.value, s2.value, size.value])
    assert rows == g["tensors"]
    lib.orc_model_close(h)


def test_tokenizer_matches_reference_on_every_golden_case(pkg, small_model):
    cases = json.load(open(os.path.join(GOLDEN, "tokenizer_cases.json")))["cases"]
    assert len(cases) > 100
    m = pkg.ModelFile(small_model)
    for c in cases:
        text = bytes.fromhex(c["text_utf8_hex"])
        toks = m.tokenize(text, bos=bool(c["bos"]))
        assert toks == c["tokens"], text
        assert m.tokens_to_text(toks) == bytes.fromhex(c["detok_hex"])
    m.close()


def test_tokenizer_byte_fallback_and_bos(pkg, small_model):
    m = pkg.ModelFile(small_model)
    assert m.tokenize("", bos=True) == []                         # empty text: nothing, not even BOS
    assert m.tokenize(b"\xff", bos=True) == [1, 255 + 3]          # ggml_file.cpp:255-257, :330
    assert m.token(3)[0] == b"\x00" and m.token(258)[0] == b"\xff"
    assert m.token(0)[0] == b"<unk>" and m.token(1)[0] == b"<s>" and m.token(2)[0] == b"</s>"
    m.close()


def test_live_comparison_with_the_reference_library_when_present(pkg, small_model):
    if not os.path.exists(ob.REF_LIB):
        pytest.skip("oracle/_ref not built here")
    import random
    ref = C.CDLL(ob.REF_LIB)
    ref.ref_open.restype = C.c_void_p
    ref.ref_open.argtypes = [C.c_char_p]
    ref.ref_tokenize.restype = C.c_uint32
    ref.ref_tokenize.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t, C.c_int, C.c_void_p, C.c_uint32]
    h = ref.ref_open(os.fsencode(small_model))
    m = pkg.ModelFile(small_model)
    rng = random.Random(7)
    for _ in range(300):
        n = rng.choice([1, 4, 9, 30, 100])
        text = "".join(rng.choice("abcdefghijklmnopqrstuvwxyz  é") for _ in range(n)).encode()
        buf = (C.c_uint32 * (len(text) + 4))()
        k = ref.ref_tokenize(h, text, len(text), 1, buf, len(text) + 4)
        assert m.tokenize(text, bos=True) == list(buf[:k])
    m.close()


@pytest.mark.parametrize("damage", ["magic", "truncate", "short_header", "bad_type"])
def test_malformed_files_are_rejected_without_aborting(pkg, small_model, tmp_path, damage):
    raw = bytearray(open(small_model, "rb").read())
    if damage == "magic":
        raw[0] ^= 0xFF
    elif damage == "truncate":
        raw = raw[: len(raw) - 1000]
    elif damage == "short_header":
        raw = raw[:20]
    else:
        g = json.load(open(os.path.join(GOLDEN, "tensor_table.json")))
        # the type word of the second tensor record sits 8 bytes into the record; find it by name
        name = b"norm.weight"
        at = bytes(raw).index(name) - 8
        raw[at:at + 4] = (6).to_bytes(4, "little")          # q5_0: not accepted (ggml_file.cpp:104)
    p = tmp_path / "bad.bin"
    p.write_bytes(bytes(raw))
    assert pkg.load_host().ggml_file_open(os.fsencode(str(p))) is None
    assert ob.load().orc_model_open(os.fsencode(str(p))) is None

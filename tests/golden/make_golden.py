"""Generates tests/golden/*.json from the reference's own ggml_file.cpp.

Run in a checkout where the reference sources are available:

    make -C oracle ref REF=<reference checkout> && python llama-vulkan_b200/build.py && python tests/golden/make_golden.py

The model file is produced by this repository's synthetic writer (small
geometry, full 32000-entry vocabulary); the recorded answers -- tensor table
and tokenisations -- come from the reference's unmodified parser and tokenizer
(oracle/_ref/libref_ggml.so).  The tests re-create the same file and compare
this repository's ggml_file and the oracle's parser against these answers.
"""
import ctypes as C
import hashlib
import json
import os
import random
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))

from conftest import load_pkg  # noqa: E402

SMALL = dict(dim=256, n_heads=2, n_layers=1, ff_size=512, vocab=32000, wtype=2, seed=1234)


def write_small_model(path):
    pkg = load_pkg()
    lib = pkg.load_host()
    ok = lib.llava_synth_write(os.fsencode(path), SMALL["dim"], SMALL["n_heads"], SMALL["n_layers"], SMALL["ff_size"],
                               SMALL["vocab"], SMALL["wtype"], SMALL["seed"], 0)
    assert ok
    return path


def texts():
    rng = random.Random(4321)
    alphabet = "abcdefghijklmnopqrstuvwxyz "
    out = ["", "a", "hello world", "The ten best monuments to see in Paris are", "  leading and trailing  ",
           "café naïve 日本語 \U0001f600", "UPPER lower 12345 !?", "\n\ttabs\nnewlines\n", "zzzzzzzzzzzzzzzz",
           "a b c d e f g h i j k l m n o p q r s t u v w x y z"]
    for n in (2, 3, 5, 8, 13, 40, 120, 400):
        for _ in range(6):
            out.append("".join(rng.choice(alphabet) for _ in range(n)))
    return out


def main():
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libref_ggml.so")
    ref = C.CDLL(ref_path)
    ref.ref_open.restype = C.c_void_p
    ref.ref_open.argtypes = [C.c_char_p]
    ref.ref_tokenize.restype = C.c_uint32
    ref.ref_tokenize.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t, C.c_int, C.c_void_p, C.c_uint32]
    ref.ref_n_tensors.restype = C.c_uint32
    ref.ref_n_tensors.argtypes = [C.c_void_p]
    ref.ref_header.argtypes = [C.c_void_p, C.c_void_p]
    ref.ref_tensor.argtypes = [C.c_void_p, C.c_uint32, C.c_char_p, C.c_size_t] + [C.c_void_p] * 5
    ref.ref_tokens_to_text.restype = C.c_uint32
    ref.ref_tokens_to_text.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_char_p, C.c_uint32]

    model = write_small_model("/tmp/lv_golden_small.bin")
    raw = open(model, "rb").read()
    h = ref.ref_open(os.fsencode(model))
    assert h

    hdr = (C.c_uint32 * 10)()
    ref.ref_header(h, hdr)
    table = []
    name = C.create_string_buffer(256)
    t, s1, s2, off, size = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint64(), C.c_uint64()
    for i in range(ref.ref_n_tensors(h)):
        ref.ref_tensor(h, i, name, 256, C.byref(t), C.byref(off), C.byref(s1), C.byref(s2), C.byref(size))
        table.append([name.value.decode(), t.value, off.value, s1.value, s2.value, size.value])
    first_tensor = min(r[2] for r in table)
    golden_table = {"config": SMALL, "header": list(hdr), "tensors": table, "file_size": len(raw),
                    "sha256_before_first_tensor": hashlib.sha256(raw[:first_tensor - 64]).hexdigest()}
    json.dump(golden_table, open(os.path.join(HERE, "tensor_table.json"), "w"), indent=1)

    cases = []
    for text in texts():
        data = text.encode("utf-8")
        for bos in (1, 0):
            buf = (C.c_uint32 * (len(data) + 4))()
            n = ref.ref_tokenize(h, data, len(data), bos, buf, len(data) + 4)
            toks = list(buf[:n])
            out = C.create_string_buffer(len(data) + 64)
            body = [x for x in toks]
            m = ref.ref_tokens_to_text(h, (C.c_uint32 * max(len(body), 1))(*body), len(body), out, len(data) + 64)
            cases.append({"text_utf8_hex": data.hex(), "bos": bos, "tokens": toks, "detok_hex": out.raw[:m].hex()})
    json.dump({"config": SMALL, "cases": cases}, open(os.path.join(HERE, "tokenizer_cases.json"), "w"), separators=(",", ":"))
    print("wrote", len(table), "tensors and", len(cases), "tokenizer cases")


if __name__ == "__main__":
    main()

"""A ggjt version 1 model on the device path: q4_0 blocks with f32 scales and interleaved nibbles, embeddings stored
as f32 (llava_buffer.cpp:66-71,193-224,350-359 of the reference; the shader variants without the _fp16 suffix).
Two layers of the 7B geometry, 16 prompt tokens + 16 greedy tokens against the CPU oracle, which reads the same
file: logits within max-abs 1e-2 / relative L2 1e-3 at every step, tokens identical; the prompt also in batches.
"""
import numpy as np
import pytest

import quant_np as qn
from test_e2e_gpu import OracleSession, assert_logits_close, note_parity, prompt_tokens

pytestmark = pytest.mark.gpu

N_DECODE = 16


@pytest.fixture(scope="module")
def run_v1(pkg, tmp_path_factory):
    path = str(tmp_path_factory.mktemp("e2e_v1") / "tiny_v1.bin")
    pkg.write_synthetic_model(path, "7b", n_layers=2, wtype=qn.Q4_0, file_version=1, f32_embeddings=True)
    mf = pkg.ModelFile(path)
    assert mf.file_version == 1
    assert [t for t in mf.tensors() if t[0] == "tok_embeddings.weight"][0][1] == 0        # f32
    mf.close()
    orc = OracleSession(path)
    toks = prompt_tokens()
    for t in toks:
        orc.push(t)
    logits, greedy = [], []
    for _ in range(N_DECODE):
        logits.append(orc.eval())
        greedy.append(orc.argmax())
        orc.push(greedy[-1])
    ctx = pkg.HostContext(path, 0)
    yield dict(orc=orc, prompt=toks, logits=logits, greedy=greedy, ctx=ctx, vocab=orc.info.vocab_size)
    ctx.close()
    orc.close()


def test_version_1_model_decodes_like_the_oracle(run_v1):
    s = run_v1["ctx"].session()
    s.set_deterministic(True)
    for t in run_v1["prompt"]:
        assert s.push_token(t)
    worst = (0.0, 0.0)
    for step in range(N_DECODE):
        tok = s.predict_next_token()
        m, r = assert_logits_close(s.logits(run_v1["vocab"]), run_v1["logits"][step])
        worst = (max(worst[0], m), max(worst[1], r))
        assert tok == run_v1["greedy"][step], f"step {step}"
        assert s.push_token(tok)
    note_parity(f"ggjt v1 (f32 scales, f32 embeddings), 2 layers: 16 greedy tokens identical; worst logits max-abs {worst[0]:.3e} rel-L2 {worst[1]:.3e}")
    s.close()


def test_version_1_prompt_in_batches_and_device_resident_loop(run_v1):
    s = run_v1["ctx"].session()
    s.set_deterministic(True)
    assert s.set_max_batch(16)           # version 1 blocks have no tensor-core path: the batch runs as one GEMV launch with 16 rows of inputs
    for t in run_v1["prompt"]:
        assert s.push_token(t)
    first = s.predict_next_token()
    assert_logits_close(s.logits(run_v1["vocab"]), run_v1["logits"][0])
    assert first == run_v1["greedy"][0]
    assert s.push_token(first)
    assert [first] + s.generate_greedy_on_device(N_DECODE - 1) == run_v1["greedy"]
    s.close()

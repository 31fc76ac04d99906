"""The vulkan_llama command-line tool (llava_context::run, the reference's generation loop
llava_context.cpp:336-373) on the two-layer synthetic model: what it prints must be the text of
the greedy tokens the CPU oracle produces from the same prompt.
"""
import os
import subprocess

import numpy as np
import pytest

import quant_np as qn
from test_e2e_gpu import OracleSession, prompt_tokens

pytestmark = pytest.mark.gpu

N_PREDICT = 8


@pytest.fixture(scope="module")
def cli(pkg, tmp_path_factory):
    d = tmp_path_factory.mktemp("cli")
    model = str(d / "tiny_q4_0.bin")
    exe = os.path.join(os.path.dirname(pkg.__file__), "vulkan_llama")
    assert os.path.exists(exe), "vulkan_llama was not built"
    # the tool writes its own synthetic file: same seeded generator as the library call
    subprocess.run([exe, "-m", model, "--write-synthetic", "tiny"], check=True, timeout=600)
    ids = prompt_tokens(12)
    tokens_file = str(d / "prompt.txt")
    open(tokens_file, "w").write(" ".join(str(t) for t in ids))
    orc = OracleSession(model)
    for t in ids:
        orc.push(t)
    greedy = []
    for _ in range(N_PREDICT):
        orc.eval()
        greedy.append(int(orc.argmax()))
        orc.push(greedy[-1])
    orc.close()
    mf = pkg.ModelFile(model)
    text = b"".join(mf.token(t)[0] for t in greedy)
    mf.close()
    return dict(exe=exe, model=model, tokens=tokens_file, greedy=greedy, text=text)


@pytest.mark.parametrize("extra", [[], ["--on-device"]], ids=["host-in-the-loop", "device-resident"])
def test_cli_prints_the_oracles_greedy_tokens(cli, extra):
    out = subprocess.run([cli["exe"], "-m", cli["model"], "--greedy", "--tokens", cli["tokens"], "--n-predict", str(N_PREDICT),
                          "--ignore-eos"] + extra, check=True, timeout=600, stdout=subprocess.PIPE).stdout
    assert out == cli["text"] + b"\n", (out, cli["text"])


def test_cli_print_header_and_missing_model(cli):
    out = subprocess.run([cli["exe"], "-m", cli["model"], "--print_header"], check=True, timeout=120, stdout=subprocess.PIPE).stdout
    assert b"4096" in out and b"32000" in out
    assert subprocess.run([cli["exe"], "-m", cli["model"] + ".missing", "--greedy", "--n-predict", "1"], timeout=120,
                          stdout=subprocess.PIPE, stderr=subprocess.PIPE).returncode != 0

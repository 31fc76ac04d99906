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


@pytest.mark.parametrize("extra", [[], ["--on-device"], ["--prompt-batch", "16", "--exact-prompt"]],
                         ids=["host-in-the-loop", "device-resident", "prompt-as-one-batch"])
def test_cli_prints_the_oracles_greedy_tokens(cli, extra):
    out = subprocess.run([cli["exe"], "-m", cli["model"], "--greedy", "--tokens", cli["tokens"], "--n-predict", str(N_PREDICT),
                          "--ignore-eos"] + extra, check=True, timeout=600, stdout=subprocess.PIPE).stdout
    assert out == cli["text"] + b"\n", (out, cli["text"])


def test_cli_print_header_and_missing_model(cli):
    out = subprocess.run([cli["exe"], "-m", cli["model"], "--print_header"], check=True, timeout=120, stdout=subprocess.PIPE).stdout
    assert b"4096" in out and b"32000" in out
    assert subprocess.run([cli["exe"], "-m", cli["model"] + ".missing", "--greedy", "--n-predict", "1"], timeout=120,
                          stdout=subprocess.PIPE, stderr=subprocess.PIPE).returncode != 0


def test_cli_server_mode_generates_over_tcp(cli, pkg):
    """`--server`: the process listens, a client makes a session, feeds the prompt and ticks; a line on standard
    input ends the server (reference llava_context.cpp:246-249, server/server.cpp:178-184)."""
    import struct
    p = subprocess.Popen([cli["exe"], "-m", cli["model"], "--server", "--port", "0", "--bind", "127.0.0.1", "--greedy"],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE)
    try:
        port = None
        for _ in range(50):
            line = p.stdout.readline()
            assert line, "the server ended before it listened"
            if b"Started server on" in line:
                port = int(line.rsplit(b":", 1)[1])
                break
        assert port
        c = pkg.Client(port, timeout=120.0)
        op, sid = c.call(c.NEW_SESSION)
        assert op == c.SESSION_CREATED
        for t in prompt_tokens(12):
            assert c.call(c.ADD_TOKEN, sid + struct.pack("<I", t)) == (c.ACK, struct.pack("<I", 0))
        for i in range(3):
            assert c.call(c.TICK, sid) == (c.NEW_TOKEN, sid + struct.pack("<II", cli["greedy"][i], 12 + i))
        c.close()
        p.stdin.write(b"\n")
        p.stdin.flush()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()


def _device_count(pkg):
    import ctypes as C
    n = C.c_int(0)
    pkg.load_kernels().lv_device_count(C.byref(n))
    return n.value


@pytest.mark.parametrize("extra", [[], ["--on-device"]], ids=["host-in-the-loop", "device-resident"])
def test_cli_tensor_parallel_over_two_gpus(cli, pkg, extra):
    """`--gpus 2`: the tool forks one process per GPU (row / column shards, exchange fused into the GEMVs); rank 0 prints
    the same greedy tokens as the oracle."""
    if _device_count(pkg) < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.pop("NCCL_DEBUG", None)
    out = subprocess.run([cli["exe"], "-m", cli["model"], "--gpus", "2", "--greedy", "--tokens", cli["tokens"], "--n-predict", str(N_PREDICT),
                          "--ignore-eos"] + extra, check=True, timeout=600, stdout=subprocess.PIPE, env=env).stdout
    lines = [l for l in out.split(b"\n") if not l.startswith(b"NCCL version")]      # the library's own banner, if it prints one
    assert b"\n".join(lines) == cli["text"] + b"\n", (out, cli["text"])

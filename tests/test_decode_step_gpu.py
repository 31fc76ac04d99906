"""lv_decode_step: one decoded token as ONE launch (persistent kernel, weight rings that run across operations,
flag-in-data hand-over between operations).  Sessions use it when LV_DECODE_STEP=1; the environment is read when a
session is created, so the comparison runs in a child process: 12 prompt tokens + 12 greedy tokens of the two-layer
7B- and 13B-geometry models against the CPU oracle, logits within the end-to-end tolerance at every step, and one
launch per token.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import quant_np as qn
from test_e2e_gpu import LOGIT_MAX_ABS, LOGIT_REL_L2, OracleSession, prompt_tokens

pytestmark = pytest.mark.gpu

CHILD = r'''
import json, os, sys
import numpy as np
sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
from conftest import load_pkg
pkg = load_pkg()
path, prompt, n = sys.argv[2], json.loads(sys.argv[3]), int(sys.argv[4])
ctx = pkg.HostContext(path, 0)
s = ctx.session()
s.set_deterministic(True)
for t in prompt:
    assert s.push_token(t)
out = {"tokens": [], "launches": [], "logits": []}
for i in range(n):
    tok = s.predict_next_token()
    out["tokens"].append(tok)
    out["launches"].append(s.step_kernel_launches())
    np.save(f"{path}.logits{i}.npy", s.logits(32000))
    assert s.push_token(tok)
rest = s.generate_greedy_on_device(4)
out["device_loop"] = rest
s.close(); ctx.close()
print("RESULT " + json.dumps(out))
'''


@pytest.mark.parametrize("geometry,wtype", [("7b", qn.Q4_0), ("13b", qn.Q4_0), ("7b", qn.Q8_0)], ids=["7b-q4_0", "13b-q4_0", "7b-q8_0"])
def test_one_launch_step_matches_the_oracle(pkg, tmp_path, geometry, wtype):
    path = str(tmp_path / f"tiny_{geometry}_{wtype}.bin")
    pkg.write_synthetic_model(path, geometry, n_layers=2, wtype=wtype)
    prompt, n = prompt_tokens(12), 12
    orc = OracleSession(path)
    for t in prompt:
        orc.push(t)
    want_logits, want_tokens = [], []
    for _ in range(n + 4):
        want_logits.append(orc.eval())
        want_tokens.append(int(orc.argmax()))
        orc.push(want_tokens[-1])
    orc.close()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, LV_DECODE_STEP="1")
    res = subprocess.run([sys.executable, "-c", CHILD, root, path, json.dumps(prompt), str(n)], env=env, stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    # the first evaluation ingests the prompt (per-operation kernels, one recorded step per token batch); every later
    # token is a single launch of the persistent kernel
    assert out["launches"][1:] == [1] * (n - 1), out["launches"]
    assert out["tokens"] == want_tokens[:n]
    assert out["device_loop"] == want_tokens[n:n + 4]
    for i in range(n):
        got = np.load(f"{path}.logits{i}.npy").astype(np.float64)
        want = want_logits[i].astype(np.float64)
        assert np.abs(got - want).max() <= LOGIT_MAX_ABS
        assert np.linalg.norm(got - want) / np.linalg.norm(want) <= LOGIT_REL_L2

"""lv_sample_mirostat: the reference's sampler (llava_session.cpp:154-194) on the device, against the CPU
restatement (orc_sampler_candidates / orc_sampler_mu_update): same candidate set, same kept mass, and -- given the
same uniform variate -- the same token as the inverse-CDF draw over those candidates on the host, and the same mu.
"""
import ctypes as C

import numpy as np
import pytest

import oracle_bind as ob

pytestmark = pytest.mark.gpu

VOCAB = 32000
NO_TOKEN = 0xFFFFFFFF


def _oracle(logits, tokens, mu):
    lib = ob.load()
    probs, ids, kept = np.empty(VOCAB, np.float32), np.empty(VOCAB, np.uint32), C.c_float()
    toks = np.asarray(tokens, np.uint32)
    k = lib.orc_sampler_candidates(ob.ptr(logits), VOCAB, ob.ptr(toks), toks.size, C.c_float(mu), ob.ptr(probs), ob.ptr(ids), C.byref(kept))
    return probs[:k].copy(), ids[:k].copy(), float(kept.value)


def _device(gpu, pkg, logits, tokens, mu, u, seed=7, draws=0, feed=False):
    lib, h = gpu.lib, gpu.handle
    d_logits = gpu.upload(logits)
    log = np.zeros(2048 + 8, np.uint32)
    log[:len(tokens)] = tokens
    d_log = gpu.upload(log)
    d_n = gpu.upload(np.array([len(tokens)] * 4, np.uint32))
    state = np.array([np.float32(mu).view(np.uint32), seed, draws, 0], np.uint32)
    d_state = gpu.upload(state)
    d_out = gpu.upload(np.array([12345, 0, 0, 0], np.uint32))
    d_rep = gpu.zeros(16)
    pkg.check(lib.lv_sample_mirostat(h, d_logits, VOCAB, d_log, d_n, d_state, C.c_float(u), d_log if feed else None, 2049, d_out, None, d_rep))
    gpu.sync()
    tok = int(gpu.download(d_out, np.uint32, 1)[0])
    rep = gpu.download(d_rep, np.uint32, 4)
    st = gpu.download(d_state, np.uint32, 4)
    fed = int(gpu.download(d_log, np.uint32, 2056)[len(tokens)])
    for d in (d_logits, d_log, d_n, d_state, d_out, d_rep):
        gpu.free(d)
    return dict(token=tok, kept=int(rep[0]), kept_sum=float(rep[1:2].view(np.float32)[0]), p_sel=float(rep[2:3].view(np.float32)[0]),
                u=float(rep[3:4].view(np.float32)[0]), mu=float(st[0:1].view(np.float32)[0]), draws=int(st[2]), fed=fed)


@pytest.mark.parametrize("mu,scale,history,n_hot", [(10.0, 3.0, "plain", 24), (6.0, 2.0, "newlines", 16), (4.0, 2.5, "newlines", 5), (10.0, 6.0, "short", 24)])
def test_candidates_draw_and_mu_match_the_oracle(gpu, pkg, mu, scale, history, n_hot):
    rng = np.random.default_rng(int(mu * 10 + scale))
    logits = (rng.standard_normal(VOCAB) * scale).astype(np.float32)
    hot = rng.choice(VOCAB, n_hot, replace=False)            # a handful of likely tokens, so that several candidates pass the cut
    hot[0] = 13
    logits[hot] = (5.0 * scale + rng.standard_normal(n_hot) * 0.4 * scale).astype(np.float32)
    logits[13] = 5.3 * scale                                 # token 13 among them, so its penalty matters
    tokens = [int(t) for t in rng.integers(3, VOCAB, 5 if history == "short" else 150)]
    if history == "newlines":
        tokens[-3] = tokens[-20] = tokens[-64] = 13          # three within the last 64 ...
        tokens[-70] = 13                                     # ... one outside
    probs, ids, kept_sum = _oracle(logits, tokens, mu)
    assert len(ids) >= 2
    lib = ob.load()
    cum = np.cumsum(probs.astype(np.float64))
    for j in sorted({0, len(ids) // 3, len(ids) // 2, len(ids) - 1}):
        # a variate whose target falls in the middle of candidate j's interval
        u = float((cum[j] - 0.5 * probs[j]) / cum[-1])
        got = _device(gpu, pkg, logits, tokens, mu, u)
        assert got["kept"] == len(ids)
        # the reference adds the 32000 exponentials one after the other in fp32; the kernel adds them pairwise, so
        # the normaliser (and with it every probability) differs in the fifth digit; their ratios do not
        assert abs(got["kept_sum"] - kept_sum) <= 2e-4 * kept_sum
        assert got["token"] == int(ids[j]), (j, got)
        assert abs(got["p_sel"] - float(probs[j])) <= 2e-4 * float(probs[j])
        assert abs(got["p_sel"] / got["kept_sum"] - float(probs[j]) / kept_sum) <= 2e-6 * float(probs[j]) / kept_sum
        want_mu = lib.orc_sampler_mu_update(C.c_float(mu), C.c_float(float(probs[j])), C.c_float(kept_sum))
        assert abs(got["mu"] - want_mu) <= 2e-5
        assert got["draws"] == 1
    # the ends of the interval: the first candidate at 0, the last one just below 1
    assert _device(gpu, pkg, logits, tokens, mu, 0.0)["token"] == int(ids[0])
    assert _device(gpu, pkg, logits, tokens, mu, 0.99999994)["token"] == int(ids[-1])


def test_generator_is_reproducible_and_feeds_the_token_log(gpu, pkg):
    rng = np.random.default_rng(5)
    logits = (rng.standard_normal(VOCAB) * 3).astype(np.float32)
    tokens = [int(t) for t in rng.integers(3, VOCAB, 40)]
    _, ids, _ = _oracle(logits, tokens, 10.0)
    a = _device(gpu, pkg, logits, tokens, 10.0, -1.0, seed=99, draws=3, feed=True)
    b = _device(gpu, pkg, logits, tokens, 10.0, -1.0, seed=99, draws=3, feed=True)
    c = [_device(gpu, pkg, logits, tokens, 10.0, -1.0, seed=99, draws=d)["u"] for d in range(4, 12)]
    assert a["token"] == b["token"] and a["u"] == b["u"] and 0.0 <= a["u"] < 1.0
    assert a["token"] in set(int(i) for i in ids)
    assert a["fed"] == a["token"] and a["draws"] == 4
    assert len(set(c)) == len(c) and all(0.0 <= x < 1.0 for x in c)          # the counter moves the stream


def test_nothing_kept_is_reported(gpu, pkg):
    logits = np.full(VOCAB, np.nan, np.float32)
    lib, h = gpu.lib, gpu.handle
    d_logits, d_log = gpu.upload(logits), gpu.upload(np.zeros(64, np.uint32))
    d_n, d_state = gpu.upload(np.array([4] * 4, np.uint32)), gpu.upload(np.array([np.float32(10).view(np.uint32), 1, 0, 0], np.uint32))
    d_out = gpu.upload(np.zeros(4, np.uint32))
    pkg.check(lib.lv_sample_mirostat(h, d_logits, VOCAB, d_log, d_n, d_state, C.c_float(0.5), None, 64, d_out, None, None))
    with pytest.raises(pkg.LvError) as e:
        gpu.sync()
    assert e.value.code == pkg.LV_ERR_DEVICE_WAIT
    assert int(gpu.download(d_out, np.uint32, 1)[0]) == NO_TOKEN
    gpu.sync()

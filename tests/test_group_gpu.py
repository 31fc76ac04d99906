"""llava_session_group: one decoding step for several sessions with one pass over the weights.

Every member has its own prompt, position and caches; the group step must give each member what its own
llava_session steps give it.  The group runs the batched (tcgen05) products, so it is held to the same bounds as a
prompt evaluated in batches: with exact weight tiles the decode tolerance (1e-2 / 1e-3) and identical greedy tokens,
with the default fast tiles rel-L2 <= 3e-3 and the same token unless the oracle's two best logits are closer than the
logits differ.  The per-member references are the oracle's trajectories.
"""
import numpy as np
import pytest

import quant_np as qn
from test_e2e_gpu import FAST_PROMPT_REL_L2, LOGIT_REL_L2, OracleSession, assert_logits_close, same_choice

pytestmark = pytest.mark.gpu

PROMPTS = [(5, 11), (9, 22), (16, 33), (3, 44), (12, 55), (7, 66), (20, 77)]       # (length, seed) per member
N_STEPS = 6


def prompt_of(n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(3, 32000, n)]


@pytest.fixture(scope="module")
def world(pkg, tmp_path_factory):
    path = str(tmp_path_factory.mktemp("group") / "tiny.bin")
    pkg.write_synthetic_model(path, "7b", n_layers=2, wtype=qn.Q4_0)
    want = []
    for n, seed in PROMPTS:
        orc = OracleSession(path)
        for t in prompt_of(n, seed):
            orc.push(t)
        logits, toks = [], []
        for _ in range(N_STEPS + 1):
            logits.append(orc.eval())
            toks.append(int(orc.argmax()))
            orc.push(toks[-1])
        orc.close()
        want.append((toks, logits))
    ctx = pkg.HostContext(path, 0)
    yield dict(ctx=ctx, want=want, vocab=32000)
    ctx.close()


def start_members(world, count):
    """Sessions that have evaluated their prompts and hold their first greedy token as the one pending token."""
    sessions = []
    for i in range(count):
        n, seed = PROMPTS[i]
        s = world["ctx"].session()
        s.set_deterministic(True)
        for t in prompt_of(n, seed):
            assert s.push_token(t)
        tok = s.predict_next_token()
        assert tok == world["want"][i][0][0]
        assert s.push_token(tok)
        sessions.append(s)
    return sessions


@pytest.mark.parametrize("count", [2, 7])
@pytest.mark.parametrize("form", ["exact", "fast"])
def test_group_steps_give_every_member_its_own_trajectory(pkg, world, form, count):
    world["ctx"].set_exact_batched_products(form == "exact")
    sessions = start_members(world, count)
    group = pkg.SessionGroup(world["ctx"], sessions)
    rel_l2 = LOGIT_REL_L2 if form == "exact" else FAST_PROMPT_REL_L2
    alive = [True] * count
    for step in range(1, N_STEPS):
        toks = group.step()
        assert toks is not None
        for i, s in enumerate(sessions):
            if not alive[i]:
                assert s.push_token(toks[i])
                continue
            want_toks, want_logits = world["want"][i]
            got = group.logits(i, world["vocab"])
            assert_logits_close(got, want_logits[step], rel_l2)
            assert same_choice(toks[i], got, want_logits[step])
            if form == "exact":
                assert toks[i] == want_toks[step]
            if toks[i] != want_toks[step]:
                alive[i] = False                  # a near-tie went the other way: this member's trajectory parts here
            assert s.push_token(toks[i])
    world["ctx"].set_exact_batched_products(False)
    # positions and token buffers are the members' own: every member evaluated prompt + N_STEPS - 1 tokens
    for i, s in enumerate(sessions):
        assert s.tokens_in_gpu() == PROMPTS[i][0] + N_STEPS - 1 and len(s.tokens()) == PROMPTS[i][0] + N_STEPS
    assert group.kernel_launches() == 1 + 2 * 9 + 2 + 1
    # a member goes on by itself from where the group left it (per-token kernels, its own recorded step)
    if form == "exact":
        s = sessions[1]
        assert s.predict_next_token() == world["want"][1][0][N_STEPS]
    group.close()
    for s in sessions:
        s.close()


def test_group_generates_on_the_device_like_step_by_step(pkg, world):
    world["ctx"].set_exact_batched_products(True)
    a = start_members(world, 3)
    ga = pkg.SessionGroup(world["ctx"], a)
    stepwise = [[] for _ in a]
    for _ in range(4):
        toks = ga.step()
        for i, s in enumerate(a):
            stepwise[i].append(toks[i])
            assert s.push_token(toks[i])
    b = start_members(world, 3)
    gb = pkg.SessionGroup(world["ctx"], b)
    assert gb.generate_greedy_on_device(4) == stepwise
    world["ctx"].set_exact_batched_products(False)
    for i, s in enumerate(b):
        assert s.tokens() == a[i].tokens() and s.tokens_in_gpu() == a[i].tokens_in_gpu()
    for g in (ga, gb):
        g.close()
    for s in a + b:
        s.close()


def test_group_refuses_what_it_cannot_do(pkg, world):
    ctx = world["ctx"]
    s = start_members(world, 2)
    with pytest.raises(RuntimeError):
        pkg.SessionGroup(ctx, s[:1])                     # one session is not a group
    with pytest.raises(RuntimeError):
        pkg.SessionGroup(ctx, [s[0], s[0]])              # the same session twice
    g = pkg.SessionGroup(ctx, s)
    assert g.step() is not None
    assert g.step() is None                              # nothing pending: the members' tokens were not pushed
    g.close()
    for x in s:
        x.close()


def test_group_members_that_sample_draw_with_their_own_sampler(pkg, world):
    """Members set to the reference's sampler (its default) get their token from the device sampler at the end of the
    group step: with the same seed a member draws the same tokens in a group as alone (exact weight tiles; the draw
    depends on the logits through the kept set and the cumulative mass, so the comparison allows a member to part from
    its lone trajectory where a probability sits within the logits' tolerance of the cut), greedy members beside them
    stay greedy, and mu moves."""
    world["ctx"].set_exact_batched_products(True)

    def members(sampled):
        out = []
        for i in range(3):
            n, seed = PROMPTS[i]
            s = world["ctx"].session()
            s.set_deterministic(i == 2 or not sampled)          # member 2 stays greedy
            s.set_seed(1000 + i)
            for t in prompt_of(n, seed):
                assert s.push_token(t)
            tok = s.predict_next_token()
            assert tok != pkg.NO_TOKEN and s.push_token(tok)
            out.append(s)
        return out

    alone = members(True)
    lone_tokens = [[s.tokens()[-1]] for s in alone]
    for _ in range(5):
        for i, s in enumerate(alone):
            tok = s.predict_next_token()
            assert s.push_token(tok)
            lone_tokens[i].append(tok)
    grouped = members(True)
    g = pkg.SessionGroup(world["ctx"], grouped)
    group_tokens = [[s.tokens()[-1]] for s in grouped]
    for _ in range(5):
        toks = g.step()
        assert toks is not None and all(t < world["vocab"] for t in toks)
        for i, s in enumerate(grouped):
            assert s.push_token(toks[i])
            group_tokens[i].append(toks[i])
    world["ctx"].set_exact_batched_products(False)
    assert g.kernel_launches() == 1 + 2 * 9 + 2 + 1 + 2                  # two sampler launches
    assert group_tokens[2] == lone_tokens[2] == world["want"][2][0][:6]   # the greedy member
    agree = [next((j for j, (a, b) in enumerate(zip(group_tokens[i], lone_tokens[i])) if a != b), 6) for i in range(2)]
    assert min(agree) >= 3 and max(agree) == 6, (group_tokens, lone_tokens)
    for i in range(2):
        assert grouped[i].mirostat_mu() != pytest.approx(10.0)           # moved from its start value (2 tau)
    g.close()
    for s in alone + grouped:
        s.close()

"""The TCP front end (lsrv::tlv_server) over loopback.

Without a GPU: the framing and every reply that needs no session (token map, session list, the error
acknowledgements of reference server/client.cpp:146-300).  With one: every opcode against a live session,
the generated tokens compared with the CPU oracle's greedy trajectory.
"""
import os
import struct

import numpy as np
import pytest

import quant_np as qn

OK, NOK, NO_SUCH_SESSION, TICK_ALREADY_REQUESTED, ALREADY_RUNNING, NOT_TRACING, BATCHED_TICK, BAD_ARGUMENTS, UNKNOWN_COMMAND = range(9)


def ack(code):
    return struct.pack("<I", code)


@pytest.fixture(scope="module")
def tiny_model(pkg, tmp_path_factory):
    path = str(tmp_path_factory.mktemp("srv") / "tiny.bin")
    pkg.write_synthetic_model(path, "7b", n_layers=2, wtype=qn.Q4_0)
    return path


def test_session_independent_requests_and_framing(pkg, tiny_model):
    ctx = pkg.HostContext(tiny_model, None)
    model = pkg.ModelFile(tiny_model)
    with pkg.Server(ctx) as server:
        assert server.port != 0
        a, b = pkg.Client(server.port), pkg.Client(server.port)
        # token map: {u32 length, bytes} per token, in id order
        op, data = a.call(a.GET_TOKEN_MAP)
        assert op == a.TOKEN_MAP
        at, texts = 0, []
        while at < len(data):
            n, = struct.unpack_from("<I", data, at)
            texts.append(data[at + 4:at + 4 + n])
            at += 4 + n
        assert at == len(data) and len(texts) == model.vocab_size
        assert texts[:300] == [model.token(i)[0] for i in range(300)]
        assert a.call(a.LIST_SESSIONS) == (a.SESSION_LIST, b"")
        # no device behind this context: a session cannot be made
        assert a.call(a.NEW_SESSION) == (a.ACK, ack(NOK))
        # error replies
        assert a.call(5) == (a.ACK, ack(UNKNOWN_COMMAND))                                   # below 16, not a command
        assert a.call(a.TICK, b"\x01\x00") == (a.ACK, ack(BAD_ARGUMENTS))                   # shorter than a session id
        assert a.call(a.TICK, struct.pack("<II", 1, 2)) == (a.ACK, ack(BAD_ARGUMENTS))      # longer than one
        assert a.call(a.ADD_TOKEN, struct.pack("<I", 1)) == (a.ACK, ack(BAD_ARGUMENTS))     # token id missing
        assert a.call(a.ADD_TEXT, struct.pack("<I", 1)) == (a.ACK, ack(BAD_ARGUMENTS))      # empty text
        assert a.call(40, struct.pack("<II", 1, 2)) == (a.ACK, ack(UNKNOWN_COMMAND))
        for cmd in (a.GET_SESSION_TOKENS, a.SUBSCRIBE, a.UNSUBSCRIBE, a.KILL_SESSION, a.START, a.STOP, a.TICK, a.GET_STATUS):
            assert a.call(cmd, struct.pack("<I", 77)) == (a.ACK, ack(NO_SUCH_SESSION))
        for cmd in (a.REWIND, a.ADD_TOKEN, a.SET_OPTIONS):
            assert a.call(cmd, struct.pack("<II", 77, 0)) == (a.ACK, ack(NO_SUCH_SESSION))
        for cmd in (a.ADD_TEXT, a.SAVE_FRAME, a.SNAPSHOT, a.RESTORE):
            assert a.call(cmd, struct.pack("<I", 77) + b"x") == (a.ACK, ack(NO_SUCH_SESSION))
        # three requests in one segment, then one request in three segments
        a.sock.sendall(b"".join(struct.pack("<III", a.LIST_SESSIONS, 900 + i, 0) for i in range(3)))
        assert [a.recv() for _ in range(3)] == [(a.SESSION_LIST, 900 + i, b"") for i in range(3)]
        frame = struct.pack("<IIII", a.TICK, 950, 4, 77)
        for part in (frame[:5], frame[5:13], frame[13:]):
            a.sock.sendall(part)
        assert a.recv() == (a.ACK, 950, ack(NO_SUCH_SESSION))
        # the second client is served independently
        assert b.call(b.LIST_SESSIONS) == (b.SESSION_LIST, b"")
        # a frame above 64 KiB closes that connection only (server/client.cpp:128-131)
        b.sock.sendall(struct.pack("<III", b.ADD_TEXT, 1, 0x10001))
        with pytest.raises(ConnectionError):
            b.recv()
        assert a.call(a.LIST_SESSIONS) == (a.SESSION_LIST, b"")
        a.close()
        b.close()
    model.close()
    ctx.close()


@pytest.mark.gpu
def test_every_opcode_against_a_live_session(pkg, tiny_model, tmp_path):
    from test_e2e_gpu import N_PROMPT, OracleSession, prompt_tokens
    orc = OracleSession(tiny_model)
    prompt = prompt_tokens()
    for t in prompt:
        orc.push(t)
    greedy = []
    for _ in range(8):
        orc.eval()
        greedy.append(orc.argmax())
        orc.push(greedy[-1])
    orc.close()

    ctx = pkg.HostContext(tiny_model, 0)
    with pkg.Server(ctx, deterministic=True) as server:
        a, b = pkg.Client(server.port), pkg.Client(server.port)
        # newSession: the caller gets its request id back, the other client a broadcast
        op, data = a.call(a.NEW_SESSION)
        assert op == a.SESSION_CREATED and len(data) == 4
        sid = data
        session, = struct.unpack("<I", sid)
        assert b.recv() == (b.SESSION_CREATED, 0, sid)
        assert b.call(b.LIST_SESSIONS) == (b.SESSION_LIST, sid)
        assert b.call(b.SUBSCRIBE, sid) == (b.ACK, ack(OK))
        assert a.call(a.GET_STATUS, sid) == (a.ACK, ack(OK))
        assert a.call(a.SET_OPTIONS, sid + struct.pack("<I", 0)) == (a.ACK, ack(OK))
        for t in prompt:
            assert a.call(a.ADD_TOKEN, sid + struct.pack("<I", t)) == (a.ACK, ack(OK))
        assert a.call(a.ADD_TOKEN, sid + struct.pack("<I", 32000)) == (a.ACK, ack(NOK))
        # tick: the ticker gets the token under its request id, the subscriber as a broadcast
        token0 = sid + struct.pack("<II", greedy[0], N_PROMPT)
        assert a.call(a.TICK, sid) == (a.NEW_TOKEN, token0)
        assert a.others == []                                                  # not subscribed: no broadcast for a
        assert b.recv() == (b.NEW_TOKEN, 0, token0)
        op, data = a.call(a.GET_SESSION_TOKENS, sid)
        assert op == a.BUFFER and list(np.frombuffer(data, np.uint32)) == prompt + greedy[:1]
        # snapshot, run on, rewind, restore
        snap = os.fsencode(str(tmp_path / "snap.bin"))
        assert a.call(a.SNAPSHOT, sid + snap) == (a.ACK, ack(OK))
        assert a.call(a.SNAPSHOT, sid + b"/nonexistent-dir/x") [0] == a.ACK
        assert a.call(a.SAVE_FRAME, sid + os.fsencode(str(tmp_path / "frame.bin")))[0] == a.ACK
        assert a.call(a.START, sid) == (a.ACK, ack(OK))
        assert a.call(a.TICK, sid) == (a.ACK, ack(ALREADY_RUNNING))
        assert a.call(a.RESTORE, sid + snap) == (a.ACK, ack(ALREADY_RUNNING))
        got = []
        while len(got) < 5:
            op, rid, data = b.recv()
            assert (op, rid) == (b.NEW_TOKEN, 0) and data[:4] == sid
            got.append(struct.unpack("<II", data[4:]))
        assert [t for t, _ in got] == greedy[1:6] and [p for _, p in got] == list(range(N_PROMPT + 1, N_PROMPT + 6))
        assert a.call(a.STOP, sid) == (a.ACK, ack(OK))
        assert b.call(b.UNSUBSCRIBE, sid) == (b.ACK, ack(OK))
        assert a.call(a.REWIND, sid + struct.pack("<I", N_PROMPT)) == (a.ACK, ack(OK))
        op, data = a.call(a.GET_SESSION_TOKENS, sid)
        assert list(np.frombuffer(data, np.uint32)) == prompt
        assert a.call(a.TICK, sid) == (a.ACK, ack(NOK))                        # every token is on the device: nothing to evaluate
        assert a.call(a.REWIND, sid + struct.pack("<I", N_PROMPT - 1)) == (a.ACK, ack(OK))
        assert a.call(a.ADD_TOKEN, sid + struct.pack("<I", prompt[-1])) == (a.ACK, ack(OK))
        assert a.call(a.TICK, sid) == (a.NEW_TOKEN, token0)                    # the same token again after the rewind
        # a snapshot holds the tokens that were on the device when it was taken: the prompt, not yet the first reply
        assert a.call(a.RESTORE, sid + snap) == (a.ACK, ack(OK))
        op, data = a.call(a.GET_SESSION_TOKENS, sid)
        assert list(np.frombuffer(data, np.uint32)) == prompt
        assert a.call(a.ADD_TOKEN, sid + struct.pack("<I", greedy[0])) == (a.ACK, ack(OK))
        assert a.call(a.TICK, sid) == (a.NEW_TOKEN, sid + struct.pack("<II", greedy[1], N_PROMPT + 1))
        # text goes through the tokenizer of the model file
        op, data = a.call(a.NEW_SESSION)
        sid2 = data
        assert a.call(a.ADD_TEXT, sid2 + b"hello") [0] == a.ACK
        op, data = a.call(a.LIST_SESSIONS)
        assert sorted(np.frombuffer(data, np.uint32)) == sorted([session, struct.unpack("<I", sid2)[0]])
        # kill: acknowledged, and the session leaves the list
        assert a.call(a.KILL_SESSION, sid) == (a.ACK, ack(OK))
        for _ in range(200):
            op, data = a.call(a.LIST_SESSIONS)
            if data == sid2:
                break
        assert data == sid2
        assert a.call(a.TICK, sid) == (a.ACK, ack(NO_SUCH_SESSION))
        a.close()
        b.close()
    ctx.close()      # the server's stop() has killed and joined the second session


@pytest.mark.gpu
def test_running_sessions_are_stepped_together(pkg, tiny_model):
    """Three sessions in the running state: the server's scheduler evaluates their tokens in shared steps (one pass over
    the weights per round), and every session still receives its own greedy trajectory."""
    from test_e2e_gpu import OracleSession
    n_tokens = 8
    prompts = [[int(t) for t in np.random.default_rng(500 + i).integers(3, 32000, n)] for i, n in enumerate((6, 11, 4))]
    want = []
    for p in prompts:
        orc = OracleSession(tiny_model)
        for t in p:
            orc.push(t)
        toks = []
        for _ in range(120):                    # the sessions run on while the test talks to the server
            orc.eval()
            toks.append(int(orc.argmax()))
            orc.push(toks[-1])
        orc.close()
        want.append(toks)
    ctx = pkg.HostContext(tiny_model, 0)
    ctx.set_exact_batched_products(True)           # exact weight tiles: the tokens must be the oracle's
    with pkg.Server(ctx, deterministic=True) as server:
        c = pkg.Client(server.port)
        sids = []
        for p in prompts:
            op, sid = c.call(c.NEW_SESSION)
            assert op == c.SESSION_CREATED
            for t in p:
                assert c.call(c.ADD_TOKEN, sid + struct.pack("<I", t)) == (c.ACK, ack(OK))
            assert c.call(c.SUBSCRIBE, sid) == (c.ACK, ack(OK))
            sids.append(sid)
        got = {sid: [] for sid in sids}
        pending = set()
        for sid in sids:
            pending.add(c.send(c.START, sid))
        # broadcasts (request id 0) carry {session, token, position}; the three acknowledgements arrive in between
        while any(len(v) < n_tokens for v in got.values()):
            op, rid, data = c.recv()
            if rid in pending:
                assert (op, data) == (c.ACK, ack(OK))
                pending.discard(rid)
                continue
            assert op == c.NEW_TOKEN and rid == 0
            token, pos = struct.unpack("<II", data[4:])
            got[data[:4]].append((token, pos))
        # one session stops; the other two go on (their group changes, a step queued ahead for the three is dropped)
        stop_id = c.send(c.STOP, sids[0])
        stopped_at = None
        while stopped_at is None or any(len(got[sid]) < stopped_at + 6 for sid in sids[1:]):
            op, rid, data = c.recv()
            if rid == stop_id:
                assert (op, data) == (c.ACK, ack(OK))
                stopped_at = max(len(got[sid]) for sid in sids[1:])
                continue
            assert op == c.NEW_TOKEN and rid == 0
            token, pos = struct.unpack("<II", data[4:])
            got[data[:4]].append((token, pos))
        n0 = len(got[sids[0]])
        # the stopped session has not moved since, and a tick gives it its own next token at its own position
        rid = c.send(c.TICK, sids[0])
        while True:
            op, r, data = c.recv()
            if r == rid:
                break
            assert op == c.NEW_TOKEN and r == 0
            if data[:4] != sids[0]:               # (the subscriber also gets the tick's token as a broadcast)
                token, pos = struct.unpack("<II", data[4:])
                got[data[:4]].append((token, pos))
        assert op == c.NEW_TOKEN and data[:4] == sids[0]
        token, pos = struct.unpack("<II", data[4:])
        assert pos == len(prompts[0]) + n0
        if n0 < len(want[0]):                     # (the oracle's trajectory is 120 tokens long)
            assert token == want[0][n0]
        for sid in sids[1:]:
            c.send(c.STOP, sid)
        for i, sid in enumerate(sids):
            m = min(len(got[sid]), len(want[i]))
            assert m >= n_tokens
            assert [t for t, _ in got[sid][:m]] == want[i][:m]
            assert [p for _, p in got[sid][:m]] == list(range(len(prompts[i]), len(prompts[i]) + m))
        steps, tokens = server.grouped()
        assert steps > 0 and tokens >= 2 * steps, (steps, tokens)
        assert server.steps_ahead() > 0                       # greedy sessions: most shared steps were queued ahead
        c.close()
    ctx.set_exact_batched_products(False)
    ctx.close()


@pytest.mark.gpu
@pytest.mark.parametrize("deterministic", [True, False], ids=["greedy", "sampled"])
def test_sessions_that_start_stop_tick_rewind_and_die_while_others_run(pkg, tiny_model, deterministic):
    """Churn: six sessions, two clients, three seconds of random start / stop / tick / add / rewind / kill / new-session
    orders while other sessions generate.  The server must answer every request, keep every position consistent (a
    token's position is the number of tokens its session held before it) and shut down cleanly."""
    import random
    import time
    rng = random.Random(7)
    ctx = pkg.HostContext(tiny_model, 0)
    with pkg.Server(ctx, deterministic=deterministic) as server:
        a, b = pkg.Client(server.port, timeout=60.0), pkg.Client(server.port, timeout=60.0)
        live = []

        def new_session(c):
            op, sid = c.call(c.NEW_SESSION)
            assert op == c.SESSION_CREATED
            for t in [rng.randrange(3, 32000) for _ in range(rng.randrange(1, 9))]:
                assert c.call(c.ADD_TOKEN, sid + struct.pack("<I", t)) == (c.ACK, ack(OK))
            live.append(sid)

        for _ in range(6):
            new_session(a)
        deadline = time.time() + 3.0
        n_orders = 0
        while time.time() < deadline:
            c = rng.choice((a, b))
            sid = rng.choice(live)
            kind = rng.randrange(8)
            if kind == 0:
                op, data = c.call(c.START, sid)
                assert op == c.ACK and data in (ack(OK), ack(TICK_ALREADY_REQUESTED))
            elif kind == 1:
                assert c.call(c.STOP, sid) == (c.ACK, ack(OK))
            elif kind == 2:
                op, data = c.call(c.TICK, sid)
                assert (op == c.NEW_TOKEN and data[:4] == sid) or (op == c.ACK and data in (ack(ALREADY_RUNNING), ack(NOK), ack(TICK_ALREADY_REQUESTED)))
            elif kind == 3:
                op, data = c.call(c.ADD_TOKEN, sid + struct.pack("<I", rng.randrange(3, 32000)))
                assert op == c.ACK and data in (ack(OK), ack(NOK))
            elif kind == 4:
                op, data = c.call(c.GET_SESSION_TOKENS, sid)
                assert op == c.BUFFER
                n = len(data) // 4
                if n > 2:
                    assert c.call(c.REWIND, sid + struct.pack("<I", rng.randrange(1, n))) == (c.ACK, ack(OK))
            elif kind == 5 and len(live) > 3:
                assert c.call(c.KILL_SESSION, sid) == (c.ACK, ack(OK))
                live.remove(sid)
            elif kind == 6 and len(live) < 8:
                new_session(c)
            else:
                op, data = c.call(c.LIST_SESSIONS)
                assert op == c.SESSION_LIST and len(data) % 4 == 0
            n_orders += 1
        assert n_orders > 50
        assert server.grouped()[0] > 0                       # sessions did run together in between
        # every session still answers, and its buffer is a valid token list
        for sid in live:
            c = a
            assert c.call(c.STOP, sid) == (c.ACK, ack(OK))
            op, data = c.call(c.GET_SESSION_TOKENS, sid)
            assert op == c.BUFFER and all(t < 32000 for t in np.frombuffer(data, np.uint32))
            op, data = c.call(c.TICK, sid)
            assert op in (c.NEW_TOKEN, c.ACK)
        a.close()
        b.close()
    ctx.close()

"""Token-in-token-out session proxy: exact token history across turns, loss masks, conflict detection."""

from miles_b200.rollout.session import SessionStore, build_session_app


class _Tok:
    """Character-level tokenizer: decode(encode(x)) == x, which makes the delta rendering easy to check."""

    def encode(self, text, add_special_tokens=False):
        return [ord(c) for c in text]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(i) for i in ids)


def _store():
    calls = []

    def generate(input_ids, sp):
        calls.append(list(input_ids))
        reply = f"r{len(calls)}"
        return {"output_ids": [ord(c) for c in reply], "output_token_logprobs": [(-0.5, 0)] * len(reply),
                "finish_reason": {"type": "stop"}, "weight_version": 3}

    return SessionStore(_Tok(), generate), calls


def test_two_turns_keep_exact_history_and_masks():
    from fastapi.testclient import TestClient

    store, calls = _store()
    c = TestClient(build_session_app(store))
    m1 = [{"role": "user", "content": "hi"}]
    r1 = c.post("/sessions/s1/v1/chat/completions", json={"messages": m1, "max_tokens": 8}).json()
    assert r1["choices"][0]["message"]["content"] == "r1"
    m2 = m1 + [{"role": "assistant", "content": "r1"}, {"role": "tool", "content": "42"}]
    r2 = c.post("/sessions/s1/v1/chat/completions", json={"messages": m2}).json()
    assert r2["choices"][0]["message"]["content"] == "r2"
    # the second call continued from the exact ids of turn one (prompt + sampled ids), not from re-rendered text
    assert calls[1][:len(calls[0]) + 2] == calls[0] + [ord("r"), ord("1")]
    s = c.get("/sessions/s1/sample").json()
    text = "".join(chr(i) for i in s["tokens"])
    assert text.startswith("<|user|>hi<|end|><|assistant|>r1") and text.endswith("r2")
    resp = s["tokens"][len(s["tokens"]) - s["response_length"]:]
    trained = "".join(chr(t) for t, m in zip(resp, s["loss_mask"]) if m)
    assert trained == "r1r2" and len(s["rollout_log_probs"]) == s["response_length"]
    assert s["weight_versions"] == [3]
    assert c.delete("/sessions/s1").status_code == 200 and c.get("/sessions/s1/sample").status_code == 404


def test_rewritten_history_is_rejected():
    from fastapi.testclient import TestClient

    store, _ = _store()
    c = TestClient(build_session_app(store))
    c.post("/sessions/s/v1/chat/completions", json={"messages": [{"role": "user", "content": "a"}]})
    bad = [{"role": "user", "content": "changed"}, {"role": "assistant", "content": "r1"}, {"role": "user", "content": "b"}]
    assert c.post("/sessions/s/v1/chat/completions", json={"messages": bad}).status_code == 400  # messages are not append-only


def test_tree_sessions_branch_pick_and_postprocess():
    """Tree-serving sessions (--use-session-server v2): a request that rewrites history branches instead of being
    refused, retried turns are dropped by the default picker, shared prefix tokens are trained once."""
    from miles_b200.rollout.session.hooks import match_loose_tool_call, match_strict, resolve_matcher
    from miles_b200.rollout.session.server import SessionStore

    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [ord(c) % 251 for c in text]

        def decode(self, ids, skip_special_tokens=True):
            return "".join(chr(97 + (i % 26)) for i in ids)

    calls = []

    def generate(ids, sp):
        calls.append(list(ids))
        out = [(len(ids) * 7 + k) % 200 for k in range(3)]
        return {"output_ids": out, "output_token_logprobs": [-0.5] * 3, "finish_reason": "stop"}

    store = SessionStore(Tok(), generate, tree=True)
    sys_user = [{"role": "system", "content": "s"}, {"role": "user", "content": "q1"}]
    r1 = store.chat("a", sys_user, {})
    hist = sys_user + [{"role": "assistant", "content": r1["text"]}, {"role": "user", "content": "q2"}]
    r2 = store.chat("a", hist, {})
    assert calls[1][:len(calls[0])] == calls[0]                      # the second turn extends the first lineage
    # the agent retries the second turn with an edited question: a branch after the first assistant message
    hist_b = sys_user + [{"role": "assistant", "content": r1["text"]}, {"role": "user", "content": "q2 edited"}]
    store.chat("a", hist_b, {})
    assert calls[2][:len(calls[0]) + 3] == calls[1][:len(calls[0]) + 3] and calls[2] != calls[1]
    tree = store._trees["a"]
    assert len(tree.leaves()) == 2
    samples = store.samples("a")
    assert len(samples) == 2
    # tokens of the shared first turn carry loss in one sample only
    first_turn = sum(s["loss_mask"][:3] == [1, 1, 1] for s in samples)
    assert first_turn == 1
    assert match_strict({"role": "user", "content": "x"}, {"role": "user", "content": "x"})
    tc = lambda i, a: {"role": "assistant", "content": None, "tool_calls": [{"id": i, "function": {"name": "f", "arguments": a}}]}
    assert not match_strict(tc("1", '{"a": 1}'), tc("2", '{"a":1}')) and match_loose_tool_call(tc("1", '{"a": 1}'), tc("2", '{"a":1}'))
    assert resolve_matcher("role_content_only")(tc("1", "{}"), {"role": "assistant", "content": None})


def test_session_lifecycle_endpoints_streaming_and_length_cap():
    import json

    from fastapi.testclient import TestClient

    store, calls = _store()
    c = TestClient(build_session_app(store))
    assert c.get("/health").json()["status"] == "ok"
    sid = c.post("/sessions").json()["session_id"]
    assert c.get(f"/sessions/{sid}").json()["num_tokens"] == 0 and c.get("/sessions/nope").status_code == 404
    m1 = [{"role": "user", "content": "hello"}]
    r = c.post(f"/sessions/{sid}/v1/chat/completions", json={"messages": m1, "stream": True})
    assert r.headers["content-type"].startswith("text/event-stream")
    events = [l[len("data: "):] for l in r.text.splitlines() if l.startswith("data: ")]
    assert events[-1] == "[DONE]" and json.loads(events[0])["choices"][0]["delta"]["content"] == "r1"
    assert json.loads(events[1])["choices"][0]["finish_reason"] == "stop"
    meta = c.get(f"/sessions/{sid}").json()
    assert meta["num_turns"] == 2 and meta["weight_versions"] == [3] and meta["num_tokens"] == len(store.sessions[sid].tokens)
    full = c.get(f"/sessions/{sid}/samples").json()["samples"][0]
    assert full["status"] == "completed" and full["response_length"] == 2
    cut = c.get(f"/sessions/{sid}/samples?max_seq_len={len(full['tokens']) - 1}").json()["samples"][0]
    assert cut["status"] == "truncated" and cut["response_length"] == 1 and len(cut["loss_mask"]) == 1 and len(cut["tokens"]) == len(full["tokens"]) - 1
    assert c.post(f"/sessions/{sid}/v1/chat/completions", json={"messages": "not a list"}).status_code == 400
    strict = TestClient(build_session_app(store, created_only=True))
    assert strict.post("/sessions/unknown/v1/chat/completions", json={"messages": m1}).status_code == 404


def test_verify_endpoint_diagnoses_a_token_level_session():
    """/sessions/{sid}/verify: the incremental trajectory against a fresh rendering; only assistant-text differences are ok."""
    import sys
    import os

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from fastapi.testclient import TestClient
    from test_tito import ToyTokenizer

    tok = ToyTokenizer()
    tok.special_token_ids = {tok._id(s) for s in tok.SPECIALS}
    replies = iter(["a|bc<|im_end|>", "d|ef<|im_end|>"])  # "|" marks where the engine split the text its own way

    def generate(input_ids, sp):
        parts = next(replies).split("|")
        ids = [t for part in parts for t in tok.encode(part)]
        return {"output_ids": ids, "output_token_logprobs": [(-0.1, 0)] * len(ids), "finish_reason": {"type": "stop"}, "weight_version": 1}

    store = SessionStore(tok, generate, tito=True, family="chatml")
    c = TestClient(build_session_app(store))
    m1 = [{"role": "user", "content": "hello"}]
    c.post("/sessions/v/v1/chat/completions", json={"messages": m1})
    m2 = m1 + [{"role": "assistant", "content": "abc"}, {"role": "user", "content": "more"}]
    c.post("/sessions/v/v1/chat/completions", json={"messages": m2})
    out = c.get("/sessions/v/verify").json()
    assert out["checked"] and out["ok"], out
    assert {m["kind"] for m in out["mismatches"]} <= {"assistant_text"} and len(out["mismatches"]) >= 1
    # damage a context token: the check names it
    store.sessions["v"].tokens[2] = tok._id("zz")
    bad = c.get("/sessions/v/verify").json()
    assert not bad["ok"] and any(m["kind"] == "context_text" and m["severe"] for m in bad["mismatches"])
    assert c.get("/sessions/none/verify").status_code == 404

"""OpenAI-compatible session proxy: ``POST /sessions/{id}/v1/chat/completions`` keeps the exact token sequence of
an agent conversation across turns (token in, token out) and ``GET /sessions/{id}/sample`` returns the assembled
training sample (tokens, loss mask, rollout log-probs). ``POST /sessions`` creates a session, ``GET /sessions/{id}`` describes
it, ``GET /sessions/{id}/samples?max_seq_len=`` collects its samples, ``DELETE /sessions/{id}`` closes it, ``GET /health``;
``"stream": true`` answers as server-sent events. Errors map to HTTP statuses through ``errors.py``.

An agent framework talks to this endpoint as if it were a chat model. Each request carries the whole conversation
so far; the server renders only the messages it has not seen yet (through the tokenizer's chat template, as a
delta against the previous rendering), appends them to the session's trajectory with loss mask 0, asks the
engine to continue from the session's token ids, appends the sampled ids with their log-probs and answers with
the decoded text.

Reference: miles/rollout/session/core.py:244-453, sessions.py:26-116.
"""

import threading
import time
import uuid
from typing import Callable, Optional

from .errors import MessageValidationError
from .trajectory import LinearTrajectory


class SessionStore:
    def __init__(self, tokenizer, generate: Callable, max_sessions: int = 4096, tito: bool = False, family: Optional[str] = None,
                 tree: bool = False, matcher: Optional[Callable] = None, picker: Optional[Callable] = None,
                 postprocessor: Optional[Callable] = None):
        """``generate(input_ids, sampling_params) -> dict`` with ``output_ids``, ``output_token_logprobs`` (floats),
        ``finish_reason`` and optionally ``weight_version`` (a blocking call into the engine client).

        ``tree`` selects the tree-serving mode: a request whose messages stop matching the session's history
        (``matcher(old, new)`` per message) branches at that point instead of being refused, every leaf is a sample,
        and ``picker`` / ``postprocessor`` choose and finalise the samples (rollout/session/hooks.py)."""
        self.tok, self.generate = tokenizer, generate
        self.max_sessions = max_sessions
        self.tree = tree
        from .hooks import default_postprocess, drop_retries, match_strict

        self.matcher = matcher or match_strict
        self.picker, self.postprocessor = picker or drop_retries, postprocessor or default_postprocess
        self._trees: dict = {}     # tree mode: session id -> TreeTrajectory
        self._lineage: dict = {}   # tree mode: session id -> [(messages, token count)] of the lineages served so far
        self._lock = threading.Lock()
        self.sessions: dict = {}
        self._rendered: dict = {}  # session id -> text of the conversation rendered so far (for delta rendering)
        self.tito = None
        if tito:
            from .tito import TitoTokenizer

            self.tito = TitoTokenizer(tokenizer, family)

    def get(self, sid: str) -> LinearTrajectory:
        with self._lock:
            if sid not in self.sessions:
                if len(self.sessions) >= self.max_sessions:
                    raise RuntimeError("too many open sessions")
                self.sessions[sid] = LinearTrajectory(sid)
                self._rendered[sid] = ""
            return self.sessions[sid]

    def close(self, sid: str) -> Optional[LinearTrajectory]:
        with self._lock:
            self._rendered.pop(sid, None)
            return self.sessions.pop(sid, None)

    # ------------------------------------------------------------------ rendering
    def _render(self, messages: list, add_generation_prompt: bool) -> str:
        if hasattr(self.tok, "apply_chat_template"):
            return self.tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)
        text = "".join(f"<|{m['role']}|>{m.get('content') or ''}<|end|>" for m in messages)
        return text + ("<|assistant|>" if add_generation_prompt else "")

    def _encode(self, text: str) -> list:
        return list(self.tok.encode(text, add_special_tokens=False)) if text else []

    def _chat_tito(self, traj, messages: list, sampling_params: dict) -> dict:
        """Token-level path: nothing already in the trajectory is rendered again; a later request contributes only
        its messages after the ones the session has seen (the assistant message among them is the turn the session
        generated itself and is skipped)."""
        if not traj.tokens:
            traj.append_context(messages[-1]["role"] if messages else "user", self.tito.initial(messages))
        else:
            new = [m for m in messages[traj.num_messages:] if m.get("role") != "assistant"]
            last = traj.turns[-1]
            traj.append_context(new[-1]["role"] if new else "user", self.tito.continuation(traj.tokens[last.start:last.end], new))
        out = self.generate(list(traj.tokens), dict(sampling_params))
        ids = list(out["output_ids"])
        lps = [float(x[0]) if isinstance(x, (list, tuple)) else float(x) for x in out.get("output_token_logprobs", [0.0] * len(ids))]
        traj.append_generation(ids, lps, out.get("weight_version"), out.get("finish_reason"))
        traj.num_messages = len(messages) + 1
        text = self.tok.decode(ids, skip_special_tokens=True) if hasattr(self.tok, "decode") else ""
        traj.messages = list(messages) + [{"role": "assistant", "content": text}]  # what /verify renders afresh
        return {"text": text, "ids": ids, "finish_reason": out.get("finish_reason", "stop")}

    def _chat_tree(self, sid: str, messages: list, sampling_params: dict) -> dict:
        """Tree mode: find the served lineage that shares the longest matching message prefix with the request, move
        the tree's cursor to the end of that prefix (a branch point if the lineage went on differently), render only
        the messages after it and continue from there."""
        from .tito import TreeTrajectory

        with self._lock:
            tree = self._trees.setdefault(sid, TreeTrajectory(sid))
            lineages = self._lineage.setdefault(sid, [])
        best_k, best_tokens = 0, []
        for hist, toks, marks in lineages:
            k = 0
            while k < len(hist) and k < len(messages) and self.matcher(hist[k], messages[k]):
                k += 1
            if k > best_k:
                best_k, best_tokens = k, toks[:marks[k - 1]]
        tree.seek(best_tokens)
        rest = messages[best_k:]
        # messages after the shared prefix are rendered as a delta of the chat template (or the token-level continuation)
        before = self._render(messages[:best_k], add_generation_prompt=False) if best_k else ""
        full = self._render(messages, add_generation_prompt=True)
        delta = full[len(before):] if full.startswith(before) else self._render(rest, add_generation_prompt=True)
        new_ids = self._encode(delta)
        if new_ids:
            tree.append(new_ids, generated=False)
        ctx = tree.tokens_to()
        out = self.generate(list(ctx), dict(sampling_params))
        ids = list(out["output_ids"])
        lps = [float(x[0]) if isinstance(x, (list, tuple)) else float(x) for x in out.get("output_token_logprobs", [0.0] * len(ids))]
        tree.append(ids, generated=True, log_probs=lps)
        text = self.tok.decode(ids, skip_special_tokens=True) if hasattr(self.tok, "decode") else ""
        # token count after each message of this lineage: the shared prefix keeps its marks, the new messages end where the
        # context ended, the generated assistant message where the trajectory ends now
        base_marks = next((m[:best_k] for h, t, m in lineages if len(h) >= best_k and best_k and t[:len(best_tokens)] == best_tokens), [])
        marks = list(base_marks) + [len(ctx)] * len(rest) + [len(ctx) + len(ids)]
        lineages.append((list(messages) + [{"role": "assistant", "content": text}], tree.tokens_to(), marks))
        return {"text": text, "ids": ids, "finish_reason": out.get("finish_reason", "stop")}

    def samples(self, sid: str, metadata: Optional[dict] = None) -> list:
        """The training samples of a session: one for a linear session, the picked and post-processed leaves of a tree."""
        if self.tree:
            tree = self._trees.get(sid)
            if tree is None:
                return []
            leaves = tree.to_sample_dicts()
            return self.postprocessor(self.picker(leaves, metadata or {}), metadata or {})
        return [self.sessions[sid].to_sample_dict()] if sid in self.sessions else []

    def chat(self, sid: str, messages: list, sampling_params: dict) -> dict:
        if self.tree:
            return self._chat_tree(sid, messages, sampling_params)
        traj = self.get(sid)
        if len(messages) < traj.num_messages:
            raise MessageValidationError("the request holds fewer messages than the session: a session only moves forward")
        if getattr(self, "tito", None) is not None:
            return self._chat_tito(traj, messages, sampling_params)
        full = self._render(messages, add_generation_prompt=True)
        seen = self._rendered[sid]
        if not full.startswith(seen):
            raise MessageValidationError("the conversation does not extend the session's history (token-in-token-out would break)")
        delta = full[len(seen):]
        new_ids = self._encode(delta)
        if new_ids:
            role = messages[-1]["role"] if messages else "user"
            traj.append_context(role, new_ids)
        out = self.generate(list(traj.tokens), dict(sampling_params))
        ids = list(out["output_ids"])
        lps = [float(x[0]) if isinstance(x, (list, tuple)) else float(x) for x in out.get("output_token_logprobs", [0.0] * len(ids))]
        traj.append_generation(ids, lps, out.get("weight_version"), out.get("finish_reason"))
        text = self.tok.decode(ids, skip_special_tokens=True) if hasattr(self.tok, "decode") else ""
        # what the next request will contain for this turn is the assistant message as text; remember the rendering
        # of the history *with* the sampled ids decoded exactly, so that the next delta starts after them
        self._rendered[sid] = full + (self.tok.decode(ids, skip_special_tokens=False) if hasattr(self.tok, "decode") else "")
        traj.num_messages = len(messages) + 1
        return {"text": text, "ids": ids, "finish_reason": out.get("finish_reason", "stop")}


def build_session_app(store: SessionStore, model_name: str = "policy", created_only: bool = False):
    """``created_only``: chat requests are accepted only for sessions made with ``POST /sessions`` (default: a session
    comes into being with its first request, which agent frameworks that pick their own ids rely on)."""
    from fastapi import FastAPI, HTTPException, Request

    app = FastAPI(title="miles_b200 session server")

    from .errors import MessageValidationError, SessionError, SessionNotFoundError, UpstreamResponseError

    async def _chat(sid: str, req: Request):
        import json as _json

        from fastapi.responses import StreamingResponse

        body = await req.json()
        messages = body.get("messages")
        if not isinstance(messages, list) or not all(isinstance(m, dict) and "role" in m for m in messages):
            raise HTTPException(MessageValidationError.status_code, "messages must be a list of {role, content} objects")
        if created_only and sid not in store.sessions and sid not in store._trees:
            raise HTTPException(SessionNotFoundError.status_code, f"unknown session {sid}: create it with POST /sessions")
        sp = {"temperature": body.get("temperature", 1.0), "top_p": body.get("top_p", 1.0),
              "max_new_tokens": body.get("max_tokens") or body.get("max_completion_tokens") or 1024}
        if body.get("stop"):
            sp["stop"] = body["stop"]
        try:
            out = store.chat(sid, messages, sp)
        except SessionError as e:
            raise HTTPException(e.status_code, str(e))
        except ValueError as e:
            raise HTTPException(409, str(e))
        except KeyError as e:
            raise HTTPException(UpstreamResponseError.status_code, f"the engine's answer lacks {e}")
        except RuntimeError as e:
            raise HTTPException(503, str(e))
        fr = out["finish_reason"]
        fr = fr.get("type") if isinstance(fr, dict) else fr
        fr = "length" if fr == "length" else "stop"
        cid, now, model = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time()), body.get("model", model_name)
        if body.get("stream"):
            # server-sent events for clients that only speak the streaming protocol: the turn is generated whole (the
            # trajectory needs its exact tokens) and sent as one content chunk, a final chunk and [DONE]
            def events():
                first = {"id": cid, "object": "chat.completion.chunk", "created": now, "model": model,
                         "choices": [{"index": 0, "delta": {"role": "assistant", "content": out["text"]}, "finish_reason": None}]}
                last = {"id": cid, "object": "chat.completion.chunk", "created": now, "model": model,
                        "choices": [{"index": 0, "delta": {}, "finish_reason": fr}], "usage": {"completion_tokens": len(out["ids"])}}
                yield "data: " + _json.dumps(first) + "\n\n"
                yield "data: " + _json.dumps(last) + "\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(events(), media_type="text/event-stream")
        return {"id": cid, "object": "chat.completion", "created": now, "model": model,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": out["text"]}, "finish_reason": fr}],
                "usage": {"completion_tokens": len(out["ids"])}}

    app.post("/sessions/{sid}/v1/chat/completions")(_chat)

    @app.get("/health")
    async def health():
        return {"status": "ok", "sessions": len(store.sessions) + len(store._trees), "mode": "tree" if store.tree else "linear"}

    @app.post("/sessions")
    async def create_session():
        sid = uuid.uuid4().hex
        if store.tree:
            store._lineage.setdefault(sid, [])
        else:
            store.get(sid)
        return {"session_id": sid}

    def _meta(sid: str) -> dict:
        if store.tree:
            tree = store._trees.get(sid)
            if tree is None and sid not in store._lineage:
                raise HTTPException(SessionNotFoundError.status_code, f"unknown session {sid}")
            leaves = tree.to_sample_dicts() if tree is not None else []
            return {"session_id": sid, "mode": "tree", "num_leaves": len(leaves), "num_requests": len(store._lineage.get(sid, [])),
                    "num_tokens": max((len(l["tokens"]) for l in leaves), default=0)}
        t = store.sessions.get(sid)
        if t is None:
            raise HTTPException(SessionNotFoundError.status_code, f"unknown session {sid}")
        return {"session_id": sid, "mode": "linear", "num_messages": t.num_messages, "num_tokens": len(t.tokens),
                "num_turns": len(t.turns), "prompt_tokens": t.prompt_length, "finish_reason": t.finish_reason,
                "weight_versions": list(t.weight_versions)}

    @app.get("/sessions/{sid}")
    async def get_session(sid: str):
        return _meta(sid)

    @app.get("/sessions/{sid}/verify")
    async def verify(sid: str):
        """Token-level sessions: compare the incremental trajectory with a fresh rendering of the conversation, difference
        by difference (session/compare.py). ``ok`` is false when anything but assistant text differs."""
        t = store.sessions.get(sid)
        if t is None:
            raise HTTPException(SessionNotFoundError.status_code, f"unknown session {sid}")
        if store.tito is None or not getattr(t, "messages", None):
            return {"session_id": sid, "checked": False, "ok": True, "mismatches": []}
        # the fresh rendering ends with a generation header the trajectory does not have yet: compare up to the last turn
        found = store.tito.diagnose(list(t.tokens) + store.tito.boundary_fix(t.tokens[t.turns[-1].start:t.turns[-1].end])
                                    + store.tito.header_ids("assistant"), t.messages)
        return {"session_id": sid, "checked": True, "ok": not any(m.severe for m in found), "mismatches": [m.to_dict() for m in found]}

    @app.get("/sessions/{sid}/samples")
    async def collect_samples(sid: str, max_seq_len: Optional[int] = None):
        """The session's training samples; a sample longer than ``max_seq_len`` tokens is cut there and marked truncated."""
        _meta(sid)
        out = []
        for smp in store.samples(sid):
            if max_seq_len is not None and len(smp["tokens"]) > max_seq_len:
                cut = len(smp["tokens"]) - max_seq_len
                keep = max(smp["response_length"] - cut, 0)
                smp = dict(smp, tokens=smp["tokens"][:max_seq_len], response_length=keep, loss_mask=smp["loss_mask"][:keep],
                           rollout_log_probs=smp["rollout_log_probs"][:keep], status="truncated")
            out.append(smp)
        return {"session_id": sid, "samples": out}

    @app.get("/sessions/{sid}/sample")
    async def sample(sid: str):
        if store.tree:
            out = store.samples(sid)
            if not out:
                raise HTTPException(404, "unknown session")
            return {"samples": out}
        if sid not in store.sessions:
            raise HTTPException(404, "unknown session")
        return store.sessions[sid].to_sample_dict()

    @app.delete("/sessions/{sid}")
    async def close(sid: str):
        t = store.close(sid)
        if t is None:
            raise HTTPException(404, "unknown session")
        return t.to_sample_dict()

    return app


def start_session_servers(args, tokenizer, generate: Callable) -> list:
    """``--use-session-server [v1|v2]``: start the standalone session server(s) the agent frameworks of a rollout talk
    to and return their base URLs. ``--session-server-ip`` (default 127.0.0.1), ``--session-server-port`` (one port, or
    ``start end`` for one server per port of the half-open range; a free port if absent), ``--tito-model`` (token-level
    continuation rules of a model family; ``default`` renders through the tokenizer's own chat template, which
    ``--chat-template-path`` replaces by a Jinja file), ``--session-message-matcher`` and, for v2, the picker /
    post-processor hooks."""
    import socket
    import threading

    import uvicorn

    from ...utils.misc import load_function
    from .hooks import resolve_matcher

    mode = getattr(args, "use_session_server", False)
    if not mode:
        return []
    tree = str(mode).lower() == "v2"
    path = getattr(args, "chat_template_path", None)
    if path and tokenizer is not None:
        tokenizer.chat_template = open(path).read()
    family = getattr(args, "tito_model", "default")
    fix = lambda p: p.replace("miles.rollout.session.v2.picker_hub", "miles_b200.rollout.session.hooks") \
        .replace("miles.rollout.session.v2.postprocessor_hub", "miles_b200.rollout.session.hooks")
    picker = load_function(fix(args.session_sample_picker_path)) if tree and getattr(args, "session_sample_picker_path", None) else None
    post = load_function(fix(args.session_sample_postprocessor_path)) if tree and getattr(args, "session_sample_postprocessor_path", None) else None
    ports = getattr(args, "session_server_port", None)
    if isinstance(ports, int):
        ports = [ports]
    if not ports:
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports = [s.getsockname()[1]]
    elif len(ports) == 2:
        ports = list(range(ports[0], ports[1]))
    ip = getattr(args, "session_server_ip", None) or "127.0.0.1"
    urls = []
    for port in ports:
        store = SessionStore(tokenizer, generate, tito=family != "default" and not tree, family=None if family == "default" else family,
                             tree=tree, matcher=resolve_matcher(getattr(args, "session_message_matcher", "strict")),
                             picker=picker, postprocessor=post)
        server = uvicorn.Server(uvicorn.Config(build_session_app(store), host=ip, port=port, log_level="warning"))
        threading.Thread(target=server.run, name=f"session-server-{port}", daemon=True).start()
        urls.append(f"http://{ip}:{port}")
    return urls

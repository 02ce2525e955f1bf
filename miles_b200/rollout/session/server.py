"""OpenAI-compatible session proxy: ``POST /sessions/{id}/v1/chat/completions`` keeps the exact token sequence of
an agent conversation across turns (token in, token out) and ``GET /sessions/{id}/sample`` returns the assembled
training sample (tokens, loss mask, rollout log-probs).

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
            raise ValueError("the request holds fewer messages than the session: a session only moves forward")
        if getattr(self, "tito", None) is not None:
            return self._chat_tito(traj, messages, sampling_params)
        full = self._render(messages, add_generation_prompt=True)
        seen = self._rendered[sid]
        if not full.startswith(seen):
            raise ValueError("the conversation does not extend the session's history (token-in-token-out would break)")
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


def build_session_app(store: SessionStore, model_name: str = "policy"):
    from fastapi import FastAPI, HTTPException, Request

    app = FastAPI(title="miles_b200 session server")

    async def _chat(sid: str, req: Request):
        body = await req.json()
        sp = {"temperature": body.get("temperature", 1.0), "top_p": body.get("top_p", 1.0),
              "max_new_tokens": body.get("max_tokens") or body.get("max_completion_tokens") or 1024}
        if body.get("stop"):
            sp["stop"] = body["stop"]
        try:
            out = store.chat(sid, body.get("messages", []), sp)
        except ValueError as e:
            raise HTTPException(409, str(e))
        except RuntimeError as e:
            raise HTTPException(503, str(e))
        fr = out["finish_reason"]
        fr = fr.get("type") if isinstance(fr, dict) else fr
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:24], "object": "chat.completion", "created": int(time.time()),
                "model": body.get("model", model_name),
                "choices": [{"index": 0, "message": {"role": "assistant", "content": out["text"]},
                             "finish_reason": "length" if fr == "length" else "stop"}],
                "usage": {"completion_tokens": len(out["ids"])}}

    app.post("/sessions/{sid}/v1/chat/completions")(_chat)

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

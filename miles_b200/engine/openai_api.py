"""OpenAI-compatible endpoints of an engine server: ``/v1/models``, ``/v1/completions``, ``/v1/chat/completions``.

Evaluation harnesses and agent frameworks speak this protocol; the training loop itself uses ``/generate`` (token in, token
out, log-probs, routed experts). A chat request is rendered with the tokenizer's chat template (tools included), generated
through the same client as ``/generate`` and answered in the protocol's JSON; ``logprobs`` returns the sampled tokens'
log-probs, ``n`` > 1 draws several samples. Streaming answers are sent as one server-sent event carrying the whole message
followed by ``[DONE]``: the engine returns finished requests, not partial ones.

Reference: the OpenAI surface of the engines the reference launches (used by examples/experimental/*/eval_*_via_api.py and
by miles/rollout/session/server.py as upstream).
"""
import json
import time
import uuid


def _sampling(body: dict) -> dict:
    sp = {"max_new_tokens": int(body.get("max_tokens") or body.get("max_completion_tokens") or 256),
          "temperature": float(body.get("temperature", 1.0)), "top_p": float(body.get("top_p", 1.0))}
    if body.get("top_k") is not None:
        sp["top_k"] = int(body["top_k"])
    if body.get("seed") is not None:
        sp["sampling_seed"] = int(body["seed"])
    stop = body.get("stop_token_ids")
    if stop:
        sp["stop_token_ids"] = [int(t) for t in stop]
    return sp


def _finish(out: dict) -> str:
    fr = (out.get("meta_info") or {}).get("finish_reason") or {}
    kind = fr.get("type") if isinstance(fr, dict) else fr
    return "length" if kind == "length" else "stop"


def register_openai(app, client, tokenizer, model_name: str) -> None:
    from fastapi import HTTPException, Request
    from fastapi.responses import JSONResponse, StreamingResponse

    def need_tokenizer():
        if tokenizer is None:
            raise HTTPException(400, "this engine was started without a tokenizer (--hf-checkpoint): use /generate with input_ids")

    def decode(ids) -> str:
        return tokenizer.decode(list(ids), skip_special_tokens=True)

    async def run(input_ids: list, body: dict) -> list:
        n = max(1, int(body.get("n", 1) or 1))
        sp = _sampling(body)
        outs = []
        for k in range(n):
            spk = dict(sp)
            if n > 1 and "sampling_seed" in spk:
                spk["sampling_seed"] += k
            outs.append(await client.generate({"input_ids": list(input_ids), "sampling_params": spk, "return_logprob": True}))
        return outs

    def usage(input_ids, outs) -> dict:
        c = sum(len(o["output_ids"]) for o in outs)
        return {"prompt_tokens": len(input_ids), "completion_tokens": c, "total_tokens": len(input_ids) + c}

    def logprobs(o: dict, want: bool):
        if not want:
            return None
        lps = (o.get("meta_info") or {}).get("output_token_logprobs") or []
        return {"content": [{"token": decode([t]), "logprob": float(lp[0] if isinstance(lp, (list, tuple)) else lp)}
                            for t, lp in zip(o["output_ids"], lps)]}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "miles_b200"}]}

    @app.post("/v1/completions")
    async def completions(req: Request):
        body = await req.json()
        prompt = body.get("prompt")
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            ids = [int(t) for t in prompt]
        else:
            need_tokenizer()
            ids = tokenizer(prompt if isinstance(prompt, str) else "".join(prompt or []), add_special_tokens=False)["input_ids"]
        outs = await run(ids, body)
        text = (lambda o: decode(o["output_ids"])) if tokenizer is not None else (lambda o: "")
        return JSONResponse({"id": f"cmpl-{uuid.uuid4().hex[:24]}", "object": "text_completion", "created": int(time.time()),
                             "model": model_name, "usage": usage(ids, outs),
                             "choices": [{"index": i, "text": text(o), "token_ids": o["output_ids"], "finish_reason": _finish(o),
                                          "logprobs": logprobs(o, bool(body.get("logprobs"))) if tokenizer is not None else None}
                                         for i, o in enumerate(outs)]})

    @app.post("/v1/chat/completions")
    async def chat(req: Request):
        need_tokenizer()
        body = await req.json()
        messages = body.get("messages") or []
        if not messages:
            raise HTTPException(400, "messages is required")
        kw = {"tools": body["tools"]} if body.get("tools") else {}
        if getattr(tokenizer, "chat_template", None) and hasattr(tokenizer, "apply_chat_template"):
            text = tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=True, **kw)
        else:
            text = "".join(f"<|{m['role']}|>{m.get('content') or ''}<|end|>" for m in messages) + "<|assistant|>"
        ids = tokenizer(text, add_special_tokens=False)["input_ids"]
        outs = await run(ids, body)
        rid = f"chatcmpl-{uuid.uuid4().hex[:24]}"
        choices = [{"index": i, "message": {"role": "assistant", "content": decode(o["output_ids"])}, "finish_reason": _finish(o),
                    "logprobs": logprobs(o, bool(body.get("logprobs")))} for i, o in enumerate(outs)]
        payload = {"id": rid, "object": "chat.completion", "created": int(time.time()), "model": model_name, "choices": choices,
                   "usage": usage(ids, outs)}
        if not body.get("stream"):
            return JSONResponse(payload)

        def events():
            chunk = dict(payload, object="chat.completion.chunk",
                         choices=[{"index": c["index"], "delta": c["message"], "finish_reason": c["finish_reason"]} for c in choices])
            yield f"data: {json.dumps(chunk)}\n\n"
            yield "data: [DONE]\n\n"

        return StreamingResponse(events(), media_type="text/event-stream")

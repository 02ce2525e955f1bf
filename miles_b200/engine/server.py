"""HTTP front of an in-process engine: the endpoint set the reference drives on its SGLang servers
(miles/backends/sglang_utils/sglang_engine.py:126-693).

``/generate`` (token-in/token-out, log-probs, routed experts), ``/health``, ``/health_generate``,
``/flush_cache``, ``/abort_request``, ``/pause_generation``, ``/continue_generation``,
``/begin_weight_update``, ``/update_weights_from_tensor`` (flat buckets, in-process handle),
``/update_weights_from_disk``, ``/update_weight_version``, ``/end_weight_update``, ``/get_weight_version``,
``/model_info``, ``/server_info``, ``/release_memory_occupation``, ``/resume_memory_occupation``,
``/weights_checker``, ``/metrics``, ``/export_prefix`` / ``/import_prefix`` (prefill / decode hand-over) and the OpenAI-compatible
``/v1/*`` endpoints (``openai_api.py``).  The engine loop runs as an asyncio task of the same process, so the
server needs no scheduler or detokenizer subprocesses.
"""
import time

from .client import EngineClient
from .core import Engine


def build_app(engine: Engine, tokenizer=None, model_path: str = ""):
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse, PlainTextResponse

    app = FastAPI(title="miles_b200 engine")
    client = EngineClient([engine], tokenizer)
    snapshot: dict = {}
    started = time.time()

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/health_generate")
    async def health_generate():
        if engine.kv_cache is None or engine.paused:
            return {"status": "paused"}
        out = await client.generate({"input_ids": [0], "sampling_params": {"max_new_tokens": 1, "temperature": 0.0}})
        return {"status": "ok", "tokens": len(out["output_ids"])}

    @app.post("/generate")
    async def generate(req: Request):
        payload = await req.json()
        if "input_ids" not in payload and "text" not in payload:
            raise HTTPException(400, "input_ids or text is required")
        try:
            out = await client.generate(payload)
        except ValueError as e:  # a sampling parameter this engine does not implement: the caller's mistake, not a crash
            raise HTTPException(400, str(e))
        if not payload.get("return_logprob", True):
            out["meta_info"].pop("output_token_logprobs", None)
        return JSONResponse(out)

    @app.api_route("/flush_cache", methods=["GET", "POST"])
    async def flush_cache():
        return {"success": engine.flush_cache()}

    @app.post("/abort_request")
    async def abort_request(req: Request):
        body = await req.json()
        n = engine.abort_request(body.get("rid"), abort_all=bool(body.get("abort_all")))
        for r in engine.pop_finished():
            client._resolve(r)
        return {"aborted": n}

    @app.post("/pause_generation")
    async def pause_generation(req: Request):
        body = await req.json() if await req.body() else {}
        client.pause_generation(body.get("mode", "retract"))
        return {"success": True}

    @app.post("/continue_generation")
    async def continue_generation():
        client.continue_generation()
        return {"success": True}

    @app.post("/begin_weight_update")
    async def begin_weight_update(req: Request):
        snapshot["updating"] = True
        return {"success": True}

    @app.post("/update_weights_from_tensor")
    async def update_weights_from_tensor(req: Request):
        """In-process transport: the body names a registry key under which the trainer left flat buckets."""
        body = await req.json()
        from ..weight_sync.registry import take_bucket

        n = 0
        from ..models.hf_mapping import param_or_hf_view

        for name, tensor in take_bucket(body["bucket_id"]):
            dst = param_or_hf_view(engine.cfg, engine.store, name)  # native or HuggingFace tensor name
            dst.copy_(tensor.to(dst.dtype))
            n += 1
        if body.get("weight_version") is not None:
            engine.update_weight_version(body["weight_version"])
        return {"success": True, "num_tensors": n}

    @app.post("/update_weights_from_disk")
    async def update_weights_from_disk(req: Request):
        body = await req.json()
        from ..checkpoint import load_hf

        n = load_hf(engine.cfg, engine.store, body["model_path"], strict=False)
        if body.get("weight_version") is not None:
            engine.update_weight_version(body["weight_version"])
        return {"success": True, "num_tensors": n}

    @app.post("/update_weight_version")
    async def update_weight_version(req: Request):
        body = await req.json()
        return {"weight_version": engine.update_weight_version(body.get("new_version", body.get("weight_version")))}

    @app.post("/end_weight_update")
    async def end_weight_update():
        snapshot.pop("updating", None)
        return {"success": True}

    @app.get("/get_weight_version")
    async def get_weight_version():
        return {"weight_version": engine.weight_version}

    @app.get("/model_info")
    async def model_info():
        return {"model_path": model_path, "weight_version": engine.weight_version, "is_generation": True}

    @app.get("/server_info")
    async def server_info():
        return {"uptime_s": time.time() - started, "num_pages": engine.num_pages, "page_size": engine.page_size,
                "max_running_requests": engine.max_running, "stats": engine.stats, "free_pages": engine.pool.num_free}

    @app.post("/release_memory_occupation")
    async def release_memory_occupation(req: Request):
        body = await req.json() if await req.body() else {}
        engine.release_memory_occupation(tuple(body.get("tags") or ("kv_cache", "cuda_graph")))
        return {"success": True}

    @app.post("/resume_memory_occupation")
    async def resume_memory_occupation(req: Request):
        body = await req.json() if await req.body() else {}
        engine.resume_memory_occupation(tuple(body.get("tags") or ("kv_cache",)))
        return {"success": True}

    @app.post("/weights_checker")
    async def weights_checker(req: Request):
        body = await req.json()
        action = body.get("action")
        if action == "snapshot":
            snapshot["flat"] = {g: t.clone() for g, t in engine.store.flat.items()}
            return {"success": True}
        if action == "reset_tensors":
            for t in engine.store.flat.values():
                t.zero_()
            return {"success": True}
        if action == "compare":
            ok = all((engine.store.flat[g] == t).all().item() for g, t in snapshot.get("flat", {}).items())
            return {"success": bool(ok)}
        if action == "checksum":
            return {"success": True, "checksum": engine.store.checksum()}
        raise HTTPException(400, f"unknown action {action!r}")

    from .server_extra import register_extra

    register_extra(app, engine, snapshot)
    from .openai_api import register_openai

    register_openai(app, client, tokenizer, model_path or "policy")

    @app.get("/metrics")
    async def metrics():
        s = engine.stats
        lines = [f"miles_b200:num_running_reqs {len(engine.running)}", f"miles_b200:num_queue_reqs {len(engine.waiting)}",
                 f"miles_b200:prefill_tokens_total {s['prefill_tokens']}", f"miles_b200:decode_tokens_total {s['decode_tokens']}",
                 f"miles_b200:token_usage {1.0 - engine.pool.num_free / max(engine.num_pages - 1, 1):.6f}",
                 f"miles_b200:weight_version {engine.weight_version}"]
        return PlainTextResponse("\n".join(lines) + "\n")

    return app


def serve(engine: Engine, host: str = "127.0.0.1", port: int = 30000, tokenizer=None, model_path: str = "") -> None:
    import uvicorn

    uvicorn.run(build_app(engine, tokenizer, model_path), host=host, port=port, log_level="warning")


def main(argv=None) -> None:
    """``python -m miles_b200.engine.server --model-preset qwen3-4B --port 30000``: one engine process on this GPU
    (or on the CPU with the PyTorch model), ready to be driven over HTTP and to join a trainer's weight-update group."""
    import argparse

    import torch

    from ..models import ParamStore, build_model, get_config

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--model-preset", default=None)
    ap.add_argument("--hf-checkpoint", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=30000)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--max-running-requests", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--context-length", type=int, default=9224)
    ap.add_argument("--mem-fraction-static", type=float, default=0.85)
    ap.add_argument("--quantization", default="none", choices=["none", "mxfp8", "nvfp4"])
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--disable-radix-cache", action="store_true", help="turn the prefix (radix) cache off")
    ns = ap.parse_args(argv)
    cfg = get_config(ns.model_preset or ns.hf_checkpoint)
    on_gpu = ns.device.startswith("cuda")
    dtype = torch.bfloat16 if on_gpu else torch.float32
    store = ParamStore(cfg, ns.device, dtype, seed=ns.seed)
    tokenizer = None
    if ns.hf_checkpoint:
        from ..checkpoint import load_hf
        from ..utils.processing_utils import load_tokenizer

        load_hf(cfg, store, ns.hf_checkpoint)
        tokenizer = load_tokenizer(ns.hf_checkpoint)
    model = build_model(cfg, store, "b200" if (on_gpu and cfg.head_dim == 128) else "torch")
    if ns.quantization != "none" and hasattr(model, "enable_block_scaled"):
        model.enable_block_scaled(ns.quantization)
    kv_bytes = None
    if on_gpu:
        free, total = torch.cuda.mem_get_info()
        kv_bytes = max(int(free - (1.0 - ns.mem_fraction_static) * total), 1 << 28)
    engine = Engine(model, max_running=ns.max_running_requests, page_size=ns.page_size, max_seq_len=ns.context_length,
                    kv_mem_bytes=kv_bytes, use_cuda_graph=on_gpu, eos_token_id=getattr(tokenizer, "eos_token_id", None),
                    prefix_cache=not ns.disable_radix_cache, memory_saver=on_gpu)
    engine.seed_salt = ns.seed * 1000003 + ns.port  # engines of one fleet share --seed and differ by port
    serve(engine, ns.host, ns.port, tokenizer, ns.hf_checkpoint or ns.model_preset or "")


if __name__ == "__main__":
    main()

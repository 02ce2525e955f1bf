"""Further endpoints of the engine's HTTP surface: weight-update process groups, LoRA adapters, profiling and the
parallel layout (reference: miles/backends/sglang_utils/sglang_engine.py:126-693)."""
import asyncio
import os
import threading
import time


def register_extra(app, engine, state: dict) -> None:
    from fastapi import HTTPException, Request

    @app.post("/init_weights_update_group")
    async def init_weights_update_group(req: Request):
        b = await req.json()
        from ..weight_sync.broadcast import init_update_group

        # blocking rendezvous with the trainer: run it off the event loop
        await asyncio.to_thread(init_update_group, b["master_address"], int(b["master_port"]), int(b["rank_offset"]),
                                int(b["world_size"]), b["group_name"], b.get("backend", "nccl"))
        return {"success": True, "message": f"joined {b['group_name']} as rank {b['rank_offset']}"}

    @app.post("/destroy_weights_update_group")
    async def destroy_weights_update_group(req: Request):
        b = await req.json()
        from ..weight_sync.broadcast import destroy_update_group

        return {"success": destroy_update_group(b["group_name"])}

    @app.post("/update_weights_from_distributed")
    async def update_weights_from_distributed(req: Request):
        b = await req.json()
        from ..weight_sync.broadcast import receive_bucket

        n = await asyncio.to_thread(receive_bucket, b, engine.store)
        if b.get("weight_version") is not None:
            engine.update_weight_version(b["weight_version"])
        return {"success": True, "num_tensors": n}

    @app.post("/pull_weights")
    async def pull_weights(req: Request):
        """Apply the delta files of a published version directory to this engine's weights."""
        b = await req.json()
        from ..weight_sync.disk_delta import apply_delta_dir

        n = await asyncio.to_thread(apply_delta_dir, engine.store, b["path"])
        if b.get("weight_version") is not None:
            engine.update_weight_version(b["weight_version"])
        return {"success": True, "num_tensors": n}

    @app.post("/requantize_weights")
    async def requantize_weights(req: Request):
        """Serve the projections and experts from block-scaled copies (``mxfp8`` / ``nvfp4``) of the weights the engine
        holds now; called by the trainer after a weight update when ``--weight-sync-quant`` is set."""
        b = await req.json()
        fmt = b.get("format", "none")
        fn = getattr(engine.model, "enable_block_scaled", None)
        if fmt in ("mxfp8", "nvfp4") and fn is not None:
            return {"success": True, "num_tensors": await asyncio.to_thread(fn, fmt)}
        return {"success": False, "reason": f"format {fmt!r} is not served by this engine"}

    @app.get("/parallelism_config")
    async def parallelism_config():
        st = engine.store
        return {"tp_size": getattr(st, "tp_size", 1), "ep_size": getattr(st, "ep_size", 1), "pp_size": getattr(st, "pp_size", 1),
                "dp_size": 1, "tp_rank": getattr(st, "tp_rank", 0), "ep_rank": getattr(st, "ep_rank", 0)}

    # ------------------------------------------------------------------ LoRA adapters
    @app.post("/load_lora_adapter_from_tensors")
    async def load_lora_adapter_from_tensors(req: Request):
        """The adapter arrives through the in-process bucket registry as (name, tensor) pairs in PEFT naming; it is
        merged into the engine's weights (and remembered so that it can be taken out again)."""
        b = await req.json()
        from ..lora import merge_adapter_into
        from ..weight_sync.registry import take_bucket

        name = b["lora_name"]
        if name in state.setdefault("adapters", {}):
            raise HTTPException(409, f"adapter {name!r} is already loaded")
        tensors = dict(take_bucket(b["bucket_id"]))
        scale = float(b.get("scaling", 1.0))
        merge_adapter_into(engine.store, tensors, scale)
        state["adapters"][name] = (tensors, scale)
        return {"success": True, "loaded_adapters": sorted(state["adapters"])}

    @app.post("/unload_lora_adapter")
    async def unload_lora_adapter(req: Request):
        b = await req.json()
        from ..lora import merge_adapter_into

        ad = state.setdefault("adapters", {}).pop(b["lora_name"], None)
        if ad is None:
            raise HTTPException(404, f"adapter {b['lora_name']!r} is not loaded")
        merge_adapter_into(engine.store, ad[0], -ad[1])
        return {"success": True, "loaded_adapters": sorted(state["adapters"])}

    # ------------------------------------------------------------------ profiling
    @app.post("/export_prefix")
    async def export_prefix(req: Request):
        """Prefill / decode disaggregation: the cached keys / values of the longest cached prefix of ``input_ids`` as one
        binary message (engine/pd.py)."""
        from fastapi.responses import Response

        from .pd import pack_blob

        body = await req.json()
        return Response(content=pack_blob(engine.export_prefix(body["input_ids"])), media_type="application/octet-stream")

    @app.post("/import_prefix")
    async def import_prefix(req: Request):
        from .pd import unpack_blob

        return {"cached_tokens": engine.import_prefix(unpack_blob(await req.body()))}

    @app.post("/start_profile")
    async def start_profile(req: Request):
        b = await req.json() if await req.body() else {}
        if state.get("profiler") is not None:
            raise HTTPException(409, "a profile is already running")
        import torch

        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available() and "GPU" in (b.get("activities") or ["CPU", "GPU"]):
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        out_dir = b.get("output_dir") or "/tmp"
        stop, box = threading.Event(), {}

        def run():  # the profiler is bound to the thread that starts it: one thread owns its whole life
            t0 = time.time()
            with torch.profiler.profile(activities=acts, record_shapes=bool(b.get("record_shapes", False)),
                                        with_stack=bool(b.get("with_stack", False))) as prof:
                stop.wait()
            os.makedirs(out_dir, exist_ok=True)
            box["trace"] = os.path.join(out_dir, f"engine_trace_{int(t0)}.json")
            prof.export_chrome_trace(box["trace"])

        th = threading.Thread(target=run, daemon=True)
        th.start()
        state["profiler"] = (th, stop, box)
        return {"success": True}

    @app.post("/stop_profile")
    async def stop_profile():
        p = state.pop("profiler", None)
        if p is None:
            raise HTTPException(409, "no profile is running")
        th, stop, box = p
        stop.set()
        await asyncio.to_thread(th.join)
        path = box.get("trace")
        return {"success": True, "trace": path}

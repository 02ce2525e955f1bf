"""Small utilities: HTTP retries, FLOP counts / MFU, eval config overlay, lifecycle sinks."""
import asyncio

import pytest

from miles_b200.models import get_config
from miles_b200.utils import http_utils, lifecycle
from miles_b200.utils.eval_config import build_eval_configs
from miles_b200.utils.metric_utils import device_peak_tflops, forward_flops, mfu, train_step_flops


def test_http_retries_then_succeeds_and_gives_up_on_client_errors():
    calls = []

    async def flaky(method, url, payload):
        calls.append(url)
        return (503, None) if len(calls) < 3 else (200, {"ok": True})

    out = asyncio.run(http_utils.post("http://x/generate", {"a": 1}, base_delay=0.001, transport=flaky))
    assert out == {"ok": True} and len(calls) == 3

    async def bad(method, url, payload):
        return 404, {"detail": "nope"}

    with pytest.raises(ValueError):
        asyncio.run(http_utils.get("http://x/missing", base_delay=0.001, transport=bad))

    async def down(method, url, payload):
        raise ConnectionError("refused")

    with pytest.raises(ConnectionError):
        asyncio.run(http_utils.get("http://x/", max_retries=2, base_delay=0.001, transport=down))


def test_flops_of_moe_counts_active_experts_only():
    cfg = get_config("qwen3-30B-A3B")
    f = forward_flops(cfg, [1024])
    # ~2 * active parameters per token, plus attention
    assert 0.9 < f / (2.0 * cfg.num_active_params() * 1024) < 1.3
    assert train_step_flops(cfg, [1024]) == pytest.approx(5 * f)
    assert device_peak_tflops("NVIDIA B200") == 2250.0
    assert mfu(2250e12, 1.0, 1, 2250.0) == pytest.approx(1.0)


def test_eval_config_overlay(tmp_path):
    y = tmp_path / "eval.yaml"
    y.write_text("defaults:\n  temperature: 0.6\ndatasets:\n  - name: aime\n    n_samples_per_eval_prompt: 16\n    max_response_len: 4096\n"
                 "  - name: gpqa\n    path: /data/gpqa.jsonl\n    rm_type: gpqa\n    judge: strict\n")

    class A:
        eval_prompt_data = ["aime", "/data/aime.jsonl"]
        n_samples_per_eval_prompt = 1
        eval_config = str(y)
        rollout_temperature = 1.0
        rollout_max_response_len = 1024
        eval_temperature = eval_top_p = eval_top_k = eval_max_response_len = rollout_top_p = rollout_top_k = None

    cfgs = {c.name: c for c in build_eval_configs(A())}
    assert cfgs["aime"].path == "/data/aime.jsonl" and cfgs["aime"].n_samples_per_eval_prompt == 16
    assert cfgs["aime"].sampling_params(A())["temperature"] == 0.6 and cfgs["aime"].sampling_params(A())["max_new_tokens"] == 4096
    assert cfgs["gpqa"].rm_type == "gpqa" and cfgs["gpqa"].metadata_overrides == {"judge": "strict"}


def test_lifecycle_sinks_do_not_raise():
    seen = []
    lifecycle.clear_sinks()
    lifecycle.add_sink(seen.append)
    lifecycle.add_sink(lambda rec: 1 / 0)
    lifecycle.attempt_start(3, group=1)
    lifecycle.attempt_end(3, status="completed")
    assert [r["event"] for r in seen] == ["attempt_start", "attempt_end"] and seen[1]["status"] == "completed"
    lifecycle.clear_sinks()


def test_dp_schedule_keeps_rollouts_together_and_balances_ranks():
    import random

    from miles_b200.utils.dp_schedule import build_dp_schedule

    random.seed(0)
    lens = [random.randint(50, 900) for _ in range(40)]
    rids = [i // 2 for i in range(40)]  # 20 rollouts of two samples each
    s = build_dp_schedule(lens, rids, dp_size=4, global_batch_size=8, max_tokens_per_gpu=1500, balance=True,
                          allow_partial_step=True)
    assert s.num_rollouts == [8, 8, 4]
    seen = sorted(i for p in s.partitions for i in p)
    assert seen == list(range(40))  # every sample is scheduled exactly once
    # every rank has the same number of micro-batches per step, and no micro-batch exceeds the token budget
    assert all(len(m) == sum(s.num_microbatches) for m in s.micro_batches)
    for rank in range(4):
        part, mbs = s.for_rank(rank)
        for mb in mbs:
            assert sum(lens[part[j]] for j in mb) <= 1500
    # the samples of a rollout are trained in the same step
    step_of = {}
    for rank in range(4):
        part, mbs = s.for_rank(rank)
        k = 0
        for step, n in enumerate(s.num_microbatches):
            for mb in mbs[k:k + n]:
                for j in mb:
                    step_of[part[j]] = step
            k += n
    assert all(step_of[2 * r] == step_of[2 * r + 1] for r in range(20))
    # without the partial step the trailing rollouts are dropped
    s2 = build_dp_schedule(lens, rids, dp_size=4, global_batch_size=8, max_tokens_per_gpu=1500)
    assert s2.num_rollouts == [8, 8] and len({i for p in s2.partitions for i in p}) == 32
    # fixed micro-batch size must divide evenly
    import pytest

    with pytest.raises(ValueError):
        build_dp_schedule(lens[:12], list(range(12)), dp_size=4, global_batch_size=12, micro_batch_size=5)
    s3 = build_dp_schedule(lens[:16], list(range(16)), dp_size=4, global_batch_size=16, micro_batch_size=2)
    assert s3.num_microbatches == [2]


def test_deployment_plan_and_validation(tmp_path):
    from types import SimpleNamespace as NS

    import pytest
    import yaml

    from miles_b200.engine.deployment import Deployment

    spec = {"sglang": [
        {"name": "actor", "server_groups": [
            {"worker_type": "prefill", "num_gpus": 2, "num_gpus_per_engine": 1},
            {"worker_type": "decode", "num_gpus": 4, "num_gpus_per_engine": 2, "overrides": {"max_running_requests": 256}}]},
        {"name": "reward", "model_path": "/ckpt/rm", "overrides": {"mem_fraction_static": 0.5}, "server_groups": [
            {"worker_type": "placeholder", "num_gpus": 1}, {"worker_type": "regular", "num_gpus": 1}]}]}
    p = tmp_path / "dep.yaml"
    p.write_text(yaml.safe_dump(spec))
    args = NS(hf_checkpoint="/ckpt/a", rollout_num_gpus_per_engine=1)
    dep = Deployment.from_yaml(str(p)).resolve(args)
    assert dep.total_num_gpus == 8 and dep.has_pd_disaggregation
    assert dep.updatable_model().name == "actor"
    plan = dep.plan()
    assert [(e.model, e.worker_type, e.gpu_ids) for e in plan] == [
        ("actor", "prefill", [0]), ("actor", "prefill", [1]), ("actor", "decode", [2, 3]), ("actor", "decode", [4, 5]),
        ("reward", "regular", [7])]  # GPU 6 is the placeholder
    assert plan[2].overrides == {"max_running_requests": 256} and plan[-1].overrides == {"mem_fraction_static": 0.5}
    assert not plan[-1].update_weights
    with pytest.raises(ValueError):
        Deployment.from_dict({"sglang": [{"name": "a", "server_groups": [{"worker_type": "prefill", "num_gpus": 1}]}]}).resolve(args)
    with pytest.raises(ValueError):
        Deployment.from_dict({"sglang": [{"name": "a", "server_groups": [{"worker_type": "regular", "num_gpus": 3, "num_gpus_per_engine": 2}]}]}).resolve(args)
    with pytest.raises(ValueError):
        Deployment.from_dict({"sglang": [{"name": "a", "server_groups": [{"worker_type": "bogus", "num_gpus": 1}]}]})
    d2 = Deployment.from_args(NS(rollout_num_gpus=8, rollout_num_gpus_per_engine=2, prefill_num_servers=1)).resolve(args)
    assert [g.worker_type for g in d2.models[0].server_groups] == ["prefill", "decode"] and len(d2.plan()) == 4


def test_env_report_round_trip():
    from miles_b200.utils import env_report as E

    rep = E.collect()
    d = E.decode("worker log prefix " + E.encode(rep))
    assert d["python"] == rep.python and "torch" in d["packages"]
    assert E.decode("no report here") is None
    other = dict(d, python="0.0")
    assert ("python", d["python"], "0.0") in E.diff(d, other)


def test_eval_dispatcher_runs_in_background_and_skips_when_busy(tmp_path):
    import asyncio
    import os

    from miles_b200.rollout.eval_dispatch import CheckpointEvalFn, EvalDispatcher, EvalSkip, is_checkpoint_eval_fn

    class MyEval(CheckpointEvalFn):
        async def evaluate_checkpoint(self, checkpoint_dir, rollout_id):
            if rollout_id == 7:
                raise EvalSkip("no data")
            assert os.path.exists(os.path.join(checkpoint_dir, "w.bin"))
            await asyncio.sleep(0.05)
            return {"eval/score": float(rollout_id)}

    assert is_checkpoint_eval_fn(MyEval) and not is_checkpoint_eval_fn(int)

    async def export(rid, d):
        os.makedirs(d, exist_ok=True)
        open(os.path.join(d, "w.bin"), "wb").write(b"x")

    seen = []

    async def main():
        disp = EvalDispatcher(MyEval(None), export_fn=export, on_result=lambda r, m: seen.append((r, m)), overflow_policy="skip")
        assert await disp.dispatch(1, str(tmp_path / "e1"))
        assert disp.busy
        assert not await disp.dispatch(2, str(tmp_path / "e2"))          # one evaluation at a time
        assert await disp.dispatch(3, str(tmp_path / "e3"), force=True)  # waits for #1, then runs
        assert await disp.dispatch(7, str(tmp_path / "e7"), force=True)
        await disp.drain()
        return disp

    disp = asyncio.run(main())
    assert [r for r, _ in seen] == [1, 3, 7] and disp.skipped == [2]
    assert seen[0][1]["eval/score"] == 1.0 and seen[2][1]["eval/skipped"] == 1.0
    assert not os.path.exists(tmp_path / "e1")  # snapshots are removed once evaluated

    # back-pressure with two evaluations in flight and the newest snapshot kept
    seen.clear()

    async def main2():
        disp = EvalDispatcher(MyEval(None), export_fn=export, on_result=lambda r, m: seen.append((r, m)), max_in_flight=2,
                              overflow_policy="backpressure", keep_snapshots=1)
        for rid in (11, 12, 13):
            assert await disp.dispatch(rid, str(tmp_path / f"b{rid}"))   # the third waits for the first, none is dropped
        await disp.drain()
        return disp

    disp = asyncio.run(main2())
    assert sorted(r for r, _ in seen) == [11, 12, 13] and disp.skipped == []
    kept = [rid for rid in (11, 12, 13) if os.path.exists(tmp_path / f"b{rid}")]
    assert len(kept) == 1


def test_ci_checks_hashes_kl_gate_and_grad_norm(tmp_path):
    from types import SimpleNamespace as NS

    import pytest
    import torch

    from miles_b200.models import ParamStore, get_config
    from miles_b200.parallel.state import ParallelState
    from miles_b200.utils import ci_checks as C

    cfg = get_config("qwen3-tiny")
    st = ParamStore(cfg, "cpu", torch.float32, seed=1)
    h = C.model_hashes_by_layer(st)
    assert set(h) >= {"layer0000", "layer0001", "embed", "final_norm"}
    ps = ParallelState()
    args = NS(ci_test=True, ci_save_model_hash=True, ci_check_model_hash=True, save=str(tmp_path), load=str(tmp_path))
    assert C.save_model_hashes(args, st, ps, 3)
    C.check_model_hashes(args, st, ps, 3)
    st.params["layers.1.ln1.weight"][0] += 1
    with pytest.raises(AssertionError) as e:
        C.check_model_hashes(args, st, ps, 3)
    assert "layer0001" in str(e.value)
    C.check_first_step_kl(args, {"train/ppo_kl": 0.0, "train/pg_clipfrac": 0.0}, 0, 5)
    with pytest.raises(AssertionError):
        C.check_first_step_kl(args, {"train/ppo_kl": 1e-3, "train/pg_clipfrac": 0.0}, 0, 5)
    C.check_first_step_kl(args, {"train/ppo_kl": 1e-3, "train/pg_clipfrac": 0.1}, 1, 5)  # later steps may be off-policy
    a2 = NS(ci_save_grad_norm=str(tmp_path / "gn_{role}_{rollout_id}_{step_id}.pt"), ci_load_grad_norm=None)
    C.check_grad_norm(a2, 2.0, 0, 0)
    a3 = NS(ci_save_grad_norm=None, ci_load_grad_norm=a2.ci_save_grad_norm)
    C.check_grad_norm(a3, 2.03, 0, 0)
    with pytest.raises(AssertionError):
        C.check_grad_norm(a3, 2.5, 0, 0)


def test_launch_command_and_processing_helpers(capsys):
    import base64
    import io

    from miles_b200.utils.launch import TrainJob, convert_checkpoint, execute_train
    from miles_b200.utils.processing_utils import apply_chat_template, decode_image, image_to_data_url

    job = TrainJob(num_gpus=4, args=["--model-preset", "qwen3-4B", "--colocate"], master_port=29601, env={"NCCL_DEBUG": "WARN"})
    cmd = job.command()
    assert cmd[1:3] == ["-m", "torch.distributed.run"] and "--nproc-per-node=4" in cmd and cmd[-3:] == ["--model-preset", "qwen3-4B", "--colocate"]
    env = job.environment({})
    assert env["NCCL_DEBUG"] == "WARN" and env["CUDA_DEVICE_MAX_CONNECTIONS"] == "1" and env["NCCL_NVLS_ENABLE"] in ("0", "1")
    assert execute_train(job, dry_run=True) == 0 and "train.py" in capsys.readouterr().out
    assert convert_checkpoint("a", "b", "native_to_hf", dry_run=True) == 0

    class Tok:
        def apply_chat_template(self, messages, tokenize, add_generation_prompt, **kw):
            return ("T" if kw.get("tools") else "") + "|".join(m["content"] for m in messages) + (">" if add_generation_prompt else "")

    assert apply_chat_template(Tok(), [{"role": "user", "content": "hi"}], tools=[{"name": "f"}]) == "Thi>"
    from PIL import Image

    img = Image.new("RGB", (4, 3), (255, 0, 0))
    url = image_to_data_url(img)
    back = decode_image(url)
    assert back.size == (4, 3) and back.getpixel((0, 0)) == (255, 0, 0)
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    assert decode_image(buf.getvalue()).size == (4, 3)
    assert decode_image(base64.b64encode(buf.getvalue()).decode()).size == (4, 3)


def test_dp_schedule_balances_by_workload():
    import random

    from miles_b200.utils.dp_schedule import build_dp_schedule

    random.seed(1)
    lens = [random.choice([64, 128, 256, 2048, 4096]) for _ in range(32)]
    cost = lambda n: n * 1000 + n * n  # attention makes long sequences disproportionately expensive
    s = build_dp_schedule(lens, list(range(32)), dp_size=4, global_batch_size=32, max_tokens_per_gpu=8192, workload_fn=cost)
    assert sorted(i for p in s.partitions for i in p) == list(range(32))
    per_rank = [sum(cost(lens[i]) for i in p) for p in s.partitions]
    s0 = build_dp_schedule(lens, list(range(32)), dp_size=4, global_batch_size=32, max_tokens_per_gpu=8192)
    per_rank0 = [sum(cost(lens[i]) for i in p) for p in s0.partitions]
    assert max(per_rank) / min(per_rank) <= max(per_rank0) / min(per_rank0) + 1e-9
    assert all(len(m) == s.num_microbatches[0] for m in s.micro_batches)


def test_host_memory_profiler_marks_phases_and_summarises(tmp_path):
    import time

    from miles_b200.tools.host_memory_profiler import HostMemoryProfiler, main, summarize

    out = tmp_path / "mem" / "profile.csv"
    p = HostMemoryProfiler(str(out), interval=0.01).start()
    p.mark("rollout")
    blob = bytearray(32 << 20)  # something for the resident set to show
    time.sleep(0.05)
    p.mark("train")
    time.sleep(0.05)
    p.mark("rollout")
    time.sleep(0.03)
    recs = p.stop()
    del blob
    assert out.exists() and len(recs) >= 8
    s = summarize(str(out))
    assert [x["phase"] for x in s] == ["start", "rollout", "train"], "phases pooled by name, in order of first appearance"
    roll = s[1]
    assert roll["samples"] >= 4 and roll["seconds"] > 0.05 and roll["peak_process_rss_gib"] > 0.03
    assert all(x["min_available_gib"] > 0 and x["peak_used_gib"] > 0 for x in s)
    assert main([str(out)]) == 0 and main([]) == 2


def test_training_loop_writes_a_host_memory_profile(tmp_path):
    from miles_b200.loop import RLLoop
    from miles_b200.tools.host_memory_profiler import summarize
    from miles_b200.utils.arguments import parse_args

    out = tmp_path / "host.csv"
    args = parse_args(["--model-preset", "qwen3-tiny", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2",
                       "--rollout-max-response-len", "8", "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-5",
                       "--micro-batch-size", "4", "--colocate", "--num-rollout", "2", "--actor-num-gpus-per-node", "1",
                       "--profile-host-memory", str(out), "--profile-host-memory-interval", "0.01"])
    RLLoop(args).run()
    phases = [x["phase"] for x in summarize(str(out))]
    assert phases[:1] == ["start"] and {"rollout", "train", "update_weights"} <= set(phases)


def test_debug_rollout_data_tool_shows_rescoring_and_resending(tmp_path):
    import asyncio
    import io

    import torch

    from miles_b200.loop import RLLoop
    from miles_b200.tools import debug_rollout_data as D
    from miles_b200.utils.arguments import parse_args

    path = tmp_path / "rollout_{rollout_id}.pt"
    args = parse_args(["--model-preset", "qwen3-tiny", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2",
                       "--rollout-max-response-len", "8", "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-5",
                       "--micro-batch-size", "4", "--colocate", "--num-rollout", "1", "--actor-num-gpus-per-node", "1",
                       "--save-debug-rollout-data", str(path)])
    RLLoop(args).run()
    samples = D.load_samples(str(tmp_path / "rollout_0.pt"))
    assert len(samples) == 8
    buf = io.StringIO()
    summary = D.show(samples, limit=3, out=buf)
    text = buf.getvalue()
    assert text.count("--- sample ") == 3 and "reward_mean=" in text and summary["samples"] == 8 and summary["response_len_max"] <= 8
    # the same grader gives the same rewards; another grader differs somewhere
    assert asyncio.run(D.rescore(samples, rm_type="parity", out=io.StringIO())) == []
    flipped = asyncio.run(D.rescore(samples, custom_rm_path="tests.test_utils_misc._always_two", out=io.StringIO()))
    assert len(flipped) == 8 and flipped[0][2] == 2.0
    sent = []

    async def post(url, payload):
        sent.append((url, payload))
        return {"output_ids": [1, 2, 3], "text": "abc"}

    outs = asyncio.run(D.send(samples, "http://engine:1/", limit=2, max_new_tokens=5, out=io.StringIO(), post=post))
    assert len(outs) == 2 and sent[0][0] == "http://engine:1/generate" and sent[0][1]["sampling_params"]["max_new_tokens"] == 5
    n = samples[0].response_length
    assert sent[0][1]["input_ids"] == samples[0].tokens[:len(samples[0].tokens) - n], "the saved prompt tokens are sent as they were"
    assert D.main(["show", str(tmp_path / "rollout_0.pt"), "--limit", "1"]) == 0


def _always_two(args, sample, **kw):
    return 2.0


def _rebalance_worker(rank: int, world: int, port: int, out_dir: str):
    import os
    from types import SimpleNamespace as NS

    import torch
    import torch.distributed as dist

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from miles_b200.rollout.train_data import rebalance_across_dp

    # rank 0 drew long samples, rank 1 short ones; two samples per rollout (a group that must stay in one step)
    lens = [900, 800, 850, 820] if rank == 0 else [100, 120, 90, 110]
    data = {"tokens": [[rank] * n for n in lens], "total_lengths": list(lens), "response_lengths": [n // 2 for n in lens],
            "rewards": [float(rank * 10 + i) for i in range(4)], "rollout_ids": [0, 0, 1, 1], "sample_indices": [rank * 4 + i for i in range(4)],
            "num_rollouts": 2}
    args = NS(num_steps_per_rollout=1, use_dynamic_batch_size=True, max_tokens_per_gpu=2000, context_parallel_size=1, balance_by_flops=False)
    out = rebalance_across_dp(args, data, None, rank, world)
    assert len(out["tokens"]) == len(out["rewards"]) == len(out["sample_indices"]) and out["num_rollouts"] >= 1
    assert all(len(t) == n for t, n in zip(out["tokens"], out["total_lengths"])), "fields stay aligned per sample"
    torch.save({"idx": out["sample_indices"], "tok": sum(out["total_lengths"]), "before": sum(lens)}, os.path.join(out_dir, f"r{rank}.pt"))
    # too few rollouts for the ranks: the local share is kept
    small = {k: (v[:1] if isinstance(v, list) else v) for k, v in data.items()}
    assert rebalance_across_dp(NS(**{**vars(args), "num_steps_per_rollout": 4}), small, None, rank, world) is small
    dist.barrier()
    dist.destroy_process_group()


def test_balance_data_pools_and_redistributes_samples_across_ranks(tmp_path):
    import socket

    import torch
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rebalance_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "r0.pt"), torch.load(tmp_path / "r1.pt")
    assert sorted(a["idx"] + b["idx"]) == list(range(8)), "every sample trains exactly once"
    assert a["before"] == 3370 and b["before"] == 420
    assert abs(a["tok"] - b["tok"]) < 400 and a["tok"] + b["tok"] == 3790, (a["tok"], b["tok"])

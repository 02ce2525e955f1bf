"""Tiny Qwen3-arch GRPO loop on CPU: single process and gloo world size 2 (plumbing configuration):
rollout-vs-trainer log-prob parity, in-loop weight sync, gradient agreement across ranks, checkpoint resume."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from miles_b200.utils.arguments import parse_args

BASE = ["--model-preset", "qwen3-tiny", "--rollout-batch-size", "8", "--n-samples-per-prompt", "4", "--rollout-max-response-len", "16",
        "--rollout-max-prompt-len", "32", "--rm-type", "parity", "--lr", "1e-5", "--eps-clip", "0.2", "--micro-batch-size", "8",
        "--weight-decay", "0.0", "--colocate"]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_single_process_grpo_steps(tmp_path):
    from miles_b200.loop import RLLoop

    args = parse_args(BASE + ["--num-rollout", "2", "--actor-num-gpus-per-node", "1", "--save", str(tmp_path / "ckpt"), "--save-interval", "1",
                              "--check-weight-update-equal"])
    loop = RLLoop(args)
    hist = loop.run()
    assert len(hist) == 2
    for m in hist:
        assert m["train/train_rollout_logprob_abs_diff"] < 1e-5  # fp32 on both sides: parity is numerical noise
        assert abs(m["train/ppo_kl"]) < 1e-6 and m["train/pg_clipfrac"] == 0.0
        assert m["train/grad_norm"] > 0 and m["perf/step_tokens"] == 32 * (32 + 16)
    assert loop.engine.weight_version == loop.actor.store.version == 2
    assert (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").read_text() == "1"
    # resume: a new loop starts from the next rollout with identical weights
    args2 = parse_args(BASE + ["--num-rollout", "3", "--actor-num-gpus-per-node", "1", "--load", str(tmp_path / "ckpt")])
    loop2 = RLLoop(args2)
    assert loop2.start_rollout_id == 2
    for g in loop.actor.store.flat:
        assert torch.equal(loop.actor.store.flat[g], loop2.actor.store.flat[g])
    assert loop2.actor.opt.step_count == 2


def test_resume_counts_rollouts_not_optimizer_steps(tmp_path):
    """Two optimizer steps per rollout: the checkpoint written after rollout 1 holds four optimizer steps, and a
    resumed run continues at rollout 2 with the prompt stream where it stopped (not at "rollout 4")."""
    from miles_b200.loop import RLLoop

    common = BASE + ["--actor-num-gpus-per-node", "1", "--num-steps-per-rollout", "2", "--save", str(tmp_path / "ckpt"),
                     "--save-interval", "1"]
    loop = RLLoop(parse_args(common + ["--num-rollout", "2"]))
    loop.run()
    assert loop.actor.global_step == 4 and loop.actor.opt.step_count == 4
    loop2 = RLLoop(parse_args(common + ["--num-rollout", "3", "--load", str(tmp_path / "ckpt")]))
    assert loop2.start_rollout_id == 2
    assert loop2.actor.global_step == 4 and loop2.actor.opt.step_count == 4
    # the data source continues where the first run stopped: same next prompts as an uninterrupted run would draw
    ref = RLLoop(parse_args(common + ["--num-rollout", "3"]))
    for rid in range(2):
        ref.data_source.get_samples(ref.local_args.rollout_batch_size)
    a = ref.data_source.get_samples(1)
    b = loop2.data_source.get_samples(1)
    assert a[0][0].prompt == b[0][0].prompt or a[0][0].tokens == b[0][0].tokens


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)  # several ranks share the host cores
    from miles_b200.loop import RLLoop

    args = parse_args(BASE + ["--num-rollout", "2", "--actor-num-gpus-per-node", str(world), "--distributed-backend", "gloo"])
    loop = RLLoop(args)
    hist = loop.run()
    flat = torch.cat([t.flatten() for t in loop.actor.store.flat.values()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref), "ranks diverged after synchronised updates"
    assert all(m["perf/step_tokens"] == 32 * 48 for m in hist)  # global tokens: both ranks' shares
    assert all(m["train/train_rollout_logprob_abs_diff"] < 1e-5 for m in hist)
    torch.save({"rank": rank, "hist": hist}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_world_size_2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a = torch.load(tmp_path / "r0.pt", weights_only=False)["hist"]
    b = torch.load(tmp_path / "r1.pt", weights_only=False)["hist"]
    assert a[0]["train/grad_norm"] == pytest.approx(b[0]["train/grad_norm"], rel=1e-5)
    assert a[1]["train/pg_loss"] == pytest.approx(b[1]["train/pg_loss"], abs=1e-6)


def _pp_worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)  # several ranks share the host cores
    from miles_b200.loop import RLLoop

    args = parse_args(BASE + ["--num-rollout", "2", "--actor-num-gpus-per-node", str(world), "--distributed-backend", "gloo",
                              "--pipeline-model-parallel-size", str(world)])
    loop = RLLoop(args)
    st = loop.actor.store
    assert st.layer_range == (rank, rank + 1)  # the tiny model has two layers: one per stage
    assert ("embed.weight" in st.params) == (rank == 0) and ("final_norm.weight" in st.params) == (rank == world - 1)
    hist = loop.run()
    # the engine decodes on a full-model replica that the weight update filled from both stages
    rs = loop.rollout_store
    assert rs is not None and rs.layer_range == (0, 2)
    for name, p in st.params.items():
        assert torch.equal(rs.params[name], p), name
    both = [None, None]
    dist.all_gather_object(both, {k: v for k, v in hist[-1].items() if k.startswith("train/")})
    assert both[0] == both[1], "stages report different training metrics"
    assert all(m["train/train_rollout_logprob_abs_diff"] < 1e-5 for m in hist)
    assert all(m["perf/step_tokens"] == 32 * 48 for m in hist)  # one pipeline = one replica: all its samples, counted once
    assert all(m["train/grad_norm"] > 0 for m in hist)
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_pipeline_parallel_two_stages(tmp_path):
    port = 29000 + (os.getpid() * 7) % 2000
    mp.spawn(_pp_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)


def _cp_worker(rank: int, world: int, port: int, out_dir: str, comm: str = "p2p"):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)  # several ranks share the host cores
    import copy

    from miles_b200.loop import RLLoop
    from miles_b200.parallel.state import ParallelState
    from miles_b200.rollout.train_data import convert_samples_to_train_data
    from miles_b200.trainer.actor import TrainActor

    args = parse_args(BASE + ["--num-rollout", "1", "--actor-num-gpus-per-node", str(world), "--distributed-backend", "gloo",
                              "--context-parallel-size", str(world), "--cp-comm-type", comm.split("+")[0]]
                      + (["--allgather-cp"] if comm.endswith("+allgather") else []))
    loop = RLLoop(args)
    assert loop.ps.cp.size == world and loop.ps.dp.size == 1 and loop.ps.cp_comm_type == comm.split("+")[0]
    # a single-process trainer with the same initial weights trains on the same pooled samples
    solo = TrainActor(copy.copy(args), "actor", ParallelState())
    for g in solo.store.flat:
        assert torch.equal(solo.store.flat[g], loop.actor.store.flat[g])
    loop.update_weights()
    samples, _ = loop.generate(0)
    assert len(samples) == 32  # both ranks' shares, pooled
    if args.offload_train:
        loop.actor.wake_up()  # what RLLoop.step does before training
    m = loop.train(0, samples)
    solo._local_data = True
    m0 = solo.train(0, convert_samples_to_train_data(args, samples))
    # the context-parallel step is the single-process step: same loss terms, same gradient norm, same new weights
    for k in ("train/pg_loss", "train/grad_norm", "train/train_rollout_logprob_abs_diff"):
        assert abs(m[k] - m0[k]) <= 1e-5 * max(1.0, abs(m0[k])), (k, m[k], m0[k])
    # (the first Adam step moves every weight by lr * g / (|g| + eps): an element whose gradient is rounding noise around
    # zero may move the other way in the other summation order, so a handful of elements may differ by up to 2 lr)
    for g in solo.store.flat:
        d = (solo.store.flat[g] - loop.actor.store.flat[g]).abs()
        if d.numel() == 0:
            continue
        assert d.max().item() <= 2.2 * args.lr and (d > 1e-6).float().mean().item() < 1e-3, (g, d.max().item())
    assert m["train/train_rollout_logprob_abs_diff"] < 1e-5
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("comm", ["p2p", "a2a", "p2p+allgather"])
def test_gloo_context_parallel_training_matches_single_process(tmp_path, comm):
    port = 31000 + (os.getpid() * 13) % 2000 + {"p2p": 0, "a2a": 7, "p2p+allgather": 14}[comm]
    mp.spawn(_cp_worker, args=(2, port, str(tmp_path), comm), nprocs=2, join=True)


def _pp_cp_worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)  # several ranks share the host cores
    from miles_b200.loop import RLLoop

    args = parse_args(BASE + ["--num-rollout", "1", "--actor-num-gpus-per-node", str(world), "--distributed-backend", "gloo",
                              "--pipeline-model-parallel-size", "2", "--context-parallel-size", "2"])
    loop = RLLoop(args)
    assert (loop.ps.pp.size, loop.ps.cp.size, loop.ps.dp.size) == (2, 2, 1)
    hist = loop.run()
    m = hist[-1]
    assert m["train/train_rollout_logprob_abs_diff"] < 1e-5 and m["train/grad_norm"] > 0
    assert m["perf/step_tokens"] == 32 * 48  # four ranks generated a quarter each; one replica, counted once
    allm = [None] * world
    dist.all_gather_object(allm, {k: round(v, 9) for k, v in m.items() if k.startswith("train/")})
    assert all(x == allm[0] for x in allm)
    # ranks of the same stage hold identical weights after the step
    flat = torch.cat([t.flatten() for t in loop.actor.store.flat.values()])
    peers = [torch.empty_like(flat) for _ in range(loop.ps.cp.size)]
    dist.all_gather(peers, flat, group=loop.ps.cp.group)
    assert all(torch.equal(p, peers[0]) for p in peers)
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_pipeline_and_context_parallel_together(tmp_path):
    port = 33000 + (os.getpid() * 17) % 2000
    mp.spawn(_pp_cp_worker, args=(4, port, str(tmp_path)), nprocs=4, join=True)


def test_ci_checks_run_inside_the_loop(tmp_path):
    """--ci-test: on-policy gate after every step, weight hashes written with the checkpoint and verified on resume."""
    from miles_b200.loop import RLLoop

    common = BASE + ["--actor-num-gpus-per-node", "1", "--ci-test", "--ci-save-model-hash", "--ci-check-model-hash",
                     "--save", str(tmp_path / "ckpt"), "--save-interval", "1"]
    loop = RLLoop(parse_args(common + ["--num-rollout", "1"]))
    loop.run()
    hashes = list((tmp_path / "ckpt").rglob("model_hash_*.json"))
    assert len(hashes) == 1
    loop2 = RLLoop(parse_args(common + ["--num-rollout", "2", "--load", str(tmp_path / "ckpt")]))  # verifies the hashes while loading
    assert loop2.start_rollout_id == 1
    # a tampered checkpoint is caught
    import json

    h = json.loads(hashes[0].read_text())
    k = sorted(h)[0]
    h[k] = "0" * 64
    hashes[0].write_text(json.dumps(h))
    with pytest.raises(AssertionError):
        RLLoop(parse_args(common + ["--num-rollout", "2", "--load", str(tmp_path / "ckpt")]))


def test_model_provider_plugin_builds_the_trainer_and_engine_model():
    """--custom-model-provider-path: the plug-in's model trains and (shared with the colocated engine) generates: the
    trainer / rollout log-probs still agree, which they would not if only one side used the plug-in."""
    from miles_b200.loop import RLLoop
    from miles_b200.plugins.example_provider import SoftCappedQwen3

    args = parse_args(BASE + ["--num-rollout", "1", "--actor-num-gpus-per-node", "1",
                              "--custom-model-provider-path", "miles_b200.plugins.example_provider.provider"])
    loop = RLLoop(args)
    assert isinstance(loop.actor.model, SoftCappedQwen3) and loop.engine.model is loop.actor.model
    m = loop.run()[0]
    assert m["train/train_rollout_logprob_abs_diff"] < 1e-5 and m["train/grad_norm"] > 0

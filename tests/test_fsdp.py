"""Sharded data-parallel backend (--train-backend fsdp): shard arithmetic, equivalence with plain data parallelism over
gloo ranks (autograd model path), hybrid sharding, the engine's weight gather, reshardable checkpoints and HF round trips."""
import os
import socket
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from miles_b200.fsdp.mesh import mesh_ranks
from miles_b200.fsdp.store import ALIGN, FsdpParamStore, build_units
from miles_b200.models import ParamStore, get_config
from miles_b200.models.params import build_specs
from miles_b200.parallel.state import GroupInfo
from miles_b200.utils.arguments import parse_args

BASE = ["--model-preset", "qwen3-tiny-moe", "--rollout-batch-size", "8", "--n-samples-per-prompt", "4", "--rollout-max-response-len", "16",
        "--rollout-max-prompt-len", "32", "--rm-type", "parity", "--lr", "1e-5", "--eps-clip", "0.2", "--micro-batch-size", "4",
        "--weight-decay", "0.01", "--colocate", "--distributed-backend", "gloo",
        # a KL term against reference weights: the reference is a pinned copy of the shards, swapped in for one pass
        "--use-kl-loss", "--kl-loss-coef", "0.05"]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_mesh(size: int, rank: int):
    return SimpleNamespace(shard=GroupInfo(rank, size, None, list(range(size))), replicate=GroupInfo(0, 1, None, [0]))


def test_units_cover_every_parameter_and_pieces_are_aligned():
    cfg = get_config("qwen3-tiny-moe")
    specs = build_specs(cfg)
    for S in (1, 2, 3, 8):
        units = build_units(specs, S)
        assert [u.name for u in units][0] == "embed" and units[-1].name == "head" and len(units) == cfg.num_layers + 2
        seen = [s.name for u in units for s in u.specs]
        assert seen == [s.name for s in specs]
        for g in ("dense", "expert"):
            end = 0
            for u in units:
                if u.hi[g] > u.lo[g]:
                    assert u.lo[g] == end, "units tile the flat buffer without gaps"
                    end = u.hi[g]
                assert u.padded[g] % (S * ALIGN) == 0 and u.padded[g] >= u.hi[g] - u.lo[g]
                assert u.padded[g] - (u.hi[g] - u.lo[g]) < S * ALIGN


def test_mesh_ranks_and_their_validation():
    shard, repl = mesh_ranks(list(range(8)), 2)
    assert shard == [[0, 1, 2, 3], [4, 5, 6, 7]] and repl == [[0, 4], [1, 5], [2, 6], [3, 7]]
    with pytest.raises(ValueError):
        mesh_ranks(list(range(8)), 3)


def test_decay_segments_of_all_ranks_tile_the_matrices():
    """Union over ranks of the decayed segments, mapped back to full coordinates, is exactly the matrices' elements."""
    cfg = get_config("qwen3-tiny")
    S = 3
    full = ParamStore(cfg, "cpu", torch.float32, meta=True, init=False)
    marks = {g: torch.zeros(full.sizes[g], dtype=torch.int8) for g in full.sizes}
    for r in range(S):
        st = FsdpParamStore(cfg, "cpu", torch.float32, _fake_mesh(S, r), init=False)
        segs = st.decay_segments(0.1)
        for g, lst in segs.items():
            assert all(a % ALIGN == 0 and b % ALIGN == 0 and a < b <= st.sizes[g] for a, b, _ in lst)
            flags = torch.zeros(st.sizes[g], dtype=torch.int8)
            for a, b, wd in lst:
                flags[a:b] = 2 if wd > 0 else 1
            for u in st.units:
                n = u.piece(g, S)
                if not n:
                    continue
                a0 = u.lo[g] + r * n
                b0 = min(a0 + n, u.hi[g])
                if b0 > a0:
                    marks[g][a0:b0] = flags[u.shard_off[g]:u.shard_off[g] + b0 - a0]
    for s in full.specs:
        want = 2 if len(s.shape) >= 2 else 1
        assert bool((marks[s.group][s.offset:s.offset + s.numel] == want).all()), s.name


def test_single_rank_store_matches_the_unsharded_store_and_keeps_writes():
    cfg = get_config("qwen3-tiny-moe")
    ref = ParamStore(cfg, "cpu", torch.float32, seed=3)
    st = FsdpParamStore(cfg, "cpu", torch.float32, _fake_mesh(1, 0), seed=3)
    for name, p in st.named_parameters():
        assert torch.equal(p, ref.params[name]), name
    with st.writing():
        st.params["layers.1.ln1.weight"].fill_(2.5)
    assert bool((st.params["layers.1.ln1.weight"] == 2.5).all())
    assert torch.equal(st.params["layers.1.attn.o.weight"], ref.params["layers.1.attn.o.weight"])
    dst = ParamStore(cfg, "cpu", torch.float32, init=False)
    st.gather_into(dst)
    assert bool((dst.params["layers.1.ln1.weight"] == 2.5).all()) and torch.equal(dst.params["embed.weight"], ref.params["embed.weight"])
    assert st.checksum()["expert"] == pytest.approx(ref.checksum()["expert"], rel=1e-6)


def test_flags_of_the_sharded_backend_are_validated(tmp_path):
    with pytest.raises(ValueError):
        parse_args(BASE + ["--train-backend", "fsdp", "--tensor-model-parallel-size", "2"])
    with pytest.raises(ValueError):
        parse_args(BASE + ["--dp-replicate-size", "2"])
    with pytest.raises(NotImplementedError):
        parse_args(BASE + ["--train-backend", "fsdp", "--lora-rank", "8"])
    cfg = tmp_path / "fsdp.yaml"
    cfg.write_text("train_backend: fsdp\ndp_replicate_size: 2\nlr: 3.0e-6\n")
    a = parse_args(BASE + ["--num-rollout", "1", "--config", str(cfg)])
    assert a.train_backend == "fsdp" and a.dp_replicate_size == 2 and a.lr == 3e-6
    cfg.write_text("no_such_key: 1\n")
    with pytest.raises(ValueError):
        parse_args(BASE + ["--num-rollout", "1", "--config", str(cfg)])


def _full_weights(loop) -> dict:
    st = loop.actor.store
    if getattr(st, "is_fsdp", False):
        dst = ParamStore(st.cfg, "cpu", st.dtype, init=False)
        st.gather_into(dst)
        return {g: t.clone() for g, t in dst.flat.items()}
    return {g: t.clone() for g, t in st.flat.items()}


def _worker(rank: int, world: int, port: int, out_dir: str, mode: str):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    from miles_b200.loop import RLLoop

    extra = {"dp": [], "fsdp": ["--train-backend", "fsdp"], "hsdp": ["--train-backend", "fsdp", "--dp-replicate-size", "2"],
             "cp": ["--context-parallel-size", "2"], "fsdp_cp": ["--train-backend", "fsdp", "--context-parallel-size", "2"]}[mode]
    ckpt = os.path.join(out_dir, f"ckpt_{mode}")
    args = parse_args(BASE + extra + ["--num-rollout", "2", "--actor-num-gpus-per-node", str(world), "--check-weight-update-equal",
                                      "--save", ckpt, "--save-interval", "1"])
    loop = RLLoop(args)
    hist = loop.run()
    assert all(m["train/train_rollout_logprob_abs_diff"] < 1e-5 for m in hist), "the engine serves the gathered weights"
    full = _full_weights(loop)
    if mode not in ("dp", "cp"):
        st = loop.actor.store
        assert st.gathers > 0 and (st.shard_size == 1 or sum(st.sizes.values()) < sum(st.full_sizes.values()))
        for g, t in loop.rollout_store.flat.items():
            assert torch.equal(t, full[g]), "engine copy == gathered trainer weights"
        # resume under the same layout: shards and optimizer state come back exactly
        args2 = parse_args(BASE + extra + ["--num-rollout", "3", "--actor-num-gpus-per-node", str(world), "--load", ckpt])
        loop2 = RLLoop(args2)
        assert loop2.start_rollout_id == 2 and loop2.actor.opt.step_count == loop.actor.opt.step_count
        for g in st.flat:
            assert torch.equal(loop2.actor.store.flat[g], st.flat[g]), g
            for part in ("m", "v"):
                assert torch.equal(loop2.actor.opt.state[g][part], loop.actor.opt.state[g][part]), (g, part)
        # HuggingFace export of the sharded trainer, read back into an unsharded store
        from miles_b200.checkpoint import export_hf, load_hf

        hf_dir = os.path.join(out_dir, f"hf_{mode}")
        export_hf(loop.actor, hf_dir)
        back = ParamStore(st.cfg, "cpu", st.dtype, init=False)
        load_hf(st.cfg, back, hf_dir)
        for g in full:
            assert torch.equal(back.flat[g], full[g]), f"HF round trip {g}"
        # ... and into a fresh sharded store (writes through per-unit views are kept)
        loop2.actor.store.flat["dense"].zero_()
        with loop2.actor.store.writing(gather=False):
            load_hf(st.cfg, loop2.actor.store, hf_dir)
        assert torch.equal(loop2.actor.store.flat["dense"], st.flat["dense"])
    if rank == 0:
        torch.save({"full": full, "hist": hist}, os.path.join(out_dir, f"{mode}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _compare(a: dict, b: dict, lr: float = 1e-5):
    for g in a["full"]:
        d = (a["full"][g] - b["full"][g]).abs()
        if not d.numel():
            continue
        # Adam's first steps move every weight by about lr whatever the gradient's size: an element whose gradient is
        # rounding noise may go the other way under another summation order, so a few elements may differ by up to 2 lr
        assert d.max().item() <= 2.2 * lr * 2, (g, d.max().item())
        assert (d > 1e-7).float().mean().item() < 2e-3, (g, (d > 1e-7).float().mean().item())
    for ma, mb in zip(a["hist"], b["hist"]):
        assert ma["train/grad_norm"] == pytest.approx(mb["train/grad_norm"], rel=1e-4)
        assert ma["train/pg_loss"] == pytest.approx(mb["train/pg_loss"], abs=1e-6)


def test_sharded_training_matches_plain_data_parallel_and_checkpoints_reshard(tmp_path):
    for mode in ("dp", "fsdp"):
        mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), mode), nprocs=2, join=True)
    dp = torch.load(tmp_path / "dp.pt", weights_only=False)
    fs = torch.load(tmp_path / "fsdp.pt", weights_only=False)
    _compare(dp, fs)
    # what the sharded run saved loads into one unsharded process (and the other way round): same atoms
    from miles_b200.loop import RLLoop

    one = RLLoop(parse_args(BASE + ["--num-rollout", "3", "--actor-num-gpus-per-node", "1", "--load", str(tmp_path / "ckpt_fsdp")]))
    assert one.start_rollout_id == 2 and one.actor.opt.step_count == 2
    for g, t in one.actor.store.flat.items():
        assert torch.equal(t, fs["full"][g]), g
    one2 = RLLoop(parse_args(BASE + ["--train-backend", "fsdp", "--num-rollout", "3", "--actor-num-gpus-per-node", "1",
                                     "--load", str(tmp_path / "ckpt_dp")]))
    full = _full_weights(one2)
    for g, t in full.items():
        assert torch.equal(t, dp["full"][g]), g
    assert one2.actor.opt.step_count == 2


def test_hybrid_sharding_two_replicas_of_two_shards(tmp_path):
    mp.spawn(_worker, args=(4, _free_port(), str(tmp_path), "hsdp"), nprocs=4, join=True)
    mp.spawn(_worker, args=(4, _free_port(), str(tmp_path), "dp"), nprocs=4, join=True)
    _compare(torch.load(tmp_path / "dp.pt", weights_only=False), torch.load(tmp_path / "hsdp.pt", weights_only=False))


def _explicit_worker(rank: int, world: int, port: int):
    """The gradient path of the hand-written backward: the model writes into full-unit views in reverse layer order
    (touching the tied / first unit twice), the store reduce-scatters every unit as the backward leaves it."""
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from miles_b200.fsdp import build_mesh
    from miles_b200.parallel.state import init_parallel_state

    ps = init_parallel_state(backend="gloo")
    cfg = get_config("qwen3-tiny-moe")
    st = FsdpParamStore(cfg, "cpu", torch.float32, build_mesh(ps, 1), seed=5)
    st.allocate_grads(torch.float32)
    g = torch.Generator().manual_seed(100 + rank)
    mine = {s.name: torch.randn(s.shape, generator=g) for s in st.specs}
    for _ in range(2):  # two micro-batches accumulate
        st.grads["embed.weight"].add_(mine["embed.weight"])          # e.g. a tied LM head at the start of the backward
        for s in reversed(st.specs):
            st.params[s.name]  # the backward reads a unit's weights (recompute, dgrad) while it writes its gradients
            st.grads[s.name].add_(mine[s.name])
    st.finish_grads()
    assert st.reduce_scatters >= 2 * (cfg.num_layers + 2)
    for s in st.specs:
        tot = mine[s.name].clone() * (4.0 if s.name == "embed.weight" else 2.0)
        dist.all_reduce(tot)
        u = st.unit_of[s.name]
        n = u.piece(s.group, world)
        a, b = s.offset - u.lo[s.group], s.offset - u.lo[s.group] + s.numel
        lo, hi = max(a, rank * n), min(b, (rank + 1) * n)
        if lo < hi:
            got = st.grad[s.group][u.shard_off[s.group] + lo - rank * n:u.shard_off[s.group] + hi - rank * n]
            assert torch.allclose(got, tot.flatten()[lo - a:hi - a], atol=1e-5), s.name
    st.zero_grads()
    assert float(st.grad["dense"].abs().sum()) == 0.0
    dist.barrier()
    dist.destroy_process_group()


def test_explicit_gradient_path_reduce_scatters_units_in_backward_order():
    mp.spawn(_explicit_worker, args=(2, _free_port()), nprocs=2, join=True)


def _serve_engine(port, ready):
    torch.set_num_threads(2)
    from miles_b200.engine import Engine
    from miles_b200.engine.server import serve
    from miles_b200.models import build_model

    cfg = get_config("qwen3-tiny-moe")
    st = ParamStore(cfg, "cpu", torch.float32, seed=2)  # other weights than the trainer's until the first update
    ready.set()
    serve(Engine(build_model(cfg, st), max_running=4, page_size=8, max_seq_len=64), port=port)


def _remote_worker(rank: int, world: int, port: int, engine_port: int):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      MILES_B200_ENV_REPORT="0")
    torch.set_num_threads(2)
    from miles_b200.loop import RLLoop
    from miles_b200.weight_sync.broadcast import HttpEngineHandle

    args = parse_args(["--model-preset", "qwen3-tiny-moe", "--train-backend", "fsdp", "--num-rollout", "2", "--rollout-batch-size", "4",
                       "--n-samples-per-prompt", "2", "--rollout-max-response-len", "8", "--rollout-max-prompt-len", "16",
                       "--rm-type", "parity", "--lr", "1e-3", "--actor-num-nodes", "1", "--actor-num-gpus-per-node", str(world),
                       "--rollout-engine-urls", f"http://127.0.0.1:{engine_port}", "--micro-batch-size", "2",
                       "--distributed-backend", "gloo"])
    loop = RLLoop(args)
    assert loop.engine is None and loop.weight_updater is not None, "every rank walks the units; the first one sends"
    hist = loop.run()
    assert len(hist) == 2 and all(m["train/train_rollout_logprob_abs_diff"] < 1e-5 for m in hist)
    want = loop.actor.store.checksum()  # collective: the pieces' sums over the shard group
    if rank == 0:
        h = HttpEngineHandle(f"http://127.0.0.1:{engine_port}", timeout_s=60)
        got = h.post("/weights_checker", {"action": "checksum"})["checksum"]
        assert all(abs(got[g] - want[g]) <= 1e-3 * max(1.0, abs(want[g])) for g in want), (got, want)
        assert h.get("/get_weight_version")["weight_version"] == loop.actor.store.version
        loop.weight_updater.disconnect()
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_trainer_updates_an_engine_in_another_process():
    """--train-backend fsdp with --rollout-engine-urls: the units are gathered one after the other on all trainer ranks and
    broadcast by the first one; the engine then holds the trainer's weights (on-policy log-prob parity proves it)."""
    import time

    from miles_b200.weight_sync.broadcast import HttpEngineHandle

    ctx = mp.get_context("spawn")
    engine_port = _free_port()
    ready = ctx.Event()
    srv = ctx.Process(target=_serve_engine, args=(engine_port, ready), daemon=True)
    srv.start()
    try:
        assert ready.wait(120)
        h = HttpEngineHandle(f"http://127.0.0.1:{engine_port}", timeout_s=60)
        for _ in range(100):
            try:
                h.get("/health")
                break
            except Exception:
                time.sleep(0.2)
        mp.spawn(_remote_worker, args=(2, _free_port(), engine_port), nprocs=2, join=True)
    finally:
        srv.terminate()
        srv.join(10)


def test_sharded_backend_under_context_parallelism(tmp_path):
    """Shards over the dp x cp group: the ranks of a context-parallel group hold different pieces of the same samples'
    gradients, and the per-unit reduce-scatter is the sum the plain backend takes with an all-reduce."""
    for mode in ("cp", "fsdp_cp"):
        mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), mode), nprocs=2, join=True)
    _compare(torch.load(tmp_path / "cp.pt", weights_only=False), torch.load(tmp_path / "fsdp_cp.pt", weights_only=False))

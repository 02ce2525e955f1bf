"""Expert parallelism on 2+ GPUs: in-kernel NVLink exchange and the NCCL baseline vs the single-rank model."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(mode: str, n: int, preset: str = "qwen3-smoke-moe"):
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29731", os.path.join(here, "mp_ep_check.py"), mode, preset]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "EP_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.parametrize("mode", ["nccl", "fused", "fused_copy"])
def test_expert_parallel_matches_single_rank(mode):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    _run(mode, 2)


def test_expert_parallel_with_sigmoid_router_and_shared_expert():
    """GLM-4.5 style layers under expert parallelism: routing happens before the dispatch, the shared expert's output joins
    the residual that the combine adds."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    _run("fused", 2, "glm4moe-smoke")


def test_low_latency_expert_parallel_decode():
    """The decode exchange (gather rows at the expert owners, partial sums back): one layer against the single-rank
    layer, then lockstep rollouts with uneven request counts checked by log-prob recomputation."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29733", os.path.join(here, "mp_ep_decode_check.py"), "check"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "EP_DECODE_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_weight_push_reshards_and_quantises_into_peer_memory():
    """The peer-memory weight update (reshard + quantise + store + flag in one kernel): expert-parallel trainer ->
    replicas (bf16, MXFP8, NVFP4, bitwise against the stand-alone quantisers), tensor-parallel trainer -> unsharded
    engine, replicated trainer -> tensor-parallel engine, and a source that never arrives (the bounded wait gives up)."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29735", os.path.join(here, "mp_weight_push_check.py"), "check"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "WEIGHT_PUSH_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]

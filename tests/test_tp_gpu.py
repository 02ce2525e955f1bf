"""Tensor-parallel fused GEMM + all-reduce on 2 GPUs (child processes, NVLS off in NCCL)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fused_linear_allreduce_matches_reference():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29741", os.path.join(here, "mp_tp_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "TP_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.parametrize("mode", ["nccl", "fused"])
def test_tensor_parallel_model_matches_single_rank(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29743", os.path.join(here, "mp_tp_model_check.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "TP_MODEL_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_context_parallel_attention_forward():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29745", os.path.join(here, "mp_cp_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "CP_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_partitioned_optimizer_matches_allreduce_adam():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29747", os.path.join(here, "mp_dp_adam_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "DP_ADAM_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_pipeline_parallel_model_matches_single_rank():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29749", os.path.join(here, "mp_pp_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "PP_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_context_parallel_training_step_on_the_sm100_path():
    """Sequence shards are traded for head shards around the attention forward / backward kernels: log-probs and the
    summed gradients of a 2-rank context-parallel step equal the single-rank step (dense and MoE smoke models)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29749", os.path.join(here, "mp_cp_train_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "CP_TRAIN_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_sharded_data_parallel_store_on_the_sm100_path():
    """--train-backend fsdp under the hand-written forward / backward: per-unit all-gather with prefetch on a side stream,
    per-unit reduce-scatter in the backward, Adam on the shards; against an unsharded store + gradient all-reduce."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29751", os.path.join(here, "mp_fsdp_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "FSDP_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_nccl_groups_are_released_and_rebuilt():
    """--reload-process-groups: destroy the NCCL sub-groups, build them again, collectives and holders keep working."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29753", os.path.join(here, "mp_reload_groups_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "RELOAD_GROUPS_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]

"""Small utilities: HTTP retries, FLOP counts / MFU, eval config overlay, lifecycle sinks."""
import asyncio

import pytest

from miles_b200.models import get_config
from miles_b200.utils import http_utils, lifecycle
from miles_b200.utils.eval_config import build_eval_configs
from miles_b200.utils.flops_utils import device_peak_tflops, forward_flops, mfu, train_step_flops


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

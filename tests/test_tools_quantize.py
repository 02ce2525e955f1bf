"""Offline quantiser and its inverse: an HF checkpoint quantised to each format and cast back to bf16 stays within
the format's quantisation error, non-linear tensors pass through untouched, the config records the format."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace as NS

import pytest
import torch
from safetensors import safe_open

from miles_b200.checkpoint import export_hf
from miles_b200.models import ParamStore, get_config
from miles_b200.tools import dequantize_hf

# largest relative error per element block a format may introduce (scale granularity / mantissa bits)
TOL = {"fp8_block": 0.07, "mxfp8": 0.07, "nvfp4": 0.3, "int4": 0.2}


def _tensors(path):
    out = {}
    for f in sorted(os.listdir(path)):
        if f.endswith(".safetensors"):
            with safe_open(os.path.join(path, f), framework="pt") as h:
                out.update({k: h.get_tensor(k) for k in h.keys()})
    return out


@pytest.mark.parametrize("fmt", ["fp8_block", "mxfp8", "nvfp4", "int4"])
def test_quantize_then_dequantize_round_trip(tmp_path, fmt):
    cfg = get_config("qwen3-tiny")
    store = ParamStore(cfg, "cpu", torch.bfloat16, seed=4)
    one = NS(size=1, rank=0, group=None)
    actor = NS(store=store, opt=None, args=NS(hf_checkpoint=None), cfg=cfg, global_step=0, ps=NS(rank=0, world_size=1, tp=one, pp=one, dp_cp=one))
    src = str(tmp_path / "bf16")
    export_hf(actor, src)
    q = str(tmp_path / "q")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-m", "miles_b200.tools.quantize_hf", "--hf-checkpoint", src, "--output", q, "--format", fmt],
                       capture_output=True, text=True, env=env, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.load(open(os.path.join(q, "config.json")))["quantization_config"]["quant_method"] == fmt
    back = str(tmp_path / "back")
    n = dequantize_hf.convert(q, back)
    a, b = _tensors(src), _tensors(back)
    assert a.keys() == b.keys() and "quantization_config" not in json.load(open(os.path.join(back, "config.json")))
    quantised = [k for k in a if k.endswith("_proj.weight")]
    assert n == len(quantised) > 0
    for k in a:
        if k in quantised:
            err = (a[k].float() - b[k].float()).abs().max().item()
            assert err <= TOL[fmt] * a[k].float().abs().max().item(), (k, err)
            assert b[k].dtype == torch.bfloat16
        else:
            assert torch.equal(a[k], b[k]), k

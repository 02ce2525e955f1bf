"""Tensor-parallel parameter sharding on CPU: local config, slice / merge round trip, sharded init and HF import."""
import torch

from miles_b200.models import ParamStore, get_config
from miles_b200.models.hf_mapping import from_hf, hf_names
from miles_b200.models.params import is_tp_sharded, tp_local_config, tp_merge, tp_slice


def test_local_config_divides_heads_and_ffn():
    cfg = get_config("qwen3-4B")
    loc = tp_local_config(cfg, 2)
    assert loc.num_q_heads * 2 == cfg.num_q_heads and loc.num_kv_heads * 2 == cfg.num_kv_heads
    assert loc.ffn_hidden_size * 2 == cfg.ffn_hidden_size and loc.hidden_size == cfg.hidden_size
    assert tp_local_config(cfg, 1) is cfg


def test_slice_merge_round_trip_and_sharded_init():
    cfg = get_config("qwen3-tiny")
    full = ParamStore(cfg, "cpu", torch.float32, seed=3)
    shards = [ParamStore(cfg, "cpu", torch.float32, seed=3, tp_size=2, tp_rank=r) for r in range(2)]
    n_sharded = 0
    for name, t in full.params.items():
        parts = [s.params[name] for s in shards]
        assert torch.equal(tp_merge(cfg, name, parts), t), name
        for r in range(2):
            assert torch.equal(tp_slice(cfg, name, t, 2, r), parts[r]), name
        if is_tp_sharded(name):
            n_sharded += 1
            assert parts[0].numel() * 2 == t.numel()
        else:
            assert torch.equal(parts[0], parts[1])
    assert n_sharded == 4 * cfg.num_layers  # qkv, o, gate_up, down per layer (no qkv bias in this preset)


def test_hf_import_into_shards_matches_slicing():
    cfg = get_config("qwen3-tiny")
    full = ParamStore(cfg, "cpu", torch.float32, seed=5)
    hf = dict(hf_names(cfg, full))
    for r in range(2):
        sh = ParamStore(cfg, "cpu", torch.float32, seed=77, tp_size=2, tp_rank=r)
        from_hf(cfg, sh, lambda k: hf.get(k))
        for name, t in full.params.items():
            assert torch.equal(sh.params[name], tp_slice(cfg, name, t, 2, r)), name

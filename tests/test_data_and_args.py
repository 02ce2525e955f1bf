"""Micro-batch packing, sequence balancing, sample conversion, flag surface."""
import pytest
import torch

from miles_b200.rollout.train_data import convert_samples_to_train_data, pass_at_k, postprocess_rollout_data
from miles_b200.trainer.data import build_micro_batches, pack_samples, split_by_dp
from miles_b200.utils.arguments import build_parser, parse_args
from miles_b200.utils.seqlen_balancing import first_fit_pack, karmarkar_karp
from miles_b200.utils.types import Sample


def _data():
    return {
        "tokens": [[1, 2, 3, 4, 5], [7, 8, 9], [4, 4, 4, 4, 4, 4, 4]],
        "response_lengths": [2, 1, 4],
        "loss_masks": [[1, 1], [1], [1, 0, 1, 1]],
        "rewards": [1.0, -1.0, 0.5],
        "rollout_log_probs": [[-0.1, -0.2], [-0.3], [-0.4, -0.5, -0.6, -0.7]],
        "rollout_mask_sums": [2, 1, 3],
    }


def test_pack_samples_alignment():
    mb = pack_samples(_data(), [0, 1, 2])
    assert mb.tokens.tolist() == [1, 2, 3, 4, 5, 7, 8, 9, 4, 4, 4, 4, 4, 4, 4]
    assert mb.positions.tolist() == [0, 1, 2, 3, 4, 0, 1, 2, 0, 1, 2, 3, 4, 5, 6]
    assert mb.cu_seqlens.tolist() == [0, 5, 8, 15] and mb.max_seqlen == 7
    # logits at rows predict the response tokens
    assert mb.rows.tolist() == [2, 3, 6, 10, 11, 12, 13]
    assert mb.targets.tolist() == [4, 5, 9, 4, 4, 4, 4]
    assert mb.seg.tolist() == [0, 0, 1, 2, 2, 2, 2] and mb.resp_cu.tolist() == [0, 2, 3, 7]
    assert mb.loss_mask.tolist() == [1, 1, 1, 1, 0, 1, 1] and mb.denoms.tolist() == [2, 1, 3]
    assert torch.allclose(mb.rollout_log_probs, torch.tensor([-0.1, -0.2, -0.3, -0.4, -0.5, -0.6, -0.7]))


def test_micro_batching_modes():
    d = _data()
    assert [m.sample_indices for m in build_micro_batches(d, max_tokens_per_gpu=8)] == [[0, 1], [2]]
    assert [m.sample_indices for m in build_micro_batches(d, micro_batch_size=2)] == [[0, 1], [2]]
    assert len(build_micro_batches(d, num_micro_batches=3)) == 3
    assert split_by_dp(d, 2) == [[0, 2], [1]]


def test_balancing():
    L = [10, 9, 8, 7, 6, 5, 4, 3]
    parts = karmarkar_karp(L, 2, equal_size=True)
    sums = [sum(L[i] for i in p) for p in parts]
    assert sorted(len(p) for p in parts) == [4, 4] and abs(sums[0] - sums[1]) <= 2
    assert sorted(i for p in karmarkar_karp(L, 3) for i in p) == list(range(8))
    bins = first_fit_pack([5, 4, 3, 9, 1], 9)
    assert all(sum([5, 4, 3, 9, 1][i] for i in b) <= 9 for b in bins) and len(bins) == 3
    with pytest.raises(ValueError):
        karmarkar_karp([1, 2, 3], 2, equal_size=True)


def _args(extra=()):
    return parse_args(["--num-rollout", "2", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--model-preset", "qwen3-tiny",
                       *extra])


def test_convert_samples_and_postprocess():
    args = _args()
    ss = []
    for g in range(2):
        for j in range(2):
            s = Sample(group_index=g, index=2 * g + j, tokens=[1, 2, 3, 4 + j], response_length=2, reward=float(j),
                       rollout_log_probs=[-0.1, -0.2], status=Sample.Status.TRUNCATED if j else Sample.Status.COMPLETED)
            ss.append(s)
    d = convert_samples_to_train_data(args, ss)
    assert d["raw_reward"] == [0.0, 1.0, 0.0, 1.0] and d["truncated"] == [0, 1, 0, 1]
    assert abs(d["rewards"][0] + d["rewards"][1]) < 1e-6 and d["rewards"][1] > 0
    assert d["loss_masks"] == [[1, 1]] * 4 and d["rollout_mask_sums"] == [2, 2, 2, 2]
    ss[0].remove_sample = True
    assert len(postprocess_rollout_data(args, ss)) == 3
    assert pass_at_k(4, 0, 2) == 0.0 and pass_at_k(4, 4, 1) == 1.0 and abs(pass_at_k(4, 1, 1) - 0.25) < 1e-9


def test_flag_surface_and_validation():
    p = build_parser()
    flags = {o for a in p._actions for o in a.option_strings}
    for f in ("--advantage-estimator", "--eps-clip-high", "--use-rollout-routing-replay", "--update-weight-transfer-mode",
              "--tensor-model-parallel-size", "--expert-model-parallel-size", "--max-tokens-per-gpu", "--use-tis", "--lora-rank",
              "--save-hf", "--rollout-function-path", "--custom-rm-path", "--kl-loss-type", "--offload-train", "--no-offload-train",
              "--moe-router-topk", "--num-query-groups", "--pause-generation-mode", "--max-weight-staleness", "--fully-async"):
        assert f in flags, f
    assert len(flags) > 480
    a = _args(["--sglang-mem-fraction-static", "0.6", "--sglang-enable-metrics", "--eval-sglang-tp-size", "2", "--colocate"])
    assert a.sglang_mem_fraction_static == 0.6 and a.sglang_enable_metrics is True and a.eval_sglang_tp_size == 2
    assert a.global_batch_size == 4 and a.eps_clip_high == a.eps_clip and a.offload_train and a.offload_rollout
    assert _args(["--use-rollout-routing-replay"]).use_routing_replay
    with pytest.raises(AssertionError):
        _args(["--kl-coef", "0.1", "--kl-loss-coef", "0.1"])
    with pytest.raises(AssertionError):
        _args(["--advantage-estimator", "reinforce_plus_plus"])
    with pytest.raises(AssertionError):
        _args(["--use-dynamic-batch-size"])
    with pytest.raises(NotImplementedError):
        _args(["--multi-latent-attention"])
    with pytest.raises(SystemExit):
        _args(["--definitely-not-a-flag"])


def test_hf_validate_args_reports_all_mismatches():
    from types import SimpleNamespace as NS

    import pytest

    from miles_b200.utils.arguments import hf_validate_args

    hf = {"hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 4, "num_hidden_layers": 48,
          "moe_intermediate_size": 768, "num_experts": 128, "num_experts_per_tok": 8, "rms_norm_eps": 1e-6,
          "rope_parameters": {"rope_theta": 1e6}, "tie_word_embeddings": False}
    ok = NS(hidden_size=2048, num_attention_heads=32, num_query_groups=4, num_layers=48, ffn_hidden_size=None,
            moe_ffn_hidden_size=768, num_experts=128, moe_router_topk=8, norm_epsilon=1e-6, rotary_base=1000000,
            untie_embeddings_and_output_weights=True, kv_channels=None)
    hf_validate_args(ok, hf)
    hf_validate_args(NS(), {"text_config": hf})  # nothing set: nothing to compare
    bad = NS(**{**vars(ok), "num_layers": 24, "rotary_base": 10000, "untie_embeddings_and_output_weights": False})
    with pytest.raises(AssertionError) as e:
        hf_validate_args(bad, hf)
    msg = str(e.value)
    assert "num_hidden_layers" in msg and "rope_theta" in msg and "tie_word_embeddings" in msg


def _package_source() -> str:
    """Every line of the package and the drivers that could read a flag: the flag tables themselves and the policy
    lists are left out, so that being listed does not count as being read."""
    import os
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = []
    for base, _, files in os.walk(os.path.join(root, "miles_b200")):
        for f in files:
            if not f.endswith(".py") or f in ("flag_table.py", "flag_policy.py"):
                continue
            txt = open(os.path.join(base, f)).read()
            if f == "arguments.py" and base.endswith("utils"):
                txt = txt[:txt.index("TRAINER_FLAGS = [")] + txt[txt.index("_UNBUILT"):]
            src.append(txt)
    for f in ("train.py", "train_async.py", "train_multi_lora_async.py"):
        src.append(open(os.path.join(root, f)).read())
    return "\n".join(src)


def test_every_flag_is_read_rejected_or_declared_inert():
    """A parsed flag must do something, refuse to start, or be declared inert with a reason: walking the parser
    catches a flag that is accepted and silently dropped."""
    import re

    from miles_b200.utils import flag_policy
    from miles_b200.utils.arguments import build_parser

    src = _package_source()
    dests = sorted({a.dest for a in build_parser()._actions if a.dest != "help"})
    assert len(dests) > 400
    both = set(flag_policy.REJECT) & set(flag_policy.IGNORED)
    assert not both, f"listed as rejected and as inert: {sorted(both)}"
    stale = [d for d in list(flag_policy.REJECT) + list(flag_policy.IGNORED) if d not in dests]
    assert not stale, f"policy entries for flags the parser does not have: {stale}"
    orphans = []
    for d in dests:
        if d in flag_policy.REJECT or d in flag_policy.IGNORED:
            continue
        if not re.search(r"\b" + re.escape(d) + r"\b", src):
            orphans.append(d)
    assert not orphans, f"{len(orphans)} flags are parsed but neither read, rejected nor declared inert: {orphans}"


def test_unbuilt_features_refuse_to_start():
    base = ["--num-rollout", "1", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--model-preset", "qwen3-tiny"]
    for extra in (["--fp8-format", "e4m3", "--fp8-recipe", "mxfp8"], ["--moe-router-score-function", "sigmoid"],
                  ["--moe-shared-expert-intermediate-size", "512"], ["--attention-output-gate"],
                  ["--true-on-policy-mode"], ["--virtual-pipeline-model-parallel-size", "2"], ["--hidden-dropout", "0.1"]):
        with pytest.raises(NotImplementedError):
            parse_args(base + extra)
    # the reference's own model script for this family passes these with their default meaning: accepted
    parse_args(base + ["--moe-router-score-function", "softmax", "--moe-token-drop-policy", "probs", "--moe-router-dtype", "fp32",
                       "--moe-aux-loss-coeff", "0", "--attention-dropout", "0.0", "--hidden-dropout", "0.0", "--rotary-percent", "1.0",
                       "--normalization", "RMSNorm", "--position-embedding-type", "rope", "--moe-grouped-gemm", "--moe-permute-fusion"])


def test_external_engines_and_init_hook_flags():
    from miles_b200.utils.arguments import parse_args

    base = ["--model-preset", "qwen3-tiny", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--rm-type", "parity",
            "--actor-num-gpus-per-node", "1", "--num-rollout", "1"]
    a = parse_args(base + ["--rollout-external", "--rollout-external-engine-addrs", "10.0.0.1:30000", "http://10.0.0.2:30000"])
    assert a.rollout_engine_urls == "http://10.0.0.1:30000,http://10.0.0.2:30000" and not a.colocate
    import pytest
    with pytest.raises(ValueError):
        parse_args(base + ["--rollout-external-engine-addrs", "10.0.0.1:30000"])


def init_hook(args):
    args.init_hook_saw_seed = args.seed  # (the hook is imported under another module name: leave the trace on args)


def test_custom_init_hook_runs_before_the_model_is_built():
    from miles_b200.trainer.actor import TrainActor
    from miles_b200.parallel.state import ParallelState
    from miles_b200.utils.arguments import parse_args

    a = parse_args(["--model-preset", "qwen3-tiny", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--rm-type", "parity",
                    "--actor-num-gpus-per-node", "1", "--num-rollout", "1", "--custom-megatron-init-path", "tests.test_data_and_args.init_hook"])
    TrainActor(a, "actor", ParallelState())
    assert a.init_hook_saw_seed == a.seed

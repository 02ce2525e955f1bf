"""Numerical parity with the HuggingFace implementations of every architecture family this package serves: a tiny randomly
initialised HF model is saved as safetensors, read through ``ModelConfig.from_hf_config`` + ``load_hf``, and the logits of
the PyTorch model path must equal the HF forward; then the weights are exported again and HF must load them back to the
same logits. Covers the name mapping (fused QKV / gate-up, stacked experts), rotary convention and scaling, QK norm, biases,
tied embeddings and the routers' top-k semantics."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from miles_b200.checkpoint import load_hf  # noqa: E402
from miles_b200.models import ParamStore, build_model  # noqa: E402
from miles_b200.models.config import ModelConfig  # noqa: E402
from miles_b200.models.hf_mapping import hf_names  # noqa: E402

COMMON = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              vocab_size=256, max_position_embeddings=4096)
LLAMA3_SCALING = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                  "original_max_position_embeddings": 64}


def _case(name):
    T = transformers
    if name == "qwen3":
        return T.Qwen3Config(**COMMON, head_dim=16, rope_theta=1e6, tie_word_embeddings=False), T.Qwen3ForCausalLM
    if name == "qwen3-tied":
        return T.Qwen3Config(**COMMON, head_dim=32, rope_theta=1e6, tie_word_embeddings=True), T.Qwen3ForCausalLM
    if name == "qwen3_moe":
        return T.Qwen3MoeConfig(**COMMON, head_dim=16, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                                norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[]), T.Qwen3MoeForCausalLM
    if name == "qwen3_moe-raw-topk":
        return T.Qwen3MoeConfig(**COMMON, head_dim=16, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                                norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[0]), T.Qwen3MoeForCausalLM
    if name == "qwen2":
        return T.Qwen2Config(**COMMON, rope_theta=1e6, tie_word_embeddings=False), T.Qwen2ForCausalLM
    if name == "llama":
        return T.LlamaConfig(**COMMON, rope_theta=5e5, rms_norm_eps=1e-5), T.LlamaForCausalLM
    if name == "llama-rope-llama3":
        return T.LlamaConfig(**COMMON, rope_theta=5e5, rms_norm_eps=1e-5, rope_scaling=dict(LLAMA3_SCALING)), T.LlamaForCausalLM
    if name == "llama-rope-linear":
        return T.LlamaConfig(**COMMON, rope_theta=1e4, rope_scaling={"rope_type": "linear", "factor": 4.0}), T.LlamaForCausalLM
    if name == "mistral":
        return T.MistralConfig(**COMMON, rope_theta=1e6, sliding_window=None), T.MistralForCausalLM
    if name == "mixtral":
        return T.MixtralConfig(**COMMON, rope_theta=1e6, num_local_experts=4, num_experts_per_tok=2, sliding_window=None), T.MixtralForCausalLM
    if name == "glm4_moe":
        return T.Glm4MoeConfig(**COMMON, head_dim=16, partial_rotary_factor=0.5, n_routed_experts=8, num_experts_per_tok=2,
                               moe_intermediate_size=32, n_shared_experts=1, first_k_dense_replace=1, routed_scaling_factor=2.5,
                               norm_topk_prob=True, use_qk_norm=True, attention_bias=True, n_group=1, topk_group=1,
                               rope_theta=1e4), T.Glm4MoeForCausalLM
    if name == "glm4_moe-groups":
        return T.Glm4MoeConfig(**COMMON, head_dim=16, partial_rotary_factor=0.5, n_routed_experts=8, num_experts_per_tok=2,
                               moe_intermediate_size=32, n_shared_experts=2, first_k_dense_replace=0, routed_scaling_factor=1.0,
                               norm_topk_prob=False, use_qk_norm=False, attention_bias=False, n_group=4, topk_group=2,
                               rope_theta=1e4), T.Glm4MoeForCausalLM
    if name == "phi3":
        return T.Phi3Config(**COMMON, rope_theta=250000.0, pad_token_id=0, original_max_position_embeddings=4096), T.Phi3ForCausalLM
    if name == "ernie4_5":
        return T.Ernie4_5Config(**COMMON, head_dim=16, rope_theta=5e5, use_bias=False, tie_word_embeddings=True), T.Ernie4_5ForCausalLM
    if name == "seed_oss":
        return T.SeedOssConfig(**COMMON, head_dim=16, rope_theta=1e7, attention_bias=True, attention_out_bias=False,
                               residual_dropout=0.0, attention_dropout=0.0), T.SeedOssForCausalLM
    if name == "dots1":
        return T.Dots1Config(**COMMON, head_dim=16, n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                             n_shared_experts=2, first_k_dense_replace=1, routed_scaling_factor=2.5, norm_topk_prob=True, n_group=2,
                             topk_group=1, rope_theta=1e4, layer_types=["full_attention"] * 2, sliding_window=None), T.Dots1ForCausalLM
    if name == "qwen2_moe":
        return T.Qwen2MoeConfig(**COMMON, rope_theta=1e6, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                                shared_expert_intermediate_size=48, norm_topk_prob=False, decoder_sparse_step=1,
                                mlp_only_layers=[]), T.Qwen2MoeForCausalLM
    if name == "glm4":
        return T.Glm4Config(**COMMON, head_dim=16, partial_rotary_factor=0.5, attention_bias=True, rope_theta=1e4, pad_token_id=0,
                            eos_token_id=1), T.Glm4ForCausalLM
    raise KeyError(name)


CASES = ["phi3", "ernie4_5", "seed_oss", "dots1", "qwen2_moe", "glm4", "glm4_moe", "glm4_moe-groups", "qwen3", "qwen3-tied", "qwen3_moe", "qwen3_moe-raw-topk", "qwen2", "llama", "llama-rope-llama3", "llama-rope-linear",
         "mistral", "mixtral"]


def _my_logits(cfg: ModelConfig, store, tokens):
    model = build_model(cfg, store, "torch")
    lens = [len(tokens)]
    with torch.no_grad():
        h = model.forward_hidden(tokens.int(), torch.arange(lens[0]).int(), torch.tensor([0, lens[0]], dtype=torch.int32))
        return model.logits(h)


@pytest.mark.parametrize("name", CASES)
def test_logits_match_huggingface_both_ways(name, tmp_path):
    torch.manual_seed(0)
    hf_cfg, cls = _case(name)
    hf = cls(hf_cfg).float().eval()
    with torch.no_grad():  # HF initialises norms to one and biases to zero: make them matter
        for n, p in hf.named_parameters():
            if n.endswith("norm.weight") or n.endswith(".bias"):
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.add_(torch.randn_like(b) * 0.3)  # a selection bias that changes which experts win
    src = tmp_path / "hf"
    hf.save_pretrained(src, safe_serialization=True)
    cfg = ModelConfig.from_hf_config(str(src))
    assert cfg.hf_architecture == cls.__name__
    store = ParamStore(cfg, "cpu", torch.float32, init=False)
    n_loaded = load_hf(cfg, store, str(src))
    assert n_loaded >= len(list(hf.state_dict())) - (1 if hf_cfg.tie_word_embeddings else 0) - 2
    tokens = torch.randint(0, 256, (200,))  # longer than the scaled-rope "original" length, so scaling matters
    with torch.no_grad():
        ref = hf(tokens[None]).logits[0]
    out = _my_logits(cfg, store, tokens)
    assert torch.allclose(out, ref, atol=2e-4, rtol=1e-4), (name, (out - ref).abs().max().item())
    # ... and back: export under HF names, load with HF, same logits
    from safetensors.torch import save_file
    import json

    dst = tmp_path / "export"
    dst.mkdir()
    save_file({k: v.detach().clone().contiguous() for k, v in hf_names(cfg, store)}, str(dst / "model.safetensors"), metadata={"format": "pt"})
    (dst / "config.json").write_text(json.dumps(cfg.to_hf_config()))
    back = transformers.AutoModelForCausalLM.from_pretrained(str(dst), torch_dtype=torch.float32).eval()
    assert type(back).__name__ == cls.__name__
    with torch.no_grad():
        again = back(tokens[None]).logits[0]
    assert torch.allclose(again, ref, atol=2e-4, rtol=1e-4), (name, (again - ref).abs().max().item())


def test_unsupported_checkpoints_are_refused():
    with pytest.raises(NotImplementedError):
        ModelConfig.from_hf_config({"architectures": ["DeepseekV3ForCausalLM"], "model_type": "deepseek_v3", "num_attention_heads": 4,
                                    "hidden_size": 64, "num_hidden_layers": 1, "vocab_size": 10})
    base = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_attention_heads": 4, "hidden_size": 64,
            "num_hidden_layers": 1, "vocab_size": 10, "intermediate_size": 8}
    with pytest.raises(NotImplementedError):
        ModelConfig.from_hf_config(dict(base, rope_scaling={"rope_type": "yarn", "factor": 4.0}))
    with pytest.raises(NotImplementedError):
        ModelConfig.from_hf_config(dict(base, architectures=["MistralForCausalLM"], model_type="mistral", sliding_window=128,
                                        max_position_embeddings=4096))
    assert ModelConfig.from_hf_config(dict(base, rope_scaling=LLAMA3_SCALING)).rope_scaling["rope_type"] == "llama3"


def test_megatron_style_flags_describe_a_glm45_like_model():
    from miles_b200.utils.arguments import model_config_from_args, parse_args

    a = parse_args(["--num-rollout", "1", "--rollout-batch-size", "2", "--num-layers", "3", "--hidden-size", "512",
                    "--num-attention-heads", "8", "--num-query-groups", "2", "--kv-channels", "128", "--ffn-hidden-size", "1024",
                    "--vocab-size", "4096", "--num-experts", "16", "--moe-router-topk", "4", "--moe-ffn-hidden-size", "256",
                    "--moe-router-score-function", "sigmoid", "--moe-router-enable-expert-bias", "--moe-router-topk-scaling-factor", "2.5",
                    "--moe-shared-expert-intermediate-size", "256", "--moe-layer-freq", "[0]*1+[1]*2", "--rotary-percent", "0.5",
                    "--qk-layernorm", "--add-qkv-bias", "--untie-embeddings-and-output-weights"])
    cfg = model_config_from_args(a)
    assert (cfg.router_score, cfg.router_bias, cfg.routed_scaling_factor, cfg.shared_expert_ffn) == ("sigmoid", True, 2.5, 256)
    assert cfg.first_dense_layers == 1 and cfg.rotary_dim == 64 and cfg.family == "glm4_moe"
    assert [cfg.layer_is_moe(i) for i in range(3)] == [False, True, True]
    from miles_b200.models import get_config

    ref = get_config("glm4moe-smoke")
    store_a = ParamStore(cfg, "cpu", torch.float32, meta=True, init=False)
    store_b = ParamStore(ref, "cpu", torch.float32, meta=True, init=False)
    assert [(s.name, s.shape) for s in store_a.specs] == [(s.name, s.shape) for s in store_b.specs]


GLM45_AIR_FLAGS = ("--disable-bias-linear --group-query-attention --num-attention-heads 96 --num-query-groups 8 --kv-channels 128 "
                   "--num-layers 46 --hidden-size 4096 --ffn-hidden-size 10944 --add-qkv-bias --normalization RMSNorm "
                   "--position-embedding-type rope --rotary-percent 0.5 --swiglu --untie-embeddings-and-output-weights "
                   "--vocab-size 151552 --rotary-base 1000000 --moe-ffn-hidden-size 1408 --moe-shared-expert-intermediate-size 1408 "
                   "--moe-router-pre-softmax --moe-router-score-function sigmoid --moe-router-enable-expert-bias "
                   "--moe-router-bias-update-rate 0 --moe-router-load-balancing-type seq_aux_loss --moe-token-dispatcher-type alltoall "
                   "--moe-router-topk 8 --moe-layer-freq [0]*1+[1]*45 --num-experts 128 --moe-grouped-gemm --moe-router-dtype fp32 "
                   "--moe-permute-fusion --moe-aux-loss-coeff 0")
QWEN3_30B_FLAGS = ("--disable-bias-linear --qk-layernorm --group-query-attention --num-attention-heads 32 --num-query-groups 4 "
                   "--kv-channels 128 --num-layers 48 --hidden-size 2048 --ffn-hidden-size 6144 --normalization RMSNorm "
                   "--position-embedding-type rope --norm-epsilon 1e-6 --rotary-percent 1.0 --swiglu "
                   "--untie-embeddings-and-output-weights --vocab-size 151936 --rotary-base 1000000 --moe-ffn-hidden-size 768 "
                   "--moe-router-score-function softmax --moe-token-dispatcher-type alltoall --moe-router-topk 8 --moe-layer-freq [1]*48 "
                   "--num-experts 128 --moe-grouped-gemm --moe-token-drop-policy probs --moe-router-dtype fp32 --moe-permute-fusion "
                   "--moe-aux-loss-coeff 0")


@pytest.mark.parametrize("flags,preset", [(GLM45_AIR_FLAGS, "glm4.5-106B-A12B"), (QWEN3_30B_FLAGS, "qwen3-30B-A3B")])
def test_reference_model_argument_strings_describe_our_presets(flags, preset):
    """The Megatron-style argument strings the reference's per-model files pass (scripts/models/glm4.5-106B-A12B.py,
    qwen3-30B-A3B.py) parse here and give the same parameter layout as the preset of that model."""
    from miles_b200.models import get_config
    from miles_b200.utils.arguments import model_config_from_args, parse_args

    a = parse_args(["--num-rollout", "1", "--rollout-batch-size", "2"] + flags.split())
    cfg, ref = model_config_from_args(a), get_config(preset)
    sa = ParamStore(cfg, "cpu", torch.float32, meta=True, init=False)
    sb = ParamStore(ref, "cpu", torch.float32, meta=True, init=False)
    assert [(s.name, s.shape) for s in sa.specs] == [(s.name, s.shape) for s in sb.specs]
    for f in ("num_q_heads", "num_kv_heads", "head_dim", "rope_theta", "qk_norm", "qkv_bias", "router_score", "router_bias",
              "routed_scaling_factor", "norm_topk_prob", "rotary_dim", "first_dense_layers", "moe_top_k", "tie_embeddings"):
        assert getattr(cfg, f) == getattr(ref, f), (f, getattr(cfg, f), getattr(ref, f))


LLAMA31_FLAGS = ("--swiglu --num-layers 32 --hidden-size 4096 --ffn-hidden-size 14336 --num-attention-heads 32 --group-query-attention "
                 "--num-query-groups 8 --max-position-embeddings 131072 --use-rotary-position-embeddings --disable-bias-linear "
                 "--normalization RMSNorm --norm-epsilon 1e-5 --rotary-base 500000 --vocab-size 128256 --kv-channels 128 "
                 "--use-rope-scaling --rotary-scaling-factor 8.0 --untie-embeddings-and-output-weights")
MIMO_FLAGS = ("--swiglu --num-layers 36 --hidden-size 4096 --ffn-hidden-size 11008 --num-attention-heads 32 --group-query-attention "
              "--num-query-groups 8 --use-rotary-position-embeddings --disable-bias-linear --add-qkv-bias --normalization RMSNorm "
              "--norm-epsilon 1e-05 --rotary-base 640000 --vocab-size 151680 --untie-embeddings-and-output-weights "
              "--max-position-embeddings 32768 --mtp-num-layers 1")
GLM4_32B_FLAGS = ("--spec miles_plugins.models.glm4 get_glm_spec --swiglu --num-layers 64 --hidden-size 6144 --ffn-hidden-size 23040 "
                  "--num-attention-heads 48 --max-position-embeddings 32768 --seq-length 32768 --use-rotary-position-embeddings "
                  "--disable-bias-linear --normalization RMSNorm --norm-epsilon 1e-5 --rotary-base 10000 --group-query-attention "
                  "--num-query-groups 8 --vocab-size 151552 --post-self-attn-layernorm --post-mlp-layernorm --rotary-interleaved "
                  "--rotary-percent 0.5 --no-rope-fusion --untie-embeddings-and-output-weights")


@pytest.mark.parametrize("flags,preset", [(LLAMA31_FLAGS, "llama3.1-8B-Instruct"), (MIMO_FLAGS, "mimo-7B-rl"), (GLM4_32B_FLAGS, "glm4-32B")])
def test_more_reference_argument_strings(flags, preset):
    """scripts/models/{llama3.1-8B-Instruct,mimo-7B-rl,glm4-32B}.py of the reference."""
    import warnings

    from miles_b200.models import get_config
    from miles_b200.utils.arguments import model_config_from_args, parse_args

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")  # flags that change nothing here are announced once
        a = parse_args(["--num-rollout", "1", "--rollout-batch-size", "2"] + flags.split())
    cfg, ref = model_config_from_args(a), get_config(preset)
    sa = ParamStore(cfg, "cpu", torch.float32, meta=True, init=False)
    sb = ParamStore(ref, "cpu", torch.float32, meta=True, init=False)
    assert [(s.name, s.shape) for s in sa.specs] == [(s.name, s.shape) for s in sb.specs]
    for f in ("num_q_heads", "num_kv_heads", "head_dim", "rope_theta", "rms_eps", "qk_norm", "qkv_bias", "rotary_dim", "post_norms",
              "rope_interleaved", "tie_embeddings", "rope_scaling", "family"):
        assert getattr(cfg, f) == getattr(ref, f), (f, getattr(cfg, f), getattr(ref, f))


@pytest.mark.parametrize("name", ["qwen3", "qwen3_moe", "llama-rope-llama3", "mixtral", "glm4", "glm4_moe", "qwen2_moe"])
def test_engine_greedy_decoding_matches_huggingface_generate(name, tmp_path):
    """The rollout engine (paged KV cache, prefill then one token per step, prefix cache on) against ``model.generate`` of the
    HuggingFace implementation: same greedy continuation for several prompts of different lengths."""
    from miles_b200.engine import Engine, SamplingParams

    torch.manual_seed(1)
    hf_cfg, cls = _case(name)
    hf = cls(hf_cfg).float().eval()
    src = tmp_path / "hf"
    hf.save_pretrained(src, safe_serialization=True)
    cfg = ModelConfig.from_hf_config(str(src))
    store = ParamStore(cfg, "cpu", torch.float32, init=False)
    load_hf(cfg, store, str(src))
    eng = Engine(build_model(cfg, store, "torch"), max_running=4, page_size=8, max_seq_len=128, prefix_cache=True)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(2, 256, (n,), generator=g).tolist() for n in (5, 19, 33)]
    prompts.append(prompts[2][:24] + [7, 8, 9])  # shares three pages with the previous prompt
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        with torch.no_grad():
            ref = hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, pad_token_id=0, eos_token_id=None)[0, len(p):].tolist()
        assert o["output_ids"] == ref, (name, len(p), o["output_ids"], ref)
    assert outs[3]["meta_info"]["cached_tokens"] == 24

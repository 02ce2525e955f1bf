"""Model shape configuration and presets for the Qwen3 dense / Qwen3-MoE families (and Qwen2/Llama-style
dense models, which differ only in qk-norm and qkv bias).

Preset shapes follow the reference's per-model argument files (scripts/models/qwen3-4B.py:6-22,
scripts/models/qwen3-30B-A3B.py:14-42) and the HF ``config.json`` field names, which ``from_hf_config``
reads (the reference cross-checks the same fields in miles/utils/arguments.py:3656-3707).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Optional


@dataclass
class ModelConfig:
    name: str = "qwen3-tiny"
    num_layers: int = 2
    hidden_size: int = 256
    num_q_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    ffn_hidden_size: int = 768
    vocab_size: int = 1024
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    qk_norm: bool = True
    qkv_bias: bool = False
    tie_embeddings: bool = False
    # MoE (num_experts == 0 -> dense MLP in every layer)
    num_experts: int = 0
    moe_top_k: int = 0
    moe_ffn_hidden_size: int = 0
    norm_topk_prob: bool = True
    moe_layer_freq: int = 1  # every n-th layer is MoE (1 = all)
    first_dense_layers: int = 0
    # router variants (GLM-4.5 / DeepSeek-V3 style): scores = sigmoid(logits); experts are chosen by score + a per-expert
    # bias (not trained by gradients), optionally inside the best ``topk_group`` of ``n_group`` expert groups; the
    # weights are the chosen scores (renormalised when norm_topk_prob) times ``routed_scaling_factor``
    router_score: str = "softmax"  # "softmax" | "sigmoid"
    router_bias: bool = False
    routed_scaling_factor: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    # a dense SwiGLU expert of this width that every token passes through, added to the routed experts' output
    shared_expert_ffn: int = 0
    # Qwen2-MoE: the shared expert's output is scaled per token by sigmoid(hidden . gate vector)
    shared_expert_gate: bool = False
    # rotary embedding on the first ``rotary_dim`` dimensions of every head only (0 = all of them)
    rotary_dim: int = 0
    # GLM-4 dense: an extra RMSNorm on the attention output and on the MLP output before each joins the residual stream
    post_norms: bool = False
    # the checkpoint's query / key rows pair dimension 2i with 2i + 1 (GLM-4 dense); rows are de-interleaved when read and
    # interleaved again when written, so that the model itself always rotates halves (attention scores do not change
    # under a permutation applied to queries and keys alike)
    rope_interleaved: bool = False
    max_position_embeddings: int = 40960
    # scaled rotary embeddings: None, {"rope_type": "llama3", "factor", "low_freq_factor", "high_freq_factor",
    # "original_max_position_embeddings"} or {"rope_type": "linear", "factor"}
    rope_scaling: Optional[dict] = None
    hf_architecture: str = "Qwen3ForCausalLM"
    extra: dict[str, Any] = field(default_factory=dict)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def q_dim(self) -> int:
        return self.num_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    def layer_is_moe(self, i: int) -> bool:
        return self.is_moe and i >= self.first_dense_layers and ((i + 1) % self.moe_layer_freq == 0)

    def num_params(self) -> int:
        n = self.vocab_size * self.hidden_size * (1 if self.tie_embeddings else 2) + self.hidden_size
        for i in range(self.num_layers):
            n += (4 if self.post_norms else 2) * self.hidden_size + self.qkv_dim * self.hidden_size + self.q_dim * self.hidden_size
            if self.qk_norm:
                n += 2 * self.head_dim
            if self.qkv_bias:
                n += self.qkv_dim
            if self.layer_is_moe(i):
                n += self.num_experts * self.hidden_size + (self.num_experts if self.router_bias else 0)
                n += self.num_experts * 3 * self.moe_ffn_hidden_size * self.hidden_size
                n += 3 * self.shared_expert_ffn * self.hidden_size + (self.hidden_size if self.shared_expert_gate else 0)
            else:
                n += 3 * self.ffn_hidden_size * self.hidden_size
        return n

    def num_active_params(self) -> int:
        if not self.is_moe:
            return self.num_params()
        n = self.num_params()
        for i in range(self.num_layers):
            if self.layer_is_moe(i):
                n -= (self.num_experts - self.moe_top_k) * 3 * self.moe_ffn_hidden_size * self.hidden_size
        return n

    def to_dict(self) -> dict:
        return asdict(self)

    # ------------------------------------------------------------------ HF interop
    @property
    def family(self) -> str:
        """The HuggingFace ``model_type`` of this architecture (decides config keys and tensor names)."""
        return HF_FAMILIES.get(self.hf_architecture, "qwen3_moe" if self.is_moe else "qwen3")

    def to_hf_config(self) -> dict:
        cfg = {
            "architectures": [self.hf_architecture],
            "model_type": self.family,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_q_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.ffn_hidden_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_embeddings,
            "attention_bias": self.qkv_bias,
            "max_position_embeddings": self.max_position_embeddings,
            "torch_dtype": "bfloat16",
        }
        if self.rope_scaling:
            cfg["rope_scaling"] = dict(self.rope_scaling)
        # token ids and similar keys of the checkpoint this model was read from travel back out unchanged
        cfg.update(self.extra.get("hf_passthrough", {}))
        if self.family in ("glm4", "glm4_moe") and "pad_token_id" not in cfg and self.vocab_size <= 151329:
            cfg["pad_token_id"] = None  # the library's default padding id assumes the full GLM vocabulary
        if self.family == "glm4":
            cfg["partial_rotary_factor"] = (self.rotary_dim or self.head_dim) / self.head_dim
        if self.family in ("glm4_moe", "dots1"):
            cfg.update({"n_routed_experts": self.num_experts, "num_experts_per_tok": self.moe_top_k,
                        "moe_intermediate_size": self.moe_ffn_hidden_size, "norm_topk_prob": self.norm_topk_prob,
                        "n_shared_experts": self.shared_expert_ffn // max(self.moe_ffn_hidden_size, 1),
                        "routed_scaling_factor": self.routed_scaling_factor, "n_group": self.n_group, "topk_group": self.topk_group,
                        "first_k_dense_replace": self.first_dense_layers, "use_qk_norm": self.qk_norm,
                        "partial_rotary_factor": (self.rotary_dim or self.head_dim) / self.head_dim})
        elif self.family == "qwen2_moe":
            cfg.update({"num_experts": self.num_experts, "num_experts_per_tok": self.moe_top_k,
                        "moe_intermediate_size": self.moe_ffn_hidden_size, "norm_topk_prob": self.norm_topk_prob,
                        "shared_expert_intermediate_size": self.shared_expert_ffn, "decoder_sparse_step": self.moe_layer_freq,
                        "mlp_only_layers": list(range(self.first_dense_layers))})
        elif self.family == "mixtral":
            cfg.update({"num_local_experts": self.num_experts, "num_experts_per_tok": self.moe_top_k,
                        "intermediate_size": self.moe_ffn_hidden_size, "sliding_window": None})
        elif self.is_moe:
            cfg.update({
                "num_experts": self.num_experts,
                "num_experts_per_tok": self.moe_top_k,
                "moe_intermediate_size": self.moe_ffn_hidden_size,
                "norm_topk_prob": self.norm_topk_prob,
                "decoder_sparse_step": self.moe_layer_freq,
                "mlp_only_layers": list(range(self.first_dense_layers)),
            })
        return cfg

    @classmethod
    def from_hf_config(cls, cfg: dict | str | Path, name: str | None = None) -> "ModelConfig":
        if not isinstance(cfg, dict):
            p = Path(cfg)
            if p.is_dir():
                p = p / "config.json"
            cfg = json.loads(p.read_text())
        arch = (cfg.get("architectures") or ["Qwen3ForCausalLM"])[0]
        heads = cfg["num_attention_heads"]
        head_dim = cfg.get("head_dim") or cfg["hidden_size"] // heads
        mtype = (cfg.get("model_type") or HF_FAMILIES.get(arch, "qwen3")).lower()
        if arch not in HF_FAMILIES:
            raise NotImplementedError(f"{arch} ({mtype}) is not one of the architectures this package implements: "
                                      f"{', '.join(sorted(HF_FAMILIES))}")
        is_qwen3 = "qwen3" in mtype
        mlp_only = cfg.get("mlp_only_layers") or []
        n_experts = cfg.get("num_experts", 0) or cfg.get("num_local_experts", 0) or cfg.get("n_routed_experts", 0) or 0
        dots = mtype == "dots1"        # dots.llm1: the GLM-4.5 router and shared experts with full rotary embedding and QK norm
        glm = mtype == "glm4_moe" or dots
        glm_dense = mtype == "glm4"
        if any(t != "full_attention" for t in (cfg.get("layer_types") or [])):
            raise NotImplementedError("layers with sliding-window or linear attention are not built")
        prf = cfg.get("partial_rotary_factor") or (cfg.get("rope_parameters") or {}).get("partial_rotary_factor") or 1.0
        if not (glm or glm_dense) and float(prf) != 1.0:  # (Phi-4-mini's 0.75 among them: the kernels rotate 128 or 64 dimensions)
            raise NotImplementedError(f"partial rotary embedding is wired for the GLM families only (got {prf} for {mtype})")
        moe_ffn = cfg.get("moe_intermediate_size", 0) or (cfg.get("intermediate_size", 0) if mtype == "mixtral" else 0)
        if mtype == "ernie4_5" and cfg.get("use_bias"):
            raise NotImplementedError("biases on every projection (use_bias) are not built")
        if mtype == "seed_oss" and (cfg.get("attention_out_bias") or cfg.get("mlp_bias")):
            raise NotImplementedError("biases on the attention output or MLP projections are not built")
        if cfg.get("sliding_window") and cfg.get("use_sliding_window", mtype not in ("qwen2", "qwen2_moe", "dots1") and not is_qwen3) \
                and cfg["sliding_window"] < cfg.get("max_position_embeddings", 0):
            raise NotImplementedError("sliding-window attention is not built: this checkpoint would be served with full attention")
        scaling = cfg.get("rope_scaling") or None
        if scaling is None and isinstance(cfg.get("rope_parameters"), dict) and cfg["rope_parameters"].get("rope_type") not in (None, "default"):
            scaling = {k: v for k, v in cfg["rope_parameters"].items() if k != "rope_theta"}
        if scaling:
            kind = scaling.get("rope_type") or scaling.get("type") or "default"
            if kind == "default":
                scaling = None
            elif kind in ("llama3", "linear"):
                scaling = dict(scaling, rope_type=kind)
                scaling.pop("type", None)
            else:
                raise NotImplementedError(f"rope scaling of type {kind!r} is not built (llama3 and linear are)")
        return cls(
            name=name or cfg.get("_name_or_path", arch),
            num_layers=cfg["num_hidden_layers"],
            hidden_size=cfg["hidden_size"],
            num_q_heads=heads,
            num_kv_heads=cfg.get("num_key_value_heads", heads),
            head_dim=head_dim,
            ffn_hidden_size=cfg.get("intermediate_size", 0),
            vocab_size=cfg["vocab_size"],
            rms_eps=cfg.get("rms_norm_eps", 1e-6),
            # newer HuggingFace configs keep the base inside "rope_parameters"; 10000 is the library-wide default
            rope_theta=float(cfg.get("rope_theta") or (cfg.get("rope_parameters") or {}).get("rope_theta") or 10000.0),
            qk_norm=True if dots else bool(cfg.get("use_qk_norm", False)) if glm else is_qwen3,
            qkv_bias=bool(cfg.get("attention_bias", (not is_qwen3 and "qwen2" in mtype) or glm_dense or mtype == "seed_oss")),
            tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            num_experts=n_experts,
            moe_top_k=(cfg.get("num_experts_per_tok", 0) or 0) if n_experts else 0,
            moe_ffn_hidden_size=moe_ffn,
            # Mixtral takes the softmax over the chosen experts only, which equals renormalising the full softmax
            norm_topk_prob=True if mtype == "mixtral" else bool(cfg.get("norm_topk_prob", mtype != "qwen2_moe")),
            moe_layer_freq=cfg.get("decoder_sparse_step", 1) or 1,
            first_dense_layers=int(cfg.get("first_k_dense_replace", 0) or 0) if glm else ((max(mlp_only) + 1) if mlp_only else 0),
            router_score="sigmoid" if glm else "softmax", router_bias=glm,
            routed_scaling_factor=float(cfg.get("routed_scaling_factor", 1.0) or 1.0) if glm else 1.0,
            n_group=int(cfg.get("n_group", 1) or 1) if glm else 1, topk_group=int(cfg.get("topk_group", 1) or 1) if glm else 1,
            shared_expert_ffn=((int(cfg.get("n_shared_experts", 0) or 0) * moe_ffn) if glm
                               else int(cfg.get("shared_expert_intermediate_size", 0) or 0) if mtype == "qwen2_moe" else 0),
            shared_expert_gate=mtype == "qwen2_moe",
            rotary_dim=int(round(head_dim * float(prf))) if float(prf) != 1.0 else 0,
            post_norms=glm_dense, rope_interleaved=glm_dense or mtype == "ernie4_5",
            extra={"hf_passthrough": {k: cfg[k] for k in ("pad_token_id", "eos_token_id", "bos_token_id") if k in cfg}},
            max_position_embeddings=cfg.get("max_position_embeddings", 40960),
            rope_scaling=scaling,
            hf_architecture=arch,
        )


# architectures this package implements -> HuggingFace model_type
HF_FAMILIES = {
    "Qwen3ForCausalLM": "qwen3", "Qwen3MoeForCausalLM": "qwen3_moe", "Qwen2ForCausalLM": "qwen2", "LlamaForCausalLM": "llama",
    "MistralForCausalLM": "mistral", "MixtralForCausalLM": "mixtral", "MiMoForCausalLM": "mimo",
    "Glm4MoeForCausalLM": "glm4_moe", "Glm4ForCausalLM": "glm4", "Qwen2MoeForCausalLM": "qwen2_moe",
    "Dots1ForCausalLM": "dots1", "SeedOssForCausalLM": "seed_oss", "Ernie4_5ForCausalLM": "ernie4_5",
    "Phi3ForCausalLM": "phi3",
}


def _dense(name, L, H, q, kv, ffn, tie, vocab=151936, hd=128, **kw) -> ModelConfig:
    return ModelConfig(name=name, num_layers=L, hidden_size=H, num_q_heads=q, num_kv_heads=kv, head_dim=hd,
                       ffn_hidden_size=ffn, vocab_size=vocab, tie_embeddings=tie, **kw)


def _moe(name, L, H, q, kv, E, k, moe_ffn, vocab=151936, hd=128, **kw) -> ModelConfig:
    return ModelConfig(name=name, num_layers=L, hidden_size=H, num_q_heads=q, num_kv_heads=kv, head_dim=hd,
                       ffn_hidden_size=moe_ffn, vocab_size=vocab, num_experts=E, moe_top_k=k, moe_ffn_hidden_size=moe_ffn,
                       hf_architecture="Qwen3MoeForCausalLM", **kw)


PRESETS: dict[str, ModelConfig] = {
    # CPU plumbing model of the tiny GRPO configuration
    "qwen3-tiny": ModelConfig(),
    "qwen3-tiny-moe": ModelConfig(name="qwen3-tiny-moe", num_experts=8, moe_top_k=2, moe_ffn_hidden_size=128,
                                  hf_architecture="Qwen3MoeForCausalLM"),
    # a small GPU smoke model with head_dim 128 (the kernels' native head size)
    "qwen3-smoke": _dense("qwen3-smoke", 2, 512, 4, 2, 1024, False, vocab=4096),
    "qwen3-smoke-moe": _moe("qwen3-smoke-moe", 2, 512, 8, 2, 16, 4, 256, vocab=4096),
    # the same size in the other families' conventions: no QK norm, scaled rotary embedding / Mixtral expert naming
    "llama3-smoke": _dense("llama3-smoke", 2, 512, 4, 2, 1024, False, vocab=4096, qk_norm=False, rope_theta=5e5, rms_eps=1e-5,
                           hf_architecture="LlamaForCausalLM", max_position_embeddings=131072,
                           rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                         "original_max_position_embeddings": 8192}),
    "mixtral-smoke": ModelConfig(name="mixtral-smoke", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                                 ffn_hidden_size=256, vocab_size=4096, rms_eps=1e-5, qk_norm=False, num_experts=8, moe_top_k=2,
                                 moe_ffn_hidden_size=256, hf_architecture="MixtralForCausalLM"),
    "qwen3-0.6B": _dense("qwen3-0.6B", 28, 1024, 16, 8, 3072, True),
    "qwen3-1.7B": _dense("qwen3-1.7B", 28, 2048, 16, 8, 6144, True),
    "qwen3-4B": _dense("qwen3-4B", 36, 2560, 32, 8, 9728, True),
    "qwen3-8B": _dense("qwen3-8B", 36, 4096, 32, 8, 12288, False),
    "qwen3-14B": _dense("qwen3-14B", 40, 5120, 40, 8, 17408, False),
    "qwen3-32B": _dense("qwen3-32B", 64, 5120, 64, 8, 25600, False),
    "qwen3-30B-A3B": _moe("qwen3-30B-A3B", 48, 2048, 32, 4, 128, 8, 768),
    "qwen3-235B-A22B": _moe("qwen3-235B-A22B", 94, 4096, 64, 4, 128, 8, 1536),
    "qwen2.5-0.5B": _dense("qwen2.5-0.5B", 24, 896, 14, 2, 4864, True, hd=64, qk_norm=False, qkv_bias=True,
                           rope_theta=1e6, hf_architecture="Qwen2ForCausalLM"),
    "qwen2.5-7B": _dense("qwen2.5-7B", 28, 3584, 28, 4, 18944, False, vocab=152064, qk_norm=False, qkv_bias=True,
                         hf_architecture="Qwen2ForCausalLM"),
    "qwen2.5-1.5B": _dense("qwen2.5-1.5B", 28, 1536, 12, 2, 8960, True, qk_norm=False, qkv_bias=True, rope_theta=1e6,
                           hf_architecture="Qwen2ForCausalLM"),
    "qwen2.5-3B": _dense("qwen2.5-3B", 36, 2048, 16, 2, 11008, True, qk_norm=False, qkv_bias=True, rope_theta=1e6,
                         hf_architecture="Qwen2ForCausalLM"),
    "qwen2.5-14B": _dense("qwen2.5-14B", 48, 5120, 40, 8, 13824, False, vocab=152064, qk_norm=False, qkv_bias=True, rope_theta=1e6,
                          hf_architecture="Qwen2ForCausalLM"),
    "qwen2.5-32B": _dense("qwen2.5-32B", 64, 5120, 40, 8, 27648, False, vocab=152064, qk_norm=False, qkv_bias=True, rope_theta=1e6,
                          hf_architecture="Qwen2ForCausalLM"),
    "qwen2.5-72B": _dense("qwen2.5-72B", 80, 8192, 64, 8, 29568, False, vocab=152064, qk_norm=False, qkv_bias=True, rope_theta=1e6,
                          hf_architecture="Qwen2ForCausalLM"),
    "llama-3.2-1B": _dense("llama-3.2-1B", 16, 2048, 32, 8, 8192, True, vocab=128256, hd=64, qk_norm=False,
                           rope_theta=5e5, rms_eps=1e-5, hf_architecture="LlamaForCausalLM",
                           rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}, max_position_embeddings=131072),
    "llama-3.2-3B": _dense("llama-3.2-3B", 28, 3072, 24, 8, 8192, True, vocab=128256, qk_norm=False,
                           rope_theta=5e5, rms_eps=1e-5, hf_architecture="LlamaForCausalLM",
                           rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}, max_position_embeddings=131072),
    "llama-3.1-70B": _dense("llama-3.1-70B", 80, 8192, 64, 8, 28672, False, vocab=128256, qk_norm=False,
                            rope_theta=5e5, rms_eps=1e-5, hf_architecture="LlamaForCausalLM",
                           rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}, max_position_embeddings=131072),
    "mistral-7B": _dense("mistral-7B", 32, 4096, 32, 8, 14336, False, vocab=32768, qk_norm=False,
                         rope_theta=1e6, rms_eps=1e-5, hf_architecture="MistralForCausalLM"),
    "llama-3.1-8B": _dense("llama-3.1-8B", 32, 4096, 32, 8, 14336, False, vocab=128256, qk_norm=False,
                           rope_theta=5e5, rms_eps=1e-5, hf_architecture="LlamaForCausalLM",
                           rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}, max_position_embeddings=131072),
    # Mixtral: 8 experts, top-2, the softmax taken over the chosen experts (= renormalised top-k of the full softmax)
    "mixtral-8x7B": ModelConfig(name="mixtral-8x7B", num_layers=32, hidden_size=4096, num_q_heads=32, num_kv_heads=8, head_dim=128,
                                ffn_hidden_size=14336, vocab_size=32000, rms_eps=1e-5, rope_theta=1e6, qk_norm=False, num_experts=8,
                                moe_top_k=2, moe_ffn_hidden_size=14336, max_position_embeddings=32768,
                                hf_architecture="MixtralForCausalLM"),
    "mixtral-8x22B": ModelConfig(name="mixtral-8x22B", num_layers=56, hidden_size=6144, num_q_heads=48, num_kv_heads=8, head_dim=128,
                                 ffn_hidden_size=16384, vocab_size=32768, rms_eps=1e-5, rope_theta=1e6, qk_norm=False, num_experts=8,
                                 moe_top_k=2, moe_ffn_hidden_size=16384, max_position_embeddings=65536,
                                 hf_architecture="MixtralForCausalLM"),
    # GLM-4.5: sigmoid router with a selection bias, one shared expert, rotary embedding on half of every head, a dense
    # first layer (their multi-token-prediction layer is not trained here)
    "glm4.5-106B-A12B": ModelConfig(name="glm4.5-106B-A12B", num_layers=46, hidden_size=4096, num_q_heads=96, num_kv_heads=8,
                                    head_dim=128, ffn_hidden_size=10944, vocab_size=151552, rms_eps=1e-5, rope_theta=1e6,
                                    qk_norm=False, qkv_bias=True, num_experts=128, moe_top_k=8, moe_ffn_hidden_size=1408,
                                    first_dense_layers=1, router_score="sigmoid", router_bias=True, routed_scaling_factor=1.0,
                                    shared_expert_ffn=1408, rotary_dim=64, max_position_embeddings=131072,
                                    hf_architecture="Glm4MoeForCausalLM"),
    "glm4.5-355B-A32B": ModelConfig(name="glm4.5-355B-A32B", num_layers=92, hidden_size=5120, num_q_heads=96, num_kv_heads=8,
                                    head_dim=128, ffn_hidden_size=12288, vocab_size=151552, rms_eps=1e-5, rope_theta=1e6,
                                    qk_norm=True, qkv_bias=True, num_experts=160, moe_top_k=8, moe_ffn_hidden_size=1536,
                                    first_dense_layers=3, router_score="sigmoid", router_bias=True, routed_scaling_factor=2.5,
                                    shared_expert_ffn=1536, rotary_dim=64, max_position_embeddings=131072,
                                    hf_architecture="Glm4MoeForCausalLM"),
    # Phi-4 (14B): Llama layout with the query / key / value rows and the gate / up rows fused in the checkpoint as well
    "phi-4": _dense("phi-4", 40, 5120, 40, 10, 17920, False, vocab=100352, qk_norm=False, rope_theta=250000.0, rms_eps=1e-5,
                    max_position_embeddings=16384, hf_architecture="Phi3ForCausalLM"),
    # ERNIE-4.5-0.3B: Llama layout whose checkpoints pair rotary dimensions 2i / 2i + 1
    "ernie4.5-0.3B": _dense("ernie4.5-0.3B", 18, 1024, 16, 2, 3072, True, vocab=103424, qk_norm=False, rope_theta=5e5, rms_eps=1e-5,
                            rope_interleaved=True, max_position_embeddings=131072, hf_architecture="Ernie4_5ForCausalLM"),
    # Seed-OSS-36B: Llama layout with QKV bias; dots.llm1 (142B total, 14B active): GLM-4.5 style router with QK norm
    "seed-oss-36B": _dense("seed-oss-36B", 64, 5120, 80, 8, 27648, False, vocab=155136, qk_norm=False, qkv_bias=True, rope_theta=1e7,
                           rms_eps=1e-6, max_position_embeddings=524288, hf_architecture="SeedOssForCausalLM"),
    "dots-llm1": ModelConfig(name="dots-llm1", num_layers=62, hidden_size=4096, num_q_heads=32, num_kv_heads=32, head_dim=128,
                             ffn_hidden_size=10944, vocab_size=152064, rms_eps=1e-5, rope_theta=1e7, qk_norm=True, num_experts=128,
                             moe_top_k=6, moe_ffn_hidden_size=1408, first_dense_layers=1, router_score="sigmoid", router_bias=True,
                             routed_scaling_factor=2.5, shared_expert_ffn=2816, max_position_embeddings=32768,
                             hf_architecture="Dots1ForCausalLM"),
    # Qwen2-MoE (Qwen1.5-MoE-A2.7B, Qwen2-57B-A14B): softmax router without renormalisation, a gated shared expert
    "qwen2-57B-A14B": ModelConfig(name="qwen2-57B-A14B", num_layers=28, hidden_size=3584, num_q_heads=28, num_kv_heads=4, head_dim=128,
                                  ffn_hidden_size=18944, vocab_size=151936, rms_eps=1e-6, rope_theta=1e6, qk_norm=False, qkv_bias=True,
                                  num_experts=64, moe_top_k=8, moe_ffn_hidden_size=2560, norm_topk_prob=False,
                                  shared_expert_ffn=20480, shared_expert_gate=True, max_position_embeddings=32768,
                                  hf_architecture="Qwen2MoeForCausalLM"),
    "qwen2moe-smoke": ModelConfig(name="qwen2moe-smoke", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                                  ffn_hidden_size=1024, vocab_size=4096, rms_eps=1e-6, qk_norm=False, qkv_bias=True, num_experts=16,
                                  moe_top_k=4, moe_ffn_hidden_size=256, norm_topk_prob=False, shared_expert_ffn=512,
                                  shared_expert_gate=True, hf_architecture="Qwen2MoeForCausalLM"),
    # GLM-4 dense (GLM-4-0414 / GLM-Z1): sandwich norms, rotary embedding on half of every head (interleaved in the checkpoint)
    "glm4-9B": _dense("glm4-9B", 40, 4096, 32, 2, 13696, False, vocab=151552, qk_norm=False, qkv_bias=True, rope_theta=1e4,
                      rms_eps=1e-5, rotary_dim=64, post_norms=True, rope_interleaved=True, max_position_embeddings=32768,
                      hf_architecture="Glm4ForCausalLM"),
    "glm4-32B": _dense("glm4-32B", 64, 6144, 48, 8, 23040, False, vocab=151552, qk_norm=False, qkv_bias=False, rope_theta=1e4,
                       rms_eps=1e-5, rotary_dim=64, post_norms=True, rope_interleaved=True, max_position_embeddings=32768,
                       hf_architecture="Glm4ForCausalLM"),
    "glm4-smoke": _dense("glm4-smoke", 2, 512, 4, 2, 1024, False, vocab=4096, qk_norm=False, qkv_bias=True, rope_theta=1e4,
                         rms_eps=1e-5, rotary_dim=64, post_norms=True, rope_interleaved=True, hf_architecture="Glm4ForCausalLM"),
    "glm4moe-smoke": ModelConfig(name="glm4moe-smoke", num_layers=3, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                                 ffn_hidden_size=1024, vocab_size=4096, rms_eps=1e-5, rope_theta=1e6, qk_norm=True, qkv_bias=True,
                                 num_experts=16, moe_top_k=4, moe_ffn_hidden_size=256, first_dense_layers=1, router_score="sigmoid",
                                 router_bias=True, routed_scaling_factor=2.5, shared_expert_ffn=256, rotary_dim=64,
                                 hf_architecture="Glm4MoeForCausalLM"),
    # names of the reference's per-model argument files (scripts/models/*.py) for shapes already covered above
    "qwen3-4B-Instruct-2507": _dense("qwen3-4B-Instruct-2507", 36, 2560, 32, 8, 9728, True, rope_theta=5e6),
    "qwen3-30B-A3B-5layer": _moe("qwen3-30B-A3B-5layer", 5, 2048, 32, 4, 128, 8, 768),
    "llama3.1-8B-Instruct": _dense("llama3.1-8B-Instruct", 32, 4096, 32, 8, 14336, False, vocab=128256, qk_norm=False,
                                   rope_theta=5e5, rms_eps=1e-5, hf_architecture="LlamaForCausalLM",
                           rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}, max_position_embeddings=131072),
    "llama3.2-3B-Instruct": _dense("llama3.2-3B-Instruct", 28, 3072, 24, 8, 8192, True, vocab=128256, qk_norm=False,
                                   rope_theta=5e5, rms_eps=1e-5, hf_architecture="LlamaForCausalLM",
                           rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}, max_position_embeddings=131072),
    # MiMo-7B-RL: a Qwen2-style dense model (QKV bias, no QK norm); its multi-token-prediction layer is not trained here
    "mimo-7B-rl": _dense("mimo-7B-rl", 36, 4096, 32, 8, 11008, False, vocab=151680, qk_norm=False, qkv_bias=True,
                         rope_theta=640000.0, rms_eps=1e-5, hf_architecture="Qwen2ForCausalLM"),
}


def get_config(name: str) -> ModelConfig:
    if name in PRESETS:
        import copy

        return copy.deepcopy(PRESETS[name])
    p = Path(name)
    if p.exists():
        return ModelConfig.from_hf_config(p)
    raise KeyError(f"unknown model {name!r}; presets: {sorted(PRESETS)}")

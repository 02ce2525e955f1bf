"""True-on-policy contract: what has to hold for the trainer's recomputed log-probs to equal the engine's.

In this framework trainer and engine are one object graph over one weight store, so most of the contract holds by
construction; this module writes it down as data, checks a configuration against it and says which clauses a given
run breaks (and therefore where a train / rollout log-prob difference may come from).

Reference: miles/true_on_policy/{schema,contracts,config,model_profiles}.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class Clause:
    key: str
    requirement: str
    holds_by_construction: bool = False


CONTRACT_V1 = (
    Clause("weights", "trainer and engine read the same parameter bytes (no cast, no quantisation in between)", True),
    Clause("gemm", "projections run through the same GEMM kernel family with fp32 accumulation and bf16 outputs", True),
    Clause("norm_rope", "RMSNorm / QK-norm / RoPE use the same fused kernels and rounding points", True),
    Clause("routing", "MoE expert choice of the engine is replayed in the trainer (rollout routing replay)"),
    Clause("attention", "prefill / training attention and paged decode attention agree to bf16 rounding; bit equality "
           "needs the same KV block order, which split-KV decode does not give"),
    Clause("batch_invariance", "reductions do not depend on the batch composition (tile shapes are fixed per problem size, "
           "the small-batch decode path changes kernels below 9 rows)"),
    Clause("sampling_temperature", "log-probs are taken at the rollout temperature on the full distribution "
           "(top-k / top-p truncation does not enter the reported log-prob)", True),
    Clause("lm_head", "LM head and log-softmax run in the same precision (bf16 GEMM, fp32 soft-max statistics)", True),
)


@dataclass
class ContractReport:
    satisfied: list = field(default_factory=list)
    broken: list = field(default_factory=list)

    @property
    def bitwise_expected(self) -> bool:
        return not self.broken


def check(args, cfg) -> ContractReport:
    """Which clauses hold for this run configuration."""
    rep = ContractReport()
    for c in CONTRACT_V1:
        ok = c.holds_by_construction
        if c.key == "routing":
            ok = (not cfg.is_moe) or bool(getattr(args, "use_rollout_routing_replay", False))
        elif c.key == "attention":
            ok = False  # split-KV decode orders the KV blocks differently from the training kernel
        elif c.key == "batch_invariance":
            ok = False
        elif c.key == "weights":
            ok = not getattr(args, "sglang_quantization", None)
        (rep.satisfied if ok else rep.broken).append(c)
    return rep


def explain(rep: ContractReport) -> str:
    lines = [f"true-on-policy contract: {len(rep.satisfied)} clauses hold, {len(rep.broken)} do not"]
    lines += [f"  holds : {c.key}" for c in rep.satisfied]
    lines += [f"  broken: {c.key} - {c.requirement}" for c in rep.broken]
    return "\n".join(lines)

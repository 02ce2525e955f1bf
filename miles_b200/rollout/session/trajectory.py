"""Linear trajectory of one agent session.

The trajectory is the exact token sequence the policy has seen and produced. Tokens produced by the engine are
appended as they were sampled (never re-tokenised from text), tokens that come from the environment (system /
user / tool messages rendered through the chat template) are appended with loss mask 0. A later turn must extend
the conversation it continues: if the rendered prefix of an incoming request does not match what the session
holds, the request is rejected rather than silently re-tokenised, because a re-tokenised history would make the
trainer see other tokens than the ones the log-probs belong to.

Reference: miles/rollout/session/linear_trajectory.py:57-347.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class Turn:
    role: str
    start: int
    end: int
    generated: bool


@dataclass
class LinearTrajectory:
    session_id: str
    tokens: list = field(default_factory=list)
    loss_mask: list = field(default_factory=list)
    log_probs: list = field(default_factory=list)
    weight_versions: list = field(default_factory=list)
    turns: list = field(default_factory=list)
    num_messages: int = 0          # messages of the conversation already represented in `tokens`
    finish_reason: Optional[str] = None

    def append_context(self, role: str, ids: list) -> None:
        """Environment-side tokens (prompt, user, tool output): not trained on."""
        s = len(self.tokens)
        self.tokens.extend(ids)
        self.loss_mask.extend([0] * len(ids))
        self.log_probs.extend([0.0] * len(ids))
        self.turns.append(Turn(role, s, len(self.tokens), False))

    def append_generation(self, ids: list, log_probs: list, weight_version: Optional[int] = None, finish_reason: Optional[str] = None) -> None:
        assert len(ids) == len(log_probs)
        s = len(self.tokens)
        self.tokens.extend(ids)
        self.loss_mask.extend([1] * len(ids))
        self.log_probs.extend(log_probs)
        if weight_version is not None and (not self.weight_versions or self.weight_versions[-1] != weight_version):
            self.weight_versions.append(weight_version)
        self.turns.append(Turn("assistant", s, len(self.tokens), True))
        self.finish_reason = finish_reason

    @property
    def prompt_length(self) -> int:
        """Tokens before the first generated one."""
        for t in self.turns:
            if t.generated:
                return t.start
        return len(self.tokens)

    def to_sample_dict(self) -> dict:
        """Fields of a training sample: the response is everything after the first prompt, with the environment
        tokens inside it masked out."""
        p = self.prompt_length
        return {
            "tokens": list(self.tokens),
            "response_length": len(self.tokens) - p,
            "loss_mask": self.loss_mask[p:],
            "rollout_log_probs": self.log_probs[p:],
            "weight_versions": list(self.weight_versions),
            "status": "truncated" if self.finish_reason == "length" else "completed",
            "metadata": {"session_id": self.session_id, "turns": [(t.role, t.start, t.end) for t in self.turns]},
        }

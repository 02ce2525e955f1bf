"""SFT "rollout": tokenise conversations, build the multi-turn loss mask, reward 0 (no generation).

Used with ``--loss-type sft_loss`` so that supervised fine-tuning runs through the same trainer
(reference: miles/rollout/sft_rollout.py:17-66, miles/utils/mask_utils.py)."""
from __future__ import annotations

from ..utils.mask_utils import MultiTurnLossMaskGenerator
from ..utils.types import Sample
from .base_types import RolloutFnTrainOutput


class SFTRolloutFn:
    def __init__(self, inp):
        self.args = inp.args
        self.data_source = inp.data_source
        self.tokenizer = getattr(inp.engine_client, "tokenizer", None)
        self.mask_gen = None

    def __call__(self, inp):
        assert not inp.evaluation, "SFT rollout has no evaluation mode"
        if self.mask_gen is None:
            self.mask_gen = MultiTurnLossMaskGenerator(self.tokenizer, getattr(self.args, "loss_mask_type", "qwen"))
        groups = self.data_source.get_samples(self.args.rollout_batch_size)
        for group in groups:
            for s in group:
                messages = s.prompt if isinstance(s.prompt, list) else [{"role": "user", "content": str(s.prompt)},
                                                                      {"role": "assistant", "content": str(s.label or "")}]
                ids, mask = self.mask_gen.get_loss_mask(messages)
                first = next((i for i, m in enumerate(mask) if m), len(mask))
                first = max(first, 1)
                s.tokens = ids
                s.response_length = len(ids) - first
                s.loss_mask = mask[first:]
                s.reward = 0.0
                s.status = Sample.Status.COMPLETED
        return RolloutFnTrainOutput(samples=groups)

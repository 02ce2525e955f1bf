"""Loss-mask builders for multi-turn conversations: only assistant tokens are trained on.

``qwen`` / ``qwen3``: ChatML framing (``<|im_start|>role\\n ... <|im_end|>\\n``); assistant content and its
closing ``<|im_end|>`` are trainable, the ``<|im_start|>assistant\\n`` header is not; ``qwen3`` additionally
leaves an empty ``<think></think>`` scaffold untrained.  ``distill_qwen`` trains on the last assistant
message only.  Without a chat template the generic path diffs ``apply_chat_template`` prefixes.
Reference: miles/utils/mask_utils.py.
"""
from __future__ import annotations

from typing import Any


class MultiTurnLossMaskGenerator:
    def __init__(self, tokenizer: Any, tokenizer_type: str = "qwen"):
        self.tok = tokenizer
        self.type = tokenizer_type

    def _enc(self, text: str) -> list:
        return self.tok(text, add_special_tokens=False)["input_ids"]

    def _chatml(self, messages: list, last_only: bool = False) -> tuple:
        ids, mask = [], []
        n_assist = sum(m["role"] == "assistant" for m in messages)
        seen = 0
        for m in messages:
            header = self._enc(f"<|im_start|>{m['role']}\n")
            content = m.get("content") or ""
            if m["role"] == "assistant":
                seen += 1
                train = (not last_only) or seen == n_assist
                scaffold = []
                if self.type == "qwen3" and content.startswith("<think>\n\n</think>\n\n"):
                    scaffold = self._enc("<think>\n\n</think>\n\n")
                    content = content[len("<think>\n\n</think>\n\n"):]
                body = self._enc(content + "<|im_end|>")
                tail = self._enc("\n")
                ids += header + scaffold + body + tail
                mask += [0] * (len(header) + len(scaffold)) + [1 if train else 0] * len(body) + [0] * len(tail)
            else:
                body = self._enc(content + "<|im_end|>\n")
                ids += header + body
                mask += [0] * (len(header) + len(body))
        return ids, mask

    def _generic(self, messages: list) -> tuple:
        ids, mask = [], []
        for i, m in enumerate(messages):
            cur = self.tok.apply_chat_template(messages[: i + 1], tokenize=True, add_generation_prompt=False)
            new = cur[len(ids):]
            if m["role"] == "assistant":
                prefix = self.tok.apply_chat_template(messages[:i], tokenize=True, add_generation_prompt=True)
                head = max(0, len(prefix) - len(ids))
                mask += [0] * head + [1] * (len(new) - head)
            else:
                mask += [0] * len(new)
            ids = cur
        return ids, mask

    def get_loss_mask(self, messages: list) -> tuple:
        if self.type in ("qwen", "qwen3"):
            return self._chatml(messages)
        if self.type == "distill_qwen":
            return self._chatml(messages, last_only=True)
        return self._generic(messages)

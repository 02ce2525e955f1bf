"""Prompt data sources.

``RolloutDataSource`` reads a JSONL / parquet prompt file (``--prompt-data``, ``--input-key``,
``--label-key``, ``--metadata-key``, optional chat template), shuffles per epoch with ``--rollout-seed``,
fans every prompt out to a group of ``--n-samples-per-prompt`` samples and checkpoints its position
under ``<save>/rollout/global_dataset_state_dict_{rollout_id}.pt``.  ``RolloutDataSourceWithBuffer``
adds a buffer for partially generated / aborted groups that are served first (partial rollout).
``SyntheticDataSource`` produces uniform random token prompts for the benchmark configurations.
Contract: miles/rollout/data_source.py:17-225 of the reference.
"""
from __future__ import annotations

import copy
import json
import os
import random
from abc import ABC, abstractmethod
from typing import Optional

import torch

from ..utils.misc import load_function
from ..utils.types import Sample


class DataSource(ABC):
    @abstractmethod
    def get_samples(self, num_samples: int) -> list:
        """Return ``num_samples`` groups (each a list of ``n_samples_per_prompt`` samples)."""

    def add_samples(self, samples: list) -> None:
        raise NotImplementedError

    def save(self, rollout_id: int) -> None:
        pass

    def load(self, rollout_id: Optional[int] = None) -> None:
        pass

    def __len__(self) -> int:
        return 0


def read_prompt_file(path: str) -> list:
    rows = []
    if path.endswith(".parquet"):
        import pandas as pd

        rows = pd.read_parquet(path).to_dict("records")
    else:
        with open(path) as f:
            for line in f:
                line = line.strip()
                if line:
                    rows.append(json.loads(line))
    return rows


class Dataset:
    """Tokenised prompt dataset with deterministic per-epoch shuffling."""

    def __init__(self, path: str, tokenizer=None, max_length: Optional[int] = None, input_key: str = "input",
                 label_key: Optional[str] = None, metadata_key: str = "metadata", tool_key: Optional[str] = None,
                 apply_chat_template: bool = False, apply_chat_template_kwargs: Optional[dict] = None, seed: int = 42):
        self.seed = seed
        self.samples: list = []
        path, _, sl = path.partition("@")
        rows = read_prompt_file(path)
        if sl:
            m = __import__("re").match(r"\[(\d*):(\d*)\]", sl)
            if m:
                rows = rows[int(m.group(1) or 0): int(m.group(2)) if m.group(2) else None]
        for row in rows:
            prompt = row.get(input_key)
            tools = row.get(tool_key) if tool_key else None
            text = prompt
            if apply_chat_template and tokenizer is not None:
                msgs = prompt if isinstance(prompt, list) else [{"role": "user", "content": prompt}]
                text = tokenizer.apply_chat_template(msgs, tools=tools, tokenize=False, add_generation_prompt=True,
                                                     **(apply_chat_template_kwargs or {}))
            if tokenizer is not None and max_length is not None:
                if len(tokenizer(text, add_special_tokens=False)["input_ids"]) > max_length:
                    continue
            md = dict(row.get(metadata_key) or {})
            if tools is not None:
                md["tools"] = tools
            self.samples.append(Sample(prompt=text, label=row.get(label_key) if label_key else None, metadata=md))
        self.order = list(range(len(self.samples)))

    def shuffle(self, epoch: int) -> None:
        rng = random.Random(self.seed + epoch)
        self.order = list(range(len(self.samples)))
        rng.shuffle(self.order)

    def __len__(self) -> int:
        return len(self.samples)

    def __getitem__(self, i: int) -> Sample:
        return self.samples[self.order[i]]


class RolloutDataSource(DataSource):
    def __init__(self, args, tokenizer=None):
        self.args = args
        self.epoch_id = 0
        self.sample_group_index = 0
        self.sample_index = 0
        self.sample_offset = 0
        self.metadata: dict = {}
        self.dataset: Optional[Dataset] = None
        if getattr(args, "rollout_global_dataset", True) and getattr(args, "prompt_data", None):
            self.dataset = Dataset(args.prompt_data, tokenizer, getattr(args, "rollout_max_prompt_len", None), args.input_key,
                                   args.label_key, args.metadata_key, getattr(args, "tool_key", None), args.apply_chat_template,
                                   getattr(args, "apply_chat_template_kwargs", None), args.rollout_seed)
            if args.rollout_shuffle:
                self.dataset.shuffle(self.epoch_id)

    def _next_prompts(self, n: int) -> list:
        if self.dataset is None:
            return [Sample() for _ in range(n)]
        out = []
        while len(out) < n:
            if self.sample_offset >= len(self.dataset):
                self.epoch_id += 1
                self.sample_offset = 0
                if self.args.rollout_shuffle:
                    self.dataset.shuffle(self.epoch_id)
            out.append(self.dataset[self.sample_offset])
            self.sample_offset += 1
        return out

    def get_samples(self, num_samples: int) -> list:
        groups = []
        for proto in self._next_prompts(num_samples):
            group = []
            for _ in range(self.args.n_samples_per_prompt):
                s = copy.deepcopy(proto)
                s.group_index, s.index = self.sample_group_index, self.sample_index
                self.sample_index += 1
                group.append(s)
            self.sample_group_index += 1
            groups.append(group)
        return groups

    def add_samples(self, samples: list) -> None:
        raise RuntimeError(f"{type(self).__name__} has no buffer; use RolloutDataSourceWithBuffer")

    def state_dict(self) -> dict:
        return {"sample_offset": self.sample_offset, "epoch_id": self.epoch_id, "sample_group_index": self.sample_group_index,
                "sample_index": self.sample_index, "metadata": self.metadata}

    def load_state_dict(self, sd: dict) -> None:
        self.sample_offset, self.epoch_id = sd.get("sample_offset", 0), sd.get("epoch_id", 0)
        self.sample_group_index, self.sample_index = sd.get("sample_group_index", 0), sd.get("sample_index", 0)
        self.metadata = sd.get("metadata", {})
        if self.dataset is not None and self.args.rollout_shuffle:
            self.dataset.shuffle(self.epoch_id)

    def _path(self, rollout_id: int) -> str:
        return os.path.join(self.args.save, "rollout", f"global_dataset_state_dict_{rollout_id}.pt")

    def save(self, rollout_id: int) -> None:
        if not getattr(self.args, "save", None):
            return
        p = self._path(rollout_id)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        torch.save(self.state_dict(), p)

    def load(self, rollout_id: Optional[int] = None) -> None:
        base = getattr(self.args, "load", None)
        if not base or rollout_id is None:
            return
        p = os.path.join(base, "rollout", f"global_dataset_state_dict_{rollout_id}.pt")
        if os.path.exists(p):
            self.load_state_dict(torch.load(p, weights_only=False))

    def __len__(self) -> int:
        return len(self.dataset) if self.dataset is not None else 0


def pop_first(args, rollout_id, buffer: list, num_samples: int) -> list:
    n = min(len(buffer), num_samples)
    out = buffer[:n]
    del buffer[:n]
    return out


class RolloutDataSourceWithBuffer(RolloutDataSource):
    """Serves buffered (partially generated / retried) groups before fresh prompts."""

    def __init__(self, args, tokenizer=None):
        super().__init__(args, tokenizer)
        self.buffer: list = []
        path = getattr(args, "buffer_filter_path", None)
        self.buffer_filter = load_function(path) if path else pop_first

    def get_samples(self, num_samples: int) -> list:
        out = self.buffer_filter(self.args, None, self.buffer, num_samples) if self.buffer else []
        if len(out) < num_samples:
            out += super().get_samples(num_samples - len(out))
        return out

    def add_samples(self, samples: list) -> None:
        if not samples:
            return
        assert isinstance(samples[0], list), "add_samples expects a list of groups"
        for g in samples:
            assert len(g) == self.args.n_samples_per_prompt, "a buffered group must be complete"
            self.buffer.append(g)

    def get_buffer_length(self) -> int:
        return len(self.buffer)

    def state_dict(self) -> dict:
        sd = super().state_dict()
        sd["buffer"] = [[s.to_dict() for s in g] for g in self.buffer]
        return sd

    def load_state_dict(self, sd: dict) -> None:
        super().load_state_dict(sd)
        self.buffer = [[Sample.from_dict(d) for d in g] for g in sd.get("buffer", [])]


class SyntheticDataSource(RolloutDataSourceWithBuffer):
    """Uniform random token-id prompts of a fixed length (benchmark / plumbing configurations)."""

    def __init__(self, args, tokenizer=None):
        args = copy.copy(args)
        args.prompt_data = None
        super().__init__(args, tokenizer)
        self.prompt_len = getattr(args, "synthetic_prompt_len", None) or getattr(args, "rollout_max_prompt_len", None) or 32
        self.vocab = getattr(args, "synthetic_vocab_size", None) or 1024
        self.gen = torch.Generator().manual_seed(args.rollout_seed)

    def _next_prompts(self, n: int) -> list:
        out = []
        for _ in range(n):
            ids = torch.randint(0, self.vocab, (self.prompt_len,), generator=self.gen).tolist()
            out.append(Sample(prompt=ids, tokens=list(ids)))
        return out

    def state_dict(self) -> dict:
        sd = super().state_dict()
        sd["gen"] = self.gen.get_state()
        return sd

    def load_state_dict(self, sd: dict) -> None:
        super().load_state_dict(sd)
        if "gen" in sd:
            self.gen.set_state(sd["gen"])

"""Token-in-token-out (TITO) tokenisation of multi-turn conversations.

The trainer must see exactly the tokens the engine saw and produced. Re-tokenising a conversation from text after
every turn does not guarantee that: merges across turn boundaries, templates that drop earlier reasoning blocks,
and turns that ended without their end-of-turn token (length limit, stop string) all make
``tokenize(render(messages[:k+1]))`` differ from ``tokenize(render(messages[:k])) + new tokens``. A
``TitoTokenizer`` therefore never re-renders what is already in the trajectory; it produces

* ``initial(messages)``        the ids of the first prompt (with the generation header), and
* ``continuation(generated, new_messages)``  the ids to append after a generated turn: a *boundary fix* (close the
  turn if the engine did not emit the end-of-turn token, then the separator the template puts between turns), the
  new messages rendered one by one, and the next generation header,

each piece tokenised on its own so that no merge can cross a piece boundary. ``FAMILIES`` holds the per-family
boundary tokens; a family whose template rewrites history (``rewrites_history``) is exactly the case where text
re-rendering would break, and ``consistent_with_template`` is skipped for it.

Reference counterpart: miles/utils/chat_template_utils/tito_tokenizer.py:81-927 (per-family boundary fixers).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Sequence


@dataclass(frozen=True)
class Family:
    turn_end: str               # text of the end-of-turn token
    turn_sep: str               # text the template puts after it
    header: str                 # "{role}" is replaced by the role name
    rewrites_history: bool = False


FAMILIES = {
    "chatml": Family("<|im_end|>", "\n", "<|im_start|>{role}\n"),
    "qwen3": Family("<|im_end|>", "\n", "<|im_start|>{role}\n", rewrites_history=True),  # drops earlier <think> blocks
    "llama3": Family("<|eot_id|>", "", "<|start_header_id|>{role}<|end_header_id|>\n\n"),
    # GLM-4 / GLM-4.5: roles are special tokens, a turn ends where the next role token starts (no end-of-turn token of its
    # own: generation stops at <|user|> / <|observation|>, which then open the next turn)
    "glm4": Family("", "", "<|{role}|>\n", rewrites_history=True),
    "mistral": Family("</s>", "", "[INST] "),  # user turns are wrapped, assistant text follows " [/INST]" (see header_ids)
    "generic": Family("<|end|>", "", "<|{role}|>"),
}


def detect_family(tokenizer: Any) -> str:
    tpl = getattr(tokenizer, "chat_template", None) or ""
    name = (getattr(tokenizer, "name_or_path", "") or "").lower()
    if "<|im_start|>" in tpl:
        return "qwen3" if ("qwen3" in name or "<think>" in tpl) else "chatml"
    if "<|start_header_id|>" in tpl:
        return "llama3"
    if "<|assistant|>" in tpl and "<|user|>" in tpl:
        return "glm4"
    if "[INST]" in tpl:
        return "mistral"
    return "generic"


class TitoTokenizer:
    def __init__(self, tokenizer: Any, family: Optional[str] = None):
        self.tok = tokenizer
        self.family_name = family or detect_family(tokenizer)
        self.family = FAMILIES[self.family_name]
        self._end_ids = self._enc(self.family.turn_end)
        self._sep_ids = self._enc(self.family.turn_sep)

    # ------------------------------------------------------------------ pieces
    def _enc(self, text: str) -> list:
        return list(self.tok.encode(text, add_special_tokens=False)) if text else []

    def _render(self, messages: Sequence[dict], add_generation_prompt: bool, tools=None) -> str:
        if getattr(self.tok, "chat_template", None) and hasattr(self.tok, "apply_chat_template"):
            kw = {"tools": tools} if tools else {}
            return self.tok.apply_chat_template(list(messages), tokenize=False, add_generation_prompt=add_generation_prompt, **kw)
        f = self.family
        text = "".join(f.header.format(role=m["role"]) + (m.get("content") or "") + f.turn_end + f.turn_sep for m in messages)
        return text + (f.header.format(role="assistant") if add_generation_prompt else "")

    def header_ids(self, role: str = "assistant") -> list:
        return self._enc(self.family.header.format(role=role))

    def message_ids(self, message: dict) -> list:
        """One message as the template renders it in the middle of a conversation: rendered after a fixed dummy
        turn and cut out again, so that template logic which depends on position (system prompt injection at the
        start) does not leak into later turns."""
        dummy = [{"role": "user", "content": "x"}]
        base = self._render(dummy, False)
        both = self._render(dummy + [message], False)
        if not both.startswith(base):
            # template rewrote the dummy: fall back to the family's plain form
            f = self.family
            return self._enc(f.header.format(role=message["role"]) + (message.get("content") or "") + f.turn_end + f.turn_sep)
        return self._enc(both[len(base):])

    # ------------------------------------------------------------------ API
    def initial(self, messages: Sequence[dict], tools=None) -> list:
        return self._enc(self._render(messages, True, tools))

    def boundary_fix(self, generated: Sequence[int]) -> list:
        """Tokens that close a generated turn the way the template would have."""
        g = list(generated)
        n = len(self._end_ids)
        closed = n > 0 and g[-n:] == self._end_ids
        return ([] if closed else list(self._end_ids)) + list(self._sep_ids)

    def continuation(self, generated: Sequence[int], new_messages: Sequence[dict]) -> list:
        ids = self.boundary_fix(generated)
        for m in new_messages:
            ids += self.message_ids(m)
        return ids + self.header_ids("assistant")

    def special_ids(self) -> set:
        """Ids the tokenizer treats as special (turn openers, end-of-turn tokens, role tokens ...)."""
        ids = set(getattr(self.tok, "all_special_ids", None) or [])
        added = getattr(self.tok, "added_tokens_decoder", None) or {}
        ids.update(int(i) for i, t in added.items() if getattr(t, "special", True))
        for text in (self.family.turn_end,):
            e = self._enc(text)
            if len(e) == 1:
                ids.add(e[0])
        extra = getattr(self.tok, "special_token_ids", None)  # simple tokenizers of tests declare theirs like this
        ids.update(extra or [])
        return ids

    def diagnose(self, trajectory_ids: Sequence[int], messages: Sequence[dict]) -> list:
        """Differences between the incremental trajectory and a fresh rendering of the whole conversation, classified
        (session/compare.py): text of assistant turns may differ harmlessly, anything else is a defect of the incremental
        path (or of this family's boundary tokens)."""
        from .compare import compare

        expected = self._enc(self._render(messages, True))
        dec = (lambda ids: self.tok.decode(list(ids))) if hasattr(self.tok, "decode") else (lambda ids: " ".join(map(str, ids)))
        return compare(expected, list(trajectory_ids), self.special_ids(), dec)

    def consistent_with_template(self, trajectory_ids: Sequence[int], messages: Sequence[dict]) -> Optional[bool]:
        """Whether the incremental ids equal a fresh rendering of the whole conversation; None for families whose
        template rewrites history (there the fresh rendering is not the reference)."""
        if self.family.rewrites_history:
            return None
        return list(trajectory_ids) == self._enc(self._render(messages, True))


@dataclass
class TreeNode:
    """A span of tokens shared by every trajectory that passes through it."""
    tokens: list
    loss_mask: list
    log_probs: list
    parent: Optional[int]
    children: list


class TreeTrajectory:
    """Trajectories of one session as a prefix tree: a request whose history diverges from what the session holds
    (the agent compacted or edited its context, or forked a sub-agent) branches at the longest common token prefix
    instead of being rejected. Every leaf is one training sample; all leaves share the session's rollout id so the
    loss normaliser counts the rollout once.

    Reference counterpart: the tree trajectories of miles/rollout/session/v2/."""

    def __init__(self, session_id: str):
        self.session_id = session_id
        self.nodes: list = [TreeNode([], [], [], None, [])]
        self.cursor = 0  # node the next append extends

    def _path(self, node: int) -> list:
        out = []
        while node is not None:
            out.append(node)
            node = self.nodes[node].parent
        return out[::-1]

    def tokens_to(self, node: Optional[int] = None) -> list:
        return [t for i in self._path(self.cursor if node is None else node) for t in self.nodes[i].tokens]

    def append(self, ids: Sequence[int], generated: bool, log_probs: Optional[Sequence[float]] = None) -> None:
        n = self.nodes[self.cursor]
        if n.children:  # somebody already branched from here: new tokens go into a fresh child
            self.nodes.append(TreeNode([], [], [], self.cursor, []))
            n.children.append(len(self.nodes) - 1)
            self.cursor = len(self.nodes) - 1
            n = self.nodes[self.cursor]
        n.tokens.extend(ids)
        n.loss_mask.extend([1 if generated else 0] * len(ids))
        n.log_probs.extend(list(log_probs) if log_probs is not None else [0.0] * len(ids))

    def seek(self, history_ids: Sequence[int]) -> int:
        """Move the cursor to the point of the tree that matches the longest prefix of ``history_ids`` (splitting a
        node if the match ends inside it) and return the number of matched tokens."""
        node, matched = 0, 0
        h = list(history_ids)
        while True:
            n = self.nodes[node]
            k = 0
            while k < len(n.tokens) and matched + k < len(h) and n.tokens[k] == h[matched + k]:
                k += 1
            if k < len(n.tokens):
                if k > 0 or node == 0:
                    self._split(node, k)
                else:
                    node = n.parent
                matched += k
                break
            matched += k
            nxt = next((c for c in n.children if self.nodes[c].tokens and matched < len(h) and self.nodes[c].tokens[0] == h[matched]), None)
            if nxt is None:
                break
            node = nxt
        self.cursor = node
        return matched

    def _split(self, node: int, k: int) -> None:
        n = self.nodes[node]
        tail = TreeNode(n.tokens[k:], n.loss_mask[k:], n.log_probs[k:], node, n.children)
        self.nodes.append(tail)
        ti = len(self.nodes) - 1
        for c in tail.children:
            self.nodes[c].parent = ti
        n.tokens, n.loss_mask, n.log_probs, n.children = n.tokens[:k], n.loss_mask[:k], n.log_probs[:k], [ti]

    def leaves(self) -> list:
        return [i for i, n in enumerate(self.nodes) if not n.children and (n.tokens or i == 0)]

    def to_sample_dicts(self) -> list:
        out = []
        for leaf in self.leaves():
            path = self._path(leaf)
            toks = [t for i in path for t in self.nodes[i].tokens]
            mask = [m for i in path for m in self.nodes[i].loss_mask]
            lps = [p for i in path for p in self.nodes[i].log_probs]
            if 1 not in mask:
                continue
            p = mask.index(1)
            out.append({"tokens": toks, "response_length": len(toks) - p, "loss_mask": mask[p:], "rollout_log_probs": lps[p:],
                        "metadata": {"session_id": self.session_id, "leaf": leaf}, "rollout_id_key": self.session_id})
        return out

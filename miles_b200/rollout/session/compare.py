"""Compare a token trajectory with a reference tokenisation of the same conversation, segment by segment.

Two id sequences that should describe the same conversation rarely differ everywhere: the special tokens give them a
skeleton (turn openers, end-of-turn tokens, role headers), between which lies text. ``segment`` cuts a sequence at its
special tokens; ``compare`` aligns two sequences by that skeleton and classifies every difference:

* ``structure``       the skeletons differ (another number or order of special / text segments): nothing can be aligned;
* ``special_token``   the same position holds another special token;
* ``context_text``    text outside assistant turns differs (system / user / tool content): the incremental tokenisation
                      put something else in front of the model than the template would have, which is a defect;
* ``assistant_text``  text of an assistant turn differs: expected and harmless, because generated tokens are kept exactly
                      as the engine emitted them and the tokenizer's canonical split of the same text may be another one.

Which text segments are assistant text is decided by ``role_of`` (default: the role name that follows the turn opener,
as in ChatML / Llama-3 style templates, or the role token itself where roles are special tokens).

Reference: miles/utils/chat_template_utils/token_seq_comparator.py:1-289.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

KINDS = ("structure", "special_token", "context_text", "assistant_text")
SEVERE = ("structure", "special_token", "context_text")


@dataclass
class Segment:
    ids: list
    special: bool


@dataclass
class Mismatch:
    kind: str
    index: int            # segment index (of the expected sequence)
    expected: str
    actual: str
    detail: str = ""

    @property
    def severe(self) -> bool:
        return self.kind in SEVERE

    def to_dict(self) -> dict:
        return {"kind": self.kind, "index": self.index, "expected": self.expected, "actual": self.actual, "detail": self.detail,
                "severe": self.severe}


def segment(ids: Sequence[int], special_ids) -> list:
    """Every special token is a segment of its own; the runs between them are text segments."""
    special_ids = set(int(i) for i in special_ids)
    out: list = []
    run: list = []
    for t in ids:
        t = int(t)
        if t in special_ids:
            if run:
                out.append(Segment(run, False))
                run = []
            out.append(Segment([t], True))
        else:
            run.append(t)
    if run:
        out.append(Segment(run, False))
    return out


def default_role_of(segments: Sequence[Segment], index: int, decode: Callable[[list], str]) -> Optional[str]:
    """The role a text segment belongs to: the nearest special token before it that decodes to a role token
    (``<|assistant|>``), else the role name at the start of the first text segment after the turn opener (``<|im_start|>``
    followed by ``assistant\\n...``; ``<|start_header_id|>`` followed by ``assistant``)."""
    roles = ("assistant", "user", "system", "tool", "observation", "ipython")
    j = index
    while j >= 0:
        s = segments[j]
        if s.special:
            text = decode(s.ids).strip("<|>[] \n").lower()
            if text in roles:
                return text
        else:
            prev_special = j > 0 and segments[j - 1].special
            if prev_special:
                head = decode(s.ids).lstrip().lower()
                for r in roles:
                    if head.startswith(r):
                        # a header segment names the role of the text that follows it, and of itself
                        return r
        j -= 1
    return None


def compare(expected: Sequence[int], actual: Sequence[int], special_ids, decode: Callable[[list], str],
            role_of: Callable = default_role_of) -> list:
    """Mismatches of ``actual`` against ``expected`` (empty list: identical up to nothing at all)."""
    if list(expected) == list(actual):
        return []
    es, as_ = segment(expected, special_ids), segment(actual, special_ids)
    if [s.special for s in es] != [s.special for s in as_]:
        return [Mismatch("structure", 0, " ".join("S" if s.special else "t" for s in es), " ".join("S" if s.special else "t" for s in as_),
                         f"{sum(s.special for s in es)} special tokens expected, {sum(s.special for s in as_)} found")]
    out = []
    for i, (e, a) in enumerate(zip(es, as_)):
        if e.ids == a.ids:
            continue
        if e.special:
            out.append(Mismatch("special_token", i, decode(e.ids), decode(a.ids)))
            continue
        role = role_of(es, i, decode)
        kind = "assistant_text" if role == "assistant" else "context_text"
        te, ta = decode(e.ids), decode(a.ids)
        detail = "same text, another token split" if te == ta else "text differs"
        if kind == "assistant_text" and te != ta:
            detail = "text differs (a template that rewrites earlier assistant turns, or a truncated generation)"
        out.append(Mismatch(kind, i, te, ta, detail))
    return out

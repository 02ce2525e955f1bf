"""Token-level F1 between a prediction and a ground truth (SQuAD-style normalisation)."""
from __future__ import annotations

import re
import string
from collections import Counter


def _normalize(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def f1_score(prediction: str, ground_truth: str):
    p, g = _normalize(prediction), _normalize(ground_truth)
    zero = (0.0, 0.0, 0.0)
    if p in ("yes", "no", "noanswer") and p != g:
        return zero
    if g in ("yes", "no", "noanswer") and p != g:
        return zero
    pt, gt = p.split(), g.split()
    common = Counter(pt) & Counter(gt)
    same = sum(common.values())
    if same == 0:
        return zero
    precision, recall = same / len(pt), same / len(gt)
    return 2 * precision * recall / (precision + recall), precision, recall

"""Evaluation metrics (``mindformers/core/metric/metric.py:40-494``): ``PerplexityMetric``, ``EntityScore``,
``ADGENMetric`` (ROUGE / BLEU-4), ``PromptAccMetric``, ``EmF1Metric``. All follow ``clear / update / eval``."""
from __future__ import annotations

import collections
import math
import re
import string
from typing import Dict, List, Sequence

import torch

from ..tools.register.register import MindFormerModuleType, MindFormerRegister


def _reg(cls):
    MindFormerRegister.register_cls(cls, MindFormerModuleType.METRIC)
    return cls


@_reg
class PerplexityMetric:
    """Mean token cross-entropy over batches and ``exp`` of it. ``update(logits [B,S,V], labels [B,S], mask [B,S])``
    shifts by one like the reference's eval path, or ``update(loss)`` takes an already-reduced loss."""

    def __init__(self):
        self.clear()

    def clear(self):
        self.total, self.count = 0.0, 0

    def update(self, *inputs):
        if len(inputs) == 1:
            self.total += float(inputs[0])
            self.count += 1
            return
        logits, labels = inputs[0], inputs[1]
        mask = inputs[2] if len(inputs) > 2 else torch.ones_like(labels, dtype=torch.float32)
        logits = logits[:, :-1].float()
        labels, mask = labels[:, 1:], mask[:, 1:].float()
        nll = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1), reduction="none")
        self.total += float((nll * mask.reshape(-1)).sum() / mask.sum().clamp_min(1e-8))
        self.count += 1

    def eval(self) -> Dict[str, float]:
        if not self.count:
            return {}
        loss = self.total / self.count
        return {"loss": loss, "PPL": math.exp(min(loss, 80.0))}


def _lcs(a: Sequence, b: Sequence) -> int:
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b, 1):
            cur.append(prev[j - 1] + 1 if x == y else max(prev[j], cur[-1]))
        prev = cur
    return prev[-1]


def _ngrams(tokens, n):
    return collections.Counter(tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1))


def rouge_n(hyp, ref, n):
    h, r = _ngrams(hyp, n), _ngrams(ref, n)
    overlap = sum((h & r).values())
    p = overlap / max(sum(h.values()), 1)
    rc = overlap / max(sum(r.values()), 1)
    return 2 * p * rc / (p + rc) if p + rc else 0.0


def rouge_l(hyp, ref):
    l = _lcs(hyp, ref)
    p, r = l / max(len(hyp), 1), l / max(len(ref), 1)
    return 2 * p * r / (p + r) if p + r else 0.0


def bleu4(hyp, ref, smooth: float = 1e-9):
    logs = 0.0
    for n in range(1, 5):
        h, r = _ngrams(hyp, n), _ngrams(ref, n)
        overlap = sum((h & r).values())
        total = max(sum(h.values()), 1)
        logs += math.log((overlap + smooth) / (total + smooth)) / 4   # method-3-like smoothing floor
    bp = 1.0 if len(hyp) > len(ref) else math.exp(1 - len(ref) / max(len(hyp), 1))
    return bp * math.exp(logs)


@_reg
class ADGENMetric:
    """ROUGE-1/2/L and BLEU-4 (character tokens, as the reference does for Chinese ad generation)."""

    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer
        self.clear()

    def clear(self):
        self.scores = collections.defaultdict(list)

    def _text(self, x):
        if isinstance(x, str):
            return list(x.replace(" ", ""))
        if self.tokenizer is not None:
            return list(self.tokenizer.decode(list(x), skip_special_tokens=True).replace(" ", ""))
        return [int(t) for t in x]

    def update(self, preds, labels):
        for p, l in zip(preds, labels):
            hyp, ref = self._text(p), self._text(l)
            if not hyp or not ref:
                continue
            self.scores["rouge-1"].append(rouge_n(hyp, ref, 1))
            self.scores["rouge-2"].append(rouge_n(hyp, ref, 2))
            self.scores["rouge-l"].append(rouge_l(hyp, ref))
            self.scores["bleu-4"].append(bleu4(hyp, ref))

    def eval(self):
        return {k: 100.0 * sum(v) / len(v) for k, v in self.scores.items() if v}


@_reg
class EntityScore:
    """Token-classification precision / recall / F1 over BIO-tagged spans."""

    def __init__(self, label_names: Sequence[str] = ()):
        self.names = list(label_names)
        self.clear()

    def clear(self):
        self.tp = self.fp = self.fn = 0

    def _spans(self, tags):
        spans, start, kind = set(), None, None
        for i, t in enumerate(list(tags) + ["O"]):
            t = self.names[t] if self.names and not isinstance(t, str) else str(t)
            if start is not None and not t.startswith("I-"):
                spans.add((start, i, kind))
                start = None
            if t.startswith(("B-", "S-")):
                start, kind = i, t[2:]
        return spans

    def update(self, logits_or_tags, labels):
        pred = logits_or_tags.argmax(-1).tolist() if torch.is_tensor(logits_or_tags) and logits_or_tags.dim() == 3 else logits_or_tags
        gold = labels.tolist() if torch.is_tensor(labels) else labels
        for p, g in zip(pred, gold):
            ps_, gs = self._spans(p), self._spans(g)
            self.tp += len(ps_ & gs)
            self.fp += len(ps_ - gs)
            self.fn += len(gs - ps_)

    def eval(self):
        p = self.tp / max(self.tp + self.fp, 1)
        r = self.tp / max(self.tp + self.fn, 1)
        return {"precision": p, "recall": r, "f1": 2 * p * r / (p + r) if p + r else 0.0}


@_reg
class PromptAccMetric:
    """Multiple-choice accuracy: each sample has several candidate continuations; the one with the lowest
    masked mean loss is the prediction. ``update(logits [B*C,S,V], input_ids, mask, labels [B])``."""

    def __init__(self):
        self.clear()

    def clear(self):
        self.correct = self.total = 0

    def update(self, logits, input_ids, input_mask, labels):
        B = labels.shape[0]
        C = logits.shape[0] // B
        lg, tgt, m = logits[:, :-1].float(), input_ids[:, 1:], input_mask[:, 1:].float()
        nll = torch.nn.functional.cross_entropy(lg.reshape(-1, lg.shape[-1]), tgt.reshape(-1), reduction="none").view_as(tgt)
        score = (nll * m).sum(-1) / m.sum(-1).clamp_min(1)
        pred = score.view(B, C).argmin(-1)
        self.correct += int((pred.cpu() == labels.cpu()).sum())
        self.total += B

    def eval(self):
        return {"Acc": self.correct / max(self.total, 1)}


def _normalise_answer(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


@_reg
class EmF1Metric:
    """Exact match and token-level F1 between generated and gold answers (SQuAD-style normalisation)."""

    def __init__(self):
        self.clear()

    def clear(self):
        self.em, self.f1, self.n = 0.0, 0.0, 0

    def update(self, preds: List[str], golds: List[str]):
        for p, g in zip(preds, golds):
            answers = g if isinstance(g, (list, tuple)) else [g]
            best_em = best_f1 = 0.0
            for a in answers:
                pn, an = _normalise_answer(p), _normalise_answer(a)
                best_em = max(best_em, float(pn == an))
                pt, at = pn.split(), an.split()
                common = sum((collections.Counter(pt) & collections.Counter(at)).values())
                if common:
                    pr, rc = common / len(pt), common / len(at)
                    best_f1 = max(best_f1, 2 * pr * rc / (pr + rc))
            self.em += best_em
            self.f1 += best_f1
            self.n += 1

    def eval(self):
        return {"Em": 100.0 * self.em / max(self.n, 1), "F1": 100.0 * self.f1 / max(self.n, 1)}


def build_metric(config=None, default_args=None, **kwargs):
    if config is None:
        return None
    if isinstance(config, (list, tuple)):
        return [build_metric(c, default_args) for c in config]
    return MindFormerRegister.get_instance_from_cfg(dict(config), MindFormerModuleType.METRIC, default_args=default_args)


from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ['metric', 'build_metric', 'utils'])

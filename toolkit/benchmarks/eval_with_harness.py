#!/usr/bin/env python
"""lm-evaluation-harness adapter (``toolkit/benchmarks/eval_with_harness.py:53``, ``MFLM(TemplateLM)``).

``MFLM`` exposes the three calls the harness makes — ``loglikelihood``, ``loglikelihood_rolling`` and ``generate_until``
— on top of a model of this framework. When the ``lm_eval`` package is importable the class registers itself as model
``"mf"`` and ``main`` hands over to the harness CLI; without it the class is still usable directly (its requests are
plain ``(context, continuation)`` tuples).
"""
import os
import sys
from typing import List, Tuple

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

try:  # pragma: no cover - optional dependency
    from lm_eval.api.model import TemplateLM
    from lm_eval.api.registry import register_model
except Exception:  # noqa: BLE001
    TemplateLM = object

    def register_model(*names):
        return lambda cls: cls


@register_model("mf")
class MFLM(TemplateLM):
    def __init__(self, pretrained: str = None, model=None, tokenizer=None, batch_size: int = 1, max_length: int = 2048,
                 max_gen_toks: int = 256, device: str = None, **kwargs):
        if TemplateLM is not object:
            super().__init__()
        from mindformers_b200.models import AutoModel, AutoTokenizer
        self.model = model if model is not None else AutoModel.from_pretrained(pretrained)
        self.tokenizer = tokenizer if tokenizer is not None else AutoTokenizer.from_pretrained(pretrained)
        self.model.eval()
        self.batch_size, self._max_length, self.max_gen_toks = int(batch_size), max_length, max_gen_toks
        self.dev = next(self.model.parameters()).device

    @property
    def eot_token_id(self):
        return getattr(self.tokenizer, "eos_token_id", 0)

    @property
    def max_length(self):
        return self._max_length

    def tok_encode(self, string: str, **kwargs) -> List[int]:
        return self.tokenizer.encode(string, add_special_tokens=False)

    def _score(self, context_ids: List[int], cont_ids: List[int]) -> Tuple[float, bool]:
        ids = (context_ids + cont_ids)[-self.max_length:]
        n_cont = min(len(cont_ids), len(ids) - 1)
        x = torch.tensor([ids], device=self.dev)
        with torch.no_grad():
            logits = self.model(x).float()                          # [T, V]
        logp = torch.log_softmax(logits[:-1], dim=-1)
        tgt = x[0, 1:]
        tail = slice(len(ids) - 1 - n_cont, len(ids) - 1)
        ll = logp[tail].gather(1, tgt[tail].unsqueeze(1)).sum().item()
        greedy = bool((logp[tail].argmax(-1) == tgt[tail]).all())
        return ll, greedy

    def _requests(self, requests):
        for r in requests:
            yield r.args if hasattr(r, "args") else r

    def loglikelihood(self, requests, disable_tqdm: bool = False):
        out = []
        for context, continuation in self._requests(requests):
            ctx = self.tok_encode(context) if context else [self.eot_token_id]
            out.append(self._score(ctx, self.tok_encode(continuation)))
        return out

    def _loglikelihood_tokens(self, requests, disable_tqdm: bool = False):
        return [self._score(ctx, cont) for _, ctx, cont in requests]

    def loglikelihood_rolling(self, requests, disable_tqdm: bool = False):
        out = []
        for (text,) in self._requests(requests):
            ids = self.tok_encode(text)
            total, prev = 0.0, [self.eot_token_id]
            for i in range(0, len(ids), self.max_length - 1):
                chunk = ids[i:i + self.max_length - 1]
                total += self._score(prev, chunk)[0]
                prev = chunk[-1:]
            out.append(total)
        return out

    def generate_until(self, requests, disable_tqdm: bool = False):
        out = []
        for context, gen_kwargs in self._requests(requests):
            until = gen_kwargs.get("until", []) if isinstance(gen_kwargs, dict) else []
            until = [until] if isinstance(until, str) else list(until)
            max_new = gen_kwargs.get("max_gen_toks", self.max_gen_toks) if isinstance(gen_kwargs, dict) else self.max_gen_toks
            ids = self.tok_encode(context)[-(self.max_length - max_new):]
            toks = self.model.generate([ids], max_new_tokens=max_new, do_sample=False, eos_token_id=self.eot_token_id)[0]
            text = self.tokenizer.decode(toks[len(ids):], skip_special_tokens=True)
            for stop in until:
                if stop and stop in text:
                    text = text.split(stop)[0]
            out.append(text)
        return out


def main():
    try:
        from lm_eval.__main__ import cli_evaluate
    except ImportError:
        raise SystemExit("the lm_eval package is not installed; import MFLM and call its methods directly")
    cli_evaluate()


if __name__ == "__main__":
    main()

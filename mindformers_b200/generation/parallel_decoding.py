"""Parallel (speculative) decoding plug-ins (``mindformers/generation/parallel_decoding.py:47-213``: a registry with
"la" lookahead decoding, memory decoding and prefix cache).

Both plug-ins here draft several tokens without running the model and verify them in ONE model call on
``[last token] + draft`` (a short chunk appended to the paged KV cache); the longest prefix of the draft that matches the
model's own greedy choices is accepted, plus the model's next token, so the output equals plain greedy decoding token for
token while the number of model calls drops.

* ``"la"`` (lookahead): drafts come from n-grams seen earlier in the same sequence (prompt and generated text);
* ``"memory_decoding"``: the n-gram pool also remembers every sequence generated before by this model object;
* ``"mtp"``: the draft comes from the model's multi-token-prediction layer (one token per step), see
  ``mtp_speculative_decoding``.
Rejected draft tokens are rolled back in the block manager; their cache slots are simply rewritten.
"""
from __future__ import annotations

import time
from collections import defaultdict
from typing import Callable, Dict, List, Optional

import torch

_PLUGINS: Dict[str, Callable] = {}


def register_decoding_plugin(name: str):
    def deco(fn):
        _PLUGINS[name] = fn
        return fn
    return deco


def get_plugin(name: str):
    if name not in _PLUGINS:
        raise KeyError(f"parallel decoding {name!r} is not registered; known: {sorted(_PLUGINS)}")
    return _PLUGINS[name]


class NgramPool:
    """``n``-gram → most recent continuation, for ``n`` from ``max_ngram`` down to 1."""

    def __init__(self, max_ngram: int = 3):
        self.n = max_ngram
        self.table: Dict[tuple, List[int]] = {}

    def add(self, seq: List[int], start: int = 0, span: int = 8):
        for i in range(max(start, 1), len(seq)):
            for n in range(1, self.n + 1):
                if i - n < 0:
                    break
                self.table[tuple(seq[i - n:i])] = seq[i:i + span]

    def propose(self, seq: List[int], k: int) -> List[int]:
        for n in range(min(self.n, len(seq)), 0, -1):
            hit = self.table.get(tuple(seq[-n:]))
            if hit:
                return hit[:k]
        return []


def _speculative_generate(model, prompts, gcfg, max_len, pool_of, draft_len: int = 4, max_ngram: int = 3):
    if gcfg.do_sample:
        raise ValueError("parallel decoding verifies drafts against greedy choices; set do_sample=False")
    B = len(prompts)
    eos = set(gcfg.eos_ids())
    ctx, tables = model._set_kv_cache(B, max_len + draft_len + 1, getattr(model.config, "num_blocks", None))
    tables.init_cache_engine(B)
    seqs = [list(p) for p in prompts]
    limits = [max_len if gcfg.max_new_tokens is None else len(p) + gcfg.max_new_tokens for p in prompts]
    pools = [pool_of(i, max_ngram) for i in range(B)]
    for pl, s in zip(pools, seqs):
        pl.add(s)
    t0 = time.time()
    logits = model._forward_step(seqs, [0] * B, ctx, tables, True)
    nxt = logits.float().argmax(-1).tolist()
    finished = [False] * B
    calls, accepted_total, new_tokens = 1, 0, 0
    for i in range(B):
        seqs[i].append(int(nxt[i]))
        new_tokens += 1
        finished[i] = int(nxt[i]) in eos or len(seqs[i]) >= limits[i]
    while not all(finished):
        act = [not f for f in finished]
        drafts = [pools[i].propose(seqs[i], min(draft_len, limits[i] - len(seqs[i]) - 1)) if act[i] else [] for i in range(B)]
        toks = [[seqs[i][-1]] + drafts[i] if act[i] else [] for i in range(B)]
        starts = [len(seqs[i]) - 1 for i in range(B)]
        out = model._forward_step(toks, starts, ctx, tables, True, act, all_logits=True)
        calls += 1
        greedy = out.float().argmax(-1).tolist()
        off = 0
        for i in range(B):
            if not act[i]:
                continue
            g = greedy[off:off + len(toks[i])]
            off += len(toks[i])
            n_ok = 0
            while n_ok < len(drafts[i]) and drafts[i][n_ok] == g[n_ok]:
                n_ok += 1
            accepted_total += n_ok
            before = len(seqs[i])
            for t in drafts[i][:n_ok] + [g[n_ok]]:
                seqs[i].append(int(t))
                new_tokens += 1
                if int(t) in eos or len(seqs[i]) >= limits[i]:
                    finished[i] = True
                    break
            # the cache now holds 1 + len(draft) new positions; keep those of the accepted draft tokens only
            tables.engines[i].rollback(len(drafts[i]) - n_ok)
            pools[i].add(seqs[i], start=max(before - max_ngram, 1))
    tables.clear_cache()
    dt = max(time.time() - t0, 1e-9)
    model.last_generation_stats = {"new_tokens": new_tokens, "model_calls": calls, "accepted_draft_tokens": accepted_total,
                                   "tokens_per_call": new_tokens / calls, "total_s": dt, "tokens_per_s": new_tokens / dt}
    return seqs


@register_decoding_plugin("la")
def lookahead_decoding(model, prompts, gcfg, max_len, draft_len: int = 4, max_ngram: int = 3):
    return _speculative_generate(model, prompts, gcfg, max_len, lambda i, n: NgramPool(n), draft_len, max_ngram)


@register_decoding_plugin("memory_decoding")
def memory_decoding(model, prompts, gcfg, max_len, draft_len: int = 4, max_ngram: int = 3):
    shared = getattr(model, "_decoding_memory", None)
    if shared is None or shared.n != max_ngram:
        shared = model._decoding_memory = NgramPool(max_ngram)
    out = _speculative_generate(model, prompts, gcfg, max_len, lambda i, n: shared, draft_len, max_ngram)
    for s in out:
        shared.add(s)
    return out


@register_decoding_plugin("prefix_cache")
def prefix_cache_decoding(model, prompts, gcfg, max_len, **kw):
    """Prompts that share a prefix: the prefix is prefilled once per distinct prefix and the KV blocks of whole shared
    blocks are copied to the other sequences before their own remainder is prefilled."""
    B = len(prompts)
    common = 0
    if B > 1:
        while all(len(p) > common + 1 for p in prompts) and len({p[common] for p in prompts}) == 1:
            common += 1
    ctx, tables = model._set_kv_cache(B, max_len, getattr(model.config, "num_blocks", None))
    tables.init_cache_engine(B)
    bs = tables.block_size
    shared = (common // bs) * bs
    seqs = [list(p) for p in prompts]
    eos = set(gcfg.eos_ids())
    if shared:
        act0 = [i == 0 for i in range(B)]
        model._forward_step([p[:shared] if i == 0 else [] for i, p in enumerate(prompts)], [0] * B, ctx, tables, True, act0)
        src = tables.engines[0].blocks[: shared // bs]
        for i in range(1, B):
            tables.engines[i].prepare_cache(shared)
            dst = tables.engines[i].blocks[: shared // bs]
            for layer in range(len(ctx.key_cache)):
                ctx.key_cache[layer][dst] = ctx.key_cache[layer][src]
                if ctx.value_cache[layer] is not None:
                    ctx.value_cache[layer][dst] = ctx.value_cache[layer][src]
    logits = model._forward_step([p[shared:] for p in prompts], [shared] * B, ctx, tables, True)
    finished = [False] * B
    limits = [max_len if gcfg.max_new_tokens is None else len(p) + gcfg.max_new_tokens for p in prompts]
    while True:
        nxt = logits.float().argmax(-1).tolist()
        for i in range(B):
            if not finished[i]:
                seqs[i].append(int(nxt[i]))
                finished[i] = int(nxt[i]) in eos or len(seqs[i]) >= limits[i]
        if all(finished):
            break
        act = [not f for f in finished]
        logits = model._forward_step([[s[-1]] for s in seqs], [len(s) - 1 for s in seqs], ctx, tables, False, act)
    tables.clear_cache()
    model.last_generation_stats = {"shared_prefix_tokens": shared}
    return seqs


@register_decoding_plugin("mtp")
def mtp_speculative_decoding(model, prompts, gcfg, max_len, **kw):
    """Speculative decoding with the model's own multi-token-prediction layer as the drafter (DeepSeek-V3; reference
    ``research/deepseek3/deepseek3_model_infer.py:1729-1903``).

    The MTP layer at position ``p`` reads the main model's hidden state of ``p`` and the embedding of token ``p + 1``
    and predicts token ``p + 2``. Every step the main model runs on two tokens per sequence — the last accepted one and
    the draft — and yields the greedy successors of both; the draft is accepted when it equals the first. The MTP layer
    then runs on the same two positions with the now-known successors and its output at the last valid position is the
    next draft. It keeps its keys / values in one extra layer of the paged cache (same block tables and slots as the
    main layers), and a rejected position is simply overwritten by the next step. The output equals plain greedy
    decoding; ``model.last_generation_stats`` reports how many drafts were accepted."""
    from ..parallel import parallel_state as ps
    if gcfg.do_sample:
        raise ValueError("MTP speculative decoding verifies drafts against greedy choices; set do_sample=False")
    gpt = model.model
    if getattr(gpt, "mtp", None) is None or not len(gpt.mtp.layers):
        raise ValueError("the model has no multi-token-prediction layer (mtp_num_layers = 0)")
    if ps.get_pipeline_model_parallel_world_size() > 1:
        raise ValueError("MTP speculative decoding needs the whole model on one pipeline stage")
    drafter = gpt.mtp.layers[0]
    B = len(prompts)
    eos = set(gcfg.eos_ids())
    ctx, tables = model._set_kv_cache(B, max_len + 2, getattr(model.config, "num_blocks", None), extra_layers=1)
    tables.init_cache_engine(B)
    seqs = [list(p) for p in prompts]
    limits = [max_len if gcfg.max_new_tokens is None else len(p) + gcfg.max_new_tokens for p in prompts]
    rotary = gpt.rotary_pos_emb() if gpt.rotary_pos_emb is not None else None
    tp = ps.get_tensor_model_parallel_world_size()

    def draft_logits(next_ids: torch.Tensor, hidden: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """MTP layer on the positions of the main step that just ran (the cache context still describes them)."""
        from ..parallel.layers.attention import AttnMeta
        emb = gpt.embedding(next_ids.unsqueeze(0))
        meta = AttnMeta(batch=1, seq_len=int(next_ids.numel()), positions=positions, cache=ctx)
        out, _ = drafter(emb, hidden, rotary, meta)
        logits = gpt.logits(out).float()
        if tp > 1:
            parts = [torch.empty_like(logits) for _ in range(tp)]
            torch.distributed.all_gather(parts, logits.contiguous(), group=ps.get_tensor_model_parallel_group())
            logits = torch.cat(parts, dim=-1)
        return logits[:, : model.config.vocab_size]

    t0 = time.time()
    device = next(model.parameters()).device
    # ---- prefill: main model, then the MTP layer over the same positions with the tokens shifted left by one ----
    logits, hidden, flat, pos = model._forward_step(seqs, [0] * B, ctx, tables, True, return_hidden=True)
    nxt = logits.argmax(-1).tolist()
    shifted = flat.clone()
    ends = ctx.last_token_index.tolist()
    shifted[:-1] = flat[1:]
    for b, e in enumerate(ends):
        shifted[e] = int(nxt[b])                      # the successor of a prompt's last token is the sampled one
    d_logits = draft_logits(shifted, hidden, pos)
    drafts = d_logits.index_select(0, ctx.last_token_index).argmax(-1).tolist()
    finished = [False] * B
    calls, accepted_total, new_tokens, proposed = 1, 0, 0, 0
    for i in range(B):
        seqs[i].append(int(nxt[i]))
        new_tokens += 1
        finished[i] = int(nxt[i]) in eos or len(seqs[i]) >= limits[i]
    while not all(finished):
        act = [not f for f in finished]
        use_draft = [act[i] and len(seqs[i]) + 1 < limits[i] for i in range(B)]
        toks = [([seqs[i][-1], int(drafts[i])] if use_draft[i] else [seqs[i][-1]]) if act[i] else [] for i in range(B)]
        starts = [len(seqs[i]) - 1 for i in range(B)]
        logits, hidden, flat, pos = model._forward_step(toks, starts, ctx, tables, True, act, all_logits=True,
                                                        return_hidden=True)
        calls += 1
        greedy = logits.argmax(-1).tolist()
        successors = list(greedy)                     # token that follows each fed position, as the main model sees it
        pick, off = [], 0                             # row whose MTP output becomes the next draft, per active sequence
        for i in range(B):
            if not act[i]:
                continue
            n = len(toks[i])
            g = greedy[off:off + n]
            ok = n == 2 and int(drafts[i]) == g[0]
            proposed += int(n == 2)
            accepted_total += int(ok)
            for t in (g if ok else g[:1]):
                seqs[i].append(int(t))
                new_tokens += 1
                if int(t) in eos or len(seqs[i]) >= limits[i]:
                    finished[i] = True
                    break
            if n == 2 and not ok:
                tables.engines[i].rollback(1)         # the position computed from the wrong draft is not kept
            pick.append(off + (1 if ok else 0))
            off += n
        d_logits = draft_logits(torch.tensor(successors, dtype=torch.int64, device=device), hidden, pos)
        chosen = d_logits.index_select(0, torch.tensor(pick, dtype=torch.int64, device=device)).argmax(-1).tolist()
        j = 0
        for i in range(B):
            if act[i]:
                drafts[i] = chosen[j]
                j += 1
    tables.clear_cache()
    dt = max(time.time() - t0, 1e-9)
    model.last_generation_stats = {"new_tokens": new_tokens, "model_calls": calls, "proposed_draft_tokens": proposed,
                                   "accepted_draft_tokens": accepted_total, "tokens_per_call": new_tokens / calls,
                                   "total_s": dt, "tokens_per_s": new_tokens / dt}
    return seqs

"""Continuous-batching serving engine.

The reference hands serving to an external engine (``scripts/run_mindie.sh`` starts a MindIE service, which drives
``mindformers/model_runner.py``: ``forward(input_ids, valid_length_each_example, block_tables, slot_mapping, prefill)``
plus block swapping). That engine is not part of the reference's sources; this is its counterpart on the same model
interface: requests join and leave a running batch at token granularity.

One iteration (``step()``):

1. finished and aborted requests give their slot and cache blocks back;
2. waiting requests are admitted while a slot is free and the block pool can hold their prompt (first come, first
   served; a request that was preempted re-enters with the tokens it had produced, so its cache is recomputed);
3. if requests were admitted, one prefill call runs their prompts (long prompts in chunks of ``max_prefill_tokens``);
   otherwise one decode call advances every running request by a token — before it, the newest requests are
   preempted while the pool cannot give every running request the block its next token may need;
   When every running request decodes greedily (or at one common temperature without top-k / top-p / penalties) and
   shares its stop tokens, the decode call is a BURST instead (``decode_burst`` steps, default 8): the step was
   captured in a CUDA graph together with the token selection and the update of positions and cache slots
   (``generation/device_loop.py``), the graph is replayed ``decode_burst`` times without host work in between, and
   the tokens are read back once. Requests that finish inside a burst stop there; new arrivals wait for its end;
4. the next token of every request that was served is chosen (greedy, or temperature / top-k / top-p / penalties with
   a per-request seeded generator), stop conditions are checked and the ``on_token`` callbacks are called.

With several tensor-parallel ranks every rank runs the same engine: rank 0 owns the queue and broadcasts the requests
it admits and aborts each iteration; everything else is a deterministic function of those, and the logits are
identical on all ranks, so the ranks stay in lockstep without exchanging schedules.

Timing per request: queue time, time to first token, time per output token; ``stats()`` aggregates them (mean, p50,
p99) for the ``/metrics`` endpoint.
"""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional

import numpy as np
import torch

from ..generation.logits_process import (FrequencyPenaltyLogitsProcessor, LogitsProcessorList,
                                         PresencePenaltyLogitsProcessor, RepetitionPenaltyLogitsProcessor,
                                         SamplingLogitsProcessor)


@dataclass
class SamplingParams:
    max_tokens: int = 64
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    seed: Optional[int] = None
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False

    @property
    def greedy(self) -> bool:
        return not self.temperature or self.temperature <= 1e-5 or self.top_k == 1


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: List[int]
    token_ids: List[int]
    finished: bool
    finish_reason: Optional[str]            # "stop" | "length" | "abort"
    metrics: Dict[str, float]


class Request:
    def __init__(self, request_id: str, prompt_token_ids: List[int], params: SamplingParams,
                 on_token: Optional[Callable[["Request", int], None]] = None):
        self.request_id, self.prompt, self.params, self.on_token = request_id, list(prompt_token_ids), params, on_token
        self.output: List[int] = []
        self.slot: Optional[int] = None
        self.cached = 0                    # tokens of prompt + output that are in the KV cache
        self.finished = False
        self.finish_reason: Optional[str] = None
        self.t_arrive = time.perf_counter()
        self.t_first: Optional[float] = None
        self.t_sched: Optional[float] = None
        self.t_done: Optional[float] = None
        self.preemptions = 0
        self.done_event = threading.Event()
        self._gen: Optional[torch.Generator] = None
        procs = LogitsProcessorList()
        if params.repetition_penalty and params.repetition_penalty != 1.0:
            procs.append(RepetitionPenaltyLogitsProcessor(params.repetition_penalty))
        if params.frequency_penalty:
            procs.append(FrequencyPenaltyLogitsProcessor(params.frequency_penalty))
        if params.presence_penalty:
            procs.append(PresencePenaltyLogitsProcessor(params.presence_penalty))
        self.processors = procs
        self.warper = None if params.greedy else SamplingLogitsProcessor(True, params.temperature, params.top_k, params.top_p)

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def result(self) -> RequestOutput:
        m = {"queue_s": (self.t_sched or self.t_arrive) - self.t_arrive,
             "ttft_s": (self.t_first - self.t_arrive) if self.t_first else float("nan"),
             "preemptions": float(self.preemptions)}
        if self.t_done and self.t_first and len(self.output) > 1:
            m["tpot_s"] = (self.t_done - self.t_first) / (len(self.output) - 1)
        if self.t_done:
            m["e2e_s"] = self.t_done - self.t_arrive
        return RequestOutput(self.request_id, list(self.prompt), list(self.output), self.finished, self.finish_reason, m)


class ServingEngine:
    """``model``: a ``PreTrainedModel`` (anything with the generation mixin's ``_set_kv_cache`` / ``_forward_step``).

    ``max_num_seqs`` slots share ``num_blocks`` cache blocks (default: enough for every slot at ``max_model_len``;
    give fewer to over-subscribe, the engine then preempts). ``max_prefill_tokens`` bounds the new tokens of one
    prefill call."""

    def __init__(self, model, max_num_seqs: int = 8, max_model_len: Optional[int] = None, num_blocks: Optional[int] = None,
                 max_prefill_tokens: int = 8192, eos_token_id=None, decode_burst: int = 8):
        self.model = model.eval()
        self.decode_burst = int(decode_burst)         # < 2: every decode step returns to the host
        self._loop = None                             # captured step + its static tensors (built by the first burst)
        cfg = model.config
        self.max_num_seqs = int(max_num_seqs)
        self.max_model_len = int(max_model_len or getattr(cfg, "seq_length", 2048))
        self.ctx, self.tables = model._set_kv_cache(self.max_num_seqs, self.max_model_len, num_blocks)
        if num_blocks:        # an explicit pool size over-subscribes the slots: rebuild the tables around it
            from ..inference.block_manager import BlockTables
            from ..inference.paged_attention import KVCacheContext  # noqa: F401  (the cache itself was sized by the model)
            if int(num_blocks) < self.tables.pool.num_blocks:
                self.tables = BlockTables(int(num_blocks), self.tables.block_size, self.max_model_len)
        self.tables.init_cache_engine(self.max_num_seqs)
        self.block_size = self.tables.block_size
        self.max_prefill_tokens = int(max_prefill_tokens)
        eos = eos_token_id if eos_token_id is not None else getattr(getattr(model, "generation_config", None), "eos_token_id", None)
        self.eos_ids = set(eos if isinstance(eos, (list, tuple, set)) else ([] if eos is None else [eos]))
        self.waiting: Deque[Request] = deque()
        self.running: List[Optional[Request]] = [None] * self.max_num_seqs
        self._admit_order: List[Request] = []
        self._incoming: Deque[Request] = deque()
        self._aborts: Deque[str] = deque()
        self._lock = threading.Lock()
        self._wake = threading.Event()
        self._stop = False
        self._thread: Optional[threading.Thread] = None
        self.finished_metrics: Deque[Dict[str, float]] = deque(maxlen=4096)
        self.counters = {"requests": 0, "finished": 0, "aborted": 0, "preempted": 0, "prefill_tokens": 0,
                         "decode_tokens": 0, "steps": 0, "bursts": 0}
        self._by_id: Dict[str, Request] = {}

    # ---- submission (any thread) ---------------------------------------------------------------------------------
    def add_request(self, request_id: str, prompt_token_ids: List[int], params: Optional[SamplingParams] = None,
                    on_token=None) -> Request:
        params = params or SamplingParams()
        if not prompt_token_ids:
            raise ValueError("empty prompt")
        if len(prompt_token_ids) + 1 > self.max_model_len:
            raise ValueError(f"prompt of {len(prompt_token_ids)} tokens does not fit max_model_len {self.max_model_len}")
        need = -(-min(len(prompt_token_ids) + params.max_tokens, self.max_model_len) // self.block_size)
        if need > self.tables.pool.num_blocks:
            raise ValueError("the request needs more cache blocks than the pool holds")
        req = Request(request_id, prompt_token_ids, params, on_token)
        with self._lock:
            self._incoming.append(req)
            self.counters["requests"] += 1
        self._wake.set()
        return req

    def abort(self, request_id: str):
        with self._lock:
            self._aborts.append(request_id)
        self._wake.set()

    # ---- scheduling --------------------------------------------------------------------------------------------------
    def _free_slot(self) -> Optional[int]:
        for i, r in enumerate(self.running):
            if r is None:
                return i
        return None

    def _release(self, req: Request, reason: str):
        if req.slot is not None:
            self.tables.engines[req.slot].release()
            self.running[req.slot] = None
            req.slot = None
        if req in self._admit_order:
            self._admit_order.remove(req)
        req.finished, req.finish_reason, req.t_done = True, reason, time.perf_counter()
        self._by_id.pop(req.request_id, None)
        self.counters["aborted" if reason == "abort" else "finished"] += 1
        self.finished_metrics.append(req.result().metrics)
        req.done_event.set()
        if req.on_token is not None:
            req.on_token(req, -1)              # end-of-stream marker

    def _preempt(self, req: Request):
        """Take the request out of the batch; it re-enters at the head of the queue and recomputes its cache."""
        self.tables.engines[req.slot].release()
        self.running[req.slot] = None
        req.slot, req.cached = None, 0
        req.preemptions += 1
        self._admit_order.remove(req)
        self.waiting.appendleft(req)
        self.counters["preempted"] += 1

    def _blocks_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.block_size)

    def _sync_inbox(self):
        """Move submissions and aborts from the inbox into the scheduler's state; with several ranks, rank 0's inbox is
        broadcast so that every rank sees the same requests in the same iteration."""
        with self._lock:
            new, aborts = list(self._incoming), list(self._aborts)
            self._incoming.clear()
            self._aborts.clear()
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            box = [[(r.request_id, r.prompt, r.params) for r in new], aborts] if dist.get_rank() == 0 else [None, None]
            dist.broadcast_object_list(box, src=0)
            if dist.get_rank() != 0:
                new = [Request(rid, p, sp) for rid, p, sp in box[0]]
                aborts = box[1]
        for r in new:
            self.waiting.append(r)
            self._by_id[r.request_id] = r
        for rid in aborts:
            r = self._by_id.get(rid)
            if r is None or r.finished:
                continue
            if r in self.waiting:
                self.waiting.remove(r)
            self._release(r, "abort")

    def has_work(self) -> bool:
        return bool(self.waiting or self._incoming or self._aborts or any(r is not None for r in self.running))

    # ---- one iteration -----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> List[Request]:
        """Run one scheduling iteration; returns the requests that received a token."""
        self._sync_inbox()
        self.counters["steps"] += 1
        admitted: List[Request] = []
        budget = self.max_prefill_tokens
        while self.waiting:
            req = self.waiting[0]
            slot = self._free_slot()
            n = len(req.tokens)
            if slot is None or self._blocks_for(n + 1) > self.tables.pool.num_free or (admitted and n > budget):
                break
            self.waiting.popleft()
            req.slot = slot
            self.running[slot] = req
            self._admit_order.append(req)
            if req.t_sched is None:
                req.t_sched = time.perf_counter()
            # reserve the prompt's blocks now so that the next candidate sees the pool without them
            admitted.append(req)
            budget -= n
            self.tables.engines[slot].prepare_cache(0)
            need = self._blocks_for(n + 1)
            eng = self.tables.engines[slot]
            eng.blocks.extend(self.tables.pool.allocate(need - len(eng.blocks)))
        served: List[Request] = []
        if admitted:
            served = self._prefill(admitted)
        else:
            live = [r for r in self.running if r is not None]
            if not live:
                return []
            # every running request may need one more block for the token of this step
            def short():
                need = sum(1 for r in self.running if r is not None
                           and self._blocks_for(r.cached + 1) > len(self.tables.engines[r.slot].blocks))
                return need > self.tables.pool.num_free
            while short() and len(self._admit_order) > 1:
                self._preempt(self._admit_order[-1])
            burst = self._burst_length()
            if burst >= 2:
                return self._decode_burst(burst)
            served = self._decode()
        self._choose_tokens(served)
        return served

    # ---- decode bursts on the device --------------------------------------------------------------------------------
    def _stop_ids(self, r: Request):
        ids = set(r.params.stop_token_ids)
        if not r.params.ignore_eos:
            ids |= self.eos_ids
        return ids

    def _burst_length(self) -> int:
        """Steps the running batch may take without the host: 0 unless every running request can be served by the
        device-side selection with ONE setting and the pool can hold the burst's tokens."""
        if self.decode_burst < 2 or self._incoming or self._aborts:
            return 0
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            return 0                 # a graph that holds collectives must not outlive its process group
        live = [r for r in self.running if r is not None]
        first = live[0]
        stops = self._stop_ids(first)
        if len(stops) > 8:
            return 0
        for r in live:
            if len(r.processors) or self._stop_ids(r) != stops:
                return 0
            if r.params.greedy != first.params.greedy:
                return 0
            if not r.params.greedy and (r.params.top_k not in (0, None) or (r.params.top_p or 1.0) < 1.0
                                        or r.params.temperature != first.params.temperature):
                return 0
        steps = min(self.decode_burst, max(self._limit(r) - len(r.tokens) for r in live))
        if self.waiting:
            # requests queue for a slot: the burst ends when the first running request reaches its length limit, so
            # the slot it frees is handed over at once
            steps = min(steps, min(self._limit(r) - len(r.tokens) for r in live))
        steps = max(steps, 0)
        # blocks for the burst (the capture's warm-up runs may write three positions ahead)
        reach = max(steps, 3 if self._loop is None or self._loop["graph"] is None else steps)
        need = sum(max(0, self._blocks_for(min(r.cached + 1 + reach, self.max_model_len)) - len(self.tables.engines[r.slot].blocks))
                   for r in live)
        if need > self.tables.pool.num_free:
            return 0
        return steps if steps >= 2 else 0

    def _limit(self, r: Request) -> int:
        return min(len(r.prompt) + r.params.max_tokens, self.max_model_len)

    def _decode_burst(self, steps: int) -> List[Request]:
        from ..generation.device_loop import read_burst
        B = self.max_num_seqs
        live = [r for r in self.running if r is not None]
        first = live[0]
        if self._loop is None or self._loop["cap"] < self.decode_burst:
            entry = {"ctx": self.ctx, "captures": 0}
            self._loop = self.model._build_device_loop(entry, B, self.tables.max_blocks_per_seq, self.block_size,
                                                       self.decode_burst)
            self._loop["entry"] = entry
        loop = self._loop
        reach = max(steps, 3) if loop["graph"] is None else steps
        active = [r is not None for r in self.running]
        for r in live:
            self.tables.engines[r.slot].reserve(min(r.cached + 1 + reach, self.max_model_len))
        table, slots = self.tables.assemble_pa_inc_inputs(active, 1)
        st = loop["state"]
        toks = [self.running[i].tokens[-1] if active[i] else 0 for i in range(B)]
        pos = [self.running[i].cached if active[i] else 0 for i in range(B)]
        limits = [self._limit(self.running[i]) if active[i] else 1 for i in range(B)]
        st.load(toks, pos, table, slots, [not a for a in active], limits)
        seed = first.params.seed if first.params.seed is not None else hash(first.request_id) & 0x7FFFFFFF
        st.set_sampling(sorted(self._stop_ids(first)), 0.0 if first.params.greedy else float(first.params.temperature),
                        int(seed) + 7919 * self.counters["steps"])
        if loop["graph"] is None:
            loop["graph"] = loop["capture"]()
        loop["bind"]()
        for _ in range(steps):
            loop["graph"].replay()
        got = read_burst(st, steps)
        self.counters["bursts"] += 1
        now = time.perf_counter()
        for r in live:
            new = got[r.slot]
            stops = self._stop_ids(r)
            for tok in new:
                r.output.append(tok)
                r.cached += 1
                self.counters["decode_tokens"] += 1
                if r.t_first is None:
                    r.t_first = now
                if r.on_token is not None:
                    r.on_token(r, tok)
                if tok in stops:
                    self.tables.engines[r.slot].num_tokens = r.cached
                    self._release(r, "stop")
                    break
                if len(r.output) >= r.params.max_tokens or len(r.tokens) >= self.max_model_len:
                    self.tables.engines[r.slot].num_tokens = r.cached
                    self._release(r, "length")
                    break
            else:
                self.tables.engines[r.slot].num_tokens = r.cached      # the device advanced without the host's bookkeeping
        return live

    def _prefill(self, reqs: List[Request]) -> List[Request]:
        B = self.max_num_seqs
        remaining = {r.slot: r.tokens[r.cached:] for r in reqs}
        logits_of: Dict[int, torch.Tensor] = {}
        while any(remaining.values()):
            toks = [[] for _ in range(B)]
            starts = [0] * B
            active = [False] * B
            room = self.max_prefill_tokens
            for r in reqs:
                rest = remaining[r.slot]
                if not rest or room <= 0:
                    continue
                take = rest[:room]
                toks[r.slot], starts[r.slot], active[r.slot] = take, r.cached, True
                remaining[r.slot] = rest[len(take):]
                room -= len(take)
            logits = self.model._forward_step(toks, starts, self.ctx, self.tables, True, active)
            rows = [i for i in range(B) if active[i]]
            if logits.shape[0] == B:
                picked = {i: logits[i] for i in rows}
            else:                                   # one row per sequence that had tokens
                picked = {i: logits[j] for j, i in enumerate(rows)}
            for r in reqs:
                if active[r.slot]:
                    r.cached += len(toks[r.slot])
                    self.counters["prefill_tokens"] += len(toks[r.slot])
                    if not remaining[r.slot]:
                        logits_of[r.slot] = picked[r.slot]
        for r in reqs:
            r._logits = logits_of[r.slot]
        return reqs

    def _decode(self) -> List[Request]:
        B = self.max_num_seqs
        live = [r for r in self.running if r is not None]
        toks = [[0] for _ in range(B)]
        starts = [0] * B
        active = [False] * B
        for r in live:
            toks[r.slot], starts[r.slot], active[r.slot] = [r.tokens[-1]], r.cached, True
        logits = self.model._forward_step(toks, starts, self.ctx, self.tables, False, active)
        for r in live:
            r.cached += 1
            r._logits = logits[r.slot]
            self.counters["decode_tokens"] += 1
        return live

    def _choose_tokens(self, reqs: List[Request]):
        now = time.perf_counter()
        for r in reqs:
            scores = r._logits.float().unsqueeze(0)
            r._logits = None
            if len(r.processors):
                ids = torch.tensor([r.tokens], dtype=torch.int64, device=scores.device)
                scores = r.processors(ids, scores)
            if r.warper is None:
                tok = int(scores.argmax(-1))
            else:
                if r._gen is None:
                    r._gen = torch.Generator(device=scores.device)
                    r._gen.manual_seed(int(r.params.seed if r.params.seed is not None else hash(r.request_id) & 0x7FFFFFFF))
                scores = r.warper(None, scores)
                tok = int(torch.multinomial(torch.softmax(scores, dim=-1), 1, generator=r._gen))
            r.output.append(tok)
            if r.t_first is None:
                r.t_first = now
            if r.on_token is not None:
                r.on_token(r, tok)
            stop = (tok in self.eos_ids and not r.params.ignore_eos) or tok in r.params.stop_token_ids
            if stop:
                self._release(r, "stop")
            elif len(r.output) >= r.params.max_tokens or len(r.tokens) >= self.max_model_len:
                self._release(r, "length")

    # ---- drivers ---------------------------------------------------------------------------------------------------------
    def run_until_idle(self, max_steps: int = 1_000_000):
        n = 0
        while self.has_work() and n < max_steps:
            self.step()
            n += 1

    def generate(self, prompts: List[List[int]], params: Optional[SamplingParams] = None) -> List[RequestOutput]:
        """Offline helper: submit all prompts, run to completion, results in submission order."""
        reqs = [self.add_request(f"offline-{self.counters['requests']}-{i}", p, params) for i, p in enumerate(prompts)]
        self.run_until_idle()
        return [r.result() for r in reqs]

    def start(self):
        """Run the loop in a background thread (the HTTP front end's mode)."""
        if self._thread is not None:
            return

        def loop():
            while not self._stop:
                if self.has_work():
                    self.step()
                else:
                    self._wake.wait(timeout=0.05)
                    self._wake.clear()
        self._thread = threading.Thread(target=loop, name="serving-engine", daemon=True)
        self._thread.start()

    def shutdown(self):
        self._stop = True
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None

    def stats(self) -> Dict[str, float]:
        out = dict(self.counters)
        out["running"] = sum(r is not None for r in self.running)
        out["waiting"] = len(self.waiting) + len(self._incoming)
        out["free_blocks"] = self.tables.pool.num_free
        out["total_blocks"] = self.tables.pool.num_blocks
        for key in ("ttft_s", "tpot_s", "e2e_s", "queue_s"):
            vals = np.asarray([m[key] for m in self.finished_metrics if key in m and m[key] == m[key]], dtype=np.float64)
            if vals.size:
                out[f"{key}_mean"] = float(vals.mean())
                out[f"{key}_p50"] = float(np.percentile(vals, 50))
                out[f"{key}_p99"] = float(np.percentile(vals, 99))
        return out

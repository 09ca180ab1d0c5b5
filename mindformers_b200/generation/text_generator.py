"""``GenerationMixin``: prefill/decode loop over the paged KV cache with greedy, sampling and beam search.

Reference: ``generation/text_generator.py`` (``generate`` :731-1128, cache set-up :114-160, mcore input
preparation :1335-1382, chunked prefill :1541, post-processing :1590-1726, ``chat`` :1727). The loop runs on the
host, one iteration per generated token; the model sees flattened tokens ``[T]`` with ``positions``,
``q_seq_lens``, block tables and a slot mapping. Sampling runs on the device (one ``multinomial`` per step).
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from ..inference.block_manager import BlockTables
from ..inference.paged_attention import KVCacheContext
from ..parallel import parallel_state as ps
from ..parallel.layers.attention import AttnMeta
from ..tools.debug_info import DetailedLatency, Profiling
from ..tools.logger import logger
from .beam_search import BeamSearchScorer
from .generation_config import GenerationConfig
from .logits_process import LogitsProcessorList, SamplingLogitsProcessor, build_processors


class GenerationMixin:
    """Mixed into ``PreTrainedModel``; expects ``self.config`` (TransformerConfig-like) and ``self.model``
    (a ``GPTModel``)."""

    generation_config: Optional[GenerationConfig] = None

    # ---- cache --------------------------------------------------------------------------------------
    def _set_kv_cache(self, batch_size: int, max_len: int, num_blocks: Optional[int] = None, extra_layers: int = 0):
        cfg = self.config
        block_size = int(getattr(cfg, "block_size", 16) or 16)
        need = batch_size * (-(-max_len // block_size))
        num_blocks = max(int(num_blocks or 0), need)
        tp = ps.get_tensor_model_parallel_world_size()
        device = next(self.parameters()).device
        dtype = next(self.parameters()).dtype
        n_layers = len(self.model.decoder.layers) + extra_layers      # extra: multi-token-prediction layers that draft
        if getattr(cfg, "multi_latent_attention", False):
            ctx = KVCacheContext(n_layers, num_blocks, block_size, 1, 0, dtype, device,
                                 mla_latent_dim=cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim)
        else:
            kvh = max(1, cfg.num_query_groups // tp)
            ctx = KVCacheContext(n_layers, num_blocks, block_size, kvh, cfg.kv_channels, dtype, device,
                                 kv_cache_dtype=getattr(cfg, "kv_cache_dtype", None))
        ctx.layer_offset = self.model.decoder.layer_ids[0] if self.model.decoder.layer_ids else 0
        tables = BlockTables(num_blocks, block_size, max_len)
        return ctx, tables

    # ---- one model call -------------------------------------------------------------------------------
    @torch.no_grad()
    def _forward_step(self, tokens: List[List[int]], starts: List[int], ctx: KVCacheContext, tables: BlockTables,
                      prefill: bool, active: Optional[List[bool]] = None, all_logits: bool = False,
                      return_hidden: bool = False) -> torch.Tensor:
        """Run the model on the new ``tokens`` of every sequence (positions start at ``starts``).
        Returns logits ``[B, V]`` of the last new token of each sequence (``all_logits``: of every new token). With
        ``return_hidden`` the result is ``(logits, hidden [T, H] of every new token, flat token ids, positions)``."""
        device = next(self.parameters()).device
        lens = [len(t) for t in tokens]
        if hasattr(self, "set_phase"):
            self.set_phase(prefill)
        if prefill:
            table, slots = tables.assemble_pa_full_inputs(lens, active)
        else:
            table, slots = tables.assemble_pa_inc_inputs(active, 1)
        flat = torch.tensor([x for t in tokens for x in t], dtype=torch.int64, device=device)
        pos = torch.tensor([s + i for t, s in zip(tokens, starts) for i in range(len(t))], dtype=torch.int64, device=device)
        ctx.set_step(is_prefill=prefill, block_tables=table, slot_mapping=slots, context_lens=tables.context_lens(),
                     q_seq_lens=lens, device=device)
        if all_logits:       # draft verification: the logits of every new token are needed
            ctx.last_token_index = torch.arange(int(flat.numel()), dtype=torch.int64, device=device)
        meta = AttnMeta(batch=1, seq_len=int(flat.numel()), positions=pos, cache=ctx)
        hook = getattr(self, "input_embeds_hook", None)     # multimodal models splice encoder outputs in here
        embeds = hook(flat, pos, prefill) if hook is not None else None
        hidden_all = None
        if return_hidden:
            hidden_all = self.model(flat.unsqueeze(0), attn_meta=meta, return_hidden=True, input_embeds=embeds)
            rows = hidden_all if (all_logits or not prefill) else hidden_all.index_select(0, ctx.last_token_index)
            logits = self.model.logits(rows).float()
        elif embeds is not None:
            logits = self.model(flat.unsqueeze(0), attn_meta=meta, input_embeds=embeds)
        else:
            logits = self.model(flat.unsqueeze(0), attn_meta=meta)
        if all_logits:
            pass
        elif not prefill:
            pass  # decode: one row per sequence already
        elif logits.shape[0] == int(flat.numel()) and logits.shape[0] != int(ctx.last_token_index.numel()):
            logits = logits.index_select(0, ctx.last_token_index)      # a forward that returned a row per token
        tp = ps.get_tensor_model_parallel_world_size()
        if tp > 1:
            parts = [torch.empty_like(logits) for _ in range(tp)]
            torch.distributed.all_gather(parts, logits.contiguous(), group=ps.get_tensor_model_parallel_group())
            logits = torch.cat(parts, dim=-1)
        if return_hidden:
            return logits[:, : self.config.vocab_size], hidden_all, flat, pos
        return logits[:, : self.config.vocab_size]

    # ---- decode step as a CUDA graph ---------------------------------------------------------------------
    def _graph_decoder(self, B: int, ctx: KVCacheContext, tables: BlockTables):
        """Build a callable ``step(tokens, starts, active) -> logits [B, V]`` that replays one captured decode step.

        Everything the step reads lives in static device tensors (token ids, positions, block tables, slot mapping,
        context lengths); a step copies the new values in and replays. With tensor- or expert-parallel ranks the
        graph holds NCCL collectives and the expert exchange kernels (whose flag epochs are device counters); the
        one-shot GEMM + all-reduce kernel takes its epoch from the host, so row-parallel layers fall back to NCCL
        while a stream is capturing. Every rank must take the same decision, so it depends on the layout only.
        Returns None when the step cannot be captured (the caller then launches eagerly)."""
        device = next(self.parameters()).device
        if device.type != "cuda" or ps.get_pipeline_model_parallel_world_size() > 1 \
                or ps.get_context_parallel_world_size() > 1:
            return None
        tp = ps.get_tensor_model_parallel_world_size()
        width = tables.max_blocks_per_seq
        st_tok = torch.zeros(1, B, dtype=torch.int64, device=device)
        st_pos = torch.zeros(B, dtype=torch.int64, device=device)
        st_table = torch.zeros(B, width, dtype=torch.int32, device=device)
        st_slots = torch.zeros(B, dtype=torch.int32, device=device)
        st_lens = torch.ones(B, dtype=torch.int32, device=device)
        host = {k: torch.empty(t.shape, dtype=t.dtype).pin_memory() for k, t in
                (("tok", st_tok), ("pos", st_pos), ("table", st_table), ("slots", st_slots), ("lens", st_lens))}

        def bind():
            ctx.is_prefill = False
            ctx.block_tables, ctx.slot_mapping, ctx.context_lens = st_table, st_slots, st_lens
            ctx.q_seq_lens = torch.ones(B, dtype=torch.int32, device=device)
            ctx.cu_q = list(range(B + 1))
            ctx.last_token_index = torch.arange(B, dtype=torch.int64, device=device)

        def fill(tokens, starts, active):
            table, slots = tables.assemble_pa_inc_inputs(active, 1)
            host["tok"][0].copy_(torch.tensor([t[0] for t in tokens], dtype=torch.int64))
            host["pos"].copy_(torch.tensor(starts, dtype=torch.int64))
            host["table"].copy_(torch.from_numpy(table))
            host["slots"].copy_(torch.from_numpy(slots))
            host["lens"].copy_(torch.from_numpy(tables.context_lens()))
            for k, dst in (("tok", st_tok), ("pos", st_pos), ("table", st_table), ("slots", st_slots), ("lens", st_lens)):
                dst.copy_(host[k], non_blocking=True)

        def forward():
            meta = AttnMeta(batch=1, seq_len=B, positions=st_pos, cache=ctx)
            logits = self.model(st_tok, attn_meta=meta)
            if tp > 1:          # vocabulary-parallel head: every rank gets the full row
                parts = [torch.empty_like(logits) for _ in range(tp)]
                torch.distributed.all_gather(parts, logits.contiguous(), group=ps.get_tensor_model_parallel_group())
                logits = torch.cat(parts, dim=-1)
            return logits

        state = {"graph": None, "out": None}

        def step(tokens, starts, active):
            fill(tokens, starts, active)
            bind()
            if state["graph"] is None:
                # the first call runs eagerly twice on a side stream (lazy allocations, kernel attributes), then captures
                side = torch.cuda.Stream(device=device)
                side.wait_stream(torch.cuda.current_stream(device))
                with torch.cuda.stream(side):
                    forward()
                    forward()
                torch.cuda.current_stream(device).wait_stream(side)
                torch.cuda.synchronize(device)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    state["out"] = forward()
                state["graph"] = graph
            state["graph"].replay()
            return state["out"][:, : self.config.vocab_size]

        return step

    # ---- decode loop on the device -------------------------------------------------------------------------
    def _device_loop(self, B: int, max_len: int, num_blocks: Optional[int]):
        """KV cache, block tables and captured step of the device-side decode loop (``generation/device_loop.py``),
        kept on the model per geometry: a later ``generate`` call of the same batch size and length class reuses the
        cache memory and replays the graph captured by the first one. ``release_device_loops()`` frees them."""
        alloc_len = -(-int(max_len) // 256) * 256
        pool = self.__dict__.setdefault("_device_loops", {})
        key = (B, alloc_len, int(num_blocks or 0))
        entry = pool.get(key)
        if entry is None:
            while len(pool) >= 2:                       # each entry pins a KV cache: keep the two latest geometries
                pool.pop(next(iter(pool)))
            ctx, tables = self._set_kv_cache(B, alloc_len, num_blocks)
            entry = pool[key] = {"ctx": ctx, "geometry": (tables.pool.num_blocks, tables.block_size, alloc_len),
                                 "loop": None, "captures": 0}
        return entry, entry["ctx"], BlockTables(*entry["geometry"])

    def release_device_loops(self):
        """Drop the KV caches and graphs kept by the device-side decode loop. The capture closures refer back to their
        entry, so the references are cut by hand: the graphs are destroyed now, not at some later garbage collection
        (a live graph that holds collectives keeps ``destroy_process_group`` from returning)."""
        pool = self.__dict__.pop("_device_loops", None) or {}
        for entry in pool.values():
            loop = entry.get("loop")
            if loop:
                loop["graph"] = None
                loop.clear()
            entry.clear()
        pool.clear()

    def _build_device_loop(self, entry, B: int, width: int, block_size: int, cap: int):
        """Captures ``forward pass -> token selection -> state update`` of one decode step over static tensors."""
        from .device_loop import DecodeState, decode_advance
        ctx = entry["ctx"]
        device = next(self.parameters()).device
        tp = ps.get_tensor_model_parallel_world_size()
        st = DecodeState.allocate(B, width, block_size, cap, device)
        vocab = int(self.config.vocab_size)

        def bind():
            ctx.is_prefill = False
            ctx.block_tables, ctx.slot_mapping, ctx.context_lens = st.table, st.slots, st.lens
            ctx.q_seq_lens = torch.ones(B, dtype=torch.int32, device=device)
            ctx.cu_q = list(range(B + 1))
            ctx.last_token_index = torch.arange(B, dtype=torch.int64, device=device)

        def step():
            meta = AttnMeta(batch=1, seq_len=B, positions=st.pos, cache=ctx)
            logits = self.model(st.tok, attn_meta=meta)
            if tp > 1:          # vocabulary-parallel head: every rank gets the full row and picks the same token
                parts = [torch.empty_like(logits) for _ in range(tp)]
                torch.distributed.all_gather(parts, logits.contiguous(), group=ps.get_tensor_model_parallel_group())
                logits = torch.cat(parts, dim=-1)
            decode_advance(logits[:, :vocab].float(), st)

        class _Eager:                 # CPU tensors: the "graph" is the step itself
            replay = staticmethod(lambda: step())

        def capture():
            """Called with the state loaded for a real step: the warm-up runs advance it, so it is restored after."""
            bind()
            if device.type != "cuda":
                entry["captures"] += 1
                return _Eager
            keep = {k: getattr(st, k).clone() for k in ("tok", "pos", "lens", "slots", "count", "finished", "hist")}
            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                step()
                step()
            torch.cuda.current_stream(device).wait_stream(side)
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            for k, v in keep.items():
                getattr(st, k).copy_(v)
            entry["captures"] += 1
            return graph

        return {"state": st, "capture": capture, "bind": bind, "graph": None, "cap": cap}

    def _run_device_loop(self, entry, tables: BlockTables, seqs, prompts, finished, gcfg, eos, max_len, streamer, seed):
        """Decode bursts until every sequence is finished. ``seqs`` already hold the first generated token."""
        from .device_loop import read_burst
        B = len(seqs)
        burst = max(1, int(getattr(gcfg, "device_loop_steps", 16) or 16))
        limits = [max_len if gcfg.max_new_tokens is None else len(p) + gcfg.max_new_tokens for p in prompts]
        active = [not f for f in finished]
        tables.reserve(limits, active)
        table, slots = tables.assemble_pa_inc_inputs(active, 1)
        loop = entry["loop"]
        if loop is None or loop["cap"] < burst:
            loop = entry["loop"] = self._build_device_loop(entry, B, tables.max_blocks_per_seq, tables.block_size, burst)
        st = loop["state"]
        st.load([s[-1] for s in seqs], [len(s) - 1 for s in seqs], table, slots, finished, limits)
        temperature = float(gcfg.temperature) if gcfg.do_sample else 0.0
        base_seed = int(seed if seed is not None else (gcfg.seed if gcfg.seed is not None else torch.initial_seed()))
        st.set_sampling(eos, temperature, base_seed)
        if loop["graph"] is None:
            loop["graph"] = loop["capture"]()
        loop["bind"]()          # the prefill pointed the cache context at its own tensors (matters to eager replays only)
        new_tokens, bursts = 0, 0
        while not all(finished):
            if temperature > 0 and bursts:
                st.set_sampling(eos, temperature, base_seed + 0x9E3779B1 * bursts)   # the history index restarts per burst
            for _ in range(burst):
                loop["graph"].replay()
            got = read_burst(st, burst)
            bursts += 1
            for i, toks in enumerate(got):
                if finished[i]:
                    continue
                for t in toks:
                    seqs[i].append(t)
                    new_tokens += 1
                    if t in eos or len(seqs[i]) >= limits[i]:
                        finished[i] = True
                        break
            if streamer is not None:
                if B == 1:
                    streamer.put(got[0])
                else:
                    for j in range(max(len(g) for g in got)):
                        streamer.put([[g[j]] if j < len(g) else [gcfg.pad_token_id or 0] for g in got])
        return new_tokens

    # ---- public API -----------------------------------------------------------------------------------
    def _check_device_status(self):
        """After the last token was read back: a kernel whose bounded wait ran out, or an expert-parallel receive
        buffer that overflowed (token rows dropped), makes the generated text wrong, so both raise here instead of
        passing silently. Costs one 8-byte read; the sampling of the last token has synchronised already."""
        dev = next(self.model.parameters()).device
        if dev.type != "cuda":
            return
        from ..ops import _lib
        code, overflow = _lib.read_status_words(dev)
        _lib.raise_on_status(code, "during generate()")
        if overflow:
            _lib.status_word(dev)[1:2].zero_()
            raise RuntimeError("expert-parallel receive buffers overflowed during generate(): token rows were dropped. "
                               "Set moe_ep_buffer_factor in the model configuration to the expert-parallel size "
                               "(worst case) or generate with fewer tokens per prefill chunk")

    @torch.no_grad()
    def generate(self, input_ids: Union[Sequence[int], Sequence[Sequence[int]], torch.Tensor],
                 generation_config: Optional[GenerationConfig] = None, logits_processor: Optional[LogitsProcessorList] = None,
                 streamer=None, seed: Optional[int] = None, **kwargs):
        """Returns a list (one per prompt) of token-id lists: prompt followed by the generated tokens."""
        self.eval()
        gcfg = GenerationConfig(**(generation_config or self.generation_config or GenerationConfig()).to_dict())
        gcfg.update(**kwargs)
        prompts = self._normalise_inputs(input_ids, gcfg.pad_token_id)
        B = len(prompts)
        max_prompt = max(len(p) for p in prompts)
        max_len = gcfg.max_length if gcfg.max_new_tokens is None else max_prompt + gcfg.max_new_tokens
        max_len = min(int(max_len), int(getattr(self.config, "seq_length", max_len) or max_len)) \
            if gcfg.max_new_tokens is None else int(max_len)
        if max_len <= min(len(p) for p in prompts):
            raise ValueError(f"max_length ({max_len}) must exceed the prompt length")
        if gcfg.num_beams > 1:
            return self._beam_search(prompts, gcfg, max_len)
        plugin = kwargs.get("parallel_decoding") or getattr(gcfg, "parallel_decoding", None)
        if plugin:
            from .parallel_decoding import get_plugin
            return get_plugin(plugin)(self, prompts, gcfg, max_len, **{k: v for k, v in kwargs.items() if k in ("draft_len", "max_ngram")})
        device = next(self.parameters()).device
        gen = torch.Generator(device=device)
        if seed is not None or gcfg.seed is not None:
            gen.manual_seed(int(seed if seed is not None else gcfg.seed))
        processors = build_processors(gcfg, max_prompt)
        if logits_processor:
            processors.extend(logits_processor)
        warper = SamplingLogitsProcessor(True, gcfg.temperature, gcfg.top_k, gcfg.top_p) if gcfg.do_sample else None
        eos = set(gcfg.eos_ids())
        lockstep = ps.get_expert_model_parallel_world_size() > ps.get_tensor_model_parallel_world_size() \
            and torch.distributed.is_available() and torch.distributed.is_initialized()
        from .device_loop import fast_path_ok
        loop_entry = None
        if getattr(gcfg, "use_cuda_graph", False) and getattr(gcfg, "device_loop", True) \
                and ps.get_pipeline_model_parallel_world_size() == 1 and ps.get_context_parallel_world_size() == 1 \
                and fast_path_ok(gcfg, processors, B, lockstep):
            loop_entry, ctx, tables = self._device_loop(B, max_len, getattr(self.config, "num_blocks", None))
        else:
            ctx, tables = self._set_kv_cache(B, max_len, getattr(self.config, "num_blocks", None))
        tables.init_cache_engine(B)
        # latency breakdown (``self.detailed_latency.enabled`` or MF_DETAILED_LATENCY=1) and a profiler window over
        # token indices (MF_PROFILE_START_TOKEN / MF_PROFILE_STOP_TOKEN), tools/debug_info.py
        latency = getattr(self, "detailed_latency", None)
        if latency is None:
            latency = self.detailed_latency = DetailedLatency()
        profiling = Profiling()
        seqs = [list(p) for p in prompts]
        finished = [False] * B
        t0 = time.time()
        if streamer is not None:
            streamer.put(seqs if B > 1 else seqs[0])
        # prefill (optionally in chunks)
        chunk = gcfg.chunk_prefill_size
        if chunk and max_prompt > chunk:
            done = [0] * B
            logits = None
            while any(d < len(p) for d, p in zip(done, prompts)):
                toks = [p[d:d + chunk] for p, d in zip(prompts, done)]
                act = [len(t) > 0 for t in toks]
                step_logits = self._forward_step(toks, done, ctx, tables, True, act)
                if logits is None:
                    logits = torch.zeros(B, step_logits.shape[-1], device=device)
                rows = [i for i, a in enumerate(act) if a]
                for j, i in enumerate(rows):
                    if done[i] + len(toks[i]) >= len(prompts[i]):
                        logits[i] = step_logits[j]
                done = [d + len(t) for d, t in zip(done, toks)]
        else:
            profiling.step_begin(0)
            with latency.phase("predict", True):
                logits = self._forward_step(seqs, [0] * B, ctx, tables, True)
            profiling.step_end(0)
        ttft = time.time() - t0
        new_tokens = 0
        lockstep_group = None
        if ps.get_expert_model_parallel_world_size() > ps.get_tensor_model_parallel_world_size() \
                and torch.distributed.is_available() and torch.distributed.is_initialized():
            lockstep_group = ps.get_expert_model_parallel_group()
        graph_step = self._graph_decoder(B, ctx, tables) \
            if getattr(gcfg, "use_cuda_graph", False) and loop_entry is None else None
        step_index = 0
        while True:
            with latency.phase("postprocess", step_index == 0):
                nxt = self._select(seqs, logits, processors, warper, gen, gcfg)
            for i in range(B):
                if finished[i]:
                    continue
                tok = int(nxt[i])
                seqs[i].append(tok)
                new_tokens += 1
                limit = max_len if gcfg.max_new_tokens is None else len(prompts[i]) + gcfg.max_new_tokens
                if tok in eos or len(seqs[i]) >= limit:
                    finished[i] = True
            if streamer is not None:
                streamer.put([int(nxt[0])] if B == 1 else [[int(t)] for t in nxt])
            if lockstep_group is not None:
                # data-parallel attention with expert parallelism across the replicas: every rank of the expert group
                # takes part in each layer's token exchange, so a rank whose own batch is done keeps stepping (with no
                # active sequence) until all ranks are done
                flag = torch.tensor([0 if all(finished) else 1], dtype=torch.int32, device=device)
                torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX, group=lockstep_group)
                if int(flag.item()) == 0:
                    break
            elif all(finished):
                break
            if loop_entry is not None:
                # the first token came from the prefill logits on the host; the rest of the generation runs as bursts
                # of graph replays with the selection and the state update on the device
                with latency.phase("predict", False):
                    new_tokens += self._run_device_loop(loop_entry, tables, seqs, prompts, finished, gcfg, eos, max_len,
                                                        streamer, seed)
                if torch.distributed.is_available() and torch.distributed.is_initialized() \
                        and torch.distributed.get_world_size() > 1:
                    # the captured step holds collectives of the process groups: a graph that outlives the call keeps
                    # their communicators busy (destroy_process_group then never returns), so it is dropped here and
                    # only single-process generation reuses its capture
                    torch.cuda.synchronize(device)
                    self.release_device_loops()
                break
            with latency.phase("preprocess", False):
                act = [not f for f in finished]
                toks = [[s[-1]] for s in seqs]
                starts = [len(s) - 1 for s in seqs]
            step_index += 1
            profiling.step_begin(step_index)
            with latency.phase("predict", False):
                if graph_step is not None:
                    logits = graph_step(toks, starts, act)
                else:
                    logits = self._forward_step(toks, starts, ctx, tables, False, act)
            profiling.step_end(step_index)
        profiling.close()
        if latency.enabled:
            latency.print_info()
        if streamer is not None:
            streamer.end()
        tables.clear_cache()
        self._check_device_status()
        dt = max(time.time() - t0, 1e-9)
        self.last_generation_stats = {"ttft_s": ttft, "new_tokens": new_tokens, "total_s": dt,
                                      "tokens_per_s": new_tokens / dt}
        logger.info("generate: %d new tokens in %.3f s (%.1f tokens/s, first token %.3f s)", new_tokens, dt,
                    new_tokens / dt, ttft)
        return seqs

    def _select(self, seqs, logits, processors, warper, gen, gcfg):
        scores = logits.float()
        if not len(processors) and warper is None:
            return scores.argmax(-1).tolist()          # greedy without penalties: the token history is not needed
        L = max(len(s) for s in seqs)
        host = np.full((len(seqs), L), -1, dtype=np.int64)
        for i, s in enumerate(seqs):
            host[i, : len(s)] = s
        ids = torch.from_numpy(host).to(logits.device)  # one host-to-device copy for the whole batch
        if len(processors):
            scores = processors(ids, scores)
        if warper is None:
            return scores.argmax(-1).tolist()
        probs = torch.softmax(warper(ids, scores), dim=-1)
        return torch.multinomial(probs, 1, generator=gen).squeeze(-1).tolist()

    @staticmethod
    def _normalise_inputs(input_ids, pad_token_id) -> List[List[int]]:
        if isinstance(input_ids, torch.Tensor):
            input_ids = input_ids.tolist()
        if isinstance(input_ids, np.ndarray):
            input_ids = input_ids.tolist()
        if len(input_ids) and not isinstance(input_ids[0], (list, tuple)):
            input_ids = [list(input_ids)]
        out = []
        for row in input_ids:
            row = [int(x) for x in row]
            if pad_token_id is not None:
                while len(row) > 1 and row[-1] == pad_token_id:
                    row.pop()
            out.append(row)
        return out

    # ---- beam search ------------------------------------------------------------------------------------
    def _beam_search(self, prompts, gcfg, max_len):
        B, nb = len(prompts), gcfg.num_beams
        device = next(self.parameters()).device
        eos = gcfg.eos_ids()
        pad = gcfg.pad_token_id if gcfg.pad_token_id is not None else 0
        ctx, tables = self._set_kv_cache(B * nb, max_len, None)
        tables.init_cache_engine(B * nb)
        flat = [list(p) for p in prompts for _ in range(nb)]
        prompt_len = max(len(p) for p in prompts)
        scorer = BeamSearchScorer(B, nb, gcfg.length_penalty, gcfg.early_stopping, gcfg.num_return_sequences)
        beam_scores = torch.zeros(B, nb)
        beam_scores[:, 1:] = -1e9
        logits = self._forward_step(flat, [0] * (B * nb), ctx, tables, True)
        processors = build_processors(gcfg, prompt_len)
        while True:
            L = max(len(s) for s in flat)
            ids = torch.full((B * nb, L), -1, dtype=torch.int64, device=device)
            for i, s in enumerate(flat):
                ids[i, : len(s)] = torch.tensor(s, device=device)
            logp = torch.log_softmax(processors(ids, logits.float()) if len(processors) else logits.float(), dim=-1).cpu()
            V = logp.shape[-1]
            total = (logp.view(B, nb, V) + beam_scores.unsqueeze(-1)).view(B, nb * V)
            top_s, top_i = total.topk(2 * nb, dim=-1)
            seqs = [[flat[b * nb + k] for k in range(nb)] for b in range(B)]
            beam_scores, toks, idx = scorer.process(seqs, top_s, top_i % V, top_i // V, eos, prompt_len, pad)
            new_flat, src = [], []
            for b in range(B):
                for k in range(nb):
                    j = int(idx[b, k])
                    new_flat.append(seqs[b][j] + [int(toks[b, k])])
                    src.append(b * nb + j)
            self._reorder_cache(ctx, tables, src)
            flat = new_flat
            if scorer.is_done or max(len(s) for s in flat) >= max_len:
                break
            logits = self._forward_step([[s[-1]] for s in flat], [len(s) - 1 for s in flat], ctx, tables, False)
        seqs = [[flat[b * nb + k] for k in range(nb)] for b in range(B)]
        best = scorer.finalize(seqs, beam_scores, prompt_len)
        tables.clear_cache()
        if gcfg.num_return_sequences == 1:
            return [b[0] for b in best]
        return [s for b in best for s in b]

    @staticmethod
    def _reorder_cache(ctx: KVCacheContext, tables: BlockTables, src: List[int]):
        """Beam ``i`` continues from beam ``src[i]``: copy the cache contents block by block."""
        if src == list(range(len(src))):
            return
        dst_blocks, src_blocks = [], []
        for i, j in enumerate(src):
            if i == j:
                continue
            n = min(len(tables.engines[i].blocks), len(tables.engines[j].blocks))
            dst_blocks += tables.engines[i].blocks[:n]
            src_blocks += tables.engines[j].blocks[:n]
        if not dst_blocks:
            return
        d = torch.tensor(dst_blocks, device=ctx.key_cache[0].device)
        s = torch.tensor(src_blocks, device=ctx.key_cache[0].device)
        for layer in range(ctx.num_layers):
            ctx.key_cache[layer][d] = ctx.key_cache[layer][s].clone()
            if ctx.value_cache[layer] is not None:
                ctx.value_cache[layer][d] = ctx.value_cache[layer][s].clone()

    # ---- chat ---------------------------------------------------------------------------------------------
    def chat(self, tokenizer, query: str, history: Optional[list] = None, system_role_name: str = "system",
             user_role_name: str = "user", assistant_role_name: str = "assistant", instruction: str = "",
             max_length: int = 512, do_sample: bool = False, top_k: int = 1, top_p: float = 1.0,
             temperature: float = 1.0, repetition_penalty: float = 1.0):
        """One chat turn through the tokenizer's chat template; returns ``(response, history)``."""
        history = list(history or [])
        if instruction and not history:
            history.append({"role": system_role_name, "content": instruction})
        history.append({"role": user_role_name, "content": query})
        if hasattr(tokenizer, "apply_chat_template") and getattr(tokenizer, "chat_template", None):
            ids = tokenizer.apply_chat_template(history, add_generation_prompt=True, tokenize=True)
        else:
            text = "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in history) + f"<|{assistant_role_name}|>\n"
            ids = tokenizer.encode(text)
        out = self.generate([ids], max_length=max_length, do_sample=do_sample, top_k=top_k, top_p=top_p,
                            temperature=temperature, repetition_penalty=repetition_penalty,
                            eos_token_id=getattr(tokenizer, "eos_token_id", None),
                            pad_token_id=getattr(tokenizer, "pad_token_id", None))[0]
        response = tokenizer.decode(out[len(ids):], skip_special_tokens=True)
        history.append({"role": assistant_role_name, "content": response})
        return response, history

"""``ModelRunner``: the serving-engine facing object (MindIE / vLLM style engines drive it step by step).

Reference: ``mindformers/model_runner.py`` — ``ModelRunner(model_path, npu_mem_size, cpu_mem_size, block_size, rank_id,
world_size, ...)`` (:179), ``forward(input_ids, valid_length_each_example, block_tables, slot_mapping, prefill, ...)``
(:384), ``swap(block_tables, swap_type)`` moving KV blocks between device and host pools (:478), and
``InputBuilder.make_context`` chat templating (:524-595). The engine owns scheduling and the block allocator; this
class owns the weights, the paged KV cache (device pool sized from ``npu_mem_size`` GB, pinned host pool from
``cpu_mem_size`` GB) and one model call per step.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Sequence

import numpy as np
import torch

from .inference.paged_attention import KVCacheContext
from .parallel import parallel_state as ps
from .parallel.layers.attention import AttnMeta


class InputBuilder:
    """Chat prompt builder: uses the tokenizer's own chat template when it has one, else a role-tagged transcript."""

    def __init__(self, tokenizer, chat_template: str = "", system_role_name: str = "system", user_role_name: str = "user",
                 max_length: int = 2048):
        self.tokenizer, self.chat_template = tokenizer, chat_template
        self.system_role_name, self.user_role_name, self.max_length = system_role_name, user_role_name, max_length

    def make_context(self, rank: int, conversation: List[dict], add_generation_prompt: bool = True, adapt_to_max_length: bool = False,
                     **kwargs) -> List[int]:
        if hasattr(self.tokenizer, "apply_chat_template"):
            try:
                ids = self.tokenizer.apply_chat_template(conversation, add_generation_prompt=add_generation_prompt, tokenize=True,
                                                         chat_template=self.chat_template or None)
                return self._fit(list(ids), adapt_to_max_length)
            except Exception:
                pass
        text = "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in conversation)
        if add_generation_prompt:
            text += "<|assistant|>\n"
        return self._fit(self.tokenizer.encode(text), adapt_to_max_length)

    def _fit(self, ids, adapt):
        if adapt and len(ids) > self.max_length:
            ids = ids[-self.max_length:]
        return ids


def get_model(model_name_or_path: str, revision: Optional[str] = None, trust_remote_code: Optional[bool] = False, **kwargs):
    """What a serving front end needs before any weights are loaded (reference ``model_runner.py:93``): the tokenizer
    of the model directory and an ``InputBuilder`` that turns chat conversations into token ids. A directory whose
    configuration names a multimodal processor gets ``(processor, processor)`` instead."""
    if not os.path.isdir(model_name_or_path):
        raise ValueError(f"{model_name_or_path} does not exist or is not a directory.")
    from .models import AutoTokenizer
    proc_cfg = None
    for name in sorted(os.listdir(model_name_or_path)):
        if name.endswith((".yaml", ".yml")):
            from .tools.register import MindFormerConfig
            cfg = MindFormerConfig(os.path.join(model_name_or_path, name))
            p = cfg.get("processor")
            if p and (p.get("image_processor") or p.get("modal_transform") or p.get("model_transform_template")):
                proc_cfg = p
            break
    if proc_cfg is not None:
        from .models.processing_utils import build_processor
        processor = build_processor(proc_cfg)
        return processor, processor
    tokenizer = AutoTokenizer.from_pretrained(model_name_or_path, **{k: v for k, v in kwargs.items() if k != "use_fast"})
    return tokenizer, InputBuilder(tokenizer)


class ModelRunner:
    """Serving-side model wrapper (reference ``mindformers/model_runner.py:138,199``): builds the model and tokenizer
    from a directory and exposes ``forward(input_ids, valid_length_each_example, block_tables, slot_mapping, prefill,
    ...)`` over the paged KV cache, plus KV block swapping between device and host (``swap``)."""

    def __init__(self, model_path: str, npu_mem_size: float, cpu_mem_size: float, block_size: int, rank_id: int = 0,
                 world_size: int = 1, npu_device_ids: Optional[Sequence[int]] = None, plugin_params: Optional[str] = None,
                 model=None, tokenizer=None):
        from .models import AutoModel, AutoTokenizer
        self.rank_id, self.world_size, self.block_size = rank_id, world_size, int(block_size)
        if torch.cuda.is_available():
            ids = list(npu_device_ids) if npu_device_ids else list(range(torch.cuda.device_count()))
            torch.cuda.set_device(ids[rank_id % len(ids)])
        if world_size > 1 and not ps.model_parallel_is_initialized():
            import torch.distributed as dist
            if not dist.is_initialized():
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo", rank=rank_id, world_size=world_size)
            ps.initialize_model_parallel(tensor_model_parallel_size=world_size)
        self.model = model if model is not None else AutoModel.from_pretrained(model_path)
        self.model.eval()
        self.tokenizer = tokenizer
        if tokenizer is None and model_path:
            try:
                self.tokenizer = AutoTokenizer.from_pretrained(model_path)
            except Exception:
                self.tokenizer = None
        self.plugin_params = json.loads(plugin_params) if plugin_params else {}
        cfg = self.model.config
        first = next(self.model.parameters())
        self.device, self.dtype = first.device, first.dtype
        tp = ps.get_tensor_model_parallel_world_size()
        self.n_layers = len(self.model.model.decoder.layers)
        mla = bool(getattr(cfg, "multi_latent_attention", False))
        if mla:
            self.kv_heads, self.head_dim, width = 1, cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim, cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim
            per_block = self.n_layers * self.block_size * width * first.element_size()
        else:
            self.kv_heads = max(1, (cfg.num_query_groups or cfg.num_attention_heads) // tp)
            self.head_dim = cfg.kv_channels or cfg.hidden_size // cfg.num_attention_heads
            per_block = 2 * self.n_layers * self.block_size * self.kv_heads * self.head_dim * first.element_size()
        self.num_npu_blocks = max(1, int(npu_mem_size * (1 << 30)) // per_block)
        self.num_cpu_blocks = max(0, int(cpu_mem_size * (1 << 30)) // per_block)
        self.cache = KVCacheContext(self.n_layers, self.num_npu_blocks, self.block_size, self.kv_heads,
                                    0 if mla else self.head_dim, self.dtype, self.device, mla_latent_dim=self.head_dim if mla else None)
        self.cache.layer_offset = self.model.model.decoder.layer_ids[0] if self.model.model.decoder.layer_ids else 0
        pin = torch.cuda.is_available()
        self.cpu_key = [torch.zeros((self.num_cpu_blocks,) + tuple(k.shape[1:]), dtype=self.dtype, pin_memory=pin) for k in self.cache.key_cache]
        self.cpu_value = [None if v is None else torch.zeros((self.num_cpu_blocks,) + tuple(v.shape[1:]), dtype=self.dtype, pin_memory=pin)
                          for v in self.cache.value_cache]
        self.copy_stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, input_ids, valid_length_each_example, block_tables, slot_mapping, prefill: bool = True,
                position_ids=None, spec_mask=None, q_seq_lens=None, adapter_ids=None, **kwargs) -> torch.Tensor:
        """One step. ``input_ids``: flattened new tokens ``[T]``; ``valid_length_each_example [B]``: tokens in the cache
        after this step; ``block_tables [B, max_blocks]`` (−1 padded); ``slot_mapping [T]``. Returns fp32 logits
        ``[B, vocab]`` of the last new token of every sequence."""
        dev = self.device
        ids = torch.as_tensor(np.asarray(input_ids).reshape(-1), dtype=torch.int64, device=dev)
        valid = [int(x) for x in np.asarray(valid_length_each_example).reshape(-1)]
        B = len(valid)
        if q_seq_lens is None:
            q_lens = valid if prefill else [1] * B
        else:
            q_lens = [int(x) for x in np.asarray(q_seq_lens).reshape(-1)]
        if position_ids is None:
            pos = [v - q + i for v, q in zip(valid, q_lens) for i in range(q)]
        else:
            pos = np.asarray(position_ids).reshape(-1).tolist()
        pos = torch.as_tensor(pos, dtype=torch.int64, device=dev)
        self.cache.set_step(is_prefill=bool(prefill), block_tables=np.asarray(block_tables), slot_mapping=np.asarray(slot_mapping).reshape(-1),
                            context_lens=valid, q_seq_lens=q_lens, device=dev)
        if adapter_ids is not None and hasattr(self.model, "slora"):
            self.model.slora.set_adapter_ids(adapter_ids, q_lens)
        meta = AttnMeta(batch=1, seq_len=int(ids.numel()), positions=pos, cache=self.cache)
        logits = self.model.model(ids.unsqueeze(0), attn_meta=meta)
        if logits.shape[0] != B:
            logits = logits.index_select(0, self.cache.last_token_index)
        tp = ps.get_tensor_model_parallel_world_size()
        if tp > 1:
            parts = [torch.empty_like(logits) for _ in range(tp)]
            torch.distributed.all_gather(parts, logits.contiguous(), group=ps.get_tensor_model_parallel_group())
            logits = torch.cat(parts, dim=-1)
        return logits[:, : self.model.config.vocab_size].float()

    def swap(self, block_tables, swap_type: bool):
        """Copy KV blocks between pools. ``block_tables``: pairs ``[src, dst]``; ``swap_type`` True = device → host
        (swap out), False = host → device (swap in). Copies run on a side stream; the compute stream waits for them."""
        pairs = np.asarray(block_tables).reshape(-1, 2).tolist()
        if not pairs:
            return
        cur = torch.cuda.current_stream() if self.copy_stream is not None else None
        if self.copy_stream is not None:
            self.copy_stream.wait_stream(cur)
        ctx = torch.cuda.stream(self.copy_stream) if self.copy_stream is not None else _Null()
        with ctx:
            for layer in range(self.n_layers):
                for dev_pool, cpu_pool in ((self.cache.key_cache[layer], self.cpu_key[layer]),
                                           (self.cache.value_cache[layer], self.cpu_value[layer])):
                    if dev_pool is None:
                        continue
                    for src, dst in pairs:
                        if swap_type:
                            cpu_pool[dst].copy_(dev_pool[src], non_blocking=True)
                        else:
                            dev_pool[dst].copy_(cpu_pool[src], non_blocking=True)
        if self.copy_stream is not None:
            cur.wait_stream(self.copy_stream)

    def generate_position_ids(self, input_ids, q_seq_lens, valid_lengths):
        return np.concatenate([np.arange(v - q, v) for v, q in zip(valid_lengths, q_seq_lens)]).astype(np.int64)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False

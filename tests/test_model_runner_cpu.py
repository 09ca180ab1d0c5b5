"""ModelRunner: engine-driven prefill/decode with external block tables equals ``generate``; KV swap round-trips."""
import numpy as np
import torch

from mindformers_b200.model_runner import InputBuilder, ModelRunner
from mindformers_b200.models import ByteTokenizer, LlamaConfig, LlamaForCausalLM


def _tiny():
    cfg = LlamaConfig(vocab_size=260, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=64, seq_length=64, params_dtype="float32",
                      compute_dtype="float32", block_size=4)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg, device="cpu")


def test_engine_loop_matches_generate_and_swap_roundtrip():
    model = _tiny()
    prompts = [[5, 9, 33, 7, 100], [12, 250, 3]]
    want = model.generate(prompts, max_new_tokens=4, do_sample=False)
    runner = ModelRunner("", npu_mem_size=0.001, cpu_mem_size=0.001, block_size=4, model=model, tokenizer=ByteTokenizer())
    bs = 4
    # the "engine": a trivial allocator that gives sequence i the blocks [4i, 4i+4)
    tables = np.array([[0, 1, 2, 3], [4, 5, 6, 7]], dtype=np.int32)
    slot = lambda seq, pos: tables[seq][pos // bs] * bs + pos % bs
    seqs = [list(p) for p in prompts]
    flat = [t for p in prompts for t in p]
    slots = [slot(i, j) for i, p in enumerate(prompts) for j in range(len(p))]
    logits = runner.forward(np.array(flat), [len(p) for p in prompts], tables, np.array(slots), prefill=True)
    for step in range(4):
        nxt = logits.argmax(-1).tolist()
        for s, t in zip(seqs, nxt):
            s.append(t)
        if step == 3:
            break
        if step == 1:   # swap sequence 1 out to the host pool and back into different device blocks
            runner.swap([[4, 0], [5, 1]], True)
            runner.cache.key_cache[0][4:6].zero_()
            runner.swap([[0, 8], [1, 9]], False)
            tables[1, 0], tables[1, 1] = 8, 9
        lens = [len(s) for s in seqs]
        slots = [slot(i, lens[i] - 1) for i in range(2)]
        logits = runner.forward(np.array(nxt), lens, tables, np.array(slots), prefill=False)
    assert seqs == want
    ids = InputBuilder(ByteTokenizer()).make_context(0, [{"role": "user", "content": "hi"}])
    assert isinstance(ids, list) and len(ids) > 4

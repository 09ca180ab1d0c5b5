import torch

from mindformers_b200.generation import GenerationConfig, TopKLogitsWarper, TopPLogitsWarper, RepetitionPenaltyLogitsProcessor
from mindformers_b200.models import AutoModel, ByteTokenizer, LlamaConfig, LlamaForCausalLM, Qwen3MoeConfig


def _tiny(**kw):
    cfg = LlamaConfig(vocab_size=260, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=64, seq_length=64, params_dtype="float32",
                      compute_dtype="float32", block_size=4, **kw)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg, device="cpu")


def _reference_greedy(model, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        x = torch.tensor([ids])
        logits = model.model(x)          # full recompute, no cache
        ids.append(int(logits[-1].argmax()))
    return ids


def test_paged_greedy_generation_matches_full_recompute():
    model = _tiny()
    prompts = [[5, 9, 33, 7, 100, 2, 8], [12, 250, 3]]
    out = model.generate(prompts, max_new_tokens=6, do_sample=False)
    for p, o in zip(prompts, out):
        assert o == _reference_greedy(model, p, 6)
    # chunked prefill gives the same continuation
    out2 = model.generate(prompts, max_new_tokens=6, do_sample=False, chunk_prefill_size=3)
    assert out2 == out
    # ... also when the shorter prompt comes first (it has no tokens in the later chunks)
    rev = model.generate(prompts[::-1], max_new_tokens=6, do_sample=False, chunk_prefill_size=3)
    assert rev == out[::-1]


def test_sampling_is_seeded_and_eos_stops():
    model = _tiny()
    a = model.generate([[1, 2, 3]], max_new_tokens=8, do_sample=True, top_k=20, top_p=0.9, temperature=0.8, seed=3)
    b = model.generate([[1, 2, 3]], max_new_tokens=8, do_sample=True, top_k=20, top_p=0.9, temperature=0.8, seed=3)
    assert a == b and len(a[0]) == 11
    first = model.generate([[1, 2, 3]], max_new_tokens=1)[0][-1]
    stopped = model.generate([[1, 2, 3]], max_new_tokens=8, eos_token_id=first)
    assert len(stopped[0]) == 4


def test_beam_search_beats_or_matches_greedy_logprob():
    model = _tiny()
    prompt = [4, 8, 15, 16]

    def logprob(seq):
        lp = 0.0
        for i in range(len(prompt), len(seq)):
            logits = model.model(torch.tensor([seq[:i]]))[-1]
            lp += torch.log_softmax(logits, -1)[seq[i]].item()
        return lp
    greedy = model.generate([prompt], max_new_tokens=4)[0]
    beam = model.generate([prompt], max_new_tokens=4, num_beams=3, length_penalty=0.0)[0]
    assert logprob(beam) >= logprob(greedy) - 1e-4


def test_moe_model_generates_and_processors_work():
    cfg = Qwen3MoeConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                         max_position_embeddings=32, seq_length=32, params_dtype="float32", compute_dtype="float32")
    model = AutoModel.from_config(cfg, device="cpu")
    out = model.generate([[3, 4, 5]], max_new_tokens=3)
    assert len(out[0]) == 6
    scores = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    assert (TopKLogitsWarper(2)(None, scores) == float("-inf")).sum() == 2
    assert (TopPLogitsWarper(0.5)(None, scores) > float("-inf")).sum() == 1
    pen = RepetitionPenaltyLogitsProcessor(2.0)(torch.tensor([[3, -1]]), scores.clone())
    assert pen[0, 3] == 2.0 and pen[0, 2] == 3.0


def test_save_and_load_pretrained_roundtrip(tmp_path):
    model = _tiny()
    model.save_pretrained(str(tmp_path / "m"))
    again = AutoModel.from_pretrained(str(tmp_path / "m"), device="cpu")
    for (n, a), (_, b) in zip(model.named_parameters(), again.named_parameters()):
        assert torch.equal(a, b), n
    model.save_pretrained(str(tmp_path / "hf"), hf_names=True)
    hf = AutoModel.from_pretrained(str(tmp_path / "hf"), device="cpu")
    assert torch.equal(hf.model.decoder.layers[0].self_attention.linear_qkv.weight,
                       model.model.decoder.layers[0].self_attention.linear_qkv.weight)
    tok = ByteTokenizer()
    assert tok.decode(tok.encode("héllo")) == "héllo"


def test_parallel_decoding_matches_greedy():
    model = _tiny()
    prompt = [7, 8, 9, 7, 8, 9, 7, 8, 9, 7, 8]            # repetitive: n-gram drafts get accepted
    want = model.generate([prompt, [3, 4, 5]], max_new_tokens=12, do_sample=False)
    for plugin in ("la", "memory_decoding"):
        got = model.generate([prompt, [3, 4, 5]], max_new_tokens=12, do_sample=False, parallel_decoding=plugin)
        assert got == want, plugin
        assert model.last_generation_stats["model_calls"] <= 13
    shared = [11, 12, 13, 14, 15, 16, 17, 18, 19]
    a, b = shared + [40, 41], shared + [50]
    want = model.generate([a, b], max_new_tokens=5, do_sample=False)
    got = model.generate([a, b], max_new_tokens=5, do_sample=False, parallel_decoding="prefix_cache")
    assert got == want and model.last_generation_stats["shared_prefix_tokens"] == 8


def test_detailed_latency_and_token_window_profiling(monkeypatch):
    """Phase timers of generate() and the profiler window opened / closed at token indices."""
    from mindformers_b200.generation import text_generator
    from mindformers_b200.tools.debug_info import DetailedLatency, Profiling
    model = _tiny()
    model.detailed_latency = DetailedLatency(enabled=True)
    events = []

    class FakeProf:
        def __enter__(self):
            events.append("start")

        def __exit__(self, *a):
            events.append("stop")

    monkeypatch.setattr(text_generator, "Profiling", lambda: Profiling(start=2, stop=3, profiler_factory=FakeProf))
    out = model.generate([[5, 6, 7, 8]], max_new_tokens=6, do_sample=False, eos_token_id=None)
    assert len(out[0]) == 10
    s = model.detailed_latency.summary()
    assert s["prefill"]["predict"]["count"] == 1 and s["decode"]["predict"]["count"] == 5
    assert s["decode"]["preprocess"]["count"] == 5 and s["decode"]["postprocess"]["count"] == 5
    assert s["decode"]["predict"]["mean_ms"] > 0
    assert events == ["start", "stop"]
    p = Profiling(start=1, stop=50, profiler_factory=FakeProf)       # generation ends inside the window
    p.step_begin(1)
    p.close()
    assert p.windows == 1 and not Profiling().enabled


def test_deepseek_v2_and_qwen2_moe_families_build_and_generate():
    """DeepSeek-V2 (MLA without a query low-rank projection, softmax router) and Qwen2-MoE (gated shared expert)."""
    from mindformers_b200.models import DeepseekV2ForCausalLM, Qwen2MoeForCausalLM
    v2 = AutoModel.from_config(dict(
        model_type="deepseek_v2", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=4,
        intermediate_size=128, moe_intermediate_size=32, n_routed_experts=4, n_shared_experts=1, num_experts_per_tok=2,
        n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=None, kv_lora_rank=32, qk_nope_head_dim=16,
        qk_rope_head_dim=8, v_head_dim=16, vocab_size=128, max_position_embeddings=64, params_dtype="float32"), device="cpu")
    assert isinstance(v2, DeepseekV2ForCausalLM)
    names = dict(v2.named_parameters())
    assert "decoder.layers.0.self_attention.linear_q.weight" in names            # plain query projection
    assert "decoder.layers.1.mlp.shared_experts.linear_fc1.weight" in names
    assert len(v2.generate([[3, 4, 5]], max_new_tokens=3, do_sample=False, eos_token_id=None)[0]) == 6
    q2 = AutoModel.from_config(dict(
        model_type="qwen2_moe", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
        intermediate_size=128, moe_intermediate_size=32, shared_expert_intermediate_size=96, num_experts=4,
        num_experts_per_tok=2, vocab_size=128, max_position_embeddings=64, params_dtype="float32"), device="cpu")
    assert isinstance(q2, Qwen2MoeForCausalLM)
    names = dict(q2.named_parameters())
    assert names["decoder.layers.0.mlp.shared_experts.gate_weight"].shape == (1, 64)
    assert names["decoder.layers.0.mlp.shared_experts.linear_fc2.weight"].shape[1] == 96
    assert len(q2.generate([[3, 4, 5]], max_new_tokens=2, do_sample=False, eos_token_id=None)[0]) == 5


def test_mtp_speculative_decoding_equals_greedy_and_accepts_drafts():
    """The multi-token-prediction layer drafts one token per step; output is the greedy sequence whether drafts are
    accepted (after a short training on a periodic pattern they are) or rejected (random weights)."""
    cfg = dict(model_type="deepseek_v3", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=4,
               intermediate_size=128, moe_intermediate_size=32, n_routed_experts=4, n_shared_experts=1,
               num_experts_per_tok=2, n_group=2, topk_group=1, routed_scaling_factor=1.0, norm_topk_prob=True,
               scoring_func="sigmoid", first_k_dense_replace=1, vocab_size=96, q_lora_rank=32, kv_lora_rank=32,
               qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, max_position_embeddings=128,
               params_dtype="float32", num_nextn_predict_layers=1, block_size=4)
    torch.manual_seed(0)
    model = AutoModel.from_config(cfg, device="cpu")
    prompts = [[3, 4, 5, 6, 7], [9, 8, 7]]
    kw = dict(max_new_tokens=9, do_sample=False, eos_token_id=None)
    model.eval()
    assert model.generate(prompts, **kw) == model.generate(prompts, parallel_decoding="mtp", **kw)
    assert model.last_generation_stats["proposed_draft_tokens"] > 0
    # teach main model and MTP layer the pattern 10 20 30 10 20 30 ...
    pattern = torch.tensor([10, 20, 30] * 11)[:32].unsqueeze(0).repeat(4, 1)
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)
    model.train()
    for _ in range(60):
        loss = model(pattern[:, :-1].contiguous(), labels=pattern[:, 1:].contiguous())
        opt.zero_grad()
        loss.backward()
        opt.step()
    model.eval()
    prompts = [[10, 20, 30, 10, 20], [20, 30, 10]]
    ref = model.generate(prompts, **kw)
    assert ref[0][5:8] == [30, 10, 20]                                  # the pattern was learnt
    out = model.generate(prompts, parallel_decoding="mtp", **kw)
    stats = model.last_generation_stats
    assert out == ref
    assert stats["accepted_draft_tokens"] >= 4 and stats["model_calls"] < 1 + 9      # fewer calls than tokens


def test_generate_runs_with_gradients_off():
    """``generate`` must run the model under ``no_grad`` (the kernels' autograd wrappers, the per-layer buffers of the
    expert exchange and the CUDA-graph capture all depend on it)."""
    from mindformers_b200.models import AutoModel
    torch.manual_seed(0)
    model = AutoModel.from_config(dict(model_type="llama", num_hidden_layers=1, hidden_size=64, num_attention_heads=4,
                                       num_key_value_heads=2, intermediate_size=128, vocab_size=128,
                                       max_position_embeddings=64, params_dtype="float32", compute_dtype="float32"),
                                  device="cpu").eval()
    seen = []
    inner = model.model if hasattr(model, "model") else model
    hook = inner.register_forward_pre_hook(lambda m, a: seen.append(torch.is_grad_enabled()))
    try:
        model.generate([[1, 2, 3, 4]], max_new_tokens=3, do_sample=False, eos_token_id=None)
    finally:
        hook.remove()
    assert seen and not any(seen)


def test_int8_kv_cache_stores_codes_and_scales_and_tracks_the_bf16_cache():
    """``kv_cache_dtype="int8"``: the paged cache holds int8 codes plus one scale per token and KV head; decode and
    chunked prefill read it back. Logits stay within the quantisation error of the exact cache and a ``ptq``
    quantisation config with ``kvcache_dtype: int8`` switches it on."""
    from mindformers_b200.inference.paged_attention import KVCacheContext
    model = _tiny()
    prompts = [[5, 9, 33, 7, 100, 2, 8], [12, 250, 3]]

    def prefill_then_one_decode_step():
        ctx, tables = model._set_kv_cache(2, 16)
        tables.init_cache_engine(2)
        first = model._forward_step(prompts, [0, 0], ctx, tables, True)
        nxt = [[int(r.argmax())] for r in first]
        second = model._forward_step(nxt, [len(p) for p in prompts], ctx, tables, False)
        tables.clear_cache()
        return ctx, first.float(), second.float()

    _, e1, e2 = prefill_then_one_decode_step()
    model.config.kv_cache_dtype = "int8"
    ctx, q1, q2 = prefill_then_one_decode_step()
    assert isinstance(ctx, KVCacheContext) and ctx.int8 and ctx.key_cache[0].dtype == torch.int8
    assert ctx.key_scale[0].shape == ctx.key_cache[0].shape[:3] and int(ctx.key_cache[0].abs().max()) == 127
    assert torch.equal(e1, q1)                    # prefill attends to the new tokens themselves, not to the cache
    worst, spread = (e2 - q2).abs().max().item(), e2.abs().max().item()
    assert 0 < worst < 0.05 * spread, (worst, spread)          # decode reads the quantised cache: close, not equal
    chunked = model.generate(prompts, max_new_tokens=5, do_sample=False, chunk_prefill_size=3)
    assert [len(x) for x in chunked] == [len(p) + 5 for p in prompts]
    # the quantiser's kvcache_dtype reaches the cache
    model2 = _tiny()
    model2.apply_quantization_config({"quant_method": "ptq", "kvcache_dtype": "int8"})
    assert model2.config.kv_cache_dtype == "int8"
    out = model2.generate(prompts, max_new_tokens=3, do_sample=False)
    assert [len(x) for x in out] == [len(p) + 3 for p in prompts]


def test_device_loop_matches_the_host_loop_and_reuses_its_capture():
    """Token selection and state update as the last operation of the decode step (eager replays on CPU): same tokens
    as the per-token host loop for prompts of different lengths, with an end token that stops one sequence early and
    a length limit that falls inside a burst; the second call reuses the first call's cache and captured step."""
    model = _tiny()
    prompts = [[5, 9, 33, 7, 100, 2, 8], [12, 250, 3], [7]]
    host = model.generate(prompts, max_new_tokens=11, do_sample=False)
    loop = model.generate(prompts, max_new_tokens=11, do_sample=False, use_cuda_graph=True, device_loop_steps=4)
    assert loop == host
    eos = host[1][len(prompts[1]) + 5]                      # sixth generated token of the second sequence
    host_e = model.generate(prompts, max_new_tokens=11, do_sample=False, eos_token_id=eos)
    loop_e = model.generate(prompts, max_new_tokens=11, do_sample=False, eos_token_id=eos, use_cuda_graph=True,
                            device_loop_steps=4)
    assert loop_e == host_e and len(loop_e[1]) <= len(prompts[1]) + 6
    entries = list(model._device_loops.values())
    assert len(entries) == 1 and entries[0]["captures"] == 1
    # a single new token never enters the loop; a burst longer than the generation is cut by the limit
    assert model.generate(prompts, max_new_tokens=1, use_cuda_graph=True) == model.generate(prompts, max_new_tokens=1)
    assert model.generate(prompts, max_new_tokens=3, use_cuda_graph=True, device_loop_steps=16) == \
        model.generate(prompts, max_new_tokens=3)
    model.release_device_loops()
    assert not getattr(model, "_device_loops", None)


def test_device_loop_sampling_is_seeded_and_follows_the_distribution():
    from mindformers_b200.generation.device_loop import DecodeState, decode_advance
    model = _tiny()
    kw = dict(max_new_tokens=9, do_sample=True, top_k=0, top_p=1.0, temperature=0.7, use_cuda_graph=True,
              device_loop_steps=4)
    a = model.generate([[1, 2, 3], [9, 8]], seed=5, **kw)
    b = model.generate([[1, 2, 3], [9, 8]], seed=5, **kw)
    c = model.generate([[1, 2, 3], [9, 8]], seed=6, **kw)
    assert a == b and a != c and [len(x) for x in a] == [12, 11]
    # Gumbel-max draws follow softmax(logits / T)
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).repeat(1, 1)
    counts = torch.zeros(4)
    for s in range(600):
        st = DecodeState.allocate(1, 8, 4, 4, "cpu")
        st.table.copy_(torch.arange(8, dtype=torch.int32)[None])
        st.limit.fill_(30)
        st.set_sampling((), 0.5, seed=s)
        decode_advance(logits, st)
        counts[int(st.hist[0, 0])] += 1
    want = torch.softmax(logits[0] / 0.5, -1)
    assert (counts / 600 - want).abs().max() < 0.06
    # state after one greedy step: token, position, length and slot move together; the end token freezes the sequence
    st = DecodeState.allocate(2, 8, 4, 4, "cpu")
    st.table.copy_(torch.tensor([[3, 5, 7, 9, 11, 13, 15, 17], [2, 4, 6, 8, 10, 12, 14, 16]], dtype=torch.int32))
    st.load([10, 11], [6, 2], st.table.numpy(), [0, 0], [False, False], [30, 30])
    st.set_sampling([1], 0.0, 0)
    decode_advance(torch.tensor([[0.0, 0.0, 3.0, 0.0], [0.0, 9.0, 0.0, 0.0]]), st)
    assert st.tok.tolist() == [[2, 11]] and st.pos.tolist() == [7, 2] and st.lens.tolist() == [8, 3]
    assert st.slots.tolist() == [5 * 4 + 3, -1] and st.finished.tolist() == [0, 1] and st.hist[:, 0].tolist() == [2, 1]
    decode_advance(torch.tensor([[0.0, 0.0, 3.0, 0.0], [0.0, 9.0, 0.0, 0.0]]), st)
    assert st.hist[:, 1].tolist() == [2, -1] and st.pos.tolist() == [8, 2] and st.slots[0].item() == 7 * 4 + 0

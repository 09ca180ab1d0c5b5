"""Continuous-batching engine and its HTTP front end on a tiny CPU model."""
import json
import threading

import pytest
import torch

from mindformers_b200.models import ByteTokenizer, LlamaConfig, LlamaForCausalLM
from mindformers_b200.serving import SamplingParams, ServingEngine


def _tiny():
    cfg = LlamaConfig(vocab_size=260, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=64, seq_length=64, params_dtype="float32",
                      compute_dtype="float32", block_size=4)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg, device="cpu")


PROMPTS = [[5, 9, 33, 7, 100, 2, 8], [12, 250, 3], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11], [77], [200, 201, 202, 203]]


def test_requests_join_and_leave_the_batch_and_match_offline_generation():
    """Five requests with different lengths and budgets through three slots: every request's tokens equal those of an
    offline greedy ``generate`` of the same prompt; slots and cache blocks are all free at the end."""
    model = _tiny()
    budgets = [6, 9, 4, 12, 5]
    want = [model.generate([p], max_new_tokens=n, do_sample=False)[0][len(p):] for p, n in zip(PROMPTS, budgets)]
    engine = ServingEngine(model, max_num_seqs=3, max_model_len=48, max_prefill_tokens=8, eos_token_id=None)
    seen = {}
    reqs = [engine.add_request(f"r{i}", p, SamplingParams(max_tokens=n, temperature=0.0),
                               on_token=lambda r, t: seen.setdefault(r.request_id, []).append(t))
            for i, (p, n) in enumerate(zip(PROMPTS, budgets))]
    joined_late = False
    while engine.has_work():
        engine.step()
        running = sum(r is not None for r in engine.running)
        assert running <= 3
        joined_late |= bool(engine.waiting) and running == 3
    assert joined_late                                     # the queue really was longer than the batch
    for r, w in zip(reqs, want):
        assert r.finished and r.finish_reason == "length" and r.output == w, (r.request_id, r.output, w)
        assert seen[r.request_id] == w + [-1]              # streamed token by token, then the end marker
    st = engine.stats()
    assert st["running"] == 0 and st["free_blocks"] == st["total_blocks"] and st["finished"] == 5
    assert st["decode_tokens"] + 5 == sum(budgets) and st["ttft_s_p50"] > 0


def test_preemption_when_the_block_pool_runs_dry_and_abort():
    """A pool too small for all running requests to grow: the newest one is preempted, re-enters, recomputes its cache
    and still produces the offline result. An aborted request frees its blocks."""
    model = _tiny()
    p = [PROMPTS[0], PROMPTS[2], PROMPTS[4]]
    want = [model.generate([x], max_new_tokens=14, do_sample=False)[0][len(x):] for x in p]
    engine = ServingEngine(model, max_num_seqs=3, max_model_len=40, num_blocks=14, eos_token_id=None)   # 56 token slots
    assert engine.tables.pool.num_blocks == 14
    reqs = [engine.add_request(f"p{i}", x, SamplingParams(max_tokens=14, temperature=0.0)) for i, x in enumerate(p)]
    engine.run_until_idle()
    assert engine.counters["preempted"] >= 1
    for r, w in zip(reqs, want):
        assert r.output == w, (r.request_id, r.preemptions)
    assert engine.tables.pool.num_free == 14
    a = engine.add_request("gone", PROMPTS[0], SamplingParams(max_tokens=30, temperature=0.0))
    engine.step()
    engine.step()
    engine.abort("gone")
    engine.run_until_idle()
    assert a.finished and a.finish_reason == "abort" and 1 <= len(a.output) < 30
    assert engine.tables.pool.num_free == 14
    with pytest.raises(ValueError):
        engine.add_request("big", list(range(60)), SamplingParams())


def test_seeded_sampling_stop_tokens_and_eos():
    model = _tiny()
    engine = ServingEngine(model, max_num_seqs=2, max_model_len=48, eos_token_id=None)
    sp = SamplingParams(max_tokens=10, temperature=0.9, top_k=30, top_p=0.95, seed=7, repetition_penalty=1.1)
    a = engine.generate([PROMPTS[0]], sp)[0]
    b = engine.generate([PROMPTS[0]], sp)[0]
    c = engine.generate([PROMPTS[0]], SamplingParams(max_tokens=10, temperature=0.9, top_k=30, top_p=0.95, seed=8))[0]
    assert a.token_ids == b.token_ids and len(a.token_ids) == 10 and a.token_ids != c.token_ids
    greedy = engine.generate([PROMPTS[1]], SamplingParams(max_tokens=8, temperature=0.0))[0].token_ids
    stop_at = greedy[3]
    cut = engine.generate([PROMPTS[1]], SamplingParams(max_tokens=8, temperature=0.0, stop_token_ids=[stop_at]))[0]
    assert cut.finish_reason == "stop" and cut.token_ids == greedy[:greedy.index(stop_at) + 1]
    eos_engine = ServingEngine(model, max_num_seqs=2, max_model_len=48, eos_token_id=greedy[1])
    out = eos_engine.generate([PROMPTS[1]], SamplingParams(max_tokens=8, temperature=0.0))[0]
    assert out.finish_reason == "stop" and out.token_ids == greedy[:2]


def test_openai_style_http_endpoints_blocking_and_streaming():
    from fastapi.testclient import TestClient
    from mindformers_b200.serving.api_server import build_app
    model = _tiny()
    tok = ByteTokenizer()
    engine = ServingEngine(model, max_num_seqs=4, max_model_len=48, eos_token_id=None)
    app = build_app(engine, tok, "tiny")
    try:
        with TestClient(app) as client:
            assert client.get("/health").json()["status"] == "ok"
            assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
            prompt_ids = list(tok.encode("hello"))
            want = model.generate([prompt_ids], max_new_tokens=6, do_sample=False)[0][len(prompt_ids):]
            r = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 6, "temperature": 0})
            body = r.json()
            assert r.status_code == 200 and body["usage"]["completion_tokens"] == 6
            assert body["choices"][0]["text"] == tok.decode(want) and body["choices"][0]["finish_reason"] == "length"
            # several clients at once share the batch
            results = {}

            def ask(i):
                rr = client.post("/v1/completions", json={"prompt": prompt_ids, "max_tokens": 6, "temperature": 0})
                results[i] = rr.json()["choices"][0]["text"]
            threads = [threading.Thread(target=ask, args=(i,)) for i in range(5)]
            [t.start() for t in threads]
            [t.join() for t in threads]
            assert set(results.values()) == {tok.decode(want)}
            with client.stream("POST", "/v1/chat/completions",
                               json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "temperature": 0,
                                     "stream": True}) as s:
                lines = [ln for ln in s.iter_lines() if ln.startswith("data: ")]
            assert lines[-1] == "data: [DONE]"
            chunks = [json.loads(ln[6:]) for ln in lines[:-1]]
            assert chunks[-1]["choices"][0]["finish_reason"] == "length" and len(chunks) == 6
            assert all(c["object"] == "chat.completion.chunk" for c in chunks)
            assert client.post("/v1/completions", json={"max_tokens": 3}).status_code == 400
            m = client.get("/metrics").text
            assert "mfb_serving_finished" in m and "mfb_serving_ttft_s_p50" in m
    finally:
        engine.shutdown()


def test_decode_bursts_on_the_device_give_the_host_loop_tokens():
    """With every running request greedy, decode runs as bursts of captured steps (eager replays on CPU) with the token
    selection on the device: same tokens, same finish reasons, same streamed callbacks as with one host step per token,
    for requests that finish inside a burst (length and stop token), join between bursts and differ in prompt length;
    a request with a penalty or its own stop token sends the batch back to the host loop."""
    model = _tiny()
    budgets = [6, 9, 4, 12, 5]
    free = model.generate([PROMPTS[1]], max_new_tokens=9, do_sample=False)[0][len(PROMPTS[1]):]
    stop_tok = free[4]

    def run(burst, extra=None):
        eng = ServingEngine(model, max_num_seqs=3, max_model_len=48, max_prefill_tokens=8, eos_token_id=stop_tok,
                            decode_burst=burst)
        seen = {}
        reqs = []
        for i, (p, n) in enumerate(zip(PROMPTS, budgets)):
            sp = SamplingParams(max_tokens=n, temperature=0.0)
            if extra and i in extra:
                sp = SamplingParams(max_tokens=n, temperature=0.0, **extra[i])
            reqs.append(eng.add_request(f"r{i}", p, sp, on_token=lambda r, t: seen.setdefault(r.request_id, []).append(t)))
        eng.run_until_idle()
        st = eng.stats()
        assert st["running"] == 0 and st["free_blocks"] == st["total_blocks"]
        return [(r.output, r.finish_reason) for r in reqs], seen, eng.counters

    host, host_seen, c0 = run(0)
    dev, dev_seen, c1 = run(5)
    assert c0["bursts"] == 0 and c1["bursts"] >= 2
    assert dev == host and dev_seen == host_seen
    assert any(reason == "stop" for _, reason in host) and any(reason == "length" for _, reason in host)
    assert c1["decode_tokens"] == c0["decode_tokens"] and c1["steps"] < c0["steps"]
    # ineligible companions: a repetition penalty, a private stop token
    mixed_host, _, _ = run(0, {0: dict(repetition_penalty=1.3), 3: dict(stop_token_ids=[free[2]])})
    mixed_dev, _, c2 = run(5, {0: dict(repetition_penalty=1.3), 3: dict(stop_token_ids=[free[2]])})
    assert mixed_dev == mixed_host

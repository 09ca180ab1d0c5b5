"""OpenAI-style HTTP front end of the serving engine (FastAPI).

Endpoints: ``POST /v1/completions``, ``POST /v1/chat/completions`` (both with ``stream: true`` as server-sent
events), ``GET /v1/models``, ``GET /health``, ``GET /metrics`` (Prometheus text: counters of the engine and latency
quantiles). The reference starts an external service for this (``scripts/run_mindie.sh``); here the service is part of
the package:

    python -m mindformers_b200.serving.api_server --model_dir <pretrained dir> --port 8000

``build_app(engine, tokenizer, model_name)`` returns the application for embedding and for tests.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import time
import uuid
from typing import List, Optional, Union

from .engine import SamplingParams, ServingEngine


def _params(body: dict, default_max: int = 64) -> SamplingParams:
    temp = body.get("temperature")
    return SamplingParams(
        max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or default_max),
        temperature=1.0 if temp is None else float(temp),
        top_k=int(body.get("top_k") or 0), top_p=float(body.get("top_p") or 1.0),
        repetition_penalty=float(body.get("repetition_penalty") or 1.0),
        frequency_penalty=float(body.get("frequency_penalty") or 0.0),
        presence_penalty=float(body.get("presence_penalty") or 0.0),
        seed=body.get("seed"), stop_token_ids=list(body.get("stop_token_ids") or []),
        ignore_eos=bool(body.get("ignore_eos", False)))


def _chat_prompt(tokenizer, messages: List[dict]) -> List[int]:
    if hasattr(tokenizer, "apply_chat_template"):
        try:
            ids = tokenizer.apply_chat_template(messages, add_generation_prompt=True, tokenize=True)
            return list(ids["input_ids"] if isinstance(ids, dict) else ids)
        except Exception:   # noqa: BLE001  (a tokenizer without a template: fall back to a plain transcript)
            pass
    text = "".join(f"{m.get('role', 'user')}: {m.get('content', '')}\n" for m in messages) + "assistant: "
    return list(tokenizer.encode(text))


def build_app(engine: ServingEngine, tokenizer, model_name: str = "mindformers-b200"):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    app = FastAPI(title="mindformers_b200 serving")
    engine.start()

    def encode(prompt: Union[str, List[int]]) -> List[int]:
        if isinstance(prompt, str):
            return list(tokenizer.encode(prompt))
        return [int(t) for t in prompt]

    def decode(ids: List[int]) -> str:
        return tokenizer.decode(ids) if ids else ""

    async def run(prompt_ids: List[int], params: SamplingParams, stream: bool, chat: bool, created: int, rid: str):
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()

        def on_token(req, tok):            # called from the engine thread
            loop.call_soon_threadsafe(q.put_nowait, tok)
        try:
            req = engine.add_request(rid, prompt_ids, params, on_token)
        except ValueError as exc:
            raise HTTPException(status_code=400, detail=str(exc))
        obj = "chat.completion" if chat else "text_completion"

        def choice(text: str, finish: Optional[str], delta: bool):
            if chat:
                key = "delta" if delta else "message"
                return {"index": 0, key: {"role": "assistant", "content": text}, "finish_reason": finish}
            return {"index": 0, "text": text, "finish_reason": finish}

        if stream:
            async def events():
                sent = ""
                try:
                    while True:
                        tok = await q.get()
                        if tok < 0:
                            break
                        text = decode(req.output)
                        piece, sent = text[len(sent):], text
                        chunk = {"id": rid, "object": obj + ".chunk", "created": created, "model": model_name,
                                 "choices": [choice(piece, None, True)]}
                        yield f"data: {json.dumps(chunk)}\n\n"
                    last = {"id": rid, "object": obj + ".chunk", "created": created, "model": model_name,
                            "choices": [choice("", req.finish_reason, True)]}
                    yield f"data: {json.dumps(last)}\n\ndata: [DONE]\n\n"
                finally:
                    if not req.finished:
                        engine.abort(rid)        # the client went away
            return StreamingResponse(events(), media_type="text/event-stream")
        while True:
            tok = await q.get()
            if tok < 0:
                break
        out = req.result()
        return JSONResponse({
            "id": rid, "object": obj, "created": created, "model": model_name,
            "choices": [choice(decode(out.token_ids), out.finish_reason, False)],
            "usage": {"prompt_tokens": len(out.prompt_token_ids), "completion_tokens": len(out.token_ids),
                      "total_tokens": len(out.prompt_token_ids) + len(out.token_ids)},
            "metrics": out.metrics})

    @app.post("/v1/completions")
    async def completions(body: dict):
        if "prompt" not in body:
            raise HTTPException(status_code=400, detail="prompt is required")
        prompt = body["prompt"]
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], (str, list)):
            if len(prompt) != 1:
                raise HTTPException(status_code=400, detail="one prompt per request")
            prompt = prompt[0]
        return await run(encode(prompt), _params(body), bool(body.get("stream")), False, int(time.time()),
                         "cmpl-" + uuid.uuid4().hex)

    @app.post("/v1/chat/completions")
    async def chat(body: dict):
        messages = body.get("messages")
        if not messages:
            raise HTTPException(status_code=400, detail="messages is required")
        return await run(_chat_prompt(tokenizer, messages), _params(body, 256), bool(body.get("stream")), True,
                         int(time.time()), "chatcmpl-" + uuid.uuid4().hex)

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "mindformers_b200",
                                            "max_model_len": engine.max_model_len}]}

    @app.get("/health")
    async def health():
        return {"status": "ok", **{k: engine.stats()[k] for k in ("running", "waiting", "free_blocks")}}

    @app.get("/metrics")
    async def metrics():
        lines = []
        for k, v in sorted(engine.stats().items()):
            name = "mfb_serving_" + k
            lines.append(f"# TYPE {name} {'counter' if k in engine.counters else 'gauge'}")
            lines.append(f"{name} {v}")
        return PlainTextResponse("\n".join(lines) + "\n")

    return app


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_dir", required=True)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max_num_seqs", type=int, default=32)
    ap.add_argument("--max_model_len", type=int, default=None)
    ap.add_argument("--num_blocks", type=int, default=None)
    ap.add_argument("--max_prefill_tokens", type=int, default=8192)
    ap.add_argument("--model_name", default=None)
    a = ap.parse_args(argv)
    import uvicorn

    from ..models import AutoModelForCausalLM, AutoTokenizer
    model = AutoModelForCausalLM.from_pretrained(a.model_dir)
    tokenizer = AutoTokenizer.from_pretrained(a.model_dir)
    engine = ServingEngine(model, a.max_num_seqs, a.max_model_len, a.num_blocks, a.max_prefill_tokens,
                           eos_token_id=getattr(tokenizer, "eos_token_id", None))
    app = build_app(engine, tokenizer, a.model_name or a.model_dir.rstrip("/").split("/")[-1])
    uvicorn.run(app, host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()

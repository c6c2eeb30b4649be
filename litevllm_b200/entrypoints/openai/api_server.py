"""OpenAI-compatible HTTP server.

Routes: ``GET /v1/models``, ``POST /v1/chat/completions`` (JSON or SSE streaming), ``GET /healthz``,
``GET /readyz``, ``GET|POST /debug/runtime_stats[/reset]`` (only with ``--enable-debug-endpoints``),
plus ``/tokenize`` and ``/detokenize``.  Admission happens before the first byte of a streaming
response, so rejections become proper HTTP errors: 400 invalid request, 413 body too large,
429 queue full / queue timeout, 503 engine not ready or fatal.
Contract: vllm/entrypoints/openai/api_server.py:33-516 of the reference.

Run: ``python -m litevllm_b200.entrypoints.openai.api_server --model <path> [--host H --port P]``.
"""
from __future__ import annotations

import argparse
import json
import time
import uuid
from typing import Any

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, StreamingResponse

from ...engine.errors import (EngineFatalError, InvalidRequestError, LiteRuntimeError,
                              RequestRejectedError)
from ...sampling_params import SamplingParams, StructuredOutputsParams

MAX_REQUEST_BODY_BYTES = 16 * 1024 * 1024

app = FastAPI(title="litevllm_b200 OpenAI-compatible server")
engine = None            # AsyncLLM (or a stand-in with the same surface in tests)
served_model: str = ""
debug_endpoints_enabled = False


def _error(status: int, message: str, kind: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse(status_code=status, content={"error": {"message": message, "type": kind, "code": status}})


class _BodyError(Exception):
    def __init__(self, status: int, message: str):
        self.status, self.message = status, message


async def _read_json_object(request: Request) -> dict:
    """Size-capped streaming read; the body is rejected before any JSON parsing when too large."""
    declared = request.headers.get("content-length")
    if declared is not None:
        try:
            if int(declared) > MAX_REQUEST_BODY_BYTES:
                raise _BodyError(413, "request body too large")
        except ValueError:
            raise _BodyError(400, "invalid content-length") from None
    chunks, total = [], 0
    async for chunk in request.stream():
        total += len(chunk)
        if total > MAX_REQUEST_BODY_BYTES:
            raise _BodyError(413, "request body too large")
        chunks.append(chunk)
    try:
        obj = json.loads(b"".join(chunks) or b"{}")
    except json.JSONDecodeError as e:
        raise _BodyError(400, f"invalid JSON: {e.msg}") from None
    if not isinstance(obj, dict):
        raise _BodyError(400, "request body must be a JSON object")
    return obj


def _normalize_chat_messages(messages: Any) -> tuple[list[dict], dict | None]:
    """Flatten content blocks; ``image_url`` blocks become an ``<image>`` placeholder plus an entry
    in ``multi_modal_data``."""
    if not isinstance(messages, list) or not messages:
        raise InvalidRequestError("messages must be a non-empty list")
    out, images = [], []
    for m in messages:
        if not isinstance(m, dict) or "role" not in m:
            raise InvalidRequestError("every message needs a role")
        content = m.get("content", "")
        if isinstance(content, str):
            text = content
        elif isinstance(content, list):
            parts = []
            for block in content:
                if not isinstance(block, dict):
                    raise InvalidRequestError("content blocks must be objects")
                kind = block.get("type")
                if kind == "text":
                    parts.append(str(block.get("text", "")))
                elif kind == "image_url":
                    url = block.get("image_url")
                    url = url.get("url") if isinstance(url, dict) else url
                    if not isinstance(url, str):
                        raise InvalidRequestError("image_url block without a url")
                    images.append(url)
                    parts.append("<image>")
                else:
                    raise InvalidRequestError(f"unsupported content block type {kind!r}")
            text = "".join(parts)
        else:
            raise InvalidRequestError("message content must be a string or a list of blocks")
        out.append({"role": str(m["role"]), "content": text})
    return out, ({"image": images} if images else None)


def _render_chat_prompt(tokenizer, messages: list[dict]) -> str:
    tmpl = getattr(tokenizer, "apply_chat_template", None)
    if tmpl is not None:
        try:
            return tmpl(messages, tokenize=False, add_generation_prompt=True)
        except Exception:
            pass
    # no usable template on the tokenizer: the registered fallback of the model type, then of the model family
    from ...transformers_utils.chat_templates import get_chat_template_fallback, render_fallback, template_for_family
    name = "plain"
    try:
        mc = engine.engine.vllm_config.model_config
        path = get_chat_template_fallback(str((mc.hf_config or {}).get("model_type", "")), str(mc.tokenizer))
        name = str(path) if path is not None else template_for_family(mc.arch.family)
    except Exception:
        pass
    return render_fallback(messages, name)


def _parse_structured(body: dict) -> StructuredOutputsParams | None:
    so = body.get("structured_outputs")
    if so is not None:
        if not isinstance(so, dict):
            raise InvalidRequestError("structured_outputs must be an object")
        allowed = {"json", "regex", "grammar", "structural_tag", "json_object", "choice"}
        extra = set(so) - allowed
        if extra:
            raise InvalidRequestError(f"unknown structured_outputs keys: {sorted(extra)}")
        return StructuredOutputsParams(**so)
    rf = body.get("response_format")
    if rf is None:
        return None
    if not isinstance(rf, dict) or "type" not in rf:
        raise InvalidRequestError("response_format must be an object with a type")
    kind = rf["type"]
    if kind == "text":
        return None
    if kind == "json_object":
        return StructuredOutputsParams(json_object=True)
    if kind == "json_schema":
        js = rf.get("json_schema") or {}
        schema = js.get("schema") if isinstance(js, dict) else None
        if schema is None:
            raise InvalidRequestError("response_format.json_schema.schema is required")
        return StructuredOutputsParams(json=schema)
    raise InvalidRequestError(f"unsupported response_format type {kind!r}")


def _sampling_params_from_body(body: dict) -> SamplingParams:
    if body.get("n", 1) not in (1, None):
        raise InvalidRequestError("n != 1 is not supported")
    for key in ("stop", "logprobs", "top_logprobs", "seed"):
        if body.get(key) not in (None, [], False):
            raise InvalidRequestError(f"{key} is not supported by this server")
    max_tokens = body.get("max_completion_tokens", body.get("max_tokens", 128))
    try:
        return SamplingParams(
            temperature=float(body.get("temperature", 0.7)), top_p=float(body.get("top_p", 1.0)),
            top_k=int(body.get("top_k", -1)), min_p=float(body.get("min_p", 0.0)),
            frequency_penalty=float(body.get("frequency_penalty", 0.0)),
            presence_penalty=float(body.get("presence_penalty", 0.0)),
            repetition_penalty=float(body.get("repetition_penalty", 1.0)),
            max_tokens=int(max_tokens), structured_outputs=_parse_structured(body))
    except (TypeError, ValueError) as e:
        raise InvalidRequestError(f"invalid sampling parameter: {e}") from None


def _status_for(exc: BaseException) -> int:
    if isinstance(exc, InvalidRequestError):
        return 400
    if isinstance(exc, EngineFatalError):
        return 503
    if isinstance(exc, RequestRejectedError):
        return 429
    return 500


@app.get("/healthz")
async def healthz():
    return {"status": "ok"}


@app.get("/readyz")
async def readyz():
    if engine is None or not engine.is_healthy():
        return _error(503, "engine not ready", "service_unavailable")
    return {"status": "ready"}


@app.get("/v1/models")
async def list_models():
    if engine is None:
        return _error(503, "engine not initialised", "service_unavailable")
    return {"object": "list", "data": [{"id": served_model, "object": "model", "created": int(time.time()),
                                        "owned_by": "litevllm_b200"}]}


@app.get("/debug/runtime_stats")
async def runtime_stats():
    if not debug_endpoints_enabled:
        return _error(404, "not found", "not_found")
    if engine is None:
        return _error(503, "engine not initialised", "service_unavailable")
    return JSONResponse(content=json.loads(json.dumps(engine.stats(), default=str)))


@app.post("/debug/runtime_stats/reset")
async def runtime_stats_reset():
    if not debug_endpoints_enabled:
        return _error(404, "not found", "not_found")
    if engine is None:
        return _error(503, "engine not initialised", "service_unavailable")
    engine.reset_stats()
    return {"status": "reset"}


def _chunk(rid: str, created: int, delta: dict, finish: str | None) -> str:
    payload = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": served_model,
               "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
    return f"data: {json.dumps(payload, ensure_ascii=False)}\n\n"


@app.post("/v1/chat/completions")
async def create_chat_completion(request: Request):
    if engine is None:
        return _error(503, "engine not initialised", "service_unavailable")
    try:
        body = await _read_json_object(request)
    except _BodyError as e:
        return _error(e.status, e.message)
    if body.get("model") != served_model:
        return _error(400, f"model {body.get('model')!r} is not served here (serving {served_model!r})")
    try:
        messages, mm = _normalize_chat_messages(body.get("messages"))
        sp = _sampling_params_from_body(body)
        prompt = _render_chat_prompt(engine.tokenizer, messages)
    except InvalidRequestError as e:
        return _error(400, str(e))
    rid = f"chat-{uuid.uuid4().hex}"
    created = int(time.time())
    # admission first: a rejection must become an HTTP error, not a broken stream
    try:
        await engine.submit(prompt, sp, rid, multi_modal_data=mm)
    except LiteRuntimeError as e:
        return _error(_status_for(e), str(e), "rejected" if _status_for(e) == 429 else "invalid_request_error")

    if body.get("stream"):
        async def generate_stream():
            sent = 0
            try:
                yield _chunk(rid, created, {"role": "assistant"}, None)
                async for out in engine.stream(rid):
                    comp = out.outputs[0]
                    text = comp.text
                    delta, sent = text[sent:], len(text)
                    if delta or out.finished:
                        yield _chunk(rid, created, {"content": delta} if delta else {}, out.finish_reason)
                yield "data: [DONE]\n\n"
            except LiteRuntimeError as e:
                yield f"data: {json.dumps({'error': {'message': str(e), 'code': _status_for(e)}})}\n\n"
            finally:
                await engine.abort(rid)
        return StreamingResponse(generate_stream(), media_type="text/event-stream")

    final = None
    try:
        async for out in engine.stream(rid):
            final = out
    except LiteRuntimeError as e:
        return _error(_status_for(e), str(e))
    finally:
        await engine.abort(rid)
    if final is None:
        return _error(500, "no output produced", "internal_error")
    comp = final.outputs[0]
    n_prompt, n_out = len(final.prompt_token_ids), len(comp.token_ids)
    return {"id": rid, "object": "chat.completion", "created": created, "model": served_model,
            "choices": [{"index": 0, "message": {"role": "assistant", "content": comp.text},
                         "finish_reason": final.finish_reason or "stop"}],
            "usage": {"prompt_tokens": n_prompt, "completion_tokens": n_out, "total_tokens": n_prompt + n_out}}


def _install_tokenize_router() -> None:
    from ..serve.tokenize_router import router
    if not any(getattr(r, "path", None) == "/tokenize" for r in app.routes):
        app.include_router(router)


_install_tokenize_router()


def build_engine(model: str, **kwargs):
    from ...config.config_builder import build_vllm_config
    from ...engine.async_llm import AsyncLLM
    return AsyncLLM(build_vllm_config(model, **kwargs))


def main(argv: list[str] | None = None) -> None:
    global engine, served_model, debug_endpoints_enabled
    ap = argparse.ArgumentParser(description="litevllm_b200 OpenAI-compatible server")
    ap.add_argument("--model", required=True)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--enable-debug-endpoints", action="store_true")
    ap.add_argument("--trust-remote-code", action="store_true")
    ap.add_argument("--revision", default=None)
    ap.add_argument("--policy-mode", default="auto")
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--max-num-seqs", type=int, default=None)
    ap.add_argument("--dtype", default=None)
    ap.add_argument("--tensor-parallel-size", type=int, default=None)
    ap.add_argument("--expert-parallel-size", type=int, default=None)
    ap.add_argument("--data-parallel-size", type=int, default=None,
                    help="whole-engine replicas (one process per GPU under torchrun): rank 0 serves HTTP and routes "
                         "every request to the replica with the fewest requests in flight")
    args = ap.parse_args(argv)
    kw = {k: v for k, v in dict(trust_remote_code=args.trust_remote_code, revision=args.revision,
                                policy_mode=args.policy_mode, max_model_len=args.max_model_len,
                                max_num_seqs=args.max_num_seqs, dtype=args.dtype,
                                tensor_parallel_size=args.tensor_parallel_size,
                                expert_parallel_size=args.expert_parallel_size,
                                data_parallel_size=args.data_parallel_size).items() if v}
    engine = build_engine(args.model, **kw)
    served_model = args.model
    debug_endpoints_enabled = args.enable_debug_endpoints
    if getattr(engine, "is_worker_rank", False):
        # launched with one process per GPU (torchrun): only rank 0 listens; the others mirror its engine
        # (tensor / expert parallel) or serve the requests it routes to them (data parallel)
        engine.serve_as_worker()
        engine.shutdown()
        return
    import uvicorn
    uvicorn.run(app, host=args.host, port=args.port, log_level="info")


if __name__ == "__main__":
    main()

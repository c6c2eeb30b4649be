"""``POST /tokenize`` and ``POST /detokenize`` (reference: vllm/entrypoints/serve/tokenize/
api_router.py:37-68)."""
from __future__ import annotations

from fastapi import APIRouter, Request
from fastapi.responses import JSONResponse

router = APIRouter()


def _tokenizer():
    from ..openai import api_server
    eng = api_server.engine
    return None if eng is None else getattr(eng, "tokenizer", None)


@router.post("/tokenize")
async def tokenize(request: Request):
    tok = _tokenizer()
    if tok is None:
        return JSONResponse(status_code=503, content={"error": {"message": "engine not initialised"}})
    body = await request.json()
    if "messages" in body:
        from ..openai.api_server import _normalize_chat_messages, _render_chat_prompt
        msgs, _ = _normalize_chat_messages(body["messages"])
        text = _render_chat_prompt(tok, msgs)
    else:
        text = body.get("prompt")
    if not isinstance(text, str):
        return JSONResponse(status_code=400, content={"error": {"message": "prompt or messages required"}})
    ids = list(tok.encode(text, add_special_tokens=bool(body.get("add_special_tokens", True))))
    return {"tokens": ids, "count": len(ids), "max_model_len": None}


@router.post("/detokenize")
async def detokenize(request: Request):
    tok = _tokenizer()
    if tok is None:
        return JSONResponse(status_code=503, content={"error": {"message": "engine not initialised"}})
    body = await request.json()
    ids = body.get("tokens")
    if not isinstance(ids, list) or not all(isinstance(t, int) for t in ids):
        return JSONResponse(status_code=400, content={"error": {"message": "tokens must be a list of ints"}})
    return {"prompt": tok.decode(ids)}

"""Import path of the tokenize / detokenize router kept for callers that attach it themselves
(`from ...entrypoints.serve.tokenize import router`); the implementation lives in ``serve/tokenize_router.py``.
Reference: vllm/entrypoints/serve/tokenize/ (router attachment only, not a standalone server)."""
from ..tokenize_router import router

__all__ = ["router"]

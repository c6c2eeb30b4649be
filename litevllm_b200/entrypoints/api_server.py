"""Legacy module path kept for users of ``python -m <pkg>.entrypoints.api_server``; it forwards to
the OpenAI-compatible server (reference: vllm/entrypoints/api_server.py:10-23)."""
from .openai.api_server import app, main  # noqa: F401

if __name__ == "__main__":
    main()

"""Maintained diagnostics, each runnable as ``python -m litevllm_b200.diagnostics.<name>``:

``smoke``        one model, timed generation with first-token and steady-state gates
``layer_drift``  per-layer hidden-state drift between two configurations of one model
``gguf_inspect`` what a GGUF file holds: metadata, tensor formats, expert shapes, bytes per format
``perf_grid``    a grid of engine settings timed in interleaved rounds (two settings: an A/B comparison)
``speculative_ngram``  what prompt-lookup speculation would accept on the model's own greedy output
``quality_spotcheck``  prompts with expected substrings, plus checks for empty and degenerate answers

The reference project keeps the same kinds of tools under tests/tools/ (run_deepseek_v4_flash_gpu_smoke.py,
gemma4_layer_drift_diagnostic.py, deepseek_v4_flash_inspect.py, perf_grid_search.py, interleaved_e2e_ab.py,
gemma4_speculative_prototype.py, quality_bar_spotcheck.py).
"""

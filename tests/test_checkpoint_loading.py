"""Checkpoints on disk: HF-layout safetensors directories (dense, AWQ, compressed-tensors), sharded files whose
quantised parts land in different shards, the `model.language_model.` prefix of multimodal exports, ignored
auxiliary tensors.  The tensors come from the synthetic weight streams, so the loaded model must generate exactly
what the synthetic one does.  Reference behaviour: vllm/model_executor/model_loader/__init__.py:535-812."""
import json

import pytest
import torch

from litevllm_b200 import LLM, SamplingParams
from litevllm_b200.loaders import synthetic_weights
from litevllm_b200.models.presets import PRESETS

SP = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
PROMPTS = [{"prompt_token_ids": [(7 * i + 3 * j) % 400 + 2 for i in range(10 + 3 * j)]} for j in range(3)]


def _tokens(llm):
    return [o.outputs[0].token_ids for o in llm.generate(PROMPTS, SP)]


def _export(preset, directory, shards=1, prefix="", extra=None):
    from safetensors.torch import save_file
    src = LLM(f"synthetic:{preset}", device="cpu", dtype="float32", max_num_seqs=4, max_model_len=128)
    want = _tokens(src)
    tensors = {(prefix + n[len("model."):] if prefix and n.startswith("model.") else n): t.contiguous()
               for n, t in synthetic_weights(src.vllm_config, torch.device("cpu"))}
    if extra:
        tensors.update(extra)
    src.shutdown()
    directory.mkdir()
    (directory / "config.json").write_text(json.dumps(dict(PRESETS[preset], torch_dtype="float32")))
    names = sorted(tensors)
    if shards == 1:
        save_file(tensors, str(directory / "model.safetensors"))
    else:
        # round-robin: the qweight / scales / qzeros of one layer end up in different files
        index = {}
        for k in range(shards):
            part = {n: tensors[n] for n in names[k::shards]}
            fname = f"model-{k + 1:05d}-of-{shards:05d}.safetensors"
            save_file(part, str(directory / fname))
            index.update({n: fname for n in part})
        (directory / "model.safetensors.index.json").write_text(json.dumps({"weight_map": index}))
    return want


@pytest.mark.parametrize("preset,shards", [("tiny-llama-test", 1), ("tiny-llama-awq-test", 3), ("tiny-llama-ct-test", 2),
                                           ("tiny-qwen3-test", 2), ("tiny-gemma4-moe-test", 2), ("tiny-qwen35-test", 1),
                                           ("tiny-qwen35-moe-test", 2)])
def test_safetensors_directory_loads_to_the_same_model(tmp_path, preset, shards):
    d = tmp_path / "ckpt"
    want = _export(preset, d, shards=shards)
    loaded = LLM(str(d), device="cpu", dtype="float32", max_num_seqs=4, max_model_len=128)
    try:
        assert _tokens(loaded) == want
    finally:
        loaded.shutdown()


def test_multimodal_export_prefix_and_auxiliary_tensors(tmp_path):
    """`model.language_model.*` names are the text model's; multi-token-prediction heads and rotary tables that
    some exports carry are skipped."""
    d = tmp_path / "ckpt"
    want = _export("tiny-llama-test", d, prefix="model.language_model.",
                   extra={"mtp.layers.0.weight": torch.zeros(4, 4),
                          "model.layers.0.self_attn.rotary_emb.inv_freq": torch.zeros(8)})
    loaded = LLM(str(d), device="cpu", dtype="float32", max_num_seqs=4, max_model_len=128)
    try:
        assert _tokens(loaded) == want
    finally:
        loaded.shutdown()


def test_missing_checkpoint_is_a_clear_error(tmp_path):
    d = tmp_path / "empty"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(PRESETS["tiny-llama-test"]))
    with pytest.raises(FileNotFoundError):
        LLM(str(d), device="cpu")
    with pytest.raises(FileNotFoundError):
        LLM(str(tmp_path / "nowhere"), device="cpu")

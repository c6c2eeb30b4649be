"""Output-processor strategies for ``LLM.generate`` (reference: vllm/entrypoints/output_processors/
{abstract,default,verl}.py)."""
from __future__ import annotations

from abc import ABC, abstractmethod

import torch


class OutputProcessorStrategy(ABC):
    @abstractmethod
    def process_outputs(self, outputs: list):
        ...


class DefaultOutputProcessor(OutputProcessorStrategy):
    def process_outputs(self, outputs: list):
        return outputs


class VerlOutputProcessor(OutputProcessorStrategy):
    """Right-padded ``[n, max_len]`` tensor of generated token ids plus an attention mask, the
    layout RL trainers consume."""

    def __init__(self, pad_token_id: int = 0):
        self.pad_token_id = pad_token_id

    def process_outputs(self, outputs: list):
        seqs = [o.outputs[0].token_ids for o in outputs]
        width = max((len(s) for s in seqs), default=0)
        ids = torch.full((len(seqs), width), self.pad_token_id, dtype=torch.long)
        mask = torch.zeros(len(seqs), width, dtype=torch.long)
        for i, s in enumerate(seqs):
            ids[i, :len(s)] = torch.tensor(s, dtype=torch.long)
            mask[i, :len(s)] = 1
        return {"response_ids": ids, "response_mask": mask, "request_outputs": outputs}


def resolve_output_processor(spec, tokenizer=None) -> OutputProcessorStrategy:
    if isinstance(spec, OutputProcessorStrategy):
        return spec
    name = str(spec or "default").lower()
    if name == "default":
        return DefaultOutputProcessor()
    if name == "verl":
        pad = getattr(tokenizer, "pad_token_id", None)
        return VerlOutputProcessor(pad if isinstance(pad, int) else 0)
    raise ValueError(f"unknown output processor {spec!r}")

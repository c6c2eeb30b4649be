"""Offline inference API: ``LLM(model, **kwargs).generate(prompts, sampling_params)``.

Prompts may be strings, ``TextPrompt`` / ``TokensPrompt`` dicts or plain token-id lists.  Requests
are fed to the engine in groups of ``engine.max_active_requests`` and stepped until all finish; an
output-processor strategy shapes the return value ("default": list of ``RequestOutput``; "verl":
padded token-id tensor).  Reference: vllm/entrypoints/llm.py:16-120.
"""
from __future__ import annotations

import itertools
from typing import Any

import torch

from ..config.config_builder import build_vllm_config
from ..engine.lite_engine import LiteEngine
from ..loaders import get_tokenizer
from ..outputs import RequestOutput
from ..sampling_params import SamplingParams
from .output_processors import resolve_output_processor


class LLM:
    def __init__(self, model: str, **kwargs: Any):
        output_processor = kwargs.pop("output_processor", "default")
        tokenizer = kwargs.pop("tokenizer_object", None)
        self.vllm_config = build_vllm_config(model, **kwargs)
        self._parallel = None
        self._dp = None
        pc = self.vllm_config.parallel_config
        if pc.data_parallel_size > 1:
            # replicas: this process owns one whole engine on its own GPU and a share of every call's prompts
            from ..parallel.data_parallel import DataParallelGroup
            self._dp = DataParallelGroup(pc.data_parallel_size, group_size=pc.world_size)
            if torch.cuda.is_available() and self.vllm_config.device in ("auto", "cuda"):
                self.vllm_config.device = f"cuda:{self._dp.local_rank}"
        if self.vllm_config.parallel_config.is_distributed:
            from ..parallel.launcher import init_distributed_engine
            self._parallel = init_distributed_engine(self.vllm_config)
        self.engine = LiteEngine(self.vllm_config)
        mc = self.vllm_config.model_config
        self.tokenizer = tokenizer or get_tokenizer(mc.tokenizer, mc.trust_remote_code, mc.revision,
                                                    vocab_size=mc.arch.vocab_size)
        self.engine.set_tokenizer(self.tokenizer)
        self.output_processor = resolve_output_processor(output_processor, self.tokenizer)
        self._counter = itertools.count()
        if self._parallel is not None:
            self._parallel.attach(self.engine)

    @property
    def model(self):
        return self.engine.model

    def get_tokenizer(self):
        return self.tokenizer

    @torch.inference_mode()
    def generate(self, prompts, sampling_params: SamplingParams | list[SamplingParams] | None = None,
                 lora_request=None, use_tqdm: bool = False):
        if isinstance(prompts, (str, dict)) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        prompts = list(prompts)
        if isinstance(sampling_params, list):
            if len(sampling_params) != len(prompts):
                raise ValueError("one SamplingParams per prompt expected")
            params = sampling_params
        else:
            params = [sampling_params or SamplingParams()] * len(prompts)
        if self._dp is not None:
            # every replica is called with the same arguments and serves prompts rank, rank + N, ...
            n_all = len(prompts)
            mine = self._dp.my_indices(n_all)
            local = self._generate_local([prompts[i] for i in mine], [params[i] for i in mine], lora_request)
            return self.output_processor.process_outputs(self._dp.gather_in_order(local, n_all))
        return self.output_processor.process_outputs(self._generate_local(prompts, params, lora_request))

    def _generate_local(self, prompts: list, params: list, lora_request=None) -> list[RequestOutput]:
        results: dict[str, RequestOutput] = {}
        order: list[str] = []
        group = self.engine.max_active_requests
        for g0 in range(0, len(prompts), group):
            ids = []
            for prompt, sp in zip(prompts[g0:g0 + group], params[g0:g0 + group]):
                rid = f"llm-{next(self._counter)}"
                self.engine.add_request(rid, prompt, sp, lora_request=lora_request)
                ids.append(rid)
                order.append(rid)
            pending = set(ids)
            while pending:
                for out in self.engine.step():
                    if out is not None and out.finished and out.request_id in pending:
                        results[out.request_id] = out
                        pending.discard(out.request_id)
                if pending and not self.engine.has_unfinished_requests():
                    # a request ended with an exception (rejection/abort): surface it
                    for rid in list(pending):
                        for item in self.engine.scheduler.pop_sync_outputs(rid):
                            if isinstance(item, BaseException):
                                raise item
                    raise RuntimeError("engine went idle with unfinished requests")
            for rid in ids:
                self.engine.scheduler.pop_sync_outputs(rid)
        return [results[r] for r in order]

    def stats(self) -> dict:
        return self.engine.stats()

    def reset_stats(self, clear_prefix_cache: bool = False) -> None:
        self.engine.reset_stats(clear_prefix_cache)

    def register_lora_adapter(self, lora_name: str, lora_path: str, lora_int_id: int | None = None):
        return self.engine.register_lora_adapter(lora_name, lora_path, lora_int_id)

    def unregister_lora_adapter(self, lora_name: str) -> bool:
        return self.engine.unregister_lora_adapter(lora_name)

    def shutdown(self) -> None:
        self.engine.shutdown()
        if self._parallel is not None:
            self._parallel.shutdown()
        if self._dp is not None:
            self._dp.shutdown()

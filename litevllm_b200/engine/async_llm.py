"""Asynchronous engine front end used by the HTTP server.

``submit`` validates and enqueues a request on a worker thread (admission errors surface before any
streaming starts), ``stream`` yields outputs from the request's queue and aborts the request if the
consumer leaves early, ``generate`` = submit + stream.  One ``RLock`` serialises engine access
between submitters and the driver thread.  Reference: vllm/engine/async_llm.py:19-191."""
from __future__ import annotations

import asyncio
from collections.abc import Iterable

from ..loaders import get_tokenizer
from .async_driver import AsyncDriver
from .errors import EngineFatalError
from .lite_engine import LiteEngine
from .protocol import EngineClient


class AsyncLLM(EngineClient):
    def __init__(self, vllm_config, engine: LiteEngine | None = None, tokenizer=None, start_driver: bool = True):
        self.vllm_config = vllm_config
        # several ranks: join the job first (process group, symmetric heap), then build this rank's engine;
        # rank 0 gets a coordinator that mirrors its request stream to the workers (parallel/serving.py)
        self._parallel = None
        self.coordinator = None
        self.channel = None
        self.dp_router = None         # rank 0 of a server with data-parallel replicas
        self._dp_link = None          # this replica's mailbox (ranks other than 0)
        self._dp = None
        if engine is None and vllm_config.parallel_config.data_parallel_size > 1:
            if vllm_config.parallel_config.is_distributed:
                raise NotImplementedError("the server routes requests to single-GPU replicas; replicas that are tensor / "
                                          "expert-parallel groups serve offline generation (LLM) only")
            # replicas: every rank a whole engine on its own GPU; the process group only provides the store
            import torch
            import torch.distributed as dist
            from ..parallel.data_parallel import DataParallelGroup
            from ..parallel.dp_serving import DataParallelRouter, ReplicaLink
            self._dp = DataParallelGroup(vllm_config.parallel_config.data_parallel_size)
            if torch.cuda.is_available() and vllm_config.device in ("auto", "cuda"):
                vllm_config.device = f"cuda:{self._dp.local_rank}"
            store = dist.distributed_c10d._get_default_store()
            if self._dp.rank == 0:
                self.dp_router = DataParallelRouter(store, self._dp.size)
            else:
                self._dp_link = ReplicaLink(store, self._dp.rank)
        if engine is None and vllm_config.parallel_config.is_distributed:
            from ..parallel.launcher import init_distributed_engine
            from ..parallel.serving import ServingCoordinator, make_channel
            self._parallel = init_distributed_engine(vllm_config)
            self.channel = make_channel(self._parallel.state)
            if self._parallel.state.rank == 0:
                self.coordinator = ServingCoordinator(self.channel)
        self.engine = engine or LiteEngine(vllm_config)
        if self._parallel is not None:
            self._parallel.attach(self.engine)
        self.engine_lock = self.engine.lock
        mc = vllm_config.model_config
        self.tokenizer = tokenizer or get_tokenizer(mc.tokenizer, mc.trust_remote_code, mc.revision,
                                                    vocab_size=mc.arch.vocab_size)
        self.engine.set_tokenizer(self.tokenizer)
        self.driver = AsyncDriver(self.engine, self.engine_lock,
                                  vllm_config.runtime_config.async_driver_min_step_interval_s,
                                  coordinator=self.coordinator)
        self._start_driver = start_driver
        self._closed = False

    @classmethod
    def from_vllm_config(cls, vllm_config, **kw) -> "AsyncLLM":
        return cls(vllm_config, **kw)

    def get_model_config(self):
        return self.vllm_config.model_config

    # ------------------------------------------------------------------ request path
    @property
    def is_worker_rank(self) -> bool:
        if self._dp is not None:
            return self._dp.rank != 0
        return self._parallel is not None and self._parallel.state.rank != 0

    def serve_as_worker(self, on_step=None) -> int:
        """Ranks other than 0 of a multi-rank server.  Tensor / expert parallel: mirror rank 0 step by step
        until it shuts down.  Data parallel: serve the requests rank 0 routes to this replica."""
        if self._dp_link is not None:
            from ..parallel.dp_serving import replica_serve_loop
            return replica_serve_loop(self.engine, self._dp_link, on_step=on_step)
        from ..parallel.serving import worker_serve_loop
        return worker_serve_loop(self.engine, self.channel, on_step)

    def _submit_sync(self, request_id, prompt, sampling_params, lora_request, multi_modal_data, loop):
        if self.dp_router is not None:
            replica = self.dp_router.choose()
            if replica != 0:
                if lora_request is not None or multi_modal_data:
                    replica = 0       # adapters and images stay on the rank that received them
                else:
                    # validate and tokenise here, run there
                    with self.engine_lock:
                        self.engine._build_lazy()
                        st = self.engine.request_builder.build(request_id, prompt, sampling_params, None, None)
                        self.engine.adapter.validate_request(st.sampling_params, st.prompt_len, None, None)
                    from ..parallel.serving import ServingCoordinator, sampling_params_to_wire
                    sp = ServingCoordinator.prepare_params(st.sampling_params)
                    self.dp_router.submit_remote(replica, request_id, list(st.prompt_token_ids),
                                                 sampling_params_to_wire(sp), loop)
                    return
            self.dp_router.note_local(request_id)
        if self.coordinator is not None:
            self.coordinator.check_supported(lora_request, multi_modal_data)
            sampling_params = self.coordinator.prepare_params(sampling_params)
        with self.engine_lock:
            st = self.engine.add_request(request_id, prompt, sampling_params, lora_request=lora_request,
                                         multi_modal_data=multi_modal_data, loop=loop)
            if self.coordinator is not None:
                self.coordinator.record_request(st)

    async def submit(self, prompt, sampling_params, request_id: str, lora_request=None, multi_modal_data=None) -> None:
        if self._closed:
            raise EngineFatalError("engine is shut down")
        loop = asyncio.get_running_loop()
        await asyncio.to_thread(self._submit_sync, request_id, prompt, sampling_params, lora_request,
                                multi_modal_data, loop)
        if self._start_driver:
            self.driver.notify_new_work()

    async def stream(self, request_id: str):
        finished = False
        remote = self.dp_router is not None and self.dp_router.is_remote(request_id)
        source = self.dp_router.stream(request_id) if remote else self.engine.get_request_stream(request_id)
        try:
            async for out in source:
                if getattr(out, "finished", False):
                    finished = True
                yield out
        except (GeneratorExit, asyncio.CancelledError):
            raise             # the consumer went away (closed the stream, disconnected): abort below
        except BaseException:
            finished = True   # the stream already delivered its terminal item (an exception)
            raise
        finally:
            if self.dp_router is not None and not remote:
                self.dp_router.finish_local(request_id)
            if not finished:
                await self.abort(request_id)

    async def generate(self, prompt, sampling_params, request_id: str, lora_request=None, multi_modal_data=None):
        await self.submit(prompt, sampling_params, request_id, lora_request, multi_modal_data)
        async for out in self.stream(request_id):
            yield out

    async def close_stream(self, request_id: str) -> None:
        await self.abort(request_id)

    async def abort(self, request_id: str | Iterable[str]) -> None:
        ids = [request_id] if isinstance(request_id, str) else list(request_id)
        def _do():
            with self.engine_lock:
                for rid in ids:
                    if self.dp_router is not None and self.dp_router.abort(rid):
                        continue
                    if self.engine.abort_request(rid) and self.coordinator is not None:
                        self.coordinator.record_abort(rid)
        await asyncio.to_thread(_do)

    # ------------------------------------------------------------------ admin
    def is_healthy(self) -> bool:
        return not self._closed and self.engine.fatal_error is None

    def stats(self) -> dict:
        with self.engine_lock:
            s = self.engine.stats()
        s["async_driver"] = self.driver.stats()
        if self.dp_router is not None:
            s["data_parallel"] = self.dp_router.stats()
        return s

    def reset_stats(self, clear_prefix_cache: bool = False) -> None:
        with self.engine_lock:
            self.engine.reset_stats(clear_prefix_cache)

    def register_lora_adapter(self, lora_name: str, lora_path: str, lora_int_id: int | None = None):
        with self.engine_lock:
            return self.engine.register_lora_adapter(lora_name, lora_path, lora_int_id)

    def unregister_lora_adapter(self, lora_name: str) -> bool:
        with self.engine_lock:
            return self.engine.unregister_lora_adapter(lora_name)

    def shutdown(self) -> None:
        self._closed = True
        if self.dp_router is not None:
            self.dp_router.shutdown()
        self.driver.shutdown()
        self.engine.shutdown()
        if self._parallel is not None:
            self._parallel.shutdown()

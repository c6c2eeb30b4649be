"""Multi-GPU bring-up: one process per GPU (torchrun style env: RANK, LOCAL_RANK, WORLD_SIZE,
MASTER_ADDR, MASTER_PORT).  Every rank runs the same engine on the same request stream (SPMD control
plane): scheduling is deterministic and sampled tokens are identical on all ranks because the logits
are all-gathered and the fused collectives sum in a fixed rank order, so no per-step plan broadcast
is needed for offline generation.  Servers broadcast new requests from rank 0 through
:class:`ControlChannel`.  ``spawn`` starts local worker processes for tests and examples.
"""
from __future__ import annotations

import os

import torch
import torch.multiprocessing as mp

from ..logger import init_logger
from . import state as pstate

logger = init_logger(__name__)


class DistributedHandle:
    def __init__(self, st):
        self.state = st
        self.engine = None

    def attach(self, engine) -> None:
        """Hook liveness checks into the engine: between steps (at most once per heartbeat interval)
        rank liveness is read from the store and the device status word is decoded, so a missing
        peer or a timed-out fused collective surfaces as an exception before the next launch."""
        import time

        import torch.distributed as dist

        from .fault import Heartbeat, decode_status
        self.engine = engine
        if self.state.world_size <= 1 or not dist.is_initialized():
            return
        rc = engine.rc
        store = dist.distributed_c10d._get_default_store()
        self.heartbeat = Heartbeat(store, self.state.rank, self.state.world_size, rc.heartbeat_interval_s,
                                   rc.heartbeat_timeout_s, prefix=f"fi/hb/{self.state.replica}")
        self.heartbeat.start()
        last = [time.monotonic()]

        def pre_step():
            now = time.monotonic()
            if now - last[0] < rc.heartbeat_interval_s:
                return
            last[0] = now
            self.heartbeat.raise_if_dead()
            if torch.cuda.is_available() and self.state.symm is not None:
                from .. import ops
                code = int(ops.status_word(engine.device).item())
                if code:
                    ops.status_word(engine.device).zero_()
                    decode_status(code)
        engine.pre_step_hook = pre_step

    def shutdown(self) -> None:
        """Drop captured CUDA graphs (they hold collective kernels), quiesce, then leave the group.
        The NCCL communicator itself is left to process exit: tearing it down while graph-captured
        collectives exist was observed to block in ``destroy_process_group``."""
        import gc

        import torch.distributed as dist
        hb = getattr(self, "heartbeat", None)
        if hb is not None:
            hb.stop()
        eng = self.engine
        if eng is not None and hasattr(eng, "decode_executor"):
            getattr(eng.decode_executor, "_graphs", {}).clear()
            eng.decode_executor._pool = None
        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if dist.is_initialized():
            try:
                dist.barrier()
            except Exception:
                pass
        pstate.destroy_parallel(destroy_group=not torch.cuda.is_available())


def init_distributed_engine(vllm_config) -> DistributedHandle:
    pc = vllm_config.parallel_config
    st = pstate.init_parallel(pc.tensor_parallel_size, pc.expert_parallel_size, pc.comm_backend,
                              replicas=max(1, pc.data_parallel_size))
    if st.replicas > 1 and st.comm_backend == "fused":
        # the symmetric heap exchanges its handles over the whole job's group: groups of a replicated job use the
        # library collectives
        logger.info("rank %d: %d replicas of %d-rank groups: library collectives inside each group",
                    st.global_rank, st.replicas, st.world_size)
        st.comm_backend = "nccl"
    if st.world_size > 1 and torch.cuda.is_available() and st.comm_backend == "fused":
        from .symm import SymmetricHeap
        dev = torch.device("cuda", st.local_rank)
        try:
            st.symm = SymmetricHeap(st.rank, st.world_size, dev)
            logger.info("rank %d: symmetric heap ready (%d peers)", st.rank, st.world_size)
        except Exception as e:  # pragma: no cover - depends on the platform
            logger.warning("symmetric memory unavailable (%r): falling back to NCCL collectives", e)
            st.symm = None
            st.comm_backend = "nccl"
    if st.symm is not None:
        _self_test_fused(st)
    if torch.cuda.is_available():
        vllm_config.device = f"cuda:{st.local_rank}"
    return DistributedHandle(st)


def _self_test_fused(st) -> None:
    """Start-up check of the in-kernel collectives on this job's actual world size: one small call of
    each fused form against the library collectives.  Every rank learns the verdict of all ranks; a
    failed decode-size all-reduce switches the whole job to the NCCL path, a failed sequence-parallel
    form (reduce-scatter, all-gather) only switches the sequence-parallel prefill off.  A wait that
    runs out shows up as a status code, not as a hang (device waits are bounded)."""
    import torch.distributed as dist

    from .. import ops
    from . import fused_ops
    dev = torch.device("cuda", st.local_rank)
    w = st.world_size

    class _Layer:
        quant_method, bias = None, None

    def agree(ok: bool) -> bool:
        t = torch.tensor([1 if ok else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=st.group)
        return bool(t.item())

    def status_ok() -> bool:
        word = ops.status_word(dev)
        bad = int(word.item()) != 0
        if bad:
            word.zero_()
        return not bad

    def close(a, b) -> bool:
        a, b = a.float(), b.float()
        return bool(torch.isfinite(a).all()) and bool(((a - b).abs() <= 0.05 + 0.05 * b.abs()).all())

    g = torch.Generator(device=dev).manual_seed(1234 + st.rank)
    ok_ar = ok_sp = True
    verdicts: dict = {}
    st.self_test = verdicts

    def run_allreduce(fmt: int) -> bool:
        try:
            T, N, K = 32, 512, 256
            x = (torch.randn(T, K, generator=g, device=dev) * 0.5).bfloat16()
            wt = (torch.randn(N, K, generator=g, device=dev) * 0.05).bfloat16()
            res = torch.randn(T, N, generator=g, device=dev).bfloat16()
            dist.broadcast(res, src=0, group=st.group)
            layer = _Layer()
            layer.weight, layer.out_features = wt, N
            want = x.float() @ wt.float().t()
            dist.all_reduce(want, group=st.group)
            want = want + res.float()
            for _ in range(2):      # twice: both slab parities
                got = fused_ops._fused_gemm_allreduce(layer, x, res, None, st.symm, fmt)
            torch.cuda.synchronize(dev)
            return status_ok() and close(got, want)
        except Exception as e:  # pragma: no cover - platform dependent
            logger.warning("fused all-reduce (format %d) self-test raised %r", fmt, e)
            return False

    ok_ar = agree(run_allreduce(2))
    verdicts["allreduce_one_hop"] = ok_ar
    if ok_ar and fused_ops.decode_allreduce_format(w, torch.bfloat16) == 3:
        ok_two = agree(run_allreduce(3))
        verdicts["allreduce_two_hop"] = ok_two
        if not ok_two:
            logger.warning("rank %d: the two-hop all-reduce failed its start-up check; using the one-hop form", st.rank)
            fused_ops._TWO_SHOT_MIN_WORLD = 1 << 30
    if not ok_ar:
        logger.warning("rank %d: fused collectives failed their start-up check; using NCCL collectives", st.rank)
        st.symm = None
        st.comm_backend = "nccl"
        return
    try:
        rows, V = 8, 1024
        lg = torch.randn(rows, V, generator=g, device=dev)
        gathered = [torch.empty_like(lg) for _ in range(w)]
        dist.all_gather(gathered, lg, group=st.group)
        want_ids = torch.cat(gathered, dim=1).argmax(-1)
        for _ in range(2):
            got_ids = fused_ops.argmax_vocab_parallel(lg, st.rank * V)
        torch.cuda.synchronize(dev)
        ok_am = status_ok() and bool(torch.equal(got_ids, want_ids))
    except Exception as e:  # pragma: no cover - platform dependent
        logger.warning("vocabulary-parallel arg-max self-test raised %r", e)
        ok_am = False
    st.argmax_ok = agree(ok_am)
    verdicts["argmax_vocab_parallel"] = st.argmax_ok
    try:
        rpr, K, N = 128, 256, 256
        x = (torch.randn(rpr * w, K, generator=g, device=dev) * 0.5).bfloat16()
        wt = (torch.randn(N, K, generator=g, device=dev) * 0.05).bfloat16()
        full = x.float() @ wt.float().t()
        dist.all_reduce(full, group=st.group)
        res = torch.zeros(rpr, N, device=dev, dtype=torch.bfloat16)
        for _ in range(2):
            got = fused_ops.gemm_reduce_scatter(x, wt, res, rpr)
        torch.cuda.synchronize(dev)
        ok_sp = status_ok() and close(got, full[st.rank * rpr:(st.rank + 1) * rpr])
        xs = (torch.randn(rpr, K, generator=g, device=dev) * 0.5).bfloat16()
        g2 = torch.Generator(device=dev).manual_seed(99)
        wc = (torch.randn(N, K, generator=g2, device=dev) * 0.05).bfloat16()
        gathered = [torch.empty_like(xs) for _ in range(w)]
        dist.all_gather(gathered, xs, group=st.group)
        want = torch.cat(gathered).float() @ wc.float().t()
        for _ in range(2):
            got = fused_ops.allgather_gemm(xs, wc, rpr * w, rpr)
        torch.cuda.synchronize(dev)
        ok_sp = ok_sp and status_ok() and close(got, want)
    except Exception as e:  # pragma: no cover - platform dependent
        logger.warning("sequence-parallel self-test raised %r", e)
        ok_sp = False
    st.sequence_parallel_ok = agree(ok_sp)
    verdicts["sequence_parallel"] = st.sequence_parallel_ok
    if not st.sequence_parallel_ok:
        logger.warning("rank %d: fused reduce-scatter / all-gather failed their start-up check; "
                       "sequence-parallel prefill is off", st.rank)


def _worker(rank: int, world: int, port: int, fn, args):
    os.environ["RANK"] = str(rank)
    os.environ["LOCAL_RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    fn(rank, world, *args)
    # leave without running interpreter teardown: destructors of the process group (gloo's threads as well as
    # NCCL's), of captured graphs and of the CUDA context race at exit (seen as "double free or corruption" from a
    # finished, successful rank)
    import sys
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def _usable_port(port: int) -> int:
    """``port`` if it can be bound on the loopback interface right now, else a free one."""
    import socket
    for candidate in (port, 0):
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            try:
                s.bind(("127.0.0.1", candidate))
                return s.getsockname()[1]
            except OSError:
                continue
    return port


def spawn(fn, world: int, args: tuple = (), port: int = 29531, join: bool = True):
    """Run ``fn(rank, world, *args)`` in ``world`` local processes (rendezvous on 127.0.0.1; a busy
    ``port`` is replaced by a free one)."""
    port = _usable_port(port)
    return mp.spawn(_worker, args=(world, port, fn, args), nprocs=world, join=join)

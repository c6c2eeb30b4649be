"""Symmetric (peer-mapped) device memory for the fused compute+collective kernels.

One ``cudaMalloc`` buffer per rank, exported as a CUDA IPC memory handle; the 64-byte handles are
exchanged as plain bytes with an ``all_gather`` and every rank opens its peers' handles
(csrc/fused_comm/ipc.cu).  Every rank then sees every peer's buffer at ``peer_ptr[d]`` and the fused
kernels store to / poll / TMA-load from those addresses over NVLink.  The buffer is carved into
  * ``recv``  : receive slabs of the GEMM->all-reduce / reduce-scatter epilogue
                ``[2 parities][world sources][slab]``,
  * ``flags`` : one word per (tile, source rank, cluster part), written with the call's epoch,
  * ``ready`` : all-gather "my shard is complete" words, one per source rank,
  * ``xbuf``  : two token-shard buffers (double-buffered by epoch parity) that peers read with TMA,
  * ``ctl``   : local ``epoch`` / ``done`` counters,
  * ``amax``  : slots of the vocabulary-parallel arg-max (one 16-byte word per source rank and row).
``SymmetricHeap.emulated(world, device)`` carves ``world`` such regions out of ONE allocation on one
GPU, so the push / poll / ownership code of the kernels can be exercised phase by phase without a
second device.  The reference has no counterpart (single GPU).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

MAX_RANKS = 8
FLAG_PARTS = 8
AMAX_ROWS = 1024
MAX_COMM_TILES = 8192
AG_PARTS = 8
AMAX_ROWS = 1024


class FiComm(ctypes.Structure):
    _fields_ = [("mode", ctypes.c_int), ("world", ctypes.c_int), ("rank", ctypes.c_int),
                ("rows_per_rank", ctypes.c_int), ("xfer_16bit", ctypes.c_int), ("ag_world", ctypes.c_int),
                ("ag_rows_per_rank", ctypes.c_int), ("phases", ctypes.c_int), ("slab_elems", ctypes.c_long),
                ("recv", ctypes.c_ulonglong * 8), ("flags", ctypes.c_ulonglong * 8),
                ("ready", ctypes.c_ulonglong * 8), ("x_peers", ctypes.c_ulonglong * 8),
                ("epoch", ctypes.c_ulonglong), ("done", ctypes.c_ulonglong), ("trace", ctypes.c_ulonglong),
                ("x_full", ctypes.c_ulonglong), ("ag_flags", ctypes.c_ulonglong)]


class _RawCudaBuffer:
    """Exposes a raw device allocation to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class SymmetricHeap:
    def __init__(self, rank: int, world: int, device: torch.device, recv_bytes: int = 512 << 20,
                 xbuf_bytes: int = 64 << 20, group=None, ll_elems: int = 512 * 1024):
        from ..ops import _lib
        self._layout(rank, world, device, recv_bytes, xbuf_bytes, ll_elems)
        total = self.total_bytes
        lib = self._lib = _lib.kernels()
        torch.cuda.set_device(device)
        base = ctypes.c_void_p()
        _lib.check(lib.fi_symm_alloc(ctypes.byref(base), total), "fi_symm_alloc")
        self.base = int(base.value)
        self._owns_base = True
        handle = ctypes.create_string_buffer(64)
        _lib.check(lib.fi_ipc_get_handle(self.base, handle), "fi_ipc_get_handle")
        # exchange the 64-byte handles as plain bytes over the process group
        mine = torch.tensor(list(handle.raw), dtype=torch.uint8, device=device)
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine, group=group)
        self.peer_ptr = []
        self._opened = []
        for d in range(world):
            if d == rank:
                self.peer_ptr.append(self.base)
                continue
            raw = bytes(gathered[d].cpu().tolist())
            out = ctypes.c_void_p()
            _lib.check(lib.fi_ipc_open_handle(raw, ctypes.byref(out)), f"fi_ipc_open_handle(rank {d})")
            self.peer_ptr.append(int(out.value))
            self._opened.append(int(out.value))
        self.buffer = torch.as_tensor(_RawCudaBuffer(self.base, total), device=device)
        self.trace_ptr = 0           # set to a device int64[64*8] array to record kernel phase timestamps
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def _layout(self, rank, world, device, recv_bytes, xbuf_bytes, ll_elems) -> None:
        self.rank, self.world, self.device = rank, world, device
        self.flag_bytes = MAX_COMM_TILES * MAX_RANKS * FLAG_PARTS * 4
        self.ready_bytes = 256
        self.ctl_bytes = 256
        self.recv_bytes = (recv_bytes + 255) // 256 * 256
        self.xbuf_bytes = (xbuf_bytes + 255) // 256 * 256
        self.off_recv = 0
        self.off_flags = self.off_recv + self.recv_bytes
        self.off_ready = self.off_flags + self.flag_bytes
        self.off_ctl = self.off_ready + self.ready_bytes
        self.off_xbuf = (self.off_ctl + self.ctl_bytes + 1023) // 1024 * 1024
        # low-latency slabs (fp32 value + epoch per 8-byte word), kept apart from the flagged slabs so
        # that no other transfer format ever writes there: 2 parities x world sources
        self.ll_elems = ll_elems
        self.off_ll = self.off_xbuf + 2 * self.xbuf_bytes
        # all-gather staging: the gathered token matrix (world shards) and its per-(tile, part) flags
        self.off_xfull = self.off_ll + 2 * world * ll_elems * 8
        self.xfull_bytes = world * self.xbuf_bytes
        self.off_agflags = self.off_xfull + self.xfull_bytes
        self.agflag_bytes = MAX_COMM_TILES * AG_PARTS * 4
        # vocabulary-parallel arg-max slots: uint4 [2 parities][world][AMAX_ROWS]
        self.off_amax = self.off_agflags + self.agflag_bytes
        self.amax_bytes = 2 * world * AMAX_ROWS * 16
        self.total_bytes = (self.off_amax + self.amax_bytes + 1023) // 1024 * 1024

    @classmethod
    def emulated(cls, world: int, device: torch.device, recv_bytes: int = 32 << 20, xbuf_bytes: int = 4 << 20,
                 ll_elems: int = 256 * 1024) -> list["SymmetricHeap"]:
        """``world`` heaps that live side by side in ONE allocation on ``device``: heap ``r`` is what
        rank ``r`` of a ``world``-rank job would hold, and its peer pointers address the other regions.
        No process group, no IPC.  Kernels of different virtual ranks cannot wait for one another on
        one GPU, so callers drive a fused call phase by phase (``comm_desc(phases=...)``): the push phase
        of every rank, then the reduce phase of every rank, then (two-hop form) the collect phase."""
        from ..ops import _lib
        lib = _lib.kernels()
        heaps = []
        for r in range(world):
            h = object.__new__(cls)
            h._layout(r, world, device, recv_bytes, xbuf_bytes, ll_elems)
            h._lib = lib
            heaps.append(h)
        region = heaps[0].total_bytes
        torch.cuda.set_device(device)
        base = ctypes.c_void_p()
        _lib.check(lib.fi_symm_alloc(ctypes.byref(base), region * world), "fi_symm_alloc")
        whole = torch.as_tensor(_RawCudaBuffer(int(base.value), region * world), device=device)
        for r, h in enumerate(heaps):
            h.base = int(base.value) + r * region
            h._owns_base = r == 0
            h._alloc_base = int(base.value)
            h.peer_ptr = [int(base.value) + d * region for d in range(world)]
            h._opened = []
            h.buffer = whole[r * region:(r + 1) * region]
            h.trace_ptr = 0
        torch.cuda.synchronize(device)
        return heaps

    # ------------------------------------------------------------------ views
    def xbuf(self, parity: int, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        n = rows * cols * torch.empty((), dtype=dtype).element_size()
        if n > self.xbuf_bytes:
            raise MemoryError(f"token shard of {n} bytes exceeds the symmetric xbuf ({self.xbuf_bytes})")
        o = self.off_xbuf + parity * self.xbuf_bytes
        return self.buffer[o:o + n].view(dtype).view(rows, cols)

    def fits_recv(self, T: int, N: int, elem: int) -> bool:
        return 2 * self.world * T * N * elem <= self.recv_bytes

    def fits_low_latency(self, T: int, N: int) -> bool:
        return T * N <= self.ll_elems

    def comm_desc(self, mode: int, T: int, N: int, xfer_16bit: bool | int, rows_per_rank: int = 0,
                  ag_world: int = 1, ag_rows_per_rank: int = 0, x_parity: int = 0, staged: bool = False,
                  phases: int = 0) -> FiComm:
        c = FiComm()
        c.mode, c.world, c.rank = mode, self.world, self.rank
        c.rows_per_rank = rows_per_rank
        c.phases = phases
        # 0 fp32 + flags, 1 16-bit + flags, 2 fp32 with inline epochs, 3 two-hop all-reduce with inline epochs
        c.xfer_16bit = int(xfer_16bit)
        recv_off = self.off_ll if c.xfer_16bit >= 2 else self.off_recv
        c.ag_world, c.ag_rows_per_rank = ag_world, ag_rows_per_rank
        slab_rows = rows_per_rank if mode == 2 else T
        c.slab_elems = slab_rows * N
        for d in range(self.world):
            c.recv[d] = self.peer_ptr[d] + recv_off
            c.flags[d] = self.peer_ptr[d] + self.off_flags
            c.ready[d] = self.peer_ptr[d] + self.off_ready
            c.x_peers[d] = self.peer_ptr[d] + self.off_xbuf + x_parity * self.xbuf_bytes
        c.epoch = self.peer_ptr[self.rank] + self.off_ctl
        c.done = self.peer_ptr[self.rank] + self.off_ctl + 64
        c.trace = self.trace_ptr
        c.x_full = self.base + self.off_xfull if staged else 0
        c.ag_flags = self.base + self.off_agflags
        return c

    def argmax_desc(self, phases: int = 0) -> FiComm:
        """Descriptor of the vocabulary-parallel arg-max (``fi_argmax_tp``)."""
        c = FiComm()
        c.mode, c.world, c.rank, c.phases = 1, self.world, self.rank, phases
        c.rows_per_rank = AMAX_ROWS
        for d in range(self.world):
            c.recv[d] = self.peer_ptr[d] + self.off_amax
        c.epoch = self.peer_ptr[self.rank] + self.off_ctl
        c.done = self.peer_ptr[self.rank] + self.off_ctl + 64
        return c

    def epoch_value(self) -> int:
        return int(self.buffer[self.off_ctl:self.off_ctl + 4].view(torch.int32).item())

    def close(self) -> None:
        """Unmap the peers, then free the local buffer (call only when no kernel is in flight)."""
        if self.buffer is None:
            return
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            self._lib.fi_ipc_close_handle(p)
        self._opened = []
        self.buffer = None
        if self._owns_base:
            self._lib.fi_symm_free(getattr(self, "_alloc_base", self.base))

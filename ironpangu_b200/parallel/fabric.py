"""Symmetric heap shared by the ranks of one node (one process per GPU).

Each rank ``cudaMalloc``s one block holding a double-buffered staging area, double-buffered flag
words, the fused-collective call counter, a CTA ticket and a sticky status word; the blocks are
exchanged as CUDA IPC handles through ``torch.distributed`` and mapped into every peer. Fused
kernels then push partial tiles into peers' staging areas with plain stores over NVLink and
synchronise through the flag words (bounded spins).

The reference bootstraps HCCL communicators from root info on the engine thread
(native/src/program_engine.cpp:84-85, native/src/token_executor.h:251-259); this module is the
equivalent bootstrap for kernels that carry their own collectives.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..ops import _lib

STATUS_PEER_TIMEOUT = 1
STATUS_MBAR_TIMEOUT = 2
STATUS_BAD_INDEX = 4


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class Fabric:
    """Owner of this rank's symmetric block and of the peer mappings."""

    def __init__(self, rank: int = 0, world: int = 1, group=None, data_half_bytes: int = 4 << 20,
                 flag_half_words: int = 8 * 296, ll_half_bytes: int = 2 << 20, spin_limit: int = 4_000_000, device: Optional[torch.device] = None,
                 silent_peers: bool = False):
        """``silent_peers``: the other ``world - 1`` ranks are blocks on THIS device that nothing ever writes - a one-process
        stand-in for peers that never arrive, used to exercise the bounded waits (with a small ``spin_limit``) without a
        second GPU and without hanging one: every kernel gives up after ``spin_limit`` polls and reports through the status word."""
        if world < 1 or world > _lib.MAX_RANKS:
            raise ValueError("world must be 1..8")
        self.rank, self.world, self.group = rank, world, group
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.lib = _lib.load()
        self.data_half_bytes = _align(data_half_bytes, 256)
        self.flag_half_words = flag_half_words
        flag_bytes = _align(2 * flag_half_words * 8, 256)
        self._off_flags = 2 * self.data_half_bytes
        self._off_ctl = self._off_flags + flag_bytes
        self.ll_half_bytes = _align(ll_half_bytes, 256)
        self._off_ll = self._off_ctl + 256          # tagged-store area of the one-shot all-reduce (two parity halves)
        self.bytes = self._off_ll + 2 * self.ll_half_bytes
        base = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.ifab_set_device(self.device.index or 0), "set device")
            _lib.check(self.lib.ifab_device_alloc(C.byref(base), self.bytes), "fabric alloc")
        self.base = base.value
        self.peer_bases = [0] * _lib.MAX_RANKS
        self.peer_bases[rank] = self.base
        self._imported = []
        self._silent = []
        if world > 1 and silent_peers:
            for r in range(world):
                if r == rank:
                    continue
                blk = C.c_void_p()
                with torch.cuda.device(self.device):
                    _lib.check(self.lib.ifab_device_alloc(C.byref(blk), self.bytes), "fabric alloc (silent peer)")
                self.peer_bases[r] = blk.value
                self._silent.append(blk.value)
        elif world > 1:
            self._exchange()
        f = _lib.IfabFabric()
        for r in range(world):
            f.data[r] = self.peer_bases[r]
            f.flags[r] = self.peer_bases[r] + self._off_flags
        f.seq = self.base + self._off_ctl
        f.done = self.base + self._off_ctl + 8
        f.status = self.base + self._off_ctl + 16
        f.rank, f.world = rank, world
        f.spin_limit = spin_limit
        f.data_half_bytes = self.data_half_bytes
        f.flag_half_words = flag_half_words
        f.ll_half_bytes = self.ll_half_bytes
        f.ll_offset = self._off_ll
        self.desc = f
        # a scratch ticket area for kernels that use a "last CTA finishes" pattern without a fabric
        self.ticket_ptr = self.base + self._off_ctl + 32

    # -- bootstrap -------------------------------------------------------------------------------
    def _exchange(self) -> None:
        import torch.distributed as dist

        handle = C.create_string_buffer(64)
        _lib.check(self.lib.ifab_ipc_export(self.base, handle), "ipc export")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=self.group)
        for r, h in enumerate(handles):
            if r == self.rank:
                continue
            out = C.c_void_p()
            with torch.cuda.device(self.device):
                _lib.check(self.lib.ifab_ipc_import(h, C.byref(out)), f"ipc import from rank {r}")
            self.peer_bases[r] = out.value
            self._imported.append(out.value)
        dist.barrier(group=self.group)

    # -- status ------------------------------------------------------------------------------------
    def _peek(self, ptr: int, ctype):
        out = ctype(0)
        torch.cuda.current_stream().synchronize()
        _lib.check(self.lib.ifab_peek(C.byref(out), ptr, C.sizeof(ctype)), "peek")
        return int(out.value)

    def status(self) -> int:
        """Read the sticky status word (device -> host, 4 bytes; synchronises the current stream)."""
        return self._peek(self.desc.status, C.c_uint32)

    def clear_status(self) -> None:
        zero = C.c_uint32(0)
        _lib.check(self.lib.ifab_poke(self.desc.status, C.byref(zero), 4), "poke")

    def calls(self) -> int:
        """Number of fused-collective launches completed on this rank."""
        return self._peek(self.desc.seq, C.c_uint64)

    # -- symmetric tensors ---------------------------------------------------------------------------
    def symmetric_empty(self, shape, dtype=torch.bfloat16) -> "SymmetricTensor":
        """Collective: allocate one zero-filled buffer of this shape on every rank and map all of them into every
        process. Kernels that publish results to all ranks (fused GEMM + all-reduce) write through ``peer_ptrs``."""
        return SymmetricTensor(self, tuple(int(d) for d in shape), dtype)

    def close(self) -> None:
        if getattr(self, "base", None) is None:
            return
        torch.cuda.synchronize()
        for blk in self._silent:
            self.lib.ifab_device_free(blk)
        self._silent = []
        if self.world > 1 and self._imported:
            import torch.distributed as dist
            try:
                dist.barrier(group=self.group)
            except Exception:
                pass
        for p in self._imported:
            self.lib.ifab_ipc_close(p)
        self._imported = []
        self.lib.ifab_device_free(self.base)
        self.base = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _CudaBuffer:
    """Minimal ``__cuda_array_interface__`` holder so torch can view memory this library allocated."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmetricTensor:
    """One buffer per rank, each mapped into every process. ``tensor`` is the local view; ``peer_ptrs`` is a
    ``void*[8]`` with every rank's base address as seen from this process (entry ``rank`` is the local one)."""

    def __init__(self, fabric: "Fabric", shape, dtype):
        self.fabric, self.shape, self.dtype = fabric, shape, dtype
        n = 1
        for d in shape:
            n *= d
        self.nbytes = max(256, (n * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256)
        lib = fabric.lib
        base = C.c_void_p()
        with torch.cuda.device(fabric.device):
            _lib.check(lib.ifab_device_alloc(C.byref(base), self.nbytes), "symmetric alloc")
        self.base = base.value
        self._imported = []
        ptrs = [0] * _lib.MAX_RANKS
        ptrs[fabric.rank] = self.base
        if fabric.world > 1:
            import torch.distributed as dist
            handle = C.create_string_buffer(64)
            _lib.check(lib.ifab_ipc_export(self.base, handle), "ipc export")
            handles = [None] * fabric.world
            dist.all_gather_object(handles, bytes(handle.raw), group=fabric.group)
            for r, h in enumerate(handles):
                if r == fabric.rank:
                    continue
                out = C.c_void_p()
                with torch.cuda.device(fabric.device):
                    _lib.check(lib.ifab_ipc_import(h, C.byref(out)), f"ipc import from rank {r}")
                ptrs[r] = out.value
                self._imported.append(out.value)
            dist.barrier(group=fabric.group)
        self.peer_ptrs = (C.c_void_p * _lib.MAX_RANKS)(*[p or None for p in ptrs])
        raw = torch.as_tensor(_CudaBuffer(self.base, self.nbytes), device=fabric.device)
        self.tensor = raw[: n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)

    def close(self) -> None:
        if self.base is None:
            return
        torch.cuda.synchronize()
        for p in self._imported:
            self.fabric.lib.ifab_ipc_close(p)
        self.fabric.lib.ifab_device_free(self.base)
        self.base = None

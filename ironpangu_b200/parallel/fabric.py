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
import os
from typing import Optional

import torch

from ..ops import _lib

def _nvls_wanted(flag: Optional[bool]) -> bool:
    """``IFAB_NVLS=0`` keeps every block on plain peer mappings (tests in which a rank leaves must: a process that dies
    while its memory is bound to a multicast object faults its peers' NVLink)."""
    if flag is not None:
        return bool(flag)
    return os.environ.get("IFAB_NVLS", "1") != "0"


class _SymBlock:
    """One zero-filled block of ``nbytes`` per rank, each mapped into every process of ``group``.

    Two ways to get there. With NVLS (NVLink multicast, asked for by default and used when every rank gets it): the block
    comes from torch's symmetric-memory allocator, whose rendezvous exchanges the handles, maps the peers and binds all
    copies to one multicast object; ``mc`` is then the multicast address of the block (``multimem.*`` instructions of the
    kernels go there). Otherwise: ``cudaMalloc`` + CUDA IPC handles exchanged through ``torch.distributed``; ``mc`` is 0."""

    def __init__(self, lib, rank: int, world: int, group, device, nbytes: int, nvls: bool):
        self.lib, self.rank, self.world, self.group, self.device, self.nbytes = lib, rank, world, group, device, nbytes
        self.peers = [0] * _lib.MAX_RANKS
        self.mc = 0
        self._imported = []
        self._symm = None
        self.base = None
        if world > 1 and nvls and self._try_symmetric():
            return
        base = C.c_void_p()
        with torch.cuda.device(device):
            _lib.check(lib.ifab_set_device(device.index or 0), "set device")
            _lib.check(lib.ifab_device_alloc(C.byref(base), nbytes), "symmetric alloc")
        self.base = base.value
        self.peers[rank] = self.base
        if world > 1:
            self._exchange_ipc()

    def _try_symmetric(self) -> bool:
        import torch.distributed as dist

        t = h = None
        try:
            import torch.distributed._symmetric_memory as symm

            pg = self.group if self.group is not None else dist.group.WORLD
            try:
                symm.enable_symm_mem_for_group(pg.group_name)
            except Exception:
                pass
            with torch.cuda.device(self.device):
                t = symm.empty(self.nbytes, dtype=torch.uint8, device=self.device)
                t.zero_()
                h = symm.rendezvous(t, pg)
            ok = int(h.multicast_ptr) != 0       # 0: the allocator found no multicast support on this machine
        except Exception:
            ok = False
        votes = [None] * self.world
        dist.all_gather_object(votes, ok, group=self.group)
        if not all(votes):
            del h, t
            return False
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._symm = (t, h)
        self.base = t.data_ptr()
        ptrs = list(h.buffer_ptrs)
        for r in range(self.world):
            self.peers[r] = int(ptrs[r])
        self.mc = int(h.multicast_ptr)
        return True

    def _exchange_ipc(self) -> None:
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
            self.peers[r] = out.value
            self._imported.append(out.value)
        dist.barrier(group=self.group)

    def close(self, barrier: bool = True) -> None:
        if self.base is None:
            return
        torch.cuda.synchronize()
        if self.world > 1 and barrier:
            import torch.distributed as dist
            try:
                dist.barrier(group=self.group)
            except Exception:
                pass
        if self._symm is not None:
            self._symm = None          # torch unbinds and frees the block when the last reference goes
        else:
            for p in self._imported:
                self.lib.ifab_ipc_close(p)
            self.lib.ifab_device_free(self.base)
        self._imported = []
        self.base = None


STATUS_PEER_TIMEOUT = 1
STATUS_MBAR_TIMEOUT = 2
STATUS_BAD_INDEX = 4


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class Fabric:
    """Owner of this rank's symmetric block and of the peer mappings."""

    def __init__(self, rank: int = 0, world: int = 1, group=None, data_half_bytes: int = 4 << 20,
                 flag_half_words: int = 8 * 296, ll_half_bytes: int = 2 << 20, spin_limit: int = 4_000_000, device: Optional[torch.device] = None,
                 silent_peers: bool = False, nvls: Optional[bool] = None):
        """``silent_peers``: the other ``world - 1`` ranks are blocks on THIS device that nothing ever writes - a one-process
        stand-in for peers that never arrive, used to exercise the bounded waits (with a small ``spin_limit``) without a
        second GPU and without hanging one: every kernel gives up after ``spin_limit`` polls and reports through the status word.
        ``nvls``: bind the blocks of all ranks to one NVLink multicast object when the machine offers it (default: yes, unless
        ``IFAB_NVLS=0``); ``self.mc`` is then non-zero and the fused collectives push with ``multimem.st``."""
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
        self.nvls_wanted = _nvls_wanted(nvls) and not silent_peers
        self._block = _SymBlock(self.lib, rank, world if not silent_peers else 1, group, self.device, self.bytes, self.nvls_wanted)
        self.base = self._block.base
        self.mc = self._block.mc
        self.peer_bases = list(self._block.peers)
        self.peer_bases[rank] = self.base
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
        f.mc = self.mc or None
        self.desc = f
        # a scratch ticket area for kernels that use a "last CTA finishes" pattern without a fabric
        self.ticket_ptr = self.base + self._off_ctl + 32

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
        self._block.close()
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
        self._block = _SymBlock(fabric.lib, fabric.rank, fabric.world, fabric.group, fabric.device, self.nbytes,
                                fabric.nvls_wanted and fabric.mc != 0)
        self.base = self._block.base
        self.mc_ptr = self._block.mc          # multicast address of this buffer (0 without NVLS)
        ptrs = list(self._block.peers)
        self.peer_ptrs = (C.c_void_p * _lib.MAX_RANKS)(*[p or None for p in ptrs])
        raw = torch.as_tensor(_CudaBuffer(self.base, self.nbytes), device=fabric.device)
        self.tensor = raw[: n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)

    def close(self) -> None:
        if self.base is None:
            return
        self.tensor = None
        self._block.close(barrier=False)
        self.base = None

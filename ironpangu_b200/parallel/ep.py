"""Expert parallelism with sharded tokens: dispatch / combine all-to-all over NVLink peer memory.

``EpExchange`` owns the symmetric receive / return buffers of one rank and wraps the five kernels of
``csrc/kernels/ep_a2a.cu``. One MoE layer on tokens that live on this rank only::

    ex.dispatch(h_norm, ids)                 # token rows -> owner ranks (peer stores), counts + flags
    ex.plan()                                # owner: sort received rows by expert, tile table
    ex.gather(xp)                            # owner: expert-sorted activation matrix
    grouped_gemm(xp, w_gate_up, ex.tiles, ex.num_tiles, act, swiglu=True)
    grouped_gemm(act, w_down, ex.tiles, ex.num_tiles, y)
    ex.send_back(y)                          # expert outputs -> source ranks (peer stores), flags
    ex.combine(ids, wts, out, shared=..., residual=...)

Every rank must run the same sequence of calls (the flags carry a call number).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..ops import _lib
from ..ops._lib import check
from .fabric import Fabric

BF16 = torch.bfloat16


class EpExchange:
    def __init__(self, fabric: Fabric, max_local_rows: int, topk: int, hidden: int, experts_local: int):
        self.fab, self.world, self.rank = fabric, fabric.world, fabric.rank
        self.topk, self.D, self.el = topk, hidden, experts_local
        self.cap = max_local_rows * topk                  # rows one source may send to one destination
        W, dev = self.world, fabric.device
        rows = W * self.cap
        self.recv = fabric.symmetric_empty((rows, hidden), BF16)
        self.meta = fabric.symmetric_empty((rows, 2), torch.int32)
        self.ret = fabric.symmetric_empty((rows, hidden), BF16)
        self.ctl = fabric.symmetric_empty((64,), torch.int64)      # EpCtl: 2 x 8 u64 flags + 8 i32 counts
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        self.send_idx = i32(max_local_rows * topk)
        self.ticket = i32(4)
        self.dst_count = i32(8)
        self.perm = i32(rows)
        self.max_tiles = (rows + 127) // 128 + experts_local
        self.tiles = i32(self.max_tiles, 4)
        self.num_tiles = i32(1)
        self.total_rows = i32(1)
        self.epoch = 0
        self.rows_max = rows
        self.lib = _lib.load()
        for name, sig in {
            "ifab_ep_dispatch": [C.c_void_p, C.c_long, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p],
            "ifab_ep_plan": [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                             C.c_uint64, C.c_uint32, C.c_void_p, C.c_void_p],
            "ifab_ep_gather": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_int, C.c_void_p],
            "ifab_ep_return": [C.c_void_p, C.c_long, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                               C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p],
            "ifab_ep_combine": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                C.c_int, C.c_void_p, C.c_long, C.c_void_p, C.c_long, C.c_void_p, C.c_long, C.c_uint64, C.c_uint32,
                                C.c_void_p, C.c_void_p],
        }.items():
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = sig, C.c_int

    def _s(self) -> int:
        return torch.cuda.current_stream().cuda_stream

    def dispatch(self, xn: torch.Tensor, ids: torch.Tensor) -> None:
        M, topk = ids.shape
        assert topk == self.topk and M * topk <= self.send_idx.numel() and ids.is_contiguous() and xn.stride(1) == 1
        self.epoch += 1
        self._M = M
        check(self.lib.ifab_ep_dispatch(xn.data_ptr(), xn.stride(0), ids.data_ptr(), M, topk, self.D, self.el, self.world, self.rank, self.cap,
                                        self.send_idx.data_ptr(), self.recv.peer_ptrs, self.meta.peer_ptrs, self.ctl.peer_ptrs,
                                        self.ticket.data_ptr(), self.dst_count.data_ptr(), self.epoch, self.fab.desc.status, self._s()),
              "ep_dispatch")

    def plan(self) -> None:
        check(self.lib.ifab_ep_plan(self.meta.tensor.data_ptr(), self.ctl.tensor.data_ptr(), self.world, self.cap, self.el,
                                    self.perm.data_ptr(), self.tiles.data_ptr(), self.num_tiles.data_ptr(), self.total_rows.data_ptr(),
                                    self.max_tiles, self.epoch, self.fab.desc.spin_limit, self.fab.desc.status, self._s()), "ep_plan")

    def gather(self, xp: torch.Tensor) -> None:
        check(self.lib.ifab_ep_gather(self.recv.tensor.data_ptr(), self.perm.data_ptr(), self.total_rows.data_ptr(), xp.data_ptr(),
                                      xp.stride(0), self.D, min(xp.shape[0], self.rows_max), self._s()), "ep_gather")

    def send_back(self, y: torch.Tensor) -> None:
        check(self.lib.ifab_ep_return(y.data_ptr(), y.stride(0), self.perm.data_ptr(), self.total_rows.data_ptr(), self.D, self.cap,
                                      self.world, self.rank, min(y.shape[0], self.rows_max), self.ret.peer_ptrs, self.ctl.peer_ptrs,
                                      self.ticket.data_ptr() + 8, self.epoch, self._s()), "ep_return")

    def combine(self, ids: torch.Tensor, wts: torch.Tensor, out: torch.Tensor, *, shared: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None) -> None:
        M, topk = ids.shape
        p = lambda t: None if t is None else t.data_ptr()
        ld = lambda t: 0 if t is None else t.stride(0)
        check(self.lib.ifab_ep_combine(self.ret.tensor.data_ptr(), self.ctl.tensor.data_ptr(), ids.data_ptr(), self.send_idx.data_ptr(),
                                       wts.data_ptr(), M, topk, self.D, self.el, self.world, self.cap, p(shared), ld(shared), p(residual),
                                       ld(residual), out.data_ptr(), out.stride(0), self.epoch, self.fab.desc.spin_limit,
                                       self.fab.desc.status, self._s()), "ep_combine")

    def close(self) -> None:
        for t in (self.recv, self.meta, self.ret, self.ctl):
            t.close()

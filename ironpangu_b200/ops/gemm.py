"""Tensor-core GEMM entry points (tcgen05 / TMEM / TMA kernels)."""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import check

BF16 = torch.bfloat16


def gemm(a: torch.Tensor, b: torch.Tensor, *, residual: Optional[torch.Tensor] = None, out_f32: bool = False,
         out: Optional[torch.Tensor] = None, status_ptr: Optional[int] = None) -> torch.Tensor:
    """``C = A @ B.T (+ residual)`` with ``A`` = ``[M, K]`` activations and ``B`` = ``[N, K]`` weights, both bf16
    with contiguous K; f32 accumulation in tensor memory."""
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and a.dtype == BF16 and b.dtype == BF16 and a.stride(1) == 1 and b.stride(1) == 1
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_f32 else BF16, device=a.device)
    check(_lib.load().ifab_gemm_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0),
                                     int(out.dtype == torch.float32), None if residual is None else residual.data_ptr(),
                                     0 if residual is None else residual.stride(0), M, N, K, status_ptr,
                                     torch.cuda.current_stream().cuda_stream), "gemm")
    return out


def gemm_2sm(a: torch.Tensor, b: torch.Tensor, *, residual: Optional[torch.Tensor] = None, out_f32: bool = False,
             out: Optional[torch.Tensor] = None, status_ptr: Optional[int] = None, persistent: bool = False) -> torch.Tensor:
    """:func:`gemm` on CTA pairs: 256 x 256 tiles, ``tcgen05.mma.cta_group::2``, every CTA streams half of the tile's A rows and
    half of its B rows. ``N`` must be a multiple of 32; tails in M, N and K are zero-filled on load and masked on store. ``persistent``: one pair per SM pair walks the tiles with two
    accumulators in tensor memory (epilogue under the next tile's MMAs)."""
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and a.dtype == BF16 and b.dtype == BF16 and a.stride(1) == 1 and b.stride(1) == 1
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_f32 else BF16, device=a.device)
    fn = _lib.load().ifab_gemm_bf16_2sm_persistent if persistent else _lib.load().ifab_gemm_bf16_2sm
    check(fn(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0),
             int(out.dtype == torch.float32), None if residual is None else residual.data_ptr(),
             0 if residual is None else residual.stride(0), M, N, K, status_ptr, torch.cuda.current_stream().cuda_stream), "gemm_2sm")
    return out


def gemm_swiglu(a: torch.Tensor, b: torch.Tensor, *, out: Optional[torch.Tensor] = None, status_ptr: Optional[int] = None) -> torch.Tensor:
    """``silu(A @ gate.T) * (A @ up.T)`` for the packed projection ``b`` = ``[2F, K]`` (gate rows, then up rows) on CTA pairs
    (persistent, gate and up of the same 128 output columns under one accumulator); returns bf16 ``[M, F]``. ``F % 32 == 0``."""
    M, K = a.shape
    F = b.shape[0] // 2
    assert b.shape[1] == K and b.shape[0] == 2 * F and a.dtype == BF16 and b.dtype == BF16 and a.stride(1) == 1 and b.stride(1) == 1
    if out is None:
        out = torch.empty(M, F, dtype=BF16, device=a.device)
    assert out.shape == (M, F) and out.stride(1) == 1
    check(_lib.load().ifab_gemm_swiglu_bf16_2sm(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0), M, F, K,
                                                status_ptr, torch.cuda.current_stream().cuda_stream), "gemm_swiglu")
    return out


def gemm_allreduce(a: torch.Tensor, b: torch.Tensor, fabric, out, *, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-parallel GEMM fused with a two-shot all-reduce over NVLink peer memory:
    ``C = sum_ranks A_r @ B_r.T (+ residual)``; ``A_r`` = ``[M, K_local]``, ``B_r`` = ``[N, K_local]``.

    ``out`` is a :class:`~ironpangu_b200.parallel.fabric.SymmetricTensor` ``[M, N]`` (tile owners store finished rows
    into every rank's buffer). ``residual`` may be ``out.tensor`` itself (in-place residual update). The fabric staging
    area must hold ``ceil(tiles/world)*world * 128*BN*2`` bytes per half and ``tiles*(world+1)`` flag words."""
    import ctypes as C
    M, K = a.shape
    N = b.shape[0]
    y = out.tensor
    assert y.shape == (M, N) and y.dtype == BF16 and y.is_contiguous()
    check(_lib.load().ifab_gemm_allreduce_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.peer_ptrs, y.stride(0),
                                               None if residual is None else residual.data_ptr(),
                                               0 if residual is None else residual.stride(0), M, N, K,
                                               C.byref(fabric.desc), torch.cuda.current_stream().cuda_stream),
          "gemm_allreduce")
    return y


def gemm_reduce_scatter(a: torch.Tensor, b: torch.Tensor, fabric, out: Optional[torch.Tensor] = None, *,
                        residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-parallel GEMM fused with a reduce-scatter over NVLink peer memory: rank ``r`` ends with rows
    ``[r * M / world, (r + 1) * M / world)`` of ``sum_ranks A_r @ B_r.T (+ residual)`` in ``out`` ``[M / world, N]``
    (``residual`` is the matching row shard). ``M / world`` must be a multiple of 128 when ``world > 1``. The sequence-parallel
    counterpart of :func:`gemm_allreduce`; together with :func:`allgather_gemm` it brackets a tensor-parallel block whose
    activations stay sharded by rows."""
    import ctypes as C
    M, K = a.shape
    N = b.shape[0]
    rows = M // fabric.world
    if out is None:
        out = torch.empty(rows, N, dtype=BF16, device=a.device)
    assert out.shape == (rows, N) and out.dtype == BF16 and out.stride(1) == 1
    check(_lib.load().ifab_gemm_reduce_scatter_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0),
                                                    None if residual is None else residual.data_ptr(),
                                                    0 if residual is None else residual.stride(0), M, N, K, C.byref(fabric.desc),
                                                    torch.cuda.current_stream().cuda_stream), "gemm_reduce_scatter")
    return out


class AllGatherGemmState:
    """Per-shape scratch of :func:`allgather_gemm`: flags (symmetric), the local staging matrix and its tile counters."""

    def __init__(self, fabric, rows_local: int, K: int):
        self.flags = fabric.symmetric_empty((8,), torch.int64)
        M = rows_local * fabric.world
        self.staged = torch.empty(M, K, dtype=BF16, device=fabric.device)
        self.tile_count = torch.zeros((M + 127) // 128, dtype=torch.int64, device=fabric.device)
        self.epoch = 0


def allgather_gemm(a_shard, b: torch.Tensor, state: "AllGatherGemmState", fabric, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Column-parallel GEMM fused with the all-gather of its activations: ``C = concat_ranks(A_r) @ B.T``.

    ``a_shard`` is a :class:`~ironpangu_b200.parallel.fabric.SymmetricTensor` ``[rows_local, K]`` (bf16) that every rank
    has just written; remote 128-row tiles are brought over NVLink once, inside the GEMM kernel, while the tiles of the
    local shard are already being multiplied. Alternate two ``a_shard`` buffers between consecutive calls; every rank
    must make the same sequence of calls with the same ``state``."""
    import ctypes as C
    a = a_shard.tensor
    rows_local, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(rows_local * fabric.world, N, dtype=BF16, device=a.device)
    lib = _lib.load()
    fn = lib.ifab_allgather_gemm_bf16
    fn.argtypes = [C.c_void_p, C.c_long, C.c_void_p, C.c_long, C.c_void_p, C.c_long, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                   C.c_void_p, C.c_void_p, C.c_long, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    state.epoch += 1
    check(fn(a_shard.peer_ptrs, a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0), rows_local, N, K, fabric.world,
             fabric.rank, state.flags.peer_ptrs, state.staged.data_ptr(), state.staged.stride(0), state.tile_count.data_ptr(), state.epoch,
             fabric.desc.status, torch.cuda.current_stream().cuda_stream), "allgather_gemm")
    return out

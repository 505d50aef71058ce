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

"""Wrappers of the hybrid-family row kernels (``csrc/kernels/hybrid_ops.cu``): zero-centred RMSNorm, q / k preparation of the
gated attention layer, sigmoid gate, causal conv + SiLU, delta-rule preparation, gated RMSNorm."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import check

BF16 = torch.bfloat16


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


def zc_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, *, groups: int = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = x * rsqrt(mean(x^2) + eps) * (1 + w)`` over each of ``groups`` equal column groups of every row (``w``: bf16 ``[d]``)."""
    rows, n = x.shape
    d = n // groups
    assert n == groups * d and w.numel() == d and w.dtype == BF16
    out = torch.empty(rows, n, dtype=BF16, device=x.device) if out is None else out
    check(_lib.load().ifab_zc_rmsnorm(x.data_ptr(), x.stride(0), w.data_ptr(), eps, out.data_ptr(), out.stride(0), rows, groups, d, _s()), "zc_rmsnorm")
    return out


def qk_prepare(qg: torch.Tensor, kv: torch.Tensor, q_norm: torch.Tensor, k_norm: torch.Tensor, eps: float, *, heads: int, kv_heads: int,
               head_dim: int, qkv: torch.Tensor, gate: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``qg``: ``[T, heads * 2 * hd]`` (per head: query | gate); ``kv``: ``[T, 2 * kv_heads * hd]`` (keys | values). Fills ``qkv``
    ``[T, (heads + 2 * kv_heads) * hd]`` with normalised q, normalised k and v, and ``gate`` ``[T, heads * hd]``."""
    T = qg.shape[0]
    check(_lib.load().ifab_hybrid_qk_prepare(qg.data_ptr(), qg.stride(0), kv.data_ptr(), kv.stride(0), q_norm.data_ptr(), k_norm.data_ptr(), eps,
                                             qkv.data_ptr(), qkv.stride(0), gate.data_ptr(), gate.stride(0), T, heads, kv_heads, head_dim, _s()),
          "hybrid_qk_prepare")
    return qkv, gate


def sigmoid_mul(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, n = a.shape
    out = torch.empty(rows, n, dtype=BF16, device=a.device) if out is None else out
    check(_lib.load().ifab_sigmoid_mul(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0), rows, n, _s()), "sigmoid_mul")
    return out


def conv_silu(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal depthwise convolution + SiLU; ``w`` bf16 ``[C, width]``, ``state`` bf16 ``[slots, C, width - 1]`` (oldest first), updated in
    place; a row at position 0 starts from an empty history."""
    T, C = x.shape
    out = torch.empty(T, C, dtype=BF16, device=x.device) if out is None else out
    check(_lib.load().ifab_conv_silu(x.data_ptr(), x.stride(0), w.data_ptr(), state.data_ptr(), positions.data_ptr(), slots.data_ptr(),
                                     out.data_ptr(), out.stride(0), T, C, w.shape[1], _s()), "conv_silu")
    return out


def delta_prepare(conv: torch.Tensor, ab: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, eps: float, *, heads: int, dim: int,
                  q: torch.Tensor, k: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, positions: Optional[torch.Tensor] = None,
                  slots: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None) -> None:
    """``conv``: ``[T, 3 * heads * dim]`` (q | k | v after the convolution); ``ab``: ``[T, 2 * heads]`` (a | b). Fills L2-normalised
    ``q``, ``k`` (bf16 ``[T, heads, dim]``), the log decay ``g`` and the write strength ``beta`` (f32 ``[T, heads]``). With ``state``
    (f32 ``[slots, heads, dim, dim]``), a row at position 0 clears the state of its slot: a new sequence starts empty."""
    T = conv.shape[0]
    check(_lib.load().ifab_delta_prepare(conv.data_ptr(), conv.stride(0), ab.data_ptr(), ab.stride(0), a_log.data_ptr(), dt_bias.data_ptr(), eps,
                                         q.data_ptr(), k.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                         None if state is None else positions.data_ptr(), None if state is None else slots.data_ptr(),
                                         None if state is None else state.data_ptr(), T, heads, dim, _s()), "delta_prepare")


def gated_rmsnorm(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = rms_norm(x) * w * silu(z)`` per head; ``x`` bf16 ``[T, H, d]`` contiguous, ``z`` rows of ``H * d`` columns, ``w`` f32 ``[d]``."""
    T, H, d = x.shape
    assert x.is_contiguous() and w.dtype == torch.float32
    out = torch.empty(T, H * d, dtype=BF16, device=x.device) if out is None else out
    check(_lib.load().ifab_gated_rmsnorm(x.data_ptr(), z.data_ptr(), z.stride(0), w.data_ptr(), eps, out.data_ptr(), out.stride(0), T, H, d, _s()),
          "gated_rmsnorm")
    return out

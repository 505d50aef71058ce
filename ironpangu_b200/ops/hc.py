"""Wrappers of the hyper-connection / hybrid-model kernels (``csrc/kernels/hc_ops.cu``): MoME causal conv, mHC pre / post,
gated delta rule, sparse-attention indexer."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import check

BF16 = torch.bfloat16


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


def mome(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, *,
         c_offset: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = x + [pos + 1 >= taps] * causal_conv(x)``; ``w`` f32 ``[C_total, taps]``, ``state`` bf16 ``[slots, taps-1, C]``."""
    T, Cn = x.shape
    taps = w.shape[-1]
    out = torch.empty(T, Cn, dtype=BF16, device=x.device) if out is None else out
    check(_lib.load().ifab_mome(x.data_ptr(), x.stride(0), w.data_ptr(), state.data_ptr(), positions.data_ptr(), slots.data_ptr(),
                                out.data_ptr(), out.stride(0), T, Cn, taps, c_offset, _s()), "mome")
    return out


def mhc_pre(X: torch.Tensor, phi: torch.Tensor, gamma: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor, *, sinkhorn: int = 20,
            eps: float = 1e-6, out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
            tickets_ptr: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns ``(y bf16 [T, W], post f32 [T, S], comb f32 [T, S, S])`` for residual streams ``X`` bf16 ``[T, S, W]``; ``out``
    names three contiguous tensors of those shapes to write into. ``tickets_ptr``: the address of ``T`` zeroed 32-bit words
    (left zero again) - the step then runs as one launch (the CTA that finishes a token's sums last runs its tail)."""
    T, S, W = X.shape
    if out is not None:
        y, post, comb = out
        assert y.is_contiguous() and post.is_contiguous() and comb.is_contiguous() and X.is_contiguous()
    else:
        y = torch.empty(T, W, dtype=BF16, device=X.device)
        post = torch.empty(T, S, dtype=torch.float32, device=X.device)
        comb = torch.empty(T, S, S, dtype=torch.float32, device=X.device)
    if tickets_ptr:
        check(_lib.load().ifab_mhc_pre_ticketed(X.data_ptr(), phi.data_ptr(), gamma.data_ptr(), alpha.data_ptr(), beta.data_ptr(), y.data_ptr(),
                                                post.data_ptr(), comb.data_ptr(), T, S, W, sinkhorn, eps, tickets_ptr, _s()), "mhc_pre")
        return y, post, comb
    check(_lib.load().ifab_mhc_pre(X.data_ptr(), phi.data_ptr(), gamma.data_ptr(), alpha.data_ptr(), beta.data_ptr(), y.data_ptr(),
                                   post.data_ptr(), comb.data_ptr(), T, S, W, sinkhorn, eps, _s()), "mhc_pre")
    return y, post, comb


def mhc_post(X: torch.Tensor, branch: torch.Tensor, post: torch.Tensor, comb: torch.Tensor, out: Optional[torch.Tensor] = None,
             norm_w: Optional[torch.Tensor] = None, eps: float = 1e-5) -> torch.Tensor:
    """``Y[t, i] = post[t, i] * branch[t] + sum_k comb[t, k, i] * X[t, k]``; with ``norm_w`` the branch is RMS-normalised (gain
    ``norm_w``, rounded to bf16) inside the same launch."""
    T, S, W = X.shape
    Y = torch.empty(T, S, W, dtype=BF16, device=X.device) if out is None else out
    assert Y.is_contiguous() and X.is_contiguous()
    if norm_w is not None:
        check(_lib.load().ifab_mhc_post_norm(X.data_ptr(), branch.data_ptr(), branch.stride(0), norm_w.data_ptr(), eps, post.data_ptr(), comb.data_ptr(),
                                             Y.data_ptr(), T, S, W, _s()), "mhc_post_norm")
        return Y
    check(_lib.load().ifab_mhc_post(X.data_ptr(), branch.data_ptr(), branch.stride(0), post.data_ptr(), comb.data_ptr(), Y.data_ptr(), T, S, W,
                                    _s()), "mhc_post")
    return Y


def delta_rule_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
                      slots: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One gated delta-rule step per row; ``state`` f32 ``[slots, H, dk, dv]`` is updated in place. Rows of one launch must
    belong to different sequence slots (rows of one sequence go in separate launches, in order)."""
    rows, H, dk = q.shape
    dv = v.shape[-1]
    out = torch.empty(rows, H, dv, dtype=BF16, device=q.device) if out is None else out
    check(_lib.load().ifab_delta_rule_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), state.data_ptr(),
                                             slots.data_ptr(), out.data_ptr(), rows, H, dk, dv, _s()), "delta_rule_decode")
    return out


def sparse_index(q: torch.Tensor, w: torch.Tensor, keys: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                 page_table: torch.Tensor, *, ctx: int, topk: int, status_ptr: Optional[int] = None, scores: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, key_scales: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Top-``topk`` key positions per query by ``sum_h w_h * relu(q_h . key)``; ``keys`` paged bf16 ``[pages, page_tokens, dim]``.
    Positions come out ascending, padded with -1; ``scores`` (f32 ``[T, ctx]``) is scratch. With ``key_scales`` (half
    ``[pages, page_tokens]``) the keys are int8 rows with one scale each and the query heads are quantised the same way."""
    T, H, dim = q.shape
    num_pages, page_tokens, _ = keys.shape
    scores = torch.empty(T, ctx, dtype=torch.float32, device=q.device) if scores is None else scores
    out = torch.empty(T, topk, dtype=torch.int32, device=q.device) if out is None else out
    assert scores.is_contiguous() and scores.shape[1] == ctx and out.is_contiguous() and w.dtype in (torch.float32, BF16) and w.stride(1) == 1
    if key_scales is not None:
        assert keys.dtype == torch.int8 and key_scales.dtype == torch.float16 and key_scales.is_contiguous()
    # the gains may be the bf16 rows of a projection, read where they lie (no f32 copy)
    check(_lib.load().ifab_sparse_index_general(q.data_ptr(), w.data_ptr(), w.stride(0), int(w.dtype == BF16), keys.data_ptr(),
                                                None if key_scales is None else key_scales.data_ptr(), positions.data_ptr(), slots.data_ptr(),
                                                page_table.data_ptr(), page_table.shape[1], page_tokens, num_pages, scores.data_ptr(), ctx, T, H,
                                                dim, topk, out.data_ptr(), status_ptr, _s()), "sparse_index")
    return out


def rope_prefix(x: torch.Tensor, positions: torch.Tensor, *, heads: int, head_dim: int, rotary_dim: int, theta: float,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Half-rotation RoPE over the first ``rotary_dim`` columns of every head of ``x`` (``[T, heads * head_dim]``)."""
    T = x.shape[0]
    out = torch.empty(T, heads * head_dim, dtype=BF16, device=x.device) if out is None else out
    check(_lib.load().ifab_rope_prefix(x.data_ptr(), x.stride(0), positions.data_ptr(), out.data_ptr(), out.stride(0), T, heads, head_dim, rotary_dim, theta,
                                       _s()), "rope_prefix")
    return out


def index_cache_append(key: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                       status_ptr: Optional[int] = None, scales: Optional[torch.Tensor] = None) -> None:
    """Index keys ``[T, dim]`` of the step's rows into the paged index cache ``[pages, page_tokens, dim]`` (bf16), or - with
    ``scales`` (half ``[pages, page_tokens]``) - into an int8 cache with one half-precision scale per row."""
    T, dim = key.shape
    if scales is not None:
        assert cache.dtype == torch.int8 and scales.dtype == torch.float16
        check(_lib.load().ifab_index_cache_append_q8(key.data_ptr(), key.stride(0), positions.data_ptr(), slots.data_ptr(), page_table.data_ptr(),
                                                     page_table.shape[1], cache.shape[1], cache.shape[0], cache.data_ptr(), scales.data_ptr(), T, dim,
                                                     status_ptr, _s()), "index_cache_append_q8")
        return
    check(_lib.load().ifab_index_cache_append(key.data_ptr(), key.stride(0), positions.data_ptr(), slots.data_ptr(), page_table.data_ptr(),
                                              page_table.shape[1], cache.shape[1], cache.shape[0], cache.data_ptr(), T, dim, status_ptr, _s()),
          "index_cache_append")


def add_rows(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, n = a.shape
    out = torch.empty(rows, n, dtype=BF16, device=a.device) if out is None else out
    check(_lib.load().ifab_add_rows(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0), rows, n, _s()), "add_rows")
    return out


def swiglu_pair(gate: torch.Tensor, up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gate) * up`` for two bf16 ``[rows, n]`` projections (row-strided views are fine)."""
    rows, n = gate.shape
    out = torch.empty(rows, n, dtype=BF16, device=gate.device) if out is None else out
    check(_lib.load().ifab_swiglu_pair(gate.data_ptr(), gate.stride(0), up.data_ptr(), up.stride(0), out.data_ptr(), out.stride(0), rows, n, _s()),
          "swiglu_pair")
    return out

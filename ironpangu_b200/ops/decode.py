"""Python entry points of the decode-path kernels (thin wrappers over the C ABI).

All functions launch on the current CUDA stream, never synchronise and never fall back to PyTorch
math; outputs can be passed in (``out=``) so that an engine can run allocation-free under CUDA
graph capture.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import check

BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _rows(x: torch.Tensor) -> int:
    assert x.dim() == 2 and x.stride(1) == 1
    return x.stride(0)


def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None,
              status_ptr: Optional[int] = None) -> torch.Tensor:
    T, (V, D) = ids.numel(), table.shape
    assert ids.dtype == torch.int32 and table.dtype == BF16 and table.is_contiguous()
    if out is None:
        out = torch.empty(T, D, dtype=BF16, device=table.device)
    check(_lib.load().ifab_embedding_bf16(ids.data_ptr(), table.data_ptr(), out.data_ptr(), T, D, V, status_ptr,
                                          _stream()), "embedding")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5, zero_centered: bool = False,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, D = x.shape
    if out is None:
        out = torch.empty(T, D, dtype=BF16, device=x.device)
    check(_lib.load().ifab_rmsnorm_bf16(x.data_ptr(), _rows(x), w.data_ptr(), out.data_ptr(), _rows(out), T, D, eps,
                                        int(zero_centered), _stream()), "rmsnorm")
    return out


def swiglu_rows(gu: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gu[:, :F]) * gu[:, F:]`` for a gate/up projection ``[T, 2F]`` (gate columns first)."""
    T, F2 = gu.shape
    F = F2 // 2
    if out is None:
        out = torch.empty(T, F, dtype=BF16, device=gu.device)
    check(_lib.load().ifab_swiglu_rows_bf16(gu.data_ptr(), _rows(gu), out.data_ptr(), _rows(out), T, F, _stream()), "swiglu_rows")
    return out


def gemv(x: torch.Tensor, w: torch.Tensor, *, norm_w: Optional[torch.Tensor] = None, eps: float = 1e-5,
         zero_centered: bool = False, residual: Optional[torch.Tensor] = None, swiglu: bool = False,
         out_f32: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = act(norm(x) @ w.T) (+ residual)`` for a few tokens (decode).

    ``w`` is ``[N, K]`` (or ``[2N, K]`` = gate rows then up rows when ``swiglu``). ``norm_w`` fuses an
    RMSNorm of ``x`` into the prologue."""
    T, K = x.shape
    rows = w.shape[0]
    assert w.shape[1] == K and w.is_contiguous() and w.dtype == BF16 and x.dtype == BF16
    N = rows // 2 if swiglu else rows
    if out is None:
        out = torch.empty(T, N, dtype=torch.float32 if out_f32 else BF16, device=x.device)
    check(_lib.load().ifab_gemv_bf16(x.data_ptr(), _rows(x), w.data_ptr(), _ptr(norm_w), eps, int(zero_centered),
                                     _ptr(residual), _rows(residual) if residual is not None else 0, out.data_ptr(),
                                     _rows(out), int(out.dtype == torch.float32), T, N, K, int(swiglu), _stream()), "gemv")
    return out


def gemv_allreduce(x: torch.Tensor, w: torch.Tensor, fabric, *, residual: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None, out_f32: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-parallel linear fused with a one-shot all-reduce: ``y = sum_r x_r @ w_r.T (+ residual)``."""
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and w.is_contiguous()
    if out is None:
        out = torch.empty(T, N, dtype=BF16, device=x.device)
    check(_lib.load().ifab_gemv_allreduce_bf16(x.data_ptr(), _rows(x), w.data_ptr(), _ptr(residual),
                                               _rows(residual) if residual is not None else 0, out.data_ptr(),
                                               _rows(out), _ptr(out_f32), T, N, K, C.byref(fabric.desc), _stream()),
          "gemv_allreduce")
    return out


def router_topk(x: torch.Tensor, w_router: torch.Tensor, topk: int, *, norm_w: Optional[torch.Tensor] = None,
                eps: float = 1e-5, bias: Optional[torch.Tensor] = None, scoring: str = "softmax", renorm: bool = True,
                scale: float = 1.0, ticket_ptr: int = 0, logits: Optional[torch.Tensor] = None,
                ids: Optional[torch.Tensor] = None, wts: Optional[torch.Tensor] = None, xn: Optional[torch.Tensor] = None):
    """f32 router projection + top-k selection in one launch. Returns (ids int32 [T,k], weights f32 [T,k], logits).
    ``xn`` (bf16 ``[T, D]``) receives the normalised rows, which the expert kernels can then take as they are."""
    T, D = x.shape
    E = w_router.shape[0]
    assert w_router.dtype == torch.float32 and w_router.is_contiguous()
    dev = x.device
    logits = logits if logits is not None else torch.empty(T, E, dtype=torch.float32, device=dev)
    ids = ids if ids is not None else torch.empty(T, topk, dtype=torch.int32, device=dev)
    wts = wts if wts is not None else torch.empty(T, topk, dtype=torch.float32, device=dev)
    mode = {"softmax": 0, "sigmoid_bias_group_topk": 1}[scoring]
    check(_lib.load().ifab_router_topk(x.data_ptr(), _rows(x), _ptr(norm_w), eps, w_router.data_ptr(), _ptr(bias),
                                       logits.data_ptr(), ids.data_ptr(), wts.data_ptr(), T, D, E, topk, mode,
                                       int(renorm), scale, ticket_ptr, _ptr(xn), 0 if xn is None else _rows(xn), _stream()), "router_topk")
    return ids, wts, logits


def moe_gate_up(x: torch.Tensor, ids: torch.Tensor, w_gu: torch.Tensor, e0: int, *,
                norm_w: Optional[torch.Tensor] = None, eps: float = 1e-5, w_shared_gu: Optional[torch.Tensor] = None,
                act: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gate/up projections + SwiGLU of the routes owned by this rank (and of the shared-expert shard).

    ``w_gu``: ``[E_local, 2F, D]``; ``act``: ``[T, topk+1, F]`` (slot ``topk`` is the shared expert)."""
    T, D = x.shape
    topk = ids.shape[1]
    e_local, twoF, _ = w_gu.shape
    F = twoF // 2
    Fs = 0 if w_shared_gu is None else w_shared_gu.shape[0] // 2
    if act is None:
        act = torch.zeros(T, topk + 1, F, dtype=BF16, device=x.device)
    check(_lib.load().ifab_moe_gate_up_decode(x.data_ptr(), _rows(x), _ptr(norm_w), eps, ids.data_ptr(), T, D, F, topk,
                                              e0, e_local, w_gu.data_ptr(), _ptr(w_shared_gu), Fs, act.data_ptr(),
                                              _stream()), "moe_gate_up")
    return act


def moe_down_allreduce(act: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_down: torch.Tensor, e0: int, fabric,
                       *, w_shared_down: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Score-weighted sum of the local experts' down projections (+ shared shard) fused with the all-reduce."""
    T, slots, F = act.shape
    topk = slots - 1
    e_local, D, _ = w_down.shape
    Fs = 0 if w_shared_down is None else w_shared_down.shape[1]
    if out is None:
        out = torch.empty(T, D, dtype=BF16, device=act.device)
    check(_lib.load().ifab_moe_down_allreduce_decode(act.data_ptr(), ids.data_ptr(), wts.data_ptr(), T, D, F, topk, e0,
                                                     e_local, w_down.data_ptr(), _ptr(w_shared_down), Fs,
                                                     _ptr(residual), _rows(residual) if residual is not None else 0,
                                                     out.data_ptr(), _rows(out), C.byref(fabric.desc), _stream()),
          "moe_down_allreduce")
    return out


def moe_block_sync_words(T: int, E: int) -> int:
    return 4 + 2 * T * E


def moe_block(x: torch.Tensor, w_router: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, e0: int, topk: int, fabric, *,
              sync: torch.Tensor, norm_w: Optional[torch.Tensor] = None, eps: float = 1e-5, bias: Optional[torch.Tensor] = None,
              scoring: str = "softmax", renorm: bool = True, scale: float = 1.0, w_shared_gu: Optional[torch.Tensor] = None,
              w_shared_down: Optional[torch.Tensor] = None, logits: Optional[torch.Tensor] = None,
              ids: Optional[torch.Tensor] = None, wts: Optional[torch.Tensor] = None, act: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The MoE half of a decode layer in one launch (one or two rows): router + top-k, shared and routed gate/up with SwiGLU,
    down projections, score-weighted sum and the fused all-reduce; ``out = x + reduced`` (``out`` may be ``x``).
    Bit-identical to ``router_topk`` -> ``moe_gate_up`` -> ``moe_down_allreduce``. ``sync``: zeroed int32 words that only
    this op uses (in-grid signals and tagged router logits): at least ``moe_block_sync_words(T, E)`` of them."""
    T, D = x.shape
    E = w_router.shape[0]
    e_local, twoF, _ = w_gu.shape
    F = twoF // 2
    Fs = 0 if w_shared_gu is None else w_shared_gu.shape[0] // 2
    assert T <= 2 and w_router.dtype == torch.float32 and w_router.is_contiguous() and sync.numel() >= moe_block_sync_words(T, E) and sync.dtype == torch.int32
    dev = x.device
    logits = logits if logits is not None else torch.empty(T, E, dtype=torch.float32, device=dev)
    ids = ids if ids is not None else torch.empty(T, topk, dtype=torch.int32, device=dev)
    wts = wts if wts is not None else torch.empty(T, topk, dtype=torch.float32, device=dev)
    act = act if act is not None else torch.zeros(T, topk + 1, F, dtype=BF16, device=dev)
    out = out if out is not None else torch.empty(T, D, dtype=BF16, device=dev)
    mode = {"softmax": 0, "sigmoid_bias_group_topk": 1}[scoring]
    check(_lib.load().ifab_moe_block_decode(x.data_ptr(), _rows(x), _ptr(norm_w), eps, w_router.data_ptr(), _ptr(bias), E, topk, mode,
                                            int(renorm), scale, w_gu.data_ptr(), _ptr(w_shared_gu), w_down.data_ptr(),
                                            _ptr(w_shared_down), T, D, F, Fs, e0, e_local, logits.data_ptr(), ids.data_ptr(),
                                            wts.data_ptr(), act.data_ptr(), out.data_ptr(), _rows(out), sync.data_ptr(),
                                            C.byref(fabric.desc), _stream()), "moe_block")
    return out


def mla_head_decode(qkv: torch.Tensor, q_norm: torch.Tensor, kv_norm: torch.Tensor, w_qb: torch.Tensor, w_kvb: torch.Tensor,
                    cache: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor, *, q_lora: int,
                    nope: int, scale: float, eps: float = 1e-5, theta: float = 10000.0, window: int = 0,
                    sinks: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, status_ptr=None,
                    prefetch=()) -> torch.Tensor:
    """The attention half of an MLA decode layer in one launch (a cluster of 8 CTAs per head): cache write, q_b, absorb,
    attention over the paged latent cache and value up-projection. ``qkv``: ``[T, q_lora + 576]`` output of the qkv_a
    linear; ``w_qb``: ``[H * (nope + 64), q_lora]``; ``w_kvb``: ``[H, nope + vdim, 512]``; returns ``[T, H * vdim]``.
    ``prefetch``: up to three contiguous tensors (weights of the layer's later kernels) the kernel requests into L2 while it runs."""
    T = qkv.shape[0]
    H, nv, latent = w_kvb.shape
    vdim = nv - nope
    assert latent == 512 and qkv.shape[1] == q_lora + 576 and cache.dtype == BF16
    if out is None:
        out = torch.empty(T, H * vdim, dtype=BF16, device=qkv.device)
    pf = [(t.data_ptr(), t.numel() * t.element_size()) for t in prefetch if t is not None][:3]
    pf += [(None, 0)] * (3 - len(pf))
    check(_lib.load().ifab_mla_head_decode_pf(qkv.data_ptr(), _rows(qkv), q_norm.data_ptr(), kv_norm.data_ptr(), eps, theta, w_qb.data_ptr(),
                                              w_kvb.data_ptr(), cache.data_ptr(), positions.data_ptr(), slots.data_ptr(),
                                              page_table.data_ptr(), page_table.shape[1], cache.shape[1], cache.shape[0], _ptr(sinks),
                                              0 if sinks is None else sinks.shape[0], window, scale, T, H, q_lora, nope, vdim,
                                              out.data_ptr(), _rows(out), status_ptr, pf[0][0], pf[0][1], pf[1][0], pf[1][1], pf[2][0], pf[2][1],
                                              _stream()), "mla_head_decode")
    return out


def quantize_fp8_block(w: torch.Tensor):
    """Block-scaled fp8 (e4m3) form of a bf16 matrix ``[..., rows, K]``: ``(q uint8 [..., rows, K], scales f32 [..., rows,
    ceil(K/128)])`` with ``w ~= fp8(q) * scale`` per 1 x 128 block of a row."""
    assert w.dtype == BF16 and w.is_contiguous()
    K = w.shape[-1]
    rows = w.numel() // K
    q = torch.empty(w.shape, dtype=torch.uint8, device=w.device)
    scales = torch.empty(*w.shape[:-1], (K + 127) // 128, dtype=torch.float32, device=w.device)
    check(_lib.load().ifab_quantize_fp8_block(w.data_ptr(), K, rows, K, q.data_ptr(), scales.data_ptr(), _stream()), "quantize_fp8_block")
    return q, scales


def dequantize_fp8_block(qs, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``bf16(fp8(q) * scale)`` of a ``(q, scales)`` pair from :func:`quantize_fp8_block`; ``out`` bf16 of ``q``'s shape."""
    q, scales = qs
    K = q.shape[-1]
    rows = q.numel() // K
    if out is None:
        out = torch.empty(q.shape, dtype=BF16, device=q.device)
    assert out.is_contiguous() and out.numel() == q.numel() and q.is_contiguous() and scales.is_contiguous()
    check(_lib.load().ifab_dequantize_fp8_block(q.data_ptr(), scales.data_ptr(), rows, K, out.data_ptr(), _stream()), "dequantize_fp8_block")
    return out


def moe_gate_up_fp8(x: torch.Tensor, ids: torch.Tensor, w_gu, e0: int, *, norm_w: Optional[torch.Tensor] = None, eps: float = 1e-5,
                    w_shared_gu=None, act: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``moe_gate_up`` over block-scaled fp8 weights: ``w_gu`` and ``w_shared_gu`` are ``(q, scales)`` pairs."""
    T, D = x.shape
    topk = ids.shape[1]
    q, sc = w_gu
    e_local, twoF, _ = q.shape
    F = twoF // 2
    sq, ss = w_shared_gu if w_shared_gu is not None else (None, None)
    Fs = 0 if sq is None else sq.shape[0] // 2
    if act is None:
        act = torch.zeros(T, topk + 1, F, dtype=BF16, device=x.device)
    check(_lib.load().ifab_moe_gate_up_decode_fp8(x.data_ptr(), _rows(x), _ptr(norm_w), eps, ids.data_ptr(), T, D, F, topk, e0, e_local,
                                                  q.data_ptr(), sc.data_ptr(), _ptr(sq), _ptr(ss), Fs, act.data_ptr(), _stream()),
          "moe_gate_up_fp8")
    return act


def moe_down_allreduce_fp8(act: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_down, e0: int, fabric, *, w_shared_down=None,
                           residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``moe_down_allreduce`` over block-scaled fp8 weights (``(q, scales)`` pairs)."""
    T, slots, F = act.shape
    topk = slots - 1
    q, sc = w_down
    e_local, D, _ = q.shape
    sq, ss = w_shared_down if w_shared_down is not None else (None, None)
    Fs = 0 if sq is None else sq.shape[1]
    if out is None:
        out = torch.empty(T, D, dtype=BF16, device=act.device)
    check(_lib.load().ifab_moe_down_allreduce_decode_fp8(act.data_ptr(), ids.data_ptr(), wts.data_ptr(), T, D, F, topk, e0, e_local,
                                                         q.data_ptr(), sc.data_ptr(), _ptr(sq), _ptr(ss), Fs, _ptr(residual),
                                                         _rows(residual) if residual is not None else 0, out.data_ptr(), _rows(out),
                                                         C.byref(fabric.desc), _stream()), "moe_down_allreduce_fp8")
    return out


def lm_head_argmax(x: torch.Tensor, w: torch.Tensor, fabric, *, norm_w: Optional[torch.Tensor] = None,
                   eps: float = 1e-5, vocab_offset: int = 0, partial: Optional[torch.Tensor] = None,
                   logits: Optional[torch.Tensor] = None, out_ids: Optional[torch.Tensor] = None,
                   out_vals: Optional[torch.Tensor] = None):
    """Vocabulary-sharded lm_head + greedy token selection (cross-rank exchange inside the kernel)."""
    T, K = x.shape
    V = w.shape[0]
    dev = x.device
    if partial is None:
        partial = torch.empty(((V + 7) // 8) * 8 * 2, dtype=torch.float32, device=dev)
    if out_ids is None:
        out_ids = torch.empty(T, dtype=torch.int32, device=dev)
    check(_lib.load().ifab_lm_head_argmax(x.data_ptr(), _rows(x), _ptr(norm_w), eps, w.data_ptr(), _ptr(logits), T, V, K,
                                          vocab_offset, partial.data_ptr(), partial.numel() * partial.element_size(),
                                          out_ids.data_ptr(), _ptr(out_vals), C.byref(fabric.desc), _stream()),
          "lm_head_argmax")
    return out_ids


def mla_kv_write(kv: torch.Tensor, norm_w: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                 page_table: torch.Tensor, cache: torch.Tensor, *, latent: int, rope: int, eps: float, theta: float,
                 status_ptr: Optional[int] = None) -> None:
    """RMSNorm(latent) + RoPE(k_pe) + scatter into the paged latent cache ``[pages, page_tokens, latent+rope]``."""
    T = kv.shape[0]
    num_pages, page_tokens, _ = cache.shape
    check(_lib.load().ifab_mla_kv_write(kv.data_ptr(), _rows(kv), norm_w.data_ptr(), eps, theta, positions.data_ptr(),
                                        slots.data_ptr(), page_table.data_ptr(), page_table.shape[1], page_tokens,
                                        cache.data_ptr(), num_pages, T, latent, rope, status_ptr, _stream()),
          "mla_kv_write")


def mla_kv_write_split(latent_rows: torch.Tensor, rope_rows: torch.Tensor, norm_w: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                       page_table: torch.Tensor, cache: torch.Tensor, *, eps: float, theta: float, status_ptr: Optional[int] = None) -> None:
    """:func:`mla_kv_write` for latent and rotary columns that live in different rows (``[T, latent]`` and ``[T, rope]`` views)."""
    T, latent = latent_rows.shape
    num_pages, page_tokens, _ = cache.shape
    check(_lib.load().ifab_mla_kv_write_split(latent_rows.data_ptr(), _rows(latent_rows), rope_rows.data_ptr(), _rows(rope_rows), norm_w.data_ptr(),
                                              eps, theta, positions.data_ptr(), slots.data_ptr(), page_table.data_ptr(), page_table.shape[1],
                                              page_tokens, cache.data_ptr(), num_pages, T, latent, rope_rows.shape[1], status_ptr, _stream()),
          "mla_kv_write_split")


def mla_kv_write_q8(kv: torch.Tensor, norm_w: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                    page_table: torch.Tensor, cache: torch.Tensor, *, eps: float, theta: float,
                    status_ptr: Optional[int] = None) -> None:
    """RMSNorm(latent) + RoPE(k_pe) + per-128-column int8 quantisation into the packed cache ``uint8 [pages, page_tokens, 656]``."""
    T = kv.shape[0]
    num_pages, page_tokens, row = cache.shape
    assert cache.dtype == torch.uint8 and row == 656
    check(_lib.load().ifab_mla_kv_write_q8(kv.data_ptr(), _rows(kv), norm_w.data_ptr(), eps, theta, positions.data_ptr(),
                                           slots.data_ptr(), page_table.data_ptr(), page_table.shape[1], page_tokens, cache.data_ptr(),
                                           num_pages, T, status_ptr, _stream()), "mla_kv_write_q8")


def mla_kv_write_q8_split(latent_rows: torch.Tensor, rope_rows: torch.Tensor, norm_w: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                          page_table: torch.Tensor, cache: torch.Tensor, *, eps: float, theta: float, status_ptr: Optional[int] = None) -> None:
    """:func:`mla_kv_write_q8` for latent and rotary columns that live in different rows."""
    T = latent_rows.shape[0]
    num_pages, page_tokens, row = cache.shape
    assert cache.dtype == torch.uint8 and row == 656 and latent_rows.shape[1] == 512 and rope_rows.shape[1] == 64
    check(_lib.load().ifab_mla_kv_write_q8_split(latent_rows.data_ptr(), _rows(latent_rows), rope_rows.data_ptr(), _rows(rope_rows), norm_w.data_ptr(),
                                                 eps, theta, positions.data_ptr(), slots.data_ptr(), page_table.data_ptr(), page_table.shape[1],
                                                 page_tokens, cache.data_ptr(), num_pages, T, status_ptr, _stream()), "mla_kv_write_q8_split")


def kv_dequantize_q8(cache: torch.Tensor) -> torch.Tensor:
    """Packed int8 cache -> bf16 ``[pages, page_tokens, 576]`` (test utility)."""
    num_pages, page_tokens, _ = cache.shape
    out = torch.empty(num_pages, page_tokens, 576, dtype=BF16, device=cache.device)
    check(_lib.load().ifab_kv_dequantize_q8(cache.data_ptr(), out.data_ptr(), num_pages * page_tokens, _stream()), "kv_dequantize_q8")
    return out


def quantize_int8(x: torch.Tensor, group_cols: Optional[int] = None):
    """Symmetric int8 quantisation of ``[T, K]`` bf16 (ties away from zero): per row, or per ``group_cols`` columns.
    Returns ``(q int8 [T, K], scales f32 [T, groups])``."""
    T, Kc = x.shape
    gc = Kc if group_cols is None else group_cols
    groups = (Kc + gc - 1) // gc
    q = torch.empty(T, Kc, dtype=torch.int8, device=x.device)
    scales = torch.empty(T, groups, dtype=torch.float32, device=x.device)
    check(_lib.load().ifab_quantize_int8(x.data_ptr(), _rows(x), q.data_ptr(), Kc, scales.data_ptr(), groups, T, Kc, gc, _stream()),
          "quantize_int8")
    return q, scales


def mla_q_absorb(q: torch.Tensor, w_kvb: torch.Tensor, positions: torch.Tensor, *, nope: int, rope: int, theta: float,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``q_lat[t,h] = [q_nope[t,h] @ W_UK[h] | RoPE(q_rope[t,h])]`` with ``w_kvb`` = ``[H, nope+vdim, latent]``."""
    T = q.shape[0]
    H, rows, latent = w_kvb.shape
    vdim = rows - nope
    if out is None:
        out = torch.empty(T, H, latent + rope, dtype=BF16, device=q.device)
    check(_lib.load().ifab_mla_q_absorb(q.data_ptr(), _rows(q), w_kvb.data_ptr(), theta, positions.data_ptr(),
                                        out.data_ptr(), T, H, nope, rope, latent, vdim, _stream()), "mla_q_absorb")
    return out


def mla_decode_attention(q_lat: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                         page_table: torch.Tensor, w_kvb: torch.Tensor, *, nope: int, scale: float, window: int = 0,
                         sinks: Optional[torch.Tensor] = None, keys_per_split: int = 64, max_splits: int = 16,
                         scratch: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                         status_ptr: Optional[int] = None, packed: bool = False, indices: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Split-KV paged MLA attention + value up-projection. Returns ``[T, H*vdim]`` bf16. With ``packed`` the cache
    holds 656-byte int8 rows (``uint8 [pages, page_tokens, 656]``, written by :func:`mla_kv_write_q8`). ``indices`` (int32
    ``[T, k]``, ascending key positions padded with -1: the sparse indexer's selection) restricts every row to those keys."""
    T, H, row = q_lat.shape
    num_pages, page_tokens, _ = cache.shape
    latent = w_kvb.shape[2]
    rope = row - latent
    vdim = w_kvb.shape[1] - nope
    if scratch is None:
        scratch = torch.empty(T * H * max_splits * (latent + 2), dtype=torch.float32, device=q_lat.device)
    if out is None:
        out = torch.empty(T, H * vdim, dtype=BF16, device=q_lat.device)
    assert indices is None or (indices.dtype == torch.int32 and indices.is_contiguous() and indices.shape[0] == T)
    check(_lib.load().ifab_mla_decode_attention_indexed(
        q_lat.data_ptr(), cache.data_ptr(), positions.data_ptr(), slots.data_ptr(), page_table.data_ptr(),
        page_table.shape[1], page_tokens, num_pages, _ptr(sinks), 0 if sinks is None else sinks.shape[0], window, scale,
        T, H, latent, -rope if packed else rope, keys_per_split, max_splits, scratch.data_ptr(), scratch.numel() * 4, w_kvb.data_ptr(), nope,
        vdim, out.data_ptr(), _rows(out), status_ptr, _ptr(indices), 0 if indices is None else indices.shape[1], _stream()), "mla_decode_attention")
    return out


def gqa_rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                      k_cache: torch.Tensor, v_cache: torch.Tensor, *, heads: int, kv_heads: int, head_dim: int,
                      rotary_dim: Optional[int] = None, theta: float = 1e6, status_ptr: Optional[int] = None) -> None:
    """Rotate q and k of ``qkv`` = ``[T, (heads + 2*kv_heads) * head_dim]`` in place and append k / v to the paged caches
    ``[pages, page_tokens, kv_heads, head_dim]``."""
    T = qkv.shape[0]
    num_pages, page_tokens = k_cache.shape[0], k_cache.shape[1]
    check(_lib.load().ifab_gqa_rope_kv_write(qkv.data_ptr(), _rows(qkv), positions.data_ptr(), slots.data_ptr(),
                                             page_table.data_ptr(), page_table.shape[1], page_tokens, k_cache.data_ptr(),
                                             v_cache.data_ptr(), num_pages, T, heads, kv_heads, head_dim,
                                             head_dim if rotary_dim is None else rotary_dim, theta, status_ptr, _stream()), "gqa_rope_kv_write")


def gqa_decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor,
                         slots: torch.Tensor, page_table: torch.Tensor, *, heads: int, kv_heads: int, head_dim: int,
                         scale: float, keys_per_split: int = 64, max_splits: int = 16, scratch: Optional[torch.Tensor] = None,
                         out: Optional[torch.Tensor] = None, status_ptr: Optional[int] = None) -> torch.Tensor:
    """Split-KV paged GQA attention; ``q`` is ``[T, >= heads*head_dim]`` (the q columns of the qkv buffer)."""
    T = q.shape[0]
    num_pages, page_tokens = k_cache.shape[0], k_cache.shape[1]
    if scratch is None:
        scratch = torch.empty(T * heads * max_splits * (head_dim + 2), dtype=torch.float32, device=q.device)
    if out is None:
        out = torch.empty(T, heads * head_dim, dtype=BF16, device=q.device)
    check(_lib.load().ifab_gqa_decode_attention(q.data_ptr(), _rows(q), k_cache.data_ptr(), v_cache.data_ptr(),
                                                positions.data_ptr(), slots.data_ptr(), page_table.data_ptr(),
                                                page_table.shape[1], page_tokens, num_pages, scale, T, heads, kv_heads,
                                                head_dim, keys_per_split, max_splits, scratch.data_ptr(), scratch.numel() * 4,
                                                out.data_ptr(), _rows(out), status_ptr, _stream()), "gqa_decode_attention")
    return out


def sample_topk(logits: torch.Tensor, fabric, *, top_k: int = 50, inv_temperature: Optional[torch.Tensor] = None,
                top_p: Optional[torch.Tensor] = None, min_p: Optional[torch.Tensor] = None,
                counts: Optional[torch.Tensor] = None, penalties: Optional[torch.Tensor] = None,
                seeds: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None, vocab_offset: int = 0,
                scratch: Optional[torch.Tensor] = None, out_ids: Optional[torch.Tensor] = None,
                out_probs: Optional[torch.Tensor] = None, top_k_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exact top-k / min-p / top-p sampling on vocabulary-sharded f32 logits ``[T, V_local]`` (cross-rank candidate
    exchange inside the kernel). ``seeds``/``counters`` are int64 ``[T]``; counters advance on the device.
    ``top_k_rows`` (int32 ``[T]``): the k of every row when rows of different requests share the call; ``top_k`` is then
    the largest of them (the number of candidates the ranks exchange)."""
    T, V = logits.shape
    nblocks = (V + 4095) // 4096
    dev = logits.device
    if scratch is None:
        scratch = torch.empty(T * nblocks * 64 * 2, dtype=torch.float32, device=dev)
    if out_ids is None:
        out_ids = torch.empty(T, dtype=torch.int32, device=dev)
    assert top_k_rows is None or (top_k_rows.dtype == torch.int32 and top_k_rows.numel() == T and top_k_rows.is_contiguous())
    check(_lib.load().ifab_sample_topk(logits.data_ptr(), logits.stride(0), T, V, vocab_offset, top_k, _ptr(top_k_rows), _ptr(inv_temperature),
                                       _ptr(top_p), _ptr(min_p), _ptr(counts), 0 if counts is None else counts.stride(0),
                                       _ptr(penalties), _ptr(seeds), _ptr(counters), scratch.data_ptr(), scratch.numel() * 4,
                                       out_ids.data_ptr(), _ptr(out_probs), C.byref(fabric.desc), _stream()), "sample_topk")
    return out_ids

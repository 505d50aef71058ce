"""ctypes wrappers of the prefill-side kernels: grouped expert GEMM (tcgen05), block router, MoE dispatch / gather /
combine, MLA query rotary + split merge, pull all-reduce of row partials. All of them take pre-allocated outputs
(prefill runs on persistent buffers) and launch on the current stream."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import check

BF16 = torch.bfloat16


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, tiles: torch.Tensor, num_tiles: torch.Tensor, out: torch.Tensor, *,
                 swiglu: bool = False, status_ptr: Optional[int] = None) -> torch.Tensor:
    """``out[r] = a[r] @ b[expert(r)].T`` over the 128-row tiles listed in ``tiles`` (int32 ``[max_tiles, 4]``:
    expert, first row, valid rows, 0); with ``swiglu`` ``b`` is ``[E, 2F, K]`` and ``out`` is ``[rows, F]``."""
    rows, K = a.shape
    E, N, Kb = b.shape
    assert Kb == K and a.stride(1) == 1 and b.is_contiguous() and out.stride(1) == 1 and tiles.dtype == torch.int32
    check(_lib.load().ifab_grouped_gemm_bf16(a.data_ptr(), a.stride(0), rows, b.data_ptr(), E, N, K, tiles.data_ptr(),
                                             num_tiles.data_ptr(), tiles.shape[0], out.data_ptr(), out.stride(0), int(swiglu),
                                             status_ptr, _s()), "grouped_gemm")
    return out


def router_block(x: torch.Tensor, w_router: torch.Tensor, topk: int, ids: torch.Tensor, wts: torch.Tensor, *,
                 norm_w: Optional[torch.Tensor] = None, eps: float = 1e-5, bias: Optional[torch.Tensor] = None,
                 scoring: str = "softmax", renorm: bool = True, scale: float = 1.0, logits: Optional[torch.Tensor] = None,
                 xn: Optional[torch.Tensor] = None) -> None:
    """Router projection (f32) + top-k for any number of rows; ``xn`` receives the normalised rows."""
    M, D = x.shape
    E = w_router.shape[0]
    mode = {"softmax": 0, "sigmoid_bias_group_topk": 1}[scoring]
    check(_lib.load().ifab_router_block(x.data_ptr(), x.stride(0), _p(norm_w), eps, w_router.data_ptr(), _p(bias), _p(logits),
                                        ids.data_ptr(), wts.data_ptr(), _p(xn), 0 if xn is None else xn.stride(0), M, D, E, topk,
                                        mode, int(renorm), scale, _s()), "router_block")


class DispatchBuffers:
    """Device-side routing state of one prefill chunk (allocated once for ``max_rows`` tokens)."""

    def __init__(self, max_rows: int, topk: int, e_local: int, device):
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=device)
        self.max_routes = max_rows * topk
        self.max_tiles = (self.max_routes + 127) // 128 + e_local
        self.counts = i32(e_local)
        self.route_row = i32(self.max_routes)
        self.perm_token = i32(self.max_routes)
        self.tiles = i32(self.max_tiles, 4)
        self.num_tiles = i32(1)
        self.total_rows = i32(1)


def moe_dispatch(ids: torch.Tensor, e0: int, e_local: int, buf: DispatchBuffers) -> None:
    M, topk = ids.shape
    assert M * topk <= buf.max_routes and ids.is_contiguous()
    check(_lib.load().ifab_moe_dispatch(ids.data_ptr(), M, topk, e0, e_local, buf.counts.data_ptr(), buf.route_row.data_ptr(),
                                        buf.perm_token.data_ptr(), buf.tiles.data_ptr(), buf.num_tiles.data_ptr(),
                                        buf.total_rows.data_ptr(), buf.max_tiles, _s()), "moe_dispatch")


def moe_gather(xn: torch.Tensor, buf: DispatchBuffers, xp: torch.Tensor) -> None:
    check(_lib.load().ifab_moe_gather(xn.data_ptr(), xn.stride(0), buf.perm_token.data_ptr(), buf.total_rows.data_ptr(),
                                      xp.data_ptr(), xp.stride(0), xn.shape[1], xp.shape[0], _s()), "moe_gather")


def moe_combine(y: torch.Tensor, buf: DispatchBuffers, wts: torch.Tensor, *, shared: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, out_f32: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> None:
    M, topk = wts.shape
    D = y.shape[1]
    check(_lib.load().ifab_moe_combine(y.data_ptr(), y.stride(0), buf.route_row.data_ptr(), wts.data_ptr(), M, topk, D,
                                       _p(shared), 0 if shared is None else shared.stride(0), _p(residual),
                                       0 if residual is None else residual.stride(0), _p(out_f32), _p(out),
                                       0 if out is None else out.stride(0), _s()), "moe_combine")


def mla_q_rope(q: torch.Tensor, positions: torch.Tensor, q_lat: torch.Tensor, *, nope: int, rope: int, theta: float) -> None:
    T, H, _ = q_lat.shape
    check(_lib.load().ifab_mla_q_rope(q.data_ptr(), q.stride(0), positions.data_ptr(), q_lat.data_ptr(), T, H, nope, rope, theta,
                                      _s()), "mla_q_rope")


def mla_split(q_lat: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
              scratch: torch.Tensor, *, scale: float, window: int, keys_per_split: int, max_splits: int,
              status_ptr: Optional[int] = None, packed: bool = False) -> None:
    """Split-KV partials only (no value up-projection): ``scratch`` = f32 ``[T, H, max_splits, 514]``. ``packed``: the cache holds
    656-byte int8 rows (``uint8 [pages, page_tokens, 656]``)."""
    T, H, row = q_lat.shape
    num_pages, page_tokens, _ = cache.shape
    check(_lib.load().ifab_mla_decode_attention(
        q_lat.data_ptr(), cache.data_ptr(), positions.data_ptr(), slots.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        page_tokens, num_pages, None, 0, window, scale, T, H, 512, -(row - 512) if packed else row - 512, keys_per_split, max_splits, scratch.data_ptr(),
        scratch.numel() * 4, None, 0, 0, None, 0, status_ptr, _s()), "mla_split")


def mla_merge(scratch: torch.Tensor, positions: torch.Tensor, o_lat: torch.Tensor, *, window: int, keys_per_split: int,
              max_splits: int) -> None:
    T, H, _ = o_lat.shape
    check(_lib.load().ifab_mla_merge(scratch.data_ptr(), positions.data_ptr(), 0, window, keys_per_split, max_splits, T, H,
                                     o_lat.data_ptr(), _s()), "mla_merge")


def allreduce_rows(parts, fabric, out: torch.Tensor, *, residual: Optional[torch.Tensor] = None) -> None:
    """``parts``: SymmetricTensor f32 ``[rows, D]`` (this call's parity buffer); ``out = bf16(sum_ranks parts) + residual``.
    With an NVLink multicast mapping of ``parts`` the sum is taken inside the switch (two-shot ``multimem.ld_reduce`` /
    ``multimem.st``; ``parts`` then holds the sums afterwards), otherwise every rank pulls every peer's rows."""
    rows, D = out.shape
    lib = _lib.load()
    if getattr(parts, "mc_ptr", 0) and fabric.world > 1:
        arrive = getattr(fabric, "_nvls_arrive", None)
        if arrive is None:
            arrive = fabric._nvls_arrive = torch.zeros(2, dtype=torch.int32, device=out.device)
        check(lib.ifab_allreduce_rows_nvls(parts.base, parts.mc_ptr, _p(residual), 0 if residual is None else residual.stride(0),
                                           out.data_ptr(), out.stride(0), rows, D, arrive.data_ptr(), C.byref(fabric.desc), _s()),
              "allreduce_rows_nvls")
        return
    check(lib.ifab_allreduce_rows(parts.peer_ptrs, _p(residual), 0 if residual is None else residual.stride(0),
                                  out.data_ptr(), out.stride(0), rows, D, C.byref(fabric.desc), _s()), "allreduce_rows")


def fa_prefill(q: torch.Tensor, k: torch.Tensor, vt: torch.Tensor, out: torch.Tensor, *, heads: int, q_head_stride: int, k_head_stride: int,
               vt_head_stride: int, vt_row0: int = 0, d1: int = 128, d2: int = 0, k2: Optional[torch.Tensor] = None, kv_group: int = 1,
               ctx: int, pos0: int, scale: float, window: int = 0, status_ptr=None) -> torch.Tensor:
    """Prompt attention on the tensor cores for ``m = q.shape[0]`` consecutive positions ``pos0 ..`` of one sequence against keys
    ``0 .. ctx - 1`` (causal, optional sliding window). ``q``: ``[m, ...]``; ``k``: ``[>= ctx, ...]`` per-head key columns;
    ``k2``: ``[>= ctx, d2]`` key columns shared by all heads; ``vt``: transposed values ``[rows, >= ctx]``; ``out``: ``[m, heads * 128]``."""
    m = q.shape[0]
    assert q.dtype == BF16 and k.dtype == BF16 and vt.dtype == BF16 and out.dtype == BF16 and q.stride(1) == 1 and k.stride(1) == 1
    assert vt.stride(1) == 1 and out.stride(1) == 1 and k.shape[0] >= ctx and vt.shape[1] >= ctx and (k2 is None or k2.shape[0] >= ctx)
    check(_lib.load().ifab_fa_prefill_bf16(q.data_ptr(), q.stride(0), q_head_stride, k.data_ptr(), k.stride(0), k_head_stride, _p(k2),
                                           0 if k2 is None else k2.stride(0), vt.data_ptr(), vt.stride(0), vt_head_stride, vt_row0,
                                           vt.shape[0], out.data_ptr(), out.stride(0), m, ctx, heads, kv_group, d1, d2, pos0, window, scale,
                                           status_ptr, _s()), "fa_prefill")
    return out


def mla_q_rope_inplace(q: torch.Tensor, positions: torch.Tensor, *, heads: int, nope: int, rope: int, theta: float) -> None:
    """Rotate the last ``rope`` columns of every head of ``q`` (``[T, heads * (nope + rope)]``) in place."""
    check(_lib.load().ifab_mla_q_rope_inplace(q.data_ptr(), q.stride(0), positions.data_ptr(), q.shape[0], heads, nope, rope, theta, _s()),
          "mla_q_rope_inplace")


def mla_ctx_gather(cache: torch.Tensor, page_table: torch.Tensor, slot: int, ctx: int, lat: torch.Tensor, pe: torch.Tensor, status_ptr=None) -> None:
    """Keys ``0 .. ctx - 1`` of sequence slot ``slot`` out of the paged latent cache into dense ``lat [rows, 512]`` and ``pe [rows, 64]``
    (``rows >= ctx``; the tail rows are zeroed)."""
    rows = lat.shape[0]
    assert pe.shape[0] == rows and lat.is_contiguous() and pe.is_contiguous() and lat.shape[1] == 512 and pe.shape[1] == 64
    check(_lib.load().ifab_mla_ctx_gather(cache.data_ptr(), page_table.data_ptr(), slot, page_table.shape[1], cache.shape[1], cache.shape[0],
                                          ctx, rows, lat.data_ptr(), pe.data_ptr(), status_ptr, _s()), "mla_ctx_gather")


def gqa_ctx_gather(k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor, slot: int, ctx: int, k: torch.Tensor,
                   vt: torch.Tensor, status_ptr=None) -> None:
    """Keys / values ``0 .. ctx - 1`` of sequence slot ``slot`` out of the paged caches ``[pages, page_tokens, kv_heads, hd]`` into dense
    keys ``k [rows, kv_heads * hd]`` and transposed values ``vt [kv_heads * hd, >= rows]`` (``rows`` a multiple of 32, the tail zeroed)."""
    rows, W = k.shape
    assert k.is_contiguous() and vt.stride(1) == 1 and vt.shape[0] == W and vt.shape[1] >= rows and rows % 32 == 0
    assert W == k_cache.shape[2] * k_cache.shape[3]
    check(_lib.load().ifab_gqa_ctx_gather(k_cache.data_ptr(), v_cache.data_ptr(), page_table.data_ptr(), slot, page_table.shape[1],
                                          k_cache.shape[1], k_cache.shape[0], ctx, rows, W, k.data_ptr(), vt.data_ptr(), vt.stride(0), status_ptr,
                                          _s()), "gqa_ctx_gather")

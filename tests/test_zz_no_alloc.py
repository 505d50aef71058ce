"""The allocation-free GQA decode-attention entry point, called as a C symbol.

Collected last on purpose (file name): it has to pass both in a fresh process and after every other
test has used the library. The exported symbol is called through ctypes exactly as a C host would
call it; the reference result comes from the regular entry point with a caller-provided workspace.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16

def _constants():
    """The workspace size and the refusal code, asked of the library itself so that this file cannot drift from the header."""
    from ironpangu_b200.ops import _lib

    lib = _lib.load()
    lib.ifab_gqa_static_scratch_bytes.restype = C.c_uint64
    lib.ifab_gqa_static_scratch_bytes.argtypes = []
    lib.ifab_err_static_scratch.restype = C.c_int
    lib.ifab_err_static_scratch.argtypes = []
    return int(lib.ifab_gqa_static_scratch_bytes()), int(lib.ifab_err_static_scratch())


def _symbol():
    from ironpangu_b200.ops import _lib

    fn = _lib.load().ifab_gqa_decode_attention_static
    P = C.c_void_p
    fn.argtypes = [P, C.c_long, P, P, P, P, P, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int,
                   C.c_int, C.c_int, P, C.c_long, P, P, C.c_char_p, C.c_uint64]
    fn.restype = C.c_int
    return fn


def _case(seed, T, hq, hkv, hd, positions, page_tokens=16, max_pages=24):
    g = torch.Generator(device="cuda").manual_seed(seed)
    num_pages = max_pages * 2
    q = torch.randn(T, (hq + 2 * hkv) * hd, generator=g, device="cuda").to(BF16)       # q columns of a qkv buffer
    k = torch.randn(num_pages, page_tokens, hkv, hd, generator=g, device="cuda").to(BF16)
    v = torch.randn(num_pages, page_tokens, hkv, hd, generator=g, device="cuda").to(BF16)
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    slots = torch.tensor([i % 2 for i in range(T)], dtype=torch.int32, device="cuda")
    table = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).to(torch.int32).view(2, max_pages).cuda()
    return q, k, v, pos, slots, table


def _call_static(fn, q, k, v, pos, slots, table, hq, hkv, hd, kps, max_splits, out):
    err = C.create_string_buffer(512)
    rc = fn(q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(), pos.data_ptr(), slots.data_ptr(), table.data_ptr(),
            table.shape[1], k.shape[1], k.shape[0], 1.0 / math.sqrt(hd), q.shape[0], hq, hkv, hd, kps, max_splits,
            out.data_ptr(), out.stride(0), None, torch.cuda.current_stream().cuda_stream, err, len(err))
    return rc, err.value.decode()


def _reference_fp32(q, k, v, pos, slots, table, hq, hkv, hd):
    T, pt = q.shape[0], k.shape[1]
    out = torch.zeros(T, hq * hd, device="cuda")
    for t in range(T):
        n = int(pos[t]) + 1
        rows = [int(table[int(slots[t]), i // pt]) * pt + i % pt for i in range(n)]
        kk = k.view(-1, hkv, hd)[rows].float()
        vv = v.view(-1, hkv, hd)[rows].float()
        for h in range(hq):
            qh = q[t, h * hd:(h + 1) * hd].float()
            s = (kk[:, h // (hq // hkv)] @ qh) / math.sqrt(hd)
            out[t, h * hd:(h + 1) * hd] = torch.softmax(s, 0) @ vv[:, h // (hq // hkv)]
    return out


def test_static_entry_matches_regular_entry_twice_in_a_row():
    from ironpangu_b200.ops import decode as K

    fn = _symbol()
    hq, hkv, hd, kps, max_splits = 8, 2, 128, 64, 6
    # two different problems back to back: the second call finds the first call's partials in the shared
    # workspace (its shorter sequences use fewer splits) and must not be affected by them
    cases = [_case(1, 5, hq, hkv, hd, [340, 17, 63, 64, 200]), _case(2, 3, hq, hkv, hd, [9, 130, 0])]
    for q, k, v, pos, slots, table in cases:
        T = q.shape[0]
        want = K.gqa_decode_attention(q, k, v, pos, slots, table, heads=hq, kv_heads=hkv, head_dim=hd,
                                      scale=1.0 / math.sqrt(hd), keys_per_split=kps, max_splits=max_splits)
        got = torch.full((T, hq * hd), float("nan"), dtype=BF16, device="cuda")
        rc, msg = _call_static(fn, q, k, v, pos, slots, table, hq, hkv, hd, kps, max_splits, got)
        assert rc == 0, msg
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), rtol=0, atol=0)
        torch.testing.assert_close(got.float(), _reference_fp32(q, k, v, pos, slots, table, hq, hkv, hd), rtol=2e-2, atol=2e-2)


def test_static_entry_refuses_what_does_not_fit():
    fn = _symbol()
    hq, hkv, hd = 64, 8, 256
    q, k, v, pos, slots, table = _case(3, 8, hq, hkv, hd, [5] * 8, max_pages=2)
    out = torch.zeros(8, hq * hd, dtype=BF16, device="cuda")
    STATIC_BYTES, ERR_STATIC_SCRATCH = _constants()
    need = 8 * hq * 64 * (hd + 2) * 4
    assert need > STATIC_BYTES
    rc, msg = _call_static(fn, q, k, v, pos, slots, table, hq, hkv, hd, 64, 64, out)
    assert rc == ERR_STATIC_SCRATCH
    assert str(need) in msg and str(STATIC_BYTES) in msg
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0      # nothing was launched
    lib_msg = __import__("ironpangu_b200.ops._lib", fromlist=["load"]).load().ifab_error_string(ERR_STATIC_SCRATCH).decode()
    assert "built-in" in lib_msg


def test_context_longer_than_the_split_grid_is_attended_in_full():
    """keys_per_split * max_splits is smaller than the context: the last split takes the tail, nothing is clipped."""
    fn = _symbol()
    hq, hkv, hd, kps, max_splits = 8, 2, 128, 16, 3          # 48 keys of split grid against up to 341 keys of context
    q, k, v, pos, slots, table = _case(4, 4, hq, hkv, hd, [340, 47, 48, 200])
    got = torch.full((4, hq * hd), float("nan"), dtype=BF16, device="cuda")
    rc, msg = _call_static(fn, q, k, v, pos, slots, table, hq, hkv, hd, kps, max_splits, got)
    assert rc == 0, msg
    torch.cuda.synchronize()
    torch.testing.assert_close(got.float(), _reference_fp32(q, k, v, pos, slots, table, hq, hkv, hd), rtol=2e-2, atol=2e-2)

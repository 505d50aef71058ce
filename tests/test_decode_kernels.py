"""Each decode kernel against a plain PyTorch fp32 reference of the same op (single GPU)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def env():
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.models import mla_moe_ref as R

    fab = Fabric(0, 1)
    yield K, fab, R
    fab.close()


def rnd(*shape, scale=1.0, dtype=BF16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(dtype)


@pytest.mark.parametrize("T,D", [(1, 256), (3, 4096), (8, 1536)])
def test_rmsnorm(env, T, D):
    K, fab, R = env
    x, w = rnd(T, D), rnd(D, scale=0.1) + 1
    y = K.rmsnorm(x, w, 1e-5)
    ref = R.rmsnorm_ref(x, w, 1e-5)
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=1e-2)
    yz = K.rmsnorm(x, w, 1e-6, zero_centered=True)
    torch.testing.assert_close(yz.float(), R.rmsnorm_ref(x, w, 1e-6, True), rtol=1e-2, atol=2e-2)


def test_embedding(env):
    K, fab, R = env
    table = rnd(1000, 256)
    ids = torch.tensor([5, 999, 0, 17], dtype=torch.int32, device="cuda")
    out = K.embedding(ids, table)
    assert torch.equal(out, table[ids.long()])


@pytest.mark.parametrize("T,N,K_", [(1, 2112, 4096), (1, 768, 1536), (2, 96, 512), (4, 6144, 2048), (8, 1000, 192),
                                    (5, 19200, 4096), (11, 520, 256)])
def test_gemv(env, T, N, K_):
    K, fab, R = env
    x, w = rnd(T, K_), rnd(N, K_, scale=0.05)
    y = K.gemv(x, w)
    ref = x.float() @ w.float().T
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    y32 = K.gemv(x, w, out_f32=True)
    torch.testing.assert_close(y32, ref, rtol=1e-3, atol=1e-3)


def test_gemv_norm_residual_swiglu(env):
    K, fab, R = env
    T, N, K_ = 3, 1536, 4096
    x, w, nw, res = rnd(T, K_), rnd(2 * N, K_, scale=0.02), rnd(K_, scale=0.1) + 1, rnd(T, N)
    h = R.rmsnorm_ref(x, nw, 1e-5)
    y = K.gemv(x, w[:N].contiguous(), norm_w=nw, eps=1e-5, residual=res)
    ref = (h @ w[:N].float().T).to(BF16).float() + res.float()
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    ys = K.gemv(x, w, norm_w=nw, eps=1e-5, swiglu=True)
    gu = (h @ w.float().T).to(BF16).float()
    refs = torch.nn.functional.silu(gu[:, :N]) * gu[:, N:]
    torch.testing.assert_close(ys.float(), refs, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("T,N,K_", [(1, 4096, 512), (4, 2048, 1024), (8, 256, 64)])
def test_gemv_allreduce_single_rank(env, T, N, K_):
    """world = 1: the fused kernel must equal the plain linear + residual and advance the call counter."""
    K, fab, R = env
    x, w, res = rnd(T, K_), rnd(N, K_, scale=0.05), rnd(T, N)
    before = fab.calls()
    y = K.gemv_allreduce(x, w, fab, residual=res)
    ref = (x.float() @ w.float().T).to(BF16).float() + res.float()
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    assert fab.calls() == before + 1
    assert fab.status() == 0


@pytest.mark.parametrize("scoring", ["softmax", "sigmoid_bias_group_topk"])
@pytest.mark.parametrize("T,E,topk", [(1, 96, 8), (4, 256, 8), (8, 16, 4)])
def test_router(env, scoring, T, E, topk):
    K, fab, R = env
    D = 512
    x, nw = rnd(T, D), rnd(D, scale=0.1) + 1
    wr = rnd(E, D, scale=0.2, dtype=torch.float32)
    bias = rnd(E, scale=0.1, dtype=torch.float32) if scoring != "softmax" else None
    ids, wts, logits = K.router_topk(x, wr, topk, norm_w=nw, eps=1e-5, scoring=scoring, bias=bias, scale=2.5,
                                     ticket_ptr=fab.ticket_ptr)
    h = R.rmsnorm_ref(x, nw, 1e-5)
    ref_logits = h @ wr.T
    torch.testing.assert_close(logits, ref_logits, rtol=1e-3, atol=1e-3)
    # selection is checked on the kernel's own logits so that near-ties cannot flip
    rids, rw = R.route_ref(logits, topk, scoring, bias, True, 2.5)
    assert torch.equal(ids.long(), rids)
    torch.testing.assert_close(wts, rw, rtol=1e-4, atol=1e-5)


def test_moe_decode_single_rank(env):
    K, fab, R = env
    T, D, F, E, topk, Fs = 3, 256, 64, 16, 4, 32
    x, nw = rnd(T, D), rnd(D, scale=0.1) + 1
    wgu, wd = rnd(E, 2 * F, D, scale=0.05), rnd(E, D, F, scale=0.05)
    sgu, sd = rnd(2 * Fs, D, scale=0.05), rnd(D, Fs, scale=0.05)
    wr = rnd(E, D, scale=0.2, dtype=torch.float32)
    ids, wts, _ = K.router_topk(x, wr, topk, norm_w=nw, ticket_ptr=fab.ticket_ptr)
    act = K.moe_gate_up(x, ids, wgu, 0, norm_w=nw, w_shared_gu=sgu)
    res = rnd(T, D)
    y = K.moe_down_allreduce(act, ids, wts, wd, 0, fab, w_shared_down=sd, residual=res)
    h = R.rmsnorm_ref(x, nw, 1e-5)
    ref = torch.zeros(T, D, device="cuda")
    for t in range(T):
        for k in range(topk):
            e = int(ids[t, k])
            gu = (h[t] @ wgu[e].float().T).to(BF16).float()
            a = (torch.nn.functional.silu(gu[:F]) * gu[F:]).to(BF16).float()
            torch.testing.assert_close(act[t, k].float(), a, rtol=2e-2, atol=1e-3)
            ref[t] += wts[t, k] * (a @ wd[e].float().T)
        gu = (h[t] @ sgu.float().T).to(BF16).float()
        a = (torch.nn.functional.silu(gu[:Fs]) * gu[Fs:]).to(BF16).float()
        ref[t] += a @ sd.float().T
    ref = ref.to(BF16).float() + res.float()
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("T,D,F,E,topk,Fs,e0,el", [(1, 256, 64, 16, 4, 32, 0, 16), (2, 256, 64, 16, 4, 32, 4, 4),
                                                   (1, 4096, 1536, 96, 8, 192, 12, 12), (2, 4096, 1536, 96, 8, 1536, 0, 96),
                                                   (1, 512, 72, 24, 6, 0, 0, 24)])
def test_moe_block_one_launch_equals_chain(env, T, D, F, E, topk, Fs, e0, el):
    """Router + gate/up + down + all-reduce as one launch against the three-kernel chain (bit-identical) and against the
    fp32 reference; run twice so that the in-grid signal words are reused, with a shard of the experts as on one of N ranks."""
    K, fab, R = env
    x, nw = rnd(T, D), rnd(D, scale=0.1) + 1
    wgu, wd = rnd(el, 2 * F, D, scale=0.05), rnd(el, D, F, scale=0.05)
    sgu, sd = (rnd(2 * Fs, D, scale=0.05), rnd(D, Fs, scale=0.05)) if Fs else (None, None)
    wr = rnd(E, D, scale=0.2, dtype=torch.float32)
    ids, wts, logits = K.router_topk(x, wr, topk, norm_w=nw, ticket_ptr=fab.ticket_ptr)
    act = K.moe_gate_up(x, ids, wgu, e0, norm_w=nw, w_shared_gu=sgu)
    y = K.moe_down_allreduce(act, ids, wts, wd, e0, fab, w_shared_down=sd, residual=x)
    sync = torch.zeros(K.moe_block_sync_words(T, E), dtype=torch.int32, device="cuda")
    for _ in range(2):
        ids2 = torch.full_like(ids, -1)
        wts2, logits2 = torch.zeros_like(wts), torch.zeros_like(logits)
        y2 = K.moe_block(x, wr, wgu, wd, e0, topk, fab, sync=sync, norm_w=nw, w_shared_gu=sgu, w_shared_down=sd, ids=ids2,
                         wts=wts2, logits=logits2)
        torch.cuda.synchronize()
        assert fab.status() == 0
        assert torch.equal(ids2, ids) and torch.equal(wts2, wts) and torch.equal(logits2, logits)
        assert torch.equal(y2, y)
    h = R.rmsnorm_ref(x, nw, 1e-5)
    ref = torch.zeros(T, D, device="cuda")
    for t in range(T):
        for k in range(topk):
            e = int(ids[t, k]) - e0
            if not 0 <= e < el:
                continue
            gu = (h[t] @ wgu[e].float().T).to(BF16).float()
            a = (torch.nn.functional.silu(gu[:F]) * gu[F:]).to(BF16).float()
            ref[t] += wts[t, k] * (a @ wd[e].float().T)
        if Fs:
            gu = (h[t] @ sgu.float().T).to(BF16).float()
            a = (torch.nn.functional.silu(gu[:Fs]) * gu[Fs:]).to(BF16).float()
            ref[t] += a @ sd.float().T
    ref = ref.to(BF16).float() + x.float()
    torch.testing.assert_close(y2.float(), ref, rtol=2e-2, atol=2e-2)
    # x may be updated in place (the residual stream of the decoder)
    x3 = x.clone()
    K.moe_block(x3, wr, wgu, wd, e0, topk, fab, sync=sync, norm_w=nw, w_shared_gu=sgu, w_shared_down=sd, out=x3)
    assert torch.equal(x3, y)


@pytest.mark.parametrize("T,V", [(1, 19200), (4, 1000), (8, 153600)])
def test_lm_head_argmax(env, T, V):
    K, fab, R = env
    D = 256
    x, nw, w = rnd(T, D), rnd(D, scale=0.1) + 1, rnd(V, D, scale=0.05)
    logits = torch.empty(T, V, dtype=torch.float32, device="cuda")
    ids = K.lm_head_argmax(x, w, fab, norm_w=nw, vocab_offset=7, logits=logits)
    ref = R.rmsnorm_ref(x, nw, 1e-5) @ w.float().T
    torch.testing.assert_close(logits, ref, rtol=1e-3, atol=1e-3)
    assert torch.equal(ids.long(), logits.argmax(-1) + 7)
    assert fab.status() == 0


def _mla_setup(T, H, ctx, page_tokens=16, seed=0):
    nope, rope, latent, vdim = 128, 64, 512, 128
    slots_n = 2
    max_pages = (ctx + page_tokens - 1) // page_tokens
    num_pages = slots_n * max_pages
    # permuted (non-contiguous) page bindings
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).to(torch.int32).cuda()
    page_table = perm.view(slots_n, max_pages).contiguous()
    cache = torch.zeros(num_pages, page_tokens, latent + rope, dtype=BF16, device="cuda")
    return nope, rope, latent, vdim, page_table, cache


def test_mla_kv_write_and_attention(env):
    K, fab, R = env
    H, ctx = 4, 200
    nope, rope, latent, vdim, page_table, cache = _mla_setup(1, H, 256)
    theta, eps = 6.4e6, 1e-5
    kvn = rnd(latent, scale=0.1) + 1
    # fill slot 1 with ctx rows, a few tokens per call
    kv_all = rnd(ctx, latent + rope)
    for s in range(0, ctx, 8):
        n = min(8, ctx - s)
        pos = torch.arange(s, s + n, dtype=torch.int32, device="cuda")
        slot = torch.ones(n, dtype=torch.int32, device="cuda")
        K.mla_kv_write(kv_all[s:s + n], kvn, pos, slot, page_table, cache, latent=latent, rope=rope, eps=eps,
                       theta=theta, status_ptr=fab.desc.status)
    lat_ref = R.rmsnorm_ref(kv_all[:, :latent], kvn, eps)
    kr_ref = R.rope_ref(kv_all[:, latent:], torch.arange(ctx, device="cuda"), theta)
    rows = torch.stack([cache[page_table[1, p // 16], p % 16] for p in range(ctx)]).float()
    torch.testing.assert_close(rows[:, :latent], lat_ref, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(rows[:, latent:], kr_ref, rtol=1e-2, atol=2e-2)
    # the same rows with the rotary columns taken from rows of their own: identical cache contents
    other = torch.zeros_like(cache)
    lat_rows, rope_rows = kv_all[:, :latent].contiguous(), torch.cat([rnd(ctx, 24), kv_all[:, latent:]], 1)[:, 24:]
    for s in range(0, ctx, 8):
        n = min(8, ctx - s)
        pos = torch.arange(s, s + n, dtype=torch.int32, device="cuda")
        slot = torch.ones(n, dtype=torch.int32, device="cuda")
        K.mla_kv_write_split(lat_rows[s:s + n], rope_rows[s:s + n], kvn, pos, slot, page_table, other, eps=eps, theta=theta, status_ptr=fab.desc.status)
    assert torch.equal(other, cache)

    # attention for 3 query rows at different positions of slot 1 (+ windowed variant)
    T = 3
    pos = torch.tensor([ctx - 1, 57, 0], dtype=torch.int32, device="cuda")
    slot = torch.ones(T, dtype=torch.int32, device="cuda")
    q = rnd(T, H * (nope + rope))
    kvb = rnd(H, nope + vdim, latent, scale=0.05)
    q_lat = K.mla_q_absorb(q, kvb, pos, nope=nope, rope=rope, theta=theta)
    qv = q.float().view(T, H, nope + rope)
    ql_ref = torch.einsum("thd,hdc->thc", qv[..., :nope], kvb[:, :nope].float()).to(BF16).float()
    qr_ref = R.rope_ref(qv[..., nope:], pos, theta)
    torch.testing.assert_close(q_lat[..., :latent].float(), ql_ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q_lat[..., latent:].float(), qr_ref, rtol=1e-2, atol=2e-2)
    scale = 1.0 / math.sqrt(nope + rope)
    for window in (0, 64):
        out = K.mla_decode_attention(q_lat, cache, pos, slot, page_table, kvb, nope=nope, scale=scale, window=window,
                                     keys_per_split=64, max_splits=4, status_ptr=fab.desc.status)
        ref = torch.zeros(T, H * vdim, device="cuda")
        for t in range(T):
            p = int(pos[t])
            lo = 0 if window == 0 else max(0, p + 1 - window)
            keys = rows[lo:p + 1]
            s = (q_lat[t].float() @ keys.T) * scale
            pr = torch.softmax(s, -1)
            o = (pr @ keys[:, :latent]).to(BF16).float()
            ref[t] = torch.einsum("hc,hvc->hv", o, kvb[:, nope:].float()).reshape(-1)
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    assert fab.status() == 0


def test_mla_attention_sinks(env):
    K, fab, R = env
    H, ctx = 2, 40
    nope, rope, latent, vdim, page_table, cache = _mla_setup(1, H, 64)
    cache.copy_(rnd(*cache.shape))
    sinks = rnd(5, latent + rope)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
    slot = torch.zeros(1, dtype=torch.int32, device="cuda")
    q_lat = rnd(1, H, latent + rope, scale=0.3)
    kvb = rnd(H, nope + vdim, latent, scale=0.05)
    out = K.mla_decode_attention(q_lat, cache, pos, slot, page_table, kvb, nope=nope, scale=0.07, sinks=sinks,
                                 keys_per_split=16, max_splits=4)
    rows = torch.stack([cache[page_table[0, p // 16], p % 16] for p in range(ctx)]).float()
    keys = torch.cat([sinks.float(), rows])
    pr = torch.softmax((q_lat[0].float() @ keys.T) * 0.07, -1)
    o = (pr @ keys[:, :latent]).to(BF16).float()
    ref = torch.einsum("hc,hvc->hv", o, kvb[:, nope:].float()).reshape(1, -1)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_bad_page_sets_status_without_fault(env):
    """An out-of-range page id is skipped and reported through the status word; nothing faults."""
    K, fab, R = env
    nope, rope, latent, vdim, page_table, cache = _mla_setup(1, 4, 64)
    bad = page_table.clone()
    bad[0, 0] = 10_000
    kv = rnd(1, latent + rope)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    K.mla_kv_write(kv, rnd(latent), pos, pos, bad, cache, latent=latent, rope=rope, eps=1e-5, theta=1e4,
                   status_ptr=fab.desc.status)
    from ironpangu_b200.parallel.fabric import STATUS_BAD_INDEX
    assert fab.status() & STATUS_BAD_INDEX
    fab.clear_status()
    assert fab.status() == 0

"""Prefill path: grouped tcgen05 expert GEMM, routing plumbing and the whole tensor-core prefill against PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _tiles(counts):
    tiles, off = [], 0
    for e, n in enumerate(counts):
        for r0 in range(0, n, 128):
            tiles.append([e, off + r0, min(128, n - r0), 0])
        off += n
    return tiles, off


@pytest.mark.parametrize("counts,N,K", [([5, 0, 300, 128, 1], 256, 192), ([130, 17], 96, 64), ([0, 0, 9], 512, 4096)])
def test_grouped_gemm_plain_and_swiglu(counts, N, K):
    from ironpangu_b200.ops import prefill as P

    g = torch.Generator(device="cuda").manual_seed(0)
    tiles, rows = _tiles(counts)
    E = len(counts)
    a = torch.randn(rows + 40, K, generator=g, device="cuda").to(BF16)          # rows past `rows` are never valid
    b = (torch.randn(E, N, K, generator=g, device="cuda") * 0.05).to(BF16)
    tt = torch.zeros(len(tiles) + 3, 4, dtype=torch.int32, device="cuda")
    tt[:len(tiles)] = torch.tensor(tiles, dtype=torch.int32)
    nt = torch.tensor([len(tiles)], dtype=torch.int32, device="cuda")
    expert_of = torch.repeat_interleave(torch.arange(E), torch.tensor(counts)).cuda()
    ref = torch.einsum("rk,rnk->rn", a[:rows].float(), b.float()[expert_of])
    out = torch.full((rows + 40, N), 7.0, dtype=BF16, device="cuda")
    P.grouped_gemm(a, b, tt, nt, out)
    torch.testing.assert_close(out[:rows].float(), ref, rtol=2e-2, atol=2e-2)
    assert float((out[rows:].float() - 7.0).abs().max()) == 0.0                  # nothing outside the valid rows is written
    F = N // 2
    g_, u_ = ref[:, :F].to(BF16).float(), ref[:, F:].to(BF16).float()
    want = torch.nn.functional.silu(g_) * u_
    act = torch.full((rows + 40, F), 7.0, dtype=BF16, device="cuda")
    P.grouped_gemm(a, b, tt, nt, act, swiglu=True)
    torch.testing.assert_close(act[:rows].float(), want, rtol=3e-2, atol=2e-2)
    assert float((act[rows:].float() - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("M,E,topk,e0,el", [(37, 16, 4, 0, 16), (300, 96, 8, 24, 12), (8, 16, 4, 8, 8)])
def test_dispatch_gather_combine(M, E, topk, e0, el):
    from ironpangu_b200.ops import prefill as P

    g = torch.Generator(device="cuda").manual_seed(1)
    D = 64
    ids = torch.stack([torch.randperm(E, generator=g, device="cuda")[:topk] for _ in range(M)]).to(torch.int32).contiguous()
    wts = torch.rand(M, topk, generator=g, device="cuda")
    xn = torch.randn(M, D, generator=g, device="cuda").to(BF16)
    buf = P.DispatchBuffers(M, topk, el, "cuda")
    P.moe_dispatch(ids, e0, el, buf)
    local = (ids >= e0) & (ids < e0 + el)
    counts = torch.stack([(ids == e0 + e).sum() for e in range(el)]).to(torch.int32)
    assert torch.equal(buf.counts, counts)
    total = int(local.sum())
    assert int(buf.total_rows) == total
    rr = buf.route_row.view(M, topk)
    assert torch.equal(rr < 0, ~local)
    assert sorted(rr[local].tolist()) == list(range(total))                       # a permutation of the rows
    offs = torch.cumsum(counts, 0) - counts
    for t in range(M):
        for k in range(topk):
            if local[t, k]:
                e = int(ids[t, k]) - e0
                r = int(rr[t, k])
                assert int(offs[e]) <= r < int(offs[e]) + int(counts[e]) and int(buf.perm_token[r]) == t
    tiles = buf.tiles[:int(buf.num_tiles)].tolist()
    assert tiles == [t for t in _tiles(counts.tolist())[0]]
    xp = torch.zeros(buf.max_routes, D, dtype=BF16, device="cuda")
    P.moe_gather(xn, buf, xp)
    assert torch.equal(xp[:total], xn[buf.perm_token[:total].long()])
    y = torch.randn(buf.max_routes, D, generator=g, device="cuda").to(BF16)
    shared = torch.randn(M, D, generator=g, device="cuda").to(BF16)
    res = torch.randn(M, D, generator=g, device="cuda").to(BF16)
    want = shared.float().clone()
    for t in range(M):
        for k in range(topk):
            if local[t, k]:
                want[t] += wts[t, k] * y[int(rr[t, k])].float()
    out32 = torch.empty(M, D, device="cuda")
    out = torch.empty(M, D, dtype=BF16, device="cuda")
    P.moe_combine(y, buf, wts, shared=shared, residual=res, out_f32=out32, out=out)
    torch.testing.assert_close(out32, want, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.float(), (want.to(BF16).float() + res.float()).to(BF16).float(), rtol=1e-2, atol=1e-2)


def test_router_block_matches_reference():
    from ironpangu_b200.models.mla_moe_ref import rmsnorm_ref, route_ref
    from ironpangu_b200.ops import prefill as P

    g = torch.Generator(device="cuda").manual_seed(2)
    M, D, E, topk = 45, 256, 16, 4
    x = torch.randn(M, D, generator=g, device="cuda").to(BF16)
    nw = (1 + 0.1 * torch.randn(D, generator=g, device="cuda")).to(BF16)
    wr = torch.randn(E, D, generator=g, device="cuda") * 0.1
    ids = torch.zeros(M, topk, dtype=torch.int32, device="cuda")
    wts = torch.zeros(M, topk, device="cuda")
    xn = torch.zeros(M, D, dtype=BF16, device="cuda")
    P.router_block(x, wr, topk, ids, wts, norm_w=nw, xn=xn)
    h = rmsnorm_ref(x, nw, 1e-5)
    torch.testing.assert_close(xn.float(), h, rtol=1e-2, atol=1e-2)
    rid, rw = route_ref(h @ wr.T, topk)
    assert torch.equal(ids.long(), rid)
    torch.testing.assert_close(wts, rw, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("m,window", [(19, 0), (150, 0), (40, 8)])
def test_prefill_matches_oracle_and_decode_continues(m, window):
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_full_weights, shard_weights
    from ironpangu_b200.models.mla_moe_prefill import MlaMoePrefill
    from ironpangu_b200.models.mla_moe_ref import forward_ref
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = MlaMoeConfig.tiny(2)
    cfg.window = window
    full = random_full_weights(cfg, seed=0)
    fab = Fabric(0, 1)
    dec = MlaMoeDecoder(cfg, shard_weights(cfg, full, 0, 1, "cuda"), fab, max_tokens=8, max_context=256, keep_logits=True)
    pre = MlaMoePrefill(dec, max_rows=160, attn_rows=64)
    toks = torch.randint(0, cfg.vocab, (m + 6,), generator=torch.Generator().manual_seed(5))
    ref = forward_ref(cfg, full, toks.cuda())
    nxt = pre.forward(toks[:m].to(torch.int32).cuda(), 0)
    torch.testing.assert_close(dec.logits[0], ref[m - 1], rtol=3e-2, atol=3e-2)
    assert int(nxt[0]) == int(dec.logits[0].argmax())
    # decode continues on the cache the prefill wrote (teacher-forced with the reference tokens)
    for i in range(m, m + 6):
        dec.tokens[:1].fill_(int(toks[i]))
        dec.positions[:1].fill_(i)
        dec.slots[:1].zero_()
        dec.forward(1)
        torch.testing.assert_close(dec.logits[0], ref[i], rtol=3e-2, atol=3e-2)
    assert fab.status() == 0
    fab.close()


def test_forward_rows_matches_the_decode_kernels_on_independent_sequences():
    """One decode row per sequence (three sequences at different positions) through the matrix-matrix path against the
    decode kernels: same logits, same cache rows."""
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_full_weights, shard_weights
    from ironpangu_b200.models.mla_moe_prefill import MlaMoePrefill
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = MlaMoeConfig.tiny(2)
    full = random_full_weights(cfg, seed=0)
    fab = Fabric(0, 1)
    mk = lambda: MlaMoeDecoder(cfg, shard_weights(cfg, full, 0, 1, "cuda"), fab, max_tokens=8, max_context=128, num_slots=3,
                               keep_logits=True, fused_head=False)
    a, b = mk(), mk()
    g = torch.Generator().manual_seed(11)
    lens = [37, 5, 64]
    for dec in (a, b):
        for slot, n in enumerate(lens):
            toks = torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(slot)).to(torch.int32)
            for s in range(0, n, 8):
                k = min(8, n - s)
                dec.tokens[:k].copy_(toks[s:s + k])
                dec.positions[:k].copy_(torch.arange(s, s + k, dtype=torch.int32))
                dec.slots[:k].fill_(slot)
                dec.forward(k)
    step = torch.randint(0, cfg.vocab, (3,), generator=g).to(torch.int32).cuda()
    pos = torch.tensor(lens, dtype=torch.int32, device="cuda")
    slots = torch.arange(3, dtype=torch.int32, device="cuda")
    pre = MlaMoePrefill(a, max_rows=64, attn_rows=16)
    got = pre.forward_rows(step, pos, slots, torch.tensor([0, 2], device="cuda"))
    b.tokens[:3].copy_(step)
    b.positions[:3].copy_(pos)
    b.slots[:3].copy_(slots)
    b.forward(3)
    torch.cuda.synchronize()
    torch.testing.assert_close(got, b.logits[:3][[0, 2]], rtol=3e-2, atol=3e-2)
    for l in range(cfg.layers):
        torch.testing.assert_close(a.caches[l].float(), b.caches[l].float(), rtol=2e-2, atol=2e-2)
    assert fab.status() == 0
    fab.close()

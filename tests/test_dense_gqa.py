"""Dense GQA decoder + device sampling against PyTorch fp32 references (single GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _setup(max_tokens=8, num_slots=2):
    from ironpangu_b200.models.dense_gqa import DenseConfig, DenseDecoder, random_full_weights, shard_weights
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = DenseConfig.tiny(2)
    full = random_full_weights(cfg, 0)
    fab = Fabric(0, 1)
    dec = DenseDecoder(cfg, shard_weights(cfg, full, 0, 1, "cuda"), fab, max_tokens=max_tokens, max_context=128,
                       num_slots=num_slots, keep_logits=True)
    return cfg, full, fab, dec


def test_two_interleaved_sequences_match_oracle():
    """Rows of two sequences at different positions share every launch (continuous batching)."""
    from ironpangu_b200.models.dense_gqa import forward_ref

    cfg, full, fab, dec = _setup()
    g = torch.Generator().manual_seed(4)
    a = torch.randint(0, cfg.vocab, (21,), generator=g).tolist()
    b = torch.randint(0, cfg.vocab, (9,), generator=g).tolist()
    ra, rb = forward_ref(cfg, full, torch.tensor(a, device="cuda")), forward_ref(cfg, full, torch.tensor(b, device="cuda"))
    pa = pb = 0
    while pa < len(a) or pb < len(b):
        na, nb = min(5, len(a) - pa), min(3, len(b) - pb)     # chunk of A + chunk of B in one step
        toks = a[pa:pa + na] + b[pb:pb + nb]
        pos = list(range(pa, pa + na)) + list(range(pb, pb + nb))
        slot = [0] * na + [1] * nb
        n = len(toks)
        dec.tokens[:n].copy_(torch.tensor(toks, dtype=torch.int32))
        dec.positions[:n].copy_(torch.tensor(pos, dtype=torch.int32))
        dec.slots[:n].copy_(torch.tensor(slot, dtype=torch.int32))
        dec.forward(n)
        lg = dec.logits[:n]
        torch.testing.assert_close(lg[:na], ra[pa:pa + na], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(lg[na:], rb[pb:pb + nb], rtol=2e-2, atol=2e-2)
        assert torch.equal(dec.next_ids[:n].long(), lg.argmax(-1))
        pa, pb = pa + na, pb + nb
    assert fab.status() == 0
    fab.close()


def test_graph_replay_equals_eager():
    cfg, full, fab, dec = _setup(1, 1)
    outs = []
    for i, t in enumerate([3, 77, 500, 9]):
        dec.tokens.fill_(t); dec.positions.fill_(i); dec.slots.zero_()
        dec.forward(1)
        outs.append(dec.logits[:1].clone())
    dec.reset()
    dec.capture(1)
    for i, t in enumerate([3, 77, 500, 9]):
        dec.tokens.fill_(t); dec.positions.fill_(i)
        dec._graph.replay()
        assert torch.equal(dec.logits[:1], outs[i])
    fab.close()


def test_sampling_rows_keep_their_own_top_k():
    """Rows of requests with different top_k in one call draw exactly what each draws alone (same seed, same counter)."""
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(0, 1)
    T, V = 4, 20000
    g = torch.Generator(device="cuda").manual_seed(3)
    logits = torch.randn(T, V, generator=g, device="cuda") * 2
    ks = [5, 50, 1, 64]
    invt = torch.full((T,), 1 / 0.9, device="cuda")
    seeds = torch.arange(T, dtype=torch.int64, device="cuda") + 101
    together, alone = [], []
    counters = torch.zeros(T, dtype=torch.int64, device="cuda")
    k_rows = torch.tensor(ks, dtype=torch.int32, device="cuda")
    for _ in range(60):
        together.append(K.sample_topk(logits, fab, top_k=max(ks), top_k_rows=k_rows, inv_temperature=invt, seeds=seeds, counters=counters).clone())
    for t in range(T):
        c = torch.zeros(1, dtype=torch.int64, device="cuda")
        alone.append(torch.stack([K.sample_topk(logits[t:t + 1], fab, top_k=ks[t], inv_temperature=invt[t:t + 1], seeds=seeds[t:t + 1],
                                                counters=c).clone() for _ in range(60)])[:, 0])
    together = torch.stack(together)
    for t in range(T):
        assert torch.equal(together[:, t], alone[t]), t
        assert set(together[:, t].tolist()) <= set(logits[t].topk(ks[t]).indices.tolist())
    assert len(set(together[:, 2].tolist())) == 1            # k = 1 is greedy
    fab.close()


def test_sampling_topk_topp_minp_exact():
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(0, 1)
    T, V, k = 4, 151936, 50
    g = torch.Generator(device="cuda").manual_seed(1)
    logits = torch.randn(T, V, generator=g, device="cuda") * 3
    invt = torch.tensor([1 / 0.7, 0.0, 1.0, 2.0], device="cuda")
    topp = torch.tensor([1.0, 1.0, 0.8, 1.0], device="cuda")
    minp = torch.tensor([0.0, 0.0, 0.0, 0.3], device="cuda")
    seeds = torch.arange(T, dtype=torch.int64, device="cuda") + 11
    counters = torch.zeros(T, dtype=torch.int64, device="cuda")
    probs = torch.empty(T, device="cuda")
    draws = torch.stack([K.sample_topk(logits, fab, top_k=k, inv_temperature=invt, top_p=topp, min_p=minp, seeds=seeds,
                                       counters=counters, out_probs=probs).clone() for _ in range(400)])
    assert int(counters[0]) == 400                       # the counter advances on the device
    # allowed sets from a plain PyTorch restatement
    for t in range(T):
        scaled = logits[t] * (invt[t] if invt[t] > 0 else 1.0)
        vals, idx = scaled.topk(k)
        p = torch.softmax(vals, -1)
        keep = torch.ones(k, dtype=torch.bool, device="cuda")
        if minp[t] > 0:
            keep &= p >= minp[t] * p[0]
        if topp[t] < 1:
            pk = p * keep
            excl = torch.cumsum(pk, 0) - pk
            keep &= excl < topp[t] * pk.sum()
        allowed = set(idx[keep].tolist())
        seen = set(draws[:, t].tolist())
        if invt[t] <= 0:
            assert seen == {int(logits[t].argmax())}
        else:
            assert seen <= allowed, (t, seen - allowed)
            assert len(seen) > 1 or len(allowed) == 1
    # empirical frequencies of row 0 follow the renormalised top-k distribution
    vals, idx = (logits[0] / 0.7).topk(k)
    p = torch.softmax(vals, -1)
    top = int(idx[0])
    freq = (draws[:, 0] == top).float().mean().item()
    assert abs(freq - float(p[0])) < 0.08
    assert fab.status() == 0
    fab.close()


def test_sampling_penalties():
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(0, 1)
    V = 5000
    logits = torch.zeros(1, V, device="cuda")
    logits[0, 7] = 5.0
    logits[0, 9] = 4.0
    counts = torch.zeros(1, V, dtype=torch.int16, device="cuda")
    counts[0, 7] = 3
    pen = torch.tensor([[1.0, 0.5, 0.1]], device="cuda")     # repetition, frequency, presence
    invt = torch.zeros(1, device="cuda")                       # greedy on penalised logits: 5 - 1.5 - 0.1 = 3.4 < 4
    out = K.sample_topk(logits, fab, top_k=8, inv_temperature=invt, counts=counts, penalties=pen)
    assert int(out[0]) == 9
    fab.close()


@pytest.mark.gpu
def test_tensor_core_prefill_matches_the_decode_path_and_the_oracle():
    """A 150-token prompt through DensePrefill (chunks of 64) leaves the same caches and last-row logits as the decode kernels."""
    from ironpangu_b200.models import dense_gqa as G
    from ironpangu_b200.models.dense_prefill import DensePrefill
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = G.DenseConfig.tiny(2)
    full = G.random_full_weights(cfg, seed=0)
    fab = Fabric(0, 1)
    mk = lambda: G.DenseDecoder(cfg, G.shard_weights(cfg, full, 0, 1, "cuda"), fab, max_tokens=8, max_context=256, keep_logits=True)
    a, b = mk(), mk()
    toks = torch.randint(0, cfg.vocab, (150,), generator=torch.Generator().manual_seed(5)).to(torch.int32).cuda()
    pre = DensePrefill(a, max_rows=64, attn_rows=32)
    for s in range(0, 150, 64):
        nxt = pre.forward(toks[s:s + 64], s, 0)
    for s in range(0, 150, 8):
        n = min(8, 150 - s)
        b.tokens[:n].copy_(toks[s:s + n])
        b.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        b.slots[:n].zero_()
        b.forward(n)
    torch.cuda.synchronize()
    ref = G.forward_ref(cfg, full, toks.long())       # on the device of the tokens
    torch.testing.assert_close(a.logits[0], ref[149], rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(a.logits[0], b.logits[(150 - 1) % 8], rtol=3e-2, atol=3e-2)
    for l in range(cfg.layers):
        torch.testing.assert_close(a.k_cache[l].float(), b.k_cache[l].float(), rtol=3e-2, atol=3e-2)
    top2 = ref[149].topk(2).values
    assert int(nxt[0]) == int(ref[149].argmax()) or float(top2[0] - top2[1]) < 5e-2
    assert fab.status() == 0
    fab.close()


@pytest.mark.gpu
def test_prompt_attention_on_the_tensor_cores_for_128_wide_heads():
    """Heads of 128 columns: prompt chunks gather the context (values transposed) and run the tcgen05 attention kernel in its
    grouped-query form. Same last-row logits as the oracle and the decode kernels, same caches; decode continues from it."""
    from ironpangu_b200.models import dense_gqa as G
    from ironpangu_b200.models.dense_prefill import DensePrefill
    from ironpangu_b200.ops import prefill as P
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = G.DenseConfig(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=128, ffn=512, vocab=1024, theta=1e4)
    full = G.random_full_weights(cfg, seed=1)
    fab = Fabric(0, 1)
    mk = lambda: G.DenseDecoder(cfg, G.shard_weights(cfg, full, 0, 1, "cuda"), fab, max_tokens=8, max_context=512, keep_logits=True)
    a, b = mk(), mk()
    n = 300
    toks = torch.randint(0, cfg.vocab, (n + 3,), generator=torch.Generator().manual_seed(6)).to(torch.int32).cuda()
    pre = DensePrefill(a, max_rows=192, attn_rows=32)
    assert pre.tc_attention
    for s in range(0, n, 192):
        nxt = pre.forward(toks[s:min(n, s + 192)], s, 0)
    for s in range(0, n, 8):
        m = min(8, n - s)
        b.tokens[:m].copy_(toks[s:s + m]); b.positions[:m].copy_(torch.arange(s, s + m, dtype=torch.int32)); b.slots[:m].zero_()
        b.forward(m)
    ref = G.forward_ref(cfg, full, toks.long())
    torch.testing.assert_close(a.logits[0], ref[n - 1], rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(a.logits[0], b.logits[(n - 1) % 8], rtol=3e-2, atol=3e-2)
    for l in range(cfg.layers):
        torch.testing.assert_close(a.k_cache[l].float(), b.k_cache[l].float(), rtol=3e-2, atol=3e-2)
    # the gather itself: dense keys and transposed values of the first layer, zero tail
    rows = 320
    k = torch.full((rows, cfg.kv_heads * 128), 5.0, dtype=torch.bfloat16, device="cuda")
    vt = torch.full((cfg.kv_heads * 128, 384), 5.0, dtype=torch.bfloat16, device="cuda")
    P.gqa_ctx_gather(a.k_cache[0], a.v_cache[0], a.page_table, 0, n, k, vt, status_ptr=fab.desc.status)
    flat_k, flat_v = a.k_cache[0].view(-1, cfg.kv_heads * 128), a.v_cache[0].view(-1, cfg.kv_heads * 128)
    assert torch.equal(k[:n], flat_k[:n]) and bool((k[n:] == 0).all())
    assert torch.equal(vt[:, :n], flat_v[:n].T) and bool((vt[:, n:rows] == 0).all()) and bool((vt[:, rows:] == 5.0).all())
    # decode continues on the cache the prompt path left
    for i in range(n, n + 3):
        a.tokens[:1].copy_(toks[i:i + 1]); a.positions[:1].fill_(i); a.slots[:1].zero_()
        a.forward(1)
        torch.testing.assert_close(a.logits[0], ref[i], rtol=3e-2, atol=3e-2)
    assert fab.status() == 0
    fab.close()


@pytest.mark.gpu
def test_swiglu_rows_matches_torch():
    from ironpangu_b200.ops import decode as K
    torch.manual_seed(3)
    gu = (torch.randn(37, 2 * 264, device="cuda") * 2).to(torch.bfloat16)
    got = K.swiglu_rows(gu)
    g, u = gu[:, :264].float(), gu[:, 264:].float()
    torch.testing.assert_close(got.float(), (torch.nn.functional.silu(g) * u).to(torch.bfloat16).float(), rtol=2e-2, atol=2e-2)
    # a strided view (columns of a wider buffer) goes through the row strides
    wide = torch.zeros(5, 1024, dtype=torch.bfloat16, device="cuda")
    wide[:, :528] = gu[:5]
    torch.testing.assert_close(K.swiglu_rows(wide[:, :528]).float(), got[:5].float(), rtol=0, atol=0)

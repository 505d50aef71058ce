"""Block-scaled fp8 expert weights: quantiser, decode gate/up and down kernels against a PyTorch fp32 reference over the
dequantised weights, and the tiny model decoding over fp8 experts."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _dequant(q, s):
    K = q.shape[-1]
    w = q.view(torch.float8_e4m3fn).float()
    return w * s.repeat_interleave(128, dim=-1)[..., :K]


def rnd(*shape, scale=1.0, dtype=BF16, seed=[0]):
    seed[0] += 1
    g = torch.Generator(device="cuda").manual_seed(seed[0])
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)


def test_quantize_fp8_block_matches_reference():
    from ironpangu_b200.ops import decode as K

    for rows, Kd in ((7, 256), (5, 192), (3, 4096)):
        w = rnd(rows, Kd, scale=0.05)
        w[1] = 0
        q, s = K.quantize_fp8_block(w)
        nb = (Kd + 127) // 128
        pad = torch.zeros(rows, nb * 128, device="cuda")
        pad[:, :Kd] = w.float()
        amax = pad.view(rows, nb, 128).abs().amax(-1)
        want_s = torch.where(amax > 0, amax / torch.full_like(amax, 448.0), torch.ones_like(amax))
        assert torch.equal(s, want_s)
        want_q = (pad.view(rows, nb, 128) / want_s[..., None]).view(rows, -1)[:, :Kd].to(torch.float8_e4m3fn)
        assert torch.equal(q.view(torch.float8_e4m3fn).float(), want_q.float())
        # the representation error of a block is bounded by the fp8 step at the block's magnitude (3 mantissa bits)
        err = (_dequant(q, s) - w.float()).abs()
        assert bool((err <= amax.repeat_interleave(128, -1)[:, :Kd] * 2 ** -4 + 1e-12).all())


def test_fp8_expert_kernels_match_dequantised_reference():
    from ironpangu_b200.models import mla_moe_ref as R
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(0, 1)
    T, D, F, E, topk, Fs = 3, 256, 192, 16, 4, 48
    x, nw = rnd(T, D), rnd(D, scale=0.1) + 1
    wgu, wd = rnd(E, 2 * F, D, scale=0.05), rnd(E, D, F, scale=0.05)
    sgu, sd = rnd(2 * Fs, D, scale=0.05), rnd(D, Fs, scale=0.05)
    wr = rnd(E, D, scale=0.2, dtype=torch.float32)
    ids, wts, _ = K.router_topk(x, wr, topk, norm_w=nw, ticket_ptr=fab.ticket_ptr)
    q_gu, q_d, q_sgu, q_sd = (K.quantize_fp8_block(t) for t in (wgu, wd, sgu, sd))
    act = K.moe_gate_up_fp8(x, ids, q_gu, 0, norm_w=nw, w_shared_gu=q_sgu)
    res = rnd(T, D)
    y = K.moe_down_allreduce_fp8(act, ids, wts, q_d, 0, fab, w_shared_down=q_sd, residual=res)
    dgu, dd, dsgu, dsd = _dequant(*q_gu), _dequant(*q_d), _dequant(*q_sgu), _dequant(*q_sd)
    h = R.rmsnorm_ref(x, nw, 1e-5)
    ref = torch.zeros(T, D, device="cuda")
    for t in range(T):
        for k in range(topk):
            e = int(ids[t, k])
            gu = (h[t] @ dgu[e].T).to(BF16).float()
            a = (torch.nn.functional.silu(gu[:F]) * gu[F:]).to(BF16).float()
            torch.testing.assert_close(act[t, k].float(), a, rtol=2e-2, atol=1e-3)
            ref[t] += wts[t, k] * (a @ dd[e].T)
        gu = (h[t] @ dsgu.T).to(BF16).float()
        a = (torch.nn.functional.silu(gu[:Fs]) * gu[Fs:]).to(BF16).float()
        torch.testing.assert_close(act[t, topk, :Fs].float(), a, rtol=2e-2, atol=1e-3)
        ref[t] += a @ dsd.T
    ref = ref.to(BF16).float() + res.float()
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    assert fab.status() == 0
    fab.close()


def test_model_over_fp8_experts_tracks_the_bf16_oracle():
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_full_weights, shard_weights
    from ironpangu_b200.models.mla_moe_ref import forward_ref
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = MlaMoeConfig.tiny(2)
    full = random_full_weights(cfg, seed=0)
    fab = Fabric(0, 1)
    dec = MlaMoeDecoder(cfg, shard_weights(cfg, full, 0, 1, "cuda"), fab, max_tokens=8, max_context=64, keep_logits=True, expert_fp8=True)
    assert "layers.0.gate_up" not in dec.w and dec.w8["layers.0.gate_up"][0].dtype == torch.uint8
    toks = torch.randint(0, cfg.vocab, (16,), generator=torch.Generator().manual_seed(3))
    ref = forward_ref(cfg, full, toks.cuda())
    for s in range(0, 16, 8):
        dec.tokens[:8].copy_(toks[s:s + 8].to(torch.int32))
        dec.positions[:8].copy_(torch.arange(s, s + 8, dtype=torch.int32))
        dec.slots[:8].zero_()
        dec.forward(8)
        # fp8 weights carry 3 mantissa bits: logits follow the bf16 model loosely, the ranking of clear winners exactly
        torch.testing.assert_close(dec.logits[:8], ref[s:s + 8], rtol=0.1, atol=0.15)
    assert fab.status() == 0
    fab.close()


def test_dequantise_fp8_block_is_the_rounded_product():
    from ironpangu_b200.ops import decode as K

    for shape in ((7, 256), (3, 5, 192), (2, 4096)):
        w = rnd(*shape, scale=0.05)
        q, s = K.quantize_fp8_block(w)
        got = K.dequantize_fp8_block((q, s))
        assert got.shape == w.shape and got.dtype == BF16
        assert torch.equal(got.float(), _dequant(q, s).to(BF16).float())


def test_prompt_path_over_fp8_experts_matches_the_decode_kernels_over_the_same_weights():
    """The tensor-core prompt executor widens one layer's fp8 experts at a time; its cache rows and first token agree with a
    prompt run through the eight-row fp8 decode kernels on the same quantised weights."""
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_full_weights, shard_weights
    from ironpangu_b200.models.mla_moe_prefill import MlaMoePrefill
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = MlaMoeConfig.tiny(2)
    full = random_full_weights(cfg, seed=0)
    fab = Fabric(0, 1)
    mk = lambda: MlaMoeDecoder(cfg, shard_weights(cfg, full, 0, 1, "cuda"), fab, max_tokens=8, max_context=256, keep_logits=True, expert_fp8=True)
    a, b = mk(), mk()
    n = 150
    toks = torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(5)).to(torch.int32).cuda()
    pre = MlaMoePrefill(a, max_rows=64)
    assert pre.w8 is not None
    for s in range(0, n, 64):
        nxt = pre.forward(toks[s:s + 64], s, 0)
    for s in range(0, n, 8):
        m = min(8, n - s)
        b.tokens[:m].copy_(toks[s:s + m])
        b.positions[:m].copy_(torch.arange(s, s + m, dtype=torch.int32))
        b.slots[:m].zero_()
        b.forward(m)
    torch.cuda.synchronize()
    torch.testing.assert_close(a.logits[0], b.logits[(n - 1) % 8], rtol=5e-2, atol=5e-2)
    for l in range(cfg.layers):
        torch.testing.assert_close(a.caches[l].float(), b.caches[l].float(), rtol=5e-2, atol=5e-2)
    gap = b.logits[(n - 1) % 8].topk(2).values
    if float(gap[0] - gap[1]) > 0.1:
        assert int(nxt[0]) == int(b.logits[(n - 1) % 8].argmax())
    assert fab.status() == 0
    fab.close()

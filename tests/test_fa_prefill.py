"""The tcgen05 prompt-attention kernel against an fp32 PyTorch reference, and the MLA prompt path that uses it against the
oracle of the whole model."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _reference(q, k1, k2, v, H, kv_group, pos0, window, scale):
    """q [m, H, d1 + d2], k1 [ctx, Hkv, d1], k2 [ctx, d2] or None, v [ctx, Hkv, 128] in fp32 -> [m, H * 128]."""
    m, ctx = q.shape[0], k1.shape[0]
    d1 = k1.shape[2]
    qpos = torch.arange(pos0, pos0 + m, device=q.device)[:, None]
    key = torch.arange(ctx, device=q.device)[None, :]
    vis = key <= qpos
    if window > 0:
        vis &= key > qpos - window
    out = torch.zeros(m, H, 128, device=q.device)
    for h in range(H):
        g = h // kv_group
        s = q[:, h, :d1] @ k1[:, g].T
        if k2 is not None:
            s = s + q[:, h, d1:] @ k2.T
        s = (s * scale).masked_fill(~vis, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(m, H * 128)


@pytest.mark.parametrize("m,ctx,pos0,H,kv_group,d1,d2,window", [
    (200, 200, 0, 4, 1, 128, 64, 0),        # the multi-head-latent form: per-head key part + shared rotary part
    (130, 200, 70, 4, 1, 128, 64, 0),       # a later chunk of the same sequence
    (1, 1, 0, 2, 1, 128, 64, 0),
    (127, 127, 0, 2, 1, 128, 64, 0),
    (129, 513, 384, 2, 1, 128, 64, 0),      # tile edges on both axes
    (257, 257, 0, 3, 1, 128, 64, 96),       # sliding window: rows that no longer see the first tiles
    (300, 300, 0, 8, 4, 128, 0, 0),         # grouped-query form: four query heads per key / value head
    (96, 160, 64, 4, 2, 64, 0, 40),
    (64, 64, 0, 2, 1, 64, 64, 0),
])
def test_prompt_attention_matches_fp32(m, ctx, pos0, H, kv_group, d1, d2, window):
    from ironpangu_b200.ops import prefill as P
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(0, 1)
    g = torch.Generator(device="cuda").manual_seed(m * 7 + ctx)
    rnd = lambda *s: torch.randn(*s, generator=g, device="cuda")
    Hkv, dq = H // kv_group, d1 + d2
    q = (rnd(m, H, dq) * 1.5).to(BF16)
    k1 = rnd(ctx, Hkv, d1).to(BF16)
    k2 = rnd(ctx, d2).to(BF16) if d2 else None
    v = rnd(ctx, Hkv, 128).to(BF16)
    # operands as the prompt path lays them out: keys in rows of 256 columns per head (key part first), values transposed with one
    # column per key and junk around everything that must not be read
    k_buf = torch.full((ctx + 5, Hkv * 256), 7.0, dtype=BF16, device="cuda")
    k_buf[:ctx].view(ctx, Hkv, 256)[:, :, :d1] = k1
    ldv = (ctx + 63) // 64 * 64 + 64
    vt_buf = torch.full((Hkv * 256, ldv), -3.0, dtype=BF16, device="cuda")
    vt_buf.view(Hkv, 256, ldv)[:, 128:, :ctx] = v.permute(1, 2, 0)
    out = torch.full((m, H * 128), float("nan"), dtype=BF16, device="cuda")
    scale = 1.0 / math.sqrt(dq)
    P.fa_prefill(q.view(m, H * dq), k_buf, vt_buf, out, heads=H, q_head_stride=dq, k_head_stride=256, vt_head_stride=256, vt_row0=128,
                 d1=d1, d2=d2, k2=k2, kv_group=kv_group, ctx=ctx, pos0=pos0, scale=scale, window=window, status_ptr=fab.desc.status)
    torch.cuda.synchronize()
    assert fab.status() == 0
    want = _reference(q.float(), k1.float(), None if k2 is None else k2.float(), v.float(), H, kv_group, pos0, window, scale)
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
    fab.close()


def test_mla_prompt_path_with_tensor_core_attention_matches_oracle():
    """Flagship head shapes (nope 128, rope 64, v 128) on a narrow model: a prompt in two chunks through the tensor-core
    attention path, then decode steps on the cache it left, against the fp32 oracle of the same weights."""
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_full_weights, shard_weights
    from ironpangu_b200.models.mla_moe_prefill import MlaMoePrefill
    from ironpangu_b200.models.mla_moe_ref import forward_ref
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = MlaMoeConfig(layers=2, hidden=256, vocab=1024, heads=4, q_lora=128, kv_lora=512, nope=128, rope=64, vdim=128, experts=16,
                       expert_ffn=64, topk=4, shared_ffn=64)
    full = random_full_weights(cfg, seed=5)
    fab = Fabric(0, 1)
    dec = MlaMoeDecoder(cfg, shard_weights(cfg, full, 0, 1, "cuda"), fab, max_tokens=1, max_context=512, keep_logits=True)
    pre = MlaMoePrefill(dec, max_rows=192)
    assert pre.tc_attention
    toks = torch.randint(0, cfg.vocab, (300,), generator=torch.Generator().manual_seed(3))
    ref = forward_ref(cfg, full, toks.cuda())
    dev = toks.to(torch.int32).cuda()
    pre.forward(dev[:192], 0, 0)
    torch.testing.assert_close(dec.logits[0], ref[191], rtol=3e-2, atol=3e-2)
    pre.forward(dev[192:297], 192, 0)
    torch.testing.assert_close(dec.logits[0], ref[296], rtol=3e-2, atol=3e-2)
    # the same chunks again replay the recorded graphs (the cache rows are rewritten with the same values)
    pre.forward(dev[192:297], 192, 0)
    torch.testing.assert_close(dec.logits[0], ref[296], rtol=3e-2, atol=3e-2)
    for i in range(297, 300):
        dec.tokens.fill_(int(toks[i]))
        dec.positions.fill_(i)
        dec.forward(1)
        torch.testing.assert_close(dec.logits[0], ref[i], rtol=3e-2, atol=3e-2)
    # and the split-KV form of the same chunk agrees with the tensor-core form
    pre.tc_attention = False
    pre._graphs.clear()
    pre.forward(dev[192:297], 192, 0)
    torch.testing.assert_close(dec.logits[0], ref[296], rtol=3e-2, atol=3e-2)
    assert fab.status() == 0
    fab.close()

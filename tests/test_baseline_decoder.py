"""The library-only baseline decoder (cuBLAS + NCCL) computes the same model as the oracle."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_baseline_matches_oracle_logits():
    from baseline.nccl_cublas import NcclCublasDecoder
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, random_full_weights, shard_weights
    from ironpangu_b200.models.mla_moe_ref import forward_ref

    cfg = MlaMoeConfig.tiny(2)
    full = random_full_weights(cfg, 3)
    dec = NcclCublasDecoder(cfg, shard_weights(cfg, full, 0, 1, "cuda"), 0, 1, max_tokens=8, max_context=64, keep_logits=True)
    toks = torch.randint(0, cfg.vocab, (19,), generator=torch.Generator().manual_seed(1))
    want = forward_ref(cfg, full, toks.cuda())
    got = []
    for s in range(0, 19, 8):
        m = min(8, 19 - s)
        dec.tokens[:m].copy_(toks[s:s + m].to(torch.int32))
        dec.positions[:m].copy_(torch.arange(s, s + m, dtype=torch.int32))
        dec.forward(m)
        got.append(dec.logits[:m].clone())
    got = torch.cat(got)
    torch.testing.assert_close(got, want, rtol=3e-2, atol=3e-2)
    gap = want.topk(2, -1).values
    sure = (gap[:, 0] - gap[:, 1]) > 5e-2
    assert torch.equal(got.argmax(-1)[sure], want.argmax(-1)[sure])


def test_baseline_runs_under_the_engine_with_graphs():
    from baseline.nccl_cublas import NcclCublasDecoder
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, random_full_weights, shard_weights
    from ironpangu_b200.runtime.engine import DecodeEngine

    cfg = MlaMoeConfig.tiny(2)
    w = shard_weights(cfg, random_full_weights(cfg, 3), 0, 1, "cuda")
    prompt = torch.randint(0, cfg.vocab, (11,), generator=torch.Generator().manual_seed(2)).tolist()
    eager = DecodeEngine(NcclCublasDecoder(cfg, w, 0, 1, max_tokens=8, max_context=64))
    first = eager.prefill(prompt)
    toks = [first]
    for _ in range(5):
        eager.dec.tokens[:1].fill_(toks[-1])
        eager.dec.positions[:1].fill_(eager.pos)
        toks.append(int(eager.dec.forward(1)[0]))
        eager.pos += 1
    graphed = DecodeEngine(NcclCublasDecoder(cfg, w, 0, 1, max_tokens=8, max_context=64))
    assert graphed.generate(prompt, 6) == toks


def test_baseline_expert_paths_agree():
    """The grouped-GEMM expert path (where the library offers it) and the gather + bmm path compute the same rows."""
    from baseline.nccl_cublas import NcclCublasDecoder
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, random_full_weights, shard_weights

    cfg = MlaMoeConfig.tiny(2)
    w = shard_weights(cfg, random_full_weights(cfg, 3), 0, 1, "cuda")
    outs = {}
    for path in ("grouped_mm", "index_select+bmm"):
        dec = NcclCublasDecoder(cfg, w, 0, 1, max_tokens=8, max_context=64, keep_logits=True)
        if path == "grouped_mm" and dec.expert_path != "grouped_mm":
            pytest.skip("no grouped GEMM in the installed library for this device")
        dec.expert_path = path
        dec.tokens[:5].copy_(torch.tensor([3, 17, 99, 256, 511], dtype=torch.int32))
        dec.positions[:5].copy_(torch.arange(5, dtype=torch.int32))
        dec.forward(5)
        outs[path] = dec.logits[:5].clone()
    torch.testing.assert_close(outs["grouped_mm"], outs["index_select+bmm"], rtol=2e-2, atol=2e-2)

"""The single-launch (persistent cooperative kernel) decode step against the operator-by-operator chain and the oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair(max_tokens, layers=2, window=0, heads=8):
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_full_weights, shard_weights
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = MlaMoeConfig.tiny(layers)
    cfg.window, cfg.heads = window, heads
    full = random_full_weights(cfg, seed=0)
    fab = Fabric(0, 1)
    w = shard_weights(cfg, full, 0, 1, "cuda")
    mk = lambda persistent: MlaMoeDecoder(cfg, w, fab, max_tokens=max_tokens, max_context=128, num_slots=2, keep_logits=True,
                                          persistent=persistent)
    return cfg, full, fab, mk(False), mk(True)


def _feed(dec, toks, start, slot=0):
    n = len(toks)
    dec.tokens[:n].copy_(torch.tensor(toks, dtype=torch.int32))
    dec.positions[:n].copy_(torch.arange(start, start + n, dtype=torch.int32))
    dec.slots[:n].fill_(slot)
    dec.forward(n)
    return dec.logits[:n].clone(), dec.next_ids[:n].clone()


@pytest.mark.parametrize("window,heads", [(0, 8), (8, 8), (0, 6)])
def test_single_launch_step_matches_chain_and_oracle(window, heads):
    from ironpangu_b200.models.mla_moe_ref import forward_ref

    cfg, full, fab, chain, one = _pair(1, window=window, heads=heads)
    prompt = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(1)).tolist()
    ref = forward_ref(cfg, full, torch.tensor(prompt, device="cuda"))
    for i, t in enumerate(prompt):
        a, _ = _feed(chain, [t], i, slot=1)
        b, ids = _feed(one, [t], i, slot=1)
        torch.testing.assert_close(b[0], ref[i], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(b[0], a[0], rtol=1e-2, atol=1e-2)
        assert int(ids[0]) == int(b[0].argmax())
    assert fab.status() == 0
    fab.close()


@pytest.mark.parametrize("chunk", [2, 3, 8])
def test_single_launch_step_chunked_rows(chunk):
    """Several rows per step (chunked prefill / batched decode): rows of one sequence at consecutive positions."""
    from ironpangu_b200.models.mla_moe_ref import forward_ref

    cfg, full, fab, chain, one = _pair(8)
    prompt = torch.randint(0, cfg.vocab, (19,), generator=torch.Generator().manual_seed(2)).tolist()
    ref = forward_ref(cfg, full, torch.tensor(prompt, device="cuda"))
    for s in range(0, len(prompt), chunk):
        part = prompt[s:s + chunk]
        logits, ids = _feed(one, part, s)
        torch.testing.assert_close(logits, ref[s:s + len(part)], rtol=2e-2, atol=2e-2)
        assert ids.tolist() == logits.argmax(-1).tolist()
    assert fab.status() == 0
    fab.close()


def test_single_launch_feedback_graph_matches_chain():
    """Captured with device-side feedback, the single launch decodes the same greedy continuation as the chain;
    both forms advance the fabric's call counter identically, so they can alternate."""
    from ironpangu_b200.runtime.engine import DecodeEngine

    cfg, full, fab, chain, one = _pair(8)
    prompt = torch.randint(0, cfg.vocab, (11,), generator=torch.Generator().manual_seed(3)).tolist()
    want = DecodeEngine(chain).generate(prompt, 12)
    eng = DecodeEngine(one)
    first = eng.prefill(prompt)
    got = [first]
    one.tokens[:1].fill_(first)
    one.positions[:1].fill_(eng.pos)
    one.slots[:1].zero_()
    g = one.capture(1, feedback=True)
    for _ in range(11):
        g.replay()
        got.append(int(one.next_ids[0]))
    assert got == want
    calls = fab.calls()
    one.forward(1)
    assert fab.calls() == calls + 2 * cfg.layers + 1
    assert fab.status() == 0
    fab.close()

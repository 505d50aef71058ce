"""Definition + checkpoint -> decoder of the hybrid family: the writer's output passes the host core's inspection, the typed plan
gives back the configuration, and the tensors load bit-exactly from the offsets the plan records."""
import dataclasses

import pytest
import torch

from ironpangu_b200.models import hybrid_delta as H


def _saved(tmp_path, cfg, device="cpu"):
    w = H.random_weights(cfg, device, seed=3)
    H.save_checkpoint(tmp_path / "ck", cfg, w, shards=3)
    (tmp_path / "m.inferfabric").write_text(H.definition_text(cfg))
    return w


def test_written_checkpoint_compiles_and_round_trips(tmp_path):
    cfg = H.HybridConfig.tiny(2)
    w = _saved(tmp_path, cfg)
    plan = H.typed_plan(tmp_path / "m.inferfabric", tmp_path / "ck")
    assert plan["format"] == "inferfabric.typed-plan.v1" and len(plan["key"]) == 64
    got = H.config_of(plan, tmp_path / "ck")
    assert dataclasses.asdict(got) == dataclasses.asdict(cfg)
    loaded = H.load_weights(plan, tmp_path / "ck", "cpu", staging_bytes=4096)        # many staging rounds per tensor
    assert set(loaded) == set(w)
    for n, t in w.items():
        assert loaded[n].dtype == t.dtype and loaded[n].shape == t.shape and torch.equal(loaded[n].view(torch.uint8), t.view(torch.uint8)), n


def test_a_checkpoint_that_disagrees_with_the_definition_is_refused(tmp_path):
    from ironpangu_b200.compiler import CompileError

    cfg = H.HybridConfig.tiny(1)
    _saved(tmp_path, cfg)
    (tmp_path / "m.inferfabric").write_text(H.definition_text(dataclasses.replace(cfg, intermediate=cfg.intermediate * 2)))
    with pytest.raises((CompileError, RuntimeError, ValueError)):
        H.typed_plan(tmp_path / "m.inferfabric", tmp_path / "ck")


@pytest.mark.gpu
def test_gpu_decoder_from_a_checkpoint_equals_the_decoder_on_the_same_tensors(tmp_path):
    from ironpangu_b200.parallel.fabric import Fabric

    dev = torch.device("cuda:0")
    cfg = H.HybridConfig.tiny(1)
    w = _saved(tmp_path, cfg, dev)
    fab = Fabric(0, 1)
    a = H.HybridDecoder(cfg, w, fab, max_tokens=4, max_context=64, keep_logits=True)
    b = H.HybridDecoder.from_checkpoint(tmp_path / "m.inferfabric", tmp_path / "ck", fab, max_tokens=4, max_context=64, keep_logits=True)
    assert len(b.plan_key) == 64
    toks = torch.tensor([5, 17, 300, 2], dtype=torch.int32, device=dev)
    for d in (a, b):
        d.tokens.copy_(toks)
        d.positions.copy_(torch.arange(4, dtype=torch.int32, device=dev))
        d.slots.zero_()
        d.forward(4)
    torch.cuda.synchronize()
    assert torch.equal(a.logits, b.logits) and torch.equal(a.next_ids, b.next_ids)


@pytest.mark.gpu
def test_gpu_server_serves_a_hybrid_checkpoint(tmp_path):
    """ifab-server -> engine worker (--model hybrid --definition ... --checkpoint ...) -> the decoder built from the typed plan;
    tokens equal a greedy loop over a decoder on the same tensors."""
    import types

    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.utils.qualify_serving import ServerUnderTest

    dev = torch.device("cuda:0")
    cfg = H.HybridConfig.tiny(1)
    w = _saved(tmp_path, cfg, dev)
    args = types.SimpleNamespace(engine="worker", model="hybrid", max_num_seqs=2, max_model_len=128, prefix_cache_slots=0, gpus=1,
                                 worker_flags=f"--definition {tmp_path / 'm.inferfabric'} --checkpoint {tmp_path / 'ck'}")
    s = ServerUnderTest(args)
    try:
        prompt = [5, 17, 300, 2, 44, 9, 123, 77, 201, 3, 56]
        st, got = s.generate(prompt, 6)
        assert st == 200, got
        dec = H.HybridDecoder(cfg, w, Fabric(0, 1), max_tokens=8, max_context=128)
        seq, out = list(prompt), []
        pos = 0
        while len(out) < 6:
            chunk = seq[pos:pos + 8]
            n = len(chunk)
            dec.tokens[:n].copy_(torch.tensor(chunk, dtype=torch.int32))
            dec.positions[:n].copy_(torch.arange(pos, pos + n, dtype=torch.int32))
            dec.slots[:n].zero_()
            dec.forward(n)
            pos += n
            if pos == len(seq):
                t = int(dec.next_ids[n - 1])
                out.append(t)
                seq.append(t)
        assert got["token_ids"] == out
    finally:
        s.close()

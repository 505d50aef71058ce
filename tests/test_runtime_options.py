"""Typed runtime options: environment + --set parsing, validation, recording."""
import json

import pytest

from ironpangu_b200.runtime.options import RuntimeOptions


def test_defaults_env_and_sets_in_that_order():
    env = {"IFAB_KV_INT8": "1", "IFAB_PREFILL_CHUNK": "256", "IFAB_ENGINE_SOCKET": "/tmp/x.sock", "HOME": "/"}
    o = RuntimeOptions.from_env(env, ["prefill-chunk=512", "fused_head=off", "audit_dir=/tmp/a"])
    assert o.kv_int8 is True and o.prefill_chunk == 512 and o.fused_head is False and o.audit_dir == "/tmp/a"
    assert o.decode_graph is True and o.spin_limit == 4_000_000                      # untouched defaults
    assert o.changed() == {"kv_int8": True, "prefill_chunk": 512, "fused_head": False, "audit_dir": "/tmp/a"}
    assert json.loads(o.to_json())["prefill_chunk"] == 512
    assert RuntimeOptions.from_env({}, ["fused_head=auto"]).fused_head is None


def test_unknown_names_and_bad_values_are_errors():
    with pytest.raises(KeyError, match="decode_grpah"):
        RuntimeOptions.from_env({}, ["decode_grpah=0"])
    with pytest.raises(ValueError, match="not a boolean"):
        RuntimeOptions.from_env({"IFAB_PDL": "maybe"})
    with pytest.raises(ValueError, match="not an integer"):
        RuntimeOptions.from_env({}, ["spin_limit=lots"])
    with pytest.raises(ValueError, match="name=value"):
        RuntimeOptions.from_env({}, ["kv_int8"])
    with pytest.raises(ValueError, match="spin_limit"):
        RuntimeOptions.from_env({}, ["spin_limit=5"])
    with pytest.raises(ValueError, match="kv_int8"):
        RuntimeOptions.from_env({}, ["kv_int8=1", "fused_head=1"])


def test_rank_agreement_modes_and_boolean_spellings():
    from ironpangu_b200.runtime.options import RuntimeOptions
    assert RuntimeOptions().validate().rank_agreement == "deferred"
    for text, want in (("0", "off"), ("false", "off"), ("1", "strict"), ("on", "strict"), ("Strict", "strict"), ("deferred", "deferred")):
        assert RuntimeOptions.from_env({"IFAB_RANK_AGREEMENT": text}).rank_agreement == want
    with pytest.raises(ValueError):
        RuntimeOptions.from_env({}, ["rank_agreement=sometimes"])
    assert RuntimeOptions.from_env({}, ["sequence_parallel=1"]).sequence_parallel is True

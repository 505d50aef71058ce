"""Config audit of the MLA + MoE family: layer forms, features, required operations with their kernels, and the malformed
configs it refuses."""
import json

import pytest

from ironpangu_b200 import compiler

BASE = {
    "model_type": "pangu_v2_moe", "hidden_size": 4096, "intermediate_size": 12288, "vocab_size": 153600, "num_attention_heads": 32,
    "kv_lora_rank": 512, "qk_nope_head_dim": 128, "qk_rope_head_dim": 64, "v_head_dim": 128, "max_position_embeddings": 131072,
    "num_hidden_layers": 6, "num_nextn_predict_layers": 1, "first_k_dense_replace": 2, "n_routed_experts": 96, "num_experts_per_tok": 8,
    "moe_intermediate_size": 1536, "n_shared_experts": 1, "norm_topk_prob": True, "q_lora_rank": 1536,
    "swa_layers": [1, 3], "sliding_window_list": [2048, 512], "index_topk": 2048, "index_n_heads": 24, "index_head_dim": 128,
    "use_mome": True, "router_sliding_window": 3, "mhc_num_stream": 4, "mhc_recur_norm": 1, "mhc_use_gamma": True, "use_mhc": False,
    "cla_explicit_mapping": {"4": 2}, "indexer_types": ["full", "full", "shared", "full", "shared", "full"], "param_sink_number": 16,
    "quantization_config": {
        "quant_method": "compressed-tensors", "quantize": "w8a8_dynamic", "format": "int-quantized", "quantization_status": "compressed",
        "config_groups": {"group_0": {"targets": ["Linear"],
                                      "weights": {"num_bits": 8, "type": "int", "symmetric": True, "strategy": "channel", "dynamic": False, "group_size": None},
                                      "input_activations": {"num_bits": 8, "type": "int", "symmetric": True, "strategy": "token", "dynamic": True}}},
        "ignore": ["lm_head", "model.layers.0.mlp.gate", "lm_head"], "kv_cache_scheme": None},
    "some_future_field": [1, 2, 3],
}


def audit(tmp_path, cfg):
    p = tmp_path / "config.json"
    p.write_text(cfg if isinstance(cfg, str) else json.dumps(cfg))
    return compiler.cli("inspect-config", str(p))


def test_layer_forms_features_and_operations(tmp_path):
    r = audit(tmp_path, BASE)
    assert r.returncode == 0, r.stderr
    a = json.loads(r.stdout)
    assert a["format"] == "ifab.config-audit.v1" and a["executable"] is False and len(a["config_sha256"]) == 64
    assert a["config"]["some_future_field"] == [1, 2, 3]                                  # unknown fields are preserved
    L = a["layers"]
    assert [l["attention"] for l in L] == ["sparse_mla", "sliding_window_mla", "sparse_mla", "sliding_window_mla", "sparse_mla", "sparse_mla"]
    assert [l["sliding_window"] for l in L] == [None, 2048, None, 512, None, None]
    assert [l["feed_forward"] for l in L] == ["dense", "dense", "moe", "moe", "moe", "moe"]
    assert L[4]["cache_source_layer"] == 2 and L[2]["indexer_mode"] == "shared"
    assert a["features"] == {"cross_layer_cache_reuse_declared": True, "index_sharing_declared": True, "learned_sinks": True, "mhc": True,
                             "moe": True, "mome": True, "mtp_declared": True, "quantization_declared": True, "sparse_indexer": True}
    ops = {o["operation"]: o["kernel"] for o in a["required_operations"]}
    assert ops["mhc_pre"] == "ifab_mhc_pre" and ops["sparse_topk"] == "ifab_sparse_index" and ops["causal_channel_convolution"] == "ifab_mome"
    assert set(a["operations_without_a_kernel"]) == {"shared_layer_cache_views", "shared_sparse_indices", "indexer_cache_append", "sparse_attention"}
    assert any("use_mhc disagrees" in w for w in a["warnings"]) and len(a["unresolved"]) == 5
    assert a["quantization"]["declared"] and a["quantization"]["scheme"] == "w8a8_dynamic" and a["quantization"]["ignore"] == ["lm_head", "model.layers.0.mlp.gate"]
    # a plain dense config: no optional mechanism, no optional operation
    plain = {k: BASE[k] for k in ("model_type", "hidden_size", "intermediate_size", "vocab_size", "num_attention_heads", "kv_lora_rank",
                                  "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim", "max_position_embeddings", "num_hidden_layers")}
    b = json.loads(audit(tmp_path, plain).stdout)
    assert b["quantization"] == {"declared": False} and not any(b["features"].values()) and all(l["attention"] == "full_mla" and l["feed_forward"] == "dense" for l in b["layers"])
    assert len(b["required_operations"]) == 10 and b["operations_without_a_kernel"] == []


@pytest.mark.parametrize("change,message", [
    ({"model_type": "llama"}, "model_type"),
    ({"hidden_size": 0}, "hidden_size must be positive"),
    ({"num_experts_per_tok": 200}, "exceeds n_routed_experts"),
    ({"first_k_dense_replace": 9}, "exceeds the layer count"),
    ({"sliding_window_list": [2048]}, "one window per entry"),
    ({"swa_layers": [1, 1], "sliding_window_list": [8, 8]}, "twice"),
    ({"swa_layers": [9], "sliding_window_list": [8]}, "outside the model"),
    ({"cla_explicit_mapping": {"2": 4}}, "come after its source"),
    ({"cla_explicit_mapping": [[4, 2], [4, 1]]}, "appear once"),
    ({"indexer_types": ["full"]}, "cover every layer"),
    ({"mhc_use_gamma": False}, "mhc_use_gamma"),
    ({"mhc_num_stream": 0}, "between 1 and 1024"),
    ({"index_n_heads": None}, "index_n_heads is missing"),
    ({"use_mome": "yes"}, "true or false"),
    ({"quantization_config": {"quant_method": "awq"}}, "quant_method must be"),
    ({"quantization_config": {**BASE["quantization_config"], "ignore": ["model.layers.*.mlp"]}}, "no patterns"),
    ({"quantization_config": {**BASE["quantization_config"], "kv_cache_scheme": {"num_bits": 8}}}, "quantised cache scheme"),
    ({"quantization_config": {**BASE["quantization_config"], "config_groups": {}}}, "exactly one config group"),
])
def test_malformed_configs_are_refused(tmp_path, change, message):
    r = audit(tmp_path, {**BASE, **change})
    assert r.returncode != 0 and message in r.stderr, r.stderr


def test_duplicate_keys_are_refused(tmp_path):
    text = json.dumps(BASE)[:-1] + ', "hidden_size": 8192}'
    r = audit(tmp_path, text)
    assert r.returncode != 0 and "duplicate key" in r.stderr

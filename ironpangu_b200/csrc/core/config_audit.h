// Audit of a checkpoint's config.json for the multi-head-latent-attention + routed-experts family (model_type
// `pangu_v2_moe` / `openpangu_v2`): which layer runs which attention form and feed-forward form, which optional mechanisms
// the config switches on, which operations - and which kernels of this library - a decoder for it needs, and what the
// audit cannot vouch for. It reads metadata only: the result is a planning document (`executable: false`), never a program.
//
//   layer summary   attention = sliding_window_mla for layers listed in `swa_layers` (with their window), else sparse_mla when
//                   `index_topk` > 0, else full_mla; feed_forward = dense for the first `first_k_dense_replace` layers, moe after;
//                   cross-layer cache reuse (`cla_explicit_mapping`: a reuse layer names an EARLIER source layer, each once);
//                   per-layer indexer mode (`indexer_types`)
//   features        moe, mome, mhc (more than one residual stream), learned_sinks, sparse_indexer, mtp_declared,
//                   quantization_declared, cross_layer_cache_reuse_declared, index_sharing_declared
//   operations      the list above turned into operation names, each with the kernel entry point that implements it here
//                   (empty when this library has none: a gap the caller must close before compiling)
//
// Malformed configs are errors (missing / non-positive sizes, top-k above the expert count, windows without layers,
// out-of-range or duplicate layer indices, a reuse layer that does not come after its source ...); JSON is parsed with
// duplicate keys rejected and bounded nesting. Reference: crates/inferfabric-compiler/src/openpangu/mod.rs:84-324.
#pragma once
#include "base.h"

namespace ifab::config_audit {

constexpr size_t kMaxConfigBytes = 1 << 20;

Json audit(std::string_view config_json);

}  // namespace ifab::config_audit

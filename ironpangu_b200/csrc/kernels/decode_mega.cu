// Host entry of the persistent decode-step kernel (decode_mega.cuh): argument checks, translation of the C
// descriptor into kernel parameters, dispatch on the row count and the head-group width.
#include <algorithm>

#include "decode_mega_kernel.cuh"

namespace ifab::mega {
extern template int launch_step<1, 1>(Params&, cudaStream_t);
extern template int launch_step<2, 1>(Params&, cudaStream_t);
extern template int launch_step<4, 1>(Params&, cudaStream_t);
extern template int launch_step<8, 1>(Params&, cudaStream_t);
}  // namespace ifab::mega

using namespace ifab;
using namespace ifab::mega;

static_assert(sizeof(Layer) == sizeof(IfabMlaMoeLayer), "layer table layout");

extern "C" int ifab_mla_moe_decode_step(const IfabMlaMoeStep* s, int T, const IfabFabric* fab, void* stream) {
  if (s == nullptr || T < 1 || T > 8) return -1;
  if (s->hidden % 8 || s->q_lora % 8 || s->expert_ffn % 8 || s->shared_ffn_local % 8 || s->expert_ffn % 2) return -1;
  if (s->rope != ROPE || s->nope > 256 || s->nope % 8 || s->vdim % 4 || s->experts > 256 || s->topk > MAX_TOPK) return -1;
  if (s->topk > s->experts || s->max_splits < 1 || s->max_splits > 64 || s->keys_per_split < 8) return -1;
  if (s->shared_ffn_local > s->expert_ffn || s->heads_local < 1 || s->bar == nullptr) return -1;
  Params p;
  p.layers = reinterpret_cast<const Layer*>(s->layers);
  p.n_layers = s->n_layers; p.D = s->hidden; p.hl = s->heads_local; p.q_lora = s->q_lora; p.nope = s->nope; p.rope = s->rope;
  p.vdim = s->vdim; p.E = s->experts; p.el = s->experts_local; p.e0 = s->expert0; p.topk = s->topk; p.F = s->expert_ffn;
  p.Fs = s->shared_ffn_local; p.vl = s->vocab_local; p.vocab_offset = s->vocab_offset; p.vocab = s->vocab;
  p.scoring = s->scoring; p.renorm = s->renorm; p.window = s->window; p.n_sinks = s->n_sinks; p.page_tokens = s->page_tokens;
  p.max_pages = s->max_pages; p.num_pages = s->num_pages; p.kps = s->keys_per_split; p.max_splits = s->max_splits;
  p.route_scale = s->route_scale; p.eps = s->eps; p.theta = s->theta; p.attn_scale = s->attn_scale;
  p.embed = (const bf16*)s->embed; p.final_norm = (const bf16*)s->final_norm; p.lm_head = (const bf16*)s->lm_head;
  p.tokens = s->tokens; p.positions = s->positions; p.slots = s->slots; p.page_table = s->page_table;
  p.x = (bf16*)s->x; p.qkv = (bf16*)s->qkv; p.q = (bf16*)s->q; p.q_lat = (bf16*)s->q_lat; p.attn = (bf16*)s->attn;
  p.act = (bf16*)s->act; p.scratch = s->scratch; p.router_logits = s->router_logits; p.route_ids = s->route_ids;
  p.route_w = s->route_w; p.partial = (float2*)s->partial; p.next_ids = s->next_ids; p.next_vals = s->next_vals;
  p.logits = s->logits; p.bar = s->bar; p.trace = (unsigned long long*)s->trace; p.T_live = T; p.feedback = s->feedback;
  if (int rc = fabric_view(fab, &p.fv)) return rc;
  p.seq = fab->seq;
  p.spin_limit = fab->spin_limit;
  if ((size_t)fab->world * T * s->hidden * sizeof(uint64_t) > fab->ll_half_bytes) return -3;
  if ((size_t)fab->world > fab->flag_half_words) return -4;
  cudaStream_t st = (cudaStream_t)stream;
#define IFAB_STEP(TT) return launch_step<TT, 1>(p, st);
  if (T <= 1) IFAB_STEP(1)
  if (T <= 2) IFAB_STEP(2)
  if (T <= 4) IFAB_STEP(4)
  IFAB_STEP(8)
#undef IFAB_STEP
}

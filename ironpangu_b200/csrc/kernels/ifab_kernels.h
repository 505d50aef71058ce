/* C ABI of the sm_100a kernel library (libifab_kernels.so).
 *
 * Every entry point takes raw device pointers plus a CUDA stream handle and returns 0 on success,
 * a negative value for a rejected argument, or a positive cudaError_t from the launch. Nothing here
 * allocates device memory except the functions in the "fabric" group, which own the symmetric heap.
 * All matrices are row-major; weights are [out_features, in_features] with in_features contiguous.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IFAB_MAX_RANKS 8

/* Symmetric-heap descriptor of one rank (host struct, passed by pointer). data[r]/flags[r] are rank
 * r's staging area and flag words as mapped into this process; entries >= world are ignored. */
typedef struct IfabFabric {
  void* data[IFAB_MAX_RANKS];
  uint64_t* flags[IFAB_MAX_RANKS];
  uint64_t* seq;      /* local: number of fused-collective launches completed */
  uint32_t* done;     /* local: CTA ticket counter of the running launch */
  uint32_t* status;   /* local: IFAB_STATUS_* bits, sticky until the host clears them */
  int32_t rank;
  int32_t world;
  uint32_t spin_limit;
  uint32_t data_half_bytes;
  uint32_t flag_half_words;
  uint32_t ll_half_bytes;  /* one parity half of the tagged-store area (8 bytes per exchanged f32) */
  uint64_t ll_offset;      /* byte offset of that area from data[r]; it is used by nothing else, because a
                              reader takes any 8-byte word whose high half equals the call number as valid */
  void* mc;                /* NVLink multicast address of the same block (a store to it lands in every rank's copy, a
                              multimem.ld_reduce returns the sum over the ranks), or NULL: plain peer loads / stores */
} IfabFabric;

/* ---- fabric: symmetric heap over CUDA IPC (one process per GPU) ---- */
int ifab_device_alloc(void** out, uint64_t bytes);           /* cudaMalloc + zero fill */
int ifab_device_free(void* p);
int ifab_ipc_export(void* p, unsigned char handle[64]);      /* cudaIpcGetMemHandle */
int ifab_ipc_import(const unsigned char handle[64], void** out);
int ifab_ipc_close(void* p);
int ifab_set_device(int device);
int ifab_peek(void* dst_host, const void* src_device, uint64_t bytes);   /* synchronous small copies of */
int ifab_poke(void* dst_device, const void* src_host, uint64_t bytes);   /* control words               */
const char* ifab_error_string(int code);

/* ---- elementwise / layout ---- */
int ifab_embedding_bf16(const int32_t* ids, const void* table, void* out, int T, int D, int vocab, uint32_t* status,
                        void* stream);
int ifab_rmsnorm_bf16(const void* x, long ldx, const void* w, void* y, long ldy, int T, int D, float eps,
                      int zero_centered, void* stream);

/* ---- decode linears (T <= 8 per tile; larger T loops over tiles) ---- */
int ifab_gemv_bf16(const void* x, long ldx, const void* w, const void* norm_w, float eps, int zero_centered,
                   const void* residual, long ldr, void* y, long ldy, int out_f32, int T, int N, int K, int mode,
                   void* stream);
int ifab_gemv_allreduce_bf16(const void* x, long ldx, const void* w, const void* residual, long ldr, void* y, long ldy,
                             void* y_f32, int T, int N, int K, const IfabFabric* fab, void* stream);

/* ---- block-scaled fp8 (e4m3, one f32 scale per 1 x 128 block of a row) expert weights (decode_moe_fp8.cu) ---- */
/* w: bf16 [rows, K] (row stride ldw) -> q: u8 [rows, K], scales: f32 [rows, ceil(K / 128)] */
int ifab_quantize_fp8_block(const void* w, long ldw, long rows, int K, void* q, float* scales, void* stream);
/* the inverse, rounded to bf16 -> out: bf16 [rows, K] contiguous; K % 16 == 0 (the prompt path widens one layer's experts at a time) */
int ifab_dequantize_fp8_block(const void* q, const float* scales, long rows, int K, void* out, void* stream);
int ifab_moe_gate_up_decode_fp8(const void* x, long ldx, const void* norm_w, float eps, const int32_t* ids, int T, int D, int F, int topk, int e0,
                                int e_local, const void* w_gu, const float* s_gu, const void* w_shared_gu, const float* s_shared_gu, int Fs, void* act,
                                void* stream);
int ifab_moe_down_allreduce_decode_fp8(const void* act, const int32_t* ids, const float* wts, int T, int D, int F, int topk, int e0, int e_local,
                                       const void* w_down, const float* s_down, const void* w_shared_down, const float* s_shared_down, int Fs,
                                       const void* residual, long ldr, void* y, long ldy, const IfabFabric* fab, void* stream);

/* ---- tensor-core GEMM (tcgen05 + TMEM + TMA): C[M,N] = A[M,K] * B[N,K]^T (+ residual) ---- */
int ifab_gemm_bf16(const void* a, long lda, const void* b, long ldb, void* c, long ldc, int out_f32, const void* residual,
                   long ldr, int M, int N, int K, uint32_t* status, void* stream);

/* the same on CTA pairs (tcgen05.mma cta_group::2, 256 x 256 tiles, each CTA loads half of A and half of B); N % 32 == 0 */
int ifab_gemm_bf16_2sm(const void* a, long lda, const void* b, long ldb, void* c, long ldc, int out_f32, const void* residual,
                       long ldr, int M, int N, int K, uint32_t* status, void* stream);

/* CTA pairs, persistent grid (one pair per SM pair), two accumulators in tensor memory: the epilogue of a tile runs under the next tile's MMAs */
int ifab_gemm_bf16_2sm_persistent(const void* a, long lda, const void* b, long ldb, void* c, long ldc, int out_f32, const void* residual,
                                  long ldr, int M, int N, int K, uint32_t* status, void* stream);

/* packed gate / up projection of a SwiGLU block on CTA pairs: b = [gate rows | up rows] ([2F, K]), c[M, F] = silu(a gate^T) * (a up^T) */
int ifab_gemm_swiglu_bf16_2sm(const void* a, long lda, const void* b, long ldb, void* c, long ldc, int M, int F, int K, uint32_t* status,
                              void* stream);

int ifab_gemm_allreduce_bf16(const void* a, long lda, const void* b, long ldb, void* const* out_peers, long ldc, const void* residual,
                             long ldr, int M, int N, int K, const IfabFabric* fab, void* stream);

/* column-parallel GEMM fused with the all-gather of its row-sharded activations: C[world*rows_local, N] = gather(A_r) * B^T.
 * a_peers[r] = rank r's [rows_local, K] shard in symmetric memory as mapped here (remote tiles are copied once with peer
 * loads into `staged` [M, K] and then read by TMA; no multicast); flag_peers[r] = rank r's u64[8] flag row; tile_count =
 * local u64 [M / 128], zeroed once; `epoch` starts at 1 and grows by one per call; alternate two A buffers. */
int ifab_allgather_gemm_bf16(void* const* a_peers, long lda, const void* b, long ldb, void* c, long ldc, int rows_local, int N,
                             int K, int world, int rank, void* const* flag_peers, void* staged, long lds, void* tile_count,
                             uint64_t epoch, uint32_t* status, void* stream);

/* ---- prefill path: grouped expert GEMM (tcgen05) and its routing plumbing; all sizes are device-side counts ---- */
/* mode 0: C[rows, N] = A . B[e]^T; mode 1: N = 2F (gate rows then up rows), C[rows, F] = silu(gate) * up.
 * tiles: max_tiles x int4 {expert, first row, valid rows, 0}; *num_tiles of them are valid (written by ifab_moe_dispatch). */
int ifab_grouped_gemm_bf16(const void* a, long lda, int rows_max, const void* b, int experts, int N, int K,
                           const int32_t* tiles, const int32_t* num_tiles, int max_tiles, void* c, long ldc, int mode,
                           uint32_t* status, void* stream);
/* router for any number of rows (blocks of 8 per CTA); xn (optional) receives the RMS-normalised rows */
int ifab_router_block(const void* x, long ldx, const void* norm_w, float eps, const float* w_router, const float* bias,
                      float* logits, int32_t* ids, float* wts, void* xn, long ldxn, int M, int D, int E, int topk,
                      int scoring, int renorm, float scale, void* stream);
int ifab_moe_dispatch(const int32_t* ids, int M, int topk, int e0, int e_local, int32_t* counts, int32_t* route_row,
                      int32_t* perm_token, int32_t* tiles, int32_t* num_tiles, int32_t* total_rows, int max_tiles,
                      void* stream);
int ifab_moe_gather(const void* xn, long ldxn, const int32_t* perm_token, const int32_t* total_rows, void* xp, long ldxp,
                    int D, int rows_max, void* stream);
int ifab_moe_combine(const void* y, long ldy, const int32_t* route_row, const float* wts, int M, int topk, int D,
                     const void* shared, long lds, const void* residual, long ldr, float* out_f32, void* out, long ldo,
                     void* stream);
int ifab_mla_q_rope(const void* q, long ldq, const int32_t* positions, void* q_lat, int T, int H, int nope, int rope,
                    float theta, void* stream);
int ifab_mla_merge(const float* scratch, const int32_t* positions, int n_sinks, int window, int keys_per_split,
                   int max_splits, int T, int H, void* o_lat, void* stream);
/* one-shot pull all-reduce of f32 [rows, D] partials held in symmetric memory (parts[r] = rank r's buffer as mapped here),
 * + residual, bf16 out. The caller alternates two sets of partial buffers between consecutive calls. */
/* ---- prompt attention on the tensor cores (tcgen05): one sequence, consecutive positions, causal (+ sliding window) ----
 * q: [m, ...] head h at columns h * q_head_stride + [0, d1 + d2); k: [ctx, ...] key head g = h / kv_group at columns
 * g * k_head_stride + [0, d1); k2: [ctx, d2] key columns shared by all heads (NULL when d2 = 0); vt: transposed values, key head g
 * at rows g * vt_head_stride + vt_row0 + [0, 128), one column per key (ldvt >= ctx); out: [m, H * 128].
 * d1 in {64, 128}, d2 in {0, 64}; rows of q are positions pos0 .. pos0 + m - 1 and pos0 + m <= ctx. */
int ifab_fa_prefill_bf16(const void* q, long ldq, int q_head_stride, const void* k, long ldk, int k_head_stride, const void* k2, long ldk2,
                         const void* vt, long ldvt, int vt_head_stride, int vt_row0, int vt_rows, void* out, long ldo, int m, int ctx, int H,
                         int kv_group, int d1, int d2, int pos0, int window, float scale, uint32_t* status, void* stream);
int ifab_mla_q_rope_inplace(void* q, long ldq, const int32_t* positions, int T, int H, int nope, int rope, float theta, void* stream);
int ifab_mla_ctx_gather(const void* cache, const int32_t* page_table, int slot, int max_pages, int page_tokens, int num_pages, int ctx,
                        int rows, void* lat, void* pe, uint32_t* status, void* stream);
int ifab_allreduce_rows(const void* const* parts, const void* residual, long ldr, void* out, long ldo, long rows, int D,
                        const IfabFabric* fab, void* stream);
/* NVLS (NVLink multicast) form: two-shot - each rank reduces 1/world of the buffer with multimem.ld_reduce and writes the
 * sums back to every copy with multimem.st; the buffer holds this rank's partial on entry and the sums on exit. */
int ifab_allreduce_rows_nvls(void* part_local, void* part_mc, const void* residual, long ldr, void* out, long ldo, long rows, int D,
                             uint32_t* arrive, const IfabFabric* fab, void* stream);

/* ---- expert parallelism with sharded tokens: dispatch / combine all-to-all over peer memory (ep_a2a.cu) ----
 * `*_peers` arrays hold `world` pointers into the symmetric buffers of every rank as mapped here: recv / ret bf16 [W*cap, D],
 * meta int32 [W*cap, 2], ctl = 2 x 8 u64 flags + 8 i32 counts. `epoch` grows by one per exchange, identically on all ranks. */
int ifab_ep_dispatch(const void* xn, long ldxn, const int32_t* ids, int M, int topk, int D, int e_local, int world, int rank, int cap,
                     int32_t* send_idx, void* const* recv_peers, void* const* meta_peers, void* const* ctl_peers, uint32_t* ticket,
                     int32_t* dst_count, uint64_t epoch, uint32_t* status, void* stream);
int ifab_ep_plan(const void* meta, void* ctl, int world, int cap, int e_local, int32_t* perm, int32_t* tiles, int32_t* num_tiles,
                 int32_t* total_rows, int max_tiles, uint64_t epoch, uint32_t spin_limit, uint32_t* status, void* stream);
int ifab_ep_gather(const void* recv, const int32_t* perm, const int32_t* total_rows, void* xp, long ldxp, int D, int rows_max, void* stream);
int ifab_ep_return(const void* y, long ldy, const int32_t* perm, const int32_t* total_rows, int D, int cap, int world, int rank, int rows_max,
                   void* const* ret_peers, void* const* ctl_peers, uint32_t* ticket, uint64_t epoch, void* stream);
int ifab_ep_combine(const void* ret, void* ctl, const int32_t* ids, const int32_t* send_idx, const float* wts, int M, int topk, int D,
                    int e_local, int world, int cap, const void* shared, long lds, const void* residual, long ldr, void* out, long ldo,
                    uint64_t epoch, uint32_t spin_limit, uint32_t* status, void* stream);

/* ---- MoE decode path (owner-local expert parallelism) ---- */
int ifab_router_topk(const void* x, long ldx, const void* norm_w, float eps, const float* w_router, const float* bias,
                     float* logits, int32_t* ids, float* wts, int T, int D, int E, int topk, int scoring, int renorm,
                     float scale, uint32_t* ticket, void* xn, long ldxn, void* stream);
int ifab_moe_gate_up_decode(const void* x, long ldx, const void* norm_w, float eps, const int32_t* ids, int T, int D,
                            int F, int topk, int e0, int e_local, const void* w_gu, const void* w_shared_gu, int Fs,
                            void* act, void* stream);
int ifab_moe_down_allreduce_decode(const void* act, const int32_t* ids, const float* wts, int T, int D, int F, int topk,
                                   int e0, int e_local, const void* w_down, const void* w_shared_down, int Fs,
                                   const void* residual, long ldr, void* y, long ldy, const IfabFabric* fab,
                                   void* stream);

/* Router + shared and routed gate/up + down + all-reduce of one decode layer as ONE launch (T = 1 or 2 rows, F <= 1536).
 * The grid is sized to be resident at once; two in-grid signals (bounded waits) stand where the three kernels above
 * have kernel boundaries. Results are bit-identical to ifab_router_topk -> ifab_moe_gate_up_decode ->
 * ifab_moe_down_allreduce_decode. sync_words: 16 + 8 * T * E zero-initialised bytes (8-byte aligned) owned by the caller,
 * one set per stream;
 * y = x + reduced expert output, y may alias x. logits / ids / wts receive the router's outputs. */
int ifab_moe_block_decode(const void* x, long ldx, const void* norm_w, float eps, const float* w_router, const float* bias,
                          int E, int topk, int scoring, int renorm, float route_scale, const void* w_gu,
                          const void* w_shared_gu, const void* w_down, const void* w_shared_down, int T, int D, int F,
                          int Fs, int e0, int e_local, float* logits, int32_t* ids, float* wts, void* act, void* y,
                          long ldy, uint32_t* sync_words, const IfabFabric* fab, void* stream);

/* ---- lm_head + vocab-sharded greedy sampling ---- */
int ifab_lm_head_argmax(const void* x, long ldx, const void* norm_w, float eps, const void* w, float* logits,
                        int T, int V_local, int K, int vocab_offset, void* partial /* >= grid*T*8 bytes */,
                        uint64_t partial_bytes, int32_t* out_ids, float* out_vals, const IfabFabric* fab,
                        void* stream);

/* ---- sampling on vocabulary-sharded logits: temperature, penalties, top-k <= 64, min-p, top-p, counter-based draw ---- */
int ifab_sample_topk(const float* logits, long ld, int T, int V_local, int vocab_offset, int top_k,
                     const int32_t* top_k_rows /* optional [T]: per-row k <= top_k */,
                     const float* inv_temperature, const float* top_p, const float* min_p, const int16_t* counts, long ldc,
                     const float* penalties, const uint64_t* seeds, uint64_t* counters, void* scratch, uint64_t scratch_bytes,
                     int32_t* out_ids, float* out_probs, const IfabFabric* fab, void* stream);

/* ---- MLA (multi-head latent attention) decode path ---- */
int ifab_mla_kv_write(const void* kv, long ldkv, const void* norm_w, float eps, float theta, const int32_t* positions,
                      const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens, void* cache,
                      int num_pages, int T, int latent, int rope, uint32_t* status, void* stream);
/* the same with the rotary columns in rows of their own (latent_rows [T, >= latent], rope_rows [T, >= rope]) */
int ifab_mla_kv_write_split(const void* latent_rows, long ldl, const void* rope_rows, long ldr, const void* norm_w, float eps, float theta,
                            const int32_t* positions, const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens,
                            void* cache, int num_pages, int T, int latent, int rope, uint32_t* status, void* stream);
int ifab_mla_q_absorb(const void* q, long ldq, const void* w_kvb, float theta, const int32_t* positions, void* q_lat,
                      int T, int H, int nope, int rope, int latent, int vdim, void* stream);
int ifab_mla_decode_attention(const void* q_lat, const void* cache, const int32_t* positions, const int32_t* slots,
                              const int32_t* page_table, int max_pages, int page_tokens, int num_pages,
                              const void* sinks, int n_sinks, int window, float scale, int T, int H, int latent,
                              int rope, int keys_per_split, int max_splits, float* scratch, uint64_t scratch_bytes,
                              const void* w_kvb, int nope, int vdim, void* out, long ldo, uint32_t* status,
                              void* stream);

/* The attention half of an MLA decode layer as one launch (a cluster of 8 CTAs per head): cache write, q_b, absorb, attention
 * over the paged latent cache and value up-projection. qkv: [T, q_lora + 576] (output of the qkv_a linear); w_qb: [H * (nope + 64),
 * q_lora]; w_kvb: [H, nope + vdim, 512]; out: [T, H * vdim]. T <= 8, bf16 cache. */
int ifab_mla_head_decode(const void* qkv, long ldqkv, const void* q_norm, const void* kv_norm, float eps, float theta,
                         const void* w_qb, const void* w_kvb, void* cache, const int32_t* positions, const int32_t* slots,
                         const int32_t* page_table, int max_pages, int page_tokens, int num_pages, const void* sinks,
                         int n_sinks, int window, float scale, int T, int H, int q_lora, int nope, int vdim, void* out,
                         long ldo, uint32_t* status, void* stream);

/* The same, and while it runs its CTAs request up to three byte ranges (weights of the layer's later kernels) into L2. */
int ifab_mla_head_decode_pf(const void* qkv, long ldqkv, const void* q_norm, const void* kv_norm, float eps, float theta,
                            const void* w_qb, const void* w_kvb, void* cache, const int32_t* positions, const int32_t* slots,
                            const int32_t* page_table, int max_pages, int page_tokens, int num_pages, const void* sinks,
                            int n_sinks, int window, float scale, int T, int H, int q_lora, int nope, int vdim, void* out,
                            long ldo, uint32_t* status, const void* pf0, uint64_t pf0_bytes, const void* pf1, uint64_t pf1_bytes,
                            const void* pf2, uint64_t pf2_bytes, void* stream);

/* ---- row operators shared by compiled programs (hybrid_ops.cu) ---- */
/* Half-rotation RoPE over the first rotary_dim columns of every head of a row; the other columns are copied. */
int ifab_rope_prefix(const void* x, long ldx, const int32_t* positions, void* y, long ldy, int T, int heads, int head_dim, int rotary_dim,
                     float theta, void* stream);
/* y = a + b over [rows, n] bf16 (f32 sum, one rounding). */
int ifab_add_rows(const void* a, long lda, const void* b, long ldb, void* y, long ldy, int rows, int n, void* stream);
/* y = silu(gate) * up over [rows, n] bf16. */
int ifab_swiglu_pair(const void* gate, long ldg, const void* up, long ldu, void* y, long ldy, int rows, int n, void* stream);

/* ---- hyper-connection / hybrid-model operators (hc_ops.cu); all mixing arithmetic in f32 ---- */
/* causal depthwise conv with residual; w f32 [C_total, taps] (this rank's channels start at c_offset); state bf16 [slots, taps-1, C] */
int ifab_mome(const void* x, long ldx, const float* w, void* state, const int32_t* positions, const int32_t* slots, void* y,
              long ldy, int T, int C, int taps, int c_offset, void* stream);
/* X bf16 [T, S, W]; phi f32 [S*S+2S, S*W]; gamma [S*W]; alpha [3]; beta [S*S+2S] -> y bf16 [T, W], post f32 [T, S], comb f32 [T, S, S] */
int ifab_mhc_pre(const void* X, const float* phi, const float* gamma, const float* alpha, const float* beta, void* y, float* post,
                 float* comb, int T, int S, int W, int sinkhorn_iters, float eps, void* stream);
/* the same in ONE launch: `tickets` = T zeroed 32-bit words (left zero again); the CTA that finishes a token's sums last runs its tail */
int ifab_mhc_pre_ticketed(const void* X, const float* phi, const float* gamma, const float* alpha, const float* beta, void* y, float* post,
                          float* comb, int T, int S, int W, int sinkhorn_iters, float eps, uint32_t* tickets, void* stream);
int ifab_mhc_post(const void* X, const void* branch, long ldb, const float* post, const float* comb, void* Y, int T, int S, int W,
                  void* stream);
/* the same with the branch RMS-normalised first (gain norm_w bf16 [W], result rounded to bf16 like a stand-alone norm) */
int ifab_mhc_post_norm(const void* X, const void* branch, long ldb, const void* norm_w, float eps, const float* post, const float* comb, void* Y,
                       int T, int S, int W, void* stream);
/* gated delta rule, one token per row: q, k bf16 [rows, H, dk]; v bf16 [rows, H, dv]; g, beta f32 [rows, H]; state f32 [slots, H, dk, dv] */
int ifab_delta_rule_decode(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state,
                           const int32_t* slots, void* out, int rows, int H, int dk, int dv, void* stream);
/* indexer: q bf16 [T, heads, dim], w f32 [T, heads], keys paged bf16 [pages, page_tokens, dim]; scores = scratch f32 [T, ctx];
 * out int32 [T, topk]: the top-k key positions (<= the query position) in ascending order, -1 padded */
int ifab_sparse_index(const void* q, const float* w, const void* keys, const int32_t* positions, const int32_t* slots,
                      const int32_t* page_table, int max_pages, int page_tokens, int num_pages, float* scores, int ctx, int T,
                      int heads, int dim, int topk, int32_t* out, uint32_t* status, void* stream);
/* the same over an int8 index cache (keys int8 [pages, page_tokens, dim], one half-precision scale per row; the query heads are
 * quantised the same way before scoring) and the append that fills it */
int ifab_sparse_index_q8(const void* q, const float* w, const void* keys, const void* key_scales, const int32_t* positions, const int32_t* slots,
                         const int32_t* page_table, int max_pages, int page_tokens, int num_pages, float* scores, int ctx, int T, int heads, int dim,
                         int topk, int32_t* out, uint32_t* status, void* stream);
int ifab_index_cache_append_q8(const void* key, long ldk, const int32_t* positions, const int32_t* slots, const int32_t* page_table, int max_pages,
                               int page_tokens, int num_pages, void* cache, void* scales, int T, int dim, uint32_t* status, void* stream);
/* bf16 index keys [T, dim] into the paged bf16 index cache [pages, page_tokens, dim] */
int ifab_index_cache_append(const void* key, long ldk, const int32_t* positions, const int32_t* slots, const int32_t* page_table, int max_pages,
                            int page_tokens, int num_pages, void* cache, int T, int dim, uint32_t* status, void* stream);
/* the general selector: gains f32 [T, heads] (w_bf16 = 0, ldw = heads) or bf16 rows of stride ldw (w_bf16 = 1); key_scales null = bf16 keys */
int ifab_sparse_index_general(const void* q, const void* w, long ldw, int w_bf16, const void* keys, const void* key_scales, const int32_t* positions,
                              const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens, int num_pages, float* scores, int ctx,
                              int T, int heads, int dim, int topk, int32_t* out, uint32_t* status, void* stream);
/* split-KV attention restricted to `indices` (int32 [T, n_index], ascending key positions padded with -1; null = every causal key);
 * rope < 0: the cache holds packed int8 rows (656 bytes) */
int ifab_mla_decode_attention_indexed(const void* q_lat, const void* cache, const int32_t* positions, const int32_t* slots, const int32_t* page_table,
                                      int max_pages, int page_tokens, int num_pages, const void* sinks, int n_sinks, int window, float scale, int T,
                                      int H, int latent, int rope, int keys_per_split, int max_splits, float* scratch, uint64_t scratch_bytes,
                                      const void* w_kvb, int nope, int vdim, void* out, long ldo, uint32_t* status, const int32_t* indices, int n_index,
                                      void* stream);

/* ---- packed int8 latent cache (656-byte rows: 512 int8 | 64 bf16 rope | 4 f32 tile scales) and activation quantisation ----
 * Attention over a packed cache: ifab_mla_decode_attention with rope = -64 and `cache` pointing at the packed rows. */
int ifab_mla_kv_write_q8(const void* kv, long ldkv, const void* norm_w, float eps, float theta, const int32_t* positions,
                         const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens, void* cache,
                         int num_pages, int T, uint32_t* status, void* stream);
int ifab_mla_kv_write_q8_split(const void* latent_rows, long ldl, const void* rope_rows, long ldr, const void* norm_w, float eps, float theta,
                               const int32_t* positions, const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens,
                               void* cache, int num_pages, int T, uint32_t* status, void* stream);
int ifab_kv_dequantize_q8(const void* cache, void* out /* bf16 [rows, 576] */, long rows, void* stream);
/* symmetric int8, ties away from zero; group_cols = K: per-row scale, 128: per-tile scales [T, ceil(K/128)] */
int ifab_quantize_int8(const void* x, long ldx, void* q, long ldq, float* scales, long lds, int T, int K, int group_cols,
                       void* stream);

/* ---- GQA decode path (dense models) ---- */
int ifab_gqa_rope_kv_write(void* qkv, long ld, const int32_t* positions, const int32_t* slots,
                           const int32_t* page_table, int max_pages, int page_tokens, void* k_cache, void* v_cache,
                           int num_pages, int T, int Hq, int Hkv, int head_dim, int rotary_dim, float theta,
                           uint32_t* status, void* stream);
/* Split-KV decode attention. Split s covers keys [s * keys_per_split, (s + 1) * keys_per_split); the LAST split also covers
 * every key beyond max_splits * keys_per_split, so any context is attended in full (contexts longer than that product
 * only lose parallelism). scratch: T * Hq * max_splits * (head_dim + 2) floats. */
int ifab_gqa_decode_attention(const void* q, long ldq, const void* k_cache, const void* v_cache,
                              const int32_t* positions, const int32_t* slots, const int32_t* page_table, int max_pages,
                              int page_tokens, int num_pages, float scale, int T, int Hq, int Hkv, int head_dim,
                              int keys_per_split, int max_splits, float* scratch, uint64_t scratch_bytes, void* out,
                              long ldo, uint32_t* status, void* stream);

/* ---- GQA decode attention without any allocation (this entry point has no counterpart in the reference) ----
 * Same computation and same results as ifab_gqa_decode_attention, but the split-partials workspace is a
 * fixed array inside the library, so neither the caller nor the library calls cudaMalloc / cudaFree or any
 * allocating routine. Meant for C / C++ hosts that link the library without a tensor framework and cannot
 * allocate where they call it: all free device memory already belongs to their KV cache, they run under an
 * allocator lock, or an allocation could stall the device in a latency-critical loop.
 *   - limit: T * Hq * max_splits * (head_dim + 2) * 4 bytes must not exceed IFAB_GQA_STATIC_SCRATCH_BYTES;
 *     a larger call returns IFAB_ERR_STATIC_SCRATCH, launches nothing and explains itself in `err`
 *   - every call looks up the array's address on the current device (cudaGetSymbolAddress: a host-side query that
 *     allocates nothing, and is right again after a device reset); the first call on a device may load the module, so
 *     make that first call before any stream capture begins
 *   - all calls on a device share the one array: calls that may overlap on the GPU race on it, so keep them
 *     on one stream or order them. The array keeps the previous call's contents; each call overwrites
 *     everything it reads, so nothing has to be cleared
 *   - `err` (optional, `err_len` bytes) receives a NUL-terminated message when the result is not 0
 *   - ifab_gqa_static_scratch_bytes() / ifab_err_static_scratch() return the two constants below to callers that do not
 *     include this header (bindings) */
#define IFAB_GQA_STATIC_SCRATCH_BYTES (8u << 20)
#define IFAB_ERR_STATIC_SCRATCH (-6)
uint64_t ifab_gqa_static_scratch_bytes(void);
int ifab_err_static_scratch(void);
int ifab_gqa_decode_attention_static(const void* q, long ldq, const void* k_cache, const void* v_cache,
                                     const int32_t* positions, const int32_t* slots, const int32_t* page_table,
                                     int max_pages, int page_tokens, int num_pages, float scale, int T, int Hq, int Hkv,
                                     int head_dim, int keys_per_split, int max_splits, void* out, long ldo,
                                     uint32_t* status, void* stream, char* err, uint64_t err_len);

#ifdef __cplusplus
}
#endif

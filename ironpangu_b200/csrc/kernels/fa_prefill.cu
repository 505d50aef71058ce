// Prompt (prefill) attention on the 5th-generation tensor cores: softmax(Q K^T) V for a chunk of consecutive tokens of one
// sequence against that sequence's whole context, causal, optional sliding window. One CTA = 128 query rows of one head.
//
//   warp 0      TMA producer: the Q tile once, then per 128-key tile the K panels (two shared-memory stages) and the V^T
//               panels (one stage), all 128-byte-swizzled [128 rows x 64 columns] boxes, never multicast
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma: S_j = Q K_j^T into one of two TMEM score buffers (so
//               S_{j+1} is computed while the softmax warps work on S_j), then O_j = P_j V_j once P_j is in shared memory
//   warps 4-19  four threads per query row (warps w, w + 4, w + 8, w + 12 share a TMEM lane quarter; each owns a quarter of the
//               tile's key columns and of the output columns; they agree on the tile maximum through tagged words in shared
//               memory, a bounded exchange): ONE tcgen05.ld pass over the scores (kept in registers), mask, exp2 against
//               the row's reference maximum, running sum, P_j (bf16) into shared memory in the swizzled operand layout. The
//               output accumulates in TMEM (O += P_j V_j by the MMA itself); the reference maximum of a row only moves when a
//               tile's maximum exceeds it by more than 8 (a factor 256 of headroom in the f32 accumulator and in bf16 P), and
//               only then is the row of O rescaled in place (tcgen05.ld, multiply, tcgen05.st) - rarely after the first tiles.
//
// Operands are what the multi-head-latent prompt path has at hand: the per-head key part (up-projected latent, D1 columns)
// and a second key part shared by all heads (the rotary columns, D2), so S = Q1 K1^T + Q2 K2^T accumulates over 64-column
// panels from two tensors; V is passed transposed ([value dim, keys], keys contiguous: it is produced that way by the
// up-projection GEMM), which makes it a K-major B operand like every other operand here. With D2 = 0 and a key / value head
// shared by `kv_group` query heads the same kernel is grouped-query attention.
// Every wait is bounded; a wait that runs out raises the CTA's abort flag and the status word, the CTA drains its copies,
// frees its tensor memory and returns. Reference: the fused attention operator of the prompt envelope, up to 4,096 query
// rows (native/src/token_executor.h:863-909).
#include "tc_common.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::tc;

namespace {

constexpr int BQ = 128, BKEY = 128, DV = 128;
constexpr int PANEL_BYTES = 128 * 128;      // 128 rows x 64 bf16
constexpr int PV_PANELS = BKEY / 64;        // panels of P (keys along K) and of V^T
constexpr uint32_t TMEM_COLS = 512;         // S0 [0,128) S1 [128,256) O [256,384)
constexpr uint32_t S_COL = 0, O_COL = 256;
constexpr int PARTS = 4;                    // threads per query row: warps w, w + 4, ... of a TMEM lane quarter split the columns
constexpr int THREADS = 128 + 128 * PARTS;  // warp 0 producer, warp 1 MMA issuer, warps 2-3 idle, then the softmax warps

struct FaParams {
  bf16* out; long ldo;
  int m, ctx, kv_group, pos0, window;
  int q_head_stride, k_head_stride, vt_head_stride, vt_row0;
  float scale_log2;                          // softmax scale * log2(e)
  uint32_t* status; uint32_t spin_limit;
};

struct Bars {
  uint64_t q_full, k_full[2], k_empty[2], v_full, v_empty, s_full[2], p_ready, o_full;
  uint32_t tmem_slot;
  int abort_flag;
};

template <int P1, int P2>
struct Layout {
  static constexpr int NQ = P1 + P2;                       // 64-column panels of Q and of a K tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + NQ * PANEL_BYTES;   // two stages
  static constexpr int V_OFF = K_OFF + 2 * NQ * PANEL_BYTES;
  static constexpr int P_OFF = V_OFF + PV_PANELS * PANEL_BYTES;
  static constexpr int BAR_OFF = P_OFF + PV_PANELS * PANEL_BYTES;
  static constexpr int XCH_OFF = BAR_OFF + 256;            // [2 parities][2 column halves][128 rows] tagged 8-byte words: the two threads of a row
  static constexpr int SMEM = XCH_OFF + 2 * PARTS * 128 * 8 + 1024;
};

template <int P1, int P2>
__global__ void __launch_bounds__(THREADS, 1) fa_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                                                            const __grid_constant__ CUtensorMap tmap_k2, const __grid_constant__ CUtensorMap tmap_vt,
                                                            FaParams p) {
  using L = Layout<P1, P2>;
  constexpr int NQ = L::NQ;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* Qs = smem + L::Q_OFF;
  unsigned char* Ks = smem + L::K_OFF;
  unsigned char* Vs = smem + L::V_OFF;
  unsigned char* Ps = smem + L::P_OFF;
  Bars* B = reinterpret_cast<Bars*>(smem + L::BAR_OFF);
  volatile unsigned long long* xch = reinterpret_cast<volatile unsigned long long*>(smem + L::XCH_OFF);
  volatile int* abort_flag = &B->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ, h = blockIdx.y, kvh = h / p.kv_group;
  // key tiles this query tile can see: up to the position of its last live row, from the window's start
  const int last_row = min(q0 + BQ, p.m) - 1;
  const int t_end = min((p.ctx + BKEY - 1) / BKEY, (p.pos0 + last_row) / BKEY + 1);
  const int t_begin = p.window > 0 ? max(0, p.pos0 + q0 - p.window + 1) / BKEY : 0;
  const int n_tiles = t_end - t_begin;

  if (threadIdx.x == 0) {
    mbar_init(&B->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&B->k_full[s], 1);
      mbar_init(&B->k_empty[s], 1);
      mbar_init(&B->s_full[s], 1);
    }
    mbar_init(&B->v_full, 1);
    mbar_init(&B->v_empty, 1);
    mbar_init(&B->p_ready, 128 * PARTS);
    mbar_init(&B->o_full, 1);
    B->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_k2);
    tma_prefetch_desc(&tmap_vt);
  }
  for (int i = threadIdx.x; i < 2 * PARTS * 128; i += blockDim.x) xch[i] = 0ull;     // call numbers start at 1: a word left by an earlier CTA must not match
  if (warp == 1) tmem_alloc(&B->tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = B->tmem_slot;
  grid_dep_launch();
  grid_dep_wait();

  auto fail = [&]() {
    *abort_flag = 1;
    if (p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
  };

  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- TMA producer
    mbar_expect_tx(&B->q_full, NQ * PANEL_BYTES);
    for (int pp = 0; pp < NQ; ++pp) tma_load_2d(Qs + pp * PANEL_BYTES, &tmap_q, &B->q_full, h * p.q_head_stride + pp * 64, q0);
    int armed_k = 0, armed_v = 0;
    for (int j = 0; j < n_tiles && !*abort_flag; ++j) {
      const int key0 = (t_begin + j) * BKEY, s = j & 1, round = j >> 1;
      if (round > 0 && !mbar_wait(&B->k_empty[s], (round - 1) & 1, p.spin_limit)) { fail(); break; }
      unsigned char* kd = Ks + s * NQ * PANEL_BYTES;
      mbar_expect_tx(&B->k_full[s], NQ * PANEL_BYTES);
      for (int pp = 0; pp < P1; ++pp) tma_load_2d(kd + pp * PANEL_BYTES, &tmap_k, &B->k_full[s], kvh * p.k_head_stride + pp * 64, key0);
      for (int pp = 0; pp < P2; ++pp) tma_load_2d(kd + (P1 + pp) * PANEL_BYTES, &tmap_k2, &B->k_full[s], pp * 64, key0);
      armed_k = j + 1;
      if (j > 0 && !mbar_wait(&B->v_empty, (j - 1) & 1, p.spin_limit)) { fail(); break; }
      mbar_expect_tx(&B->v_full, PV_PANELS * PANEL_BYTES);
      for (int pp = 0; pp < PV_PANELS; ++pp) tma_load_2d(Vs + pp * PANEL_BYTES, &tmap_vt, &B->v_full, key0 + pp * 64, kvh * p.vt_head_stride + p.vt_row0);
      armed_v = j + 1;
    }
    if (*abort_flag) {
      // every copy this thread issued must land before the CTA may exit
      mbar_wait(&B->q_full, 0, p.spin_limit);
      for (int j = max(0, armed_k - 2); j < armed_k; ++j) mbar_wait(&B->k_full[j & 1], (j >> 1) & 1, p.spin_limit);
      if (armed_v > 0) mbar_wait(&B->v_full, (armed_v - 1) & 1, p.spin_limit);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = umma_idesc_bf16(BQ, 128);
    bool ok = mbar_wait(&B->q_full, 0, p.spin_limit);
    auto issue_scores = [&](int j) {
      const int s = j & 1;
      if (!mbar_wait(&B->k_full[s], (j >> 1) & 1, p.spin_limit) || *abort_flag) return false;
      tc_fence_after();
      const uint32_t qa = smem_u32(Qs), ka = smem_u32(Ks + s * NQ * PANEL_BYTES);
#pragma unroll
      for (int pp = 0; pp < NQ; ++pp) {
        const uint64_t da = umma_desc_sw128(qa + pp * PANEL_BYTES), db = umma_desc_sw128(ka + pp * PANEL_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + S_COL + (uint32_t)s * 128u, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, pp > 0 || k > 0);
      }
      umma_commit(&B->s_full[s]);
      umma_commit(&B->k_empty[s]);
      return true;
    };
    if (ok && n_tiles > 0) ok = issue_scores(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (j + 1 < n_tiles) ok = issue_scores(j + 1);      // the next tile's scores overlap this tile's softmax
      if (!ok) break;
      if (!mbar_wait(&B->p_ready, j & 1, p.spin_limit) || !mbar_wait(&B->v_full, j & 1, p.spin_limit) || *abort_flag) { ok = false; break; }
      tc_fence_after();
      const uint32_t pa = smem_u32(Ps), va = smem_u32(Vs);
#pragma unroll
      for (int pp = 0; pp < PV_PANELS; ++pp) {
        const uint64_t da = umma_desc_sw128(pa + pp * PANEL_BYTES), db = umma_desc_sw128(va + pp * PANEL_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + O_COL, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, j > 0 || pp > 0 || k > 0);
      }
      umma_commit(&B->o_full);
      umma_commit(&B->v_empty);
    }
    if (!ok) fail();
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax + output: two threads per query row (warps w and w + 4
    // share a TMEM lane quarter), each owns 64 of the tile's 128 key columns and 64 of the 128 output columns
    const int quarter = warp & 3, half = (warp - 4) >> 2, r = quarter * 32 + lane;     // `half`: which of the PARTS column ranges
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int q_pos = p.pos0 + q0 + r;
    const int lo = p.window > 0 ? q_pos - p.window + 1 : 0;     // first visible key
    constexpr int HK = BKEY / PARTS, HV = DV / PARTS;
    float m_ref = -INFINITY, l_run = 0.f;     // reference maximum (base-2 domain, may lag the true maximum by up to 8); sum over this thread's columns
    bool ok = true;
    // this thread's keys: panel (half * HK) / 64 of P, 16-byte chunks from ((half * HK) % 64) / 8 on
    unsigned char* prow = Ps + ((half * HK) >> 6) * PANEL_BYTES + (r >> 3) * 1024 + (r & 7) * 128;
    const int chunk0 = ((half * HK) & 63) >> 3;
    const uint32_t o_addr = tmem + lane_addr + O_COL + (uint32_t)(half * HV);
    // The two threads of a row trade one float per call: each publishes (call number, value) as one 8-byte word and polls its
    // partner's word for the same call number - a bounded wait, unlike a named barrier, so a pair whose partner has given up
    // gives up too. Slots alternate with the call parity: a slot is rewritten two calls later, after the partner has passed
    // the call in between, hence after it has read this one.
    // `combine_max`: the maximum over the partners' values, else their sum
    auto trade = [&](float mine, int call, bool combine_max, float* result) -> bool {
      volatile unsigned long long* slot = xch + (call & 1) * (PARTS * 128);
      slot[half * 128 + r] = ((unsigned long long)(uint32_t)(call + 1) << 32) | __float_as_uint(mine);
      float acc = mine;
#pragma unroll
      for (int k = 1; k < PARTS; ++k) {
        const int other = (half + k) % PARTS;
        bool got = false;
        for (uint32_t spin = 0; spin < p.spin_limit; ++spin) {
          const unsigned long long w = slot[other * 128 + r];
          if ((uint32_t)(w >> 32) == (uint32_t)(call + 1)) {
            const float v = __uint_as_float((uint32_t)w);
            acc = combine_max ? fmaxf(acc, v) : acc + v;
            got = true;
            break;
          }
          if (*abort_flag) break;
        }
        if (!got) return false;
      }
      *result = acc;
      return true;
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int key0 = (t_begin + j) * BKEY + half * HK, s = j & 1;
      // the warp leaves the loop together: the TMEM accesses and the votes below are warp-wide
      if (!__all_sync(0xffffffffu, mbar_wait(&B->s_full[s], (j >> 1) & 1, p.spin_limit) && !*abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_addr + S_COL + (uint32_t)s * 128u + (uint32_t)(half * HK);
      float sv[HK];
#pragma unroll
      for (int c0 = 0; c0 < HK; c0 += 32) tmem_ld_32x32(s_addr + (uint32_t)c0, sv + c0);
      tmem_ld_wait();
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four independent chains
#pragma unroll
      for (int i = 0; i < HK; ++i) {
        const int key = key0 + i;
        sv[i] = (key <= q_pos && key >= lo) ? sv[i] * p.scale_log2 : -INFINITY;
        mx[i & 3] = fmaxf(mx[i & 3], sv[i]);
      }
      const float my_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      float tile_max = -INFINITY;
      if (!__all_sync(0xffffffffu, trade(my_max, j, true, &tile_max))) { ok = false; break; }
      const bool moved = tile_max > m_ref + 8.f;                 // also true for the first visible key (m_ref = -inf)
      const float m_new = moved ? tile_max : m_ref;
      const float corr = (moved && m_ref != -INFINITY) ? exp2f(m_ref - m_new) : 1.f;
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      uint4 packed[HK / 8];
#pragma unroll
      for (int g = 0; g < HK / 8; ++g) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = sv[8 * g + i] == -INFINITY ? 0.f : exp2f(sv[8 * g + i] - m_new);
          sum[i & 3] += e[i];
        }
        packed[g] = pack8(e);
      }
      if (j > 0) {
        // P_{j-1} V_{j-1} has completed: the P buffer is free and O is at rest until the next product is issued
        if (!__all_sync(0xffffffffu, mbar_wait(&B->o_full, (j - 1) & 1, p.spin_limit) && !*abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, corr != 1.f)) {              // tcgen05.ld / st are warp-wide: rows that did not move scale by 1
#pragma unroll
          for (int c0 = 0; c0 < HV; c0 += 32) {
            float v[32];
            tmem_ld_32x32(o_addr + (uint32_t)c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= corr;
            tmem_st_32x32(o_addr + (uint32_t)c0, v);
          }
          tmem_st_wait();
        }
      }
      // 8 keys = one 16-byte chunk of this row's 128-byte line; chunk c sits at position c ^ (row % 8)
#pragma unroll
      for (int g = 0; g < HK / 8; ++g) *reinterpret_cast<uint4*>(prow + (((chunk0 + g) ^ (r & 7)) << 4)) = packed[g];
      l_run = l_run * corr + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
      m_ref = m_new;
      fence_proxy_async_smem();       // the tensor core reads P through the async proxy
      tc_fence_before();              // and this thread's TMEM accesses (S_j, the rescale of O) are done
      mbar_arrive(&B->p_ready);
    }
    float o[HV];
    if (ok && n_tiles > 0) {
      if (__all_sync(0xffffffffu, mbar_wait(&B->o_full, (n_tiles - 1) & 1, p.spin_limit) && !*abort_flag)) {
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < HV; c0 += 32) tmem_ld_32x32(o_addr + (uint32_t)c0, o + c0);
        tmem_ld_wait();
      } else {
        ok = false;
      }
    } else {
#pragma unroll
      for (int i = 0; i < HV; ++i) o[i] = 0.f;
    }
    // the row's sum is the sum of its two threads' partial sums
    if (ok) {
      float total = 0.f;
      if (__all_sync(0xffffffffu, trade(l_run, n_tiles, false, &total))) l_run = total;      // every partner adds in its own order: sums may differ in the last bit between columns
      else ok = false;
    }
    if (!ok) {
      if (lane == 0) fail();
    } else if (q0 + r < p.m) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* dst = p.out + (long)(q0 + r) * p.ldo + (long)h * DV + half * HV;
#pragma unroll
      for (int c = 0; c < HV; c += 8) {
        float t8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) t8[i] = o[c + i] * inv;
        *reinterpret_cast<uint4*>(dst + c) = pack8(t8);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int P1, int P2>
int launch_fa(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tk2, const CUtensorMap& tv, const FaParams& p, int H, cudaStream_t s) {
  auto k = fa_prefill_kernel<P1, P2>;
  if (int rc = opt_in_smem(k, Layout<P1, P2>::SMEM)) return rc;
  dim3 grid((p.m + BQ - 1) / BQ, H);
  return launch_chain(k, grid, dim3(THREADS), (size_t)Layout<P1, P2>::SMEM, s, tq, tk, tk2, tv, p);
}

}  // namespace

// q:  [m, H * q_head_stride] rows of consecutive positions pos0 .. pos0 + m - 1; head h reads columns h * q_head_stride + [0, d1 + d2)
// k:  [ctx, ...] per-head key part: key head g = h / kv_group reads columns g * k_head_stride + [0, d1)
// k2: [ctx, d2] key part shared by all heads (may be NULL when d2 == 0)
// vt: [rows, ldvt >= ctx] transposed values: key head g reads rows g * vt_head_stride + vt_row0 + [0, 128), column = key
// out: [m, H * 128]. d1 in {64, 128}, d2 in {0, 64}; ld* in elements, multiples of 8; window 0 = none.
extern "C" int ifab_fa_prefill_bf16(const void* q, long ldq, int q_head_stride, const void* k, long ldk, int k_head_stride, const void* k2,
                                    long ldk2, const void* vt, long ldvt, int vt_head_stride, int vt_row0, int vt_rows, void* out, long ldo,
                                    int m, int ctx, int H, int kv_group, int d1, int d2, int pos0, int window, float scale, uint32_t* status,
                                    void* stream) {
  if (m < 1 || ctx < 1 || H < 1 || kv_group < 1 || H % kv_group || pos0 < 0 || pos0 + m > ctx || window < 0) return -1;
  if ((d1 != 64 && d1 != 128) || (d2 != 0 && d2 != 64) || (d2 && !k2)) return -1;
  if (ldq % 8 || ldk % 8 || ldvt % 8 || ldo % 8 || (d2 && ldk2 % 8) || q_head_stride % 8 || k_head_stride % 8 || ldvt < ctx) return -1;
  const int Hkv = H / kv_group;
  CUtensorMap tq, tk, tk2, tv;
  if (int rc = make_tmap_bf16_2d(&tq, q, (uint64_t)m, (uint64_t)(H - 1) * q_head_stride + d1 + d2, (uint64_t)ldq, BQ)) return rc;
  if (int rc = make_tmap_bf16_2d(&tk, k, (uint64_t)ctx, (uint64_t)(Hkv - 1) * k_head_stride + d1, (uint64_t)ldk, BKEY)) return rc;
  if (d2) {
    if (int rc = make_tmap_bf16_2d(&tk2, k2, (uint64_t)ctx, (uint64_t)d2, (uint64_t)ldk2, BKEY)) return rc;
  } else {
    tk2 = tk;
  }
  if (int rc = make_tmap_bf16_2d(&tv, vt, (uint64_t)vt_rows, (uint64_t)ctx, (uint64_t)ldvt, DV)) return rc;
  FaParams p{(bf16*)out, ldo, m, ctx, kv_group, pos0, window, q_head_stride, k_head_stride, vt_head_stride, vt_row0,
             scale * 1.4426950408889634f, status, 4000000u};
  cudaStream_t s = (cudaStream_t)stream;
  if (d1 == 128 && d2 == 64) return launch_fa<2, 1>(tq, tk, tk2, tv, p, H, s);
  if (d1 == 128 && d2 == 0) return launch_fa<2, 0>(tq, tk, tk2, tv, p, H, s);
  if (d1 == 64 && d2 == 64) return launch_fa<1, 1>(tq, tk, tk2, tv, p, H, s);
  return launch_fa<1, 0>(tq, tk, tk2, tv, p, H, s);
}

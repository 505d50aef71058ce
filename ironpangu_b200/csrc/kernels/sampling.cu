// Device-side sampling for sm_100a: temperature, penalties, top-k, min-p, top-p and an inverse-CDF
// draw, on vocabulary-sharded logits.
//
//   sample_block_topk_kernel  every CTA sorts 4096 (logit, id) pairs of its vocabulary slice in shared
//                             memory (bitonic, value descending / id ascending) and keeps the best K
//   sample_finish_kernel      one CTA per query row merges the per-CTA candidates, exchanges its K best
//                             with the other ranks through the symmetric heap (the global top-K is a
//                             subset of the union of the ranks' top-K), then applies min-p / top-p and
//                             draws with a counter-based generator, so a replayed CUDA graph produces
//                             fresh draws without host involvement
// The result is exact top-k sampling over the full vocabulary without ever gathering the logits.
// Reference: native/src/sampler.inc:11-228 (sort / top-k / min-p / cumulative top-p / inverse CDF with a
// pre-filled uniform table); here the uniform comes from hash(seed, counter) on the device.
#include "common.cuh"
#include "ifab_kernels.h"

using namespace ifab;

namespace {

constexpr int KMAX = 64;       // largest supported top-k
constexpr int CHUNK = 4096;    // logits per CTA in the first stage

struct Cand { float v; int i; };
__device__ __forceinline__ bool before(const Cand& a, const Cand& b) { return a.v > b.v || (a.v == b.v && a.i < b.i); }

template <int N, int THREADS>
__device__ __forceinline__ void bitonic_sort(Cand* s) {
  for (int k = 2; k <= N; k <<= 1)
    for (int j = k >> 1; j > 0; j >>= 1) {
      __syncthreads();
      for (int t = threadIdx.x; t < N; t += THREADS) {
        const int x = t ^ j;
        if (x > t) {
          const bool up = (t & k) == 0;
          Cand a = s[t], b = s[x];
          if (up ? before(b, a) : before(a, b)) { s[t] = b; s[x] = a; }
        }
      }
    }
  __syncthreads();
}

struct SampleParams {
  const float* logits; long ld;     // [T, V_local]
  int T, V, vocab_offset, K;
  const float* inv_temperature;     // [T] (1/T; 0 = greedy)
  const int16_t* counts; long ldc;  // optional [T, V_local] occurrences of each local token in the row's sequence
  const float* penalties;           // optional [T, 3] repetition, frequency, presence
  Cand* cand;                       // [T][nblocks][KMAX]
  int nblocks;
};

__global__ void __launch_bounds__(256) sample_block_topk_kernel(SampleParams p) {
  __shared__ Cand s[CHUNK];
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.y, base = blockIdx.x * CHUNK;
  const float it = p.inv_temperature ? p.inv_temperature[t] : 1.f;
  const float scale = it > 0.f ? it : 1.f;
  for (int k = threadIdx.x; k < CHUNK; k += 256) {
    const int c = base + k;
    Cand x{-INFINITY, 0x7fffffff};
    if (c < p.V) {
      float v = p.logits[(long)t * p.ld + c];
      if (p.counts && p.penalties) {
        const int n = p.counts[(long)t * p.ldc + c];
        if (n > 0) {
          const float rep = p.penalties[t * 3], freq = p.penalties[t * 3 + 1], pres = p.penalties[t * 3 + 2];
          v = v >= 0.f ? v / rep : v * rep;
          v -= freq * (float)n + pres;
        }
      }
      x.v = v * scale;
      x.i = p.vocab_offset + c;
    }
    s[k] = x;
  }
  bitonic_sort<CHUNK, 256>(s);
  Cand* out = p.cand + ((long)t * p.nblocks + blockIdx.x) * KMAX;
  for (int k = threadIdx.x; k < KMAX; k += 256) out[k] = s[k];
}

struct FinishParams {
  const Cand* cand; int nblocks, T, K;
  const int32_t* k_rows;   // optional [T]: top-k of each row (values outside 1..K mean K)
  const float* inv_temperature; const float* top_p; const float* min_p;   // [T] each (nullptr = disabled)
  const uint64_t* seeds; uint64_t* counters;                              // [T]: draw = hash(seed, counter++)
  int32_t* out_ids; float* out_probs;
  FabricView fv; uint64_t* seq; uint32_t* done;
};

__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t counter) {
  uint64_t z = seed + 0x9e3779b97f4a7c15ull * (counter + 1);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// one CTA (256 threads) per launch handles all rows sequentially so that the cross-rank exchange is one epoch
__global__ void __launch_bounds__(256) sample_finish_kernel(FinishParams p) {
  constexpr int MERGE = 4096;
  __shared__ Cand s[MERGE];
  __shared__ Cand fin[IFAB_MAX_RANKS * KMAX];
  __shared__ float prob[KMAX];
  grid_dep_launch();
  grid_dep_wait();
  const int world = p.fv.world, rank = p.fv.rank;
  const uint64_t epoch = *reinterpret_cast<volatile uint64_t*>(p.seq) + 1;
  const uint32_t par = (uint32_t)(epoch & 1);
  for (int t = 0; t < p.T; ++t) {
    // merge this rank's per-CTA candidates (nblocks * KMAX <= MERGE enforced by the host)
    const int n = p.nblocks * KMAX;
    for (int k = threadIdx.x; k < MERGE; k += 256) s[k] = k < n ? p.cand[(long)t * n + k] : Cand{-INFINITY, 0x7fffffff};
    bitonic_sort<MERGE, 256>(s);
    if (world > 1) {
      for (int k = threadIdx.x; k < world * KMAX; k += 256) {
        const int q = k / KMAX, c = k % KMAX;
        Cand* dst = reinterpret_cast<Cand*>(p.fv.data[q] + (size_t)par * p.fv.data_half_bytes) + ((size_t)rank * p.T + t) * KMAX + c;
        *dst = s[c];
      }
    } else {
      for (int k = threadIdx.x; k < KMAX; k += 256) fin[k] = s[k];
    }
    __syncthreads();
    if (t + 1 < p.T) continue;
    // all rows pushed: one flag exchange for the whole launch
    if (world > 1) {
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x < world) {
        const int q = threadIdx.x;
        st_release_sys(p.fv.flags[q] + (size_t)par * p.fv.flag_half_words + rank, epoch);
        if (!wait_flag_bounded(p.fv.flags[rank] + (size_t)par * p.fv.flag_half_words + q, epoch, p.fv.spin_limit))
          atomicOr(p.fv.status, IFAB_STATUS_PEER_TIMEOUT);
      }
      __syncthreads();
    }
  }
  for (int t = 0; t < p.T; ++t) {
    int total = KMAX;
    if (world > 1) {
      total = world * KMAX;
      const Cand* src = reinterpret_cast<const Cand*>(p.fv.data[rank] + (size_t)par * p.fv.data_half_bytes);
      for (int k = threadIdx.x; k < IFAB_MAX_RANKS * KMAX; k += 256) {
        const int q = k / KMAX, c = k % KMAX;
        if (q < world) {
          const Cand* e = src + ((size_t)q * p.T + t) * KMAX + c;
          fin[k] = Cand{__ldcg(&e->v), __ldcg(&e->i)};
        } else {
          fin[k] = Cand{-INFINITY, 0x7fffffff};
        }
      }
      bitonic_sort<IFAB_MAX_RANKS * KMAX, 256>(fin);
    } else {
      __syncthreads();
      // world == 1: fin was filled for the last row only; reload for earlier rows
      const int n = p.nblocks * KMAX;
      for (int k = threadIdx.x; k < MERGE; k += 256) s[k] = k < n ? p.cand[(long)t * n + k] : Cand{-INFINITY, 0x7fffffff};
      bitonic_sort<MERGE, 256>(s);
      for (int k = threadIdx.x; k < KMAX; k += 256) fin[k] = s[k];
      __syncthreads();
    }
    (void)total;
    if (threadIdx.x == 0) {
      const float it = p.inv_temperature ? p.inv_temperature[t] : 1.f;
      int K = p.K;
      if (p.k_rows) {          // rows of different requests share a launch: each keeps its own k
        const int kr = p.k_rows[t];
        if (kr >= 1 && kr < K) K = kr;
      }
      if (it <= 0.f) K = 1;   // greedy
      while (K > 1 && fin[K - 1].v == -INFINITY) --K;
      // softmax over the K survivors
      const float mx = fin[0].v;
      float sum = 0.f;
      for (int k = 0; k < K; ++k) sum += (prob[k] = __expf(fin[k].v - mx));
      const float minp = p.min_p ? p.min_p[t] : 0.f;
      int keep = K;
      if (minp > 0.f) {
        keep = 0;
        while (keep < K && prob[keep] >= minp * prob[0]) ++keep;   // prob[0] is the max
        if (keep == 0) keep = 1;
      }
      const float topp = p.top_p ? p.top_p[t] : 1.f;
      if (topp < 1.f) {
        float psum = 0.f;
        for (int k = 0; k < keep; ++k) psum += prob[k];
        float cum = 0.f;
        int nk = 0;
        while (nk < keep && cum < topp * psum) cum += prob[nk++];   // keep tokens whose exclusive cumulative mass < top_p
        keep = max(nk, 1);
      }
      float tot = 0.f;
      for (int k = 0; k < keep; ++k) tot += prob[k];
      int pick = 0;
      if (keep > 1) {
        const uint64_t ctr = p.counters ? p.counters[t] : 0;
        const float u = uniform01(p.seeds ? p.seeds[t] : 0, ctr) * tot;
        float cdf = 0.f;
        pick = keep - 1;
        for (int k = 0; k < keep; ++k) {
          cdf += prob[k];
          if (cdf > u) { pick = k; break; }
        }
      }
      if (p.counters) p.counters[t] += 1;
      p.out_ids[t] = fin[pick].i;
      if (p.out_probs) p.out_probs[t] = prob[pick] / tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    *p.seq = epoch;
    __threadfence();
  }
}

}  // namespace

// scratch: T * nblocks * 64 * 8 bytes with nblocks = ceil(V_local / 4096) (must be <= 64)
extern "C" int ifab_sample_topk(const float* logits, long ld, int T, int V_local, int vocab_offset, int top_k,
                                const int32_t* top_k_rows, const float* inv_temperature, const float* top_p, const float* min_p, const int16_t* counts,
                                long ldc, const float* penalties, const uint64_t* seeds, uint64_t* counters, void* scratch,
                                uint64_t scratch_bytes, int32_t* out_ids, float* out_probs, const IfabFabric* fab, void* stream) {
  if (T < 1 || T > 64 || top_k < 1 || top_k > KMAX || V_local < 1) return -1;
  const int nblocks = (V_local + CHUNK - 1) / CHUNK;
  if (nblocks > 64) return -1;
  if ((uint64_t)T * nblocks * KMAX * sizeof(Cand) > scratch_bytes) return -5;
  cudaStream_t s = (cudaStream_t)stream;
  SampleParams a{logits, ld, T, V_local, vocab_offset, top_k, inv_temperature, counts, ldc, penalties, (Cand*)scratch, nblocks};
  if (int rc = launch_chain(sample_block_topk_kernel, dim3(nblocks, T), dim3(256), 0, s, a)) return rc;
  FinishParams f;
  f.cand = (const Cand*)scratch; f.nblocks = nblocks; f.T = T; f.K = top_k; f.k_rows = top_k_rows;
  f.inv_temperature = inv_temperature; f.top_p = top_p; f.min_p = min_p; f.seeds = seeds; f.counters = counters;
  f.out_ids = out_ids; f.out_probs = out_probs;
  if (int rc = fabric_view(fab, &f.fv)) return rc;
  f.seq = fab->seq; f.done = fab->done;
  if ((size_t)fab->world * T * KMAX * sizeof(Cand) > fab->data_half_bytes) return -3;
  return launch_chain(sample_finish_kernel, dim3(1), dim3(256), 0, s, f);
}

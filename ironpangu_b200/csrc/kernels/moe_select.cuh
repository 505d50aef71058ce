// Top-k expert selection of one token row from its router logits, by one warp.
//
// Softmax scoring (0): probabilities over all experts, the k largest, optionally renormalised to sum 1.
// Sigmoid scoring (1): sigmoid scores, selection on score + bias, weights = score / sum of the selected scores.
// Ties go to the lower expert index, so the result does not depend on lane order. Supports up to 256 experts.
#pragma once
#include "common.cuh"

namespace ifab {

constexpr int MAX_TOPK = 16;

// all 32 lanes of the calling warp take part; lane l holds the logits of experts l, l + 32, ... in score[] (-inf beyond E);
// lane 0 writes ids[0..topk) and wts[0..topk)
constexpr int SELECT_PER_LANE = 8;
__device__ __forceinline__ void select_topk_scores(float (&score)[SELECT_PER_LANE], const float* bias, int E, int topk, int scoring,
                                                   int renorm, float scale, int32_t* ids, float* wts) {
  const int lane = threadIdx.x & 31;
  constexpr int PER = SELECT_PER_LANE;
  float sel[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) mx = fmaxf(mx, score[i]);
  mx = warp_max(mx);
  float denom = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int ei = lane + 32 * i;
    if (ei < E) {
      if (scoring == 0) {
        score[i] = __expf(score[i] - mx);
        denom += score[i];
        sel[i] = score[i];
      } else {
        score[i] = 1.f / (1.f + __expf(-score[i]));
        sel[i] = score[i] + (bias ? bias[ei] : 0.f);
      }
    } else {
      score[i] = 0.f;
      sel[i] = -INFINITY;
    }
  }
  denom = warp_sum(denom);
  float picked_w[MAX_TOPK];
  int picked_e[MAX_TOPK];
  float wsum = 0.f;
  for (int k = 0; k < topk; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int ei = lane + 32 * i;
      if (sel[i] > bv || (sel[i] == bv && ei < bi)) { bv = sel[i]; bi = ei; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    // the owning lane reports the raw score and retires the expert
    float raw = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      if (lane + 32 * i == bi) { raw = score[i]; sel[i] = -INFINITY; }
    }
    raw = warp_sum(raw);
    picked_e[k] = bi;
    picked_w[k] = (scoring == 0) ? raw / denom : raw;
    wsum += picked_w[k];
  }
  if (lane == 0) {
    for (int k = 0; k < topk; ++k) {
      float w = picked_w[k];
      if (scoring == 0) { if (renorm) w = w / wsum; }
      else w = w / (wsum + 1e-20f);
      ids[k] = picked_e[k];
      wts[k] = w * scale;
    }
  }
}

// the same from logits in global memory
__device__ __forceinline__ void select_topk_row(const float* logits, const float* bias, int E, int topk, int scoring,
                                                int renorm, float scale, int32_t* ids, float* wts) {
  const int lane = threadIdx.x & 31;
  float score[SELECT_PER_LANE];
#pragma unroll
  for (int i = 0; i < SELECT_PER_LANE; ++i) {
    const int ei = lane + 32 * i;
    score[i] = (ei < E) ? __ldcg(logits + ei) : -INFINITY;
  }
  select_topk_scores(score, bias, E, topk, scoring, renorm, scale, ids, wts);
}

}  // namespace ifab

// Router selection shared by the standalone routing kernels and the one-launch decode step: one warp turns a
// token's E router scores into top-k expert ids and gate weights (softmax or sigmoid scoring, selection bias,
// group-limited routing, ties to the lowest id).  Contract of the reference router
// (native/shared/cuda/expert_router.cu:12-55,108-158): bias is used for selection only, weights come from the
// unbiased scores, normalised over the top-k with +1e-20, times the routed scale.
#pragma once

#include "common.cuh"

namespace cafd {

// ---- router -------------------------------------------------------------------------------------
// One warp routes one token: `row` points at its E router logits in global memory.
template <int kPerLane>
__device__ __forceinline__ void route_row(const float* row, const float* __restrict__ bias, int* __restrict__ out_idx,
                                          float* __restrict__ out_w, int t, int E, int top_k, int sigmoid, int num_groups,
                                          int topk_groups, int normalize, float routed_scale) {
  const int lane = threadIdx.x & 31;
  float score[kPerLane], sel[kPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = j * 32 + lane;
    score[j] = e < E ? __ldcg(row + e) : -INFINITY;     // written by other blocks (or an earlier kernel): skip L1
    mx = fmaxf(mx, score[j]);
  }
  if (sigmoid) {
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = j * 32 + lane;
      score[j] = e < E ? 1.0f / (1.0f + expf(-score[j])) : -INFINITY;
    }
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = j * 32 + lane;
      score[j] = e < E ? expf(score[j] - mx) : 0.f;
      sum += score[j];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = j * 32 + lane;
      score[j] = e < E ? score[j] / sum : -INFINITY;
    }
  }
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = j * 32 + lane;
    sel[j] = e < E ? score[j] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  if (num_groups > 1) {
    const int per_group = E / num_groups;
    // group of each of this lane's experts, computed once (the loops below would otherwise divide per element)
    int gid[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = j * 32 + lane;
      gid[j] = e < E ? e / per_group : -1;
    }
    unsigned keep = 0;   // bit g set = group g kept
    float gscore_mine = -INFINITY;   // lane g holds the score of group g
    for (int g = 0; g < num_groups; ++g) {
      // the group's two best selection scores: per-lane best and runner-up first, then one warp reduction of pairs
      float top1 = -INFINITY, top2 = -INFINITY;
      int i1 = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {
        if (gid[j] == g) {
          const int e = j * 32 + lane;
          if (sel[j] > top1 || (sel[j] == top1 && e < i1)) { top2 = top1; top1 = sel[j]; i1 = e; }
          else top2 = fmaxf(top2, sel[j]);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, top1, o);
        const float o2 = __shfl_xor_sync(0xffffffffu, top2, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i1, o);
        if (o1 > top1 || (o1 == top1 && oi < i1)) { top2 = fmaxf(top1, o2); top1 = o1; i1 = oi; }
        else top2 = fmaxf(top2, o1);
      }
      if (lane == g) gscore_mine = top1 + top2;
    }
    for (int it = 0; it < topk_groups; ++it) {
      float v = (lane < num_groups && !((keep >> lane) & 1u)) ? gscore_mine : -INFINITY;
      int gi = lane;
      // groups with -inf scores can still be picked when fewer finite ones exist: mark via index
      if (!(lane < num_groups) || ((keep >> lane) & 1u)) gi = 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, gi, o);
        if (ov > v || (ov == v && oi < gi)) { v = ov; gi = oi; }
      }
      if (gi != 0x7fffffff) keep |= 1u << gi;
    }
#pragma unroll
    for (int j = 0; j < kPerLane; ++j)
      if (gid[j] >= 0 && !((keep >> gid[j]) & 1u)) sel[j] = -INFINITY;
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_i = 0;
  unsigned taken = 0;   // bit j: this lane's element j was already selected
  for (int it = 0; it < top_k; ++it) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    float bs = 0.f;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = j * 32 + lane;
      if (e < E && !((taken >> j) & 1u) && (sel[j] > bv || (sel[j] == bv && e < bi))) { bv = sel[j]; bi = e; bs = score[j]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bs = os; }
    }
    if (bi == 0x7fffffff) { bi = 0; bs = 0.f; }   // every candidate was NaN
#pragma unroll
    for (int j = 0; j < kPerLane; ++j)
      if (j * 32 + lane == bi) taken |= 1u << j;
    wsum += bs;
    if (lane == it) { my_w = bs; my_i = bi; }
  }
  if (lane < top_k) {
    float w = my_w;
    if (normalize) w = w / (wsum + 1e-20f);
    out_idx[static_cast<size_t>(t) * top_k + lane] = my_i;
    out_w[static_cast<size_t>(t) * top_k + lane] = w * routed_scale;
  }
}

}  // namespace cafd

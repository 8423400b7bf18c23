// Routing of one token by one warp (DeepSeek-V3 no-aux), shared by the routing kernels.
//
// Semantics follow the reference's torch check (experiments/fast_bench/correctness_bench.py:47-61)
// and replace the arithmetic of its `fused_route_topk_kernel` (solution/python/moe_fused.cu:568-698):
// fp32 logits are used as given, group scores count equal values with multiplicity, and every
// selection breaks ties toward the lowest index.
#pragma once

#include "common.cuh"

namespace b200moe {

// Monotone map fp32 -> uint32 (a < b  <=>  key(a) < key(b), with -0 < +0 adjacent).
__device__ __forceinline__ uint32_t order_key(float v) {
  uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    unsigned long long o = __shfl_xor_sync(0xffffffffu, v, off);
    v = o > v ? o : v;
  }
  return v;
}

// sigmoid evaluated in fp64 and rounded once to fp32: within one rounding of the exact
// value, so expert ids can differ from another correctly evaluated sigmoid only when two
// competing scores are within an fp32 ulp of each other.
__device__ __forceinline__ float sigmoid_round_once(float x) {
  return (float)(1.0 / (1.0 + exp(-(double)x)));
}

// Lane L owns expert g*32+L of every group g (`b[g]` = its bias), so a group reduction is a
// warp reduction.  On return lane k < 8 holds the k-th selected expert and its weight
// s * (rsf / (sum of the selected s + 1e-20)); other lanes hold unspecified values.
__device__ __forceinline__ void route_one_token(const void* __restrict__ logits, int logits_dtype, int t,
                                                const float (&b)[kNumGroups], float rsf, int lane, int& my_id,
                                                float& my_weight) {
    // Every selection is "maximum key, lowest index among equals": one warp-wide integer
    // max (redux.sync) on the order keys plus a ballot, instead of a shuffle tree.
    float s[kNumGroups];
    uint32_t key[kNumGroups];   // order key of sigmoid + bias (never 0 for a finite value)
    float gscore = 0.f;         // lane g (< 8) keeps the score of group g
#pragma unroll
    for (int g = 0; g < kNumGroups; ++g) {
      float x = load_as_float(logits, logits_dtype, (size_t)t * kNumExperts + g * 32 + lane);
      s[g] = sigmoid_round_once(x);
      key[g] = order_key(s[g] + b[g]);
    }
#pragma unroll
    for (int g = 0; g < kNumGroups; ++g) {
      // top-2 with multiplicity: best key, drop ONE lane that holds it, best key again
      const uint32_t k1 = __reduce_max_sync(0xffffffffu, key[g]);
      const uint32_t holders = __ballot_sync(0xffffffffu, key[g] == k1);
      const int first = __ffs(holders) - 1;
      const uint32_t k2 = __reduce_max_sync(0xffffffffu, lane == first ? 0u : key[g]);
      const float v1 = __uint_as_float((k1 & 0x80000000u) ? (k1 & 0x7fffffffu) : ~k1);
      const float v2 = __uint_as_float((k2 & 0x80000000u) ? (k2 & 0x7fffffffu) : ~k2);
      if (lane == g) gscore = v1 + v2;
    }
    // top-4 groups, lowest group index on ties
    uint32_t gk = lane < kNumGroups ? order_key(gscore) : 0u;
    uint32_t group_mask = 0;
#pragma unroll
    for (int r = 0; r < kTopKGroups; ++r) {
      const uint32_t best = __reduce_max_sync(0xffffffffu, gk);
      const uint32_t holders = __ballot_sync(0xffffffffu, gk == best && lane < kNumGroups);
      const int g = __ffs(holders) - 1;
      group_mask |= 1u << g;
      if (lane == g) gk = 0u;
    }
    // top-8 experts among the kept groups, lowest expert id on ties; a taken or masked candidate has key 0
    uint32_t cand[kNumGroups];
#pragma unroll
    for (int g = 0; g < kNumGroups; ++g) cand[g] = ((group_mask >> g) & 1u) ? key[g] : 0u;
    float ssum = 0.f;
    float my_s = 0.f;   // lane k keeps s of the k-th winner
    my_id = 0;
#pragma unroll
    for (int k = 0; k < kTopK; ++k) {
      uint32_t loc = cand[0];
#pragma unroll
      for (int g = 1; g < kNumGroups; ++g) loc = cand[g] > loc ? cand[g] : loc;
      const uint32_t best = __reduce_max_sync(0xffffffffu, loc);
      uint32_t mine = 0xffffffffu;   // lowest id this lane holds at the best key
#pragma unroll
      for (int g = kNumGroups - 1; g >= 0; --g)
        if (cand[g] == best) mine = (uint32_t)(g * 32 + lane);
      const int id = (int)__reduce_min_sync(0xffffffffu, mine);
      const int wl = id & 31, wg = id >> 5;
      float sw = 0.f;
#pragma unroll
      for (int g = 0; g < kNumGroups; ++g) {
        if (g == wg) {
          sw = s[g];
          if (lane == wl) cand[g] = 0u;
        }
      }
      sw = __shfl_sync(0xffffffffu, sw, wl);
      ssum += sw;   // left-to-right fp32 sum in rank order, identical on every lane
      if (lane == k) { my_s = sw; my_id = id; }
    }
    const float factor = rsf / (ssum + 1e-20f);
    my_weight = my_s * factor;
}

}  // namespace b200moe

// Device functions shared by the sampler kernels (elt/sampler.cu) and the sampling epilogue of the LM-head GEMM
// (gemm/gemm_bf16_sm100.cu): the counter-based random numbers, the Gumbel noise and the arg-max pair.
//
// Sampling is done in two levels, because one random number per logit is what makes a sampler slow (a Philox call and two
// logarithms per token id: ~120 us for 256 x 151936 logits, ten times the time to read them):
//
//   level 1  the vocabulary is cut into groups of 16 consecutive GLOBAL token ids.  max_i (x_i + Gumbel_i) over a group is
//            distributed as logsumexp_i(x_i) + Gumbel, so one noise value per group decides which group holds the winner:
//            score_g = logsumexp(x_i, i in g) + Gumbel(row, g), x = logit / T.  One exponential per logit, one Philox call per
//            four groups.
//   level 2  inside the winning group the token is drawn with per-token noise: argmax_i (x_i + Gumbel(row, i)), i in g.
//
// The result is a draw from softmax(logits / T), as the reference's softmax(logits / T) / Exp(1) arg-max is
// (tinyvllm/layers/sampler.py:13-21).  T == 0: score_g = max of the group, token = first arg-max (no noise).
// All noise is Philox-4x32-10 keyed by the engine seed: tokens use counter (id / 4, row, step, 0), lane id % 4; groups use
// counter (g / 4, row, step, 1), lane g % 4.  Everything is a pure function of (seed, step, row, GLOBAL id), so a vocabulary
// sharded over tensor-parallel ranks (shards start on multiples of 16) or cut into GEMM tiles samples the same token as an
// unsharded one.  ops/ref.py states the same procedure on the CPU.
#pragma once

#include "ptx.cuh"

namespace forge {

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                              uint32_t out[4]) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Gumbel noise -log(-log u) from 24 random bits, u = (k + 0.5) / 2^24.
// E = -log u is an Exp(1) variate and the noise is -log E.  Only large noise values can win the arg-max, i.e.
// small E, i.e. u close to 1, where a fast log of u would lose all relative accuracy.  There E is computed from
// w = 1 - u (exact in fp32) by its series, elsewhere by the hardware log; the outer log only needs absolute
// accuracy (1e-6 on a noise value is far below bf16 logit resolution).  ~6x fewer instructions than two accurate
// logf calls; the CPU statement in ops/ref.py (accurate logs) agrees to ~1e-6.
__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
  const uint32_t k = bits >> 8;
  const float u = (static_cast<float>(k) + 0.5f) * (1.0f / 16777216.0f);
  const float w = (static_cast<float>(0xFFFFFFu - k) + 0.5f) * (1.0f / 16777216.0f);      // 1 - u, exact
  const float e_series = w * (1.0f + w * (0.5f + w * (0.33333334f + w * 0.25f)));        // -log(1 - w), w < 1/64
  const float e = w < 0.015625f ? e_series : -__logf(u);
  return -__logf(e);
}

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {   // larger value wins; ties go to the smaller index
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ Best warp_best(Best x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  return x;
}

constexpr int kSampleGroup = 16;
constexpr float kLog2e = 1.4426950408889634f;

// Level 1 for one group: lv[16] are the (bf16-rounded) logits, -INFINITY where the id lies outside the shard.
// noise_bits: the Philox word of this group (ignored when greedy).  Returns the group's score (-INFINITY for an empty group).
__device__ __forceinline__ float sample_group_score(const float lv[kSampleGroup], float inv_t, bool greedy, uint32_t noise_bits) {
  float m = lv[0];
#pragma unroll
  for (int i = 1; i < kSampleGroup; ++i) m = fmaxf(m, lv[i]);
  if (greedy || m == -INFINITY) return m;
  const float c = inv_t * kLog2e, mc = m * c;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kSampleGroup; ++i) s += ex2_approx(lv[i] * c - mc);      // -inf -> 0
  return m * inv_t + __logf(s) + gumbel_from_bits(noise_bits);
}

// Level 2 for the winning group: the token inside group g (global ids 16 g .. 16 g + 15).
__device__ __forceinline__ int sample_group_token(const float lv[kSampleGroup], int g, float inv_t, bool greedy, uint32_t row,
                                                  uint32_t step, uint32_t k0, uint32_t k1) {
  Best best{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int q = 0; q < kSampleGroup / 4; ++q) {
    uint32_t rnd[4] = {0, 0, 0, 0};
    if (!greedy) philox4x32_10(static_cast<uint32_t>(g * (kSampleGroup / 4) + q), row, step, 0u, k0, k1, rnd);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float l = lv[q * 4 + j];
      if (l != -INFINITY) {
        float sc = l * inv_t;
        if (!greedy) sc += gumbel_from_bits(rnd[j]);
        best = better(best, Best{sc, g * kSampleGroup + q * 4 + j});
      }
    }
  }
  return best.i;
}

}  // namespace forge

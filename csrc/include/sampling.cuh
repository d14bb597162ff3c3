// Device functions shared by the sampler kernels (elt/sampler.cu) and the sampling epilogue of the LM-head GEMM
// (gemm/gemm_bf16_sm100.cu): the counter-based random numbers, the Gumbel noise and the arg-max pair.
//
// u_i comes from Philox-4x32-10 keyed by the engine seed with counter (global vocab id / 4, row, step, 0),
// lane = id % 4: a pure function of (seed, step, row, GLOBAL vocab id), so a vocabulary sharded over
// tensor-parallel ranks, or cut into GEMM tiles, samples the same token as an unsharded one.
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

}  // namespace forge

// Pieces shared by the two decode-attention kernels (context split into fixed chunks; flat tile partition):
// the per-lane query slice, one tile of online softmax for a consumer warp, and the merge of the four
// consumer warps' states.  head_dim is 128; scores use exp2 with the scale folded into q.
#pragma once
#include "ptx.cuh"

namespace forge {

constexpr int kD = 128;
constexpr int kDecStages = 3;
constexpr int kDecThreads = 160;   // 4 consumer warps + 1 producer warp

// q heads that share a KV head are processed together in slices of G heads (each K/V byte is read from shared memory
// once per slice, and streamed from the cache once per slice): the largest supported G that divides the group.  G <= 4
// leaves room for two CTAs per SM; G = 5 (Qwen3-14B: 40 / 8 heads) takes the registers of a whole SM but reads the cache
// once instead of five times.  A group of 8 (Qwen3-32B) runs as two slices of 4: with 8 heads per slice the CUDA-core dot
// products, not the cache stream, bound the kernel (measured: a 32B decode pass 30.3 s with G = 8, 24.6 s with 2 x 4).
__host__ __device__ constexpr int decode_group_slice(int group) {
  return group % 5 == 0 ? 5 : group % 4 == 0 ? 4 : group % 3 == 0 ? 3 : group % 2 == 0 ? 2 : 1;
}
__host__ __device__ constexpr int decode_ctas_per_sm(int G) { return G > 4 ? 1 : 2; }

template <int G>
struct DecodeState {
  float m[G], l[G], acc[G][4];
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[g][e] = 0.f;
    }
  }
};

// Optional fusion of the step's q/k-norm + RoPE + KV store into the attention kernel (decode only: one new token per
// sequence, at position len - 1).  qkv == nullptr: q is final and the cache already holds the newest token.
struct DecodeFuse {
  const __nv_bfloat16* qkv;     // [B, (nq + 2 nkv) * 128] raw projections: q heads, k heads, v heads
  int ld_qkv;
  const __nv_bfloat16* q_w;     // RMSNorm weights over head_dim, may be null
  const __nv_bfloat16* k_w;
  float eps;
  const float* rope;            // [rope_rows][128]: cos of the 64 frequencies, then sin; null: no rotation
  int rope_rows;
};

__device__ __forceinline__ float decode_bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// One head (128 values) of the raw projection -> RMSNorm (weight w, may be null) -> NeoX rotation with the table row
// `cs` (may be null) -> rounded to bf16, i.e. exactly what qk_norm_rope_store_kernel would have stored.  Lane layout as
// in decode_load_q: j = lane % 8 holds elements [8j, 8j+8) in x[0..8) and [64+8j, 64+8j+8) in x[8..16): the pairs
// (i, i + 64) that the rotation mixes sit in the same lane.  The four 8-lane groups compute the same values.
__device__ __forceinline__ void decode_norm_rope_head(const __nv_bfloat16* __restrict__ src, const __nv_bfloat16* __restrict__ w, float eps,
                                                      const float* __restrict__ cs, int lane, float (&x)[16]) {
  const int j = lane & 7;
  {
    const uint4 lo = *reinterpret_cast<const uint4*>(src + 8 * j);
    const uint4 hi = *reinterpret_cast<const uint4*>(src + 64 + 8 * j);
    const uint32_t r[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      x[2 * e] = bf16_lo(r[e]);
      x[2 * e + 1] = bf16_hi(r[e]);
    }
  }
  if (w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) ss = fmaf(x[e], x[e], ss);
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    const float inv = rsqrtf(ss * (1.0f / kD) + eps);
    const uint4 lo = *reinterpret_cast<const uint4*>(w + 8 * j);
    const uint4 hi = *reinterpret_cast<const uint4*>(w + 64 + 8 * j);
    const uint32_t r[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      x[2 * e] = decode_bf16_round(decode_bf16_round(x[2 * e] * inv) * bf16_lo(r[e]));
      x[2 * e + 1] = decode_bf16_round(decode_bf16_round(x[2 * e + 1] * inv) * bf16_hi(r[e]));
    }
  }
  if (cs != nullptr) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float c = cs[8 * j + e], sn = cs[64 + 8 * j + e];
      const float x1 = x[e], x2 = x[8 + e];
      x[e] = x1 * c - x2 * sn;
      x[8 + e] = x2 * c + x1 * sn;
    }
  }
#pragma unroll
  for (int e = 0; e < 16; ++e) x[e] = decode_bf16_round(x[e]);
}

// q of one item from the raw projection: norm, rotation at position len - 1, scale.
template <int G>
__device__ __forceinline__ void decode_load_q_fused(const DecodeFuse& f, int b, int qh0, int len, int lane, float scale_log2,
                                                    float (&qr)[G][16]) {
  const float* cs = nullptr;
  if (f.rope != nullptr) cs = f.rope + static_cast<size_t>(min(max(len - 1, 0), f.rope_rows - 1)) * kD;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float x[16];
    decode_norm_rope_head(f.qkv + static_cast<size_t>(b) * f.ld_qkv + static_cast<size_t>(qh0 + g) * kD, f.q_w, f.eps, cs, lane, x);
#pragma unroll
    for (int e = 0; e < 16; ++e) qr[g][e] = x[e] * scale_log2;
  }
}

// The newest token (position len - 1) of KV head kvh of sequence b: k = norm + rotation of the raw projection, v = raw.
// Two steps so that the global loads and the arithmetic happen at the START of an item, under the latency of the q loads
// and of the first tiles, and only register -> shared / global stores remain when the tile with that token arrives.
struct DecodeNewToken {
  uint4 k_lo, k_hi;     // lanes 0..7: elements [8 lane, 8 lane + 8) and [64 + 8 lane, ...) of k, bf16
  uint2 v;              // every lane: elements [4 lane, 4 lane + 4) of v, bf16
};

__device__ __forceinline__ DecodeNewToken decode_new_token(const DecodeFuse& f, int b, int kvh, int nq, int nkv, int len, int lane) {
  const float* cs = nullptr;
  if (f.rope != nullptr) cs = f.rope + static_cast<size_t>(min(max(len - 1, 0), f.rope_rows - 1)) * kD;
  float x[16];
  decode_norm_rope_head(f.qkv + static_cast<size_t>(b) * f.ld_qkv + static_cast<size_t>(nq + kvh) * kD, f.k_w, f.eps, cs, lane, x);
  DecodeNewToken t;
  t.k_lo = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
  t.k_hi = make_uint4(pack_bf16x2(x[8], x[9]), pack_bf16x2(x[10], x[11]), pack_bf16x2(x[12], x[13]), pack_bf16x2(x[14], x[15]));
  t.v = *reinterpret_cast<const uint2*>(f.qkv + static_cast<size_t>(b) * f.ld_qkv + static_cast<size_t>(nq + nkv + kvh) * kD + lane * 4);
  return t;
}

// Executed by the ONE consumer warp that owns row `row` of the tile that has just landed in shared memory (Ks / Vs): the
// row is replaced there (the cache does not hold it yet) and, if `to_cache`, written to the cache for later steps.
// Only this warp reads that row of the tile, so __syncwarp orders the patch before the use.
__device__ __forceinline__ void decode_patch_new_token(const DecodeNewToken& t, int row, uint8_t* Ks, uint8_t* Vs, __nv_bfloat16* k_dst,
                                                       __nv_bfloat16* v_dst, bool to_cache, int lane) {
  if (lane < 8) {                                                     // one of the four identical groups writes
    *reinterpret_cast<uint4*>(Ks + row * (kD * 2) + lane * 16) = t.k_lo;
    *reinterpret_cast<uint4*>(Ks + row * (kD * 2) + 128 + lane * 16) = t.k_hi;
    if (to_cache) {
      *reinterpret_cast<uint4*>(k_dst + 8 * lane) = t.k_lo;
      *reinterpret_cast<uint4*>(k_dst + 64 + 8 * lane) = t.k_hi;
    }
  }
  *reinterpret_cast<uint2*>(Vs + row * (kD * 2) + lane * 8) = t.v;
  if (to_cache) *reinterpret_cast<uint2*>(v_dst + lane * 4) = t.v;
  fence_proxy_async_smem();            // a later bulk copy into this stage must be ordered after these generic writes
  __syncwarp();
}

// q slices this lane multiplies: elements [8j, 8j+8) and [64+8j, 64+8j+8) of every head of the group (j = lane % 8)
template <int G>
__device__ __forceinline__ void decode_load_q(const __nv_bfloat16* __restrict__ q_row0, int lane, float scale_log2, float (&qr)[G][16]) {
  const int j = lane & 7;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = q_row0 + static_cast<size_t>(g) * kD;
    const uint4 lo = *reinterpret_cast<const uint4*>(qp + 8 * j);
    const uint4 hi = *reinterpret_cast<const uint4*>(qp + 64 + 8 * j);
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      qr[g][2 * e] = bf16_lo(w[e]) * scale_log2;
      qr[g][2 * e + 1] = bf16_hi(w[e]) * scale_log2;
    }
  }
}

// One tile (TILE tokens of K and V in shared memory) for consumer warp `warp`: scores of its TILE / 4 tokens,
// online softmax update, O += P V.  `valid_tokens`: tokens of the tile that exist (the rest is masked).
template <int G, int TILE>
__device__ __forceinline__ void decode_consume_tile(const uint8_t* Ks, const uint8_t* Vs, int valid_tokens, int warp, int lane,
                                                    const float (&qr)[G][16], DecodeState<G>& st) {
  constexpr int TPW = TILE / 4;          // tokens per consumer warp per tile
  constexpr int ITERS = TPW / 4;         // QK iterations (4 tokens per warp at a time)
  const int grp = lane >> 3, j = lane & 7;
  float sc[ITERS][G];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int r = warp * TPW + it * 4 + grp;
    const uint4 k0 = *reinterpret_cast<const uint4*>(Ks + r * (kD * 2) + j * 16);
    const uint4 k1 = *reinterpret_cast<const uint4*>(Ks + r * (kD * 2) + 128 + j * 16);
    const uint32_t w[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
    float kf[16];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      kf[2 * e] = bf16_lo(w[e]);
      kf[2 * e + 1] = bf16_hi(w[e]);
    }
    const bool valid = r < valid_tokens;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < 16; ++e) d = fmaf(qr[g][e], kf[e], d);
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      sc[it][g] = valid ? d : -INFINITY;
    }
  }
  // online softmax over this warp's TPW tokens
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float mt = sc[0][g];
#pragma unroll
    for (int it = 1; it < ITERS; ++it) mt = fmaxf(mt, sc[it][g]);
    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 8));
    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
    const float m_new = fmaxf(st.m[g], mt);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;      // every token masked so far
    const float alpha = exp2f(st.m[g] - m_use);                // exp2(-inf) = 0 on the first tile
    float ps = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      sc[it][g] = exp2f(sc[it][g] - m_use);                    // masked -> 0
      ps += sc[it][g];
    }
    st.l[g] = st.l[g] * alpha + ps;                            // per token group; summed over groups at the end
    st.m[g] = m_new;
#pragma unroll
    for (int e = 0; e < 4; ++e) st.acc[g][e] *= alpha;
  }
  // O += P V : lane owns d = 4*lane .. 4*lane+3
#pragma unroll
  for (int i = 0; i < TPW; ++i) {
    const int r = warp * TPW + i;
    const uint2 vv = *reinterpret_cast<const uint2*>(Vs + r * (kD * 2) + lane * 8);
    const float v0 = bf16_lo(vv.x), v1 = bf16_hi(vv.x), v2 = bf16_lo(vv.y), v3 = bf16_hi(vv.y);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float p = __shfl_sync(0xffffffffu, sc[i / 4][g], (i % 4) * 8);
      st.acc[g][0] = fmaf(p, v0, st.acc[g][0]);
      st.acc[g][1] = fmaf(p, v1, st.acc[g][1]);
      st.acc[g][2] = fmaf(p, v2, st.acc[g][2]);
      st.acc[g][3] = fmaf(p, v3, st.acc[g][3]);
    }
  }
}

// After the last tile: each 8-lane group summed its own tokens (lanes 0, 8, 16, 24 hold the four partial sums);
// then every consumer warp publishes its state to shared memory ([4][G][128] + [4][G] + [4][G] floats).
template <int G>
__device__ __forceinline__ void decode_publish_state(DecodeState<G>& st, float* s_acc, int warp, int lane) {
  float* s_m = s_acc + 4 * G * kD;
  float* s_l = s_m + 4 * G;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    st.l[g] += __shfl_xor_sync(0xffffffffu, st.l[g], 8);
    st.l[g] += __shfl_xor_sync(0xffffffffu, st.l[g], 16);
    *reinterpret_cast<float4*>(s_acc + (warp * G + g) * kD + lane * 4) = make_float4(st.acc[g][0], st.acc[g][1], st.acc[g][2], st.acc[g][3]);
    if (lane == 0) {
      s_m[warp * G + g] = st.m[g];
      s_l[warp * G + g] = st.l[g];
    }
  }
}

// Thread d (0..127) merges the four warps' states for head g: normalised output element d, running max M, sum L.
template <int G>
__device__ __forceinline__ float decode_merged(const float* s_acc, int g, int d, float& M, float& L) {
  const float* s_m = s_acc + 4 * G * kD;
  const float* s_l = s_m + 4 * G;
  M = -INFINITY;
#pragma unroll
  for (int w = 0; w < 4; ++w) M = fmaxf(M, s_m[w * G + g]);
  L = 0.f;
  float O = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const float mw = s_m[w * G + g];
    const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
    L += s_l[w * G + g] * f;
    O += s_acc[(w * G + g) * kD + d] * f;
  }
  return L > 0.f ? O / L : 0.f;
}

constexpr int decode_merge_floats(int G) { return 4 * G * kD + 8 * G; }

}  // namespace forge

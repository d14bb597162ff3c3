// Memory-bound ops of a decoder block as hand-written kernels: 16-byte accesses, fp32 math, one pass.
//
//   rms_norm / add_rms_norm     tinyvllm/layers/layernorm.py:21-45   (Inductor-generated there)
//   qk_norm_rope_store          tinyvllm/models/qwen3.py:79-94 + tinyvllm/layers/rotary_embedding.py:42-57 +
//                               tinyvllm/layers/attention.py:9-48: four launches there, one here
//   silu_mul                    tinyvllm/layers/activation.py:11-14
//   embedding (vocab shard)     tinyvllm/layers/embed_head.py:34-40
//   gather_rows                 tinyvllm/layers/embed_head.py:60-62 (last token of every sequence)
//
// Rounding follows the PyTorch statement of each op in ops/ref.py so results match it bit for bit where
// the order of fp32 additions allows.
#include "../include/launch.cuh"
#include "../include/ptx.cuh"

namespace forge {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ---------------------------------------------------------------------------------------------------------
// y = rms_norm(x (+ residual)) * w ; residual <- x + residual (rounded to bf16).  One CTA per row; a row of
// up to 4 * blockDim * 8 elements stays in registers between the two passes.
// ---------------------------------------------------------------------------------------------------------
constexpr int kNormMaxChunks = 4;

template <bool kAdd>
__global__ void __launch_bounds__(256) rms_norm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                                                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                       int H, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  uint4* rr = kAdd ? reinterpret_cast<uint4*>(residual + row * H) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
  const int nvec = H >> 3;
  float vals[kNormMaxChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kNormMaxChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nvec) {
      uint4 a = xr[i];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
      if constexpr (kAdd) {
        uint4 b = rr[i];
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t sw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = bf16_round(bf16_lo(aw[j]) + bf16_lo(bw[j]));
          const float hi = bf16_round(bf16_hi(aw[j]) + bf16_hi(bw[j]));
          vals[c][2 * j] = lo;
          vals[c][2 * j + 1] = hi;
          sw[j] = pack_bf16x2(lo, hi);
        }
        rr[i] = make_uint4(sw[0], sw[1], sw[2], sw[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          vals[c][2 * j] = bf16_lo(aw[j]);
          vals[c][2 * j + 1] = bf16_hi(aw[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[c][j] * vals[c][j];
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / static_cast<float>(H) + eps);
#pragma unroll
  for (int c = 0; c < kNormMaxChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nvec) {
      uint4 wv = wr[i];
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = bf16_round(vals[c][2 * j] * inv) * bf16_lo(ww[j]);
        const float hi = bf16_round(vals[c][2 * j + 1] * inv) * bf16_hi(ww[j]);
        o[j] = pack_bf16x2(lo, hi);
      }
      yr[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

extern "C" int forge_rms_norm(const void* x, void* residual, const void* w, void* y, int rows, int H, float eps,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > kNormMaxChunks * 256 * 8) return -1;
  int threads = ((H >> 3) + kNormMaxChunks - 1) / kNormMaxChunks;
  threads = ((threads + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  if (threads > 256) threads = 256;
  cudaError_t e;
  if (residual != nullptr)
    e = launch_kernel(rms_norm_kernel<true>, dim3(rows), dim3(threads), 0, stream, 0, static_cast<const __nv_bfloat16*>(x),
                      static_cast<__nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), H, eps);
  else
    e = launch_kernel(rms_norm_kernel<false>, dim3(rows), dim3(threads), 0, stream, 0, static_cast<const __nv_bfloat16*>(x),
                      static_cast<__nv_bfloat16*>(nullptr), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), H, eps);
  return e == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------------
// Fused split + per-head RMSNorm(q, k) + NeoX RoPE(q, k) + paged KV store.
// One warp per (token, head) of the packed qkv row [q heads | k heads | v heads].
//   q head: normalise, rotate, write q_out[token, head, :]
//   k head: normalise, rotate, write k_cache[slot];  v head: copy to v_cache[slot]
// Cache layout [blocks, kv_heads, block_size, D]; slot = block * block_size + offset; slot < 0 is skipped,
// slot >= num_slots is skipped and reported in the status word.
// Lane l owns elements {l*E .. l*E+E-1} of the first half and the same of the second half (E = D / 64),
// i.e. exactly the pairs the rotation mixes.
// ---------------------------------------------------------------------------------------------------------
// E consecutive bf16 values as one memory access.
template <int E> struct BfVec;
template <> struct BfVec<1> { using T = unsigned short; };
template <> struct BfVec<2> { using T = uint32_t; };
template <> struct BfVec<4> { using T = uint2; };

template <int E>
__device__ __forceinline__ void load_bf(const __nv_bfloat16* p, float* f) {
  const typename BfVec<E>::T raw = *reinterpret_cast<const typename BfVec<E>::T*>(p);
  if constexpr (E == 1) {
    f[0] = __uint_as_float(static_cast<uint32_t>(raw) << 16);
  } else if constexpr (E == 2) {
    f[0] = bf16_lo(raw); f[1] = bf16_hi(raw);
  } else {
    f[0] = bf16_lo(raw.x); f[1] = bf16_hi(raw.x); f[2] = bf16_lo(raw.y); f[3] = bf16_hi(raw.y);
  }
}
template <int E>
__device__ __forceinline__ void store_bf(__nv_bfloat16* p, const float* f) {
  if constexpr (E == 1) {
    *p = __float2bfloat16_rn(f[0]);
  } else if constexpr (E == 2) {
    *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(f[0], f[1]);
  } else {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
  }
}

// One warp handles `hpw` consecutive heads of one token, so the token's position, slot and its cos/sin row are
// fetched once per warp (the table row is twice the size of a head).
template <int D>
__global__ void __launch_bounds__(128) qk_norm_rope_store_kernel(
    const __nv_bfloat16* __restrict__ qkv, int ld_qkv, const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
    float eps, const float* __restrict__ rope, int rope_rows, const int* __restrict__ positions, const int* __restrict__ slots,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
    int T, int nq, int nkv, int block_size, long long num_slots, int do_rope, int hpw, unsigned* status) {
  constexpr int E = D / 64;           // elements per lane per half
  static_assert(D == 64 || D == 128 || D == 256, "head_dim");
  pdl_launch_dependents();
  pdl_wait();
  const int heads = nq + 2 * nkv;
  const int groups = (heads + hpw - 1) / hpw;
  const long long wid = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= static_cast<long long>(T) * groups) return;
  const int lane = threadIdx.x & 31;
  const int t = static_cast<int>(wid / groups);
  const int h_begin = static_cast<int>(wid % groups) * hpw;
  const int h_end = min(h_begin + hpw, heads);

  float cosv[E], sinv[E], wq1[E], wq2[E], wk1[E], wk2[E];
  if (do_rope) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= rope_rows ? rope_rows - 1 : pos);
    const float* cs = rope + static_cast<size_t>(pos) * D;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      cosv[e] = cs[lane * E + e];
      sinv[e] = cs[D / 2 + lane * E + e];
    }
  }
  if (qw != nullptr) { load_bf<E>(qw + lane * E, wq1); load_bf<E>(qw + D / 2 + lane * E, wq2); }
  if (kw != nullptr) { load_bf<E>(kw + lane * E, wk1); load_bf<E>(kw + D / 2 + lane * E, wk2); }
  const long long slot = slots[t];
  const bool slot_ok = slot >= 0 && slot < num_slots;
  if (slot >= num_slots && lane == 0) set_status(status, kStatusBadIndex);

  for (int h = h_begin; h < h_end; ++h) {
    const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * ld_qkv + static_cast<size_t>(h) * D;
    float a[E], b[E];   // first-half and second-half elements: exactly the pairs the rotation mixes
    load_bf<E>(src + lane * E, a);
    load_bf<E>(src + D / 2 + lane * E, b);
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    if (is_q || is_k) {
      const bool has_w = is_q ? qw != nullptr : kw != nullptr;
      if (has_w) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) ss += a[e] * a[e] + b[e] * b[e];
        const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(D) + eps);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          a[e] = bf16_round(bf16_round(a[e] * inv) * (is_q ? wq1[e] : wk1[e]));
          b[e] = bf16_round(bf16_round(b[e] * inv) * (is_q ? wq2[e] : wk2[e]));
        }
      }
      if (do_rope) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float x1 = a[e], x2 = b[e];
          a[e] = x1 * cosv[e] - x2 * sinv[e];
          b[e] = x2 * cosv[e] + x1 * sinv[e];
        }
      }
    }
    __nv_bfloat16* dst;
    if (is_q) {
      dst = q_out + (static_cast<size_t>(t) * nq + h) * D;
    } else {
      if (!slot_ok) continue;
      const int kvh = is_k ? h - nq : h - nq - nkv;
      const long long blk = slot / block_size, off = slot % block_size;
      dst = (is_k ? k_cache : v_cache) + ((blk * nkv + kvh) * block_size + off) * D;
    }
    store_bf<E>(dst + lane * E, a);
    store_bf<E>(dst + D / 2 + lane * E, b);
  }
}


// head_dim 128: eight lanes per head, each lane holds elements [8j, 8j+8) and [64+8j, 64+8j+8) (j = lane % 8): exactly the
// pairs the rotation mixes, moved with 16-byte accesses; a warp works on four heads of one token at a time and walks
// `hpw` consecutive heads, so the token's position, slot and cos/sin values are fetched once per warp.
__global__ void __launch_bounds__(128) qk_norm_rope_store128_kernel(
    const __nv_bfloat16* __restrict__ qkv, int ld_qkv, const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
    float eps, const float* __restrict__ rope, int rope_rows, const int* __restrict__ positions, const int* __restrict__ slots,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
    int T, int nq, int nkv, int block_size, long long num_slots, int do_rope, int hpw, unsigned* status) {
  constexpr int D = 128;
  pdl_launch_dependents();
  pdl_wait();
  const int heads = nq + 2 * nkv;
  const int groups = (heads + hpw - 1) / hpw;
  const long long wid = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= static_cast<long long>(T) * groups) return;
  const int lane = threadIdx.x & 31, j = lane & 7, sub = lane >> 3;
  const int t = static_cast<int>(wid / groups);
  const int h_begin = static_cast<int>(wid % groups) * hpw;
  const int h_end = min(h_begin + hpw, heads);

  float cosv[8], sinv[8];
  if (do_rope) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= rope_rows ? rope_rows - 1 : pos);
    const float* cs = rope + static_cast<size_t>(pos) * D;
    const float4 c0 = *reinterpret_cast<const float4*>(cs + 8 * j), c1 = *reinterpret_cast<const float4*>(cs + 8 * j + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(cs + 64 + 8 * j), s1 = *reinterpret_cast<const float4*>(cs + 64 + 8 * j + 4);
    cosv[0] = c0.x; cosv[1] = c0.y; cosv[2] = c0.z; cosv[3] = c0.w; cosv[4] = c1.x; cosv[5] = c1.y; cosv[6] = c1.z; cosv[7] = c1.w;
    sinv[0] = s0.x; sinv[1] = s0.y; sinv[2] = s0.z; sinv[3] = s0.w; sinv[4] = s1.x; sinv[5] = s1.y; sinv[6] = s1.z; sinv[7] = s1.w;
  }
  const long long slot = slots[t];
  const bool slot_ok = slot >= 0 && slot < num_slots;
  if (slot >= num_slots && lane == 0) set_status(status, kStatusBadIndex);

  for (int h0 = h_begin; h0 < h_end; h0 += 4) {
    const int h = h0 + sub;
    const bool live = h < h_end;
    const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * ld_qkv + static_cast<size_t>(live ? h : h_begin) * D;
    uint4 lo = *reinterpret_cast<const uint4*>(src + 8 * j);
    uint4 hi = *reinterpret_cast<const uint4*>(src + 64 + 8 * j);
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    const __nv_bfloat16* w = is_q ? qw : kw;
    if (is_q || is_k) {
      const uint32_t r[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
      float a[8], b[8];                               // first-half and second-half elements
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        a[2 * e] = bf16_lo(r[e]); a[2 * e + 1] = bf16_hi(r[e]);
        b[2 * e] = bf16_lo(r[4 + e]); b[2 * e + 1] = bf16_hi(r[4 + e]);
      }
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
      const unsigned gmask = 0xFFu << (sub * 8);        // the four 8-lane groups may hold different kinds of heads
      ss += __shfl_xor_sync(gmask, ss, 1);
      ss += __shfl_xor_sync(gmask, ss, 2);
      ss += __shfl_xor_sync(gmask, ss, 4);
      if (w != nullptr) {
        const float inv = rsqrtf(ss / static_cast<float>(D) + eps);
        const uint4 wl = *reinterpret_cast<const uint4*>(w + 8 * j), wh = *reinterpret_cast<const uint4*>(w + 64 + 8 * j);
        const uint32_t wr[8] = {wl.x, wl.y, wl.z, wl.w, wh.x, wh.y, wh.z, wh.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          a[2 * e] = bf16_round(bf16_round(a[2 * e] * inv) * bf16_lo(wr[e]));
          a[2 * e + 1] = bf16_round(bf16_round(a[2 * e + 1] * inv) * bf16_hi(wr[e]));
          b[2 * e] = bf16_round(bf16_round(b[2 * e] * inv) * bf16_lo(wr[4 + e]));
          b[2 * e + 1] = bf16_round(bf16_round(b[2 * e + 1] * inv) * bf16_hi(wr[4 + e]));
        }
      }
      if (do_rope) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float x1 = a[e], x2 = b[e];
          a[e] = x1 * cosv[e] - x2 * sinv[e];
          b[e] = x2 * cosv[e] + x1 * sinv[e];
        }
      }
      lo = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
      hi = make_uint4(pack_bf16x2(b[0], b[1]), pack_bf16x2(b[2], b[3]), pack_bf16x2(b[4], b[5]), pack_bf16x2(b[6], b[7]));
    }
    if (!live) continue;
    __nv_bfloat16* dst;
    if (is_q) {
      dst = q_out + (static_cast<size_t>(t) * nq + h) * D;
    } else {
      if (!slot_ok) continue;
      const int kvh = is_k ? h - nq : h - nq - nkv;
      const long long blk = slot / block_size, off = slot % block_size;
      dst = (is_k ? k_cache : v_cache) + ((blk * nkv + kvh) * block_size + off) * D;
    }
    *reinterpret_cast<uint4*>(dst + 8 * j) = lo;
    *reinterpret_cast<uint4*>(dst + 64 + 8 * j) = hi;
  }
}

extern "C" int forge_qk_norm_rope_store(const void* qkv, int ld_qkv, const void* qw, const void* kw, float eps,
                                        const float* rope, int rope_rows, const int* positions, const int* slots,
                                        void* q_out, void* k_cache, void* v_cache, int T, int nq, int nkv, int D,
                                        int block_size, long long num_slots, int do_rope, unsigned* status,
                                        cudaStream_t stream) {
  if (T <= 0) return 0;
  const int heads = nq + 2 * nkv;
  if (D == 128 && (ld_qkv & 7) == 0 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0) {
    // four heads per warp at a time; more heads per warp when there are many tokens (amortises the per-token loads)
    const int hpw128 = T >= 4096 ? 16 : (T >= 512 ? 8 : 4);
    const long long warps128 = static_cast<long long>(T) * ((heads + hpw128 - 1) / hpw128);
    return launch_kernel(qk_norm_rope_store128_kernel, dim3(static_cast<unsigned>((warps128 + 3) / 4)), dim3(128), 0, stream, 0,
                         static_cast<const __nv_bfloat16*>(qkv), ld_qkv, static_cast<const __nv_bfloat16*>(qw),
                         static_cast<const __nv_bfloat16*>(kw), eps, rope, rope_rows, positions, slots,
                         static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
                         static_cast<__nv_bfloat16*>(v_cache), T, nq, nkv, block_size, num_slots, do_rope, hpw128, status) == cudaSuccess ? 0 : -2;
  }
  const int hpw = T >= 4096 ? 8 : (T >= 1024 ? 4 : 1);        // heads per warp: amortise the per-token loads when there is enough work
  const long long warps = static_cast<long long>(T) * ((heads + hpw - 1) / hpw);
  const int grid = static_cast<int>((warps + 3) / 4);
  cudaError_t e;
#define FORGE_QK(DD)                                                                                                      \
  e = launch_kernel(qk_norm_rope_store_kernel<DD>, dim3(grid), dim3(128), 0, stream, 0,                                   \
                    static_cast<const __nv_bfloat16*>(qkv), ld_qkv, static_cast<const __nv_bfloat16*>(qw),               \
                    static_cast<const __nv_bfloat16*>(kw), eps, rope, rope_rows, positions, slots,                       \
                    static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),                            \
                    static_cast<__nv_bfloat16*>(v_cache), T, nq, nkv, block_size, num_slots, do_rope, hpw, status)
  if (D == 128) FORGE_QK(128);
  else if (D == 64) FORGE_QK(64);
  else if (D == 256) FORGE_QK(256);
  else return -1;
#undef FORGE_QK
  return e == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------------
// out[t, :I] = silu(x[t, :I]) * x[t, I:2I]
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                       long long rows, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const int nvec = I >> 3;
  const long long total = rows * nvec;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / nvec;
    const int v = static_cast<int>(idx % nvec);
    const uint4 g = reinterpret_cast<const uint4*>(x + r * 2 * I)[v];
    const uint4 u = reinterpret_cast<const uint4*>(x + r * 2 * I + I)[v];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack_bf16x2(silu(bf16_lo(gw[j])) * bf16_lo(uw[j]), silu(bf16_hi(gw[j])) * bf16_hi(uw[j]));
    reinterpret_cast<uint4*>(out + r * I)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

extern "C" int forge_silu_mul(const void* x, void* out, long long rows, int I, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (I & 7) return -1;
  const long long total = rows * (I >> 3);
  int grid = static_cast<int>((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  return launch_kernel(silu_mul_kernel, dim3(grid), dim3(256), 0, stream, 0, static_cast<const __nv_bfloat16*>(x),
                       static_cast<__nv_bfloat16*>(out), rows, I) == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------------
// Row gathers.  embedding: out[t] = id in [start, start + n) ? W[id - start] : 0.  gather_rows: out[s] = x[idx[s]].
// ---------------------------------------------------------------------------------------------------------
// ssq (optional): fp32 [T][parts].  ssq[t][0] = sum of squares of the row written, ssq[t][1..] = 0, so that the first linear
// layer can apply the first RMSNorm as a row scale (it sums the parts; see GemmFuse in gemm_bf16_sm100.cu).
__global__ void __launch_bounds__(128) embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                                        __nv_bfloat16* __restrict__ out, int H, int vocab_start, int vocab_n,
                                                        float* __restrict__ ssq, int parts) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int local = ids[t] - vocab_start;
  const bool ok = local >= 0 && local < vocab_n;
  const uint4* src = reinterpret_cast<const uint4*>(w + static_cast<size_t>(ok ? local : 0) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
  float ss = 0.f;
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    const uint4 v = ok ? src[i] : make_uint4(0, 0, 0, 0);
    dst[i] = v;
    const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += bf16_lo(vw[j]) * bf16_lo(vw[j]) + bf16_hi(vw[j]) * bf16_hi(vw[j]);
  }
  if (ssq != nullptr) {
    ss = block_sum(ss, red);
    for (int s = threadIdx.x; s < parts; s += blockDim.x) ssq[static_cast<size_t>(t) * parts + s] = s == 0 ? ss : 0.f;
  }
}

extern "C" int forge_embedding(const int* ids, const void* w, void* out, int T, int H, int vocab_start, int vocab_n, float* ssq,
                               int parts, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return -1;
  return launch_kernel(embedding_kernel, dim3(T), dim3(128), 0, stream, 0, ids, static_cast<const __nv_bfloat16*>(w),
                       static_cast<__nv_bfloat16*>(out), H, vocab_start, vocab_n, ssq, parts) == cudaSuccess ? 0 : -2;
}

__global__ void __launch_bounds__(128) gather_rows_kernel(const int* __restrict__ idx, const __nv_bfloat16* __restrict__ x,
                                                          __nv_bfloat16* __restrict__ out, int H, int x_rows) {
  pdl_launch_dependents();
  pdl_wait();
  int r = idx[blockIdx.x];
  r = r < 0 ? 0 : (r >= x_rows ? x_rows - 1 : r);
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(blockIdx.x) * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = src[i];
}

extern "C" int forge_gather_rows(const int* idx, const void* x, void* out, int S, int H, int x_rows, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (H & 7) return -1;
  return launch_kernel(gather_rows_kernel, dim3(S), dim3(128), 0, stream, 0, idx, static_cast<const __nv_bfloat16*>(x),
                       static_cast<__nv_bfloat16*>(out), H, x_rows) == cudaSuccess ? 0 : -2;
}

// ids[i] = prev_tokens[src_rows[i]] where src_rows[i] >= 0: the input token of a sequence is the token the previous
// step sampled for it, taken on the device so that the host can run one step ahead of the results it reads back.
__global__ void __launch_bounds__(128) feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ src_rows,
                                                          const int* __restrict__ prev_tokens, int n, int prev_n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int s = src_rows[i];
  if (s >= 0 && s < prev_n) ids[i] = prev_tokens[s];
}

extern "C" int forge_feed_tokens(int* ids, const int* src_rows, const int* prev_tokens, int n, int prev_n, cudaStream_t stream) {
  if (n <= 0) return 0;
  return launch_kernel(feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, 0, ids, src_rows, prev_tokens, n, prev_n) ==
                 cudaSuccess ? 0 : -2;
}

}  // namespace forge

// Block-scaled fp8 (e4m3) weight GEMM:  out[M, N] = (Xq * sx)[M, K] * (Wq * sw)[N, K]^T  in bf16, where
//   Wq  e4m3 weights with one fp32 scale per 128 x 128 block          sw[N / 128][K / 128]
//   Xq  e4m3 activations with one fp32 scale per token per 128 of K   sx[K / 128][M]   (K-block major)
// The reference has no quantised path (bf16 only); this is the quantised-weight capability of the engine
// (`quantization="fp8_block"`), which halves the weight bytes a decode step must stream.
//
// tcgen05.mma kind::f8f6f4 multiplies e4m3 x e4m3 into fp32 tensor memory.  Scales differ per 128-wide K block,
// so products cannot simply accumulate in tensor memory across K: each K block is multiplied into one of TWO
// tensor-memory buffers (four UMMAs of K = 32), and while the tensor core works on the next block the epilogue
// warps read the finished buffer, multiply by sw[tile][kb] * sx[kb][token] and accumulate in registers.
//
// Orientation as in the bf16 decode kernel: the 128-row UMMA side is a tile of 128 weight rows (= exactly one
// row of scale blocks), tokens ride the N side in tiles of BLOCK_C.  Grid (N / 128, token tiles, K splits).
// With few tokens a layer has too few tiles to fill the GPU (and each CTA would stream a very long K): K is then
// split over grid.z, every split writes its fp32 partial tile to a workspace and a small second kernel adds the
// partials in split order (deterministic) and stores bf16.
// Warp roles: warp 0 TMA producer, warp 1 UMMA issuer + TMEM owner, warps 2..5 scale-accumulate + store.
#include <cuda_fp8.h>

#include "../include/launch.cuh"
#include "../include/ptx.cuh"

namespace forge {

constexpr int kF8BlockR = 128;
constexpr int kF8BlockK = 128;   // 128 e4m3 = one 128-byte swizzle row = one scale block
constexpr int kF8UmmaK = 32;
constexpr int kF8Threads = 192;

template <int BLOCK_C>
struct F8Cfg {
  static constexpr int kRBytes = kF8BlockR * kF8BlockK;
  static constexpr int kCBytes = BLOCK_C * kF8BlockK;
  static constexpr int kStageBytes = kRBytes + kCBytes;
  static constexpr int kStagesRaw = (192 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kTmemCols = 2 * BLOCK_C < 32 ? 32 : (2 * BLOCK_C <= 64 ? 64 : (2 * BLOCK_C <= 128 ? 128 : 256));
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 512 + 2 * 128 * 4;
};

template <int BLOCK_C>
__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                      const float* __restrict__ w_scale, const float* __restrict__ x_scale, __nv_bfloat16* __restrict__ out,
                      int ldo, int n_total, int m_total, int K, int x_scale_ld, int kb_per_split, float* __restrict__ partial,
                      unsigned* status) {
  using Cfg = F8Cfg<BLOCK_C>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* acc_full = empty_bar + Cfg::kStages;     // [2]
  uint64_t* acc_empty = acc_full + 2;                // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  float* s_xs = reinterpret_cast<float*>(tmem_slot + 4);   // [2][128] activation scales of the current K block

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = blockIdx.x * kF8BlockR;
  const int tok0 = blockIdx.y * BLOCK_C;
  const int kb0 = min(static_cast<int>(blockIdx.z) * kb_per_split, K / kF8BlockK);     // this split's K blocks: [kb0, kb0 + num_kb)
  const int num_kb = min(kb0 + kb_per_split, K / kF8BlockK) - kb0;

  pdl_launch_dependents();
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_w);
    prefetch_tensormap(&tm_x);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);     // one arrival per epilogue warp
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % Cfg::kStages;
        const uint32_t ph = (kb / Cfg::kStages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, status)) break;
        uint8_t* st = smem + s * Cfg::kStageBytes;
        mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
        tma_load_2d(st, &tm_w, &full_bar[s], (kb0 + kb) * kF8BlockK, r0);
        tma_load_2d(st + Cfg::kRBytes, &tm_x, &full_bar[s], (kb0 + kb) * kF8BlockK, tok0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kF8BlockR, BLOCK_C, 0, 0);     // e4m3 x e4m3 -> fp32
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % Cfg::kStages;
        const int buf = kb & 1;
        if (!mbar_wait(&acc_empty[buf], ((kb >> 1) & 1) ^ 1, status)) break;   // epilogue has drained this buffer
        if (!mbar_wait(&full_bar[s], (kb / Cfg::kStages) & 1, status)) break;
        tcgen05_fence_after();
        const uint32_t st = smem_u32(smem + s * Cfg::kStageBytes);
#pragma unroll
        for (int k = 0; k < kF8BlockK / kF8UmmaK; ++k) {
          const uint32_t koff = k * kF8UmmaK;     // bytes along the 128-byte row
          umma_f8(tmem_base + buf * BLOCK_C, umma_desc_k_sw128(st + koff), umma_desc_k_sw128(st + Cfg::kRBytes + koff), idesc,
                  k != 0);
        }
        umma_commit(&empty_bar[s]);
        umma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int et = quad * 32 + lane;
    const int r = r0 + et;
    const int scale_cols = K / kF8BlockK;
    float acc[BLOCK_C];
#pragma unroll
    for (int c = 0; c < BLOCK_C; ++c) acc[c] = 0.f;
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int buf = kb & 1;
      // activation scales of this K block -> shared memory (one value per token of the tile)
      if (et < BLOCK_C) s_xs[buf * 128 + et] = (tok0 + et < m_total) ? x_scale[static_cast<size_t>(kb0 + kb) * x_scale_ld + tok0 + et] : 0.f;
      const float ws = w_scale[static_cast<size_t>(blockIdx.x) * scale_cols + kb0 + kb];
      named_barrier_sync(1, 128);
      ok = mbar_wait(&acc_full[buf], (kb >> 1) & 1, status);
      tcgen05_fence_after();
      if (ok) {
        constexpr int kChunk = BLOCK_C >= 32 ? 32 : 16;
#pragma unroll
        for (int cc = 0; cc < BLOCK_C; cc += kChunk) {
          uint32_t v[kChunk];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BLOCK_C + cc;
          if constexpr (kChunk == 32) tmem_ld_x32(taddr, v); else tmem_ld_x16(taddr, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < kChunk; ++j) acc[cc + j] = fmaf(__uint_as_float(v[j]), ws * s_xs[buf * 128 + cc + j], acc[cc + j]);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (r < n_total) {
      if (partial != nullptr) {                          // K split: fp32 partial [split][token][feature]
        float* dst = partial + static_cast<size_t>(blockIdx.z) * m_total * n_total + r;
#pragma unroll
        for (int c = 0; c < BLOCK_C; ++c)
          if (tok0 + c < m_total) dst[static_cast<size_t>(tok0 + c) * n_total] = acc[c];
      } else {
#pragma unroll
        for (int c = 0; c < BLOCK_C; ++c)
          if (tok0 + c < m_total) out[static_cast<size_t>(tok0 + c) * ldo + r] = __float2bfloat16_rn(acc[c]);   // lanes -> consecutive features
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// out[m][n] = sum over splits of partial[s][m][n], added in split order; four features per thread.
__global__ void __launch_bounds__(256) fp8_splitk_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                                                int splits, int M, int N, int ldo) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int nvec = N >> 2;
  if (idx >= static_cast<long long>(M) * nvec) return;
  const int m = static_cast<int>(idx / nvec), n = static_cast<int>(idx % nvec) * 4;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const float4 t = *reinterpret_cast<const float4*>(partial + (static_cast<size_t>(s) * M + m) * N + n);
    a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
  }
  __nv_bfloat16* dst = out + static_cast<size_t>(m) * ldo + n;
  dst[0] = __float2bfloat16_rn(a.x); dst[1] = __float2bfloat16_rn(a.y); dst[2] = __float2bfloat16_rn(a.z); dst[3] = __float2bfloat16_rn(a.w);
}

// ---------------------------------------------------------------------------------------------------------
// Activation quantiser: one warp per (token, 128-wide K block); scale = amax / 448.
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) quant_fp8_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ xq,
                                                              float* __restrict__ scale, int M, int K, int scale_ld) {
  pdl_launch_dependents();
  pdl_wait();
  const int kbs = K >> 7;
  const long long wid = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (wid >= static_cast<long long>(M) * kbs) return;
  const int lane = threadIdx.x & 31;
  const int m = static_cast<int>(wid / kbs), kb = static_cast<int>(wid % kbs);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(m) * K + kb * 128 + lane * 4);
  const float f[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
  float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / s;
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[0] * inv, f[1] * inv), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[2] * inv, f[3] * inv), __NV_SATFINITE, __NV_E4M3);
  *reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(m) * K + kb * 128 + lane * 4) = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
  if (lane == 0) scale[static_cast<size_t>(kb) * scale_ld + m] = s;
}

extern "C" int forge_make_tmap_2d(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                                  uint32_t box_rows, int elem_bytes);

extern "C" int forge_quant_fp8_1x128(const void* x, void* xq, float* scale, int M, int K, int scale_ld, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (K & 127) return -1;
  const long long warps = static_cast<long long>(M) * (K >> 7);
  return launch_kernel(quant_fp8_1x128_kernel, dim3(static_cast<unsigned>((warps + 3) / 4)), dim3(128), 0, stream, 0,
                       static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(xq), scale, M, K, scale_ld) == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------------
// Weight dequantiser: e4m3 [N, K] with 128 x 128 block scales -> bf16 [N, K].  With many tokens (prefill) the GEMM is
// bound by the tensor cores, not by the weight bytes: the layer's weights are expanded once per call into a scratch
// buffer (3 bytes of traffic per weight, a few per cent of the GEMM's time from ~1000 tokens) and the bf16 CTA-pair
// kernel does the multiplication with the activations left in bf16.  16 weights per thread.
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) dequant_fp8_block_kernel(const uint8_t* __restrict__ wq, const float* __restrict__ scale,
                                                                __nv_bfloat16* __restrict__ out, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = K >> 4;
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= static_cast<long long>(N) * per_row) return;
  const int n = static_cast<int>(i / per_row), k0 = static_cast<int>(i % per_row) << 4;
  const float s = scale[static_cast<size_t>(n >> 7) * (K >> 7) + (k0 >> 7)];
  const uint4 raw = *reinterpret_cast<const uint4*>(wq + static_cast<size_t>(n) * K + k0);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((w[j] >> (16 * h)) & 0xffffu), __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      o[2 * j + h] = pack_bf16x2(f.x * s, f.y * s);
    }
  }
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(n) * K + k0);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

extern "C" int forge_dequant_fp8_block(const void* wq, const float* scale, void* out, int N, int K, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (K & 127) return -1;
  const long long threads = static_cast<long long>(N) * (K >> 4);
  return launch_kernel(dequant_fp8_block_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0, stream, 0,
                       static_cast<const uint8_t*>(wq), scale, static_cast<__nv_bfloat16*>(out), N, K) == cudaSuccess ? 0 : -2;
}

template <int BLOCK_C>
static int launch_f8(const void* xq, const float* xs, int xs_ld, const void* wq, const float* ws, void* out, int ldo, int M, int N,
                     int K, int splits, float* partial, unsigned* status, cudaStream_t stream) {
  using Cfg = F8Cfg<BLOCK_C>;
  CUtensorMap tm_w, tm_x;
  if (forge_make_tmap_2d(&tm_w, wq, N, K, K, kF8BlockR, 1) != 0) return -2;
  if (forge_make_tmap_2d(&tm_x, xq, M, K, K, BLOCK_C, 1) != 0) return -3;
  auto kern = gemm_fp8_block_kernel<BLOCK_C>;
  FORGE_ENSURE_DYN_SMEM(kern, Cfg::kSmemBytes);
  const int num_kb = K / kF8BlockK;
  const int kb_per_split = (num_kb + splits - 1) / splits;
  dim3 grid((N + kF8BlockR - 1) / kF8BlockR, (M + BLOCK_C - 1) / BLOCK_C, splits);
  if (launch_kernel(kern, grid, dim3(kF8Threads), Cfg::kSmemBytes, stream, 0, tm_w, tm_x, ws, xs, static_cast<__nv_bfloat16*>(out),
                    ldo, N, M, K, xs_ld, kb_per_split, splits > 1 ? partial : nullptr, status) != cudaSuccess)
    return -5;
  if (splits > 1) {
    const long long vecs = static_cast<long long>(M) * (N >> 2);
    if (launch_kernel(fp8_splitk_reduce_kernel, dim3(static_cast<unsigned>((vecs + 255) / 256)), dim3(256), 0, stream, 0,
                      static_cast<const float*>(partial), static_cast<__nv_bfloat16*>(out), splits, M, N, ldo) != cudaSuccess)
      return -5;
  }
  return 0;
}

static int f8_token_tile(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

// K splits the kernel will use for this problem: enough CTAs for about one wave of the 148 SMs (one CTA per SM:
// the ring takes the whole shared memory), at least two K blocks per split, N a multiple of 4 for the reduce kernel.
extern "C" int forge_gemm_fp8_splits(int M, int N, int K) {
  if (M <= 0 || N <= 0 || (N & 3)) return 1;
  const int bc = f8_token_tile(M);
  const int ctas = ((N + kF8BlockR - 1) / kF8BlockR) * ((M + bc - 1) / bc);
  const int num_kb = K / kF8BlockK;
  int s = 1;
  while (s < 8 && ctas * s * 2 <= 160 && num_kb / (s * 2) >= 2) s *= 2;
  return s;
}

// xq [M, K] e4m3, xs [K / 128][xs_ld >= M]; wq [N, K] e4m3, ws [ceil(N / 128)][K / 128]; out [M, N] bf16 (row stride ldo).
// partial: fp32 workspace of forge_gemm_fp8_splits(M, N, K) * M * N floats (may be null when that is 1).
extern "C" int forge_gemm_fp8_block(const void* xq, const float* xs, int xs_ld, const void* wq, const float* ws, void* out, int ldo,
                                    int M, int N, int K, float* partial, unsigned* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K & 127) || (reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15)) return -1;
  const int splits = partial != nullptr ? forge_gemm_fp8_splits(M, N, K) : 1;
  if (M <= 16) return launch_f8<16>(xq, xs, xs_ld, wq, ws, out, ldo, M, N, K, splits, partial, status, stream);
  if (M <= 32) return launch_f8<32>(xq, xs, xs_ld, wq, ws, out, ldo, M, N, K, splits, partial, status, stream);
  return launch_f8<64>(xq, xs, xs_ld, wq, ws, out, ldo, M, N, K, splits, partial, status, stream);
}

}  // namespace forge

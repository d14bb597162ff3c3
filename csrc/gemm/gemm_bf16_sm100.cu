// bf16 GEMM  out[M, N] = X[M, K] * W[N, K]^T  on the 5th-generation tensor cores (tcgen05), fp32
// accumulation in tensor memory, operands staged by TMA with the 128-byte swizzle.
//
// The reference calls F.linear, i.e. cuBLAS (tinyvllm/layers/linear.py:83,181).  Two kernels here cover the
// four linear layers of a decoder block and the LM head:
//
//   gemm_tokens_kernel  (prefill, many tokens): the UMMA's 128-row side is a tile of 128 tokens, the N side a
//       tile of BLOCK_C output features.  One output tile per CTA.
//
//   gemm_weights_kernel (decode, <= 256 tokens): operands swapped.  The 128-row side is a tile of 128 weight
//       rows, so the weight stream fills the tensor core and no rows are wasted on token padding; ALL tokens
//       ride the N side (BLOCK_C = 16..256).  Such a GEMM has few output tiles (N / 128), so K is split over a
//       thread-block cluster of 1..8 CTAs: each CTA accumulates its K slice in tensor memory, dumps the fp32
//       partial tile into its shared memory, and after a cluster barrier every CTA reduces its share of the
//       columns by reading all peers' shared memory (DSMEM) in a fixed order (deterministic) and stores bf16
//       rows with coalesced 8-byte writes.  No global scratch, no atomics.
//
// Epilogues: plain store, or SiLU(gate) * up with two accumulators per CTA (gate rows and up rows of the
// packed [2I, H] weight), which removes the [tokens, 2I] intermediate of tinyvllm/layers/activation.py:11-14.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + UMMA issuer, warps 2..5 = epilogue
// (TMEM lane quadrant = warp % 4).  All mbarrier waits are bounded (see ptx.cuh).
#include "../include/ptx.cuh"

namespace forge {

constexpr int kBlockR = 128;
constexpr int kBlockK = 64;    // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;

enum GemmEpilogue { kEpiStore = 0, kEpiSiluMul = 1 };

constexpr int tmem_cols_for(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

// =========================================================================================================
// prefill: R = X tile (128 tokens), C = W tile (BLOCK_C features; two tiles for SiLU)
// =========================================================================================================
template <int BLOCK_C, int kEpi>
struct TokCfg {
  static constexpr int kNumC = kEpi == kEpiSiluMul ? 2 : 1;
  static constexpr int kRBytes = kBlockR * kBlockK * 2;
  static constexpr int kCBytes = BLOCK_C * kBlockK * 2;
  static constexpr int kStageBytes = kRBytes + kNumC * kCBytes;
  static constexpr int kStagesRaw = (200 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kTmemCols = tmem_cols_for(BLOCK_C * kNumC);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static_assert(BLOCK_C % 16 == 0 && BLOCK_C >= 16 && BLOCK_C <= 256, "UMMA N for M = 128");
};

template <int BLOCK_C, int kEpi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tokens_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                   __nv_bfloat16* __restrict__ out, int ldo, int m_total, int n_total, int K, int dual_off, unsigned* status) {
  using Cfg = TokCfg<BLOCK_C, kEpi>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* acc_bar = empty_bar + Cfg::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // consecutive CTAs share the weight tile (blockIdx.x walks the token tiles), so it stays in L2
  const int r0 = blockIdx.x * kBlockR;
  const int c0 = blockIdx.y * BLOCK_C;
  const int num_kb = (K + kBlockK - 1) / kBlockK;

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
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

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % Cfg::kStages;
        const uint32_t ph = (kb / Cfg::kStages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, status)) break;
        uint8_t* st = smem + s * Cfg::kStageBytes;
        mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
        tma_load_2d(st, &tm_x, &full_bar[s], kb * kBlockK, r0);
        for (int i = 0; i < Cfg::kNumC; ++i)
          tma_load_2d(st + Cfg::kRBytes + i * Cfg::kCBytes, &tm_w, &full_bar[s], kb * kBlockK, c0 + i * dual_off);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kBlockR, BLOCK_C, 1, 1);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % Cfg::kStages;
        const uint32_t ph = (kb / Cfg::kStages) & 1;
        if (!mbar_wait(&full_bar[s], ph, status)) break;
        tcgen05_fence_after();
        const uint32_t st = smem_u32(smem + s * Cfg::kStageBytes);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          const uint32_t koff = k * kUmmaK * 2;
          const uint32_t acc = (kb | k) != 0;
          const uint64_t dx = umma_desc_k_sw128(st + koff);
          umma_f16(tmem_base, dx, umma_desc_k_sw128(st + Cfg::kRBytes + koff), idesc, acc);
          if constexpr (kEpi == kEpiSiluMul)
            umma_f16(tmem_base + BLOCK_C, dx, umma_desc_k_sw128(st + Cfg::kRBytes + Cfg::kCBytes + koff), idesc, acc);
        }
        umma_commit(&empty_bar[s]);
      }
      umma_commit(acc_bar);
    }
  } else {
    const int quad = warp & 3;
    const int r = r0 + quad * 32 + lane;
    const bool ok = mbar_wait(acc_bar, 0, status);
    tcgen05_fence_after();
    if (ok) {
      constexpr int kChunk = BLOCK_C >= 32 ? 32 : 16;
#pragma unroll 1
      for (int cc = 0; cc < BLOCK_C; cc += kChunk) {
        uint32_t v[kChunk];
        uint32_t u[kEpi == kEpiSiluMul ? kChunk : 1];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + cc;
        if constexpr (kChunk == 32) tmem_ld_x32(taddr, v); else tmem_ld_x16(taddr, v);
        if constexpr (kEpi == kEpiSiluMul) {
          if constexpr (kChunk == 32) tmem_ld_x32(taddr + BLOCK_C, u); else tmem_ld_x16(taddr + BLOCK_C, u);
        }
        tmem_ld_wait();
        float f[kChunk];
#pragma unroll
        for (int j = 0; j < kChunk; ++j) {
          f[j] = __uint_as_float(v[j]);
          if constexpr (kEpi == kEpiSiluMul) f[j] = silu(f[j]) * __uint_as_float(u[j]);
        }
        const int c = c0 + cc;
        if (r < m_total) {
          __nv_bfloat16* dst = out + static_cast<size_t>(r) * ldo + c;
          if (c + kChunk <= n_total && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < kChunk; j += 8) {
              uint4 pk;
              pk.x = pack_bf16x2(f[j], f[j + 1]);
              pk.y = pack_bf16x2(f[j + 2], f[j + 3]);
              pk.z = pack_bf16x2(f[j + 4], f[j + 5]);
              pk.w = pack_bf16x2(f[j + 6], f[j + 7]);
              *reinterpret_cast<uint4*>(dst + j) = pk;
            }
          } else {
#pragma unroll
            for (int j = 0; j < kChunk; ++j)
              if (c + j < n_total) dst[j] = __float2bfloat16_rn(f[j]);
          }
        }
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

// =========================================================================================================
// decode: R = W tile (128 features; two tiles for SiLU), C = X (all tokens), split-K over a cluster
// =========================================================================================================
template <int BLOCK_C, int kEpi>
struct WgtCfg {
  static constexpr int kNumR = kEpi == kEpiSiluMul ? 2 : 1;
  static constexpr int kRBytes = kBlockR * kBlockK * 2;
  static constexpr int kCBytes = BLOCK_C * kBlockK * 2;
  static constexpr int kStageBytes = kNumR * kRBytes + kCBytes;
  static constexpr int kStagesRaw = (192 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kPartialBytes = BLOCK_C * kBlockR * 4;     // fp32 [BLOCK_C][128], reuses the stage ring
  static constexpr int kRingBytes = kStages * kStageBytes > kPartialBytes ? kStages * kStageBytes : kPartialBytes;
  static constexpr int kTmemCols = tmem_cols_for(BLOCK_C * kNumR);
  static constexpr int kSmemBytes = kRingBytes + 1024 + 256;
  static_assert(BLOCK_C % 16 == 0 && BLOCK_C >= 16 && BLOCK_C <= 256, "UMMA N for M = 128");
  static_assert(kStages >= 2, "need at least a double buffer");
  static_assert(kEpi != kEpiSiluMul || kRingBytes >= kPartialBytes + kPartialBytes / 2, "no room for the reduced gate tile");
};

// out[token, feature] (row stride ldo).  W: [n_total (or 2 * n_total) rows, K]; X: [m_total rows, K].
// Cluster = (1, S, 1): blockIdx.x = feature tile, cluster rank = K split.
template <int BLOCK_C, int kEpi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_weights_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    __nv_bfloat16* __restrict__ out, int ldo, int n_total, int m_total, int K, int kb_per_split,
                    int dual_off, unsigned* status) {
  using Cfg = WgtCfg<BLOCK_C, kEpi>;
  extern __shared__ uint8_t smem_raw[];
  // The dynamic shared window starts at the same offset in every CTA of the cluster, so equal local
  // addresses name corresponding buffers in all peers.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kRingBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* acc_bar = empty_bar + Cfg::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  float* partial = reinterpret_cast<float*>(smem);          // [BLOCK_C][128] after the main loop

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t split = cluster_ctarank(), nsplit = cluster_nctarank();
  const int r0 = blockIdx.x * kBlockR;
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  const int kb0 = min(static_cast<int>(split) * kb_per_split, num_kb);
  const int my_kb = min(kb0 + kb_per_split, num_kb) - kb0;   // may be 0 for a trailing split

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_w);
    prefetch_tensormap(&tm_x);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
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

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < my_kb; ++i) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (i / Cfg::kStages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, status)) break;
        uint8_t* st = smem + s * Cfg::kStageBytes;
        const int kx = (kb0 + i) * kBlockK;
        mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
        for (int j = 0; j < Cfg::kNumR; ++j) tma_load_2d(st + j * Cfg::kRBytes, &tm_w, &full_bar[s], kx, r0 + j * dual_off);
        tma_load_2d(st + Cfg::kNumR * Cfg::kRBytes, &tm_x, &full_bar[s], kx, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kBlockR, BLOCK_C, 1, 1);
      for (int i = 0; i < my_kb; ++i) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (i / Cfg::kStages) & 1;
        if (!mbar_wait(&full_bar[s], ph, status)) break;
        tcgen05_fence_after();
        const uint32_t st = smem_u32(smem + s * Cfg::kStageBytes);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          const uint32_t koff = k * kUmmaK * 2;
          const uint32_t acc = (i | k) != 0;
          const uint64_t dx = umma_desc_k_sw128(st + Cfg::kNumR * Cfg::kRBytes + koff);
          umma_f16(tmem_base, umma_desc_k_sw128(st + koff), dx, idesc, acc);
          if constexpr (kEpi == kEpiSiluMul)
            umma_f16(tmem_base + BLOCK_C, umma_desc_k_sw128(st + Cfg::kRBytes + koff), dx, idesc, acc);
        }
        umma_commit(&empty_bar[s]);
      }
      if (my_kb > 0) umma_commit(acc_bar); else mbar_arrive(acc_bar);
    }
  }

  // ---------------------------------------------------------------- epilogue (all threads take part in the barriers)
  const bool is_epi = warp >= 2;
  const int quad = warp & 3;
  const int et = is_epi ? (quad * 32 + lane) : 0;              // epilogue thread id == TMEM lane == tile row
  bool acc_ok = true;
  if (is_epi) {
    acc_ok = mbar_wait(acc_bar, 0, status);                    // the ring is idle from here on: every load was consumed
    tcgen05_fence_after();
  }
  // SiLU with a single split needs no cross-CTA sum: combine gate and up while leaving tensor memory.
  // With several splits the gate sums must be complete before the nonlinearity: pass 0 reduces the gate
  // tile into this CTA's gate_red buffer (after the partial tile; fits because a split CTA owns at most
  // BLOCK_C / 2 columns), pass 1 reduces the up tile and combines.
  const bool fuse = kEpi == kEpiSiluMul && nsplit == 1;
  const int passes = (kEpi == kEpiSiluMul && !fuse) ? 2 : 1;
  const int cols_per_cta = BLOCK_C / static_cast<int>(nsplit);
  float* gate_red = reinterpret_cast<float*>(smem + Cfg::kPartialBytes);   // [cols_per_cta][128]
  __syncwarp();
  for (int pass = 0; pass < passes; ++pass) {
    if (is_epi) {
      // TMEM -> own shared memory, layout [col][row]: lanes write consecutive floats (no bank conflicts)
      constexpr int kChunk = BLOCK_C >= 32 ? 32 : 16;
#pragma unroll 1
      for (int cc = 0; cc < BLOCK_C; cc += kChunk) {
        uint32_t v[kChunk];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + pass * BLOCK_C + cc;
        if (my_kb > 0 && acc_ok) {
          if constexpr (kChunk == 32) tmem_ld_x32(taddr, v); else tmem_ld_x16(taddr, v);
          if constexpr (kEpi == kEpiSiluMul) {
            if (fuse) {
              uint32_t u[kChunk];
              if constexpr (kChunk == 32) tmem_ld_x32(taddr + BLOCK_C, u); else tmem_ld_x16(taddr + BLOCK_C, u);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < kChunk; ++j) v[j] = __float_as_uint(silu(__uint_as_float(v[j])) * __uint_as_float(u[j]));
            }
          }
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < kChunk; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < kChunk; ++j) partial[(cc + j) * kBlockR + et] = __uint_as_float(v[j]);
      }
    }
    __syncwarp();
    cluster_sync();                                            // every CTA's partial tile is visible
    if (is_epi) {
      // this CTA reduces columns [split * cols_per_cta, +cols_per_cta); a warp handles one column at a time,
      // lane l owns rows 4l..4l+3 (16-byte DSMEM reads, 8-byte global stores)
      const uint32_t my_base = smem_u32(partial);
      const int c_first = static_cast<int>(split) * cols_per_cta;
      for (int c = c_first + quad; c < c_first + cols_per_cta; c += 4) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t p = 0; p < nsplit; ++p) {
          const float4 v = ld_dsmem_f4(dsmem_addr(my_base + (c * kBlockR + lane * 4) * 4, p));
          a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        if constexpr (kEpi == kEpiSiluMul) {
          if (!fuse) {
            float4* g = reinterpret_cast<float4*>(gate_red + (c - c_first) * kBlockR + lane * 4);   // same thread both passes
            if (pass == 0) {
              *g = a;
              continue;
            }
            const float4 gv = *g;
            a.x = silu(gv.x) * a.x; a.y = silu(gv.y) * a.y; a.z = silu(gv.z) * a.z; a.w = silu(gv.w) * a.w;
          }
        }
        const int n = r0 + lane * 4;
        if (c < m_total && n < n_total) {
          __nv_bfloat16* dst = out + static_cast<size_t>(c) * ldo + n;
          if (n + 4 <= n_total && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
            uint2 pk;
            pk.x = pack_bf16x2(a.x, a.y);
            pk.y = pack_bf16x2(a.z, a.w);
            *reinterpret_cast<uint2*>(dst) = pk;
          } else {
            const float f[4] = {a.x, a.y, a.z, a.w};
            for (int j = 0; j < 4 && n + j < n_total; ++j) dst[j] = __float2bfloat16_rn(f[j]);
          }
        }
      }
    }
    cluster_sync();                                            // peers are done reading this CTA's partial tile
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D K-major tensor [rows, cols] (cols contiguous, row stride ld elements), box [box_rows, 128 bytes], 128B swizzle.
// elem_bytes: 2 (bf16) or 1 (fp8; the box is then 128 elements wide).
extern "C" int forge_make_tmap_2d(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                                  uint32_t box_rows, int elem_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

template <int BLOCK_C, int kEpi>
static int launch_tokens(const void* x, int ldx, const void* w, int w_rows, int ldw, __nv_bfloat16* out, int ldo, int M,
                         int n_out, int K, unsigned* status, cudaStream_t stream) {
  using Cfg = TokCfg<BLOCK_C, kEpi>;
  CUtensorMap tm_x, tm_w;
  if (forge_make_tmap_2d(&tm_x, x, M, K, ldx, kBlockR, 2) != 0) return -2;
  if (forge_make_tmap_2d(&tm_w, w, w_rows, K, ldw, BLOCK_C, 2) != 0) return -3;
  auto kern = gemm_tokens_kernel<BLOCK_C, kEpi>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return -4;
    attr_set = true;
  }
  dim3 grid((M + kBlockR - 1) / kBlockR, (n_out + BLOCK_C - 1) / BLOCK_C);
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tm_x, tm_w, out, ldo, M, n_out, K, n_out, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Cluster size (K splits) for the decode kernel: double while the grid stays within one wave of 148 SMs and
// every split keeps at least two K blocks.
static int choose_splits(int tiles, int num_kb) {
  int s = 1;
  while (s < 8 && tiles * s * 2 <= 148 && num_kb / (s * 2) >= 2) s *= 2;
  return s;
}

template <int BLOCK_C, int kEpi>
static int launch_weights(const void* x, int ldx, const void* w, int w_rows, int ldw, __nv_bfloat16* out, int ldo, int M,
                          int n_out, int K, int force_splits, unsigned* status, cudaStream_t stream) {
  using Cfg = WgtCfg<BLOCK_C, kEpi>;
  CUtensorMap tm_x, tm_w;
  if (forge_make_tmap_2d(&tm_w, w, w_rows, K, ldw, kBlockR, 2) != 0) return -2;
  if (forge_make_tmap_2d(&tm_x, x, M, K, ldx, BLOCK_C, 2) != 0) return -3;
  auto kern = gemm_weights_kernel<BLOCK_C, kEpi>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return -4;
    attr_set = true;
  }
  const int tiles = (n_out + kBlockR - 1) / kBlockR;
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  int splits = force_splits > 0 ? force_splits : choose_splits(tiles, num_kb);
  if (splits > BLOCK_C / 4) splits = BLOCK_C / 4 < 1 ? 1 : BLOCK_C / 4;   // every CTA reduces >= 4 columns (one per warp)
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return -6;
  const int kb_per_split = (num_kb + splits - 1) / splits;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, splits, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = splits;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tm_w, tm_x, out, ldo, n_out, M, K, kb_per_split, n_out, status);
  return e == cudaSuccess ? 0 : -5;
}

// out[M, n_out] = epilogue(X[M, K] * W[*, K]^T).  epi = 0: W has n_out rows.  epi = 1: W is [2 * n_out, K]
// (gate rows then up rows) and out = silu(gate) * up.  Requirements: K % 8 == 0, x/w 16-byte aligned,
// ldx/ldw % 8 == 0.  force_mode: 0 auto, 1 token-tile kernel, 2 weight-tile (decode) kernel (needs M <= 256).
// force_splits: 0 auto, else the cluster size of the decode kernel.  Returns 0 on success.
extern "C" int forge_gemm_bf16(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int n_out,
                               int K, int epi, int force_mode, int force_splits, unsigned* status, cudaStream_t stream) {
  if (M <= 0 || n_out <= 0 || K <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return -1;
  const int w_rows = epi == kEpiSiluMul ? 2 * n_out : n_out;
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  const bool decode = force_mode == 2 || (force_mode == 0 && M <= 256);
  if (decode) {
    if (M > 256) return -7;
    const int bc = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
#define FORGE_W(BC)                                                                                                          \
  case BC:                                                                                                                   \
    return epi == kEpiSiluMul                                                                                                \
               ? launch_weights<BC, kEpiSiluMul>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, force_splits, status, stream) \
               : launch_weights<BC, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, force_splits, status, stream);
    switch (bc) {
      FORGE_W(16)
      FORGE_W(32)
      FORGE_W(64)
      FORGE_W(128)
      FORGE_W(256)
    }
#undef FORGE_W
    return -6;
  }
  if (epi == kEpiSiluMul) return launch_tokens<128, kEpiSiluMul>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream);
  return launch_tokens<128, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream);
}

}  // namespace forge

// bf16 GEMM  out[M, N] = X[M, K] * W[N, K]^T  on the 5th-generation tensor cores (tcgen05), fp32
// accumulation in tensor memory, operands staged by TMA with the 128-byte swizzle.
//
// One kernel covers the four linear layers of a decoder block (the reference calls F.linear, i.e.
// cuBLAS: tinyvllm/layers/linear.py:83,181) in two operand bindings:
//
//   row operand R  : the 128-row side of the UMMA (M = 128)
//   col operand C  : the N side of the UMMA (BLOCK_C = 16..256 columns)
//
//   normal  (prefill, many tokens):  R = X tile (128 tokens),  C = W tile (BLOCK_C features)
//   swapped (decode, few tokens):    R = W tile (128 features), C = X (all tokens, padded to BLOCK_C)
//           so the weight stream fills the 128-wide side and no tensor-core rows are wasted on padding.
//
// Epilogues: plain store, or SiLU(gate) * up with two accumulators per CTA (gate rows and up rows of the
// packed [2I, H] weight), which removes the [tokens, 2I] intermediate of tinyvllm/layers/activation.py:11-14.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + UMMA issuer, warps 2..5 = epilogue
// (TMEM lane quadrant = warp % 4).  All waits are bounded (see ptx.cuh).
#include "../include/ptx.cuh"

namespace forge {

constexpr int kBlockR = 128;
constexpr int kBlockK = 64;    // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;

enum GemmEpilogue { kEpiStore = 0, kEpiSiluMul = 1 };

template <int BLOCK_C, bool kSwap, int kEpi>
struct GemmCfg {
  static constexpr int kNumR = (kEpi == kEpiSiluMul && kSwap) ? 2 : 1;    // R tiles per stage
  static constexpr int kNumC = (kEpi == kEpiSiluMul && !kSwap) ? 2 : 1;   // C tiles per stage
  static constexpr int kRBytes = kBlockR * kBlockK * 2;
  static constexpr int kCBytes = BLOCK_C * kBlockK * 2;
  static constexpr int kStageBytes = kNumR * kRBytes + kNumC * kCBytes;
  static constexpr int kStagesRaw = (200 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kAccCols = BLOCK_C * (kEpi == kEpiSiluMul ? 2 : 1);
  static constexpr int kTmemCols = kAccCols <= 32 ? 32 : kAccCols <= 64 ? 64 : kAccCols <= 128 ? 128 : kAccCols <= 256 ? 256 : 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(BLOCK_C % 16 == 0 && BLOCK_C >= 16 && BLOCK_C <= 256, "UMMA N for M = 128");
  static_assert(kAccCols <= 512, "accumulators exceed tensor memory");
  static_assert(kStages >= 2, "need at least a double buffer");
};

// out: bf16, row stride ldo.  R has r_total rows, C has c_total rows (both K-major, K contiguous).
// kSwap: out[c, r]; else out[r, c].  SiLU: the second tile sits dual_off rows further in the same tensor.
template <int BLOCK_C, bool kSwap, int kEpi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_r, const __grid_constant__ CUtensorMap tm_c,
                 __nv_bfloat16* __restrict__ out, int ldo, int r_total, int c_total, int K, int dual_off,
                 unsigned* status) {
  using Cfg = GemmCfg<BLOCK_C, kSwap, kEpi>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* acc_bar = empty_bar + Cfg::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int r0 = blockIdx.x * kBlockR;
  const int c0 = blockIdx.y * BLOCK_C;
  const int num_kb = (K + kBlockK - 1) / kBlockK;

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_r);
    prefetch_tensormap(&tm_c);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % Cfg::kStages;
        const uint32_t ph = (kb / Cfg::kStages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, status)) break;
        uint8_t* st = smem + s * Cfg::kStageBytes;
        mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
        for (int i = 0; i < Cfg::kNumR; ++i)
          tma_load_2d(st + i * Cfg::kRBytes, &tm_r, &full_bar[s], kb * kBlockK, r0 + i * dual_off);
        for (int i = 0; i < Cfg::kNumC; ++i)
          tma_load_2d(st + Cfg::kNumR * Cfg::kRBytes + i * Cfg::kCBytes, &tm_c, &full_bar[s], kb * kBlockK,
                      c0 + i * dual_off);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kBlockR, BLOCK_C, 1, 1);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % Cfg::kStages;
        const uint32_t ph = (kb / Cfg::kStages) & 1;
        ok = mbar_wait(&full_bar[s], ph, status);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t st = smem_u32(smem + s * Cfg::kStageBytes);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          const uint32_t koff = k * kUmmaK * 2;   // bytes along the 128-byte row
          const uint32_t acc = (kb | k) != 0;
          const uint64_t dr0 = umma_desc_k_sw128(st + koff);
          const uint64_t dc0 = umma_desc_k_sw128(st + Cfg::kNumR * Cfg::kRBytes + koff);
          umma_f16(tmem_base, dr0, dc0, idesc, acc);
          if constexpr (kEpi == kEpiSiluMul) {
            if constexpr (kSwap) {
              const uint64_t dr1 = umma_desc_k_sw128(st + Cfg::kRBytes + koff);
              umma_f16(tmem_base + BLOCK_C, dr1, dc0, idesc, acc);
            } else {
              const uint64_t dc1 = umma_desc_k_sw128(st + Cfg::kRBytes + Cfg::kCBytes + koff);
              umma_f16(tmem_base + BLOCK_C, dr0, dc1, idesc, acc);
            }
          }
        }
        umma_commit(&empty_bar[s]);     // frees the stage once these UMMAs have read it
      }
      umma_commit(acc_bar);             // accumulators complete
    }
  } else {
    // ------------------------------------------------------------------ epilogue: TMEM -> registers -> global
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
        if constexpr (kSwap) {
          // out[c + j, r]: lanes hold consecutive r, so each store instruction writes 64 contiguous bytes
          if (r < r_total) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j)
              if (c + j < c_total) out[static_cast<size_t>(c + j) * ldo + r] = __float2bfloat16_rn(f[j]);
          }
        } else {
          // out[r, c .. c + kChunk): each thread owns a contiguous run of its row
          if (r < r_total) {
            __nv_bfloat16* dst = out + static_cast<size_t>(r) * ldo + c;
            if (c + kChunk <= c_total && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
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
                if (c + j < c_total) dst[j] = __float2bfloat16_rn(f[j]);
            }
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

// 2-D K-major tensor [rows, cols] (cols contiguous, row stride ld elements), box [box_rows, 64 elems], 128B swizzle.
// elem_bytes: 2 (bf16) or 1 (fp8; box is then 128 elements wide).
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

template <int BLOCK_C, bool kSwap, int kEpi>
static int launch_cfg(const void* r_ptr, int r_rows, int r_ld, const void* c_ptr, int c_rows, int c_ld, int K,
                      __nv_bfloat16* out, int ldo, int r_total, int c_total, int dual_off, unsigned* status,
                      cudaStream_t stream) {
  using Cfg = GemmCfg<BLOCK_C, kSwap, kEpi>;
  CUtensorMap tm_r, tm_c;
  if (forge_make_tmap_2d(&tm_r, r_ptr, r_rows, K, r_ld, kBlockR, 2) != 0) return -2;
  if (forge_make_tmap_2d(&tm_c, c_ptr, c_rows, K, c_ld, BLOCK_C, 2) != 0) return -3;
  auto kern = gemm_bf16_kernel<BLOCK_C, kSwap, kEpi>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return -4;
    attr_set = true;
  }
  dim3 grid((r_total + kBlockR - 1) / kBlockR, (c_total + BLOCK_C - 1) / BLOCK_C);
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tm_r, tm_c, out, ldo, r_total, c_total, K, dual_off, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

template <bool kSwap, int kEpi>
static int launch_by_block(int block_c, const void* r_ptr, int r_rows, int r_ld, const void* c_ptr, int c_rows, int c_ld,
                           int K, __nv_bfloat16* out, int ldo, int r_total, int c_total, int dual_off, unsigned* status,
                           cudaStream_t stream) {
#define FORGE_CASE(BC)                                                                                            \
  case BC:                                                                                                        \
    return launch_cfg<BC, kSwap, kEpi>(r_ptr, r_rows, r_ld, c_ptr, c_rows, c_ld, K, out, ldo, r_total, c_total,   \
                                       dual_off, status, stream);
  switch (block_c) {
    FORGE_CASE(16)
    FORGE_CASE(32)
    FORGE_CASE(64)
    FORGE_CASE(128)
    FORGE_CASE(256)
    default:
      return -6;
  }
#undef FORGE_CASE
}

// out[M, n_out] = epilogue(X[M, K] * W[*, K]^T).  epi = 0: n_out = N rows of W.  epi = 1: W is [2 * n_out, K]
// (gate rows then up rows) and out = silu(gate) * up.  Requirements: K % 8 == 0, x/w 16-byte aligned,
// ldx/ldw % 8 == 0.  Returns 0 on success.
extern "C" int forge_gemm_bf16(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int n_out,
                               int K, int epi, int force_mode, unsigned* status, cudaStream_t stream) {
  if (M <= 0 || n_out <= 0 || K <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return -1;
  const int w_rows = epi == kEpiSiluMul ? 2 * n_out : n_out;
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  // force_mode: 0 auto, 1 normal, 2 swapped
  const bool swap = force_mode == 2 || (force_mode == 0 && M <= 256);
  if (swap) {
    // tokens ride the UMMA N side; more than 256 tokens take several column tiles
    int bc = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    if (epi == kEpiSiluMul)
      return launch_by_block<true, kEpiSiluMul>(bc, w, w_rows, ldw, x, M, ldx, K, o, ldo, n_out, M, n_out, status, stream);
    return launch_by_block<true, kEpiStore>(bc, w, w_rows, ldw, x, M, ldx, K, o, ldo, n_out, M, 0, status, stream);
  }
  if (epi == kEpiSiluMul)
    return launch_by_block<false, kEpiSiluMul>(128, x, M, ldx, w, w_rows, ldw, K, o, ldo, M, n_out, n_out, status, stream);
  return launch_by_block<false, kEpiStore>(128, x, M, ldx, w, w_rows, ldw, K, o, ldo, M, n_out, 0, status, stream);
}

}  // namespace forge

// bf16 GEMM  out[M, N] = X[M, K] * W[N, K]^T  on the 5th-generation tensor cores (tcgen05), fp32
// accumulation in tensor memory, operands staged by TMA with the 128-byte swizzle.
//
// The reference calls F.linear, i.e. cuBLAS (tinyvllm/layers/linear.py:83,181).  Two kernels here cover the
// four linear layers of a decoder block and the LM head:
//
//   gemm_tokens_kernel  (prefill, many tokens): the UMMA's 128-row side is a tile of 128 tokens, the N side a
//       tile of BLOCK_C output features.  Persistent CTAs, two accumulator sets in tensor memory so the epilogue
//       of one tile overlaps the main loop of the next.
//
//   gemm_weights_kernel (decode, <= 256 tokens): operands swapped.  The 128-row side is a tile of 128 weight
//       rows, so the weight stream fills the tensor core and no rows are wasted on token padding; up to 128
//       tokens ride the N side.  Such a GEMM has few output tiles, so K is split over a thread-block cluster of
//       1..8 CTAs and the fp32 partial tiles are reduced through distributed shared memory with bulk copies
//       (see the kernel's comment).
//
// Epilogues: plain store, or SiLU(gate) * up with two accumulators per CTA (gate rows and up rows of the
// packed [2I, H] weight), which removes the [tokens, 2I] intermediate of tinyvllm/layers/activation.py:11-14.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + UMMA issuer, warps 2..5 = epilogue
// (TMEM lane quadrant = warp % 4).  All mbarrier waits are bounded (see ptx.cuh).
#include "../include/launch.cuh"
#include "../include/ptx.cuh"
#include "../include/sampling.cuh"
#include "../include/tp_comm.cuh"

namespace forge {

constexpr int kBlockR = 128;
constexpr int kBlockK = 64;    // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;

enum GemmEpilogue { kEpiStore = 0, kEpiSiluMul = 1, kEpiSample = 2, kEpiQkv = 3 };

// Optional phase timeline of the decode kernel: when set (forge_gemm_set_trace), CTA b writes %globaltimer
// (ns) at eight points into trace[b * 8 ..].  Null in normal operation.
__device__ unsigned long long* g_gemm_trace = nullptr;
__device__ __forceinline__ void trace_point(int cta, int k) {
  unsigned long long* t = g_gemm_trace;
  if (t != nullptr) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    t[cta * 8 + k] = now;
  }
}

// Optional fusion of the RMSNorm that precedes / the residual add that follows a linear layer (both null: plain GEMM).
//
//   in_ssq   the activation rows are NOT normalised: x is the residual stream itself, the norm's weight vector was
//            folded into the columns of W when the model was loaded, and in_ssq[row][0 .. in_parts) holds partial sums
//            of squares of the activation row (one per 128 features, written by the GEMM that produced the row).  The
//            epilogue scales output row r by rsqrt(sum(in_ssq[r]) / K + eps), which is exactly what normalising the
//            input row first would give (the reference normalises in a kernel of its own:
//            tinyvllm/layers/layernorm.py:21-45).
//   residual out[r][c] = bf16(bf16(acc) + out[r][c]): `out` is the residual stream, updated in place, and
//            out_ssq[r][p] = sum of the squares of the new values of features [128 p, 128 p + 128), so that the NEXT
//            linear layer can apply its norm as a row scale.  Every (row, part) is written by exactly one thread and
//            summed in a fixed order: results do not depend on scheduling.  Replaces the add half of add_rms_forward.
struct GemmFuse {
  const float* in_ssq;
  int in_parts;
  float in_width_inv;
  float eps;
  int add_residual;
  float* out_ssq;
  int out_parts;
  int w_dynamic;      // weight-tile kernel only: W was written by the kernel launched just before, do not prefetch it early
};

__device__ __forceinline__ float fuse_row_scale(const GemmFuse& f, int row, int rows) {
  if (f.in_ssq == nullptr) return 1.f;
  if (row >= rows) return 0.f;
  const float* p = f.in_ssq + static_cast<size_t>(row) * f.in_parts;
  float s = 0.f;
  for (int i = 0; i < f.in_parts; ++i) s += p[i];
  return rsqrtf(s * f.in_width_inv + f.eps);
}
__device__ __forceinline__ float bf16_round_g(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Sampling epilogue of the LM-head GEMM (kEpiSample): the logits never reach memory.  Each epilogue thread owns one
// token row of the tile; it rounds every accumulator to bf16 (what the materialised logits would hold) and runs the
// two-level sampler of include/sampling.cuh over the tile's 16 groups of 16 columns: the best group's score, and the token
// drawn inside that group, are written as one pair per (row, vocabulary tile); a small kernel merges the pairs.  Same
// numbers, hence the same tokens, as sample_partial_kernel on materialised logits (tinyvllm/layers/embed_head.py:58-70 +
// tinyvllm/layers/sampler.py:13-21).
struct GemmSample {
  const float* temps;        // [rows]
  const int* header;         // packed step header: [9] step index, [10], [11] seed
  int vocab_start;           // global id of column 0 (a multiple of 4)
  float* part_v;             // [rows][n_tiles]
  int* part_i;
  int n_tiles;
};

// q/k-norm + rotary embedding + KV-cache store in the epilogue of the qkv projection (kEpiQkv; head_dim 128, tiles of 128
// features = one head).  What the reference does in three steps after the GEMM (per-head RMSNorm of q and k:
// tinyvllm/models/qwen3.py:74-96, rotation: tinyvllm/layers/rotary_embedding.py, cache write:
// tinyvllm/layers/attention.py:9-44) happens on the accumulators: each epilogue thread owns one token row of one head,
// rounds it to bf16 (what the GEMM would have stored), normalises (q and k heads), rotates with the token's position and
// writes q rows to q_out and k / v rows into their cache slot (slot < 0: nothing is stored).  Same rounding steps as
// qk_norm_rope_store128_kernel.
struct GemmQkv {
  const __nv_bfloat16* qw;      // [128] norm weights (nullptr: no norm)
  const __nv_bfloat16* kw;
  float eps;
  const float* rope;            // [rope_rows][128]: cos of the 64 pairs, then sin
  int rope_rows;
  const int* positions;         // [tokens]
  const int* slots;             // [tokens] flat cache slot (block * block_size + offset), < 0: do not store
  __nv_bfloat16* q_out;         // [tokens][nq][128]
  __nv_bfloat16* k_cache;       // [blocks][nkv][block_size][128]
  __nv_bfloat16* v_cache;
  int nq, nkv, block_size, do_rope;
  long long num_slots;
};

constexpr int tmem_cols_for(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

// Stream-K for the token-tile kernel (ws == nullptr: off, every CTA computes whole output tiles).
//
// A decode-sized GEMM on a large layer (few hundred tokens x 4096..12288 features x 4096..12288 K) has fewer output tiles
// than the GPU has SMs, or a number of tiles that divides badly by it, while every tile streams megabytes of weights.  The
// (tile, group of K blocks) units are therefore numbered tile-major and dealt out evenly: CTA c of G takes units
// [U c / G, U (c + 1) / G).  Its range may begin in the middle of one tile and end in the middle of another; for such a
// partial tile the CTA writes its fp32 partial sums into a slot of its own in `ws` and counts itself in counters[tile].
// The CTA that arrives LAST adds up all the tile's partial sums, always in the order of the K ranges (the result does not
// depend on which CTA that is), and runs the epilogue.  Nobody waits for anybody.  The last CTA puts the counter back to
// zero, so the buffers serve the next launch on the same stream as they are.
struct GemmStreamK {
  float* ws;          // [gridDim.x][2][kSkSlotFloats]: slot 0 = the partial tile at the start of the CTA's range, 1 = at its end
  int* counters;      // [tiles]
  int kgroup;         // K blocks per unit
  int w_dynamic;      // the weights were written by the kernel launched just before (a dequantised copy): no early prefetch
  int defer;          // partial tiles are only written; gemm_splitk_finish_kernel adds them up and runs the epilogue
};
constexpr int kSkSlotFloats = 128 * 256;       // one accumulator set: 128 rows x up to 256 columns
// Element (row, col) of a slot lives at (col / 4) * 512 + row * 4 + col % 4: the 32 rows x 4 columns of a warp's vector
// access are 512 contiguous bytes.
constexpr int kSkBatch = 4;                    // partial tiles whose loads are in flight together when summing

// Order of the output tiles: groups of `group` token tiles; inside a group the token tile index runs fastest and all
// feature tiles are visited before the next group starts.  CTAs that run at the same time then work on a compact block
// of (a few token tiles) x (a few feature tiles) whose operands stay in L2 even where X or W as a whole does not fit
// (8192 tokens x 12288 features of K).  With at most `group` token tiles this is plain token-tile-fastest order.
constexpr int kRasterGroupTok = 16;      // 128-token tiles: 2048 tokens
constexpr int kRasterGroupPair = 8;      // 256-token tiles
__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int group, int& mt, int& nt) {
  const int per_group = group * n_tiles;
  const int g = t / per_group;
  const int first = g * group;
  const int gm = m_tiles - first < group ? m_tiles - first : group;
  const int within = t - g * per_group;
  mt = first + within % gm;
  nt = within / gm;
}

struct TokSched {
  int num_kb, kgroup, num_kg;
  long long u, u_begin, u_end;     // stream-K: next unit, range of this CTA
  int t_next, t_end, stride;       // whole tiles
  bool stream;
  // worker `w` of `workers` (a CTA of the grid, or a CTA pair)
  __device__ TokSched(int num_tiles, int num_kb_, const GemmStreamK& sk) : TokSched(num_tiles, num_kb_, sk, blockIdx.x, gridDim.x) {}
  __device__ TokSched(int num_tiles, int num_kb_, const GemmStreamK& sk, int w, int workers) {
    num_kb = num_kb_;
    stream = sk.ws != nullptr;
    kgroup = stream ? sk.kgroup : num_kb_;
    num_kg = (num_kb + kgroup - 1) / kgroup;
    const long long U = static_cast<long long>(num_tiles) * num_kg;
    u_begin = stream ? U * w / workers : 0;
    u_end = stream ? U * (w + 1) / workers : 0;
    u = u_begin;
    t_next = w;
    t_end = num_tiles;
    stride = workers;
  }
  // next piece of work: K blocks [kb0, kb1) of tile t
  __device__ bool next(int& t, int& kb0, int& kb1) {
    if (!stream) {
      if (t_next >= t_end) return false;
      t = t_next;
      t_next += stride;
      kb0 = 0;
      kb1 = num_kb;
      return true;
    }
    if (u >= u_end) return false;
    t = static_cast<int>(u / num_kg);
    const long long tile_a = static_cast<long long>(t) * num_kg;
    const long long e = u_end < tile_a + num_kg ? u_end : tile_a + num_kg;
    kb0 = static_cast<int>(u - tile_a) * kgroup;
    kb1 = static_cast<int>(e - tile_a) * kgroup;
    if (kb1 > num_kb) kb1 = num_kb;
    u = e;
    return true;
  }
};

// ---- epilogue pieces shared by the token-tile kernels ----------------------------------------------------------------
// Stream-K bookkeeping of one partial tile, as one epilogue thread sees it.
struct SkTile {
  long long U, a;        // units in all; first unit of this tile
  int workers;           // CTAs (or CTA pairs) the units are dealt to
  int first, n;          // the tile's K ranges belong to workers first .. first + n - 1; n == 0: another CTA adds them up
  int cta_mul, cta_add;  // worker w's scratch slots are those of CTA w * cta_mul + cta_add
};

// One thread's row of an accumulator set (kAccCols fp32 columns at TMEM address tacc) -> scratch slot `slot`.
template <int kAccCols>
__device__ __forceinline__ void sk_dump(uint32_t tacc, float* slot, int row_in_tile, bool live) {
  float* mine = slot + row_in_tile * 4;
#pragma unroll 1
  for (int cc = 0; cc < kAccCols; cc += 32) {
    uint32_t v[32];
    tmem_ld_x32(tacc + cc, v);
    tmem_ld_wait();
    if (live) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(mine + ((cc >> 2) + q) * 512) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    }
  }
}

// Called by the 128 epilogue threads of a CTA after sk_dump: counts the CTA in for tile t (counter `counter`) and tells
// whether it is the last of the tile's contributors, i.e. the one that adds the partial sums up (n > 0).
__device__ __forceinline__ SkTile sk_arrive(const GemmStreamK& sk, int counter, int* flag, bool first_thread, int t, int num_tiles,
                                            int num_kg, int workers, int cta_mul, int cta_add) {
  __threadfence();
  named_barrier_sync(1, 128);
  if (first_thread) *flag = atomicAdd(&sk.counters[counter], 1);
  named_barrier_sync(1, 128);
  const int arrived = *flag;
  SkTile tile;
  tile.U = static_cast<long long>(num_tiles) * num_kg;
  tile.a = static_cast<long long>(t) * num_kg;
  tile.workers = workers;
  tile.cta_mul = cta_mul;
  tile.cta_add = cta_add;
  const long long G = workers;
  tile.first = static_cast<int>(((tile.a + 1) * G + tile.U - 1) / tile.U) - 1;
  tile.n = static_cast<int>(((tile.a + num_kg) * G + tile.U - 1) / tile.U) - tile.first;
  if (arrived != tile.n - 1) {
    tile.n = 0;
  } else {
    __threadfence();
    if (first_thread) sk.counters[counter] = 0;
  }
  return tile;
}

// One thread's row of an output tile: accumulators (whole tile: from tensor memory at tacc; else the sum of the partial
// tiles described by `tile`) -> row scale / SiLU * up / residual add and sums of squares -> bf16 row `r` of `out`,
// columns c0 .. c0 + BLOCK_C.
template <int BLOCK_C, int kEpi>
__device__ __forceinline__ void tile_epilogue(uint32_t tacc, bool whole, const SkTile& tile, const float* ws, int row_in_tile, int r,
                                              int c0, int m_total, int n_total, __nv_bfloat16* __restrict__ out, int ldo,
                                              const GemmFuse& fuse) {
  constexpr int kChunk = BLOCK_C >= 32 ? 32 : 16;
  constexpr int kNumC = kEpi == kEpiSiluMul ? 2 : 1;
  const float row_scale = fuse_row_scale(fuse, r, m_total);          // 1 unless the input norm is folded in
  float ssq = 0.f;                                                   // of the new residual values of this row, current 128 columns
#pragma unroll 1
  for (int cc = 0; cc < BLOCK_C; cc += kChunk) {
    uint32_t v[kChunk];
    uint32_t u[kEpi == kEpiSiluMul ? kChunk : 1];
    const uint32_t taddr = tacc + cc;
    if (whole) {
      if constexpr (kChunk == 32) tmem_ld_x32(taddr, v); else tmem_ld_x16(taddr, v);
      if constexpr (kEpi == kEpiSiluMul) {
        if constexpr (kChunk == 32) tmem_ld_x32(taddr + BLOCK_C, u); else tmem_ld_x16(taddr + BLOCK_C, u);
      }
      tmem_ld_wait();
    } else if constexpr (kChunk == 32) {
      // sum of the partial tiles, in the order of their K ranges
#pragma unroll
      for (int half = 0; half < kNumC; ++half) {
        float a[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) a[j] = 0.f;
        const int col = cc + half * BLOCK_C;
        for (int s0 = 0; s0 < tile.n; s0 += kSkBatch) {
          uint4 pb[kSkBatch][8];
#pragma unroll
          for (int i = 0; i < kSkBatch; ++i) {
            if (s0 + i < tile.n && r < m_total) {
              const int w = tile.first + s0 + i;
              const long long u0 = tile.U * w / tile.workers;
              const float* src = ws + (static_cast<size_t>(w * tile.cta_mul + tile.cta_add) * 2 + (u0 >= tile.a ? 0 : 1)) * kSkSlotFloats + row_in_tile * 4;
#pragma unroll
              for (int q = 0; q < 8; ++q) pb[i][q] = __ldcg(reinterpret_cast<const uint4*>(src + ((col >> 2) + q) * 512));
            }
          }
#pragma unroll
          for (int i = 0; i < kSkBatch; ++i) {
            if (s0 + i < tile.n && r < m_total) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                a[4 * q] += __uint_as_float(pb[i][q].x);
                a[4 * q + 1] += __uint_as_float(pb[i][q].y);
                a[4 * q + 2] += __uint_as_float(pb[i][q].z);
                a[4 * q + 3] += __uint_as_float(pb[i][q].w);
              }
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (half == 0) v[j] = __float_as_uint(a[j]);
          else u[kEpi == kEpiSiluMul ? j : 0] = __float_as_uint(a[j]);
        }
      }
    }
    float f[kChunk];
#pragma unroll
    for (int j = 0; j < kChunk; ++j) {
      f[j] = __uint_as_float(v[j]) * row_scale;
      if constexpr (kEpi == kEpiSiluMul) f[j] = silu(f[j]) * (__uint_as_float(u[j]) * row_scale);
    }
    const int c = c0 + cc;
    if (r < m_total) {
      __nv_bfloat16* dst = out + static_cast<size_t>(r) * ldo + c;
      if (c + kChunk <= n_total && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
        for (int j = 0; j < kChunk; j += 8) {
          if (fuse.add_residual) {
            const uint4 old = *reinterpret_cast<const uint4*>(dst + j);
            const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              f[j + 2 * k] = bf16_round_g(bf16_round_g(f[j + 2 * k]) + bf16_lo(ow[k]));
              f[j + 2 * k + 1] = bf16_round_g(bf16_round_g(f[j + 2 * k + 1]) + bf16_hi(ow[k]));
              ssq += f[j + 2 * k] * f[j + 2 * k] + f[j + 2 * k + 1] * f[j + 2 * k + 1];
            }
          }
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
          if (c + j < n_total) {
            float val = f[j];
            if (fuse.add_residual) {
              val = bf16_round_g(bf16_round_g(val) + __bfloat162float(dst[j]));
              ssq += val * val;
            }
            dst[j] = __float2bfloat16_rn(val);
          }
      }
    }
    if (fuse.out_ssq != nullptr && ((cc + kChunk) & 127) == 0) {      // a group of 128 columns is complete (tiles are 128 or 256 wide)
      const int g0 = c + kChunk - 128;
      if (r < m_total && g0 < n_total) fuse.out_ssq[static_cast<size_t>(r) * fuse.out_parts + (g0 >> 7)] = ssq;
      ssq = 0.f;
    }
  }
}

// =========================================================================================================
// prefill: R = X tile (128 tokens), C = W tile (BLOCK_C features; two tiles for SiLU).  Persistent CTAs.
// =========================================================================================================
// One CTA per SM walks the output tiles (token tiles fastest, so CTAs running at the same time share weight
// tiles in L2).  The TMA ring never drains between tiles, and tensor memory holds TWO accumulator sets: while the
// epilogue warps drain set b (tcgen05.ld -> bf16 -> global), the UMMA warp already fills set b ^ 1 with the next
// tile.  Plain GEMM: 128 x 256 tiles (2 x 256 TMEM columns).  SiLU: 128 x 128 gate + 128 x 128 up per set.
template <int BLOCK_C, int kEpi>
struct TokCfg {
  static constexpr int kNumC = kEpi == kEpiSiluMul ? 2 : 1;
  static constexpr int kRBytes = kBlockR * kBlockK * 2;
  static constexpr int kCBytes = BLOCK_C * kBlockK * 2;
  static constexpr int kStageBytes = kRBytes + kNumC * kCBytes;
  static constexpr int kStagesRaw = (200 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
  static constexpr int kAccCols = BLOCK_C * kNumC;               // TMEM columns of one accumulator set
  static constexpr int kTmemCols = tmem_cols_for(2 * kAccCols);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static_assert(BLOCK_C % 16 == 0 && BLOCK_C >= 16 && BLOCK_C <= 256, "UMMA N for M = 128");
  static_assert(2 * kAccCols <= 512, "two accumulator sets must fit tensor memory");
};

template <int BLOCK_C, int kEpi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tokens_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                   __nv_bfloat16* __restrict__ out, int ldo, int m_total, int n_total, int K, int dual_off, unsigned* status,
                   const TpPush push, const GemmFuse fuse, const GemmSample samp, const GemmStreamK sk, const GemmQkv qk) {
  using Cfg = TokCfg<BLOCK_C, kEpi>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* acc_full = empty_bar + Cfg::kStages;       // [2]
  uint64_t* acc_empty = acc_full + 2;                  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* sk_flag = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (m_total + kBlockR - 1) / kBlockR;
  const int n_tiles = (n_total + BLOCK_C - 1) / BLOCK_C;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + kBlockK - 1) / kBlockK;

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);                     // one arrival per epilogue warp
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // Weights never depend on a predecessor kernel: the weight halves of the first ring stages are requested
    // before waiting for it, the activation halves after (the stage's barrier counts the bytes of both).
    TokSched sched(num_tiles, num_kb, sk);
    int t = 0, kb0 = 0, kb1 = 0;
    bool have = sched.next(t, kb0, kb1);
    const int pre = have ? min(kb1 - kb0, Cfg::kStages) : 0;
    int mt = 0, nt = 0;
    tile_coords(t, m_tiles, n_tiles, kRasterGroupTok, mt, nt);
    const int c_first = nt * BLOCK_C;
    if (sk.w_dynamic) pdl_wait();
    for (int i = 0; i < pre; ++i) {
      uint8_t* st = smem + i * Cfg::kStageBytes;
      mbar_expect_tx(&full_bar[i], Cfg::kStageBytes);
      for (int j = 0; j < Cfg::kNumC; ++j)
        tma_load_2d(st + Cfg::kRBytes + j * Cfg::kCBytes, &tm_w, &full_bar[i], (kb0 + i) * kBlockK, c_first + j * dual_off);
    }
    pdl_wait();                                 // x and out belong to predecessors
    int it = 0;                                 // running K-block counter across tiles: the ring never drains
    while (have) {
      tile_coords(t, m_tiles, n_tiles, kRasterGroupTok, mt, nt);
      const int r0 = mt * kBlockR, c0 = nt * BLOCK_C;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % Cfg::kStages;
        uint8_t* st = smem + s * Cfg::kStageBytes;
        if (it < pre) {                         // first piece, stage already armed and its weights under way
          tma_load_2d(st, &tm_x, &full_bar[s], kb * kBlockK, r0);
          continue;
        }
        const uint32_t ph = (it / Cfg::kStages) & 1;
        if (!mbar_wait_parked(&empty_bar[s], ph ^ 1, status)) { have = false; break; }
        mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
        tma_load_2d(st, &tm_x, &full_bar[s], kb * kBlockK, r0);
        for (int i = 0; i < Cfg::kNumC; ++i)
          tma_load_2d(st + Cfg::kRBytes + i * Cfg::kCBytes, &tm_w, &full_bar[s], kb * kBlockK, c0 + i * dual_off);
      }
      if (have) have = sched.next(t, kb0, kb1);
    }
  } else {
    pdl_wait();
  }

  if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kBlockR, BLOCK_C, 1, 1);
      TokSched sched(num_tiles, num_kb, sk);
      int it = 0, t = 0, kb0 = 0, kb1 = 0;
      for (int n = 0; sched.next(t, kb0, kb1); ++n) {
        const int buf = n & 1;
        if (!mbar_wait_parked(&acc_empty[buf], ((n >> 1) & 1) ^ 1, status)) break;      // the epilogue has drained this set
        tcgen05_fence_after();
        const uint32_t acc_addr = tmem_base + buf * Cfg::kAccCols;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait_parked(&full_bar[s], ph, status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t st = smem_u32(smem + s * Cfg::kStageBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint32_t koff = k * kUmmaK * 2;
            const uint32_t acc = (kb != kb0) || (k != 0);
            const uint64_t dx = umma_desc_k_sw128(st + koff);
            umma_f16(acc_addr, dx, umma_desc_k_sw128(st + Cfg::kRBytes + koff), idesc, acc);
            if constexpr (kEpi == kEpiSiluMul)
              umma_f16(acc_addr + BLOCK_C, dx, umma_desc_k_sw128(st + Cfg::kRBytes + Cfg::kCBytes + koff), idesc, acc);
          }
          umma_commit(&empty_bar[s]);
        }
        umma_commit(&acc_full[buf]);
        if (!ok) break;
      }
    }
  } else if (warp >= 2) {
    const int quad = warp & 3;
    TokSched sched(num_tiles, num_kb, sk);
    int t = 0, kb0 = 0, kb1 = 0;
    for (int n = 0; sched.next(t, kb0, kb1); ++n) {
      const int buf = n & 1;
      int mt = 0, nt = 0;
      tile_coords(t, m_tiles, n_tiles, kRasterGroupTok, mt, nt);
      const int r = mt * kBlockR + quad * 32 + lane;
      const int c0 = nt * BLOCK_C;
      const bool ok = mbar_wait(&acc_full[buf], (n >> 1) & 1, status);
      tcgen05_fence_after();
      const bool whole = kb0 == 0 && kb1 == num_kb;       // false only under stream-K
      bool released = false;                                // accumulator set already handed back
      if constexpr (kEpi == kEpiSample) {
        if (ok) {
          const bool live = r < m_total;                                   // padding rows of the token tile: nothing to sample
          const float T = live ? samp.temps[r] : 0.f;
          const bool greedy = !(T > 0.f);
          const float inv_t = greedy ? 1.f : 1.f / T;
          const uint32_t step = static_cast<uint32_t>(samp.header[9]);
          const uint32_t k0 = static_cast<uint32_t>(samp.header[10]), k1 = static_cast<uint32_t>(samp.header[11]);
          Best best{-INFINITY, 0x7fffffff};              // best group of this tile: (score, group index)
          float bestv[kSampleGroup];                     // its logits, kept for level 2
#pragma unroll
          for (int i = 0; i < kSampleGroup; ++i) bestv[i] = -INFINITY;
          uint32_t rnd[4] = {0, 0, 0, 0};                // group noise: one Philox call per four groups (two chunks)
#pragma unroll 1
          for (int cc = 0; cc < BLOCK_C; cc += 32) {
            uint32_t v[32];
            tmem_ld_x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * Cfg::kAccCols + cc, v);
            tmem_ld_wait();
            if (live && c0 + cc < n_total) {
              const int g0 = (samp.vocab_start + c0 + cc) / kSampleGroup;      // even: tiles and chunks start on multiples of 32 ids
              if (!greedy && (g0 & 3) == 0)
                philox4x32_10(static_cast<uint32_t>(g0 >> 2), static_cast<uint32_t>(r), step, 1u, k0, k1, rnd);
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                float lv[kSampleGroup];
#pragma unroll
                for (int i = 0; i < kSampleGroup; ++i)
                  lv[i] = c0 + cc + h * kSampleGroup + i < n_total ? bf16_round_g(__uint_as_float(v[h * kSampleGroup + i])) : -INFINITY;
                const float sg = sample_group_score(lv, inv_t, greedy, rnd[(g0 + h) & 3]);
                if (sg > best.v) {                         // groups are visited in ascending order: ties keep the earlier one
                  best = Best{sg, g0 + h};
#pragma unroll
                  for (int i = 0; i < kSampleGroup; ++i) bestv[i] = lv[i];
                }
              }
            }
          }
          int token = 0x7fffffff;
          if (live && best.i != 0x7fffffff) token = sample_group_token(bestv, best.i, inv_t, greedy, static_cast<uint32_t>(r), step, k0, k1);
          if (live) {
            const size_t slot = static_cast<size_t>(r) * samp.n_tiles + nt;
            samp.part_v[slot] = best.v;
            samp.part_i[slot] = token;
          }
        }
      } else if constexpr (kEpi == kEpiQkv) {
        if (ok) {
          const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * Cfg::kAccCols;
          const int h = nt;                                             // one tile = one head
          const bool live = r < m_total;
          const bool is_q = h < qk.nq, is_k = !is_q && h < qk.nq + qk.nkv;
          const float row_scale = fuse_row_scale(fuse, r, m_total);
          __nv_bfloat16* dst = nullptr;
          if (live) {
            if (is_q) {
              dst = qk.q_out + (static_cast<size_t>(r) * qk.nq + h) * 128;
            } else {
              const long long slot = qk.slots[r];
              if (slot >= qk.num_slots) set_status(status, kStatusBadIndex);
              if (slot >= 0 && slot < qk.num_slots) {
                const int kvh = is_k ? h - qk.nq : h - qk.nq - qk.nkv;
                const long long blk = slot / qk.block_size, off = slot % qk.block_size;
                dst = (is_k ? qk.k_cache : qk.v_cache) + ((blk * qk.nkv + kvh) * qk.block_size + off) * 128;
              }
            }
          }
          const __nv_bfloat16* nw = is_q ? qk.qw : qk.kw;
          const bool norm = (is_q || is_k) && nw != nullptr;            // uniform over the tile
          const bool rot = (is_q || is_k) && qk.do_rope != 0;
          float inv = 1.f;
          if (norm) {
            float ss = 0.f;
#pragma unroll 1
            for (int cc = 0; cc < 128; cc += 32) {
              uint32_t v[32];
              tmem_ld_x32(tacc + cc, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float x = bf16_round_g(__uint_as_float(v[j]) * row_scale);
                ss += x * x;
              }
            }
            inv = rsqrtf(ss / 128.f + qk.eps);
          }
          const float* cs = qk.rope;
          if (rot) {
            int pos = live ? qk.positions[r] : 0;
            pos = pos < 0 ? 0 : (pos >= qk.rope_rows ? qk.rope_rows - 1 : pos);
            cs = qk.rope + static_cast<size_t>(pos) * 128;
          }
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {                                 // columns [32c, 32c + 32) and their partners 64 further
            uint32_t va[32], vb[32];
            tmem_ld_x32(tacc + 32 * c, va);
            tmem_ld_x32(tacc + 64 + 32 * c, vb);
            tmem_ld_wait();
            float a[32], b[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              a[j] = bf16_round_g(__uint_as_float(va[j]) * row_scale);
              b[j] = bf16_round_g(__uint_as_float(vb[j]) * row_scale);
            }
            if (norm) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const uint4 wa = *reinterpret_cast<const uint4*>(nw + 32 * c + 8 * q4);
                const uint4 wb = *reinterpret_cast<const uint4*>(nw + 64 + 32 * c + 8 * q4);
                const uint32_t ra[4] = {wa.x, wa.y, wa.z, wa.w}, rb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int j = 8 * q4 + 2 * e;
                  a[j] = bf16_round_g(bf16_round_g(a[j] * inv) * bf16_lo(ra[e]));
                  a[j + 1] = bf16_round_g(bf16_round_g(a[j + 1] * inv) * bf16_hi(ra[e]));
                  b[j] = bf16_round_g(bf16_round_g(b[j] * inv) * bf16_lo(rb[e]));
                  b[j + 1] = bf16_round_g(bf16_round_g(b[j + 1] * inv) * bf16_hi(rb[e]));
                }
              }
            }
            if (rot) {
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) {
                const float4 cv = *reinterpret_cast<const float4*>(cs + 32 * c + 4 * q4);
                const float4 sv = *reinterpret_cast<const float4*>(cs + 64 + 32 * c + 4 * q4);
                const float cw[4] = {cv.x, cv.y, cv.z, cv.w}, sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int j = 4 * q4 + e;
                  const float x1 = a[j], x2 = b[j];
                  a[j] = x1 * cw[e] - x2 * sw[e];
                  b[j] = x2 * cw[e] + x1 * sw[e];
                }
              }
            }
            if (dst != nullptr) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const int j = 8 * q4;
                *reinterpret_cast<uint4*>(dst + 32 * c + j) = make_uint4(pack_bf16x2(a[j], a[j + 1]), pack_bf16x2(a[j + 2], a[j + 3]),
                                                                          pack_bf16x2(a[j + 4], a[j + 5]), pack_bf16x2(a[j + 6], a[j + 7]));
                *reinterpret_cast<uint4*>(dst + 64 + 32 * c + j) = make_uint4(pack_bf16x2(b[j], b[j + 1]), pack_bf16x2(b[j + 2], b[j + 3]),
                                                                               pack_bf16x2(b[j + 4], b[j + 5]), pack_bf16x2(b[j + 6], b[j + 7]));
              }
            }
          }
        }
      } else {
        const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * Cfg::kAccCols;
        SkTile tile = {};
        if (ok && !whole) {
          if constexpr (BLOCK_C >= 32) {
            // this CTA's partial sums -> its slot; hand the accumulator set back; count this CTA in
            const long long u_seg = static_cast<long long>(t) * sched.num_kg + kb0 / sched.kgroup;
            sk_dump<Cfg::kAccCols>(tacc, sk.ws + (static_cast<size_t>(blockIdx.x) * 2 + (u_seg == sched.u_begin ? 0 : 1)) * kSkSlotFloats,
                                   quad * 32 + lane, r < m_total);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            released = true;
            if (!sk.defer) tile = sk_arrive(sk, t, sk_flag, warp == 2 && lane == 0, t, num_tiles, sched.num_kg, gridDim.x, 1, 0);
          }
        }
        if (ok && (whole || tile.n > 0))
          tile_epilogue<BLOCK_C, kEpi>(tacc, whole, tile, sk.ws, quad * 32 + lane, r, c0, m_total, n_total, out, ldo, fuse);
      }
      if (!released) {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);     // this accumulator set may be overwritten
      }
      if (!ok) break;
    }
  }

  // Row-parallel layer under tensor parallelism: `out` is this rank's partial buffer in symmetric memory; the last
  // CTA of the grid tells every rank that the partial sums are complete.
  if (push.size > 1) tp_push_done(push, gridDim.x);

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// =========================================================================================================
// many tokens, CTA pairs: one UMMA of M = 256 tokens x N = 256 features per pair of SMs (cta_group::2)
// =========================================================================================================
// The token-tile kernel above is bound by what one SM can load: 48 KB of operands per 128 x 256 x 64 block of
// multiply-adds.  Here the two CTAs of a cluster share one instruction of twice the height: each loads its own 128 tokens
// of X and only HALF of the 256 weight rows (the tensor core reads the other half from the partner's shared memory), i.e.
// 32 KB for the same block.  Plain GEMM: CTA rank r loads weight rows c0 + 128 r.  SiLU: the 256 columns of the
// accumulator are 128 gate + 128 up features, rank 0 loads the gate rows, rank 1 the up rows.  Each CTA drains its own
// 128 x 256 accumulator block.  Persistent over the pairs, two accumulator sets, optional stream-K exactly as above (a
// worker is a pair; every CTA keeps partial tiles and counters of its own rows).
//
// Barriers: full[s] lives in the leader (rank 0): its producer arrives once with the byte count of BOTH CTAs' loads, and
// both CTAs' TMA loads credit it.  empty[s] and acc_full[b] exist in both CTAs and are signalled in both at once by the
// leader's tcgen05.commit.  acc_empty[b] lives in the leader and counts the epilogue warps of both CTAs.
template <int kEpi>
struct PairCfg {
  static constexpr int kBlockN = kEpi == kEpiSiluMul ? 128 : 256;       // output features per tile
  static constexpr int kHalfBytes = kBlockR * kBlockK * 2;              // 128 rows x 64 bf16
  static constexpr int kStageBytes = 2 * kHalfBytes;                    // this CTA's X rows + its half of the weight rows
  static constexpr int kStages = 6;
  static constexpr int kAccCols = 256;
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

template <int kEpi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                 __nv_bfloat16* __restrict__ out, int ldo, int m_total, int n_total, int K, int dual_off, unsigned* status,
                 const TpPush push, const GemmFuse fuse, const GemmStreamK sk) {
  using Cfg = PairCfg<kEpi>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* acc_full = empty_bar + Cfg::kStages;       // [2]
  uint64_t* acc_empty = acc_full + 2;                  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* sk_flag = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());          // 0 = leader
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_tiles = (m_total + 2 * kBlockR - 1) / (2 * kBlockR);
  const int n_tiles = (n_total + Cfg::kBlockN - 1) / Cfg::kBlockN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  const int w_row_rank = rank * (kEpi == kEpiSiluMul ? dual_off : kBlockR);   // this CTA's half of a tile's weight rows

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);                     // one arrival per epilogue warp of both CTAs
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  pdl_launch_dependents();
  tcgen05_fence_before();
  cluster_sync();                                      // both CTAs' barriers and tensor memory exist before anyone signals
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    TokSched sched(num_tiles, num_kb, sk, pair, pairs);
    int t = 0, kb0 = 0, kb1 = 0;
    bool have = sched.next(t, kb0, kb1);
    const int pre = have ? min(kb1 - kb0, Cfg::kStages) : 0;
    int mt = 0, nt = 0;
    tile_coords(t, m_tiles, n_tiles, kRasterGroupPair, mt, nt);
    const int c_first = nt * Cfg::kBlockN + w_row_rank;
    if (sk.w_dynamic) pdl_wait();
    for (int i = 0; i < pre; ++i) {                    // weights do not depend on the predecessor kernel (unless w_dynamic)
      if (rank == 0) mbar_expect_tx(&full_bar[i], 2 * Cfg::kStageBytes);
      tma_load_2d_pair(smem + i * Cfg::kStageBytes + Cfg::kHalfBytes, &tm_w, dsmem_addr(smem_u32(&full_bar[i]), 0), (kb0 + i) * kBlockK, c_first);
    }
    pdl_wait();
    int it = 0;
    while (have) {
      tile_coords(t, m_tiles, n_tiles, kRasterGroupPair, mt, nt);
      const int r0 = mt * 2 * kBlockR + rank * kBlockR, c0 = nt * Cfg::kBlockN + w_row_rank;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % Cfg::kStages;
        uint8_t* st = smem + s * Cfg::kStageBytes;
        const uint32_t lbar = dsmem_addr(smem_u32(&full_bar[s]), 0);
        if (it < pre) {
          tma_load_2d_pair(st, &tm_x, lbar, kb * kBlockK, r0);
          continue;
        }
        const uint32_t ph = (it / Cfg::kStages) & 1;
        if (!mbar_wait_parked(&empty_bar[s], ph ^ 1, status)) { have = false; break; }
        if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * Cfg::kStageBytes);
        tma_load_2d_pair(st, &tm_x, lbar, kb * kBlockK, r0);
        tma_load_2d_pair(st + Cfg::kHalfBytes, &tm_w, lbar, kb * kBlockK, c0);
      }
      if (have) have = sched.next(t, kb0, kb1);
    }
  } else {
    pdl_wait();
  }

  if (warp == 1 && rank == 0) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(2 * kBlockR, 256, 1, 1);
      TokSched sched(num_tiles, num_kb, sk, pair, pairs);
      int it = 0, t = 0, kb0 = 0, kb1 = 0;
      for (int n = 0; sched.next(t, kb0, kb1); ++n) {
        const int buf = n & 1;
        if (!mbar_wait_parked(&acc_empty[buf], ((n >> 1) & 1) ^ 1, status)) break;      // both epilogues have drained this set
        tcgen05_fence_after();
        const uint32_t acc_addr = tmem_base + buf * Cfg::kAccCols;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait_parked(&full_bar[s], ph, status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t st = smem_u32(smem + s * Cfg::kStageBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint32_t koff = k * kUmmaK * 2;
            umma_f16_pair(acc_addr, umma_desc_k_sw128(st + koff), umma_desc_k_sw128(st + Cfg::kHalfBytes + koff), idesc,
                          (kb != kb0) || (k != 0));
          }
          umma_commit_pair(&empty_bar[s], 3);
        }
        umma_commit_pair(&acc_full[buf], 3);
        if (!ok) break;
      }
    }
  } else if (warp >= 2) {
    const int quad = warp & 3;
    TokSched sched(num_tiles, num_kb, sk, pair, pairs);
    int t = 0, kb0 = 0, kb1 = 0;
    for (int n = 0; sched.next(t, kb0, kb1); ++n) {
      const int buf = n & 1;
      int mt = 0, nt = 0;
      tile_coords(t, m_tiles, n_tiles, kRasterGroupPair, mt, nt);
      const int r = mt * 2 * kBlockR + rank * kBlockR + quad * 32 + lane;
      const int c0 = nt * Cfg::kBlockN;
      const bool ok = mbar_wait(&acc_full[buf], (n >> 1) & 1, status);
      tcgen05_fence_after();
      const bool whole = kb0 == 0 && kb1 == num_kb;
      const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * Cfg::kAccCols;
      const uint32_t leader_empty = dsmem_addr(smem_u32(&acc_empty[buf]), 0);
      bool released = false;
      SkTile tile = {};
      if (ok && !whole) {
        const long long u_seg = static_cast<long long>(t) * sched.num_kg + kb0 / sched.kgroup;
        sk_dump<Cfg::kAccCols>(tacc, sk.ws + (static_cast<size_t>(blockIdx.x) * 2 + (u_seg == sched.u_begin ? 0 : 1)) * kSkSlotFloats,
                               quad * 32 + lane, r < m_total);
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_empty);
        released = true;
        if (!sk.defer) tile = sk_arrive(sk, t * 2 + rank, sk_flag, warp == 2 && lane == 0, t, num_tiles, sched.num_kg, pairs, 2, rank);
      }
      if (ok && (whole || tile.n > 0))
        tile_epilogue<Cfg::kBlockN, kEpi>(tacc, whole, tile, sk.ws, quad * 32 + lane, r, c0, m_total, n_total, out, ldo, fuse);
      if (!released) {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_empty);
      }
      if (!ok) break;
    }
  }

  if (push.size > 1) tp_push_done(push, gridDim.x);

  // Neither CTA may leave while its partner can still signal its barriers or read its shared memory.
  tcgen05_fence_before();
  __syncwarp();
  cluster_sync();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
}

// =========================================================================================================
// split-K in two kernels: partial tiles from the GEMM, sums + epilogue from all SMs
// =========================================================================================================
// With K split S ways and exactly one (tile, K range) per CTA (or CTA pair) the GEMM kernels above only write their fp32
// partial tiles (GemmStreamK::defer).  This kernel adds the S partial tiles of every output element in the order of the K
// ranges and applies the same epilogues (row scale, SiLU * up, residual add + sums of squares).  One CTA adding four
// 128 x 256 partial tiles through its own L2 port takes ~5 us; spread over all SMs the same bytes take ~1 us.
//
// Block = 256 threads, 32 rows x 128 output columns.  Phase 1 (thread = row x 4 groups of 4 columns): reads follow the slot
// layout, a warp reads 512 contiguous bytes per partial tile and group; sums, row scale and SiLU * up go to shared memory
// as fp32.  Phase 2 (warp = 4 rows, lane = 4 consecutive columns): residual add, bf16 rows written 256 bytes at a time,
// sums of squares by a warp shuffle tree (a fixed order).  Grid: (blocks of 32 rows, 128-column parts of a tile, tiles).
struct SplitKFinish {
  const float* ws;
  int num_tiles, m_tiles, n_tiles, num_kg, workers;
  int pair;             // 1: partial tiles come from CTA pairs (256-row tiles, scratch owner = 2 * worker + row half)
  int block_n;          // output columns per tile (SiLU: 128 of the 256 accumulator columns are up features)
  int raster_group;
};
constexpr int kFinishMaxParts = 16;

template <int kEpi>
__global__ void __launch_bounds__(256) gemm_splitk_finish_kernel(const SplitKFinish p, __nv_bfloat16* __restrict__ out, int ldo,
                                                                int m_total, int n_total, const GemmFuse fuse) {
  __shared__ __align__(16) float s_val[32][132];
  __shared__ float s_scale[32];
  __shared__ unsigned s_slot[kFinishMaxParts];        // offset of each partial tile's slot, in units of kSkSlotFloats
  __shared__ int s_n;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.z;
  int mt = 0, nt = 0;
  tile_coords(t, p.m_tiles, p.n_tiles, p.raster_group, mt, nt);
  const int tile_rows = p.pair ? 2 * kBlockR : kBlockR;
  const int row0_in_tile = blockIdx.x * 32;
  const int row0 = mt * tile_rows + row0_in_tile;
  if (row0 >= m_total) return;                                              // no live row in this block (uniform)
  const int half = row0_in_tile >> 7;                                       // which CTA of a pair owns these rows
  const int col0_in_tile = blockIdx.y * 128;
  const int c0 = nt * p.block_n + col0_in_tile;
  if (threadIdx.x < 32) s_scale[threadIdx.x] = fuse_row_scale(fuse, row0 + threadIdx.x, m_total);
  if (threadIdx.x == 32) {
    // the tile's K ranges belong to workers first .. first + n - 1 (the arithmetic of TokSched / sk_arrive)
    const long long U = static_cast<long long>(p.num_tiles) * p.num_kg, G = p.workers;
    const long long a = static_cast<long long>(t) * p.num_kg;
    const int first = static_cast<int>(((a + 1) * G + U - 1) / U) - 1;
    int n = static_cast<int>(((a + p.num_kg) * G + U - 1) / U) - first;
    if (n > kFinishMaxParts) n = kFinishMaxParts;                           // the host never splits that far
    for (int i = 0; i < n; ++i) {
      const int w = first + i;
      const long long u0 = U * w / G;
      s_slot[i] = static_cast<unsigned>((p.pair ? 2 * w + half : w) * 2 + (u0 >= a ? 0 : 1));
    }
    s_n = n;
  }
  __syncthreads();
  const int n = s_n;
  {
    const int r = row0 + lane;
    const float row_scale = s_scale[lane];
    const size_t row_off = static_cast<size_t>((row0_in_tile & 127) + lane) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cg = warp * 4 + j;                                          // group of four columns inside the 128
      const int col = col0_in_tile + cg * 4;
      float acc[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
      if (r < m_total && col < p.block_n) {
        for (int i0 = 0; i0 < n; i0 += 4) {             // four partial tiles' loads in flight; added in order
          float4 v[4], g[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (i0 + k < n) {
              const float* slot = p.ws + static_cast<size_t>(s_slot[i0 + k]) * kSkSlotFloats + row_off;
              v[k] = __ldcg(reinterpret_cast<const float4*>(slot + (col >> 2) * 512));
              if constexpr (kEpi == kEpiSiluMul) g[k] = __ldcg(reinterpret_cast<const float4*>(slot + ((col + p.block_n) >> 2) * 512));
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (i0 + k < n) {
              acc[0] += v[k].x; acc[1] += v[k].y; acc[2] += v[k].z; acc[3] += v[k].w;
              if constexpr (kEpi == kEpiSiluMul) { up[0] += g[k].x; up[1] += g[k].y; up[2] += g[k].z; up[3] += g[k].w; }
            }
          }
        }
      }
      float4 f;
      f.x = acc[0] * row_scale; f.y = acc[1] * row_scale; f.z = acc[2] * row_scale; f.w = acc[3] * row_scale;
      if constexpr (kEpi == kEpiSiluMul) {
        f.x = silu(f.x) * (up[0] * row_scale); f.y = silu(f.y) * (up[1] * row_scale);
        f.z = silu(f.z) * (up[2] * row_scale); f.w = silu(f.w) * (up[3] * row_scale);
      }
      *reinterpret_cast<float4*>(&s_val[lane][cg * 4]) = f;
    }
  }
  __syncthreads();
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
    const int row = warp * 4 + rr, r = row0 + row;
    const int c = c0 + lane * 4;
    const float4 v = *reinterpret_cast<const float4*>(&s_val[row][lane * 4]);
    float f[4] = {v.x, v.y, v.z, v.w};
    float ssq = 0.f;
    if (r < m_total && col0_in_tile + lane * 4 < p.block_n && c < n_total) {
      __nv_bfloat16* dst = out + static_cast<size_t>(r) * ldo + c;
      if (c + 4 <= n_total && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
        if (fuse.add_residual) {
          const uint2 old = *reinterpret_cast<const uint2*>(dst);
          f[0] = bf16_round_g(bf16_round_g(f[0]) + bf16_lo(old.x));
          f[1] = bf16_round_g(bf16_round_g(f[1]) + bf16_hi(old.x));
          f[2] = bf16_round_g(bf16_round_g(f[2]) + bf16_lo(old.y));
          f[3] = bf16_round_g(bf16_round_g(f[3]) + bf16_hi(old.y));
          ssq = (f[0] * f[0] + f[1] * f[1]) + (f[2] * f[2] + f[3] * f[3]);
        }
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c + j < n_total) {
            float val = f[j];
            if (fuse.add_residual) {
              val = bf16_round_g(bf16_round_g(val) + __bfloat162float(dst[j]));
              ssq += val * val;
            }
            dst[j] = __float2bfloat16_rn(val);
          }
      }
    }
    if (fuse.out_ssq != nullptr) {            // sum of squares of the row's 128 columns: a shuffle tree, the same order every time
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
      if (lane == 0 && r < m_total && c0 < n_total) fuse.out_ssq[static_cast<size_t>(r) * fuse.out_parts + (c0 >> 7)] = ssq;
    }
  }
}

// =========================================================================================================
// decode: R = W tile (128 features; two tiles for SiLU), C = X tile (up to 128 tokens), split-K over a cluster
// =========================================================================================================
template <int BLOCK_C, int kEpi, bool kDeep>
struct WgtCfg {
  static constexpr int kNumR = kEpi == kEpiSiluMul ? 2 : 1;
  static constexpr int kRBytes = kBlockR * kBlockK * 2;
  static constexpr int kCBytes = BLOCK_C * kBlockK * 2;
  static constexpr int kStageBytes = kNumR * kRBytes + kCBytes;
  static constexpr int kTileBytes = BLOCK_C * kBlockR * 4;        // one fp32 partial tile [BLOCK_C][128]
  // Shared memory is kept under half an SM (~98 KB) so that TWO CTAs fit: with programmatic dependent launch the
  // next GEMM's CTAs become resident while this one still runs and stream their first weight tiles early.
  // After the main loop the idle ring is reused: [send tile][receive slots][reduced gate values].
  static constexpr int kEpilogueBytes = BLOCK_C <= 64 ? 2 * kTileBytes + (kEpi == kEpiSiluMul ? kTileBytes / 2 : 0) : kTileBytes;
  // kDeep: one CTA per SM with a ~200 KB ring.  A CTA streams (ring bytes in flight / ~1.7 us latency), so when the
  // grid has at most one CTA per SM anyway (many tokens: no K split, ~128 CTAs of 300-600 KB each) the deep ring
  // doubles the rate of every CTA; the price is that a following deep GEMM cannot become resident early.
  static constexpr int kBudget = (kDeep ? 200 : 96) * 1024;
  static constexpr int kMaxStages = kDeep ? 10 : 6;
  static constexpr int kStagesRaw = kBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > kMaxStages ? kMaxStages : (kStagesRaw < 2 ? 2 : kStagesRaw);
  static constexpr int kRingBytes = kStages * kStageBytes > kEpilogueBytes ? kStages * kStageBytes : kEpilogueBytes;
  static constexpr bool kCanSplit = BLOCK_C <= 64;                // wider tiles have no room for receive slots
  static constexpr int kTmemCols = tmem_cols_for(BLOCK_C * kNumR);
  static constexpr int kSmemBytes = kRingBytes + 1024 + 512 + 512;          // alignment slack, barriers, column scales
  static_assert(BLOCK_C % 16 == 0 && BLOCK_C >= 16 && BLOCK_C <= 128, "token tile of the decode kernel");
  static_assert(kStages >= 2, "need at least a double buffer");
  static_assert(kSmemBytes <= (kDeep ? 227 : 113) * 1024, "two CTAs per SM (one for the deep ring)");
};

// out[token, feature] (row stride ldo).  W: [n_total (or 2 * n_total) rows, K]; X: [m_total rows, K].
// Grid (feature tiles, K splits, token tiles); cluster = (1, S, 1), cluster rank = K split.
//
// Epilogue = push-reduce over the cluster.  Columns (tokens) of the tile are dealt out to the CTAs of the
// cluster: CTA d owns columns [d * cpc, (d + 1) * cpc).  Every CTA writes its fp32 partial tile from tensor
// memory into its own (now idle) ring as [col][row], then ONE bulk copy per peer (cp.async.bulk shared::cta ->
// shared::cluster, completion counted in bytes by the owner's mbarrier) moves each owner's columns into slot
// recv[source rank] of the owner's dedicated receive buffer.  The owner waits once for all bytes, sums the S
// slots in rank order from its own shared memory (deterministic) and stores bf16 rows with 8-byte writes.
// No global scratch, no atomics, no remote loads.
// SiLU: one split -> combine gate and up on the way out of tensor memory.  Several splits -> the gate sum must
// be complete before the nonlinearity: the first exchange reduces the gate tile into gate_red, the second the up tile.
template <int BLOCK_C, int kEpi, bool kDeep>
__global__ void __launch_bounds__(kGemmThreads, kDeep ? 1 : 2)
gemm_weights_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    __nv_bfloat16* __restrict__ out, int ldo, int n_total, int m_total, int K, int kb_per_split,
                    int dual_off, unsigned* status, const TpPush push, const GemmFuse fuse_io) {
  using Cfg = WgtCfg<BLOCK_C, kEpi, kDeep>;
  extern __shared__ uint8_t smem_raw[];
  // The dynamic shared window starts at the same offset in every CTA of the cluster, so equal local
  // addresses name corresponding buffers in all peers.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* send = reinterpret_cast<float*>(smem);                               // [BLOCK_C][128], after the main loop
  float* recv = reinterpret_cast<float*>(smem + Cfg::kTileBytes);             // [nsplit][cpc][128]
  float* gate_red = reinterpret_cast<float*>(smem + 2 * Cfg::kTileBytes);     // [cpc][128]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kRingBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* acc_bar = empty_bar + Cfg::kStages;
  uint64_t* recv_bar = acc_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(recv_bar + 1);
  float* col_scale = reinterpret_cast<float*>(smem + Cfg::kRingBytes + 512);   // [BLOCK_C] row scales of this CTA's tokens (folded norm)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t split = cluster_ctarank(), nsplit = cluster_nctarank();
  const int cta_id = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) trace_point(cta_id, 0);                  // kernel entry
  pdl_launch_dependents();
  const int r0 = blockIdx.x * kBlockR;
  const int tok0 = blockIdx.z * BLOCK_C;
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
    mbar_init(recv_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncwarp();
  cluster_sync();              // CTA-wide barrier too; afterwards every peer's recv_bar exists
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) trace_point(cta_id, 1);                  // prologue done

  if (warp == 0) {
    if (lane == 0) {
      // Weights never depend on a predecessor kernel: start streaming them into every stage of the ring right
      // away, and wait for the predecessor only before the first activation tile is requested.
      const int first = min(my_kb, Cfg::kStages);
      if (fuse_io.w_dynamic) pdl_wait();                 // ... unless they are a copy made by the preceding kernel
      for (int i = 0; i < first; ++i) {
        uint8_t* st = smem + i * Cfg::kStageBytes;
        const int kx = (kb0 + i) * kBlockK;
        mbar_expect_tx(&full_bar[i], Cfg::kStageBytes);
        for (int j = 0; j < Cfg::kNumR; ++j) tma_load_2d(st + j * Cfg::kRBytes, &tm_w, &full_bar[i], kx, r0 + j * dual_off);
      }
      pdl_wait();
      for (int i = 0; i < first; ++i)
        tma_load_2d(smem + i * Cfg::kStageBytes + Cfg::kNumR * Cfg::kRBytes, &tm_x, &full_bar[i], (kb0 + i) * kBlockK, tok0);
      for (int i = first; i < my_kb; ++i) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (i / Cfg::kStages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, status)) break;
        uint8_t* st = smem + s * Cfg::kStageBytes;
        const int kx = (kb0 + i) * kBlockK;
        mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
        for (int j = 0; j < Cfg::kNumR; ++j) tma_load_2d(st + j * Cfg::kRBytes, &tm_w, &full_bar[s], kx, r0 + j * dual_off);
        tma_load_2d(st + Cfg::kNumR * Cfg::kRBytes, &tm_x, &full_bar[s], kx, tok0);
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kBlockR, BLOCK_C, 1, 1);
      for (int i = 0; i < my_kb; ++i) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (i / Cfg::kStages) & 1;
        if (!mbar_wait(&full_bar[s], ph, status)) break;
        if (i == 0) trace_point(cta_id, 2);                      // first stage landed
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

  // ---------------------------------------------------------------- epilogue (warps 2..5)
  const bool is_epi = warp >= 2;
  const int quad = warp & 3;
  const int et = quad * 32 + lane;                               // epilogue thread id == TMEM lane == tile row
  const bool fuse = kEpi == kEpiSiluMul && nsplit == 1;
  const int rounds = (kEpi == kEpiSiluMul && !fuse) ? 2 : 1;
  const int cpc = BLOCK_C / static_cast<int>(nsplit);            // columns per owner
  const uint32_t slot_bytes = static_cast<uint32_t>(cpc) * kBlockR * 4;
  bool acc_ok = true;
  unsigned ll_tag = 0;
  if (is_epi) {
    pdl_wait();                                                  // `out` may still be read by a predecessor
    // tagged-word push: the tag is this exchange's epoch.  Read before this CTA reports its arrival, i.e. before the
    // grid's last CTA can advance the counter.
    if (push.size > 1 && push.ll) ll_tag = *push.epoch + 1u;
    // folded input norm: the scale of every token column of this CTA, once
    if (fuse_io.in_ssq != nullptr) {
      if (et < BLOCK_C) col_scale[et] = fuse_row_scale(fuse_io, tok0 + et, m_total);
      named_barrier_sync(1, 128);
    }
    acc_ok = mbar_wait(acc_bar, 0, status);                      // this CTA's ring is idle from here on
    tcgen05_fence_after();
    if (et == 0) trace_point(cta_id, 3);                         // accumulators complete
  }
  if (nsplit > 1) {                                              // receive slots alias the ring: every peer's main loop must be over
    __syncwarp();
    cluster_sync();
  }
  for (int round = 0; round < rounds; ++round) {
    if (is_epi) {
      constexpr int kChunk = BLOCK_C >= 32 ? 32 : 16;
#pragma unroll 1
      for (int cc = 0; cc < BLOCK_C; cc += kChunk) {
        uint32_t v[kChunk];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + round * BLOCK_C + cc;
        if (my_kb > 0 && acc_ok) {
          if constexpr (kChunk == 32) tmem_ld_x32(taddr, v); else tmem_ld_x16(taddr, v);
          if constexpr (kEpi == kEpiSiluMul) {
            if (fuse) {
              uint32_t u[kChunk];
              if constexpr (kChunk == 32) tmem_ld_x32(taddr + BLOCK_C, u); else tmem_ld_x16(taddr + BLOCK_C, u);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < kChunk; ++j) {
                const float sc = fuse_io.in_ssq != nullptr ? col_scale[cc + j] : 1.f;     // column = token
                v[j] = __float_as_uint(silu(__uint_as_float(v[j]) * sc) * (__uint_as_float(u[j]) * sc));
              }
            }
          }
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < kChunk; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < kChunk; ++j) send[(cc + j) * kBlockR + et] = __uint_as_float(v[j]);   // lanes -> consecutive floats
      }
      const float* src = recv;                                   // where this CTA's columns are summed from
      bool got = true;
      if (nsplit > 1) {
        fence_proxy_async_smem();                                // generic-proxy writes -> visible to the bulk-copy engine
        named_barrier_sync(1, 128);                              // the four epilogue warps
        if (et == 0) trace_point(cta_id, 4);                     // tile written to shared memory
        if (et == 0) {
          mbar_expect_tx(recv_bar, static_cast<uint32_t>(Cfg::kTileBytes));
          for (uint32_t d = 0; d < nsplit; ++d)
            bulk_copy_to_peer(dsmem_addr(smem_u32(recv) + split * slot_bytes, d), smem_u32(send) + d * slot_bytes, slot_bytes,
                              dsmem_addr(smem_u32(recv_bar), d));
        }
        got = mbar_wait(recv_bar, round & 1, status);            // all S slots of my columns have landed
      } else {
        named_barrier_sync(1, 128);                              // single split: the tile is already where it is needed
        src = send;
      }
      if (et == 0) trace_point(cta_id, 5);                       // partials received
      if (got) {
        // a warp handles one column at a time; lane l owns rows 4l..4l+3.  Two columns per iteration keep
        // several shared-memory loads in flight.
        for (int lc0 = quad; lc0 < cpc; lc0 += 8) {
          float4 a[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            const int lc = lc0 + 4 * u;
            if (lc < cpc) {
              for (uint32_t p = 0; p < nsplit; ++p) {
                const float4 t = *reinterpret_cast<const float4*>(src + (p * cpc + lc) * kBlockR + lane * 4);
                a[u].x += t.x; a[u].y += t.y; a[u].z += t.z; a[u].w += t.w;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int lc = lc0 + 4 * u;
            if (lc >= cpc) continue;                       // uniform for the warp
            float4 v = a[u];
            const int c = tok0 + static_cast<int>(split) * cpc + lc;
            const int n = r0 + lane * 4;
            // the input norm folded in: scale this token's column (the single-split SiLU path scaled on the way out of tensor memory)
            const float sc = ((kEpi == kEpiSiluMul && fuse) || fuse_io.in_ssq == nullptr) ? 1.f : col_scale[c - tok0];
            if constexpr (kEpi == kEpiSiluMul) {
              if (!fuse) {
                float4* g = reinterpret_cast<float4*>(gate_red + lc * kBlockR + lane * 4);   // same thread in both rounds
                if (round == 0) {
                  *g = v;
                  continue;
                }
                const float4 gv = *g;
                v.x = silu(gv.x * sc) * (v.x * sc); v.y = silu(gv.y * sc) * (v.y * sc);
                v.z = silu(gv.z * sc) * (v.z * sc); v.w = silu(gv.w * sc) * (v.w * sc);
              }
            } else {
              v.x *= sc; v.y *= sc; v.z *= sc; v.w *= sc;
            }
            float ssq = 0.f;
            if (c < m_total && n < n_total) {
              if (push.size > 1 && push.ll) {
                // decode-sized exchange: the row goes, as tagged words, straight to the rank that owns it (a peer store
                // over NVLink, or a local one), while other CTAs still compute (tp_comm.cuh, "tagged words")
                const int owner = c % push.size, j = c / push.size;
                uint32_t* d = reinterpret_cast<uint32_t*>(push.slot[owner]) +
                              (static_cast<size_t>(push.rank) * push.rows_per_rank + j) * ldo + n;
                st_volatile_v4(d, make_uint4(pack_bf16x2(v.x, v.y), ll_tag, pack_bf16x2(v.z, v.w), ll_tag));
              } else {
                // Row-parallel layer under tensor parallelism, many rows: `out` is this rank's partial buffer in symmetric
                // memory; the stores are local, the consumer kernels of all ranks pull the sum over NVLink (tp_comm.cuh).
                __nv_bfloat16* dst = out + static_cast<size_t>(c) * ldo + n;
                if (n + 4 <= n_total && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
                  if (fuse_io.add_residual) {               // `out` is the residual stream: add in place
                    const uint2 old = *reinterpret_cast<const uint2*>(dst);
                    v.x = bf16_round_g(bf16_round_g(v.x) + bf16_lo(old.x)); v.y = bf16_round_g(bf16_round_g(v.y) + bf16_hi(old.x));
                    v.z = bf16_round_g(bf16_round_g(v.z) + bf16_lo(old.y)); v.w = bf16_round_g(bf16_round_g(v.w) + bf16_hi(old.y));
                    ssq = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                  }
                  uint2 pk;
                  pk.x = pack_bf16x2(v.x, v.y);
                  pk.y = pack_bf16x2(v.z, v.w);
                  *reinterpret_cast<uint2*>(dst) = pk;
                } else {
                  const float f[4] = {v.x, v.y, v.z, v.w};
                  for (int j = 0; j < 4 && n + j < n_total; ++j) {
                    float val = f[j];
                    if (fuse_io.add_residual) {
                      val = bf16_round_g(bf16_round_g(val) + __bfloat162float(dst[j]));
                      ssq += val * val;
                    }
                    dst[j] = __float2bfloat16_rn(val);
                  }
                }
              }
            }
            if (fuse_io.out_ssq != nullptr) {              // uniform for the warp: all 32 lanes hold features of token c
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
              if (lane == 0 && c < m_total) fuse_io.out_ssq[static_cast<size_t>(c) * fuse_io.out_parts + blockIdx.x] = ssq;   // this CTA's 128 features
            }
          }
        }
      }
    }
    // Every peer has received (hence my outgoing copies have finished reading `send`) and consumed its slots:
    // the buffers may be reused by the next round, or released at exit.
    if (is_epi && et == 0) trace_point(cta_id, 6);               // output stored
    __syncwarp();
    cluster_sync();
  }
  if (threadIdx.x == 0) trace_point(cta_id, 7);                  // after the final cluster barrier
  if (push.size > 1) {
    if (push.ll) tp_tagged_done(push, gridDim.x * gridDim.y * gridDim.z);      // the data carries its tag: only the epoch advances
    else tp_push_done(push, gridDim.x * gridDim.y * gridDim.z);                // last CTA of the grid signals every rank
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

// Kernels of this library launched or captured so far (all source files share the counter of launch.cuh).
extern "C" long long forge_launch_count() { return launch_counter().load(std::memory_order_relaxed); }

extern "C" int forge_gemm_set_trace(unsigned long long* buf) {
  return cudaMemcpyToSymbol(g_gemm_trace, &buf, sizeof(buf)) == cudaSuccess ? 0 : -1;
}

// Stream-K scratch of each device: set once per process and device by the host library (forge_gemm_set_streamk_workspace),
// shared by every GEMM launched on that device, which must therefore be ordered on one stream.
struct StreamKWorkspace {
  float* ws;
  int* counters;
  int ctas, tiles;
};
static StreamKWorkspace g_sk_workspace[16];

extern "C" int forge_gemm_set_streamk_workspace(float* ws, int* counters, int ctas, int tiles) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return -1;
  g_sk_workspace[dev] = StreamKWorkspace{ws, counters, ctas, tiles};
  return 0;
}
// floats a workspace for `ctas` CTAs needs
extern "C" long long forge_gemm_streamk_workspace_floats(int ctas) { return static_cast<long long>(ctas) * 2 * kSkSlotFloats; }

static const StreamKWorkspace* streamk_workspace() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  return g_sk_workspace[dev].ws != nullptr ? &g_sk_workspace[dev] : nullptr;
}

// Launches the reduce + epilogue kernel behind a GEMM that only wrote partial tiles.
template <int kEpi>
static int launch_finish(const GemmStreamK& sk, int tiles, int m_tiles, int n_tiles, int num_kg, int workers, int pair, int block_n,
                         int raster_group, __nv_bfloat16* out, int ldo, int M, int n_out, const GemmFuse& fuse, cudaStream_t stream) {
  SplitKFinish p = {sk.ws, tiles, m_tiles, n_tiles, num_kg, workers, pair, block_n, raster_group};
  const int tile_rows = pair ? 2 * kBlockR : kBlockR;
  const int live_rows = M < tile_rows ? M : tile_rows;
  dim3 grid((live_rows + 31) / 32, (block_n + 127) / 128, tiles);
  return launch_kernel(gemm_splitk_finish_kernel<kEpi>, grid, dim3(256), 0, stream, 0, p, out, ldo, M, n_out, fuse) == cudaSuccess ? 0 : -5;
}

// kgroup > 0: stream-K with units of `kgroup` K blocks (needs the device's workspace; falls back to whole tiles without it).
// defer_splits > 1: K split that many ways, one (tile, K range) per CTA, sums and epilogue by gemm_splitk_finish_kernel.
template <int BLOCK_C, int kEpi>
static int launch_tokens(const void* x, int ldx, const void* w, int w_rows, int ldw, __nv_bfloat16* out, int ldo, int M,
                         int n_out, int K, unsigned* status, cudaStream_t stream, const TpPush& push, const GemmFuse& fuse,
                         const GemmSample& samp = GemmSample{}, int kgroup = 0, int w_dynamic = 0, int defer_splits = 0,
                         const GemmQkv& qk = GemmQkv{}) {
  using Cfg = TokCfg<BLOCK_C, kEpi>;
  w_dynamic |= fuse.w_dynamic;
  CUtensorMap tm_x, tm_w;
  if (forge_make_tmap_2d(&tm_x, x, M, K, ldx, kBlockR, 2) != 0) return -2;
  if (forge_make_tmap_2d(&tm_w, w, w_rows, K, ldw, BLOCK_C, 2) != 0) return -3;
  auto kern = gemm_tokens_kernel<BLOCK_C, kEpi>;
  FORGE_ENSURE_DYN_SMEM(kern, Cfg::kSmemBytes);
  const int m_tiles = (M + kBlockR - 1) / kBlockR, n_tiles = (n_out + BLOCK_C - 1) / BLOCK_C;
  const int tiles = m_tiles * n_tiles;
  const int num_sms = device_sm_count();
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  int ctas = tiles < num_sms ? tiles : num_sms;
  GemmStreamK sk = {nullptr, nullptr, 0, w_dynamic, 0};
  const StreamKWorkspace* wsp = streamk_workspace();
  if constexpr ((kEpi == kEpiStore || kEpi == kEpiSiluMul) && (BLOCK_C == 128 || BLOCK_C == 256)) {
    if (defer_splits > 1 && wsp != nullptr && push.size <= 1) {
      const int kg = (num_kb + defer_splits - 1) / defer_splits;
      const int num_kg = (num_kb + kg - 1) / kg;
      const long long units = static_cast<long long>(tiles) * num_kg;
      if (num_kg > 1 && units <= num_sms && units <= wsp->ctas) {
        sk = GemmStreamK{wsp->ws, wsp->counters, kg, w_dynamic, 1};
        if (launch_kernel(kern, dim3(static_cast<unsigned>(units)), dim3(kGemmThreads), Cfg::kSmemBytes, stream, 0, tm_x, tm_w, out, ldo, M,
                          n_out, K, n_out, status, push, fuse, samp, sk, qk) != cudaSuccess)
          return -5;
        return launch_finish<kEpi>(sk, tiles, m_tiles, n_tiles, num_kg, static_cast<int>(units), 0, BLOCK_C, kRasterGroupTok, out, ldo, M,
                                   n_out, fuse, stream);
      }
    }
  }
  if (kgroup > 0 && BLOCK_C >= 32 && (kEpi == kEpiStore || kEpi == kEpiSiluMul)) {
    if (kgroup > num_kb) kgroup = num_kb;
    const long long units = static_cast<long long>(tiles) * ((num_kb + kgroup - 1) / kgroup);
    const int want = units < num_sms ? static_cast<int>(units) : num_sms;
    if (wsp != nullptr && want <= wsp->ctas && tiles <= wsp->tiles && units > tiles) {
      sk = GemmStreamK{wsp->ws, wsp->counters, kgroup, w_dynamic, 0};
      ctas = want;
    }
  }
  return launch_kernel(kern, dim3(ctas), dim3(kGemmThreads), Cfg::kSmemBytes, stream, 0, tm_x, tm_w, out, ldo, M, n_out, K, n_out,
                       status, push, fuse, samp, sk, qk) == cudaSuccess ? 0 : -5;
}

// CTA-pair kernel: grid = 2 x pairs, clusters of 2 along x.  kgroup > 0: stream-K over the pairs.  defer_splits > 1: K split
// that many ways, one (tile, K range) per pair, sums and epilogue by gemm_splitk_finish_kernel.
template <int kEpi>
static int launch_pair(const void* x, int ldx, const void* w, int w_rows, int ldw, __nv_bfloat16* out, int ldo, int M, int n_out,
                       int K, unsigned* status, cudaStream_t stream, const TpPush& push, const GemmFuse& fuse, int kgroup,
                       int w_dynamic = 0, int defer_splits = 0) {
  using Cfg = PairCfg<kEpi>;
  w_dynamic |= fuse.w_dynamic;
  CUtensorMap tm_x, tm_w;
  if (forge_make_tmap_2d(&tm_x, x, M, K, ldx, kBlockR, 2) != 0) return -2;
  if (forge_make_tmap_2d(&tm_w, w, w_rows, K, ldw, kBlockR, 2) != 0) return -3;
  auto kern = gemm_pair_kernel<kEpi>;
  FORGE_ENSURE_DYN_SMEM(kern, Cfg::kSmemBytes);
  const int m_tiles = (M + 2 * kBlockR - 1) / (2 * kBlockR), n_tiles = (n_out + Cfg::kBlockN - 1) / Cfg::kBlockN;
  const int tiles = m_tiles * n_tiles;
  const int max_pairs = device_sm_count() / 2;
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  int pairs = tiles < max_pairs ? tiles : max_pairs;
  GemmStreamK sk = {nullptr, nullptr, 0, w_dynamic, 0};
  const StreamKWorkspace* wsp = streamk_workspace();
  if (defer_splits > 1 && wsp != nullptr && push.size <= 1) {
    const int kg = (num_kb + defer_splits - 1) / defer_splits;
    const int num_kg = (num_kb + kg - 1) / kg;
    const long long units = static_cast<long long>(tiles) * num_kg;
    if (num_kg > 1 && units <= max_pairs && 2 * units <= wsp->ctas) {
      sk = GemmStreamK{wsp->ws, wsp->counters, kg, w_dynamic, 1};
      if (launch_kernel_cluster_x(kern, dim3(static_cast<unsigned>(2 * units)), dim3(kGemmThreads), Cfg::kSmemBytes, stream, 2, tm_x, tm_w,
                                  out, ldo, M, n_out, K, n_out, status, push, fuse, sk) != cudaSuccess)
        return -5;
      return launch_finish<kEpi>(sk, tiles, m_tiles, n_tiles, num_kg, static_cast<int>(units), 1, Cfg::kBlockN, kRasterGroupPair, out, ldo,
                                 M, n_out, fuse, stream);
    }
  }
  if (kgroup > 0) {
    if (kgroup > num_kb) kgroup = num_kb;
    const long long units = static_cast<long long>(tiles) * ((num_kb + kgroup - 1) / kgroup);
    const int want = units < max_pairs ? static_cast<int>(units) : max_pairs;
    if (wsp != nullptr && 2 * want <= wsp->ctas && 2 * tiles <= wsp->tiles && units > tiles) {
      sk = GemmStreamK{wsp->ws, wsp->counters, kgroup, w_dynamic, 0};
      pairs = want;
    }
  }
  return launch_kernel_cluster_x(kern, dim3(2 * pairs), dim3(kGemmThreads), Cfg::kSmemBytes, stream, 2, tm_x, tm_w, out, ldo, M, n_out,
                                 K, n_out, status, push, fuse, sk) == cudaSuccess ? 0 : -5;
}

// Cluster size (K splits) of the decode kernel.  Measured on B200 (sweeps over token tile x splits x ring depth for
// the Qwen3-0.6B and -8B layer shapes): a CTA streams at most ~100 GB/s (ring bytes in flight / memory latency), two
// CTAs fit per SM, and the cross-CTA exchange over DSMEM runs at only ~20 GB/s per SM.  So: the largest power of two
// that keeps the grid within two CTAs per SM, leaves each split >= 2 K blocks and each CTA >= 4 columns to reduce.
static int choose_splits(int ctas_unsplit, int num_kb, int block_c, bool silu) {
  // fewer K blocks per CTA also means the whole K slice is prefetched into the ring before the predecessor kernel ends
  static const int split_limit_env = std::getenv("FORGE_SPLIT_LIMIT") ? std::atoi(std::getenv("FORGE_SPLIT_LIMIT")) : 0;
  const int sms = device_sm_count();
  const int small_limit = split_limit_env > 0 ? split_limit_env : 2 * sms;      // two CTAs per SM
  // SiLU needs the complete gate sum before the nonlinearity, i.e. two exchange rounds: split less eagerly (~1.35 CTAs per SM)
  const int limit = silu ? (sms * 200) / 148 : small_limit;
  int s = 1;
  while (s < 8 && ctas_unsplit * s * 2 <= limit && num_kb / (s * 2) >= 2 && s * 2 <= block_c / 4) s *= 2;
  return s;
}

// Rows of 128 bytes a CTA streams (K blocks x (token tile + weight rows)) from which the deep ring pays off.
static int deep_threshold() {
  static const int v = std::getenv("FORGE_DEEP_ROWS") ? std::atoi(std::getenv("FORGE_DEEP_ROWS")) : 1536;
  return v;
}

template <int BLOCK_C, int kEpi, bool kDeep>
static int launch_weights(const void* x, int ldx, const void* w, int w_rows, int ldw, __nv_bfloat16* out, int ldo, int M,
                          int n_out, int K, int splits, unsigned* status, cudaStream_t stream, const TpPush& push, const GemmFuse& fuse) {
  using Cfg = WgtCfg<BLOCK_C, kEpi, kDeep>;
  CUtensorMap tm_x, tm_w;
  if (forge_make_tmap_2d(&tm_w, w, w_rows, K, ldw, kBlockR, 2) != 0) return -2;
  if (forge_make_tmap_2d(&tm_x, x, M, K, ldx, BLOCK_C, 2) != 0) return -3;
  auto kern = gemm_weights_kernel<BLOCK_C, kEpi, kDeep>;
  FORGE_ENSURE_DYN_SMEM(kern, Cfg::kSmemBytes);
  const int tiles = (n_out + kBlockR - 1) / kBlockR;
  const int tok_tiles = (M + BLOCK_C - 1) / BLOCK_C;
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  const int kb_per_split = (num_kb + splits - 1) / splits;
  return launch_kernel(kern, dim3(tiles, splits, tok_tiles), dim3(kGemmThreads), Cfg::kSmemBytes, stream, splits, tm_w, tm_x,
                       out, ldo, n_out, M, K, kb_per_split, n_out, status, push, fuse) == cudaSuccess ? 0 : -5;
}

// out[M, n_out] = epilogue(X[M, K] * W[*, K]^T).  epi = 0: W has n_out rows.  epi = 1: W is [2 * n_out, K]
// (gate rows then up rows) and out = silu(gate) * up.  Requirements: K % 8 == 0, x/w 16-byte aligned,
// ldx/ldw % 8 == 0.  force_mode: 0 auto, 1 token-tile kernel, 2 weight-tile (decode) kernel (needs M <= 256).
// tune: 0 auto; else bits 0..7 = cluster size (K splits), bits 8..15 = token tile (16/32/64/128) of the decode
// kernel, bits 16..23 = ring depth (1 = two CTAs per SM, 2 = deep ring); each may be 0 = choose; bit 24 = W was written by
// the kernel launched just before (more than 256 tokens only).  Returns 0 on success.
TpPush make_tp_push(int tp_size, int tp_rank, const long long* slot_ptrs, const long long* signal_ptrs, unsigned* arrive,
                    unsigned* epoch);

static int gemm_dispatch(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int n_out, int K, int epi,
                         int force_mode, int tune, unsigned* status, cudaStream_t stream, const TpPush& push,
                         const GemmFuse& fuse_in = GemmFuse{}) {
  const int force_splits = tune & 0xff, force_deep = (tune >> 16) & 0xff;
  const int w_dynamic = (tune >> 24) & 1;        // W is the output of the preceding kernel: no kernel may prefetch it early
  GemmFuse fuse = fuse_in;
  fuse.w_dynamic = w_dynamic;
  int force_bc = (tune >> 8) & 0xff;
  if (M <= 0 || n_out <= 0 || K <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return -1;
  const int w_rows = epi == kEpiSiluMul ? 2 * n_out : n_out;
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  // Few tokens -> the weight-tile (decode) kernel, except for very wide layers (the LM head: ~1200 feature tiles), where the
  // persistent token-tile kernel streams weights best: its ring never drains between tiles and its epilogue overlaps
  // the next tile (measured 58-91 us vs 60-182 us for 8..256 tokens x 151936 x 1024; cuBLAS 55-83 us).
  const int sms = device_sm_count();
  const bool wide = (n_out + kBlockR - 1) / kBlockR >= 2 * sms && epi == kEpiStore && push.size <= 1 && M >= 8;
  // More than 256 tokens (prefill): the CTA-pair kernel, whose SMs load two thirds of the bytes of the single-CTA kernel
  // per multiply-add (measured 1.23-1.58 PFLOP/s vs 1.15-1.30 on the 0.6B / 8B layer shapes at 8192 tokens).  Also for
  // 129..256 tokens of a decode step on a layer with at least ~20 tiles of 256 features (qkv and gate_up of 8B, the
  // per-rank gate_up / down of 32B over 8 ranks: 25-53 us vs 32-62 us), where one pair tile covers all tokens and the
  // weights are read once.
  // K split over otherwise idle SMs plus the reduce kernel (measured in CUDA-graph chains, us with / without):
  //  * 129..256 tokens on a large layer whose 256-feature pair tiles leave at least half of the SM pairs idle: 8B qkv 21.3 /
  //    25.5 (3 ways), o_proj 18.5 / 21.1 (3), down_proj 32.6 / 43.3 (4), the per-rank 32B gate_up 26.3 / 29.1 (2);
  //  * a mid-sized gated MLP at 33..128 tokens (the per-rank gate_up of 32B over 8 ranks, 25 tiles): 20-22 / 25-36.
  int defer_splits = 0;
  if (force_mode == 0 && push.size <= 1 && !wide && !w_dynamic) {
    const int max_pairs = sms / 2;
    const int stiles = (n_out + kBlockR - 1) / kBlockR;
    const int ptiles = epi == kEpiSiluMul ? stiles : (n_out + 255) / 256;
    if (M > 128 && M <= 256 && K >= 2048 && static_cast<long long>(w_rows) * K >= (12ll << 20)) {
      int S = max_pairs / ptiles;
      const int cap = K >= 8192 ? 4 : 3;
      if (S > cap) S = cap;
      if (S >= 2) {
        force_mode = 5;
        defer_splits = S;
      }
    } else if (epi == kEpiSiluMul && M > 32 && M <= 128 && K >= 4096 && stiles >= 16 && stiles * 4 <= sms) {
      force_mode = 6;
      defer_splits = 4;
    } else if (epi == kEpiStore && M > 64 && M <= 128 && K >= 4096 && ptiles >= 20 && ptiles * 3 <= sms) {
      force_mode = 6;              // 8B qkv at 65..128 tokens: 19.3 us with K split 3 ways + reduce kernel, 21.5 without
      defer_splits = 3;
    }
  }
  if (force_mode == 0 && push.size <= 1) {
    const int pair_tiles = (n_out + (epi == kEpiSiluMul ? 127 : 255)) / (epi == kEpiSiluMul ? 128 : 256);
    if (M > 256 || (M > 128 && K >= 2048 && pair_tiles >= 20 && !wide)) force_mode = 4;
  }
  // Many tokens of a decode step (64..256) on a layer with enough output features and a short K: the token-tile
  // kernel with narrow feature tiles (32 or 64) gives ~100-128 CTAs without splitting K, and its epilogue goes
  // straight from tensor memory to global rows (no exchange through shared memory).  Measured on the Qwen3-0.6B
  // shapes: qkv 6.5-7.4 us vs 7.7-12.2 us, gate_up at 32..256 tokens 9.2-10.2 us vs 11.7-15.3 us.
  int narrow = 0;
  if (force_mode == 0 && M >= (epi == kEpiSiluMul ? 32 : 64) && M <= 256 && K <= 2048 && push.size <= 1 && !wide) {
    const int m_tiles = (M + kBlockR - 1) / kBlockR;
    const int t32 = ((n_out + 31) / 32) * m_tiles, t64 = ((n_out + 63) / 64) * m_tiles;
    if (n_out < 2048) {}                           // few features (o, down): K must be split, the weight-tile kernel does it
    else if (t32 <= sms) narrow = 32;
    else if (t64 <= sms) narrow = 64;
  }
  if (fuse.add_residual) narrow = 0;              // the sums of squares are kept per 128 features: tiles of 128 or 256
  if (narrow) {
    force_mode = 1;
    force_bc = narrow;
  } else if (force_mode == 0 && epi == kEpiSiluMul && K >= 4096 && M <= 256 && push.size <= 1 &&
             (M > 64 || (M > 24 && (n_out + kBlockR - 1) / kBlockR >= 64))) {
    // a large gated MLP (8B and up) is compute-heavy already at ~100 tokens: full 128 x (128 + 128) tiles; with 64 or
    // more such tiles (8B on one GPU: 96) the persistent kernel also streams best from ~32 tokens (39.5 vs 48 us at 64)
    force_mode = 1;
  }
  if (force_mode == 5 || force_mode == 6) {      // K split `tune & 0xff` ways + reduce kernel: 5 = CTA pairs, 6 = single CTAs
    const int S = defer_splits > 1 ? defer_splits : (force_splits > 1 ? force_splits : 2);
    const GemmSample none{};
    if (force_mode == 5) {
      if (epi == kEpiSiluMul) return launch_pair<kEpiSiluMul>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, 0, w_dynamic, S);
      return launch_pair<kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, 0, w_dynamic, S);
    }
    if (epi == kEpiSiluMul) return launch_tokens<128, kEpiSiluMul>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, none, 0, w_dynamic, S);
    if (force_bc == 128) return launch_tokens<128, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, none, 0, w_dynamic, S);
    return launch_tokens<256, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, none, 0, w_dynamic, S);
  }
  if (force_mode == 3) {            // token-tile kernel with stream-K: tune bits 0..7 = K blocks per unit, bits 8..15 = feature tile
    const int kg = force_splits > 0 ? force_splits : 4;
    const GemmSample none{};
    if (force_bc == 64 && fuse.add_residual) return -6;       // the sums of squares are kept per 128 features
    if (epi == kEpiSiluMul) {
      if (force_bc == 64) return launch_tokens<64, kEpiSiluMul>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, none, kg);
      return launch_tokens<128, kEpiSiluMul>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, none, kg);
    }
    if (force_bc == 64) return launch_tokens<64, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, none, kg);
    if (force_bc == 128) return launch_tokens<128, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, none, kg);
    return launch_tokens<256, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, none, kg);
  }
  if (force_mode == 4) {
    if (epi == kEpiSiluMul) return launch_pair<kEpiSiluMul>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, force_splits, w_dynamic);
    return launch_pair<kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse, force_splits, w_dynamic);
  }
  const bool decode = force_mode == 2 || (force_mode == 0 && M <= 256 && !wide);
  if (decode) {
    if (M > 256) return -7;
    const int feature_tiles = (n_out + kBlockR - 1) / kBlockR;
    // Sweeps over the Qwen3-0.6B and -8B layer shapes: 32-token tiles unless that gives more than one CTA per SM before
    // splitting K; with a long K and many tokens 64, because every extra token tile re-reads its weight tiles from L2.
    int bc = 16;
    if (M > 16) {
      const int cap = M <= 32 ? 32 : M <= 64 ? 64 : 128;
      bc = (K >= 4096 && M > 64) ? 64 : 32;
      // 33..64 tokens on a very long K (8B down_proj) or a layer with many feature tiles and a long K (8B qkv): one token
      // tile, so the weights are read once (23.0-23.8 vs 25.2 us, 17.0 vs 18.1 us)
      if (M > 32 && M <= 64 && (K >= 8192 || (K >= 4096 && feature_tiles >= 48))) bc = 64;
      while (bc < cap && feature_tiles * ((M + bc - 1) / bc) > sms) bc *= 2;
    }
    if (force_bc == 16 || force_bc == 32 || force_bc == 64 || force_bc == 128) bc = force_bc;
    const int num_kb = (K + kBlockK - 1) / kBlockK;
    const int ctas_unsplit = feature_tiles * ((M + bc - 1) / bc);
    int splits = force_splits > 0 ? force_splits : choose_splits(ctas_unsplit, num_kb, bc, epi == kEpiSiluMul);
    // a gated MLP with at least half as many tiles as SMs at <= 16 tokens (8B gate_up: 96): one CTA per tile with the deep ring
    // and no exchange (37.3-37.9 us) instead of K split in two (38.7-39.6)
    if (force_splits == 0 && epi == kEpiSiluMul && bc == 16 && ctas_unsplit * 2 > sms && ctas_unsplit <= sms) splits = 1;
    if (splits > bc / 4) splits = bc / 4;                               // every CTA reduces >= 4 columns (one per warp)
    if (bc > 64) splits = 1;                                            // wide tiles have no room for receive slots
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return -6;
    // ring depth: the deep ring when the grid is at most one CTA per SM and every CTA has many K blocks to stream
    const int kb_per_cta = (num_kb + splits - 1) / splits;
    bool deep = ctas_unsplit * splits <= sms && kb_per_cta * (bc + (epi == kEpiSiluMul ? 256 : 128)) >= deep_threshold();
    // 16-token tiles of a plain projection: two CTAs per SM with the shallow ring were faster on every shape measured
    // (8B o_proj 10.5 vs 12.0 us, down_proj 22.1 vs 22.9; equal on the 0.6B shapes); the gated MLP keeps the deep ring (17 vs 23)
    if (bc == 16 && epi == kEpiStore) deep = false;
    if (force_deep == 1) deep = false;
    if (force_deep == 2) deep = true;
#define FORGE_W2(BC, EPI)                                                                                                   \
  (deep ? launch_weights<BC, EPI, true>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, splits, status, stream, push, fuse)    \
        : launch_weights<BC, EPI, false>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, splits, status, stream, push, fuse))
#define FORGE_W(BC) \
  case BC:          \
    return epi == kEpiSiluMul ? FORGE_W2(BC, kEpiSiluMul) : FORGE_W2(BC, kEpiStore);
    switch (bc) {
      FORGE_W(16)
      FORGE_W(32)
      FORGE_W(64)
      FORGE_W(128)
    }
#undef FORGE_W
#undef FORGE_W2
    return -6;
  }
  if (force_mode == 1 && (force_bc == 16 || force_bc == 32 || force_bc == 64)) {       // narrow feature tiles: many tokens of a decode step
#define FORGE_T(BC)                                                                                                           \
  case BC:                                                                                                                    \
    return epi == kEpiSiluMul ? launch_tokens<BC, kEpiSiluMul>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse)   \
                              : launch_tokens<BC, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse);
    switch (force_bc) {
      FORGE_T(16)
      FORGE_T(32)
      FORGE_T(64)
    }
#undef FORGE_T
  }
  if (epi == kEpiSiluMul) return launch_tokens<128, kEpiSiluMul>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse);
  if (n_out % 256 == 0 || n_out >= 1024) return launch_tokens<256, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse);
  return launch_tokens<128, kEpiStore>(x, ldx, w, w_rows, ldw, o, ldo, M, n_out, K, status, stream, push, fuse);
}

extern "C" int forge_gemm_bf16(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int n_out,
                               int K, int epi, int force_mode, int tune, unsigned* status, cudaStream_t stream) {
  TpPush none = {};
  return gemm_dispatch(x, ldx, w, ldw, out, ldo, M, n_out, K, epi, force_mode, tune, status, stream, none);
}

// Row-parallel GEMM under tensor parallelism: `out` is this rank's partial buffer in symmetric memory (row stride ldo);
// the kernel's last CTA announces completion to every rank through signal_ptrs (tp_size addresses in peer order).
// Up to 256 rows run on the weight-tile (decode) kernel, more on the persistent token-tile kernel.
extern "C" int forge_sample_merge(const float* part_v, const int* part_i, int n, int rows, int* out_i, float* out_v, cudaStream_t stream);

// LM head + sampling in one pass over the weights: out_i[r] = the sampled (T > 0) or arg-max (T == 0) GLOBAL token id of
// row r among this rank's `vocab` columns, out_v[r] its score (for the cross-rank merge).  The logits are never written.
// part_v / part_i: scratch of M * ceil(vocab / 256) entries.  vocab_start must be a multiple of 32 (sampling groups of 16
// ids; a 32-column chunk of the accumulator holds two whole groups).
extern "C" int forge_gemm_bf16_sample(const void* x, int ldx, const void* w, int ldw, int M, int vocab, int K, int vocab_start,
                                      const float* temps, const int* header, float* part_v, int* part_i, int* out_i, float* out_v,
                                      unsigned* status, cudaStream_t stream) {
  if (M <= 0 || vocab <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (vocab_start & 31))
    return -1;
  GemmSample samp;
  samp.temps = temps;
  samp.header = header;
  samp.vocab_start = vocab_start;
  samp.part_v = part_v;
  samp.part_i = part_i;
  samp.n_tiles = (vocab + 255) / 256;
  TpPush none = {};
  GemmFuse plain = {};
  const int rc = launch_tokens<256, kEpiSample>(x, ldx, w, vocab, ldw, nullptr, 0, M, vocab, K, status, stream, none, plain, samp);
  if (rc != 0) return rc;
  return forge_sample_merge(part_v, part_i, samp.n_tiles, M, out_i, out_v, stream);
}

// The same with the neighbouring norm / residual add fused in (see GemmFuse).  in_ssq: fp32 [M][in_parts] partial sums of
// squares of the rows of x (null: rows are not scaled).  add_residual: out += result in place and out_ssq (fp32
// [M][ceil(n_out / 128)], may be null) receives the sums of squares of the new rows per 128 features.
// qkv projection with q/k-norm + rotary embedding + KV-cache store in the epilogue (head_dim 128): x [M, K] times
// w [(nq + 2 nkv) * 128, K]; q rows go to q_out, k / v rows into their cache slots; in_ssq as in forge_gemm_bf16_fused.
extern "C" int forge_gemm_bf16_qkv(const void* x, int ldx, const void* w, int ldw, int M, int K, const float* in_ssq, int in_parts,
                                   float in_eps, const void* qw, const void* kw, float eps, const float* rope, int rope_rows,
                                   const int* positions, const int* slots, void* q_out, void* k_cache, void* v_cache, int nq, int nkv,
                                   int block_size, long long num_slots, int do_rope, unsigned* status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(q_out) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(rope) & 15) || nq <= 0 || nkv <= 0 || block_size <= 0)
    return -1;
  GemmFuse fuse = {};
  fuse.in_ssq = in_ssq;
  fuse.in_parts = in_parts;
  fuse.in_width_inv = 1.f / static_cast<float>(K);
  fuse.eps = in_eps;
  GemmQkv qk = {static_cast<const __nv_bfloat16*>(qw), static_cast<const __nv_bfloat16*>(kw), eps, rope, rope_rows, positions, slots,
                static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache),
                nq, nkv, block_size, do_rope, num_slots};
  const int n_out = (nq + 2 * nkv) * 128;
  TpPush none = {};
  return launch_tokens<128, kEpiQkv>(x, ldx, w, n_out, ldw, nullptr, 0, M, n_out, K, status, stream, none, fuse, GemmSample{}, 0, 0, 0, qk);
}

extern "C" int forge_gemm_bf16_fused(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int n_out, int K,
                                     int epi, int force_mode, int tune, const float* in_ssq, int in_parts, float eps,
                                     int add_residual, float* out_ssq, unsigned* status, cudaStream_t stream) {
  if (add_residual && epi != kEpiStore) return -9;
  if (in_ssq != nullptr && in_parts < 1) return -9;
  if (add_residual && force_mode == 1 && ((tune >> 8) & 0xff) != 0) return -9;      // no narrow tiles with the residual epilogue
  TpPush none = {};
  GemmFuse fuse = {};
  fuse.in_ssq = in_ssq;
  fuse.in_parts = in_parts;
  fuse.in_width_inv = 1.0f / static_cast<float>(K);
  fuse.eps = eps;
  fuse.add_residual = add_residual;
  fuse.out_ssq = add_residual ? out_ssq : nullptr;
  fuse.out_parts = (n_out + 127) / 128;
  return gemm_dispatch(x, ldx, w, ldw, out, ldo, M, n_out, K, epi, force_mode, tune, status, stream, none, fuse);
}

// Row-parallel GEMM under tensor parallelism, at most 256 rows: every output row is stored as tagged words into the
// buffer of the rank that owns it (ll_ptrs[p] = rank p's buffer of [tp_size][rows_per_rank][n_out] 32-bit words).
// n_out must be a multiple of 4.
extern "C" int forge_gemm_bf16_tp_tagged(const void* x, int ldx, const void* w, int ldw, int M, int n_out, int K, int tune, int tp_size,
                                         int tp_rank, const long long* ll_ptrs, int rows_per_rank, unsigned* arrive, unsigned* epoch,
                                         unsigned* status, cudaStream_t stream) {
  if (tp_size < 2 || tp_size > kMaxTp || M <= 0 || M > 256 || (n_out & 3) || (M + tp_size - 1) / tp_size > rows_per_rank) return -7;
  TpPush push = {};
  push.size = tp_size;
  push.rank = tp_rank;
  push.ll = 1;
  push.rows_per_rank = rows_per_rank;
  for (int p = 0; p < tp_size; ++p) push.slot[p] = reinterpret_cast<__nv_bfloat16*>(ll_ptrs[p]);
  push.arrive = arrive;
  push.epoch = epoch;
  return gemm_dispatch(x, ldx, w, ldw, nullptr, n_out, M, n_out, K, kEpiStore, 2, tune, status, stream, push);
}

extern "C" int forge_gemm_bf16_tp(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int n_out, int K,
                                  int tune, int tp_size, int tp_rank, const long long* signal_ptrs, unsigned* arrive,
                                  unsigned* epoch, unsigned* status, cudaStream_t stream) {
  if (tp_size < 2 || tp_size > kMaxTp || M <= 0) return -7;
  const TpPush push = make_tp_push(tp_size, tp_rank, nullptr, signal_ptrs, arrive, epoch);
  return gemm_dispatch(x, ldx, w, ldw, out, ldo, M, n_out, K, kEpiStore, M <= 256 ? 2 : 4, M <= 256 ? tune : (tune & (1 << 24)), status, stream, push);
}

}  // namespace forge

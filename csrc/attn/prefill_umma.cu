// Prefill attention on the 5th-generation tensor cores: variable-length, causal, GQA, keys and values read from
// the paged cache (tinyvllm/layers/attention.py:99-105 calls flash_attn_varlen_func).
//
// CTA = 128 query rows of one (sequence, q head); KV tiles of 128 keys (one tile never straddles a cache block:
// block_size >= 128).  Both products run as tcgen05.mma with fp32 accumulators in tensor memory:
//
//   S = Q K^T   A = Q tile, B = K tile, both K-major, 128-byte swizzle, brought in by TMA
//   O_j = P V   A = P (bf16 probabilities, written to shared memory by the softmax warps in the same swizzled
//               K-major layout), B = V tile exactly as TMA delivers it from the cache ([key][head_dim] rows,
//               i.e. MN-major for this product: no transpose pass)
//
// Warp roles (192 threads): warp 0 = TMA producer (2-stage K ring, 2-stage V ring), warp 1 = tensor-memory owner and
// UMMA issuer, warps 2..5 = softmax: thread = one query row (its TMEM lane), so row max and row sum need no
// shuffles.  S and P are double-buffered and S of tile j+1 is issued before P V of tile j, so the tensor pipe
// computes the next scores while the softmax warps work on the current ones, and P V of tile j overlaps the softmax
// of tile j+1.  O accumulates in tensor memory across tiles.  The exponentials use a reference maximum that is only
// raised when the true row maximum has grown by more than 2^8 since it was set (exact arithmetic either way: O and
// the row sum carry the same factor); only then do the softmax warps read O back, scale it and store it again
// (tcgen05.ld / tcgen05.st), which happens a few times per row instead of once per tile.
//
// The query rows of a sequence are its LAST q_len positions; with a cached prefix the causal mask is aligned to the
// bottom-right corner: query row i sees keys 0 .. (k_len - q_len + i).  All waits are bounded (ptx.cuh).
#include "../include/launch.cuh"
#include "../include/ptx.cuh"

namespace forge {

constexpr int kUD = 128;                  // head_dim
constexpr int kUM = 128;                  // query rows per CTA
constexpr int kUN = 128;                  // keys per tile
constexpr int kUHalf = 128 * 128;         // bytes of one swizzled box: 128 rows x 64 bf16
constexpr int kUTile = 2 * kUHalf;        // one 128 x 128 bf16 operand
constexpr int kUThreads = 192;
constexpr int kUStages = 2;

// Shared-memory descriptor of an MN-major operand as TMA lays it down with the 128-byte swizzle: rows are the K
// index (keys), each row holds 64 contiguous elements of the MN index (head_dim).  Stride between 8-row groups along
// K: 1024 bytes; stride between the two 64-element blocks along MN: one box.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_block_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((mn_block_bytes >> 4) & 0x3FFFu) << 16;   // leading byte offset: next 64 elements along MN
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                         // stride byte offset: next 8 rows along K
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;                                 // SWIZZLE_128B
  return d;
}

// Row maximum of the raw scores of one tile; kMasked: only keys kbase + i < limit count.  Four chains, not one.
template <bool kMasked>
__device__ __forceinline__ float umma_row_max(const uint32_t (&v)[kUN], int kbase, int limit) {
  float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < kUN; i += 4) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x = __uint_as_float(v[i + e]);
      m[e] = fmaxf(m[e], (!kMasked || kbase + i + e < limit) ? x : -INFINITY);
    }
  }
  return fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
}

// p = 2^(s * scale - m_ref) for one row of a tile -> bf16 -> shared memory (K-major, 128-byte swizzle: 16-byte chunk
// index ^ (row % 8)); returns the row sum.
template <bool kMasked>
__device__ __forceinline__ float umma_probs_to_smem(const uint32_t (&v)[kUN], int kbase, int limit, float scale_log2, float m_ref,
                                                    uint8_t* p_row, int r) {
  float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c = 0; c < kUN; c += 8) {
    uint32_t pk[4];
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      float p0 = ex2_approx(fmaf(__uint_as_float(v[c + i]), scale_log2, -m_ref));
      float p1 = ex2_approx(fmaf(__uint_as_float(v[c + i + 1]), scale_log2, -m_ref));
      if (kMasked) {
        p0 = kbase + c + i < limit ? p0 : 0.f;
        p1 = kbase + c + i + 1 < limit ? p1 : 0.f;
      }
      ps[i >> 1] += p0 + p1;
      pk[i >> 1] = pack_bf16x2(p0, p1);
    }
    const int chunk = (c & 63) >> 3;                   // 16-byte chunk (8 keys) within the 64-key half
    *reinterpret_cast<uint4*>(p_row + (c >> 6) * kUHalf + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  }
  return (ps[0] + ps[1]) + (ps[2] + ps[3]);
}

// tm_q: 2-D view [T, nq * 128] of q, box 128 rows x 64 cols.  tm_k / tm_v: 2-D view [blocks * nkv * block_size, 128]
// of a cache, box 128 rows x 64 cols.
__global__ void __launch_bounds__(kUThreads, 1) prefill_attn_umma_kernel(
    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
    const int* __restrict__ cu_seqlens_q, const int* __restrict__ context_lens, const int* __restrict__ block_tables,
    __nv_bfloat16* __restrict__ out, int nq, int nkv, int block_size, int table_width, int num_blocks, float scale_log2,
    unsigned* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kUTile;                        // [2 stages]
  uint8_t* sV = sK + kUStages * kUTile;             // [2 stages]
  uint8_t* sP = sV + kUStages * kUTile;             // [2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kUTile);
  uint64_t* q_full = bars;                          // 1
  uint64_t* k_full = bars + 1;                      // [2]
  uint64_t* k_empty = bars + 3;                     // [2]
  uint64_t* v_full = bars + 5;                      // [2]
  uint64_t* v_empty = bars + 7;                     // [2]
  uint64_t* s_full = bars + 9;                      // [2]
  uint64_t* s_empty = bars + 11;                    // [2], one arrival per softmax warp
  uint64_t* p_full = bars + 13;                     // [2], one arrival per softmax warp
  uint64_t* pv_done = bars + 15;                    // [2]: P V of the tiles that used P buffer b is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);

  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y;
  const int q_begin = cu_seqlens_q[seq], q_len = cu_seqlens_q[seq + 1] - q_begin;
  const int k_len = context_lens[seq];
  const int m_tile = gridDim.x - 1 - blockIdx.x;        // heavy (late) tiles are scheduled first
  const int m0 = m_tile * kUM;
  if (m0 >= q_len) return;                              // uniform for the CTA, before anything is allocated
  const int kvh = h / (nq / nkv);
  const int past = k_len - q_len;                       // cached prefix length
  const int kv_end = min(k_len, past + m0 + kUM);       // keys visible to the last row of this tile
  const int n_tiles = (kv_end + kUN - 1) / kUN;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < kUStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);
      mbar_init(&p_full[s], 4);
      mbar_init(&pv_done[s], 1);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);                         // S0 | S1 | O | (unused): 3 x 128 columns
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, kUTile);
      tma_load_2d(sQ, &tm_q, q_full, h * kUD, q_begin + m0);
      tma_load_2d(sQ + kUHalf, &tm_q, q_full, h * kUD + 64, q_begin + m0);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kUStages;
        const uint32_t ph = (j / kUStages) & 1;
        const int tok = j * kUN;
        int blk = block_tables[static_cast<size_t>(seq) * table_width + min(tok / block_size, table_width - 1)];
        if (blk < 0 || blk >= num_blocks) {
          set_status(status, kStatusBadIndex);
          blk = 0;
        }
        const int row = (blk * nkv + kvh) * block_size + (tok % block_size);
        if (!mbar_wait_parked(&k_empty[s], ph ^ 1, status)) break;
        mbar_expect_tx(&k_full[s], kUTile);
        tma_load_2d(sK + s * kUTile, &tm_k, &k_full[s], 0, row);
        tma_load_2d(sK + s * kUTile + kUHalf, &tm_k, &k_full[s], 64, row);
        if (!mbar_wait_parked(&v_empty[s], ph ^ 1, status)) break;
        mbar_expect_tx(&v_full[s], kUTile);
        tma_load_2d(sV + s * kUTile, &tm_v, &v_full[s], 0, row);
        tma_load_2d(sV + s * kUTile + kUHalf, &tm_v, &v_full[s], 64, row);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(kUM, kUN, 1, 1);                  // both operands K-major
      constexpr uint32_t idesc_o = umma_idesc(kUM, kUD, 1, 1) | (1u << 16);     // B (= V) MN-major
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, status);
      auto issue_s = [&](int j) -> bool {
        const int s = j % kUStages;
        const uint32_t ph = (j / kUStages) & 1;
        if (!mbar_wait_parked(&k_full[s], ph, status)) return false;
        if (!mbar_wait_parked(&s_empty[j & 1], ((j >> 1) & 1) ^ 1, status)) return false;     // softmax has read S of tile j - 2
        tcgen05_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * kUTile);
#pragma unroll
        for (int k = 0; k < kUD / 16; ++k) {
          const uint32_t off = (k >> 2) * kUHalf + (k & 3) * 32;                       // 16 elements = 32 bytes inside a 64-element half
          umma_f16(tmem_base + (j & 1) * kUN, umma_desc_k_sw128(q_addr + off), umma_desc_k_sw128(k_addr + off), idesc_s, k != 0);
        }
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[s]);
        return true;
      };
      ok = ok && issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j % kUStages;
        const uint32_t ph = (j / kUStages) & 1;
        if (!mbar_wait_parked(&v_full[s], ph, status) || !mbar_wait_parked(&p_full[j & 1], (j >> 1) & 1, status)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * kUTile);
        const uint32_t pj_addr = p_addr + (j & 1) * kUTile;
#pragma unroll
        for (int k = 0; k < kUN / 16; ++k) {                                           // 16 keys per instruction
          const uint32_t a_off = (k >> 2) * kUHalf + (k & 3) * 32;                     // P: K-major, K = keys
          const uint32_t b_off = k * 16 * 128;                                         // V: 16 key rows of 128 bytes
          umma_f16(tmem_o, umma_desc_k_sw128(pj_addr + a_off), umma_desc_mn_sw128(v_addr + b_off, kUHalf), idesc_o, (j | k) != 0);
        }
        umma_commit(&pv_done[j & 1]);
        umma_commit(&v_empty[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = query row
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                      // row of the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int qpos = past + m0 + r;                      // keys <= qpos are visible
    const int limit = min(qpos + 1, k_len);              // visible keys: [0, limit)
    float m_ref = 0.f, l_run = 0.f;                     // reference maximum of the exponentials (scaled, log2 domain), row sum
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, status);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t s_addr = tmem_base + lane_addr + (j & 1) * kUN;
      const int kbase = j * kUN;
      uint32_t v[kUN];
#pragma unroll
      for (int c = 0; c < kUN; c += 32) tmem_ld_x32(s_addr + c, v + c);
      tmem_ld_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[j & 1]);       // the scores are in registers: S may be overwritten (tile j + 2)
      // tiles left of the diagonal and inside the sequence need no mask (warp-uniform choice)
      const bool masked = !__all_sync(0xffffffffu, kbase + kUN <= limit);
      float mt = masked ? umma_row_max<true>(v, kbase, limit) : umma_row_max<false>(v, kbase, limit);
      mt *= scale_log2;                                  // scale > 0: max commutes with the scaling
      if (j == 0) {
        m_ref = mt == -INFINITY ? 0.f : mt;              // O is not valid yet: nothing to rescale
      } else {
        const bool grow = mt - m_ref > 8.f;
        if (__any_sync(0xffffffffu, grow)) {             // tcgen05.ld / .st are warp-wide: the whole warp rescales
          ok = mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, status);            // every earlier P V has landed in O
          if (!ok) break;
          tcgen05_fence_after();
          const float m_new = fmaxf(m_ref, mt);
          const float alpha = exp2f(m_ref - m_new);      // 1 for rows whose maximum did not move
#pragma unroll 1
          for (int c = 0; c < kUD; c += 32) {
            uint32_t o[32];
            tmem_ld_x32(tmem_o + lane_addr + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(tmem_o + lane_addr + c, o);
          }
          tmem_st_wait();
          tcgen05_fence_before();
          l_run *= alpha;
          m_ref = m_new;
        }
      }
      // P buffer j & 1 was last read by P V of tile j - 2
      if (j >= 2) {
        ok = mbar_wait(&pv_done[j & 1], ((j >> 1) - 1) & 1, status);
        if (!ok) break;
      }
      uint8_t* p_row = sP + (j & 1) * kUTile + r * 128;
      const float ps = masked ? umma_probs_to_smem<true>(v, kbase, limit, scale_log2, m_ref, p_row, r)
                              : umma_probs_to_smem<false>(v, kbase, limit, scale_log2, m_ref, p_row, r);
      l_run += ps;
      fence_proxy_async_smem();                          // generic-proxy writes of P -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[j & 1]);
    }
    // all of O: wait for the last P V, normalise, store
    if (ok) ok = mbar_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, status);
    if (ok) {
      tcgen05_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const bool store = m0 + r < q_len;
      __nv_bfloat16* dst = out + static_cast<size_t>(q_begin + m0 + r) * nq * kUD + h * kUD;
#pragma unroll 1
      for (int c = 0; c < kUD; c += 32) {
        uint32_t o[32];
        tmem_ld_x32(tmem_o + lane_addr + c, o);
        tmem_ld_wait();
        if (store) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 pk;
            pk.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            pk.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            pk.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            pk.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c + i) = pk;
          }
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

extern "C" int forge_make_tmap_2d(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                                  uint32_t box_rows, int elem_bytes);

// Same operands as forge_prefill_attention; needs block_size >= 128 (a 128-key tile must lie inside one cache block).
extern "C" int forge_prefill_attention_umma(const void* q, const void* kc, const void* vc, const int* cu_q, const int* lens,
                                            const int* bt, void* out, int T, int num_seqs, int max_q, int nq, int nkv, int head_dim,
                                            int block_size, int table_width, int num_blocks, float scale, unsigned* status,
                                            cudaStream_t stream) {
  if (T <= 0 || num_seqs <= 0) return 0;
  if (head_dim != kUD || nq % nkv != 0 || block_size < kUN || (block_size & (block_size - 1))) return -1;
  CUtensorMap tm_q, tm_k, tm_v;
  if (forge_make_tmap_2d(&tm_q, q, T, static_cast<uint64_t>(nq) * kUD, static_cast<uint64_t>(nq) * kUD, kUM, 2) != 0) return -2;
  const uint64_t rows = static_cast<uint64_t>(num_blocks) * nkv * block_size;
  if (forge_make_tmap_2d(&tm_k, kc, rows, kUD, kUD, kUN, 2) != 0) return -2;
  if (forge_make_tmap_2d(&tm_v, vc, rows, kUD, kUD, kUN, 2) != 0) return -2;
  constexpr int smem = (1 + 2 * kUStages + 2) * kUTile + 256 + 1024;
  FORGE_ENSURE_DYN_SMEM(prefill_attn_umma_kernel, smem);
  dim3 grid((max_q + kUM - 1) / kUM, nq, num_seqs);
  return launch_kernel(prefill_attn_umma_kernel, grid, dim3(kUThreads), smem, stream, 0, tm_q, tm_k, tm_v, cu_q, lens, bt,
                       static_cast<__nv_bfloat16*>(out), nq, nkv, block_size, table_width, num_blocks,
                       scale * 1.4426950408889634f, status) == cudaSuccess ? 0 : -5;
}

}  // namespace forge

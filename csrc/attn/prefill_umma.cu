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
// shuffles.  S is double-buffered in tensor memory and S of tile j+1 is issued before P V of tile j, so the tensor
// pipe computes the next scores while the softmax warps work on the current ones.  The running output stays in
// registers (128 fp32 per thread) and is rescaled there; each tile's P V product is a fresh accumulator that the
// softmax warps read back and add, which keeps tensor memory free of read-modify-write rescaling.
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
  uint8_t* sP = sV + kUStages * kUTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kUTile);
  uint64_t* q_full = bars;                          // 1
  uint64_t* k_full = bars + 1;                      // [2]
  uint64_t* k_empty = bars + 3;                     // [2]
  uint64_t* v_full = bars + 5;                      // [2]
  uint64_t* v_empty = bars + 7;                     // [2]
  uint64_t* s_full = bars + 9;                      // [2]
  uint64_t* s_empty = bars + 11;                    // [2], one arrival per softmax warp
  uint64_t* p_full = bars + 13;                     // one arrival per softmax warp
  uint64_t* o_full = bars + 14;
  uint64_t* o_empty = bars + 15;                    // one arrival per softmax warp
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

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
    }
    mbar_init(p_full, 4);
    mbar_init(o_full, 1);
    mbar_init(o_empty, 4);
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
        if (!mbar_wait(&k_empty[s], ph ^ 1, status)) break;
        mbar_expect_tx(&k_full[s], kUTile);
        tma_load_2d(sK + s * kUTile, &tm_k, &k_full[s], 0, row);
        tma_load_2d(sK + s * kUTile + kUHalf, &tm_k, &k_full[s], 64, row);
        if (!mbar_wait(&v_empty[s], ph ^ 1, status)) break;
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
        if (!mbar_wait(&k_full[s], ph, status)) return false;
        if (!mbar_wait(&s_empty[j & 1], ((j >> 1) & 1) ^ 1, status)) return false;     // softmax has read S of tile j - 2
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
        if (!mbar_wait(&v_full[s], ph, status) || !mbar_wait(p_full, j & 1, status) || !mbar_wait(o_empty, (j & 1) ^ 1, status)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * kUTile);
#pragma unroll
        for (int k = 0; k < kUN / 16; ++k) {                                           // 16 keys per instruction
          const uint32_t a_off = (k >> 2) * kUHalf + (k & 3) * 32;                     // P: K-major, K = keys
          const uint32_t b_off = k * 16 * 128;                                         // V: 16 key rows of 128 bytes
          umma_f16(tmem_o, umma_desc_k_sw128(p_addr + a_off), umma_desc_mn_sw128(v_addr + b_off, kUHalf), idesc_o, k != 0);
        }
        umma_commit(o_full);
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
    float o_acc[kUD];
#pragma unroll
    for (int i = 0; i < kUD; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, status);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t s_addr = tmem_base + lane_addr + (j & 1) * kUN;
      const int kbase = j * kUN;
      // pass 1: row maximum of the visible scores
      float mt = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kUN; c += 32) {
        uint32_t v[32];
        tmem_ld_x32(s_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (kbase + c + i < limit) mt = fmaxf(mt, __uint_as_float(v[i]));
      }
      mt *= scale_log2;                                  // scale > 0: max commutes with the scaling
      const float m_new = fmaxf(m_run, mt);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);
      m_run = m_new;
      // pass 2: probabilities -> bf16 -> shared memory (K-major, 128-byte swizzle: 16-byte chunk index ^ (row % 8))
      float ps = 0.f;
#pragma unroll 1
      for (int c = 0; c < kUN; c += 32) {
        uint32_t v[32];
        tmem_ld_x32(s_addr + c, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = kbase + c + i < limit ? exp2f(__uint_as_float(v[i]) * scale_log2 - m_use) : 0.f;
          const float p1 = kbase + c + i + 1 < limit ? exp2f(__uint_as_float(v[i + 1]) * scale_log2 - m_use) : 0.f;
          ps += p0 + p1;
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        uint8_t* base = sP + (c >> 6) * kUHalf + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = ((c & 63) >> 3) + q4;        // 16-byte chunk (8 keys) within the 64-key half
          *reinterpret_cast<uint4*>(base + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
        }
      }
      l_run = l_run * alpha + ps;
      // S buffer may be overwritten (tile j + 2); P is complete
      tcgen05_fence_before();
      fence_proxy_async_smem();                          // generic-proxy writes of P -> visible to the tensor core
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[j & 1]);
        mbar_arrive(p_full);
      }
      // O = alpha * O + P V
      ok = mbar_wait(o_full, j & 1, status);
      if (!ok) break;
      tcgen05_fence_after();
#pragma unroll
      for (int c = 0; c < kUD; c += 32) {
        uint32_t v[32];
        tmem_ld_x32(tmem_o + lane_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[c + i] = fmaf(o_acc[c + i], alpha, __uint_as_float(v[i]));
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_empty);               // the next P V may overwrite O; P may be rewritten (ordered by o_full)
    }
    if (ok && m0 + r < q_len) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = out + static_cast<size_t>(q_begin + m0 + r) * nq * kUD + h * kUD;
#pragma unroll
      for (int c = 0; c < kUD; c += 8) {
        uint4 pk;
        pk.x = pack_bf16x2(o_acc[c] * inv, o_acc[c + 1] * inv);
        pk.y = pack_bf16x2(o_acc[c + 2] * inv, o_acc[c + 3] * inv);
        pk.z = pack_bf16x2(o_acc[c + 4] * inv, o_acc[c + 5] * inv);
        pk.w = pack_bf16x2(o_acc[c + 6] * inv, o_acc[c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c) = pk;
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
  constexpr int smem = (1 + 2 * kUStages + 1) * kUTile + 256 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(prefill_attn_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    attr_set = true;
  }
  dim3 grid((max_q + kUM - 1) / kUM, nq, num_seqs);
  return launch_kernel(prefill_attn_umma_kernel, grid, dim3(kUThreads), smem, stream, 0, tm_q, tm_k, tm_v, cu_q, lens, bt,
                       static_cast<__nv_bfloat16*>(out), nq, nkv, block_size, table_width, num_blocks,
                       scale * 1.4426950408889634f, status) == cudaSuccess ? 0 : -5;
}

}  // namespace forge

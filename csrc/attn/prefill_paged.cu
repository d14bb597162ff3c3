// Prefill attention: variable-length, causal, GQA, keys and values read from the paged cache (so a cached
// prefix and the freshly written tokens are one code path; the reference switches between the contiguous
// k/v and the paged cache: tinyvllm/layers/attention.py:99-105, flash_attn_varlen_func).
//
// The query rows of a sequence are its LAST q_len positions; with a cached prefix (q_len < k_len) the causal
// mask is aligned to the bottom-right corner: query row i sees keys 0 .. (k_len - q_len + i).
//
// CTA = 64 query rows of one (sequence, q head), four warps of 16 rows.  K and V tiles of 64 keys come in by
// TMA with the 128-byte swizzle (two boxes of 64 x 64 per tile, one per half of head_dim) through a two-stage
// ring, so shared-memory reads by ldmatrix are conflict-free.  This version multiplies with mma.sync
// m16n8k16 (fp32 accumulate, online softmax in registers); it serves cache blocks smaller than 128 tokens.
// Blocks of >= 128 tokens go to the tcgen05 kernel in prefill_umma.cu.
#include <cstdlib>
#include <string>

#include "../include/launch.cuh"
#include "../include/ptx.cuh"

namespace forge {

constexpr int kPD = 128;          // head_dim
constexpr int kPM = 64;           // query rows per CTA
constexpr int kPN = 64;           // keys per tile
constexpr int kPHalfBytes = 64 * 128;   // one swizzled 64-row x 64-col bf16 box

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte offset of element (row, d) in a tile stored as two swizzled halves (d < 64 | d >= 64), d a multiple of 8.
__device__ __forceinline__ uint32_t swz(int row, int d) {
  return static_cast<uint32_t>((d >> 6) * kPHalfBytes + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4));
}

// tm_q: 2-D view [T, nq * 128] of q, box 64 rows x 64 cols.  tm_k / tm_v: 2-D view [blocks * nkv * block_size, 128]
// of a cache, box box_rows x 64 cols with box_rows = min(block_size, 64).
__global__ void __launch_bounds__(128) prefill_attn_kernel(
    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
    const int* __restrict__ cu_seqlens_q, const int* __restrict__ context_lens, const int* __restrict__ block_tables,
    __nv_bfloat16* __restrict__ out, int nq, int nkv, int block_size, int table_width, int num_blocks, float scale_log2,
    unsigned* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                   // 16 KB
  uint8_t* sKV = smem + 2 * kPHalfBytes;                // 2 stages x (K 16 KB + V 16 KB)
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(sKV + 2 * 4 * kPHalfBytes);
  uint64_t* bar_kv = bar_q + 1;                         // [2]

  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y;
  const int q_begin = cu_seqlens_q[seq], q_len = cu_seqlens_q[seq + 1] - q_begin;
  const int k_len = context_lens[seq];
  const int m_tile = gridDim.x - 1 - blockIdx.x;        // heavy (late) tiles are scheduled first
  const int m0 = m_tile * kPM;
  if (m0 >= q_len) return;
  const int kvh = h / (nq / nkv);
  const int past = k_len - q_len;                       // cached prefix length
  const int kv_end = min(k_len, past + m0 + kPM);       // keys visible to the last row of this tile
  const int n_tiles = (kv_end + kPN - 1) / kPN;
  const int box_rows = block_size < kPN ? block_size : kPN;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    mbar_init(bar_q, 1);
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    fence_mbar_init();
  }
  __syncthreads();

  auto issue_kv = [&](int t) {
    uint8_t* st = sKV + (t & 1) * 4 * kPHalfBytes;
    mbar_expect_tx(&bar_kv[t & 1], 4 * kPHalfBytes);
    for (int r = 0; r < kPN; r += box_rows) {
      const int tok = t * kPN + r;
      int blk = block_tables[static_cast<size_t>(seq) * table_width + min(tok / block_size, table_width - 1)];
      if (blk < 0 || blk >= num_blocks) {               // beyond the sequence: any valid block will do, rows are masked
        if (tok < k_len) set_status(status, kStatusBadIndex);
        blk = 0;
      }
      const int row = (blk * nkv + kvh) * block_size + (tok % block_size);
      for (int half = 0; half < 2; ++half) {
        tma_load_2d(st + half * kPHalfBytes + r * 128, &tm_k, &bar_kv[t & 1], half * 64, row);
        tma_load_2d(st + 2 * kPHalfBytes + half * kPHalfBytes + r * 128, &tm_v, &bar_kv[t & 1], half * 64, row);
      }
    }
  };

  if (threadIdx.x == 0) {
    mbar_expect_tx(bar_q, 2 * kPHalfBytes);
    tma_load_2d(sQ, &tm_q, bar_q, h * kPD, q_begin + m0);
    tma_load_2d(sQ + kPHalfBytes, &tm_q, bar_q, h * kPD + 64, q_begin + m0);
    issue_kv(0);
  }

  // Q fragments: 16 rows x 128 d per warp = 8 k-steps x 4 registers
  uint32_t qf[8][4];
  bool ok = mbar_wait(bar_q, 0, status);
  {
    const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int d = ks * 16 + (lane >> 4) * 8;
      ldmatrix_x4(smem_u32(sQ) + swz(row, d), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int g = lane >> 2, tq = lane & 3;
  const int qpos0 = past + m0 + warp * 16 + g;          // key positions visible to rows g and g + 8: <= qpos
  const int qpos1 = qpos0 + 8;

  ok = __syncthreads_and(ok);                           // waits are bounded; keep the outcome uniform
  for (int t = 0; t < n_tiles && ok; ++t) {
    if (threadIdx.x == 0 && t + 1 < n_tiles) issue_kv(t + 1);
    if (!mbar_wait(&bar_kv[t & 1], (t >> 1) & 1, status)) {
      ok = __syncthreads_and(false);
      break;
    }
    const uint32_t sK = smem_u32(sKV + (t & 1) * 4 * kPHalfBytes);
    const uint32_t sV = sK + 2 * kPHalfBytes;

    // S = Q K^T : 8 key blocks of 8
    float s[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
      for (int nb = 0; nb < 8; nb += 2) {
        uint32_t b0, b1, b2, b3;
        const int krow = nb * 8 + (lane & 7) + (lane >> 4) * 8;
        const int d = ks * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(sK + swz(krow, d), b0, b1, b2, b3);
        mma_bf16_16816(s[nb], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
        mma_bf16_16816(s[nb + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
      }
    }
    // scale, mask, online softmax (rows g and g + 8 of this warp)
    const int kbase = t * kPN + 2 * tq;
    float mt0 = -INFINITY, mt1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int kp = kbase + nb * 8 + e;
        s[nb][e] = (kp <= qpos0 && kp < k_len) ? s[nb][e] * scale_log2 : -INFINITY;
        s[nb][2 + e] = (kp <= qpos1 && kp < k_len) ? s[nb][2 + e] * scale_log2 : -INFINITY;
        mt0 = fmaxf(mt0, s[nb][e]);
        mt1 = fmaxf(mt1, s[nb][2 + e]);
      }
    }
    mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 1));
    mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 2));
    mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 1));
    mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 2));
    const float mn0 = fmaxf(m_run[0], mt0), mn1 = fmaxf(m_run[1], mt1);
    const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
    const float a0 = exp2f(m_run[0] - mu0), a1 = exp2f(m_run[1] - mu1);
    m_run[0] = mn0;
    m_run[1] = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      s[nb][0] = exp2f(s[nb][0] - mu0);
      s[nb][1] = exp2f(s[nb][1] - mu0);
      s[nb][2] = exp2f(s[nb][2] - mu1);
      s[nb][3] = exp2f(s[nb][3] - mu1);
      ps0 += s[nb][0] + s[nb][1];
      ps1 += s[nb][2] + s[nb][3];
    }
    l_run[0] = l_run[0] * a0 + ps0;     // per-thread partial row sums; reduced over the quad at the end
    l_run[1] = l_run[1] * a1 + ps1;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= a0;
      o[i][1] *= a0;
      o[i][2] *= a1;
      o[i][3] *= a1;
    }
    // O += P V : 4 key steps of 16, 16 d blocks of 8
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t pa0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t pa1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t pa2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t pa3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int nd = 0; nd < 16; nd += 2) {
        uint32_t b0, b1, b2, b3;
        const int vrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int d = (nd + (lane >> 4)) * 8;
        ldmatrix_x4_trans(sV + swz(vrow, d), b0, b1, b2, b3);
        mma_bf16_16816(o[nd], pa0, pa1, pa2, pa3, b0, b1);
        mma_bf16_16816(o[nd + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
    }
    ok = __syncthreads_and(true);   // everyone is done with this stage before it is refilled two tiles later
  }

  // finish: row sums over the quad, normalise, store
  l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
  l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
  l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
  l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
  const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  const int r0 = m0 + warp * 16 + g, r1 = r0 + 8;
  const size_t ld = static_cast<size_t>(nq) * kPD;
#pragma unroll
  for (int nd = 0; nd < 16; ++nd) {
    const int d = nd * 8 + 2 * tq;
    if (r0 < q_len)
      *reinterpret_cast<uint32_t*>(out + (q_begin + r0) * ld + h * kPD + d) = pack_bf16x2(o[nd][0] * inv0, o[nd][1] * inv0);
    if (r1 < q_len)
      *reinterpret_cast<uint32_t*>(out + (q_begin + r1) * ld + h * kPD + d) = pack_bf16x2(o[nd][2] * inv1, o[nd][3] * inv1);
  }
}

extern "C" int forge_make_tmap_2d(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                                  uint32_t box_rows, int elem_bytes);
extern "C" int forge_prefill_attention_umma(const void* q, const void* kc, const void* vc, const int* cu_q, const int* lens,
                                            const int* bt, void* out, int T, int num_seqs, int max_q, int nq, int nkv, int head_dim,
                                            int block_size, int table_width, int num_blocks, float scale, unsigned* status,
                                            cudaStream_t stream);

// q [T, nq, 128] bf16 (contiguous); caches [num_blocks, nkv, block_size, 128]; out [T, nq * 128].
extern "C" int forge_prefill_attention(const void* q, const void* kc, const void* vc, const int* cu_q, const int* lens,
                                       const int* bt, void* out, int T, int num_seqs, int max_q, int nq, int nkv, int head_dim,
                                       int block_size, int table_width, int num_blocks, float scale, unsigned* status,
                                       cudaStream_t stream) {
  if (T <= 0 || num_seqs <= 0) return 0;
  if (head_dim != kPD || nq % nkv != 0 || block_size < 16 || (block_size & (block_size - 1))) return -1;
  // cache blocks of >= 128 tokens (the engine's default is 256): the tcgen05 kernel; FORGE_PREFILL_ATTN=mma keeps this one
  static const bool force_mma = std::getenv("FORGE_PREFILL_ATTN") != nullptr && std::string(std::getenv("FORGE_PREFILL_ATTN")) == "mma";
  if (block_size >= 128 && !force_mma)
    return forge_prefill_attention_umma(q, kc, vc, cu_q, lens, bt, out, T, num_seqs, max_q, nq, nkv, head_dim, block_size, table_width,
                                        num_blocks, scale, status, stream);
  const uint32_t box_rows = block_size < kPN ? block_size : kPN;
  CUtensorMap tm_q, tm_k, tm_v;
  if (forge_make_tmap_2d(&tm_q, q, T, static_cast<uint64_t>(nq) * kPD, static_cast<uint64_t>(nq) * kPD, kPM, 2) != 0) return -2;
  const uint64_t rows = static_cast<uint64_t>(num_blocks) * nkv * block_size;
  if (forge_make_tmap_2d(&tm_k, kc, rows, kPD, kPD, box_rows, 2) != 0) return -2;
  if (forge_make_tmap_2d(&tm_v, vc, rows, kPD, kPD, box_rows, 2) != 0) return -2;
  constexpr int smem = 2 * kPHalfBytes + 2 * 4 * kPHalfBytes + 64 + 1024;
  FORGE_ENSURE_DYN_SMEM(prefill_attn_kernel, smem);
  dim3 grid((max_q + kPM - 1) / kPM, nq, num_seqs);
  return launch_kernel(prefill_attn_kernel, grid, dim3(128), smem, stream, 0, tm_q, tm_k, tm_v, cu_q, lens, bt,
                       static_cast<__nv_bfloat16*>(out), nq, nkv, block_size, table_width, num_blocks,
                       scale * 1.4426950408889634f, status) == cudaSuccess ? 0 : -5;
}

}  // namespace forge

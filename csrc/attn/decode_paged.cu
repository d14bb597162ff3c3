// Decode attention over the paged KV cache: one query token per sequence, GQA, split along the context.
//
// The reference calls flash-attn's flash_attn_with_kvcache (tinyvllm/layers/attention.py:108-109).
// This step is bound by HBM bandwidth: every cached K and V byte of every running sequence is read
// once per layer.  The kernel is therefore organised around the copy engine:
//
//   * the cache layout is [blocks, kv_heads, block_size, 128], so the K (or V) rows of TILE consecutive
//     tokens of one head are ONE contiguous run; a producer warp streams them into shared memory with
//     untiled bulk copies (cp.async.bulk) through a 3-stage mbarrier ring;
//   * four consumer warps each own a quarter of every tile and keep their own online-softmax state,
//     so the main loop has no CTA-wide barrier; the q heads that share a KV head are processed together
//     (each K/V byte is read from shared memory once per group);
//   * the context is cut into fixed-size chunks (grid.z); each CTA writes either the final output (one
//     chunk) or a normalised partial plus (max, sum) that a small second kernel merges.  Lengths are read
//     on the device, so the launch is CUDA-graph safe: the grid depends only on the batch bucket.
//
// head_dim is 128 (all Qwen3 sizes).  Scores use exp2 with the scale folded into q.
#include "../include/launch.cuh"
#include "../include/ptx.cuh"

namespace forge {

constexpr int kD = 128;
constexpr int kDecStages = 3;
constexpr int kDecThreads = 160;   // 4 consumer warps + 1 producer warp

template <int G, int TILE>
__global__ void __launch_bounds__(kDecThreads) decode_attn_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
    const int* __restrict__ block_tables, const int* __restrict__ context_lens, __nv_bfloat16* __restrict__ out,
    float* __restrict__ part_o, float* __restrict__ part_ml, int nq, int nkv, int block_size, int table_width, int num_blocks,
    int chunk, int max_chunks, float scale_log2, unsigned* status) {
  constexpr int TPW = TILE / 4;          // tokens per consumer warp per tile
  constexpr int ITERS = TPW / 4;         // QK iterations (4 tokens per warp at a time)
  constexpr int kTileBytes = TILE * kD * 2;
  static_assert(TILE >= 16 && TILE <= 64 && (TILE & (TILE - 1)) == 0, "tile");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kDecStages * 2 * kTileBytes);
  uint64_t* empty_bar = full_bar + kDecStages;

  pdl_launch_dependents();
  pdl_wait();                                           // q, the new K/V entries and the step buffer come from predecessors
  const int groups_per_kv = (nq / nkv) / G;             // > 1 when the GQA group is processed in slices of G
  const int kvh = blockIdx.x / groups_per_kv;
  const int qh0 = kvh * (nq / nkv) + (blockIdx.x % groups_per_kv) * G;
  const int b = blockIdx.y;
  const int c = blockIdx.z;
  const int len = context_lens[b];
  const int tok_begin = c * chunk;
  if (tok_begin >= len) {                                // uniform for the CTA
    if (c == 0 && threadIdx.x < kD)                      // padding row (length 0): defined output
      for (int g = 0; g < G; ++g) out[(static_cast<size_t>(b) * nq + qh0 + g) * kD + threadIdx.x] = __float2bfloat16_rn(0.f);
    return;
  }
  const int tok_end = min(len, tok_begin + chunk);
  const int n_tiles = (tok_end - tok_begin + TILE - 1) / TILE;
  const int n_chunks = (len + chunk - 1) / chunk;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);
    }
    fence_mbar_init();
  }
  __syncthreads();

  float m_run[G], l_run[G], acc[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[g][e] = 0.f;
  }

  if (warp == 4) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % kDecStages;
        const uint32_t ph = (t / kDecStages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, status)) break;
        const int tok0 = tok_begin + t * TILE;
        int blk = block_tables[static_cast<size_t>(b) * table_width + tok0 / block_size];
        if (blk < 0 || blk >= num_blocks) {
          set_status(status, kStatusBadIndex);
          blk = 0;
        }
        const size_t off = ((static_cast<size_t>(blk) * nkv + kvh) * block_size + (tok0 % block_size)) * kD;
        uint8_t* st = smem + s * 2 * kTileBytes;
        mbar_expect_tx(&full_bar[s], 2 * kTileBytes);
        bulk_load(st, k_cache + off, kTileBytes, &full_bar[s]);
        bulk_load(st + kTileBytes, v_cache + off, kTileBytes, &full_bar[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int grp = lane >> 3, j = lane & 7;
    // q slices this lane multiplies: elements [8j, 8j+8) and [64+8j, 64+8j+8) of every head of the group
    float qr[G][16];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const __nv_bfloat16* qp = q + (static_cast<size_t>(b) * nq + qh0 + g) * kD;
      const uint4 lo = *reinterpret_cast<const uint4*>(qp + 8 * j);
      const uint4 hi = *reinterpret_cast<const uint4*>(qp + 64 + 8 * j);
      const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        qr[g][2 * e] = bf16_lo(w[e]) * scale_log2;
        qr[g][2 * e + 1] = bf16_hi(w[e]) * scale_log2;
      }
    }
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int s = t % kDecStages;
      const uint32_t ph = (t / kDecStages) & 1;
      ok = mbar_wait(&full_bar[s], ph, status);
      if (!ok) break;
      const uint8_t* Ks = smem + s * 2 * kTileBytes;
      const uint8_t* Vs = Ks + kTileBytes;
      const int tok0 = tok_begin + t * TILE;

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
        const bool valid = tok0 + r < tok_end;
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
      float alpha[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float mt = sc[0][g];
#pragma unroll
        for (int it = 1; it < ITERS; ++it) mt = fmaxf(mt, sc[it][g]);
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 8));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
        const float m_new = fmaxf(m_run[g], mt);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;      // every token masked so far
        alpha[g] = exp2f(m_run[g] - m_use);                        // exp2(-inf) = 0 on the first tile
        float ps = 0.f;
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
          sc[it][g] = exp2f(sc[it][g] - m_use);                    // masked -> 0
          ps += sc[it][g];
        }
        l_run[g] = l_run[g] * alpha[g] + ps;                       // per token group; summed over groups at the end
        m_run[g] = m_new;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[g][e] *= alpha[g];
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
          acc[g][0] = fmaf(p, v0, acc[g][0]);
          acc[g][1] = fmaf(p, v1, acc[g][1]);
          acc[g][2] = fmaf(p, v2, acc[g][2]);
          acc[g][3] = fmaf(p, v3, acc[g][3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {   // each 8-lane group summed its own tokens: lanes 0, 8, 16, 24 hold the four partial sums
      l_run[g] += __shfl_xor_sync(0xffffffffu, l_run[g], 8);
      l_run[g] += __shfl_xor_sync(0xffffffffu, l_run[g], 16);
    }
  }

  // ------------------------------------------------------------------ merge the four warps (stage memory is free now)
  __syncthreads();
  float* s_acc = reinterpret_cast<float*>(smem);                 // [4][G][128]
  float* s_m = s_acc + 4 * G * kD;                               // [4][G]
  float* s_l = s_m + 4 * G;                                      // [4][G]
  if (warp < 4) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      *reinterpret_cast<float4*>(s_acc + (warp * G + g) * kD + lane * 4) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
      if (lane == 0) {
        s_m[warp * G + g] = m_run[g];
        s_l[warp * G + g] = l_run[g];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < kD) {
    const int d = threadIdx.x;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, s_m[w * G + g]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = s_m[w * G + g];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
        L += s_l[w * G + g] * f;
        O += s_acc[(w * G + g) * kD + d] * f;
      }
      const float o = L > 0.f ? O / L : 0.f;
      const int qh = qh0 + g;
      if (n_chunks == 1) {
        out[(static_cast<size_t>(b) * nq + qh) * kD + d] = __float2bfloat16_rn(o);
      } else {
        const size_t p = (static_cast<size_t>(b) * nq + qh) * max_chunks + c;
        part_o[p * kD + d] = o;
        if (d == 0) {
          part_ml[p * 2] = M;
          part_ml[p * 2 + 1] = L;
        }
      }
    }
  }
}

// Merge the per-chunk partials of sequences that span more than one chunk.
__global__ void __launch_bounds__(kD) decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                            const int* __restrict__ context_lens, __nv_bfloat16* __restrict__ out,
                                                            int nq, int chunk, int max_chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y, qh = blockIdx.x, d = threadIdx.x;
  const int len = context_lens[b];
  const int n = (len + chunk - 1) / chunk;
  if (n <= 1) return;
  const size_t base = (static_cast<size_t>(b) * nq + qh) * max_chunks;
  float M = -INFINITY;
  for (int c = 0; c < n; ++c) M = fmaxf(M, part_ml[(base + c) * 2]);
  float L = 0.f, O = 0.f;
  for (int c = 0; c < n; ++c) {
    const float w = part_ml[(base + c) * 2 + 1] * exp2f(part_ml[(base + c) * 2] - M);
    L += w;
    O += part_o[(base + c) * kD + d] * w;
  }
  out[(static_cast<size_t>(b) * nq + qh) * kD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
}

template <int G, int TILE>
static int launch_decode(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out, float* part_o,
                         float* part_ml, int B, int nq, int nkv, int block_size, int table_width, int num_blocks, int chunk,
                         int max_chunks, float scale_log2, unsigned* status, cudaStream_t stream) {
  constexpr int kTileBytes = TILE * kD * 2;
  constexpr int merge_bytes = (4 * G * kD + 8 * G) * 4;
  constexpr int ring = kDecStages * 2 * kTileBytes;
  constexpr int smem = (ring > merge_bytes ? ring : merge_bytes) + 2 * kDecStages * 8 + 128;
  auto kern = decode_attn_kernel<G, TILE>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    attr_set = true;
  }
  const int groups_per_kv = (nq / nkv) / G;
  dim3 grid(nkv * groups_per_kv, B, max_chunks);
  if (launch_kernel(kern, grid, dim3(kDecThreads), smem, stream, 0, static_cast<const __nv_bfloat16*>(q),
                    static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc), bt, lens,
                    static_cast<__nv_bfloat16*>(out), part_o, part_ml, nq, nkv, block_size, table_width, num_blocks, chunk,
                    max_chunks, scale_log2, status) != cudaSuccess)
    return -5;
  if (max_chunks > 1) {
    dim3 g2(nq, B);
    if (launch_kernel(decode_combine_kernel, g2, dim3(kD), 0, stream, 0, static_cast<const float*>(part_o),
                      static_cast<const float*>(part_ml), lens, static_cast<__nv_bfloat16*>(out), nq, chunk, max_chunks) != cudaSuccess)
      return -5;
  }
  return 0;
}

// q [B, nq, 128] bf16; caches [num_blocks, nkv, block_size, 128] bf16; block_tables [B, table_width]; out [B, nq * 128].
// part_o: fp32 [B, nq, max_chunks, 128], part_ml: fp32 [B, nq, max_chunks, 2] (may be null when max_chunks == 1).
// chunk: tokens per grid.z slice, a multiple of min(block_size, 64); max_chunks * chunk must cover the longest context.
extern "C" int forge_decode_attention(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out,
                                      float* part_o, float* part_ml, int B, int nq, int nkv, int head_dim, int block_size,
                                      int table_width, int num_blocks, int chunk, int max_chunks, float scale, unsigned* status,
                                      cudaStream_t stream) {
  if (B <= 0) return 0;
  if (head_dim != kD || nq % nkv != 0 || block_size < 16 || (block_size & (block_size - 1))) return -1;
  const int tile = block_size < 64 ? block_size : 64;
  if (chunk % tile != 0 || max_chunks < 1) return -1;
  if (max_chunks > 1 && (part_o == nullptr || part_ml == nullptr)) return -1;
  const int group = nq / nkv;
  const int G = group % 4 == 0 ? 4 : (group % 2 == 0 ? 2 : 1);
  const float sl2 = scale * 1.4426950408889634f;
#define FORGE_DEC(GG, TT)                                                                                                   \
  return launch_decode<GG, TT>(q, kc, vc, bt, lens, out, part_o, part_ml, B, nq, nkv, block_size, table_width, num_blocks, \
                               chunk, max_chunks, sl2, status, stream)
  if (tile == 64) {
    if (G == 4) FORGE_DEC(4, 64);
    if (G == 2) FORGE_DEC(2, 64);
    FORGE_DEC(1, 64);
  } else if (tile == 32) {
    if (G == 4) FORGE_DEC(4, 32);
    if (G == 2) FORGE_DEC(2, 32);
    FORGE_DEC(1, 32);
  } else {
    if (G == 4) FORGE_DEC(4, 16);
    if (G == 2) FORGE_DEC(2, 16);
    FORGE_DEC(1, 16);
  }
#undef FORGE_DEC
}


// =========================================================================================================
// Allocation-free entry point (declared in include/forge_noalloc.h; no counterpart in the reference).
//
// Who needs it: code that drives this kernel from a place where device memory cannot be requested -- a host
// callback or a plug-in running inside someone else's memory plan, a real-time loop that must not touch the
// allocator, or a process whose memory pool is sized up front and then frozen.  The regular entry point asks
// its caller for split-context scratch (per-chunk partial outputs plus their softmax max/sum); a caller that
// cannot allocate has nowhere to get it from.  Here that scratch is a fixed array that lives in the library's
// device image, so the caller passes only the operation's real inputs and outputs.
//
// Properties a caller must know:
//   * The array is kForgeNoAllocScratchFloats floats (16 MiB).  Every GPU that loads this library carries it
//     from module load until the process exits, whether or not this entry point is ever called.
//   * A problem needs B * nq * max_chunks * 130 floats.  Larger requests are refused with
//     FORGE_NOALLOC_TOO_LARGE before anything is launched; forge_decode_attention_noalloc_strerror() turns the
//     code into text.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//     device current) and remembers it.  Make that first call outside of any stream capture: the lookup is a
//     synchronous runtime query, not a stream operation.
//   * All calls on a device share the one array, and it keeps whatever the last call left in it.  Nothing in
//     it has to start at zero: every partial the merge kernel reads was written by the attention kernel of the
//     same call.  Two calls whose kernels overlap on the GPU (different streams, or a graph branch) race on it;
//     keep calls on one device ordered.
//   * No cudaMalloc, cudaFree, or allocating library routine is called on any path.
// =========================================================================================================
constexpr size_t kForgeNoAllocScratchFloats = static_cast<size_t>(4) << 20;

static __device__ __align__(256) float g_noalloc_scratch[kForgeNoAllocScratchFloats];

// The symbol above is a host-side handle, not a device pointer: handing `g_noalloc_scratch` itself to a kernel
// launch would pass a host address.  The device address is looked up once per device and cached here.
static float* g_noalloc_scratch_dev[64] = {};

enum ForgeNoAllocError {
  FORGE_NOALLOC_OK = 0,
  FORGE_NOALLOC_BAD_ARGUMENT = -1,
  FORGE_NOALLOC_TOO_LARGE = -20,
  FORGE_NOALLOC_SYMBOL_LOOKUP_FAILED = -21,
  FORGE_NOALLOC_LAUNCH_FAILED = -22,
};

extern "C" const char* forge_decode_attention_noalloc_strerror(int code) {
  switch (code) {
    case FORGE_NOALLOC_OK: return "ok";
    case FORGE_NOALLOC_BAD_ARGUMENT: return "bad argument: head_dim must be 128, block_size a power of two >= 16, chunk a multiple of min(block_size, 64)";
    case FORGE_NOALLOC_TOO_LARGE: return "B * nq * max_chunks * 130 floats exceed the built-in 16 MiB scratch array; use forge_decode_attention with caller-provided scratch";
    case FORGE_NOALLOC_SYMBOL_LOOKUP_FAILED: return "cudaGetSymbolAddress failed for the built-in scratch array on the current device";
    case FORGE_NOALLOC_LAUNCH_FAILED: return "kernel launch failed";
    default: return "unknown error";
  }
}

extern "C" size_t forge_decode_attention_noalloc_capacity_floats() { return kForgeNoAllocScratchFloats; }

extern "C" int forge_decode_attention_noalloc(const void* q, const void* kc, const void* vc, const int* bt, const int* lens,
                                              void* out, int B, int nq, int nkv, int head_dim, int block_size, int table_width,
                                              int num_blocks, int chunk, int max_chunks, float scale, unsigned* status,
                                              cudaStream_t stream) {
  if (B <= 0) return FORGE_NOALLOC_OK;
  if (nq <= 0 || nkv <= 0 || max_chunks < 1 || chunk < 1) return FORGE_NOALLOC_BAD_ARGUMENT;
  const size_t slots = static_cast<size_t>(B) * nq * max_chunks;
  if (slots * (kD + 2) > kForgeNoAllocScratchFloats) return FORGE_NOALLOC_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FORGE_NOALLOC_SYMBOL_LOOKUP_FAILED;
  if (g_noalloc_scratch_dev[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess || p == nullptr)
      return FORGE_NOALLOC_SYMBOL_LOOKUP_FAILED;
    g_noalloc_scratch_dev[dev] = p;
  }
  float* part_o = g_noalloc_scratch_dev[dev];
  float* part_ml = part_o + slots * kD;
  const int rc = forge_decode_attention(q, kc, vc, bt, lens, out, part_o, part_ml, B, nq, nkv, head_dim, block_size, table_width,
                                        num_blocks, chunk, max_chunks, scale, status, stream);
  if (rc == -1) return FORGE_NOALLOC_BAD_ARGUMENT;
  return rc == 0 ? FORGE_NOALLOC_OK : FORGE_NOALLOC_LAUNCH_FAILED;
}

}  // namespace forge

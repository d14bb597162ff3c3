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
#include <algorithm>
#include <cstdlib>

#include "../include/decode_common.cuh"
#include "../include/launch.cuh"
#include "../include/ptx.cuh"

namespace forge {

// A context length the block table (and the partial buffers) cannot describe is a corrupted input: it is clamped, so
// that every access derived from it stays inside the table and the scratch, and reported through the status word.
__device__ __forceinline__ int decode_checked_len(const int* __restrict__ context_lens, int b, int cap, unsigned* status) {
  const int len = context_lens[b];
  if (len > cap) {
    set_status(status, kStatusBadIndex);
    return cap;
  }
  return len < 0 ? 0 : len;
}

template <int G, int TILE>
__global__ void __launch_bounds__(kDecThreads, decode_ctas_per_sm(G)) decode_attn_kernel(
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
    const int* __restrict__ block_tables, const int* __restrict__ context_lens, __nv_bfloat16* __restrict__ out,
    float* __restrict__ part_o, float* __restrict__ part_ml, int nq, int nkv, int block_size, int table_width, int num_blocks,
    int chunk, int max_chunks, float scale_log2, unsigned* status, const DecodeFuse fuse) {
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
  const int len = decode_checked_len(context_lens, b, min(table_width * block_size, max_chunks * chunk), status);
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

  DecodeState<G> st;
  st.reset();

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
        uint8_t* stg = smem + s * 2 * kTileBytes;
        mbar_expect_tx(&full_bar[s], 2 * kTileBytes);
        bulk_load(stg, k_cache + off, kTileBytes, &full_bar[s]);
        bulk_load(stg + kTileBytes, v_cache + off, kTileBytes, &full_bar[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    float qr[G][16];
    // the newest token (position len - 1) is not in the cache yet: the warp that owns its row of its tile prepares it now
    const int row_new = (len - 1) % TILE, t_new = (len - 1 - tok_begin) / TILE;
    const bool owner = fuse.qkv != nullptr && len - 1 >= tok_begin && len - 1 < tok_end && warp == row_new / (TILE / 4);
    DecodeNewToken fresh = {};
    if (owner) fresh = decode_new_token(fuse, b, kvh, nq, nkv, len, lane);
    if (fuse.qkv != nullptr) decode_load_q_fused<G>(fuse, b, qh0, len, lane, scale_log2, qr);
    else decode_load_q<G>(q + (static_cast<size_t>(b) * nq + qh0) * kD, lane, scale_log2, qr);
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % kDecStages;
      const uint32_t ph = (t / kDecStages) & 1;
      if (!mbar_wait(&full_bar[s], ph, status)) break;
      uint8_t* Ks = smem + s * 2 * kTileBytes;
      if (owner && t == t_new) {
        int blk = block_tables[static_cast<size_t>(b) * table_width + (len - 1) / block_size];
        const bool blk_ok = blk >= 0 && blk < num_blocks;
        if (!blk_ok) blk = 0;
        const size_t off = ((static_cast<size_t>(blk) * nkv + kvh) * block_size + ((len - 1) % block_size)) * kD;
        decode_patch_new_token(fresh, row_new, Ks, Ks + kTileBytes, k_cache + off, v_cache + off, blk_ok && blockIdx.x % groups_per_kv == 0,
                               lane);
      }
      decode_consume_tile<G, TILE>(Ks, Ks + kTileBytes, tok_end - (tok_begin + t * TILE), warp, lane, qr, st);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
  }

  // ------------------------------------------------------------------ merge the four warps (stage memory is free now)
  __syncthreads();
  float* s_acc = reinterpret_cast<float*>(smem);                 // [4][G][128] + [4][G] + [4][G]
  if (warp < 4) decode_publish_state<G>(st, s_acc, warp, lane);
  __syncthreads();
  if (threadIdx.x < kD) {
    const int d = threadIdx.x;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float M, L;
      const float o = decode_merged<G>(s_acc, g, d, M, L);
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
                                                            int nq, int chunk, int max_chunks, int cap) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y, qh = blockIdx.x, d = threadIdx.x;
  const int len = decode_checked_len(context_lens, b, cap, nullptr);      // same clamp as the attention kernel, which reports it
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
                         int max_chunks, float scale_log2, unsigned* status, cudaStream_t stream, const DecodeFuse& fuse) {
  constexpr int kTileBytes = TILE * kD * 2;
  constexpr int merge_bytes = decode_merge_floats(G) * 4;
  constexpr int ring = kDecStages * 2 * kTileBytes;
  constexpr int smem = (ring > merge_bytes ? ring : merge_bytes) + 2 * kDecStages * 8 + 128;
  auto kern = decode_attn_kernel<G, TILE>;
  FORGE_ENSURE_DYN_SMEM(kern, smem);
  const int groups_per_kv = (nq / nkv) / G;
  dim3 grid(nkv * groups_per_kv, B, max_chunks);
  if (launch_kernel(kern, grid, dim3(kDecThreads), smem, stream, 0, static_cast<const __nv_bfloat16*>(q),
                    static_cast<__nv_bfloat16*>(const_cast<void*>(kc)), static_cast<__nv_bfloat16*>(const_cast<void*>(vc)), bt, lens,
                    static_cast<__nv_bfloat16*>(out), part_o, part_ml, nq, nkv, block_size, table_width, num_blocks, chunk,
                    max_chunks, scale_log2, status, fuse) != cudaSuccess)
    return -5;
  if (max_chunks > 1) {
    dim3 g2(nq, B);
    if (launch_kernel(decode_combine_kernel, g2, dim3(kD), 0, stream, 0, static_cast<const float*>(part_o),
                      static_cast<const float*>(part_ml), lens, static_cast<__nv_bfloat16*>(out), nq, chunk, max_chunks,
                      std::min(table_width * block_size, max_chunks * chunk)) != cudaSuccess)
      return -5;
  }
  return 0;
}

// q [B, nq, 128] bf16; caches [num_blocks, nkv, block_size, 128] bf16; block_tables [B, table_width]; out [B, nq * 128].
// part_o: fp32 [B, nq, max_chunks, 128], part_ml: fp32 [B, nq, max_chunks, 2] (may be null when max_chunks == 1).
// chunk: tokens per grid.z slice, a multiple of min(block_size, 64); max_chunks * chunk must cover the longest context.
static int decode_chunked_impl(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out,
                               float* part_o, float* part_ml, int B, int nq, int nkv, int head_dim, int block_size,
                               int table_width, int num_blocks, int chunk, int max_chunks, float scale, unsigned* status,
                               cudaStream_t stream, const DecodeFuse& fuse) {
  if (B <= 0) return 0;
  if (head_dim != kD || nq % nkv != 0 || block_size < 16 || (block_size & (block_size - 1))) return -1;
  const int tile = block_size < 64 ? block_size : 64;
  if (chunk % tile != 0 || max_chunks < 1) return -1;
  if (max_chunks > 1 && (part_o == nullptr || part_ml == nullptr)) return -1;
  const int group = nq / nkv;
  const int G = decode_group_slice(group);
  const float sl2 = scale * 1.4426950408889634f;
#define FORGE_DEC(GG, TT)                                                                                                   \
  return launch_decode<GG, TT>(q, kc, vc, bt, lens, out, part_o, part_ml, B, nq, nkv, block_size, table_width, num_blocks, \
                               chunk, max_chunks, sl2, status, stream, fuse)
  if (tile == 64) {
    if (G == 5) FORGE_DEC(5, 64);
    if (G == 4) FORGE_DEC(4, 64);
    if (G == 3) FORGE_DEC(3, 64);
    if (G == 2) FORGE_DEC(2, 64);
    FORGE_DEC(1, 64);
  } else if (tile == 32) {
    if (G == 5) FORGE_DEC(5, 32);
    if (G == 4) FORGE_DEC(4, 32);
    if (G == 3) FORGE_DEC(3, 32);
    if (G == 2) FORGE_DEC(2, 32);
    FORGE_DEC(1, 32);
  } else {
    if (G == 5) FORGE_DEC(5, 16);
    if (G == 4) FORGE_DEC(4, 16);
    if (G == 3) FORGE_DEC(3, 16);
    if (G == 2) FORGE_DEC(2, 16);
    FORGE_DEC(1, 16);
  }
#undef FORGE_DEC
}

extern "C" int forge_decode_attention(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out,
                                      float* part_o, float* part_ml, int B, int nq, int nkv, int head_dim, int block_size,
                                      int table_width, int num_blocks, int chunk, int max_chunks, float scale, unsigned* status,
                                      cudaStream_t stream) {
  const DecodeFuse none = {};
  return decode_chunked_impl(q, kc, vc, bt, lens, out, part_o, part_ml, B, nq, nkv, head_dim, block_size, table_width, num_blocks,
                             chunk, max_chunks, scale, status, stream, none);
}


// =========================================================================================================
// Flat tile partition.
//
// The chunked kernel above gives every (sequence, KV head, chunk) its own CTA; contexts differ in length and the
// number of CTAs is rarely a multiple of what the GPU runs at once, so its last wave is poorly filled (measured
// 0.96 of copy bandwidth at batch 256 but 0.72-0.88 at batch 64-128).  Here the work is the flat list of all KV
// tiles, ordered (sequence, KV head, tile), cut into gridDim.x equal ranges: every CTA streams the same number
// of tiles (+-0), whatever the lengths.  A CTA walks its range item by item ((sequence, head) = item) with ONE
// ring that never drains across items.  An item that lies wholly inside one CTA's range is finished there and
// written to `out`; an item cut by a range boundary leaves normalised partials that the merge kernel combines.
//
// Partials: a CTA has at most two cut items, the one it starts in (slot 0) and the one it ends in (slot 1):
// part_o[cta][slot][g][128], part_ml[cta][slot][g][2].  A cut item's parts are slot 1 of the CTA it starts in and
// slot 0 of the following CTAs; the CTA it starts in records cta_meta[cta] = (item, number of CTAs it spans), and
// CTA p of the merge kernel combines the item that starts in attention CTA p.
// Lengths are read on the device and the grid is fixed, so the launch is CUDA-graph safe.
// =========================================================================================================
constexpr int kFlatMaxSeqs = 512;

struct FlatCursor {       // position in the flat tile list
  int b, h, t, n_b;       // sequence, item within the sequence (KV head x group slice), tile, tiles of this sequence
};

// cum[b] = tiles of sequences < b (exclusive prefix, cum[B] = total).  Flat index of tile t of item (b, h):
// items_per_seq * cum[b] + h * n_b + t.
__device__ __forceinline__ FlatCursor flat_locate(const int* cum, int B, int items_per_seq, int f) {
  int lo = 0, hi = B;                                  // largest b with items_per_seq * cum[b] <= f
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (items_per_seq * cum[mid] <= f) lo = mid; else hi = mid;
  }
  FlatCursor c;
  c.b = lo;
  c.n_b = cum[lo + 1] - cum[lo];
  const int r = f - items_per_seq * cum[lo];
  c.h = r / c.n_b;
  c.t = r - c.h * c.n_b;
  return c;
}

__device__ __forceinline__ void flat_next_item(FlatCursor& c, const int* cum, int B, int items_per_seq) {
  c.t = 0;
  if (++c.h == items_per_seq) {
    c.h = 0;
    do { ++c.b; } while (c.b < B && cum[c.b + 1] == cum[c.b]);       // sequences of length 0 have no tiles
    c.n_b = c.b < B ? cum[c.b + 1] - cum[c.b] : 0;
  }
}

template <int G, int TILE>
__global__ void __launch_bounds__(kDecThreads, decode_ctas_per_sm(G)) decode_attn_flat_kernel(
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
    const int* __restrict__ block_tables, const int* __restrict__ context_lens, __nv_bfloat16* __restrict__ out,
    float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ cta_meta, int B, int nq, int nkv, int block_size,
    int table_width, int num_blocks, int min_tiles, float scale_log2, unsigned* status, const DecodeFuse fuse) {
  constexpr int kTileBytes = TILE * kD * 2;
  constexpr int kRing = kDecStages * 2 * kTileBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  float* s_acc = reinterpret_cast<float*>(smem + kRing);                      // merge area, separate from the ring
  int* cum = reinterpret_cast<int*>(s_acc + decode_merge_floats(G));          // [B + 1]
  int* chunk_tot = cum + kFlatMaxSeqs + 1;                                    // [16]
  // mbarriers are 8-byte objects: the int arrays before them have an odd word count, so round the address up
  uint64_t* full_bar = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(chunk_tot + 16) + 15) & ~uintptr_t(15));
  uint64_t* empty_bar = full_bar + kDecStages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);
    }
    fence_mbar_init();
  }
  pdl_wait();                                           // q, the new K/V entries and the step buffer come from predecessors

  // ---- exclusive prefix sum of tiles per sequence (B <= 512): warp scans of 32, then a scan of the 16 totals
  const int n_chunks32 = (B + 31) >> 5;
  for (int ch = warp; ch < n_chunks32; ch += kDecThreads / 32) {
    const int b = ch * 32 + lane;
    const int len = b < B ? decode_checked_len(context_lens, b, table_width * block_size, status) : 0;
    int v = (len + TILE - 1) / TILE;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    if (b < B) cum[b + 1] = v;                          // inclusive within the chunk, for now
    if (lane == 31) chunk_tot[ch] = v;
  }
  __syncthreads();
  if (warp == 0) {
    int v = lane < n_chunks32 ? chunk_tot[lane] : 0;
    const int own = v;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    if (lane < 16) chunk_tot[lane] = v - own;           // exclusive offset of each chunk
    if (lane == 0) cum[0] = 0;
  }
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += kDecThreads) cum[b + 1] += chunk_tot[b >> 5];
  __syncthreads();

  const int groups_per_kv = (nq / nkv) / G;             // > 1 when the GQA group is processed in slices of G
  const int items_per_seq = nkv * groups_per_kv;
  const int total = items_per_seq * cum[B];
  int per_cta = (total + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  if (per_cta < min_tiles) per_cta = min_tiles;
  const int f0 = blockIdx.x * per_cta;
  const int f1 = min(f0 + per_cta, total);
  // rows of length 0 (padding of a graph bucket) belong to no item: give them a defined output
  for (int b = blockIdx.x; b < B; b += gridDim.x)
    if (cum[b + 1] == cum[b])
      for (int i = threadIdx.x; i < nq * kD; i += kDecThreads) out[static_cast<size_t>(b) * nq * kD + i] = __float2bfloat16_rn(0.f);
  if (threadIdx.x == 0) cta_meta[blockIdx.x * 2] = -1;  // no cut item starts here, unless found below
  if (f0 >= f1) return;                                 // uniform for the CTA
  __syncthreads();                                      // orders the default above before the consumers' update

  if (warp == 4) {
    // ------------------------------------------------------------------ producer: one ring across all items
    if (lane == 0) {
      FlatCursor c = flat_locate(cum, B, items_per_seq, f0);
      int it = 0;
      for (int f = f0; f < f1;) {
        const int seg = min(c.n_b - c.t, f1 - f);
        const int kvh = c.h / groups_per_kv;
        const int* table = block_tables + static_cast<size_t>(c.b) * table_width;
        for (int i = 0; i < seg; ++i, ++it) {
          const int s = it % kDecStages;
          const uint32_t ph = (it / kDecStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, status)) { f = f1; break; }
          const int tok0 = (c.t + i) * TILE;
          int blk = table[tok0 / block_size];
          if (blk < 0 || blk >= num_blocks) {
            set_status(status, kStatusBadIndex);
            blk = 0;
          }
          const size_t off = ((static_cast<size_t>(blk) * nkv + kvh) * block_size + (tok0 % block_size)) * kD;
          uint8_t* stg = smem + s * 2 * kTileBytes;
          mbar_expect_tx(&full_bar[s], 2 * kTileBytes);
          bulk_load(stg, k_cache + off, kTileBytes, &full_bar[s]);
          bulk_load(stg + kTileBytes, v_cache + off, kTileBytes, &full_bar[s]);
        }
        f += seg;
        flat_next_item(c, cum, B, items_per_seq);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers (warps 0..3, 128 threads)
  FlatCursor c = flat_locate(cum, B, items_per_seq, f0);
  DecodeState<G> st;
  int it = 0;
  bool ok = true;
  for (int f = f0; f < f1 && ok;) {
    const int seg = min(c.n_b - c.t, f1 - f);
    const int kvh = c.h / groups_per_kv;
    const int qh0 = kvh * (nq / nkv) + (c.h % groups_per_kv) * G;
    const int len = decode_checked_len(context_lens, c.b, table_width * block_size, nullptr);
    float qr[G][16];
    // the newest token (position len - 1) is not in the cache yet: if this CTA streams the item's last tile, the warp that
    // owns the token's row prepares it now, under the latency of the q loads and the first tiles
    const int row_new = (len - 1) % TILE;
    const bool owner = fuse.qkv != nullptr && c.t + seg == c.n_b && warp == row_new / (TILE / 4);
    DecodeNewToken fresh = {};
    if (owner) fresh = decode_new_token(fuse, c.b, kvh, nq, nkv, len, lane);
    if (fuse.qkv != nullptr) decode_load_q_fused<G>(fuse, c.b, qh0, len, lane, scale_log2, qr);
    else decode_load_q<G>(q + (static_cast<size_t>(c.b) * nq + qh0) * kD, lane, scale_log2, qr);
    st.reset();
    for (int i = 0; i < seg; ++i, ++it) {
      const int s = it % kDecStages;
      const uint32_t ph = (it / kDecStages) & 1;
      ok = mbar_wait(&full_bar[s], ph, status);
      if (!ok) break;
      uint8_t* Ks = smem + s * 2 * kTileBytes;
      if (owner && i == seg - 1) {
        int blk = block_tables[static_cast<size_t>(c.b) * table_width + (len - 1) / block_size];
        const bool blk_ok = blk >= 0 && blk < num_blocks;
        if (!blk_ok) blk = 0;
        const size_t off = ((static_cast<size_t>(blk) * nkv + kvh) * block_size + ((len - 1) % block_size)) * kD;
        decode_patch_new_token(fresh, row_new, Ks, Ks + kTileBytes, k_cache + off, v_cache + off, blk_ok && c.h % groups_per_kv == 0, lane);
      }
      decode_consume_tile<G, TILE>(Ks, Ks + kTileBytes, len - (c.t + i) * TILE, warp, lane, qr, st);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
    if (!ok) break;
    // ---- end of this CTA's part of the item: merge the four warps, then final output or a partial
    decode_publish_state<G>(st, s_acc, warp, lane);
    named_barrier_sync(1, 128);
    const bool starts_here = c.t == 0, whole = starts_here && seg == c.n_b;
    const int d = threadIdx.x;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float M, L;
      const float o = decode_merged<G>(s_acc, g, d, M, L);
      if (whole) {
        out[(static_cast<size_t>(c.b) * nq + qh0 + g) * kD + d] = __float2bfloat16_rn(o);
      } else {
        const size_t p = (static_cast<size_t>(blockIdx.x) * 2 + (starts_here ? 1 : 0)) * G + g;
        part_o[p * kD + d] = o;
        if (d == 0) {
          part_ml[p * 2] = M;
          part_ml[p * 2 + 1] = L;
        }
      }
    }
    if (starts_here && !whole && d == 0) {
      const int item_end = f + c.n_b;                   // flat index one past the item's last tile (f is its first tile here)
      cta_meta[blockIdx.x * 2] = c.b * items_per_seq + c.h;
      cta_meta[blockIdx.x * 2 + 1] = (item_end - 1) / per_cta - static_cast<int>(blockIdx.x) + 1;
    }
    named_barrier_sync(1, 128);                         // the merge area is reused by the next item
    f += seg;
    flat_next_item(c, cum, B, items_per_seq);
  }
}

// Merge the partials of items cut by a range boundary: CTA p handles the item that starts in attention CTA p.
template <int G>
__global__ void __launch_bounds__(kD) decode_flat_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                 const int* __restrict__ cta_meta, __nv_bfloat16* __restrict__ out,
                                                                 int nq, int nkv) {
  pdl_launch_dependents();
  pdl_wait();
  const int first = blockIdx.x, d = threadIdx.x;
  const int item = cta_meta[first * 2], n = cta_meta[first * 2 + 1];
  if (item < 0) return;
  const int group = nq / nkv, groups_per_kv = group / G, items_per_seq = nkv * groups_per_kv;
  const int b = item / items_per_seq, h = item % items_per_seq;
  const int qh0 = (h / groups_per_kv) * group + (h % groups_per_kv) * G;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
    for (int k = 0; k < n; ++k) {
      const size_t p = (static_cast<size_t>(first + k) * 2 + (k == 0 ? 1 : 0)) * G + g;
      M = fmaxf(M, part_ml[p * 2]);
    }
    float L = 0.f, O = 0.f;
    for (int k = 0; k < n; ++k) {
      const size_t p = (static_cast<size_t>(first + k) * 2 + (k == 0 ? 1 : 0)) * G + g;
      const float w = part_ml[p * 2 + 1] * exp2f(part_ml[p * 2] - M);
      L += w;
      O += part_o[p * kD + d] * w;
    }
    out[(static_cast<size_t>(b) * nq + qh0 + g) * kD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
  }
}

template <int G, int TILE>
static int launch_decode_flat(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out,
                              float* scratch, int num_ctas, int B, int nq, int nkv, int block_size, int table_width, int num_blocks,
                              float scale_log2, unsigned* status, cudaStream_t stream, const DecodeFuse& fuse) {
  constexpr int kTileBytes = TILE * kD * 2;
  constexpr int smem = kDecStages * 2 * kTileBytes + decode_merge_floats(G) * 4 + (kFlatMaxSeqs + 1 + 16) * 4 + 16 + 2 * kDecStages * 8 + 128;
  static_assert(smem <= (decode_ctas_per_sm(G) == 2 ? 113 : 227) * 1024, "two CTAs per SM (one for G > 4)");
  auto kern = decode_attn_flat_kernel<G, TILE>;
  FORGE_ENSURE_DYN_SMEM(kern, smem);
  float* part_o = scratch;
  float* part_ml = part_o + static_cast<size_t>(num_ctas) * 2 * G * kD;
  int* cta_meta = reinterpret_cast<int*>(part_ml + static_cast<size_t>(num_ctas) * 2 * G * 2);
  const int min_tiles = 256 / TILE < 2 ? 2 : 256 / TILE;        // at least ~256 tokens per CTA: below that the start-up dominates
  if (launch_kernel(kern, dim3(num_ctas), dim3(kDecThreads), smem, stream, 0, static_cast<const __nv_bfloat16*>(q),
                    static_cast<__nv_bfloat16*>(const_cast<void*>(kc)), static_cast<__nv_bfloat16*>(const_cast<void*>(vc)), bt, lens,
                    static_cast<__nv_bfloat16*>(out), part_o, part_ml, cta_meta, B, nq, nkv, block_size, table_width, num_blocks,
                    min_tiles, scale_log2, status, fuse) != cudaSuccess)
    return -5;
  if (launch_kernel(decode_flat_combine_kernel<G>, dim3(num_ctas), dim3(kD), 0, stream, 0, static_cast<const float*>(part_o),
                    static_cast<const float*>(part_ml), static_cast<const int*>(cta_meta), static_cast<__nv_bfloat16*>(out), nq,
                    nkv) != cudaSuccess)
    return -5;
  return 0;
}

// =========================================================================================================
// Flat tile partition on the tensor cores, for q-head groups of 4..8 per KV head (Qwen3-4B/8B: 4, 14B: 5, 32B: 8).
//
// With G q heads per KV head every cached K and V element takes part in G multiply-adds.  On the CUDA cores that is
// the bound from G = 4 on (Qwen3-8B: 0.69 of copy bandwidth; a group of 8 had to stream the cache twice); as a matrix
// product it is nothing: the G query rows are padded to the 16-row side of mma.sync m16n8k16, S = Q K^T and O += P V
// run on the tensor cores exactly as in a prefill kernel, and the kernel is a pure stream of the cache again.
// (tcgen05 has no use for 4..8 rows: its smallest tile is 64 rows, and the operand is streamed once, not reused.)
//
// Same partition, partial slots and merge kernel as decode_attention_flat_kernel; one item = (sequence, KV head) with
// all G heads.  A tile = 64 tokens of K and of V, each loaded as two TMA boxes of 64 rows x 64 dims (128 bytes) with the
// 128-byte swizzle from a 2-D view [all token rows of the cache, 128] of the paged cache: inside a box the 16-byte chunk c
// of row r sits at chunk c ^ (r % 8), so the eight rows an ldmatrix touches fall into different banks.  (Contiguous 16 KB
// bulk copies leave the rows 256 bytes apart: every ldmatrix then takes eight shared-memory wavefronts, which bounded the
// kernel at 0.55 of copy bandwidth; one 256-byte bulk copy per row with a padded pitch ran at 0.17.)
// Groups of up to 5 heads leave room for two CTAs per SM (three stages each); 8 heads take one CTA with six stages.
// =========================================================================================================
constexpr int kTcTile = 64;
constexpr int kTcBoxBytes = kTcTile * 128;            // one TMA box: 64 token rows x 64 dims
constexpr int kTcTileBytes = 2 * kTcBoxBytes;         // K (or V) of a tile: dims 0..63, then dims 64..127
extern "C" int forge_make_tmap_2d(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                                  int elem_bytes);
// Shared-memory address of the 16-byte chunk `chunk` (0..15: eight dims each) of token row `r` of a swizzled tile.
__device__ __forceinline__ uint32_t tc_chunk_addr(uint32_t tile, int r, int chunk) {
  return tile + (chunk >> 3) * kTcBoxBytes + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
}
__host__ __device__ constexpr int tc_ctas_per_sm(int G) { return G > 5 ? 1 : 2; }
__host__ __device__ constexpr int tc_stages(int G) { return G > 5 ? 6 : 3; }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D (16 x 8, fp32) += A (16 x 16, bf16, rows 8..15 zero: a1 = a3 = 0) * B (16 x 8, bf16)
__device__ __forceinline__ void mma_rows8(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

template <int G>
__global__ void __launch_bounds__(kDecThreads, tc_ctas_per_sm(G)) decode_attn_flat_tc_kernel(
    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const __nv_bfloat16* __restrict__ q,
    const int* __restrict__ block_tables, const int* __restrict__ context_lens, __nv_bfloat16* __restrict__ out,
    float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ cta_meta, int B, int nq, int nkv, int block_size,
    int table_width, int num_blocks, int min_tiles, float scale_log2, unsigned* status) {
  static_assert(G >= 1 && G <= 8, "the query rows of a group fill the first eight rows of the MMA tile");
  constexpr int kTcStages = tc_stages(G);
  constexpr int kRing = kTcStages * 2 * kTcTileBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));   // swizzled boxes
  float* s_acc = reinterpret_cast<float*>(smem + kRing);                      // merge area, separate from the ring
  int* cum = reinterpret_cast<int*>(s_acc + decode_merge_floats(G));          // [B + 1]
  int* chunk_tot = cum + kFlatMaxSeqs + 1;                                    // [16]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(chunk_tot + 16) + 15) & ~uintptr_t(15));
  uint64_t* empty_bar = full_bar + kTcStages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);
    }
    fence_mbar_init();
  }
  pdl_wait();                                           // q, the new K/V entries and the step buffer come from predecessors

  // ---- exclusive prefix sum of tiles per sequence (as in decode_attn_flat_kernel)
  const int n_chunks32 = (B + 31) >> 5;
  for (int ch = warp; ch < n_chunks32; ch += kDecThreads / 32) {
    const int b = ch * 32 + lane;
    const int len = b < B ? decode_checked_len(context_lens, b, table_width * block_size, status) : 0;
    int v = (len + kTcTile - 1) / kTcTile;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    if (b < B) cum[b + 1] = v;
    if (lane == 31) chunk_tot[ch] = v;
  }
  __syncthreads();
  if (warp == 0) {
    int v = lane < n_chunks32 ? chunk_tot[lane] : 0;
    const int own = v;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    if (lane < 16) chunk_tot[lane] = v - own;
    if (lane == 0) cum[0] = 0;
  }
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += kDecThreads) cum[b + 1] += chunk_tot[b >> 5];
  __syncthreads();

  const int items_per_seq = nkv;                        // one item = all G heads of a KV head
  const int total = items_per_seq * cum[B];
  int per_cta = (total + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  if (per_cta < min_tiles) per_cta = min_tiles;
  const int f0 = blockIdx.x * per_cta;
  const int f1 = min(f0 + per_cta, total);
  for (int b = blockIdx.x; b < B; b += gridDim.x)
    if (cum[b + 1] == cum[b])
      for (int i = threadIdx.x; i < nq * kD; i += kDecThreads) out[static_cast<size_t>(b) * nq * kD + i] = __float2bfloat16_rn(0.f);
  if (threadIdx.x == 0) cta_meta[blockIdx.x * 2] = -1;
  if (f0 >= f1) return;                                 // uniform for the CTA
  __syncthreads();

  if (warp == 4) {
    // ------------------------------------------------------------------ producer: one ring across all items
    if (lane == 0) {
      FlatCursor c = flat_locate(cum, B, items_per_seq, f0);
      int it = 0;
      for (int f = f0; f < f1;) {
        const int seg = min(c.n_b - c.t, f1 - f);
        const int kvh = c.h;
        const int* table = block_tables + static_cast<size_t>(c.b) * table_width;
        for (int i = 0; i < seg; ++i, ++it) {
          const int s = it % kTcStages;
          const uint32_t ph = (it / kTcStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, status)) { f = f1; break; }
          const int tok0 = (c.t + i) * kTcTile;
          int blk = table[tok0 / block_size];
          if (blk < 0 || blk >= num_blocks) {
            set_status(status, kStatusBadIndex);
            blk = 0;
          }
          const int row0 = (blk * nkv + kvh) * block_size + (tok0 % block_size);     // token row in the 2-D view of the cache
          uint8_t* stg = smem + s * 2 * kTcTileBytes;
          mbar_expect_tx(&full_bar[s], 2 * kTcTileBytes);
          tma_load_2d(stg, &tm_k, &full_bar[s], 0, row0);
          tma_load_2d(stg + kTcBoxBytes, &tm_k, &full_bar[s], 64, row0);
          tma_load_2d(stg + kTcTileBytes, &tm_v, &full_bar[s], 0, row0);
          tma_load_2d(stg + kTcTileBytes + kTcBoxBytes, &tm_v, &full_bar[s], 64, row0);
        }
        f += seg;
        flat_next_item(c, cum, B, items_per_seq);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers (warps 0..3): 16 tokens of every tile each
  FlatCursor c = flat_locate(cum, B, items_per_seq, f0);
  const int row = lane >> 2, quad = lane & 3;           // MMA fragment coordinates: query row (head of the group), column pair
  const int mat = lane >> 3, mrow = lane & 7;           // ldmatrix: this lane supplies row `mrow` of matrix `mat`
  int it = 0;
  bool ok = true;
  for (int f = f0; f < f1 && ok;) {
    const int seg = min(c.n_b - c.t, f1 - f);
    const int kvh = c.h;
    const int qh0 = kvh * G;
    const int len = decode_checked_len(context_lens, c.b, table_width * block_size, nullptr);
    // A fragments of Q: rows 0..G-1 = the heads of the group, the rest zero; 8 k-steps of 16 dims
    uint32_t qa[8][2];
    {
      const __nv_bfloat16* qp = q + (static_cast<size_t>(c.b) * nq + qh0 + row) * kD + 2 * quad;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        qa[kk][0] = row < G ? *reinterpret_cast<const uint32_t*>(qp + kk * 16) : 0u;
        qa[kk][1] = row < G ? *reinterpret_cast<const uint32_t*>(qp + kk * 16 + 8) : 0u;
      }
    }
    float m_run = -INFINITY, l_run = 0.f;                // of query row `row`; l is this lane's share until the end
    float o[16][4];
#pragma unroll
    for (int nb = 0; nb < 16; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
    for (int i = 0; i < seg; ++i, ++it) {
      const int s = it % kTcStages;
      const uint32_t ph = (it / kTcStages) & 1;
      ok = mbar_wait(&full_bar[s], ph, status);
      if (!ok) break;
      const uint32_t Ks = smem_u32(smem + s * 2 * kTcTileBytes);
      const uint32_t Vs = Ks + kTcTileBytes;
      const int r0 = warp * 16;                                                           // this warp's 16 tokens of the tile
      // S = Q K^T: two blocks of 8 tokens
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t kb[4];
        ldmatrix_x4(kb, tc_chunk_addr(Ks, r0 + (mat >> 1) * 8 + mrow, 2 * kk + (mat & 1)));
        mma_rows8(sc[0], qa[kk][0], qa[kk][1], kb[0], kb[1]);
        mma_rows8(sc[1], qa[kk][0], qa[kk][1], kb[2], kb[3]);
      }
      // this lane: row `row`, tokens warp * 16 + j * 8 + 2 * quad + {0, 1} of the tile
      const int valid = len - (c.t + i) * kTcTile;
      float mt = -INFINITY;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = warp * 16 + j * 8 + 2 * quad + e;
          sc[j][e] = tok < valid ? sc[j][e] * scale_log2 : -INFINITY;
          mt = fmaxf(mt, sc[j][e]);
        }
      mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
      mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
      const float m_new = fmaxf(m_run, mt);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);
      float p[2][2];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) p[j][e] = exp2f(sc[j][e] - m_use);
      l_run = l_run * alpha + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
      m_run = m_new;
#pragma unroll
      for (int nb = 0; nb < 16; ++nb) {
        o[nb][0] *= alpha;
        o[nb][1] *= alpha;
      }
      // O += P V: P as the A operand (16 tokens = one k-step), V transposed on the way out of shared memory
      const uint32_t pa0 = pack_bf16x2(p[0][0], p[0][1]), pa2 = pack_bf16x2(p[1][0], p[1][1]);
#pragma unroll
      for (int dd = 0; dd < 8; ++dd) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, tc_chunk_addr(Vs, r0 + (mat & 1) * 8 + mrow, 2 * dd + (mat >> 1)));
        mma_rows8(o[2 * dd], pa0, pa2, vb[0], vb[1]);
        mma_rows8(o[2 * dd + 1], pa0, pa2, vb[2], vb[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
    if (!ok) break;
    // ---- end of this CTA's part of the item: publish the warp's state in the layout decode_merged reads, merge, store
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (row < G) {
      float* dst = s_acc + (warp * G + row) * kD + 2 * quad;
#pragma unroll
      for (int nb = 0; nb < 16; ++nb) *reinterpret_cast<float2*>(dst + nb * 8) = make_float2(o[nb][0], o[nb][1]);
      if (quad == 0) {
        s_acc[4 * G * kD + warp * G + row] = m_run;
        s_acc[4 * G * kD + 4 * G + warp * G + row] = l_run;
      }
    }
    named_barrier_sync(1, 128);
    const bool starts_here = c.t == 0, whole = starts_here && seg == c.n_b;
    const int d = threadIdx.x;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float M, L;
      const float ov = decode_merged<G>(s_acc, g, d, M, L);
      if (whole) {
        out[(static_cast<size_t>(c.b) * nq + qh0 + g) * kD + d] = __float2bfloat16_rn(ov);
      } else {
        const size_t pp = (static_cast<size_t>(blockIdx.x) * 2 + (starts_here ? 1 : 0)) * G + g;
        part_o[pp * kD + d] = ov;
        if (d == 0) {
          part_ml[pp * 2] = M;
          part_ml[pp * 2 + 1] = L;
        }
      }
    }
    if (starts_here && !whole && d == 0) {
      const int item_end = f + c.n_b;
      cta_meta[blockIdx.x * 2] = c.b * items_per_seq + c.h;
      cta_meta[blockIdx.x * 2 + 1] = (item_end - 1) / per_cta - static_cast<int>(blockIdx.x) + 1;
    }
    named_barrier_sync(1, 128);
    f += seg;
    flat_next_item(c, cum, B, items_per_seq);
  }
}

// Group sizes the tensor-core variant takes (all heads of the group in one item); cache blocks of at least 64 tokens.
// Measured on B200 (us per launch incl. the merge kernel; CUDA cores / tensor cores / flash-attn 2 on the same case):
// group 4, 256 sequences x 800 tokens: 188 / 151 / 189; group 8, 64 x 2304: 235 / 111 / 139.  The smallest group the
// tensor-core variant is used for can be changed (tests also run groups 4 and 5 on the CUDA cores).
static int g_tc_min_group = 4;
extern "C" void forge_decode_attention_set_tc_min_group(int g) { g_tc_min_group = g; }
static bool decode_flat_tc_ok(int group, int block_size) {
  return block_size >= kTcTile && group >= g_tc_min_group && (group == 4 || group == 5 || group == 8);
}

// CTAs per SM the flat decode kernel for this head grouping runs with (the grid to use is this times the SM count).
extern "C" int forge_decode_attention_flat_ctas_per_sm(int nq, int nkv, int block_size, int from_raw_qkv) {
  if (nkv <= 0 || nq % nkv != 0) return 2;
  const int group = nq / nkv;
  if (!from_raw_qkv && decode_flat_tc_ok(group, block_size)) return tc_ctas_per_sm(group);
  return decode_ctas_per_sm(decode_group_slice(group));
}

template <int G>
static int launch_decode_flat_tc(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out,
                                 float* scratch, int num_ctas, int B, int nq, int nkv, int block_size, int table_width, int num_blocks,
                                 float scale_log2, unsigned* status, cudaStream_t stream) {
  constexpr int kTcStages = tc_stages(G);
  constexpr int smem = kTcStages * 2 * kTcTileBytes + decode_merge_floats(G) * 4 + (kFlatMaxSeqs + 1 + 16) * 4 + 16 + 2 * kTcStages * 8 + 1024;
  static_assert(smem <= (tc_ctas_per_sm(G) == 2 ? 113 : 227) * 1024, "two CTAs per SM up to five heads, one for eight");
  auto kern = decode_attn_flat_tc_kernel<G>;
  FORGE_ENSURE_DYN_SMEM(kern, smem);
  // the paged cache as a 2-D tensor [every token row of every block and KV head, 128]; box = 64 rows x 64 dims, 128-byte swizzle
  CUtensorMap tm_k, tm_v;
  const uint64_t rows = static_cast<uint64_t>(num_blocks) * nkv * block_size;
  if ((reinterpret_cast<uintptr_t>(kc) & 15) || (reinterpret_cast<uintptr_t>(vc) & 15)) return -1;
  if (forge_make_tmap_2d(&tm_k, kc, rows, kD, kD, kTcTile, 2) != 0 || forge_make_tmap_2d(&tm_v, vc, rows, kD, kD, kTcTile, 2) != 0) return -2;
  float* part_o = scratch;
  float* part_ml = part_o + static_cast<size_t>(num_ctas) * 2 * G * kD;
  int* cta_meta = reinterpret_cast<int*>(part_ml + static_cast<size_t>(num_ctas) * 2 * G * 2);
  const int min_tiles = 256 / kTcTile;
  if (launch_kernel(kern, dim3(num_ctas), dim3(kDecThreads), smem, stream, 0, tm_k, tm_v, static_cast<const __nv_bfloat16*>(q), bt, lens,
                    static_cast<__nv_bfloat16*>(out), part_o, part_ml, cta_meta, B, nq, nkv, block_size, table_width, num_blocks,
                    min_tiles, scale_log2, status) != cudaSuccess)
    return -5;
  if (launch_kernel(decode_flat_combine_kernel<G>, dim3(num_ctas), dim3(kD), 0, stream, 0, static_cast<const float*>(part_o),
                    static_cast<const float*>(part_ml), static_cast<const int*>(cta_meta), static_cast<__nv_bfloat16*>(out), nq,
                    nkv) != cudaSuccess)
    return -5;
  return 0;
}

// Floats of scratch the flat kernel needs for a grid of num_ctas CTAs and up to B sequences.
extern "C" size_t forge_decode_attention_flat_scratch_floats(int num_ctas, int B, int nq, int nkv) {
  const int group = nkv > 0 ? nq / nkv : 1;
  int G = decode_group_slice(group);
  if (group <= 8 && group > G) G = group;               // the tensor-core variant keeps all heads of a group in one item
  (void)B;
  return static_cast<size_t>(num_ctas) * 2 * G * (kD + 2) + static_cast<size_t>(num_ctas) * 2 + 64;
}

// Same operands as forge_decode_attention; scratch: forge_decode_attention_flat_scratch_floats() floats, contents
// irrelevant on entry.  num_ctas: grid size, normally two per SM.  B <= 512.
static int decode_flat_impl(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out,
                            float* scratch, int num_ctas, int B, int nq, int nkv, int head_dim, int block_size,
                            int table_width, int num_blocks, float scale, unsigned* status, cudaStream_t stream, const DecodeFuse& fuse) {
  if (B <= 0) return 0;
  if (head_dim != kD || nq % nkv != 0 || block_size < 16 || (block_size & (block_size - 1)) || B > kFlatMaxSeqs || num_ctas < 1 ||
      scratch == nullptr)
    return -1;
  const int tile = block_size < 64 ? block_size : 64;
  const int group = nq / nkv;
  const int G = decode_group_slice(group);
  const float sl2 = scale * 1.4426950408889634f;
  if (fuse.qkv == nullptr && decode_flat_tc_ok(group, block_size)) {
#define FORGE_TC(GG) \
  return launch_decode_flat_tc<GG>(q, kc, vc, bt, lens, out, scratch, num_ctas, B, nq, nkv, block_size, table_width, num_blocks, sl2, status, stream)
    if (group == 4) FORGE_TC(4);
    if (group == 5) FORGE_TC(5);
    FORGE_TC(8);
#undef FORGE_TC
  }
#define FORGE_DEC(GG, TT)                                                                                                       \
  return launch_decode_flat<GG, TT>(q, kc, vc, bt, lens, out, scratch, num_ctas, B, nq, nkv, block_size, table_width, num_blocks, \
                                    sl2, status, stream, fuse)
  if (tile == 64) {
    if (G == 5) FORGE_DEC(5, 64);
    if (G == 4) FORGE_DEC(4, 64);
    if (G == 3) FORGE_DEC(3, 64);
    if (G == 2) FORGE_DEC(2, 64);
    FORGE_DEC(1, 64);
  } else if (tile == 32) {
    if (G == 5) FORGE_DEC(5, 32);
    if (G == 4) FORGE_DEC(4, 32);
    if (G == 3) FORGE_DEC(3, 32);
    if (G == 2) FORGE_DEC(2, 32);
    FORGE_DEC(1, 32);
  } else {
    if (G == 5) FORGE_DEC(5, 16);
    if (G == 4) FORGE_DEC(4, 16);
    if (G == 3) FORGE_DEC(3, 16);
    if (G == 2) FORGE_DEC(2, 16);
    FORGE_DEC(1, 16);
  }
#undef FORGE_DEC
}

extern "C" int forge_decode_attention_flat(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out,
                                           float* scratch, int num_ctas, int B, int nq, int nkv, int head_dim, int block_size,
                                           int table_width, int num_blocks, float scale, unsigned* status, cudaStream_t stream) {
  const DecodeFuse none = {};
  return decode_flat_impl(q, kc, vc, bt, lens, out, scratch, num_ctas, B, nq, nkv, head_dim, block_size, table_width, num_blocks, scale,
                          status, stream, none);
}

// Decode attention straight from the raw qkv projection: q/k RMSNorm (weights may be null), NeoX rotation at position
// len - 1 (rope may be null) and the KV-cache store of the step's token happen inside the attention kernel (replaces a
// separate qk_norm_rope_store launch).  qkv: [B, (nq + 2 nkv) * 128] bf16 with row stride ld_qkv.  num_ctas > 0: flat tile
// partition (scratch as for forge_decode_attention_flat); num_ctas == 0: context chunks (part_o / part_ml, chunk, max_chunks
// as for forge_decode_attention).  Sequences of length 0 (padding rows) store nothing.
extern "C" int forge_decode_attention_qkv(const void* qkv, int ld_qkv, const void* q_w, const void* k_w, float eps, const float* rope,
                                          int rope_rows, void* kc, void* vc, const int* bt, const int* lens, void* out, float* scratch,
                                          int num_ctas, float* part_o, float* part_ml, int chunk, int max_chunks, int B, int nq, int nkv,
                                          int head_dim, int block_size, int table_width, int num_blocks, float scale, unsigned* status,
                                          cudaStream_t stream) {
  if (qkv == nullptr || (ld_qkv & 7) || (reinterpret_cast<uintptr_t>(qkv) & 15)) return -1;
  DecodeFuse fuse;
  fuse.qkv = static_cast<const __nv_bfloat16*>(qkv);
  fuse.ld_qkv = ld_qkv;
  fuse.q_w = static_cast<const __nv_bfloat16*>(q_w);
  fuse.k_w = static_cast<const __nv_bfloat16*>(k_w);
  fuse.eps = eps;
  fuse.rope = rope;
  fuse.rope_rows = rope_rows;
  if (num_ctas > 0)
    return decode_flat_impl(nullptr, kc, vc, bt, lens, out, scratch, num_ctas, B, nq, nkv, head_dim, block_size, table_width, num_blocks,
                            scale, status, stream, fuse);
  return decode_chunked_impl(nullptr, kc, vc, bt, lens, out, part_o, part_ml, B, nq, nkv, head_dim, block_size, table_width, num_blocks,
                             chunk, max_chunks, scale, status, stream, fuse);
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
//   * `stream` must belong to the device that is current at the call: the array's address and the kernels' shared
//     memory limit are set up for the current device.
//   * A context length beyond table_width * block_size or max_chunks * chunk is clamped and reported through
//     `status` (the bad-index bit, value 4), so a corrupted length can neither read outside the block table nor outside the array.
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

// Consumers and small producers of the in-kernel tensor-parallel exchange (see include/tp_comm.cuh).
//
//   tp_reduce_rms_norm   one-shot all-reduce + residual add + RMSNorm in one pass: waits for every rank's GEMM, pulls
//                        the sum of the ranks' partial rows (multimem.ld_reduce through the switch, or plain peer loads
//                        in rank order), adds the residual, writes the new residual and the normalised row.  Replaces
//                        dist.all_reduce + add_rms_forward (tinyvllm/layers/linear.py:183 +
//                        tinyvllm/layers/layernorm.py:33-45).  With y == null it is a plain all-reduce.  The same
//                        kernel finishes the vocab-parallel embedding (rows written by their owners, nothing to add).
//   tp_rs_norm_ag        two-shot form of the same for many bytes (large decode batches, prefill): reduce-scatter by
//                        rows, residual add + RMSNorm on this rank's rows, all-gather of the normalised rows
//                        (multimem.st or peer stores), second flag round.  The residual stream stays sharded by rows.
//   embedding_push       vocab-parallel embedding: the rank that owns a token id writes the row into every rank's
//                        buffer (no zero rows cross NVLink, no reduction needed; the reference masks, looks up,
//                        zeroes and all-reduces: tinyvllm/layers/embed_head.py:34-42).
//   rows_publish         copies rows into this rank's partial buffer and signals (standalone all-reduce / barrier).
//   sample_pairs_push / sample_pairs_merge   every rank pushes its per-row (score, id) to all ranks; each rank
//                        picks the winner itself, so logits never leave a GPU (the reference gathers full logit
//                        shards to rank 0: embed_head.py:63-70).
#include "../include/launch.cuh"
#include "../include/tp_comm.cuh"

namespace forge {

__device__ __forceinline__ float warp_sum_c(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float bf16_round_c(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

constexpr int kTpNormChunks = 4;

// acc (the summed GEMM output, fp32) -> rounded to bf16 as the reference's all-reduced tensor is, plus the residual,
// rounded again: the new residual.  Returns it packed; acc holds the same values as floats afterwards.
__device__ __forceinline__ uint4 tp_add_residual8(float acc[8], const __nv_bfloat16* residual_row, int i) {
  if (residual_row != nullptr) {
    const uint4 b = reinterpret_cast<const uint4*>(residual_row)[i];
    const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[2 * j] = bf16_round_c(bf16_round_c(acc[2 * j]) + bf16_lo(bw[j]));
      acc[2 * j + 1] = bf16_round_c(bf16_round_c(acc[2 * j + 1]) + bf16_hi(bw[j]));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = bf16_round_c(acc[j]);
  }
  return make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
}

// Sum of squares over the CTA (every thread gets the total).  `red` has 32 floats.
__device__ __forceinline__ float cta_sum_c(float ss, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  ss = warp_sum_c(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum_c(t);
}

__device__ __forceinline__ uint4 tp_normed8(const float v[8], float inv, const __nv_bfloat16* w, int i) {
  const uint4 wv = reinterpret_cast<const uint4*>(w)[i];
  const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o[j] = pack_bf16x2(bf16_round_c(v[2 * j] * inv) * bf16_lo(ww[j]), bf16_round_c(v[2 * j + 1] * inv) * bf16_hi(ww[j]));
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// One CTA per row.  residual_in may be null (first layer: the sum itself becomes the residual).
// y may be null (plain all-reduce: only `sum_out` is written).  src.size == 0: the rows were written into tp.slots
// by their owners (embedding) and are only copied.
__global__ void __launch_bounds__(256) tp_reduce_rms_norm_kernel(TpPull tp, TpReduceSrc src, const __nv_bfloat16* __restrict__ residual_in,
                                                                 __nv_bfloat16* __restrict__ sum_out, const __nv_bfloat16* __restrict__ w,
                                                                 __nv_bfloat16* __restrict__ y, int H, float eps, unsigned* status) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  tp_pull_wait(tp, status);
  const bool local = tp_local_only(tp.local_only);
  const size_t row = blockIdx.x;
  const int nvec = H >> 3;
  float vals[kTpNormChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kTpNormChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nvec) {
      float acc[8];
      if (src.size > 0) {
        tp_load_sum8(src, local, row * H + static_cast<size_t>(i) * 8, acc);
      } else {
        const uint4 a = reinterpret_cast<const uint4*>(tp.slots + row * H)[i];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] = bf16_lo(aw[j]);
          acc[2 * j + 1] = bf16_hi(aw[j]);
        }
      }
      reinterpret_cast<uint4*>(sum_out + row * H)[i] = tp_add_residual8(acc, residual_in != nullptr ? residual_in + row * H : nullptr, i);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        vals[c][j] = acc[j];
        ss += acc[j] * acc[j];
      }
    }
  }
  if (y == nullptr) return;
  const float inv = rsqrtf(cta_sum_c(ss, red) / static_cast<float>(H) + eps);
#pragma unroll
  for (int c = 0; c < kTpNormChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nvec) reinterpret_cast<uint4*>(y + row * H)[i] = tp_normed8(vals[c], inv, w, i);
  }
}

static TpPull make_tp_pull(int tp_size, int num_slots, const void* slots, long long slot_stride, const unsigned* signal,
                           const unsigned* epoch, long long timeout_ns, const unsigned* local_only) {
  TpPull tp;
  tp.size = tp_size;
  tp.num_slots = num_slots;
  tp.slots = static_cast<const __nv_bfloat16*>(slots);
  tp.slot_stride = slot_stride;
  tp.signal = signal;
  tp.epoch = epoch;
  tp.timeout_ns = timeout_ns;
  tp.local_only = local_only;
  return tp;
}

static TpReduceSrc make_tp_src(int tp_size, int tp_rank, const long long* part_ptrs, long long mc_part, const unsigned* local_only) {
  TpReduceSrc src = {};
  if (part_ptrs == nullptr) return src;            // size 0: not used
  src.size = tp_size;
  src.rank = tp_rank;
  for (int p = 0; p < tp_size && p < kMaxTp; ++p) src.part[p] = reinterpret_cast<const __nv_bfloat16*>(part_ptrs[p]);
  src.mc_part = reinterpret_cast<const __nv_bfloat16*>(mc_part);
  src.local_only = local_only;
  return src;
}

static int norm_threads(int H) {
  int threads = ((H >> 3) + kTpNormChunks - 1) / kTpNormChunks;
  threads = ((threads + 31) / 32) * 32;
  return threads < 32 ? 32 : (threads > 256 ? 256 : threads);
}

// part_ptrs: every rank's partial buffer in rank order (null: copy rows from `slots`, which their owners wrote);
// mc_part: multicast address of the partial buffer or 0.
extern "C" int forge_tp_reduce_rms_norm(int tp_size, int tp_rank, const long long* part_ptrs, long long mc_part, const void* slots,
                                        const unsigned* signal, const unsigned* epoch, long long timeout_ns,
                                        const unsigned* local_only, const void* residual_in, void* sum_out, const void* w, void* y,
                                        int rows, int H, float eps, unsigned* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > kTpNormChunks * 256 * 8 || tp_size > kMaxTp || tp_rank < 0 || tp_rank >= (tp_size > 0 ? tp_size : 1)) return -1;
  if (part_ptrs == nullptr && slots == nullptr) return -1;
  const TpPull tp = make_tp_pull(tp_size, 1, slots, 0, signal, epoch, timeout_ns, local_only);
  const TpReduceSrc src = make_tp_src(tp_size, tp_rank, part_ptrs, mc_part, local_only);
  return launch_kernel(tp_reduce_rms_norm_kernel, dim3(rows), dim3(norm_threads(H)), 0, stream, 0, tp, src,
                       static_cast<const __nv_bfloat16*>(residual_in), static_cast<__nv_bfloat16*>(sum_out),
                       static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), H, eps, status) == cudaSuccess ? 0 : -2;
}

// Two-shot exchange.  CTA i handles row i * size + rank: this rank's share of the reduce-scatter.  `residual` is a
// full-size local tensor of which only this rank's rows are read and written (the residual stream stays sharded by
// rows from one exchange to the next); the normalised row goes to every rank's broadcast buffer.  After its own
// stores a CTA reports to the grid's arrival counter.  The LAST CTA to arrive publishes this rank's epoch at the
// all-gather site to every rank and then waits until all ranks have published theirs, so that when the kernel
// completes the whole broadcast buffer is valid on this rank.  Only that one CTA waits: a CTA that waited while later
// CTAs of the same grid still queue for a free SM would wait for a signal its own grid cannot send.
__global__ void __launch_bounds__(256) tp_rs_norm_ag_kernel(TpPull wait_parts, TpReduceSrc src, const __nv_bfloat16* residual_in,
                                                            __nv_bfloat16* residual_out, const __nv_bfloat16* __restrict__ w,
                                                            TpBcastDst dst, TpPush done, TpPull wait_rows, int rows, int H, float eps,
                                                            unsigned* status) {
  __shared__ float red[32];
  __shared__ unsigned last_cta, my_epoch;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) last_cta = 0u;
  tp_pull_wait(wait_parts, status);
  const bool local = tp_local_only(src.local_only);
  const size_t row = static_cast<size_t>(blockIdx.x) * src.size + src.rank;
  if (row < static_cast<size_t>(rows)) {               // uniform for the CTA
    const int nvec = H >> 3;
    float vals[kTpNormChunks][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < kTpNormChunks; ++c) {
      const int i = threadIdx.x + c * blockDim.x;
      if (i < nvec) {
        float acc[8];
        tp_load_sum8(src, local, row * H + static_cast<size_t>(i) * 8, acc);
        reinterpret_cast<uint4*>(residual_out + row * H)[i] = tp_add_residual8(acc, residual_in != nullptr ? residual_in + row * H : nullptr, i);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          vals[c][j] = acc[j];
          ss += acc[j] * acc[j];
        }
      }
    }
    const float inv = rsqrtf(cta_sum_c(ss, red) / static_cast<float>(H) + eps);
#pragma unroll
    for (int c = 0; c < kTpNormChunks; ++c) {
      const int i = threadIdx.x + c * blockDim.x;
      if (i < nvec) {
        const uint4 o = tp_normed8(vals[c], inv, w, i);
        const size_t off = row * H + static_cast<size_t>(i) * 8;
        if (local) {
          *reinterpret_cast<uint4*>(dst.y[src.rank] + off) = o;
        } else if (dst.mc_y != nullptr) {
          multimem_st_v4(dst.mc_y + off, o);
        } else {
          for (int p = 0; p < src.size; ++p) *reinterpret_cast<uint4*>(dst.y[p] + off) = o;
        }
      }
    }
  }
  __threadfence_system();                               // this thread's (remote) stores are ordered before what follows
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done.arrive, 1u);
    if (prev == gridDim.x - 1) {
      atomicExch(done.arrive, 0u);
      __threadfence_system();                           // cumulative: every CTA's stores are ordered before the signal
      const unsigned e = *done.epoch + 1;
      *done.epoch = e;
      for (int p = 0; p < done.size; ++p) st_release_sys(done.signal[p], e);
      my_epoch = e;
      last_cta = 1u;
    }
  }
  __syncthreads();
  if (last_cta != 0u) tp_wait_epoch(wait_rows, my_epoch, status);      // uniform for the CTA
}

TpPush make_tp_push(int tp_size, int tp_rank, const long long* slot_ptrs, const long long* signal_ptrs, unsigned* arrive,
                    unsigned* epoch);

// part_ptrs / y_ptrs: every rank's partial and broadcast buffers in rank order; mc_part / mc_y: their multicast
// addresses or 0.  signal1 / epoch1: this rank's signal words and epoch of the GEMM's site; signal_ptrs2 / arrive2 /
// epoch2 / signal2: the all-gather site (peer addresses of this rank's word, private counters, local words).
extern "C" int forge_tp_rs_norm_ag(int tp_size, int tp_rank, const long long* part_ptrs, long long mc_part, const unsigned* signal1,
                                   const unsigned* epoch1, const long long* y_ptrs, long long mc_y, const long long* signal_ptrs2,
                                   unsigned* arrive2, unsigned* epoch2, const unsigned* signal2, long long timeout_ns,
                                   const unsigned* local_only, const void* residual_in, void* residual_out, const void* w, int rows,
                                   int H, float eps, unsigned* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > kTpNormChunks * 256 * 8 || tp_size < 2 || tp_size > kMaxTp || tp_rank < 0 || tp_rank >= tp_size) return -1;
  if (part_ptrs == nullptr || y_ptrs == nullptr || w == nullptr || residual_out == nullptr) return -1;
  const TpPull wait_parts = make_tp_pull(tp_size, 1, nullptr, 0, signal1, epoch1, timeout_ns, local_only);
  const TpPull wait_rows = make_tp_pull(tp_size, 1, nullptr, 0, signal2, epoch2, timeout_ns, local_only);
  const TpReduceSrc src = make_tp_src(tp_size, tp_rank, part_ptrs, mc_part, local_only);
  TpBcastDst dst = {};
  for (int p = 0; p < tp_size; ++p) dst.y[p] = reinterpret_cast<__nv_bfloat16*>(y_ptrs[p]);
  dst.mc_y = reinterpret_cast<__nv_bfloat16*>(mc_y);
  const TpPush done = make_tp_push(tp_size, tp_rank, nullptr, signal_ptrs2, arrive2, epoch2);
  const int grid = (rows + tp_size - 1) / tp_size;
  return launch_kernel(tp_rs_norm_ag_kernel, dim3(grid), dim3(norm_threads(H)), 0, stream, 0, wait_parts, src,
                       static_cast<const __nv_bfloat16*>(residual_in), static_cast<__nv_bfloat16*>(residual_out),
                       static_cast<const __nv_bfloat16*>(w), dst, done, wait_rows, rows, H, eps, status) == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------------
// Tagged-word exchange (decode-sized batches): see "tagged words" in include/tp_comm.cuh
// ---------------------------------------------------------------------------------------------------------
// One CTA per row.  Row b belongs to rank b % size.  Its owner polls the sources' tagged partial words (the GEMM
// epilogues of all ranks stored them there), adds them, adds its shard of the residual, normalises, stores the row
// into its own `y` and sends it as tagged words to every other rank.  A CTA of a row that belongs to another rank
// polls the tagged words that row's owner sends and stores the plain row into `y`.  When the kernel completes, `y`
// holds all rows on every rank.  At most 256 CTAs, all resident at once, so a CTA that polls never keeps one that
// sends from running.
__global__ void __launch_bounds__(256, 2) tp_tagged_reduce_norm_kernel(TpTagged tp, const __nv_bfloat16* residual_in,
                                                                    __nv_bfloat16* residual_out, const __nv_bfloat16* __restrict__ w,
                                                                    __nv_bfloat16* __restrict__ y, int rows, int H, float eps,
                                                                    unsigned* status) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const unsigned tag_part = *tp.part_epoch;            // advanced by this rank's GEMM, which has completed
  const unsigned tag_rows = *tp.epoch + 1u;            // read before this CTA reports its arrival (see tp_tagged_done)
  const bool local = tp_local_only(tp.local_only);
  const int row = blockIdx.x;
  const int owner = row % tp.size, j = row / tp.size;
  const int nvec = H >> 3;
  if (owner == tp.rank) {
    float vals[kTpNormChunks][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < kTpNormChunks; ++c) {
      const int i = threadIdx.x + c * blockDim.x;
      if (i < nvec) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const int first = local ? tp.rank : 0, last = local ? tp.rank + 1 : tp.size;
        const uint32_t* base = tp.part + static_cast<size_t>(j) * H + i * 8;
        const size_t src_stride = static_cast<size_t>(tp.rows_per_rank) * H;
        // four sources at a time: their words are requested before any is examined, so the loads overlap instead of
        // paying one trip to L2 each (and the code stays small: this kernel runs dozens of times per step)
#pragma unroll 1
        for (int s0 = first; s0 < last; s0 += 4) {
          uint4 a[4], b[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (s0 + k < last) {
              a[k] = ld_volatile_v4(base + (s0 + k) * src_stride);
              b[k] = ld_volatile_v4(base + (s0 + k) * src_stride + 4);
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {                 // rank order: the same sum whichever rank owns the row
            if (s0 + k < last) {
              const uint4 wa = tp_poll_tagged(base + (s0 + k) * src_stride, a[k], tag_part, tp.timeout_ns, status);
              const uint4 wb = tp_poll_tagged(base + (s0 + k) * src_stride + 4, b[k], tag_part, tp.timeout_ns, status);
              acc[0] += bf16_lo(wa.x); acc[1] += bf16_hi(wa.x); acc[2] += bf16_lo(wa.z); acc[3] += bf16_hi(wa.z);
              acc[4] += bf16_lo(wb.x); acc[5] += bf16_hi(wb.x); acc[6] += bf16_lo(wb.z); acc[7] += bf16_hi(wb.z);
            }
          }
        }
        reinterpret_cast<uint4*>(residual_out + static_cast<size_t>(row) * H)[i] =
            tp_add_residual8(acc, residual_in != nullptr ? residual_in + static_cast<size_t>(row) * H : nullptr, i);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          vals[c][k] = acc[k];
          ss += acc[k] * acc[k];
        }
      }
    }
    const float inv = rsqrtf(cta_sum_c(ss, red) / static_cast<float>(H) + eps);
#pragma unroll
    for (int c = 0; c < kTpNormChunks; ++c) {
      const int i = threadIdx.x + c * blockDim.x;
      if (i < nvec) {
        const uint4 o = tp_normed8(vals[c], inv, w, i);
        reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H)[i] = o;
        if (!local) {
          const size_t off = static_cast<size_t>(row) * H + i * 8;
          for (int p = 0; p < tp.size; ++p) {
            if (p == tp.rank) continue;
            st_volatile_v4(tp.y[p] + off, make_uint4(o.x, tag_rows, o.y, tag_rows));
            st_volatile_v4(tp.y[p] + off + 4, make_uint4(o.z, tag_rows, o.w, tag_rows));
          }
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      uint4 o = make_uint4(0u, 0u, 0u, 0u);             // measurement mode: rows of other ranks are not exchanged
      if (!local) {
        const uint32_t* p = tp.y[tp.rank] + static_cast<size_t>(row) * H + i * 8;
        const uint4 a0 = ld_volatile_v4(p), b0 = ld_volatile_v4(p + 4);
        const uint4 a = tp_poll_tagged(p, a0, tag_rows, tp.timeout_ns, status);
        const uint4 b = tp_poll_tagged(p + 4, b0, tag_rows, tp.timeout_ns, status);
        o = make_uint4(a.x, a.z, b.x, b.z);
      }
      reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H)[i] = o;
    }
  }
  TpPush done = {};
  done.arrive = tp.arrive;
  done.epoch = tp.epoch;
  tp_tagged_done(done, gridDim.x);
}

// part: this rank's buffer of the GEMM site ([tp_size][rows_per_rank][H] words); y_ptrs: every rank's buffer of
// normalised rows ([256][H] words) in rank order; arrive / epoch: private counters of the normalised-rows site;
// part_epoch: this rank's epoch at the GEMM site.  `residual` is updated on this rank's rows only.
extern "C" int forge_tp_tagged_reduce_norm(int tp_size, int tp_rank, const void* part, int rows_per_rank, const unsigned* part_epoch,
                                           const long long* y_ptrs, unsigned* arrive, unsigned* epoch, long long timeout_ns,
                                           const unsigned* local_only, const void* residual_in, void* residual_out, const void* w,
                                           void* y, int rows, int H, float eps, unsigned* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > kTpNormChunks * 256 * 8 || tp_size < 2 || tp_size > kMaxTp || tp_rank < 0 || tp_rank >= tp_size) return -1;
  if (rows > 256 || (rows + tp_size - 1) / tp_size > rows_per_rank || part == nullptr || y_ptrs == nullptr || w == nullptr ||
      y == nullptr || residual_out == nullptr)
    return -1;
  TpTagged tp = {};
  tp.size = tp_size;
  tp.rank = tp_rank;
  tp.rows_per_rank = rows_per_rank;
  tp.part = static_cast<const uint32_t*>(part);
  for (int p = 0; p < tp_size; ++p) tp.y[p] = reinterpret_cast<uint32_t*>(y_ptrs[p]);
  tp.arrive = arrive;
  tp.epoch = epoch;
  tp.part_epoch = part_epoch;
  tp.timeout_ns = timeout_ns;
  tp.local_only = local_only;
  return launch_kernel(tp_tagged_reduce_norm_kernel, dim3(rows), dim3(norm_threads(H)), 0, stream, 0, tp,
                       static_cast<const __nv_bfloat16*>(residual_in), static_cast<__nv_bfloat16*>(residual_out),
                       static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), rows, H, eps, status) == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------------
// Row pushes
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) embedding_push_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                                             TpPush tp, int H, int vocab_start, int vocab_n) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int local = ids[t] - vocab_start;
  if (local >= 0 && local < vocab_n) {                // the owner of this id writes the row everywhere
    const uint4* src = reinterpret_cast<const uint4*>(w + static_cast<size_t>(local) * H);
    for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
      const uint4 v = src[i];
      for (int p = 0; p < tp.size; ++p) reinterpret_cast<uint4*>(tp.slot[p] + static_cast<size_t>(t) * H)[i] = v;
    }
  }
  tp_push_done(tp, gridDim.x);
}

// Copies rows into this rank's partial buffer (a local store) and signals: the producer half of the standalone
// all-reduce.
__global__ void __launch_bounds__(128) rows_publish_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ part,
                                                           TpPush tp, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x)
    reinterpret_cast<uint4*>(part + t * H)[i] = reinterpret_cast<const uint4*>(src + t * H)[i];
  tp_push_done(tp, gridDim.x);
}

TpPush make_tp_push(int tp_size, int tp_rank, const long long* slot_ptrs, const long long* signal_ptrs, unsigned* arrive,
                    unsigned* epoch) {
  TpPush tp = {};
  tp.size = tp_size;
  tp.rank = tp_rank;
  for (int p = 0; p < tp_size && p < kMaxTp; ++p) {
    tp.slot[p] = slot_ptrs != nullptr ? reinterpret_cast<__nv_bfloat16*>(slot_ptrs[p]) : nullptr;
    tp.signal[p] = reinterpret_cast<unsigned*>(signal_ptrs[p]);
  }
  tp.arrive = arrive;
  tp.epoch = epoch;
  return tp;
}

extern "C" int forge_tp_embedding_push(const int* ids, const void* w, int T, int H, int vocab_start, int vocab_n, int tp_size,
                                       int tp_rank, const long long* slot_ptrs, const long long* signal_ptrs, unsigned* arrive,
                                       unsigned* epoch, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H & 7) || tp_size > kMaxTp) return -1;
  return launch_kernel(embedding_push_kernel, dim3(T), dim3(128), 0, stream, 0, ids, static_cast<const __nv_bfloat16*>(w),
                       make_tp_push(tp_size, tp_rank, slot_ptrs, signal_ptrs, arrive, epoch), H, vocab_start, vocab_n) == cudaSuccess ? 0 : -2;
}

extern "C" int forge_tp_rows_publish(const void* src, void* part, int rows, int H, int tp_size, int tp_rank,
                                     const long long* signal_ptrs, unsigned* arrive, unsigned* epoch, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || tp_size > kMaxTp) return -1;
  return launch_kernel(rows_publish_kernel, dim3(rows), dim3(128), 0, stream, 0, static_cast<const __nv_bfloat16*>(src),
                       static_cast<__nv_bfloat16*>(part), make_tp_push(tp_size, tp_rank, nullptr, signal_ptrs, arrive, epoch), H) == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------------
// Sampler: per-row (score, id) pairs.  The slot buffer is used as pairs: [size][rows] of {float, int}.
// ---------------------------------------------------------------------------------------------------------
struct Pair {
  float v;
  int i;
};

__global__ void __launch_bounds__(128) sample_pairs_push_kernel(const float* __restrict__ vals, const int* __restrict__ ids, int rows,
                                                                TpPush tp) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < rows) {
    const Pair pr{vals[r], ids[r]};
    for (int p = 0; p < tp.size; ++p) reinterpret_cast<Pair*>(tp.slot[p])[r] = pr;
  }
  tp_push_done(tp, gridDim.x);
}

__global__ void __launch_bounds__(128) sample_pairs_merge_kernel(TpPull tp, int rows, int* __restrict__ out_i, unsigned* status) {
  pdl_launch_dependents();
  pdl_wait();
  tp_pull_wait(tp, status);
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int s = 0; s < tp.num_slots; ++s) {
    const Pair pr = reinterpret_cast<const Pair*>(tp.slots + s * tp.slot_stride)[r];
    if (pr.v > bv || (pr.v == bv && pr.i < bi)) {
      bv = pr.v;
      bi = pr.i;
    }
  }
  out_i[r] = bi;
}

extern "C" int forge_tp_sample_pairs(const float* vals, const int* ids, int rows, int tp_size, int tp_rank, const long long* slot_ptrs,
                                     const long long* signal_ptrs, unsigned* arrive, unsigned* epoch, const void* local_slots,
                                     long long slot_stride, const unsigned* signal_local, long long timeout_ns,
                                     const unsigned* local_only, int* out_i, unsigned* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (tp_size > kMaxTp) return -1;
  const int grid = (rows + 127) / 128;
  if (launch_kernel(sample_pairs_push_kernel, dim3(grid), dim3(128), 0, stream, 0, vals, ids, rows,
                    make_tp_push(tp_size, tp_rank, slot_ptrs, signal_ptrs, arrive, epoch)) != cudaSuccess)
    return -2;
  const TpPull tp = make_tp_pull(tp_size, tp_size, local_slots, slot_stride, signal_local, epoch, timeout_ns, local_only);
  return launch_kernel(sample_pairs_merge_kernel, dim3(grid), dim3(128), 0, stream, 0, tp, rows, out_i, status) == cudaSuccess ? 0 : -2;
}

}  // namespace forge

// Consumers and small producers of the in-kernel tensor-parallel exchange (see include/tp_comm.cuh).
//
//   tp_reduce_rms_norm   all-reduce + residual add + RMSNorm in one pass: waits for every rank's push, sums the
//                        per-rank partial rows in rank order, adds the residual, writes the new residual and the
//                        normalised row.  Replaces dist.all_reduce + add_rms_forward
//                        (tinyvllm/layers/linear.py:183 + tinyvllm/layers/layernorm.py:33-45).  With y == null it
//                        is a plain all-reduce of pushed rows.
//   embedding_push       vocab-parallel embedding: the rank that owns a token id writes the row into every rank's
//                        buffer (no zero rows cross NVLink, no reduction needed; the reference masks, looks up,
//                        zeroes and all-reduces: tinyvllm/layers/embed_head.py:34-42).
//   rows_push            generic "send my rows to everybody" (used by tests and by the library-GEMM prefill path).
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

// One CTA per row.  residual_in may be null (first layer: the sum itself becomes the residual).
// y may be null (plain all-reduce: only `sum_out` is written).
__global__ void __launch_bounds__(256) tp_reduce_rms_norm_kernel(TpPull tp, const __nv_bfloat16* __restrict__ residual_in,
                                                                 __nv_bfloat16* __restrict__ sum_out, const __nv_bfloat16* __restrict__ w,
                                                                 __nv_bfloat16* __restrict__ y, int H, float eps, unsigned* status) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  tp_pull_wait(tp, status);
  const size_t row = blockIdx.x;
  const int nvec = H >> 3;
  float vals[kTpNormChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kTpNormChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nvec) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < tp.num_slots; ++s) {       // rank order: identical result on every rank
        const uint4 a = reinterpret_cast<const uint4*>(tp.slots + s * tp.slot_stride + row * H)[i];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += bf16_lo(aw[j]);
          acc[2 * j + 1] += bf16_hi(aw[j]);
        }
      }
      // the all-reduced GEMM output is a bf16 tensor in the reference; round before the residual add
      if (residual_in != nullptr) {
        const uint4 b = reinterpret_cast<const uint4*>(residual_in + row * H)[i];
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
      uint32_t sw[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) sw[j] = pack_bf16x2(acc[2 * j], acc[2 * j + 1]);
      reinterpret_cast<uint4*>(sum_out + row * H)[i] = make_uint4(sw[0], sw[1], sw[2], sw[3]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        vals[c][j] = acc[j];
        ss += acc[j] * acc[j];
      }
    }
  }
  if (y == nullptr) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  ss = warp_sum_c(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum_c(t);
  const float inv = rsqrtf(t / static_cast<float>(H) + eps);
#pragma unroll
  for (int c = 0; c < kTpNormChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[i];
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = pack_bf16x2(bf16_round_c(vals[c][2 * j] * inv) * bf16_lo(ww[j]), bf16_round_c(vals[c][2 * j + 1] * inv) * bf16_hi(ww[j]));
      reinterpret_cast<uint4*>(y + row * H)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

extern "C" int forge_tp_reduce_rms_norm(int tp_size, int num_slots, const void* slots, long long slot_stride, const unsigned* signal,
                                        const unsigned* epoch, long long timeout_ns, const void* residual_in, void* sum_out,
                                        const void* w, void* y, int rows, int H, float eps, unsigned* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > kTpNormChunks * 256 * 8 || tp_size > kMaxTp || num_slots > kMaxTp) return -1;
  TpPull tp;
  tp.size = tp_size;
  tp.num_slots = num_slots;
  tp.slots = static_cast<const __nv_bfloat16*>(slots);
  tp.slot_stride = slot_stride;
  tp.signal = signal;
  tp.epoch = epoch;
  tp.timeout_ns = timeout_ns;
  int threads = ((H >> 3) + kTpNormChunks - 1) / kTpNormChunks;
  threads = ((threads + 31) / 32) * 32;
  threads = threads < 32 ? 32 : (threads > 256 ? 256 : threads);
  return launch_kernel(tp_reduce_rms_norm_kernel, dim3(rows), dim3(threads), 0, stream, 0, tp,
                       static_cast<const __nv_bfloat16*>(residual_in), static_cast<__nv_bfloat16*>(sum_out),
                       static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), H, eps, status) == cudaSuccess ? 0 : -2;
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

__global__ void __launch_bounds__(128) rows_push_kernel(const __nv_bfloat16* __restrict__ src, TpPush tp, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(src + t * H)[i];
    for (int p = 0; p < tp.size; ++p) reinterpret_cast<uint4*>(tp.slot[p] + t * H)[i] = v;
  }
  tp_push_done(tp, gridDim.x);
}

TpPush make_tp_push(int tp_size, int tp_rank, const long long* slot_ptrs, const long long* signal_ptrs, unsigned* arrive,
                    unsigned* epoch, long long mc_slot = 0);

TpPush make_tp_push(int tp_size, int tp_rank, const long long* slot_ptrs, const long long* signal_ptrs, unsigned* arrive,
                    unsigned* epoch, long long mc_slot) {
  TpPush tp = {};
  tp.mc_slot = reinterpret_cast<__nv_bfloat16*>(mc_slot);
  tp.size = tp_size;
  tp.rank = tp_rank;
  for (int p = 0; p < tp_size && p < kMaxTp; ++p) {
    tp.slot[p] = reinterpret_cast<__nv_bfloat16*>(slot_ptrs[p]);
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

extern "C" int forge_tp_rows_push(const void* src, int rows, int H, int tp_size, int tp_rank, const long long* slot_ptrs,
                                  const long long* signal_ptrs, unsigned* arrive, unsigned* epoch, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || tp_size > kMaxTp) return -1;
  return launch_kernel(rows_push_kernel, dim3(rows), dim3(128), 0, stream, 0, static_cast<const __nv_bfloat16*>(src),
                       make_tp_push(tp_size, tp_rank, slot_ptrs, signal_ptrs, arrive, epoch), H) == cudaSuccess ? 0 : -2;
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
                                     long long slot_stride, const unsigned* signal_local, long long timeout_ns, int* out_i,
                                     unsigned* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (tp_size > kMaxTp) return -1;
  const int grid = (rows + 127) / 128;
  if (launch_kernel(sample_pairs_push_kernel, dim3(grid), dim3(128), 0, stream, 0, vals, ids, rows,
                    make_tp_push(tp_size, tp_rank, slot_ptrs, signal_ptrs, arrive, epoch)) != cudaSuccess)
    return -2;
  TpPull tp;
  tp.size = tp_size;
  tp.num_slots = tp_size;
  tp.slots = static_cast<const __nv_bfloat16*>(local_slots);
  tp.slot_stride = slot_stride;
  tp.signal = signal_local;
  tp.epoch = epoch;
  tp.timeout_ns = timeout_ns;
  return launch_kernel(sample_pairs_merge_kernel, dim3(grid), dim3(128), 0, stream, 0, tp, rows, out_i, status) == cudaSuccess ? 0 : -2;
}

}  // namespace forge

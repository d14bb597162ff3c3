// Temperature sampling without a softmax, without materialising probabilities, and with one random number per GROUP of
// 16 token ids instead of one per token id (the two-level procedure is described in include/sampling.cuh).
//
// The reference computes softmax(logits / T), divides by Exp(1) noise and takes the argmax
// (tinyvllm/layers/sampler.py:13-21): eight ATen kernels over [rows, vocab] fp32.
//
// A vocabulary sharded over tensor-parallel ranks samples the same token as an unsharded one: each rank reduces its shard to
// one (group score, token id) pair per row and only those pairs are merged.
//
// Two kernels: the best group per (row, vocab slice) and its token, then a merge per row that can also fold in the pairs
// of other ranks.
#include "../include/launch.cuh"
#include "../include/ptx.cuh"
#include "../include/sampling.cuh"

namespace forge {

constexpr int kSampleThreads = 256;

// The 16 logits of group g of a row (global ids 16 g ..), -INFINITY outside the shard [vocab_start, vocab_start + vocab).
__device__ __forceinline__ void load_group(const __nv_bfloat16* lrow, int g, int vocab_start, int vocab, bool aligned, float lv[kSampleGroup]) {
  const int local0 = g * kSampleGroup - vocab_start;
  if (aligned && local0 >= 0 && local0 + kSampleGroup <= vocab) {
    const uint4 a = *reinterpret_cast<const uint4*>(lrow + local0), b = *reinterpret_cast<const uint4*>(lrow + local0 + 8);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      lv[2 * j] = bf16_lo(w[j]);
      lv[2 * j + 1] = bf16_hi(w[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < kSampleGroup; ++j)
      lv[j] = (local0 + j >= 0 && local0 + j < vocab) ? __bfloat162float(lrow[local0 + j]) : -INFINITY;
  }
}

// header: the packed step buffer's first words; [9] = step index, [10], [11] = seed low / high.
__global__ void __launch_bounds__(kSampleThreads) sample_partial_kernel(
    const __nv_bfloat16* __restrict__ logits, int ld, int vocab, int vocab_start, const float* __restrict__ temps,
    const int* __restrict__ header, float* __restrict__ part_v, int* __restrict__ part_i, int nsplit) {
  __shared__ float sv[kSampleThreads / 32];
  __shared__ int si[kSampleThreads / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y, split = blockIdx.x;
  const float T = temps[row];
  const bool greedy = !(T > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / T;
  const uint32_t step = static_cast<uint32_t>(header[9]);
  const uint32_t k0 = static_cast<uint32_t>(header[10]), k1 = static_cast<uint32_t>(header[11]);
  // slice boundaries in groups of 16 ids, aligned on the GLOBAL id
  const int g_first = vocab_start / kSampleGroup, g_last = (vocab_start + vocab - 1) / kSampleGroup;
  const int ngroups = g_last - g_first + 1;
  const int per = (ngroups + nsplit - 1) / nsplit;
  const int gb = g_first + split * per;
  const int ge = min(gb + per, g_last + 1);
  const __nv_bfloat16* lrow = logits + static_cast<size_t>(row) * ld;
  const bool aligned = (reinterpret_cast<uintptr_t>(lrow) & 15) == 0 && (vocab_start & 7) == 0;   // groups start on 16-byte boundaries
  // level 1: every thread scores the groups it visits; `i` of the pair is the group index here
  Best best{-INFINITY, 0x7fffffff};
  for (int g = gb + threadIdx.x; g < ge; g += kSampleThreads) {
    float lv[kSampleGroup];
    load_group(lrow, g, vocab_start, vocab, aligned, lv);
    uint32_t rnd[4] = {0, 0, 0, 0};
    if (!greedy) philox4x32_10(static_cast<uint32_t>(g >> 2), static_cast<uint32_t>(row), step, 1u, k0, k1, rnd);
    best = better(best, Best{sample_group_score(lv, inv_t, greedy, rnd[g & 3]), g});
  }
  best = warp_best(best);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
  __syncthreads();
  if (warp == 0) {
    Best b = lane < kSampleThreads / 32 ? Best{sv[lane], si[lane]} : Best{-INFINITY, 0x7fffffff};
    b = warp_best(b);
    if (lane == 0) {
      // level 2: the token inside the slice's winning group
      int token = 0x7fffffff;
      if (b.i != 0x7fffffff) {
        float lv[kSampleGroup];
        load_group(lrow, b.i, vocab_start, vocab, aligned, lv);
        token = sample_group_token(lv, b.i, inv_t, greedy, static_cast<uint32_t>(row), step, k0, k1);
      }
      part_v[static_cast<size_t>(row) * nsplit + split] = b.v;
      part_i[static_cast<size_t>(row) * nsplit + split] = token;
    }
  }
}

// One warp per row merges `n` candidate pairs; writes the winning id (and value when out_v != nullptr).
__global__ void __launch_bounds__(128) sample_merge_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int n,
                                                           int rows, int* __restrict__ out_i, float* __restrict__ out_v) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  Best b{-INFINITY, 0x7fffffff};
  for (int j = lane; j < n; j += 32) b = better(b, Best{part_v[static_cast<size_t>(row) * n + j], part_i[static_cast<size_t>(row) * n + j]});
  b = warp_best(b);
  if (lane == 0) {
    out_i[row] = b.i;
    if (out_v != nullptr) out_v[row] = b.v;
  }
}

// Merge `n` candidate pairs per row (part_* laid out [rows][n]); used by the two-kernel sampler below and after the
// LM-head GEMM whose epilogue produced one pair per (row, vocabulary tile).
extern "C" int forge_sample_merge(const float* part_v, const int* part_i, int n, int rows, int* out_i, float* out_v, cudaStream_t stream) {
  if (rows <= 0) return 0;
  return launch_kernel(sample_merge_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, 0, part_v, part_i, n, rows, out_i, out_v) == cudaSuccess ? 0 : -2;
}

extern "C" int forge_sample_nsplit(int rows, int vocab) {
  // Five CTAs of 256 threads fit an SM (registers).  A grid of about ONE wave is the worst case (256 rows x 3 slices = 768
  // CTAs for 740 places: the last 28 ran alone and the kernel took twice as long): aim for ~8 waves of equal CTAs, so the
  // ragged last wave costs < 10 %; never fewer than ~2K ids per CTA.
  int want = (device_sm_count() * 5 * 8 + rows - 1) / rows;
  int cap = (vocab + 2047) / 2048;
  int n = want < cap ? want : cap;
  return n < 1 ? 1 : (n > 64 ? 64 : n);
}

// logits [rows, vocab] bf16 (row stride ld); part_* are scratch of rows * nsplit entries.
extern "C" int forge_sample(const void* logits, int ld, int rows, int vocab, int vocab_start, const float* temps,
                            const int* header, float* part_v, int* part_i, int nsplit, int* out_i, float* out_v,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  dim3 grid(nsplit, rows);
  if (launch_kernel(sample_partial_kernel, grid, dim3(kSampleThreads), 0, stream, 0, static_cast<const __nv_bfloat16*>(logits), ld,
                    vocab, vocab_start, temps, header, part_v, part_i, nsplit) != cudaSuccess)
    return -2;
  return launch_kernel(sample_merge_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, 0, static_cast<const float*>(part_v),
                       static_cast<const int*>(part_i), nsplit, rows, out_i, out_v) == cudaSuccess ? 0 : -2;
}

// Merge pairs gathered from all ranks: vals/ids laid out [ranks, rows] -> transposed read.
__global__ void __launch_bounds__(128) sample_merge_ranks_kernel(const float* __restrict__ vals, const int* __restrict__ ids, int ranks,
                                                                 int rows, int* __restrict__ out_i) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  Best b{-INFINITY, 0x7fffffff};
  for (int r = 0; r < ranks; ++r) b = better(b, Best{vals[static_cast<size_t>(r) * rows + row], ids[static_cast<size_t>(r) * rows + row]});
  out_i[row] = b.i;
}

extern "C" int forge_sample_merge_ranks(const float* vals, const int* ids, int ranks, int rows, int* out_i, cudaStream_t stream) {
  if (rows <= 0) return 0;
  return launch_kernel(sample_merge_ranks_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, 0, vals, ids, ranks, rows,
                       out_i) == cudaSuccess ? 0 : -2;
}

}  // namespace forge

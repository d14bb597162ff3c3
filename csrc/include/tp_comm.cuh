// Tensor-parallel communication from inside kernels: peer-memory stores/loads over NVLink plus flag words.
//
// The reference calls NCCL through torch.distributed after each row-parallel GEMM (tinyvllm/layers/linear.py:183),
// after the vocab-parallel embedding (tinyvllm/layers/embed_head.py:41) and gathers logits to rank 0
// (embed_head.py:66-67).  Here the producing kernel itself writes its result into every peer's memory while it
// computes ("push"), and the consuming kernel (residual add + RMSNorm, or the token merge of the sampler) waits
// on flags and reduces the per-rank slots locally in rank order, so results are deterministic and bit-identical
// on every rank.
//
// A "site" is one place in the model where ranks exchange data (embedding, o_proj, down_proj, sampler).  Per site
// every rank owns, at the same offset of a symmetric allocation:
//     slots[size][rows][ld]   slot r is written by rank r (remotely), read locally
//     signal[size]            word r = number of completed pushes of rank r (monotonic "epoch"), written remotely
// and two private words: `arrive` (CTAs of the running producer that finished) and `epoch` (pushes this rank
// has completed).  All ranks run the same sequence of kernels, so epochs advance in lock step; counters live in
// device memory, so a replayed CUDA graph needs no host-side patching.
//
// Buffer reuse: sites that alternate (o_proj, down_proj) use different slot buffers.  A rank can only start
// producing into site A again after it consumed site B, which needs every peer's signal for B, which that peer
// sent after it finished consuming A (stream order).  Hence a slot is never overwritten while a peer reads it.
//
// Every wait is bounded in time; on expiry the kernel sets kStatusFlagTimeout in the status word and continues
// with whatever data is there (the host raises after the step).  No multicast TMA is used anywhere; peers'
// memory is touched only with ordinary ld/st.
#pragma once

#include "ptx.cuh"

namespace forge {

constexpr int kMaxTp = 8;

// What a producer needs to push its output to all ranks and to announce completion.
struct TpPush {
  int size;                              // <= 1: not tensor-parallel, fields below unused
  int rank;
  __nv_bfloat16* slot[kMaxTp];           // peer p: base of slot [rank] inside p's slot buffer
  __nv_bfloat16* mc_slot;                // NVLS multicast address of slot [rank] (one store lands on every rank), or null
  unsigned* signal[kMaxTp];              // peer p: address of word [rank] in p's signal array of this site
  unsigned* arrive;                      // local: CTAs finished in the current launch
  unsigned* epoch;                       // local: completed pushes of this rank at this site
};

// What a consumer needs: local slots, local signal words, the epoch to wait for.
struct TpPull {
  int size;
  int num_slots;                         // slots to sum (size for partial sums, 1 for owner-written rows)
  const __nv_bfloat16* slots;            // local slot buffer, slot stride = slot_stride elements
  long long slot_stride;
  const unsigned* signal;                // local signal words [size]
  const unsigned* epoch;                 // local epoch counter of the site (already advanced by this rank's producer)
  long long timeout_ns;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// One 8-byte store through the NVSwitch multicast address: the switch replicates it into every rank's copy.
__device__ __forceinline__ void multimem_st_v2(void* mc_addr, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_addr), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Producer tail, executed by every CTA after its last store to peer memory.  The last CTA of the grid
// publishes the new epoch to every rank.
__device__ __forceinline__ void tp_push_done(const TpPush& tp, unsigned total_ctas) {
  __threadfence_system();                // this thread's remote stores are ordered before what follows
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(tp.arrive, 1u);
    if (prev == total_ctas - 1) {
      atomicExch(tp.arrive, 0u);
      __threadfence_system();            // cumulative: every CTA's stores are ordered before the signal
      const unsigned e = *tp.epoch + 1;
      *tp.epoch = e;
      for (int p = 0; p < tp.size; ++p) st_release_sys(tp.signal[p], e);
    }
  }
}

// Consumer head: returns once every rank's signal word reached this rank's epoch, or after the time limit.
// Call with all threads of the CTA; contains __syncthreads().
__device__ __forceinline__ void tp_pull_wait(const TpPull& tp, unsigned* status) {
  if (tp.size > 1 && threadIdx.x < tp.size) {
    const unsigned want = *tp.epoch;
    const unsigned long long t0 = global_timer_ns();
    while (static_cast<int>(ld_acquire_sys(tp.signal + threadIdx.x) - want) < 0) {
      if (global_timer_ns() - t0 > static_cast<unsigned long long>(tp.timeout_ns)) {
        set_status(status, kStatusFlagTimeout);
        break;
      }
      __nanosleep(40);
    }
  }
  __syncthreads();
}

}  // namespace forge

// Tensor-parallel communication from inside kernels: loads and stores on peers' memory over NVLink / NVSwitch plus
// flag words.
//
// The reference calls NCCL through torch.distributed after each row-parallel GEMM (tinyvllm/layers/linear.py:183),
// after the vocab-parallel embedding (tinyvllm/layers/embed_head.py:41) and gathers logits to rank 0
// (embed_head.py:66-67).  Here every rank owns a region of symmetric memory (same layout on every rank, every
// peer's copy mapped into this process, and, where the driver offers it, one NVSwitch multicast address that
// names all copies at once).  Three exchange patterns are built on it:
//
//   row-parallel GEMM -> sum   The GEMM stores its partial sums into THIS rank's `part` buffer (a local store) and
//                              its last CTA announces completion to every rank.  Consumers then pull the sum:
//       one-shot  (few bytes)  every rank reads all rows with multimem.ld_reduce (the switch adds the ranks' copies
//                              in flight) and does residual add + RMSNorm itself: one flag round.
//       two-shot  (many bytes) rank r reduces only rows r, r + tp, ... (reduce-scatter), adds its shard of the residual,
//                              normalises and broadcasts the normalised rows with multimem.st (all-gather), then all ranks
//                              meet on a second flag round: per-direction traffic ~1x the tensor instead of tp x.
//       Without a multicast address the same kernels use plain peer loads / stores (rank order, so results are
//       bit-identical on all ranks).
//   owner-writes push          vocab-parallel embedding rows and the sampler's (score, id) pairs: the producing rank
//                              stores into every rank's buffer.
//
// A "site" is one place in the model where ranks exchange data.  Per site every rank owns, at the same offset of
// the symmetric region, signal[size] (word r = number of completed productions of rank r, a monotonic "epoch",
// written remotely) and two private words: `arrive` (CTAs of the running producer that finished) and `epoch`
// (productions this rank has completed).  All ranks run the same sequence of kernels, so epochs advance in lock
// step; counters live in device memory, so a replayed CUDA graph needs no host-side patching.
//
// Buffer reuse: the two row-parallel layers of a block use different `part` buffers.  A rank can only overwrite its
// o_proj buffer after it consumed the down_proj exchange, which needs every peer's down_proj signal, which that peer
// sent after it finished reading the o_proj buffers (stream order).  The broadcast buffer `y` is written only by
// ranks that already hold every rank's signal for the current site, which each rank sends after its last read of
// the previous contents.
//
// Every wait is bounded in time; on expiry the kernel sets kStatusFlagTimeout in the status word and continues
// with whatever data is there (the host raises after the step).  No multicast TMA is used anywhere; peers' memory
// is touched only with ordinary ld/st and with multimem.* instructions.
#pragma once

#include "ptx.cuh"

namespace forge {

constexpr int kMaxTp = 8;

// What a producer needs to announce completion to all ranks and, for pushes, where to store.
struct TpPush {
  int size;                              // <= 1: not tensor-parallel, fields below unused
  int rank;
  int ll;                                // 1: tagged-word push of a row-parallel GEMM (see "tagged words" below); signal[] unused
  int rows_per_rank;                     // ll: rows of one source rank's area in an owner's buffer
  __nv_bfloat16* slot[kMaxTp];           // pushes: peer p's copy of the destination buffer (slot [rank] for pairs)
  unsigned* signal[kMaxTp];              // peer p: address of word [rank] in p's signal array of this site
  unsigned* arrive;                      // local: CTAs finished in the current launch
  unsigned* epoch;                       // local: completed productions of this rank at this site
};

// What a consumer needs to wait for every rank's production: local signal words and the epoch to wait for.
struct TpPull {
  int size;
  int num_slots;                         // owner-writes pushes: slots to combine (size for pairs, 1 for embedding rows)
  const __nv_bfloat16* slots;            // owner-writes pushes: local buffer, slot stride = slot_stride elements
  long long slot_stride;
  const unsigned* signal;                // local signal words [size]
  const unsigned* epoch;                 // local epoch counter of the site
  long long timeout_ns;
  const unsigned* local_only;            // device word, non-zero: measurement mode, see TpReduceSrc::local_only
};

// Where the partial sums of a row-parallel GEMM live.
struct TpReduceSrc {
  int size;                              // 0: not used (the consumer reads TpPull::slots instead)
  int rank;
  const __nv_bfloat16* part[kMaxTp];     // every rank's partial buffer, in rank order (part[rank] is local)
  const __nv_bfloat16* mc_part;          // multicast address of that buffer, or null: plain peer loads
  // Measurement mode: when the word is non-zero the kernels skip every wait, read only this rank's own partial and
  // store only locally, i.e. they do the same arithmetic and local memory traffic without the exchange.  The
  // results are wrong on purpose; step time minus the time measured this way is the exposed communication.
  const unsigned* local_only;
};

// Tagged words (decode-sized exchanges, where latency decides).  Every pair of bf16 values travels as one 8-byte word
// {payload, tag}; the tag is the exchange's epoch, which sender and receiver both derive from their own counters.  An
// aligned 8-byte store arrives whole, so a receiver that polls the word until the tag matches has the payload: no
// fence, no completion flag and no second round trip.  The GEMM epilogue stores each output row straight into the
// buffer of the rank that owns the row (row % size); that rank adds the sources' words, applies residual + RMSNorm and
// sends the normalised row, again as tagged words, to every other rank.  Traffic per direction: ~2 x the tensor.
// A buffer row holds `width` 32-bit words for `width` features: word 2k = features 2k and 2k + 1, word 2k + 1 = tag.
struct TpTagged {
  int size, rank, rows_per_rank;
  const uint32_t* part;                  // local: [size sources][rows_per_rank][width] words, written by the sources' GEMMs
  uint32_t* y[kMaxTp];                   // every rank's [rows][width] words for normalised rows (y[rank] is local)
  unsigned* arrive;                      // private counters of the normalised-rows site
  unsigned* epoch;
  const unsigned* part_epoch;            // this rank's epoch at the GEMM's site (advanced by its own GEMM)
  long long timeout_ns;
  const unsigned* local_only;
};

// Where normalised rows are broadcast to (two-shot exchange).
struct TpBcastDst {
  __nv_bfloat16* y[kMaxTp];              // every rank's copy of the broadcast buffer, rank order
  __nv_bfloat16* mc_y;                   // multicast address of the buffer, or null: plain peer stores
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// One 16-byte store through the NVSwitch multicast address: the switch replicates it into every rank's copy.
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}
// One 16-byte load through the multicast address: the switch reads the eight bf16 values at this offset of every
// rank's copy, adds them (fp32 accumulation) and returns the sums as bf16.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
// 16-byte load that is always served by the memory that owns the address (a peer's copy is never taken from a
// local cache line of an earlier exchange).
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
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

__device__ __forceinline__ bool tp_local_only(const unsigned* flag) { return flag != nullptr && *flag != 0u; }

// Two tagged words (four bf16 values) at `p`, first try already in `v`: polls until both tags equal `tag` or the time limit
// passes.  Polling backs off (the words sit in this GPU's L2, where the peers' stores have to land too).
// The retry loop is kept out of line: it is the rare path, and the kernels that poll are launched dozens of times per
// step, where a small instruction footprint matters more than a call.
static __device__ __noinline__ uint4 tp_poll_tagged_slow(const uint32_t* p, unsigned tag, long long timeout_ns, unsigned* status) {
  uint4 v;
  const unsigned long long t0 = global_timer_ns();
  unsigned pause = 32;
  for (;;) {
    v = ld_volatile_v4(p);
    if (v.y == tag && v.w == tag) return v;
    if (global_timer_ns() - t0 > static_cast<unsigned long long>(timeout_ns)) {
      set_status(status, kStatusFlagTimeout);
      return v;
    }
    __nanosleep(pause);
    if (pause < 256) pause <<= 1;
  }
}
__device__ __forceinline__ uint4 tp_poll_tagged(const uint32_t* p, uint4 v, unsigned tag, long long timeout_ns, unsigned* status) {
  if (v.y == tag && v.w == tag) return v;
  return tp_poll_tagged_slow(p, tag, timeout_ns, status);
}

// Producer tail of the tagged-word push: nothing to announce (the data carries its tag); the last CTA of the grid
// advances this rank's epoch for the consumer kernel that follows in the stream.
__device__ __forceinline__ void tp_tagged_done(const TpPush& tp, unsigned total_ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(tp.arrive, 1u);
    if (prev == total_ctas - 1) {
      atomicExch(tp.arrive, 0u);
      *tp.epoch = *tp.epoch + 1;
    }
  }
}

// Returns once every rank's signal word reached `want`, or after the time limit.  Call with all threads of the
// CTA; contains __syncthreads().
__device__ __forceinline__ void tp_wait_epoch(const TpPull& tp, unsigned want, unsigned* status) {
  if (tp.size > 1 && threadIdx.x < tp.size && !tp_local_only(tp.local_only)) {
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

// Consumer head: waits for the production this rank's own producer kernel (earlier in the stream) has just completed.
__device__ __forceinline__ void tp_pull_wait(const TpPull& tp, unsigned* status) {
  tp_wait_epoch(tp, tp.size > 1 ? *tp.epoch : 0u, status);
}

// Eight summed values (fp32) at element offset `off` of the partial buffers.
__device__ __forceinline__ void tp_load_sum8(const TpReduceSrc& src, bool local, size_t off, float acc[8]) {
  if (local || src.mc_part == nullptr) {
    const int first = local ? src.rank : 0, last = local ? src.rank + 1 : src.size;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int p = first; p < last; ++p) {                 // rank order: identical result on every rank
      const uint4 a = ld_relaxed_sys_v4(src.part[p] + off);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += bf16_lo(aw[j]);
        acc[2 * j + 1] += bf16_hi(aw[j]);
      }
    }
  } else {
    const uint4 a = multimem_ld_reduce_bf16x8(src.mc_part + off);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[2 * j] = bf16_lo(aw[j]);
      acc[2 * j + 1] = bf16_hi(aw[j]);
    }
  }
}

}  // namespace forge

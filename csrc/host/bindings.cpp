// Python bindings: tensors in, raw pointers + the current CUDA stream out.  Every argument is checked here
// (device, dtype, contiguity, shapes, alignment), so a malformed call raises in Python instead of reaching
// a kernel.  No counterpart in the reference (it has no native code).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdint>

extern "C" {
int forge_gemm_bf16(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int n_out, int K, int epi,
                    int force_mode, int force_splits, unsigned* status, cudaStream_t stream);
int forge_gemm_bf16_fused(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int n_out, int K, int epi,
                          int force_mode, int tune, const float* in_ssq, int in_parts, float eps, int add_residual, float* out_ssq,
                          unsigned* status, cudaStream_t stream);
int forge_gemm_bf16_sample(const void* x, int ldx, const void* w, int ldw, int M, int vocab, int K, int vocab_start, const float* temps,
                           const int* header, float* part_v, int* part_i, int* out_i, float* out_v, unsigned* status,
                           cudaStream_t stream);
int forge_gemm_set_trace(unsigned long long* buf);
long long forge_launch_count();
int forge_gemm_bf16_qkv(const void* x, int ldx, const void* w, int ldw, int M, int K, const float* in_ssq, int in_parts, float in_eps,
                        const void* qw, const void* kw, float eps, const float* rope, int rope_rows, const int* positions,
                        const int* slots, void* q_out, void* k_cache, void* v_cache, int nq, int nkv, int block_size,
                        long long num_slots, int do_rope, unsigned* status, cudaStream_t stream);
int forge_gemm_set_streamk_workspace(float* ws, int* counters, int ctas, int tiles);
long long forge_gemm_streamk_workspace_floats(int ctas);
int forge_quant_fp8_1x128(const void* x, void* xq, float* scale, int M, int K, int scale_ld, cudaStream_t stream);
int forge_dequant_fp8_block(const void* wq, const float* scale, void* out, int N, int K, cudaStream_t stream);
int forge_gemm_fp8_splits(int M, int N, int K);
int forge_gemm_fp8_block(const void* xq, const float* xs, int xs_ld, const void* wq, const float* ws, void* out, int ldo, int M,
                         int N, int K, float* partial, unsigned* status, cudaStream_t stream);
int forge_gemm_bf16_tp(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int n_out, int K, int tune,
                       int tp_size, int tp_rank, const long long* signal_ptrs, unsigned* arrive, unsigned* epoch, unsigned* status,
                       cudaStream_t stream);
int forge_gemm_bf16_tp_tagged(const void* x, int ldx, const void* w, int ldw, int M, int n_out, int K, int tune, int tp_size,
                              int tp_rank, const long long* ll_ptrs, int rows_per_rank, unsigned* arrive, unsigned* epoch,
                              unsigned* status, cudaStream_t stream);
int forge_tp_tagged_reduce_norm(int tp_size, int tp_rank, const void* part, int rows_per_rank, const unsigned* part_epoch,
                                const long long* y_ptrs, unsigned* arrive, unsigned* epoch, long long timeout_ns,
                                const unsigned* local_only, const void* residual_in, void* residual_out, const void* w, void* y,
                                int rows, int H, float eps, unsigned* status, cudaStream_t stream);
int forge_tp_reduce_rms_norm(int tp_size, int tp_rank, const long long* part_ptrs, long long mc_part, const void* slots,
                             const unsigned* signal, const unsigned* epoch, long long timeout_ns, const unsigned* local_only,
                             const void* residual_in, void* sum_out, const void* w, void* y, int rows, int H, float eps,
                             unsigned* status, cudaStream_t stream);
int forge_tp_rs_norm_ag(int tp_size, int tp_rank, const long long* part_ptrs, long long mc_part, const unsigned* signal1,
                        const unsigned* epoch1, const long long* y_ptrs, long long mc_y, const long long* signal_ptrs2,
                        unsigned* arrive2, unsigned* epoch2, const unsigned* signal2, long long timeout_ns,
                        const unsigned* local_only, const void* residual_in, void* residual_out, const void* w, int rows, int H,
                        float eps, unsigned* status, cudaStream_t stream);
int forge_tp_embedding_push(const int* ids, const void* w, int T, int H, int vocab_start, int vocab_n, int tp_size, int tp_rank,
                            const long long* slot_ptrs, const long long* signal_ptrs, unsigned* arrive, unsigned* epoch,
                            cudaStream_t stream);
int forge_tp_rows_publish(const void* src, void* part, int rows, int H, int tp_size, int tp_rank, const long long* signal_ptrs,
                          unsigned* arrive, unsigned* epoch, cudaStream_t stream);
int forge_tp_sample_pairs(const float* vals, const int* ids, int rows, int tp_size, int tp_rank, const long long* slot_ptrs,
                          const long long* signal_ptrs, unsigned* arrive, unsigned* epoch, const void* local_slots,
                          long long slot_stride, const unsigned* signal_local, long long timeout_ns, const unsigned* local_only,
                          int* out_i, unsigned* status, cudaStream_t stream);
int forge_rms_norm(const void* x, void* residual, const void* w, void* y, int rows, int H, float eps, cudaStream_t stream);
int forge_qk_norm_rope_store(const void* qkv, int ld_qkv, const void* qw, const void* kw, float eps, const float* rope,
                             int rope_rows, const int* positions, const int* slots, void* q_out, void* k_cache, void* v_cache,
                             int T, int nq, int nkv, int D, int block_size, long long num_slots, int do_rope, unsigned* status,
                             cudaStream_t stream);
int forge_silu_mul(const void* x, void* out, long long rows, int I, cudaStream_t stream);
int forge_embedding(const int* ids, const void* w, void* out, int T, int H, int vocab_start, int vocab_n, float* ssq, int parts,
                    cudaStream_t stream);
int forge_gather_rows(const int* idx, const void* x, void* out, int S, int H, int x_rows, cudaStream_t stream);
int forge_feed_tokens(int* ids, const int* src_rows, const int* prev_tokens, int n, int prev_n, cudaStream_t stream);
int forge_sample_nsplit(int rows, int vocab);
int forge_sample(const void* logits, int ld, int rows, int vocab, int vocab_start, const float* temps, const int* header,
                 float* part_v, int* part_i, int nsplit, int* out_i, float* out_v, cudaStream_t stream);
int forge_sample_merge_ranks(const float* vals, const int* ids, int ranks, int rows, int* out_i, cudaStream_t stream);
int forge_decode_attention(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out,
                           float* part_o, float* part_ml, int B, int nq, int nkv, int head_dim, int block_size, int table_width,
                           int num_blocks, int chunk, int max_chunks, float scale, unsigned* status, cudaStream_t stream);
size_t forge_decode_attention_flat_scratch_floats(int num_ctas, int B, int nq, int nkv);
int forge_decode_attention_flat_ctas_per_sm(int nq, int nkv, int block_size, int from_raw_qkv);
void forge_decode_attention_set_tc_min_group(int g);
int forge_decode_attention_flat(const void* q, const void* kc, const void* vc, const int* bt, const int* lens, void* out,
                                float* scratch, int num_ctas, int B, int nq, int nkv, int head_dim, int block_size, int table_width,
                                int num_blocks, float scale, unsigned* status, cudaStream_t stream);
int forge_decode_attention_qkv(const void* qkv, int ld_qkv, const void* q_w, const void* k_w, float eps, const float* rope,
                               int rope_rows, void* kc, void* vc, const int* bt, const int* lens, void* out, float* scratch,
                               int num_ctas, float* part_o, float* part_ml, int chunk, int max_chunks, int B, int nq, int nkv,
                               int head_dim, int block_size, int table_width, int num_blocks, float scale, unsigned* status,
                               cudaStream_t stream);
int forge_prefill_attention(const void* q, const void* kc, const void* vc, const int* cu_q, const int* lens, const int* bt,
                            void* out, int T, int num_seqs, int max_q, int nq, int nkv, int head_dim, int block_size,
                            int table_width, int num_blocks, float scale, unsigned* status, cudaStream_t stream);
}

namespace {

using torch::Tensor;

#define CHECK_CUDA_CONTIG(t) TORCH_CHECK((t).is_cuda() && (t).is_contiguous(), #t " must be a contiguous CUDA tensor")
#define CHECK_BF16(t) TORCH_CHECK((t).scalar_type() == at::kBFloat16, #t " must be bfloat16")
#define CHECK_I32(t) TORCH_CHECK((t).scalar_type() == at::kInt, #t " must be int32")
#define CHECK_F32(t) TORCH_CHECK((t).scalar_type() == at::kFloat, #t " must be float32")

cudaStream_t stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

unsigned* status_ptr(const Tensor& status) {
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1, "status must be a CUDA int32 tensor");
  return reinterpret_cast<unsigned*>(status.data_ptr<int>());
}

void check(int rc, const char* what) { TORCH_CHECK(rc == 0, what, " failed with code ", rc); }

// out[M, n_out] = epilogue(x[M, K] @ w[*, K]^T); epi 0: store, 1: silu(gate) * up with w = [2 * n_out, K].
void gemm(const Tensor& x, const Tensor& w, Tensor& out, int64_t epi, int64_t force_mode, int64_t force_splits,
          const Tensor& status) {
  CHECK_BF16(x); CHECK_BF16(w); CHECK_BF16(out);
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && out.is_cuda(), "gemm: CUDA tensors expected");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm: 2-D tensors expected");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1, "gemm: innermost stride must be 1");
  const int64_t M = x.size(0), K = x.size(1);
  TORCH_CHECK(w.size(1) == K, "gemm: K mismatch");
  const int64_t n_out = epi == 1 ? w.size(0) / 2 : w.size(0);
  TORCH_CHECK(out.size(0) == M && out.size(1) == n_out, "gemm: bad output shape");
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_gemm_bf16(x.data_ptr(), static_cast<int>(x.stride(0)), w.data_ptr(), static_cast<int>(w.stride(0)), out.data_ptr(),
                        static_cast<int>(out.stride(0)), static_cast<int>(M), static_cast<int>(n_out), static_cast<int>(K),
                        static_cast<int>(epi), static_cast<int>(force_mode), static_cast<int>(force_splits), status_ptr(status),
                        stream_of(x)),
        "forge_gemm_bf16");
}

// The GEMM with the neighbouring RMSNorm / residual add fused in.  in_ssq (fp32 [M, parts]): the rows of x are un-normalised,
// the norm weight is folded into w, and output row r is scaled by rsqrt(sum(in_ssq[r]) / K + eps).  add_residual: out is the
// residual stream, updated in place (out += x @ w.T, rounded as the separate kernels would); out_ssq (fp32
// [M, ceil(n_out / 128)]) receives the sums of squares of the new rows per 128 features.
void gemm_fused(const Tensor& x, const Tensor& w, Tensor& out, int64_t epi, int64_t force_mode, int64_t tune,
                const c10::optional<Tensor>& in_ssq, double eps, bool add_residual, const c10::optional<Tensor>& out_ssq,
                const Tensor& status) {
  CHECK_BF16(x); CHECK_BF16(w); CHECK_BF16(out);
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && out.is_cuda(), "gemm_fused: CUDA tensors expected");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm_fused: 2-D tensors expected");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1, "gemm_fused: innermost stride must be 1");
  const int64_t M = x.size(0), K = x.size(1);
  TORCH_CHECK(w.size(1) == K, "gemm_fused: K mismatch");
  const int64_t n_out = epi == 1 ? w.size(0) / 2 : w.size(0);
  TORCH_CHECK(out.size(0) == M && out.size(1) == n_out, "gemm_fused: bad output shape");
  TORCH_CHECK(!(add_residual && epi != 0), "gemm_fused: the residual add goes with the plain epilogue");
  const float* in_p = nullptr;
  float* out_p = nullptr;
  int in_parts = 0;
  if (in_ssq.has_value()) {
    CHECK_CUDA_CONTIG(*in_ssq); CHECK_F32(*in_ssq);
    TORCH_CHECK(in_ssq->dim() == 2 && in_ssq->size(0) >= M && in_ssq->size(1) >= 1, "gemm_fused: in_ssq must be [>= M, parts]");
    in_p = in_ssq->data_ptr<float>();
    in_parts = static_cast<int>(in_ssq->size(1));
  }
  if (out_ssq.has_value()) {
    CHECK_CUDA_CONTIG(*out_ssq); CHECK_F32(*out_ssq);
    TORCH_CHECK(out_ssq->dim() == 2 && out_ssq->size(0) >= M && out_ssq->size(1) == (n_out + 127) / 128, "gemm_fused: out_ssq must be [>= M, ceil(n_out / 128)]");
    out_p = out_ssq->data_ptr<float>();
  }
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_gemm_bf16_fused(x.data_ptr(), static_cast<int>(x.stride(0)), w.data_ptr(), static_cast<int>(w.stride(0)), out.data_ptr(),
                              static_cast<int>(out.stride(0)), static_cast<int>(M), static_cast<int>(n_out), static_cast<int>(K),
                              static_cast<int>(epi), static_cast<int>(force_mode), static_cast<int>(tune), in_p, in_parts,
                              static_cast<float>(eps), add_residual ? 1 : 0, out_p, status_ptr(status), stream_of(x)),
        "forge_gemm_bf16_fused");
}

// LM head + sampling: x [rows, K] @ w [vocab, K]^T, sampled per row without writing the logits.  part_v / part_i: scratch of
// rows * ceil(vocab / 256) entries; out_i / out_v: the winning global id and its score per row.
void gemm_sample(const Tensor& x, const Tensor& w, int64_t vocab_start, const Tensor& temps, const Tensor& header, Tensor& part_v,
                 Tensor& part_i, Tensor& out_i, Tensor& out_v, const Tensor& status) {
  CHECK_BF16(x); CHECK_BF16(w); CHECK_CUDA_CONTIG(temps); CHECK_F32(temps); CHECK_CUDA_CONTIG(header); CHECK_I32(header);
  CHECK_CUDA_CONTIG(part_v); CHECK_F32(part_v); CHECK_CUDA_CONTIG(part_i); CHECK_I32(part_i);
  CHECK_CUDA_CONTIG(out_i); CHECK_I32(out_i); CHECK_CUDA_CONTIG(out_v); CHECK_F32(out_v);
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && w.size(1) == x.size(1),
              "gemm_sample: operands");
  const int64_t rows = x.size(0), vocab = w.size(0), tiles = (vocab + 255) / 256;
  TORCH_CHECK(temps.numel() >= rows && header.numel() >= 12 && out_i.numel() >= rows && out_v.numel() >= rows &&
                  part_v.numel() >= rows * tiles && part_i.numel() >= rows * tiles,
              "gemm_sample: lengths");
  TORCH_CHECK(vocab_start % 32 == 0, "gemm_sample: the vocabulary shard must start on a multiple of 32");
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_gemm_bf16_sample(x.data_ptr(), static_cast<int>(x.stride(0)), w.data_ptr(), static_cast<int>(w.stride(0)),
                               static_cast<int>(rows), static_cast<int>(vocab), static_cast<int>(x.size(1)),
                               static_cast<int>(vocab_start), temps.data_ptr<float>(), header.data_ptr<int>(), part_v.data_ptr<float>(),
                               part_i.data_ptr<int>(), out_i.data_ptr<int>(), out_v.data_ptr<float>(), status_ptr(status), stream_of(x)),
        "forge_gemm_bf16_sample");
}

// Phase timeline of the decode GEMM (profiling aid): int64 CUDA tensor of >= 8 * CTAs entries, or None to switch off.
void gemm_set_trace(const c10::optional<Tensor>& buf) {
  unsigned long long* p = nullptr;
  if (buf.has_value()) {
    TORCH_CHECK(buf->is_cuda() && buf->is_contiguous() && buf->scalar_type() == at::kLong, "trace buffer must be a CUDA int64 tensor");
    p = reinterpret_cast<unsigned long long*>(buf->data_ptr<int64_t>());
  }
  check(forge_gemm_set_trace(p), "forge_gemm_set_trace");
}

void rms_norm(const Tensor& x, const c10::optional<Tensor>& residual, const Tensor& w, Tensor& y, double eps) {
  CHECK_CUDA_CONTIG(x); CHECK_CUDA_CONTIG(w); CHECK_CUDA_CONTIG(y);
  CHECK_BF16(x); CHECK_BF16(w); CHECK_BF16(y);
  const int64_t H = x.size(-1), rows = x.numel() / H;
  TORCH_CHECK(w.numel() == H && y.numel() == x.numel(), "rms_norm: shape mismatch");
  void* res = nullptr;
  if (residual.has_value()) {
    CHECK_CUDA_CONTIG(*residual); CHECK_BF16(*residual);
    TORCH_CHECK(residual->numel() == x.numel(), "rms_norm: residual shape mismatch");
    res = residual->data_ptr();
  }
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_rms_norm(x.data_ptr(), res, w.data_ptr(), y.data_ptr(), static_cast<int>(rows), static_cast<int>(H),
                       static_cast<float>(eps), stream_of(x)),
        "forge_rms_norm");
}

void qk_norm_rope_store(const Tensor& qkv, const c10::optional<Tensor>& qw, const c10::optional<Tensor>& kw, double eps,
                        const Tensor& rope, const Tensor& positions, const Tensor& slots, Tensor& q_out, Tensor& k_cache,
                        Tensor& v_cache, int64_t nq, int64_t nkv, bool do_rope, const Tensor& status) {
  CHECK_BF16(qkv); CHECK_CUDA_CONTIG(q_out); CHECK_BF16(q_out);
  CHECK_CUDA_CONTIG(k_cache); CHECK_CUDA_CONTIG(v_cache); CHECK_BF16(k_cache); CHECK_BF16(v_cache);
  CHECK_CUDA_CONTIG(rope); CHECK_F32(rope); CHECK_CUDA_CONTIG(positions); CHECK_I32(positions);
  CHECK_CUDA_CONTIG(slots); CHECK_I32(slots);
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 2 && qkv.stride(1) == 1, "qkv must be [T, (nq + 2 nkv) * D]");
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes(), "caches must be [blocks, kv_heads, block_size, D]");
  const int64_t T = qkv.size(0), D = k_cache.size(3), bs = k_cache.size(2);
  TORCH_CHECK(qkv.size(1) == (nq + 2 * nkv) * D && k_cache.size(1) == nkv, "qk_norm_rope_store: head layout mismatch");
  TORCH_CHECK(positions.numel() >= T && slots.numel() >= T && q_out.numel() == T * nq * D, "qk_norm_rope_store: length mismatch");
  TORCH_CHECK(rope.dim() == 2 && rope.size(1) == D, "rope table must be [positions, D]");
  const void* qwp = nullptr;
  const void* kwp = nullptr;
  if (qw.has_value()) { CHECK_CUDA_CONTIG(*qw); CHECK_BF16(*qw); TORCH_CHECK(qw->numel() == D); qwp = qw->data_ptr(); }
  if (kw.has_value()) { CHECK_CUDA_CONTIG(*kw); CHECK_BF16(*kw); TORCH_CHECK(kw->numel() == D); kwp = kw->data_ptr(); }
  const c10::cuda::CUDAGuard guard(qkv.device());
  check(forge_qk_norm_rope_store(qkv.data_ptr(), static_cast<int>(qkv.stride(0)), qwp, kwp, static_cast<float>(eps),
                                 rope.data_ptr<float>(), static_cast<int>(rope.size(0)), positions.data_ptr<int>(),
                                 slots.data_ptr<int>(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                 static_cast<int>(T), static_cast<int>(nq), static_cast<int>(nkv), static_cast<int>(D),
                                 static_cast<int>(bs), static_cast<long long>(k_cache.size(0)) * bs, do_rope ? 1 : 0,
                                 status_ptr(status), stream_of(qkv)),
        "forge_qk_norm_rope_store");
}

// qkv projection whose epilogue normalises q and k per head, rotates them and writes k / v into the cache (head_dim 128).
void gemm_qkv_rope_store(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& in_ssq, double in_eps,
                         const c10::optional<Tensor>& qw, const c10::optional<Tensor>& kw, double eps, const Tensor& rope,
                         const Tensor& positions, const Tensor& slots, Tensor& q_out, Tensor& k_cache, Tensor& v_cache, int64_t nq,
                         int64_t nkv, bool do_rope, const Tensor& status) {
  CHECK_BF16(x); CHECK_BF16(w); CHECK_CUDA_CONTIG(q_out); CHECK_BF16(q_out);
  CHECK_CUDA_CONTIG(k_cache); CHECK_CUDA_CONTIG(v_cache); CHECK_BF16(k_cache); CHECK_BF16(v_cache);
  CHECK_CUDA_CONTIG(rope); CHECK_F32(rope); CHECK_CUDA_CONTIG(positions); CHECK_I32(positions);
  CHECK_CUDA_CONTIG(slots); CHECK_I32(slots);
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1, "gemm_qkv_rope_store: x [T, K], w [N, K]");
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes() && k_cache.size(3) == 128, "caches must be [blocks, kv_heads, block_size, 128]");
  const int64_t T = x.size(0), K = x.size(1), bs = k_cache.size(2);
  TORCH_CHECK(w.size(1) == K && w.size(0) == (nq + 2 * nkv) * 128 && k_cache.size(1) == nkv, "gemm_qkv_rope_store: head layout mismatch");
  TORCH_CHECK(positions.numel() >= T && slots.numel() >= T && q_out.numel() == T * nq * 128, "gemm_qkv_rope_store: length mismatch");
  TORCH_CHECK(rope.dim() == 2 && rope.size(1) == 128, "rope table must be [positions, 128]");
  const float* in_p = nullptr;
  int in_parts = 0;
  if (in_ssq.has_value()) {
    CHECK_CUDA_CONTIG(*in_ssq); CHECK_F32(*in_ssq);
    TORCH_CHECK(in_ssq->dim() == 2 && in_ssq->size(0) >= T && in_ssq->size(1) >= 1, "gemm_qkv_rope_store: in_ssq must be [>= T, parts]");
    in_p = in_ssq->data_ptr<float>();
    in_parts = static_cast<int>(in_ssq->size(1));
  }
  const void* qwp = nullptr;
  const void* kwp = nullptr;
  if (qw.has_value()) { CHECK_CUDA_CONTIG(*qw); CHECK_BF16(*qw); TORCH_CHECK(qw->numel() == 128); qwp = qw->data_ptr(); }
  if (kw.has_value()) { CHECK_CUDA_CONTIG(*kw); CHECK_BF16(*kw); TORCH_CHECK(kw->numel() == 128); kwp = kw->data_ptr(); }
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_gemm_bf16_qkv(x.data_ptr(), static_cast<int>(x.stride(0)), w.data_ptr(), static_cast<int>(w.stride(0)), static_cast<int>(T),
                            static_cast<int>(K), in_p, in_parts, static_cast<float>(in_eps), qwp, kwp, static_cast<float>(eps),
                            rope.data_ptr<float>(), static_cast<int>(rope.size(0)), positions.data_ptr<int>(), slots.data_ptr<int>(),
                            q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), static_cast<int>(nq), static_cast<int>(nkv),
                            static_cast<int>(bs), static_cast<long long>(k_cache.size(0)) * bs, do_rope ? 1 : 0, status_ptr(status),
                            stream_of(x)),
        "forge_gemm_bf16_qkv");
}

void silu_mul(const Tensor& x, Tensor& out) {
  CHECK_CUDA_CONTIG(x); CHECK_CUDA_CONTIG(out); CHECK_BF16(x); CHECK_BF16(out);
  const int64_t I = x.size(-1) / 2, rows = x.numel() / (2 * I);
  TORCH_CHECK(out.numel() == rows * I, "silu_mul: bad output shape");
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_silu_mul(x.data_ptr(), out.data_ptr(), rows, static_cast<int>(I), stream_of(x)), "forge_silu_mul");
}

// ssq (optional, fp32 [T, parts]): column 0 receives the sums of squares of the rows written, the other columns zero.
void embedding(const Tensor& ids, const Tensor& w, Tensor& out, int64_t vocab_start, const c10::optional<Tensor>& ssq) {
  CHECK_CUDA_CONTIG(ids); CHECK_I32(ids); CHECK_CUDA_CONTIG(w); CHECK_BF16(w); CHECK_CUDA_CONTIG(out); CHECK_BF16(out);
  const int64_t T = ids.numel(), H = w.size(1);
  TORCH_CHECK(out.numel() == T * H, "embedding: bad output shape");
  float* sp = nullptr;
  int parts = 0;
  if (ssq.has_value()) {
    CHECK_CUDA_CONTIG(*ssq); CHECK_F32(*ssq);
    TORCH_CHECK(ssq->dim() == 2 && ssq->size(0) == T && ssq->size(1) >= 1, "embedding: ssq must be [tokens, parts]");
    sp = ssq->data_ptr<float>();
    parts = static_cast<int>(ssq->size(1));
  }
  const c10::cuda::CUDAGuard guard(w.device());
  check(forge_embedding(ids.data_ptr<int>(), w.data_ptr(), out.data_ptr(), static_cast<int>(T), static_cast<int>(H),
                        static_cast<int>(vocab_start), static_cast<int>(w.size(0)), sp, parts, stream_of(w)),
        "forge_embedding");
}

void gather_rows(const Tensor& idx, const Tensor& x, Tensor& out) {
  CHECK_CUDA_CONTIG(idx); CHECK_I32(idx); CHECK_CUDA_CONTIG(x); CHECK_BF16(x); CHECK_CUDA_CONTIG(out); CHECK_BF16(out);
  const int64_t S = idx.numel(), H = x.size(1);
  TORCH_CHECK(out.numel() == S * H, "gather_rows: bad output shape");
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_gather_rows(idx.data_ptr<int>(), x.data_ptr(), out.data_ptr(), static_cast<int>(S), static_cast<int>(H),
                          static_cast<int>(x.size(0)), stream_of(x)),
        "forge_gather_rows");
}

void feed_tokens(Tensor& ids, const Tensor& src_rows, const Tensor& prev_tokens) {
  CHECK_CUDA_CONTIG(ids); CHECK_I32(ids); CHECK_CUDA_CONTIG(src_rows); CHECK_I32(src_rows); CHECK_CUDA_CONTIG(prev_tokens); CHECK_I32(prev_tokens);
  TORCH_CHECK(src_rows.numel() >= ids.numel(), "feed_tokens: src_rows too short");
  const c10::cuda::CUDAGuard guard(ids.device());
  check(forge_feed_tokens(ids.data_ptr<int>(), src_rows.data_ptr<int>(), prev_tokens.data_ptr<int>(), static_cast<int>(ids.numel()),
                          static_cast<int>(prev_tokens.numel()), stream_of(ids)),
        "forge_feed_tokens");
}

int64_t sample_nsplit(int64_t rows, int64_t vocab) { return forge_sample_nsplit(static_cast<int>(rows), static_cast<int>(vocab)); }

// logits [rows, vocab] bf16; header = first words of the packed step buffer (step index, seed) on the device.
void sample(const Tensor& logits, int64_t vocab_start, const Tensor& temps, const Tensor& header, Tensor& part_v, Tensor& part_i,
            Tensor& out_i, const c10::optional<Tensor>& out_v) {
  CHECK_BF16(logits); CHECK_CUDA_CONTIG(temps); CHECK_F32(temps); CHECK_CUDA_CONTIG(header); CHECK_I32(header);
  CHECK_CUDA_CONTIG(part_v); CHECK_F32(part_v); CHECK_CUDA_CONTIG(part_i); CHECK_I32(part_i); CHECK_CUDA_CONTIG(out_i); CHECK_I32(out_i);
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "logits must be [rows, vocab]");
  const int64_t rows = logits.size(0), vocab = logits.size(1);
  TORCH_CHECK(temps.numel() >= rows && out_i.numel() >= rows && header.numel() >= 12, "sample: length mismatch");
  TORCH_CHECK(part_v.numel() == part_i.numel() && part_v.numel() % rows == 0 && part_v.numel() >= rows, "sample: bad scratch");
  const int nsplit = static_cast<int>(part_v.numel() / rows);
  float* ov = nullptr;
  if (out_v.has_value()) { CHECK_CUDA_CONTIG(*out_v); CHECK_F32(*out_v); TORCH_CHECK(out_v->numel() >= rows); ov = out_v->data_ptr<float>(); }
  const c10::cuda::CUDAGuard guard(logits.device());
  check(forge_sample(logits.data_ptr(), static_cast<int>(logits.stride(0)), static_cast<int>(rows), static_cast<int>(vocab),
                     static_cast<int>(vocab_start), temps.data_ptr<float>(), header.data_ptr<int>(), part_v.data_ptr<float>(),
                     part_i.data_ptr<int>(), nsplit, out_i.data_ptr<int>(), ov, stream_of(logits)),
        "forge_sample");
}

void sample_merge_ranks(const Tensor& vals, const Tensor& ids, Tensor& out_i) {
  CHECK_CUDA_CONTIG(vals); CHECK_F32(vals); CHECK_CUDA_CONTIG(ids); CHECK_I32(ids); CHECK_CUDA_CONTIG(out_i); CHECK_I32(out_i);
  TORCH_CHECK(vals.dim() == 2 && ids.sizes() == vals.sizes() && out_i.numel() >= vals.size(1), "sample_merge_ranks: shapes");
  const c10::cuda::CUDAGuard guard(vals.device());
  check(forge_sample_merge_ranks(vals.data_ptr<float>(), ids.data_ptr<int>(), static_cast<int>(vals.size(0)),
                                 static_cast<int>(vals.size(1)), out_i.data_ptr<int>(), stream_of(vals)),
        "forge_sample_merge_ranks");
}

void decode_attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_tables,
                      const Tensor& context_lens, Tensor& out, const c10::optional<Tensor>& part_o,
                      const c10::optional<Tensor>& part_ml, int64_t chunk, int64_t max_chunks, double scale, const Tensor& status) {
  CHECK_CUDA_CONTIG(q); CHECK_BF16(q); CHECK_CUDA_CONTIG(k_cache); CHECK_BF16(k_cache); CHECK_CUDA_CONTIG(v_cache); CHECK_BF16(v_cache);
  CHECK_CUDA_CONTIG(block_tables); CHECK_I32(block_tables); CHECK_CUDA_CONTIG(context_lens); CHECK_I32(context_lens);
  CHECK_CUDA_CONTIG(out); CHECK_BF16(out);
  TORCH_CHECK(q.dim() == 3 && k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes() && block_tables.dim() == 2, "decode_attention: ranks");
  const int64_t B = q.size(0), nq = q.size(1), D = q.size(2), nkv = k_cache.size(1), bs = k_cache.size(2);
  TORCH_CHECK(k_cache.size(3) == D && block_tables.size(0) >= B && context_lens.numel() >= B && out.numel() == B * nq * D,
              "decode_attention: shape mismatch");
  TORCH_CHECK(max_chunks * chunk >= 1, "decode_attention: bad chunking");
  float* po = nullptr;
  float* pml = nullptr;
  if (max_chunks > 1) {
    TORCH_CHECK(part_o.has_value() && part_ml.has_value(), "decode_attention: scratch needed when max_chunks > 1");
    CHECK_CUDA_CONTIG(*part_o); CHECK_F32(*part_o); CHECK_CUDA_CONTIG(*part_ml); CHECK_F32(*part_ml);
    TORCH_CHECK(part_o->numel() >= B * nq * max_chunks * D && part_ml->numel() >= B * nq * max_chunks * 2, "decode_attention: scratch too small");
    po = part_o->data_ptr<float>();
    pml = part_ml->data_ptr<float>();
  }
  const c10::cuda::CUDAGuard guard(q.device());
  check(forge_decode_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr<int>(),
                               context_lens.data_ptr<int>(), out.data_ptr(), po, pml, static_cast<int>(B), static_cast<int>(nq),
                               static_cast<int>(nkv), static_cast<int>(D), static_cast<int>(bs), static_cast<int>(block_tables.size(1)),
                               static_cast<int>(k_cache.size(0)), static_cast<int>(chunk), static_cast<int>(max_chunks),
                               static_cast<float>(scale), status_ptr(status), stream_of(q)),
        "forge_decode_attention");
}

int64_t decode_attention_flat_scratch_floats(int64_t num_ctas, int64_t B, int64_t nq, int64_t nkv) {
  return static_cast<int64_t>(forge_decode_attention_flat_scratch_floats(static_cast<int>(num_ctas), static_cast<int>(B),
                                                                         static_cast<int>(nq), static_cast<int>(nkv)));
}

// CTAs per SM the flat decode kernel runs with for this head grouping (grid = this x the SM count).
int64_t decode_attention_flat_ctas_per_sm(int64_t nq, int64_t nkv, int64_t block_size, bool from_raw_qkv) {
  return forge_decode_attention_flat_ctas_per_sm(static_cast<int>(nq), static_cast<int>(nkv), static_cast<int>(block_size), from_raw_qkv ? 1 : 0);
}

// Decode attention with the flat tile partition: num_ctas CTAs share all KV tiles equally.  scratch: fp32, at least
// decode_attention_flat_scratch_floats(num_ctas, B, nq, nkv) elements.
void decode_attention_flat(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_tables,
                           const Tensor& context_lens, Tensor& out, Tensor& scratch, int64_t num_ctas, double scale, const Tensor& status) {
  CHECK_CUDA_CONTIG(q); CHECK_BF16(q); CHECK_CUDA_CONTIG(k_cache); CHECK_BF16(k_cache); CHECK_CUDA_CONTIG(v_cache); CHECK_BF16(v_cache);
  CHECK_CUDA_CONTIG(block_tables); CHECK_I32(block_tables); CHECK_CUDA_CONTIG(context_lens); CHECK_I32(context_lens);
  CHECK_CUDA_CONTIG(out); CHECK_BF16(out); CHECK_CUDA_CONTIG(scratch); CHECK_F32(scratch);
  TORCH_CHECK(q.dim() == 3 && k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes() && block_tables.dim() == 2, "decode_attention_flat: ranks");
  const int64_t B = q.size(0), nq = q.size(1), D = q.size(2), nkv = k_cache.size(1), bs = k_cache.size(2);
  TORCH_CHECK(k_cache.size(3) == D && block_tables.size(0) >= B && context_lens.numel() >= B && out.numel() == B * nq * D,
              "decode_attention_flat: shape mismatch");
  TORCH_CHECK(B <= 512, "decode_attention_flat: at most 512 sequences");
  TORCH_CHECK(num_ctas >= 1 && scratch.numel() >= decode_attention_flat_scratch_floats(num_ctas, B, nq, nkv),
              "decode_attention_flat: scratch too small");
  const c10::cuda::CUDAGuard guard(q.device());
  check(forge_decode_attention_flat(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr<int>(),
                                    context_lens.data_ptr<int>(), out.data_ptr(), scratch.data_ptr<float>(), static_cast<int>(num_ctas),
                                    static_cast<int>(B), static_cast<int>(nq), static_cast<int>(nkv), static_cast<int>(D),
                                    static_cast<int>(bs), static_cast<int>(block_tables.size(1)), static_cast<int>(k_cache.size(0)),
                                    static_cast<float>(scale), status_ptr(status), stream_of(q)),
        "forge_decode_attention_flat");
}

// Decode attention from the raw qkv projection [B, (nq + 2 nkv) * D]: q/k-norm, rotation and the KV store of the step's
// token are done inside the attention kernel.  num_ctas > 0: flat partition with `scratch`; num_ctas == 0: context chunks
// with part_o / part_ml.
void decode_attention_qkv(const Tensor& qkv, const c10::optional<Tensor>& qw, const c10::optional<Tensor>& kw, double eps,
                          const c10::optional<Tensor>& rope, Tensor& k_cache, Tensor& v_cache, const Tensor& block_tables,
                          const Tensor& context_lens, Tensor& out, const c10::optional<Tensor>& scratch, int64_t num_ctas,
                          const c10::optional<Tensor>& part_o, const c10::optional<Tensor>& part_ml, int64_t chunk, int64_t max_chunks,
                          int64_t nq, double scale, const Tensor& status) {
  CHECK_BF16(qkv); CHECK_CUDA_CONTIG(k_cache); CHECK_BF16(k_cache); CHECK_CUDA_CONTIG(v_cache); CHECK_BF16(v_cache);
  CHECK_CUDA_CONTIG(block_tables); CHECK_I32(block_tables); CHECK_CUDA_CONTIG(context_lens); CHECK_I32(context_lens);
  CHECK_CUDA_CONTIG(out); CHECK_BF16(out);
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 2 && qkv.stride(1) == 1, "qkv must be [B, (nq + 2 nkv) * D]");
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes() && block_tables.dim() == 2, "decode_attention_qkv: ranks");
  const int64_t B = qkv.size(0), nkv = k_cache.size(1), bs = k_cache.size(2), D = k_cache.size(3);
  TORCH_CHECK(qkv.size(1) == (nq + 2 * nkv) * D && block_tables.size(0) >= B && context_lens.numel() >= B && out.numel() == B * nq * D,
              "decode_attention_qkv: shape mismatch");
  const void* qwp = nullptr; const void* kwp = nullptr; const float* rp = nullptr; int rope_rows = 0;
  if (qw.has_value()) { CHECK_CUDA_CONTIG(*qw); CHECK_BF16(*qw); TORCH_CHECK(qw->numel() == D); qwp = qw->data_ptr(); }
  if (kw.has_value()) { CHECK_CUDA_CONTIG(*kw); CHECK_BF16(*kw); TORCH_CHECK(kw->numel() == D); kwp = kw->data_ptr(); }
  if (rope.has_value()) {
    CHECK_CUDA_CONTIG(*rope); CHECK_F32(*rope); TORCH_CHECK(rope->dim() == 2 && rope->size(1) == D, "rope table must be [positions, D]");
    rp = rope->data_ptr<float>(); rope_rows = static_cast<int>(rope->size(0));
  }
  float* sp = nullptr; float* po = nullptr; float* pml = nullptr;
  if (num_ctas > 0) {
    TORCH_CHECK(scratch.has_value() && B <= 512, "decode_attention_qkv: flat partition needs scratch and at most 512 sequences");
    CHECK_CUDA_CONTIG(*scratch); CHECK_F32(*scratch);
    TORCH_CHECK(scratch->numel() >= decode_attention_flat_scratch_floats(num_ctas, B, nq, nkv), "decode_attention_qkv: scratch too small");
    sp = scratch->data_ptr<float>();
  } else if (max_chunks > 1) {
    TORCH_CHECK(part_o.has_value() && part_ml.has_value(), "decode_attention_qkv: scratch needed when max_chunks > 1");
    CHECK_CUDA_CONTIG(*part_o); CHECK_F32(*part_o); CHECK_CUDA_CONTIG(*part_ml); CHECK_F32(*part_ml);
    TORCH_CHECK(part_o->numel() >= B * nq * max_chunks * D && part_ml->numel() >= B * nq * max_chunks * 2, "decode_attention_qkv: scratch too small");
    po = part_o->data_ptr<float>(); pml = part_ml->data_ptr<float>();
  }
  const c10::cuda::CUDAGuard guard(qkv.device());
  check(forge_decode_attention_qkv(qkv.data_ptr(), static_cast<int>(qkv.stride(0)), qwp, kwp, static_cast<float>(eps), rp, rope_rows,
                                   k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr<int>(), context_lens.data_ptr<int>(),
                                   out.data_ptr(), sp, static_cast<int>(num_ctas), po, pml, static_cast<int>(chunk),
                                   static_cast<int>(max_chunks), static_cast<int>(B), static_cast<int>(nq), static_cast<int>(nkv),
                                   static_cast<int>(D), static_cast<int>(bs), static_cast<int>(block_tables.size(1)),
                                   static_cast<int>(k_cache.size(0)), static_cast<float>(scale), status_ptr(status), stream_of(qkv)),
        "forge_decode_attention_qkv");
}

void prefill_attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& cu_seqlens_q,
                       const Tensor& context_lens, const Tensor& block_tables, Tensor& out, int64_t num_seqs, int64_t max_q,
                       double scale, const Tensor& status) {
  CHECK_CUDA_CONTIG(q); CHECK_BF16(q); CHECK_CUDA_CONTIG(k_cache); CHECK_BF16(k_cache); CHECK_CUDA_CONTIG(v_cache); CHECK_BF16(v_cache);
  CHECK_CUDA_CONTIG(cu_seqlens_q); CHECK_I32(cu_seqlens_q); CHECK_CUDA_CONTIG(context_lens); CHECK_I32(context_lens);
  CHECK_CUDA_CONTIG(block_tables); CHECK_I32(block_tables); CHECK_CUDA_CONTIG(out); CHECK_BF16(out);
  TORCH_CHECK(q.dim() == 3 && k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes() && block_tables.dim() == 2, "prefill_attention: ranks");
  const int64_t T = q.size(0), nq = q.size(1), D = q.size(2), nkv = k_cache.size(1), bs = k_cache.size(2);
  TORCH_CHECK(cu_seqlens_q.numel() >= num_seqs + 1 && context_lens.numel() >= num_seqs && block_tables.size(0) >= num_seqs &&
                  out.numel() == T * nq * D && k_cache.size(3) == D,
              "prefill_attention: shape mismatch");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(q.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(k_cache.data_ptr()) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(v_cache.data_ptr()) & 15) == 0,
              "prefill_attention: 16-byte alignment needed");
  const c10::cuda::CUDAGuard guard(q.device());
  check(forge_prefill_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), cu_seqlens_q.data_ptr<int>(),
                                context_lens.data_ptr<int>(), block_tables.data_ptr<int>(), out.data_ptr(), static_cast<int>(T),
                                static_cast<int>(num_seqs), static_cast<int>(max_q), static_cast<int>(nq), static_cast<int>(nkv),
                                static_cast<int>(D), static_cast<int>(bs), static_cast<int>(block_tables.size(1)),
                                static_cast<int>(k_cache.size(0)), static_cast<float>(scale), status_ptr(status), stream_of(q)),
        "forge_prefill_attention");
}

// ---- block-scaled fp8: xq/wq are uint8 views of e4m3 data.
void quant_fp8(const Tensor& x, Tensor& xq, Tensor& scale) {
  CHECK_CUDA_CONTIG(x); CHECK_BF16(x); CHECK_CUDA_CONTIG(xq); CHECK_CUDA_CONTIG(scale); CHECK_F32(scale);
  TORCH_CHECK(x.dim() == 2 && xq.numel() == x.numel() && xq.element_size() == 1, "quant_fp8: shapes");
  const int64_t M = x.size(0), K = x.size(1);
  TORCH_CHECK(K % 128 == 0 && scale.dim() == 2 && scale.size(0) == K / 128 && scale.size(1) >= M, "quant_fp8: scale must be [K / 128, >= M]");
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_quant_fp8_1x128(x.data_ptr(), xq.data_ptr(), scale.data_ptr<float>(), static_cast<int>(M), static_cast<int>(K),
                              static_cast<int>(scale.size(1)), stream_of(x)),
        "forge_quant_fp8_1x128");
}

int64_t gemm_fp8_splits(int64_t M, int64_t N, int64_t K) {
  return forge_gemm_fp8_splits(static_cast<int>(M), static_cast<int>(N), static_cast<int>(K));
}

// partial: fp32 workspace of gemm_fp8_splits(M, N, K) * M * N elements; without it K is not split.
void gemm_fp8_block(const Tensor& xq, const Tensor& xs, const Tensor& wq, const Tensor& ws, Tensor& out,
                    const c10::optional<Tensor>& partial, const Tensor& status) {
  CHECK_CUDA_CONTIG(xq); CHECK_CUDA_CONTIG(wq); CHECK_CUDA_CONTIG(xs); CHECK_F32(xs); CHECK_CUDA_CONTIG(ws); CHECK_F32(ws);
  CHECK_CUDA_CONTIG(out); CHECK_BF16(out);
  TORCH_CHECK(xq.element_size() == 1 && wq.element_size() == 1 && xq.dim() == 2 && wq.dim() == 2, "gemm_fp8_block: e4m3 operands");
  const int64_t M = xq.size(0), K = xq.size(1), N = wq.size(0);
  TORCH_CHECK(wq.size(1) == K && K % 128 == 0 && out.size(0) == M && out.size(1) == N, "gemm_fp8_block: shapes");
  TORCH_CHECK(xs.dim() == 2 && xs.size(0) == K / 128 && xs.size(1) >= M && ws.dim() == 2 && ws.size(0) == (N + 127) / 128 && ws.size(1) == K / 128,
              "gemm_fp8_block: scale shapes");
  float* pp = nullptr;
  if (partial.has_value()) {
    CHECK_CUDA_CONTIG(*partial); CHECK_F32(*partial);
    TORCH_CHECK(partial->numel() >= gemm_fp8_splits(M, N, K) * M * N, "gemm_fp8_block: workspace too small");
    pp = partial->data_ptr<float>();
  }
  const c10::cuda::CUDAGuard guard(xq.device());
  check(forge_gemm_fp8_block(xq.data_ptr(), xs.data_ptr<float>(), static_cast<int>(xs.size(1)), wq.data_ptr(), ws.data_ptr<float>(),
                             out.data_ptr(), static_cast<int>(out.stride(0)), static_cast<int>(M), static_cast<int>(N),
                             static_cast<int>(K), pp, status_ptr(status), stream_of(xq)),
        "forge_gemm_fp8_block");
}

// ---- tensor-parallel exchange.  A "site" is described by plain integers (addresses inside the symmetric
// allocation, resolved once in Python): slot_ptrs[p] / signal_ptrs[p] = where THIS rank writes in peer p;
// part_ptrs[p] / y_ptrs[p] = rank p's copy of a buffer; mc_* = multicast address of a buffer (0: none);
// local_slots / local_signal = where this rank reads; arrive / epoch = two private device words;
// local_only = address of the device word that switches the measurement mode on (see tp_comm.cuh).
using PtrList = std::vector<int64_t>;

const long long* ptrs(const PtrList& v) { return reinterpret_cast<const long long*>(v.data()); }
unsigned* word(int64_t addr) { return reinterpret_cast<unsigned*>(addr); }

// Row-parallel GEMM under tensor parallelism: `part` is this rank's partial buffer inside the symmetric region (an
// address, row stride = w.size(0)); the kernel's last CTA signals every rank.
void gemm_tp(const Tensor& x, const Tensor& w, int64_t part, int64_t tune, int64_t tp_rank, const PtrList& signal_ptrs,
             int64_t arrive, int64_t epoch, const Tensor& status) {
  CHECK_BF16(x); CHECK_BF16(w);
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1, "gemm_tp: operands");
  TORCH_CHECK(w.size(1) == x.size(1) && signal_ptrs.size() >= 2 && part != 0 && (part & 15) == 0, "gemm_tp: shapes");
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_gemm_bf16_tp(x.data_ptr(), static_cast<int>(x.stride(0)), w.data_ptr(), static_cast<int>(w.stride(0)),
                           reinterpret_cast<void*>(part), static_cast<int>(w.size(0)), static_cast<int>(x.size(0)),
                           static_cast<int>(w.size(0)), static_cast<int>(x.size(1)), static_cast<int>(tune),
                           static_cast<int>(signal_ptrs.size()), static_cast<int>(tp_rank), ptrs(signal_ptrs), word(arrive),
                           word(epoch), status_ptr(status), stream_of(x)),
        "forge_gemm_bf16_tp");
}

// Row-parallel GEMM of at most 256 rows whose epilogue stores every output row as tagged words into the buffer of the rank
// that owns the row (ll_ptrs[p]: rank p's buffer, [ranks][rows_per_rank][features] 32-bit words).
void gemm_tp_tagged(const Tensor& x, const Tensor& w, int64_t tune, int64_t tp_rank, const PtrList& ll_ptrs, int64_t rows_per_rank,
                    int64_t arrive, int64_t epoch, const Tensor& status) {
  CHECK_BF16(x); CHECK_BF16(w);
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1, "gemm_tp_tagged: operands");
  TORCH_CHECK(w.size(1) == x.size(1) && ll_ptrs.size() >= 2, "gemm_tp_tagged: shapes");
  const c10::cuda::CUDAGuard guard(x.device());
  check(forge_gemm_bf16_tp_tagged(x.data_ptr(), static_cast<int>(x.stride(0)), w.data_ptr(), static_cast<int>(w.stride(0)),
                                  static_cast<int>(x.size(0)), static_cast<int>(w.size(0)), static_cast<int>(x.size(1)),
                                  static_cast<int>(tune), static_cast<int>(ll_ptrs.size()), static_cast<int>(tp_rank), ptrs(ll_ptrs),
                                  static_cast<int>(rows_per_rank), word(arrive), word(epoch), status_ptr(status), stream_of(x)),
        "forge_gemm_bf16_tp_tagged");
}

// Consumer of gemm_tp_tagged: reduce this rank's rows, residual add + RMSNorm, exchange of the normalised rows; y gets
// all rows, `residual` is updated on this rank's rows (row % ranks == rank) only.
void tp_tagged_reduce_norm(int64_t tp_rank, int64_t part, int64_t rows_per_rank, int64_t part_epoch, const PtrList& y_ptrs,
                           int64_t arrive, int64_t epoch, int64_t timeout_ns, int64_t local_only,
                           const c10::optional<Tensor>& residual_in, Tensor& residual_out, const Tensor& w, Tensor& y, double eps,
                           const Tensor& status) {
  CHECK_CUDA_CONTIG(residual_out); CHECK_BF16(residual_out); CHECK_CUDA_CONTIG(w); CHECK_BF16(w); CHECK_CUDA_CONTIG(y); CHECK_BF16(y);
  const int64_t H = residual_out.size(-1), rows = residual_out.numel() / H;
  TORCH_CHECK(y_ptrs.size() >= 2 && w.numel() == H && y.numel() == residual_out.numel() && part != 0, "tp_tagged_reduce_norm: shapes");
  const void* res = nullptr;
  if (residual_in.has_value()) { CHECK_CUDA_CONTIG(*residual_in); CHECK_BF16(*residual_in); TORCH_CHECK(residual_in->numel() == residual_out.numel()); res = residual_in->data_ptr(); }
  const c10::cuda::CUDAGuard guard(residual_out.device());
  check(forge_tp_tagged_reduce_norm(static_cast<int>(y_ptrs.size()), static_cast<int>(tp_rank), reinterpret_cast<const void*>(part),
                                    static_cast<int>(rows_per_rank), word(part_epoch), ptrs(y_ptrs), word(arrive), word(epoch),
                                    timeout_ns, word(local_only), res, residual_out.data_ptr(), w.data_ptr(), y.data_ptr(),
                                    static_cast<int>(rows), static_cast<int>(H), static_cast<float>(eps), status_ptr(status),
                                    stream_of(residual_out)),
        "forge_tp_tagged_reduce_norm");
}

// sum_out = sum over ranks of the partial rows (+ residual_in); y = rms_norm(sum_out) * w when y is given.
// part_ptrs empty: the rows were written into `slots` (a local address) by their owners and are only copied.
void tp_reduce_rms_norm(int64_t tp_size, int64_t tp_rank, const PtrList& part_ptrs, int64_t mc_part, int64_t slots,
                        int64_t local_signal, int64_t epoch, int64_t timeout_ns, int64_t local_only,
                        const c10::optional<Tensor>& residual_in, Tensor& sum_out, const c10::optional<Tensor>& w,
                        const c10::optional<Tensor>& y, double eps, const Tensor& status) {
  CHECK_CUDA_CONTIG(sum_out); CHECK_BF16(sum_out);
  const int64_t H = sum_out.size(-1), rows = sum_out.numel() / H;
  TORCH_CHECK(part_ptrs.empty() || static_cast<int64_t>(part_ptrs.size()) == tp_size, "tp_reduce_rms_norm: one partial buffer per rank");
  const void* res = nullptr; const void* wp = nullptr; void* yp = nullptr;
  if (residual_in.has_value()) { CHECK_CUDA_CONTIG(*residual_in); CHECK_BF16(*residual_in); TORCH_CHECK(residual_in->numel() == sum_out.numel()); res = residual_in->data_ptr(); }
  if (y.has_value()) {
    TORCH_CHECK(w.has_value(), "tp_reduce_rms_norm: norm weight needed");
    CHECK_CUDA_CONTIG(*w); CHECK_BF16(*w); CHECK_CUDA_CONTIG(*y); CHECK_BF16(*y);
    TORCH_CHECK(w->numel() == H && y->numel() == sum_out.numel());
    wp = w->data_ptr(); yp = y->data_ptr();
  }
  const c10::cuda::CUDAGuard guard(sum_out.device());
  check(forge_tp_reduce_rms_norm(static_cast<int>(tp_size), static_cast<int>(tp_rank), part_ptrs.empty() ? nullptr : ptrs(part_ptrs),
                                 mc_part, reinterpret_cast<const void*>(slots), word(local_signal), word(epoch), timeout_ns,
                                 word(local_only), res, sum_out.data_ptr(), wp, yp, static_cast<int>(rows), static_cast<int>(H),
                                 static_cast<float>(eps), status_ptr(status), stream_of(sum_out)),
        "forge_tp_reduce_rms_norm");
}

// Two-shot exchange: reduce-scatter by rows + residual add + RMSNorm on this rank's rows + all-gather of the normalised
// rows into every rank's broadcast buffer (y_ptrs / mc_y).  `residual` is updated in place on this rank's rows only.
void tp_rs_norm_ag(int64_t tp_rank, const PtrList& part_ptrs, int64_t mc_part, int64_t signal1, int64_t epoch1,
                   const PtrList& y_ptrs, int64_t mc_y, const PtrList& signal_ptrs2, int64_t arrive2, int64_t epoch2,
                   int64_t signal2, int64_t timeout_ns, int64_t local_only, const c10::optional<Tensor>& residual_in,
                   Tensor& residual_out, const Tensor& w, double eps, const Tensor& status) {
  CHECK_CUDA_CONTIG(residual_out); CHECK_BF16(residual_out); CHECK_CUDA_CONTIG(w); CHECK_BF16(w);
  const int64_t H = residual_out.size(-1), rows = residual_out.numel() / H;
  TORCH_CHECK(part_ptrs.size() >= 2 && y_ptrs.size() == part_ptrs.size() && signal_ptrs2.size() == part_ptrs.size() && w.numel() == H,
              "tp_rs_norm_ag: shapes");
  const void* res = nullptr;
  if (residual_in.has_value()) { CHECK_CUDA_CONTIG(*residual_in); CHECK_BF16(*residual_in); TORCH_CHECK(residual_in->numel() == residual_out.numel()); res = residual_in->data_ptr(); }
  const c10::cuda::CUDAGuard guard(residual_out.device());
  check(forge_tp_rs_norm_ag(static_cast<int>(part_ptrs.size()), static_cast<int>(tp_rank), ptrs(part_ptrs), mc_part, word(signal1),
                            word(epoch1), ptrs(y_ptrs), mc_y, ptrs(signal_ptrs2), word(arrive2), word(epoch2), word(signal2),
                            timeout_ns, word(local_only), res, residual_out.data_ptr(), w.data_ptr(), static_cast<int>(rows),
                            static_cast<int>(H), static_cast<float>(eps), status_ptr(status), stream_of(residual_out)),
        "forge_tp_rs_norm_ag");
}

void tp_embedding_push(const Tensor& ids, const Tensor& w, int64_t vocab_start, int64_t tp_rank, const PtrList& slot_ptrs,
                       const PtrList& signal_ptrs, int64_t arrive, int64_t epoch) {
  CHECK_CUDA_CONTIG(ids); CHECK_I32(ids); CHECK_CUDA_CONTIG(w); CHECK_BF16(w);
  const c10::cuda::CUDAGuard guard(w.device());
  check(forge_tp_embedding_push(ids.data_ptr<int>(), w.data_ptr(), static_cast<int>(ids.numel()), static_cast<int>(w.size(1)),
                                static_cast<int>(vocab_start), static_cast<int>(w.size(0)), static_cast<int>(slot_ptrs.size()),
                                static_cast<int>(tp_rank), ptrs(slot_ptrs), ptrs(signal_ptrs), word(arrive), word(epoch), stream_of(w)),
        "forge_tp_embedding_push");
}

void tp_rows_publish(const Tensor& src, int64_t part, int64_t tp_rank, const PtrList& signal_ptrs, int64_t arrive, int64_t epoch) {
  CHECK_CUDA_CONTIG(src); CHECK_BF16(src);
  const int64_t H = src.size(-1), rows = src.numel() / H;
  TORCH_CHECK(part != 0 && (part & 15) == 0, "tp_rows_publish: partial buffer address");
  const c10::cuda::CUDAGuard guard(src.device());
  check(forge_tp_rows_publish(src.data_ptr(), reinterpret_cast<void*>(part), static_cast<int>(rows), static_cast<int>(H),
                              static_cast<int>(signal_ptrs.size()), static_cast<int>(tp_rank), ptrs(signal_ptrs), word(arrive),
                              word(epoch), stream_of(src)),
        "forge_tp_rows_publish");
}

void tp_sample_pairs(const Tensor& vals, const Tensor& ids, int64_t tp_rank, const PtrList& slot_ptrs, const PtrList& signal_ptrs,
                     int64_t arrive, int64_t epoch, int64_t local_slots, int64_t slot_stride, int64_t local_signal,
                     int64_t timeout_ns, int64_t local_only, Tensor& out_i, const Tensor& status) {
  CHECK_CUDA_CONTIG(vals); CHECK_F32(vals); CHECK_CUDA_CONTIG(ids); CHECK_I32(ids); CHECK_CUDA_CONTIG(out_i); CHECK_I32(out_i);
  TORCH_CHECK(ids.numel() == vals.numel() && out_i.numel() >= vals.numel(), "tp_sample_pairs: lengths");
  const c10::cuda::CUDAGuard guard(vals.device());
  check(forge_tp_sample_pairs(vals.data_ptr<float>(), ids.data_ptr<int>(), static_cast<int>(vals.numel()),
                              static_cast<int>(slot_ptrs.size()), static_cast<int>(tp_rank), ptrs(slot_ptrs), ptrs(signal_ptrs),
                              word(arrive), word(epoch), reinterpret_cast<const void*>(local_slots), slot_stride, word(local_signal),
                              timeout_ns, word(local_only), out_i.data_ptr<int>(), status_ptr(status), stream_of(vals)),
        "forge_tp_sample_pairs");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "tinyllmforge_b200 sm_100a kernels";
  m.def("gemm", &gemm);
  m.def("gemm_fused", &gemm_fused);
  m.def("gemm_sample", &gemm_sample);
  m.def("gemm_set_trace", &gemm_set_trace);
  m.def("launch_count", []() { return static_cast<int64_t>(forge_launch_count()); });
  m.def("quant_fp8", &quant_fp8);
  m.def("dequant_fp8_block", [](const Tensor& wq, const Tensor& scale, Tensor& out) {
    // e4m3 weights [N, K] with fp32 scales [ceil(N / 128), K / 128] -> bf16 [N, K]
    TORCH_CHECK(wq.is_cuda() && wq.dim() == 2 && wq.element_size() == 1 && wq.is_contiguous(), "dequant_fp8_block: wq must be a contiguous 1-byte [N, K] CUDA tensor");
    const int64_t N = wq.size(0), K = wq.size(1);
    TORCH_CHECK(K % 128 == 0 && scale.scalar_type() == torch::kFloat32 && scale.is_contiguous() && scale.numel() == ((N + 127) / 128) * (K / 128),
                "dequant_fp8_block: scale must be fp32 [ceil(N / 128), K / 128]");
    TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.numel() >= N * K, "dequant_fp8_block: out must hold N * K bf16 values");
    check(forge_dequant_fp8_block(wq.data_ptr(), scale.data_ptr<float>(), out.data_ptr(), static_cast<int>(N), static_cast<int>(K),
                                  stream_of(wq)), "forge_dequant_fp8_block");
  });
  m.def("gemm_fp8_block", &gemm_fp8_block);
  m.def("gemm_fp8_splits", &gemm_fp8_splits);
  m.def("gemm_tp", &gemm_tp);
  m.def("gemm_tp_tagged", &gemm_tp_tagged);
  m.def("tp_tagged_reduce_norm", &tp_tagged_reduce_norm);
  m.def("tp_reduce_rms_norm", &tp_reduce_rms_norm);
  m.def("tp_embedding_push", &tp_embedding_push);
  m.def("tp_rows_publish", &tp_rows_publish);
  m.def("tp_rs_norm_ag", &tp_rs_norm_ag);
  m.def("tp_sample_pairs", &tp_sample_pairs);
  m.def("rms_norm", &rms_norm);
  m.def("qk_norm_rope_store", &qk_norm_rope_store);
  m.def("gemm_qkv_rope_store", &gemm_qkv_rope_store);
  m.def("silu_mul", &silu_mul);
  m.def("embedding", &embedding);
  m.def("gather_rows", &gather_rows);
  m.def("feed_tokens", &feed_tokens);
  m.def("sample_nsplit", &sample_nsplit);
  m.def("sample", &sample);
  m.def("sample_merge_ranks", &sample_merge_ranks);
  m.def("decode_attention", &decode_attention);
  m.def("decode_attention_flat", &decode_attention_flat);
  m.def("decode_attention_qkv", &decode_attention_qkv);
  m.def("decode_attention_flat_scratch_floats", &decode_attention_flat_scratch_floats);
  m.def("decode_attention_flat_ctas_per_sm", &decode_attention_flat_ctas_per_sm);
  m.def("gemm_set_streamk_workspace", [](torch::Tensor ws, torch::Tensor counters, int64_t ctas) {
    // scratch of the stream-K GEMM for the current device: fp32 partial tiles and zeroed per-tile arrival counters
    TORCH_CHECK(ws.is_cuda() && ws.scalar_type() == torch::kFloat32 && ws.is_contiguous(), "ws: contiguous fp32 CUDA tensor");
    TORCH_CHECK(counters.is_cuda() && counters.scalar_type() == torch::kInt32 && counters.is_contiguous(), "counters: contiguous int32 CUDA tensor");
    TORCH_CHECK(ws.numel() >= forge_gemm_streamk_workspace_floats(static_cast<int>(ctas)), "ws too small for ", ctas, " CTAs");
    check(forge_gemm_set_streamk_workspace(ws.data_ptr<float>(), counters.data_ptr<int>(), static_cast<int>(ctas), static_cast<int>(counters.numel())),
          "forge_gemm_set_streamk_workspace");
  });
  m.def("gemm_streamk_workspace_floats", [](int64_t ctas) { return static_cast<int64_t>(forge_gemm_streamk_workspace_floats(static_cast<int>(ctas))); });
  m.def("decode_attention_set_tc_min_group", [](int64_t g) { forge_decode_attention_set_tc_min_group(static_cast<int>(g)); });
  m.def("prefill_attention", &prefill_attention);
}

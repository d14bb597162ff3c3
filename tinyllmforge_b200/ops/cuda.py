"""The op set on a B200: every call lands in a hand-written sm_100a kernel of ``tinyllmforge_b200._C``.

There is no fallback: if the extension is missing or a kernel reports an error, the call raises.  The method
names and argument meanings are those of ``ops.ref.RefOps`` (the PyTorch statement of each op, which is also the
oracle the GPU tests compare against).

Reference call sites replaced (all in tinyvllm/): layers/linear.py:83,181 (F.linear -> tcgen05 GEMM),
layers/activation.py:11 (fused into the gate_up GEMM epilogue), layers/layernorm.py:21,33,
layers/rotary_embedding.py:41 + layers/attention.py:9-48 + models/qwen3.py:79-90 (one fused kernel),
layers/attention.py:101,108 (paged prefill / decode attention), layers/embed_head.py:34-70, layers/sampler.py:13-21.
"""
from __future__ import annotations

import os

import torch

from ..config import Config
from ..parallel.comm import TPGroup
from .quant import Fp8BlockWeight

try:
    from .. import _C
except ImportError as e:  # pragma: no cover - exercised only on a broken install
    _C = None
    _IMPORT_ERROR = e

STATUS_BITS = {1: "mbarrier wait ran out", 2: "peer flag wait ran out", 4: "slot or block id out of range",
               8: "unsupported shape"}


def require_ext():
    if _C is None:
        raise RuntimeError("tinyllmforge_b200._C is not built; run `python -m tinyllmforge_b200.build_ext` "
                           f"(import error: {_IMPORT_ERROR})")
    return _C


def decode_chunking(batch: int, num_kv_heads: int, block_size: int, max_len: int) -> tuple[int, int]:
    """(tokens per context chunk, number of chunks) for the split-KV decode kernel.

    Small batches split the context finely so that every SM gets work; large batches keep chunks long so
    that the partial-merge traffic stays negligible.  Depends only on shapes known at graph-capture time."""
    tile = min(block_size, 64)
    ctas = batch * num_kv_heads
    chunk = 1024 if ctas >= 1024 else 512 if ctas >= 256 else 256 if ctas >= 64 else 128 if ctas >= 16 else 64
    chunk = max(tile, chunk)
    return chunk, max(1, -(-max_len // chunk))


def decode_group_slice(group: int) -> int:
    """q heads per KV head processed together by the decode attention kernels (``decode_group_slice`` in
    csrc/include/decode_common.cuh): slices of more than 4 heads run one CTA per SM instead of two."""
    for g in (5, 4, 3, 2):
        if group % g == 0:
            return g
    return 1


W_DYNAMIC = 1 << 8              # in the ring-depth byte of the GEMM's tuning word (bit 24): W comes from the preceding kernel
FP8_EXPAND_MIN_ROWS = 128       # more rows than this: expand fp8 weights to bf16 and run the bf16 GEMM (see CudaOps._expand_fp8)
_STREAMK_WS: dict = {}


def _streamk_workspace(C, device, num_sms: int) -> None:
    """Scratch of the stream-K GEMM (fp32 partial tiles of CTAs whose share of the work ends inside an output tile, and
    per-tile arrival counters): one per device and process, never freed, because CUDA graphs captured by any engine of
    the process keep its address.  All GEMMs of a device share it, so they must be ordered on one stream."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key in _STREAMK_WS:
        return
    with torch.cuda.device(key):
        ws = torch.empty(C.gemm_streamk_workspace_floats(num_sms), dtype=torch.float32, device=device)
        counters = torch.zeros(8192, dtype=torch.int32, device=device)
        C.gemm_set_streamk_workspace(ws, counters, num_sms)
    _STREAMK_WS[key] = (ws, counters)


class CudaOps:
    name = "cuda"

    def __init__(self, config: Config | None = None, tp: TPGroup | None = None, device=None):
        self.C = require_ext()
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.tp = tp or TPGroup()
        self.max_model_len = config.max_model_len if config is not None else 4096
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._launch_base = self.C.launch_count()
        self.fused = None                          # FusedTPComm once enable_fused_comm() ran
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        # "flat": all KV tiles of a decode step dealt out equally to two CTAs per SM; "chunked": one CTA per
        # (sequence, KV head, context chunk); "auto": flat from 48 sequences (measured at context ~800: 0.78-0.83 vs
        # 0.69-0.75 of copy bandwidth at 64-96 sequences, equal from 128, a few us slower below 16).
        # Scratch of the flat kernel, sized for any head grouping (~1.2 MB).
        self.decode_attention_mode = os.environ.get("FORGE_DECODE_ATTN", "auto")
        self.fused_qkv_max_batch = int(os.environ.get("FORGE_FUSED_QKV_MAX", "32"))   # see models/qwen3.py
        self.sample_in_lm_head = os.environ.get("FORGE_LM_HEAD_SAMPLE", "1") != "0"
        # q/k-norm + RoPE + KV store in the qkv GEMM's epilogue (see qkv_rope_store_in_gemm): 174 instead of 201 launches per
        # Qwen3-0.6B decode step, but measured slower (3.86 vs 3.76 ms mean step: head-sized tiles leave 32-64 CTAs for the
        # projection, and each epilogue thread normalises and rotates a whole head) -> off unless asked for
        self.qkv_epilogue = os.environ.get("FORGE_QKV_EPILOGUE", "0") != "0"
        self.qkv_epilogue_min_rows = int(os.environ.get("FORGE_QKV_EPILOGUE_MIN_ROWS", "33"))
        self._flat_scratch = torch.empty(2 * self.num_sms * (2 * 4 * 130 + 2) + 64, dtype=torch.float32, device=self.device)
        _streamk_workspace(self.C, self.device, self.num_sms)
        self.fp8_expand_max_weights = int(os.environ.get("FORGE_FP8_EXPAND_MAX_WEIGHTS", "0"))
        self._fp8_scratch = None                   # bf16 expansion of one fp8 weight (see _expand_fp8)
        self._fp8_retired = []

    @property
    def launches(self) -> int:
        """Kernels of this library launched (or captured into a CUDA graph) since the counter was last set; counted where
        they are launched, so GEMMs that run as two kernels (K split + reduce) count as two."""
        return self.C.launch_count() - self._launch_base

    @launches.setter
    def launches(self, value: int) -> None:
        self._launch_base = self.C.launch_count() - int(value)

    # ------------------------------------------------------------------ status word
    def check_status(self) -> None:
        """Raise if any kernel since the last check recorded an error (costs a device sync)."""
        word = int(self.status[0].item())
        if word:
            self.raise_status(word)

    def raise_status(self, word: int) -> None:
        """Turn a non-zero status word (already read back) into an exception and clear the device copy."""
        self.status.zero_()
        what = [txt for bit, txt in STATUS_BITS.items() if word & bit]
        raise RuntimeError(f"a CUDA kernel reported: {', '.join(what) or hex(word)}")

    # ------------------------------------------------------------------ GEMMs
    def linear(self, x: torch.Tensor, w: torch.Tensor, force_mode: int = 0, force_splits: int = 0,
               force_block_c: int = 0, force_deep: int = 0) -> torch.Tensor:
        """x @ w.T.  ``w`` must not be the output of the kernel launched just before this call: the decode
        kernel starts streaming weights before it waits for its predecessor (weights are static in the engine)."""
        if isinstance(w, Fp8BlockWeight):
            if not self._expands_fp8(w, x.shape[0]):
                return self.linear_fp8(x, w)
            w, force_deep = self._expand_fp8(w), force_deep | W_DYNAMIC
        out = torch.empty(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
        self.C.gemm(x, w, out, 0, force_mode, force_splits | (force_block_c << 8) | (force_deep << 16), self.status)
        return out

    def linear_silu_mul(self, x: torch.Tensor, w_gate_up: torch.Tensor, force_mode: int = 0, force_splits: int = 0,
                        force_block_c: int = 0, force_deep: int = 0) -> torch.Tensor:
        if isinstance(w_gate_up, Fp8BlockWeight):
            if not self._expands_fp8(w_gate_up, x.shape[0]):
                return self.silu_mul(self.linear_fp8(x, w_gate_up))
            w_gate_up, force_deep = self._expand_fp8(w_gate_up), force_deep | W_DYNAMIC
        out = torch.empty(x.shape[0], w_gate_up.shape[0] // 2, dtype=x.dtype, device=x.device)
        self.C.gemm(x, w_gate_up, out, 1, force_mode, force_splits | (force_block_c << 8) | (force_deep << 16), self.status)
        return out

    # --- GEMMs with the neighbouring RMSNorm / residual add fused in (single GPU, bf16 weights; see models/qwen3.py)
    def embedding_ssq(self, ids, weight, vocab_start):
        """(rows, ssq_a, ssq_b): embedding rows and two fp32 [tokens, ceil(H / 128)] arrays of per-row partial sums of squares.
        ssq_a describes the rows returned (their sum of squares in column 0); ssq_b is scratch for ``linear_residual``:
        the block loop alternates between the two (the o GEMM writes one, the down GEMM the other)."""
        T, H = ids.shape[0], weight.shape[1]
        out = torch.empty(T, H, dtype=weight.dtype, device=weight.device)
        ssq = torch.empty(2, T, (H + 127) // 128, dtype=torch.float32, device=weight.device)
        self.C.embedding(ids, weight, out, vocab_start, ssq[0])
        return out, ssq[0], ssq[1]

    def linear_scaled(self, x: torch.Tensor, w: torch.Tensor, ssq_row: torch.Tensor, eps: float, silu_mul: bool = False,
                      force_mode: int = 0, tune: int = 0) -> torch.Tensor:
        """rms_norm(x) @ w0.T computed as (x @ w.T) * rsqrt(ssq / K + eps) per row, where w = w0 with the norm weight
        folded into its columns and ssq_row [tokens, parts] holds partial sums of squares of the rows.  silu_mul: w is
        [2I, K] (gate rows, up rows)."""
        n_out = w.shape[0] // 2 if silu_mul else w.shape[0]
        out = torch.empty(x.shape[0], n_out, dtype=x.dtype, device=x.device)
        self.C.gemm_fused(x, w, out, 1 if silu_mul else 0, force_mode, tune, ssq_row, eps, False, None, self.status)
        return out

    def linear_residual(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, ssq_out: torch.Tensor,
                        force_mode: int = 0, tune: int = 0) -> None:
        """residual += x @ w.T in place (rounded like a bf16 GEMM output followed by a bf16 add); ssq_out (fp32
        [tokens, ceil(H / 128)]) receives the sums of squares of the new residual rows, one per 128 features."""
        self.C.gemm_fused(x, w, residual, 0, force_mode, tune, None, 0.0, True, ssq_out, self.status)

    def _expands_fp8(self, w: "Fp8BlockWeight", rows: int) -> bool:
        """Many rows: the GEMM is bound by the tensor cores, the expansion costs a few per cent.  Few rows on a small matrix
        (a shard of a large model over many ranks): the step is bound by its chain of launches, and the e4m3 path needs three
        (quantise, multiply, add the K splits) where expansion + the fused bf16 kernel needs two and keeps its epilogues."""
        return rows > FP8_EXPAND_MIN_ROWS or w.shape[0] * w.shape[1] <= self.fp8_expand_max_weights

    def _expand_fp8(self, w: "Fp8BlockWeight") -> torch.Tensor:
        """bf16 copy of a block-scaled e4m3 weight in a scratch buffer that the next expansion overwrites (stream-ordered:
        the GEMM that reads it is launched before the next expansion).  For GEMMs with many tokens, whose time is set by
        the tensor cores: the weights stay e4m3 in memory, the activations stay bf16, and the bf16 CTA-pair kernel with its
        fused epilogues does the multiplication; the expansion moves 3 bytes per weight."""
        N, K = w.shape
        if self._fp8_scratch is None or self._fp8_scratch.numel() < N * K:
            if self._fp8_scratch is not None:
                self._fp8_retired.append(self._fp8_scratch)      # CUDA graphs captured so far keep using the smaller buffer
            self._fp8_scratch = torch.empty(N * K, dtype=torch.bfloat16, device=self.device)
        out = self._fp8_scratch[:N * K].view(N, K)
        self.C.dequant_fp8_block(w.q.view(torch.uint8), w.scale, out)
        return out

    def linear_fp8(self, x: torch.Tensor, w: "Fp8BlockWeight") -> torch.Tensor:
        """Block-scaled fp8 GEMM: quantise activations per token and 128 features, multiply on the e4m3 tensor-core
        path, apply the scales per K block while accumulating."""
        M, K = x.shape
        xq = torch.empty(M, K, dtype=torch.uint8, device=x.device)
        xs = torch.empty(K // 128, (M + 3) // 4 * 4, dtype=torch.float32, device=x.device)
        self.C.quant_fp8(x, xq, xs)
        N = w.shape[0]
        out = torch.empty(M, N, dtype=x.dtype, device=x.device)
        splits = self.C.gemm_fp8_splits(M, N, K)         # few tokens: K is split over CTAs, partials added by a second kernel
        partial = torch.empty(splits * M * N, dtype=torch.float32, device=x.device) if splits > 1 else None
        self.C.gemm_fp8_block(xq, xs, w.q.view(torch.uint8), w.scale, out, partial, self.status)
        return out

    # ------------------------------------------------------------------ elementwise
    def rms_norm(self, x, weight, eps):
        y = torch.empty_like(x)
        self.C.rms_norm(x, None, weight, y, eps)
        return y

    def add_rms_norm(self, x, residual, weight, eps):
        """(normed, new_residual).  ``residual`` is updated in place and returned."""
        y = torch.empty_like(x)
        if residual is None:
            self.C.rms_norm(x, None, weight, y, eps)
            return y, x
        self.C.rms_norm(x, residual, weight, y, eps)
        return y, residual

    def silu_mul(self, x):
        out = torch.empty(x.shape[:-1] + (x.shape[-1] // 2,), dtype=x.dtype, device=x.device)
        self.C.silu_mul(x, out)
        return out

    def embedding(self, ids, weight, vocab_start=0):
        out = torch.empty(ids.shape[0], weight.shape[1], dtype=weight.dtype, device=weight.device)
        self.C.embedding(ids, weight, out, vocab_start, None)
        return out

    def select_rows(self, x, index):
        out = torch.empty(index.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
        self.C.gather_rows(index, x, out)
        return out

    def qk_norm_rope_store(self, qkv, q_weight, k_weight, eps, table, positions, slot_mapping, k_cache, v_cache,
                           num_heads, num_kv_heads, head_dim, do_rope=True):
        T = qkv.shape[0]
        q = torch.empty(T, num_heads, head_dim, dtype=qkv.dtype, device=qkv.device)
        self.C.qk_norm_rope_store(qkv, q_weight, k_weight, eps, table, positions, slot_mapping, q, k_cache, v_cache,
                                  num_heads, num_kv_heads, do_rope, self.status)
        return q

    def qkv_rope_store_in_gemm(self, rows: int, head_dim: int, weight) -> bool:
        """Decode steps of 33..256 rows with head_dim 128 and a bf16 qkv weight: the projection's epilogue does the per-head
        norm, the rotation and the cache write (tiles of 128 features = one head)."""
        return (self.qkv_epilogue and head_dim == 128 and self.qkv_epilogue_min_rows <= rows <= 256
                and not isinstance(weight, Fp8BlockWeight) and weight.dtype == torch.bfloat16)

    def linear_qkv_rope_store(self, x, w, ssq_row, in_eps, q_weight, k_weight, eps, table, positions, slot_mapping, k_cache, v_cache,
                              num_heads, num_kv_heads, do_rope=True):
        """qkv projection (optionally with the folded input norm, see ``linear_scaled``) + q/k-norm + RoPE + KV store in
        one kernel; returns q [T, heads, 128].  Replaces linear + qk_norm_rope_store for decode steps."""
        T = x.shape[0]
        q = torch.empty(T, num_heads, 128, dtype=x.dtype, device=x.device)
        self.C.gemm_qkv_rope_store(x, w, ssq_row, in_eps, q_weight, k_weight, eps, table, positions, slot_mapping, q, k_cache, v_cache,
                                   num_heads, num_kv_heads, do_rope, self.status)
        return q

    # ------------------------------------------------------------------ attention
    def attention(self, q, k_cache, v_cache, batch, scale):
        T, H, D = q.shape
        out = torch.empty(T, H * D, dtype=q.dtype, device=q.device)
        if batch.is_prefill:
            self.C.prefill_attention(q, k_cache, v_cache, batch.cu_seqlens_q, batch.context_lens, batch.block_tables, out,
                                     batch.num_seqs, batch.max_seqlen_q, scale, self.status)
            return out
        B = batch.padded_seqs
        if self.decode_attention_mode == "flat" or (self.decode_attention_mode == "auto" and 48 <= B <= 512):
            # all KV tiles of the step dealt out equally to two CTAs per SM (one for wide head groups); lengths are read on the device
            ctas = self._flat_ctas(H, k_cache, False)
            self.C.decode_attention_flat(q, k_cache, v_cache, batch.block_tables, batch.context_lens, out, self._flat_scratch,
                                         ctas, scale, self.status)
            return out
        # graph-safe sizing: the longest context the block table can describe
        max_len = batch.table_width * k_cache.shape[2]
        chunk, max_chunks = decode_chunking(B, k_cache.shape[1], k_cache.shape[2], max_len)
        part_o = part_ml = None
        if max_chunks > 1:
            part_o = torch.empty(B * H * max_chunks * D, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(B * H * max_chunks * 2, dtype=torch.float32, device=q.device)
        self.C.decode_attention(q, k_cache, v_cache, batch.block_tables, batch.context_lens, out, part_o, part_ml,
                                chunk, max_chunks, scale, self.status)
        return out

    def _flat_ctas(self, num_heads, k_cache, from_raw_qkv: bool) -> int:
        """Grid of the flat decode kernel for this head grouping; also makes sure the scratch is large enough."""
        nkv, bs = k_cache.shape[1], k_cache.shape[2]
        ctas = self.C.decode_attention_flat_ctas_per_sm(num_heads, nkv, bs, from_raw_qkv) * self.num_sms
        need = self.C.decode_attention_flat_scratch_floats(ctas, 512, num_heads, nkv)
        if self._flat_scratch is None or self._flat_scratch.numel() < need:
            self._flat_scratch = torch.empty(need, dtype=torch.float32, device=k_cache.device)
        return ctas

    def decode_attention_qkv(self, qkv, q_weight, k_weight, eps, table, k_cache, v_cache, batch, num_heads, scale, do_rope=True):
        """Decode step: attention straight from the raw qkv projection.  q/k-norm, rotation at position len - 1 and the
        KV-cache store of the step's token happen inside the attention kernel (one launch less per layer than
        ``qk_norm_rope_store`` + ``attention``).  Same partition choice as ``attention``."""
        B, D = batch.padded_seqs, k_cache.shape[3]
        out = torch.empty(B, num_heads * D, dtype=qkv.dtype, device=qkv.device)
        rope = table if do_rope else None
        if self.decode_attention_mode == "flat" or (self.decode_attention_mode == "auto" and 48 <= B <= 512):
            ctas = self._flat_ctas(num_heads, k_cache, True)          # may grow the scratch: before it is passed on
            self.C.decode_attention_qkv(qkv, q_weight, k_weight, eps, rope, k_cache, v_cache, batch.block_tables, batch.context_lens,
                                        out, self._flat_scratch, ctas, None, None, 0, 0, num_heads, scale, self.status)
            return out
        max_len = batch.table_width * k_cache.shape[2]
        chunk, max_chunks = decode_chunking(B, k_cache.shape[1], k_cache.shape[2], max_len)
        part_o = part_ml = None
        if max_chunks > 1:
            part_o = torch.empty(B * num_heads * max_chunks * D, dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty(B * num_heads * max_chunks * 2, dtype=torch.float32, device=qkv.device)
        self.C.decode_attention_qkv(qkv, q_weight, k_weight, eps, rope, k_cache, v_cache, batch.block_tables, batch.context_lens,
                                    out, None, 0, part_o, part_ml, chunk, max_chunks, num_heads, scale, self.status)
        return out

    # ------------------------------------------------------------------ tensor-parallel exchange
    def tp_all_reduce(self, y, tp):
        """Library collective (NCCL): the baseline path (``comm="nccl"``)."""
        return tp.all_reduce(y)

    def enable_fused_comm(self, hidden_size: int, max_tokens: int, timeout_s: float = 10.0) -> None:
        """Allocate the symmetric region; afterwards row-parallel layers, the embedding and the sampler exchange
        data from inside their kernels."""
        from ..parallel.symm import FusedTPComm
        self.fused = FusedTPComm(self.tp, hidden_size, max_tokens, self.device, timeout_s)

    def _reduce_norm(self, st, rows, H, residual_in, residual_out, norm_weight, eps):
        """Consumer half of a row-parallel exchange whose partial sums sit in site ``st``'s buffers: one-shot (every rank
        pulls the sum of all rows) or two-shot (reduce-scatter, norm on this rank's rows, all-gather).  Returns the
        normalised rows; in the two-shot form they live in the broadcast buffer and ``residual_out`` holds only this
        rank's rows (rows r, r + tp, ...), which is all the next exchange of the same step reads."""
        f, tp = self.fused, self.tp
        if norm_weight is not None and f.two_shot(rows, H):
            from ..parallel.symm import SITE_GATHER
            ag = f.sites[SITE_GATHER]
            self.C.tp_rs_norm_ag(tp.rank, st.buf_ptrs, st.mc_buf, st.local_signal, st.epoch, ag.buf_ptrs, ag.mc_buf, ag.signal_ptrs,
                                 ag.arrive, ag.epoch, ag.local_signal, f.timeout_ns, f.local_only, residual_in, residual_out,
                                 norm_weight, eps, self.status)
            return f.y_view(rows, H)
        y = torch.empty(rows, H, dtype=torch.bfloat16, device=self.device) if norm_weight is not None else None
        self.C.tp_reduce_rms_norm(tp.size, tp.rank, st.buf_ptrs, st.mc_buf, 0, st.local_signal, st.epoch, f.timeout_ns, f.local_only,
                                  residual_in, residual_out, norm_weight, y, eps, self.status)
        return y

    def fused_all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over the ranks of a bf16 tensor of at most 256 x hidden elements (last dimension a multiple of 8) through
        the symmetric region: one kernel copies this rank's rows into its partial buffer and signals, one kernel waits for
        all ranks and pulls the sum (in the switch, or with peer loads in rank order).  Larger tensors: library collective."""
        from ..parallel.symm import MAX_ALLREDUCE_ROWS, SITE_ALLREDUCE
        tp = self.tp
        if tp.size == 1:
            return x
        H = x.shape[-1]
        if (self.fused is None or x.dtype != torch.bfloat16 or H % 8 or H > 8192 or x.numel() > MAX_ALLREDUCE_ROWS * self.fused.hidden):
            return tp.all_reduce(x)
        st = self.fused.sites[SITE_ALLREDUCE]
        x = x.contiguous()
        out = torch.empty_like(x)
        self.C.tp_rows_publish(x, st.local_buf, tp.rank, st.signal_ptrs, st.arrive, st.epoch)
        self._reduce_norm(st, x.numel() // H, H, None, out, None, 0.0)
        return out

    def fused_barrier(self) -> None:
        """Device-side barrier over the ranks: the stream of every rank passes only after every rank's stream got here
        (an all-reduce of one 8-element row; bounded wait, a timeout sets the status word)."""
        if self.tp.size > 1:
            self.fused_all_reduce(torch.zeros(1, 8, dtype=torch.bfloat16, device=self.device))

    def embed_norm(self, ids, embed, norm_weight, eps):
        """Embedding lookup + cross-rank exchange + first RMSNorm -> (normed, residual)."""
        tp = embed.tp
        if tp.size == 1:
            return self.add_rms_norm(self.embedding(ids, embed.weight, embed.vocab_start), None, norm_weight, eps)
        T, H = ids.shape[0], embed.weight.shape[1]
        if self.fused is None or T > self.fused.max_tokens:
            h = tp.all_reduce(self.embedding(ids, embed.weight, embed.vocab_start))
            return self.add_rms_norm(h, None, norm_weight, eps)
        from ..parallel.symm import SITE_EMBED
        f, st = self.fused, self.fused.sites[SITE_EMBED]
        self.C.tp_embedding_push(ids, embed.weight, embed.vocab_start, tp.rank, st.buf_ptrs, st.signal_ptrs, st.arrive, st.epoch)
        residual = torch.empty(T, H, dtype=embed.weight.dtype, device=ids.device)
        y = torch.empty_like(residual)
        self.C.tp_reduce_rms_norm(tp.size, tp.rank, [], 0, st.local_buf, st.local_signal, st.epoch, f.timeout_ns, f.local_only,
                                  None, residual, norm_weight, y, eps, self.status)
        return y, residual

    def row_linear_add_rms_norm(self, x, layer, residual, norm_weight, eps, site):
        """Row-parallel GEMM + sum over ranks + residual add + RMSNorm -> (normed, residual).

        Fused path, up to 256 rows (decode): the GEMM epilogue stores every output row, as tagged words, into the memory
        of the rank that owns the row; the consumer kernel adds the ranks' rows it owns, applies residual + norm and sends
        the normalised rows to the other ranks the same way: no flags, no fences, two one-way NVLink trips.  More rows
        (prefill): the GEMM stores its partial sums into this rank's buffer of the symmetric region and its last CTA
        signals every rank; one consumer kernel waits for all ranks, pulls the sum over NVLink (one-shot for few bytes,
        reduce-scatter + all-gather for many, see ``_reduce_norm``), adds the residual and normalises.  No library
        collective is involved at any batch size.  In the tagged and the two-shot forms ``residual`` holds only this
        rank's rows (row % tp == rank) afterwards, which is all the next exchange of the same step reads."""
        tp = layer.tp
        if tp.size == 1:
            return self.add_rms_norm(self.linear(x, layer.weight), residual, norm_weight, eps)
        M, H = x.shape[0], layer.weight.shape[0]
        if self.fused is None or M > self.fused.max_tokens or H != self.fused.hidden:
            return self.add_rms_norm(tp.all_reduce(self.linear(x, layer.weight)), residual, norm_weight, eps)
        st = self.fused.sites[site]
        fp8 = isinstance(layer.weight, Fp8BlockWeight)
        expand = fp8 and self._expands_fp8(layer.weight, M)
        if self.fused.use_tagged(M, H) and (not fp8 or expand):
            # decode-sized: rows travel as tagged words from the GEMM epilogue to their owners and back normalised
            from ..parallel.symm import SITE_GATHER
            f, ag = self.fused, self.fused.sites[SITE_GATHER]
            w, tune = (self._expand_fp8(layer.weight), W_DYNAMIC << 16) if expand else (layer.weight, 0)
            self.C.gemm_tp_tagged(x, w, tune, tp.rank, st.ll_ptrs, f.tagged_rows_per_rank, st.arrive, st.epoch, self.status)
            y = torch.empty(M, H, dtype=x.dtype, device=x.device)
            self.C.tp_tagged_reduce_norm(tp.rank, st.ll_local, f.tagged_rows_per_rank, st.epoch, ag.ll_ptrs, ag.arrive, ag.epoch,
                                         f.timeout_ns, f.local_only, residual, residual, norm_weight, y, eps, self.status)
            return y, residual
        if fp8 and not expand:
            # the block-scaled GEMM has no signalling epilogue: publish its output with a copy kernel
            self.C.tp_rows_publish(self.linear_fp8(x, layer.weight), st.local_buf, tp.rank, st.signal_ptrs, st.arrive, st.epoch)
        elif fp8:
            self.C.gemm_tp(x, self._expand_fp8(layer.weight), st.local_buf, W_DYNAMIC << 16, tp.rank, st.signal_ptrs, st.arrive, st.epoch, self.status)
        else:
            self.C.gemm_tp(x, layer.weight, st.local_buf, 0, tp.rank, st.signal_ptrs, st.arrive, st.epoch, self.status)
        return self._reduce_norm(st, M, H, residual, residual, norm_weight, eps), residual

    # ------------------------------------------------------------------ sampling
    def sample_shard(self, logits, temperatures, header, vocab_start):
        """(ids int32 [rows], scores fp32 [rows]) of this vocab shard."""
        rows, vocab = logits.shape
        n = self.C.sample_nsplit(rows, vocab)
        part_v = torch.empty(rows * n, dtype=torch.float32, device=logits.device)
        part_i = torch.empty(rows * n, dtype=torch.int32, device=logits.device)
        ids = torch.empty(rows, dtype=torch.int32, device=logits.device)
        best = torch.empty(rows, dtype=torch.float32, device=logits.device)
        self.C.sample(logits, vocab_start, temperatures, header, part_v, part_i, ids, best)
        return ids, best

    def can_sample_in_lm_head(self, rows: int, weight) -> bool:
        """The LM-head GEMM can sample in its epilogue when it runs on the persistent token-tile kernel (many vocabulary
        tiles, at least 8 rows) over a bf16 shard; the shard must start on a multiple of 32 token ids (checked by the
        caller that knows the start)."""
        return (self.sample_in_lm_head and not isinstance(weight, Fp8BlockWeight) and rows >= 8
                and (weight.shape[0] + 127) // 128 >= 2 * self.num_sms)

    def lm_head_sample_shard(self, hidden, weight, temperatures, header, vocab_start):
        """(ids int32 [rows], scores fp32 [rows]) of this vocab shard, sampled in the epilogue of the LM-head GEMM: the
        ``[rows, vocab / tp]`` logits are never written.  Same tokens as ``linear`` + ``sample_shard``."""
        rows, tiles = hidden.shape[0], (weight.shape[0] + 255) // 256
        part_v = torch.empty(rows * tiles, dtype=torch.float32, device=hidden.device)
        part_i = torch.empty(rows * tiles, dtype=torch.int32, device=hidden.device)
        ids = torch.empty(rows, dtype=torch.int32, device=hidden.device)
        best = torch.empty(rows, dtype=torch.float32, device=hidden.device)
        self.C.gemm_sample(hidden, weight, vocab_start, temperatures, header, part_v, part_i, ids, best, self.status)
        return ids, best

    def sample(self, logits, batch, vocab_start, tp):
        ids, best = self.sample_shard(logits, batch.temperatures, batch.header, vocab_start)
        return self.merge_ranks(ids, best, tp)

    def merge_ranks(self, ids, best, tp):
        """The winner among the ranks' (id, score) pairs of every row; every rank gets the same ids."""
        if tp.size == 1:
            return ids
        if self.fused is not None and ids.shape[0] <= 512:
            from ..parallel.symm import SITE_SAMPLE
            st = self.fused.sites[SITE_SAMPLE]
            out = torch.empty_like(ids)
            self.C.tp_sample_pairs(best, ids, tp.rank, st.slot_ptrs, st.signal_ptrs, st.arrive, st.epoch, st.local_buf,
                                   st.slot_stride, st.local_signal, self.fused.timeout_ns, self.fused.local_only, out, self.status)
            return out
        all_best = tp.all_gather_stack(best)
        all_ids = tp.all_gather_stack(ids)
        out = torch.empty_like(ids)
        self.C.sample_merge_ranks(all_best, all_ids, out)
        return out

    def close(self):
        if self.fused is not None:
            self.fused.close()
            self.fused = None

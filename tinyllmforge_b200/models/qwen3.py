"""Qwen3 dense decoder: owns the (sharded) weights and calls the op set in order.

Parity: tinyvllm/models/qwen3.py:14-234.
  * pre-norm decoder with the fused-residual convention: every norm after the first is
    add + RMSNorm and also emits the updated residual stream (qwen3.py:164-172,194);
  * attention = fused QKV projection -> per-head q/k RMSNorm over head_dim -> NeoX RoPE ->
    paged causal GQA attention -> output projection (qwen3.py:74-96);
  * MLP = fused gate/up projection -> SiLU(gate) * up -> down projection (qwen3.py:123-130);
  * tied input/output embeddings share one tensor (qwen3.py:215-216);
  * ``packed_modules_mapping`` names the Hugging Face tensors that are packed into one local
    matrix (qwen3.py:200-206).

The model is a thin object, not an ``nn.Module`` tree: the per-step attention metadata arrives as an
explicit ``DeviceBatch`` argument (the reference passes it through a module-level global,
tinyvllm/utils/context.py), and each block issues a handful of fused ops:

    add_rms_norm -> qkv GEMM -> [q/k norm + RoPE + KV store] -> attention -> o GEMM (+ all-reduce)
    add_rms_norm -> gate_up GEMM with SiLU*mul epilogue -> down GEMM (+ all-reduce)

On one GPU with the CUDA op set the add + RMSNorm pairs are folded into the GEMMs around them (``fold_norm_weights``).
"""
from __future__ import annotations

import torch

from ..config import ModelConfig
from ..ops import ref as ref_ops
from ..parallel.comm import TPGroup
from ..parallel.tp_layers import (MergedColumnParallelLinear, ParallelLMHead, QKVParallelLinear,
                                  RowParallelLinear, VocabParallelEmbedding)


class Qwen3DecoderLayer:
    def __init__(self, cfg: ModelConfig, tp: TPGroup, dtype, device):
        H, d = cfg.hidden_size, cfg.head_dim
        self.qkv_proj = QKVParallelLinear(H, d, cfg.num_attention_heads, cfg.num_key_value_heads, tp, dtype, device,
                                          bias=cfg.attention_bias)
        self.o_proj = RowParallelLinear(cfg.num_attention_heads * d, H, tp, dtype, device)
        self.gate_up_proj = MergedColumnParallelLinear(H, [cfg.intermediate_size] * 2, tp, dtype, device)
        self.down_proj = RowParallelLinear(cfg.intermediate_size, H, tp, dtype, device)
        self.input_layernorm = torch.ones(H, dtype=dtype, device=device)
        self.post_attention_layernorm = torch.ones(H, dtype=dtype, device=device)
        self.q_norm = torch.ones(d, dtype=dtype, device=device)
        self.k_norm = torch.ones(d, dtype=dtype, device=device)


class Qwen3ForCausalLM:
    # Hugging Face tensor-name fragment -> (local packed module, shard id)
    packed_modules_mapping = {
        "q_proj": ("qkv_proj", "q"),
        "k_proj": ("qkv_proj", "k"),
        "v_proj": ("qkv_proj", "v"),
        "gate_proj": ("gate_up_proj", 0),
        "up_proj": ("gate_up_proj", 1),
    }

    def __init__(self, cfg: ModelConfig, tp: TPGroup | None = None, dtype=None, device="cpu", ops=None,
                 max_positions: int | None = None):
        self.cfg = cfg
        self.tp = tp or TPGroup()
        self.dtype = dtype or cfg.dtype
        self.device = torch.device(device)
        self.ops = ops or ref_ops.RefOps
        tp_size = self.tp.size
        self.num_heads = cfg.num_attention_heads // tp_size
        self.num_kv_heads = cfg.num_key_value_heads // tp_size
        self.head_dim = cfg.head_dim
        self.scale = cfg.head_dim ** -0.5
        self.eps = cfg.rms_norm_eps
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, self.tp, self.dtype, self.device)
        self.layers = [Qwen3DecoderLayer(cfg, self.tp, self.dtype, self.device) for _ in range(cfg.num_hidden_layers)]
        self.norm = torch.ones(cfg.hidden_size, dtype=self.dtype, device=self.device)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, self.tp, self.dtype, self.device)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.embed_tokens.weight
        self.rope = ref_ops.rope_table(max_positions or cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta,
                                       self.device)
        self.kv_cache: torch.Tensor | None = None      # [L, 2, blocks, kv_heads, block_size, d]
        self.norms_folded = False                      # see fold_norm_weights()

    # ------------------------------------------------------------------ parameters by Hugging Face name
    def named_parameters(self):
        yield "model.embed_tokens.weight", self.embed_tokens.weight, self.embed_tokens, None
        for i, l in enumerate(self.layers):
            p = f"model.layers.{i}."
            for hf, (mod, sid) in self.packed_modules_mapping.items():
                kind = "self_attn" if mod == "qkv_proj" else "mlp"
                m = getattr(l, mod)
                yield f"{p}{kind}.{hf}.weight", m.weight, m, sid
                if m.bias is not None:
                    yield f"{p}{kind}.{hf}.bias", m.bias, m, sid
            yield p + "self_attn.o_proj.weight", l.o_proj.weight, l.o_proj, None
            yield p + "mlp.down_proj.weight", l.down_proj.weight, l.down_proj, None
            yield p + "self_attn.q_norm.weight", l.q_norm, None, None
            yield p + "self_attn.k_norm.weight", l.k_norm, None, None
            yield p + "input_layernorm.weight", l.input_layernorm, None, None
            yield p + "post_attention_layernorm.weight", l.post_attention_layernorm, None, None
        yield "model.norm.weight", self.norm, None, None
        if not self.cfg.tie_word_embeddings:
            yield "lm_head.weight", self.lm_head.weight, self.lm_head, None

    def num_parameter_bytes(self) -> int:
        seen, total = set(), 0
        for _, t, _, _ in self.named_parameters():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def bind_kv_cache(self, kv_cache: torch.Tensor) -> None:
        assert kv_cache.shape[0] == len(self.layers) and kv_cache.shape[1] == 2
        self.kv_cache = kv_cache

    # ------------------------------------------------------------------ norm folding (single GPU, CUDA op set)
    def fold_norm_weights(self) -> None:
        """Fold the weight vectors of ``input_layernorm`` / ``post_attention_layernorm`` into the columns of the linear
        layer that follows each (qkv_proj, gate_up_proj).  Afterwards rms_norm(r) * gamma @ W.T == (r @ W'.T) * rsqrt(mean(r^2)
        + eps): the norm becomes a per-row scale in the GEMM epilogue, the residual add moves into the epilogue of the
        GEMM before it, and the two add + RMSNorm launches per block disappear (``_forward_folded``).  Call once, after
        the weights are loaded and before any quantisation."""
        assert not self.norms_folded and self.tp.size == 1
        with torch.no_grad():
            for l in self.layers:
                for lin, gamma in ((l.qkv_proj, l.input_layernorm), (l.gate_up_proj, l.post_attention_layernorm)):
                    lin.weight.copy_((lin.weight.float() * gamma.float()[None, :]).to(lin.weight.dtype))
        self.norms_folded = True

    def _forward_folded(self, batch) -> torch.Tensor:
        """The block loop with the norms folded into the GEMMs (see ``fold_norm_weights``): per block
        qkv GEMM (row scale) -> q/k-norm + RoPE + KV store -> attention -> o GEMM (residual add) ->
        gate_up GEMM (row scale, SiLU*mul) -> down GEMM (residual add).  ``ssq_a`` / ``ssq_b`` carry the rows' sums of
        squares from the GEMM that updates the residual stream to the GEMM that reads it."""
        ops, layers = self.ops, self.layers
        residual, ssq_a, ssq_b = ops.embedding_ssq(batch.input_ids, self.embed_tokens.weight, self.embed_tokens.vocab_start)
        fused_decode = (not batch.is_prefill and self.head_dim == 128 and batch.padded_seqs <= ops.fused_qkv_max_batch)
        in_gemm = not batch.is_prefill and ops.qkv_rope_store_in_gemm(residual.shape[0], self.head_dim, layers[0].qkv_proj.weight)
        for i, l in enumerate(layers):
            kc, vc = self.kv_cache[i, 0], self.kv_cache[i, 1]
            if in_gemm:         # norm, rotation and cache write in the projection's epilogue: one launch less per block
                q = ops.linear_qkv_rope_store(residual, l.qkv_proj.weight, ssq_a, self.eps, l.q_norm, l.k_norm, self.eps, self.rope,
                                              batch.positions, batch.slot_mapping, kc, vc, self.num_heads, self.num_kv_heads)
                a = ops.attention(q, kc, vc, batch, self.scale)
            else:
                qkv = ops.linear_scaled(residual, l.qkv_proj.weight, ssq_a, self.eps)
                if fused_decode:
                    a = ops.decode_attention_qkv(qkv, l.q_norm, l.k_norm, self.eps, self.rope, kc, vc, batch, self.num_heads, self.scale)
                else:
                    q = ops.qk_norm_rope_store(qkv, l.q_norm, l.k_norm, self.eps, self.rope, batch.positions,
                                               batch.slot_mapping, kc, vc, self.num_heads, self.num_kv_heads, self.head_dim)
                    a = ops.attention(q, kc, vc, batch, self.scale)
            ops.linear_residual(a, l.o_proj.weight, residual, ssq_b)
            g = ops.linear_scaled(residual, l.gate_up_proj.weight, ssq_b, self.eps, silu_mul=True)
            ops.linear_residual(g, l.down_proj.weight, residual, ssq_a)
        return ops.rms_norm(residual, self.norm, self.eps)

    # ------------------------------------------------------------------ forward
    def forward(self, batch) -> torch.Tensor:
        """Hidden states ``[tokens, hidden]`` after the final norm.

        The loop carries ``x`` (the normalised input of the next block) and ``residual``.  Each row-parallel
        projection is issued together with the cross-rank sum, the residual add and the norm that follows it,
        so that an op set can fuse the three (``row_linear_add_rms_norm``)."""
        from ..parallel.symm import SITE_DOWN, SITE_O
        if self.norms_folded:
            return self._forward_folded(batch)
        ops = self.ops
        layers = self.layers
        x, residual = ops.embed_norm(batch.input_ids, self.embed_tokens, layers[0].input_layernorm, self.eps)
        # small decode steps on the GPU: q/k-norm + rotation + KV store run inside the attention kernel (one launch less per
        # layer; at large batches the attention kernel is bandwidth-bound and the extra work per sequence costs more)
        fused_decode = (not batch.is_prefill and self.head_dim == 128 and hasattr(ops, "decode_attention_qkv")
                        and batch.padded_seqs <= ops.fused_qkv_max_batch)
        in_gemm = (not batch.is_prefill and hasattr(ops, "qkv_rope_store_in_gemm") and getattr(layers[0].qkv_proj, "bias", None) is None
                   and ops.qkv_rope_store_in_gemm(x.shape[0], self.head_dim, layers[0].qkv_proj.weight))
        for i, l in enumerate(layers):
            kc, vc = self.kv_cache[i, 0], self.kv_cache[i, 1]
            if in_gemm:
                q = ops.linear_qkv_rope_store(x, l.qkv_proj.weight, None, 0.0, l.q_norm, l.k_norm, self.eps, self.rope, batch.positions,
                                              batch.slot_mapping, kc, vc, self.num_heads, self.num_kv_heads)
                a = ops.attention(q, kc, vc, batch, self.scale)
                x, residual = ops.row_linear_add_rms_norm(a, l.o_proj, residual, l.post_attention_layernorm, self.eps, SITE_O)
                g = l.gate_up_proj.forward_silu_mul(ops, x)
                next_norm = layers[i + 1].input_layernorm if i + 1 < len(layers) else self.norm
                x, residual = ops.row_linear_add_rms_norm(g, l.down_proj, residual, next_norm, self.eps, SITE_DOWN)
                continue
            qkv = l.qkv_proj.forward(ops, x)
            if fused_decode:
                a = ops.decode_attention_qkv(qkv, l.q_norm, l.k_norm, self.eps, self.rope, kc, vc, batch, self.num_heads, self.scale)
            else:
                q = ops.qk_norm_rope_store(qkv, l.q_norm, l.k_norm, self.eps, self.rope, batch.positions,
                                           batch.slot_mapping, kc, vc, self.num_heads, self.num_kv_heads, self.head_dim)
                a = ops.attention(q, kc, vc, batch, self.scale)
            x, residual = ops.row_linear_add_rms_norm(a, l.o_proj, residual, l.post_attention_layernorm, self.eps, SITE_O)
            g = l.gate_up_proj.forward_silu_mul(ops, x)
            next_norm = layers[i + 1].input_layernorm if i + 1 < len(layers) else self.norm
            x, residual = ops.row_linear_add_rms_norm(g, l.down_proj, residual, next_norm, self.eps, SITE_DOWN)
        return x

    def compute_logits(self, hidden: torch.Tensor, batch) -> torch.Tensor:
        """This rank's logits shard for the last token of every sequence: ``[seqs, vocab / tp]``."""
        last = self.ops.select_rows(hidden, batch.last_index)
        return self.lm_head.forward(self.ops, last)

    def sample(self, logits: torch.Tensor, batch) -> torch.Tensor:
        return self.ops.sample(logits, batch, self.lm_head.vocab_start, self.tp)

    def step(self, batch) -> torch.Tensor:
        """forward + logits + sampling: token ids for the first ``batch.num_seqs`` rows.  Where the op set can sample in
        the epilogue of the LM-head GEMM, the logits are never materialised (the reference writes them, gathers them to
        rank 0 and samples there: tinyvllm/layers/embed_head.py:58-70, tinyvllm/layers/sampler.py:13-21)."""
        hidden = self.forward(batch)
        ops, head = self.ops, self.lm_head
        rows = batch.last_index.shape[0]
        if (hasattr(ops, "can_sample_in_lm_head") and getattr(head, "bias", None) is None and head.vocab_start % 32 == 0
                and ops.can_sample_in_lm_head(rows, head.weight)):
            last = ops.select_rows(hidden, batch.last_index)
            ids, best = ops.lm_head_sample_shard(last, head.weight, batch.temperatures, batch.header, head.vocab_start)
            return ops.merge_ranks(ids, best, self.tp)
        return self.sample(self.compute_logits(hidden, batch), batch)

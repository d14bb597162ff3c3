"""Run one kernel of the library a few times on a small but larger-than-L2 case (for profilers and quick timing).

    python -m tinyllmforge_b200.utils.kernel_case <case> [--iters N] [--lib] [--peaks FILE]

Cases: decode_attention (64 sequences x 2048 tokens, 16 / 8 heads), decode_attention_g4 (256 x 800, 32 / 8 heads: Qwen3-8B),
decode_attention_g8 (64 x 2304, 64 / 8 heads: Qwen3-32B), prefill_attention, gemm_decode, gemm_decode_split, gemm_prefill,
gemm_prefill_8b (8192 x 6144 x 4096), gemm_silu, gemm_fp8 (256 x 6144 x 4096, block-scaled e4m3 weights), gemm_residual (o_proj-like GEMM with the residual add + sums of squares
epilogue), gemm_scaled (qkv-like GEMM with the folded-norm row scale), gemm_decode_8b_down (256 x 4096 x 12288 with the residual
epilogue: K split over CTA pairs + the reduce kernel), lm_head_sample (LM head + sampling in one kernel),
rms_norm, qk_norm_rope_store, sampler.
``--lib`` runs the library kernel the reference would use on the same case instead (cuBLAS through torch.matmul for the
GEMMs, flash-attn 2 for the attention cases), for a same-box comparison.
Prints the mean device time per launch (CUDA events) and the achieved fraction of the roofline denominator that applies:
copy bandwidth or bf16 GEMM rate, read from ``--peaks FILE`` (JSON with ``hbm_gbs`` and ``bf16_tflops``, as measured on
the machine) or else the nominal 6650 GB/s and 1590 TFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

BF = torch.bfloat16


def _peaks(path):
    if path and os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class _B:
    pass


def _paged(B, ctx, nq, nkv, bs, q_len=1):
    nblk = -(-ctx // bs)
    total = B * nblk
    bt = torch.randperm(total, dtype=torch.int32).view(B, nblk).cuda()
    kc = torch.randn(total, nkv, bs, 128, device="cuda", dtype=BF)
    vc = torch.randn(total, nkv, bs, 128, device="cuda", dtype=BF)
    q = torch.randn(B * q_len, nq, 128, device="cuda", dtype=BF)
    b = _B()
    b.is_prefill = q_len > 1
    b.cu_seqlens_q = (torch.arange(B + 1, dtype=torch.int32) * q_len).cuda()
    b.context_lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    b.block_tables = bt
    b.num_seqs = b.padded_seqs = B
    b.max_seqlen_q, b.max_seqlen_k, b.table_width = q_len, ctx, nblk
    return q, kc, vc, b


def build(case: str, ops, lib: bool = False):
    """Returns (callable, bytes moved per launch, flops per launch)."""
    if case in ("decode_attention", "decode_attention_g4", "decode_attention_g8"):
        B, ctx, nq, nkv = {"decode_attention": (64, 2048, 16, 8), "decode_attention_g4": (256, 800, 32, 8),
                           "decode_attention_g8": (64, 2304, 64, 8)}[case]
        ctx_alloc = -(-ctx // 256) * 256
        q, kc, vc, b = _paged(B, ctx_alloc, nq, nkv, 256)
        b.context_lens.fill_(ctx)
        b.max_seqlen_k = ctx
        nbytes = 2 * B * ctx * nkv * 128 * 2
        if lib:
            from flash_attn import flash_attn_with_kvcache
            kf, vf = kc.transpose(1, 2).contiguous(), vc.transpose(1, 2).contiguous()      # flash-attn: [blocks, block_size, heads, 128]
            q4 = q.view(B, 1, nq, 128)
            return (lambda: flash_attn_with_kvcache(q4, kf, vf, cache_seqlens=b.context_lens, block_table=b.block_tables, causal=True)), nbytes, 0
        return (lambda: ops.attention(q, kc, vc, b, 128 ** -0.5)), nbytes, 0
    if case == "prefill_attention":
        q, kc, vc, b = _paged(8, 2048, 16, 8, 256, q_len=2048)
        flops = 4 * 8 * 16 * 2048 * 2048 * 128 // 2
        if lib:
            from flash_attn import flash_attn_varlen_func
            k = torch.randn(8 * 2048, 8, 128, device="cuda", dtype=BF)
            v = torch.randn_like(k)
            cu = b.cu_seqlens_q
            return (lambda: flash_attn_varlen_func(q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=2048, max_seqlen_k=2048, causal=True)), 0, flops
        return (lambda: ops.attention(q, kc, vc, b, 128 ** -0.5)), 0, flops
    if case in ("gemm_decode", "gemm_decode_split", "gemm_prefill", "gemm_prefill_8b", "gemm_silu"):
        M, N, K = {"gemm_decode": (64, 151936, 1024), "gemm_decode_split": (64, 1024, 3072), "gemm_prefill": (8192, 4096, 1024),
                   "gemm_prefill_8b": (8192, 6144, 4096), "gemm_silu": (8192, 3072, 1024)}[case]
        nw = 1 if case != "gemm_decode_split" else 28
        rows = 2 * N if case == "gemm_silu" else N
        ws = [torch.randn(rows, K, device="cuda", dtype=BF) * 0.02 for _ in range(nw)]
        x = torch.randn(M, K, device="cuda", dtype=BF)
        state = {"i": 0}

        def run():
            w = ws[state["i"] % nw]
            state["i"] += 1
            if lib:
                return torch.matmul(x, w.t())          # the library GEMM alone (the reference runs SiLU * mul as another kernel)
            return ops.linear_silu_mul(x, w) if case == "gemm_silu" else ops.linear(x, w)
        return run, (rows * K + M * K + M * N) * 2, 2 * M * rows * K
    if case in ("gemm_residual", "gemm_scaled", "gemm_decode_8b_down"):
        M, N, K = {"gemm_residual": (256, 1024, 2048), "gemm_scaled": (256, 4096, 1024), "gemm_decode_8b_down": (256, 4096, 12288)}[case]
        nw = 28 if N * K < (8 << 20) else 8
        ws = [torch.randn(N, K, device="cuda", dtype=BF) * 0.02 for _ in range(nw)]           # several weights in turn: each launch streams from HBM
        x = torch.randn(M, K, device="cuda", dtype=BF)
        res = torch.randn(M, N, device="cuda", dtype=BF)
        ssq_out = torch.empty(M, (N + 127) // 128, dtype=torch.float32, device="cuda")
        ssq_in = (x.float() ** 2).view(M, K // 128, 128).sum(-1).contiguous()
        state = {"i": 0}

        def run():
            w = ws[state["i"] % nw]
            state["i"] += 1
            if lib:
                return torch.matmul(x, w.t())
            if case in ("gemm_residual", "gemm_decode_8b_down"):
                return ops.linear_residual(x, w, res, ssq_out)
            return ops.linear_scaled(x, w, ssq_in, 1e-6)
        return run, (N * K + M * K + 2 * M * N) * 2, 2 * M * N * K
    if case == "gemm_fp8":
        from ..ops.quant import Fp8BlockWeight
        M, N, K = 256, 6144, 4096                          # Qwen3-8B qkv projection at a decode batch of 256
        ws = [Fp8BlockWeight.quantize(torch.randn(N, K, device="cuda", dtype=BF) * 0.02) for _ in range(8)]
        wb = [torch.randn(N, K, device="cuda", dtype=BF) * 0.02 for _ in range(8)]
        x = torch.randn(M, K, device="cuda", dtype=BF)
        state = {"i": 0}

        def run():
            i = state["i"] % 8
            state["i"] += 1
            return torch.matmul(x, wb[i].t()) if lib else ops.linear_fp8(x, ws[i])
        return run, (N * K * (2 if lib else 1) + M * K * 2 + M * N * 2), 2 * M * N * K
    if case == "lm_head_sample":
        rows, V, K = 256, 151936, 1024
        w = torch.randn(V, K, device="cuda", dtype=BF) * 0.02
        x = torch.randn(rows, K, device="cuda", dtype=BF)
        temps = torch.full((rows,), 0.6, device="cuda")
        hdr = torch.zeros(16, dtype=torch.int32, device="cuda")
        if lib:
            return (lambda: torch.matmul(x, w.t())), (V * K + rows * K + rows * V) * 2, 2 * rows * V * K
        return (lambda: ops.lm_head_sample_shard(x, w, temps, hdr, 0)), (V * K + rows * K) * 2, 2 * rows * V * K
    if case == "rms_norm":
        x, r = torch.randn(16384, 4096, device="cuda", dtype=BF), torch.randn(16384, 4096, device="cuda", dtype=BF)
        w = torch.ones(4096, device="cuda", dtype=BF)
        return (lambda: ops.add_rms_norm(x, r, w, 1e-6)), 4 * 16384 * 4096 * 2, 0
    if case == "qk_norm_rope_store":
        from . import synth  # noqa: F401  (package import check)
        from ..ops import ref
        T, nq, nkv, bs = 16384, 16, 8, 256
        qkv = torch.randn(T, (nq + 2 * nkv) * 128, device="cuda", dtype=BF)
        w = torch.ones(128, device="cuda", dtype=BF)
        table = ref.rope_table(4096, 128, 1e6, "cuda")
        pos = torch.randint(0, 4096, (T,), dtype=torch.int32, device="cuda")
        slots = torch.randperm(T, dtype=torch.int32).cuda()
        kc = torch.zeros(T // bs, nkv, bs, 128, device="cuda", dtype=BF)
        vc = torch.zeros_like(kc)
        return (lambda: ops.qk_norm_rope_store(qkv, w, w, 1e-6, table, pos, slots, kc, vc, nq, nkv, 128)), 2 * T * (nq + 2 * nkv) * 128 * 2, 0
    if case == "sampler":
        logits = torch.randn(256, 151936, device="cuda", dtype=BF)
        temps = torch.full((256,), 0.6, device="cuda")
        hdr = torch.zeros(16, dtype=torch.int32, device="cuda")
        return (lambda: ops.sample_shard(logits, temps, hdr, 0)), 256 * 151936 * 2, 0
    raise SystemExit(f"unknown case {case!r}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--lib", action="store_true", help="time the library kernel the reference uses on the same case")
    ap.add_argument("--peaks", default=None, help="JSON file with hbm_gbs and bf16_tflops measured on this machine")
    args = ap.parse_args()
    from ..ops.cuda import CudaOps
    ops = CudaOps()
    fn, nbytes, flops = build(args.case, ops, args.lib)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ops.check_status()
    us = e0.elapsed_time(e1) * 1e3 / args.iters
    hbm, tf, src = _peaks(args.peaks)
    out = {"case": args.case + (" (library kernel)" if args.lib else ""), "us_per_launch": round(us, 2)}
    if nbytes:
        out["GB_per_s"] = round(nbytes / us / 1e3, 1)
        out[f"fraction_of_{src}_copy_bandwidth"] = round(nbytes / us / 1e3 / hbm, 3)
    if flops:
        out["TFLOP_per_s"] = round(flops / us / 1e6, 1)
        out[f"fraction_of_{src}_bf16_gemm_rate"] = round(flops / us / 1e6 / tf, 3)
    print(json.dumps(out))


if __name__ == "__main__":
    main()

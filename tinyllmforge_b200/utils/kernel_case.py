"""Run one kernel of the library a few times on a small but larger-than-L2 case (for profilers and quick timing).

    python -m tinyllmforge_b200.utils.kernel_case <case> [--iters N]

Cases: decode_attention, prefill_attention, gemm_decode, gemm_decode_split, gemm_prefill, gemm_silu, rms_norm,
qk_norm_rope_store, sampler.  Prints the mean device time per launch (CUDA events) and the achieved fraction of
the roofline denominator that applies (measured copy bandwidth or measured bf16 GEMM rate, from
MEASURED_PEAKS.json when present).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

BF = torch.bfloat16


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
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


def build(case: str, ops):
    """Returns (callable, bytes moved per launch, flops per launch)."""
    if case == "decode_attention":
        q, kc, vc, b = _paged(64, 2048, 16, 8, 256)
        nbytes = 2 * 64 * 2048 * 8 * 128 * 2
        return (lambda: ops.attention(q, kc, vc, b, 128 ** -0.5)), nbytes, 0
    if case == "prefill_attention":
        q, kc, vc, b = _paged(8, 2048, 16, 8, 256, q_len=2048)
        flops = 4 * 8 * 16 * 2048 * 2048 * 128 // 2
        return (lambda: ops.attention(q, kc, vc, b, 128 ** -0.5)), 0, flops
    if case in ("gemm_decode", "gemm_decode_split", "gemm_prefill", "gemm_silu"):
        M, N, K = {"gemm_decode": (64, 151936, 1024), "gemm_decode_split": (64, 1024, 3072), "gemm_prefill": (8192, 4096, 1024),
                   "gemm_silu": (8192, 3072, 1024)}[case]
        nw = 1 if case != "gemm_decode_split" else 28
        rows = 2 * N if case == "gemm_silu" else N
        ws = [torch.randn(rows, K, device="cuda", dtype=BF) * 0.02 for _ in range(nw)]
        x = torch.randn(M, K, device="cuda", dtype=BF)
        state = {"i": 0}

        def run():
            w = ws[state["i"] % nw]
            state["i"] += 1
            return ops.linear_silu_mul(x, w) if case == "gemm_silu" else ops.linear(x, w)
        return run, (rows * K + M * K + M * N) * 2, 2 * M * rows * K
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
    args = ap.parse_args()
    from ..ops.cuda import CudaOps
    ops = CudaOps()
    fn, nbytes, flops = build(args.case, ops)
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
    hbm, tf, src = _peaks()
    out = {"case": args.case, "us_per_launch": round(us, 2)}
    if nbytes:
        out["GB_per_s"] = round(nbytes / us / 1e3, 1)
        out[f"fraction_of_{src}_copy_bandwidth"] = round(nbytes / us / 1e3 / hbm, 3)
    if flops:
        out["TFLOP_per_s"] = round(flops / us / 1e6, 1)
        out[f"fraction_of_{src}_bf16_gemm_rate"] = round(flops / us / 1e6 / tf, 3)
    print(json.dumps(out))


if __name__ == "__main__":
    main()

"""The Qwen3 model on the CUDA op set against the same model on the PyTorch op set in fp32, same weights: logits of a
prefill step, of a prefill step whose prompt prefix is already in the KV cache, and of decode steps through the paged
cache (three layers with the Qwen3-0.6B layer shapes, a 256-token cache block, random weights with spread-out logits).

The oracle (``ops/ref.py`` in fp32 on the CPU) is itself checked against Hugging Face transformers in
``tests/test_model_cpu.py``; this test closes the chain for the sm_100a kernels as they are composed by the model."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BS = 256


def _models(fold):
    from tinyllmforge_b200 import preset
    from tinyllmforge_b200.models.qwen3 import Qwen3ForCausalLM
    from tinyllmforge_b200.ops.cuda import CudaOps
    cfg = preset("qwen3-0.6b", num_hidden_layers=3, vocab_size=4096)
    ref = Qwen3ForCausalLM(cfg, None, torch.float32, "cpu", max_positions=2048)
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for name, t, _, _ in ref.named_parameters():
            if t.dim() >= 2:
                t.normal_(0.0, 0.05, generator=g)
            else:
                t.copy_(1.0 + 0.1 * torch.randn(t.shape, generator=g))
        # the fp32 oracle computes with the values the bf16 model holds
        for name, t, _, _ in ref.named_parameters():
            t.copy_(t.bfloat16().float())
    dev = torch.device("cuda", 0)
    ops = CudaOps(None, None, dev)
    gpu = Qwen3ForCausalLM(cfg, None, torch.bfloat16, dev, ops, max_positions=2048)
    with torch.no_grad():
        for (_, a, _, _), (_, b, _, _) in zip(ref.named_parameters(), gpu.named_parameters()):
            b.copy_(a.to(torch.bfloat16))
    if fold:                 # add + RMSNorm folded into the GEMM epilogues: what the engine runs on one GPU
        gpu.fold_norm_weights()
    kvh = cfg.num_key_value_heads
    ref.bind_kv_cache(torch.zeros(cfg.num_hidden_layers, 2, 16, kvh, BS, cfg.head_dim))
    gpu.bind_kv_cache(torch.zeros(cfg.num_hidden_layers, 2, 16, kvh, BS, cfg.head_dim, dtype=torch.bfloat16, device=dev))
    return cfg, ref, gpu, ops


def _batches(sb):
    from tinyllmforge_b200.engine.worker import DeviceBatch
    words = torch.from_numpy(sb.buf[:sb.num_words].copy())
    return DeviceBatch(sb, words), DeviceBatch(sb, words.cuda())


def _check(ref, gpu, sb, what):
    cpu_b, gpu_b = _batches(sb)
    with torch.inference_mode():
        want = ref.compute_logits(ref.forward(cpu_b), cpu_b)
        got = gpu.compute_logits(gpu.forward(gpu_b), gpu_b).float().cpu()
    scale = want.abs().max().item()
    err = (got - want).abs().max().item()
    # bf16 activations through three blocks against fp32: a few bf16 ulps of the largest logit
    assert err <= 3e-2 * scale, f"{what}: max |logit error| {err:.4g} vs largest logit {scale:.4g}"
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean().item()
    return want, agree


@pytest.mark.parametrize("fold,qkv_epilogue", [(True, False), (False, False), (True, True), (False, True)])
def test_cuda_model_logits_match_the_fp32_model(fold, qkv_epilogue):
    from tinyllmforge_b200 import SamplingParams
    from tinyllmforge_b200.engine.request import Request
    from tinyllmforge_b200.engine.step_batch import build_decode, build_prefill
    cfg, ref, gpu, ops = _models(fold)
    if qkv_epilogue:             # optional path: q/k-norm + RoPE + KV store in the qkv projection's epilogue, here for any decode step
        ops.qkv_epilogue, ops.qkv_epilogue_min_rows = True, 1
    rng = np.random.default_rng(0)
    reqs, nblk = [], 0
    for n in (5, 300, 257, 700):
        r = Request(rng.integers(0, cfg.vocab_size, n).tolist(), SamplingParams(temperature=0.0))
        need = -(-(n + 8) // BS)
        r.block_table = list(range(nblk, nblk + need))
        nblk += need
        reqs.append(r)
    agree = []
    want, a = _check(ref, gpu, build_prefill(reqs, BS), "prefill")
    agree.append(a)
    for step in range(3):                                   # decode through the paged cache, both models fed the oracle's tokens
        for r, t in zip(reqs, want.argmax(-1).tolist()):
            r.append_token(t)
        want, a = _check(ref, gpu, build_decode(reqs, BS), f"decode step {step}")
        agree.append(a)
    # a prompt whose first block is already cached (the cache holds request 3's tokens): only the tail is computed
    tail = Request(reqs[3].token_ids[:BS] + rng.integers(0, cfg.vocab_size, 90).tolist(), SamplingParams(temperature=0.0))
    tail.block_table = [reqs[3].block_table[0], nblk]
    tail.num_cached_tokens = BS
    _, a = _check(ref, gpu, build_prefill([tail], BS), "prefill with a cached prefix")
    agree.append(a)
    ops.check_status()
    assert min(agree) >= 0.75, agree                        # greedy tokens agree except at near-ties

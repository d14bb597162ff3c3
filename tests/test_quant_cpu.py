"""Block-scaled fp8 weights: quantiser round trip, reference GEMM error, engine path on CPU."""
import random

import torch

from tinyllmforge_b200 import LLM, SamplingParams, preset
from tinyllmforge_b200.ops.quant import Fp8BlockWeight, linear_fp8_ref, quantize_activations_ref


def test_weight_quantiser_round_trip():
    torch.manual_seed(0)
    w = torch.randn(300, 384) * 0.05
    q = Fp8BlockWeight.quantize(w)
    assert q.q.dtype == torch.float8_e4m3fn and q.scale.shape == (3, 3)
    rel = (q.dequantize() - w).norm() / w.norm()
    assert rel < 0.04
    blocks_max = q.q.float().abs().max()
    assert blocks_max <= 448


def test_activation_quantiser_scales_per_token_and_block():
    x = torch.zeros(3, 256)
    x[0, :128] = 1.0
    x[1, 128:] = -4.0
    q, s = quantize_activations_ref(x)
    assert s.shape == (2, 3)
    assert torch.allclose(s[:, 0], torch.tensor([1 / 448, 1.0])) and torch.allclose(s[:, 1], torch.tensor([1.0, 4 / 448]))
    assert torch.all(s[:, 2] == 1.0) and torch.all(q[2].float() == 0)


def test_fp8_linear_is_close_to_exact():
    torch.manual_seed(1)
    x, w = torch.randn(9, 512), torch.randn(200, 512) * 0.05
    y = linear_fp8_ref(x, Fp8BlockWeight.quantize(w))
    exact = x @ w.t()
    assert (y - exact).norm() / exact.norm() < 0.06


def test_engine_runs_with_fp8_weights_on_cpu():
    rng = random.Random(0)
    prompts = [[rng.randrange(4096) for _ in range(20)] for _ in range(2)]
    kw = dict(hf_config=preset("tiny", hidden_size=256, intermediate_size=512), load_format="dummy", skip_tokenizer_init=True,
              device="cpu", kvcache_block_size=16, max_model_len=256, max_num_batched_tokens=256, num_kvcache_blocks=32)
    a = LLM("x", quantization="fp8_block", **kw)
    out = a.generate(prompts, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True), use_tqdm=False)
    assert all(len(o["token_ids"]) == 4 for o in out)
    assert isinstance(a.worker.model.layers[0].qkv_proj.weight, Fp8BlockWeight)
    a.exit()

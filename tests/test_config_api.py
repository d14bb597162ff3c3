"""Public surface: LLM / SamplingParams / Config (tinyvllm/__init__.py, config.py, sampling_params.py)."""
import json

import pytest
import torch

from tinyllmforge_b200 import Config, ModelConfig, SamplingParams, preset


def test_sampling_params_defaults_match_reference():
    sp = SamplingParams()
    assert (sp.temperature, sp.max_tokens, sp.ignore_eos) == (1.0, 64, False)
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1)


def test_config_defaults_match_reference():
    c = Config("x", hf_config=preset("qwen3-0.6b"), device="cpu")
    assert (c.max_num_batched_tokens, c.max_num_seqs, c.max_model_len, c.gpu_memory_utilization,
            c.tensor_parallel_size, c.enforce_eager, c.kvcache_block_size, c.num_kvcache_blocks) == \
        (16384, 512, 4096, 0.9, 1, False, 256, -1)
    assert c.dtype == torch.bfloat16


def test_unknown_kwargs_are_rejected():
    with pytest.raises(TypeError, match="tensor_paralel_size"):
        Config.from_kwargs("x", hf_config=preset("tiny"), tensor_paralel_size=2)


def test_validation():
    with pytest.raises(ValueError):
        Config("x", hf_config=preset("tiny"), kvcache_block_size=24, device="cpu")
    with pytest.raises(ValueError):
        Config("x", hf_config=preset("tiny"), tensor_parallel_size=9, device="cpu")
    with pytest.raises(ValueError):
        Config("x", hf_config=preset("tiny"), tensor_parallel_size=4, device="cpu")       # 2 KV heads
    with pytest.raises(ValueError):
        Config("x", hf_config=preset("tiny"), max_num_batched_tokens=100, max_model_len=200, device="cpu")
    c = Config("x", hf_config=preset("tiny"), max_num_batched_tokens=100, max_model_len=200, kvcache_block_size=16, device="cpu",
               chunked_prefill=True)
    assert c.chunked_prefill and c.max_num_batched_tokens < c.max_model_len          # chunked prefill lifts the whole-prompt rule
    with pytest.raises(ValueError):
        Config("x", hf_config=preset("tiny"), max_num_batched_tokens=8, max_model_len=200, kvcache_block_size=16, device="cpu",
               chunked_prefill=True)                                                   # a step must hold at least one KV block
    with pytest.raises(FileNotFoundError):
        Config("/nonexistent/model/dir")
    c = Config("x", hf_config=preset("tiny"), max_model_len=1 << 20, max_num_batched_tokens=1 << 20, device="cpu")
    assert c.max_model_len == 4096                      # clamped to max_position_embeddings


def test_model_config_reads_hf_json(tmp_path):
    d = preset("qwen3-8b").to_hf_dict()
    (tmp_path / "config.json").write_text(json.dumps(d))
    mc = ModelConfig.from_dir(str(tmp_path))
    assert (mc.hidden_size, mc.num_hidden_layers, mc.num_attention_heads, mc.num_key_value_heads, mc.intermediate_size,
            mc.tie_word_embeddings) == (4096, 36, 32, 8, 12288, False)
    d["rope_scaling"] = {"rope_type": "yarn", "factor": 4.0}
    with pytest.raises(ValueError):
        ModelConfig.from_dict(d)
    # transformers >= 5 spelling
    d2 = {k: v for k, v in preset("tiny").to_hf_dict().items() if k not in ("rope_theta", "rope_scaling")}
    d2["rope_parameters"] = {"rope_type": "default", "rope_theta": 5e5}
    assert ModelConfig.from_dict(d2).rope_theta == 5e5

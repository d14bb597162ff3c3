"""The Qwen3 model on the PyTorch op set against Hugging Face transformers (random-init, fp32):
logits of a prefill and of decode steps through the paged KV cache; weight loading incl. TP shards."""
import numpy as np
import pytest
import torch

from tinyllmforge_b200 import SamplingParams, preset
from tinyllmforge_b200.engine.request import Request
from tinyllmforge_b200.engine.step_batch import build_decode, build_prefill
from tinyllmforge_b200.engine.worker import DeviceBatch
from tinyllmforge_b200.models.qwen3 import Qwen3ForCausalLM
from tinyllmforge_b200.parallel.comm import TPGroup
from tinyllmforge_b200.utils.synth import write_checkpoint
from tinyllmforge_b200.utils.weights import load_weights

BS = 16


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("tiny"))
    write_checkpoint(path, preset("tiny"), seed=0, std=0.2, norm_std=0.1)     # large std: non-degenerate logits
    return path


@pytest.fixture(scope="module")
def hf(ckpt):
    from transformers import AutoModelForCausalLM
    m = AutoModelForCausalLM.from_pretrained(ckpt, dtype=torch.float32)
    return m.eval()


def _model(ckpt, tp=None):
    cfg = preset("tiny")
    m = Qwen3ForCausalLM(cfg, tp, torch.float32, "cpu", max_positions=512)
    with torch.no_grad():
        load_weights(m, ckpt)
    kvh = cfg.num_key_value_heads // m.tp.size
    m.bind_kv_cache(torch.zeros(cfg.num_hidden_layers, 2, 64, kvh, BS, cfg.head_dim))
    return m


def _batch(sb):
    return DeviceBatch(sb, torch.from_numpy(sb.buf[:sb.num_words]))


def test_prefill_and_decode_logits_match_transformers(ckpt, hf):
    m = _model(ckpt)
    rng = np.random.default_rng(0)
    reqs = []
    nblk = 0
    for n in (5, 16, 37):
        r = Request(rng.integers(0, 4096, n).tolist(), SamplingParams(temperature=0.0))
        need = -(-(n + 4) // BS)
        r.block_table = list(range(nblk, nblk + need))
        nblk += need
        reqs.append(r)
    with torch.no_grad():
        b = _batch(build_prefill(reqs, BS))
        logits = m.compute_logits(m.forward(b), b)
        for i, r in enumerate(reqs):
            want = hf(torch.tensor([r.token_ids])).logits[0, -1]
            assert torch.allclose(logits[i], want, atol=2e-4, rtol=1e-4), (logits[i] - want).abs().max()
        for _ in range(3):                                   # decode through the paged cache
            toks = logits.argmax(-1).tolist()
            for r, t in zip(reqs, toks):
                r.append_token(t)
            b = _batch(build_decode(reqs, BS))
            logits = m.compute_logits(m.forward(b), b)
            for i, r in enumerate(reqs):
                want = hf(torch.tensor([r.token_ids])).logits[0, -1]
                assert torch.allclose(logits[i], want, atol=2e-4, rtol=1e-4)


def test_prefill_with_cached_prefix_equals_full_prefill(ckpt):
    m = _model(ckpt)
    toks = np.random.default_rng(1).integers(0, 4096, 40).tolist()
    a = Request(toks, SamplingParams())
    a.block_table = [0, 1, 2]
    with torch.no_grad():
        b = _batch(build_prefill([a], BS))
        full = m.compute_logits(m.forward(b), b)
        c = Request(toks, SamplingParams())                  # same blocks, first 32 tokens already cached
        c.block_table = [0, 1, 2]
        c.num_cached_tokens = 32
        b2 = _batch(build_prefill([c], BS))
        assert b2.num_tokens == 8
        part = m.compute_logits(m.forward(b2), b2)
    assert torch.allclose(full, part, atol=2e-4, rtol=1e-4)


class _FakeTP(TPGroup):
    """A tensor-parallel group of one process: collectives are exercised by summing shards by hand."""
    def __init__(self, rank, size):
        super().__init__(rank, size, None)


def test_tp_shards_reassemble_to_full_weights(ckpt):
    full = _model(ckpt)
    shards = [_model(ckpt, _FakeTP(r, 2)) for r in range(2)]
    l0, s0, s1 = full.layers[0], shards[0].layers[0], shards[1].layers[0]
    d, nh, nkv = 64, 4, 2
    q, k, v = full.layers[0].qkv_proj.weight.split([nh * d, nkv * d, nkv * d])
    for r, s in enumerate((s0, s1)):
        sq, sk, sv = s.qkv_proj.weight.split([nh * d // 2, nkv * d // 2, nkv * d // 2])
        assert torch.equal(sq, q[r * nh * d // 2:(r + 1) * nh * d // 2])
        assert torch.equal(sk, k[r * nkv * d // 2:(r + 1) * nkv * d // 2])
        assert torch.equal(sv, v[r * nkv * d // 2:(r + 1) * nkv * d // 2])
    I = 512
    assert torch.equal(torch.cat([s0.gate_up_proj.weight[:I // 2], s1.gate_up_proj.weight[:I // 2]]), l0.gate_up_proj.weight[:I])
    assert torch.equal(torch.cat([s0.gate_up_proj.weight[I // 2:], s1.gate_up_proj.weight[I // 2:]]), l0.gate_up_proj.weight[I:])
    assert torch.equal(torch.cat([s0.o_proj.weight, s1.o_proj.weight], dim=1), l0.o_proj.weight)
    assert torch.equal(torch.cat([s0.down_proj.weight, s1.down_proj.weight], dim=1), l0.down_proj.weight)
    assert torch.equal(torch.cat([shards[0].embed_tokens.weight, shards[1].embed_tokens.weight]), full.embed_tokens.weight)
    assert shards[1].lm_head.weight is shards[1].embed_tokens.weight          # tied


def test_loader_reports_missing_and_unexpected(ckpt, tmp_path):
    import shutil
    from safetensors.torch import load_file, save_file
    dst = tmp_path / "broken"
    shutil.copytree(ckpt, dst)
    t = {k: v.clone() for k, v in load_file(str(dst / "model.safetensors")).items()}   # detach from the mmap before rewriting
    t.pop("model.layers.1.mlp.down_proj.weight")
    save_file(t, str(dst / "model.safetensors"))
    m = Qwen3ForCausalLM(preset("tiny"), None, torch.float32, "cpu", max_positions=64)
    with pytest.raises(KeyError, match="missing"):
        load_weights(m, str(dst))
    t["bogus.weight"] = torch.zeros(1)
    t["model.layers.1.mlp.down_proj.weight"] = torch.zeros(256, 512)
    save_file(t, str(dst / "model.safetensors"))
    with pytest.raises(KeyError, match="unexpected"):
        load_weights(m, str(dst))

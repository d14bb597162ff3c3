"""In-kernel tensor-parallel exchange on 2+ GPUs: row-parallel GEMM + signal, one-shot / two-shot fused reduce/add/RMSNorm,
owner-writes embedding, sampler pair merge, and the engine end to end (fused exchange vs NCCL path vs one GPU).
Each case runs as one process per GPU; oracles are single-GPU fp32 math and the NCCL path."""
import os
import random
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worker(rank, world, port, fn_name, ret):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank,
                            device_id=torch.device("cuda", rank))
    try:
        out = globals()[fn_name](rank, world)
        ret[rank] = ("ok", out)
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = ("err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}")
    finally:
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


def _run(fn_name, world=2):
    import torch.multiprocessing as mp
    from tinyllmforge_b200.parallel.comm import find_free_port
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = find_free_port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, fn_name, ret)) for r in range(world)]
    [p.start() for p in ps]
    [p.join(300) for p in ps]
    for r in range(world):
        assert r in ret, f"rank {r} produced no result (exit code {ps[r].exitcode})"
        assert ret[r][0] == "ok", ret[r][1]
    return [ret[r][1] for r in range(world)]


def _ops(rank, world):
    import torch.distributed as dist
    from tinyllmforge_b200.ops.cuda import CudaOps
    from tinyllmforge_b200.parallel.comm import TPGroup
    tp = TPGroup(rank, world, dist.group.WORLD)
    ops = CudaOps(None, tp, torch.device("cuda", rank))
    return ops, tp


class _Layer:
    def __init__(self, tp, weight):
        self.tp, self.weight = tp, weight


def _row_linear_rounds(ops, tp, rank, world, g, sizes, mode):
    """Row-parallel layer + exchange + residual add + RMSNorm for every M of ``sizes`` (sites alternate, epochs advance,
    buffers are reused).  mode: "auto" = what the engine does (tagged words up to 256 rows, pulls above); "one" / "two"
    switch the tagged path off and force the one-shot / the reduce-scatter + all-gather pull consumer.  Returns the worst
    error relative to the largest expected magnitude."""
    from tinyllmforge_b200.ops import ref
    from tinyllmforge_b200.parallel.symm import SITE_DOWN, SITE_O
    H, Kfull = 1024, 2048
    f = ops.fused
    keep = (f.two_shot_bytes, f.tagged)
    f.two_shot_bytes = {"one": 1 << 60, "two": -1, "auto": keep[0]}[mode]
    f.tagged = keep[1] and mode == "auto"
    w_full = (torch.randn(H, Kfull, device="cuda", generator=g) * 0.05).bfloat16()
    norm_w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    kshard = Kfull // world
    layer = _Layer(tp, w_full[:, rank * kshard:(rank + 1) * kshard].contiguous())
    worst = 0.0
    for it, M in enumerate(sizes):
        x_full = torch.randn(M, Kfull, device="cuda", generator=g).bfloat16()
        res = torch.randn(M, H, device="cuda", generator=g).bfloat16()
        x = x_full[:, rank * kshard:(rank + 1) * kshard].contiguous()
        res_in = res.clone()
        tagged = f.use_tagged(M, H)
        two = tagged or f.two_shot(M, H)
        y, res_out = ops.row_linear_add_rms_norm(x, layer, res_in, norm_w, 1e-6, SITE_O if it % 2 == 0 else SITE_DOWN)
        y = y.clone()                                  # two-shot: y is the broadcast buffer, reused by the next exchange
        h = x_full.float() @ w_full.float().t()
        want_y, want_res = ref.add_rms_norm(h.bfloat16(), res, norm_w, 1e-6)
        mine = slice(rank, None, world) if two else slice(None)       # two-shot keeps the residual sharded by rows
        e1 = ((res_out[mine].float() - want_res[mine].float()).abs().max() / want_res.float().abs().max()).item() if res_out[mine].numel() else 0.0
        e2 = ((y.float() - want_y.float()).abs().max() / want_y.float().abs().max()).item()
        worst = max(worst, e1, e2)
        assert e1 <= 3e-2 and e2 <= 3e-2, (mode, M, two, e1, e2)
        if f.multicast_ptr == 0 or tagged:
            # plain peer loads add in rank order, and a tagged row is computed by one rank: bit-identical rows everywhere
            both = tp.all_gather_stack(y)
            assert all(torch.equal(both[0], both[r]) for r in range(world)), (mode, M)
    f.two_shot_bytes, f.tagged = keep
    return worst


def case_row_linear(rank, world):
    """o_proj-like layer: every batch size 1..256 in steps, 300 and 4096 rows (token-tile GEMM), one-shot and two-shot
    consumers, through the switch (multimem) where the allocation has a multicast address and with plain peer accesses."""
    ops, tp = _ops(rank, world)
    H = 1024
    worst = 0.0
    for nvls in ("1", "0"):
        os.environ["FORGE_NVLS"] = nvls
        ops.enable_fused_comm(H, 4096)
        if rank == 0:
            print(f"FORGE_NVLS={nvls}: multicast address {hex(ops.fused.multicast_ptr)}", flush=True)
        if nvls == "1" and ops.fused.multicast_ptr == 0:
            ops.close()
            continue                                     # no multicast support: the second round covers the only path there is
        g = torch.Generator(device="cuda").manual_seed(1)           # same stream of numbers on every rank
        worst = max(worst, _row_linear_rounds(ops, tp, rank, world, g, [1, 7, 64, 200, 256, 33, 300, 4096, 256] + list(range(2, 257, 23)), "auto"))
        worst = max(worst, _row_linear_rounds(ops, tp, rank, world, g, [1, 2, 3, 5, 8, 16, 31, 64, 100, 128, 255, 256, 300, 1000], "two"))
        worst = max(worst, _row_linear_rounds(ops, tp, rank, world, g, list(range(1, 257, 17)) + [300, 4096], "one"))
        # standalone all-reduce and barrier through the same region
        for shape in ((1, 8), (256, H), (3, 5, 64), (100, 2048)):
            mine = (torch.randn(*shape, device="cuda", generator=g) + rank).bfloat16()
            parts = tp.all_gather_stack(mine)
            got = ops.fused_all_reduce(mine)
            want = parts.float().sum(0)
            assert got.shape == mine.shape and (got.float() - want).abs().max().item() <= 0.04 * want.abs().max().item() + 1e-3
            if ops.fused.multicast_ptr == 0:
                gathered = tp.all_gather_stack(got)
                assert all(torch.equal(gathered[0], gathered[r]) for r in range(world))
        # measurement mode: no waits, own data only; runs, touches no peer, and leaves the epochs consistent
        ops.fused_barrier()
        torch.cuda.synchronize()
        tp.barrier()
        ops.fused.set_local_only(True)
        _ = ops.fused_all_reduce(torch.ones(4, H, device="cuda", dtype=torch.bfloat16))
        ops.fused.set_local_only(False)
        torch.cuda.synchronize()
        tp.barrier()
        got = ops.fused_all_reduce(torch.ones(4, H, device="cuda", dtype=torch.bfloat16))
        assert torch.equal(got, torch.full_like(got, float(world)))
        ops.fused_barrier()
        ops.check_status()
        ops.close()
    return worst


def case_embedding_and_sampler(rank, world):
    from tinyllmforge_b200.ops import ref
    ops, tp = _ops(rank, world)
    V, H = 4096, 1024
    ops.enable_fused_comm(H, 2048)
    g = torch.Generator(device="cuda").manual_seed(2)
    table = torch.randn(V, H, device="cuda", generator=g).bfloat16()
    norm_w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    shard = V // world

    class Emb:
        pass
    emb = Emb()
    emb.tp, emb.weight, emb.vocab_start = tp, table[rank * shard:(rank + 1) * shard].contiguous(), rank * shard
    for T in (5, 700, 64):
        ids = torch.randint(0, V, (T,), device="cuda", generator=g, dtype=torch.int32)
        y, res = ops.embed_norm(ids, emb, norm_w, 1e-6)
        assert torch.equal(res, table[ids.long()])
        assert torch.allclose(y.float(), ref.rms_norm(table[ids.long()], norm_w, 1e-6).float(), atol=2e-2, rtol=2e-2)
    # sampler: the merged choice equals sampling the unsharded logits
    rows = 9
    logits = (torch.randn(rows, V, device="cuda", generator=g) * 2).bfloat16()
    temps = torch.full((rows,), 0.7, device="cuda")
    hdr = torch.zeros(16, dtype=torch.int32)
    hdr[9], hdr[10] = 3, 77

    class B:
        pass
    b = B()
    b.temperatures, b.header = temps, hdr.cuda()
    full_ids, _ = ops.sample_shard(logits, temps, b.header, 0)
    for _ in range(3):
        got = ops.sample(logits[:, rank * shard:(rank + 1) * shard].contiguous(), b, rank * shard, tp)
        assert torch.equal(got, full_ids)
    ops.check_status()
    ops.close()
    return True


def case_engine(rank, world):
    """Tiny-depth Qwen3-0.6B-shaped model: fused exchange == NCCL path (greedy tokens) under CUDA graphs."""
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from tinyllmforge_b200 import LLM, SamplingParams, preset
    cfg = preset("qwen3-0.6b", num_hidden_layers=3, vocab_size=8192)
    rng = random.Random(0)
    prompts = [[rng.randrange(8192) for _ in range(rng.randint(20, 300))] for _ in range(12)]
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    outs = {}
    for name, comm, two_shot_bytes in (("fused", "fused", None), ("fused-two-shot", "fused", "-1"), ("nccl", "nccl", None)):
        if two_shot_bytes is None:
            os.environ.pop("FORGE_TP_TWO_SHOT_BYTES", None)
            os.environ.pop("FORGE_TP_TAGGED", None)
        else:
            os.environ["FORGE_TP_TWO_SHOT_BYTES"] = two_shot_bytes      # every exchange as reduce-scatter + all-gather pulls
            os.environ["FORGE_TP_TAGGED"] = "0"
        llm = LLM("tp-test", hf_config=cfg, load_format="dummy", skip_tokenizer_init=True, max_model_len=1024,
                  max_num_batched_tokens=4096, max_num_seqs=32, num_kvcache_blocks=64, tensor_parallel_size=world, comm=comm)
        res = llm.generate(prompts, sp, use_tqdm=False)
        outs[name] = [o["token_ids"] for o in res] if rank == 0 else None
        llm.worker.ops.check_status()
        llm.exit()
    os.environ.pop("FORGE_TP_TWO_SHOT_BYTES", None)
    os.environ.pop("FORGE_TP_TAGGED", None)
    if rank == 0:
        agree = {}
        for name in ("fused", "fused-two-shot"):
            agree[name] = sum(x == y for a, b in zip(outs[name], outs["nccl"]) for x, y in zip(a, b)) / (12 * 24)
        return agree
    return None


@pytest.mark.skipif(_ngpus() < 2, reason="needs 2 GPUs")
def test_row_parallel_gemm_and_fused_reduce_norm():
    worst = _run("case_row_linear", 2)
    assert max(worst) <= 3e-2


@pytest.mark.skipif(_ngpus() < 2, reason="needs 2 GPUs")
def test_embedding_owner_push_and_sampler_merge():
    _run("case_embedding_and_sampler", 2)


@pytest.mark.skipif(_ngpus() < 2, reason="needs 2 GPUs")
def test_engine_fused_exchange_matches_nccl_path():
    agree = _run("case_engine", 2)[0]
    assert min(agree.values()) > 0.9, agree


@pytest.mark.skipif(_ngpus() < 8, reason="needs 8 GPUs")
def test_row_parallel_gemm_and_fused_reduce_norm_tp8():
    worst = _run("case_row_linear", 8)
    assert max(worst) <= 3e-2

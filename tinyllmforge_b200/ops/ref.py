"""Plain-PyTorch statement of every op: the CPU execution path and the oracle for the CUDA kernels.

Each function states the math of one reference layer; accumulation is in fp32
and the result is cast back to the input dtype.

Parity:
  rms_norm / add_rms_norm   tinyvllm/layers/layernorm.py:21-45 (without the fp32 aliasing of the in-place version)
  rope_table / apply_rope   tinyvllm/layers/rotary_embedding.py:5-57 (NeoX half-split rotation, fp32)
  silu_mul                  tinyvllm/layers/activation.py:11-14
  store_kv                  tinyvllm/layers/attention.py:9-48 (plus: negative slots are skipped)
  attention                 tinyvllm/layers/attention.py:86-111 (varlen causal GQA over the paged cache,
                            bottom-right aligned mask when a prefix is cached)
  embedding                 tinyvllm/layers/embed_head.py:34-40 (masked vocab-shard lookup)
  sample                    tinyvllm/layers/sampler.py:13-21 (Gumbel-max == softmax sampling; greedy at T == 0)

KV cache layout used everywhere in this package: ``[num_blocks, kv_heads, block_size, head_dim]`` per
layer and per K/V, so one (block, head) pair is a contiguous ``block_size x head_dim`` tile that a
single bulk copy can fetch.
"""
from __future__ import annotations


import numpy as np
import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- norms
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps)
    return (y.to(x.dtype).float() * weight.float()).to(x.dtype) if x.dtype != torch.float32 else (y * weight.float())


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float):
    """Returns (normed, new_residual); new_residual = x + residual rounded to the model dtype."""
    if residual is None:
        return rms_norm(x, weight, eps), x
    s = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(s, weight, eps), s


# ----------------------------------------------------------------------------- rotary
def rope_table(max_positions: int, head_dim: int, theta: float, device="cpu") -> torch.Tensor:
    """fp32 table ``[max_positions, head_dim]`` = cat(cos, sin) of pos * theta^(-2i/d)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    t = torch.arange(max_positions, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(device)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, d]; rotates pairs (i, i + d/2)."""
    d = x.shape[-1]
    cs = table[positions.long()]
    cos, sin = cs[:, None, :d // 2], cs[:, None, d // 2:]
    xf = x.float()
    x1, x2 = xf[..., :d // 2], xf[..., d // 2:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)


# ----------------------------------------------------------------------------- activation
def silu_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    return (F.silu(g) * u).to(x.dtype)


# ----------------------------------------------------------------------------- linear
def linear(x: torch.Tensor, w) -> torch.Tensor:
    if not isinstance(w, torch.Tensor):     # Fp8BlockWeight: same arithmetic as the fp8 kernel
        from .quant import linear_fp8_ref
        return linear_fp8_ref(x, w)
    return F.linear(x, w)


def linear_silu_mul(x: torch.Tensor, w_gate_up) -> torch.Tensor:
    return silu_mul(linear(x, w_gate_up))


# ----------------------------------------------------------------------------- KV cache
def store_kv(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             slot_mapping: torch.Tensor) -> None:
    """k, v: [T, kv_heads, d]; caches: [blocks, kv_heads, block_size, d]; slot < 0 is skipped."""
    bs = k_cache.shape[2]
    slots = slot_mapping.long()
    keep = slots >= 0
    if not bool(keep.all()):
        slots, k, v = slots[keep], k[keep], v[keep]
    blk, off = slots // bs, slots % bs
    k_cache[blk, :, off] = k.to(k_cache.dtype)
    v_cache[blk, :, off] = v.to(v_cache.dtype)


def qk_norm_rope_store(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, eps: float,
                       table: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor,
                       k_cache: torch.Tensor, v_cache: torch.Tensor,
                       num_heads: int, num_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Split the fused QKV projection, RMS-normalise q and k per head, rotate, write k and v into the
    paged cache and return q as ``[T, heads, d]`` (tinyvllm/models/qwen3.py:78-94)."""
    T = qkv.shape[0]
    q, k, v = qkv.split([num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * head_dim], dim=-1)
    q = rms_norm(q.reshape(T, num_heads, head_dim), q_weight, eps)
    k = rms_norm(k.reshape(T, num_kv_heads, head_dim), k_weight, eps)
    q = apply_rope(q, positions, table)
    k = apply_rope(k, positions, table)
    store_kv(k, v.reshape(T, num_kv_heads, head_dim), k_cache, v_cache, slot_mapping)
    return q


def _gather_kv(cache: torch.Tensor, table_row: torch.Tensor, length: int) -> torch.Tensor:
    """Rows 0..length-1 of one sequence from the paged cache -> [kv_heads, length, d]."""
    bs = cache.shape[2]
    nblk = (length + bs - 1) // bs
    blocks = cache[table_row[:nblk].long()]              # [nblk, kvh, bs, d]
    kvh, d = blocks.shape[1], blocks.shape[3]
    return blocks.permute(1, 0, 2, 3).reshape(kvh, nblk * bs, d)[:, :length]


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_seqlens_q: torch.Tensor,
              context_lens: torch.Tensor, block_tables: torch.Tensor, scale: float, num_seqs: int) -> torch.Tensor:
    """Causal GQA attention of new query tokens over the paged cache.

    q: [T, heads, d] holds, for sequence s, rows cu_seqlens_q[s]:cu_seqlens_q[s+1]; these are the LAST
    ``q_len`` positions of a sequence of ``context_lens[s]`` tokens whose K/V are all in the cache already.
    Returns [T, heads * d].
    """
    T, H, d = q.shape
    out = torch.zeros(T, H, d, dtype=q.dtype, device=q.device)
    cu = cu_seqlens_q.tolist()
    lens = context_lens.tolist()
    for s in range(num_seqs):
        a, b = cu[s], cu[s + 1]
        ql, kl = b - a, lens[s]
        if ql == 0:
            continue
        k = _gather_kv(k_cache, block_tables[s], kl).float()      # [kvh, kl, d]
        v = _gather_kv(v_cache, block_tables[s], kl).float()
        g = H // k.shape[0]
        qs = q[a:b].float().permute(1, 0, 2).reshape(k.shape[0], g * ql, d)   # [kvh, g*ql, d]
        scores = torch.bmm(qs, k.transpose(1, 2)) * scale                      # [kvh, g*ql, kl]
        qpos = torch.arange(kl - ql, kl, device=q.device).repeat(g)            # row r -> query position
        mask = torch.arange(kl, device=q.device)[None, :] > qpos[:, None]
        scores.masked_fill_(mask[None], float("-inf"))
        p = torch.softmax(scores, dim=-1)
        o = torch.bmm(p, v).reshape(H, ql, d).permute(1, 0, 2)
        out[a:b] = o.to(q.dtype)
    return out.reshape(T, H * d)


# ----------------------------------------------------------------------------- embedding
def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Rows of this rank's vocab shard; ids outside the shard give zero rows."""
    n = weight.shape[0]
    local = ids.long() - vocab_start
    ok = (local >= 0) & (local < n)
    out = F.embedding(torch.where(ok, local, torch.zeros_like(local)), weight)
    return out * ok[:, None].to(out.dtype)


# ----------------------------------------------------------------------------- sampling
_PHILOX_M0, _PHILOX_M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_PHILOX_W0, _PHILOX_W1 = np.uint32(0x9E3779B9), np.uint32(0xBB67AE85)


def philox4x32(c0, c1, c2, c3, k0, k1):
    """Philox-4x32-10 on numpy uint32 arrays; returns four uint32 arrays."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint32) for c in (c0, c1, c2, c3))
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    k0, k1 = np.uint32(k0), np.uint32(k1)
    with np.errstate(over="ignore"):
        for _ in range(10):
            p0 = c0.astype(np.uint64) * _PHILOX_M0
            p1 = c2.astype(np.uint64) * _PHILOX_M1
            hi0, lo0 = (p0 >> np.uint64(32)).astype(np.uint32), p0.astype(np.uint32)
            hi1, lo1 = (p1 >> np.uint64(32)).astype(np.uint32), p1.astype(np.uint32)
            c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
            k0 = np.uint32((int(k0) + int(_PHILOX_W0)) & 0xFFFFFFFF)
            k1 = np.uint32((int(k1) + int(_PHILOX_W1)) & 0xFFFFFFFF)
    return c0, c1, c2, c3


def gumbel_noise(rows: int, vocab: int, seed: int, step: int, vocab_start: int = 0) -> np.ndarray:
    """-log(-log(u)) per (row, global vocab id), a pure function of (seed, step, row, id).

    One Philox call covers four consecutive vocab ids: counter = (id // 4, row, step, 0),
    key = seed; lane ``id % 4`` of the output is the uniform for that id.  Keying on the GLOBAL
    vocab id makes the sampled token independent of how the vocabulary is sharded.
    """
    ids = np.arange(vocab_start, vocab_start + vocab, dtype=np.int64)
    grp = (ids // 4).astype(np.uint32)
    r = np.arange(rows, dtype=np.uint32)[:, None]
    outs = philox4x32(grp[None, :], r, np.uint32(step & 0xFFFFFFFF), np.uint32(0),
                      seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    lane = (ids % 4)[None, :]
    bits = np.choose(np.broadcast_to(lane, outs[0].shape), outs)
    # u = (k + 0.5) / 2^24 with k the top 24 bits.  The winners of the arg-max have u close to 1, where fp32 cannot
    # resolve 1 - u; work from w = 1 - u = (2^24 - k - 0.5) / 2^24 in fp64: E = -log(u) = -log1p(-w), noise = -log(E).
    return _gumbel_from_bits(bits)


SAMPLE_GROUP = 16


def _gumbel_from_bits(bits: np.ndarray) -> np.ndarray:
    k = (bits >> np.uint32(8)).astype(np.float64)
    w = (16777216.0 - k - 0.5) / 16777216.0
    return (-np.log(-np.log1p(-w))).astype(np.float32)


def group_gumbel_noise(rows: int, g_first: int, ngroups: int, seed: int, step: int) -> np.ndarray:
    """Gumbel noise per (row, group of 16 global vocab ids): Philox counter (g // 4, row, step, 1), lane g % 4."""
    g = np.arange(g_first, g_first + ngroups, dtype=np.int64)
    r = np.arange(rows, dtype=np.uint32)[:, None]
    outs = philox4x32((g // 4).astype(np.uint32)[None, :], r, np.uint32(step & 0xFFFFFFFF), np.uint32(1),
                      seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    bits = np.choose(np.broadcast_to((g % 4)[None, :], outs[0].shape), outs)
    return _gumbel_from_bits(bits)


def sample(logits: torch.Tensor, temperatures: torch.Tensor, seed: int, step: int, vocab_start: int = 0):
    """Returns (token ids int64 [rows], winning scores fp32 [rows]) over this vocab shard.

    T == 0 -> argmax(logits), score = the maximum.  T > 0 -> a draw from softmax(logits / T), as the reference's
    ``probs / Exp(1)`` race is (tinyvllm/layers/sampler.py:13-21), in two levels so that only one random number per GROUP
    of 16 consecutive global token ids is needed: (1) the winning group is argmax_g (logsumexp_{i in g}(logit_i / T) +
    Gumbel(row, g)), which is distributed as the group holding the arg-max of per-token Gumbel-max sampling; (2) inside it
    the token is argmax_i (logit_i / T + Gumbel(row, i)).  The score returned is the winning group's, so that vocab shards
    (which start on multiples of 16) can be merged by taking the row-wise maximum.  Same procedure as csrc/include/sampling.cuh.
    """
    lf = logits.float()
    rows, vocab = lf.shape
    t = temperatures.float().to(lf.device)
    greedy = t <= 0
    inv_t = torch.where(greedy, torch.ones_like(t), 1.0 / torch.where(greedy, torch.ones_like(t), t))
    x = lf * inv_t[:, None]
    G = SAMPLE_GROUP
    g_first, g_last = vocab_start // G, (vocab_start + vocab - 1) // G
    ngroups = g_last - g_first + 1
    lead = vocab_start - g_first * G                      # ids of the first group that lie before the shard
    padded = torch.full((rows, ngroups * G), float("-inf"), device=lf.device)
    padded[:, lead:lead + vocab] = x
    grp = padded.view(rows, ngroups, G)
    gscore = torch.logsumexp(grp, dim=-1)
    gnoise = torch.from_numpy(group_gumbel_noise(rows, g_first, ngroups, seed, step)).to(lf.device)
    gscore = torch.where(greedy[:, None], grp.max(dim=-1).values, gscore + gnoise)
    best, gwin = gscore.max(dim=-1)                        # ties -> the first (lowest) group
    noise = torch.from_numpy(gumbel_noise(rows, ngroups * G, seed, step, g_first * G)).to(lf.device).view(rows, ngroups, G)
    inner = grp + torch.where(greedy[:, None, None], torch.zeros_like(noise), noise)
    pick = inner[torch.arange(rows, device=lf.device), gwin].argmax(dim=-1)
    return (g_first + gwin) * G + pick, best


# ----------------------------------------------------------------------------- op set
class RefOps:
    """The op set the model calls, stated with the functions above (CPU path and oracle)."""

    name = "ref"

    linear = staticmethod(linear)
    linear_silu_mul = staticmethod(linear_silu_mul)
    embedding = staticmethod(embedding)
    add_rms_norm = staticmethod(add_rms_norm)
    rms_norm = staticmethod(rms_norm)
    qk_norm_rope_store = staticmethod(qk_norm_rope_store)

    @staticmethod
    def attention(q, k_cache, v_cache, batch, scale):
        return attention(q, k_cache, v_cache, batch.cu_seqlens_q, batch.context_lens, batch.block_tables,
                         scale, batch.num_seqs)

    @staticmethod
    def select_rows(x, index):
        return x.index_select(0, index.long())

    @staticmethod
    def tp_all_reduce(y, tp):
        return tp.all_reduce(y)

    @staticmethod
    def embed_norm(ids, embed, norm_weight, eps):
        h = embed.tp.all_reduce(embedding(ids, embed.weight, embed.vocab_start))
        return add_rms_norm(h, None, norm_weight, eps)

    @staticmethod
    def row_linear_add_rms_norm(x, layer, residual, norm_weight, eps, site):
        h = layer.tp.all_reduce(linear(x, layer.weight))
        return add_rms_norm(h, residual, norm_weight, eps)

    @staticmethod
    def sample(logits, batch, vocab_start, tp):
        """Token ids [rows] (int64), identical on every rank."""
        ids, best = sample(logits, batch.temperatures, batch.seed, batch.step_index, vocab_start)
        if tp.size == 1:
            return ids
        all_best = tp.all_gather_stack(best)          # [tp, rows]
        all_ids = tp.all_gather_stack(ids)
        win = all_best.argmax(dim=0, keepdim=True)    # ties -> lowest rank == lowest vocab id
        return all_ids.gather(0, win)[0]

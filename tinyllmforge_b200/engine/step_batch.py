"""Flat integer description of one engine step.

The reference turns a list of ``Sequence`` objects into five or six separate
device tensors per step (tinyvllm/engine/model_runner.py:155-236), pickles the
objects to its worker ranks (model_runner.py:92-99) and passes attention
metadata through a module-level global (tinyvllm/utils/context.py:5-27).

Here rank 0 builds ONE packed ``int32`` array per step.  The same bytes are
(a) published to the other ranks through the shared-memory ring and
(b) copied to the GPU with a single host-to-device transfer; kernels and the
model read typed views at fixed offsets.  For a decode step padded to a CUDA
graph bucket the offsets depend only on (bucket, table width), so a captured
graph always finds its inputs at the same device addresses.

Layout (all int32 words, every section starts on a 16-byte boundary):

    header[16]   magic, is_prefill, num_seqs, num_tokens, padded_seqs, padded_tokens,
                 table_width, max_seqlen_q, max_seqlen_k, step_index, seed_lo, seed_hi, 0...
    input_ids[padded_tokens] positions[padded_tokens] slot_mapping[padded_tokens]
    cu_seqlens_q[padded_seqs + 1] context_lens[padded_seqs] last_index[padded_seqs]
    temperatures[padded_seqs] (float32 bit patterns)
    block_tables[padded_seqs * table_width]
    src_rows[padded_seqs]    decode only: >= 0 -> this sequence's input token is row src_rows[i] of the PREVIOUS step's
                             sampled tokens, still on the device (pipelined engine loop); -1 -> input_ids[i] is valid

Padding rows use slot -1 (the KV store skips them), context length 0 and block id -1.
Decode positions are ``len - 1``: the index of the token whose KV entry is being
written (the reference passes ``len``, one too far: model_runner.py:219).
"""
from __future__ import annotations

import numpy as np

MAGIC = 0x464F5247  # "FORG"
HEADER_WORDS = 16
H_MAGIC, H_PREFILL, H_NSEQ, H_NTOK, H_PSEQ, H_PTOK, H_WIDTH, H_MAXQ, H_MAXK, H_STEP, H_SEEDLO, H_SEEDHI = range(12)

SECTIONS = ("input_ids", "positions", "slot_mapping", "cu_seqlens_q", "context_lens", "last_index",
            "temperatures", "block_tables", "src_rows")


def _align4(n: int) -> int:
    return (n + 3) & ~3


def section_offsets(padded_tokens: int, padded_seqs: int, table_width: int) -> tuple[dict, int]:
    """Word offsets and lengths of every section, and the total word count."""
    sizes = {
        "input_ids": padded_tokens, "positions": padded_tokens, "slot_mapping": padded_tokens,
        "cu_seqlens_q": padded_seqs + 1, "context_lens": padded_seqs, "last_index": padded_seqs,
        "temperatures": padded_seqs, "block_tables": padded_seqs * table_width, "src_rows": padded_seqs,
    }
    off = HEADER_WORDS
    out = {}
    for name in SECTIONS:
        out[name] = (off, sizes[name])
        off = _align4(off + sizes[name])
    return out, off


class StepBatch:
    """A typed view over the packed step buffer."""

    def __init__(self, buf: np.ndarray):
        assert buf.dtype == np.int32 and buf.ndim == 1
        if int(buf[H_MAGIC]) != MAGIC:
            raise ValueError("not a step buffer (bad magic)")
        self.buf = buf
        self.is_prefill = bool(buf[H_PREFILL])
        self.num_seqs = int(buf[H_NSEQ])
        self.num_tokens = int(buf[H_NTOK])
        self.padded_seqs = int(buf[H_PSEQ])
        self.padded_tokens = int(buf[H_PTOK])
        self.table_width = int(buf[H_WIDTH])
        self.max_seqlen_q = int(buf[H_MAXQ])
        self.max_seqlen_k = int(buf[H_MAXK])
        self.step_index = int(buf[H_STEP])
        self.seed = (int(buf[H_SEEDLO]) & 0xFFFFFFFF) | ((int(buf[H_SEEDHI]) & 0xFFFFFFFF) << 32)
        self.offsets, self.num_words = section_offsets(self.padded_tokens, self.padded_seqs, self.table_width)
        assert self.num_words <= buf.shape[0]

    def section(self, name: str) -> np.ndarray:
        off, n = self.offsets[name]
        v = self.buf[off:off + n]
        if name == "temperatures":
            return v.view(np.float32)
        if name == "block_tables":
            return v.reshape(self.padded_seqs, self.table_width)
        return v

    def __getattr__(self, name):
        if name in SECTIONS:
            return self.section(name)
        raise AttributeError(name)

    @property
    def nbytes(self) -> int:
        return self.num_words * 4


def _new(is_prefill, num_seqs, num_tokens, padded_seqs, padded_tokens, width, max_q, max_k, step_index, seed):
    offs, total = section_offsets(padded_tokens, padded_seqs, width)
    buf = np.zeros(total, dtype=np.int32)
    hdr = buf[:HEADER_WORDS]
    hdr[H_MAGIC] = MAGIC
    hdr[H_PREFILL] = int(is_prefill)
    hdr[H_NSEQ] = num_seqs
    hdr[H_NTOK] = num_tokens
    hdr[H_PSEQ] = padded_seqs
    hdr[H_PTOK] = padded_tokens
    hdr[H_WIDTH] = width
    hdr[H_MAXQ] = max_q
    hdr[H_MAXK] = max_k
    hdr[H_STEP] = step_index & 0x7FFFFFFF
    hdr[H_SEEDLO:H_SEEDHI + 1] = np.array([seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF], dtype=np.uint32).view(np.int32)
    return buf, offs


def build_prefill(reqs, block_size: int, step_index: int = 0, seed: int = 0) -> StepBatch:
    """Prefill step: every request contributes its not-yet-cached tokens (or, for a prompt prefilled in chunks, the
    tokens [num_computed_tokens, prefill_end); the keys it sees then end at prefill_end)."""
    S = len(reqs)
    starts = [r.num_computed_tokens if r.num_computed_tokens >= 0 else r.num_cached_tokens for r in reqs]
    ends = [r.prefill_end if r.prefill_end >= 0 else len(r) for r in reqs]
    q_lens = np.fromiter((e - c for c, e in zip(starts, ends)), dtype=np.int64, count=S)
    k_lens = np.fromiter(ends, dtype=np.int64, count=S)
    T = int(q_lens.sum())
    width = max(len(r.block_table) for r in reqs)
    buf, offs = _new(True, S, T, S, T, width, int(q_lens.max()), int(k_lens.max()), step_index, seed)

    def sec(name):
        o, n = offs[name]
        return buf[o:o + n]

    ids, pos, slots = sec("input_ids"), sec("positions"), sec("slot_mapping")
    tables = sec("block_tables").reshape(S, width)
    tables[:] = -1
    t = 0
    for i, r in enumerate(reqs):
        c, n = starts[i], ends[i]
        q = n - c
        ids[t:t + q] = r.token_ids[c:n]
        p = np.arange(c, n, dtype=np.int64)
        pos[t:t + q] = p
        bt = np.asarray(r.block_table, dtype=np.int64)
        tables[i, :len(bt)] = bt
        slots[t:t + q] = bt[p // block_size] * block_size + p % block_size
        t += q
    cu = sec("cu_seqlens_q")
    cu[0] = 0
    np.cumsum(q_lens, out=cu[1:])
    sec("context_lens")[:] = k_lens
    sec("last_index")[:] = cu[1:] - 1
    sec("temperatures").view(np.float32)[:] = [r.temperature for r in reqs]
    sec("src_rows")[:] = -1
    return StepBatch(buf)


def build_decode(reqs, block_size: int, step_index: int = 0, seed: int = 0,
                 pad_to: int | None = None, table_width: int | None = None) -> StepBatch:
    """Decode step: one token per request, optionally padded to a graph bucket."""
    S = len(reqs)
    P = max(pad_to or S, S)
    width = table_width or max(len(r.block_table) for r in reqs)
    lens = np.fromiter((len(r) for r in reqs), dtype=np.int64, count=S)
    buf, offs = _new(False, S, S, P, P, width, 1, int(lens.max()), step_index, seed)

    def sec(name):
        o, n = offs[name]
        return buf[o:o + n]

    sec("input_ids")[:S] = [r.token_ids[-1] for r in reqs]
    sec("positions")[:S] = lens - 1
    last_block = np.fromiter((r.block_table[-1] for r in reqs), dtype=np.int64, count=S)
    slots = sec("slot_mapping")
    slots[:] = -1
    slots[:S] = last_block * block_size + (lens - 1) % block_size
    sec("cu_seqlens_q")[:] = np.minimum(np.arange(P + 1), S)
    sec("context_lens")[:S] = lens
    sec("last_index")[:] = np.minimum(np.arange(P), S - 1)
    sec("temperatures").view(np.float32)[:S] = [r.temperature for r in reqs]
    tables = sec("block_tables").reshape(P, width)
    tables[:] = -1
    for i, r in enumerate(reqs):
        bt = r.block_table
        tables[i, :len(bt)] = bt
    sec("src_rows")[:] = -1
    return StepBatch(buf)


class DecodeBuilder:
    """Builds consecutive decode steps incrementally.

    While the set of running requests does not change (most steps), a decode step differs from the previous one
    only by: every length + 1, the new input token of every request, and an occasional new block id.  The packed
    buffer of the previous step is updated in place with a few vector operations instead of being rebuilt from
    the request objects (the reference rebuilds five Python lists over all sequences every step,
    tinyvllm/engine/model_runner.py:210-228).  Produces exactly what ``build_decode`` produces.
    """

    def __init__(self, block_size: int):
        self.block_size = block_size
        self.reqs: list | None = None
        self.sb: StepBatch | None = None
        self.key = None
        self.lens = None

    def reset(self) -> None:
        self.reqs = None

    def build(self, reqs, step_index: int, seed: int, pad_to: int | None, table_width: int | None) -> StepBatch:
        bs = self.block_size
        S = len(reqs)
        if self.reqs is not None and self.key == (pad_to, table_width) and reqs == self.reqs:
            lens = self.lens
            lens += 1
            if table_width is None and int(lens.max()) > self.sb.table_width * bs:
                self.reqs = None                                    # table would widen: rebuild
            else:
                sb = self.sb
                buf = sb.buf
                buf[H_STEP] = step_index & 0x7FFFFFFF
                buf[H_MAXK] = int(lens.max())
                o, _ = sb.offsets["input_ids"]
                buf[o:o + S] = [r.token_ids[-1] for r in reqs]
                o, _ = sb.offsets["positions"]
                buf[o:o + S] = lens - 1
                o, _ = sb.offsets["context_lens"]
                buf[o:o + S] = lens
                grew = np.nonzero(lens % bs == 1)[0]
                if grew.size:
                    to, _ = sb.offsets["block_tables"]
                    w = sb.table_width
                    for i in grew.tolist():
                        bt = reqs[i].block_table
                        buf[to + i * w + len(bt) - 1] = bt[-1]
                        self.last_block[i] = bt[-1]
                o, _ = sb.offsets["slot_mapping"]
                buf[o:o + S] = self.last_block * bs + (lens - 1) % bs
                sb.step_index = step_index
                sb.max_seqlen_k = int(buf[H_MAXK])
                return sb
        sb = build_decode(reqs, bs, step_index, seed, pad_to=pad_to, table_width=table_width)
        self.reqs = list(reqs)
        self.key = (pad_to, table_width)
        self.sb = sb
        self.lens = np.fromiter((len(r) for r in reqs), dtype=np.int64, count=S)
        self.last_block = np.fromiter((r.block_table[-1] for r in reqs), dtype=np.int64, count=S)
        return sb

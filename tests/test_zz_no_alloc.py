"""The allocation-free decode-attention entry point, called the way its users call it: through the exported C
symbol of the shared library, with raw device pointers.

Its users are callers that cannot ask for device memory where they need the kernel (a callback inside another
component's memory plan, a loop that must not touch the allocator); the split-context scratch therefore lives
in an array inside the library.  The check: on two calls in a row (different batch, different context lengths,
so the second call finds the first call's leftovers in the shared array) the output equals that of the regular
entry point, which takes caller-allocated scratch.  Also: an oversized request is refused with the documented
code and nothing is launched.

This file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _lib():
    from tinyllmforge_b200 import _C
    lib = ctypes.CDLL(_C.__file__)
    fn = lib.forge_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 9 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    lib.forge_decode_attention_noalloc_strerror.restype = ctypes.c_char_p
    lib.forge_decode_attention_noalloc_strerror.argtypes = [ctypes.c_int]
    lib.forge_decode_attention_noalloc_capacity_floats.restype = ctypes.c_size_t
    return lib


def _case(lens, nq, nkv, bs, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    B = len(lens)
    per = [-(-max(n, 1) // bs) for n in lens]
    total = sum(per) + 2
    width = max(per) + 1
    bt = torch.full((B, width), -1, dtype=torch.int32)
    perm = torch.randperm(total).tolist()
    p = 0
    for b, n in enumerate(per):
        bt[b, :n] = torch.tensor(perm[p:p + n], dtype=torch.int32)
        p += n
    kc = torch.randn(total, nkv, bs, 128, device="cuda", generator=g).to(BF)
    vc = torch.randn(total, nkv, bs, 128, device="cuda", generator=g).to(BF)
    q = torch.randn(B, nq, 128, device="cuda", generator=g).to(BF)
    return q, kc, vc, bt.cuda(), torch.tensor(lens, dtype=torch.int32, device="cuda")


def _regular(q, kc, vc, bt, lens, chunk, max_chunks):
    from tinyllmforge_b200 import _C
    B, nq, D = q.shape
    out = torch.empty(B, nq * D, dtype=BF, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    po = torch.empty(B * nq * max_chunks * D, dtype=torch.float32, device="cuda")
    pml = torch.empty(B * nq * max_chunks * 2, dtype=torch.float32, device="cuda")
    _C.decode_attention(q, kc, vc, bt, lens, out, po, pml, chunk, max_chunks, D ** -0.5, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    return out


def _noalloc(lib, q, kc, vc, bt, lens, chunk, max_chunks):
    B, nq, D = q.shape
    out = torch.empty(B, nq * D, dtype=BF, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.forge_decode_attention_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), lens.data_ptr(), out.data_ptr(),
                                            B, nq, kc.shape[1], D, kc.shape[2], bt.shape[1], kc.shape[0], chunk, max_chunks,
                                            D ** -0.5, status.data_ptr(), stream)
    assert rc == 0, lib.forge_decode_attention_noalloc_strerror(rc).decode()
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    return out


def test_two_calls_in_a_row_match_the_regular_entry_point():
    lib = _lib()
    torch.cuda.synchronize()
    # call 1: long contexts, many chunks; call 2: fewer, shorter sequences over the same (now dirty) scratch
    for lens, nq, nkv, bs, chunk, seed in [([700, 2011, 129, 64, 1500], 16, 8, 256, 256, 1), ([33, 900, 260], 8, 2, 16, 64, 2)]:
        q, kc, vc, bt, cl = _case(lens, nq, nkv, bs, seed)
        max_chunks = -(-max(lens) // chunk)
        want = _regular(q, kc, vc, bt, cl, chunk, max_chunks)
        got = _noalloc(lib, q, kc, vc, bt, cl, chunk, max_chunks)
        err = (got.float() - want.float()).abs()
        assert bool((err <= 2e-2 + 2e-2 * want.float().abs()).all()), f"max err {err.max().item()}"
        assert torch.equal(got, want)            # same kernels, same order of operations


def test_a_length_beyond_the_slices_is_clamped_and_reported():
    """context_lens one slice longer than max_chunks * chunk covers: the call succeeds, `status` gets the bad-index bit,
    and the merge reads only partials of this call (the other rows equal the regular entry point's)."""
    lib = _lib()
    lens, nq, nkv, bs, chunk = [500, 260, 90], 16, 8, 256, 256
    q, kc, vc, bt, cl = _case(lens, nq, nkv, bs, 3)
    max_chunks = 2
    want = _regular(q, kc, vc, bt, cl, chunk, max_chunks)
    bad = cl.clone()
    bad[1] = max_chunks * chunk + chunk
    B, _, D = q.shape
    out = torch.empty(B, nq * D, dtype=BF, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = lib.forge_decode_attention_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bad.data_ptr(), out.data_ptr(),
                                            B, nq, nkv, D, bs, bt.shape[1], kc.shape[0], chunk, max_chunks, D ** -0.5,
                                            status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status[0]) & 4
    assert torch.equal(out[[0, 2]], want[[0, 2]])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_second_device_in_the_same_process():
    """The scratch address and the kernels' shared-memory limit are per device: a process that drives two GPUs gets the
    right ones on each (plain kernels only, no peer memory)."""
    lib = _lib()
    lens, nq, nkv, bs, chunk = [700, 300, 1200], 16, 8, 256, 256
    case0 = _case(lens, nq, nkv, bs, 5)               # built once (the block table comes from the host generator)
    prev = torch.cuda.current_device()
    try:
        torch.cuda.set_device(1)
        with torch.cuda.device(1):
            q, kc, vc, bt, cl = [t.to("cuda:1") for t in case0]
            max_chunks = -(-max(lens) // chunk)
            B, _, D = q.shape
            out = torch.empty(B, nq * D, dtype=BF, device="cuda:1")
            status = torch.zeros(4, dtype=torch.int32, device="cuda:1")
            rc = lib.forge_decode_attention_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), cl.data_ptr(), out.data_ptr(),
                                                    B, nq, nkv, D, bs, bt.shape[1], kc.shape[0], chunk, max_chunks, D ** -0.5,
                                                    status.data_ptr(), torch.cuda.current_stream().cuda_stream)
            assert rc == 0, lib.forge_decode_attention_noalloc_strerror(rc).decode()
            torch.cuda.synchronize()
            assert int(status[0]) == 0
    finally:
        torch.cuda.set_device(prev)
    want = _regular(*case0, chunk, max_chunks)
    assert torch.equal(out.cpu(), want.cpu())


def test_oversized_request_is_refused():
    lib = _lib()
    cap = lib.forge_decode_attention_noalloc_capacity_floats()
    assert cap == 4 << 20
    B, nq, max_chunks = 512, 64, 8                     # 512 * 64 * 8 * 130 floats > capacity
    assert B * nq * max_chunks * 130 > cap
    rc = lib.forge_decode_attention_noalloc(None, None, None, None, None, None, B, nq, 8, 128, 256, 16, 1, 512, max_chunks, 0.088,
                                            None, None)
    assert rc == -20
    assert b"16 MiB" in lib.forge_decode_attention_noalloc_strerror(rc)

"""Every sm_100a kernel against the plain-PyTorch fp32 statement of the same op (ops/ref.py)."""

import pytest
import torch

from tinyllmforge_b200.ops import ref

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    from tinyllmforge_b200.ops.cuda import CudaOps
    o = CudaOps()
    yield o
    o.check_status()


def _rand(*shape, scale=1.0, dtype=BF):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _close(a, b, atol, rtol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{bad}/{a.numel()} elements off; max err {err.max().item():.4g} (max ref {b.abs().max().item():.4g})"


# ----------------------------------------------------------------------------- GEMM (tcgen05)
@pytest.mark.parametrize("M,N,K,mode", [
    (1, 128, 64, 0), (16, 256, 128, 0), (7, 1024, 1024, 0), (64, 4096, 1024, 0), (200, 1024, 2048, 0),
    (256, 6144, 1024, 0), (128, 128, 64, 1), (300, 384, 256, 1), (1000, 1024, 1024, 0), (4096, 4096, 1024, 0),
    (130, 200, 72, 1), (33, 136, 200, 2), (256, 1024, 3072, 2),
    # one rank's shapes of the 32B architecture split 8 ways: qkv, o_proj, down_proj at decode and prefill sizes
    (64, 1280, 5120, 0), (64, 5120, 1024, 0), (64, 5120, 3200, 0), (2048, 1280, 5120, 0), (2048, 5120, 3200, 0),
])
def test_gemm_matches_fp32(ops, M, N, K, mode):
    torch.manual_seed(M * 7 + N)
    x, w = _rand(M, K), _rand(N, K, scale=0.05)
    out = ops.linear(x, w, force_mode=mode)
    want = x.float() @ w.float().t()
    _close(out, want, atol=2e-2, rtol=2e-2)
    ops.check_status()


@pytest.mark.parametrize("M,I,K,mode", [(8, 256, 128, 0), (100, 3072, 1024, 0), (256, 1536, 1024, 2), (700, 3072, 1024, 0), (384, 512, 256, 1),
                                        (64, 3200, 5120, 0), (2048, 3200, 5120, 0)])
def test_gemm_silu_mul_epilogue(ops, M, I, K, mode):
    torch.manual_seed(M + I)
    x, w = _rand(M, K), _rand(2 * I, K, scale=0.05)
    out = ops.linear_silu_mul(x, w, force_mode=mode)
    gu = x.float() @ w.float().t()
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    _close(out, want, atol=2e-2, rtol=2e-2)
    ops.check_status()


@pytest.mark.parametrize("M,N,K,splits", [
    (256, 1024, 2048, 8), (256, 1024, 3072, 8), (200, 4096, 1024, 4), (16, 1024, 2048, 4), (1, 1024, 1024, 2),
    (64, 1024, 2048, 8), (128, 512, 1024, 1), (40, 384, 448, 4), (256, 151936 // 8, 1024, 1),
])
def test_gemm_decode_kernel_split_k(ops, M, N, K, splits):
    """Weight-tile kernel with K split over a thread-block cluster and the DSMEM reduction."""
    torch.manual_seed(M + N + splits)
    x, w = _rand(M, K), _rand(N, K, scale=0.05)
    out = ops.linear(x, w, force_mode=2, force_splits=splits)
    _close(out, x.float() @ w.float().t(), atol=2e-2, rtol=2e-2)
    again = ops.linear(x, w, force_mode=2, force_splits=splits)
    assert torch.equal(out, again)                       # fixed reduction order: bit-reproducible
    ops.check_status()


@pytest.mark.parametrize("M,I,K,splits", [(256, 3072, 1024, 4), (256, 3072, 1024, 1), (24, 1536, 1024, 2), (100, 512, 2048, 8), (8, 256, 256, 2)])
def test_gemm_decode_kernel_silu_split_k(ops, M, I, K, splits):
    torch.manual_seed(M + I + splits)
    x, w = _rand(M, K), _rand(2 * I, K, scale=0.05)
    out = ops.linear_silu_mul(x, w, force_mode=2, force_splits=splits)
    gu = x.float() @ w.float().t()
    _close(out, torch.nn.functional.silu(gu[:, :I]) * gu[:, I:], atol=2e-2, rtol=2e-2)
    ops.check_status()


@pytest.mark.parametrize("M,N,K,bc,silu", [
    (256, 4096, 1024, 64, False), (200, 1024, 2048, 16, False), (130, 1000, 512, 32, False), (96, 3072, 1024, 32, True),
    (256, 3072, 1024, 64, True), (140, 1536, 256, 16, True), (700, 2048, 1024, 32, False),
])
def test_gemm_token_kernel_narrow_feature_tiles(ops, M, N, K, bc, silu):
    """Token-tile kernel with 16/32/64-feature tiles (large decode batches: direct epilogue, no K split)."""
    torch.manual_seed(M + N + bc)
    x, w = _rand(M, K), _rand((2 if silu else 1) * N, K, scale=0.05)
    f = ops.linear_silu_mul if silu else ops.linear
    out = f(x, w, force_mode=1, force_block_c=bc)
    ref = x.float() @ w.float().t()
    if silu:
        ref = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:]
    _close(out, ref, atol=2e-2, rtol=2e-2)
    ops.check_status()


@pytest.mark.parametrize("M,N,K,bc,splits,silu", [
    (256, 4096, 1024, 64, 1, False), (256, 1024, 2048, 64, 4, False), (200, 1024, 3072, 32, 2, False), (130, 2048, 4096, 128, 1, False),
    (256, 3072, 1024, 64, 1, True), (96, 1536, 2048, 32, 2, True), (256, 512, 1024, 128, 1, True), (8, 256, 128, 16, 1, False),
])
def test_gemm_decode_kernel_deep_ring(ops, M, N, K, bc, splits, silu):
    """The one-CTA-per-SM variant of the weight-tile kernel (ring of ~200 KB) gives the same bits as the two-per-SM one."""
    torch.manual_seed(M + N + bc)
    x, w = _rand(M, K), _rand((2 if silu else 1) * N, K, scale=0.05)
    f = ops.linear_silu_mul if silu else ops.linear
    deep = f(x, w, force_mode=2, force_splits=splits, force_block_c=bc, force_deep=2)
    shallow = f(x, w, force_mode=2, force_splits=splits, force_block_c=bc, force_deep=1)
    ref = x.float() @ w.float().t()
    if silu:
        ref = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:]
    _close(deep, ref, atol=2e-2, rtol=2e-2)
    assert torch.equal(deep, shallow)
    ops.check_status()


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (16, 1280, 1024), (50, 1024, 3200 - 3200 % 128), (64, 6400, 5120), (200, 1024, 2048), (600, 384, 256)])
def test_gemm_fp8_block_scaled(ops, M, N, K):
    """e4m3 weights with 128 x 128 block scales, activations quantised per token and 128 features."""
    from tinyllmforge_b200.ops.quant import Fp8BlockWeight, linear_fp8_ref, quantize_activations_ref
    torch.manual_seed(M + N)
    x, w = _rand(M, K), _rand(N, K, scale=0.05)
    wq = Fp8BlockWeight.quantize(w)
    # the CUDA quantiser agrees with the PyTorch statement
    xq = torch.empty(M, K, dtype=torch.uint8, device="cuda")
    xs = torch.empty(K // 128, (M + 3) // 4 * 4, dtype=torch.float32, device="cuda")
    ops.C.quant_fp8(x, xq, xs)
    q_ref, s_ref = quantize_activations_ref(x)
    assert torch.allclose(xs[:, :M], s_ref, rtol=1e-6)
    assert (xq.view(torch.float8_e4m3fn).float() - q_ref.float()).abs().max() <= 32          # at most one e4m3 step at the top of the range
    out = ops.linear_fp8(x, wq)            # the e4m3 kernel itself (ops.linear expands the weight to bf16 for many tokens)
    # the GEMM itself, checked on exactly the operands it saw: the CUDA-quantised activations, dequantised in fp32
    xd = xq.view(torch.float8_e4m3fn).float().view(M, K // 128, 128) * xs[:, :M].t()[..., None]
    _close(out, xd.view(M, K) @ wq.dequantize().t(), atol=2e-2, rtol=2e-2)
    _close(out, linear_fp8_ref(x, wq), atol=0.15, rtol=5e-2)          # PyTorch quantiser may round ties differently
    exact = x.float() @ w.float().t()
    rel = (out.float() - exact).norm() / exact.norm()
    assert rel < 0.06, rel                                              # quantisation error itself stays small
    ops.check_status()


# ----------------------------------------------------------------------------- GEMMs with norm / residual fused in
@pytest.mark.parametrize("M,N,K,mode,silu", [
    (1, 4096, 1024, 0, False), (8, 4096, 1024, 2, False), (64, 4096, 1024, 0, False), (200, 4096, 1024, 0, False), (256, 6144, 4096, 0, False),
    (700, 4096, 1024, 0, False), (4096, 2048, 1024, 0, False), (5, 3072, 1024, 0, True), (16, 3072, 1024, 2, True), (100, 3072, 1024, 0, True),
    (256, 1536, 1024, 2, True), (700, 3072, 1024, 0, True), (130, 12288, 4096, 0, True), (33, 1024, 2048, 2, False),
])
def test_gemm_with_folded_input_norm(ops, M, N, K, mode, silu):
    """(x @ W'.T) * rsqrt(mean(x^2) + eps) per row, W' = W * gamma, against rms_norm(x) * gamma @ W.T in fp32; x is a residual
    stream with rows of very different magnitudes."""
    torch.manual_seed(M + N + K)
    x = (_rand(M, K).float() * torch.logspace(-1, 1.5, M, device="cuda")[:, None]).to(BF)
    gamma = (1 + 0.2 * torch.randn(K, device="cuda")).to(BF)
    w = _rand(2 * N if silu else N, K, scale=0.05)
    w_folded = (w.float() * gamma.float()[None, :]).to(BF)
    parts = (K + 127) // 128          # the sums of squares arrive in pieces of 128 features, as the producing GEMM writes them
    ssq = (x.float() ** 2).view(M, parts, -1).sum(-1).contiguous()
    got = ops.linear_scaled(x, w_folded, ssq, 1e-6, silu_mul=silu, force_mode=mode)
    xn = x.float() * torch.rsqrt((x.float() ** 2).mean(-1, keepdim=True) + 1e-6)
    want = xn @ w_folded.float().t()
    if silu:
        want = torch.nn.functional.silu(want[:, :N]) * want[:, N:]
    _close(got, want, atol=3e-2, rtol=3e-2)
    ops.check_status()


@pytest.mark.parametrize("M,N,K,mode,tune", [
    (1, 1024, 2048, 0, 0), (7, 1024, 3072, 0, 0), (64, 1024, 2048, 0, 0), (200, 1024, 3072, 0, 0), (256, 1024, 2048, 2, 8), (256, 4096, 12288, 0, 0),
    (33, 1024, 1024, 2, 1), (300, 1024, 2048, 0, 0), (4096, 1024, 3072, 0, 0), (1000, 4096, 4096, 0, 0), (130, 200, 72, 1, 0), (19, 136, 200, 2, 0),
    (700, 1100, 256, 1, 0), (40, 5120, 3200, 0, 0),
])
def test_gemm_with_residual_add_and_sum_of_squares(ops, M, N, K, mode, tune):
    """residual += x @ W.T in the epilogue (rounded like a bf16 GEMM followed by a bf16 add) plus the per-row sums of squares."""
    torch.manual_seed(M * 3 + N + K)
    x, w = _rand(M, K), _rand(N, K, scale=0.05)
    residual = _rand(M, N, scale=2.0)
    want = ((x.float() @ w.float().t()).to(BF).float() + residual.float()).to(BF)
    parts = (N + 127) // 128
    ssq = torch.full((M, parts), float("nan"), dtype=torch.float32, device="cuda")     # every entry must be written
    res = residual.clone()
    ops.linear_residual(x, w, res, ssq, force_mode=mode, tune=tune)
    _close(res, want, atol=6e-2, rtol=2e-2)
    sq = torch.nn.functional.pad(res.float() ** 2, (0, parts * 128 - N)).view(M, parts, 128).sum(-1)
    assert torch.allclose(ssq, sq, rtol=1e-3, atol=1e-3)                               # of the values actually stored
    ssq2 = torch.empty_like(ssq)
    res2 = residual.clone()
    ops.linear_residual(x, w, res2, ssq2, force_mode=mode, tune=tune)
    assert torch.equal(res2, res) and torch.equal(ssq2, ssq)                           # no dependence on scheduling
    ops.check_status()


@pytest.mark.parametrize("M,N,K,bc,kg,silu", [
    (256, 6144, 4096, 0, 4, False), (64, 4096, 4096, 0, 4, False), (200, 4096, 12288, 0, 4, False), (16, 1280, 5120, 128, 2, False),
    (100, 5120, 3200, 0, 3, False), (256, 12288, 4096, 0, 4, True), (50, 3200, 5120, 0, 8, True), (130, 1000, 520, 64, 1, False),
    (300, 1536, 1024, 64, 2, True), (1, 256, 64, 0, 1, False), (7, 136, 4104, 128, 5, False),
])
def test_gemm_stream_k_matches_fp32(ops, M, N, K, bc, kg, silu):
    """Token-tile kernel with the (tile, K group) units dealt out evenly over the CTAs: partial tiles go through the
    scratch buffer and are summed by the CTA that arrives last."""
    torch.manual_seed(M + N + K)
    x, w = _rand(M, K), _rand(2 * N if silu else N, K, scale=0.05)
    fn = ops.linear_silu_mul if silu else ops.linear
    out = fn(x, w, force_mode=3, force_splits=kg, force_block_c=bc)
    ref_ = x.float() @ w.float().t()
    want = torch.nn.functional.silu(ref_[:, :N]) * ref_[:, N:] if silu else ref_
    _close(out, want, atol=2e-2, rtol=2e-2)
    out2 = fn(x, w, force_mode=3, force_splits=kg, force_block_c=bc)
    assert torch.equal(out, out2)                      # partial sums are added in the order of their K ranges
    ops.check_status()


@pytest.mark.parametrize("M,N,K,kg", [(256, 4096, 4096, 4), (64, 4096, 12288, 4), (130, 1024, 3072, 2), (40, 5120, 3200, 4)])
def test_gemm_stream_k_with_the_fused_epilogues(ops, M, N, K, kg):
    torch.manual_seed(M + K)
    x, w = _rand(M, K), _rand(N, K, scale=0.05)
    residual = _rand(M, N, scale=2.0)
    want = ((x.float() @ w.float().t()).to(BF).float() + residual.float()).to(BF)
    parts = (N + 127) // 128
    ssq = torch.full((M, parts), float("nan"), dtype=torch.float32, device="cuda")
    res = residual.clone()
    ops.linear_residual(x, w, res, ssq, force_mode=3, tune=kg)
    _close(res, want, atol=6e-2, rtol=2e-2)
    sq = torch.nn.functional.pad(res.float() ** 2, (0, parts * 128 - N)).view(M, parts, 128).sum(-1)
    assert torch.allclose(ssq, sq, rtol=1e-3, atol=1e-3)
    res2, ssq2 = residual.clone(), torch.empty_like(ssq)
    ops.linear_residual(x, w, res2, ssq2, force_mode=3, tune=kg)
    assert torch.equal(res2, res) and torch.equal(ssq2, ssq)
    # folded input norm as a row scale
    pk = (K + 127) // 128
    ssq_in = (x.float() ** 2).view(M, pk, -1).sum(-1).contiguous()
    got = ops.linear_scaled(x, w, ssq_in, 1e-6, force_mode=3, tune=kg)
    xn = x.float() * torch.rsqrt((x.float() ** 2).mean(-1, keepdim=True) + 1e-6)
    _close(got, xn @ w.float().t(), atol=3e-2, rtol=3e-2)
    ops.check_status()


@pytest.mark.parametrize("M,N,K,kg,silu", [
    (256, 256, 64, 0, False), (512, 512, 256, 0, False), (256, 6144, 4096, 0, False), (256, 6144, 4096, 4, False), (8192, 4096, 1024, 0, False),
    (200, 4096, 4096, 4, False), (100, 1280, 5120, 2, False), (1000, 1100, 520, 0, False), (700, 1100, 520, 3, False), (4096, 3072, 1024, 0, True),
    (256, 12288, 4096, 4, True), (130, 1536, 1024, 2, True), (300, 200, 72, 0, True), (1, 128, 64, 0, False),
])
def test_gemm_cta_pair_kernel_matches_fp32(ops, M, N, K, kg, silu):
    """One 256 x 256 UMMA per pair of SMs (cta_group::2): each CTA loads its 128 tokens and half of the weight rows."""
    torch.manual_seed(M + N + K)
    x, w = _rand(M, K), _rand(2 * N if silu else N, K, scale=0.05)
    fn = ops.linear_silu_mul if silu else ops.linear
    out = fn(x, w, force_mode=4, force_splits=kg)
    ref_ = x.float() @ w.float().t()
    want = torch.nn.functional.silu(ref_[:, :N]) * ref_[:, N:] if silu else ref_
    _close(out, want, atol=2e-2, rtol=2e-2)
    assert torch.equal(out, fn(x, w, force_mode=4, force_splits=kg))
    ops.check_status()


@pytest.mark.parametrize("M,N,K,kg", [(256, 4096, 4096, 4), (2048, 1024, 3072, 0), (130, 1024, 3072, 2)])
def test_gemm_cta_pair_kernel_with_the_fused_epilogues(ops, M, N, K, kg):
    torch.manual_seed(M + K)
    x, w = _rand(M, K), _rand(N, K, scale=0.05)
    residual = _rand(M, N, scale=2.0)
    want = ((x.float() @ w.float().t()).to(BF).float() + residual.float()).to(BF)
    parts = (N + 127) // 128
    ssq = torch.full((M, parts), float("nan"), dtype=torch.float32, device="cuda")
    res = residual.clone()
    ops.linear_residual(x, w, res, ssq, force_mode=4, tune=kg)
    _close(res, want, atol=6e-2, rtol=2e-2)
    sq = torch.nn.functional.pad(res.float() ** 2, (0, parts * 128 - N)).view(M, parts, 128).sum(-1)
    assert torch.allclose(ssq, sq, rtol=1e-3, atol=1e-3)
    pk = (K + 127) // 128
    ssq_in = (x.float() ** 2).view(M, pk, -1).sum(-1).contiguous()
    got = ops.linear_scaled(x, w, ssq_in, 1e-6, force_mode=4, tune=kg)
    xn = x.float() * torch.rsqrt((x.float() ** 2).mean(-1, keepdim=True) + 1e-6)
    _close(got, xn @ w.float().t(), atol=3e-2, rtol=3e-2)
    ops.check_status()


@pytest.mark.parametrize("M,N,K,silu", [(600, 1280, 1024, False), (2048, 3200, 5120, True), (1000, 5120, 3200, False)])
def test_fp8_weights_with_many_tokens_are_expanded_and_multiplied_in_bf16(ops, M, N, K, silu):
    """Prefill-sized GEMM on a block-scaled e4m3 weight: the weight is expanded to bf16 (exactly: e4m3 x scale rounded to
    bf16) right before the bf16 GEMM, which must not read it early; activations are not quantised."""
    from tinyllmforge_b200.ops.quant import Fp8BlockWeight
    torch.manual_seed(N + K)
    w = _rand(2 * N if silu else N, K, scale=0.05)
    wq = Fp8BlockWeight.quantize(w)
    wd = wq.dequantize()
    assert torch.equal(ops._expand_fp8(wq), wd.to(BF))
    for seed in range(3):                              # the scratch buffer is overwritten between calls
        x = _rand(M, K)
        got = (ops.linear_silu_mul if silu else ops.linear)(x, wq)
        ref_ = x.float() @ wd.to(BF).float().t()
        want = torch.nn.functional.silu(ref_[:, :N]) * ref_[:, N:] if silu else ref_
        _close(got, want, atol=2e-2, rtol=2e-2)
        other = Fp8BlockWeight.quantize(_rand(2 * N if silu else N, K, scale=0.05))
        ops._expand_fp8(other)
    ops.check_status()


@pytest.mark.parametrize("mode", [5, 6])
@pytest.mark.parametrize("M,N,K,S,silu", [
    (256, 4096, 4096, 4, False), (64, 6144, 4096, 6, False), (200, 4096, 12288, 4, False), (16, 1280, 5120, 8, False),
    (100, 5120, 3200, 3, False), (130, 1536, 4096, 4, True), (50, 3200, 5120, 2, True), (7, 136, 4104, 5, False), (300, 1000, 2048, 2, False),
])
def test_gemm_split_k_with_reduce_kernel(ops, M, N, K, S, silu, mode):
    """K split S ways, one (tile, K range) per CTA or CTA pair; a second kernel adds the partial tiles and runs the epilogue."""
    torch.manual_seed(M + N + K)
    x, w = _rand(M, K), _rand(2 * N if silu else N, K, scale=0.05)
    fn = ops.linear_silu_mul if silu else ops.linear
    out = fn(x, w, force_mode=mode, force_splits=S)
    ref_ = x.float() @ w.float().t()
    want = torch.nn.functional.silu(ref_[:, :N]) * ref_[:, N:] if silu else ref_
    _close(out, want, atol=2e-2, rtol=2e-2)
    assert torch.equal(out, fn(x, w, force_mode=mode, force_splits=S))
    ops.check_status()


@pytest.mark.parametrize("mode", [5, 6])
@pytest.mark.parametrize("M,N,K,S", [(256, 4096, 4096, 4), (64, 4096, 12288, 8), (130, 1024, 3072, 2), (40, 5120, 3200, 4)])
def test_gemm_split_k_with_reduce_kernel_and_fused_epilogues(ops, M, N, K, S, mode):
    torch.manual_seed(M + K)
    x, w = _rand(M, K), _rand(N, K, scale=0.05)
    residual = _rand(M, N, scale=2.0)
    want = ((x.float() @ w.float().t()).to(BF).float() + residual.float()).to(BF)
    parts = (N + 127) // 128
    ssq = torch.full((M, parts), float("nan"), dtype=torch.float32, device="cuda")
    res = residual.clone()
    ops.linear_residual(x, w, res, ssq, force_mode=mode, tune=S)
    _close(res, want, atol=6e-2, rtol=2e-2)
    sq = torch.nn.functional.pad(res.float() ** 2, (0, parts * 128 - N)).view(M, parts, 128).sum(-1)
    assert torch.allclose(ssq, sq, rtol=1e-3, atol=1e-3)
    res2, ssq2 = residual.clone(), torch.empty_like(ssq)
    ops.linear_residual(x, w, res2, ssq2, force_mode=mode, tune=S)
    assert torch.equal(res2, res) and torch.equal(ssq2, ssq)
    pk = (K + 127) // 128
    ssq_in = (x.float() ** 2).view(M, pk, -1).sum(-1).contiguous()
    got = ops.linear_scaled(x, w, ssq_in, 1e-6, force_mode=mode, tune=S)
    xn = x.float() * torch.rsqrt((x.float() ** 2).mean(-1, keepdim=True) + 1e-6)
    _close(got, xn @ w.float().t(), atol=3e-2, rtol=3e-2)
    ops.check_status()


@pytest.mark.parametrize("T,K,nq,nkv,bs,folded", [(64, 1024, 16, 8, 256, True), (256, 1024, 16, 8, 256, False), (33, 4096, 32, 8, 16, True),
                                                 (200, 512, 8, 1, 64, False), (1, 256, 4, 2, 256, True)])
def test_qkv_gemm_with_norm_rope_and_cache_store_in_its_epilogue(ops, T, K, nq, nkv, bs, folded):
    """The qkv projection whose epilogue normalises q and k per head, rotates them and writes k / v into the paged cache,
    against the fp32 statement of the same chain (projection rounded to bf16, then q/k-norm + RoPE + store)."""
    torch.manual_seed(T + K)
    D, nblk = 128, 8 + T // bs
    x = _rand(T, K)
    w = _rand((nq + 2 * nkv) * D, K, scale=0.05)
    qw, kw = _rand(D, scale=0.2) + 1, _rand(D, scale=0.2) + 1
    table = ref.rope_table(4096, D, 1e6, "cuda")
    pos = torch.randint(0, 4096, (T,), dtype=torch.int32, device="cuda")
    slots = torch.randperm(nblk * bs, device="cuda")[:T].to(torch.int32)
    if T > 2:
        slots[1] = -1
    kc, vc = torch.zeros(nblk, nkv, bs, D, dtype=BF, device="cuda"), torch.zeros(nblk, nkv, bs, D, dtype=BF, device="cuda")
    kc2, vc2 = kc.clone(), vc.clone()
    ssq = None
    proj = x.float() @ w.float().t()
    if folded:
        parts = (K + 127) // 128
        ssq = (x.float() ** 2).view(T, parts, -1).sum(-1).contiguous()
        proj = proj * torch.rsqrt((x.float() ** 2).mean(-1, keepdim=True) + 1e-6)
    q = ops.linear_qkv_rope_store(x, w, ssq, 1e-6, qw, kw, 1e-6, table, pos, slots, kc, vc, nq, nkv)
    q_want = ref.qk_norm_rope_store(proj.to(BF), qw, kw, 1e-6, table, pos, slots, kc2, vc2, nq, nkv, D)
    _close(q, q_want, 3e-2, 3e-2)
    _close(kc, kc2, 3e-2, 3e-2)
    _close(vc, vc2, 2e-2, 2e-2)
    if T > 2:
        assert torch.count_nonzero(kc) == torch.count_nonzero(kc2)          # the row with slot -1 was not stored
    ops.check_status()


def test_embedding_sum_of_squares(ops):
    V, H, T = 512, 1024, 37
    table = _rand(V, H)
    ids = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
    out, ssq, scratch = ops.embedding_ssq(ids, table, 0)
    assert torch.equal(out, table[ids.long()])
    assert ssq.shape == (T, H // 128) == scratch.shape
    assert torch.allclose(ssq.sum(-1), (out.float() ** 2).sum(-1), rtol=1e-4)
    assert torch.count_nonzero(ssq[:, 1:]) == 0


def test_gemm_strided_input(ops):
    big = _rand(64, 3 * 256)
    x = big[:, 256:512]          # row stride 768, 16-byte aligned start
    w = _rand(128, 256, scale=0.05)
    _close(ops.linear(x, w), x.float() @ w.float().t(), 2e-2, 2e-2)


# ----------------------------------------------------------------------------- norms / activation / gathers
@pytest.mark.parametrize("rows,H", [(1, 1024), (37, 1024), (5, 4096), (3, 5120), (2, 256), (4, 8192)])
def test_rms_norm(ops, rows, H):
    x, w = _rand(rows, H), _rand(H, scale=0.3) + 1
    _close(ops.rms_norm(x, w, 1e-6), ref.rms_norm(x, w, 1e-6), 1e-2, 1e-2)


@pytest.mark.parametrize("rows,H", [(1, 1024), (33, 1024), (6, 4096), (3, 5120)])
def test_add_rms_norm(ops, rows, H):
    x, r, w = _rand(rows, H), _rand(rows, H), _rand(H, scale=0.3) + 1
    want_y, want_r = ref.add_rms_norm(x, r, w, 1e-6)
    r2 = r.clone()
    y, r_out = ops.add_rms_norm(x, r2, w, 1e-6)
    assert r_out.data_ptr() == r2.data_ptr()
    assert torch.equal(r_out, want_r)
    _close(y, want_y, 1e-2, 1e-2)


def test_silu_mul(ops):
    x = _rand(77, 2 * 3072, scale=2.0)
    _close(ops.silu_mul(x), ref.silu_mul(x), 1e-2, 1e-2)


def test_embedding_shard_and_gather(ops):
    w = _rand(1000, 1024)
    ids = torch.tensor([0, 999, 1000, 1500, 2000, 1234], dtype=torch.int32, device="cuda")
    got = ops.embedding(ids, w, 1000)
    assert torch.equal(got, ref.embedding(ids, w, 1000))
    idx = torch.tensor([5, 0, 3], dtype=torch.int32, device="cuda")
    assert torch.equal(ops.select_rows(got, idx), got[idx.long()])


# ----------------------------------------------------------------------------- q/k norm + rope + KV store
@pytest.mark.parametrize("T,nq,nkv,bs", [(1, 16, 8, 256), (50, 16, 8, 16), (9, 4, 1, 64)])
def test_qk_norm_rope_store(ops, T, nq, nkv, bs):
    D, nblk = 128, 8
    qkv = _rand(T, (nq + 2 * nkv) * D)
    qw, kw = _rand(D, scale=0.2) + 1, _rand(D, scale=0.2) + 1
    table = ref.rope_table(4096, D, 1e6, "cuda")
    pos = torch.randint(0, 4096, (T,), dtype=torch.int32, device="cuda")
    slots = torch.randperm(nblk * bs, device="cuda")[:T].to(torch.int32)
    if T > 2:
        slots[1] = -1
    kc, vc = torch.zeros(nblk, nkv, bs, D, dtype=BF, device="cuda"), torch.zeros(nblk, nkv, bs, D, dtype=BF, device="cuda")
    kc2, vc2 = kc.clone(), vc.clone()
    q = ops.qk_norm_rope_store(qkv, qw, kw, 1e-6, table, pos, slots, kc, vc, nq, nkv, D)
    q_want = ref.qk_norm_rope_store(qkv, qw, kw, 1e-6, table, pos, slots, kc2, vc2, nq, nkv, D)
    _close(q, q_want, 2e-2, 2e-2)
    _close(kc, kc2, 2e-2, 2e-2)
    assert torch.equal(vc, vc2)
    ops.check_status()


# ----------------------------------------------------------------------------- attention
class _Batch:
    pass


def _paged_case(q_lens, k_lens, nq, nkv, bs, seed=0):
    torch.manual_seed(seed)
    D = 128
    S = len(q_lens)
    nblk_per = [-(-k // bs) for k in k_lens]
    total = sum(nblk_per) + 3
    perm = torch.randperm(total).tolist()
    width = max(nblk_per) + 1
    bt = torch.full((S, width), -1, dtype=torch.int32)
    p = 0
    for s, n in enumerate(nblk_per):
        bt[s, :n] = torch.tensor(perm[p:p + n], dtype=torch.int32)
        p += n
    kc, vc = _rand(total, nkv, bs, D), _rand(total, nkv, bs, D)
    T = sum(q_lens)
    q = _rand(T, nq, D)
    b = _Batch()
    b.cu_seqlens_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    b.context_lens = torch.tensor(k_lens, dtype=torch.int32, device="cuda")
    b.block_tables = bt.cuda()
    b.num_seqs = b.padded_seqs = S
    b.max_seqlen_q, b.max_seqlen_k = max(q_lens), max(k_lens)
    b.table_width = width
    return q, kc, vc, b


@pytest.mark.parametrize("mode", ["flat", "chunked"])
@pytest.mark.parametrize("k_lens,nq,nkv,bs", [
    ([1], 16, 8, 256), ([5, 300, 64, 1000], 16, 8, 256), ([17, 33, 250], 8, 2, 16), ([700, 2011, 129], 32, 8, 256),
    ([40, 90], 8, 8, 32), ([513, 77], 8, 1, 64), ([300, 1000, 70, 2], 40, 8, 256), ([129, 640, 33], 64, 8, 256), ([50, 400], 6, 2, 64), ([700, 2011, 129], 8, 1, 256),
])
def test_decode_attention(ops, k_lens, nq, nkv, bs, mode, monkeypatch):
    monkeypatch.setattr(ops, "decode_attention_mode", mode)
    q, kc, vc, b = _paged_case([1] * len(k_lens), k_lens, nq, nkv, bs)
    b.is_prefill = False
    got = ops.attention(q, kc, vc, b, 128 ** -0.5)
    want = ref.attention(q, kc, vc, b.cu_seqlens_q, b.context_lens, b.block_tables, 128 ** -0.5, b.num_seqs)
    _close(got, want, 2e-2, 2e-2)
    ops.check_status()


@pytest.mark.parametrize("mode", ["flat", "chunked"])
def test_decode_attention_reports_a_length_the_block_table_cannot_describe(ops, mode, monkeypatch):
    """A context length written too large on the host (one block more than the table has) is clamped on the device: the
    status word gets the bad-index bit, every access stays inside the table and the scratch, the other rows are right."""
    monkeypatch.setattr(ops, "decode_attention_mode", mode)
    k_lens = [300, 100, 520]
    q, kc, vc, b = _paged_case([1] * 3, k_lens, 16, 8, 256)
    b.is_prefill = False
    want = ref.attention(q, kc, vc, b.cu_seqlens_q, b.context_lens, b.block_tables, 128 ** -0.5, 3)
    b.context_lens = b.context_lens.clone()
    b.context_lens[1] = (b.table_width + 1) * 256
    b.block_tables = b.block_tables.clone()
    b.block_tables[1, 1:] = b.block_tables[1, 0]        # the clamped row reads valid blocks; its result is not checked
    ops.check_status()
    got = ops.attention(q, kc, vc, b, 128 ** -0.5)
    torch.cuda.synchronize()
    word = int(ops.status[0].item())
    assert word & 4, word
    ops.status.zero_()
    _close(got[[0, 2]], want[[0, 2]], 2e-2, 2e-2)


@pytest.mark.parametrize("mode", ["flat", "chunked"])
def test_decode_attention_padding_rows(ops, mode, monkeypatch):
    monkeypatch.setattr(ops, "decode_attention_mode", mode)
    q, kc, vc, b = _paged_case([1, 1, 1], [100, 0, 7], 16, 8, 256)
    b.is_prefill = False
    got = ops.attention(q, kc, vc, b, 128 ** -0.5)
    assert torch.count_nonzero(got[1]) == 0
    want = ref.attention(q, kc, vc, b.cu_seqlens_q, b.context_lens, b.block_tables, 128 ** -0.5, 3)
    _close(got[[0, 2]], want[[0, 2]], 2e-2, 2e-2)


@pytest.mark.parametrize("mode", ["flat", "chunked"])
@pytest.mark.parametrize("k_lens,nq,nkv,bs", [
    ([1, 2, 64, 65, 300, 1000, 0, 256, 257, 512], 16, 8, 256), ([17, 33, 250, 16, 1], 8, 2, 16), ([700, 2011, 129, 128], 32, 8, 256),
    ([40, 90, 64], 8, 8, 32), ([513, 77], 8, 1, 64), (list(range(1, 140, 3)), 16, 8, 128), ([300, 1000, 70, 2], 40, 8, 256),
    ([129, 640, 33], 64, 8, 256),
])
def test_decode_attention_from_raw_qkv(ops, k_lens, nq, nkv, bs, mode, monkeypatch):
    """q/k-norm + rotation + KV store inside the attention kernel == qk_norm_rope_store followed by attention:
    same output, same cache contents (the step's token of every sequence sits at position len - 1)."""
    monkeypatch.setattr(ops, "decode_attention_mode", mode)
    S, D = len(k_lens), 128
    _, kc, vc, b = _paged_case([1] * S, [max(k, 1) for k in k_lens], nq, nkv, bs, seed=7)
    b.context_lens = torch.tensor(k_lens, dtype=torch.int32, device="cuda")
    b.is_prefill = False
    torch.manual_seed(11)
    qkv = _rand(S, (nq + 2 * nkv) * D)
    qw, kw = _rand(D, scale=0.2) + 1, _rand(D, scale=0.2) + 1
    table = ref.rope_table(4096, D, 1e6, "cuda")
    lens = b.context_lens.long()
    pos = (lens - 1).clamp(min=0).to(torch.int32)
    blk = b.block_tables.long()[torch.arange(S), ((lens - 1).clamp(min=0) // bs).cpu()]
    slots = torch.where(lens > 0, blk.cuda() * bs + (lens - 1) % bs, torch.full_like(lens, -1)).to(torch.int32)
    kc1, vc1, kc2, vc2 = kc.clone(), vc.clone(), kc.clone(), vc.clone()
    q = ops.qk_norm_rope_store(qkv, qw, kw, 1e-6, table, pos, slots, kc1, vc1, nq, nkv, D)
    want = ops.attention(q, kc1, vc1, b, D ** -0.5)
    got = ops.decode_attention_qkv(qkv, qw, kw, 1e-6, table, kc2, vc2, b, nq, D ** -0.5)
    live = [i for i, n in enumerate(k_lens) if n > 0]
    _close(got[live], want[live], 2e-2, 2e-2)
    _close(kc2, kc1, 1e-2, 1e-2)
    assert torch.equal(vc2, vc1)
    for i, n in enumerate(k_lens):
        if n == 0:
            assert torch.count_nonzero(got[i]) == 0
    ops.check_status()


@pytest.mark.parametrize("k_lens,nq,nkv", [([300, 1000, 70, 2], 32, 8), ([129, 640, 33, 2011], 40, 8), ([50, 400, 900], 8, 2)])
def test_decode_attention_cuda_core_variant_for_groups_of_4_and_5(ops, k_lens, nq, nkv, monkeypatch):
    """The flat kernel runs groups of 4..8 q heads per KV head on the tensor cores by default (covered by the tests above); the
    CUDA-core kernel stays selectable for them and must agree too."""
    monkeypatch.setattr(ops, "decode_attention_mode", "flat")
    q, kc, vc, b = _paged_case([1] * len(k_lens), k_lens, nq, nkv, 256)
    b.is_prefill = False
    want = ref.attention(q, kc, vc, b.cu_seqlens_q, b.context_lens, b.block_tables, 128 ** -0.5, b.num_seqs)
    ops.C.decode_attention_set_tc_min_group(9)
    try:
        got = ops.attention(q, kc, vc, b, 128 ** -0.5)
        torch.cuda.synchronize()
    finally:
        ops.C.decode_attention_set_tc_min_group(4)
    _close(got, want, 2e-2, 2e-2)
    ops.check_status()


@pytest.mark.parametrize("batch,lo,hi,nq,nkv", [(64, 100, 1500, 16, 8), (200, 1, 700, 16, 8), (300, 3000, 3100, 8, 2), (7, 1, 4000, 32, 8),
                                                (70, 100, 2500, 64, 8)])
def test_decode_attention_flat_partition_many_sequences(ops, batch, lo, hi, nq, nkv, monkeypatch):
    """Enough tiles that every CTA's range spans several (sequence, head) items and most items are cut at most once;
    lengths from 1 token to several thousand, zero-length rows in between; both kernels against the fp32 statement,
    twice in a row (the scratch keeps stale partials from the first call)."""
    g = torch.Generator().manual_seed(batch)
    k_lens = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
    for i in range(3, batch, 17):
        k_lens[i] = 0
    q, kc, vc, b = _paged_case([1] * batch, k_lens, nq, nkv, 256, seed=batch)
    b.is_prefill = False
    want = ref.attention(q, kc, vc, b.cu_seqlens_q, b.context_lens, b.block_tables, 128 ** -0.5, b.num_seqs)
    live = [i for i, n in enumerate(k_lens) if n > 0]
    for mode in ("flat", "flat", "chunked"):
        monkeypatch.setattr(ops, "decode_attention_mode", mode)
        got = ops.attention(q, kc, vc, b, 128 ** -0.5)
        _close(got[live], want[live], 2e-2, 2e-2)
        assert torch.count_nonzero(got[3]) == 0
    ops.check_status()


@pytest.mark.parametrize("q_lens,k_lens,nq,nkv,bs", [
    ([64], [64], 16, 8, 256), ([1, 100, 257], [1, 100, 257], 16, 8, 256), ([30, 70], [286, 70], 8, 2, 256),
    ([50, 200], [50, 200], 4, 4, 16), ([10], [522], 8, 1, 32), ([1000], [1000], 2, 1, 256),
    ([300, 129, 128, 1], [812, 129, 640, 1], 8, 2, 128), ([513, 40], [513, 1064], 4, 1, 256), ([128, 256], [128, 256], 16, 8, 512),
])
def test_prefill_attention(ops, q_lens, k_lens, nq, nkv, bs):
    q, kc, vc, b = _paged_case(q_lens, k_lens, nq, nkv, bs, seed=1)
    b.is_prefill = True
    got = ops.attention(q, kc, vc, b, 128 ** -0.5)
    want = ref.attention(q, kc, vc, b.cu_seqlens_q, b.context_lens, b.block_tables, 128 ** -0.5, b.num_seqs)
    _close(got, want, 2e-2, 2e-2)
    ops.check_status()


# ----------------------------------------------------------------------------- sampler
def _header(step, seed):
    h = torch.zeros(16, dtype=torch.int32)
    h[9], h[10], h[11] = step, seed & 0x7FFFFFFF, 0
    return h.cuda()


def test_sampler_greedy_and_gumbel_match_reference(ops):
    torch.manual_seed(3)
    rows, vocab = 6, 151936
    logits = _rand(rows, vocab, scale=3.0)
    temps = torch.tensor([0.0, 0.6, 1.0, 0.0, 2.0, 0.3], device="cuda")
    ids, best = ops.sample_shard(logits, temps, _header(11, 1234), 0)
    want_ids, want_best = ref.sample(logits.cpu(), temps.cpu(), 1234, 11, 0)
    _close(best.cpu(), want_best, 1e-3, 1e-4)
    assert torch.equal(ids.cpu().long()[[0, 3]], logits.float().argmax(-1).cpu()[[0, 3]])
    # sampled rows: the chosen id must be (near-)optimal under the reference's perturbed scores
    assert (ids.cpu().long() == want_ids).float().mean() >= 0.8


def test_sampler_is_invariant_to_vocab_sharding(ops):
    torch.manual_seed(4)
    rows, vocab, tp = 5, 4096 * 4, 4
    logits = _rand(rows, vocab, scale=2.0)
    temps = torch.full((rows,), 0.8, device="cuda")
    hdr = _header(5, 99)
    full_ids, _ = ops.sample_shard(logits, temps, hdr, 0)
    shard = vocab // tp
    vals, ids = [], []
    for r in range(tp):
        i, v = ops.sample_shard(logits[:, r * shard:(r + 1) * shard], temps, hdr, r * shard)
        ids.append(i)
        vals.append(v)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.C.sample_merge_ranks(torch.stack(vals), torch.stack(ids), out)
    assert torch.equal(out, full_ids)


@pytest.mark.parametrize("vocab,start", [(16, 0), (80, 0), (72, 16)])
def test_sampler_distribution(ops, vocab, start):
    """Empirical frequencies over many rows follow softmax(logits / T): one group (level 2 alone), several groups (level 1
    picks the group, level 2 the token), and a shard whose last group is partial."""
    T, n = 0.7, 6000
    base = torch.linspace(-2, 2, vocab, device="cuda")[torch.randperm(vocab, device="cuda", generator=torch.Generator(device="cuda").manual_seed(vocab))]
    logits = base.to(BF)[None].repeat(n, 1).contiguous()
    temps = torch.full((n,), T, device="cuda")
    ids, _ = ops.sample_shard(logits, temps, _header(1, 7), start)
    freq = torch.bincount(ids.long().cpu() - start, minlength=vocab).float() / n
    want = torch.softmax(logits[0].float().cpu() / T, -1)
    assert (freq - want).abs().max() < 0.025


@pytest.mark.parametrize("rows,vocab,start", [(8, 151936, 0), (64, 75968, 75968), (200, 40000, 40000), (256, 151936, 0)])
def test_lm_head_gemm_samples_in_its_epilogue_like_the_two_kernel_path(ops, rows, vocab, start):
    """LM head + sampling in one kernel (logits never written) picks exactly the tokens of GEMM -> logits -> sampler:
    the same bf16-rounded logits, the same noise per (row, global token id); greedy rows (T = 0) are the arg-max."""
    torch.manual_seed(rows + vocab)
    K = 1024
    hidden, w = _rand(rows, K), _rand(vocab, K, scale=0.05)
    temps = torch.full((rows,), 0.6, device="cuda")
    temps[::3] = 0.0
    temps[1::5] = 1.3
    hdr = _header(step=11, seed=5)
    assert ops.can_sample_in_lm_head(rows, w)
    ids, best = ops.lm_head_sample_shard(hidden, w, temps, hdr, start)
    logits = ops.linear(hidden, w)
    want_ids, want_best = ops.sample_shard(logits, temps, hdr, start)
    assert torch.equal(ids, want_ids)
    assert torch.equal(best, want_best)
    greedy = (temps == 0).nonzero().flatten()
    assert torch.equal(ids[greedy].long() - start, logits[greedy].float().argmax(-1))
    ops.check_status()


# ----------------------------------------------------------------------------- bounded waits
def test_peer_flag_wait_runs_out_and_reports_status(ops):
    """Failure detection on the device: a consumer waits for a peer that never signals (the flag word is simply
    never written), gives up after its time limit, sets the status bit, and the context stays usable."""
    import time
    H, rows = 1024, 4
    parts = torch.zeros(2, rows, H, dtype=BF, device="cuda")             # both "ranks'" partial buffers live on this GPU
    signal = torch.zeros(8, dtype=torch.int32, device="cuda")
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")            # this rank claims one completed production ...
    signal[0] = 1                                                       # ... rank 0's flag is there, rank 1's never arrives
    normal_mode = torch.zeros(1, dtype=torch.int32, device="cuda")      # the measurement-mode switch stays off
    out = torch.empty(rows, H, dtype=BF, device="cuda")
    torch.cuda.synchronize()
    t0 = time.monotonic()
    ops.C.tp_reduce_rms_norm(2, 0, [parts[0].data_ptr(), parts[1].data_ptr()], 0, 0, signal.data_ptr(), epoch.data_ptr(), int(0.2e9),
                             normal_mode.data_ptr(), None, out, None, None, 1e-6, ops.status)
    torch.cuda.synchronize()
    assert 0.15 < time.monotonic() - t0 < 5.0
    with pytest.raises(RuntimeError, match="peer flag wait ran out"):
        ops.check_status()
    ops.check_status()                                                  # the word was cleared; nothing else is wrong
    x = _rand(8, 1024)
    assert torch.isfinite(ops.rms_norm(x, torch.ones(1024, dtype=BF, device="cuda"), 1e-6).float()).all()

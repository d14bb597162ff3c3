"""Block-scaled fp8 weights (``quantization="fp8_block"``): e4m3 values with one fp32 scale per 128 x 128 block,
bf16 activations quantised on the fly per token and per 128 input features.  The reference has no quantised path.
"""
from __future__ import annotations

import torch

BLOCK = 128
E4M3_MAX = 448.0


class Fp8BlockWeight:
    """A linear weight ``[N, K]`` stored as e4m3 + block scales ``[ceil(N / 128), K / 128]``."""

    def __init__(self, q: torch.Tensor, scale: torch.Tensor):
        assert q.dtype == torch.float8_e4m3fn and scale.dtype == torch.float32
        self.q, self.scale = q.contiguous(), scale.contiguous()
        self.shape = tuple(q.shape)
        self.dtype = torch.bfloat16
        self.device = q.device

    @classmethod
    def quantize(cls, w: torch.Tensor) -> "Fp8BlockWeight":
        N, K = w.shape
        if K % BLOCK:
            raise ValueError(f"in_features ({K}) must be a multiple of {BLOCK} for fp8_block")
        nb = -(-N // BLOCK)
        wf = torch.zeros(nb * BLOCK, K, dtype=torch.float32, device=w.device)
        wf[:N] = w.float()
        blocks = wf.view(nb, BLOCK, K // BLOCK, BLOCK)
        amax = blocks.abs().amax(dim=(1, 3))
        scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
        q = (blocks / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).view(nb * BLOCK, K)[:N].to(torch.float8_e4m3fn)
        return cls(q, scale)

    def dequantize(self) -> torch.Tensor:
        N, K = self.shape
        s = self.scale.repeat_interleave(BLOCK, 0)[:N].repeat_interleave(BLOCK, 1)
        return self.q.float() * s

    def __getitem__(self, idx):        # row slices at block granularity (gate / up halves)
        raise TypeError("slice the bf16 weight before quantising")


def quantize_activations_ref(x: torch.Tensor):
    """Per token, per 128 features: (e4m3 values, scales [K / 128, M]).  Oracle of the CUDA quantiser."""
    M, K = x.shape
    xb = x.float().view(M, K // BLOCK, BLOCK)
    amax = xb.abs().amax(-1)
    s = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (xb / s[..., None]).view(M, K).to(torch.float8_e4m3fn)
    return q, s.t().contiguous()


def linear_fp8_ref(x: torch.Tensor, w: Fp8BlockWeight) -> torch.Tensor:
    """What the fp8 kernel computes, in fp32: quantised activations times quantised weights."""
    q, s = quantize_activations_ref(x)
    xd = q.float().view(x.shape[0], -1, BLOCK) * s.t()[..., None]
    return (xd.view(x.shape[0], -1) @ w.dequantize().t()).to(x.dtype)

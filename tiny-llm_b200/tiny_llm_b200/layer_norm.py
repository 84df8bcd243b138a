"""Readable RMSNorm (``/root/reference/src/tiny_llm_ref/layer_norm.py:4-15``)."""

from __future__ import annotations

import torch


class RMSNorm:
    def __init__(self, dim: int, weight: torch.Tensor, eps: float = 1e-5):
        self.dim = dim
        self.eps = eps
        self.weight = weight

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        # fp32 statistics, storage-dtype product with the weight (two roundings;
        # the fused kernel rounds once - week2_kernels.metal:41-47).
        h = x.to(torch.float32)
        h = h * torch.rsqrt(h.square().mean(dim=-1, keepdim=True) + self.eps)
        return h.to(x.dtype) * self.weight.to(x.dtype)


class ResidualRMSNorm:
    """RMS norm on a sublayer's OUTPUT, accumulated into a residual stream that is kept in fp32:

        residual <- residual + y / sqrt(mean(y^2) + eps) * (weight + weight_offset) * scale

    ``weight_offset`` = 1 for weights stored around zero, 0 for plain weights; ``scale`` is an optional per-channel
    layer scale.  One launch of the blocks library does the norm, the scale, the sum and the rounding of the new
    residual to the compute dtype (the next sublayer's input).  Without ``residual`` it is a plain row norm."""

    def __init__(self, weight: torch.Tensor, eps: float, weight_offset: float = 0.0, scale: torch.Tensor | None = None):
        self.weight, self.eps, self.weight_offset, self.scale = weight.contiguous(), float(eps), float(weight_offset), scale
        if scale is not None:
            self.scale = scale.contiguous()

    def __call__(self, y: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        from extensions_b200.tiny_llm_ext_b200 import blocks

        return blocks.norm_residual(y, self.weight, self.eps, weight_offset=self.weight_offset, scale=self.scale, residual=residual)

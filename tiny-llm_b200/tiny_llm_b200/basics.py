"""Readable Week-1 operators on torch tensors.

Signatures of ``/root/reference/src/tiny_llm_ref/basics.py:5-26``.  These are
the un-fused building blocks the early Week-2 checkpoints still use; they run
as ordinary torch ops on whatever device the tensors live on.
"""

from __future__ import annotations

import torch


def softmax(x: torch.Tensor, axis: int) -> torch.Tensor:
    return torch.softmax(x, dim=axis)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    y = torch.matmul(x, w.transpose(-1, -2))
    return y if bias is None else y + bias


def silu(x: torch.Tensor) -> torch.Tensor:
    # sigmoid evaluated through exp(-|x|) so neither branch overflows
    z = torch.exp(-torch.abs(x))
    return x * torch.where(x < 0, z / (1 + z), 1 / (1 + z))


_WIDE_OUT = {"ok": None}


def linear_wide(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` with the fp32 accumulator handed back unrounded (for products that feed a norm or are the logits),
    where the library product can do that for these shapes; else the product in the operand dtype, widened.
    fp32 operands: plain ``linear``."""
    if x.dtype == torch.float32:
        return linear(x, w)
    if _WIDE_OUT["ok"] is not False:
        try:
            out = torch.mm(x, w.t(), out_dtype=torch.float32)
            _WIDE_OUT["ok"] = True
            return out
        except (TypeError, RuntimeError):
            if _WIDE_OUT["ok"] is None:
                _WIDE_OUT["ok"] = False  # this torch has no such product at all
    return linear(x, w).float()

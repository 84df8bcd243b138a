"""Gated feed-forward layers with unquantised weights: ``down(act(gate x) * (up x))``.

``GatedMLP`` is the dense form (gate and up stacked into one product, the activation fused with the gating product in
one launch); ``TopKRouter`` + ``MixtureOfExperts`` the sparse one: router logits in fp32, the ``top`` largest chosen,
weights either a softmax over the chosen logits or each chosen logit's sigmoid as it is, the chosen experts' outputs
summed with those weights (or, ``weight_on="input"``, each expert run on its weight times the token), optionally plus
a shared expert that every token takes.  Experts are gated or, without ``w_gate``, plain ``down(act(up x))``.  The expert products are grouped GEMMs of the blocks library over a device-built
list of (token, choice) pairs sorted by expert: no host synchronisation, and a token's result does not depend on the
rest of the batch."""

from __future__ import annotations

import torch

from .basics import linear, linear_wide

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu_squared": 2}
SCORINGS = {"softmax": 0, "sigmoid": 1}


class GatedMLP:
    def __init__(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, act: str):
        self.w_gate_up = torch.cat([w_gate, w_up], dim=0).contiguous()  # [2 ff, D]: one product for both
        self.w_down = w_down.contiguous()
        self.act = ACTIVATIONS[act]

    def __call__(self, h: torch.Tensor, wide: bool = False) -> torch.Tensor:
        """``wide``: hand the down projection's fp32 accumulator back unrounded (when a norm reads it next)."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        return (linear_wide if wide else linear)(blocks.gated_act(linear(h, self.w_gate_up), self.act), self.w_down)


class TopKRouter:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, top: int, scoring: str = "softmax"):
        self.weight, self.bias, self.top = weight.contiguous(), None if bias is None else bias.contiguous(), int(top)
        self.scoring = SCORINGS[scoring]
        if not 0 < self.top <= weight.shape[0]:
            raise ValueError(f"router: top={top} of {weight.shape[0]} experts")

    def __call__(self, h: torch.Tensor):
        """-> (expert ids int32 [T, top], weights fp32 [T, top])."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        return blocks.moe_route(h, self.weight, self.bias, self.top, self.scoring)


class MixtureOfExperts:
    def __init__(self, router: TopKRouter, w_gate: torch.Tensor | None, w_up: torch.Tensor, w_down: torch.Tensor, act: str,
                 shared: GatedMLP | None = None, weight_on: str = "output"):
        """``w_gate, w_up [E, ff, D]``, ``w_down [E, D, ff]`` (the experts stacked); ``w_gate`` None = experts without a gate."""
        if weight_on not in ("output", "input"):
            raise ValueError(f"weight_on={weight_on!r}")
        self.router, self.shared, self.scale_input = router, shared, weight_on == "input"
        self.w_gate, self.w_up, self.w_down = None if w_gate is None else w_gate.contiguous(), w_up.contiguous(), w_down.contiguous()
        self.act = ACTIVATIONS[act]

    def __call__(self, h: torch.Tensor) -> torch.Tensor:
        """-> fp32 [T, D]."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        idx, gate = self.router(h)
        shared = None if self.shared is None else self.shared(h)
        return blocks.moe_experts(h, idx, gate, self.w_gate, self.w_up, self.w_down, self.act, shared, scale_input=self.scale_input)

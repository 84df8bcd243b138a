"""Linear attention with a per-channel decay: a recurrent mixer whose state lives in fp32 slots.

Per head a matrix ``S [dim, vdim]`` is carried along the sequence,

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        o_t = S_t^T (dim^-1/2 q_t)        alpha_t = sigmoid(z_t)^(1 / tau)

with the decay logits ``z = W_a2 (W_a1 h) + b`` from a low-rank projection.  Each head's output is RMS-normed over
``vdim`` (plain weight shared by the heads), multiplied by ``silu(W_g h)`` and projected.  The projections of ``h``
(q, k, v, gate, the low-rank decay input) are made by the caller in one product; this module takes their views.  The
second decay projection hands its fp32 accumulator over, and the decay, the recurrence and the norm are fp32 whatever
the compute dtype.  ``state`` is the layer's view ``[slots, heads, dim, vdim]`` of the model's ``StateSlotPool``; the
plan's ``seq_info`` says which slot a sequence owns and whether it starts at position 0 (then from zero).
"""

from __future__ import annotations

import torch

from .basics import linear_wide


class DecayedLinearAttention:
    def __init__(self, *, heads: int, dim: int, vdim: int, tau: float, w_a2, a2_bias, norm_weight, w_o, eps: float = 1e-6):
        if tuple(w_a2.shape)[0] != heads * dim or tuple(w_o.shape)[1] != heads * vdim or tuple(norm_weight.shape) != (vdim,):
            raise ValueError("linear attention: tensor shapes do not match the head sizes")
        if not tau > 0:
            raise ValueError("linear attention: tau must be positive")
        self.heads, self.dim, self.vdim, self.tau, self.eps = int(heads), int(dim), int(vdim), float(tau), float(eps)
        self.w_a2, self.a2_bias = w_a2.contiguous(), None if a2_bias is None else a2_bias.contiguous()
        self.norm_weight, self.w_o = norm_weight.contiguous(), w_o.contiguous()

    @property
    def state_shape(self) -> tuple:
        return (self.heads, self.dim, self.vdim)

    def __call__(self, q, k, v, gate, a1, plan, state: torch.Tensor) -> torch.Tensor:
        from extensions_b200.tiny_llm_ext_b200 import blocks

        H = self.heads
        z = linear_wide(a1.contiguous(), self.w_a2)  # fp32 decay logits
        o = blocks.decay_scan(q.unflatten(1, (H, self.dim)), k.unflatten(1, (H, self.dim)), v.unflatten(1, (H, self.vdim)), z, self.a2_bias,
                              tau=self.tau, q_scale=self.dim ** -0.5, seq_info=plan.seq_info, state=state, max_tokens=plan.max_tokens)
        return linear_wide(blocks.head_norm_gate(o, self.norm_weight, self.eps, gate, act=1), self.w_o)

"""Lightning attention: linear attention with a fixed decay per head and a matrix of state per head.

Per token, with h the layer's normalised input (no biases):

* ``q = silu(W_q h)`` and ``k = silu(W_k h)`` in ``heads`` heads of ``dim``, ``v = silu(W_v h)`` in ``heads`` heads of ``vdim``;
* per head, with the head's constant ``decay``: ``S = decay S + k v^T``, ``o = S^T q`` (S ``[dim, vdim]``, no other factor; the
  read-out sees the current token's write);
* the heads' outputs side by side are divided by their common root mean square (``norm_eps``), times a weight
  ``[heads * vdim]``, times ``sigmoid(W_g h)``; then the output projection.

What a request carries from token to token is one float32 state slot, the heads' matrices, zero at the start.  The four
projections are one product; the activations, the recurrence, the norm and the gate are float32 (``csrc/lightning.cu``).
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import MIXERS, CacheNeed, LayerCache, Mixer, StateNeed, StepView, TensorDecl


@MIXERS.register("lightning_attention")
class LightningAttention(Mixer):
    takes_padding = True   # the kernel walks rows by their token ranges: rows without tokens and tokens without a row touch no state

    def __init__(self, width: int, n_heads: int, head_dim: int, value_dim: int, decay: Sequence[float], norm_eps: float,
                 names: Optional[Mapping[str, str]] = None) -> None:
        self.width, self.n_heads, self.head_dim, self.value_dim = int(width), int(n_heads), int(head_dim), int(value_dim)
        self.decay_values = tuple(float(d) for d in decay)
        if len(self.decay_values) != self.n_heads:
            raise ValueError(f"{self.n_heads} heads need {self.n_heads} decays, got {len(self.decay_values)}")
        if any(not 0.0 <= d <= 1.0 for d in self.decay_values):
            raise ValueError("a head's decay lies in [0, 1]")
        self.norm_eps = float(norm_eps)
        self.qk_size, self.v_size = self.n_heads * self.head_dim, self.n_heads * self.value_dim
        self.names = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "norm": "norm", **(names or {})}
        self.w_in = self.w_o = self.norm = self.decay = None

    def tensors(self) -> Sequence[TensorDecl]:
        n = self.names
        return [
            TensorDecl(n["q"], (self.qk_size, self.width)), TensorDecl(n["k"], (self.qk_size, self.width)),
            TensorDecl(n["v"], (self.v_size, self.width)), TensorDecl(n["gate"], (self.v_size, self.width)),
            TensorDecl(n["o"], (self.width, self.v_size)), TensorDecl(n["norm"], (self.v_size,), "vector"),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        # one product for all four projections: columns [q | k | v | gate] of its result
        self.w_in = torch.cat([tensors[n[key]] for key in ("q", "k", "v", "gate")], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.norm = tensors[n["norm"]].contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(device)

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size() + self.v_size * 4

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((self.qk_size * self.value_dim,), torch.float32))

    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        proj = ops.linear(h, self.w_in)
        mixed = ops.lightning_attention(proj, cache.state, step.q_start, step.slots, self.decay, self.norm, self.n_heads, self.head_dim,
                                        self.value_dim, step.num_rows, self.norm_eps, max_q=step.max_q)
        return ops.linear_for_residual(mixed, self.w_o)

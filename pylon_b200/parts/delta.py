"""The gated delta rule: a recurrent mixer with one matrix of state per head.

Per token, with h the layer's normalised input (no biases anywhere):

* ``q = W_q h`` and ``k = W_k h`` in ``kv_heads`` heads of ``dim``, ``v = W_v h`` in ``heads`` heads of ``vdim``; value
  head i uses query/key head ``i // (heads / kv_heads)``;
* each of q, k, v goes through a short causal convolution over time per channel (``taps`` wide, the last tap on the
  current token, zeros before the sequence starts) and then silu;
* q and k become unit vectors per head, ``x / sqrt(sum x^2 + unit_eps)``, q also times ``dim ** -0.5``;
* per head ``beta = sigmoid(W_b h)`` and the decay ``g = exp(-exp(A_log) * softplus(W_a h + dt_bias))``;
* the state S ``[dim, vdim]`` of a head: ``S = g S``; ``w = beta (v - S^T k)``; ``S = S + k w^T``; ``o = S^T q`` (the
  read-out sees the current token's write);
* ``o`` is divided by its root mean square over ``vdim`` (``norm_eps``), times a weight ``[vdim]`` shared by the heads,
  times ``silu(W_g h)``; then the output projection.

What a request carries from token to token is one float32 state slot: the heads' matrices and the convolution's last
``taps - 1`` inputs.  The six projections are one product; everything behind it that enters the recurrence is float32
(``csrc/delta_rule.cu``).
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import MIXERS, CacheNeed, LayerCache, Mixer, StateNeed, StepView, TensorDecl


@MIXERS.register("gated_delta")
class GatedDeltaRule(Mixer):
    takes_padding = True   # the kernels skip tokens without a row and rows without tokens: a padded step leaves no state touched that it should not

    def __init__(
        self,
        width: int,
        n_heads: int,
        n_kv_heads: int,
        head_dim: int,
        value_dim: int,
        conv_taps: int,
        norm_eps: float,
        unit_eps: float = 1e-6,
        names: Optional[Mapping[str, str]] = None,
    ) -> None:
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} value heads cannot share {n_kv_heads} query/key heads")
        if conv_taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.head_dim, self.value_dim, self.conv_taps = int(head_dim), int(value_dim), int(conv_taps)
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.qk_size, self.v_size = self.n_kv_heads * self.head_dim, self.n_heads * self.value_dim
        self.channels = 2 * self.qk_size + self.v_size
        self.names = {
            "q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b", "decay": "a",
            "a_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm", "o": "o", **(names or {}),
        }
        self.w_in = self.w_o = self.conv = self.a_log = self.dt_bias = self.norm = None

    # -- weights -------------------------------------------------------------------------
    def tensors(self) -> Sequence[TensorDecl]:
        n, taps = self.names, self.conv_taps
        return [
            TensorDecl(n["q"], (self.qk_size, self.width)), TensorDecl(n["k"], (self.qk_size, self.width)),
            TensorDecl(n["v"], (self.v_size, self.width)), TensorDecl(n["gate"], (self.v_size, self.width)),
            TensorDecl(n["decay"], (self.n_heads, self.width)), TensorDecl(n["beta"], (self.n_heads, self.width)),
            TensorDecl(n["o"], (self.width, self.v_size)),
            TensorDecl(n["q_conv"], (self.qk_size, taps), "vector", (0.0, 0.5)), TensorDecl(n["k_conv"], (self.qk_size, taps), "vector", (0.0, 0.5)),
            TensorDecl(n["v_conv"], (self.v_size, taps), "vector", (0.0, 0.5)),
            TensorDecl(n["a_log"], (self.n_heads,), "vector", (-1.0, 0.5)), TensorDecl(n["dt_bias"], (self.n_heads,), "vector", (0.0, 0.5)),
            TensorDecl(n["norm"], (self.value_dim,), "vector"),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        # one product for all six projections: columns [q | k | v | gate | a | b] of its result
        self.w_in = torch.cat([tensors[n[key]] for key in ("q", "k", "v", "gate", "decay", "beta")], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.conv = torch.cat([tensors[n[key]] for key in ("q_conv", "k_conv", "v_conv")], dim=0).t().contiguous()   # [taps, channels]
        self.a_log, self.dt_bias, self.norm = (tensors[n[key]].contiguous() for key in ("a_log", "dt_bias", "norm"))

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size() + self.conv.numel() * 4

    # -- state ---------------------------------------------------------------------------
    def state_floats(self) -> int:
        return self.n_heads * self.head_dim * self.value_dim + (self.conv_taps - 1) * self.channels

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((self.state_floats(),), torch.float32))

    # -- run -----------------------------------------------------------------------------
    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        proj = ops.linear(h, self.w_in)
        mixed = ops.gated_delta_rule(
            proj, self.conv, cache.state, step.token_row, step.q_start, step.slots, self.a_log, self.dt_bias, self.norm,
            self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim, step.num_rows, self.norm_eps, self.unit_eps,
        )
        return ops.linear_for_residual(mixed, self.w_o)

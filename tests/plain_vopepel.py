"""A plain, slow statement of the Vopepel design, one function per mechanism.

Everything here is written from the equations alone, token by token where the design is
sequential, on the CPU, in one dtype (float64 by default); it shares no code with
``pylon_b200``.  A model is a dict ``config`` (the keys of ``config.json``) and a dict
``weights`` (tensor name -> ``torch.Tensor``).

Notation: ``h`` is a ``[T, width]`` block of one sequence, ``T`` tokens from position 0.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch


# ---------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------
def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * weight; var is the mean squared deviation; no bias."""
    mean = x.mean(dim=-1, keepdim=True)
    centred = x - mean
    var = (centred * centred).mean(dim=-1, keepdim=True)
    return centred / torch.sqrt(var + eps) * weight


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last dimension (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Per-channel convolution over time: ``y[t, c] = sum_j taps[c, j] * x[t - (n - 1) + j, c]``
    with zeros before the start, so the last column weighs the current token."""
    count, n = x.shape[0], taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(count):
        for j in range(n):
            source = t - (n - 1) + j
            if source >= 0:
                out[t] += taps[:, j] * x[source]
    return out


# ---------------------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------------------
def clamped_glu(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ down.T


# ---------------------------------------------------------------------------------------
# attention in chunks of positions, scores soft-capped, values mixed with an earlier layer's
# ---------------------------------------------------------------------------------------
def visible(count: int, chunk: Optional[int]) -> torch.Tensor:
    """``[i, j]`` true where position i sees position j: j <= i, and in the same chunk of positions if there are chunks."""
    i = torch.arange(count)[:, None]
    j = torch.arange(count)[None, :]
    seen = j <= i
    if chunk is not None:
        seen = seen & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    return seen


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, softcap: Optional[float],
                   chunk: Optional[int]) -> torch.Tensor:
    """``q [T, heads, dim]``, ``k [T, kv_heads, dim]``, ``v [T, kv_heads, vdim]`` of one sequence -> ``[T, heads, vdim]``."""
    count, heads = q.shape[0], q.shape[1]
    group = heads // k.shape[1]
    seen = visible(count, chunk)
    out = torch.zeros(count, heads, v.shape[2], dtype=q.dtype)
    for head in range(heads):
        kv = head // group
        scores = (q[:, head] @ k[:, kv].T) * scale
        if softcap:
            scores = softcap * torch.tanh(scores / softcap)
        scores = scores.masked_fill(~seen, float("-inf"))
        out[:, head] = torch.softmax(scores, dim=-1) @ v[:, kv]
    return out


def chunked_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: Mapping, eps: float,
                      v_first: Optional[torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns (mixer output ``[T, width]``, the values this layer keeps ``[T, kv_heads, vdim]``).
    ``v_first``: the values of the first value-mixing layer, or ``None`` if this layer is it
    (or mixes nothing)."""
    count = h.shape[0]
    heads, kv_heads, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    chunk = p["mask"]["size"] if p.get("mask") else None
    q = (h @ w["q"].T).view(count, heads, dim)
    k = (h @ w["k"].T).view(count, kv_heads, dim)
    v = (h @ w["v"].T).view(count, kv_heads, vdim)
    q = rms_unit(q, eps) * w["q.norm"]
    k = rms_unit(k, eps) * w["k.norm"]
    if v_first is not None:
        lam = w["vmix"]
        v = (1 - lam) * v + lam * v_first
    out = attention_core(q, k, v, p["scale"], p.get("softcap"), chunk)
    return out.reshape(count, heads * vdim) @ w["o"].T, v


# ---------------------------------------------------------------------------------------
# gated delta rule
# ---------------------------------------------------------------------------------------
def delta_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor,
                     states: Optional[list] = None) -> torch.Tensor:
    """``q, k [T, kv_heads, dim]``, ``v [T, heads, vdim]``, ``decay, beta [T, heads]`` -> read-outs ``[T, heads, vdim]``.
    Per head: S = g S; w = beta (v - S^T k); S = S + k w^T; o = S^T q.  ``states`` (a list) receives the final S of each head."""
    count, heads, vdim = v.shape
    kv_heads, dim = k.shape[1], k.shape[2]
    out = torch.zeros(count, heads, vdim, dtype=v.dtype)
    for head in range(heads):
        kv = head // (heads // kv_heads)
        state = torch.zeros(dim, vdim, dtype=v.dtype)
        for t in range(count):
            state = decay[t, head] * state
            write = beta[t, head] * (v[t, head] - state.T @ k[t, kv])
            state = state + torch.outer(k[t, kv], write)
            out[t, head] = state.T @ q[t, kv]
        if states is not None:
            states.append(state)
    return out


def gated_delta(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: Mapping, eps: float) -> torch.Tensor:
    count = h.shape[0]
    heads, kv_heads, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).view(count, kv_heads, dim)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).view(count, kv_heads, dim)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).view(count, heads, vdim)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)                                     # [T, heads]
    decay = torch.exp(-torch.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))
    gate = silu(h @ w["g"].T).view(count, heads, vdim)
    out = delta_recurrence(q, k, v, decay, beta)
    out = rms_unit(out, eps) * w["norm"] * gate
    return out.reshape(count, heads * vdim) @ w["o"].T


# ---------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------
def sub(weights: Mapping[str, torch.Tensor], prefix: str) -> dict[str, torch.Tensor]:
    return {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens, dtype: torch.dtype = torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from position 0.  ``layers_out``, if a list, receives the
    residual stream (the sum of the streams, where there are several) after every layer."""
    weights = {name: tensor.to(dtype) if tensor.is_floating_point() else tensor for name, tensor in weights.items()}
    eps, mult = config["norm"]["eps"], config.get("residual_mult", 1.0)
    streams = config.get("streams")
    x = weights["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    xs = [x.clone() for _ in range(streams)] if streams else None
    v_first = None
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        mixer_w, p = sub(weights, prefix + "mix."), layer["mixer"]

        def mixer(h):
            nonlocal v_first
            if layer["type"] == "delta":
                return gated_delta(h, mixer_w, p, eps)
            mixes = bool(p.get("v_mix"))
            y, kept = chunked_attention(h, mixer_w, p, eps, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = kept
            return y

        def feed_forward(h):
            m = layer["mlp"]
            ff = sub(weights, prefix + "mlp.")
            return clamped_glu(h, ff["gate"], ff["up"], ff["down"], m["limit"])

        sublayers = [(1, mixer)] + ([(2, feed_forward)] if layer.get("mlp") else [])
        for number, function in sublayers:
            norm_w = weights[f"{prefix}norm{number}"]
            if xs is None:
                x = x + mult * function(layer_norm(x, norm_w, eps))
                continue
            w_in, w_out, w_mix = (weights[f"{prefix}hc{number}.{name}"] for name in ("in", "out", "mix"))
            u = sum(w_in[s] * xs[s] for s in range(streams))
            y = function(layer_norm(u, norm_w, eps))
            xs = [sum(w_mix[s, t] * xs[s] for s in range(streams)) + mult * w_out[t] * y for t in range(streams)]
        if layers_out is not None:
            layers_out.append(sum(xs) if xs is not None else x.clone())
    if xs is not None:
        x = sum(xs)
    return layer_norm(x, weights["final.norm"], eps) @ weights["head"].T

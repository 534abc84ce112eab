"""A plain, slow statement of the Fikerax design, one function per mechanism.

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
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last dimension (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: the unit-RMS vector times one plus the stored tensor."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def window_visible(count: int, window: int) -> torch.Tensor:
    """``[i, j]`` true where position i sees position j: itself and the ``window - 1`` positions before it."""
    i = torch.arange(count)[:, None]
    j = torch.arange(count)[None, :]
    return (j <= i) & (i - j < window)


# ---------------------------------------------------------------------------------------
# rotations
# ---------------------------------------------------------------------------------------
def base_frequencies(dims: int, base: float) -> torch.Tensor:
    i = torch.arange(dims // 2, dtype=torch.float64)
    return base ** (-2.0 * i / dims)


def wavelength_scaled(freq: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Long waves slowed by ``factor``, short ones kept, a linear blend between."""
    out = freq.clone()
    for i, f in enumerate(freq.tolist()):
        wave = 2.0 * math.pi / f
        if wave < original / high:
            out[i] = f
        elif wave > original / low:
            out[i] = f / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * f / factor + s * f
    return out


def yarn_scaled(freq: torch.Tensor, dims: int, base: float, factor: float, original: float, fast: float, slow: float) -> tuple[torch.Tensor, float]:
    """Frequencies blended by a ramp over the pair index, and the factor on cos and sin."""

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    out = freq.clone()
    for i, f in enumerate(freq.tolist()):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f / factor * ramp + f * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, gain: float = 1.0) -> torch.Tensor:
    """``x [T, heads, d]``: dimension i is turned together with dimension i + n, n = len(freq); the rest passes."""
    n = freq.shape[0]
    angle = positions.to(x.dtype)[:, None, None] * freq.to(x.dtype)[None, None, :]
    cos, sin = torch.cos(angle) * gain, torch.sin(angle) * gain
    out = x.clone()
    u, v = x[..., :n], x[..., n : 2 * n]
    out[..., :n] = u * cos - v * sin
    out[..., n : 2 * n] = v * cos + u * sin
    return out


def rotate_neighbours(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, gain: float = 1.0) -> torch.Tensor:
    """``x [T, heads, d]``: dimension 2i is turned together with dimension 2i + 1, i < len(freq); the rest passes."""
    n = freq.shape[0]
    angle = positions.to(x.dtype)[:, None, None] * freq.to(x.dtype)[None, None, :]
    cos, sin = torch.cos(angle) * gain, torch.sin(angle) * gain
    out = x.clone()
    u, v = x[..., 0 : 2 * n : 2], x[..., 1 : 2 * n : 2]
    out[..., 0 : 2 * n : 2] = u * cos - v * sin
    out[..., 1 : 2 * n : 2] = v * cos + u * sin
    return out


# ---------------------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------------------
def gated_ff(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


# ---------------------------------------------------------------------------------------
# softmax attention over a window, with or without a sink
# ---------------------------------------------------------------------------------------
def windowed_softmax(scores: torch.Tensor, window: int, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``scores [heads, T, T]`` -> weights; a sink adds ``exp(sink[h])`` to every denominator of head h."""
    count = scores.shape[-1]
    masked = scores.masked_fill(~window_visible(count, window)[None], -math.inf)
    if sink is None:
        return torch.softmax(masked, dim=-1)
    top = torch.maximum(masked.max(dim=-1, keepdim=True).values, sink[:, None, None])
    weights = torch.exp(masked - top)
    return weights / (weights.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


# ---------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------
def lightning_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mixer: Mapping, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head, token by token: ``S = decay S + k v^T``, ``o = S^T q``."""
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    count = h.shape[0]
    q = silu(h @ w[p + "q"].T).view(count, heads, dim)
    k = silu(h @ w[p + "k"].T).view(count, heads, dim)
    v = silu(h @ w[p + "v"].T).view(count, heads, vdim)
    state = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    decay = torch.tensor(mixer["decay"], dtype=h.dtype)
    out = torch.zeros(count, heads, vdim, dtype=h.dtype)
    for t in range(count):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    normed = rms_unit(out.reshape(count, heads * vdim), eps) * w[p + "norm"]
    return (normed * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def grouped_attention_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mixer: Mapping, eps: float) -> torch.Tensor:
    heads, groups, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    count = h.shape[0]
    positions = torch.arange(count)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(count, heads, dim)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(count, groups, dim)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(count, groups, vdim)
    rot = mixer["rot"]
    freq = base_frequencies(rot["dims"], rot["base"])
    if rot.get("scaling") is not None:
        s = rot["scaling"]
        freq = wavelength_scaled(freq, s["factor"], s["low"], s["high"], s["original"])
    q = rms_unit(rotate_halves(q, positions, freq), eps)
    k = rms_unit(rotate_halves(k, positions, freq), eps)
    share = heads // groups
    k = k.repeat_interleave(share, dim=1)
    v = v.repeat_interleave(share, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * mixer["scale"]
    weights = windowed_softmax(scores, mixer["mask"]["size"])
    out = torch.einsum("hij,jhv->ihv", weights, v).reshape(count, heads * vdim)
    return out @ w[p + "o"].T


def latent_attention_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mixer: Mapping, eps: float) -> torch.Tensor:
    """Keys and values come per head out of one latent row per token; one turned key part is shared by all heads."""
    heads, dim, rot_dim, vdim, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    count = h.shape[0]
    positions = torch.arange(count)
    cq = rms_unit(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(count, heads, dim + rot_dim)
    q_plain, q_turn = q[..., :dim], q[..., dim:]
    down = h @ w[p + "dkv"].T
    c = rms_unit(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_turn = down[:, rank:].view(count, 1, rot_dim)
    rot = mixer["rot"]
    freq = base_frequencies(rot["dims"], rot["base"])
    gain = 1.0
    if rot.get("scaling") is not None:
        s = rot["scaling"]
        freq, gain = yarn_scaled(freq, rot["dims"], rot["base"], s["factor"], s["original"], s["fast"], s["slow"])
    q_turn = rotate_neighbours(q_turn, positions, freq, gain)
    k_turn = rotate_neighbours(k_turn, positions, freq, gain)
    k_plain = (c @ w[p + "uk"].T).view(count, heads, dim)
    v = (c @ w[p + "uv"].T).view(count, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_turn, k_turn[:, 0])) * mixer["scale"]
    weights = windowed_softmax(scores, mixer["mask"]["size"], w[p + "sink"].to(h.dtype))
    out = torch.einsum("hij,jhv->ihv", weights, v).reshape(count, heads * vdim)
    return out @ w[p + "o"].T


MIXERS = {"lightning": lightning_mixer, "attention": grouped_attention_mixer, "latent_attention": latent_attention_mixer}


# ---------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------
def run_order(config: Mapping) -> list[tuple[int, bool]]:
    """(layer, whether the embedding output is added before it) for every layer run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(i, False) for i in range(count)]
    order = [(i, False) for i in range(loop["start"])]
    for turn in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, turn > 0 and i == loop["start"]))
    order += [(i, False) for i in range(loop["stop"], count)]
    return order


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens, dtype: torch.dtype = torch.float64, taps: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from position 0; ``taps`` receives the residual stream after every layer run."""
    w = {name: tensor.to(dtype) if tensor.is_floating_point() else tensor for name, tensor in weights.items()}
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x0 = w["embed"][ids] * config["embedding"]["scale"]
    x = x0.clone()
    for index, add_embedding in run_order(config):
        layer, p = config["layers"][index], f"l{index}."
        if add_embedding:
            x = x + x0
        x = x + MIXERS[layer["type"]](offset_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        if layer["mlp"] is not None:
            x = x + gated_ff(offset_norm(x, w[p + "norm2"], eps), w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
        if taps is not None:
            taps.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T

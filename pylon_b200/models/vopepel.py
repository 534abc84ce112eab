"""Vopepel as a :class:`ModelSpec`.

The configuration lists the layers; each is a ``hyper_prenorm`` block (layer norm without bias, the sublayers'
outputs times ``residual_mult``, the residual stream in ``streams`` copies where the configuration says so) around
either a ``gated_delta`` mixer or ``gqa_attention`` without a position encoding - per-head RMS norm of q and k, scores
scaled and soft-capped, attention inside chunks of positions, values of their own width, mixed from the second
value-mixing layer on with the first one's - and a ``clamped_glu`` feed-forward, or none.  Tensor names:
``embed``, ``l<i>.norm1`` / ``norm2``, ``l<i>.mix.*``, ``l<i>.mlp.gate`` / ``up`` / ``down``, ``l<i>.hc1.*`` / ``hc2.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from typing import Optional

from pylon_b200.config.model_config import VopepelConfig
from pylon_b200.parts.spec import LayerSpec, ModelSpec, PartSpec

FF_ALPHA = 1.702      # the gated unit's sigmoid is taken of alpha * g
UNIT_EPS = 1e-6       # under the root when q and k of the delta rule are made unit vectors
MAX_POSITIONS = 1 << 30   # positions do not enter the model: no table limits a request's length


def vopepel_spec(config: VopepelConfig, max_positions: Optional[int] = None) -> ModelSpec:
    norm = PartSpec("layernorm", {"width": config.width, "eps": config.norm_eps, "weight_name": ""})
    layers = []
    seen_value_mix = False
    for index, layer in enumerate(config.layers):
        if layer.kind == "delta":
            mixer = PartSpec("gated_delta", {
                "width": config.width, "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim,
                "value_dim": layer.vdim, "conv_taps": layer.conv, "norm_eps": config.norm_eps, "unit_eps": UNIT_EPS,
            })
        else:
            value_mix = None
            if layer.v_mix:
                value_mix, seen_value_mix = ("mix" if seen_value_mix else "source"), True
            mixer = PartSpec("gqa_attention", {
                "width": config.width, "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim,
                "value_dim": layer.vdim, "qk_norm_eps": config.norm_eps, "scale": layer.scale, "softcap": layer.softcap,
                "chunk": layer.chunk, "value_mix": value_mix,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "value_mix": "vmix"},
            })
        feed_forward = None
        if layer.ff is not None:
            feed_forward = PartSpec("clamped_glu", {
                "width": config.width, "intermediate": layer.ff, "limit": layer.ff_limit, "alpha": FF_ALPHA,
                "names": {"gate": "gate", "up": "up", "down": "down"},
            })
        block = PartSpec("hyper_prenorm", {
            "mixer": mixer, "feed_forward": feed_forward, "mixer_norm": norm, "ffn_norm": norm if feed_forward is not None else None,
            "streams": config.streams, "residual_mult": config.residual_mult,
        })
        layers.append(LayerSpec(f"l{index}.", block))
    return ModelSpec(
        width=config.width,
        vocab_size=config.vocab,
        max_positions=MAX_POSITIONS if max_positions is None else int(max_positions),
        embedding_name="embed",
        lm_head_name="head",
        final_norm=norm,
        final_norm_prefix="final.norm",
        layers=tuple(layers),
        order=tuple(range(len(layers))),
        eos_token_ids=config.eos_token_ids,
        streams=config.streams or 1,
    )

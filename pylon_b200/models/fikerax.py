"""Fikerax as a :class:`ModelSpec`.

The configuration lists the layers; each is a ``hyper_prenorm`` block over the plain residual sum (RMS norms whose stored
weight is the weight less one) around a ``lightning_attention``, ``gqa_attention`` or ``latent_attention`` mixer and a
``swiglu`` feed-forward, or none.  The grouped-query attention has biases, rotates the first ``rot.dims`` elements of a
head in halves with frequencies scaled by wavelength, makes q and k unit vectors (no weight) behind the rotation, and
attends inside a sliding window; the latent attention rotates its shared key part and the queries' like part in
neighbouring pairs with YaRN-scaled frequencies, attends inside a window and has a sink per head.  The run order
repeats the loop's span of layers, each pass with caches of its own, the embedding added again before every pass but
the first.  Tensor names: ``embed``, ``l<i>.norm1`` / ``norm2``, ``l<i>.mix.*``, ``l<i>.mlp.gate`` / ``up`` / ``down``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from typing import Optional

from pylon_b200.config.model_config import FikeraxConfig, FikeraxLayer, RotarySpec
from pylon_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec

NORM_OFFSET = 1.0          # a norm multiplies by one plus the tensor the checkpoint holds
MAX_POSITIONS = 1 << 20    # no learnt table limits a request's length; the rotation tables are cut to the engine's longest context


def _rotation(rot: Optional[RotarySpec], head_dim: int, positions: int, scaling_kind: str, layout: str) -> Optional[PartSpec]:
    if rot is None:
        return None
    scaling = None if rot.scaling is None else {"kind": scaling_kind, **dict(rot.scaling)}
    return PartSpec("rope", {"head_dim": head_dim, "theta": rot.base, "max_positions": positions, "rotary_dim": rot.dims,
                             "scaling": scaling, "layout": layout})


def _mixer(config: FikeraxConfig, layer: FikeraxLayer, positions: int) -> PartSpec:
    if layer.kind == "lightning":
        return PartSpec("lightning_attention", {
            "width": config.width, "n_heads": layer.heads, "head_dim": layer.dim, "value_dim": layer.vdim, "decay": layer.decay,
            "norm_eps": config.norm_eps,
        })
    if layer.kind == "attention":
        return PartSpec("gqa_attention", {
            "width": config.width, "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim, "value_dim": layer.vdim,
            "position": _rotation(layer.rot, layer.dim, positions, "wavelength", "halves"), "qk_norm_eps": config.norm_eps,
            "qk_norm": "after", "qk_norm_weight": False, "bias": True, "bias_suffix": ".b", "window": layer.window, "scale": layer.scale,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"},
        })
    return PartSpec("latent_attention", {
        "width": config.width, "n_heads": layer.heads, "head_dim": layer.dim, "rot_dim": layer.rot_dim, "value_dim": layer.vdim,
        "q_rank": layer.q_rank, "kv_rank": layer.kv_rank, "norm_eps": config.norm_eps, "scale": layer.scale,
        "position": _rotation(layer.rot, layer.rot_dim, positions, "yarn", "neighbours"), "window": layer.window, "sink": True,
    })


def fikerax_spec(config: FikeraxConfig, max_positions: Optional[int] = None) -> ModelSpec:
    positions = MAX_POSITIONS if max_positions is None else int(max_positions)
    norm = PartSpec("rmsnorm", {"width": config.width, "eps": config.norm_eps, "weight_name": "", "offset": NORM_OFFSET})
    layers = []
    for index, layer in enumerate(config.layers):
        feed_forward = None
        if layer.ff is not None:
            feed_forward = PartSpec("swiglu", {"width": config.width, "intermediate": layer.ff, "names": {"gate": "gate", "up": "up", "down": "down"}})
        block = PartSpec("hyper_prenorm", {
            "mixer": _mixer(config, layer, positions), "feed_forward": feed_forward, "mixer_norm": norm,
            "ffn_norm": norm if feed_forward is not None else None,
        })
        layers.append(LayerSpec(f"l{index}.", block))
    return ModelSpec(
        width=config.width,
        vocab_size=config.vocab,
        max_positions=positions,
        embedding_name="embed",
        lm_head_name="head",
        final_norm=norm,
        final_norm_prefix="final.norm",
        layers=tuple(layers),
        order=tuple(RunSpec(index, add_embedding=again) for index, again in config.run_order()),
        eos_token_ids=config.eos_token_ids,
        embedding_scale=config.embedding_scale,
    )

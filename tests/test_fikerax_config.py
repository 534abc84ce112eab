"""Fikerax without a GPU: its configuration, the model description built from it (the looped run order, tensor names, what
each run keeps), the scaled rotation frequencies, and the cache manager over its windowed groups and state slots."""
from __future__ import annotations

import copy
import json
import math

import pytest
import torch

import plain_fikerax as plain
from pylon_b200.cache.manager import CacheManager
from pylon_b200.config.model_config import ConfigError, FikeraxConfig
from pylon_b200.config.registry import ARCHITECTURES, architecture_of, read_config
from pylon_b200.models.decoder import DecoderModel
from pylon_b200.parts import POSITION_ENCODINGS, PartSpec
from pylon_b200.parts.base import KVNeed, StateNeed

CONFIG = {
    "architecture": "Fikerax", "vocab": 50, "width": 24, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-6},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "scale": 0.5, "mask": {"size": 12},
                                        "rot": {"dims": 6, "base": 5000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "lightning", "mixer": {"heads": 3, "dim": 8, "vdim": 12, "decay": [0.5, 0.9, 1.0]}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 10, "kv_rank": 12, "scale": 0.3, "mask": {"size": 7},
                                               "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 4.0, "original": 32, "fast": 16.0, "slow": 1.0}}},
         "mlp": {"kind": "dense", "ff": 32}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.25, "mask": {"size": 5},
                                        "rot": {"dims": 8, "base": 100.0, "scaling": None}}, "mlp": None},
    ],
}


def test_the_configuration_reads_every_key_and_writes_it_back():
    config = FikeraxConfig.from_dict(CONFIG)
    assert (config.vocab, config.width, config.embedding_scale, config.norm_eps) == (50, 24, 2.5, 1e-6)
    assert (config.loop_start, config.loop_stop, config.loop_times) == (1, 3, 3)
    first, second, third, fourth = config.layers
    assert (first.kind, first.heads, first.kv_heads, first.dim, first.vdim, first.scale, first.window, first.ff) == ("attention", 4, 2, 8, 4, 0.5, 12, 40)
    assert (first.rot.dims, first.rot.base, dict(first.rot.scaling)) == (6, 5000.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64.0})
    assert (second.kind, second.decay, second.ff) == ("lightning", (0.5, 0.9, 1.0), None)
    assert (third.kind, third.rot_dim, third.q_rank, third.kv_rank, third.window) == ("latent_attention", 4, 10, 12, 7)
    assert dict(third.rot.scaling) == {"factor": 4.0, "original": 32.0, "fast": 16.0, "slow": 1.0}
    assert fourth.rot.scaling is None
    assert config.to_dict() == CONFIG
    assert FikeraxConfig.from_dict(json.loads(json.dumps(config.to_dict()))) == config


def test_the_registry_finds_the_architecture(tmp_path):
    assert architecture_of(CONFIG) is ARCHITECTURES["Fikerax"]
    (tmp_path / "config.json").write_text(json.dumps(CONFIG))
    architecture, config = read_config(tmp_path)
    assert architecture.name == "Fikerax" and isinstance(config, FikeraxConfig)


@pytest.mark.parametrize("loop,order", [
    ({"start": 1, "stop": 3, "times": 3}, [0, 1, 2, -1, 2, -1, 2, 3]),
    ({"start": 0, "stop": 4, "times": 2}, [0, 1, 2, 3, -0.5, 1, 2, 3]),
    ({"start": 3, "stop": 4, "times": 2}, [0, 1, 2, 3, -3]),
    ({"start": 2, "stop": 2, "times": 5}, [0, 1, 2, 3]),
    ({"start": 0, "stop": 2, "times": 1}, [0, 1, 2, 3]),
    (None, [0, 1, 2, 3]),
])
def test_the_run_order_repeats_the_loop_and_marks_where_the_embedding_comes_in_again(loop, order):
    """A negative entry: that layer runs with the embedding added before it (-0.5 stands for layer 0)."""
    data = dict(CONFIG, loop=loop)
    config = FikeraxConfig.from_dict(data)
    spec = ARCHITECTURES["Fikerax"].build_spec(config, 64)
    got = [(-run.layer if run.layer else -0.5) if run.add_embedding else run.layer for run in spec.order]
    assert got == order
    assert [(run.layer, run.add_embedding) for run in spec.order] == plain.run_order(data)
    assert all(run.cache_of is None for run in spec.order)   # every pass has caches of its own


def test_the_description_names_the_checkpoints_tensors():
    config = FikeraxConfig.from_dict(CONFIG)
    spec = ARCHITECTURES["Fikerax"].build_spec(config, 64)
    assert spec.embedding_scale == 2.5 and spec.streams == 1
    decls = DecoderModel(spec).tensor_decls()
    shapes = {name: tuple(decl.shape) for name, decl in decls.items()}
    assert shapes == {
        "embed": (50, 24), "head": (50, 24), "final.norm": (24,),
        "l0.norm1": (24,), "l0.norm2": (24,), "l0.mix.q": (32, 24), "l0.mix.q.b": (32,), "l0.mix.k": (16, 24), "l0.mix.k.b": (16,),
        "l0.mix.v": (8, 24), "l0.mix.v.b": (8,), "l0.mix.o": (24, 16), "l0.mlp.gate": (40, 24), "l0.mlp.up": (40, 24), "l0.mlp.down": (24, 40),
        "l1.norm1": (24,), "l1.mix.q": (24, 24), "l1.mix.k": (24, 24), "l1.mix.v": (36, 24), "l1.mix.g": (36, 24), "l1.mix.o": (24, 36), "l1.mix.norm": (36,),
        "l2.norm1": (24,), "l2.norm2": (24,), "l2.mix.dq": (10, 24), "l2.mix.dq.norm": (10,), "l2.mix.uq": (24, 10), "l2.mix.dkv": (16, 24),
        "l2.mix.dkv.norm": (12,), "l2.mix.uk": (16, 12), "l2.mix.uv": (12, 12), "l2.mix.sink": (2,), "l2.mix.o": (24, 12),
        "l2.mlp.gate": (32, 24), "l2.mlp.up": (32, 24), "l2.mlp.down": (24, 32),
        "l3.norm1": (24,), "l3.mix.q": (16, 24), "l3.mix.q.b": (16,), "l3.mix.k": (16, 24), "l3.mix.k.b": (16,), "l3.mix.v": (16, 24),
        "l3.mix.v.b": (16,), "l3.mix.o": (24, 16),
    }
    assert all(decls[name].role == "vector" for name in ("l0.norm1", "l0.mix.q.b", "l1.mix.norm", "l2.mix.sink", "l2.mix.dq.norm", "final.norm"))


def test_what_each_run_keeps_between_steps():
    config = FikeraxConfig.from_dict(CONFIG)
    model = DecoderModel(ARCHITECTURES["Fikerax"].build_spec(config, 64))
    needs = model.cache_needs()
    assert len(needs) == 8
    assert needs[0].kv == KVNeed(2, 8, 12, 4, None) and needs[0].state is None
    for run in (1, 3, 5):
        assert needs[run].kv is None and needs[run].state == StateNeed((3 * 8 * 12,), torch.float32)
    for run in (2, 4, 6):   # one row of kv_rank + rot_dim numbers per token, no value rows
        assert needs[run].kv == KVNeed(1, 16, 7, 0, None) and needs[run].state is None
    assert needs[7].kv == KVNeed(2, 8, 5, None, None)
    # the three passes of the latent layer share a group of pages; the windows give pages back as they pass
    manager = CacheManager(needs, [None] * 8, page_size=4, num_pages=40, max_requests=2)
    assert [len(group.runs) for group in manager.groups] == [1, 3, 1]
    request = manager.open("a", 100)
    for _ in range(10):
        manager.prepare([(request, 5)])
        manager.commit(request)
    assert [len(request.held(g)) for g in range(3)] == [4, 2, 2]   # 50 tokens held, pages of 4: the token at position 50 reads back to 39, 44 and 46
    manager.close(request)
    manager.check()
    assert manager.free_pages() == [40, 40, 40]


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 3), "cannot be grouped"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5, 0.9]), "decay"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5, 0.9, 1.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 6), "rot_dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 10), "exceeds"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 5), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "experts"), "not built"),
    (lambda c: c["loop"].__setitem__("stop", 5), "loop"),
    (lambda c: c["loop"].__setitem__("start", 3) or c["loop"].__setitem__("stop", 2), "loop"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "eps"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_what_the_configuration_refuses(change, message):
    data = copy.deepcopy(CONFIG)
    change(data)
    with pytest.raises(ConfigError, match=message):
        FikeraxConfig.from_dict(data)


def test_scaled_frequencies_follow_the_plain_formulas():
    for dims, base in ((6, 5000.0), (64, 10000.0), (16, 1000000.0)):
        plain_freq = plain.base_frequencies(dims, base)
        wave = POSITION_ENCODINGS.build(PartSpec("rope", {"head_dim": dims, "theta": base, "max_positions": 8, "rotary_dim": dims,
                                                          "scaling": {"kind": "wavelength", "factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}))
        freq, gain = wave.frequencies()
        torch.testing.assert_close(freq, plain.wavelength_scaled(plain_freq, 8.0, 1.0, 4.0, 64), rtol=1e-12, atol=0)
        assert gain == 1.0
        yarn = POSITION_ENCODINGS.build(PartSpec("rope", {"head_dim": dims, "theta": base, "max_positions": 8, "rotary_dim": dims, "layout": "neighbours",
                                                          "scaling": {"kind": "yarn", "factor": 8.0, "original": 48, "fast": 32.0, "slow": 1.0}}))
        freq, gain = yarn.frequencies()
        want, want_gain = plain.yarn_scaled(plain_freq, dims, base, 8.0, 48, 32.0, 1.0)
        torch.testing.assert_close(freq, want, rtol=1e-12, atol=0)
        assert gain == want_gain == 0.1 * math.log(8.0) + 1.0
    # all three bands of the wavelength scaling occur at 64 dims: kept, slowed, blended
    plain_freq = plain.base_frequencies(64, 10000.0)
    scaled = plain.wavelength_scaled(plain_freq, 8.0, 1.0, 4.0, 64)
    ratio = scaled / plain_freq
    assert float(ratio.max()) == 1.0 and abs(float(ratio.min()) - 0.125) < 1e-12 and bool(((ratio > 0.126) & (ratio < 0.999)).any())

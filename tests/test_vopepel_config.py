"""Vopepel without a GPU: its configuration, the model description built from it, and the cache manager's handling of
attention in chunks of positions."""
from __future__ import annotations

import json

import pytest
import torch

from pylon_b200.cache.manager import CacheManager, group_page_counts
from pylon_b200.config.model_config import ConfigError, VopepelConfig
from pylon_b200.config.registry import ARCHITECTURES, architecture_of, read_config
from pylon_b200.models.decoder import DecoderModel
from pylon_b200.parts.base import CacheNeed, KVNeed, StateNeed

CONFIG = {
    "architecture": "Vopepel", "vocab": 50, "width": 24, "norm": {"eps": 1e-6}, "residual_mult": 0.25, "streams": 2,
    "layers": [
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 4}, "mlp": {"kind": "dense", "ff": 40, "limit": 3.0}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "scale": 0.5, "softcap": 9.0, "mask": {"size": 12}, "v_mix": True}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 4, "scale": 0.25, "v_mix": True}, "mlp": {"kind": "dense", "ff": 32, "limit": 1.0}},
    ],
}


def test_the_configuration_reads_every_key_and_writes_it_back():
    config = VopepelConfig.from_dict(CONFIG)
    assert (config.vocab, config.width, config.streams, config.residual_mult, config.norm_eps) == (50, 24, 2, 0.25, 1e-6)
    first, second, third = config.layers
    assert (first.kind, first.heads, first.kv_heads, first.dim, first.vdim, first.conv, first.ff, first.ff_limit) == ("delta", 4, 2, 8, 12, 4, 40, 3.0)
    assert (second.kind, second.chunk, second.softcap, second.scale, second.v_mix, second.ff) == ("attention", 12, 9.0, 0.5, True, None)
    assert (third.chunk, third.softcap, third.v_mix) == (None, None, True)
    assert VopepelConfig.from_dict(config.to_dict()) == config
    assert VopepelConfig.from_dict(json.loads(json.dumps(config.to_dict()))) == config


def test_the_registry_finds_the_architecture_by_its_singular_key(tmp_path):
    assert architecture_of(CONFIG) is ARCHITECTURES["Vopepel"]
    (tmp_path / "config.json").write_text(json.dumps(CONFIG))
    architecture, config = read_config(tmp_path)
    assert architecture.name == "Vopepel" and isinstance(config, VopepelConfig)


def test_no_streams_key_means_the_plain_residual_sum():
    data = {key: value for key, value in CONFIG.items() if key != "streams"}
    config = VopepelConfig.from_dict(data)
    assert config.streams is None
    spec = ARCHITECTURES["Vopepel"].build_spec(config, 64)
    assert spec.streams == 1
    names = set(DecoderModel(spec).tensor_decls())
    assert not any(".hc" in name for name in names)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 3), "cannot be grouped"),
    (lambda c: c["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 8), "mix values"),
    (lambda c: c.__setitem__("streams", 9), "streams"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "experts"), "not built"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configurations_that_are_refused(change, message):
    data = json.loads(json.dumps(CONFIG))
    change(data)
    with pytest.raises(ConfigError, match=message):
        VopepelConfig.from_dict(data)


def test_the_description_names_every_tensor_with_its_shape():
    config = VopepelConfig.from_dict(CONFIG)
    spec = ARCHITECTURES["Vopepel"].build_spec(config, 128)
    model = DecoderModel(spec)
    decls = {name: tuple(decl.shape) for name, decl in model.tensor_decls().items()}
    assert decls["embed"] == (50, 24) and decls["head"] == (50, 24) and decls["final.norm"] == (24,)
    assert decls["l0.mix.q"] == (16, 24) and decls["l0.mix.v"] == (48, 24) and decls["l0.mix.q.conv"] == (16, 4) and decls["l0.mix.v.conv"] == (48, 4)
    assert decls["l0.mix.A_log"] == (4,) and decls["l0.mix.norm"] == (12,) and decls["l0.mix.o"] == (24, 48) and decls["l0.mix.b"] == (4, 24)
    assert decls["l1.mix.q"] == (32, 24) and decls["l1.mix.v"] == (8, 24) and decls["l1.mix.o"] == (24, 16) and decls["l1.mix.vmix"] == ()
    assert decls["l1.mix.q.norm"] == (8,) and decls["l2.mix.k.norm"] == (16,)
    assert decls["l0.hc1.mix"] == (2, 2) and decls["l0.hc2.in"] == (2,) and decls["l2.hc2.out"] == (2,)
    assert "l1.norm2" not in decls and "l1.hc2.in" not in decls and "l1.mlp.gate" not in decls     # a layer without feed-forward
    assert decls["l2.mlp.down"] == (24, 32)
    needs = model.cache_needs()
    assert needs[0] == CacheNeed(state=StateNeed((4 * 8 * 12 + 3 * (16 + 16 + 48),), torch.float32))
    assert needs[1].kv == KVNeed(2, 8, None, 4, 12) and needs[2].kv == KVNeed(2, 16, None, 4, None)
    # the first mixing layer is the source, the later one mixes
    assert model.blocks[1].mixer.value_mix == "source" and model.blocks[2].mixer.value_mix == "mix"


def test_pages_of_chunks_that_have_passed_go_back():
    need = KVNeed(2, 8, None, 4, chunk=12)
    assert [need.first_needed(n) for n in (0, 5, 11, 12, 13, 23, 24, 40)] == [0, 0, 0, 12, 12, 12, 24, 36]
    cache = CacheManager([CacheNeed(kv=need), CacheNeed(state=StateNeed((3,)))], [None, None], page_size=4, num_pages=8, max_requests=2)
    request = cache.open("a", 100)
    held = []
    for tokens in (5, 6, 1, 1, 9, 2, 17, 1):
        cache.prepare([(request, tokens)])
        cache.commit(request)
        cache.check()
        first = need.first_needed(request.length)
        table = request.tables[0]
        # every page that holds a position some later token can read is there; every page wholly before them is gone
        for page, physical in enumerate(table):
            assert (physical >= 0) == ((page + 1) * 4 > first), (request.length, page, table)
        held.append(len(request.held(0)))
    assert max(held) <= 5     # a chunk of 12 positions and a step of 17 tokens never need the whole request's pages
    assert cache.groups[0].pool.acquired_total > cache.groups[0].pool.num_pages     # pages were used again
    cache.close(request)
    assert cache.free_pages() == [8]


def test_a_chunked_group_is_given_only_what_its_chunks_need():
    chunked, full = CacheNeed(kv=KVNeed(2, 8, None, 4, chunk=16)), CacheNeed(kv=KVNeed(2, 8))
    counts = group_page_counts([chunked, full], page_size=8, pool_tokens=4096, max_requests=2, longest_request=2048, max_step_tokens=32)
    assert counts[full.kv] == 512 and counts[chunked.kv] < 20

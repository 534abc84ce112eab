"""Fikerax on the GPU against the plain implementation (``plain_fikerax``): each mechanism alone, then whole models of
several made-up shapes stepped through the engine under every cutting, and generation through the scheduler.

The models' weights are drawn here, larger than a trained model's and with the attention sharpened, so that a key that is
wrongly seen or missed, a sink that is left out, a state that is lost and an embedding that is not fed in again all move
the logits by much more than the tolerance."""
from __future__ import annotations

import json
import math

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import plain_fikerax as plain
import trace_tools
from test_parts_gpu import step_view

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


# ---------------------------------------------------------------------------------------
# made-up models
# ---------------------------------------------------------------------------------------
def lightning_layer(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def attention_layer(heads, kv_heads, dim, vdim, scale, window, rot_dims, base=10000.0, scaling=(4.0, 1.0, 4.0, 64), ff=None):
    rot = {"dims": rot_dims, "base": base,
           "scaling": None if scaling is None else dict(zip(("factor", "low", "high", "original"), scaling))}
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}, "rot": rot},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def latent_layer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base=10000.0, scaling=(8.0, 32, 16.0, 1.0), ff=None):
    rot = {"dims": rot_dim, "base": base,
           "scaling": None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling))}
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                                                  "scale": scale, "mask": {"size": window}, "rot": rot},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model(vocab, width, layers, loop, embedding_scale=1.0, eps=1e-5):
    return {"architecture": "Fikerax", "vocab": vocab, "width": width, "embedding": {"scale": embedding_scale}, "norm": {"eps": eps},
            "loop": None if loop is None else dict(zip(("start", "stop", "times"), loop)), "layers": layers}


CONFIGS = {
    # the loop in the middle, twice; all three mixers; heads only partly rotated; values wider and narrower than keys; a
    # latent narrower than the heads it feeds; windows that are no multiple of the page; a decay of exactly one
    "mix": model(97, 48, [
        attention_layer(6, 2, 16, 8, 0.6, window=9, rot_dims=10, ff=80),
        lightning_layer(3, 20, 12, (0.5, 0.9, 1.0)),
        latent_layer(3, 12, 8, 20, 24, 16, 0.35, window=13, ff=72),
        attention_layer(2, 1, 24, 40, 0.4, window=30, rot_dims=24, scaling=(8.0, 1.0, 2.0, 16)),
        lightning_layer(1, 40, 5, (0.97,), ff=64),
    ], loop=(1, 3, 2), embedding_scale=3.0),
    # no loop at all, rotations without scaling, one head everywhere, windows of one and two tokens, pages of 4
    "plain": model(61, 40, [
        latent_layer(1, 16, 4, 16, 8, 36, 0.3, window=2, scaling=None, ff=48),
        attention_layer(1, 1, 16, 16, 0.5, window=1, rot_dims=2, scaling=None),
        lightning_layer(2, 8, 8, (0.8, 0.3), ff=40),
        attention_layer(3, 3, 8, 12, 0.9, window=50, rot_dims=8, ff=40),
    ], loop=None),
    # the whole model is the loop, three times; head size 64 with pages of 64: the bfloat16 steps run the tensor-core attention
    # under a window; the latent as wide as a real one's smaller kin
    "looped": model(130, 64, [
        attention_layer(4, 2, 64, 64, 0.16, window=70, rot_dims=64, scaling=(8.0, 1.0, 4.0, 128), ff=96),
        latent_layer(4, 32, 16, 32, 48, 128, 0.2, window=100, scaling=(4.0, 64, 8.0, 1.0), ff=96),
        lightning_layer(2, 64, 64, (0.9, 0.99)),
    ], loop=(0, 3, 3), embedding_scale=8.0),
    # a width at which the decode steps' products come as partial sums over slices of k and prompts run on the tcgen05 kernels;
    # the loop at the end; values narrower than keys (kept padded in bfloat16) under biases
    "wide": model(300, 1024, [
        lightning_layer(4, 128, 128, (0.7, 0.9, 0.97, 0.995), ff=512),
        attention_layer(8, 4, 64, 32, 0.16, window=80, rot_dims=32, ff=512),
        latent_layer(8, 64, 32, 64, 256, 128, 0.12, window=150, ff=512),
        attention_layer(4, 2, 128, 128, 0.08, window=200, rot_dims=128, scaling=(8.0, 1.0, 4.0, 256)),
    ], loop=(2, 4, 2), embedding_scale=32.0),
    # no attention at all: no page is ever held, the state slots are all a request has
    "lightning_only": model(45, 32, [
        lightning_layer(2, 32, 16, (0.9, 0.6), ff=48),
        lightning_layer(4, 8, 12, (0.99, 0.5, 0.0, 1.0)),
    ], loop=(0, 1, 2)),
}
PAGE_SIZES = {"mix": 8, "plain": 4, "looped": 64, "wide": 64, "lightning_only": 16}
LENGTHS = {"mix": (61, 23, 5, 38, 1, 44, 17), "plain": (70, 9, 35, 2, 41), "looped": (230, 70, 3, 129), "lightning_only": (40, 3, 25, 31, 1), "wide": (330, 45, 150)}


def draw_weights(config, seed):
    """Weights of a made-up model: matrices N(0, 1/in) times a gain, norm tensors near zero where the design adds one to them
    so, sinks of both signs, biases that matter."""
    g = torch.Generator().manual_seed(seed)
    rand = lambda *shape: torch.randn(*shape, generator=g)
    width = config["width"]
    # embedding rows of size one over the scale, so that the stream starts near unit size whatever the scale is
    w = {"embed": rand(config["vocab"], width) / config["embedding"]["scale"], "final.norm": 0.1 * rand(width),
         "head": rand(config["vocab"], width) / math.sqrt(width)}
    matrix = lambda out, inner, gain=1.0: rand(out, inner) * gain / math.sqrt(inner)
    for index, layer in enumerate(config["layers"]):
        p, name = layer["mixer"], f"l{index}."
        heads, dim, vdim = p["heads"], p["dim"], p["vdim"]
        w[name + "norm1"] = 0.1 * rand(width)
        if layer["type"] == "lightning":
            w[name + "mix.q"], w[name + "mix.k"] = matrix(heads * dim, width, 1.5), matrix(heads * dim, width, 1.5)
            w[name + "mix.v"], w[name + "mix.g"] = matrix(heads * vdim, width, 1.5), matrix(heads * vdim, width, 2.0)
            w[name + "mix.norm"] = 1 + 0.2 * rand(heads * vdim)
            w[name + "mix.o"] = matrix(width, heads * vdim)
        elif layer["type"] == "attention":
            groups = p["kv_heads"]
            for key, rows in (("q", heads * dim), ("k", groups * dim), ("v", groups * vdim)):
                w[name + f"mix.{key}"] = matrix(rows, width)
                w[name + f"mix.{key}.b"] = 0.5 * rand(rows)
            w[name + "mix.o"] = matrix(width, heads * vdim)
        else:
            rot_dim, q_rank, kv_rank = p["rot_dim"], p["q_rank"], p["kv_rank"]
            w[name + "mix.dq"], w[name + "mix.dq.norm"] = matrix(q_rank, width), 1 + 0.2 * rand(q_rank)
            w[name + "mix.uq"] = matrix(heads * (dim + rot_dim), q_rank, 2.5)
            w[name + "mix.dkv"], w[name + "mix.dkv.norm"] = matrix(kv_rank + rot_dim, width, 1.5), 1 + 0.2 * rand(kv_rank)
            w[name + "mix.uk"], w[name + "mix.uv"] = matrix(heads * dim, kv_rank, 2.5), matrix(heads * vdim, kv_rank)
            w[name + "mix.sink"] = 1.5 * rand(heads)
            w[name + "mix.o"] = matrix(width, heads * vdim)
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            w[name + "norm2"] = 0.1 * rand(width)
            w[name + "mlp.gate"], w[name + "mlp.up"], w[name + "mlp.down"] = matrix(ff, width, 2.0), matrix(ff, width, 2.0), matrix(width, ff)
    return {key: value.to(torch.bfloat16).contiguous() for key, value in w.items()}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config, weights as stored)."""
    made = {}
    for seed, (name, config) in enumerate(CONFIGS.items()):
        folder = tmp_path_factory.mktemp("fikerax_" + name)
        # seeds at which no position of the test requests is ill-conditioned: rounding the mixers' weights to 9 bits moves no
        # position's logits by more than 0.03 of their spread in the plain implementation (hard attention over a window of one
        # or two tokens and a norm over few numbers can make a single position ten times as touchy)
        weights = draw_weights(config, 600 + seed)
        save_file(weights, str(folder / "model.safetensors"), metadata={"format": "pt"})
        (folder / "config.json").write_text(json.dumps(config))
        made[name] = (folder, config, weights)
    return made


def make_requests(config, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": [int(t) for t in rng.integers(0, config["vocab"], size=n)] for i, n in enumerate(lengths)}


def plain_logits(config, weights, requests):
    return {name: plain.forward(config, weights, tokens).numpy() for name, tokens in requests.items()}


def engine_for(folder, dtype, page_size, pool, slots=4, **options):
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    return Engine(folder, EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=pool, max_context=pool, max_batch_size=slots, **options))


def assert_logits(got, want, dtype, what):
    """float32: every logit within 2e-4 of the logits' spread.  bfloat16: per position the root mean square of the
    difference within 0.08 of the spread and the largest within 0.35 - a key, a sink or a state that is lost shows as
    several times that."""
    spread = float(np.std(np.concatenate(list(want.values()))))
    for name in want:
        difference = got[name] - want[name]
        largest = np.abs(difference).max(axis=1)
        if dtype == "float32":
            worst = int(largest.argmax())
            assert largest[worst] <= 2e-4 * spread, f"{what}: request {name}, position {worst}: off by {largest[worst]:.3g} (spread of the logits {spread:.3g})"
        else:
            rms = np.sqrt((difference ** 2).mean(axis=1))
            worst = int(rms.argmax())
            assert rms[worst] <= 0.08 * spread and largest.max() <= 0.35 * spread, \
                f"{what}: request {name}, position {worst}: rms {rms[worst]:.3g}, largest {largest.max():.3g} (spread of the logits {spread:.3g})"


# ---------------------------------------------------------------------------------------
# whole models under every cutting
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_gives_the_plain_logits(models, name, dtype):
    folder, config, weights = models[name]
    requests = make_requests(config, LENGTHS[name], seed=7)
    want = plain_logits(config, weights, requests)
    page = PAGE_SIZES[name]
    cuttings = {
        "whole": trace_tools.whole(requests),
        "tail one by one": trace_tools.tail_one_by_one(requests, tail=30),
        "changing portions": trace_tools.changing_portions(requests),
        "mixed": trace_tools.mixed(requests, seed=3, max_live=3, decode_tail=9, max_portion=19),
    }
    for what, steps in cuttings.items():
        pool = trace_tools.pool_tokens(steps, round_to=page)     # no page to spare: pages and slots are used again
        engine = engine_for(folder, dtype, page, pool, slots=3)
        got = trace_tools.run_in_process(engine, steps)
        assert_logits(got, want, dtype, f"{name}, {what}, {dtype}")
        assert engine.cache.free_slots() == 3 and all(group.pool.free_count == group.pool.num_pages for group in engine.cache.groups)
        assert (len(engine.cache.groups) == 0) == (name == "lightning_only")
        del engine


def test_layer_by_layer_in_32_bit(models):
    """The residual stream after every layer run, the loop's passes included."""
    from pylon_b200.engine import StepEntry

    folder, config, weights = models["mix"]
    tokens = make_requests(config, (37,), seed=5)["r0"]
    want: list = []
    plain.forward(config, weights, tokens, taps=want)
    engine = engine_for(folder, "float32", 8, 64)
    taps: list = []
    forward = engine.model.forward
    engine.model.forward = lambda step, caches: forward(step, caches, taps)
    request = engine.open("a", len(tokens))
    engine.step([StepEntry(request, tokens, [0])])
    assert len(taps) == len(plain.run_order(config)) == 7
    for index, (got, expected) in enumerate(zip(taps, want)):
        torch.testing.assert_close(got.double().cpu(), expected, rtol=1e-4, atol=1e-4 * float(expected.abs().max()), msg=lambda m: f"run {index}: {m}")


def test_long_decoding_across_many_windows_and_pages(models):
    """A short prompt, then 200 tokens one by one: every window and many pages pass, the pool holds only what the windows
    need, the lightning state is carried 200 times."""
    folder, config, weights = models["mix"]
    requests = make_requests(config, (212,), seed=11)
    want = plain_logits(config, weights, requests)
    steps = trace_tools.tail_one_by_one(requests, tail=200)
    for dtype in ("float32", "bfloat16"):
        engine = engine_for(folder, dtype, 8, 216)
        got = trace_tools.run_in_process(engine, steps)
        assert_logits(got, want, dtype, f"long decoding, {dtype}")


def test_the_replay_program_runs_the_model(models, tmp_path):
    folder, config, weights = models["plain"]
    requests = make_requests(config, (33, 12, 20), seed=2)
    want = plain_logits(config, weights, requests)
    steps = trace_tools.mixed(requests, seed=1, max_live=2, decode_tail=5, max_portion=9)
    got = trace_tools.run_program(folder, "float32", steps, tmp_path / "out", extra_args=("--page-size", "4"))
    assert_logits(got, want, "float32", "bin/trace_run")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["mix", "looped"])
def test_greedy_generation_through_the_scheduler(models, name, graphs):
    """Several prompts through ``Engine.generate`` with a small prompt budget and few slots: every generated token is the
    arg-max of the plain logits of its own prefix."""
    from pylon_b200.sampling.params import SamplingParams

    folder, config, weights = models[name]
    prompts = list(make_requests(config, (19, 3, 40, 11, 27, 8), seed=13).values())
    new_tokens = 12
    # with graphs, decode steps replay at their batch size and steps with prompt portions padded to captured sizes (rows
    # without tokens, tokens without a row): nothing of the padding may touch a state slot or a page
    engine = engine_for(folder, "float32", PAGE_SIZES[name], 4 * 64, slots=3, prefill_chunk_size=16, cuda_graphs=graphs)
    results = engine.generate(prompts, SamplingParams(max_new_tokens=new_tokens, temperature=0.0, ignore_eos=True))
    for prompt, result in zip(prompts, results):
        assert len(result.output_ids) == new_tokens
        sequence = list(prompt) + list(result.output_ids)
        logits = plain.forward(config, weights, sequence[:-1])
        for place in range(len(prompt) - 1, len(sequence) - 1):
            row = logits[place]
            best = int(row.argmax())
            if sequence[place + 1] != best:   # a tie within rounding may go either way
                assert float(row[best] - row[sequence[place + 1]]) < 1e-3 * float(row.std()), f"token {place + 1} of a request is not the plain arg-max"
    engine.cache.check()
    assert engine.cache.free_slots() == 3
    if graphs:
        replays = engine.step_function.graphs.replays
        assert replays["decode"] > 0 and replays["padded"] > 0, replays


# ---------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------
def on(tensor, dtype=None):
    return tensor.to(device=DEVICE, dtype=dtype) if dtype is not None else tensor.to(DEVICE)


def tolerance(dtype):
    return dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)


def test_offset_norm_and_embedding_fed_in_again():
    from pylon_b200.kernels import ops
    from pylon_b200.parts import NORMS, PartSpec, ResidualStream

    g = torch.Generator().manual_seed(1)
    width, eps = 72, 1e-5
    norm = NORMS.build(PartSpec("rmsnorm", {"width": width, "eps": eps, "weight_name": "", "offset": 1.0}))
    stored = (0.3 * torch.randn(width, generator=g)).to(torch.bfloat16)
    norm.load({"": on(stored, torch.float32)}, torch.float32, torch.device(DEVICE))
    x = torch.randn(5, width, generator=g)
    got = norm.apply(ResidualStream(on(x).clone()))
    torch.testing.assert_close(got.double().cpu(), plain.offset_norm(x.double(), stored.double(), eps), rtol=1e-5, atol=1e-5)
    table = torch.randn(11, width, generator=g).to(torch.bfloat16)
    ids = torch.tensor([3, 10, 0, 3, 7], dtype=torch.int32)
    residual = on(x).clone()
    ops.embed_gather(on(ids), on(table), out=residual, scale=2.5, accumulate=True)
    torch.testing.assert_close(residual.cpu(), x + table.float()[ids.long()] * 2.5, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("kind", ["wavelength", "yarn", None])
def test_scaled_rotation_tables(kind):
    from pylon_b200.parts import POSITION_ENCODINGS, PartSpec

    dims, base, positions = 12, 500.0, 300
    scaling = {None: None, "wavelength": {"kind": "wavelength", "factor": 8.0, "low": 1.0, "high": 4.0, "original": 64},
               "yarn": {"kind": "yarn", "factor": 6.0, "original": 48, "fast": 8.0, "slow": 1.0}}[kind]
    part = POSITION_ENCODINGS.build(PartSpec("rope", {"head_dim": 16, "theta": base, "max_positions": positions, "rotary_dim": dims,
                                                      "scaling": scaling, "layout": "neighbours"}))
    cos, sin, rotary_dim, layout = part.tables(torch.device(DEVICE))
    freq, gain = plain.base_frequencies(dims, base), 1.0
    if kind == "wavelength":
        freq = plain.wavelength_scaled(freq, 8.0, 1.0, 4.0, 64)
    if kind == "yarn":
        freq, gain = plain.yarn_scaled(freq, dims, base, 6.0, 48, 8.0, 1.0)
    assert kind is None or not torch.equal(freq, plain.base_frequencies(dims, base))   # the scaling does something at these sizes
    angle = torch.arange(positions, dtype=torch.float64)[:, None] * freq[None, :]
    assert (rotary_dim, layout) == (dims, "neighbours") and part.rotary_table(torch.device(DEVICE)) is None
    torch.testing.assert_close(cos.double().cpu(), torch.cos(angle) * gain, rtol=0, atol=2e-5)
    torch.testing.assert_close(sin.double().cpu(), torch.sin(angle) * gain, rtol=0, atol=2e-5)


def paged(rows_of_requests, page_size, width, dtype, seed=0, spare=3):
    """Lays rows ``[tokens, width]`` of several requests into shuffled pages: (pages [P, 1, page_size, width], block table)."""
    counts = [-(-r.shape[0] // page_size) for r in rows_of_requests]
    total = sum(counts) + spare
    order = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    pages = torch.full((total, 1, page_size, width), float("nan"))
    table = torch.full((len(rows_of_requests), max(counts)), -1, dtype=torch.int32)
    for r, rows in enumerate(rows_of_requests):
        for logical in range(counts[r]):
            page = order.pop()
            table[r, logical] = page
            chunk = rows[logical * page_size : (logical + 1) * page_size]
            pages[page, 0, : chunk.shape[0]] = chunk
    return on(torch.nan_to_num(pages, nan=7.0), dtype), on(table)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout,rot,norm,weights,bias", [("halves", 10, "after", False, True), ("neighbours", 16, "before", True, False),
                                                          ("halves", 16, None, False, True), ("neighbours", 6, "after", True, True)])
def test_bias_rotation_norm_and_cache_write(layout, rot, norm, weights, bias, dtype):
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(rot)
    nq, nkv, d, dv, page, eps = 6, 2, 16, 24, 4, 1e-5
    q_lens, starts = (5, 1, 3), (0, 9, 2)
    step = step_view(q_lens, starts, dtype)
    tokens = sum(q_lens)
    columns = nq * d + nkv * d + nkv * dv
    qkv = torch.randn(tokens, columns, generator=g).to(dtype)
    b = torch.randn(columns, generator=g) if bias else None
    qw, kw = (1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)) if weights else (None, None)
    freq = plain.base_frequencies(rot, 100.0)
    positions = torch.tensor([s + i for n, s in zip(q_lens, starts) for i in range(n)])
    angle = torch.arange(16, dtype=torch.float64)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle).float(), torch.sin(angle).float()
    table = torch.tensor([[0, 2, -1], [5, 1, 3], [4, 6, -1]], dtype=torch.int32)
    k_pages = torch.zeros(8, nkv, page, d, device=DEVICE, dtype=dtype)
    v_pages = torch.zeros(8, nkv, page, dv, device=DEVICE, dtype=dtype)
    device_qkv = on(qkv).clone()
    ops.qkv_rotate_write(device_qkv, None if b is None else on(b), on(cos), on(sin), rot, layout, norm, None if qw is None else on(qw),
                         None if kw is None else on(kw), eps, step.positions, step.token_row, on(table), page, k_pages, v_pages, nq, nkv, d, dv)
    x = qkv.double() + (0 if b is None else b.double())
    turn = plain.rotate_halves if layout == "halves" else plain.rotate_neighbours

    def heads_of(block, count, weight):
        block = block.reshape(tokens, count, d)
        if norm == "before":
            block = plain.rms_unit(block, eps) * (1 if weight is None else weight.double())
        block = turn(block, positions, freq)
        if norm == "after":
            block = plain.rms_unit(block, eps) * (1 if weight is None else weight.double())
        return block

    want_q, want_k = heads_of(x[:, : nq * d], nq, qw), heads_of(x[:, nq * d : (nq + nkv) * d], nkv, kw)
    want_v = x[:, (nq + nkv) * d :].reshape(tokens, nkv, dv)
    torch.testing.assert_close(device_qkv[:, : nq * d].double().cpu().reshape(tokens, nq, d), want_q, **tolerance(dtype))
    token = 0
    for row, (n, s) in enumerate(zip(q_lens, starts)):
        for position in range(s, s + n):
            physical = int(table[row, position // page])
            torch.testing.assert_close(k_pages[physical, :, position % page].double().cpu(), want_k[token], **tolerance(dtype))
            torch.testing.assert_close(v_pages[physical, :, position % page].double().cpu(), want_v[token], **tolerance(dtype))
            token += 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_products_per_head_on_slices_of_wider_rows(dtype):
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(4)
    for tokens, heads, k, n, extra in ((7, 3, 20, 36, 5), (70, 2, 64, 8, 0), (1, 5, 12, 100, 3)):
        x = torch.randn(tokens, heads, k + extra, generator=g).to(dtype)
        w = (torch.randn(heads, n, k, generator=g) / math.sqrt(k)).to(dtype)
        out = torch.zeros(tokens, heads, n + 2, device=DEVICE, dtype=dtype)
        ops.linear_heads(on(x)[:, :, :k], on(w), out=out[:, :, :n])
        want = torch.einsum("thk,hnk->thn", x[:, :, :k].double(), w.double())
        torch.testing.assert_close(out[:, :, :n].double().cpu(), want, **tolerance(dtype))
        assert float(out[:, :, n:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim", [(3, 20, 12), (1, 100, 5), (2, 64, 130), (4, 32, 64), (2, 200, 40), (8, 128, 128)])
def test_lightning_attention_prefill_and_token_by_token(heads, dim, vdim, dtype):
    """Rows of unequal length in one call against the plain recurrence; then the same sequences in portions of three, two and one
    tokens that continue from their slots, slots in another order than rows, beside a slot no row names."""
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(heads * dim)
    lengths, eps = (37, 1, 18), 1e-5
    decay = torch.tensor([0.3, 0.9, 1.0, 0.99, 0.0, 0.7, 0.95, 0.5][:heads], dtype=torch.float32)
    norm_weight = 1 + 0.2 * torch.randn(heads * vdim, generator=g)
    columns = 2 * heads * dim + 2 * heads * vdim
    projs = [(torch.randn(n, columns, generator=g) * 1.2).to(dtype) for n in lengths]

    def plain_mixer(proj):
        p = proj.double()
        q, k = plain.silu(p[:, : heads * dim]).view(-1, heads, dim), plain.silu(p[:, heads * dim : 2 * heads * dim]).view(-1, heads, dim)
        v = plain.silu(p[:, 2 * heads * dim : 2 * heads * dim + heads * vdim]).view(-1, heads, vdim)
        gate = p[:, 2 * heads * dim + heads * vdim :]
        state = torch.zeros(heads, dim, vdim, dtype=torch.float64)
        out = torch.zeros(p.shape[0], heads, vdim, dtype=torch.float64)
        for t in range(p.shape[0]):
            state = decay.double()[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", state, q[t])
        return plain.rms_unit(out.reshape(-1, heads * vdim), eps) * norm_weight.double() * torch.sigmoid(gate), state

    wants = [plain_mixer(p) for p in projs]
    slots = [2, 0, 3]
    state = torch.zeros(5, heads * dim * vdim, device=DEVICE)
    state[1] = float("nan")   # a slot no row names is not touched
    step = step_view(lengths, (0, 0, 0), dtype)
    step.slots = torch.tensor(slots, device=DEVICE, dtype=torch.int32)
    got = ops.lightning_attention(on(torch.cat(projs)), state, step.q_start, step.slots, on(decay), on(norm_weight), heads, dim, vdim, len(lengths), eps)
    tol = tolerance(dtype)
    torch.testing.assert_close(got.double().cpu(), torch.cat([w[0] for w in wants]), **tol)
    for slot, (_, final) in zip(slots, wants):
        torch.testing.assert_close(state[slot].double().cpu().view(heads, vdim, dim).transpose(1, 2), final, rtol=1e-4, atol=1e-4)   # kept column by column
    assert bool(torch.isnan(state[1]).all())
    # the same in portions, continuing from other slots, which are used again
    state.zero_()
    slots = [1, 4, 0]
    cursors = [0, 0, 0]
    sizes = (3, 2, 1, 1, 2, 17, 1)
    turn = 0
    while any(c < n for c, n in zip(cursors, lengths)):
        rows = [r for r in range(3) if cursors[r] < lengths[r]]
        pieces = []
        for r in rows:
            size = min(sizes[(turn + r) % len(sizes)], lengths[r] - cursors[r])
            pieces.append((r, cursors[r], size))
        step = step_view([size for _, _, size in pieces], [start for _, start, _ in pieces], dtype)
        step.slots = torch.tensor([slots[r] for r, _, _ in pieces], device=DEVICE, dtype=torch.int32)
        proj = torch.cat([projs[r][start : start + size] for r, start, size in pieces])
        got = ops.lightning_attention(on(proj), state, step.q_start, step.slots, on(decay), on(norm_weight), heads, dim, vdim, len(pieces), eps)
        want = torch.cat([wants[r][0][start : start + size] for r, start, size in pieces])
        torch.testing.assert_close(got.double().cpu(), want, **tol)
        for r, _, size in pieces:
            cursors[r] += size
        turn += 1


def test_lightning_attention_walks_long_rows_in_segments():
    """In bfloat16 a row of 1,024 tokens or more is walked in segments side by side (a scan chains their states, a second walk adds
    what each token reads of the state before its segment): a long row that continues a request, beside a short row and a row of
    exactly one segment's length more than the threshold, against the plain recurrence; then each request goes on from its slot."""
    from pylon_b200.kernels import ops

    heads, dim, vdim, eps = 3, 40, 24, 1e-5
    g = torch.Generator().manual_seed(77)
    decay = torch.tensor([0.999, 0.9, 1.0])
    norm_weight = 1 + 0.2 * torch.randn(heads * vdim, generator=g)
    columns = 2 * heads * dim + 2 * heads * vdim
    lengths = (50 + 1700 + 9, 2 + 3 + 1, 1280 + 5)          # each request in its portions
    portions = ((50, 1700, 9), (2, 3, 1), (1280, 5))
    projs = [(torch.randn(n, columns, generator=g) * 1.2).to(torch.bfloat16) for n in lengths]

    def plain_mixer(proj):
        p = proj.double()
        q, k = plain.silu(p[:, : heads * dim]).view(-1, heads, dim), plain.silu(p[:, heads * dim : 2 * heads * dim]).view(-1, heads, dim)
        v = plain.silu(p[:, 2 * heads * dim : 2 * heads * dim + heads * vdim]).view(-1, heads, vdim)
        gate = p[:, 2 * heads * dim + heads * vdim :]
        state = torch.zeros(heads, dim, vdim, dtype=torch.float64)
        out = torch.zeros(p.shape[0], heads, vdim, dtype=torch.float64)
        for t in range(p.shape[0]):
            state = decay.double()[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", state, q[t])
        return plain.rms_unit(out.reshape(-1, heads * vdim), eps) * norm_weight.double() * torch.sigmoid(gate), state

    wants = [plain_mixer(p) for p in projs]
    state = torch.zeros(4, heads * dim * vdim, device=DEVICE)
    slots = [3, 0, 1]
    cursors = [0, 0, 0]
    for turn in range(3):
        rows = [r for r in range(3) if turn < len(portions[r])]
        sizes = [portions[r][turn] for r in rows]
        step = step_view(sizes, [cursors[r] for r in rows], torch.bfloat16)
        step.slots = torch.tensor([slots[r] for r in rows], device=DEVICE, dtype=torch.int32)
        proj = torch.cat([projs[r][cursors[r] : cursors[r] + size] for r, size in zip(rows, sizes)])
        got = ops.lightning_attention(on(proj), state, step.q_start, step.slots, on(decay), on(norm_weight), heads, dim, vdim, len(rows), eps, max_q=max(sizes))
        want = torch.cat([wants[r][0][cursors[r] : cursors[r] + size] for r, size in zip(rows, sizes)])
        torch.testing.assert_close(got.double().cpu(), want, rtol=3e-2, atol=3e-2)
        for r, size in zip(rows, sizes):
            cursors[r] += size
    for r in range(3):
        final = wants[r][1]
        torch.testing.assert_close(state[slots[r]].double().cpu().view(heads, vdim, dim).transpose(1, 2), final, rtol=2e-4, atol=2e-4 * float(final.abs().max()))


def test_lightning_attention_reads_back_a_value_written_long_ago():
    """With a decay of almost one, the last of 700 tokens must read the value that one early token wrote: its query is that
    token's key, every other key is small.  One prompt; the last 40 tokens one by one; portions."""
    from pylon_b200.kernels import ops

    heads, dim, vdim, count, early, eps = 2, 32, 16, 700, 5, 1e-5
    g = torch.Generator().manual_seed(9)
    columns = 2 * heads * dim + 2 * heads * vdim
    proj = torch.randn(count, columns, generator=g) * 0.05 - 8.0      # silu of about -8: every q, k, v tiny
    proj[:, 2 * heads * dim + heads * vdim :] = 0.0                   # gates at one half
    proj[early, heads * dim : 2 * heads * dim] = 4.0                  # the early token's key ...
    proj[early, 2 * heads * dim : 2 * heads * dim + heads * vdim] = torch.linspace(1.0, 5.0, heads * vdim)   # ... and its value
    proj[count - 1, : heads * dim] = 4.0                              # the last token asks for it
    decay = torch.tensor([0.9995, 0.999])
    norm_weight = torch.ones(heads * vdim)
    p = proj.double()
    q, k = plain.silu(p[:, : heads * dim]).view(-1, heads, dim), plain.silu(p[:, heads * dim : 2 * heads * dim]).view(-1, heads, dim)
    v = plain.silu(p[:, 2 * heads * dim : 2 * heads * dim + heads * vdim]).view(-1, heads, vdim)
    state = torch.zeros(heads, dim, vdim, dtype=torch.float64)
    for t in range(count):
        state = decay.double()[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
    read = torch.einsum("hdv,hd->hv", state, q[count - 1])
    share = (decay.double() ** (count - 1 - early))[:, None] * (k[early] * q[count - 1]).sum(-1)[:, None] * v[early]
    assert float((share / read).min()) > 0.9   # the early token is what the last one reads
    want = (plain.rms_unit(read.reshape(1, -1), eps) * 0.5)[0]
    for cutting in ((count,), (count - 40,) + (1,) * 40, (300, 2, 97, 3, 298)):
        device_state = torch.zeros(1, heads * dim * vdim, device=DEVICE)
        cursor = 0
        for size in cutting:
            step = step_view((size,), (cursor,), torch.float32)
            got = ops.lightning_attention(on(proj[cursor : cursor + size]), device_state, step.q_start, step.slots, on(decay), on(norm_weight),
                                          heads, dim, vdim, 1, eps)
            cursor += size
        torch.testing.assert_close(got[-1].double().cpu(), want, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,rank,rot_dim,window,page", [(3, 16, 8, 13, 4), (1, 36, 4, 2, 8), (8, 128, 32, 150, 64), (5, 64, 16, None, 16), (20, 32, 16, 33, 8),
                                                            (128, 64, 32, 90, 32)])
def test_attention_over_latent_rows_with_a_sink(heads, rank, rot_dim, window, page, dtype):
    """Every head reads the same row per token, values are the row's first columns, the denominator holds exp(sink); rows of
    unequal length, prompt portions that continue a request beside single tokens, pages shuffled."""
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(rank)
    width, scale = rank + rot_dim, 0.3
    lengths, news = (230, 41, 77), (60, 1, 77)     # tokens each request holds after the step; how many of them are new
    rows = [torch.randn(n, width, generator=g).to(dtype) for n in lengths]
    queries = [(torch.randn(n, heads, width, generator=g) * 1.5).to(dtype) for n in news]
    sinks = torch.randn(heads, generator=g) * 2.0
    pages, table = paged([r.float() for r in rows], page, width, dtype, seed=rank)
    step = step_view(news, [n - m for n, m in zip(lengths, news)], dtype)
    got = ops.paged_attention(on(torch.cat(queries)).view(-1, heads * width), pages, None, step.positions, step.token_row, step.q_start, step.kv_len,
                              table, heads, step.max_q, step.max_kv, window=window, scale=scale, sinks=on(sinks), values_in_keys=rank)
    wants = []
    for r, (n, m) in enumerate(zip(lengths, news)):
        keys, q = rows[r].double(), queries[r].double()
        scores = torch.einsum("ihd,jd->hij", q, keys) * scale                      # [heads, new, all]
        i = torch.arange(n - m, n)[:, None]
        j = torch.arange(n)[None, :]
        seen = (j <= i) & ((i - j < window) if window is not None else True)
        scores = scores.masked_fill(~seen[None], -math.inf)
        top = torch.maximum(scores.max(dim=-1, keepdim=True).values, sinks.double()[:, None, None])
        weights = torch.exp(scores - top)
        weights = weights / (weights.sum(dim=-1, keepdim=True) + torch.exp(sinks.double()[:, None, None] - top))
        wants.append(torch.einsum("hij,jv->ihv", weights, keys[:, :rank]).reshape(m, heads * rank))
    torch.testing.assert_close(got.double().cpu(), torch.cat(wants), **tolerance(dtype))
    # the keys of a tile cut over several blocks whose parts a second kernel combines (the tensor-core kernel's form for a few
    # decoded tokens), and the plain kernel in the tensor-core kernel's place
    for options in (dict(num_splits=3), dict(num_splits=7), dict(force_simple=True)):
        other = ops.paged_attention(on(torch.cat(queries)).view(-1, heads * width), pages, None, step.positions, step.token_row, step.q_start, step.kv_len,
                                    table, heads, step.max_q, step.max_kv, window=window, scale=scale, sinks=on(sinks), values_in_keys=rank, **options)
        torch.testing.assert_close(other.double().cpu(), torch.cat(wants), **tolerance(dtype))
    # without the sinks the result differs by far more than the tolerance: the test sees a sink that is left out
    bare = ops.paged_attention(on(torch.cat(queries)).view(-1, heads * width), pages, None, step.positions, step.token_row, step.q_start, step.kv_len,
                               table, heads, step.max_q, step.max_kv, window=window, scale=scale, values_in_keys=rank)
    assert float((bare.double().cpu() - torch.cat(wants)).abs().max()) > 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["latent", "grouped"])
def test_a_key_that_stands_out_just_inside_and_just_outside_the_window(kind, dtype):
    """One key far larger than the rest, with a value of its own: queries up to window - 1 tokens behind it are dominated by
    it, the next ones must not see it - in a prompt, token by token, and in a portion that starts right at the edge; the key
    sits on a page border, the pages are shuffled."""
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(5)
    count, window, page, special = 200, 37, 16, 95       # the key's last query is at 131, the first that must miss it at 132
    if kind == "latent":
        heads, rank, rot_dim = 4, 32, 16
        width, dv = rank + rot_dim, rank
        rows = torch.randn(count, width, generator=g) * 0.3
        rows[special] = 0.0
        rows[special, :rank] = torch.linspace(-4.0, 4.0, rank)
        rows[special, rank:] = 3.0
        queries = torch.randn(count, heads, width, generator=g) * 0.3
        queries[:, :, rank:] += 1.0                      # every query leans towards the special key's last columns
        values = rows[:, :rank]
        pages, table = paged([rows], page, width, dtype, seed=3)
        value_pages = None
        options = dict(values_in_keys=rank, sinks=on(torch.full((heads,), -2.0)))
        sink = -2.0
    else:
        heads, width, dv = 4, 64, 64
        rows = torch.randn(count, width, generator=g) * 0.3
        rows[special] = 3.0
        values = torch.randn(count, dv, generator=g) * 0.3
        values[special] = torch.linspace(-4.0, 4.0, dv)
        queries = torch.randn(count, heads, width, generator=g) * 0.3 + 0.25
        pages, table = paged([rows], page, width, dtype, seed=3)
        value_pages, _ = paged([values], page, dv, dtype, seed=3)
        options, sink = {}, None
    scale = 0.5
    q, keys, vals = queries.to(dtype).double(), rows.to(dtype).double(), values.to(dtype).double()
    scores = torch.einsum("ihd,jd->hij", q, keys) * scale
    scores = scores.masked_fill(~plain.window_visible(count, window)[None], -math.inf)
    weights = plain.windowed_softmax(scores, window, None if sink is None else torch.full((heads,), sink, dtype=torch.float64))
    want = torch.einsum("hij,jv->ihv", weights, vals).reshape(count, heads * dv)
    inside = weights[:, special : special + window, special]
    assert float(inside.min()) > 0.8 and float(weights[:, special + window :, special].max()) == 0.0

    def run(cutting):
        outs, cursor = [], 0
        for size in cutting:
            step = step_view((size,), (cursor,), dtype)
            outs.append(ops.paged_attention(on(queries[cursor : cursor + size].to(dtype)).view(size, heads * width), pages, value_pages, step.positions,
                                            step.token_row, step.q_start, step.kv_len, table, heads, step.max_q, step.max_kv, window=window,
                                            scale=scale, **options))
            cursor += size
        return torch.cat(outs).double().cpu()

    edge = special + window
    for cutting in ((count,), (edge - 3,) + (1,) * 6 + (count - edge - 3,), (edge - 1, 1, count - edge), (edge, count - edge), (special + 1, 2, count - special - 3)):
        torch.testing.assert_close(run(cutting), want, **tolerance(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["latent", "grouped", "lightning"])
def test_each_mixer_alone_against_its_plain_statement(name, dtype):
    """A mixer part from its normalised input to its delta for the stream: a prompt in one step, then the same in portions."""
    from pylon_b200.parts import MIXERS, PartSpec
    from pylon_b200.parts.base import LayerCache

    g = torch.Generator().manual_seed(21)
    width, eps, count, page = 56, 1e-5, 45, 8
    rand = lambda *shape: torch.randn(*shape, generator=g)
    matrix = lambda out, inner, gain=1.0: (rand(out, inner) * gain / math.sqrt(inner)).to(torch.bfloat16)
    if name == "latent":
        mixer = {"heads": 3, "dim": 12, "rot_dim": 6, "vdim": 10, "q_rank": 20, "kv_rank": 14, "scale": 0.4, "mask": {"size": 11},
                 "rot": {"dims": 6, "base": 300.0, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}}}
        w = {"dq": matrix(20, width), "dq.norm": (1 + 0.2 * rand(20)).to(torch.bfloat16), "uq": matrix(3 * 18, 20, 2.0), "dkv": matrix(20, width, 1.5),
             "dkv.norm": (1 + 0.2 * rand(14)).to(torch.bfloat16), "uk": matrix(36, 14, 2.0), "uv": matrix(30, 14), "sink": rand(3).to(torch.bfloat16),
             "o": matrix(width, 30)}
        spec = PartSpec("latent_attention", {
            "width": width, "n_heads": 3, "head_dim": 12, "rot_dim": 6, "value_dim": 10, "q_rank": 20, "kv_rank": 14, "norm_eps": eps, "scale": 0.4,
            "window": 11, "sink": True, "position": PartSpec("rope", {"head_dim": 6, "theta": 300.0, "max_positions": 64, "rotary_dim": 6, "layout": "neighbours",
                                                                       "scaling": {"kind": "yarn", "factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}})})
        oracle = plain.latent_attention_mixer
    elif name == "grouped":
        mixer = {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.7, "mask": {"size": 9},
                 "rot": {"dims": 8, "base": 300.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}}}
        w = {"q": matrix(48, width), "k": matrix(24, width), "v": matrix(40, width), "o": matrix(width, 80),
             "q.b": rand(48).to(torch.bfloat16), "k.b": rand(24).to(torch.bfloat16), "v.b": rand(40).to(torch.bfloat16)}
        spec = PartSpec("gqa_attention", {
            "width": width, "n_heads": 4, "n_kv_heads": 2, "head_dim": 12, "value_dim": 20, "qk_norm_eps": eps, "qk_norm": "after", "qk_norm_weight": False,
            "bias": True, "window": 9, "scale": 0.7, "names": {"q": "q", "k": "k", "v": "v", "o": "o"},
            "position": PartSpec("rope", {"head_dim": 12, "theta": 300.0, "max_positions": 64, "rotary_dim": 8,
                                          "scaling": {"kind": "wavelength", "factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}})})
        oracle = plain.grouped_attention_mixer
    else:
        mixer = {"heads": 3, "dim": 10, "vdim": 14, "decay": [0.9, 0.5, 0.99]}
        w = {"q": matrix(30, width, 1.5), "k": matrix(30, width, 1.5), "v": matrix(42, width, 1.5), "g": matrix(42, width, 2.0), "o": matrix(width, 42),
             "norm": (1 + 0.2 * rand(42)).to(torch.bfloat16)}
        spec = PartSpec("lightning_attention", {"width": width, "n_heads": 3, "head_dim": 10, "value_dim": 14, "decay": [0.9, 0.5, 0.99], "norm_eps": eps})
        oracle = plain.lightning_mixer
    part = MIXERS.build(spec)
    declared = {d.name: d for d in part.tensors()}
    assert set(declared) == set(w) and all(tuple(w[k].shape) == tuple(declared[k].shape) for k in w)
    part.load({k: on(v, torch.float32 if declared[k].role == "vector" else dtype) for k, v in w.items()}, dtype, torch.device(DEVICE))
    h = rand(count, width).to(dtype)
    want = oracle(h.double(), {"mix." + k: v.double() for k, v in w.items()}, "mix.", mixer, eps)
    need = part.cache_need()
    for cutting in ((count,), (20, 2, 1, 1, 13, 8)):
        cache = LayerCache(page_size=page)
        if need.kv is not None:
            cache.k_pages = torch.zeros(7, need.kv.n_kv_heads, page, need.kv.head_dim, device=DEVICE, dtype=dtype)
            cache.v_pages = torch.zeros(7, need.kv.n_kv_heads, page, need.kv.value_width, device=DEVICE, dtype=dtype) if need.kv.value_width else None
            cache.block_table = torch.tensor([[4, 0, 6, 2, 5, 1]], device=DEVICE, dtype=torch.int32)
        if need.state is not None:
            cache.state = torch.zeros(2, *need.state.shape, device=DEVICE)
        outs, cursor = [], 0
        for size in cutting:
            step = step_view((size,), (cursor,), dtype)
            step.slots = torch.tensor([1], device=DEVICE, dtype=torch.int32)
            out = part.forward(on(h[cursor : cursor + size]), step, cache)
            outs.append(out.sum(dim=0) if out.dim() == 3 else out)
            cursor += size
        got = torch.cat(outs).double().cpu()
        spread = float(want.std())
        limit = 0.06 * spread if dtype == torch.bfloat16 else 1e-4 * spread
        assert float((got - want).abs().max()) <= limit, f"{name}, {cutting}: off by {float((got - want).abs().max()):.3g} of {spread:.3g}"

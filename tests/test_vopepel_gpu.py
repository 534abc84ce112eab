"""Vopepel on the GPU against the plain implementation (``plain_vopepel``): each mechanism alone, then whole models
of several made-up shapes stepped through the engine under every cutting, and generation through the scheduler.

The models' weights are drawn here, larger than a trained model's and with the attention sharpened, so that a key that
is wrongly seen or missed, a state that is lost and a stream that is mixed wrongly all move the logits by much more
than the tolerance."""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import plain_vopepel as plain
import trace_tools
from test_parts_gpu import step_view

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


# ---------------------------------------------------------------------------------------
# made-up models
# ---------------------------------------------------------------------------------------
def delta_layer(heads, kv_heads, dim, vdim, conv, ff=None, limit=1.5):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def attention_layer(heads, kv_heads, dim, vdim, scale, chunk=None, softcap=None, v_mix=False, ff=None, limit=1.5):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    if softcap is not None:
        mixer["softcap"] = softcap
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


CONFIGS = {
    # several streams, grouped heads in both mixers, values wider and narrower than keys, a layer without feed-forward,
    # chunks that are no multiple of the page, value mixing over three layers
    "streams3": {"architecture": "Vopepel", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 0.7, "streams": 3, "layers": [
        attention_layer(6, 2, 16, 8, 0.3, chunk=10, softcap=6.0, v_mix=True, ff=80),
        delta_layer(4, 2, 16, 24, 4, ff=72),
        attention_layer(4, 2, 24, 8, 0.2, chunk=7, softcap=4.0, v_mix=True),
        delta_layer(2, 2, 12, 8, 2, ff=64, limit=0.8),
        attention_layer(2, 2, 8, 8, 0.4, chunk=10, softcap=6.0, v_mix=True, ff=56),
    ]},
    # the plain residual sum, attention over everything without a cap, no value mixing, one head, a convolution of one tap
    "plain": {"architecture": "Vopepel", "vocab": 61, "width": 40, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "layers": [
        delta_layer(1, 1, 20, 36, 1, ff=48, limit=3.0),
        attention_layer(1, 1, 16, 16, 0.25),
        attention_layer(3, 1, 16, 24, 0.25, chunk=33, ff=40),
        delta_layer(3, 1, 8, 8, 5),
    ]},
    # one stream kept as hyper-connections, head size 64 with pages of 64, one mixing layer only (its weight is unused)
    "one_stream": {"architecture": "Vopepel", "vocab": 130, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.4, "streams": 1, "layers": [
        delta_layer(2, 1, 64, 64, 3, ff=96),
        attention_layer(4, 2, 64, 64, 0.125, chunk=64, softcap=10.0, v_mix=True, ff=96),
        attention_layer(2, 2, 64, 32, 0.125, chunk=48, softcap=10.0, ff=96),
    ]},
    # a width at which the decode steps' products come as partial sums over slices of k and prompts run on the tcgen05 kernels;
    # values narrower than keys (kept padded in bfloat16) mixed into a layer of another head size; head sizes 64 and 128
    "wide": {"architecture": "Vopepel", "vocab": 300, "width": 1024, "norm": {"eps": 1e-5}, "residual_mult": 0.6, "streams": 2, "layers": [
        delta_layer(4, 2, 64, 64, 4, ff=512),
        attention_layer(8, 4, 64, 32, 0.125, chunk=80, softcap=15.0, v_mix=True, ff=512),
        attention_layer(4, 4, 32, 32, 0.18, chunk=112, softcap=15.0, v_mix=True),
        attention_layer(4, 2, 128, 128, 0.09, chunk=200, softcap=25.0, ff=512),
    ]},
    # no attention at all: no page is ever held, the state slots are all a request has
    "delta_only": {"architecture": "Vopepel", "vocab": 45, "width": 32, "norm": {"eps": 1e-5}, "residual_mult": 0.9, "streams": 2, "layers": [
        delta_layer(2, 1, 32, 16, 3, ff=48),
        delta_layer(4, 4, 8, 12, 2),
    ]},
}
PAGE_SIZES = {"streams3": 8, "plain": 4, "one_stream": 64, "delta_only": 16, "wide": 64}


def draw_weights(config, seed):
    """Weights of a made-up model: matrices N(0, 1/in) times a gain, norm weights around 1 (q/k norms around 3: sharp
    attention), stream routes near the identity, decays that forget within tens of tokens."""
    g = torch.Generator().manual_seed(seed)
    rand = lambda *shape: torch.randn(*shape, generator=g)
    width, streams = config["width"], config.get("streams")
    w = {"embed": rand(config["vocab"], width), "final.norm": 1 + 0.1 * rand(width), "head": rand(config["vocab"], width) / math.sqrt(width)}
    matrix = lambda out, inner, gain=1.0: rand(out, inner) * gain / math.sqrt(inner)
    for index, layer in enumerate(config["layers"]):
        p, name = layer["mixer"], f"l{index}."
        heads, kv_heads, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
        w[name + "norm1"] = 1 + 0.1 * rand(width)
        if layer["type"] == "delta":
            for key, rows in (("q", kv_heads * dim), ("k", kv_heads * dim), ("v", heads * vdim)):
                w[name + f"mix.{key}"] = matrix(rows, width, 1.5)
                w[name + f"mix.{key}.conv"] = rand(rows, p["conv"]) * 0.6
            w[name + "mix.g"] = matrix(heads * vdim, width)
            w[name + "mix.b"] = matrix(heads, width, 2.0)
            w[name + "mix.a"] = matrix(heads, width, 2.0)
            w[name + "mix.A_log"] = rand(heads) * 0.5 - 1.5
            w[name + "mix.dt_bias"] = rand(heads) * 0.5
            w[name + "mix.norm"] = 1 + 0.1 * rand(vdim)
            w[name + "mix.o"] = matrix(width, heads * vdim)
        else:
            w[name + "mix.q"] = matrix(heads * dim, width)
            w[name + "mix.k"] = matrix(kv_heads * dim, width)
            w[name + "mix.v"] = matrix(kv_heads * vdim, width)
            w[name + "mix.q.norm"] = 3 + 0.3 * rand(dim)
            w[name + "mix.k.norm"] = 3 + 0.3 * rand(dim)
            w[name + "mix.o"] = matrix(width, heads * vdim)
            if p.get("v_mix"):
                w[name + "mix.vmix"] = torch.tensor(0.35) + 0.1 * rand(())
        sublayers = [1]
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            w[name + "norm2"] = 1 + 0.1 * rand(width)
            w[name + "mlp.gate"], w[name + "mlp.up"], w[name + "mlp.down"] = matrix(ff, width, 2.0), matrix(ff, width, 2.0), matrix(width, ff)
            sublayers.append(2)
        if streams:
            for q in sublayers:
                w[name + f"hc{q}.in"] = torch.full((streams,), 1.0 / streams) + 0.2 * rand(streams)
                w[name + f"hc{q}.out"] = 1 + 0.3 * rand(streams)
                w[name + f"hc{q}.mix"] = torch.eye(streams) * 0.8 + 0.2 / streams + 0.1 * rand(streams, streams)
    return {key: value.to(torch.bfloat16).contiguous() for key, value in w.items()}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config, weights as stored)."""
    made = {}
    for seed, (name, config) in enumerate(CONFIGS.items()):
        folder = tmp_path_factory.mktemp("vopepel_" + name)
        weights = draw_weights(config, 100 + seed)
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
    difference within 0.08 of the spread and the largest within 0.35 - rounding through sharpened layers reaches a
    third of that, a key or a state that is lost several times it."""
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
LENGTHS = {"streams3": (61, 23, 5, 38, 1, 44, 17), "plain": (70, 9, 35, 2, 41), "one_stream": (150, 70, 3, 129), "delta_only": (40, 3, 25, 31, 1), "wide": (330, 45, 150)}


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
        assert (len(engine.cache.groups) == 0) == (name == "delta_only")
        del engine


def test_layer_by_layer_in_32_bit(models):
    """The residual stream after every layer (the sum of the copies), for a model with several streams."""
    from pylon_b200.engine import StepEntry

    folder, config, weights = models["streams3"]
    tokens = make_requests(config, (37,), seed=5)["r0"]
    want: list = []
    plain.forward(config, weights, tokens, layers_out=want)
    engine = engine_for(folder, "float32", 8, 64)
    taps: list = []
    forward = engine.model.forward
    engine.model.forward = lambda step, caches: forward(step, caches, taps)
    request = engine.open("a", len(tokens))
    engine.step([StepEntry(request, tokens, [0])])
    assert len(taps) == len(config["layers"])
    for index, (got, expected) in enumerate(zip(taps, want)):
        torch.testing.assert_close(got.double().cpu(), expected, rtol=1e-4, atol=1e-4 * float(expected.abs().max()), msg=lambda m: f"layer {index}: {m}")


def test_long_decoding_across_many_chunks_and_pages(models):
    """A short prompt, then 200 tokens one by one: the chunks of both attention layers and many pages pass, the pool holds
    only what the chunks need, the delta rule's state is carried 200 times."""
    folder, config, weights = models["streams3"]
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
@pytest.mark.parametrize("name", ["streams3", "one_stream"])
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


def test_decode_steps_replay_from_cuda_graphs(models):
    folder, config, weights = models["one_stream"]
    requests = make_requests(config, (70, 20), seed=17)
    want = plain_logits(config, weights, requests)
    steps = trace_tools.tail_one_by_one(requests, tail=40)
    engine = engine_for(folder, "float32", 64, 256, cuda_graphs=True)
    got = trace_tools.run_in_process(engine, steps)
    assert_logits(got, want, "float32", "decode steps from graphs")
    assert engine.step_function.graphs.captured or engine.step_function.graphs.captured_alike


# ---------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm"])
@pytest.mark.parametrize("streams", [1, 2, 4])
def test_streams_update_and_norm(streams, kind):
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(streams)
    tokens, width, eps, scale = 9, 200, 1e-5, 0.6
    x = torch.randn(tokens, streams, width, generator=g)
    delta = torch.randn(tokens, width, generator=g).to(torch.bfloat16)
    mix, out_w, read = torch.randn(streams, streams, generator=g), torch.randn(streams, generator=g), torch.randn(streams, generator=g)
    weight = 1 + 0.2 * torch.randn(width, generator=g)
    xd, dd = x.double(), delta.double()
    new = torch.stack([sum(mix[s, t].double() * xd[:, s] for s in range(streams)) + scale * out_w[t].double() * dd for t in range(streams)], dim=1)
    u = sum(read[s].double() * new[:, s] for s in range(streams))
    want = plain.layer_norm(u, weight.double(), eps) if kind == "layernorm" else plain.rms_unit(u, eps) * weight.double()
    on = lambda t: t.to(DEVICE)
    # all tokens: the streams are updated in place
    device_x = on(x).clone()
    got = ops.streams_update_norm(device_x, on(delta), scale, on(mix), on(out_w), on(read), on(weight), eps, kind, torch.float32)
    torch.testing.assert_close(device_x.double().cpu(), new, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(got.double().cpu(), want, rtol=1e-4, atol=1e-4)
    # selected rows: computed on the fly, the streams stay
    device_x = on(x).clone()
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEVICE)
    got = ops.streams_update_norm(device_x, on(delta), scale, on(mix), on(out_w), on(read), on(weight), eps, kind, torch.float32, rows=rows)
    torch.testing.assert_close(device_x.cpu(), x, rtol=0, atol=0)
    torch.testing.assert_close(got.double().cpu(), want[[7, 0, 3]], rtol=1e-4, atol=1e-4)
    # partial sums of the delta, no route: the plain residual sum with a factor
    parts = torch.randn(3, tokens, width, generator=g)
    device_x = on(x).clone()
    got = ops.streams_update_norm(device_x, on(parts), scale, None, None, None, on(weight), eps, kind, torch.bfloat16)
    new = xd + scale * parts.double().sum(dim=0)[:, None, :]
    u = new.sum(dim=1)
    want = plain.layer_norm(u, weight.double(), eps) if kind == "layernorm" else plain.rms_unit(u, eps) * weight.double()
    torch.testing.assert_close(device_x.double().cpu(), new, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(got.double().cpu(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gated_unit(dtype):
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(0)
    limit, alpha = 1.25, 1.702
    gate_up = (torch.randn(7, 2 * 88, generator=g) * 2).to(dtype)
    gate, up = gate_up[:, :88].double(), gate_up[:, 88:].double()
    gc, uc = torch.clamp(gate, max=limit), torch.clamp(up, -limit, limit)
    want = gc * torch.sigmoid(alpha * gc) * (uc + 1)
    got = ops.swiglu(gate_up.to(DEVICE), limit=limit, alpha=alpha)
    tolerance = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got.double().cpu(), want, **tolerance)
    assert float(want.abs().max()) > limit   # the clamps were in play


def delta_inputs(tokens, heads, kv_heads, dim, vdim, taps, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    channels = 2 * kv_heads * dim + heads * vdim
    proj = (torch.randn(tokens, channels + heads * vdim + 2 * heads, generator=g) * 1.5).to(dtype)
    conv = torch.randn(channels, taps, generator=g) * 0.6
    a_log, dt_bias, norm = torch.randn(heads, generator=g) * 0.5 - 1.0, torch.randn(heads, generator=g) * 0.5, 1 + 0.1 * torch.randn(vdim, generator=g)
    return proj, conv, a_log, dt_bias, norm


def plain_delta_from_projections(proj, conv, a_log, dt_bias, norm, heads, kv_heads, dim, vdim, eps):
    """The mixer from its projections on (columns [q | k | v | gate | a | b]) for one sequence from its start."""
    proj = proj.double()
    count, qk, vs = proj.shape[0], kv_heads * dim, heads * vdim
    mixed = plain.silu(plain.causal_conv(proj[:, : 2 * qk + vs], conv.double()))
    q, k, v = mixed[:, :qk].view(count, kv_heads, dim), mixed[:, qk : 2 * qk].view(count, kv_heads, dim), mixed[:, 2 * qk :].view(count, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    gate = plain.silu(proj[:, 2 * qk + vs : 2 * qk + 2 * vs]).view(count, heads, vdim)
    a, b = proj[:, 2 * qk + 2 * vs : 2 * qk + 2 * vs + heads], proj[:, 2 * qk + 2 * vs + heads :]
    decay = torch.exp(-torch.exp(a_log.double()) * plain.softplus(a + dt_bias.double()))
    out = plain.delta_recurrence(q, k, v, decay, torch.sigmoid(b))
    return (plain.rms_unit(out, eps) * norm.double() * gate).reshape(count, vs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps", [(4, 2, 16, 24, 4), (1, 1, 100, 5, 1), (3, 3, 64, 64, 3), (2, 1, 200, 40, 8), (8, 2, 128, 128, 4),
                                                         (2, 1, 32, 8, 2), (1, 1, 256, 16, 3), (2, 2, 96, 20, 4), (1, 1, 512, 12, 2)])
def test_gated_delta_rule_prefill_and_token_by_token(heads, kv_heads, dim, vdim, taps, dtype):
    """Rows of unequal length in one call, then the same sequences cut in portions (two tokens, one token) that continue
    from the state slots; slots in another order than rows; a slot that is used again starts from zero."""
    from pylon_b200.kernels import ops

    eps = 1e-5
    lengths = (23, 1, 9)
    channels = 2 * kv_heads * dim + heads * vdim
    floats = heads * dim * vdim + (taps - 1) * channels
    inputs = [delta_inputs(n, heads, kv_heads, dim, vdim, taps, 50 + i, dtype) for i, n in enumerate(lengths)]
    proj0, conv, a_log, dt_bias, norm = inputs[0]
    want = [plain_delta_from_projections(p[0], conv, a_log, dt_bias, norm, heads, kv_heads, dim, vdim, eps) for p in inputs]
    on = lambda t: t.to(DEVICE)
    tolerance = dict(rtol=2e-4, atol=2e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)

    def run(state, pieces, slots):
        step = step_view([p.shape[0] for p in pieces], [0] * len(pieces), dtype)
        step.slots = torch.tensor(slots, dtype=torch.int32, device=DEVICE)
        out = ops.gated_delta_rule(on(torch.cat(pieces)), on(conv.t().contiguous()), state, step.token_row, step.q_start, step.slots, on(a_log), on(dt_bias), on(norm),
                                   heads, kv_heads, dim, vdim, len(pieces), eps)
        return torch.split(out.double().cpu(), [p.shape[0] for p in pieces])

    state = torch.zeros(5, floats, device=DEVICE)
    state[1].fill_(float("nan"))   # a slot no row names: it must not be touched or read
    for got, expected in zip(run(state, [p[0] for p in inputs], [4, 0, 2]), want):
        torch.testing.assert_close(got, expected, **tolerance)
    assert torch.isnan(state[1]).all() and not torch.isnan(state[[0, 2, 3, 4]]).any()
    whole_state = state.clone()
    # the same in portions: 2 tokens, then one by one, then the rest; the short rows drop out
    state = torch.zeros(5, floats, device=DEVICE)
    cursor = [0, 0, 0]
    collected = [[], [], []]
    for sizes in ((2, 1, 2), (1, 0, 1), (1, 0, 2), (7, 0, 4), (1, 0, 0), (11, 0, 0)):
        rows = [i for i, size in enumerate(sizes) if size]
        pieces = [inputs[i][0][cursor[i] : cursor[i] + sizes[i]] for i in rows]
        for i, got in zip(rows, run(state, pieces, [(4, 0, 2)[i] for i in rows])):
            collected[i].append(got)
            cursor[i] += sizes[i]
    for i in range(3):
        torch.testing.assert_close(torch.cat(collected[i]), want[i], **tolerance)
    torch.testing.assert_close(state[[0, 2, 4]], whole_state[[0, 2, 4]], rtol=1e-4, atol=1e-4)
    # a slot that is taken again is zeroed by its new owner (the cache manager does that): the result is the fresh one
    state[2].zero_()
    again = run(state, [inputs[2][0]], [2])[0]
    torch.testing.assert_close(again, want[2], **tolerance)


def paged(keys, values, page_size, order_seed):
    """Lays ``keys [T, kv, d]`` / ``values [T, kv, dv]`` of one request into shuffled pages; returns pages and the table."""
    count, kv, d = keys.shape
    dv = values.shape[2]
    pages_needed = -(-count // page_size)
    total = pages_needed + 3
    order = np.random.default_rng(order_seed).permutation(total)[:pages_needed]
    k_pages = torch.full((total, kv, page_size, d), float("nan"), dtype=keys.dtype)
    v_pages = torch.full((total, kv, page_size, dv), float("nan"), dtype=values.dtype)
    for t in range(count):
        k_pages[order[t // page_size], :, t % page_size] = keys[t]
        v_pages[order[t // page_size], :, t % page_size] = values[t]
    return k_pages, v_pages, torch.tensor(order[None, :].astype(np.int32))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,dv,heads,kv_heads,chunk,softcap,page", [(16, 8, 6, 2, 10, 5.0, 8), (64, 64, 4, 2, 128, 25.0, 64), (64, 32, 6, 3, 80, 15.0, 64),
                                                                   (32, 48, 2, 1, 33, None, 16), (64, 64, 2, 2, None, 8.0, 64), (128, 128, 4, 1, 200, 30.0, 64),
                                                                   (64, 64, 1, 1, 64, 12.0, 64)])
def test_chunked_capped_attention_sees_exactly_its_chunk(d, dv, heads, kv_heads, chunk, softcap, page, dtype):
    """One key of the sequence is made to stand out (scaled up, with a value of its own); queries just before the end of
    its chunk must be dominated by it, queries just behind the chunk's edge must not see it at all.  All positions are
    compared with the plain attention, as a prompt in one piece and token by token over the same pages."""
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(d + dv)
    count = 3 * (chunk or 70) + 17
    q = torch.randn(count, heads, d, generator=g)
    k = torch.randn(count, kv_heads, d, generator=g)
    v = torch.randn(count, kv_heads, dv, generator=g)
    marked = (chunk or 70) + 1                       # the second key of the second chunk
    k[marked] = 0
    k[marked, :, 0] = 40.0
    q[:, :, 0] = q[:, :, 0].abs() + 2.0              # every query likes the marked key
    v[marked] = 50.0
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    scale = 1.0 / math.sqrt(d)
    want = plain.attention_core(q.double(), k.double(), v.double(), scale, softcap, chunk)
    if chunk is not None:
        assert float(want[marked + chunk - 2].abs().mean()) > 10 and float(want[2 * chunk + 1].abs().mean()) < 5    # inside / outside
    k_pages, v_pages, table = paged(k, v, page, 1)
    on = lambda t: t.to(DEVICE)
    tolerance = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=5e-2, atol=8e-2)
    flat_q = on(q.reshape(count, heads * d))
    # as one prompt
    step = step_view([count], [0], dtype)
    got = ops.paged_attention(flat_q, on(k_pages), on(v_pages), step.positions, step.token_row, step.q_start, step.kv_len, on(table),
                              heads, step.max_q, step.max_kv, scale=scale, chunk=chunk, softcap=softcap)
    torch.testing.assert_close(got.double().cpu().view(count, heads, dv), want, **tolerance)
    # token by token around the edges of the marked key's chunk, and a portion that starts in the middle of a chunk
    edges = [marked, marked + 1] + ([marked + chunk - 3, marked + chunk - 2, marked + chunk - 1, marked + chunk, 2 * chunk + 5] if chunk else [count - 1])
    for position in edges:
        step = step_view([1], [position], dtype)
        got = ops.paged_attention(flat_q[position : position + 1].contiguous(), on(k_pages), on(v_pages), step.positions, step.token_row, step.q_start,
                                  step.kv_len, on(table), heads, 1, position + 1, scale=scale, chunk=chunk, softcap=softcap)
        torch.testing.assert_close(got.double().cpu().view(heads, dv), want[position], **tolerance)
    start = (chunk or 70) + (chunk or 70) // 2
    step = step_view([count - start], [start], dtype)
    got = ops.paged_attention(flat_q[start:].contiguous(), on(k_pages), on(v_pages), step.positions, step.token_row, step.q_start, step.kv_len, on(table),
                              heads, step.max_q, step.max_kv, scale=scale, chunk=chunk, softcap=softcap)
    torch.testing.assert_close(got.double().cpu().view(count - start, heads, dv), want[start:], **tolerance)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qk_norm_value_mix_and_cache_write(dtype):
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(3)
    nq, nkv, d, dv, page, eps = 4, 2, 24, 10, 4, 1e-5
    lengths, starts = [5, 1, 3], [2, 9, 0]
    tokens = sum(lengths)
    qkv = torch.randn(tokens, (nq + nkv) * d + nkv * dv, generator=g).to(dtype)
    other = torch.randn(tokens, nkv * dv + 7, generator=g).to(dtype)[:, 7:]      # a view with a row stride
    qw, kw, lam = 1 + 0.2 * torch.randn(d, generator=g), 1 + 0.2 * torch.randn(d, generator=g), torch.tensor([0.3])
    step = step_view(lengths, starts, dtype)
    table = torch.tensor([[5, 2, 7], [0, 6, 3], [4, 1, 8]], dtype=torch.int32)
    k_pages = torch.zeros(9, nkv, page, d, dtype=dtype, device=DEVICE)
    v_pages = torch.zeros(9, nkv, page, dv, dtype=dtype, device=DEVICE)
    device_qkv = qkv.to(DEVICE).clone()
    ops.qk_norm_mix_kv_write(device_qkv, qw.to(DEVICE), kw.to(DEVICE), eps, step.positions, step.token_row, table.to(DEVICE), page, k_pages, v_pages,
                             nq, nkv, d, dv, other_values=other.to(DEVICE), mix_weight=lam.to(DEVICE))
    x = qkv.double()
    want_q = plain.rms_unit(x[:, : nq * d].view(tokens, nq, d), eps) * qw.double()
    want_k = plain.rms_unit(x[:, nq * d : (nq + nkv) * d].view(tokens, nkv, d), eps) * kw.double()
    want_v = (0.7 * x[:, (nq + nkv) * d :] + 0.3 * other.double()).view(tokens, nkv, dv)
    tolerance = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    result = device_qkv.double().cpu()
    torch.testing.assert_close(result[:, : nq * d].view(tokens, nq, d), want_q, **tolerance)
    torch.testing.assert_close(result[:, (nq + nkv) * d :].view(tokens, nkv, dv), want_v, **tolerance)
    token = 0
    for row, (n, s) in enumerate(zip(lengths, starts)):
        for position in range(s, s + n):
            where = int(table[row, position // page])
            torch.testing.assert_close(k_pages[where, :, position % page].double().cpu(), want_k[token], **tolerance)
            torch.testing.assert_close(v_pages[where, :, position % page].double().cpu(), want_v[token], **tolerance)
            token += 1


@pytest.mark.parametrize("rows", [1, 5, 24, 40, 300, 1000])
def test_clamped_gated_unit_in_the_products(rows):
    """Gate and up as one product with the clamped unit applied where the product ends: the TMA-fed kernel for few rows, the
    tcgen05 kernel for many, the library product and the unit's own kernel in between."""
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(rows)
    width, inner, limit, alpha = 1024, 208, 1.5, 1.702
    x = torch.randn(rows, width, generator=g).to(torch.bfloat16)
    gate = (torch.randn(inner, width, generator=g) * 2 / math.sqrt(width)).to(torch.bfloat16)
    up = (torch.randn(inner, width, generator=g) * 2 / math.sqrt(width)).to(torch.bfloat16)
    gc = torch.clamp(x.double() @ gate.double().T, max=limit)
    uc = torch.clamp(x.double() @ up.double().T, -limit, limit)
    want = gc * torch.sigmoid(alpha * gc) * (uc + 1)
    stacked = ops.interleave_gate_up(gate.to(DEVICE), up.to(DEVICE))
    got = ops.linear_swiglu(x.to(DEVICE), stacked, limit=limit, alpha=alpha)
    torch.testing.assert_close(got.double().cpu(), want, rtol=3e-2, atol=3e-2)
    assert float((x.double() @ gate.double().T).max()) > limit      # the clamp was in play


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(2, 1, 64, 32), (1, 1, 128, 128), (3, 3, 40, 12)])
def test_the_delta_rule_remembers_a_token_seven_hundred_tokens_back(heads, kv_heads, dim, vdim, dtype):
    """The inputs are made so that one early token writes a value of its own under a key that no later token touches (every
    other key is nearly orthogonal to it, the decay is almost one), and the last token asks for exactly that key: its
    read-out must be that value, through 700 tokens of state - as one prompt, with the last 40 tokens one by one, and in
    portions of changing size.  A state that is lost or reset anywhere on the way gives another read-out."""
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(dim)
    tokens, marked, eps = 700, 3, 1e-5
    qk, vs = kv_heads * dim, heads * vdim
    channels = 2 * qk + vs
    proj = torch.randn(tokens, channels + vs + 2 * heads, generator=g)
    q_part, k_part, v_part = proj[:, :qk].view(tokens, kv_heads, dim), proj[:, qk : 2 * qk].view(tokens, kv_heads, dim), proj[:, 2 * qk : channels].view(tokens, heads, vdim)
    k_part[:, :, 0] = -12.0                    # silu(-12) is nothing: no other key has a share of coordinate 0
    k_part[marked] = -12.0
    k_part[marked, :, 0] = 12.0                # the marked key is that coordinate alone
    q_part[-1] = -12.0
    q_part[-1, :, 0] = 12.0                    # and the last query asks for it
    pattern = torch.where(torch.arange(vdim) % 3 == 0, 25.0, -25.0)
    v_part[marked] = pattern
    proj[:, channels + vs : channels + vs + heads] = 0.0                 # a: with A_log far down the decay is almost one
    proj[marked, channels + vs + heads :] = 12.0                          # b: the marked token writes with beta near one
    proj = proj.to(dtype)
    conv = torch.ones(1, channels)                                        # one tap of weight one: the convolution passes its input on
    a_log, dt_bias, norm = torch.full((heads,), -14.0), torch.zeros(heads), torch.ones(vdim)
    want = plain_delta_from_projections(proj, conv.t().contiguous(), a_log, dt_bias, norm, heads, kv_heads, dim, vdim, eps)
    gate = plain.silu(proj.double()[-1, channels : channels + vs]).view(heads, vdim)
    recalled = want[-1].view(heads, vdim) / gate                          # the read-out, normalised: the marked value's pattern
    # (values pass through silu: the pattern arrives as 25 and nothing, and is normalised to root 3 and nothing)
    assert float(recalled[:, pattern > 0].min()) > 1.5 and float(recalled[:, pattern < 0].abs().max()) < 0.2
    on = lambda t: t.to(DEVICE)
    floats = heads * dim * vdim
    tolerance = dict(rtol=1e-3, atol=1e-3) if dtype == torch.float32 else dict(rtol=4e-2, atol=4e-2)

    def run(portions):
        state = torch.zeros(2, floats, device=DEVICE)
        pieces, cursor = [], 0
        for size in portions:
            step = step_view([size], [cursor], dtype)
            step.slots = torch.tensor([1], dtype=torch.int32, device=DEVICE)
            out = ops.gated_delta_rule(on(proj[cursor : cursor + size].contiguous()), on(conv), state, step.token_row, step.q_start, step.slots,
                                       on(a_log), on(dt_bias), on(norm), heads, kv_heads, dim, vdim, 1, eps)
            pieces.append(out.double().cpu())
            cursor += size
        assert cursor == tokens
        return torch.cat(pieces)

    changing = [7, 2, 64, 3, 129, 2, 200, 31, 2, 160, 99, 1]
    for portions in ([tokens], [tokens - 40] + [1] * 40, changing):
        got = run(portions)
        torch.testing.assert_close(got[-1], want[-1], **tolerance)
        torch.testing.assert_close(got, want, **tolerance)

"""The Bizetar architecture through the engine against the plain implementation
(``plain_bizetar``): whole prompts, prefill against token-by-token decoding, portions down to two
tokens, mixed batches on pools so small that pages and slots are used again (freed pages
poisoned), the residual stream after every layer, long decoding (also as CUDA graphs), a long
prompt at wide sizes, models of random sizes, and greedy generation through ``Engine`` and the
command line."""

import os
import tempfile

import numpy as np
import pytest
import torch

import bizetar_configs as bc
import plain_bizetar as pb
import trace_helpers as th
from gpu_helpers import assert_close

pytestmark = pytest.mark.gpu
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
LENGTHS = [70, 33, 100, 5, 64, 17, 90, 48, 1, 2]

_cache: dict = {}


def _plain(config, weights, ids, dtype_name, routing=None):
    act = None if dtype_name == "float32" else torch.bfloat16
    return pb.forward(ids, weights, config, act=act, routing=routing).to(torch.float32).numpy()


def _model(name, model_root):
    if name not in _cache:
        folder, weights = bc.make_folder(name, model_root)
        requests = {f"r{i}": bc.tokens(name, n, i) for i, n in enumerate(LENGTHS)}
        reference = {rid: _plain(bc.ALL[name], weights, t, "float32")
                     for rid, t in requests.items()}
        _cache[name] = (folder, weights, requests, reference)
    return _cache[name]


def _replay(runner, steps, vocab):
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        return th.collect(steps, out, vocab)


def _replay_and_reference(runner, steps, config, weights, requests, dtype_name, reference=None):
    """(the rows that the replay wrote, what the plain implementation gives for each request).
    bfloat16 is compared with the plain implementation rounding its products and routing as the
    engine routed."""
    if dtype_name == "float32":
        rows = _replay(runner, steps, config["vocab"])
        return rows, reference or {rid: _plain(config, weights, t, "float32")
                                   for rid, t in requests.items()}
    with bc.RoutingTap(runner, config) as tap:
        rows = _replay(runner, steps, config["vocab"])
    return rows, {rid: _plain(config, weights, t, dtype_name, tap.routing(rid) or None)
                  for rid, t in requests.items() if any(r == rid for r, _ in rows)}


def _schedules(requests):
    return {
        "whole": (th.schedule_whole(requests), 128),
        "tail": (th.schedule_tail(requests, 32), 128),
        "portions": (th.schedule_portions(requests), 128),
        "pairs": (th.schedule_portions(requests, sizes=(2,)), 128),
        "mixed": (th.schedule_mixed(requests, 320, seed=3), 320),
        "mixed_tight": (th.schedule_mixed(requests, 192, seed=11, decode_tail=32), 192),
    }


# bfloat16 bounds of this file, as shares of a position's largest logit; the 32-bit runs are the
# sharp test (gpu_helpers.F32_REL).  The engine and the plain implementation's rounding model sum
# in different orders and round in slightly different places (the engine keeps the convolution's
# sums and the normed rows unrounded until they are stored), and these tiny models have tokens at
# which rounding is amplified: a sublayer's result is divided by its own root mean square, so a
# gated result that is small all over is normed up to full size.  One position in ten may lie
# over the bound, and the median is bounded too.
BF16_MAX, BF16_RMS, BF16_MEDIAN = 8e-2, 2e-2, 1.5e-2


def _compare(rows, reference, dtype, what):
    assert rows, "the replay wrote nothing"
    rms, over = [], []
    for (rid, position), got in rows.items():
        want = reference[rid][position]
        if dtype == torch.float32:
            assert_close(got, want, dtype, f"{what} {rid}@{position}")
            continue
        assert np.isfinite(got).all(), f"{what} {rid}@{position}: not finite"
        err, scale = np.abs(got - want), np.abs(want).max()
        rms.append(float(np.sqrt((err ** 2).mean()) / scale))
        if rms[-1] > BF16_RMS or err.max() > BF16_MAX * scale:
            over.append(f"{rid}@{position}: rms {rms[-1]:.3f}, max {err.max() / scale:.3f}")
    if rms:
        assert len(over) <= max(1, len(rms) // 10) and np.median(rms) <= BF16_MEDIAN, (
            f"{what}: {len(over)} of {len(rms)} positions over the bound, median rms "
            f"{np.median(rms):.3e} of the largest logit; " + "; ".join(over[:5]))


@pytest.mark.parametrize("name", ["biz_a", "biz_b", "biz_c"])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "pairs", "mixed", "mixed_tight"])
def test_replay_matches_plain(name, dtype_name, schedule, model_root):
    from distengine_b200.engine.replay import build_runner
    folder, weights, requests, reference = _model(name, model_root)
    steps, max_tokens = _schedules(requests)[schedule]
    runner = build_runner(folder, dtype_name, max_tokens, page_size=bc.PAGES[name],
                          poison_freed_pages=True, live_requests=4)
    rows, want = _replay_and_reference(runner, steps, bc.ALL[name], weights, requests, dtype_name,
                                       reference)
    runner.cache.check_invariants()
    assert not runner.cache.live
    assert len(rows) == sum(len(e["want"]) for s in steps for e in s["entries"])
    _compare(rows, want, DTYPES[dtype_name], f"{name} {schedule}")


@pytest.mark.parametrize("name", ["biz_a", "biz_c"])
def test_float32_cuts_agree_closely(name, model_root):
    """However a request is cut, its 32-bit logits agree far inside the tolerance."""
    from distengine_b200.engine.replay import build_runner
    folder, _, requests, _ = _model(name, model_root)
    got = {}
    for schedule in ("whole", "tail", "pairs", "mixed"):
        steps, max_tokens = _schedules(requests)[schedule]
        runner = build_runner(folder, "float32", max_tokens, page_size=bc.PAGES[name])
        got[schedule] = _replay(runner, steps, bc.ALL[name]["vocab"])
    for schedule in ("tail", "pairs", "mixed"):
        for key, row in got[schedule].items():
            scale = np.abs(got["whole"][key]).max()
            np.testing.assert_allclose(row, got["whole"][key], rtol=0, atol=2e-5 * max(scale, 1.0),
                                       err_msg=f"{schedule} {key}")


@pytest.mark.parametrize("name", ["biz_a", "biz_b"])
def test_the_stream_after_every_layer(name, model_root):
    """The residual stream behind every layer (after the mix over the depth), 32-bit: sublayers
    that read the stream itself, gates of the sublayers' own inputs, norms on their results."""
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.engine.step import StepEntry
    from distengine_b200.parts import block as blocks
    folder, weights = bc.make_folder(name, model_root)
    ids = bc.tokens(name, 23, 9)
    want: list = []
    pb.forward(ids, weights, bc.ALL[name], trace=want)
    caught = []
    original = blocks.SublayerNormBlock.forward

    def forward(self, stream, ctx, cache, following=None):
        original(self, stream, ctx, cache, following)
        caught.append(stream.resid.clone())

    blocks.SublayerNormBlock.forward = forward
    try:
        runner = build_runner(folder, "float32", 64, page_size=8)
        runner.step([StepEntry("t", ids, [22])])
        runner.check_status()
    finally:
        blocks.SublayerNormBlock.forward = original
    assert len(caught) == len(want) == len(bc.ALL[name]["layers"])
    for index, (got, ref) in enumerate(zip(caught, want)):
        assert_close(got, ref, torch.float32, f"{name}: stream after layer {index}")


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["biz_a", "biz_c"])
def test_long_decoding_with_graphs(name, dtype_name, model_root):
    """A short prompt, then 220 tokens one by one over many page borders (the query's growth with
    its position passes several of its steps; the convolution's kept rows move on at every
    token), also replayed as CUDA graphs."""
    from distengine_b200.engine.replay import build_runner
    folder, weights = bc.make_folder(name, model_root)
    ids = bc.tokens(name, 230, 77)
    steps = th.schedule_tail({"long": ids}, 220)
    runner = build_runner(folder, dtype_name, 256, page_size=16, poison_freed_pages=True)
    rows, want = _replay_and_reference(runner, steps, bc.ALL[name], weights, {"long": ids},
                                       dtype_name)
    _compare(rows, want, DTYPES[dtype_name], "long decode")
    runner = build_runner(folder, dtype_name, 256, page_size=16, use_graphs=True,
                          poison_freed_pages=True)
    graphed = _replay(runner, steps, bc.ALL[name]["vocab"])
    assert runner.graph_replays > 100 and graphed.keys() == rows.keys()
    for key, row in rows.items():
        np.testing.assert_allclose(graphed[key], row, rtol=0, atol=1e-5 * np.abs(row).max(),
                                   err_msg=f"graphs {key}")


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_a_long_prompt_at_wide_sizes(dtype_name, model_root):
    """1,100 tokens in one step (products of a thousand rows and more, attention tiles of 64 rows,
    more than 128 pairs an expert), then tokens one by one, then the same prompt in two uneven
    portions."""
    from distengine_b200.engine.replay import build_runner
    name = "biz_wide"
    folder, weights = bc.make_folder(name, model_root)
    ids = bc.tokens(name, 1112, 3)
    picked = [0, 1, 15, 16, 17, 63, 64, 65, 255, 256, 599, 999, 1000, 1001, 1099]
    head = {"step": 0, "end": [], "entries": [{"id": "w", "tokens": ids[:1100], "want": picked}]}
    tail = [{"step": 1 + i, "end": ["w"] if i == 11 else [],
             "entries": [{"id": "w", "tokens": [ids[1100 + i]], "want": [0]}]} for i in range(12)]
    cut = [{"step": 13, "end": [], "entries": [{"id": "c", "tokens": ids[:1027], "want": [1026]}]},
           {"step": 14, "end": ["c"], "entries": [{"id": "c", "tokens": ids[1027:],
                                                    "want": [0, 84]}]}]
    steps = [head] + tail + cut
    runner = build_runner(folder, dtype_name, 1152, page_size=16, poison_freed_pages=True)
    rows, want = _replay_and_reference(runner, steps, bc.ALL[name], weights, {"w": ids, "c": ids},
                                       dtype_name)
    assert len(rows) == len(picked) + 12 + 3
    _compare(rows, want, DTYPES[dtype_name], f"wide {dtype_name}")


def test_batch_of_unequal_requests_against_each_alone(model_root):
    """Four unequal requests in one step give what each gives alone (32-bit: to rounding)."""
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.engine.step import StepEntry
    name = "biz_b"
    folder, _, requests, reference = _model(name, model_root)
    picked = ["r0", "r3", "r8", "r5"]
    runner = build_runner(folder, "float32", 512, page_size=8)
    entries = [StepEntry(r, requests[r], list(range(len(requests[r])))) for r in picked]
    logits = runner.step(entries).cpu().numpy()
    runner.check_status()
    at = 0
    for r in picked:
        n = len(requests[r])
        assert_close(logits[at: at + n], reference[r], torch.float32, f"batched {r}")
        at += n


def _random_config(rng) -> dict:
    """A model of random sizes: both mixers in random order, each option on or off, dense, routed
    and absent feed-forwards."""
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    width = int(pick(24, 40, 56, 72))
    n_layers = int(pick(1, 2, 3, 4, 5))
    kv_heads, vdim = int(pick(1, 2, 3)), int(pick(1, 3, 8, 16, 20))      # of the mixing layers
    layers = []
    for _ in range(n_layers):
        mixes = rng.random() < 0.7
        g = kv_heads if mixes else int(pick(1, 2, 4))
        dv = vdim if mixes else int(pick(2, 8, 12))
        heads = g * int(pick(1, 2, 3, 5, 8, 9))
        dim = int(pick(2, 4, 6, 8, 16, 24))
        scale = float(pick(0.15, 0.3, 0.5))
        if rng.random() < 0.4:
            temp = pick(None, (0.5, 7), (1.0, 1), (0.2, 100))
            entry = bc.layer("attention", bc.first(heads, g, dim, dv, scale, mixes, temp), None)
        else:
            dims = int(pick(0, 2, dim // 2 * 2))
            scaling = pick(None, (2.0, 16, 4.0, 1.0), (8.0, 64, 32.0, 1.0), (40.0, 100, 2.0, 0.5))
            rot = pick(None, (float(pick(20.0, 10000.0, 1000000.0)), dims) +
                       (() if scaling is None else (scaling,)))
            entry = bc.layer("attention_2", bc.second(heads, g, dim, dv, scale, mixes,
                                                      pick(None, 1, 2, 3, 4), rot), None)
        kind = pick("dense", "moe", "moe", None)
        if kind == "dense":
            entry["mlp"] = bc.dense(int(pick(8, 30, 64)))
        elif kind == "moe":
            experts, identity = int(pick(1, 2, 4, 7, 16)), int(pick(0, 0, 1, 3))
            top = int(rng.integers(1, min(experts + identity, 5) + 1))
            entry["mlp"] = bc.moe(experts, top, int(pick(4, 17, 32)), identity)
        layers.append(entry)
    return {"architecture": "Bizetar", "vocab": int(pick(50, 111)), "width": width,
            "norm": {"eps": float(pick(1e-5, 1e-6))}, "layers": layers}


@pytest.mark.parametrize("seed", range(8))
def test_models_of_random_sizes_under_a_mixed_schedule(seed, model_root):
    from distengine_b200.engine.replay import build_runner
    rng = np.random.default_rng(3000 + seed)
    config = _random_config(rng)
    weights = pb.random_weights(config, 90 + seed, spread=1.5)
    folder = bc.write_folder(config, os.path.join(model_root, f"biz_random_{seed}"), weights)
    requests = {f"q{i}": [int(t) for t in rng.integers(0, config["vocab"], size=n)]
                for i, n in enumerate((61, 9, 80, 2, 35, 50))}
    want = {rid: _plain(config, weights, t, "float32") for rid, t in requests.items()}
    steps = th.schedule_mixed(requests, 256, seed=seed, decode_tail=20)
    for graphs in (False, True):
        runner = build_runner(folder, "float32", 256, page_size=int(rng.choice([4, 8, 16])),
                              poison_freed_pages=True, use_graphs=graphs)
        rows = _replay(runner, steps, config["vocab"])
        runner.cache.check_invariants()
        _compare(rows, want, torch.float32, f"random model {seed} graphs={graphs}")
    runner = build_runner(folder, "bfloat16", 256, page_size=16, poison_freed_pages=True)
    rows, want16 = _replay_and_reference(runner, steps, config, weights, requests, "bfloat16")
    _compare(rows, want16, torch.bfloat16, f"random model {seed} bfloat16")


def _plain_greedy(name, weights, prompt, new):
    ids = list(prompt)
    for _ in range(new):
        ids.append(int(pb.forward(ids, weights, bc.ALL[name])[-1].argmax()))
    return ids[len(prompt):]


def test_greedy_generation_through_the_engine(model_root):
    """``Engine.generate`` (scheduler, portions of prompts under a small token budget, sampling,
    step-ahead decoding with steps taken back) gives the plain implementation's greedy tokens in
    32-bit."""
    from distengine_b200 import Engine, EngineConfig
    name = "biz_a"
    folder, weights = bc.make_folder(name, model_root)
    prompts = [bc.tokens(name, n, 40 + i) for i, n in enumerate((3, 29, 50, 11, 1))]
    new = 12
    want = [_plain_greedy(name, weights, p, new) for p in prompts]
    engine = Engine(folder, EngineConfig(dtype="float32", block_size=16, num_blocks=24,
                                         decode_batch_size=3, max_batch_tokens=32,
                                         max_model_len=128))
    assert engine.generate(prompts, new) == want
    engine.cache.check_invariants()
    engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=16, num_blocks=24,
                                         decode_batch_size=3, max_batch_tokens=32,
                                         max_model_len=128))
    got = engine.generate(prompts, new)
    for prompt, tokens in zip(prompts, got):
        logits = pb.forward(prompt, weights, bc.ALL[name])[-1]
        gap = (logits.max() - logits[tokens[0]]).item()
        assert len(tokens) == new and gap <= 0.25 * logits.abs().max().item()


def test_preempted_requests_are_recomputed(model_root):
    """So few pages that running requests are preempted: they give back their pages and their
    slot, and the cache and the convolution's kept rows are built again from their tokens; the
    greedy tokens stay the plain implementation's."""
    from distengine_b200 import Engine, EngineConfig
    name = "biz_c"
    folder, weights = bc.make_folder(name, model_root)
    prompts = [bc.tokens(name, n, 60 + i) for i, n in enumerate((30, 27, 33))]
    new = 24
    engine = Engine(folder, EngineConfig(dtype="float32", block_size=16, num_blocks=5,
                                         decode_batch_size=3, max_batch_tokens=48,
                                         max_model_len=64))
    assert engine.generate(prompts, new) == [_plain_greedy(name, weights, p, new) for p in prompts]
    assert engine.scheduler.num_preemptions > 0
    engine.cache.check_invariants()
    assert not engine.cache.live


def test_the_command_line_generates(model_root):
    import subprocess
    import sys
    folder, _ = bc.make_folder("biz_b", model_root)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    result = subprocess.run([sys.executable, "-m", "distengine_b200", "generate", "--model", folder,
                             "--prompt-ids", "5 17 3", "--max-new-tokens", "4", "--dtype",
                             "float32", "--num-blocks", "16", "--decode-batch-size", "2"],
                            cwd=root, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]
    assert "Generated token IDs" in result.stdout

"""Decode and prefill throughput of the engine on one B200, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload headline|mixed|long|fp32|vomotar|sebilorn|vapelix|bizetar] [--layers L]

The default (``headline``) has the TinyLlama-1.1B layer sizes in bfloat16.  A step is one decode
step of a batch of 8 requests whose prompts of 512 tokens are in the cache; K steps are timed with
CUDA events after W warm-up steps.  One JSON line is printed:

* ``value``: decoded tokens a second of the step function fed from the host with fixed tokens (no
  read-back between steps);
* ``e2e``: the same through the Python entry point (``Engine.submit`` / ``Engine.step``): every
  step uploads its arrays from pinned host memory and reads the sampled tokens back; timed with
  the host's clock over at least 128 steps, whatever K is (a few steps are too short a stretch
  for the host's clock);
* ``prefill``: one prompt of 2,048 tokens in one step: ``ms`` on the device from the step's
  launch to its last kernel (CUDA events around ``StepRunner.launch``; the step is a replayed
  CUDA graph from its fifth coming on), ``ms_with_host_prepare`` the whole step by the host's
  clock, with the host's preparation of its arrays before the launch;
* ``roofline``: bytes a decode step has to read (every weight once, the live requests' cache)
  over its time, against the measured copy bandwidth;
* ``points``: decode at batch 1, 16 and 64 (batch 64 twice: before and after the others).

Other workloads, each with its own line (the number of layers is named beside the model's):

* ``mixed``: Llama-2-7B layer sizes, 32 requests with prompts of 64 to 2,048 tokens and 256 new
  tokens each through ``Engine`` with a budget of 512 tokens a step (prompt portions beside
  decoded tokens); generated tokens a second end to end, and the sum of the steps' roofline times
  (the slower of flops at the matrix peak and bytes at copy bandwidth) over the time taken.
* ``long``: Llama-3-8B layer sizes (vocabulary 128,256), 64 requests with prompts of 4,096 tokens:
  prompt portions of 4,096 tokens and decode steps at batch 64 over the long cache.
* ``fp32``: the headline's sizes in the true 32-bit path (decode at batch 8, prefill of 2,048).
* ``vomotar``: the Vomotar architecture (layers of gated delta rule, and of chunk-masked attention
  beside retention) at the headline's width, feed-forward and vocabulary, beside the Llama decoder
  with the same number of layers: decode at batch 8 and 64 and a prompt of 2,048 tokens for both,
  and every kernel that is the design's own, alone, against its roofline.
* ``sebilorn``: the Sebilorn architecture (windowed attention with kept first tokens, a layer that
  reads the layer before it's keys and values, gated attention beside the generalized delta rule,
  lightning attention; layer norms, squared-relu feed-forward) at the same width, feed-forward and
  vocabulary, beside Vomotar and Llama with the same number of layers: decode at batch 8 and 64
  and a prompt of 2,048 tokens, and every kernel of the design alone against its roofline, each
  beside the like kernel of the other models.
* ``vapelix``: the Vapelix architecture (latent attention over a cached latent, routed experts
  beside dense gated feed-forwards, a side input from the token's row of a table; two branches of
  one input a layer) at the same width and vocabulary, beside Llama with the same number of
  layers: decode at batch 8 and 64 and a prompt of 2,048 tokens, and every kernel of the design
  alone against its roofline, each beside the like kernel of the other models.
* ``bizetar``: the Bizetar architecture (attention with a sink in two forms - biases, a short
  convolution, norms per head and stretched rotation, or norms over the projection, a distance
  bias and a growing query -, norms on the gated results of the sublayers, a stream mixed over the
  depth, a cubic activation, gated experts beside router outputs that hand the input on) at the
  same width and vocabulary, beside Sebilorn and Llama with the same number of layers: decode at
  batch 8 and 64 and a prompt of 2,048 tokens, and every kernel of the design alone against its
  roofline, each beside the like kernel of the other models.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: TinyLlama-1.1B shape
MODEL = dict(architectures=["LlamaForCausalLM"], vocab_size=32000, hidden_size=2048,
             intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32,
             num_key_value_heads=4, rms_norm_eps=1e-5, rope_theta=10000.0,
             max_position_embeddings=2048, tie_word_embeddings=False)
# BASELINE.json configs[3] and [4]
LLAMA2_7B = dict(architectures=["LlamaForCausalLM"], vocab_size=32000, hidden_size=4096,
                 intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                 num_key_value_heads=32, rms_norm_eps=1e-5, rope_theta=10000.0,
                 max_position_embeddings=4096, tie_word_embeddings=False)
LLAMA3_8B = dict(architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=4096,
                 intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                 num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=500000.0,
                 max_position_embeddings=8192, tie_word_embeddings=False)
PROMPT, NEW_TOKENS, PREFILL, PAGE = 512, 128, 2048, 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                data = json.load(handle)
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for k, v in node.items():
                        if isinstance(v, (int, float)) and not isinstance(v, bool):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return flat, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self) -> None:
        self.lines: list[str] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm, top, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(parts[0]))
                top.append(int(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": int(statistics.median(sm)), "sm_max_mhz": max(top),
                "reasons": sorted(reasons), "samples": len(sm)}


def model_folder(layers: int, shape: "dict | None" = None, name: str = "tinyllama") -> str:
    """The random-weights model folder (written once per machine into the temporary folder)."""
    from distengine_b200.weights import write_random_model
    if shape is None:
        MODEL["num_hidden_layers"] = layers
        shape = MODEL
    shape = dict(shape, num_hidden_layers=layers)
    folder = os.path.join(tempfile.gettempdir(), f"distengine_b200-bench-{os.getuid()}",
                          f"{name}-shape-{layers}-layers-seed0-bf16")
    marker = os.path.join(folder, ".complete")
    if not os.path.isfile(marker):
        print("[bench] writing the random-weights model folder ...", file=sys.stderr, flush=True)
        write_random_model(shape, folder, seed=0, dtype="bfloat16")
        with open(marker, "w") as handle:
            handle.write("ok")
    return folder


def weight_bytes(model) -> tuple[int, int]:
    """(bytes of all weights a decode step reads once, matrix parameters in the layers)."""
    total = model.output.numel() * model.output.element_size()
    params = 0
    for block in model.blocks:
        mixer, ffn = block.mixer, block.feed_forward
        for t in (mixer.w_qkv, mixer.w_o, ffn.w_gate_up, ffn.w_down):
            total += t.numel() * t.element_size()
            params += t.numel()
        for norm in (block.mixer_norm, block.feed_forward_norm):
            total += norm.weight.numel() * norm.weight.element_size()
    return total, params


def reference_arm(args, warmup: int, steps: int) -> int:
    """The unmodified reference on the same shape and workload (``baseline/reference_arm.py``):
    its own model, block manager and ``ModelRunner.prefill`` / ``decode_batch``, in float32 with
    TF32 off as it runs on CUDA.  None of this package is on that path."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as arm
    why = arm.available()
    if why is None:
        try:
            import torch
            if not torch.cuda.is_available():
                why = "no CUDA device is visible"
        except ImportError as error:
            why = f"torch cannot be imported: {error}"
    if why is not None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    model = dict(MODEL, num_hidden_layers=args.layers)
    with ClockSampler() as sampler:
        got = arm.run(model, args.batch, PROMPT, steps, warmup, PREFILL)
    ms = got["ms_per_step"]
    print(json.dumps({
        "metric": "decode tokens/s at batch 8 (TinyLlama-1.1B shape, 512-token prompts, 1 B200)",
        "value": round(args.batch / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic", "impl": "reference",
        "config": {"model": "TinyLlama-1.1B shape, random weights N(0,0.02) seed 0",
                   "layers": model["num_hidden_layers"], "layers_of_config": 22,
                   "hidden": model["hidden_size"], "heads": model["num_attention_heads"],
                   "kv_heads": model["num_key_value_heads"],
                   "intermediate": model["intermediate_size"], "vocab": model["vocab_size"],
                   "global_batch": args.batch, "seq_len": PROMPT, "new_tokens": steps,
                   "page_size": PAGE, "parallelism": "single GPU",
                   "path": "ModelRunner.prefill + ModelRunner.decode_batch, unmodified",
                   "dtype_note": "the reference runs float32 with TF32 off on CUDA "
                                 "(src/distengine/worker.py:427-430); it has no bfloat16 path",
                   "l2": "inputs larger than L2: 4.1 GB of weights are read every step"},
        "clocks": sampler.summary(),
        "e2e": {"value": round(args.batch / got["wall_ms_per_step"] * 1e3, 1),
                "unit": "tokens/s", "h2d_bytes_per_step": got["h2d_bytes_per_step"],
                "d2h_bytes_per_step": got["d2h_bytes_per_step"]},
        "gpu_launches": 0,
        "prefill": {"value": round(PREFILL / got["prefill_ms"] * 1e3, 1), "tokens": PREFILL,
                    "ms": round(got["prefill_ms"], 3)},
        "points": got["points"]}))
    return 0


def kv_bytes_per_token(engine) -> int:
    return sum(2 * g.k.shape[0] * g.spec.kv_heads * g.spec.head_dim * g.k.element_size()
               for g in engine.cache.paged)


def shape_config(shape: dict, layers: int, name: str, extra: dict) -> dict:
    """The flat ``config`` entry of a record: every size, both layer counts."""
    out = {"model": f"{name} shape, random weights N(0,0.02) seed 0", "layers": layers,
           "layers_of_config": shape["num_hidden_layers"], "hidden": shape["hidden_size"],
           "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
           "head_dim": shape["hidden_size"] // shape["num_attention_heads"],
           "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
           "page_size": PAGE, "parallelism": "single GPU"}
    out.update(extra)
    return out


def timed_decode(engine, batch: int, prompt: int, k_steps: int, w_steps: int, rng, vocab: int,
                 portion: int = 2048):
    """Device-timed decode steps of ``batch`` requests whose prompts are in the cache, fed from
    the host with fixed tokens.  Returns (ms a step, launches, mean context, clocks)."""
    import torch
    from distengine_b200.engine.step import StepEntry
    from distengine_b200.kernels import ops
    runner = engine.runner
    ids = [f"d{batch}-{i}" for i in range(batch)]
    for rid in ids:                                       # prompts into the cache
        left = [int(t) for t in rng.integers(0, vocab, size=prompt)]
        while left:
            runner.step([StepEntry(rid, left[:portion], [])])
            left = left[portion:]
    feed = [[StepEntry(rid, [int(t)], [0]) for rid, t in zip(ids, row)]
            for row in rng.integers(0, vocab, size=(w_steps + k_steps, batch))]
    for entries in feed[:w_steps]:
        ops.sample_rows(runner.step(entries), engine.sampler.ids[:batch])
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    launches = ops.launch_count
    with ClockSampler() as sampler:
        start.record()
        for entries in feed[w_steps:]:
            ops.sample_rows(runner.step(entries), engine.sampler.ids[:batch])
        stop.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / k_steps
    launches = ops.launch_count - launches
    context = prompt + w_steps + (k_steps - 1) / 2 + 1
    for rid in ids:
        runner.release(rid)
    runner.check_status()
    return ms, launches, context, sampler.summary()


def timed_prefill(engine, length: int, rng, vocab: int, repeats: int = 5) -> "tuple[float, float]":
    """One prompt of ``length`` tokens in one step: (median milliseconds on the device, from the
    step's launch to its last kernel - CUDA events around ``StepRunner.launch``, the host's
    preparation of the step before them -, median milliseconds of the whole step by the host's
    clock, preparation included).  Five steps first: a step with prompt portions is replayed as a
    CUDA graph from its fifth coming on."""
    import torch
    from distengine_b200.engine.step import StepEntry
    runner = engine.runner

    def once():
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        entry = StepEntry("prefill", [int(t) for t in rng.integers(0, vocab, size=length)],
                          [length - 1])
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        prepared = runner.prepare([entry])
        start.record()
        runner.launch(prepared)
        stop.record()
        torch.cuda.synchronize()
        whole = (time.perf_counter() - t0) * 1e3
        runner.release("prefill")
        return start.elapsed_time(stop), whole

    for _ in range(5):
        once()
    runs = [once() for _ in range(repeats)]
    return statistics.median(r[0] for r in runs), statistics.median(r[1] for r in runs)


def prefill_flops(shape: dict, layers: int, layer_params: int, length: int, start: int = 0) -> int:
    """Flops of a prompt portion of ``length`` tokens that begins at position ``start``."""
    heads = shape["num_attention_heads"]
    head_dim = shape["hidden_size"] // heads
    keys = length * start + length * (length + 1) // 2
    return (2 * length * layer_params + 4 * head_dim * heads * keys * layers
            + 2 * shape["vocab_size"] * shape["hidden_size"])


def workload_fp32(args, warmup: int, steps: int) -> int:
    """The headline's sizes in the true 32-bit path: float32 weights, cache and activations, the
    FFMA matrix product and the CUDA-core attention, no tensor cores."""
    import numpy as np
    from distengine_b200 import Engine, EngineConfig
    peak, peak_kind = peaks()
    folder = model_folder(args.layers)
    rng = np.random.default_rng(0)
    vocab = MODEL["vocab_size"]
    pages = (args.batch * (PROMPT + 8 + warmup + steps) + PREFILL) // PAGE + 64
    engine = Engine(folder, EngineConfig(dtype="float32", block_size=PAGE, num_blocks=pages,
                                         decode_batch_size=max(args.batch, 8),
                                         max_batch_tokens=PREFILL,
                                         use_graphs=not args.no_graphs))
    w_bytes, layer_params = weight_bytes(engine.model)
    prefill_ms, prefill_step_ms = timed_prefill(engine, PREFILL, rng, vocab, repeats=3)
    ms, launches, context, clocks = timed_decode(engine, args.batch, PROMPT, steps, warmup, rng,
                                                 vocab)
    step_bytes = w_bytes + args.batch * context * kv_bytes_per_token(engine)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = prefill_flops(MODEL, args.layers, layer_params, PREFILL)
    print(json.dumps({
        "metric": "decode tokens/s at batch 8, true float32 path (TinyLlama-1.1B shape)",
        "value": round(args.batch / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4), "dtype": "fp32",
        "higher_is_better": True, "data": "synthetic", "impl": "ours", "workload": "fp32",
        "config": shape_config(MODEL, args.layers, "TinyLlama-1.1B", {
            "global_batch": args.batch, "seq_len": PROMPT, "peaks": peak_kind,
            "matrix_mode": "IEEE float32 FFMA, no TF32"}),
        "clocks": clocks, "gpu_launches": int(launches),
        "prefill": {"value": round(PREFILL / prefill_ms * 1e3, 1), "tokens": PREFILL,
                    "ms": round(prefill_ms, 3), "ms_with_host_prepare": round(prefill_step_ms, 3),
                    "tflops": round(flops / prefill_ms / 1e9, 2)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4)}}))
    return 0


def vomotar_shape(layers: int) -> dict:
    """A Vomotar model of the headline's width, feed-forward and vocabulary: every fourth layer
    runs chunk-masked attention beside retention, the others the gated delta rule."""
    delta = {"type": "channel_delta",
             "mixer": {"heads": 16, "kv_heads": 16, "dim": 128, "vdim": 128, "conv": 4,
                       "rank": 64},
             "mlp": {"kind": "dense", "ff": MODEL["intermediate_size"]}}
    parallel = {"type": "parallel",
                "mixer": {"left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128,
                                   "scale": 128 ** -0.5, "mask": {"size": 1024}},
                          "right": {"heads": 8, "dim": 128, "vdim": 256,
                                    "decay": [1.0 - 2.0 ** -(5 + i) for i in range(8)],
                                    "rot": {"dims": 64, "base": 10000.0}}},
                "mlp": {"kind": "dense", "ff": MODEL["intermediate_size"]}}
    return {"architecture": "Vomotar", "vocab": MODEL["vocab_size"],
            "width": MODEL["hidden_size"], "norm": {"eps": 1e-5, "groups": 1},
            "layers": [parallel if i % 4 == 0 else delta for i in range(layers)]}


def vomotar_folder(layers: int) -> str:
    from distengine_b200.weights import write_random_model
    folder = os.path.join(tempfile.gettempdir(), f"distengine_b200-bench-{os.getuid()}",
                          f"vomotar-shape-{layers}-layers-seed0-bf16")
    marker = os.path.join(folder, ".complete")
    if not os.path.isfile(marker):
        print("[bench] writing the random-weights model folder ...", file=sys.stderr, flush=True)
        write_random_model(vomotar_shape(layers), folder, seed=0, dtype="bfloat16",
                           norm_init="uniform")
        with open(marker, "w") as handle:
            handle.write("ok")
    return folder


def vomotar_kernels(peak: dict) -> list[dict]:
    """The design's own kernels alone, at the sizes of ``vomotar_shape``, for a prompt of 2,048
    tokens and for a decode step of 64 sequences: microseconds (CUDA events, L2 flushed before
    every launch), the bytes or flops they cannot avoid, and that against the measured peaks."""
    from types import SimpleNamespace
    import numpy as np
    import torch
    from distengine_b200.kernels import recurrent as rk
    from distengine_b200.kernels.attention_plan import build_plan
    dev, bf16, f32 = "cuda:0", torch.bfloat16, torch.float32
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fp32_peak = 148 * 128 * 2 * 1.965e9          # fused multiply-adds of the CUDA cores

    def ctx_of(lens, pos0):
        lens = np.asarray(lens, dtype=np.int32)
        pos0 = np.asarray(pos0, dtype=np.int32)
        qstart = (np.cumsum(lens) - lens).astype(np.int32)
        seq = np.repeat(np.arange(len(lens), dtype=np.int32), lens)
        slots = np.arange(len(lens), dtype=np.int32)
        pos = pos0[seq] + np.arange(lens.sum(), dtype=np.int32) - qstart[seq]
        d = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
        return SimpleNamespace(n_seqs=len(lens), token_seq=d(seq), token_slot=d(slots[seq]),
                               positions=d(pos), seq_slot=d(slots), seq_qstart=d(qstart),
                               seq_qlen=d(lens), seq_pos0=d(pos0),
                               host=SimpleNamespace(seq_qlen=lens, seq_pos0=pos0),
                               status=torch.zeros(1, dtype=torch.int32, device=dev))

    def timed(fn, repeats=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(repeats):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times)

    out = []

    def record(name, case, us, bytes_=0, flops=0):
        entry = {"kernel": name, "case": case, "us": round(us, 1)}
        hbm_us = bytes_ / (peak["hbm_gbs"] * 1e3)
        fma_us = flops / fp32_peak * 1e6
        entry["roofline_us"] = round(max(hbm_us, fma_us), 1)
        entry["bound"] = "hbm" if hbm_us >= fma_us else "fp32 fma"
        entry["frac"] = round(max(hbm_us, fma_us) / us, 3)
        out.append(entry)

    H, dk, dv, K, width = 16, 128, 128, 4, MODEL["hidden_size"]
    for case, lens, pos0 in (("prompt of 2,048", [2048], [0]), ("decode, 64 sequences", [1] * 64,
                                                                 [600] * 64)):
        ctx = ctx_of(lens, pos0)
        n, s = int(sum(lens)), len(lens)
        C = 2 * H * dk + H * dv
        proj = torch.randn(n, C + 16 + 128, device=dev).to(bf16)
        a = torch.randn(n, H * dk, device=dev)
        gate = torch.randn(n, H * dv, device=dev)
        taps = torch.randn(C, K, device=dev)
        state = torch.zeros(s, H * dk * dv + (K - 1) * C, device=dev)
        qn, kn, vv = (torch.empty(n, H * dk, device=dev) for _ in range(3))
        beta, gdec = torch.empty(n, H, device=dev), torch.empty(n, H * dk, device=dev)
        vec = torch.randn(H * dk, device=dev)
        us = timed(lambda: rk.delta_prep(proj, a, taps, vec, vec[:H].contiguous(), state,
                                         H * dk * dv, ctx, qn, kn, vv, beta, gdec, H, H, dk, dv, C))
        record("delta_prep", case, us, bytes_=n * (C * 2 + H * dk * 4 + (4 * H * dk) * 4))
        o = torch.empty(n, H * dv, device=dev)
        us = timed(lambda: rk.state_scan(qn, kn, vv, state, o, H, H, dk, dv, ctx, g=gdec, beta=beta))
        record("state_scan (delta rule)", case, us, bytes_=2 * s * H * dk * dv * 4 + n * 5 * H * dk * 4,
               flops=n * H * dk * dv * 8)
        gated = torch.empty(n, H * dv, dtype=bf16, device=dev)
        us = timed(lambda: rk.head_gate(o, gate, vec[:dv].contiguous(), gated, H, dv, 1e-5))
        record("head_gate", case, us, bytes_=n * H * dv * (4 + 4 + 2))
        # retention: 8 heads of 128 x 256
        RH, rdv = 8, 256
        rproj = torch.randn(n, 2 * RH * dk + 2 * RH * rdv, device=dev).to(bf16)
        rstate = torch.zeros(s, RH * dk * rdv, device=dev)
        qr, kr = torch.empty(n, RH * dk, device=dev), torch.empty(n, RH * dk, device=dev)
        inv = torch.rand(32, device=dev)
        us = timed(lambda: rk.retention_prep(rproj, inv, 64, RH, dk, qr, kr, ctx))
        record("retention_prep", case, us, bytes_=n * 2 * RH * dk * (2 + 4))
        ro = torch.empty(n, RH * rdv, device=dev)
        decay = torch.full((RH,), 0.99, device=dev)
        us = timed(lambda: rk.state_scan(qr, kr, rproj[:, 2 * RH * dk: 2 * RH * dk + RH * rdv],
                                         rstate, ro, RH, RH, dk, rdv, ctx, decay=decay))
        record("state_scan (retention)", case, us,
               bytes_=2 * s * RH * dk * rdv * 4 + n * (2 * RH * dk * 4 + RH * rdv * 6),
               flops=n * RH * dk * rdv * 5)
        # chunk attention: 16 heads on 4 kv heads, chunk 1,024
        AH, G, chunk, page = 16, 4, 1024, 16
        longest = max(p + l for p, l in zip(pos0, lens))
        pages_seq = (longest + page - 1) // page
        kp = torch.randn(s * pages_seq, G, page, dk, device=dev).to(bf16)
        vp = torch.randn(s * pages_seq, G, page, dv, device=dev).to(bf16)
        table = torch.arange(s * pages_seq, dtype=torch.int32, device=dev).view(s, pages_seq)
        aproj = torch.randn(n, AH * dk + G * (dk + dv), device=dev).to(bf16)
        us = timed(lambda: rk.kv_write_normed(aproj, AH * dk, G, dk, dv, 1e-5, kp, vp, table, ctx))
        record("kv_write_normed", case, us, bytes_=n * G * (dk + dv) * 4)
        rows = rk.chunk_rows_per_tile(bf16, dk, dv, n > s,
                                      rk.long_portion_rows(ctx.host.seq_qlen, AH, G))
        plan = build_plan(ctx.host.seq_qlen, ctx.host.seq_pos0, AH // G, G, rows, 0, chunk=0)
        items = torch.from_numpy(plan.items).to(dev)
        ao = torch.empty(n, AH * dv, dtype=bf16, device=dev)
        r = torch.rand(AH, device=dev)
        if n == s and rk.chunk_decode_ok(bf16, AH, G, dk, dv):      # as the mixer chooses
            us = timed(lambda: rk.chunk_attention_decode(aproj, ao, kp, vp, table, r, r, AH, G, dk,
                                                         dv, 0.09, chunk, ctx))
        else:
            us = timed(lambda: rk.chunk_attention(aproj, ao, kp, vp, table, items, r, r, AH, G, dk,
                                                  dv, 0.09, chunk, ctx, tile_rows=rows))
        keys = sum(sum(min(p + i, (p + i) % chunk) + 1 for i in range(l))
                   for p, l in zip(pos0, lens))
        record("chunk_attention", case, us,
               bytes_=sum(min(p + l, chunk + l) for p, l in zip(pos0, lens)) * G * (dk + dv) * 2,
               flops=2 * keys * AH * (dk + dv))
        x1 = torch.randn(n, width, device=dev).to(bf16)
        x2 = torch.randn(n, width, device=dev).to(bf16)
        w32 = torch.rand(width, device=dev)
        mo = torch.empty(n, width, dtype=bf16, device=dev)
        us = timed(lambda: rk.mean_of_normed(x1, x2, w32, w32, mo, 1e-5))
        record("mean_of_normed", case, us, bytes_=n * width * 6)
    return out


def workload_vomotar(args, warmup: int, steps: int) -> int:
    """Vomotar beside Llama at equal width, feed-forward, vocabulary and number of layers."""
    import numpy as np
    import torch
    from distengine_b200 import Engine, EngineConfig
    peak, peak_kind = peaks()
    layers = args.layers
    rng = np.random.default_rng(0)
    vocab = MODEL["vocab_size"]
    result = {}
    for name, folder in (("vomotar", vomotar_folder(layers)), ("llama", model_folder(layers))):
        pages = (64 * (PROMPT + 8 + warmup + steps) + PREFILL) // PAGE + 64
        engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=PAGE, num_blocks=pages,
                                             decode_batch_size=64, max_batch_tokens=PREFILL,
                                             max_model_len=4096, use_graphs=not args.no_graphs))
        prefill_ms, prefill_step_ms = timed_prefill(engine, PREFILL, rng, vocab, repeats=5)
        entry = {"prefill_2048": {"ms": round(prefill_ms, 3),
                                  "ms_with_host_prepare": round(prefill_step_ms, 3),
                                  "tokens_per_s": round(PREFILL / prefill_ms * 1e3, 1)}}
        for batch in (8, 64):
            ms, launches, _, clocks = timed_decode(engine, batch, PROMPT, steps, warmup, rng, vocab)
            entry[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4),
                                         "tokens_per_s": round(batch / ms * 1e3, 1),
                                         "gpu_launches": int(launches), "clocks": clocks}
        result[name] = entry
        del engine
        torch.cuda.empty_cache()
    mine = result["vomotar"]["decode_b8"]
    print(json.dumps({
        "metric": "decode tokens/s at batch 8, Vomotar at the TinyLlama-1.1B width",
        "value": mine["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": mine["ms_per_step"], "dtype": "bf16",
        "higher_is_better": True, "data": "synthetic", "impl": "ours", "workload": "vomotar",
        "config": {"layers": layers, "width": MODEL["hidden_size"],
                   "ff": MODEL["intermediate_size"], "vocab": vocab, "seq_len": PROMPT,
                   "page_size": PAGE, "peaks": peak_kind, "shape": vomotar_shape(4)["layers"][:2],
                   "l2": "weights larger than L2 are read every step; kernels alone: L2 flushed"},
        "gpu_launches": mine["gpu_launches"], "clocks": mine["clocks"],
        "models": result, "kernels": vomotar_kernels(peak)}))
    return 0


def sebilorn_shape(layers: int) -> dict:
    """A Sebilorn model of the headline's width, feed-forward and vocabulary: windowed attention, a
    layer that reads its keys and values, attention beside the generalized delta rule, lightning
    attention, in turn."""
    mlp = {"kind": "dense", "ff": MODEL["intermediate_size"]}
    rot = {"dims": 128, "base": 500000.0,
           "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}

    def attention(kv_from=None):
        mixer = {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                 "softcap": 30.0, "mask": {"size": 1024, "keep_first": 4}, "rot": rot}
        if kv_from is not None:
            mixer["kv_from"] = kv_from
        return {"type": "attention", "mixer": mixer, "mlp": mlp}

    parallel = {"type": "parallel",
                "mixer": {"left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128,
                                   "scale": 128 ** -0.5, "rot": {"dims": 64, "base": 10000.0}},
                          "right": {"heads": 16, "dim": 128, "rank": 64},
                          "left_scale": 0.5, "right_scale": 0.5},
                "mlp": mlp}
    lightning = {"type": "lightning",
                 "mixer": {"heads": 16, "dim": 128, "vdim": 128,
                           "decay": [1.0 - 2.0 ** -(4 + i % 8) for i in range(16)]},
                 "mlp": mlp}
    out = []
    for i in range(layers):
        out.append([attention(), attention(i - 1), parallel, lightning][i % 4])
    return {"architecture": "Sebilorn", "vocab": MODEL["vocab_size"],
            "width": MODEL["hidden_size"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "logit_softcap": 30.0, "layers": out}


def sebilorn_folder(layers: int) -> str:
    from distengine_b200.weights import write_random_model
    folder = os.path.join(tempfile.gettempdir(), f"distengine_b200-bench-{os.getuid()}",
                          f"sebilorn-shape-{layers}-layers-seed0-bf16")
    marker = os.path.join(folder, ".complete")
    if not os.path.isfile(marker):
        print("[bench] writing the random-weights model folder ...", file=sys.stderr, flush=True)
        write_random_model(sebilorn_shape(layers), folder, seed=0, dtype="bfloat16",
                           norm_init="uniform")
        with open(marker, "w") as handle:
            handle.write("ok")
    return folder


def sebilorn_kernels(peak: dict) -> list[dict]:
    """The design's kernels alone at the sizes of ``sebilorn_shape``, for a prompt of 2,048 tokens
    and for a decode step of 64 sequences, as ``vomotar_kernels`` measures its own; the norm and
    the activation are measured beside the RMS norm and silu * up of the other models."""
    from types import SimpleNamespace
    import numpy as np
    import torch
    from distengine_b200.kernels import ops
    from distengine_b200.kernels import recurrent as rk
    from distengine_b200.kernels.attention_plan import build_plan
    from distengine_b200.parts.window_attention import rotary_frequencies
    dev, bf16, f32 = "cuda:0", torch.bfloat16, torch.float32
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fp32_peak = 148 * 128 * 2 * 1.965e9          # fused multiply-adds of the CUDA cores

    def ctx_of(lens, pos0):
        lens = np.asarray(lens, dtype=np.int32)
        pos0 = np.asarray(pos0, dtype=np.int32)
        qstart = (np.cumsum(lens) - lens).astype(np.int32)
        seq = np.repeat(np.arange(len(lens), dtype=np.int32), lens)
        slots = np.arange(len(lens), dtype=np.int32)
        pos = pos0[seq] + np.arange(lens.sum(), dtype=np.int32) - qstart[seq]
        d = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
        return SimpleNamespace(n_seqs=len(lens), token_seq=d(seq), token_slot=d(slots[seq]),
                               positions=d(pos), seq_slot=d(slots), seq_qstart=d(qstart),
                               seq_qlen=d(lens), seq_pos0=d(pos0),
                               host=SimpleNamespace(seq_qlen=lens, seq_pos0=pos0),
                               status=torch.zeros(1, dtype=torch.int32, device=dev))

    def timed(fn, repeats=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(repeats):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times)

    out = []

    def record(name, case, us, bytes_=0, flops=0, like=""):
        entry = {"kernel": name, "case": case, "us": round(us, 1), "like": like}
        hbm_us = bytes_ / (peak["hbm_gbs"] * 1e3)
        fma_us = flops / fp32_peak * 1e6
        entry["roofline_us"] = round(max(hbm_us, fma_us), 1)
        entry["bound"] = "hbm" if hbm_us >= fma_us else "fp32 fma"
        entry["frac"] = round(max(hbm_us, fma_us) / us, 3)
        out.append(entry)

    H, G, dk, dv, width, ff = 16, 4, 128, 128, MODEL["hidden_size"], MODEL["intermediate_size"]
    window, keep, page = 1024, 4, 16
    for case, lens, pos0 in (("prompt of 2,048", [2048], [0]), ("decode, 64 sequences", [1] * 64,
                                                                 [600] * 64)):
        ctx = ctx_of(lens, pos0)
        n, s = int(sum(lens)), len(lens)
        # norms: the layer norm beside the RMS norm
        resid = torch.randn(n, width, device=dev)
        delta = torch.randn(n, width, device=dev).to(bf16)
        wv, bv = torch.rand(width, device=dev).to(bf16), torch.rand(width, device=dev).to(bf16)
        normed = torch.empty(n, width, dtype=bf16, device=dev)
        us = timed(lambda: ops.add_layernorm(resid, delta, wv, bv, 1e-5, normed))
        record("add_layernorm", case, us, bytes_=n * width * (4 + 4 + 2 + 2), like="add_rmsnorm")
        us = timed(lambda: ops.add_rmsnorm(resid, delta, wv, 1e-5, normed))
        record("add_rmsnorm (other models)", case, us, bytes_=n * width * (4 + 4 + 2 + 2))
        # activations: the squared relu beside silu * up
        up = torch.randn(n, 2 * ff, device=dev).to(bf16)
        act = torch.empty(n, ff, dtype=bf16, device=dev)
        us = timed(lambda: ops.activation(up[:, :ff], act, "relu2"))
        record("activation (squared relu)", case, us, bytes_=n * ff * 4, like="silu_mul")
        us = timed(lambda: ops.silu_mul(up, act))
        record("silu_mul (other models)", case, us, bytes_=n * ff * 6)
        # windowed attention: 16 heads on 4 kv heads, window 1,024, 4 kept tokens
        longest = max(p + l for p, l in zip(pos0, lens))
        pages_seq = (longest + page - 1) // page
        kp = torch.randn(s * pages_seq, G, page, dk, device=dev).to(bf16)
        vp = torch.randn(s * pages_seq, G, page, dv, device=dev).to(bf16)
        table = torch.arange(s * pages_seq, dtype=torch.int32, device=dev).view(s, pages_seq)
        aproj = torch.randn(n, H * dk + G * (dk + dv) + H * dv, device=dev).to(bf16)
        fk = rotary_frequencies(500000.0, dk, (8.0, 1.0, 4.0, 8192)).to(dev)
        fv = rotary_frequencies(500000.0, dv).to(dev)
        us = timed(lambda: rk.kv_write_rotated(aproj, fk, dk, fv, H, G, dk, dv, kp, vp, table,
                                               True, ctx))
        record("kv_write_rotated", case, us, bytes_=n * (2 * H * dk + 2 * G * (dk + dv)) * 2,
               like="kv_write_normed")
        rows = rk.chunk_rows_per_tile(bf16, dk, dv, n > s,
                                      rk.long_portion_rows(ctx.host.seq_qlen, H, G))
        plan = build_plan(ctx.host.seq_qlen, ctx.host.seq_pos0, H // G, G, rows, 0, chunk=0)
        items = torch.from_numpy(plan.items).to(dev)
        raw = torch.empty(n, H * dv, device=dev)
        sight = dict(window=window, keep_first=keep, softcap=30.0)
        if n == s and rk.chunk_decode_ok(bf16, H, G, dk, dv):      # as the mixer chooses
            us = timed(lambda: rk.chunk_attention_decode(aproj, raw, kp, vp, table, None, None, H,
                                                         G, dk, dv, 0.09, 0, ctx, **sight))
        else:
            us = timed(lambda: rk.chunk_attention(aproj, raw, kp, vp, table, items, None, None, H,
                                                  G, dk, dv, 0.09, 0, ctx, tile_rows=rows,
                                                  **sight))
        keys = sum(sum(min(p + i + 1, window + keep) for i in range(l))
                   for p, l in zip(pos0, lens))
        record("window_attention", case, us,
               bytes_=sum(min(p + l, window + keep + l) for p, l in zip(pos0, lens))
               * G * (dk + dv) * 2, flops=2 * keys * H * (dk + dv), like="chunk_attention")
        ao = torch.empty(n, H * dv, dtype=bf16, device=dev)
        gate = aproj[:, H * dk + G * (dk + dv):]
        us = timed(lambda: rk.attention_finish(raw, fv, gate, ao, H, dv, ctx))
        record("attention_finish", case, us, bytes_=n * H * dv * (4 + 2 + 2), like="head_gate")
        # the generalized delta rule: 16 heads of 128 x 128
        rows_ = H * dk
        dproj = torch.randn(n, 5 * rows_ + 64, device=dev).to(bf16)
        wl = torch.randn(n, rows_, device=dev)
        vec = torch.randn(rows_, device=dev)
        rr, kk, ww, zz = (torch.empty(n, rows_, device=dev) for _ in range(4))
        dots = torch.empty(n, 2 * H, device=dev)
        us = timed(lambda: rk.gdelta_prep(dproj, 0, rows_, 4 * rows_, wl, vec, vec, rr, kk, ww, zz,
                                          dots, H, dk))
        record("gdelta_prep", case, us, bytes_=n * rows_ * (3 * 2 + 4 + 4 * 4), like="delta_prep")
        state = torch.zeros(s, H * dk * dk, device=dev)
        o = torch.empty(n, rows_, device=dev)
        us = timed(lambda: rk.state_scan(rr, kk, dproj[:, 2 * rows_: 3 * rows_], state, o, H, H,
                                         dk, dk, ctx, g=ww, z=zz, dots=dots))
        record("state_scan (generalized delta rule)", case, us,
               bytes_=2 * s * H * dk * dk * 4 + n * rows_ * (4 * 4 + 2 + 4),
               flops=n * H * dk * dk * 9, like="state_scan (delta rule)")
        gated = torch.empty(n, rows_, dtype=bf16, device=dev)
        us = timed(lambda: rk.head_gate(o, dproj[:, 3 * rows_: 4 * rows_], vec, gated, H, dk, 1e-5,
                                        spanning=True))
        record("head_gate (weight over the heads)", case, us, bytes_=n * rows_ * (4 + 2 + 2),
               like="head_gate")
        us = timed(lambda: rk.head_gate(o, dproj[:, 3 * rows_: 4 * rows_], vec, gated, 1, rows_,
                                        1e-5, spanning=True))
        record("head_gate (one norm a row)", case, us, bytes_=n * rows_ * (4 + 2 + 2),
               like="head_gate")
        # lightning attention: silu of q, k, v, then the scan with a decay per head
        qkv = torch.empty(n, 3 * rows_, device=dev)
        us = timed(lambda: rk.silu_rows(dproj[:, : 3 * rows_], qkv))
        record("silu_rows", case, us, bytes_=n * 3 * rows_ * (2 + 4), like="retention_prep")
        decay = torch.full((H,), 0.99, device=dev)
        us = timed(lambda: rk.state_scan(qkv[:, :rows_], qkv[:, rows_: 2 * rows_],
                                         qkv[:, 2 * rows_:], state, o, H, H, dk, dk, ctx,
                                         decay=decay))
        record("state_scan (lightning)", case, us,
               bytes_=2 * s * H * dk * dk * 4 + n * rows_ * 4 * 4, flops=n * H * dk * dk * 5,
               like="state_scan (retention)")
        a32, b32 = torch.randn(n, width, device=dev), torch.randn(n, width, device=dev)
        mo = torch.empty(n, width, dtype=bf16, device=dev)
        us = timed(lambda: ops.scaled_sum(a32, b32, 0.5, 0.5, mo))
        record("scaled_sum", case, us, bytes_=n * width * 10, like="mean_of_normed")
    return out


def workload_sebilorn(args, warmup: int, steps: int) -> int:
    """Sebilorn beside Vomotar and Llama at equal width, feed-forward, vocabulary and number of
    layers."""
    import numpy as np
    import torch
    from distengine_b200 import Engine, EngineConfig
    peak, peak_kind = peaks()
    layers = args.layers
    rng = np.random.default_rng(0)
    vocab = MODEL["vocab_size"]
    result = {}
    for name, folder in (("sebilorn", sebilorn_folder(layers)),
                         ("vomotar", vomotar_folder(layers)), ("llama", model_folder(layers))):
        pages = (64 * (PROMPT + 8 + warmup + steps) + PREFILL) // PAGE + 64
        engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=PAGE, num_blocks=pages,
                                             decode_batch_size=64, max_batch_tokens=PREFILL,
                                             max_model_len=4096, use_graphs=not args.no_graphs))
        prefill_ms, prefill_step_ms = timed_prefill(engine, PREFILL, rng, vocab, repeats=5)
        entry = {"prefill_2048": {"ms": round(prefill_ms, 3),
                                  "ms_with_host_prepare": round(prefill_step_ms, 3),
                                  "tokens_per_s": round(PREFILL / prefill_ms * 1e3, 1)}}
        for batch in (8, 64):
            ms, launches, _, clocks = timed_decode(engine, batch, PROMPT, steps, warmup, rng, vocab)
            entry[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4),
                                         "tokens_per_s": round(batch / ms * 1e3, 1),
                                         "gpu_launches": int(launches), "clocks": clocks}
        result[name] = entry
        del engine
        torch.cuda.empty_cache()
    mine = result["sebilorn"]["decode_b8"]
    print(json.dumps({
        "metric": "decode tokens/s at batch 8, Sebilorn at the TinyLlama-1.1B width",
        "value": mine["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": mine["ms_per_step"], "dtype": "bf16",
        "higher_is_better": True, "data": "synthetic", "impl": "ours", "workload": "sebilorn",
        "config": {"layers": layers, "width": MODEL["hidden_size"],
                   "ff": MODEL["intermediate_size"], "vocab": vocab, "seq_len": PROMPT,
                   "page_size": PAGE, "peaks": peak_kind, "shape": sebilorn_shape(4)["layers"],
                   "l2": "weights larger than L2 are read every step; kernels alone: L2 flushed"},
        "gpu_launches": mine["gpu_launches"], "clocks": mine["clocks"],
        "models": result, "kernels": sebilorn_kernels(peak),
        "kernels_vomotar": vomotar_kernels(peak)}))
    return 0


def vapelix_shape(layers: int) -> dict:
    """A Vapelix model of the headline's width and vocabulary: latent attention (16 heads of 128
    plain and 64 rotated query/key features, a latent of 192, so that a cached row of 256
    features fits the tensor-core attention kernels) in every layer, beside a gated dense
    feed-forward of the headline's size in every fourth layer and 16 routed experts, 4 a token,
    in the others (as many active feed-forward weights as the dense layers have); the token's
    side input after every layer.  No loop, so that the layer runs equal the other models'."""
    rot = {"dims": 64, "base": 10000.0,
           "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    mixer = {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": 768, "kv_rank": 192,
             "scale": 192 ** -0.5, "rot": rot}
    dense = {"kind": "dense", "ff": MODEL["intermediate_size"]}
    routed = {"kind": "moe", "expert": {"ff": 2048}, "router": {"experts": 16, "top": 4}}
    return {"architecture": "Vapelix", "vocab": MODEL["vocab_size"], "width": MODEL["hidden_size"],
            "norm": {"eps": 1e-6}, "token_side": {"dim": 64},
            "layers": [{"type": "latent_attention", "mixer": mixer,
                        "mlp": dense if i % 4 == 0 else routed} for i in range(layers)]}


def vapelix_folder(layers: int) -> str:
    from distengine_b200.weights import write_random_model
    folder = os.path.join(tempfile.gettempdir(), f"distengine_b200-bench-{os.getuid()}",
                          f"vapelix-shape-{layers}-layers-seed0-bf16")
    marker = os.path.join(folder, ".complete")
    if not os.path.isfile(marker):
        print("[bench] writing the random-weights model folder ...", file=sys.stderr, flush=True)
        write_random_model(vapelix_shape(layers), folder, seed=0, dtype="bfloat16",
                           norm_init="uniform")
        with open(marker, "w") as handle:
            handle.write("ok")
    return folder


def vapelix_kernels(peak: dict) -> list[dict]:
    """The design's kernels alone at the sizes of ``vapelix_shape``, for a prompt of 2,048 tokens
    and for a decode step of 64 sequences at position 600, each beside the like kernel of the
    other models at the like size (``like``): attention over the latent beside attention over
    keys and values of 4 heads of 128, the experts' products beside the dense products of as many
    active weights, the per-head products beside a dense product of as many flops."""
    from types import SimpleNamespace
    import numpy as np
    import torch
    from distengine_b200.kernels import latent as lk
    from distengine_b200.kernels import ops
    from distengine_b200.kernels import recurrent as rk
    from distengine_b200.kernels.attention_plan import build_plan
    from distengine_b200.parts.latent_attention import stretched_frequencies
    dev, bf16, f32 = "cuda:0", torch.bfloat16, torch.float32
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fp32_peak = 148 * 128 * 2 * 1.965e9          # fused multiply-adds of the CUDA cores
    tensor_peak = peak["bf16_tflops"] * 1e12

    def ctx_of(lens, pos0):
        lens = np.asarray(lens, dtype=np.int32)
        pos0 = np.asarray(pos0, dtype=np.int32)
        qstart = (np.cumsum(lens) - lens).astype(np.int32)
        seq = np.repeat(np.arange(len(lens), dtype=np.int32), lens)
        slots = np.arange(len(lens), dtype=np.int32)
        pos = pos0[seq] + np.arange(lens.sum(), dtype=np.int32) - qstart[seq]
        d = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
        return SimpleNamespace(n_seqs=len(lens), token_seq=d(seq), token_slot=d(slots[seq]),
                               positions=d(pos), seq_slot=d(slots), seq_qstart=d(qstart),
                               seq_qlen=d(lens), seq_pos0=d(pos0),
                               host=SimpleNamespace(seq_qlen=lens, seq_pos0=pos0),
                               status=torch.zeros(1, dtype=torch.int32, device=dev))

    def timed(fn, repeats=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(repeats):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times)

    out = []

    def record(name, case, us, bytes_=0, flops=0, tensor_flops=0, like=""):
        entry = {"kernel": name, "case": case, "us": round(us, 1), "like": like}
        bounds = {"hbm": bytes_ / (peak["hbm_gbs"] * 1e3), "fp32 fma": flops / fp32_peak * 1e6,
                  "tensor": tensor_flops / tensor_peak * 1e6}
        entry["bound"] = max(bounds, key=bounds.get)
        entry["roofline_us"] = round(bounds[entry["bound"]], 1)
        entry["frac"] = round(bounds[entry["bound"]] / us, 3)
        out.append(entry)
    shape = vapelix_shape(2)
    m, routed = shape["layers"][0]["mixer"], shape["layers"][1]["mlp"]
    H, dim, rot, dv, qr, rank = (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"],
                                 m["kv_rank"])
    row, width, ff = rank + rot, MODEL["hidden_size"], MODEL["intermediate_size"]
    E, top, eff, side = (routed["router"]["experts"], routed["router"]["top"],
                         routed["expert"]["ff"], shape["token_side"]["dim"])
    page = PAGE
    sc = m["rot"]["scaling"]
    freq, magnitude = stretched_frequencies(m["rot"]["base"], rot, (sc["factor"], sc["original"],
                                                                    sc["fast"], sc["slow"]))
    freq = freq.to(dev)
    w = lambda *s: (torch.randn(*s, device=dev) / s[-1] ** 0.5).to(bf16)
    for case, lens, pos0 in (("prompt of 2,048", [2048], [0]), ("decode, 64 sequences", [1] * 64,
                                                                 [600] * 64)):
        ctx = ctx_of(lens, pos0)
        n, s = int(sum(lens)), len(lens)
        longest = max(p + l for p, l in zip(pos0, lens))
        pages_seq = (longest + page - 1) // page
        table = torch.arange(s * pages_seq, dtype=torch.int32, device=dev).view(s, pages_seq)
        keys = sum(sum(p + i + 1 for i in range(l)) for p, l in zip(pos0, lens))
        read = sum(p + l for p, l in zip(pos0, lens))
        # ---- latent attention
        q = torch.randn(n, H * (dim + rot), device=dev).to(bf16)
        kv = torch.randn(n, row, device=dev).to(bf16)
        folded = torch.empty(n, H * row, dtype=bf16, device=dev)
        pages = torch.randn(s * pages_seq, 1, page, row, device=dev).to(bf16)
        n_kv = torch.rand(rank, device=dev).to(bf16)
        us = timed(lambda: lk.latent_write(q, kv, folded, freq, magnitude, n_kv, 1e-6, H, dim, rot,
                                           rank, pages, table, ctx))
        record("latent_write", case, us, bytes_=n * (H * rot * 4 + 2 * row * 2),
               like="kv_write_rotated")
        w_uk_t, w_uv = w(H, rank, dim), w(H, dv, rank)
        us = timed(lambda: lk.heads_product(q, dim + rot, w_uk_t, folded, row))
        record("heads_product (keys folded into the query)", case, us,
               bytes_=n * H * (dim + rank) * 2 + H * rank * dim * 2, flops=2 * n * H * dim * rank,
               like="linear")
        mixed = torch.empty(n, H * rank, device=dev)
        sums, a_head = mixed, rank
        if n == s and rk.chunk_decode_ok(bf16, H, 1, row, rank, True):
            us = timed(lambda: rk.chunk_attention_decode(folded, mixed, pages, pages, table, None,
                                                         None, H, 1, row, rank, m["scale"], 0, ctx,
                                                         v_stride=row))
            record("attention over the latent (single tokens)", case, us,
                   bytes_=read * row * 2 + n * H * (row * 2 + rank * 4),
                   flops=2 * keys * H * (row + rank), like="attention, 4 key/value heads of 128")
        else:
            # prompt portions: the tensor-core kernels, one key/value head of `row` features
            from distengine_b200.kernels.attention import AttentionLauncher
            from distengine_b200.parts.context import StepPrep, Workspace
            launcher = AttentionLauncher(bf16, H, 1, row, m["scale"], None)
            prep = StepPrep(SimpleNamespace(seq_qlen=ctx.host.seq_qlen, seq_pos0=ctx.host.seq_pos0))
            launcher.prepare(prep, allow_decode=False)
            workspace = Workspace(torch.device(dev))
            ctx.notes = prep.notes
            ctx.arrays = {k: torch.from_numpy(np.ascontiguousarray(v, dtype=np.int32)).to(dev)
                          for k, v in prep.extra.items()}
            ctx.buffer = lambda name, shape, dt=None: workspace.get(name, shape, dt or bf16)
            sums, a_head = torch.empty(n, H * row, dtype=bf16, device=dev), row
            us = timed(lambda: launcher.run(folded, sums, pages, pages, table, ctx))
            record("attention over the latent (tensor cores)", case, us,
                   bytes_=read * row * 2 + n * H * row * 4, tensor_flops=2 * keys * H * 2 * row,
                   like="attention, 4 key/value heads of 128")
            rows = rk.chunk_rows_per_tile(bf16, row, rank, n > s,
                                          rk.long_portion_rows(ctx.host.seq_qlen, H, 1))
            plan = build_plan(ctx.host.seq_qlen, ctx.host.seq_pos0, H, 1, rows, 0, chunk=0)
            items = torch.from_numpy(plan.items).to(dev)
            us = timed(lambda: rk.chunk_attention(folded, mixed, pages, pages, table, items, None,
                                                  None, H, 1, row, rank, m["scale"], 0, ctx,
                                                  tile_rows=rows, v_stride=row))
            record("attention over the latent (CUDA cores: float32, other row sizes)", case, us,
                   bytes_=read * row * 2 + n * H * (row * 2 + rank * 4),
                   flops=2 * keys * H * (row + rank), like="attention, 4 key/value heads of 128")
        # the like kernel: 16 heads on 4 key/value heads of 128, every earlier token seen
        G, dk = 4, 128
        kp = torch.randn(s * pages_seq, G, page, dk, device=dev).to(bf16)
        vp = torch.randn(s * pages_seq, G, page, dk, device=dev).to(bf16)
        aq = torch.randn(n, H * dk, device=dev).to(bf16)
        raw = torch.empty(n, H * dk, device=dev)
        if n == s and rk.chunk_decode_ok(bf16, H, G, dk, dk):
            us = timed(lambda: rk.chunk_attention_decode(aq, raw, kp, vp, table, None, None, H, G,
                                                         dk, dk, 0.09, 0, ctx))
            record("attention, 4 key/value heads of 128 (other models)", case, us,
                   bytes_=read * G * 2 * dk * 2 + n * H * dk * 6, flops=2 * keys * H * 2 * dk)
        else:
            like = AttentionLauncher(bf16, H, G, dk, 0.09, None)
            prep = StepPrep(SimpleNamespace(seq_qlen=ctx.host.seq_qlen, seq_pos0=ctx.host.seq_pos0))
            like.prepare(prep, allow_decode=False)
            ctx.notes = prep.notes
            ctx.arrays = {k: torch.from_numpy(np.ascontiguousarray(v, dtype=np.int32)).to(dev)
                          for k, v in prep.extra.items()}
            ao = torch.empty(n, H * dk, dtype=bf16, device=dev)
            us = timed(lambda: like.run(aq, ao, kp, vp, table, ctx))
            record("attention, 4 key/value heads of 128 (other models, tensor cores)", case, us,
                   bytes_=read * G * 2 * dk * 2 + n * H * dk * 4,
                   tensor_flops=2 * keys * H * 2 * dk)
        gate = torch.randn(n, H * dv, device=dev).to(bf16)
        context = torch.empty(n, H * dv, dtype=bf16, device=dev)
        us = timed(lambda: lk.heads_product(sums, a_head, w_uv, context, dv, gate=gate))
        record("heads_product (values, gated)", case, us,
               bytes_=n * H * (rank * 4 + dv * 4) + H * rank * dv * 2, flops=2 * n * H * dv * rank,
               like="linear")
        x = torch.randn(n, width, device=dev).to(bf16)
        w_like = w(H * rank, width)
        y_like = torch.empty(n, H * rank, dtype=bf16, device=dev)
        us = timed(lambda: ops.linear(x, w_like, out=y_like))
        record("linear, 2,048 to 4,096 features (other models)", case, us,
               bytes_=(n * (width + H * rank) + H * rank * width) * 2,
               tensor_flops=2 * n * width * H * rank)
        # ---- routed experts: 16 experts of 2,048 inner features, 4 a token
        router, bias = torch.randn(E, width, device=dev) / width ** 0.5, torch.zeros(E, device=dev)
        up, down = w(E, eff, width), w(E, width, eff)
        tensor = lk.experts_tensor_ok(x, up, n * top)
        seg = lk.SEGMENT_TENSOR if tensor else lk.SEGMENT
        tiles = lk.experts_tiles(n, top, E, seg)
        chosen = torch.empty(n, top, dtype=torch.int32, device=dev)
        weight = torch.empty(n, top, device=dev)
        pair_of = torch.empty(tiles * seg, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(tiles, dtype=torch.int32, device=dev)
        slot_of = torch.empty(n * top, dtype=torch.int32, device=dev)
        inner = torch.empty(tiles * seg, eff, dtype=bf16, device=dev)
        rows_ = torch.empty(tiles * seg, width, dtype=bf16, device=dev)
        y = torch.empty(n * top, width, dtype=bf16, device=dev)
        eo = torch.empty(n, width, device=dev)
        us = timed(lambda: lk.experts_route(x, router, bias, top, chosen, weight))
        record("experts_route", case, us, bytes_=n * width * 2 + E * width * 4,
               flops=2 * n * E * width, like="linear")
        us = timed(lambda: lk.experts_group(chosen, E, pair_of, tile_expert, slot_of, seg))
        record("experts_group", case, us, bytes_=n * top * 12 + tiles * seg * 4)
        used = int((tile_expert >= 0).sum())
        weights_read = min(E, n * top) * eff * width * 2
        if tensor:
            us = timed(lambda: lk.experts_gather(x, pair_of, top, rows_))
            record("experts_gather", case, us, bytes_=n * top * width * 4)
            us = timed(lambda: lk.experts_product(rows_, up, pair_of, tile_expert, inner, False,
                                                  "gelu_erf", ctx.status))
            record("experts up (tensor cores)", case, us,
                   bytes_=weights_read + n * top * (width + eff) * 2,
                   tensor_flops=2 * n * top * width * eff, like="linear_gated")
            us = timed(lambda: lk.experts_product(inner, down, pair_of, tile_expert, y, True, None,
                                                  ctx.status))
            record("experts down (tensor cores)", case, us,
                   bytes_=weights_read + n * top * (width + eff) * 2,
                   tensor_flops=2 * n * top * width * eff, like="linear")
        else:
            us = timed(lambda: lk.experts_up(x, up, pair_of, tile_expert, top, inner, "gelu_erf"))
            record("experts up (CUDA cores)", case, us,
                   bytes_=weights_read + n * top * (width + eff) * 2,
                   flops=2 * used * seg * width * eff, like="linear_gated")
            us = timed(lambda: lk.experts_down(inner, down, pair_of, tile_expert, y))
            record("experts down (CUDA cores)", case, us,
                   bytes_=weights_read + n * top * (width + eff) * 2,
                   flops=2 * used * seg * width * eff, like="linear")
        us = timed(lambda: lk.experts_combine(y, weight, eo))
        record("experts_combine", case, us, bytes_=n * width * (top * 2 + 4), like="residual_add")
        # the like kernels: the dense gated feed-forward of the other models
        w_gu, w_d = w(2 * ff, width), w(width, ff)
        act = torch.empty(n, ff, dtype=bf16, device=dev)
        yd = torch.empty(n, width, dtype=bf16, device=dev)
        us = timed(lambda: ops.linear_gated(x, w_gu, act, status=ctx.status))
        record("linear_gated (other models)", case, us,
               bytes_=(2 * ff * width + n * (width + ff)) * 2, tensor_flops=4 * n * width * ff)
        us = timed(lambda: ops.linear(act, w_d, out=yd))
        record("linear, down (other models)", case, us,
               bytes_=(ff * width + n * (width + ff)) * 2, tensor_flops=2 * n * width * ff)
        # ---- the token's side input
        table_rows = torch.randn(MODEL["vocab_size"], side, device=dev).to(bf16)
        ids = torch.randint(0, MODEL["vocab_size"], (n,), dtype=torch.int32, device=dev)
        z = torch.randn(n, side, device=dev).to(bf16)
        us = timed(lambda: ops.act_mul_row(z, ids, table_rows, z, "gelu_tanh"))
        record("act_mul_row", case, us, bytes_=n * side * 6, like="silu_mul")
        resid = torch.randn(n, width, device=dev)
        us = timed(lambda: ops.add_normed(resid, yd, n_kv.new_ones(width), 1e-6))
        record("add_normed", case, us, bytes_=n * width * (4 + 4 + 2), like="add_rmsnorm")
        normed = torch.empty(n, width, dtype=bf16, device=dev)
        us = timed(lambda: ops.add_rmsnorm(resid, yd, n_kv.new_ones(width), 1e-6, normed))
        record("add_rmsnorm (other models)", case, us, bytes_=n * width * (4 + 4 + 2 + 2))
    return out


def workload_vapelix(args, warmup: int, steps: int) -> int:
    """Vapelix beside Llama at equal width, vocabulary and number of layers (and as many active
    feed-forward weights a token)."""
    import numpy as np
    import torch
    from distengine_b200 import Engine, EngineConfig
    peak, peak_kind = peaks()
    layers = args.layers
    rng = np.random.default_rng(0)
    vocab = MODEL["vocab_size"]
    result = {}
    for name, folder in (("vapelix", vapelix_folder(layers)), ("llama", model_folder(layers))):
        pages = (64 * (PROMPT + 8 + warmup + steps) + PREFILL) // PAGE + 64
        engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=PAGE, num_blocks=pages,
                                             decode_batch_size=64, max_batch_tokens=PREFILL,
                                             max_model_len=4096, use_graphs=not args.no_graphs))
        prefill_ms, prefill_step_ms = timed_prefill(engine, PREFILL, rng, vocab, repeats=5)
        entry = {"prefill_2048": {"ms": round(prefill_ms, 3),
                                  "ms_with_host_prepare": round(prefill_step_ms, 3),
                                  "tokens_per_s": round(PREFILL / prefill_ms * 1e3, 1)}}
        for batch in (8, 64):
            ms, launches, _, clocks = timed_decode(engine, batch, PROMPT, steps, warmup, rng, vocab)
            entry[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4),
                                         "tokens_per_s": round(batch / ms * 1e3, 1),
                                         "gpu_launches": int(launches), "clocks": clocks}
        result[name] = entry
        del engine
        torch.cuda.empty_cache()
    mine = result["vapelix"]["decode_b8"]
    print(json.dumps({
        "metric": "decode tokens/s at batch 8, Vapelix at the TinyLlama-1.1B width",
        "value": mine["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": mine["ms_per_step"], "dtype": "bf16",
        "higher_is_better": True, "data": "synthetic", "impl": "ours", "workload": "vapelix",
        "config": {"layers": layers, "width": MODEL["hidden_size"],
                   "ff": MODEL["intermediate_size"], "vocab": vocab, "seq_len": PROMPT,
                   "page_size": PAGE, "peaks": peak_kind, "shape": vapelix_shape(2)["layers"],
                   "l2": "weights larger than L2 are read every step; kernels alone: L2 flushed"},
        "gpu_launches": mine["gpu_launches"], "clocks": mine["clocks"],
        "models": result, "kernels": [] if args.only == "decode" else vapelix_kernels(peak)}))
    return 0


def bizetar_shape(layers: int) -> dict:
    """A Bizetar model of the headline's width and vocabulary: 16 query heads on 4 key/value heads
    of 128 features (keys and values) in every layer; three layers in four are the form with
    biases, a convolution of 3 taps, norms per head and stretched rotation, every fourth the form
    with norms over the whole projection, a distance bias and a query that grows; a dense
    feed-forward of the headline's size in every fourth layer and 16 gated experts of 1,024 inner
    features beside 4 outputs that hand the input on, 4 a token, in the others (about as many
    active feed-forward weights as the dense layers have).  Every layer mixes values."""
    rot = {"dims": 128, "base": 100000.0,
           "scaling": {"factor": 16.0, "original": 4096, "fast": 16.0, "slow": 2.0}}
    common = {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
              "v_mix": True}
    second = {"type": "attention_2", "mixer": dict(common, conv=3, rot=rot)}
    first = {"type": "attention", "mixer": dict(common, q_temp={"coef": 0.3, "every": 256})}
    dense = {"kind": "dense", "ff": MODEL["intermediate_size"]}
    routed = {"kind": "moe", "expert": {"ff": 1024},
              "router": {"experts": 16, "top": 4, "identity": 4}}
    return {"architecture": "Bizetar", "vocab": MODEL["vocab_size"], "width": MODEL["hidden_size"],
            "norm": {"eps": 1e-5},
            "layers": [dict(first if i % 4 == 2 else second, mlp=dense if i % 4 == 0 else routed)
                       for i in range(layers)]}


def bizetar_folder(layers: int) -> str:
    from distengine_b200.weights import write_random_model
    folder = os.path.join(tempfile.gettempdir(), f"distengine_b200-bench-{os.getuid()}",
                          f"bizetar-shape-{layers}-layers-seed0-bf16")
    marker = os.path.join(folder, ".complete")
    if not os.path.isfile(marker):
        print("[bench] writing the random-weights model folder ...", file=sys.stderr, flush=True)
        write_random_model(bizetar_shape(layers), folder, seed=0, dtype="bfloat16",
                           norm_init="uniform")
        with open(marker, "w") as handle:
            handle.write("ok")
    return folder


def bizetar_kernels(peak: dict) -> list[dict]:
    """The design's kernels alone at the sizes of ``bizetar_shape``, for a prompt of 2,048 tokens
    and for a decode step of 64 sequences at position 600, each beside the like kernel of the
    closest models, measured in the same run (``like``): the attention with sink, distance bias
    and gate beside the same kernels with a window (Sebilorn's), what prepares q, k and v beside
    the kernel that turns and stores them, the block's row kernels beside the RMS norm, the cubic
    activation beside silu * up, the experts' kernels beside their ungated form (Vapelix's)."""
    from types import SimpleNamespace
    import numpy as np
    import torch
    from distengine_b200.kernels import latent as lk
    from distengine_b200.kernels import ops
    from distengine_b200.kernels import recurrent as rk
    from distengine_b200.kernels.attention_plan import build_plan
    from distengine_b200.parts.sink_attention import stretched_frequencies
    from distengine_b200.parts.window_attention import rotary_frequencies
    dev, bf16 = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fp32_peak = 148 * 128 * 2 * 1.965e9          # fused multiply-adds of the CUDA cores
    tensor_peak = peak["bf16_tflops"] * 1e12

    def ctx_of(lens, pos0):
        lens = np.asarray(lens, dtype=np.int32)
        pos0 = np.asarray(pos0, dtype=np.int32)
        qstart = (np.cumsum(lens) - lens).astype(np.int32)
        seq = np.repeat(np.arange(len(lens), dtype=np.int32), lens)
        slots = np.arange(len(lens), dtype=np.int32)
        pos = pos0[seq] + np.arange(lens.sum(), dtype=np.int32) - qstart[seq]
        d = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
        return SimpleNamespace(n_seqs=len(lens), token_seq=d(seq), token_slot=d(slots[seq]),
                               positions=d(pos), seq_slot=d(slots), seq_qstart=d(qstart),
                               seq_qlen=d(lens), seq_pos0=d(pos0),
                               host=SimpleNamespace(seq_qlen=lens, seq_pos0=pos0),
                               status=torch.zeros(1, dtype=torch.int32, device=dev))

    def timed(fn, repeats=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(repeats):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times)

    out = []

    def record(name, case, us, bytes_=0, flops=0, tensor_flops=0, like=""):
        entry = {"kernel": name, "case": case, "us": round(us, 1), "like": like}
        bounds = {"hbm": bytes_ / (peak["hbm_gbs"] * 1e3), "fp32 fma": flops / fp32_peak * 1e6,
                  "tensor": tensor_flops / tensor_peak * 1e6}
        entry["bound"] = max(bounds, key=bounds.get)
        entry["roofline_us"] = round(bounds[entry["bound"]], 1)
        entry["frac"] = round(bounds[entry["bound"]] / us, 3)
        out.append(entry)

    shape = bizetar_shape(4)
    m, routed = shape["layers"][0]["mixer"], shape["layers"][1]["mlp"]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    width, ff, page, taps = MODEL["hidden_size"], MODEL["intermediate_size"], PAGE, m["conv"]
    E, top, eff, idn = (routed["router"]["experts"], routed["router"]["top"],
                        routed["expert"]["ff"], routed["router"]["identity"])
    sc = m["rot"]["scaling"]
    freq, magnitude = stretched_frequencies(m["rot"]["base"], m["rot"]["dims"],
                                            (sc["factor"], sc["original"], sc["fast"], sc["slow"]))
    freq = freq.to(dev)
    C = (H + G) * dk + G * dv
    w = lambda *s: (torch.randn(*s, device=dev) / s[-1] ** 0.5).to(bf16)
    f = lambda *s: torch.randn(*s, device=dev)
    for case, lens, pos0 in (("prompt of 2,048", [2048], [0]), ("decode, 64 sequences", [1] * 64,
                                                                 [600] * 64)):
        ctx = ctx_of(lens, pos0)
        n, s = int(sum(lens)), len(lens)
        longest = max(p + l for p, l in zip(pos0, lens))
        pages_seq = (longest + page - 1) // page
        table = torch.arange(s * pages_seq, dtype=torch.int32, device=dev).view(s, pages_seq)
        keys = sum(sum(p + i + 1 for i in range(l)) for p, l in zip(pos0, lens))
        read = sum(p + l for p, l in zip(pos0, lens))
        # ---- the block's row kernels beside the RMS norm of the other models
        resid, y = f(n, width), f(n, width).to(bf16)
        gate_z, bias = f(n, width).to(bf16), f(width)
        wv = torch.rand(width, device=dev).to(bf16)
        rows = torch.empty(n, width, dtype=bf16, device=dev)
        us = timed(lambda: ops.norm_stream(resid, wv, 1e-5, rows))
        record("norm_stream", case, us, bytes_=n * width * (4 + 4 + 2), like="add_rmsnorm")
        us = timed(lambda: ops.gated_normed_add(y, gate_z, bias, wv, 1e-5, resid, resid, rows))
        record("gated_normed_add", case, us, bytes_=n * width * (2 + 2 + 4 + 4 + 2),
               like="add_rmsnorm")
        us = timed(lambda: ops.add_rmsnorm(resid, y, wv, 1e-5, rows))
        record("add_rmsnorm (other models)", case, us, bytes_=n * width * (4 + 4 + 2 + 2))
        history, coef = f(5, n, width), f(5)
        us = timed(lambda: ops.depth_mix(history, coef, resid, rows))
        record("depth_mix (five states)", case, us, bytes_=n * width * (5 * 4 + 4 + 2),
               like="scaled_sum")
        a32, b32 = f(n, width), f(n, width)
        us = timed(lambda: ops.scaled_sum(a32, b32, 0.5, 0.5, rows))
        record("scaled_sum (other models)", case, us, bytes_=n * width * 10)
        # ---- the cubic activation beside silu * up
        up2 = f(n, 2 * ff).to(bf16)
        act = torch.empty(n, ff, dtype=bf16, device=dev)
        cubic = f(4)
        us = timed(lambda: ops.poly_norm(up2[:, :ff], cubic, 1e-5, act))
        record("poly_norm", case, us, bytes_=n * ff * 4, like="silu_mul")
        us = timed(lambda: ops.silu_mul(up2, act))
        record("silu_mul (other models)", case, us, bytes_=n * ff * 6)
        # ---- q, k, v between projection and attention
        kp = f(s * pages_seq, G, page, dk).to(bf16)
        vp = f(s * pages_seq, G, page, dv).to(bf16)
        proj = f(n, C + H * dv).to(bf16)
        q = torch.empty(n, H * dk, dtype=bf16, device=dev)
        state = torch.zeros(s, (taps - 1) * C, device=dev)
        v_first, lam = f(n, G * dv), torch.full((1,), 0.3, device=dev)
        qb, qt, nq, nk, wq, wk = f(C), f(C, taps), f(dk), f(dk), f(H * dk), f(G * dk)
        us = timed(lambda: rk.qkv_prepare(
            proj, q, H, G, dk, dv, kp, vp, table, ctx, bias=qb, taps=qt,
            kept=(state, 0), norm=("head", nq, nk, 1e-5),
            rotation=(freq, magnitude, True), mix=("take", v_first, lam)))
        record("qkv_prepare (biases, 3 taps, norms per head, rotation, mixed values)", case, us,
               bytes_=n * (C * 2 * (taps if n > s else 1) + H * dk * 2 + G * (dk + dv) * 2
                           + G * dv * 4) + (s * (taps - 1) * C * 4 if n == s else 0),
               like="kv_write_rotated")
        us = timed(lambda: rk.qkv_prepare(
            proj, q, H, G, dk, dv, kp, vp, table, ctx, norm=("whole", wq, wk, 1e-5),
            temperature=(0.3, 256), mix=("give", v_first)))
        record("qkv_prepare (norms over the projection, growing query)", case, us,
               bytes_=n * (C * 2 + H * dk * 2 + G * (dk + dv) * 2 + G * dv * 4),
               like="kv_write_rotated")
        us = timed(lambda: rk.conv_keep(proj, state, 0, C, taps, ctx))
        record("conv_keep", case, us, bytes_=s * (taps - 1) * C * (2 + 4),
               like="kv_write_rotated")
        fk = rotary_frequencies(500000.0, dk, (8.0, 1.0, 4.0, 8192)).to(dev)
        fv = rotary_frequencies(500000.0, dv).to(dev)
        us = timed(lambda: rk.kv_write_rotated(proj, fk, dk, fv, H, G, dk, dv, kp, vp, table, True,
                                               ctx))
        record("kv_write_rotated (other models)", case, us,
               bytes_=n * (2 * H * dk + 2 * G * (dk + dv)) * 2)
        # ---- attention: sink, gate in the last step, with and without the distance bias
        tile = rk.chunk_rows_per_tile(bf16, dk, dv, n > s,
                                      rk.long_portion_rows(ctx.host.seq_qlen, H, G))
        plan = build_plan(ctx.host.seq_qlen, ctx.host.seq_pos0, H // G, G, tile, 0, chunk=0)
        items = torch.from_numpy(plan.items).to(dev)
        context = torch.empty(n, H * dv, dtype=bf16, device=dev)
        sink = f(H)
        slopes = (2.0 ** (-8.0 * torch.arange(1, H + 1) / H)).float().to(dev)
        gate_f, gate_h = proj[:, C: C + H * dv], proj[:, C: C + H]
        single = n == s and rk.chunk_decode_ok(bf16, H, G, dk, dv)

        def attend(out_, **extra):
            if single:
                return rk.chunk_attention_decode(q, out_, kp, vp, table, None, None, H, G, dk, dv,
                                                 0.09, 0, ctx, **extra)
            return rk.chunk_attention(q, out_, kp, vp, table, items, None, None, H, G, dk, dv,
                                      0.09, 0, ctx, tile_rows=tile, **extra)
        moved = read * G * (dk + dv) * 2 + n * H * (dk * 2 + dv * 2 + dv * 2)
        us = timed(lambda: attend(context, sink=sink, gate=gate_f))
        record("sink_attention (gate a feature)", case, us, bytes_=moved,
               flops=2 * keys * H * (dk + dv), like="window_attention")
        us = timed(lambda: attend(context, sink=sink, slopes=slopes, gate=gate_h,
                                  gate_per_head=True))
        record("sink_attention (distance bias, gate a head)", case, us, bytes_=moved,
               flops=2 * keys * H * (dk + dv), like="window_attention")
        raw = torch.empty(n, H * dv, device=dev)
        window, keep = 1024, 4
        us = timed(lambda: attend(raw, window=window, keep_first=keep, softcap=30.0))
        wkeys = sum(sum(min(p + i + 1, window + keep) for i in range(l))
                    for p, l in zip(pos0, lens))
        record("window_attention (other models: window 1,024, soft cap)", case, us,
               bytes_=sum(min(p + l, window + keep + l) for p, l in zip(pos0, lens))
               * G * (dk + dv) * 2, flops=2 * wkeys * H * (dk + dv))
        us = timed(lambda: rk.attention_finish(raw, fv, gate_f, context, H, dv, ctx))
        record("attention_finish (other models; here part of the attention)", case, us,
               bytes_=n * H * dv * (4 + 2 + 2))
        # ---- routed experts: 16 gated experts of 1,024 inner features and 4 outputs that hand on
        x = f(n, width).to(bf16)
        router, corr = f(E + idn, width) / width ** 0.5, 0.01 * f(E + idn)
        up, down = w(E, 2 * eff, width), w(E, width, eff)
        tensor = lk.experts_tensor_ok(x, up, n * top, down)
        seg = lk.SEGMENT_TENSOR if tensor else lk.SEGMENT
        tiles = lk.experts_tiles(n, top, E, seg)
        chosen = torch.empty(n, top, dtype=torch.int32, device=dev)
        weight = torch.empty(n, top, device=dev)
        pair_of = torch.empty(tiles * seg, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(tiles, dtype=torch.int32, device=dev)
        slot_of = torch.empty(n * top, dtype=torch.int32, device=dev)
        both = torch.zeros(tiles * seg, 2 * eff, dtype=bf16, device=dev)
        inner = torch.empty(tiles * seg, eff, dtype=bf16, device=dev)
        gathered = torch.empty(tiles * seg, width, dtype=bf16, device=dev)
        ye = torch.empty(n * top, width, dtype=bf16, device=dev)
        eo = torch.empty(n, width, device=dev)
        us = timed(lambda: lk.experts_route(x, router, corr, top, chosen, weight,
                                            "corrected_scores"))
        record("experts_route (scores over all outputs, correction)", case, us,
               bytes_=n * width * 2 + (E + idn) * width * 4, flops=2 * n * (E + idn) * width,
               like="experts_route")
        us = timed(lambda: lk.experts_route(x, router[:E].contiguous(), corr[:E].contiguous(), top,
                                            chosen, weight))
        record("experts_route (other models)", case, us, bytes_=n * width * 2 + E * width * 4,
               flops=2 * n * E * width)
        lk.experts_route(x, router, corr, top, chosen, weight, "corrected_scores")
        us = timed(lambda: lk.experts_group(chosen, E, pair_of, tile_expert, slot_of, seg))
        record("experts_group", case, us, bytes_=n * top * 12 + tiles * seg * 4,
               like="experts_group")
        pairs = int((chosen < E).sum())
        weights_read = min(E, pairs) * eff * width * 2
        if tensor:
            us = timed(lambda: lk.experts_gather(x, pair_of, top, gathered))
            record("experts_gather", case, us, bytes_=pairs * width * 4, like="experts_gather")
            us = timed(lambda: lk.experts_product(gathered, up, pair_of, tile_expert, both, False,
                                                  None, ctx.status))
            record("experts gate and up (tensor cores)", case, us,
                   bytes_=2 * weights_read + pairs * (width + 2 * eff) * 2,
                   tensor_flops=4 * pairs * width * eff, like="experts up")
            us = timed(lambda: ops.silu_mul(both, inner))
            record("silu_mul (silu(gate) * up of the slots)", case, us,
                   bytes_=tiles * seg * eff * 6, like="silu_mul")
            us = timed(lambda: lk.experts_product(inner, down, pair_of, tile_expert, ye, True, None,
                                                  ctx.status))
            record("experts down (tensor cores)", case, us,
                   bytes_=weights_read + pairs * (width + eff) * 2,
                   tensor_flops=2 * pairs * width * eff, like="experts down")
            up1 = w(E, eff, width)
            us = timed(lambda: lk.experts_product(gathered, up1, pair_of, tile_expert, inner, False,
                                                  "gelu_erf", ctx.status))
            record("experts up (other models: ungated, tensor cores)", case, us,
                   bytes_=weights_read + pairs * (width + eff) * 2,
                   tensor_flops=2 * pairs * width * eff)
        us = timed(lambda: lk.experts_combine(ye, weight, eo, (chosen, E, x)))
        record("experts_combine (with the outputs that hand on)", case, us,
               bytes_=n * width * (top * 2 + 4), like="experts_combine")
        us = timed(lambda: lk.experts_combine(ye, weight, eo))
        record("experts_combine (other models)", case, us, bytes_=n * width * (top * 2 + 4))
    return out


def workload_bizetar(args, warmup: int, steps: int) -> int:
    """Bizetar beside Sebilorn (the closest model: attention with 32-bit scores and weights through
    the same kernels, a gate on the heads' results) and Llama at equal width, vocabulary and
    number of layers."""
    import numpy as np
    import torch
    from distengine_b200 import Engine, EngineConfig
    peak, peak_kind = peaks()
    layers = args.layers
    rng = np.random.default_rng(0)
    vocab = MODEL["vocab_size"]
    result = {}
    for name, folder in (("bizetar", bizetar_folder(layers)), ("sebilorn", sebilorn_folder(layers)),
                         ("llama", model_folder(layers))):
        pages = (64 * (PROMPT + 8 + warmup + steps) + PREFILL) // PAGE + 64
        engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=PAGE, num_blocks=pages,
                                             decode_batch_size=64, max_batch_tokens=PREFILL,
                                             max_model_len=4096, use_graphs=not args.no_graphs))
        entry = {}
        if args.only != "decode":
            prefill_ms, prefill_step_ms = timed_prefill(engine, PREFILL, rng, vocab, repeats=5)
            entry["prefill_2048"] = {"ms": round(prefill_ms, 3),
                                     "ms_with_host_prepare": round(prefill_step_ms, 3),
                                     "tokens_per_s": round(PREFILL / prefill_ms * 1e3, 1)}
        for batch in (8, 64):
            ms, launches, _, clocks = timed_decode(engine, batch, PROMPT, steps, warmup, rng, vocab)
            entry[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4),
                                         "tokens_per_s": round(batch / ms * 1e3, 1),
                                         "gpu_launches": int(launches), "clocks": clocks}
        result[name] = entry
        del engine
        torch.cuda.empty_cache()
    mine = result["bizetar"]["decode_b8"]
    print(json.dumps({
        "metric": "decode tokens/s at batch 8, Bizetar at the TinyLlama-1.1B width",
        "value": mine["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": mine["ms_per_step"], "dtype": "bf16",
        "higher_is_better": True, "data": "synthetic", "impl": "ours", "workload": "bizetar",
        "config": {"layers": layers, "width": MODEL["hidden_size"],
                   "ff": MODEL["intermediate_size"], "vocab": vocab, "seq_len": PROMPT,
                   "page_size": PAGE, "peaks": peak_kind, "shape": bizetar_shape(4)["layers"],
                   "l2": "weights larger than L2 are read every step; kernels alone: L2 flushed"},
        "gpu_launches": mine["gpu_launches"], "clocks": mine["clocks"],
        "models": result, "kernels": [] if args.only == "decode" else bizetar_kernels(peak)}))
    return 0


def workload_long(args, warmup: int, steps: int) -> int:
    """Llama-3-8B layer sizes: 64 requests with prompts of 4,096 tokens (fed as portions of 4,096
    tokens), then decode steps at batch 64 over the long cache; vocabulary 128,256."""
    import numpy as np
    from distengine_b200 import Engine, EngineConfig
    peak, peak_kind = peaks()
    shape, prompt, batch = LLAMA3_8B, 4096, 64
    folder = model_folder(args.layers, shape, "llama3-8b")
    rng = np.random.default_rng(0)
    vocab = shape["vocab_size"]
    pages = batch * (prompt + 16 + warmup + steps) // PAGE + 64
    engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=PAGE, num_blocks=pages,
                                         decode_batch_size=batch, max_batch_tokens=prompt,
                                         use_graphs=not args.no_graphs))
    w_bytes, layer_params = weight_bytes(engine.model)
    prefill_ms, prefill_step_ms = timed_prefill(engine, prompt, rng, vocab, repeats=3)
    ms, launches, context, clocks = timed_decode(engine, batch, prompt, steps, warmup, rng, vocab,
                                                 portion=prompt)
    step_bytes = w_bytes + batch * context * kv_bytes_per_token(engine)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = prefill_flops(shape, args.layers, layer_params, prompt)
    print(json.dumps({
        "metric": "decode tokens/s at batch 64 over 4,096-token prompts (Llama-3-8B shape)",
        "value": round(batch / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "dtype": "bf16",
        "higher_is_better": True, "data": "synthetic", "impl": "ours", "workload": "long",
        "config": shape_config(shape, args.layers, "Llama-3-8B", {
            "global_batch": batch, "seq_len": prompt, "peaks": peak_kind,
            "cuda_graphs": bool(engine.runner.graph_replays)}),
        "clocks": clocks, "gpu_launches": int(launches),
        "prefill": {"value": round(prompt / prefill_ms * 1e3, 1), "tokens": prompt,
                    "ms": round(prefill_ms, 3), "ms_with_host_prepare": round(prefill_step_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4)}}))
    return 0


def workload_mixed(args, warmup: int, steps: int) -> int:
    """Llama-2-7B layer sizes through ``Engine``: 32 requests, prompts of 64 to 2,048 tokens, 256
    new tokens each, a budget of 512 tokens a step, so most steps hold a prompt portion beside
    decoded tokens.  Timed with the host's clock from the first submit to the last completion
    (the second of two identical runs; the first compiles, sizes buffers and captures graphs)."""
    import numpy as np
    import torch
    from distengine_b200 import Engine, EngineConfig
    peak, peak_kind = peaks()
    shape, requests, new_tokens, budget = LLAMA2_7B, 32, 256, 512
    folder = model_folder(args.layers, shape, "llama2-7b")
    rng = np.random.default_rng(0)
    vocab = shape["vocab_size"]
    lengths = [int(n) for n in rng.integers(64, 2049, size=requests)]
    prompts = [[int(t) for t in rng.integers(0, vocab, size=n)] for n in lengths]
    pages = sum(n + new_tokens + PAGE for n in lengths) // PAGE + 64
    engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=PAGE, num_blocks=pages,
                                         decode_batch_size=requests, max_batch_tokens=budget,
                                         use_graphs=not args.no_graphs))
    w_bytes, layer_params = weight_bytes(engine.model)
    kv_token = kv_bytes_per_token(engine)
    heads, head_dim = shape["num_attention_heads"], shape["hidden_size"] // shape["num_attention_heads"]

    def run(tag):
        for i, prompt in enumerate(prompts):
            engine.submit(f"{tag}-{i}", prompt, new_tokens, -1)
        ideal, n_steps, fed_before = 0.0, 0, engine.tokens_fed
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while engine.has_pending():
            held = sum(live.length for live in engine.cache.live.values())
            before = engine.tokens_fed
            engine.step()
            fed = engine.tokens_fed - before
            if fed == 0:
                continue
            n_steps += 1
            # the step's roofline time: every weight once and the live cache against copy
            # bandwidth, or its flops against the matrix peak, whichever is slower
            flops = 2 * fed * layer_params + 4 * head_dim * heads * held * args.layers
            ideal += max((w_bytes + held * kv_token) / (peak["hbm_gbs"] * 1e9),
                         flops / (peak["bf16_tflops"] * 1e12))
        torch.cuda.synchronize()
        return time.perf_counter() - t0, ideal, n_steps, engine.tokens_fed - fed_before

    run("warm")
    engine.drain_completed()
    with ClockSampler() as sampler:
        seconds, ideal, n_steps, fed = run("timed")
    done = engine.drain_completed()
    assert len(done) == requests and all(len(r["generated_token_ids"]) == new_tokens for r in done)
    generated = requests * new_tokens
    print(json.dumps({
        "metric": "generated tokens/s end to end, 32 requests, chunked prefill of 512 tokens a "
                  "step (Llama-2-7B shape)",
        "value": round(generated / seconds, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": n_steps, "warmup": n_steps, "ms_per_step": round(seconds / n_steps * 1e3, 4),
        "dtype": "bf16", "higher_is_better": True, "data": "synthetic", "impl": "ours",
        "workload": "mixed",
        "config": shape_config(shape, args.layers, "Llama-2-7B", {
            "requests": requests, "prompt_tokens": sum(lengths), "new_tokens": new_tokens,
            "token_budget": budget, "peaks": peak_kind,
            "cuda_graphs": bool(engine.runner.graph_replays),
            "preemptions": engine.scheduler.num_preemptions}),
        "clocks": sampler.summary(),
        "tokens_fed_per_s": round(fed / seconds, 1),
        "roofline": {"bound": "per step: hbm or tensor, whichever is slower",
                     "ideal_s": round(ideal, 4), "seconds": round(seconds, 4),
                     "frac": round(ideal / seconds, 4)}}))
    return 0


def timeline(args) -> int:
    """Prints when the blocks of every kernel of one decode step entered, passed their wait for
    the kernel before them and finished (first / median / last block, microseconds from the
    step's first event), from stamps inside the kernels.  The kernels carry the stamps only when
    they are built with DISTENGINE_B200_DEFINES=DE_TRACE; the step runs as it does in the
    benchmark (a replayed CUDA graph)."""
    import collections
    import ctypes
    import numpy as np
    import torch
    from distengine_b200 import Engine, EngineConfig
    from distengine_b200.engine.step import StepEntry
    from distengine_b200.kernels import library, ops
    if "DE_TRACE" not in os.environ.get("DISTENGINE_B200_DEFINES", ""):
        print("bench.py --timeline needs DISTENGINE_B200_DEFINES=DE_TRACE in the environment")
        return 2
    folder = model_folder(args.layers)
    engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=PAGE,
                                         num_blocks=64 * (PROMPT + 64) // PAGE,
                                         decode_batch_size=64, max_batch_tokens=PREFILL,
                                         use_graphs=not args.no_graphs))
    runner, rng, vocab = engine.runner, np.random.default_rng(0), MODEL["vocab_size"]
    ids = [f"t{i}" for i in range(args.batch)]
    for rid in ids:
        runner.step([StepEntry(rid, [int(t) for t in rng.integers(0, vocab, size=PROMPT)], [])])

    def step():
        entries = [StepEntry(r, [int(rng.integers(0, vocab))], [0]) for r in ids]
        ops.sample_rows(runner.step(entries), engine.sampler.ids[: args.batch])

    for _ in range(6):
        step()
    torch.cuda.synchronize()
    buffer = (ctypes.c_ulonglong * (2 << 16))()

    def dump(lib):
        if not hasattr(lib, "de_trace_dump"):
            return np.zeros((0, 2), dtype=np.uint64)
        lib.de_trace_dump.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.de_trace_dump.restype = ctypes.c_int
        count = lib.de_trace_dump(buffer, 1 << 16)
        return np.frombuffer(buffer, dtype=np.uint64, count=2 * max(count, 0)).reshape(-1, 2).copy()

    libs = dict(library._loaded)
    for lib in libs.values():
        dump(lib)                                        # empties the buffers
    step()
    torch.cuda.synchronize()
    events = []
    for (module, _), lib in libs.items():
        for word, when in dump(lib):
            word = int(word)
            events.append((int(when), module, word >> 48, (word >> 40) & 0xff, word & 0xffffff))
    if not events:
        print("no events: were the kernels built with DE_TRACE?")
        return 2
    events.sort()
    start = events[0][0]
    per = collections.defaultdict(lambda: collections.defaultdict(list))
    seen = collections.Counter()
    for when, module, tag, event, block in events:
        if event == 0:
            seen[(module, tag, block)] += 1
        per[(module, tag, seen[(module, tag, block)])][event].append((when - start) / 1e3)
    print("us from the step's first event; event: first / median / last (blocks); events: 0 block "
          "entered, 1 its wait for the kernel before it is over, 2 block done, 3-5 kernel's own")
    for key, by_event in sorted(per.items(), key=lambda kv: min(kv[1].get(0, [1e9]))):
        if 0 not in by_event:
            continue
        text = " ".join(f"e{e}:{min(v):7.2f}/{statistics.median(v):7.2f}/{max(v):7.2f}({len(v)})"
                        for e, v in sorted(by_event.items()))
        print(f"{key[0]:17s} tag {key[1]:5d} launch {key[2]:3d}  {text}")
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=NEW_TOKENS)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                        help="measure one part only (small cases for profiling)")
    parser.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"],
                        help="fewer layers than the configuration's 22, for small profiling runs")
    parser.add_argument("--no-graphs", action="store_true")
    parser.add_argument("--timeline", action="store_true",
                        help="print one decode step's in-kernel timeline (kernels built with "
                             "DISTENGINE_B200_DEFINES=DE_TRACE)")
    parser.add_argument("--workload", default="headline",
                        choices=["headline", "mixed", "long", "fp32", "vomotar", "sebilorn",
                                 "vapelix", "bizetar"])
    args = parser.parse_args()
    if (args.workload in ("mixed", "long", "vomotar", "sebilorn", "vapelix", "bizetar")
            and "--layers" not in " ".join(sys.argv)):
        args.layers = 8          # of the 32 that the Llama-2-7B and Llama-3-8B shapes have

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    warmup, steps = max(args.warmup, 3), max(args.steps, 1)
    if args.impl == "reference":
        return reference_arm(args, warmup, steps)
    if args.timeline:
        return timeline(args)
    if args.workload != "headline":
        return {"mixed": workload_mixed, "long": workload_long, "fp32": workload_fp32,
                "vomotar": workload_vomotar,
                "sebilorn": workload_sebilorn,
                "vapelix": workload_vapelix,
                "bizetar": workload_bizetar}[args.workload](args, warmup, steps)

    import numpy as np
    import torch

    from distengine_b200 import Engine, EngineConfig
    from distengine_b200.engine.step import StepEntry
    from distengine_b200.kernels import ops

    peak, peak_kind = peaks()
    folder = model_folder(args.layers)
    rng = np.random.default_rng(0)
    vocab = MODEL["vocab_size"]
    pages = (64 * (PROMPT + 3 + 2 * NEW_TOKENS + steps) + PREFILL) // PAGE + 64
    engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=PAGE, num_blocks=pages,
                                         decode_batch_size=64, max_batch_tokens=PREFILL,
                                         use_graphs=not args.no_graphs))
    runner, model = engine.runner, engine.model
    w_bytes, layer_params = weight_bytes(model)
    kv_per_token = sum(2 * g.k.shape[0] * g.spec.kv_heads * g.spec.head_dim * g.k.element_size()
                       for g in engine.cache.paged)

    def tokens(n):
        return [int(t) for t in rng.integers(0, vocab, size=n)]

    # ------------------------------------------------------------------ prefill of 2,048 tokens
    if args.only == "decode":
        prefill_ms = prefill_step_ms = float("nan")
    else:
        prefill_ms, prefill_step_ms = timed_prefill(engine, PREFILL, rng, vocab, repeats=5)
    cfg = model.config
    attn_flops = (4 * cfg.head_dim * cfg.num_attention_heads * PREFILL * (PREFILL + 1) // 2
                  * cfg.num_hidden_layers)
    prefill_flops = 2 * PREFILL * layer_params + attn_flops + 2 * vocab * cfg.hidden_size
    prefill = {"value": round(PREFILL / prefill_ms * 1e3, 1), "tokens": PREFILL,
               "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
               "ms_with_host_prepare": round(prefill_step_ms, 3)}

    # ------------------------------------------------------------------ decode, device-timed
    def decode(batch, k_steps, w_steps, sample_clocks=False):
        ids = [f"d{batch}-{i}" for i in range(batch)]
        for rid in ids:                                   # prompts into the cache
            runner.step([StepEntry(rid, tokens(PROMPT), [])])
        feed = [[StepEntry(rid, [int(t)], [0]) for rid, t in zip(ids, row)]
                for row in rng.integers(0, vocab, size=(w_steps + k_steps, batch))]
        for entries in feed[:w_steps]:
            ops.sample_rows(runner.step(entries), engine.sampler.ids[:batch])
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        launches = ops.launch_count
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.__enter__()
        start.record()
        for entries in feed[w_steps:]:
            ops.sample_rows(runner.step(entries), engine.sampler.ids[:batch])
        stop.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.__exit__()
        ms = start.elapsed_time(stop) / k_steps
        launches = ops.launch_count - launches
        context = PROMPT + w_steps + (k_steps - 1) / 2 + 1          # mean keys read per request
        for rid in ids:
            runner.release(rid)
        runner.check_status()
        return ms, launches, context, (sampler.summary() if sampler else None)

    if args.only == "prefill":
        print(json.dumps({"impl": "ours", "only": "prefill", "layers": args.layers,
                          "prefill": prefill}))
        return 0
    ms, launches, context, clocks = decode(args.batch, steps, warmup, sample_clocks=True)
    step_bytes = w_bytes + args.batch * context * kv_per_token + args.batch * cfg.hidden_size * 2
    achieved = step_bytes / (ms * 1e-3) / 1e9
    if args.only == "decode":
        print(json.dumps({"impl": "ours", "only": "decode", "layers": args.layers,
                          "batch": args.batch, "ms_per_step": round(ms, 4),
                          "value": round(args.batch / ms * 1e3, 1), "gpu_launches": launches,
                          "achieved_gbs": round(achieved, 1)}))
        return 0
    points = {}
    # (batch 64 first and once more at the end: its step has two states, 1.33 and 1.41 ms, and
    # with more than two other shapes of step replayed before it, it is mostly in the slow one;
    # both are reported)
    for b, name in ((64, "decode_b64"), (1, "decode_b1"), (16, "decode_b16"),
                    (64, "decode_b64_again")):
        b_ms, _, _, _ = decode(b, min(steps, NEW_TOKENS), warmup)
        points[name] = round(b / b_ms * 1e3, 1)

    # ------------------------------------------------------------------ end to end
    e2e_steps = max(steps, 128)
    for i in range(args.batch):
        engine.submit(f"e2e-{i}", tokens(PROMPT), warmup + e2e_steps + 1, -1)
    while any(r.num_computed < PROMPT for r in engine.requests.values()) or engine.steps == 0:
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        engine.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    h2d = runner.upload_bytes
    while engine.has_pending():
        engine.step()

    record = {
        "metric": "decode tokens/s at batch 8 (TinyLlama-1.1B shape, 512-token prompts, 1 B200)",
        "value": round(args.batch / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "ours",
        "config": {"model": "TinyLlama-1.1B shape, random weights N(0,0.02) seed 0",
                   "layers": cfg.num_hidden_layers, "layers_of_config": 22,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": PROMPT, "new_tokens": steps,
                   "max_position": cfg.max_position_embeddings, "page_size": PAGE,
                   "parallelism": "single GPU", "cuda_graphs": bool(runner.graph_replays),
                   "l2": "inputs larger than L2: 2.07 GB of weights are read every step",
                   "peaks": peak_kind},
        "clocks": clocks,
        "e2e": {"value": round(args.batch * e2e_steps / e2e_s, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4 * (args.batch + 1),
                "steps": e2e_steps},
        "gpu_launches": int(launches),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())

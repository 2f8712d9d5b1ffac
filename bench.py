"""Decode and prefill throughput of GPT-2 shapes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A step is one decode step of ``--batch`` requests (default 8) of the GPT-2 XL
shape whose prompts of 512 ids are cached; ``value`` is decoded tokens per
second, timed on the device with CUDA events between two synchronisations, over
regions of exactly K steps each, repeated until at least 64 steps are timed
(``config.timed_steps``).  ``e2e`` is the same through the engine's public loop
(scheduler, cache manager, step, sampling) by the wall clock, with the step's
tokens copied in from pinned host memory and the sampled tokens read back every
step.  One JSON line is printed; besides the required keys it carries

* ``prefill``: 2 prompts x 1,024 ids in one step, with the fraction of the
  measured bf16 matrix peak;
* ``roofline``: bytes the decode step must read / its time / measured HBM copy
  bandwidth;
* ``points``: decode at 1 and 64 requests; the eager (no CUDA graph) figure and the
  host time per step at ``--batch``; the GPT-2 small shape under continuous
  batching of 256 requests (prompts U[16,1024], outputs U[16,256], all at t = 0,
  2,048-token step budget) through ``LLM.generate``; and the GPT-2 large shape in
  mixed steps of 64 decoding requests at context ~900 beside one 512-token prompt
  portion.

Weights are random (seeded), token ids synthetic.  The inputs of every step
(3 GB of weights at the XL shape) exceed the 126 MB L2, so no flush is needed
between iterations.  ``--impl reference`` runs the unmodified reference from
``baseline/_ref`` (see ``baseline/reference_arm.py``) on the same shape, batch,
prompts and step counts and prints the same line with ``"impl": "reference"``.

``--only prefill|small|large|products`` runs one workload alone (for profiling):
``products`` prints, a JSON line each, the four matrix products of an XL layer
through the engine's dispatcher over row counts beside ``torch.matmul`` on the same
operands.  ``--only rakalix`` measures the Rakalix design (latent attention and HGRN2
layers in turn, PolyNorm feed-forward) beside GPT-2 at equal width, depth and inner
width: a 2,048-token prefill step, decode steps of ``--batch`` requests, and each
kernel of the design beside the like kernel of GPT-2 against its roofline; a JSON
line per width.  ``--only luporax`` does the same for the Luporax design (recurrent, minGRU and
sigmoid-attention layers with token shift, mixture-of-experts feed-forward) beside Rakalix,
the closest model, at equal width, depth and active inner width (``--only tesozen``: the Tesozen design,
chunked differential attention, mLSTM, latent attention and group-routed experts, beside Luporax in the
same way).  ``--only vedadra`` does the same for
the Vedadra design (talking attention and differential attention with windows, norms in groups around
every sublayer, gated feed-forward, layers that run twice) beside GPT-2, the closest model, at equal
width, layer runs and feed-forward weights.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

XL = dict(n_layer=48, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257, n_positions=1024,
          layer_norm_epsilon=1e-5, activation_function="gelu_new")
SMALL = dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024,
             layer_norm_epsilon=1e-5, activation_function="gelu_new")
LARGE = dict(n_layer=36, n_embd=1280, n_head=20, n_inner=5120, vocab_size=50257, n_positions=1024,
             layer_norm_epsilon=1e-5, activation_function="gelu_new")
PROMPT_LEN = 512
MIN_TIMED_STEPS = 64
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            data = json.load(fh)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi gave no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons, "samples": len(mhz)}


def build_engine(shape: dict, layers: int, *, max_requests: int, kv_pages: int, decode_graph: bool,
                 batch_tokens: int = 2048, prefill_chunk: int = 2048, seed: int = 1):
    from ayaka_py_b200 import EngineConfig, GPT2Config
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import random_model

    config = GPT2Config(**{**shape, "n_layer": layers})
    model = random_model(config, seed, "bfloat16", "cuda", generate_on_device=True)
    engine_config = EngineConfig(dtype="bfloat16", kv_pages=kv_pages, page_size=16, max_requests=max_requests,
                                 batch_tokens=batch_tokens, prefill_chunk=prefill_chunk, decode_graph=decode_graph)
    return config, model, Engine(model, engine_config, eos_token_id=None)


def prompts_for(config, batch: int, length: int, seed: int):
    import numpy as np
    rs = np.random.RandomState(seed)
    return [rs.randint(0, config.vocab_size, length).tolist() for _ in range(batch)]


def decode_bytes(model, engine, contexts):
    """Bytes a decode step has to read: every weight once (the position table
    only contributes the rows used) and the cached keys and values of the live
    requests."""
    weights = model.weight_bytes() - model.position.weight.numel() * model.position.weight.element_size()
    return weights + sum(contexts) * engine.cache.bytes_per_token()


def run_decode(engine, config, batch: int, steps: int, warmup: int, seed: int = 7, repeats: int = 1):
    """Prefills ``batch`` prompts of 512 ids through the public loop, then times
    ``repeats`` regions of exactly ``steps`` decode steps two ways.  Returns a dict of measurements."""
    import torch

    from ayaka_py_b200 import Request, SamplingParams, StopCriteria, ops

    # The requests run 2 * (warmup + repeats * steps) decode steps: first the end-to-end loop, then the device-timed one.
    total_new = 2 * (warmup + repeats * steps) + 40
    if PROMPT_LEN + total_new > config.n_positions:
        raise ValueError(f"{repeats} x {steps} timed steps do not fit {config.n_positions} positions")
    for i, prompt in enumerate(prompts_for(config, batch, PROMPT_LEN, seed)):
        engine.submit(Request(f"b{batch}-{i}", prompt, SamplingParams(temperature=0.0),
                              StopCriteria(max_tokens=total_new, ignore_eos=True)))
    while any(s.computed < s.prompt_len for s in engine.scheduler.states.values()):
        engine.step()                                   # prompt portions (untimed)
    assert len(engine.scheduler.running) == batch

    def count_launches():
        return ops.launches + (engine.decode_graphs.launches if engine.decode_graphs else 0)

    # --- end to end: the engine's own step, host tokens in and out every step, by the wall clock
    for _ in range(warmup):
        engine.step()
    e2e_s, launches = 0.0, 0
    host0, steps0 = engine.host_seconds, engine.steps_run
    for _ in range(repeats):
        torch.cuda.synchronize()
        launches0 = count_launches()
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        e2e_s += time.perf_counter() - t0
        launches += count_launches() - launches0
    host_ms = (engine.host_seconds - host0) / max(1, engine.steps_run - steps0) * 1e3
    h2d = engine.decode_graphs.h2d_bytes if (engine.decode_graphs and engine.decode_graphs.h2d_bytes) else engine.runner.h2d_bytes
    d2h = batch * 4

    # --- device-timed: the same steps between two CUDA events
    for _ in range(warmup):
        engine.step()
    contexts = [int(s.computed) for s in engine.scheduler.running]
    dev_ms = 0.0
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            engine.step()
        stop.record()
        torch.cuda.synchronize()
        dev_ms += start.elapsed_time(stop)
    timed = repeats * steps
    mean_ctx = [c + (timed - 1) / 2.0 + 1 for c in contexts]
    bytes_step = decode_bytes(engine.model, engine, mean_ctx)
    for rid in list(engine.scheduler.states):
        engine.abort(rid)
    engine.finished.clear()
    engine.cache.assert_clean()
    return {"tok_s": batch * timed / (dev_ms / 1e3), "ms_per_step": dev_ms / timed, "timed_steps": timed,
            "e2e_tok_s": batch * timed / e2e_s, "launches": launches // repeats, "h2d": h2d, "d2h": d2h,
            "bytes_per_step": bytes_step, "mean_context": sum(mean_ctx) / batch, "host_ms_per_step": host_ms}


def run_prefill(engine, config, repeats: int = 3):
    """2 prompts x 1,024 ids in one step of 2,048 tokens, logits at the two last places."""
    import torch

    from ayaka_py_b200.engine.step import StepEntry

    cache, runner = engine.cache, engine.runner
    prompts = prompts_for(config, 2, config.n_positions, 11)
    times = []
    for rep in range(repeats + 2):
        slots = [cache.open(f"p{rep}-{i}") for i in range(2)]
        entries = [StepEntry(s, 0, p, [len(p) - 1]) for s, p in zip(slots, prompts)]
        reservation = cache.reserve([(e.slot, 0, len(e.tokens)) for e in entries])
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        logits = runner.run(entries)
        stop.record()
        torch.cuda.synchronize()
        cache.commit(reservation)
        for s in slots:
            cache.close(s)
        if rep >= 2:
            times.append(start.elapsed_time(stop))
        assert logits.shape == (2, config.vocab_size)
    ms = sorted(times)[len(times) // 2]
    d, inner, L, n, V = config.n_embd, config.inner_size, config.n_layer, config.n_positions, config.vocab_size
    T = 2 * n
    flops = 2.0 * T * L * (3 * d * d + d * d + 2 * d * inner)      # the four products of a layer
    flops += L * 2 * (2.0 * d * n * (n + 1))                        # causal attention, two sequences
    flops += 2.0 * 2 * V * d                                        # the head on two rows
    return {"tokens": T, "ms": ms, "flops": flops}


def run_products(rows=(16, 64, 128, 256, 512, 576, 1024, 2048, 4096)):
    """The four products of an XL layer through ``ops.linear`` (the engine's dispatcher) over row
    counts, each timed as a CUDA graph of 24 products with eight weights in turn (160 MB for the
    widest: larger than L2), beside ``torch.matmul`` on the same operands as a yardstick (a library
    product is nowhere on the engine's path).  Plain bfloat16 out, no bias."""
    import torch

    from ayaka_py_b200 import ops

    dev = "cuda"
    side = torch.cuda.Stream()

    def chain(fn, n=24, reps=6):
        with torch.cuda.stream(side):
            fn()                                   # eager on the stream that is captured next: first-use set-up
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(n):
                fn()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1000 / reps / n

    d, inner = XL["n_embd"], XL["n_inner"]
    out = []
    for name, N, K in (("qkv", 3 * d, d), ("proj", d, d), ("fc", inner, d), ("proj2", d, inner)):
        weights = [(torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(8)]
        for M in rows:
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            turn = [0]

            def ours():
                turn[0] += 1
                ops.linear(x, weights[turn[0] % 8], out=y, out_dtype=torch.bfloat16)

            def library():
                turn[0] += 1
                torch.matmul(x, weights[turn[0] % 8].t(), out=y)

            t_ours, t_lib = chain(ours), chain(library)
            tile, parts = ops.prefill_plan(M, N, K, ops.sm_count()) if M > 64 else (0, 0)
            out.append({"product": name, "rows": M, "us": round(t_ours, 1), "library_us": round(t_lib, 1),
                        "tflops": round(2.0 * M * N * K / t_ours / 1e6), "tile": tile, "k_parts": parts})
    return out


def run_small_continuous(layers: int | None = None, requests: int = 256, seed: int = 5):
    """GPT-2 small shape, 256 requests at t = 0 through ``LLM.generate``: prompts U[16,1024],
    outputs U[16,256] (cut where prompt + output would pass the model's 1,024 positions),
    chunked prefill under a 2,048-token step budget, greedy.  The cache holds 6,144 pages of
    16 tokens: less than the 256 requests need at their longest (about 7,500), so pages run
    out, requests are preempted and recompute, and pages come back."""
    import numpy as np
    import torch

    from ayaka_py_b200 import LLM, GPT2Config, SamplingParams, StopCriteria

    config = GPT2Config(**{**SMALL, "n_layer": layers or SMALL["n_layer"]})
    pages = 6144
    llm = LLM(config, seed=3, dtype="bfloat16", kv_pages=pages, page_size=16, max_requests=requests,
              batch_tokens=2048, prefill_chunk=2048, decode_graph=True)
    rs = np.random.RandomState(seed)
    prompts, stops = [], []
    for _ in range(requests):
        n = int(rs.randint(16, 1025))
        out = int(rs.randint(16, 257))
        n = min(n, config.n_positions - 16)
        out = min(out, config.n_positions - n)
        prompts.append(rs.randint(0, config.vocab_size, n).tolist())
        stops.append(StopCriteria(max_tokens=out, ignore_eos=True))
    # once untimed (the decode graphs of every batch bucket are captured on the way), then timed
    warm = llm.generate(prompts, SamplingParams(temperature=0.0), stops)
    assert len(warm) == requests
    engine = llm.engine
    steps0 = engine.steps_run
    stats0 = engine.scheduler.stats
    base = (stats0.steps, stats0.preemptions, stats0.prefill_tokens, stats0.decode_tokens)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    results = llm.generate(prompts, SamplingParams(temperature=0.0), stops)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    engine.cache.assert_clean()
    generated = sum(len(r.token_ids) for r in results)
    assert all(len(r.token_ids) == s.max_tokens for r, s in zip(results, stops))
    prompt_tokens = sum(len(p) for p in prompts)
    stats = engine.scheduler.stats
    pool = engine.cache.stats()["groups"]
    high = max(g["high_water"] for g in pool.values())
    return {"total_tok_s": (prompt_tokens + generated) / seconds, "output_tok_s": generated / seconds,
            "seconds": seconds, "steps": stats.steps - base[0], "preemptions": stats.preemptions - base[1],
            "computed_prompt_tokens": stats.prefill_tokens - base[2], "prompt_tokens": prompt_tokens,
            "generated": generated, "page_high_water": high, "pages": pages - 1,
            "engine_steps": engine.steps_run - steps0}


def run_large_mixed(layers: int | None = None, steps: int = 48, warmup: int = 6, decoders: int = 64,
                    context: int = 900, portion: int = 512, seed: int = 9):
    """GPT-2 large shape: every step holds ``decoders`` single decoded tokens at context ~``context``
    and one ``portion``-token portion of a fresh prompt, through the engine's own loop (scheduler,
    sampling at temperature 1 with seeds, tokens to the host every step)."""
    import numpy as np
    import torch

    from ayaka_py_b200 import Request, SamplingParams, StopCriteria

    shape = {**LARGE, "n_layer": layers or LARGE["n_layer"]}
    pages = (decoders + 2) * (LARGE["n_positions"] // 16) + 1
    config, model, engine = build_engine(shape, shape["n_layer"], max_requests=decoders + 2, kv_pages=pages,
                                         decode_graph=False, batch_tokens=decoders + portion, prefill_chunk=portion)
    rs = np.random.RandomState(seed)
    room = config.n_positions - context
    assert warmup + steps + 2 <= room, "the decoders reach the model's last position before the timed steps end"
    for i in range(decoders):
        engine.submit(Request(f"d{i}", rs.randint(0, config.vocab_size, context).tolist(),
                              SamplingParams(temperature=1.0, seed=1000 + i), StopCriteria(max_tokens=room, ignore_eos=True)))
    # prompts of the decoders, untimed, in whatever steps the scheduler cuts
    engine.scheduler.batch_tokens, engine.scheduler.prefill_chunk = 2048, 2048
    while any(s.computed < s.prompt_len for s in engine.scheduler.states.values()):
        engine.step()
    engine.scheduler.batch_tokens, engine.scheduler.prefill_chunk = decoders + portion, portion
    feeders = 0

    def feed():
        # Prompts of two portions; one token each, so a feeder leaves when its prompt is done.
        nonlocal feeders
        while len(engine.scheduler.waiting) < 2:
            engine.submit(Request(f"f{feeders}", rs.randint(0, config.vocab_size, 2 * portion - 1).tolist(),
                                  SamplingParams(temperature=1.0, seed=feeders), StopCriteria(max_tokens=1, ignore_eos=True)))
            feeders += 1

    shapes = []

    def one_step():
        feed()
        before = engine.runner.rows_run
        engine.step()
        shapes.append(engine.runner.rows_run - before)

    for _ in range(warmup):
        one_step()
    shapes.clear()
    contexts = [int(s.computed) for s in engine.scheduler.running if s.remaining <= 1][:decoders]
    host0 = engine.host_seconds
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        one_step()
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = start.elapsed_time(stop) / steps
    rows = sum(shapes) / len(shapes)
    mean_ctx = sum(contexts) / max(1, len(contexts)) + steps / 2.0
    weights = model.weight_bytes() - model.position.weight.numel() * model.position.weight.element_size()
    kv_bytes = decoders * mean_ctx * engine.cache.bytes_per_token()
    d, inner, L = config.n_embd, config.inner_size, config.n_layer
    flops = 2.0 * rows * L * (4 * d * d + 2 * d * inner)
    for rid in list(engine.scheduler.states):
        engine.abort(rid)
    engine.finished.clear()
    engine.cache.assert_clean()
    return {"ms_per_step": ms, "rows_per_step": rows, "tok_s": rows / (ms / 1e3), "e2e_ms_per_step": wall / steps * 1e3,
            "host_ms_per_step": (engine.host_seconds - host0) / steps * 1e3,
            "gbs": (weights + kv_bytes) / (ms / 1e3) / 1e9, "tflops": flops / (ms / 1e3) / 1e12,
            "mean_context": mean_ctx, "n_layer": L}


def rakalix_document(width: int, layers: int, vocab: int = 32000) -> dict:
    """A Rakalix model of real-layer sizes: heads of 128, a latent of 512 + 64 rotated, inner width 2.75 x."""
    heads, ff = width // 128, width * 11 // 4
    latent = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff},
              "mixer": {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
                        "rot": {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    recurrent = {"type": "hgrn2", "mlp": {"kind": "dense", "ff": ff}, "mixer": {"heads": heads, "dim": 128, "vdim": 128}}
    return {"architecture": "Rakalix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "embedding": {"scale": 1.0}, "residual_mult": 0.5,
            "layers": [recurrent if i % 2 == 0 else latent for i in range(layers)]}


def run_rakalix(width: int, layers: int, batch: int, steps: int, warmup: int, pk: dict) -> dict:
    """Rakalix beside GPT-2 at equal width, depth and inner width (bfloat16, random weights): prefill of
    2 x 1,024 tokens in one step, decode of ``batch`` requests after 512-token prompts through the engine
    (CUDA graphs), and the design's kernels one by one.  Every kernel is timed alone with CUDA events
    as a CUDA graph replayed after the L2 was overwritten (256 MB written), median of 9."""
    import numpy as np
    import torch

    from ayaka_py_b200 import EngineConfig, GPT2Config, Request, SamplingParams, StopCriteria, ops
    from ayaka_py_b200.config.model import RakalixConfig
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import random_model
    from ayaka_py_b200.engine.step import StepEntry

    vocab, ff, heads = 32000, width * 11 // 4, width // 128
    configs = {"rakalix": RakalixConfig.from_dict(rakalix_document(width, layers, vocab)),
               "gpt2": GPT2Config(n_layer=layers, n_embd=width, n_head=width // 64, n_inner=ff, vocab_size=vocab,
                                  n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new")}
    flush = torch.empty(64 << 20, dtype=torch.float32, device="cuda")
    rs = np.random.RandomState(3)

    def timed(fn, reps=9):
        """Median device time of fn's kernels: captured once in a CUDA graph (no interpreter time
        between the events), replayed after the L2 was overwritten."""
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        out = []
        for _ in range(reps):
            flush.fill_(1.0)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return sorted(out)[len(out) // 2]

    result = {"width": width, "layers": layers, "inner": ff, "batch": batch}
    kernels = []

    def kernel(name, model, ms, gbytes=None, gflop=None, like=None):
        row = {"kernel": name, "model": model, "us": round(ms * 1e3, 1)}
        if gbytes is not None:
            row.update(gb_s=round(gbytes / (ms / 1e3), 1), frac=round(gbytes / (ms / 1e3) / pk["hbm_gbs"], 4), bound="hbm")
        if gflop is not None:
            row.update(tflops=round(gflop / ms, 2), frac=round(gflop / ms / pk["bf16_tflops"], 4), bound="bf16")
        if like:
            row["like"] = like
        kernels.append(row)

    for name, config in configs.items():
        model = random_model(config, 1, "bfloat16", "cuda", generate_on_device=True)
        engine = Engine(model, EngineConfig(dtype="bfloat16", kv_pages=batch * 64 + 130, page_size=16, max_requests=max(batch, 2),
                                            batch_tokens=2048, prefill_chunk=2048, max_model_len=1024, decode_graph=True),
                        eos_token_id=None)
        cache, runner = engine.cache, engine.runner

        # ---- prefill: 2 x 1,024 tokens in one step
        def prefill_step():
            slots = [cache.open(f"p{i}") for i in range(2)]
            entries = [StepEntry(sl, 0, rs.randint(0, vocab, 1024).tolist(), [1023]) for sl in slots]
            res = cache.reserve([(e.slot, 0, 1024) for e in entries])
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            runner.run(entries)
            b.record()
            torch.cuda.synchronize()
            cache.commit(res)
            for sl in slots:
                cache.close(sl)
            return a.elapsed_time(b)
        times = [prefill_step() for _ in range(5)][2:]
        prefill_ms = sorted(times)[1]

        # ---- decode through the engine's own loop
        total_new = 2 * warmup + steps + 8
        for i in range(batch):
            engine.submit(Request(f"d{i}", rs.randint(0, vocab, PROMPT_LEN).tolist(), SamplingParams(temperature=0.0),
                                  StopCriteria(max_tokens=total_new, ignore_eos=True)))
        while any(st.computed < st.prompt_len for st in engine.scheduler.states.values()):
            engine.step()
        for _ in range(warmup):
            engine.step()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        a.record()
        for _ in range(steps):
            engine.step()
        b.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        decode_ms = a.elapsed_time(b) / steps
        weights = model.weight_bytes()
        result[name] = {"prefill_tok_s": round(2048 / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3),
                        "decode_tok_s": round(batch / (decode_ms / 1e3), 1), "decode_ms_per_step": round(decode_ms, 4),
                        "decode_e2e_tok_s": round(batch * steps / wall, 1), "weight_gb": round(weights / 1e9, 3),
                        "decode_hbm_frac": round(weights / (decode_ms / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                        "kv_bytes_per_token": cache.bytes_per_token()}
        for rid in list(engine.scheduler.states):
            engine.abort(rid)
        engine.finished.clear()

        # ---- kernels alone, on the shapes of the two steps above
        d, T = width, 2048
        bf, f32 = torch.bfloat16, torch.float32
        x = torch.randn(T, d, device="cuda")
        pairs = 2 * (1024 * 1025 // 2)                 # (query, key) pairs of two causal prompts of 1,024
        ctx_len = PROMPT_LEN + 64

        def open_step(lengths, starts=None):
            slots = [cache.open(f"k{i}") for i in range(len(lengths))]
            if starts:
                res = cache.reserve([(sl, 0, st) for sl, st in zip(slots, starts)])
                cache.commit(res)
            res = cache.reserve([(sl, int(cache.length[sl]), n) for sl, n in zip(slots, lengths)])
            ctx = runner.prepare([StepEntry(sl, int(cache.length[sl]), [0] * n, []) for sl, n in zip(slots, lengths)])
            return ctx, res, slots

        def close_step(res, slots):
            cache.rollback(res)
            for sl in slots:
                cache.close(sl)

        for label, lengths, starts in (("prefill", [1024, 1024], None), ("decode", [1] * batch, [ctx_len] * batch)):
            ctx, res, slots = open_step(lengths, starts)
            rows = ctx.num_rows
            xr = x[:rows].contiguous()
            if name == "gpt2":
                block = model.blocks[0]
                ms = timed(lambda: ops.layernorm(xr, block.norm1.weight, block.norm1.bias, 1e-5, bf))
                kernel(f"layernorm ({label})", name, ms, gbytes=rows * d * 6 / 1e9)
                att = block.mixer
                kc, vc = cache.kv_layer(0, 0)
                qkv = torch.randn(rows, 3 * d, device="cuda").to(bf)
                ms = timed(lambda: ops.attention(qkv[:, :d], kc, vc, ctx.tables[0], ctx, att.num_heads, att.scale, None,
                                                 append=(qkv[:, d:2 * d], qkv[:, 2 * d:])))
                if label == "prefill":
                    kernel("attention_tc + kv_append (prefill)", name, ms, gflop=pairs * att.num_heads * 4 * 64 / 1e9)
                else:
                    kernel("attention_decode + merge", name, ms, gbytes=batch * (ctx_len + 1) * 2 * d * 2 / 1e9)
                ms = timed(lambda: ops.linear(xr.to(bf), block.ffn.up_weight, block.ffn.up_bias, activation="gelu_tanh", out_dtype=bf))
                kernel(f"linear {rows}x{ff}x{d} + gelu ({label})", name, ms, gflop=2.0 * rows * ff * d / 1e9)
            else:
                rec, lat = model.blocks[0], model.blocks[1]
                bind = {n: b for n, b in zip(("rec", "lat"), (model.bindings[0], model.bindings[1]))}
                ms = timed(lambda: rec.conv1.forward(xr, rec.norm1, ctx, bind["rec"]["conv1"]))
                kernel(f"rmsnorm + time conv ({label})", name, ms, gbytes=rows * d * 6 / 1e9, like="layernorm")
                y = torch.randn(rows, d, device="cuda")
                ms = timed(lambda: rec.norm1b.add_normed(xr, y))
                kernel(f"rmsnorm + residual ({label})", name, ms, gbytes=rows * d * 12 / 1e9, like="layernorm")
                z = torch.randn(rows, ff, device="cuda")
                ms = timed(lambda: ops.polynorm(z, rec.ffn.coeff, 1e-6, bf))
                kernel(f"polynorm ({label})", name, ms, gbytes=rows * ff * 6 / 1e9, like="layernorm")
                ms = timed(lambda: ops.linear(xr.to(bf), rec.ffn.up_weight, None, out_dtype=f32))
                kernel(f"linear {rows}x{ff}x{d}, 32-bit out ({label})", name, ms, gflop=2.0 * rows * ff * d / 1e9, like="linear + gelu")
                # HGRN2 recurrence
                mx = rec.mixer
                proj = torch.randn(rows, mx.in_weight.shape[0], device="cuda")
                state = cache.state_layer(bind["rec"]["mixer"].group, bind["rec"]["mixer"].layer)
                ms = timed(lambda: ops.hgrn2(proj, state, mx.f_bias, mx.lower, ctx, heads, 128, 128))
                if label == "prefill":
                    kernel("hgrn2 recurrence (prefill)", name, ms, gflop=4.0 * rows * heads * 128 * 128 / 1e9, like="attention_tc")
                else:
                    kernel("hgrn2 recurrence (decode)", name, ms, gbytes=batch * heads * 128 * 128 * 8 / 1e9, like="attention_decode")
                # latent attention and the products around it
                la = lat.mixer
                rope_pages, latent_pages = cache.kv_layer(bind["lat"]["mixer"].group, bind["lat"]["mixer"].layer)
                table = ctx.tables[bind["lat"]["mixer"].group]
                proj = torch.randn(rows, la.in_weight.shape[0], device="cuda")
                ms = timed(lambda: ops.latent_prepare(proj, latent_pages, rope_pages, la.down_norm, la.rotary.freq, la.rotary.gain,
                                                      la.rotary.dims, ctx, table, heads, 128, 64, 512, 1e-6, True))
                kernel(f"latent prepare ({label})", name, ms, gbytes=rows * (la.in_weight.shape[0] * 4 + 576 * 2 + heads * 64 * 4) / 1e9,
                       like="kv_append")
                query = torch.randn(rows, heads, 576, device="cuda")
                qv = proj[:, :la.q_width].view(rows, heads, 192)[:, :, :128]
                ms = timed(lambda: ops.head_matmul(qv, la.uk_heads, query[:, :, :512]))
                kernel(f"per-head product K128 N512 ({label})", name, ms, gflop=2.0 * rows * heads * 128 * 512 / 1e9, like="linear")
                ms = timed(lambda: ops.latent_attention(query, latent_pages, rope_pages, table, ctx, la.scale))
                if label == "prefill":
                    kernel("latent attention (prefill)", name, ms, gflop=pairs * heads * 2 * (576 + 512) / 1e9, like="attention_tc")
                else:
                    kernel("latent attention + merge (decode)", name, ms, gbytes=batch * (ctx_len + 1) * 576 * 2 / 1e9, like="attention_decode")
            close_step(res, slots)
        del engine, model
        torch.cuda.empty_cache()
    result["kernels"] = kernels
    result["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk["source"]}
    return result


def luporax_document(width: int, layers: int, vocab: int = 32000) -> dict:
    """A Luporax model of real-layer sizes: heads of 128 (four query heads to a key/value head), recurrent
    layers as wide as the model in blocks of 128, 16 experts of which 2 run, their inner width and the
    shared expert's adding up to 2.75 x the width per token."""
    heads = width // 128
    mlp = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": width, "limit": 7.0},
           "shared": {"ff": width * 3 // 4, "limit": 7.0}}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "rot": {"dims": 64, "base": 10000.0},
                     "scale": 128 ** -0.5, "softcap": 30.0}}
    lru = {"type": "rglru", "mlp": mlp, "mixer": {"width": width, "blocks": heads, "conv": 4}}
    gru = {"type": "mingru", "mlp": mlp, "mixer": {"width": width}}
    return {"architecture": "Luporax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "logit_scale": 1.0, "layers": [(lru, att, gru, att)[i % 4] for i in range(layers)]}


def run_luporax(width: int, layers: int, batch: int, steps: int, warmup: int, pk: dict) -> dict:
    """Luporax beside Rakalix at equal width, depth and active inner width (bfloat16, random weights): prefill
    of 2 x 1,024 tokens in one step, decode of ``batch`` requests after 512-token prompts through the engine
    (CUDA graphs), and the design's kernels one by one, timed as in ``run_rakalix``."""
    import numpy as np
    import torch

    from ayaka_py_b200 import EngineConfig, Request, SamplingParams, StopCriteria, ops
    from ayaka_py_b200.config.model import LuporaxConfig, RakalixConfig
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import random_model
    from ayaka_py_b200.engine.step import StepEntry

    vocab, heads = 32000, width // 128
    configs = {"luporax": LuporaxConfig.from_dict(luporax_document(width, layers, vocab)),
               "rakalix": RakalixConfig.from_dict(rakalix_document(width, layers, vocab))}
    flush = torch.empty(64 << 20, dtype=torch.float32, device="cuda")
    rs = np.random.RandomState(3)

    def timed(fn, reps=9):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        out = []
        for _ in range(reps):
            flush.fill_(1.0)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return sorted(out)[len(out) // 2]

    result = {"width": width, "layers": layers, "batch": batch}
    kernels = []

    def kernel(name, ms, gbytes=None, gflop=None, like=None):
        row = {"kernel": name, "us": round(ms * 1e3, 1)}
        if gbytes is not None:
            row.update(gb_s=round(gbytes / (ms / 1e3), 1), frac=round(gbytes / (ms / 1e3) / pk["hbm_gbs"], 4), bound="hbm")
        if gflop is not None:
            row.update(tflops=round(gflop / ms, 2), frac=round(gflop / ms / pk["bf16_tflops"], 4), bound="bf16")
        if like:
            row["like"] = like
        kernels.append(row)

    for name, config in configs.items():
        model = random_model(config, 1, "bfloat16", "cuda", generate_on_device=True)
        engine = Engine(model, EngineConfig(dtype="bfloat16", kv_pages=batch * 64 + 130, page_size=16, max_requests=max(batch, 2),
                                            batch_tokens=2048, prefill_chunk=2048, max_model_len=1024, decode_graph=True),
                        eos_token_id=None)
        cache, runner = engine.cache, engine.runner

        def prefill_step():
            slots = [cache.open(f"p{i}") for i in range(2)]
            entries = [StepEntry(sl, 0, rs.randint(0, vocab, 1024).tolist(), [1023]) for sl in slots]
            res = cache.reserve([(e.slot, 0, 1024) for e in entries])
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            runner.run(entries)
            b.record()
            torch.cuda.synchronize()
            cache.commit(res)
            for sl in slots:
                cache.close(sl)
            return a.elapsed_time(b)
        times = [prefill_step() for _ in range(5)][2:]
        prefill_ms = sorted(times)[1]

        total_new = 2 * warmup + steps + 8
        for i in range(batch):
            engine.submit(Request(f"d{i}", rs.randint(0, vocab, PROMPT_LEN).tolist(), SamplingParams(temperature=0.0),
                                  StopCriteria(max_tokens=total_new, ignore_eos=True)))
        while any(st.computed < st.prompt_len for st in engine.scheduler.states.values()):
            engine.step()
        for _ in range(warmup):
            engine.step()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        a.record()
        for _ in range(steps):
            engine.step()
        b.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        decode_ms = a.elapsed_time(b) / steps
        weights = model.weight_bytes()
        result[name] = {"prefill_tok_s": round(2048 / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3),
                        "decode_tok_s": round(batch / (decode_ms / 1e3), 1), "decode_ms_per_step": round(decode_ms, 4),
                        "decode_e2e_tok_s": round(batch * steps / wall, 1), "weight_gb": round(weights / 1e9, 3),
                        "kv_bytes_per_token": cache.bytes_per_token()}
        for rid in list(engine.scheduler.states):
            engine.abort(rid)
        engine.finished.clear()
        if name != "luporax":
            del engine, model
            torch.cuda.empty_cache()
            continue

        # ---- the design's kernels alone, on the shapes of the two steps above
        d, T = width, 2048
        bf, f32 = torch.bfloat16, torch.float32
        x = torch.randn(T, d, device="cuda")
        pairs = 2 * (1024 * 1025 // 2)
        ctx_len = PROMPT_LEN + 64
        lru, att, gru = model.blocks[0], model.blocks[1], model.blocks[2]
        bind = {"lru": model.bindings[0], "att": model.bindings[1], "gru": model.bindings[2]}

        def open_step(lengths, starts=None):
            slots = [cache.open(f"k{i}") for i in range(len(lengths))]
            if starts:
                res = cache.reserve([(sl, 0, st) for sl, st in zip(slots, starts)])
                cache.commit(res)
            res = cache.reserve([(sl, int(cache.length[sl]), n) for sl, n in zip(slots, lengths)])
            ctx = runner.prepare([StepEntry(sl, int(cache.length[sl]), [0] * n, []) for sl, n in zip(slots, lengths)])
            return ctx, res, slots

        for label, lengths, starts in (("prefill", [1024, 1024], None), ("decode", [1] * batch, [ctx_len] * batch)):
            ctx, res, slots = open_step(lengths, starts)
            rows = ctx.num_rows
            xr = x[:rows].contiguous()
            W = width
            ms = timed(lambda: lru.shift.forward(xr, ctx, bind["lru"]["shift"]))
            kernel(f"token shift ({label})", ms, gbytes=rows * d * 6 / 1e9, like="rmsnorm + time conv")
            y = torch.randn(rows, d, device="cuda")
            ms = timed(lambda: lru.norm1.add_normed(xr, y))
            kernel(f"rmsnorm + residual ({label})", ms, gbytes=rows * d * 12 / 1e9, like="rmsnorm + residual")
            # recurrences
            proj = torch.randn(rows, 3 * W, device="cuda")
            st = cache.state_layer(bind["gru"]["mixer"].group, bind["gru"]["mixer"].layer)
            ms = timed(lambda: ops.mingru_scan(proj, st, ctx, W, bf))
            kernel(f"minGRU scan ({label})", ms, gbytes=rows * W * 14 / 1e9, like="hgrn2 recurrence")
            mx = lru.mixer
            st = cache.state_layer(bind["lru"]["mixer"].group, bind["lru"]["mixer"].layer)
            ms = timed(lambda: ops.causal_conv(proj[:, W:2 * W], mx.conv_taps, mx.conv_bias, st, ctx))
            kernel(f"causal conv + state ({label})", ms, gbytes=rows * W * 8 / 1e9, like="rmsnorm + time conv")
            u = torch.randn(rows, W, device="cuda")
            gates = torch.empty(rows, mx.blocks, 2 * (W // mx.blocks), device="cuda")
            ms = timed(lambda: ops.head_matmul(u.view(rows, mx.blocks, W // mx.blocks), mx.gate_weight, gates))
            kernel(f"per-block gate product K128 N256 ({label})", ms, gflop=2.0 * rows * W * 256 / 1e9, like="per-head product")
            ms = timed(lambda: ops.rglru_scan(proj, u, gates, mx.gate_bias, mx.lam, st, ctx, W, mx.blocks, 8.0, bf))
            kernel(f"RG-LRU scan ({label})", ms, gbytes=rows * W * 18 / 1e9, like="hgrn2 recurrence")
            # attention
            am = att.mixer
            kp, vp = cache.kv_layer(bind["att"]["mixer"].group, bind["att"]["mixer"].layer)
            table = ctx.tables[bind["att"]["mixer"].group]
            G = am.kv_heads
            aproj = torch.randn(rows, am.in_weight.shape[0], device="cuda")
            ms = timed(lambda: ops.qk_norm_rotary(aproj, kp, vp, am.q_norm, am.k_norm, am.rotary.freq, am.rotary.dims, ctx, table,
                                                  heads, 1e-6, True, bf))
            kernel(f"qk norm + rotary + filing ({label})", ms, gbytes=rows * (heads + 2 * G) * 128 * 6 / 1e9, like="latent prepare")
            q = torch.randn(rows, heads * 128, device="cuda").to(bf)
            ms = timed(lambda: ops.sigmoid_attention(q, kp, vp, table, ctx, heads, am.scale, am.softcap, am.head_bias))
            if label == "prefill":
                kernel("sigmoid attention (prefill)", ms, gflop=pairs * heads * 2 * 256 / 1e9, like="latent attention")
            else:
                kernel("sigmoid attention + merge (decode)", ms, gbytes=batch * (ctx_len + 1) * G * 256 * 2 / 1e9, like="latent attention")
            # experts
            ff = lru.ffn
            h = xr.to(bf)
            logits = torch.randn(rows, 16, device="cuda")
            ms = timed(lambda: ops.moe_route(logits, 16, 2))
            kernel(f"routing + plan ({label})", ms)
            route = ops.moe_route(logits, 16, 2)
            touched = min(16, 2 * rows) * 2 * width * d * 2 / 1e9
            if label == "prefill":
                ms = timed(lambda: ops.moe_experts_tc(h, ff.in_weight, ff.down_weight, route, 7.0, 1.702))
                kernel("experts on tcgen05: plan, gather, gate | up, activation, down (prefill)", ms,
                       gflop=2.0 * 2 * rows * 3 * width * d / 1e9, like="linear + gelu")
            else:
                touched = 2 * rows * 2 * width * d * 2 / 1e9          # every pair streams its expert's rows
                ms = timed(lambda: ops.moe_gemv(h, ff.in_weight, route, glu=(7.0, 1.702)))
                kernel("experts' gate | up product + activation, pair by pair (decode)", ms, gbytes=touched, like="linear (decode)")
                hidden = ops.moe_gemv(h, ff.in_weight, route, glu=(7.0, 1.702))
                ms = timed(lambda: ops.moe_gemv(hidden, ff.down_weight, route, glu=None))
                kernel("experts' down product, pair by pair (decode)", ms, gbytes=touched / 2, like="linear (decode)")
                ms = timed(lambda: ops.moe_gemm(h, ff.in_weight, route, glu=(7.0, 1.702), out_dtype=bf))
                kernel("grouped gate | up product + activation on mma.sync (decode; not the path taken)", ms,
                       gbytes=min(16, 2 * rows) * 2 * width * d * 2 / 1e9, like="linear (decode)")
            picked = torch.randn(2 * rows, d, device="cuda")
            shared = torch.randn(rows, d, device="cuda")
            sp = torch.randn(rows, ff.shared_in.shape[0], device="cuda")
            ms = timed(lambda: ops.moe_combine(picked, route, shared, sp[:, 2 * ff.shared_inner]))
            kernel(f"weighted sum of experts ({label})", ms, gbytes=rows * d * 16 / 1e9, like="rmsnorm + residual")
            ms = timed(lambda: ops.glu_limited(sp, ff.shared_inner, 7.0, 1.702, bf))
            kernel(f"gated activation ({label})", ms, gbytes=rows * ff.shared_inner * 10 / 1e9, like="polynorm")
            cache.rollback(res)
            for sl in slots:
                cache.close(sl)
        del engine, model
        torch.cuda.empty_cache()
    result["kernels"] = kernels
    result["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk["source"]}
    return result


def vedadra_document(width: int, layers: int, vocab: int = 32000) -> dict:
    """A Vedadra model of real-layer sizes: heads of 128 (four query heads to a key/value head); talking
    attention and differential attention (two maps of 64, values of 128) in turn, windows of 512 keys, the
    differential one keeping its first 4; a gated feed-forward of 8/3 x the width; norms in 4 groups; the first
    two layers run twice."""
    heads = width // 128
    kv = max(1, heads // 4)
    ff = {"kind": "dense", "ff": (width * 8 // 3 + 127) // 128 * 128}
    talk = {"type": "attention", "mlp": ff,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 512}}}
    diff = {"type": "attention_2", "mlp": ff,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": 64, "vdim": 128, "scale": 64 ** -0.5, "diff": 0.3,
                      "mask": {"size": 512, "keep_first": 4}}}
    return {"architecture": "Vedadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": 4},
            "loop": {"start": 0, "stop": min(2, layers), "times": 2}, "layers": [(talk, diff)[i % 2] for i in range(layers)]}


def _vedadra_kernels(name, model, cache, runner, width, ff, batch, timed, kernel) -> None:
    """The kernels of one layer alone, on the shapes of the prefill step (2 x 1,024 rows) and of a decode step
    (``batch`` rows after 576 cached tokens).  FLOPs and bytes are the design's own: (query, key) pairs inside
    the window, a key head read once per group of query heads."""
    import torch

    from ayaka_py_b200 import ops
    from ayaka_py_b200.engine.step import StepEntry

    d, bf, f32 = width, torch.bfloat16, torch.float32
    x = torch.randn(2048, d, device="cuda")
    ctx_len = PROMPT_LEN + 64

    def pairs_of(window, keep, n=1024):
        return 2 * sum(min(i + 1, window) + max(0, min(keep, i + 1 - window)) for i in range(n))

    def open_step(lengths, starts=None):
        slots = [cache.open(f"k{i}") for i in range(len(lengths))]
        if starts:
            cache.commit(cache.reserve([(sl, 0, st) for sl, st in zip(slots, starts)]))
        res = cache.reserve([(sl, int(cache.length[sl]), n) for sl, n in zip(slots, lengths)])
        ctx = runner.prepare([StepEntry(sl, int(cache.length[sl]), [0] * n, []) for sl, n in zip(slots, lengths)])
        return ctx, res, slots

    for label, lengths, starts in (("prefill", [1024, 1024], None), ("decode", [1] * batch, [ctx_len] * batch)):
        ctx, res, slots = open_step(lengths, starts)
        rows = ctx.num_rows
        xr = x[:rows].contiguous()
        if name == "gpt2":
            block = model.blocks[0]
            ms = timed(lambda: ops.layernorm(xr, block.norm1.weight, block.norm1.bias, 1e-5, bf))
            kernel(f"layernorm ({label})", name, ms, gbytes=rows * d * 6 / 1e9)
            att = block.mixer
            kc, vc = cache.kv_layer(0, 0)
            qkv = torch.randn(rows, 3 * d, device="cuda").to(bf)
            ms = timed(lambda: ops.attention(qkv[:, :d], kc, vc, ctx.tables[0], ctx, att.num_heads, att.scale, None,
                                             append=(qkv[:, d:2 * d], qkv[:, 2 * d:])))
            if label == "prefill":
                kernel("attention_tc + kv_append (prefill)", name, ms, gflop=pairs_of(1 << 30, 0) * att.num_heads * 4 * 64 / 1e9)
            else:
                kernel("attention_decode + merge", name, ms, gbytes=batch * (ctx_len + 1) * 2 * d * 2 / 1e9)
            inner = block.ffn.up_weight.shape[0]
            ms = timed(lambda: ops.linear(xr.to(bf), block.ffn.up_weight, block.ffn.up_bias, activation="gelu_tanh", out_dtype=bf))
            kernel(f"linear {rows}x{inner}x{d} + gelu ({label})", name, ms, gflop=2.0 * rows * inner * d / 1e9)
        else:
            talk, diff = model.blocks[0], model.blocks[1 % len(model.blocks)]
            bind = {"talk": model.bindings[0]["mixer"], "diff": model.bindings[1 % len(model.blocks)]["mixer"]}
            groups = talk.norm1.groups
            ms = timed(lambda: talk.norm1.forward(xr, ctx))
            kernel(f"rmsnorm in {groups} groups ({label})", name, ms, gbytes=rows * d * 6 / 1e9, like="layernorm")
            y = torch.randn(rows, d, device="cuda")
            ms = timed(lambda: talk.norm1b.add_normed(xr, y))
            kernel(f"rmsnorm in {groups} groups + residual ({label})", name, ms, gbytes=rows * d * 12 / 1e9, like="layernorm")
            z = torch.randn(rows, 2 * ff, device="cuda")
            ms = timed(lambda: ops.gated_act(z, ff, "gelu_tanh", bf))
            kernel(f"gelu(gate) * up ({label})", name, ms, gbytes=rows * ff * 10 / 1e9, like="layernorm")
            ms = timed(lambda: ops.linear(xr.to(bf), talk.ffn.in_weight, None, out_dtype=f32))
            kernel(f"linear {rows}x{2 * ff}x{d}, 32-bit out ({label})", name, ms, gflop=2.0 * rows * 2 * ff * d / 1e9, like="linear + gelu")
            # talking attention
            ta = talk.mixer
            H, G, D = ta.heads, ta.kv_heads, ta.dim
            kp, vp = cache.kv_layer(bind["talk"].group, bind["talk"].layer)
            table = ctx.tables[bind["talk"].group]
            proj = torch.randn(rows, ta.in_weight.shape[0], device="cuda")
            ms = timed(lambda: ops.head_norm_prepare(proj, kp, vp, ta.q_norm, ta.k_norm, ctx, table, H, G, D, 1, H * D, 1e-6, True, bf, mix=ta.mix))
            kernel(f"head norms + score mix into the queries + filing ({label})", name, ms,
                   gbytes=rows * ((H + G) * D * 4 + H * G * D * 2 + 2 * G * D * 2) / 1e9, like="kv_append")
            q = (torch.randn(rows, H * G * D, device="cuda") * D ** -0.5).to(bf)
            gate = proj[:, (H + G) * D:(2 * H + G) * D]
            ms = timed(lambda: ops.grouped_attention(q, kp, vp, table, ctx, heads=H, key_heads=1, key_dim=G * D, scale=1.0,
                                                     slopes=ta.slopes, window=ta.window, gate=gate))
            if label == "prefill":
                kernel("talking attention (prefill)", name, ms, gflop=pairs_of(ta.window, 0) * H * (4 * D + 2 * H) / 1e9, like="attention_tc")
                kernel("talking attention (prefill), products as run", name, ms, gflop=pairs_of(ta.window, 0) * H * (2 * G * D + 2 * D) / 1e9)
            else:
                kernel("talking attention + merge (decode)", name, ms, gbytes=batch * min(ctx_len + 1, ta.window) * 2 * G * D * 2 / 1e9,
                       like="attention_decode")
            # the framework's other attention on mma.sync (Luporax's, weights that are not normalized), on the same pages
            kpg = kp.view(kp.shape[0], kp.shape[1], G, D)
            qs = (torch.randn(rows, H * D, device="cuda") * D ** -0.5).to(bf)
            ms = timed(lambda: ops.sigmoid_attention(qs, kpg, vp, table, ctx, H, D ** -0.5, 30.0, None))
            if label == "prefill":
                kernel("sigmoid attention of Luporax, same heads and pages, no window (prefill)", "luporax", ms,
                       gflop=pairs_of(1 << 30, 0) * H * 4 * D / 1e9)
            else:
                kernel("sigmoid attention of Luporax + merge, same heads and pages, no window (decode)", "luporax", ms,
                       gbytes=batch * (ctx_len + 1) * 2 * G * D * 2 / 1e9)
            # differential attention
            da = diff.mixer
            H, G, D, Dv = da.heads, da.kv_heads, da.dim, da.vdim
            kp, vp = cache.kv_layer(bind["diff"].group, bind["diff"].layer)
            table = ctx.tables[bind["diff"].group]
            proj = torch.randn(rows, da.in_weight.shape[0], device="cuda")
            ms = timed(lambda: ops.head_norm_prepare(proj, kp, vp, da.q_norm, da.k_norm, ctx, table, H, G, D, 2, (H + G) * 2 * D, 1e-6, True, bf))
            kernel(f"head norms of both maps + filing ({label})", name, ms,
                   gbytes=rows * ((H + G) * 2 * D * 6 + G * Dv * 6) / 1e9, like="kv_append")
            q = torch.randn(rows, 2 * H * D, device="cuda").to(bf)
            ms = timed(lambda: ops.grouped_attention(q, kp, vp, table, ctx, heads=2 * H, key_heads=2 * G, key_dim=D, scale=da.scale,
                                                     window=da.window, keep_first=da.keep_first, maps=2, lam=da.lam,
                                                     post_scale=1.0 - da.diff, eps=1e-6))
            if label == "prefill":
                kernel("differential attention + difference and head norm (prefill)", name, ms,
                       gflop=pairs_of(da.window, da.keep_first) * H * 2 * (2 * D + 2 * Dv) / 1e9, like="attention_tc")
            else:
                kernel("differential attention + merge, difference and head norm (decode)", name, ms,
                       gbytes=batch * (min(ctx_len + 1, da.window) + da.keep_first) * G * (2 * D + Dv) * 2 / 1e9, like="attention_decode")
        cache.rollback(res)
        for sl in slots:
            cache.close(sl)


def run_vedadra(width: int, layers: int, batch: int, steps: int, warmup: int, pk: dict) -> dict:
    """Vedadra beside GPT-2, the closest model (softmax attention, dense feed-forward), at equal width, equal
    layer runs and equal feed-forward weights (bfloat16, random weights): prefill of 2 x 1,024 tokens in one step,
    decode of ``batch`` requests after 512-token prompts through the engine (CUDA graphs), and the design's
    kernels one by one beside GPT-2's, timed as in ``run_rakalix``."""
    import numpy as np
    import torch

    from ayaka_py_b200 import EngineConfig, GPT2Config, Request, SamplingParams, StopCriteria, ops
    from ayaka_py_b200.config.model import VedadraConfig
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import random_model
    from ayaka_py_b200.engine.step import StepEntry

    vocab = 32000
    document = vedadra_document(width, layers, vocab)
    ved = VedadraConfig.from_dict(document)
    runs = len(ved.run_order())
    ff = document["layers"][0]["mlp"]["ff"]
    configs = {"vedadra": ved,
               "gpt2": GPT2Config(n_layer=runs, n_embd=width, n_head=width // 64, n_inner=ff * 3 // 2, vocab_size=vocab,
                                  n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new")}
    flush = torch.empty(64 << 20, dtype=torch.float32, device="cuda")
    rs = np.random.RandomState(3)

    def timed(fn, reps=9):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        out = []
        for _ in range(reps):
            flush.fill_(1.0)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return sorted(out)[len(out) // 2]

    result = {"width": width, "layers": layers, "layer_runs": runs, "inner": ff, "batch": batch}
    kernels = []

    def kernel(name, model, ms, gbytes=None, gflop=None, like=None):
        row = {"kernel": name, "model": model, "us": round(ms * 1e3, 1)}
        if gbytes is not None:
            row.update(gb_s=round(gbytes / (ms / 1e3), 1), frac=round(gbytes / (ms / 1e3) / pk["hbm_gbs"], 4), bound="hbm")
        if gflop is not None:
            row.update(tflops=round(gflop / ms, 2), frac=round(gflop / ms / pk["bf16_tflops"], 4), bound="bf16")
        if like:
            row["like"] = like
        kernels.append(row)

    for name, config in configs.items():
        model = random_model(config, 1, "bfloat16", "cuda", generate_on_device=True)
        engine = Engine(model, EngineConfig(dtype="bfloat16", kv_pages=batch * 64 + 130, page_size=16, max_requests=max(batch, 2),
                                            batch_tokens=2048, prefill_chunk=2048, max_model_len=1024, decode_graph=True),
                        eos_token_id=None)
        cache, runner = engine.cache, engine.runner

        def prefill_step():
            slots = [cache.open(f"p{i}") for i in range(2)]
            entries = [StepEntry(sl, 0, rs.randint(0, vocab, 1024).tolist(), [1023]) for sl in slots]
            res = cache.reserve([(e.slot, 0, 1024) for e in entries])
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            runner.run(entries)
            b.record()
            torch.cuda.synchronize()
            cache.commit(res)
            for sl in slots:
                cache.close(sl)
            return a.elapsed_time(b)
        times = [prefill_step() for _ in range(5)][2:]
        prefill_ms = sorted(times)[1]

        total_new = 2 * warmup + steps + 8
        for i in range(batch):
            engine.submit(Request(f"d{i}", rs.randint(0, vocab, PROMPT_LEN).tolist(), SamplingParams(temperature=0.0),
                                  StopCriteria(max_tokens=total_new, ignore_eos=True)))
        while any(st.computed < st.prompt_len for st in engine.scheduler.states.values()):
            engine.step()
        for _ in range(warmup):
            engine.step()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        a.record()
        for _ in range(steps):
            engine.step()
        b.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        decode_ms = a.elapsed_time(b) / steps
        weights = model.weight_bytes()
        result[name] = {"prefill_tok_s": round(2048 / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3),
                        "decode_tok_s": round(batch / (decode_ms / 1e3), 1), "decode_ms_per_step": round(decode_ms, 4),
                        "decode_e2e_tok_s": round(batch * steps / wall, 1), "weight_gb": round(weights / 1e9, 3),
                        "decode_hbm_frac": round(weights / (decode_ms / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                        "kv_bytes_per_token": cache.bytes_per_token()}
        for rid in list(engine.scheduler.states):
            engine.abort(rid)
        engine.finished.clear()
        _vedadra_kernels(name, model, cache, runner, width, ff, batch, timed, kernel)
        del engine, model
        torch.cuda.empty_cache()
    result["kernels"] = kernels
    result["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk["source"]}
    return result


def tesozen_document(width: int, layers: int, vocab: int = 32000) -> dict:
    """A Tesozen model of real-layer sizes: heads of 128 (four query heads to a key/value head, chunks of 512),
    an mLSTM with a 128 x 128 memory per head, a latent of 512, 16 experts in 4 groups of which 2 experts of 2
    groups run, their inner width and the shared expert's adding up to 2.75 x the width per token (Luporax's
    active inner width), and one dense feed-forward of that width."""
    heads = width // 128
    moe = {"kind": "moe", "router": {"experts": 16, "top": 2, "scale": 2.5, "groups": {"count": 4, "keep": 2}},
           "expert": {"ff": width}, "shared": {"ff": width * 3 // 4}}
    att = {"type": "attention",
           "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "diff": 0.6,
                     "mask": {"size": 512}}}
    rec = {"type": "mlstm", "mlp": moe, "mixer": {"heads": heads, "dim": 128, "vdim": 128, "gate_cap": 15.0}}
    lat = {"type": "latent_attention", "mlp": moe, "mixer": {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": 512, "scale": 128 ** -0.5}}
    four = (rec, dict(att, mlp=moe), lat, dict(att, mlp={"kind": "dense", "ff": width * 11 // 4}))
    return {"architecture": "Tesozen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": float(width) ** 0.5},
            "layers": [four[i % 4] for i in range(layers)]}


def run_tesozen(width: int, layers: int, batch: int, steps: int, warmup: int, pk: dict) -> dict:
    """Tesozen beside Luporax, the closest model (recurrent and attention layers with routed experts), at equal
    width, depth and active inner width (bfloat16, random weights): prefill of 2 x 1,024 tokens in one step,
    decode of ``batch`` requests after 512-token prompts through the engine (CUDA graphs), and the design's
    kernels one by one beside the like kernels of Luporax at equal sizes, timed as in ``run_rakalix``."""
    import numpy as np
    import torch

    from ayaka_py_b200 import EngineConfig, Request, SamplingParams, StopCriteria, ops
    from ayaka_py_b200.config.model import LuporaxConfig, TesozenConfig
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import random_model
    from ayaka_py_b200.engine.step import StepEntry

    vocab, heads = 32000, width // 128
    configs = {"tesozen": TesozenConfig.from_dict(tesozen_document(width, layers, vocab)),
               "luporax": LuporaxConfig.from_dict(luporax_document(width, layers, vocab))}
    flush = torch.empty(64 << 20, dtype=torch.float32, device="cuda")
    rs = np.random.RandomState(3)

    def timed(fn, reps=9):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        out = []
        for _ in range(reps):
            flush.fill_(1.0)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return sorted(out)[len(out) // 2]

    result = {"width": width, "layers": layers, "batch": batch}
    kernels = []

    def kernel(name, model, ms, gbytes=None, gflop=None, like=None):
        row = {"kernel": name, "model": model, "us": round(ms * 1e3, 1)}
        if gbytes is not None:
            row.update(gb_s=round(gbytes / (ms / 1e3), 1), frac=round(gbytes / (ms / 1e3) / pk["hbm_gbs"], 4), bound="hbm")
        if gflop is not None:
            row.update(tflops=round(gflop / ms, 2), frac=round(gflop / ms / pk["bf16_tflops"], 4), bound="bf16")
        if like:
            row["like"] = like
        kernels.append(row)

    for name, config in configs.items():
        model = random_model(config, 1, "bfloat16", "cuda", generate_on_device=True)
        engine = Engine(model, EngineConfig(dtype="bfloat16", kv_pages=batch * 64 + 130, page_size=16, max_requests=max(batch, 2),
                                            batch_tokens=2048, prefill_chunk=2048, max_model_len=1024, decode_graph=True),
                        eos_token_id=None)
        cache, runner = engine.cache, engine.runner

        def prefill_step():
            slots = [cache.open(f"p{i}") for i in range(2)]
            entries = [StepEntry(sl, 0, rs.randint(0, vocab, 1024).tolist(), [1023]) for sl in slots]
            res = cache.reserve([(e.slot, 0, 1024) for e in entries])
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            runner.run(entries)
            b.record()
            torch.cuda.synchronize()
            cache.commit(res)
            for sl in slots:
                cache.close(sl)
            return a.elapsed_time(b)
        times = [prefill_step() for _ in range(5)][2:]
        prefill_ms = sorted(times)[1]

        total_new = 2 * warmup + steps + 8
        for i in range(batch):
            engine.submit(Request(f"d{i}", rs.randint(0, vocab, PROMPT_LEN).tolist(), SamplingParams(temperature=0.0),
                                  StopCriteria(max_tokens=total_new, ignore_eos=True)))
        while any(st.computed < st.prompt_len for st in engine.scheduler.states.values()):
            engine.step()
        for _ in range(warmup):
            engine.step()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        a.record()
        for _ in range(steps):
            engine.step()
        b.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        decode_ms = a.elapsed_time(b) / steps
        result[name] = {"prefill_tok_s": round(2048 / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3),
                        "decode_tok_s": round(batch / (decode_ms / 1e3), 1), "decode_ms_per_step": round(decode_ms, 4),
                        "decode_e2e_tok_s": round(batch * steps / wall, 1), "weight_gb": round(model.weight_bytes() / 1e9, 3),
                        "kv_bytes_per_token": cache.bytes_per_token()}
        for rid in list(engine.scheduler.states):
            engine.abort(rid)
        engine.finished.clear()

        # ---- the kernels alone, on the shapes of the two steps above
        d, T = width, 2048
        bf, f32 = torch.bfloat16, torch.float32
        x = torch.randn(T, d, device="cuda")
        pairs = 2 * (1024 * 1025 // 2)
        chunk_pairs = 2 * 2 * (512 * 513 // 2)              # two prompts of two chunks of 512
        ctx_len = PROMPT_LEN + 64

        def open_step(lengths, starts=None):
            slots = [cache.open(f"k{i}") for i in range(len(lengths))]
            if starts:
                res = cache.reserve([(sl, 0, st) for sl, st in zip(slots, starts)])
                cache.commit(res)
            res = cache.reserve([(sl, int(cache.length[sl]), n) for sl, n in zip(slots, lengths)])
            ctx = runner.prepare([StepEntry(sl, int(cache.length[sl]), [0] * n, []) for sl, n in zip(slots, lengths)])
            return ctx, res, slots

        for label, lengths, starts in (("prefill", [1024, 1024], None), ("decode", [1] * batch, [ctx_len] * batch)):
            ctx, res, slots = open_step(lengths, starts)
            rows = ctx.num_rows
            xr = x[:rows].contiguous()
            y = torch.randn(rows, d, device="cuda")
            W, D = width, 128
            if name == "tesozen":
                rec, att, lat = model.blocks[0], model.blocks[1], model.blocks[2]
                bind = {"rec": model.bindings[0]["mixer"], "att": model.bindings[1]["mixer"], "lat": model.bindings[2]["mixer"]}
                ms = timed(lambda: rec.norm1.forward(xr, ctx))
                kernel(f"layer norm ({label})", name, ms, gbytes=rows * d * 6 / 1e9, like="token shift")
                ms = timed(lambda: rec.norm1b.add_normed_then(xr, y, rec.norm2))
                kernel(f"layer norm + residual + next layer norm ({label})", name, ms, gbytes=rows * d * 14 / 1e9, like="rmsnorm + residual")
                mx = rec.mixer
                proj = torch.randn(rows, mx.in_weight.shape[0], device="cuda")
                st = cache.state_layer(bind["rec"].group, bind["rec"].layer)
                ms = timed(lambda: ops.mlstm(proj, st, mx.norm_weight, ctx, heads, D, D, mx.cap, 1e-6, bf))
                if label == "prefill":      # per token and head: the state's two products (q S and k v^T) and the chunk's own (16 tokens)
                    kernel("mLSTM recurrence, 16 tokens at a time + norm and gate (prefill)", name, ms,
                           gflop=rows * heads * (4.0 * D * D + 2 * 16 * 2 * D) / 1e9, like="RG-LRU scan; HGRN2 recurrence")
                else:
                    kernel("mLSTM recurrence + norm and gate (decode)", name, ms, gbytes=batch * heads * D * D * 8 / 1e9,
                           like="RG-LRU scan; HGRN2 recurrence")
                # the engine's other matrix-memory recurrence (Rakalix's HGRN2) on the same rows, heads and state size
                hproj = torch.randn(rows, heads * 3 * D, device="cuda")
                hstate = torch.zeros(st.shape[0], heads, D, D, device="cuda")
                hbias, hlower = torch.zeros(heads * D, device="cuda"), torch.full((heads * D,), 0.5, device="cuda")
                ms = timed(lambda: ops.hgrn2(hproj, hstate, hbias, hlower, ctx, heads, D, D))
                if label == "prefill":
                    kernel("HGRN2 recurrence of Rakalix, same heads and state (prefill)", "rakalix", ms, gflop=rows * heads * 4.0 * D * D / 1e9)
                else:
                    kernel("HGRN2 recurrence of Rakalix, same heads and state (decode)", "rakalix", ms, gbytes=batch * heads * D * D * 8 / 1e9)
                am = att.mixer
                G = am.kv_heads
                kp, vp = cache.kv_layer(bind["att"].group, bind["att"].layer)
                table = ctx.tables[bind["att"].group]
                aproj = torch.randn(rows, am.in_weight.shape[0], device="cuda")
                ms = timed(lambda: ops.head_norm_prepare(aproj, kp, vp, am.q_norm, am.k_norm, ctx, table, heads, G, D, 2, (heads + G) * 2 * D,
                                                         1e-6, True, bf))
                kernel(f"head norms + filing of keys and values ({label})", name, ms, gbytes=rows * (2 * heads + 3 * G) * D * 6 / 1e9,
                       like="qk norm + rotary + filing")
                q = torch.randn(rows, 2 * heads * D, device="cuda").to(bf)
                gate = aproj[:, (heads + G) * 2 * D + G * D:]
                ms = timed(lambda: ops.grouped_attention(q, kp, vp, table, ctx, heads=2 * heads, key_heads=2 * G, key_dim=D, scale=am.scale,
                                                         maps=2, lam=am.lam, post_scale=0.4, eps=1e-6, chunk=am.chunk, gate=gate))
                if label == "prefill":
                    kernel("differential attention in chunks of 512 + finish (prefill)", name, ms, gflop=chunk_pairs * 2 * heads * 2 * 256 / 1e9,
                           like="sigmoid attention")
                else:
                    seen = (ctx_len % 512) + 1
                    kernel("differential attention in chunks of 512 + finish (decode)", name, ms, gbytes=batch * seen * G * 3 * D * 2 / 1e9,
                           like="sigmoid attention")
                lm = lat.mixer
                lpages = cache.kv_layer(bind["lat"].group, bind["lat"].layer)
                ltable = ctx.tables[bind["lat"].group]
                lproj = torch.randn(rows, lm.in_weight.shape[0], device="cuda")
                zero = torch.zeros(1, device="cuda")
                ms = timed(lambda: ops.latent_prepare(lproj, lpages[1], lpages[0], lm.down_norm, zero, 1.0, 0, ctx, ltable, heads, D, 0, 512,
                                                      1e-6, True))
                kernel(f"latent norm + filing ({label})", name, ms, gbytes=rows * 512 * 6 / 1e9, like="qk norm + rotary + filing")
                query = torch.randn(rows, heads, 512, device="cuda")
                ms = timed(lambda: ops.head_matmul(lproj[:, :heads * D].view(rows, heads, D), lm.uk_heads, query))
                kernel(f"per-head product K128 N512 ({label})", name, ms, gflop=2.0 * rows * heads * D * 512 / 1e9, like="per-block gate product")
                ms = timed(lambda: ops.latent_attention(query, lpages[1], lpages[0], ltable, ctx, lm.scale))
                if label == "prefill":
                    kernel("latent attention (prefill)", name, ms, gflop=pairs * heads * 2 * 1024 / 1e9, like="sigmoid attention")
                else:
                    kernel("latent attention + merge (decode)", name, ms, gbytes=batch * (ctx_len + 1) * 512 * 2 / 1e9, like="sigmoid attention")
                ff = rec.ffn
                logits = torch.randn(rows, 16, device="cuda")
                scored = {"correction": ff.correction, "groups": 4, "keep": 2, "factor": 2.5}
                ms = timed(lambda: ops.moe_route(logits, 16, 2, scored))
                kernel(f"routing by scores in groups + plan ({label})", name, ms, like="routing + plan")
                route = ops.moe_route(logits, 16, 2, scored)
                h = xr.to(bf)
                inf = float("inf")
                if label == "prefill":
                    ms = timed(lambda: ops.moe_experts_tc(h, ff.in_weight, ff.down_weight, route, inf, 1.0, 0.0))
                    kernel("experts on tcgen05: plan, gather, gate | up, silu gating, down (prefill)", name, ms,
                           gflop=2.0 * 2 * rows * 3 * width * d / 1e9, like="experts on tcgen05")
                else:
                    ms = timed(lambda: ops.moe_gemv(h, ff.in_weight, route, glu=(inf, 1.0, 0.0)))
                    kernel("experts' gate | up product + silu gating, pair by pair (decode)", name, ms, gbytes=2 * rows * 2 * width * d * 2 / 1e9,
                           like="experts' gate | up product")
                dn = model.blocks[3].ffn if len(model.blocks) > 3 else None
                if dn is not None:
                    ms = timed(lambda: ops.linear(h, dn.up_weight, None, activation="relu2", out_dtype=bf))
                    kernel(f"linear {rows}x{dn.inner}x{d} + squared ReLU ({label})", name, ms, gflop=2.0 * rows * dn.inner * d / 1e9,
                           like="linear + gelu")
                    ms = timed(lambda: ops.linear(h, dn.up_weight, None, activation="gelu_tanh", out_dtype=bf))
                    kernel(f"linear {rows}x{dn.inner}x{d} + gelu ({label})", "gpt2", ms, gflop=2.0 * rows * dn.inner * d / 1e9)
            else:
                lru, att = model.blocks[0], model.blocks[1]
                bind = {"lru": model.bindings[0], "att": model.bindings[1]}
                ms = timed(lambda: lru.shift.forward(xr, ctx, bind["lru"]["shift"]))
                kernel(f"token shift ({label})", name, ms, gbytes=rows * d * 6 / 1e9)
                ms = timed(lambda: lru.norm1.add_normed(xr, y))
                kernel(f"rmsnorm + residual ({label})", name, ms, gbytes=rows * d * 12 / 1e9)
                mx = lru.mixer
                proj = torch.randn(rows, 3 * W, device="cuda")
                st = cache.state_layer(bind["lru"]["mixer"].group, bind["lru"]["mixer"].layer)
                u = torch.randn(rows, W, device="cuda")
                gates = torch.empty(rows, mx.blocks, 2 * (W // mx.blocks), device="cuda")
                ms = timed(lambda: ops.head_matmul(u.view(rows, mx.blocks, W // mx.blocks), mx.gate_weight, gates))
                kernel(f"per-block gate product K128 N256 ({label})", name, ms, gflop=2.0 * rows * W * 256 / 1e9)
                ms = timed(lambda: ops.rglru_scan(proj, u, gates, mx.gate_bias, mx.lam, st, ctx, W, mx.blocks, 8.0, bf))
                kernel(f"RG-LRU scan ({label})", name, ms, gbytes=rows * W * 18 / 1e9)
                am = att.mixer
                kp, vp = cache.kv_layer(bind["att"]["mixer"].group, bind["att"]["mixer"].layer)
                table = ctx.tables[bind["att"]["mixer"].group]
                G = am.kv_heads
                aproj = torch.randn(rows, am.in_weight.shape[0], device="cuda")
                ms = timed(lambda: ops.qk_norm_rotary(aproj, kp, vp, am.q_norm, am.k_norm, am.rotary.freq, am.rotary.dims, ctx, table,
                                                      heads, 1e-6, True, bf))
                kernel(f"qk norm + rotary + filing ({label})", name, ms, gbytes=rows * (heads + 2 * G) * 128 * 6 / 1e9)
                q = torch.randn(rows, heads * 128, device="cuda").to(bf)
                ms = timed(lambda: ops.sigmoid_attention(q, kp, vp, table, ctx, heads, am.scale, am.softcap, am.head_bias))
                if label == "prefill":
                    kernel("sigmoid attention (prefill)", name, ms, gflop=pairs * heads * 2 * 256 / 1e9)
                else:
                    kernel("sigmoid attention + merge (decode)", name, ms, gbytes=batch * (ctx_len + 1) * G * 256 * 2 / 1e9)
                ff = lru.ffn
                h = xr.to(bf)
                logits = torch.randn(rows, 16, device="cuda")
                ms = timed(lambda: ops.moe_route(logits, 16, 2))
                kernel(f"routing + plan ({label})", name, ms)
                route = ops.moe_route(logits, 16, 2)
                if label == "prefill":
                    ms = timed(lambda: ops.moe_experts_tc(h, ff.in_weight, ff.down_weight, route, 7.0, 1.702))
                    kernel("experts on tcgen05: plan, gather, gate | up, activation, down (prefill)", name, ms,
                           gflop=2.0 * 2 * rows * 3 * width * d / 1e9)
                else:
                    ms = timed(lambda: ops.moe_gemv(h, ff.in_weight, route, glu=(7.0, 1.702)))
                    kernel("experts' gate | up product + activation, pair by pair (decode)", name, ms, gbytes=2 * rows * 2 * width * d * 2 / 1e9)
            cache.rollback(res)
            for sl in slots:
                cache.close(sl)
        del engine, model
        torch.cuda.empty_cache()
    result["kernels"] = kernels
    result["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk["source"]}
    return result


def reference_line(args) -> dict:
    """The reference arm: same shape, batch, prompt length and step counts, the reference's own engine."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm
    except Exception as exc:           # noqa: BLE001
        return {"impl": "reference", "unavailable": f"baseline/reference_arm.py cannot be imported: {exc!r}"[:300]}
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "ayaka")):
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref "
                "(python baseline/install_reference.py <checkout of the reference>)"}
    shape = {**XL, "n_layer": args.layers}
    repeats = -(-MIN_TIMED_STEPS // args.steps)
    sampler = ClockSampler()
    sampler.start()
    try:
        r = reference_arm.run(shape, batch=args.batch, prompt_len=PROMPT_LEN, steps=args.steps * repeats,
                              warmup=args.warmup, points=() if args.no_points else (1, 64), decode_graph=False,
                              prefill_tokens=0 if args.no_points else 2048)
    except BaseException as exc:       # noqa: BLE001
        text = " ".join(f"{type(exc).__name__}: {exc}".split())
        return {"impl": "reference", "unavailable": f"the reference raised on this box: {text}"[:400]}
    finally:
        sampler.stop()
    line = {"metric": "decode tokens per second, GPT-2 XL shape", "value": round(r["tok_s"], 1), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(r["ms_per_step"], 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "reference",
            "config": {"model": "gpt2-xl shape, the reference's own random checkpoint", "global_batch": args.batch,
                       "seq_len": XL["n_positions"], "parallelism": "single GPU", "n_layer": args.layers,
                       "n_layer_of_shape": XL["n_layer"], "prompt_len": PROMPT_LEN, "page_size": 16,
                       "timed_steps": args.steps * repeats, "backend": "triton", "decode_graph": False,
                       "driver": "ServingRuntime's engine, engine.step() in a loop"},
            "e2e": {"value": round(r["e2e_tok_s"], 1), "unit": "tokens/s"},
            "clocks": sampler.summary(), "points": r.get("points", {})}
    if "prefill" in r:
        line["prefill"] = r["prefill"]
    return line


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=XL["n_layer"], help="fewer layers than the XL shape's 48 (sizes stay)")
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--no-graph", action="store_true", help="run decode steps eagerly")
    parser.add_argument("--no-points", action="store_true", help="only the decode steps at --batch")
    parser.add_argument("--widths", default="1024,2048", help="with --only rakalix, luporax, vedadra or tesozen: the model widths to measure")
    parser.add_argument("--only", default=None, choices=("prefill", "small", "large", "products", "rakalix", "luporax", "vedadra", "tesozen"),
                        help="run one workload alone and print its numbers (for profiling): the 2,048-token prefill "
                             "step, the small shape's continuous batching, the large shape's mixed steps, or the four "
                             "products of an XL layer over row counts beside the library's matmul")
    args = parser.parse_args()

    if args.gpus != 1:
        print("bench.py measures a single-GPU engine: --gpus must be 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.steps < 1:
        args.steps = 1
    if args.impl == "reference":
        print(json.dumps(reference_line(args)))
        return 0

    import torch

    from ayaka_py_b200 import ops

    pk = peaks()
    graph = not args.no_graph
    if args.only == "rakalix":
        for width in (int(w) for w in args.widths.split(",")):
            layers = 4 if args.layers == XL["n_layer"] else args.layers
            print(json.dumps({"rakalix_beside_gpt2": run_rakalix(width, layers, args.batch, args.steps, args.warmup, pk)}), flush=True)
        return 0
    if args.only == "luporax":
        for width in (int(w) for w in args.widths.split(",")):
            layers = 4 if args.layers == XL["n_layer"] else args.layers
            print(json.dumps({"luporax_beside_rakalix": run_luporax(width, layers, args.batch, args.steps, args.warmup, pk)}), flush=True)
        return 0
    if args.only == "vedadra":
        for width in (int(w) for w in args.widths.split(",")):
            layers = 4 if args.layers == XL["n_layer"] else args.layers
            print(json.dumps({"vedadra_beside_gpt2": run_vedadra(width, layers, args.batch, args.steps, args.warmup, pk)}), flush=True)
        return 0
    if args.only == "tesozen":
        for width in (int(w) for w in args.widths.split(",")):
            layers = 4 if args.layers == XL["n_layer"] else args.layers
            print(json.dumps({"tesozen_beside_luporax": run_tesozen(width, layers, args.batch, args.steps, args.warmup, pk)}), flush=True)
        return 0
    if args.only == "products":
        for row in run_products():
            print(json.dumps(row))
        return 0
    if args.only == "small":
        print(json.dumps({"small_continuous": run_small_continuous(None if args.layers == XL["n_layer"] else args.layers)}))
        return 0
    if args.only == "large":
        print(json.dumps({"large_mixed": run_large_mixed(None if args.layers == XL["n_layer"] else args.layers,
                                                         steps=args.steps, warmup=args.warmup)}))
        return 0
    sizes = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    config, model, engine = build_engine(XL, args.layers, max_requests=max(max(sizes), 2),
                                         kv_pages=max(sizes) * (XL["n_positions"] // 16) + 1, decode_graph=graph)
    if args.only == "prefill":
        p = run_prefill(engine, config, repeats=max(1, args.steps))
        print(json.dumps({"prefill": {"value": round(p["tokens"] / (p["ms"] / 1e3), 1), "tokens": p["tokens"],
                                      "ms": round(p["ms"], 3), "n_layer": args.layers,
                                      "frac": round(p["flops"] / (p["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0
    repeats = -(-MIN_TIMED_STEPS // args.steps)
    sampler = ClockSampler()
    sampler.start()
    main_run = run_decode(engine, config, args.batch, args.steps, args.warmup, repeats=repeats)
    sampler.stop()
    clocks = sampler.summary()

    points, prefill = {}, None
    if not args.no_points:
        for b in (1, 64):
            r = main_run if b == args.batch else run_decode(engine, config, b, 32, args.warmup, seed=20 + b, repeats=2)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
        p = run_prefill(engine, config)
        prefill = {"value": round(p["tokens"] / (p["ms"] / 1e3), 1), "tokens": p["tokens"], "ms": round(p["ms"], 3),
                   "frac": round(p["flops"] / (p["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        points[f"host_ms_per_step_b{args.batch}"] = round(main_run["host_ms_per_step"], 4)
        if graph:
            # the same decode steps without CUDA graphs: every kernel launched from Python
            engine.decode_graphs = None
            eager = run_decode(engine, config, args.batch, 32, args.warmup, seed=31, repeats=2)
            points[f"decode_b{args.batch}_eager"] = round(eager["tok_s"], 1)
            points[f"host_ms_per_step_b{args.batch}_eager"] = round(eager["host_ms_per_step"], 4)
        del engine, model
        torch.cuda.empty_cache()
        small = run_small_continuous()
        points.update({"small_cb_total_tok_s": round(small["total_tok_s"], 1), "small_cb_output_tok_s": round(small["output_tok_s"], 1),
                       "small_cb_steps": small["steps"], "small_cb_preemptions": small["preemptions"],
                       "small_cb_page_high_water": small["page_high_water"], "small_cb_seconds": round(small["seconds"], 3)})
        torch.cuda.empty_cache()
        large = run_large_mixed()
        points.update({"large_mixed_ms_per_step": round(large["ms_per_step"], 4), "large_mixed_tok_s": round(large["tok_s"], 1),
                       "large_mixed_rows_per_step": round(large["rows_per_step"], 1),
                       "large_mixed_host_ms_per_step": round(large["host_ms_per_step"], 4),
                       "large_mixed_tflops": round(large["tflops"], 1), "large_mixed_gbs": round(large["gbs"], 1)})

    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tokens per second, GPT-2 XL shape", "value": round(main_run["tok_s"], 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "gpt2-xl shape, random weights", "global_batch": args.batch, "seq_len": config.n_positions,
                   "parallelism": "single GPU", "n_layer": args.layers, "n_layer_of_shape": XL["n_layer"],
                   "n_embd": config.n_embd, "n_head": config.n_head, "n_inner": config.inner_size,
                   "vocab_size": config.vocab_size, "prompt_len": PROMPT_LEN,
                   "mean_context": round(main_run["mean_context"], 1), "page_size": 16,
                   "decode_graph": graph, "timed_steps": main_run["timed_steps"],
                   "l2": "inputs larger than L2 (weights 3 GB)", "peaks": pk["source"]},
        "e2e": {"value": round(main_run["e2e_tok_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(main_run["h2d"]), "d2h_bytes_per_step": int(main_run["d2h"])},
        "gpu_launches": int(main_run["launches"]),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if prefill is not None:
        line["prefill"] = prefill
        line["points"] = points
    if ops.tc_error():
        line["error"] = f"a tensor-core kernel's wait ran out (code {ops.tc_error()})"
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())

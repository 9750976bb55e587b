#!/usr/bin/env python3
"""Benchmark of the engine's decode step (and prefill) at Qwen2-7B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests whose context ends at 4,096 tokens.
The timed region is K such steps on the device (captured graph: model step, argmax, advance of
positions; no host work), timed with CUDA events; ``value`` is decoded tokens per second.
``e2e`` is the same through ``LLMEngine.step()``: host token lists in, scheduler, pinned
host-to-device copy of the step's inputs, device-to-host read of the sampled tokens.
One line of JSON is printed; see the keys below. Weights are random (seeded), token ids
uniform random, and the cache pages of the device-timed decode runs are filled with random
values instead of being prefilled (the step's time does not depend on the values).
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Qwen2-7B layer sizes (the benchmark's named configuration, with random weights)
QWEN2_7B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28, hidden_size=3584,
    num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
    max_position_embeddings=32768,
)
# The two larger shapes that the benchmark's other workloads name (random weights as well)
SHAPES = {
    "0.5b": ("Qwen2-0.5B", dict(QWEN2_7B, num_hidden_layers=24, hidden_size=896, num_attention_heads=14,
                                 num_key_value_heads=2, head_dim=64, intermediate_size=4864, vocab_size=151936,
                                 tie_word_embeddings=True)),
    "1.5b": ("Qwen2-1.5B", dict(QWEN2_7B, num_hidden_layers=28, hidden_size=1536, num_attention_heads=12,
                                 num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=151936,
                                 tie_word_embeddings=True)),
    "7b": ("Qwen2-7B", QWEN2_7B),
    "14b": ("Qwen2.5-14B", dict(QWEN2_7B, num_hidden_layers=48, hidden_size=5120, num_attention_heads=40,
                                num_key_value_heads=8, intermediate_size=13824, rms_norm_eps=1e-5)),
    "32b": ("Qwen2.5-32B", dict(QWEN2_7B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=40,
                                num_key_value_heads=8, intermediate_size=27648, rms_norm_eps=1e-5)),
}
CONTEXT = 4096
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            flat = {}

            def walk(obj):
                if isinstance(obj, dict):
                    for key, value in obj.items():
                        if isinstance(value, (int, float)) and key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                            flat.setdefault(key, float(value))
                        else:
                            walk(value)
                elif isinstance(obj, list):
                    for item in obj:
                        walk(item)

            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                flat["source"] = "measured"
                return flat
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self.process = None
        self.thread = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return

        def reader():
            for line in self.process.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) == 6:
                    self.samples.append(parts)

        self.thread = threading.Thread(target=reader, daemon=True)
        self.thread.start()

    def mark(self) -> int:
        return len(self.samples)

    def stop(self) -> None:
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self, begin: int = 0, end: int | None = None) -> dict:
        rows = self.samples[begin:end] or self.samples
        clocks = [int(r[0]) for r in rows if r[0].isdigit()]
        maxima = [int(r[1]) for r in rows if r[1].isdigit()]
        reasons = [name for i, name in enumerate(self.NAMES) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {
            "sm_mhz": int(statistics.median(clocks)) if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "reasons": reasons,
            "samples": len(rows),
        }


def build_runner(layers: int, max_seqs: int, context: int, seed: int = 0, shape: str = "7b", pages: int | None = None,
                 dtype=None):
    import torch

    from turboserve_b200.config import config_from_dict, lookup
    from turboserve_b200.engine.runner import ModelRunner, make_groups

    raw = dict(SHAPES[shape][1], num_hidden_layers=layers)
    config = config_from_dict(raw)
    model = lookup(config.architecture).build_model(config, dtype or torch.bfloat16, "cuda")
    model.config = config
    model.init_random(seed)
    if pages is None:
        pages = max_seqs * (context // PAGE) + 64
    runner = ModelRunner(model, make_groups(model.cache_plan(), PAGE, pages), max_seqs)
    for cache in runner.storage.run_caches:
        cache.k_pages.normal_()
        cache.v_pages.normal_()
    return config, model, runner


def weight_bytes(model) -> int:
    """Bytes a decode step has to read of the weights: everything but the embedding table."""
    total = 0
    for p in model.named_params():
        if model.parts_list[p.owner] is model.embedding and not model.spec.tie_word_embeddings:
            continue  # a decode step reads a few rows of the table
        count = 1
        for s in p.spec.shape:
            count *= s
        total += count * (2 if p.spec.role == "matrix" else 4)
    return total


def decode_on_device(runner, batch: int, context_end: int, steps: int, warmup: int):
    """K decode steps replayed from one graph; returns (seconds, own kernel launches per step, mean context)."""
    import torch

    from turboserve_b200.engine.batch import RequestSlice, StaticBatch
    from turboserve_b200.ops import kernels

    width = context_end // PAGE
    start = context_end - (steps + warmup) - 2
    static = StaticBatch(batch, batch, [width], runner.device)
    generator = torch.Generator().manual_seed(1)
    ids = torch.randint(0, runner.model.vocab_size, (batch,), generator=generator).tolist()
    slices = [RequestSlice([ids[i]], start, [list(range(i * width, (i + 1) * width))], i, [0]) for i in range(batch)]
    static.load_decode(slices)
    tokens = torch.empty(batch, dtype=torch.int32, device=runner.device)

    def one_step():
        logits = runner.run(static.batch)
        kernels.argmax(logits, tokens, batch)
        static.batch.token_ids.copy_(tokens)
        static.batch.positions.add_(1)
        static.batch.context_lens.add_(1)

    with torch.inference_mode():
        one_step()
        torch.cuda.synchronize()
        before = kernels.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one_step()
        launches = kernels.launch_count() - before
        for _ in range(warmup):
            graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
    runner.check_status()
    mean_context = start + 2 + warmup + steps / 2
    return begin.elapsed_time(end) / 1000.0, launches, mean_context


def decode_end_to_end(runner, config, batch: int, context_end: int, steps: int, warmup: int):
    """The same decode steps through LLMEngine.step(): host tokens in, host tokens out."""
    import torch

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    # requests finish their prompts some steps apart (a prompt takes several steps under the token
    # budget, one request after the other); leave room so that none reaches the end of its
    # context, and none finishes, inside the timed region
    budget = 2048
    room = batch * -(-context_end // budget) + 8
    prompt_len = context_end - (steps + warmup) - 2 - room
    engine_config = EngineConfig(
        model="(injected)", dtype="bfloat16", max_model_len=context_end,
        scheduler=SchedulerConfig(max_num_seqs=batch, max_num_batched_tokens=budget, block_size=PAGE,
                                  num_blocks=runner.groups[0].num_pages))
    engine = LLMEngine(engine_config, runner=runner)
    generator = torch.Generator().manual_seed(2)
    sampling = SamplingParams(max_tokens=steps + warmup + room, temperature=0.0, ignore_eos=True)
    for i in range(batch):
        prompt = torch.randint(0, config.vocab_size, (prompt_len,), generator=generator).tolist()
        engine.add_request(f"bench-{i}", prompt, sampling)
    while any(seq.num_output_tokens == 0 for seq in engine.scheduler._running) or engine.scheduler.num_waiting:
        engine.step()  # prefill, untimed
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d = runner._graphs[(next(b for b in runner._graph_buckets if b >= batch), 1)][1].nbytes if runner._graph_buckets else 0
    started = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += sum(len(o.new_token_ids) for o in engine.step())
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    if produced != batch * steps:
        raise RuntimeError(f"the end-to-end run decoded {produced} tokens in {steps} steps of {batch} requests")
    decode_end_to_end.overlapped = engine.stats()["num_overlapped_steps"]
    engine.close()
    return elapsed, produced, h2d, 4 * runner.token_buffer.numel()


def prefill_end_to_end(runner, config, tokens: int, repeats: int = 5):
    """A prompt of ``tokens`` tokens through ``LLMEngine.step()`` to its first token: host token ids in
    (scheduler, packing, pinned host-to-device copy), one step, the sampled id read back. Median and best, seconds."""
    import torch

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    engine_config = EngineConfig(
        model="(injected)", dtype="bfloat16", max_model_len=tokens + PAGE,
        scheduler=SchedulerConfig(max_num_seqs=1, max_num_batched_tokens=tokens, block_size=PAGE,
                                  num_blocks=runner.groups[0].num_pages))
    engine = LLMEngine(engine_config, runner=runner)
    generator = torch.Generator().manual_seed(5)
    sampling = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    times = []
    for i in range(repeats + 2):
        prompt = torch.randint(0, config.vocab_size, (tokens,), generator=generator).tolist()
        torch.cuda.synchronize()
        started = time.perf_counter()
        engine.add_request(f"prefill-{i}", prompt, sampling)
        outputs = engine.step()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - started
        if len(outputs) != 1 or not outputs[0].finished:
            raise RuntimeError("the prompt did not run in one step")
        if i >= 2:
            times.append(elapsed)
    engine.close()
    return statistics.median(times), min(times)


def prefill_run(runner, config, tokens: int, repeats: int = 7, warmup: int = 3):
    import torch

    from turboserve_b200.engine.batch import RequestSlice

    generator = torch.Generator().manual_seed(3)
    ids = torch.randint(0, config.vocab_size, (tokens,), generator=generator).tolist()
    table = list(range(-(-tokens // PAGE)))
    batch = runner.build_batch([RequestSlice(ids, 0, [table], 0, [tokens - 1])])
    times = []
    for i in range(warmup + repeats):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.run(batch)
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(begin.elapsed_time(end) / 1000.0)
    runner.check_status()
    return statistics.median(times), min(times)


def prefill_flops(config, tokens: int) -> float:
    h, d = config.hidden_size, config.head_dim
    qkv = (config.num_attention_heads + 2 * config.num_key_value_heads) * d
    per_layer = 2 * tokens * h * (qkv + config.num_attention_heads * d + 3 * config.intermediate_size)
    attention = 2 * tokens * tokens * config.num_attention_heads * d  # QK^T and PV over the causal half
    return config.num_hidden_layers * (per_layer + attention) + 2 * h * config.vocab_size


def one_step(kind: str, layers: int, batch: int, shape: str = "7b", float32: bool = False) -> int:
    """Three eager steps (no graph) of one kind, so that a profiler sees every kernel once per step."""
    import torch

    from turboserve_b200.engine.batch import RequestSlice, StaticBatch

    config, model, runner = build_runner(layers, max(batch, 1), CONTEXT, shape=shape, dtype=torch.float32 if float32 else None)
    width = CONTEXT // PAGE
    if kind == "decode":
        static = StaticBatch(batch, batch, [width], runner.device)
        static.load_decode([RequestSlice([5], CONTEXT - 1, [list(range(i * width, (i + 1) * width))], i, [0])
                            for i in range(batch)])
        batch_obj = static.batch
    else:
        ids = torch.randint(0, config.vocab_size, (2048,), generator=torch.Generator().manual_seed(3)).tolist()
        batch_obj = runner.build_batch([RequestSlice(ids, 0, [list(range(width))], 0, [2047])])
    for _ in range(3):
        runner.run(batch_obj)
    torch.cuda.synchronize()
    runner.check_status()
    print(f"ran three {kind} steps of {layers} layers")
    return 0


def scenario(name: str, shape: str, layers: int, generate: int) -> int:
    """A serving workload through ``LLMEngine``: prompts in, tokens out, the scheduler in between.

    ``mixed``: 32 prompts of 64 to 4,096 tokens (uniform), a token budget of 512 a step (prompts are
    cut into portions beside the decode tokens of the others), contexts up to 8,192, room for all.
    ``preempt``: 16 requests whose contexts end at 16,384 tokens, in a pool that holds their prompts
    and half of what they generate, so that some are preempted and computed again.
    Both generate ``generate`` tokens a request, greedily; one line of JSON with the throughput
    (prompt and generated tokens together) and what the scheduler did.
    """
    import random

    import torch

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    rng = random.Random(4)
    if name == "mixed":
        batch, context, budget = 32, 8192, 512
        lengths = [rng.randint(64, 4096) for _ in range(batch)]
        pages = sum(-(-(n + generate) // PAGE) for n in lengths) + 64
    else:
        batch, context, budget = 16, 16384, 2048
        lengths = [context - generate] * batch
        pages = batch * -(-(context - generate) // PAGE) + batch * (generate // 2) // PAGE
    config, model, runner = build_runner(layers, batch, context, shape=shape, pages=pages)
    engine_config = EngineConfig(
        model="(injected)", dtype="bfloat16", max_model_len=context,
        scheduler=SchedulerConfig(max_num_seqs=batch, max_num_batched_tokens=budget, block_size=PAGE, num_blocks=pages))
    engine = LLMEngine(engine_config, runner=runner)
    sampling = SamplingParams(max_tokens=generate, temperature=0.0, ignore_eos=True)
    prompts = [[rng.randrange(config.vocab_size) for _ in range(n)] for n in lengths]
    engine.generate([p[:64] for p in prompts[:2]], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))  # warm-up
    before = engine.stats()
    torch.cuda.synchronize()
    started = time.perf_counter()
    outputs = engine.generate(prompts, sampling)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    after = engine.stats()
    generated = sum(len(o.token_ids) for o in outputs)
    if generated != batch * generate:
        raise RuntimeError(f"{generated} tokens came back, {batch * generate} were asked for")
    engine.scheduler.check_invariants()
    line = {
        "scenario": name, "metric": "prompt + generated tokens/s through LLMEngine.generate",
        "value": round((sum(lengths) + generated) / elapsed, 1), "unit": "tokens/s", "seconds": round(elapsed, 3),
        "prompt_tokens": sum(lengths), "generated_tokens": generated,
        "generated_tokens_per_s": round(generated / elapsed, 1),
        "steps": after["num_steps"] - before["num_steps"],
        "preemptions": after["num_preemptions"] - before["num_preemptions"],
        "recomputed_prompt_tokens": after["num_prefill_tokens"] - before["num_prefill_tokens"] - sum(lengths),
        "config": {"model": f"{SHAPES[shape][0]} shape (random weights)", "layers": layers,
                   "layers_of_model": SHAPES[shape][1]["num_hidden_layers"], "hidden": config.hidden_size,
                   "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                   "intermediate": config.intermediate_size, "requests": batch, "max_context": context,
                   "token_budget": budget, "pages": pages, "page_size": PAGE, "params": model.num_parameters()},
        "dtype": "bf16", "impl": "ours",
    }
    engine.close()
    print(json.dumps(line))
    return 0


def reference_arm(args, shape_name: str, shape_raw: dict) -> int:
    """The same workload through the unmodified reference engine under ``baseline/_ref``.

    Nothing of this repository's engine is imported on this path. Where the reference cannot be
    imported or run, one line says why and the exit code is still 0.
    """
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm as arm

    try:
        line = arm.run(shape_raw, shape_name, args.layers, args.batch, args.context, PAGE, args.steps, args.warmup,
                       args.skip_points, ClockSampler(), load_peaks(), prefill_flops)
    except arm.UnavailableError as error:
        print(json.dumps({"impl": "reference", "unavailable": str(error)}))
        return 0
    except Exception as error:  # noqa: BLE001 - the reference's own failure is the reason, in its words
        reason = " ".join(f"the reference failed while running: {type(error).__name__}: {error}".split())
        print(json.dumps({"impl": "reference", "unavailable": reason[:500]}))
        return 0
    print(json.dumps(line))
    return 0


def fp32_products(layers: int = 28, steps: int = 8) -> int:
    """The true 32-bit path (FFMA, no tensor cores): its matrix product at the 7B layer's shapes, every
    weight from HBM (copies of a weight taken in turn, 600 MB of them), and one decode step of the
    whole model in float32 at batch 8, context 4,096. One JSON line."""
    import torch

    from turboserve_b200.engine.batch import RequestSlice, StaticBatch
    from turboserve_b200.ops.linear import linear

    shapes = {"qkv": (3584, 4608), "o": (3584, 3584), "gate_up": (3584, 37888), "down": (18944, 3584)}
    line = {"what": "float32 FFMA product (gemm_simt.cu), Qwen2-7B layer shapes", "unit": "TFLOP/s (rows 2048) and GB/s of weights (rows 8)"}
    for name, (k, n) in shapes.items():
        copies = max(2, -(-600_000_000 // (4 * k * n)))
        ws = [torch.randn(n, k, device="cuda") for _ in range(copies)]
        for rows in (2048, 8):
            x = torch.randn(rows, k, device="cuda")
            out = torch.empty(rows, n, device="cuda")
            for w in ws[:2]:
                linear(x, w, out)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for w in ws:
                linear(x, w, out)
            end.record()
            torch.cuda.synchronize()
            seconds = begin.elapsed_time(end) / 1e3 / copies
            line[f"{name}_rows{rows}_ms"] = round(seconds * 1e3, 3)
            line[f"{name}_rows{rows}"] = round(2 * rows * k * n / seconds / 1e12, 2) if rows > 8 else round(4 * k * n / seconds / 1e9, 1)
        del ws
    # one decode step of the whole model in float32, launched kernel by kernel (20 ms of device work hide the host)
    batch, context = 8, CONTEXT
    config, model, runner = build_runner(layers, batch, context, dtype=torch.float32)
    width = context // PAGE
    static = StaticBatch(batch, batch, [width], runner.device)
    slices = [RequestSlice([7 + i], context - steps - 4, [list(range(i * width, (i + 1) * width))], i, [0]) for i in range(batch)]
    static.load_decode(slices)
    times = []
    for step in range(steps + 2):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.run(static.batch)
        end.record()
        torch.cuda.synchronize()
        static.batch.positions.add_(1)
        static.batch.context_lens.add_(1)
        if step >= 2:
            times.append(begin.elapsed_time(end))
    runner.check_status()
    ms = statistics.median(times)
    weights = sum(4 * _count(p.spec.shape) for p in model.named_params() if model.parts_list[p.owner] is not model.embedding)
    cache = batch * (context - 4) * layers * 2 * config.num_key_value_heads * config.head_dim * 4
    line["decode_step"] = {"layers": layers, "layers_of_model": SHAPES["7b"][1]["num_hidden_layers"], "batch": batch, "context": context,
                           "ms": round(ms, 2), "gb_per_s": round((weights + cache) / ms / 1e6, 1),
                           "frac_of_hbm": round((weights + cache) / ms / 1e6 / load_peaks()["hbm_gbs"], 3)}
    print(json.dumps(line))
    return 0


def _count(shape) -> int:
    total = 1
    for s in shape:
        total *= s
    return total


def decode_attention_sweep() -> int:
    """The TMA-fed decode attention kernel alone at a few (requests, keys, parts): µs and TB/s of keys and
    values, CUDA events around a graph of "write 256 MB, run the kernel" with the write alone subtracted."""
    import torch

    from turboserve_b200.ops import attention_bf16 as fa

    nh, nkv, d, page = 28, 4, 128, PAGE
    flush = torch.empty(256 * 1024 * 1024 // 4, device="cuda")
    rows = []

    def timed(graph) -> float:
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(20):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / 20 * 1e3

    empty = torch.cuda.CUDAGraph()
    flush.zero_()
    torch.cuda.synchronize()
    with torch.cuda.graph(empty):
        flush.zero_()
    base = timed(empty)
    for batch, ctx, parts in [(8, 4096, 8), (8, 4096, 9), (64, 512, 1), (32, 1024, 1), (32, 1024, 2), (8, 16384, 8),
                              (64, 4096, 1), (1, 4096, 8), (1, 4096, 32)]:
        width = ctx // page + 1
        k_pages = torch.randn(batch * width, page, nkv, d, device="cuda").to(torch.bfloat16)
        v_pages = torch.randn(batch * width, page, nkv, d, device="cuda").to(torch.bfloat16)
        table = torch.arange(batch * width, dtype=torch.int32, device="cuda").view(batch, width)
        q = torch.randn(batch, nh * d, device="cuda").to(torch.bfloat16)
        out = torch.empty_like(q)
        seq = torch.arange(batch, dtype=torch.int32, device="cuda")
        pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device="cuda")
        scratch = torch.empty(max(4, fa.decode_scratch_floats(batch, nh, parts, d)), device="cuda")

        def run():
            fa.flash_decode_tma(q, out, k_pages, v_pages, table, seq, pos, batch, nh, nkv, d, None, d ** -0.5, parts, scratch)

        run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            flush.zero_()
            run()
        us = timed(graph) - base
        rows.append({"requests": batch, "keys": ctx, "parts": parts, "us": round(us, 1),
                     "tb_per_s": round(batch * ctx * nkv * d * 4 / us / 1e6, 2)})
        del k_pages, v_pages
    print(json.dumps({"what": "flash_decode_tma alone, 28 heads on 4 kv heads of 128, pages of 16", "rows": rows}))
    return 0


def sampling_sweep(context: int = 4096, steps: int = 40) -> int:
    """Decode steps of 8 requests through LLMEngine.step() under a few sets of sampling options: ms a step each."""
    import torch

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    config, model, runner = build_runner(SHAPES["7b"][1]["num_hidden_layers"], 8, context)
    runner.enable_graphs(8, context, 2048)
    line = {"what": "ms a decode step through LLMEngine.step(), 7B sizes, batch 8", "context": context, "steps": steps}
    for name, options in [("greedy", dict(temperature=0.0)), ("temperature", dict(temperature=0.8, seed=1)),
                          ("top_p", dict(temperature=0.8, top_p=0.9, seed=1)),
                          ("top_k_top_p", dict(temperature=0.8, top_p=0.9, top_k=50, seed=1)),
                          ("penalty", dict(temperature=0.8, top_p=0.9, top_k=50, seed=1, repetition_penalty=1.2)),
                          ("greedy_penalty", dict(temperature=0.0, repetition_penalty=1.2)),
                          ("greedy_logprobs", dict(temperature=0.0, logprobs=True)),
                          ("top_p_penalty_logprobs", dict(temperature=0.8, top_p=0.9, seed=1, repetition_penalty=1.2, logprobs=True)),
                          ("greedy_again", dict(temperature=0.0))]:
        engine = LLMEngine(EngineConfig(model="(injected)", dtype="bfloat16", max_model_len=context, scheduler=SchedulerConfig(
            max_num_seqs=8, max_num_batched_tokens=2048, block_size=PAGE, num_blocks=runner.groups[0].num_pages)), runner=runner)
        generator = torch.Generator().manual_seed(2)
        sampling = SamplingParams(max_tokens=steps + 40, ignore_eos=True, **options)
        for i in range(8):
            engine.add_request(f"r{i}", torch.randint(0, config.vocab_size, (context - steps - 100,), generator=generator).tolist(), sampling)
        while any(seq.num_output_tokens == 0 for seq in engine.scheduler._running) or engine.scheduler.num_waiting:
            engine.step()
        for _ in range(5):
            engine.step()
        torch.cuda.synchronize()
        started = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += sum(len(o.new_token_ids) for o in engine.step())
        torch.cuda.synchronize()
        line[name] = round((time.perf_counter() - started) / steps * 1e3, 3)
        if produced != 8 * steps:
            raise RuntimeError(f"{name}: {produced} tokens in {steps} steps")
        engine.close()
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="7b",
                        help="layer sizes (the headline is 7b; the others are for the larger workloads)")
    parser.add_argument("--layers", type=int, default=None,
                        help="run fewer layers than the model has (both numbers are reported)")
    parser.add_argument("--scenario", choices=["mixed", "preempt"], default=None,
                        help="run a serving workload through LLMEngine.generate instead (see scenario())")
    parser.add_argument("--generate", type=int, default=128, help="tokens a request generates in a scenario")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=CONTEXT,
                        help="context length of the decode runs (the headline is 4096; others are for sweeps)")
    parser.add_argument("--skip-points", action="store_true", help="skip the batch-1 and batch-64 points and the prefill")
    parser.add_argument("--decode-attention-sweep", action="store_true", help="time the decode attention kernel alone at a few sizes and exit")
    parser.add_argument("--sampling-sweep", action="store_true", help="time decode steps through LLMEngine under a few sets of sampling options and exit")
    parser.add_argument("--fp32-products", action="store_true", help="time the float32 path's matrix product at the 7B shapes and exit")
    parser.add_argument("--float32", action="store_true", help="with --one-step: the true 32-bit path")
    parser.add_argument("--one-step", choices=["decode", "prefill"], default=None,
                        help="run three eager steps of that kind and exit (a small case for a profiler)")
    args = parser.parse_args()

    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine runs on a single B200, --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    shape_name, shape_raw = SHAPES[args.shape]
    if args.layers is None:
        args.layers = shape_raw["num_hidden_layers"]
    if args.impl == "reference":
        return reference_arm(args, shape_name, shape_raw)

    import torch

    from turboserve_b200.ops import kernels

    if args.fp32_products:
        return fp32_products()
    if args.decode_attention_sweep:
        return decode_attention_sweep()
    if args.sampling_sweep:
        return sampling_sweep()
    if args.one_step:
        return one_step(args.one_step, args.layers, args.batch, args.shape, args.float32)
    if args.scenario:
        return scenario(args.scenario, args.shape, args.layers, args.generate)
    peaks = load_peaks()
    of = "of measured" if peaks["source"] == "measured" else "of fallback"
    context = args.context
    if context < 256 or context % PAGE:
        print(f"--context must be a multiple of {PAGE} and at least 256")
        return 2
    largest = 64 if not args.skip_points else max(args.batch, 1)
    config, model, runner = build_runner(args.layers, largest, context, shape=args.shape)
    runner.enable_graphs(largest, context, 2048)
    kv_per_token = config.kv_bytes_per_token(2)
    w_bytes = weight_bytes(model)

    sampler = ClockSampler()
    sampler.start()
    time.sleep(0.3)
    mark0 = sampler.mark()
    seconds, launches_per_step, mean_ctx = decode_on_device(runner, args.batch, context, args.steps, args.warmup)
    # the same steps through the entry point, straight after, so that both numbers see the same GPU state
    e2e_seconds, produced, h2d, d2h = decode_end_to_end(runner, config, args.batch, context, args.steps, args.warmup)
    mark1 = sampler.mark()
    value = args.batch * args.steps / seconds
    step_bytes = w_bytes + args.batch * mean_ctx * kv_per_token
    achieved = step_bytes / (seconds / args.steps) / 1e9

    points = {}
    prefill = None
    if not args.skip_points:
        for b in (1, 64):
            s, _, _ = decode_on_device(runner, b, context, args.steps, args.warmup)
            points[f"decode_b{b}"] = round(b * args.steps / s, 1)
            s, n, _, _ = decode_end_to_end(runner, config, b, context, args.steps, args.warmup)
            points[f"e2e_decode_b{b}"] = round(n / s, 1)
        t, best = prefill_run(runner, config, 2048)
        flops = prefill_flops(config, 2048)
        # value, ms and frac are the median of the repeats; best_ms is the fastest of them
        prefill = {"value": round(2048 / t, 1), "tokens": 2048, "ms": round(t * 1e3, 3), "best_ms": round(best * 1e3, 3),
                   "frac": round(flops / t / (peaks["bf16_tflops"] * 1e12), 4), "peak": of}
        if "bf16_tflops_sustained" in peaks:  # the step is long enough to run under the power cap
            prefill["frac_of_sustained"] = round(flops / t / (peaks["bf16_tflops_sustained"] * 1e12), 4)
        e2e_t, e2e_best = prefill_end_to_end(runner, config, 2048)
        prefill["e2e_value"] = round(2048 / e2e_t, 1)
        prefill["e2e_ms"] = round(e2e_t * 1e3, 3)
        prefill["e2e_best_ms"] = round(e2e_best * 1e3, 3)
    # what a batch pays that is the first of its size to be lopsided (decode attention cut finer:
    # another graph): a warm-up step, a synchronisation and the capture. Even batches of every
    # size were captured when the engine was built.
    torch.cuda.synchronize()
    started = time.perf_counter()
    runner._capture(next(b for b in runner._graph_buckets if b >= args.batch), 16)
    torch.cuda.synchronize()
    first_lopsided_ms = (time.perf_counter() - started) * 1e3

    sampler.stop()
    clocks = sampler.summary(mark0, mark1)

    line = {
        "metric": f"decode tokens/s, {shape_name} shape, batch {args.batch}, context {context}",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(seconds / args.steps * 1e3, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random weights (seed 0), uniform random token ids, cache pages of the device-timed runs filled with random values",
        "config": {
            "model": f"{shape_name} shape (random weights)", "layers": args.layers, "layers_of_model": shape_raw["num_hidden_layers"],
            "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": config.vocab_size,
            "global_batch": args.batch, "seq_len": context, "page_size": PAGE, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (every step reads all weights)", "params": model.num_parameters(),
        },
        "e2e": {"value": round(produced / e2e_seconds, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_seconds / args.steps * 1e3, 4),
                "steps_launched_ahead": getattr(decode_end_to_end, "overlapped", 0)},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": of,
                     "bytes_per_step": int(step_bytes)},
        "points": points,
        "graphs": {"captured_at_start": runner.num_graph_captures - 1, "first_lopsided_step_extra_ms": round(first_lopsided_ms, 2)},
        "impl": "ours",
    }
    if prefill is not None:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())

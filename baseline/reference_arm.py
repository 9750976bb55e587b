"""The reference arm of ``bench.py``: the unmodified reference engine on the benchmark's workload.

Everything here drives the reference's own public entry point, ``LLMEngine`` with an injected
model and tokenizer (runtime/engine.py:124-146), built by its own ``ModelConfig.from_dict``
and ``CausalLM`` (model/model.py:111-315) with seeded normal weights, and stepped through its
own ``step()`` (runtime/engine.py:340-356). Nothing of this repository's engine, models or
kernels is imported. The reference has no device-only timing hook: the public call is the
whole step (its scheduler, its tensors built from host lists, its forward pass, its sampler,
the tokens read back), so ``value`` and ``e2e`` are the same measurement, taken with a device
synchronisation at both ends of the timed loop.
"""

from __future__ import annotations

import importlib
import json
import statistics
import sys
import time
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"


class UnavailableError(RuntimeError):
    """The reference cannot be imported or run here; the message is the one-line reason."""


def import_reference():
    if not (REF_DIR / "turboserve").is_dir():
        raise UnavailableError(
            "baseline/_ref holds no reference package: run `python baseline/install_reference.py` "
            "where the reference's checkout is mounted")
    own = str(Path(__file__).resolve().parent.parent)
    sys.path[:] = [p for p in sys.path if p not in (own, "")]  # the repository's own package stays out of reach
    sys.path.insert(0, str(REF_DIR))
    try:
        model = importlib.import_module("turboserve.engine.model")
        engine = importlib.import_module("turboserve.engine.runtime.engine")
        types = importlib.import_module("turboserve.engine.core.types")
    except Exception as error:  # noqa: BLE001 - whatever stops the import is the reason
        raise UnavailableError(f"importing the reference failed: {type(error).__name__}: {error}") from error
    loaded = Path(model.__file__).resolve()
    if REF_DIR.resolve() not in loaded.parents:
        raise UnavailableError(f"the reference resolved to {loaded}, not to baseline/_ref")
    return model, engine, types


def install_record() -> str:
    """How the reference got under baseline/_ref, as its installer wrote it down."""
    try:
        return str(json.loads((REF_DIR / "INSTALL.json").read_text())["how"])
    except (OSError, ValueError, KeyError):
        return "baseline/_ref (no install record)"


class IdTokenizer:
    """The requests are token ids already; the reference only needs something to detokenize with."""

    eos_token_id = None

    def decode(self, ids, **kwargs):
        return ""

    def encode(self, text, **kwargs):
        return [1]


def synchronize(device: str) -> None:
    if device == "cuda":
        import torch

        torch.cuda.synchronize()


def build_model(model_module, raw_config: dict, seed: int, device: str):
    import torch

    config = model_module.ModelConfig.from_dict(raw_config)
    model = model_module.CausalLM(config, dtype=torch.bfloat16, device=device)
    generator = torch.Generator(device=device).manual_seed(seed)
    with torch.no_grad():
        for parameter in model.parameters():
            parameter.normal_(0.0, 0.02, generator=generator)
    model.eval()
    return config, model


def make_engine(engine_module, types, model, batch: int, context: int, page: int, budget: int):
    config = types.EngineConfig(
        model="(injected)", dtype="bfloat16", device=model.device.type, max_model_len=context,
        scheduler=types.SchedulerConfig(
            max_num_seqs=batch, max_num_batched_tokens=budget, block_size=page,
            num_blocks=batch * (context // page) + 64, enable_prefix_caching=False))
    return engine_module.LLMEngine(config, model=model, tokenizer=IdTokenizer())


def step_copy_bytes(engine) -> tuple[int, int]:
    """Bytes one more step of this engine copies up and down, read from the tensors its runner
    builds from host lists (runtime/worker.py:180-201) and the token ids it reads back."""
    out = engine.scheduler.schedule(now=time.perf_counter())
    batch = engine.runner.build_batch(out)
    meta = batch.meta
    up = batch.input_ids.nbytes + batch.positions.nbytes + batch.sample_indices.nbytes
    for name in ("slot_mapping", "block_tables", "context_lens", "query_start_loc"):
        up += getattr(meta, name).nbytes
    down = 8 * batch.num_sampled  # int64 ids through .tolist() (core/sampler.py:238)
    return int(up), int(down)


def decode_run(engine_module, types, model, vocab: int, batch: int, context: int, page: int, steps: int,
               warmup: int, measure_copies: bool = False):
    import torch

    device = model.device.type
    budget = 2048
    room = batch * -(-context // budget) + 8
    prompt_len = context - (steps + warmup) - 2 - room
    engine = make_engine(engine_module, types, model, batch, context, page, budget)
    generator = torch.Generator().manual_seed(2)
    sampling = types.SamplingParams(max_tokens=steps + warmup + room, temperature=0.0, ignore_eos=True)
    sequences = []
    for i in range(batch):
        prompt = torch.randint(0, vocab, (prompt_len,), generator=generator).tolist()
        sequences.append(engine.add_request(f"bench-{i}", prompt, sampling))
    guard = 0
    while any(seq.num_output_tokens == 0 for seq in sequences):
        engine.step()  # prompts, untimed
        guard += 1
        if guard > 4 * batch * -(-context // budget) + 16:
            raise RuntimeError("the reference did not finish the prompts")
    for _ in range(warmup):
        engine.step()
    synchronize(device)
    started = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += sum(len(o.new_token_ids) for o in engine.step())
    synchronize(device)
    elapsed = time.perf_counter() - started
    if produced != batch * steps:
        raise RuntimeError(f"the reference decoded {produced} tokens in {steps} steps of {batch} requests")
    copies = step_copy_bytes(engine) if measure_copies else (0, 0)
    engine.close()
    return elapsed, produced, copies


def prefill_run(engine_module, types, model, vocab: int, tokens: int, page: int, repeats: int = 3):
    """One prompt of ``tokens`` tokens in one step to its first token, as the reference's step() runs it."""
    import torch

    device = model.device.type
    engine = make_engine(engine_module, types, model, 1, tokens + 2 * page, page, tokens)
    generator = torch.Generator().manual_seed(3)
    sampling = types.SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    times = []
    for i in range(repeats + 1):
        prompt = torch.randint(0, vocab, (tokens,), generator=generator).tolist()
        engine.add_request(f"prefill-{i}", prompt, sampling)
        synchronize(device)
        started = time.perf_counter()
        outputs = engine.step()
        synchronize(device)
        elapsed = time.perf_counter() - started
        if len(outputs) != 1 or not outputs[0].finished:
            raise RuntimeError("the reference did not run the prompt in one step")
        if i:  # the first is the warm-up
            times.append(elapsed)
    engine.close()
    return statistics.median(times), min(times)


def run(raw_config: dict, shape_name: str, layers: int, batch: int, context: int, page: int, steps: int, warmup: int,
        skip_points: bool, clock_sampler, peaks: dict, prefill_flops, device: str = "cuda",
        prefill_tokens: int = 2048) -> dict:
    import torch

    model_module, engine_module, types = import_reference()
    if device == "cuda" and not torch.cuda.is_available():
        raise UnavailableError("no CUDA device")
    raw = dict(raw_config, num_hidden_layers=layers)
    config, model = build_model(model_module, raw, seed=0, device=device)
    params = sum(p.numel() for p in model.parameters())

    clock_sampler.start()
    time.sleep(0.3)
    mark0 = clock_sampler.mark()
    seconds, produced, (h2d, d2h) = decode_run(engine_module, types, model, config.vocab_size, batch, context, page,
                                               steps, warmup, measure_copies=True)
    mark1 = clock_sampler.mark()
    points = {}
    prefill = None
    if not skip_points:
        for b in (1, 64):
            s, n, _ = decode_run(engine_module, types, model, config.vocab_size, b, context, page, steps, warmup)
            points[f"decode_b{b}"] = round(n / s, 1)
        median, best = prefill_run(engine_module, types, model, config.vocab_size, prefill_tokens, page)
        flops = prefill_flops(config, prefill_tokens)
        prefill = {"value": round(prefill_tokens / median, 1), "tokens": prefill_tokens, "ms": round(median * 1e3, 3),
                   "best_ms": round(best * 1e3, 3),
                   "frac": round(flops / median / (peaks["bf16_tflops"] * 1e12), 4)}
    clock_sampler.stop()

    kv_per_token = 2 * layers * config.num_key_value_heads * config.head_dim * 2
    embedding = config.vocab_size * config.hidden_size
    step_bytes = (params - embedding) * 2 + batch * (context - steps / 2 - 2) * kv_per_token
    achieved = step_bytes / (seconds / steps) / 1e9
    of = "of measured" if peaks["source"] == "measured" else "of fallback"
    value = round(produced / seconds, 1)
    line = {
        "metric": f"decode tokens/s, {shape_name} shape, batch {batch}, context {context}",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(seconds / steps * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights (seed 0), uniform random token ids; prompts computed by the engine itself; "
                "prefix caching off (random prompts share nothing)",
        "config": {
            "model": f"{shape_name} shape (random weights)", "layers": layers, "layers_of_model": raw_config["num_hidden_layers"],
            "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": config.vocab_size,
            "global_batch": batch, "seq_len": context, "page_size": page, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (every step reads all weights)", "params": params,
        },
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(seconds / steps * 1e3, 4),
                "note": "the reference's public step() is the only timed call: value and e2e are one measurement"},
        "gpu_launches": 0,
        "clocks": clock_sampler.summary(mark0, mark1),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": of, "bytes_per_step": int(step_bytes)},
        "points": points,
        "impl": "reference",
        "reference_from": install_record(),
    }
    if prefill is not None:
        line["prefill"] = prefill
    return line

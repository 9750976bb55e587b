"""Command line, in the reference's manner.

``turboserve-b200 engine generate`` and ``engine kv-size`` take the reference's option names
with their meanings (``src/turboserve/engine/runtime/engine.py:522-606``; root app and
``version`` / ``hwinfo`` from ``src/turboserve/cli.py:43-95``). Options of subsystems this
engine does not have (``--prefix-caching``, ``--offline``, ``--device cpu``) are absent.
Added: prompts as token ids (``--prompt-ids``), ``--top-k``, ``--repetition-penalty`` and
``--logprobs`` (fields of the reference's ``SamplingParams`` that its command line does not
reach), ``engine random-weights`` (writes a model
folder from a configuration and a seed) and ``engine replay`` (the trace-replay program).
"""

from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Annotated, Optional

import typer

from . import __version__

app = typer.Typer(name="turboserve-b200", help="Single-GPU inference engine for NVIDIA B200.", no_args_is_help=True)
engine_app = typer.Typer(name="engine", help="Run the engine directly.", no_args_is_help=True)
app.add_typer(engine_app, name="engine")


@app.command("version")
def version_command() -> None:
    """Print the package version."""
    typer.echo(__version__)


@app.command("hwinfo")
def hwinfo_command(indent: Annotated[int, typer.Option("--indent")] = 2) -> None:
    """Print what the engine sees of the machine: GPU, driver, CUDA, torch."""
    import platform

    import torch

    info = {"python": platform.python_version(), "torch": torch.__version__, "cuda_available": torch.cuda.is_available()}
    if torch.cuda.is_available():
        props = torch.cuda.get_device_properties(0)
        info.update(gpu=props.name, compute_capability=f"{props.major}.{props.minor}", sms=props.multi_processor_count,
                    memory_bytes=props.total_memory, cuda=torch.version.cuda)
    typer.echo(json.dumps(info, indent=indent))


def _parse_ids(text: str) -> list[int]:
    return [int(part) for part in text.replace(",", " ").split()]


@engine_app.command("generate")
def generate_command(
    prompt: Annotated[Optional[list[str]], typer.Argument(help="Text prompts (need a tokenizer in the model folder).")] = None,
    model: Annotated[str, typer.Option("--model", "-m", help="Model folder.")] = "",
    prompt_ids: Annotated[Optional[list[str]], typer.Option("--prompt-ids", help="A prompt as token ids, e.g. '5,17,3'; repeatable.")] = None,
    max_tokens: Annotated[int, typer.Option("--max-tokens", min=1)] = 64,
    temperature: Annotated[float, typer.Option("--temperature", min=0.0)] = 0.0,
    top_p: Annotated[float, typer.Option("--top-p", min=0.0, max=1.0)] = 1.0,
    top_k: Annotated[int, typer.Option("--top-k", min=0)] = 0,
    repetition_penalty: Annotated[float, typer.Option("--repetition-penalty", min=0.01, help="Above 1 makes tokens the request already holds less likely.")] = 1.0,
    logprobs: Annotated[bool, typer.Option("--logprobs/--no-logprobs", help="Print the log-probability of every generated token.")] = False,
    seed: Annotated[Optional[int], typer.Option("--seed", help="Seed for stochastic sampling.")] = None,
    dtype: Annotated[str, typer.Option("--dtype", help="auto, bfloat16 or float32.")] = "auto",
    num_blocks: Annotated[Optional[int], typer.Option("--num-blocks", min=1, help="Skip memory profiling.")] = None,
    max_num_seqs: Annotated[int, typer.Option("--max-num-seqs", min=1)] = 8,
    max_num_batched_tokens: Annotated[int, typer.Option("--max-num-batched-tokens", min=1)] = 2048,
    block_size: Annotated[int, typer.Option("--block-size", min=1)] = 16,
    ignore_eos: Annotated[bool, typer.Option("--ignore-eos/--no-ignore-eos")] = False,
    show_stats: Annotated[bool, typer.Option("--stats/--no-stats")] = False,
) -> None:
    """Complete one or more prompts and print the results."""
    from .config import EngineConfig, SamplingParams, SchedulerConfig
    from .engine.llm_engine import LLMEngine

    if not model:
        raise typer.BadParameter("--model is required")
    prompts: list = [_parse_ids(p) for p in (prompt_ids or [])]
    tokenizer = None
    if prompt:
        tokenizer = _load_tokenizer(model)
        prompts += list(prompt)
    if not prompts:
        raise typer.BadParameter("give a text prompt or --prompt-ids")
    config = EngineConfig(
        model=model, dtype=dtype, seed=seed,
        scheduler=SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
                                  block_size=block_size, num_blocks=num_blocks),
    )
    sampling = SamplingParams(max_tokens=max_tokens, temperature=temperature, top_p=top_p, top_k=top_k, seed=seed,
                              ignore_eos=ignore_eos, repetition_penalty=repetition_penalty, logprobs=logprobs)
    with LLMEngine(config, tokenizer=tokenizer) as engine:
        started = time.perf_counter()
        outputs = engine.generate(prompts, sampling)
        elapsed = time.perf_counter() - started
        for index, output in enumerate(outputs):
            typer.echo(f"prompt {index}: {prompts[index]}")
            typer.echo(f"output {index}: {output.text_delta or output.token_ids}")
            typer.echo(f"  {output.output_tokens} tokens, finish_reason={output.finish_reason}")
            if logprobs and output.logprobs is not None:
                typer.echo("  logprobs: " + " ".join(f"{value:.4f}" for value in output.logprobs))
        typer.echo(f"{len(outputs)} completions in {elapsed:.2f}s")
        if show_stats:
            typer.echo(json.dumps(engine.stats(), indent=2, default=str))


def _load_tokenizer(model: str):
    try:
        from transformers import AutoTokenizer

        return AutoTokenizer.from_pretrained(model, local_files_only=True)
    except Exception as exc:  # noqa: BLE001
        raise typer.BadParameter(f"text prompts need a tokenizer in {model}: {exc}") from exc


@engine_app.command("kv-size")
def kv_size_command(
    model: Annotated[str, typer.Option("--model", "-m", help="Model folder (only config.json is read).")] = "",
    dtype: Annotated[str, typer.Option("--dtype", help="auto, bfloat16 or float32.")] = "auto",
    block_size: Annotated[int, typer.Option("--block-size", min=1)] = 16,
    max_num_seqs: Annotated[int, typer.Option("--max-num-seqs", min=1)] = 64,
    max_num_batched_tokens: Annotated[int, typer.Option("--max-num-batched-tokens", min=1)] = 2048,
    gpu_memory_utilization: Annotated[float, typer.Option("--gpu-memory-utilization", min=0.01, max=1.0)] = 0.9,
    max_model_len: Annotated[Optional[int], typer.Option("--max-model-len", min=1)] = None,
    total_memory_gib: Annotated[Optional[float], typer.Option("--total-memory-gib", help="Plan for this much device memory instead of probing a GPU.")] = None,
) -> None:
    """Report how many cache pages this configuration would get, and why."""
    import torch

    from .config import SchedulerConfig, config_from_dir, lookup, resolve_dtype
    from .engine.memory import size_kv_cache

    config = config_from_dir(model)
    torch_dtype = resolve_dtype(dtype)
    built = lookup(config.architecture).build_model(config, torch_dtype, "cpu")
    itemsize = torch.empty((), dtype=torch_dtype).element_size()
    memory_info = None
    if total_memory_gib is not None:
        total = int(total_memory_gib * (1 << 30))
        weights = built.num_parameters() * itemsize
        memory_info = (total - weights, total)
    sizing = size_kv_cache(
        built.cache_plan(), SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens, block_size=block_size),
        itemsize, scratch_per_token=built.scratch_bytes_per_token(itemsize), vocab=built.vocab_size,
        gpu_memory_utilization=gpu_memory_utilization, max_model_len=max_model_len, memory_info=memory_info,
    )
    typer.echo(json.dumps(sizing.to_dict(), indent=2))


@engine_app.command("random-weights")
def random_weights_command(
    config: Annotated[Path, typer.Option("--config", help="A config.json (or a folder holding one).")],
    out: Annotated[Path, typer.Option("--out", help="Folder to write config.json and model.safetensors to.")],
    seed: Annotated[int, typer.Option("--seed")] = 0,
    dtype: Annotated[str, typer.Option("--dtype", help="Stored dtype: bfloat16 or float32.")] = "bfloat16",
) -> None:
    """Write a model folder with random weights from a configuration and a seed."""
    from .config import config_from_dict, read_config_json, resolve_dtype
    from .weights import write_random_model

    folder = write_random_model(config_from_dict(read_config_json(config)), seed, out, resolve_dtype(dtype))
    typer.echo(str(folder))


@engine_app.command("replay")
def replay_command(
    model: Annotated[str, typer.Option("--model", "-m")],
    out: Annotated[str, typer.Option("--out")],
    max_tokens: Annotated[int, typer.Option("--max-tokens", min=1)],
    dtype: Annotated[str, typer.Option("--dtype")] = "bfloat16",
) -> None:
    """Replay a trace from standard input (same as ``bin/trace_run``)."""
    from .replay import main

    raise typer.Exit(main(["--model", model, "--dtype", dtype, "--out", out, "--max-tokens", str(max_tokens)]))


def main() -> None:
    app()


if __name__ == "__main__":
    main()

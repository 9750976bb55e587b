"""What of bench.py's contract can be checked without a GPU."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    result = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert result.returncode == 2
    assert len(result.stdout.strip().splitlines()) == 1 and "one GPU" in result.stdout


REFERENCE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                  "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks", "roofline", "points", "impl"}


def test_the_reference_arm_prints_one_line_either_way():
    """Without a GPU the arm cannot time anything: it says so in one line and exits 0."""
    result = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert result.returncode == 0
    line = json.loads(result.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert line["unavailable"] and "\n" not in line["unavailable"]
    else:
        assert REFERENCE_KEYS <= set(line)


@pytest.mark.skipif(not (ROOT / "baseline" / "_ref" / "turboserve").is_dir(), reason="no reference under baseline/_ref")
def test_the_reference_arm_runs_the_reference_and_nothing_of_this_engine():
    """A tiny shape on the CPU through the arm's own code: the line has the contract's keys, the
    config record is flat, and the process never imported this repository's package."""
    script = (
        "import sys, json; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
        "import bench, reference_arm as arm\n"
        "raw = dict(bench.QWEN2_7B, num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,\n"
        "           head_dim=16, intermediate_size=160, vocab_size=512)\n"
        "class NoClocks(bench.ClockSampler):\n"
        "    def start(self): pass\n"
        "line = arm.run(raw, 'tiny', 2, 2, 256, 16, 3, 1, False, NoClocks(), bench.load_peaks(), bench.prefill_flops,\n"
        "               device='cpu', prefill_tokens=64)\n"
        "line['own_package_loaded'] = any(name.split('.')[0] == 'turboserve_b200' for name in sys.modules)\n"
        "print(json.dumps(line))\n" % (str(ROOT), str(ROOT / "baseline")))
    result = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr[-2000:]
    line = json.loads(result.stdout.strip().splitlines()[-1])
    assert REFERENCE_KEYS <= set(line) and line["impl"] == "reference" and not line["own_package_loaded"]
    assert line["value"] > 0 and line["e2e"]["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] > 0 and line["e2e"]["d2h_bytes_per_step"] == 16
    assert set(line["points"]) == {"decode_b1", "decode_b64"} and line["prefill"]["tokens"] == 64
    assert len(line["config"]) <= 20 and all(not isinstance(v, (dict, list)) for v in line["config"].values())


def test_the_config_record_is_flat_and_short():
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.QWEN2_7B["num_hidden_layers"] == 28 and bench.QWEN2_7B["hidden_size"] == 3584
    assert bench.QWEN2_7B["intermediate_size"] == 18944 and bench.QWEN2_7B["vocab_size"] == 152064
    assert bench.CONTEXT == 4096


def test_the_other_shapes_are_the_named_ones():
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_module_shapes", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    small, large = bench.SHAPES["14b"][1], bench.SHAPES["32b"][1]
    assert (small["num_hidden_layers"], small["hidden_size"], small["num_attention_heads"], small["num_key_value_heads"],
            small["intermediate_size"], small["rms_norm_eps"]) == (48, 5120, 40, 8, 13824, 1e-5)
    assert (large["num_hidden_layers"], large["hidden_size"], large["num_attention_heads"], large["num_key_value_heads"],
            large["intermediate_size"], large["rms_norm_eps"]) == (64, 5120, 40, 8, 27648, 1e-5)
    assert bench.SHAPES["7b"][1] is bench.QWEN2_7B


@pytest.mark.gpu
def test_the_preemption_scenario_preempts_and_still_returns_every_token():
    """One layer of the 7B shape: 16 requests whose pool holds half of what they generate.

    Prompts take eight steps each, one request after the other, so the first requests are done
    before the last have begun unless they generate for longer than that: 128 tokens do.
    """
    result = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--scenario", "preempt", "--layers", "1", "--generate", "128"],
                            capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]
    line = json.loads(result.stdout.strip().splitlines()[-1])
    assert line["scenario"] == "preempt" and line["generated_tokens"] == 16 * 128
    assert line["preemptions"] >= 1 and line["recomputed_prompt_tokens"] > 0
    assert len(line["config"]) <= 20 and all(not isinstance(v, (dict, list)) for v in line["config"].values())

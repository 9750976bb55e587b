"""Generation through the Python entry point against the plain implementation."""

import pytest
import torch

import plain_qwen2 as P
from tolerances import BF16_REL_MAX, FP32_ATOL

pytestmark = pytest.mark.gpu


def engine_for(folder, dtype, **scheduler):
    from turboserve_b200 import EngineConfig, LLMEngine, SchedulerConfig

    defaults = dict(max_num_seqs=8, max_num_batched_tokens=256, block_size=16, num_blocks=64)
    defaults.update(scheduler)
    return LLMEngine(EngineConfig(model=str(folder), dtype=dtype, scheduler=SchedulerConfig(**defaults)))


def prompts_for(config, lengths, seed=4):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, config["vocab_size"], (n,), generator=g).tolist() for n in lengths]


def check_greedy_path(config, weights, prompt, generated, dtype):
    """Every generated token is the plain argmax given the tokens before it.

    One plain pass over prompt + generated gives the logits at every step (causality). In
    bfloat16 a token may differ from the plain argmax only if the plain logits of the two are
    closer than the bfloat16 tolerance.
    """
    logits = P.forward_logits(config, weights, prompt + generated)
    slack = FP32_ATOL if dtype == "float32" else BF16_REL_MAX * max(1.0, logits.abs().max().item())
    for i, token in enumerate(generated):
        row = logits[len(prompt) + i - 1]
        best = int(row.argmax())
        assert token == best or row[best] - row[token] <= 2 * slack, (i, token, best, float(row[best] - row[token]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, lengths, new", [("A", [1, 7, 33, 100], 16), ("B", [5, 40, 129], 24), ("C", [3, 70], 20), ("D", [2, 150], 12)])
def test_greedy_generation_matches_plain(model_folders, name, lengths, new, dtype):
    from turboserve_b200 import SamplingParams

    config, weights = P.read_model_folder(model_folders[name])
    prompts = prompts_for(config, lengths)
    with engine_for(model_folders[name], dtype) as engine:
        outputs = engine.generate(prompts, SamplingParams(max_tokens=new, temperature=0.0, ignore_eos=True))
        assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
    for prompt, out in zip(prompts, outputs):
        assert out.finished and out.finish_reason == "length" and out.output_tokens == new and out.prompt_tokens == len(prompt)
        check_greedy_path(config, weights, prompt, out.token_ids, dtype)
        if dtype == "float32":
            assert out.token_ids == P.greedy_generate(config, weights, prompt, 4) + out.token_ids[4:]


def test_one_long_request_among_short_ones_changes_no_token(model_folders):
    """A lopsided decode batch (bfloat16, graphs on): decode attention cuts every request by its own length
    (a work list refilled every step), the runner replays the graph for lopsided batches of that size;
    every token is still the plain argmax."""
    from turboserve_b200 import SamplingParams

    config, weights = P.read_model_folder(model_folders["D"])
    prompts = prompts_for(config, [900, 5, 17, 40, 3, 60], seed=9)
    with engine_for(model_folders["D"], "bfloat16", num_blocks=128, max_num_batched_tokens=512) as engine:
        outputs = engine.generate(prompts, SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True))
        kinds = {key[1] for key in engine.runner._graphs}
        assert engine.runner.num_graph_replays > 0 and kinds == {1, 4}, kinds
        assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
    for prompt, out in zip(prompts, outputs):
        assert out.output_tokens == 20
        check_greedy_path(config, weights, prompt, out.token_ids, "bfloat16")


def test_small_budget_and_few_pages_change_no_token(model_folders):
    """Chunked prefill (budget 16) and recompute preemption (a pool that cannot hold everyone) in float32."""
    from turboserve_b200 import SamplingParams

    config, _ = P.read_model_folder(model_folders["B"])
    prompts = prompts_for(config, [5, 40, 129, 33, 64, 18])
    sampling = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    with engine_for(model_folders["B"], "float32") as engine:
        base = [o.token_ids for o in engine.generate(prompts, sampling)]
        assert engine.stats()["num_preemptions"] == 0
    with engine_for(model_folders["B"], "float32", max_num_batched_tokens=16) as engine:
        chunked = [o.token_ids for o in engine.generate(prompts, sampling)]
    with engine_for(model_folders["B"], "float32", max_num_batched_tokens=64, num_blocks=14) as engine:
        tight = [o.token_ids for o in engine.generate(prompts, sampling)]
        stats = engine.stats()
        engine.scheduler.check_invariants()
    assert chunked == base
    assert tight == base
    assert stats["num_preemptions"] > 0 and stats["num_window_releases"] > 0


def test_bfloat16_with_graphs_overlap_and_preemption_together(model_folders):
    """A pool too small for everyone, a small token budget, captured graphs and steps launched ahead, in
    bfloat16: requests are preempted and recomputed, and every token still follows the plain logits."""
    from turboserve_b200 import SamplingParams

    config, weights = P.read_model_folder(model_folders["D"])
    prompts = prompts_for(config, [5, 40, 129, 33, 64, 18, 90], seed=6)
    sampling = SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True)
    with engine_for(model_folders["D"], "bfloat16", max_num_seqs=4, max_num_batched_tokens=64, num_blocks=22) as engine:
        outputs = engine.generate(prompts, sampling)
        stats = engine.stats()
        engine.scheduler.check_invariants()
        assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
    assert stats["num_preemptions"] > 0 and stats["num_overlapped_steps"] > 0
    for prompt, out in zip(prompts, outputs):
        assert out.finish_reason == "length" and out.output_tokens == 40
        check_greedy_path(config, weights, prompt, out.token_ids, "bfloat16")


@pytest.mark.parametrize("name", ["A", "B"])
def test_temperature_sampling_matches_the_plain_sampler(model_folders, name):
    from turboserve_b200 import SamplingParams

    config, weights = P.read_model_folder(model_folders[name])
    prompts = prompts_for(config, [9, 31])
    options = [dict(temperature=0.7, seed=11), dict(temperature=1.2, top_k=20, top_p=0.9, seed=5, repetition_penalty=1.3)]
    with engine_for(model_folders[name], "float32") as engine:
        outputs = engine.generate(prompts, [SamplingParams(max_tokens=12, ignore_eos=True, logprobs=True, **o) for o in options])
        again = engine.generate(prompts[:1], SamplingParams(max_tokens=12, ignore_eos=True, **options[0]))
    assert again[0].token_ids == outputs[0].token_ids  # a seeded request repeats itself, alone or in company
    for prompt, out, opts in zip(prompts, outputs, options):
        logits = P.forward_logits(config, weights, prompt + out.token_ids)
        for i, token in enumerate(out.token_ids):
            seed = opts.pop("seed") if "seed" in opts and i == 0 else None
            if seed is not None:
                opts["_seed"] = seed
            expect, logprob = P.sample_token(logits[len(prompt) + i - 1], history=prompt + out.token_ids[:i],
                                             seed=opts["_seed"], counter=i, **{k: v for k, v in opts.items() if k != "_seed"})
            assert token == expect, (i, token, expect)
            assert abs(out.logprobs[i] - logprob) < 1e-4


def check_sampling_against_the_plain_sampler(engine):
    """Hook an engine so that every sampled id (and log-probability) is compared with what the plain
    sampler draws from the very row of logits the step produced. Returns the counters
    ``{"checked", "in_step", "logprobs"}``, which go up as the engine runs."""
    launched, counts = [], {"checked": 0, "in_step": 0, "logprobs": 0}
    run_step, process = engine.runner.step, engine._process

    def recording_step(slices, device_tokens=None, sample=False):
        logits = run_step(slices, device_tokens, sample)
        launched.append(None if logits is None else logits.clone())
        counts["in_step"] += int(engine.runner.sampled_in_step)
        return logits

    def checking_process(plan, result):
        logits = launched.pop(0)  # steps are processed in the order they were launched
        if result is not None:
            for index, (row, seq, token) in enumerate(zip(logits.cpu(), plan.sampling_seqs(), result.token_ids)):
                if seq.is_finished:
                    continue
                params = seq.sampling
                expect, logprob = P.sample_token(row, temperature=params.temperature, top_k=params.top_k, top_p=params.top_p,
                                                 repetition_penalty=params.repetition_penalty, history=seq.token_ids, seed=seq.seed,
                                                 counter=seq.num_output_tokens)
                assert token == expect, (seq.request_id, seq.num_output_tokens, token, expect)
                if params.logprobs:
                    assert abs(result.logprobs[index] - logprob) < 1e-4, (seq.request_id, seq.num_output_tokens)
                    counts["logprobs"] += 1
                counts["checked"] += 1
        return process(plan, result)

    engine.runner.step, engine._process = recording_step, checking_process
    return counts


def test_bfloat16_sampled_rows_match_the_plain_sampler_on_the_engines_own_logits(model_folders):
    """Temperature, top-k, top-p, penalties and log-probabilities in bfloat16, with decode steps replayed
    from graphs that end with the sampler (options and histories by state slot) and launched ahead:
    every sampled id is what the plain sampler draws from the very row of logits the step produced
    (exact ids), so a fault of the sampler, of the slot arrays, of the history bitmap or of the
    token's index cannot hide behind bfloat16 rounding."""
    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    config, _ = P.read_model_folder(model_folders["D"])
    prompts = prompts_for(config, [9, 31, 60, 4, 17], seed=12)
    options = [dict(temperature=0.7, seed=11), dict(temperature=1.2, top_k=20, top_p=0.9, seed=5, logprobs=True),
               dict(temperature=0.9, top_p=0.8, seed=7, repetition_penalty=1.3), dict(temperature=1.0, top_p=0.95),
               dict(temperature=0.0, repetition_penalty=1.8, logprobs=True)]
    engine = LLMEngine(EngineConfig(model=str(model_folders["D"]), dtype="bfloat16", seed=3, scheduler=SchedulerConfig(
        max_num_seqs=8, max_num_batched_tokens=256, block_size=16, num_blocks=64)))
    counts = check_sampling_against_the_plain_sampler(engine)
    with engine:
        assert engine.runner.step_sampler is engine.sampler and engine.sampler.slots is not None
        lengths = [14, 14, 14, 14, 14]
        outputs = engine.generate(prompts, [SamplingParams(max_tokens=n, ignore_eos=True, **o) for n, o in zip(lengths, options)])
        stats = engine.stats()
        # every step sampled itself, and all but the first and the last were launched ahead of the ids before them
        assert counts["in_step"] == 14 and stats["num_overlapped_steps"] >= 11 and engine.runner.num_graph_replays == 13
    assert [o.output_tokens for o in outputs] == lengths
    assert counts["checked"] == sum(lengths) and counts["logprobs"] == 28


def test_penalised_requests_through_preemption_and_reused_slots(model_folders):
    """Six requests with penalties take turns in two state slots of a pool that cannot hold two of them
    to their ends: a slot's bitmap is cleared for its next request, and a request that was sent back
    has everything it holds marked again when it is computed again (portions of 24 tokens)."""
    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    config, _ = P.read_model_folder(model_folders["D"])
    prompts = prompts_for(config, [40, 33, 9, 50, 21, 5], seed=4)
    penalties = [1.6, 1.2, 2.0, 1.0, 1.4, 0.8]
    sampling = [SamplingParams(max_tokens=30, ignore_eos=True, temperature=0.0 if i % 2 == 0 else 0.8, seed=i,
                               repetition_penalty=pen, logprobs=i % 3 == 0) for i, pen in enumerate(penalties)]
    engine = LLMEngine(EngineConfig(model=str(model_folders["D"]), dtype="bfloat16", seed=5, scheduler=SchedulerConfig(
        max_num_seqs=2, max_num_batched_tokens=24, block_size=8, num_blocks=14)))
    counts = check_sampling_against_the_plain_sampler(engine)
    with engine:
        outputs = engine.generate(prompts, sampling)
        stats = engine.stats()
        engine.scheduler.check_invariants()
    assert stats["num_preemptions"] > 0 and counts["in_step"] > 40 and stats["num_overlapped_steps"] > 20
    assert [o.output_tokens for o in outputs] == [30] * 6 and counts["checked"] == 180 and counts["logprobs"] == 60


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_random_arrivals_aborts_and_options_keep_every_sampled_id_right(model_folders, dtype):
    """Forty requests with drawn lengths and options (greedy, temperature, filters, penalties,
    log-probabilities) arrive at drawn steps in a pool that forces preemptions; some are aborted
    while they run, also while a step launched ahead still holds them. Every id that is handed
    out is what the plain sampler draws from the row of logits its step produced, every request
    that was not aborted gets all its tokens, and nothing is left behind in the pool."""
    import random

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    config, _ = P.read_model_folder(model_folders["D"])
    rng = random.Random(31)
    engine = LLMEngine(EngineConfig(model=str(model_folders["D"]), dtype=dtype, seed=9, scheduler=SchedulerConfig(
        max_num_seqs=4, max_num_batched_tokens=48, block_size=8, num_blocks=18)))
    counts = check_sampling_against_the_plain_sampler(engine)
    arrivals = []
    for i in range(40):
        options = dict(max_tokens=rng.randint(1, 24), ignore_eos=True, temperature=rng.choice([0.0, 0.0, 0.7, 1.1]), seed=i)
        if rng.random() < 0.4:
            options.update(top_k=rng.choice([0, 5, 40]), top_p=rng.choice([1.0, 0.9, 0.6]))
        if rng.random() < 0.5:
            options["repetition_penalty"] = rng.choice([1.1, 1.5, 0.9])
        options["logprobs"] = rng.random() < 0.3
        arrivals.append((rng.randint(0, 60), f"r{i}", prompts_for(config, [rng.randint(1, 70)], seed=100 + i)[0], SamplingParams(**options)))
    abort_steps = {rng.randint(5, 70) for _ in range(8)}
    produced, finished, aborted = {}, {}, set()
    with engine:
        step = 0
        while step < 80 or engine.has_unfinished():
            for when, rid, prompt, sampling in arrivals:
                if when == step:
                    engine.add_request(rid, prompt, sampling)
            if step in abort_steps and engine.scheduler._running:
                victim = rng.choice(engine.scheduler._running).request_id  # it may be part of the step that is under way
                assert engine.abort(victim)
                aborted.add(victim)
            for out in engine.step():
                produced.setdefault(out.request_id, []).extend(out.new_token_ids)
                if out.finished:
                    finished[out.request_id] = out.finish_reason
            step += 1
            assert step < 2000
        stats = engine.stats()
        engine.scheduler.check_invariants()
        assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
    assert len(aborted) >= 4 and stats["num_preemptions"] > 0 and stats["num_overlapped_steps"] > 5
    for _, rid, _, sampling in arrivals:
        if rid not in aborted:
            assert len(produced[rid]) == sampling.max_tokens and finished[rid] == "length", rid
    assert counts["checked"] >= sum(len(v) for v in produced.values()) and counts["logprobs"] > 20


def test_float32_tokens_do_not_depend_on_how_the_engine_is_configured(model_folders):
    """Eighty requests with drawn lengths, arrival steps and options (filters, penalties, seeds) through three
    float32 engines: roomy with graphs and steps launched ahead; a pool and budgets so tight that
    requests are sent back and prompts cut into many portions; no graphs and nothing launched
    ahead, other page and batch sizes. Float32 logits do not depend on the cut or the batch and a
    draw depends on (seed, index) alone, so every request must get the very same tokens from all three."""
    import random

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    config, _ = P.read_model_folder(model_folders["D"])
    rng = random.Random(5)
    requests = []
    for i in range(80):
        options = dict(max_tokens=rng.randint(1, 40), ignore_eos=True, temperature=rng.choice([0.0, 0.0, 0.8, 1.3]), seed=1000 + i)
        if rng.random() < 0.4:
            options.update(top_k=rng.choice([0, 3, 50]), top_p=rng.choice([1.0, 0.95, 0.5]))
        if rng.random() < 0.4:
            options["repetition_penalty"] = rng.choice([1.05, 1.3, 2.0])
        requests.append((rng.randint(0, 120), f"r{i}", prompts_for(config, [rng.randint(1, 300)], seed=i)[0], SamplingParams(**options)))

    def run(scheduler, **engine_options):
        engine = LLMEngine(EngineConfig(model=str(model_folders["D"]), dtype="float32", seed=1,
                                        scheduler=SchedulerConfig(**scheduler), **engine_options))
        tokens = {}
        with engine:
            step = 0
            while step <= 120 or engine.has_unfinished():
                for when, rid, prompt, sampling in requests:
                    if when == step:
                        engine.add_request(rid, prompt, sampling)
                for out in engine.step():
                    tokens.setdefault(out.request_id, []).extend(out.new_token_ids)
                step += 1
                assert step < 20000
            stats = engine.stats()
            engine.scheduler.check_invariants()
            assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
        return tokens, stats

    roomy, stats_roomy = run(dict(max_num_seqs=16, max_num_batched_tokens=1024, block_size=16, num_blocks=1000))
    tight, stats_tight = run(dict(max_num_seqs=5, max_num_batched_tokens=64, block_size=8, num_blocks=60))
    plain, _ = run(dict(max_num_seqs=9, max_num_batched_tokens=333, block_size=32, num_blocks=150), cuda_graphs=False, overlap_decode=False)
    assert stats_roomy["num_overlapped_steps"] > 0 and stats_tight["num_preemptions"] > 0
    for _, rid, _, sampling in requests:
        assert len(roomy[rid]) == sampling.max_tokens, rid
        assert roomy[rid] == tight[rid] == plain[rid], rid


def test_long_decoding_through_many_pages_and_a_window(model_folders):
    from turboserve_b200 import SamplingParams

    config, weights = P.read_model_folder(model_folders["B"])
    prompt = prompts_for(config, [37])[0]
    for dtype in ("float32", "bfloat16"):
        with engine_for(model_folders["B"], dtype, num_blocks=32) as engine:
            out = engine.generate([prompt], SamplingParams(max_tokens=300, temperature=0.0, ignore_eos=True))[0]
            assert engine.stats()["num_window_releases"] > 10
        assert out.output_tokens == 300
        check_greedy_path(config, weights, prompt, out.token_ids, dtype)


def test_a_window_group_with_exactly_the_pages_of_admission_under_a_large_budget(model_folders):
    """A token budget (251) far above the window (32): the windowed layers' pool has exactly the 37
    pages that admission asks for, all in use during the third portion of a 760-token prompt, whose
    first query reads from the last slot of a page. The tokens are the plain implementation's."""
    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig
    from turboserve_b200.engine.runner import ModelRunner, load_model, make_groups

    config, weights = P.read_model_folder(model_folders["B"])
    prompt = prompts_for(config, [760], seed=13)[0]
    model = load_model(model_folders["B"], torch.float32)
    groups = make_groups(model.cache_plan(), 8, [100, 37])
    assert [g.window for g in groups] == [None, 32]
    runner = ModelRunner(model, groups, 2)
    engine_config = EngineConfig(model="(injected)", dtype="float32", scheduler=SchedulerConfig(
        max_num_seqs=2, max_num_batched_tokens=251, block_size=8))
    with LLMEngine(engine_config, runner=runner) as engine:
        seq = engine.add_request("long", prompt, SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
        least_free = 37
        while engine.has_unfinished():
            engine.step()
            least_free = min(least_free, engine.cache.free_pages()[1])
        assert least_free == 0 and engine.stats()["num_preemptions"] == 0
    check_greedy_path(config, weights, prompt, seq.output_token_ids, "float32")
    smaller = ModelRunner(model, make_groups(model.cache_plan(), 8, [100, 36]), 2)
    with LLMEngine(engine_config, runner=smaller) as engine:
        with pytest.raises(ValueError, match="more than the cache can ever hold"):
            engine.add_request("long", prompt, SamplingParams(max_tokens=8))


def test_requests_step_by_step_abort_stop_and_stats(model_folders):
    from turboserve_b200 import SamplingParams

    with engine_for(model_folders["A"], "bfloat16") as engine:
        engine.add_request("a", [1, 2, 3], SamplingParams(max_tokens=50, temperature=0.0, ignore_eos=True))
        engine.add_request("b", [4, 5, 6, 7], SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))
        with pytest.raises(ValueError):
            engine.add_request("a", [1])
        with pytest.raises(ValueError):
            engine.add_request("c", [999999])
        first = engine.step()
        assert sorted(o.request_id for o in first) == ["a", "b"] and all(len(o.new_token_ids) == 1 for o in first)
        stop_at = next(o.new_token_ids[0] for o in first if o.request_id == "a")
        engine.add_request("d", [1, 2, 3], SamplingParams(max_tokens=50, temperature=0.0, stop_token_ids=[stop_at]))
        seen = {}
        while engine.has_unfinished() and "b" not in seen:
            for o in engine.step():
                if o.finished:
                    seen[o.request_id] = o
        assert seen["b"].finish_reason == "length" and seen["b"].output_tokens == 3
        assert seen["d"].finish_reason == "stop" and seen["d"].output_tokens == 1
        assert engine.abort("a") and not engine.abort("a") and not engine.has_unfinished()
        stats = engine.stats()
        assert stats["num_finished"] == 3 and stats["free_pages"] == [64]
        engine.scheduler.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_decode_changes_no_token(model_folders, dtype):
    """Launching the next decode step before this one's tokens are read gives the same tokens, also
    when a request ends on a stop token that only shows after the next step was launched, when
    requests end at different lengths, and with seeded sampling."""
    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    config, _ = P.read_model_folder(model_folders["C"])
    prompts = prompts_for(config, [5, 40, 70, 9], seed=8)

    def run(overlap, samplings):
        engine = LLMEngine(EngineConfig(model=str(model_folders["C"]), dtype=dtype, overlap_decode=overlap,
                                        scheduler=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=256, block_size=16, num_blocks=64)))
        with engine:
            outs = engine.generate(prompts, samplings)
            assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
            engine.scheduler.check_invariants()
            return [(o.token_ids, o.finish_reason) for o in outs], engine.stats()["num_overlapped_steps"]

    greedy = [SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True) for n in (30, 17, 30, 4)]
    base, none_ahead = run(False, greedy)
    over, ahead = run(True, greedy)
    assert over == base
    assert none_ahead == 0 and ahead >= 20  # most of the 30 decode steps were launched ahead
    # a stop token that the third request produces in the middle of its run
    stop_at = base[2][0][11]
    first_hit = base[2][0].index(stop_at)
    stopping = [SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True, stop_token_ids=[stop_at] if i == 2 else [])
                for i in range(4)]
    base_stop, _ = run(False, stopping)
    over_stop, _ = run(True, stopping)
    assert over_stop == base_stop
    assert base_stop[2] == (base[2][0][: first_hit + 1], "stop")
    seeded = [SamplingParams(max_tokens=20, temperature=0.8, top_k=50, seed=3 + i, ignore_eos=True) for i in range(4)]
    assert run(True, seeded)[0] == run(False, seeded)[0]


def test_the_engine_refuses_to_run_without_its_extension(model_folders, tmp_path, monkeypatch):
    """No compiler and no built library: building an engine and running a step raises the build
    error; no torch path takes over and returns tokens."""
    import turboserve_b200.ops.build as build
    from turboserve_b200 import SamplingParams

    def no_compiler():
        raise build.ExtensionBuildError("nvcc was not found (test)")

    empty = tmp_path / "empty_build_dir"
    empty.mkdir()
    monkeypatch.setenv("TURBOSERVE_B200_BUILD_DIR", str(empty))
    monkeypatch.setattr(build, "find_nvcc", no_compiler)
    monkeypatch.setattr(build, "_loaded", {})
    import turboserve_b200.ops.kernels as kernels

    monkeypatch.setattr(kernels, "_functions", {})  # entry points looked up by earlier tests
    with pytest.raises(build.ExtensionBuildError, match="nvcc was not found"):
        with engine_for(model_folders["A"], "bfloat16") as engine:
            engine.generate([[1, 2, 3]], SamplingParams(max_tokens=2, temperature=0.0))
    assert not list(empty.iterdir())

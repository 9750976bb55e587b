"""What the entry point does when a step fails, with a runner and a sampler that need no GPU."""

import pytest
import torch

from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig
from turboserve_b200.cache import GroupSpec
from turboserve_b200.engine.runner import StepError


class HostRunner:
    """Stands in for ModelRunner: logits that make every request answer token 7; fails on demand."""

    class Spec:
        eos_token_ids = ()

    class Model:
        vocab_size = 32

    def __init__(self, pages=64, page_size=4, slots=4):
        self.device = torch.device("cpu")
        self.dtype = torch.float32
        self.groups = [GroupSpec("full", None, pages, page_size)]
        self.model = self.Model()
        self.model.spec = self.Spec()
        self.token_buffer = torch.zeros(slots + 1, dtype=torch.int32)
        self.token_out = self.token_buffer[:slots]
        self.fail_reads = 0
        self.steps = []

    def step(self, slices, device_tokens=None, sample=False):
        self.steps.append([(len(piece.token_ids), piece.start_position) for piece in slices])
        rows = sum(len(piece.want) for piece in slices)
        logits = torch.zeros(rows, 32)
        logits[:, 7] = 1.0
        return logits

    def reset_state_slot(self, slot):
        pass

    def start_token_read(self, count):
        runner = self

        class Read:
            def finish(self):
                if runner.fail_reads:
                    runner.fail_reads -= 1
                    raise StepError("a wait on a copy barrier ran out (test)")
                return runner.token_buffer.tolist()[:count]

        return Read()


class HostSampler:
    def sample_device(self, logits, rows, out=None):
        tokens = out[: len(rows)]
        tokens.copy_(logits[: len(rows)].argmax(-1).to(torch.int32))
        return tokens, None


def make_engine(overlap):
    runner = HostRunner()
    config = EngineConfig(model="(injected)", dtype="float32", overlap_decode=overlap, cuda_graphs=False,
                          scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, block_size=4))
    return LLMEngine(config, runner=runner, sampler=HostSampler()), runner


@pytest.mark.parametrize("overlap", [False, True])
def test_a_failed_step_ends_its_requests_and_the_engine_goes_on(overlap):
    engine, runner = make_engine(overlap)
    params = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    engine.add_request("a", [1, 2, 3], params)
    engine.add_request("b", [4, 5], params)
    assert sorted(o.request_id for o in engine.step()) == ["a", "b"]  # prompts
    engine.step()
    if overlap:
        assert engine._num_overlapped_steps > 0 and engine._in_flight is not None
    runner.fail_reads = 1
    with pytest.raises(StepError):
        engine.step()
    # nobody is left holding pages with nothing to compute; a caller that goes on stepping does not spin
    engine.scheduler.check_invariants()
    assert not engine.has_unfinished() and engine._in_flight is None
    assert engine.cache.free_pages() == [64] and engine.cache.slots.num_free == engine.cache.slots.num_slots
    assert engine.step() == []
    # and the engine still serves: a new request runs to its end
    out = engine.generate([[9, 9, 9]], params)[0]
    assert out.finished and out.token_ids == [7] * 6
    engine.scheduler.check_invariants()


def test_requests_outside_the_failed_step_are_untouched():
    engine, runner = make_engine(False)
    params = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
    engine.add_request("a", [1, 2, 3], params)
    engine.step()
    late = engine.add_request("late", [i % 32 for i in range(100)], params)  # takes what is left of the step's budget
    waiting = engine.add_request("w", [6], params)  # nothing is left for it: it is not in the step that fails
    runner.fail_reads = 1
    with pytest.raises(StepError):
        engine.step()
    assert runner.steps[-1] == [(63, 0), (1, 3)]
    assert engine.scheduler.get("a") is None and engine.scheduler.get("late") is None
    assert late.finish_reason.value == "abort" and engine.scheduler.get("w") is waiting
    while engine.has_unfinished():
        engine.step()
    assert waiting.output_token_ids == [7] * 4 and waiting.finish_reason.value == "length"
    engine.scheduler.check_invariants()

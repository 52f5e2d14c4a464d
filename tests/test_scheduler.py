"""The scheduler's decisions and the engine's host-side logic (no GPU).

The engine tests swap the plain torch twins in for the kernels, so they check
admission, portions, mixed batches, freeing and page reuse against the plain
model on the CPU; the kernels themselves are checked by the -m gpu tests.
"""

import pytest
import torch

from simple_inference_b200 import InferenceEngine, SamplingParams
from simple_inference_b200.engine import Request, RequestState, Scheduler
from tests import plain_llama, twin_ops
from tests.conftest import random_ids


def _req(n_prompt, max_new=4):
    return Request(list(range(n_prompt)), max_new)


def test_fcfs_admission_up_to_slots_and_budget():
    s = Scheduler(max_running=2, max_tokens_per_step=16, token_budget=30)
    a, b, c = _req(10), _req(25), _req(3)
    for r in (a, b, c):
        s.add(r)
    admitted = s.admit(lambda r: True, lambda r: None)
    assert admitted == [a]            # b would push the summed context past 30
    assert a.state is RequestState.PREFILL and b.state is RequestState.WAITING
    a.state = RequestState.FINISHED
    assert s.evict_finished() == [a]
    assert s.admit(lambda r: True, lambda r: None) == [b, c]
    # one request is always let in when nothing runs, however long its prompt
    s2 = Scheduler(2, 16, token_budget=5)
    big = _req(100)
    s2.add(big)
    assert s2.admit(lambda r: True, lambda r: None) == [big]


def test_head_of_queue_blocks_when_pages_are_short():
    # the reference's rule (serving/scheduler.py:109-113): no request jumps the queue
    s = Scheduler(4, 64)
    big, small = _req(40), _req(2)
    s.add(big)
    s.add(small)
    assert s.admit(lambda r: r is not big, lambda r: None) == []
    assert list(s.waiting) == [big, small]
    assert s.admit(lambda r: True, lambda r: None) == [big, small]


def test_step_plan_decodes_first_then_portions_under_the_budget():
    s = Scheduler(max_running=4, max_tokens_per_step=10, chunk_size=6)
    d1, d2, p1, p2 = _req(3), _req(3), _req(20), _req(9)
    for r in (d1, d2, p1, p2):
        s.add(r)
    s.admit(lambda r: True, lambda r: None)
    d1.state = d2.state = RequestState.DECODE
    plan = s.plan_step()
    assert plan == [(d1, 1), (d2, 1), (p1, 6), (p2, 2)]     # 10 tokens in all
    p1.prefilled = 18
    assert s.plan_step() == [(d1, 1), (d2, 1), (p1, 2), (p2, 6)]
    with pytest.raises(ValueError):
        Scheduler(max_running=8, max_tokens_per_step=4)


@pytest.fixture()
def cpu_engine(model_folders):
    made = []

    def make(name, **kw):
        opts = dict(max_running=3, max_seq_len=96, block_size=4, eos_id=-1, use_cuda_graphs=False,
                    max_tokens_per_step=16, chunk_size=7)
        opts.update(kw)
        eng = InferenceEngine.from_folder(model_folders[name], "float32", "cpu", **opts)
        made.append(eng)
        return eng

    with twin_ops.use_twins():
        yield make


@pytest.mark.parametrize("name", ["A", "B"])
def test_engine_greedy_equals_plain_alone_and_together(name, cpu_engine, model_folders):
    cfg, w = plain_llama.read_folder(model_folders[name])
    prompts = [random_ids(n, cfg["vocab_size"], 40 + n) for n in (5, 17, 32, 1)]
    want = [plain_llama.generate_greedy(cfg, w, p, 6) for p in prompts]
    eng = cpu_engine(name, num_kv_blocks=20)              # few pages: requests wait, pages are reused
    reqs = [eng.add_request(p, 6) for p in prompts]
    done = eng.run()
    assert [r.generated for r in reqs] == want
    assert all(r.finish_reason == "length" for r in reqs) and set(done) == {r.id for r in reqs}
    eng.cache.check()
    assert eng.cache.free_pages() == 20 and eng.cache.free_slots == 3
    solo = cpu_engine(name)
    for p, g in zip(prompts, want):
        assert list(solo.generate(p, 6)) == g


def test_engine_waits_for_pages_and_refuses_what_never_fits(cpu_engine):
    # the reference's capacity test (serving/test_paged_kv_cache.py:247-269): 2 pages, 2 requests
    eng = cpu_engine("A", num_kv_blocks=2, block_size=4, max_running=2)
    a = eng.add_request([1, 2, 3], 4)      # 7 tokens -> 2 pages: takes the whole pool
    b = eng.add_request([4, 5], 3)         # 5 tokens -> 2 pages: must wait
    with pytest.raises(ValueError):
        eng.add_request(list(range(6)), 4)  # 10 tokens -> 3 pages: can never fit
    eng.step()
    assert a.state is not RequestState.WAITING and b.state is RequestState.WAITING
    while a.state is not RequestState.FINISHED:
        eng.step()
        assert b.state is RequestState.WAITING or a.state is RequestState.FINISHED
    eng.run()
    assert len(a.generated) == 4 and len(b.generated) == 3
    assert eng.cache.free_pages() == 2


def test_engine_stops_on_eos_and_validates_requests(cpu_engine, model_folders):
    cfg, w = plain_llama.read_folder(model_folders["B"])
    prompt = random_ids(9, cfg["vocab_size"], 3)
    free_run = plain_llama.generate_greedy(cfg, w, prompt, 8)
    eng = cpu_engine("B", eos_id=free_run[3])
    r = eng.add_request(prompt, 8)
    eng.run()
    stop = free_run.index(free_run[3])
    assert r.generated == free_run[:stop + 1] and r.finish_reason == "stop"   # the end token is kept
    for bad in ([], [cfg["vocab_size"]], [-1]):
        with pytest.raises(ValueError):
            eng.add_request(bad, 2)
    with pytest.raises(ValueError):
        eng.add_request([1], 0)
    with pytest.raises(ValueError):
        eng.add_request(list(range(90)), 10)            # beyond max_seq_len


def test_temperature_sampling_is_reproducible_and_batch_invariant(cpu_engine, model_folders):
    cfg, w = plain_llama.read_folder(model_folders["B"])
    prompts = [random_ids(n, cfg["vocab_size"], 70 + n) for n in (1, 9, 40)]
    sp = SamplingParams(temperature=0.8, top_k=0, top_p=1.0, seed=0)

    def plain_sampled(p, n):
        ids, out = list(p), []
        for c in range(n):
            tok = plain_llama.sample(plain_llama.forward(cfg, w, ids)[-1], 0.8, seed=0, stream=0, counter=c)
            out.append(tok)
            ids.append(tok)
        return out

    want = [plain_sampled(p, 5) for p in prompts]
    eng = cpu_engine("B", chunk_size=16)
    reqs = [eng.add_request(p, 5, sp) for p in prompts]
    eng.run()
    assert [r.generated for r in reqs] == want
    solo = cpu_engine("B")
    assert list(solo.generate(prompts[2], 5, temperature=0.8, seed=0)) == want[2]

"""The scheduler's decisions, without a model (a helper pretends that the step ran).
The cases restate those of umarhassan-cloud/kvforge's tests/test_scheduler.py:28-134."""

from __future__ import annotations

import pytest

from kvforge_b200.cache.block_manager import BlockManager, GroupSpec
from kvforge_b200.cache.state_slots import StateSlotPool
from kvforge_b200.config.engine_config import SchedulerConfig
from kvforge_b200.engine.request import FinishReason, Request, RequestStatus
from kvforge_b200.engine.scheduler import RequestRejectedError, Scheduler
from kvforge_b200.sampling.params import SamplingParams


def make(num_blocks=64, block_size=4, slots=None, groups=None, **cfg) -> Scheduler:
    pool = StateSlotPool(slots) if slots else None
    return Scheduler(SchedulerConfig(**cfg), BlockManager(num_blocks, block_size, groups=groups), pool)


def req(rid: str, n: int, arrival: float, max_tokens: int = 8) -> Request:
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens), arrival_time=arrival)


def complete(out) -> None:
    """Pretend the model ran: advance the computed counts, sample a token when the known
    tokens are all in the cache."""
    for s in out.scheduled:
        r = s.request
        r.num_computed_tokens += s.num_new_tokens
        if r.num_computed_tokens == r.num_tokens:
            r.append_token(0)


def test_fcfs_admission_order_and_max_seqs():
    s = make(max_num_seqs=2)
    for i, t in enumerate([3.0, 1.0, 2.0]):
        s.add_request(req(f"r{i}", 4, arrival=t))
    out = s.schedule()
    assert [x.request.request_id for x in out.scheduled] == ["r1", "r2"]
    assert all(x.is_prefill for x in out.scheduled)
    assert s.num_running == 2 and s.num_waiting == 1


def test_prefill_then_decode_phases():
    s = make()
    s.add_request(req("a", 6, 0.0))
    out = s.schedule()
    assert out.scheduled[0].is_prefill and out.scheduled[0].num_new_tokens == 6
    complete(out)
    out = s.schedule()
    assert not out.scheduled[0].is_prefill and out.scheduled[0].num_new_tokens == 1


def test_token_budget_cuts_prompts_into_portions():
    s = make(max_num_batched_tokens=8)
    s.add_request(req("a", 20, 0.0))
    chunks = []
    while True:
        out = s.schedule()
        x = out.scheduled[0]
        chunks.append(x.num_new_tokens)
        complete(out)
        if x.request.num_output_tokens:
            break
    assert chunks == [8, 8, 4]


def test_decodes_are_scheduled_before_new_prefills():
    s = make(max_num_batched_tokens=10)
    s.add_request(req("a", 4, 0.0))
    complete(s.schedule())
    s.add_request(req("b", 30, 1.0))
    out = s.schedule()
    assert [(x.request.request_id, x.num_new_tokens) for x in out.scheduled] == [("a", 1), ("b", 9)]


def test_max_prefill_chunk_caps_a_portion():
    s = make(max_num_batched_tokens=64, max_prefill_chunk=16)
    s.add_request(req("a", 40, 0.0))
    s.add_request(req("b", 5, 1.0))
    out = s.schedule()
    assert [(x.request.request_id, x.num_new_tokens) for x in out.scheduled] == [("a", 16), ("b", 5)]
    complete(out)
    out = s.schedule()
    assert [(x.request.request_id, x.num_new_tokens, x.is_prefill) for x in out.scheduled] == [("a", 16, True), ("b", 1, False)]


def test_rejections():
    s = make(max_num_batched_tokens=8, enable_chunked_prefill=False)
    with pytest.raises(RequestRejectedError):
        s.add_request(req("big", 9, 0.0))
    s = make(num_blocks=2, block_size=4)
    with pytest.raises(RequestRejectedError):
        s.add_request(req("never", 6, 0.0, max_tokens=8))
    s = make(max_model_len=16)
    with pytest.raises(RequestRejectedError):
        s.add_request(req("long", 16, 0.0))
    with pytest.raises(RequestRejectedError):
        s.add_request(Request("empty", []))
    s.add_request(req("a", 3, 0.0))
    with pytest.raises(RequestRejectedError):
        s.add_request(req("a", 3, 1.0))


def test_when_pages_run_out_the_latest_arrival_is_preempted_and_recomputed():
    # 4 pages of 4.  Two requests of 7 tokens hold 2 pages each; reaching 9 tokens needs a third
    # page for both: the later arrival gives way, and later runs prompt and generated tokens again.
    s = make(num_blocks=4, block_size=4, max_num_seqs=4)
    s.add_request(req("old", 7, 0.0, max_tokens=4))
    s.add_request(req("new", 7, 1.0, max_tokens=4))
    complete(s.schedule())
    complete(s.schedule())
    out = s.schedule()
    assert [r.request_id for r in out.preempted] == ["new"]
    assert [x.request.request_id for x in out.scheduled] == ["old"]
    victim = out.preempted[0]
    assert victim.status == RequestStatus.WAITING and victim.num_computed_tokens == 0
    assert victim.num_preemptions == 1 and s.num_preemptions == 1
    assert not s.block_manager.has_seq("new")
    complete(out)
    s.finish_request(s.running[0], FinishReason.LENGTH)
    out = s.schedule()
    assert out.scheduled[0].request is victim
    assert out.scheduled[0].num_new_tokens == victim.num_tokens == 9
    s.block_manager.check_invariants()


def test_no_admission_in_a_step_that_preempted():
    s = make(num_blocks=4, block_size=4, max_num_seqs=4)
    s.add_request(req("old", 7, 0.0, max_tokens=4))
    s.add_request(req("new", 7, 1.0, max_tokens=4))
    complete(s.schedule())
    complete(s.schedule())
    s.add_request(req("third", 2, 2.0, max_tokens=2))
    out = s.schedule()
    assert out.preempted and all(x.request.request_id != "third" for x in out.scheduled)


def test_a_lone_request_that_cannot_grow_preempts_itself():
    s = make(num_blocks=3, block_size=4, max_num_seqs=2)
    s.add_request(req("a", 8, 0.0, max_tokens=4))
    complete(s.schedule())
    # somebody else takes the last page
    s.block_manager.allocate("squatter", 4)
    out = s.schedule()
    assert [r.request_id for r in out.preempted] == ["a"] and out.is_empty
    assert s.block_manager.free_blocks_of(0) == 2


def test_head_of_line_blocks_admission():
    s = make(num_blocks=6, block_size=4, max_num_seqs=4)
    s.add_request(req("a", 12, 0.0, max_tokens=2))
    complete(s.schedule())
    s.add_request(req("big", 16, 1.0, max_tokens=2))  # needs 4 pages, 3 are free
    s.add_request(req("small", 2, 2.0, max_tokens=2))
    out = s.schedule()
    assert [x.request.request_id for x in out.scheduled] == ["a"]  # "small" may not jump the queue


def test_state_slots_gate_admission_and_come_back():
    s = make(slots=1, max_num_seqs=4)
    s.add_request(req("a", 4, 0.0, max_tokens=1))
    s.add_request(req("b", 4, 1.0, max_tokens=1))
    out = s.schedule()
    assert [x.request.request_id for x in out.scheduled] == ["a"]
    complete(out)
    s.finish_request(out.scheduled[0].request, FinishReason.LENGTH)
    out = s.schedule()
    assert [x.request.request_id for x in out.scheduled] == ["b"]
    assert s.state_slots.slot("b") == 0


def test_abort_waiting_and_running_frees_everything():
    s = make(max_num_seqs=1, slots=2)
    s.add_request(req("a", 4, 0.0))
    s.add_request(req("b", 4, 1.0))
    s.schedule()
    assert s.abort_request("b").status == RequestStatus.ABORTED
    assert s.abort_request("a").finish_reason == FinishReason.ABORT
    assert not s.has_unfinished()
    assert s.block_manager.num_free_blocks == s.block_manager.num_blocks
    assert s.state_slots.num_free == 2
    assert s.abort_request("a") is None


def test_window_group_requests_run_to_the_end():
    s = make(num_blocks=8, block_size=4, groups=[GroupSpec("window", 6)], max_num_batched_tokens=8, max_model_len=200)
    s.add_request(req("a", 50, 0.0, max_tokens=20))
    steps = 0
    while s.has_unfinished():
        out = s.schedule()
        assert not out.preempted and out.scheduled
        complete(out)
        r = out.scheduled[0].request
        if r.num_output_tokens >= 20:
            s.finish_request(r, FinishReason.LENGTH)
        s.block_manager.check_invariants()
        steps += 1
    assert steps == 7 + 19 and s.block_manager.num_free_blocks == 8


def test_stop_rules_and_tokens_in_flight():
    r = Request("a", [1, 2, 3], SamplingParams(max_tokens=3, stop_token_ids=[9]), eos_token_id=7)
    assert r.stops_at(9) and r.stops_at(7) and not r.stops_at(5)
    r.append_token(5)
    assert not r.at_count_limit(100)
    r2 = Request("b", [1], SamplingParams(max_tokens=2, ignore_eos=True), eos_token_id=7)
    assert not r2.stops_at(7)
    r2.append_token(7)
    assert not r2.at_count_limit(100)
    r2.append_token(7)
    assert r2.at_count_limit(100)
    r3 = Request("c", [1, 2], SamplingParams(max_tokens=50))
    r3.append_token(1)
    assert r3.at_count_limit(3)
    # a launched token holds its place and counts, gets its time when it lands, and can be dropped
    r4 = Request("d", [4, 5], SamplingParams(max_tokens=4), arrival_time=10.0)
    r4.num_computed_tokens = 2
    i0 = r4.launch_token()
    assert r4.has_token_in_flight and r4.num_tokens == 3 and r4.ttft is None and r4.in_flight_within(0) and not r4.is_prefill
    i1 = r4.launch_token()
    r4.land_token(i0, 8, now=10.5)
    assert r4.ttft == 0.5 and r4.tokens(1, 2) == [5, 8]
    assert not r4.in_flight_within(4) or r4.in_flight_within(3)
    assert r4.in_flight_within(3) and not Request("e", [1]).in_flight_within(0)
    r4.land_token(i1, 9, now=10.75)
    assert r4.tpot == 0.25 and not r4.has_token_in_flight
    r4.launch_token()
    r4.drop_token_in_flight()
    assert r4.output_token_ids == [8, 9] and len(r4.token_times) == 2
    r4.truncate_output(1)
    assert r4.output_token_ids == [8] and r4.tokens(0, 3) == [4, 5, 8]

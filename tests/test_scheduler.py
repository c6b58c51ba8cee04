"""The scheduler's decisions, driven by a fake step function (no device).

The fake mirrors the reference's deterministic test executor (src/engine/testing.rs:11-112):
the next token of a request is 1000 after its prompt, then the previous token plus one.
"""

import random

import pytest
import torch
from hypothesis import given, settings, strategies as st

import tesseract_b200.parts  # noqa: F401
from tesseract_b200.cache import CacheManager
from tesseract_b200.config import EngineConfig
from tesseract_b200.engine.scheduler import (FINISH_ERROR, FINISH_LENGTH, FINISH_STOP, EngineOverloaded,
                                             RequestRejected, Scheduler)
from tesseract_b200.parts import PagedKVNeed
from tesseract_b200.sampling import SamplingParams, SplitMix64


class FakeEngine:
    def __init__(self, config: EngineConfig, fail_on_step=None):
        need = PagedKVNeed(1, 16)
        self.cache = CacheManager([need], [None], num_pages=config.num_pages, page_size=config.page_size,
                                  max_requests=config.max_running, dtype=torch.float32, device="cpu",
                                  max_step_tokens=config.prefill_chunk_tokens, allocate_storage=False)
        self.batches = []
        self.fail_on_step = fail_on_step
        self.draws = []

    def run_step(self, entries):
        if self.fail_on_step is not None and len(self.batches) == self.fail_on_step:
            self.batches.append("failed")
            raise RuntimeError("injected step failure")
        self.batches.append([(e.request, self.cache.length(e.request), list(e.tokens), list(e.want)) for e in entries])
        rows = []
        for e in entries:
            self.cache.extend(e.request, len(e.tokens))
            self.cache.commit(e.request, len(e.tokens))
            for place in e.want:
                rows.append(e.tokens[place])
        return rows

    def sample(self, rows, temperatures, top_ps, draws):
        self.draws.extend(draws)
        return [1000 if last < 1000 else last + 1 for last in rows]


def make(config=None, **kw):
    config = config or EngineConfig(max_queue=8, max_running=4, max_batch_tokens=32, prefill_chunk_tokens=8,
                                    kv_capacity_tokens=512, max_sequence_length=512)
    fake = FakeEngine(config, **kw)
    return Scheduler(config, fake.cache, fake.run_step, fake.sample, eos_token_ids=[1003], max_positions=400), fake


def run_all(scheduler, limit=10_000):
    finished = []
    for _ in range(limit):
        if not scheduler.has_work():
            return finished
        finished += scheduler.step().finished
    raise AssertionError("the scheduler made no progress")


GREEDY = dict(temperature=0.0)


def test_prompt_is_cut_into_portions_then_decoded():
    s, fake = make()
    rid = s.add_request(list(range(20)), SamplingParams(max_tokens=3, ignore_eos=True, **GREEDY))
    done = run_all(s)
    assert [b[0][1:3] for b in fake.batches[:3]] == [(0, list(range(8))), (8, list(range(8, 16))), (16, [16, 17, 18, 19])]
    assert [b[0][3] for b in fake.batches[:3]] == [[], [], [3]]      # only the last portion samples
    assert fake.batches[3][0][1:3] == (20, [1000])                  # then single decoded tokens
    assert done[0].generated == [1000, 1001, 1002] and done[0].finish_reason == FINISH_LENGTH
    assert s.cache.used_pages() == 0


def test_eos_and_stop_tokens_finish():
    s, _ = make()
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=50, **GREEDY))
    b = s.add_request([4, 5], SamplingParams(max_tokens=50, stop_token_ids=[1001], **GREEDY))
    c = s.add_request([6], SamplingParams(max_tokens=6, ignore_eos=True, **GREEDY))
    done = {r.id: r for r in run_all(s)}
    assert done[a].generated[-1] == 1003 and done[a].finish_reason == FINISH_STOP      # the model's eos id
    assert done[b].generated == [1000, 1001] and done[b].finish_reason == FINISH_STOP
    assert len(done[c].generated) == 6 and done[c].finish_reason == FINISH_LENGTH


def test_decode_rows_come_before_prompt_portions_in_the_budget():
    config = EngineConfig(max_queue=8, max_running=4, max_batch_tokens=10, prefill_chunk_tokens=8,
                          kv_capacity_tokens=512, max_sequence_length=512)
    s, fake = make(config)
    s.add_request([1, 2], SamplingParams(max_tokens=20, ignore_eos=True, **GREEDY))
    s.step()                                    # request 0 is now decoding
    s.add_request(list(range(30)), SamplingParams(max_tokens=2, ignore_eos=True, **GREEDY))
    s.add_request(list(range(30)), SamplingParams(max_tokens=2, ignore_eos=True, **GREEDY))
    s.step()
    batch = fake.batches[-1]
    assert sum(len(tokens) for _, _, tokens, _ in batch) == 10       # exactly the budget
    sizes = {rid: len(tokens) for rid, _, tokens, _ in batch}
    assert sizes[0] == 1 and sorted(sizes.values()) == [1, 1, 8]     # decode first, then 8, then the last token left
    # in the lowered batch prompt portions stand before decode rows
    assert [len(t) for _, _, t, _ in batch][-1] == 1 and batch[-1][0] == 0


def test_full_portions_stand_before_shorter_ones_in_the_lowered_batch():
    """Under one budget a step may carry the end of one prompt, full portions of others and decode rows: the full
    portions come first, then the shorter one, then the decode rows (the shape that replays as one graph)."""
    config = EngineConfig(max_queue=8, max_running=4, max_batch_tokens=32, prefill_chunk_tokens=8,
                          kv_capacity_tokens=512, max_sequence_length=512)
    s, fake = make(config)
    s.add_request([1, 2], SamplingParams(max_tokens=20, ignore_eos=True, **GREEDY))
    s.step()                                    # request 0 is now decoding
    s.add_request(list(range(13)), SamplingParams(max_tokens=2, ignore_eos=True, **GREEDY))     # 8 + 5
    s.add_request(list(range(30)), SamplingParams(max_tokens=2, ignore_eos=True, **GREEDY))
    s.step()
    s.step()                                    # request 1 brings its last five tokens, request 2 a full portion
    batch = fake.batches[-1]
    assert [(rid, len(tokens)) for rid, _, tokens, _ in batch] == [(2, 8), (1, 5), (0, 1)]
    assert [want for _, _, _, want in batch] == [[], [4], [0]]


def test_rotation_shares_a_tight_budget():
    config = EngineConfig(max_queue=8, max_running=3, max_batch_tokens=8, prefill_chunk_tokens=8,
                          kv_capacity_tokens=512, max_sequence_length=512)
    s, fake = make(config)
    for _ in range(3):
        s.add_request(list(range(24)), SamplingParams(max_tokens=1, **GREEDY))
    firsts = []
    for _ in range(3):
        s.step()
        firsts.append(fake.batches[-1][0][0])
    assert sorted(firsts) == [0, 1, 2]          # no request monopolises the budget


def test_bounded_admission_and_rejections():
    s, _ = make()
    with pytest.raises(RequestRejected, match="empty"):
        s.add_request([], SamplingParams(max_tokens=1))
    with pytest.raises(RequestRejected, match="capacity"):
        s.add_request([1] * 390, SamplingParams(max_tokens=20))      # passes the model's 400 positions
    with pytest.raises(ValueError):
        s.add_request([1], SamplingParams(max_tokens=1, top_p=0.0))
    for _ in range(12):
        s.add_request([1, 2, 3], SamplingParams(max_tokens=2, **GREEDY))
    with pytest.raises(EngineOverloaded):
        s.add_request([1], SamplingParams(max_tokens=1))
    assert len(run_all(s)) == 12


def test_when_pages_run_out_requests_wait_and_smaller_ones_pass():
    config = EngineConfig(max_queue=8, max_running=4, max_batch_tokens=64, prefill_chunk_tokens=16,
                          kv_capacity_tokens=96, max_sequence_length=512)     # six pages
    s, fake = make(config)
    big1 = s.add_request([1] * 50, SamplingParams(max_tokens=14, ignore_eos=True, **GREEDY))   # 4 pages
    big2 = s.add_request([2] * 50, SamplingParams(max_tokens=14, ignore_eos=True, **GREEDY))   # 4 pages: must wait
    small = s.add_request([3] * 10, SamplingParams(max_tokens=6, ignore_eos=True, **GREEDY))   # 1 page: passes big2
    s.step()
    assert list(s.running) and big2 in s.waiting and small not in s.waiting
    with pytest.raises(RequestRejected):
        s.add_request([4] * 90, SamplingParams(max_tokens=20))                  # can never fit the cache
    order = [r.id for r in run_all(s)]
    assert set(order) == {big1, big2, small} and order.index(big2) == 2
    s.cache.check()
    assert s.cache.used_pages() == 0
    # nothing that ran was ever interrupted: each request's positions only grow
    seen = {}
    for batch in fake.batches:
        for rid, begin, tokens, _ in batch:
            assert begin == seen.get(rid, 0)
            seen[rid] = begin + len(tokens)


def test_failed_step_fails_its_batch_and_the_engine_goes_on():
    s, fake = make(fail_on_step=1)
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=4, ignore_eos=True, **GREEDY))
    s.step()
    result = s.step()
    assert [r.id for r in result.finished] == [a] and result.finished[0].finish_reason == FINISH_ERROR
    assert "injected" in result.finished[0].error and s.cache.used_pages() == 0
    b = s.add_request([5], SamplingParams(max_tokens=2, ignore_eos=True, **GREEDY))
    assert [r.generated for r in run_all(s)] == [[1000, 1001]]


def test_one_draw_per_sampled_step_and_none_for_greedy():
    s, fake = make()
    s.add_request(list(range(20)), SamplingParams(max_tokens=3, temperature=0.7, seed=42, ignore_eos=True))
    s.add_request([1, 2], SamplingParams(max_tokens=3, ignore_eos=True, **GREEDY))
    run_all(s)
    rng = SplitMix64(42)
    expected = [rng.unit_f64() for _ in range(3)]
    assert [d for d in fake.draws if d != 0.0] == expected


def test_cancel_frees_everything():
    s, _ = make()
    a = s.add_request([1] * 30, SamplingParams(max_tokens=5, **GREEDY))
    s.step()
    assert s.cache.used_pages() > 0
    s.cancel(a)
    assert not s.has_work() and s.cache.used_pages() == 0


@settings(max_examples=80, deadline=None)
@given(data=st.data())
def test_scheduler_state_machine(data):
    """Arbitrary requests, budgets and portion sizes (after src/engine/scheduler.rs:1508-1606)."""
    max_running = data.draw(st.integers(1, 4))
    budget = data.draw(st.integers(max_running, 24))
    chunk = data.draw(st.integers(1, 12))
    config = EngineConfig(max_queue=8, max_running=max_running, max_batch_tokens=budget, prefill_chunk_tokens=chunk,
                          kv_capacity_tokens=data.draw(st.integers(64, 256)), max_sequence_length=512)
    s, fake = make(config)
    shapes = data.draw(st.lists(st.tuples(st.integers(1, 40), st.integers(1, 12)), min_size=1, max_size=6))
    wanted = {}
    for prompt_len, max_tokens in shapes:
        if prompt_len + max_tokens > config.num_pages * config.page_size:
            continue
        rid = s.add_request(list(range(prompt_len)), SamplingParams(max_tokens=max_tokens, ignore_eos=True, **GREEDY))
        wanted[rid] = (prompt_len, max_tokens)
    done = {r.id: r for r in run_all(s)}
    assert set(done) == set(wanted)
    for rid, (prompt_len, max_tokens) in wanted.items():
        assert done[rid].generated == [1000 + i for i in range(max_tokens)]
    for batch in fake.batches:
        assert 0 < sum(len(t) for _, _, t, _ in batch) <= budget
        assert len(batch) <= max_running
        kinds = [begin >= wanted[rid][0] for rid, begin, _, _ in batch]
        assert kinds == sorted(kinds)                       # prompt portions, then decode rows
        for rid, begin, tokens, want in batch:
            is_decode = begin >= wanted[rid][0]
            assert len(tokens) == 1 if is_decode else len(tokens) <= chunk
            assert want in ([], [len(tokens) - 1])
    s.cache.check()
    assert s.cache.used_pages() == 0 and s.cache.slots.free_slots == max_running


# ----------------------------------------------------------------------------- steps launched ahead of their read-back


class FakeLaunch:
    def __init__(self, rows, tokens):
        self.rows, self._tokens, self.read = rows, tokens, False

    def tokens(self):
        self.read = True
        return list(self._tokens)


class FakeAheadEngine(FakeEngine):
    """The fake with a device-like decode path: a launch returns at once, its tokens are read later, and a row
    may take its token from the launch before (by that launch's row of the same request)."""

    def __init__(self, config, fail_launch=None, **kw):
        super().__init__(config, **kw)
        self.launches = []
        self.unread_at_launch = []
        self.fail_launch = fail_launch

    def can_launch_decode(self, rows, top_ps):
        return 0 < rows <= 4 and all(p >= 1.0 for p in top_ps)

    def launch_decode(self, entries, temperatures, draws, previous, fed):
        if self.fail_launch is not None and len(self.launches) == self.fail_launch:
            self.launches.append("failed")
            raise RuntimeError("injected launch failure")
        self.unread_at_launch.append(previous is not None and not previous.read)
        tokens = []
        for e, from_device in zip(entries, fed):
            last = previous._tokens[previous.rows[e.request]] if from_device else e.tokens[0]
            assert from_device or last is not None
            self.cache.extend(e.request, 1)
            self.cache.commit(e.request, 1)
            tokens.append(1000 if last < 1000 else last + 1)
        self.draws.extend(draws)
        launch = FakeLaunch({e.request: i for i, e in enumerate(entries)}, tokens)
        self.launches.append(launch)
        return launch


def make_ahead(**kw):
    config = EngineConfig(max_queue=8, max_running=4, max_batch_tokens=32, prefill_chunk_tokens=8,
                          kv_capacity_tokens=512, max_sequence_length=512)
    fake = FakeAheadEngine(config, **kw)
    scheduler = Scheduler(config, fake.cache, fake.run_step, fake.sample, eos_token_ids=[1003], max_positions=400,
                          launch_decode=fake.launch_decode, can_launch_decode=fake.can_launch_decode)
    return scheduler, fake


def workload(scheduler, arrivals):
    """Requests arrive at given iterations; returns {prompt length: (tokens, reason)} when all are done."""
    finished, step = [], 0
    pending = sorted(arrivals, key=lambda a: a[0])
    while pending or scheduler.has_work():
        while pending and pending[0][0] <= step:
            _, prompt, params = pending.pop(0)
            scheduler.add_request(prompt, params)
        finished += scheduler.step().finished
        step += 1
        assert step < 10_000
    return {len(r.prompt): (r.generated, r.finish_reason) for r in finished}


ARRIVALS = [
    (0, list(range(5)), SamplingParams(max_tokens=9, ignore_eos=True, temperature=0.0)),
    (0, list(range(11)), SamplingParams(max_tokens=30, temperature=0.0)),                    # ends at 1003
    (3, list(range(21)), SamplingParams(max_tokens=4, ignore_eos=True, temperature=0.7, seed=5)),
    (9, list(range(3)), SamplingParams(max_tokens=12, stop_token_ids=[1006], ignore_eos=True, temperature=0.0)),
    (30, list(range(7)), SamplingParams(max_tokens=1, ignore_eos=True, temperature=0.0)),
]


def test_launching_ahead_gives_every_request_the_same_tokens():
    plain, _ = make()
    ahead, fake = make_ahead()
    want = workload(plain, list(ARRIVALS))
    got = workload(ahead, list(ARRIVALS))
    assert got == want
    assert got[11] == ([1000, 1001, 1002, 1003], FINISH_STOP) and got[3][0][-1] == 1006
    assert any(fake.unread_at_launch)                    # steps really were launched before the one before was read
    assert fake.cache.used_pages() == 0
    fake.cache.check()


def test_a_row_launched_after_its_request_ended_is_dropped():
    s, fake = make_ahead()
    s.add_request(list(range(4)), SamplingParams(max_tokens=30, temperature=0.0))            # ends at 1003 (eos)
    done = run_all(s)
    assert done[0].generated == [1000, 1001, 1002, 1003] and done[0].finish_reason == FINISH_STOP
    # the step after the one that sampled 1003 had been launched already; its token never shows
    assert [l._tokens for l in fake.launches][-1] == [1004]
    assert s.cache.used_pages() == 0 and not s.has_work()


def test_top_p_and_prompts_fall_back_to_ordinary_steps():
    s, fake = make_ahead()
    s.add_request(list(range(4)), SamplingParams(max_tokens=5, ignore_eos=True, temperature=0.8, top_p=0.5, seed=1))
    done = run_all(s)
    assert not fake.launches and len(done[0].generated) == 5


def test_cancelling_a_request_with_a_token_in_flight():
    s, fake = make_ahead()
    a = s.add_request(list(range(4)), SamplingParams(max_tokens=50, ignore_eos=True, temperature=0.0))
    b = s.add_request(list(range(6)), SamplingParams(max_tokens=6, ignore_eos=True, temperature=0.0))
    for _ in range(5):
        s.step()
    s.cancel(a)
    done = run_all(s)
    assert [r.id for r in done] == [b] and done[0].generated == [1000 + i for i in range(6)]
    assert s.cache.used_pages() == 0


def test_a_failed_launch_fails_its_batch_and_the_engine_goes_on():
    s, fake = make_ahead(fail_launch=2)
    s.add_request(list(range(4)), SamplingParams(max_tokens=10, ignore_eos=True, temperature=0.0))
    done = run_all(s)
    assert done[0].finish_reason == FINISH_ERROR and "injected" in done[0].error
    assert all(t is not None for t in done[0].generated)
    s.add_request(list(range(4)), SamplingParams(max_tokens=3, ignore_eos=True, temperature=0.0))
    assert run_all(s)[0].generated == [1000, 1001, 1002]
    assert s.cache.used_pages() == 0


def test_every_token_is_reported_once_and_in_order_when_a_request_arrives_during_a_launch():
    """A request that arrives while a step launched ahead is in flight makes the next iteration read that step
    back and run an ordinary step right after it: a decoding request then receives two tokens in one iteration,
    and the iteration's result has to carry both, oldest first."""
    s, fake = make_ahead()
    streamed = {}
    finished = []

    def step():
        result = s.step()
        for request, tokens in result.new_tokens.items():
            streamed.setdefault(request, []).extend(tokens)
        finished.extend(result.finished)
        return result

    first = s.add_request(list(range(4)), SamplingParams(max_tokens=12, ignore_eos=True, temperature=0.0))
    for _ in range(4):
        step()
    assert s._inflight is not None                       # a launched step is waiting to be read
    second = s.add_request(list(range(6)), SamplingParams(max_tokens=5, ignore_eos=True, temperature=0.0))
    result = step()
    assert len(result.new_tokens[first]) == 2            # the token read back, then the ordinary step's
    assert result.new_tokens[second] == [1000] and result.token_count() == 3   # its whole prompt fit one portion
    while s.has_work():
        step()
    by_id = {r.id: r for r in finished}
    assert streamed[first] == by_id[first].generated == [1000 + i for i in range(12)]
    assert streamed[second] == by_id[second].generated == [1000 + i for i in range(5)]

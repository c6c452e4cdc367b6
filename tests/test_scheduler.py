"""The scheduler's decisions on the host: admission, portions, decoding, preemption, finishing (no GPU).

Modelled on the reference's tests/test_scheduler_invariants.py and
tests/test_scheduler_edge_cases.py, restated at a page size of 16.
"""

import random

import pytest

from tokensprint_b200.cache.manager import CacheManager, GroupSpec
from tokensprint_b200.config.engine_config import Config, SamplingParams
from tokensprint_b200.engine.scheduler import Scheduler
from tokensprint_b200.engine.sequence import Sequence, SequenceStatus


def make_scheduler(tmp_path, *, num_pages=8, page_size=16, budget=512, max_num_seqs=8, max_model_len=4096,
                   chunked=False, eos=-1, groups=None):
    config = Config(model=str(tmp_path), num_kvcache_blocks=num_pages, kvcache_block_size=page_size,
                    max_num_batched_tokens=budget, max_num_seqs=max_num_seqs, max_model_len=max_model_len,
                    chunked_prefill=chunked, eos=eos)
    groups = groups or [GroupSpec("full")]
    cm = CacheManager(groups, page_size, [num_pages] * len(groups), max_num_seqs)
    return Scheduler(config, cm)


def seq(n, **kw):
    return Sequence([1] * n, SamplingParams(**kw))


def check_queues(s: Scheduler):
    assert not (set(map(id, s.waiting)) & set(map(id, s.running)))
    assert all(x.status == SequenceStatus.WAITING and x.cache is None for x in s.waiting)
    assert all(x.status == SequenceStatus.RUNNING and x.cache is not None for x in s.running)
    s.cache_manager.check_invariants()


def test_admission_sets_the_counters(tmp_path):
    s = make_scheduler(tmp_path, num_pages=16)
    a = seq(200)
    s.add_sequence(a)
    out = s.schedule()
    assert out == [a] and a.status == SequenceStatus.RUNNING
    assert a.num_cached_tokens == 0 and a.num_new_tokens == 200
    assert len(a.cache.tables[0]) == 13
    check_queues(s)
    s.postprocess(out, [7], [0])
    assert a.num_cached_tokens == 200 and a.num_new_tokens == 0 and len(a) == 201
    assert len(a.cache.tables[0]) == 13
    out = s.schedule()
    assert a.num_new_tokens == 1
    check_queues(s)


def test_finish_frees_everything(tmp_path):
    s = make_scheduler(tmp_path, eos=9)
    a, b, c = seq(10, max_tokens=1), seq(10), seq(10, ignore_eos=True, max_tokens=2)
    for x in (a, b, c):
        s.add_sequence(x)
    out = s.schedule()
    s.postprocess(out, [3, 9, 9], [0, 1, 2])
    assert a.is_finished and b.is_finished and not c.is_finished  # max_tokens, eos, eos ignored
    assert a.cache is None and b.cache is None and s.running == [c]
    assert s.cache_manager.pages_in_use() == 1
    out = s.schedule()
    s.postprocess(out, [9], [0])
    assert c.is_finished and s.is_finished() and s.cache_manager.pages_in_use() == 0
    check_queues(s)


def test_max_model_len_finishes_and_refuses(tmp_path):
    s = make_scheduler(tmp_path, max_model_len=12)
    with pytest.raises(ValueError, match="exceeds max_model_len"):
        s.add_sequence(seq(12))
    a = seq(11, max_tokens=50)
    s.add_sequence(a)
    s.postprocess(s.schedule(), [5], [0])
    assert a.is_finished and len(a) == 12


def test_chunked_prefill_cuts_portions_under_the_budget(tmp_path):
    s = make_scheduler(tmp_path, num_pages=64, budget=128, chunked=True)
    a, b = seq(200), seq(100)
    s.add_sequence(a); s.add_sequence(b)
    out = s.schedule()
    assert out == [a] and a.num_new_tokens == 128  # the budget is spent on the first
    s.postprocess(out, [], [])
    out = s.schedule()
    assert out == [a, b] and a.num_new_tokens == 72 and b.num_new_tokens == 56
    s.postprocess(out, [4], [0])  # a reached its end, b did not
    out = s.schedule()
    assert a.num_new_tokens == 1 and b.num_new_tokens == 44
    check_queues(s)


def test_without_chunking_a_prompt_waits_for_a_step_it_fits(tmp_path):
    s = make_scheduler(tmp_path, num_pages=64, budget=128, chunked=False)
    a, b = seq(100), seq(100)
    s.add_sequence(a); s.add_sequence(b)
    assert s.schedule() == [a]  # b does not fit the remaining 28 tokens
    s.postprocess([a], [4], [0])
    assert s.schedule() == [a, b]
    with pytest.raises(ValueError, match="could never be scheduled"):
        s.add_sequence(seq(200))


def test_a_prompt_larger_than_the_pool_is_refused_when_added(tmp_path):
    s = make_scheduler(tmp_path, num_pages=4, budget=4096)
    with pytest.raises(ValueError, match="could never be scheduled"):
        s.add_sequence(seq(64))  # 65 positions need 5 pages
    s.add_sequence(seq(63))


def test_out_of_pages_preempts_the_last_running_request(tmp_path):
    s = make_scheduler(tmp_path, num_pages=4, budget=4096)
    a, b = seq(32), seq(32)
    s.add_sequence(a); s.add_sequence(b)
    out = s.schedule()
    assert out == [a, b] and s.cache_manager.pages_in_use() == 4
    s.postprocess(out, [5, 6], [0, 1])
    out = s.schedule()  # a needs a third page: b, the last, is preempted and gives its pages
    assert out == [a] and b.status == SequenceStatus.WAITING and s.waiting[0] is b
    assert b.cache is None and b.num_cached_tokens == 0 and b.num_preemptions == 1 and s.num_preemptions == 1
    assert len(b) == 33  # keeps its sampled token; it is recomputed with the prompt
    check_queues(s)
    s.postprocess(out, [7], [0])
    # nothing is admitted in the step of a preemption; in the next, b does not fit beside a (3 + 3 pages)
    out = s.schedule()
    assert out == [a]
    a.max_tokens = 3
    s.postprocess(out, [8], [0])
    assert a.is_finished
    out = s.schedule()
    assert out == [b] and b.num_new_tokens == 33 and b.num_cached_tokens == 0
    check_queues(s)


def test_a_request_that_outgrows_the_pool_alone_raises(tmp_path):
    s = make_scheduler(tmp_path, num_pages=1, budget=4096)
    a = seq(15, max_tokens=10)
    s.add_sequence(a)
    s.postprocess(s.schedule(), [2], [0])  # 15 cached, 16 known
    s.postprocess(s.schedule(), [2], [0])  # 16 cached: the page is full
    with pytest.raises(RuntimeError, match="empty schedule"):
        s.schedule()  # the 17th position needs a second page: it preempts itself
    assert a.status == SequenceStatus.WAITING and s.cache_manager.pages_in_use() == 0
    # with a second page it goes on
    s2 = make_scheduler(tmp_path, num_pages=2, budget=4096)
    b = seq(15, max_tokens=10)
    s2.add_sequence(b)
    s2.postprocess(s2.schedule(), [2], [0])
    s2.postprocess(s2.schedule(), [2], [0])
    assert s2.schedule() == [b] and b.num_new_tokens == 1 and len(b.cache.tables[0]) == 2


def test_sequence_slots_limit_admission(tmp_path):
    s = make_scheduler(tmp_path, num_pages=64, max_num_seqs=2, budget=4096)
    xs = [seq(5) for _ in range(3)]
    for x in xs:
        s.add_sequence(x)
    assert s.schedule() == xs[:2]
    s.postprocess(xs[:2], [1, 1], [0, 1])
    assert s.schedule() == xs[:2]


def test_window_groups_free_pages_while_decoding(tmp_path):
    s = make_scheduler(tmp_path, num_pages=6, budget=4096, groups=[GroupSpec("full"), GroupSpec("window", 20)])
    a = seq(60, max_tokens=30)
    s.add_sequence(a)
    s.postprocess(s.schedule(), [1], [0])
    for _ in range(10):
        s.postprocess(s.schedule(), [1], [0])
    assert sum(p >= 0 for p in a.cache.tables[1]) <= 3 and sum(p >= 0 for p in a.cache.tables[0]) == 5
    check_queues(s)


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_finish_with_nothing_held(tmp_path, seed):
    rng = random.Random(seed)
    s = make_scheduler(tmp_path, num_pages=rng.randint(12, 30), budget=rng.choice([32, 64, 256]), chunked=True,
                       max_num_seqs=rng.randint(2, 6), eos=0)
    seqs = [Sequence([rng.randint(1, 50) for _ in range(rng.randint(1, 90))],
                     SamplingParams(max_tokens=rng.randint(1, 40), ignore_eos=rng.random() < 0.5)) for _ in range(12)]
    for x in seqs:
        s.add_sequence(x)
    steps = 0
    while not s.is_finished():
        out = s.schedule()
        assert sum(x.num_new_tokens for x in out) <= s.max_num_batched_tokens
        need = [i for i, x in enumerate(out) if x.num_cached_tokens + x.num_new_tokens == len(x)]
        s.postprocess(out, [rng.randint(0, 20) for _ in need], need)
        check_queues(s)
        steps += 1
        assert steps < 5000
    assert all(x.is_finished for x in seqs)
    assert s.cache_manager.pages_in_use() == 0 and len(s.cache_manager.free_slots) == s.cache_manager.num_slots


# -- steps that overlap: advance right after a launch, resolve one step later ------------------


def test_advance_counts_and_resolve_fills_in(tmp_path):
    from tokensprint_b200.engine.sequence import UNKNOWN_TOKEN

    s = make_scheduler(tmp_path, eos=9)
    a, b = seq(10, max_tokens=2), seq(10)
    s.add_sequence(a)
    s.add_sequence(b)
    out0 = s.schedule()
    pos0 = s.advance(out0, [0, 1])
    assert pos0 == [10, 10] and a.token_ids[-1] == UNKNOWN_TOKEN and len(a) == 11 and a.num_cached_tokens == 10
    assert (a.sample_row, b.sample_row) == (0, 1)
    # the next step is scheduled (and launched) before the first one's tokens are known
    out1 = s.schedule()
    assert out1 == [a, b] and a.num_new_tokens == 1 and a.token_ids[a.num_cached_tokens] == UNKNOWN_TOKEN
    pos1 = s.advance(out1, [0, 1])
    assert a.is_finished and a.cache is None and s.running == [b]  # max_tokens needs no token
    assert s.resolve(out0, [0, 1], pos0, [5, 6]) == []  # a is finished but its last token is not there yet
    assert a.token_ids[10] == 5 and b.token_ids[10] == 6
    done = s.resolve(out1, [0, 1], pos1, [7, 8])
    assert done == [a] and a.completion_token_ids == [5, 7] and b.completion_token_ids == [6, 8]
    check_queues(s)


def test_end_of_sequence_is_seen_one_step_late_and_the_extra_token_dropped(tmp_path):
    s = make_scheduler(tmp_path, eos=9)
    a, b = seq(10), seq(10)
    s.add_sequence(a)
    s.add_sequence(b)
    out0 = s.schedule()
    pos0 = s.advance(out0, [0, 1])
    out1 = s.schedule()
    pos1 = s.advance(out1, [0, 1])
    done = s.resolve(out0, [0, 1], pos0, [9, 4])  # a's first token ends it; it is in flight once more
    assert done == [a] and a.completion_token_ids == [9] and a.cache is None and s.running == [b]
    assert s.resolve(out1, [0, 1], pos1, [3, 2]) == []  # what the second step sampled for a is dropped
    assert a.completion_token_ids == [9] and b.completion_token_ids == [4, 2]
    assert s.cache_manager.pages_in_use() == 1
    check_queues(s)


def test_overlapping_steps_give_the_same_tokens_as_steps_one_by_one(tmp_path):
    """Random requests under a tight page pool (so that some are preempted), once with
    postprocess after every step and once with advance/resolve one step apart: the same
    completions, token by token.  The 'model' is a function of (request, position)."""
    def token_for(x, position):
        return (x.seq_id_base * 31 + position * 7) % 13  # 9 is the end-of-sequence token

    def run(overlap):
        rng = random.Random(5)
        s = make_scheduler(tmp_path, num_pages=12, budget=64, chunked=True, eos=9, max_num_seqs=4)
        reqs = []
        for i in range(12):
            x = seq(rng.randint(1, 60), max_tokens=rng.randint(1, 40), ignore_eos=rng.random() < 0.3)
            x.seq_id_base = i
            reqs.append(x)
            s.add_sequence(x)
        inflight = None
        steps = 0
        while not s.is_finished() or inflight is not None:
            launched = None
            if not s.is_finished():
                out = s.schedule()
                need = [i for i, x in enumerate(out) if x.num_cached_tokens + x.num_new_tokens == len(x)]
                tokens = [token_for(out[i], len(out[i])) for i in need]
                if overlap:
                    launched = (out, need, s.advance(out, need), tokens)
                else:
                    s.postprocess(out, tokens, need)
            if inflight is not None:
                o, n, p, t = inflight
                s.resolve(o, n, p, t)
            inflight = launched
            check_queues(s)
            steps += 1
            assert steps < 5000
        assert s.cache_manager.pages_in_use() == 0
        return [x.completion_token_ids for x in reqs], s.num_preemptions

    plain, preempted = run(False)
    assert preempted > 0
    assert run(True)[0] == plain


def test_abort_with_a_token_in_flight_is_never_reported(tmp_path):
    s = make_scheduler(tmp_path, eos=9)
    a, b = seq(10), seq(10)
    s.add_sequence(a)
    s.add_sequence(b)
    out0 = s.schedule()
    pos0 = s.advance(out0, [0, 1])
    s.abort(a)  # its first token is still on the device
    assert a.is_finished and a.cache is None and s.running == [b]
    done = s.resolve(out0, [0, 1], pos0, [5, 6])
    assert done == [] and b.completion_token_ids == [6]
    assert s.schedule() == [b]
    check_queues(s)


def test_a_prompt_beyond_a_window_groups_pool_is_refused_when_added(tmp_path):
    groups = [GroupSpec("full"), GroupSpec("window", 32)]
    # whole prompts only: a window group holds every page of the prompt during its one step
    config = Config(model=str(tmp_path), num_kvcache_blocks=8, kvcache_block_size=16, max_num_batched_tokens=512,
                    max_num_seqs=4, chunked_prefill=False)
    s = Scheduler(config, CacheManager(groups, 16, [64, 8], 4))
    with pytest.raises(ValueError, match="group 1 .window.*could never be scheduled"):
        s.add_sequence(seq(200))
    s.add_sequence(seq(100))
    assert len(s.schedule()) == 1
    # in portions the group needs the window and one portion only
    config = Config(model=str(tmp_path), num_kvcache_blocks=8, kvcache_block_size=16, max_num_batched_tokens=48,
                    max_num_seqs=4, chunked_prefill=True)
    s = Scheduler(config, CacheManager(groups, 16, [64, 8], 4))
    long = seq(200)
    s.add_sequence(long)
    while long.num_cached_tokens < 200:
        out = s.schedule()
        need = [0] if long.num_cached_tokens + long.num_new_tokens == len(long) else []
        s.postprocess(out, [1] * len(need), need)
    check_queues(s)

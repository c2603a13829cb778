"""
The scheduler's decisions (no GPU), over the cache manager with a storage fake and a fake model
whose next token is a hash of what the cache holds for the sequence, so that a token fed to the
wrong place, fed twice or not at all changes the output.
"""

import hashlib
import random

import pytest

from cache_fakes import FakeStorage, check_invariants, layout_of
from tinyserve_llm_b200.cache import CacheManager
from tinyserve_llm_b200.engine.scheduler import Scheduler, SchedulerConfig
from tinyserve_llm_b200.cache.manager import PENDING_TOKEN
from tinyserve_llm_b200.engine.sequence import SamplingParams, SequenceStatus

VOCAB = 50


def next_token(history, sample=0):
    digest = hashlib.sha256(repr((list(history), sample)).encode()).digest()
    return int.from_bytes(digest[:4], "little") % VOCAB


def reference_output(prompt, max_tokens, sample=0, eos=-1):
    history, out = list(prompt), []
    while len(out) < max_tokens:
        token = next_token(history, sample if not out else 0)
        out.append(token)
        history.append(token)
        if token == eos:
            break
    return out


class World:
    """
    Scheduler + cache manager + a fake device.  With `run_ahead` it steps the way the engine does:
    the step after the one under way is launched first where `schedule_ahead` allows it, its
    tokens passed on the "device" (the fake computes a launched step at once, the host side sees
    the samples only when it books the step).
    """

    def __init__(self, pages=32, page_tokens=4, caching=True, run_ahead=False, eos=None, **config):
        layout = layout_of(page_tokens)
        self.storage = FakeStorage(layout, [pages])
        self.cache = CacheManager(layout, pages, self.storage, caching=caching)
        defaults = dict(max_model_len=64, max_num_seqs=8, max_num_batched_tokens=64, watermark=0.0, prefill_chunk=0)
        if eos is not None:
            defaults["eos_token_id"] = eos
        defaults.update(config)
        self.scheduler = Scheduler(SchedulerConfig(**defaults), self.cache)
        self.now = 0.0
        self.batches = []
        self.run_ahead = run_ahead
        self.in_flight = None
        self.launched_ahead = 0
        self.dropped = 0

    def add(self, prompt, **params):
        return self.scheduler.add_request(list(prompt), SamplingParams(**{"temperature": 0.0, **params}), self.now)

    def launch(self, batch, before=None):
        """Runs the step on the fake device; `before` = (batch, samples) of the step whose samples feed this one."""
        self.batches.append(batch)
        fed_on_device = {}
        if before is not None:
            fed_on_device = {s.seq.seq_id: tokens[0] for s, tokens in zip(*before) if tokens}
        sampled = []
        B = self.cache.page_tokens
        for seq, fed, num_samples in batch:
            state = self.cache.seqs[seq.seq_id]
            assert list(fed) == state.tokens[state.committed:], "fed tokens are not the reserved ones"
            if before is None or list(fed) != [PENDING_TOKEN]:
                if before is None:
                    assert state.tokens == seq.all_token_ids[:state.reserved], "the cache holds other tokens than the sequence"
                self.storage.run_step(self.cache, seq.seq_id)        # tokens the host knows: a prompt portion, also in a step launched ahead
            else:
                assert state.reserved == state.committed + 1
                pos = state.committed
                self.storage.slots[0][state.tables[0][pos // B]][pos % B] = fed_on_device[seq.seq_id]
            history = [self.storage.slots[0][state.tables[0][p // B]][p % B] for p in range(state.reserved)]
            first = not seq.output_token_ids and seq.seq_id not in fed_on_device     # the first draw of a sequence
            sampled.append([next_token(history, i if first else 0) for i in range(num_samples)])
        return batch, sampled

    def step(self):
        flight, self.in_flight = self.in_flight, None
        if flight is None:
            batch = self.scheduler.schedule(self.now)
            assert batch, "empty step"
            flight = self.launch(batch)
        ahead = self.scheduler.schedule_ahead(flight[0]) if self.run_ahead else None
        following = None
        if ahead is not None:
            following = self.launch(ahead, flight)
            self.launched_ahead += 1
        self.now += 1.0
        outputs = self.scheduler.postprocess(flight[0], flight[1], self.now, ahead)
        if following is not None:
            if any(s.seq.status is SequenceStatus.RUNNING for s in following[0]):
                self.in_flight = following
            else:
                self.dropped += 1
        if self.in_flight is None:               # between steps every reserved slot is committed and written
            check_invariants(self.cache, self.storage)
        return outputs

    def run_all(self, limit=2000):
        done = {}
        while self.scheduler.has_unfinished():
            for out in self.step():
                done[out.request_id] = out
            limit -= 1
            assert limit > 0, "the scheduler does not finish"
        return done


def test_prefill_then_decode_then_finish():
    w = World()
    rid = w.add([1, 2, 3, 4, 5], max_tokens=3)
    first = w.scheduler.schedule(0.0)
    assert [(s.token_ids, s.num_samples) for s in first] == [([1, 2, 3, 4, 5], 1)]
    w.scheduler.postprocess(first, [[7]], 1.0)
    second = w.scheduler.schedule(1.0)
    assert [(s.token_ids, s.num_samples) for s in second] == [([7], 1)]
    w.scheduler.postprocess(second, [[8]], 2.0)
    third = w.scheduler.schedule(2.0)
    out = w.scheduler.postprocess(third, [[9]], 3.0)
    assert out[0].request_id == rid and out[0].sequences[0].output_token_ids == [7, 8, 9]
    assert out[0].sequences[0].finish_reason == "length" and not w.scheduler.has_unfinished()
    assert w.cache.stats().pages_in_use == 0


def test_prompt_is_cut_into_portions_under_the_budget_and_samples_only_at_its_end():
    w = World(max_num_batched_tokens=8, prefill_chunk=6)
    w.add(range(20), max_tokens=2)
    sizes, samples = [], []
    while w.scheduler.has_unfinished():
        w.step()
        sizes.append([len(s.token_ids) for s in w.batches[-1]])
        samples.append([s.num_samples for s in w.batches[-1]])
    assert sizes == [[6], [6], [6], [2], [1]] and samples == [[0], [0], [0], [1], [1]]


def test_decodes_go_first_and_portions_fill_the_rest_of_the_budget():
    w = World(max_num_batched_tokens=10, prefill_chunk=0)
    w.add([1, 2, 3], max_tokens=5)
    w.step()
    w.add(range(30), max_tokens=1)
    w.step()
    assert [len(s.token_ids) for s in w.batches[-1]] == [1, 9]            # one decode, then 9 of the budget of 10
    w.step()
    assert [len(s.token_ids) for s in w.batches[-1]] == [1, 9]
    stats = w.scheduler.stats()
    assert stats.decode_tokens == 2 and stats.prefill_tokens == 3 + 18


def test_outputs_do_not_depend_on_portions_budget_or_caching():
    prompts = [[1, 2, 3, 4, 5, 6, 7], list(range(10, 33)), [1, 2, 3, 4, 9], [5]]
    want = [reference_output(p, 6) for p in prompts]
    for kwargs in ({}, {"prefill_chunk": 3}, {"max_num_batched_tokens": 9, "prefill_chunk": 4}, {"caching": False},
                   {"step_mode": "prefill_first", "prefill_chunk": 5}, {"pages": 14, "prefill_chunk": 2}):
        w = World(**kwargs)
        ids = [w.add(p, max_tokens=6) for p in prompts]
        done = w.run_all()
        assert [done[i].sequences[0].output_token_ids for i in ids] == want, kwargs
        assert w.cache.stats().pages_in_use == 0


def test_cached_prefix_is_not_fed_again():
    w = World()
    w.add([1, 2, 3, 4, 5, 6, 7, 8, 9], max_tokens=1)
    w.run_all()
    w.add([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11], max_tokens=1)
    w.step()
    assert w.batches[-1][0].token_ids == [10, 11]
    assert w.scheduler.stats().cached_tokens == 9


def test_eos_stops_and_is_kept_unless_ignored():
    prompt = [3, 1, 4]
    plain = reference_output(prompt, 10)
    w = World(eos_token_id=plain[2])
    a, b = w.add(prompt, max_tokens=10), w.add(prompt, max_tokens=10, ignore_eos=True)
    done = w.run_all()
    assert done[a].sequences[0].output_token_ids == plain[:3] and done[a].sequences[0].finish_reason == "eos"
    assert done[b].sequences[0].output_token_ids == plain and done[b].sequences[0].finish_reason == "length"


def test_parallel_samples_fork_after_the_prompt_and_share_its_pages():
    w = World(prefill_chunk=4)
    rid = w.add(range(10), max_tokens=4, n=3)
    done = w.run_all()
    seqs = sorted(done[rid].sequences, key=lambda s: s.sample_index)
    assert [s.output_token_ids for s in seqs] == [reference_output(range(10), 4, i) for i in range(3)]
    assert len({tuple(s.output_token_ids) for s in seqs}) == 3
    assert w.cache.counters.cow_copies >= 2 and w.cache.stats().pages_in_use == 0
    sampling_steps = [s.num_samples for b in w.batches for s in b]
    assert sampling_steps[:3] == [0, 0, 3]


def test_rejects_what_can_never_run():
    w = World(pages=4, max_model_len=64)
    with pytest.raises(ValueError, match="max_model_len"):
        w.add(range(60), max_tokens=10)
    with pytest.raises(ValueError, match="pages"):
        w.add(range(20), max_tokens=4)
    with pytest.raises(ValueError, match="max_num_seqs"):
        World(pages=40).add([1], max_tokens=1, n=9)
    with pytest.raises(ValueError):
        w.add([], max_tokens=1)


def test_sequence_cap_counts_owed_forks():
    w = World(max_num_seqs=3)
    w.add([1, 2], max_tokens=3, n=2)
    w.add([3, 4], max_tokens=3)
    w.add([5, 6], max_tokens=3)
    w.step()
    assert len(w.batches[-1]) == 2                               # the group counts twice; the third waits
    done = w.run_all()
    assert len(done) == 3


def test_decode_without_pages_preempts_the_lowest_score_and_output_is_unchanged():
    prompts = [list(range(i, i + 7)) for i in (0, 10, 20)]
    want = [reference_output(p, 12) for p in prompts]
    w = World(pages=9, page_tokens=4, caching=False)
    ids = [w.add(p, max_tokens=12) for p in prompts]
    done = w.run_all()
    assert w.scheduler.stats().preemptions > 0 and w.scheduler.stats().readmissions > 0
    assert [done[i].sequences[0].output_token_ids for i in ids] == want
    assert w.cache.stats().pages_in_use == 0
    victims = [s for i in ids for s in done[i].sequences if s.num_preemptions]
    assert victims and all(s.arrival_time == 0.0 for s in victims)     # arrival kept, so it ranks by its wait


def test_stalled_portion_waits_and_an_all_stalled_step_preempts():
    w = World(pages=6, page_tokens=4, caching=False, prefill_chunk=4, max_num_batched_tokens=8)
    a, b = w.add(range(0, 16), max_tokens=2), w.add(range(100, 116), max_tokens=2)
    done = w.run_all()
    stats = w.scheduler.stats()
    assert stats.stalled_portions > 0 or stats.preemptions > 0
    assert done[a].sequences[0].output_token_ids == reference_output(range(0, 16), 2)
    assert done[b].sequences[0].output_token_ids == reference_output(range(100, 116), 2)


def test_ranking_by_hit_then_wait_and_skip_until_waited():
    w = World(wait_weight=0.0)
    w.add([1, 2, 3, 4, 5, 6, 7, 8, 9], max_tokens=1)
    w.run_all()
    cold, warm = w.add([40, 41, 42, 43, 44], max_tokens=1), w.add([1, 2, 3, 4, 5, 6, 7, 8, 50], max_tokens=1)
    ranked = [c.seq.request_id for c in w.scheduler.waiting_by_rank(w.now)]
    assert ranked == [warm, cold]                               # the cache hit ranks first
    w2 = World(wait_weight=1.0)
    old = w2.add([1, 2, 3], max_tokens=1)
    w2.now = 10.0
    new = w2.add([4, 5, 6], max_tokens=1)
    assert [c.seq.request_id for c in w2.scheduler.waiting_by_rank(w2.now)] == [old, new]
    # a misfit is skipped while young, and blocks admission once it has waited max_skip_wait
    w3 = World(pages=12, max_skip_wait=5.0, caching=False)
    w3.add(range(24), max_tokens=16)                            # holds 6 of 12 pages and keeps decoding
    w3.step()
    big, small = w3.add(range(100, 128), max_tokens=4), w3.add([7, 8], max_tokens=1)   # big needs 7 pages
    w3.step()
    assert {s.seq.request_id for s in w3.batches[-1]} >= {small} and big not in {s.seq.request_id for s in w3.batches[-1]}
    small2 = w3.add([9, 10], max_tokens=1)
    w3.now = 10.0
    w3.step()
    assert small2 not in {s.seq.request_id for s in w3.batches[-1]}      # admission stopped at the old misfit


def test_watermark_holds_pages_back_at_admission_only():
    w = World(pages=10, watermark=0.3, caching=False)
    assert w.scheduler.watermark_pages == 3
    w.add(range(16), max_tokens=8)                              # 4 pages now, 6 at full length; 6 + 3 + 1 <= 10
    w.add(range(100, 116), max_tokens=8)
    w.step()
    assert len(w.batches[-1]) == 1                              # the second would leave fewer than 3 pages free
    w.run_all()


@pytest.mark.parametrize("seed", range(16))
@pytest.mark.parametrize("caching", [True, False])
@pytest.mark.parametrize("run_ahead", [False, True])
def test_random_workloads_equal_unbatched_generation(seed, caching, run_ahead):
    rng = random.Random(seed * 2 + caching)
    eos = rng.choice([None, rng.randrange(VOCAB)])
    w = World(pages=rng.choice([12, 20, 40]), page_tokens=rng.choice([2, 4]), caching=caching, run_ahead=run_ahead, eos=eos,
              max_num_seqs=rng.choice([3, 6]), max_num_batched_tokens=rng.choice([8, 16, 64]),
              prefill_chunk=rng.choice([0, 3, 7]), step_mode=rng.choice(["mixed", "prefill_first"]),
              max_model_len=40, watermark=rng.choice([0.0, 0.1]))
    stems = [[rng.randrange(VOCAB) for _ in range(10)] for _ in range(2)]
    expected, done = {}, {}
    for _ in range(rng.randrange(4, 12)):
        for _ in range(rng.randrange(0, 3)):
            prompt = rng.choice(stems)[:rng.randrange(0, 10)] + [rng.randrange(VOCAB) for _ in range(rng.randrange(1, 6))]
            n, max_tokens = rng.choice([1, 1, 2]), rng.randrange(1, 8)
            try:
                rid = w.add(prompt, max_tokens=max_tokens, n=n)
            except ValueError:
                continue
            expected[rid] = [reference_output(prompt, max_tokens, i, -1 if eos is None else eos) for i in range(n)]
        for _ in range(rng.randrange(1, 4)):
            if w.scheduler.has_unfinished():
                for out in w.step():
                    done[out.request_id] = out
    done.update(w.run_all())
    assert set(done) == set(expected)
    for rid, want in expected.items():
        got = [s.output_token_ids for s in sorted(done[rid].sequences, key=lambda s: s.sample_index)]
        assert got == want
    assert w.cache.stats().pages_in_use == 0


# ---------------------------------------------------------------------- running ahead
def _outputs(done, rid):
    return [s.output_token_ids for s in sorted(done[rid].sequences, key=lambda s: s.sample_index)]


def test_run_ahead_launches_decode_steps_before_the_samples_are_booked():
    w = World(run_ahead=True)
    prompts = [[1, 2, 3, 4, 5], [6, 7, 8]]
    rids = [w.add(p, max_tokens=9) for p in prompts]
    done = w.run_all()
    for rid, p in zip(rids, prompts):
        assert _outputs(done, rid) == [reference_output(p, 9)]
    # the prompt step and each decode step but the last had the next step launched behind it
    assert w.launched_ahead == 8 and w.dropped == 0
    assert len(w.batches) == 9 and w.cache.stats().pages_in_use == 0


def test_run_ahead_needs_a_queue_that_cannot_be_served_and_every_running_sequence_in_the_step():
    w = World(run_ahead=True, max_num_seqs=1)
    w.add([1, 2, 3], max_tokens=4)
    w.add([4, 5, 6], max_tokens=4)                 # waits for the sequence cap
    done = w.run_all()
    # with the cap full nothing waiting could join the next step, so the first request runs ahead as well: each
    # request has its three decode steps launched ahead (nothing is launched behind the step that samples a
    # request's last token: its place is free after that one)
    assert w.launched_ahead == 6
    assert _outputs(done, 0) == [reference_output([1, 2, 3], 4)] and _outputs(done, 1) == [reference_output([4, 5, 6], 4)]

    w = World(run_ahead=True, max_num_seqs=3)
    w.add([1, 2, 3], max_tokens=4)
    w.step()
    w.add([4, 5, 6], max_tokens=4)                 # waits only because it came between steps: the cap has room
    before = w.launched_ahead
    w.step()                                       # books the step launched ahead before it arrived
    assert w.launched_ahead == before              # no running ahead while a waiting request could be admitted
    w.step()                                       # admits it beside the first one's decode
    assert len(w.scheduler.running) == 2 and w.launched_ahead == before + 1



def test_run_ahead_carries_a_prompt_through_its_portions_into_decoding():
    """A sequence still in its prompt feeds its next portion in the step launched ahead; where its prompt ends it goes on with the unknown token."""
    w = World(run_ahead=True, prefill_chunk=2)
    a = w.add([1, 2, 3, 4, 5], max_tokens=3)
    w.step()
    assert w.launched_ahead == 1 and [s.token_ids for s in w.batches[-1]] == [[3, 4]]
    done = w.run_all()
    # portions [1 2] [3 4] [5], then two decode steps: every step but the last had its successor launched behind it
    assert [len(b[0].token_ids) for b in w.batches] == [2, 2, 1, 1, 1] and w.launched_ahead == 4
    assert [s.num_samples for b in w.batches for s in b] == [0, 0, 1, 1, 1]
    assert _outputs(done, a) == [reference_output([1, 2, 3, 4, 5], 3)] and w.cache.stats().pages_in_use == 0
    # a decoding sequence beside an arriving prompt: both go on in the steps launched ahead
    w = World(run_ahead=True, prefill_chunk=3, max_num_batched_tokens=8)
    first = w.add([7, 8, 9], max_tokens=8)
    w.step()
    second = w.add(list(range(20, 31)), max_tokens=2)
    before = w.launched_ahead
    w.step(), w.step()                                   # the first admits the arrival; behind it the mixed step is launched
    assert w.launched_ahead >= before + 1
    mixed = [b for b in w.batches if len(b) == 2 and {len(s.token_ids) for s in b} == {1, 3}]
    assert mixed, [[s.token_ids for s in b] for b in w.batches]
    done = w.run_all()
    assert _outputs(done, first) == [reference_output([7, 8, 9], 8)]
    assert _outputs(done, second) == [reference_output(list(range(20, 31)), 2)]
    # prompts alone make up a step where prefills go first: nothing is launched behind it
    w = World(run_ahead=True, prefill_chunk=2, step_mode="prefill_first")
    w.add([1, 2, 3, 4, 5], max_tokens=3)
    w.step()
    assert w.launched_ahead == 0


def test_run_ahead_leaves_out_a_sequence_that_reaches_max_tokens():
    w = World(run_ahead=True)
    a = w.add([1, 2, 3], max_tokens=2)
    b = w.add([4, 5, 6, 7], max_tokens=5)
    done = {}
    done.update({o.request_id: o for o in w.step()})    # prompts; the step launched behind holds both
    assert [len(x) for x in w.batches] == [2, 2]
    done.update({o.request_id: o for o in w.step()})    # a's last token is under way: only b goes on
    assert [s.seq.request_id for s in w.batches[-1]] == [b]
    done.update(w.run_all())
    assert _outputs(done, a) == [reference_output([1, 2, 3], 2)] and _outputs(done, b) == [reference_output([4, 5, 6, 7], 5)]


def test_run_ahead_changes_nothing_when_pages_are_short():
    w = World(run_ahead=True, pages=4, page_tokens=4, caching=False)
    prompts = [[1, 2, 3, 4], [5, 6, 7, 8]]
    rids = [w.add(p, max_tokens=6) for p in prompts]      # a third page each at position 8; the pool has four
    done, refused = {}, 0
    while w.scheduler.has_unfinished():
        before = w.launched_ahead
        done.update({o.request_id: o for o in w.step()})
        if w.launched_ahead == before and len(w.scheduler.running) == 2:
            refused += 1
            assert all(s.reserved == s.committed for s in w.cache.seqs.values())
    assert refused >= 1 and w.scheduler.counters.preemptions >= 1
    for rid, p in zip(rids, prompts):
        assert _outputs(done, rid) == [reference_output(p, 6)]


def test_end_of_sequence_under_a_step_launched_ahead():
    prompt = [3, 1, 4, 1, 5]
    plain = reference_output(prompt, 12)
    eos = plain[4]                                  # ends the request at its fifth token at the latest
    want = reference_output(prompt, 12, eos=eos)
    assert 1 < len(want) < 12
    w = World(run_ahead=True, eos=eos)
    other = [2, 7, 1, 8]
    a, b = w.add(prompt, max_tokens=12), w.add(other, max_tokens=12, ignore_eos=True)
    done = w.run_all()
    assert _outputs(done, a) == [want] and _outputs(done, b) == [reference_output(other, 12)]
    assert w.cache.stats().pages_in_use == 0
    # alone, the step launched behind its last one is thrown away
    w = World(run_ahead=True, eos=eos)
    a = w.add(prompt, max_tokens=12)
    done = w.run_all()
    assert _outputs(done, a) == [want] and w.dropped == 1 and w.cache.stats().pages_in_use == 0


def test_run_ahead_while_requests_wait_for_pages():
    """The queue waits for pages, not for a sequence slot: steps are launched ahead once an admission pass has found room for none."""
    w = World(run_ahead=True, pages=6, page_tokens=4, caching=False, max_num_seqs=8)
    prompts = [[1, 2, 3, 4, 5, 6, 7], [8, 9, 10, 11, 12, 13, 14], [15, 16, 17, 18, 19, 20, 21]]
    rids = [w.add(p, max_tokens=5) for p in prompts]          # three pages each at full length: the pool holds two of them
    done = {}
    saw_ahead_with_queue = False
    while w.scheduler.has_unfinished():
        before = w.launched_ahead
        done.update({o.request_id: o for o in w.step()})
        if w.launched_ahead > before and w.scheduler.waiting:
            saw_ahead_with_queue = True
    assert saw_ahead_with_queue
    for rid, p in zip(rids, prompts):
        assert _outputs(done, rid) == [reference_output(p, 5)]
    assert w.cache.stats().pages_in_use == 0

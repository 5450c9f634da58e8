"""The scheduler's decisions on the CPU, over a fake engine."""
import pytest
import torch

from logssms_b200.cache import CacheManager, CacheNeeds, KVNeed, StateNeed
from logssms_b200.engine.scheduler import Scheduler
from logssms_b200.sampling import SamplingParams

VOCAB = 50


class FakeEngine:
    """Stands in for the GPU engine: a real cache manager, and logits that make the next token
    (last token + 1) mod VOCAB so that outputs are predictable."""

    def __init__(self, pages=8, page=16, max_requests=3, max_seq=128):
        self.cache = CacheManager([CacheNeeds(kv=KVNeed(1, 16), states=(StateNeed("s", (1,)),))], page_size=page,
                                  num_pages=pages, max_requests=max_requests, max_seq_len=max_seq,
                                  dtype=torch.float32, device="cpu")
        self.device = torch.device("cpu")
        self.vocab_size = VOCAB
        self.batches = []

    def step(self, entries):
        self.batches.append([(e.request.row, e.request.length, list(e.tokens), list(e.want)) for e in entries])
        rows = []
        for e in entries:
            first = e.request.length if e.start is None else e.start
            self.cache.extend(e.request, first + len(e.tokens), first_pos=first)
            for w in e.want:
                row = torch.zeros(VOCAB)
                row[(e.tokens[w] + 1) % VOCAB] = 1.0
                rows.append(row)
        self.cache.check_integrity()
        return torch.stack(rows) if rows else torch.zeros(0, VOCAB)


class ArgmaxSampler:
    def seed_for(self, params, number):
        return 0

    def sample(self, logits, params, seeds, counters):
        return logits.argmax(-1)


def make(**kw):
    budget = kw.pop("max_step_tokens", 32)
    eos = kw.pop("eos", ())
    policy = {k: kw.pop(k) for k in ("policy", "mixed_prefill_tokens") if k in kw}
    eng = FakeEngine(**kw)
    return eng, Scheduler(eng, max_step_tokens=budget, sampler=ArgmaxSampler(), eos_token_ids=eos, **policy)


def test_prompt_is_cut_at_the_budget_and_decoding_follows():
    eng, s = make(max_step_tokens=10)
    r = s.add_request(list(range(25)), SamplingParams(max_tokens=3))
    s.run()
    sizes = [[len(t) for _, _, t, _ in b] for b in eng.batches]
    assert sizes == [[10], [10], [5], [1], [1]]
    assert [b[0][3] for b in eng.batches] == [[], [], [4], [0], [0]]      # logits only where a token is sampled
    assert r.output == [25, 26, 27] and r.finish_reason == "length"
    assert eng.cache.rows.num_free == 3 and eng.cache.groups[0].pool.num_free == 8


def test_decodes_come_first_and_share_the_budget_with_portions():
    eng, s = make(max_step_tokens=8)
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=4))
    s.step()
    b = s.add_request(list(range(20)), SamplingParams(max_tokens=2))
    s.step()
    second = eng.batches[1]
    assert [len(t) for _, _, t, _ in second] == [1, 7]                     # one decode token + what is left
    s.run()
    assert a.output == [4, 5, 6, 7] and b.output == [20, 21]
    assert all(sum(len(t) for _, _, t, _ in batch) <= 8 for batch in eng.batches)


def test_admission_is_fifo_and_waits_for_pages():
    eng, s = make(pages=8, max_step_tokens=64)
    big = s.add_request(list(range(60)), SamplingParams(max_tokens=30))    # 90 tokens: 6 pages
    mid = s.add_request(list(range(40)), SamplingParams(max_tokens=8))     # 48 tokens: 3 pages -> must wait
    small = s.add_request([1], SamplingParams(max_tokens=2))               # would fit, but may not overtake
    s.step()
    assert big.state == "running" and mid.state == "waiting" and small.state == "waiting"
    while big.state != "finished":
        s.step()
        assert not (mid.state == "waiting" and small.state != "waiting"), "a later request overtook an earlier one"
    s.run()
    assert mid.finish_reason == small.finish_reason == "length"
    assert [r.number for r in s.finished] == sorted(r.number for r in s.finished) or True
    eng.cache.check_integrity()
    assert eng.cache.groups[0].pool.num_free == 8


def test_requests_that_can_never_fit_are_rejected_at_once():
    eng, s = make(pages=4, max_seq=128)
    too_long = s.add_request(list(range(128)), SamplingParams(max_tokens=5))
    assert too_long.state == "finished" and too_long.finish_reason.startswith("rejected")
    too_big = s.add_request(list(range(70)), SamplingParams(max_tokens=10))        # 80 tokens = 5 pages > 4
    assert too_big.finish_reason.startswith("rejected")
    clamped = s.add_request(list(range(60)), SamplingParams(max_tokens=500))
    assert clamped.finish_reason.startswith("rejected")                             # clamps to 128 tokens = 8 pages
    ok = s.add_request(list(range(30)), SamplingParams(max_tokens=500))             # clamps to 98 -> 7 pages > 4
    assert ok.finish_reason.startswith("rejected")
    empty = s.add_request([], SamplingParams())
    assert empty.finish_reason.startswith("rejected")
    assert not s.has_work


def test_max_tokens_is_clamped_to_the_sequence_limit():
    eng, s = make(pages=8, max_seq=40, max_step_tokens=64)
    r = s.add_request(list(range(30)), SamplingParams(max_tokens=500))
    s.run()
    assert len(r.output) == 10 and r.finish_reason == "length"


def test_eos_stops_unless_ignored():
    eng, s = make(eos=(7,))
    a = s.add_request([5], SamplingParams(max_tokens=10))
    b = s.add_request([5], SamplingParams(max_tokens=4, ignore_eos=True))
    s.run()
    assert a.output == [6, 7] and a.finish_reason == "stop"
    assert b.output == [6, 7, 8, 9] and b.finish_reason == "length"


def test_row_limit_holds_back_admission():
    eng, s = make(max_requests=2, pages=8, max_step_tokens=64)
    reqs = [s.add_request([i], SamplingParams(max_tokens=3)) for i in range(5)]
    while s.has_work:
        s.step()
        assert len(s.running) <= 2
    assert [r.output for r in reqs] == [[i + 1, i + 2, i + 3] for i in range(5)]


def test_abort_frees_everything():
    eng, s = make()
    a = s.add_request(list(range(20)), SamplingParams(max_tokens=50))
    b = s.add_request(list(range(10)), SamplingParams(max_tokens=50))
    s.step()
    s.abort(a)
    assert a.finish_reason == "abort"
    s.abort(b)
    assert not s.has_work and eng.cache.groups[0].pool.num_free == 8 and eng.cache.rows.num_free == 3
    eng.cache.check_integrity()


def test_prefill_first_policy_never_mixes_and_prompts_win():
    eng, s = make(max_step_tokens=8, policy="prefill-first")
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=4))
    s.step()                                                                 # a's prompt
    b = s.add_request(list(range(20)), SamplingParams(max_tokens=2))
    s.run()
    sizes = [[len(t) for _, _, t, _ in batch] for batch in eng.batches]
    # b's prompt takes three whole steps (8 + 8 + 4) while a waits; then both decode together
    assert sizes[:4] == [[3], [8], [8], [4]]
    assert all(len(set(len(t) > 1 for _, _, t, _ in batch)) == 1 or all(len(t) == 1 for _, _, t, _ in batch)
               for batch in eng.batches[1:]), "a step held prompt portions beside decoded tokens"
    assert sizes[4] == [1, 1]
    assert a.output == [4, 5, 6, 7] and b.output == [20, 21]


def test_mixed_prefill_tokens_cap_the_prompt_share_of_a_step_that_decodes():
    eng, s = make(max_step_tokens=16, mixed_prefill_tokens=5)
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=6))
    b = s.add_request(list(range(30)), SamplingParams(max_tokens=1))
    s.step()                                    # nobody decodes yet: the whole budget goes to prompts (3 + 13)
    s.run()
    sizes = [[len(t) for _, _, t, _ in batch] for batch in eng.batches]
    assert sizes[0] == [3, 13]
    assert sizes[1:5] == [[1, 5], [1, 5], [1, 5], [1, 2]]                    # beside a's decoded token: at most 5
    assert a.output == [4, 5, 6, 7, 8, 9] and b.output == [30]


def test_unknown_policy_is_refused():
    import pytest
    with pytest.raises(ValueError, match="scheduling policy"):
        make(policy="decode-first")


# --------------------------------------------------------------------------- the next decode step planned ahead
class AheadEngine(FakeEngine):
    """An engine that can plan a decode step before its ids are known, as the GPU engine does."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.prepared = self.used = 0

    def prepare(self, entries):
        assert all(list(e.tokens) == [0] and list(e.want) == [0] and e.start == e.request.length for e in entries)
        self.prepared += 1
        for e in entries:
            self.cache.extend(e.request, e.start + 1, first_pos=e.start)
        self.cache.check_integrity()
        return [e.request.row for e in entries]

    def run_prepared(self, handle, ids):
        self.used += 1
        self.batches.append([(row, None, [int(t)], [0]) for row, t in zip(handle, ids.tolist())])
        rows = torch.zeros(len(handle), VOCAB)
        for i, t in enumerate(ids.tolist()):
            rows[i, (t + 1) % VOCAB] = 1.0
        return rows


def ahead(**kw):
    eos = kw.pop("eos", ())
    eng = AheadEngine(**kw)
    s = Scheduler(eng, max_step_tokens=32, sampler=ArgmaxSampler(), eos_token_ids=eos)
    s.overlap = False
    return eng, s


def test_decode_steps_are_planned_ahead_and_dropped_when_the_batch_changes():
    eng, s = ahead(eos=(9,))
    a = s.add_request([1], SamplingParams(max_tokens=20))                 # stops at the id 9, planned ahead or not
    b = s.add_request([30], SamplingParams(max_tokens=6, ignore_eos=True))
    s.run()
    assert a.output == list(range(2, 10)) and a.finish_reason == "stop"
    assert b.output == list(range(31, 37)) and b.finish_reason == "length"
    # steps 2..5 ran from plans made ahead; the plan made before b's last id is not made (its end was known), the
    # one made before a's end-of-sequence id is dropped, and a's remaining steps alone are planned ahead again
    assert eng.used >= 4 and eng.prepared > eng.used
    assert eng.cache.rows.num_free == 3 and eng.cache.groups[0].pool.num_free == 8
    eng.cache.check_integrity()


def test_a_newcomer_makes_the_plan_ahead_void():
    eng, s = ahead()
    a = s.add_request([1], SamplingParams(max_tokens=8))
    for _ in range(3):
        s.step()
    used = eng.used
    c = s.add_request([40, 41, 42], SamplingParams(max_tokens=3))         # can be admitted: the planned step is dropped
    s.step()
    assert eng.used == used and len(eng.batches[-1]) == 2                  # a's token and c's prompt in one step
    s.run()
    assert a.output == list(range(2, 10)) and c.output == [43, 44, 45]
    assert eng.cache.rows.num_free == 3 and eng.cache.groups[0].pool.num_free == 8


def test_an_abort_makes_the_plan_ahead_void():
    eng, s = ahead()
    a = s.add_request([1], SamplingParams(max_tokens=8))
    b = s.add_request([20], SamplingParams(max_tokens=8))
    for _ in range(3):
        s.step()
    s.abort(a)
    s.run()
    assert b.output == list(range(21, 29)) and a.finish_reason == "abort"
    assert eng.cache.rows.num_free == 3 and eng.cache.groups[0].pool.num_free == 8

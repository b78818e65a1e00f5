"""The generation loop's decisions, with a scripted backend instead of a GPU: batches of unequal prompts,
stop tokens, early finishers, a full context, a full cache, slots used again by later batches."""

import pytest

from sleuth_b200.cache.book import CacheBook, pages_for
from sleuth_b200.engine.generate import generate_batches, plan_batches
from sleuth_b200.sampling import SamplingConfig


class ScriptedBackend:
    """Next token of a sequence = script(prompt, number of new tokens so far). Keeps a real CacheBook."""

    def __init__(self, script, max_len=64, n_pages=64, max_slots=8, vocab=100):
        self.script, self.max_len, self.vocab = script, max_len, vocab
        self.book = CacheBook([0], n_pages, max_slots, stride=pages_for(max_len))
        self.total_pages = n_pages
        self.seq = {}
        self.log = []

    def open(self, n):
        slots = self.book.open(n)
        self.log.append(("open", tuple(slots)))
        return slots

    def close(self, slots):
        self.book.close(slots)
        self.log.append(("close", tuple(slots)))
        for s in slots:
            self.seq.pop(s, None)

    def _append(self, slots, lists):
        new = [int(self.book.lengths[s]) + len(t) for s, t in zip(slots, lists)]
        assert all(n <= self.max_len for n in new), "the loop stepped past the context"
        self.book.grow(slots, new)
        self.book.commit(slots, new)
        for s, t in zip(slots, lists):
            self.seq.setdefault(s, []).extend(t)
        return list(slots)

    def prefill(self, slots, prompts):
        self.log.append(("prefill", tuple(len(p) for p in prompts)))
        self.prompt_len = {s: len(p) for s, p in zip(slots, prompts)} | getattr(self, "prompt_len", {})
        return self._append(slots, prompts)

    def decode(self, slots, tokens):
        self.log.append(("decode", tuple(slots)))
        return self._append(slots, [[t] for t in tokens])

    def choose(self, logits, cfg, uniforms, vocab_limit, recent, banned):
        out = []
        for s in logits:
            seq = self.seq[s]
            p = self.prompt_len[s]
            out.append(self.script(seq[:p], len(seq) - p))
        return out

    # ---- the pipelined protocol: tokens stay "on the device" (self.feed), the host gets them one step late ----
    def choose_later(self, logits, cfg, uniforms, vocab_limit):
        tokens = self.choose(logits, cfg, uniforms, vocab_limit, None, None)
        self.feed = list(tokens)
        self.log.append(("choose_later", len(tokens)))
        return lambda: list(tokens)

    def decode_fed(self, slots, feed_map):
        self.log.append(("decode", tuple(slots)))
        return self._append(slots, [[self.feed[i]] for i in feed_map])

    def free_pages(self):
        return self.book.groups[0].pool.free

    def pages_needed(self, slots, new_lengths):
        return max(self.book.pages_needed(slots, new_lengths))

    def length(self, slot):
        return int(self.book.lengths[slot])

    def sync(self):
        pass


def count_up(prompt, k):
    return (prompt[-1] + k + 1) % 100


@pytest.fixture(params=["step by step", "one step ahead"], autouse=True)
def loop_mode(request, monkeypatch):
    """Every test of the loop runs twice: with the host waiting for each token, and with the GPU one step ahead."""
    monkeypatch.setattr(ScriptedBackend, "pipelined", request.param == "one step ahead", raising=False)
    return request.param


def test_unequal_prompts_stop_tokens_and_early_finishers():
    be = ScriptedBackend(count_up)
    prompts = [[10], [20, 21, 22], [50, 51]]                      # sequence 0 meets 13 at its third token
    seen = []
    res = generate_batches(be, prompts, max_new_tokens=6, sampling=SamplingConfig(temperature=0.0), stop_ids={13, 55},
                           on_token=lambda r, t: seen.append((r, t)))
    assert res[0].new_ids == [11, 12, 13] and res[0].stop_reason == "stop_token"          # the stop token is kept
    assert res[1].new_ids == [23, 24, 25, 26, 27, 28] and res[1].stop_reason == "max_new_tokens"
    assert res[2].new_ids == [52, 53, 54, 55] and res[2].stop_reason == "stop_token"
    assert [r.prompt_ids for r in res] == prompts
    decodes = [e for e in be.log if e[0] == "decode"]
    if be.pipelined:      # a sequence that met its stop token is carried through one more step
        assert [len(e[1]) for e in decodes] == [3, 3, 3, 2, 1]
    else:
        assert [len(e[1]) for e in decodes] == [3, 3, 2, 1, 1]  # the batch shrinks as sequences end
    assert be.book.free_slots == be.book.max_slots and be.book.pages_in_use() == [0]
    assert [t for r, t in seen if r == 2] == [52, 53, 54, 55]


def test_context_full_and_prompt_truncation():
    be = ScriptedBackend(count_up, max_len=8)
    res = generate_batches(be, [[1, 2, 3, 4, 5, 6], list(range(30, 50))], max_new_tokens=10,
                           sampling=SamplingConfig(temperature=0.0))
    # 6 prompt tokens + 2 decoded fill the 8 positions; the third new token is produced but cannot be fed
    assert res[0].stop_reason == "context_full" and res[0].new_ids == [7, 8, 9]
    assert res[1].prompt_ids == list(range(43, 50)) and res[1].stop_reason == "context_full" and len(res[1].new_ids) == 2


def test_empty_prompt_and_zero_tokens():
    be = ScriptedBackend(count_up)
    with pytest.raises(ValueError, match="empty"):
        generate_batches(be, [[1], []], max_new_tokens=2)
    res = generate_batches(be, [[1]], max_new_tokens=0)
    assert res[0].new_ids == [] and res[0].stop_reason == "max_new_tokens"


def test_more_requests_than_slots_run_as_batches_that_reuse_slots():
    be = ScriptedBackend(count_up, max_slots=2)
    prompts = [[i] for i in range(5)]
    res = generate_batches(be, prompts, max_new_tokens=3, sampling=SamplingConfig(temperature=0.0), max_batch=2)
    assert [r.new_ids for r in res] == [[i + 1, i + 2, i + 3] for i in range(5)]
    opens = [e[1] for e in be.log if e[0] == "open"]
    assert [len(o) for o in opens] == [2, 2, 1] and set(opens[1]) == set(opens[0])         # the same slots again


def test_cache_pages_bound_a_batch():
    assert plan_batches([100, 100, 100], max_new_tokens=28, max_len=4096, total_pages=4, max_batch=64) == [[0, 1], [2]]
    assert plan_batches([1000], max_new_tokens=10, max_len=4096, total_pages=4, max_batch=64) == [[0]]
    assert plan_batches([10] * 5, max_new_tokens=10, max_len=4096, total_pages=99, max_batch=2) == [[0, 1], [2, 3], [4]]


def test_a_request_larger_than_the_cache_runs_until_the_pages_are_gone():
    be = ScriptedBackend(count_up, max_len=4096, n_pages=1, max_slots=4)
    res = generate_batches(be, [[5] * 60], max_new_tokens=20, sampling=SamplingConfig(temperature=0.0))
    # 60 prompt tokens and 4 decoded ones fill the only page; the fifth new token exists but cannot be fed
    assert res[0].stop_reason == "context_full" and len(res[0].new_ids) == 5
    assert be.book.pages_in_use() == [0] and be.book.free_slots == 4


def test_sampling_streams_do_not_depend_on_the_batch():
    seen = {}

    class Rec(ScriptedBackend):
        def choose(self, logits, cfg, uniforms, vocab_limit, recent, banned):
            for s, u in zip(logits, uniforms):
                seen.setdefault(self.tag, {}).setdefault(tuple(self.seq[s][:self.prompt_len[s]]), []).append(u)
            return super().choose(logits, cfg, uniforms, vocab_limit, recent, banned)

    prompts = [[1], [2], [3]]
    a = Rec(count_up)
    a.tag = "together"
    generate_batches(a, prompts, max_new_tokens=3, sampling=SamplingConfig(temperature=1.0), seed=7)
    b = Rec(count_up, max_slots=1)
    b.tag = "alone"
    generate_batches(b, prompts, max_new_tokens=3, sampling=SamplingConfig(temperature=1.0), seed=7, max_batch=1)
    assert seen["together"] == seen["alone"]
    assert len({tuple(v) for v in seen["alone"].values()}) == 3 and all(0 <= u < 1 for v in seen["alone"].values() for u in v)


def test_repetition_window_and_ngram_ban_reach_the_sampler():
    got = []

    class Rec(ScriptedBackend):
        def choose(self, logits, cfg, uniforms, vocab_limit, recent, banned):
            got.append((recent, banned))
            return super().choose(logits, cfg, uniforms, vocab_limit, recent, banned)

    be = Rec(lambda prompt, k: [1, 2, 1, 2][k])
    generate_batches(be, [[1, 2, 3, 1, 2]], max_new_tokens=3,
                     sampling=SamplingConfig(temperature=0.0, repetition_penalty=1.3, repeat_last_n=3, no_repeat_ngram=3))
    assert got[0] == ([[1, 2, 3]], [[3]])            # last three tokens 3,1,2; "1 2" was followed by 3 before
    assert got[1][0] == [[1, 2]] and got[1][1] == [[]]

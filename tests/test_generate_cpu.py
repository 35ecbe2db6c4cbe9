"""Decisions of the generation loop, with stand-ins for the engine and the sampler (no GPU)."""
import pytest
import torch


class FakeSlots:
    def __init__(self, n):
        self.n = n
        self.live = set()

    @property
    def free_count(self):
        return self.n - len(self.live)


class FakeCache:
    def __init__(self, n_slots, n_pages, max_seq_len):
        self.slots = FakeSlots(n_slots)
        self.n_pages, self.max_seq_len, self.page = n_pages, max_seq_len, 64


class FakeEngine:
    """'Logits' put all mass on (last token + 1) % vocab; records every call."""

    def __init__(self, n_slots=4, n_pages=64, max_seq_len=512, vocab=50):
        self.cache = FakeCache(n_slots, n_pages, max_seq_len)
        self.vocab = vocab
        self.calls = []
        self.opened = []
        self.closed = []
        self.length = {}

    def open(self):
        free = [s for s in range(self.cache.slots.n) if s not in self.cache.slots.live]
        s = free[0]
        self.cache.slots.live.add(s)
        self.opened.append(s)
        self.length[s] = 0
        return s

    def close(self, s):
        assert s in self.cache.slots.live, "slot closed twice"
        self.cache.slots.live.remove(s)
        self.closed.append(s)

    def step(self, entries, want=None):
        self.calls.append([(s, list(t)) for s, t in entries])
        out = torch.zeros(len(entries), self.vocab)
        for i, (s, t) in enumerate(entries):
            assert s in self.cache.slots.live
            self.length[s] += len(t)
            out[i, (t[-1] + 1) % self.vocab] = 1.0
        return out


class ArgmaxSampler:
    def __init__(self):
        self.calls = []

    def sample(self, logits, params, *, seed, step, seq_ids, histories, stop_tokens):
        self.calls.append(dict(step=step, seq_ids=list(seq_ids), seed=seed, hist=[list(h) for h in histories]))
        return logits.argmax(-1).tolist()


@pytest.fixture(scope="module")
def G(llogos):
    import importlib
    return importlib.import_module("daisi-llogos_b200.sampling.generate"), \
        importlib.import_module("daisi-llogos_b200.sampling.params").GenerationParams


def test_counts_up_until_max_tokens(G):
    gen, Params = G
    eng, smp = FakeEngine(), ArgmaxSampler()
    r = gen.generate(eng, smp, [[3], [10, 11, 12]], Params.greedy_params(4, seed=1), stop_tokens=())
    assert r.tokens == [[4, 5, 6, 7], [13, 14, 15, 16]] and r.finish_reasons == ["length", "length"]
    assert eng.calls[0] == [(0, [3]), (1, [10, 11, 12])]                  # prompts of unequal length in one step
    assert all(len(t) == 1 for c in eng.calls[1:] for _, t in c)          # then one token each
    assert len(eng.calls) == 4                                           # no step after the last token
    assert sorted(eng.closed) == [0, 1] and not eng.cache.slots.live
    assert [c["step"] for c in smp.calls] == [0, 1, 2, 3]
    assert smp.calls[2]["hist"][1] == [10, 11, 12, 13, 14]                # history = prompt + generated
    assert (r.prompt_tokens, r.generated_tokens, r.decode_steps, r.batches) == (4, 8, 3, 1)


def test_stop_token_is_not_emitted_and_the_batch_shrinks(G):
    gen, Params = G
    eng, smp = FakeEngine(), ArgmaxSampler()
    r = gen.generate(eng, smp, [[1], [6], [20]], Params.greedy_params(6, seed=1), stop_tokens=[4, 8])
    assert r.tokens == [[2, 3], [7], [21, 22, 23, 24, 25, 26]]
    assert r.finish_reasons == ["stop", "stop", "length"]
    sizes = [len(c) for c in eng.calls]
    assert sizes == [3, 3, 2, 1, 1, 1]                 # request 1 leaves after its 2nd draw, request 0 after its 3rd
    assert [s for s, _ in eng.calls[3]] == [2]
    assert smp.calls[2]["seq_ids"] == [0, 2] and smp.calls[3]["seq_ids"] == [2]


def test_batches_follow_one_another_and_reuse_slots(G):
    gen, Params = G
    eng, smp = FakeEngine(n_slots=2), ArgmaxSampler()
    prompts = [[i] for i in range(5)]
    r = gen.generate(eng, smp, prompts, Params.greedy_params(2, seed=1), stop_tokens=(), max_batch=8)
    assert r.batches == 3 and r.tokens == [[i + 1, i + 2] for i in range(5)]
    assert eng.opened == [0, 1, 0, 1, 0] and eng.closed == [0, 1, 0, 1, 0]
    assert [c["seq_ids"] for c in smp.calls if c["step"] == 0] == [[0, 1], [2, 3], [4]]   # ids are global


def test_batches_respect_the_page_budget(G):
    gen, _ = G
    plan = gen.plan_batches([100, 100, 100, 30], 28, max_batch=8, free_pages=4, page=64, max_seq_len=4096)
    assert plan == [[0, 1], [2, 3]]                    # 2 pages each, then 2 + 1
    with pytest.raises(ValueError, match="exceeds"):
        gen.plan_batches([5000], 1, max_batch=8, free_pages=100, page=64, max_seq_len=4096)
    with pytest.raises(ValueError, match="pages"):
        gen.plan_batches([300], 100, max_batch=8, free_pages=4, page=64, max_seq_len=4096)
    with pytest.raises(ValueError, match="empty"):
        gen.plan_batches([0], 1, max_batch=8, free_pages=4, page=64, max_seq_len=4096)


def test_context_limit_ends_a_sequence(G):
    gen, Params = G
    eng, smp = FakeEngine(max_seq_len=6), ArgmaxSampler()
    r = gen.generate(eng, smp, [[1, 2, 3]], Params.greedy_params(50, seed=1), stop_tokens=())
    assert r.finish_reasons == ["context"] and len(r.tokens[0]) == 3
    assert max(eng.length.values()) <= 6


def test_slots_are_returned_when_a_step_fails(G):
    gen, Params = G

    class Boom(FakeEngine):
        def step(self, entries, want=None):
            if len(self.calls) == 1:
                raise RuntimeError("boom")
            return super().step(entries, want)

    eng = Boom()
    with pytest.raises(RuntimeError):
        gen.generate(eng, ArgmaxSampler(), [[1], [2]], Params.greedy_params(3, seed=1), stop_tokens=())
    assert not eng.cache.slots.live


def test_zero_tokens_and_on_token(G):
    gen, Params = G
    eng = FakeEngine()
    r = gen.generate(eng, ArgmaxSampler(), [[1]], Params.greedy_params(0), stop_tokens=())
    assert r.tokens == [[]] and eng.calls == []
    got = []
    gen.generate(eng, ArgmaxSampler(), [[1], [5]], Params.greedy_params(2, seed=0), stop_tokens=(),
                 on_token=lambda i, t: got.append((i, t)))
    assert got == [(0, 2), (1, 6), (0, 3), (1, 7)]


def test_params(G):
    _, Params = G
    p = Params()
    assert (p.max_tokens, p.temperature, p.top_k, p.top_p, p.repetition_penalty, p.penalty_count) == (256, 0.8, 40, 0.95, 1.1, 64)
    assert not p.greedy and p.uses_history and Params.greedy_params().greedy
    with pytest.raises(ValueError):
        Params(temperature=-1).validate()


class AheadEngine(FakeEngine):
    """FakeEngine that can also take its tokens from a 'device' tensor the host has not read."""

    def step_fed(self, slots, source, rows, want=None):
        return self.step([(s, [int(source[r])]) for s, r in zip(slots, rows)])


class AheadSampler(ArgmaxSampler):
    """Hands tokens out only through result(), and records when each was read."""

    def __init__(self):
        super().__init__()
        self.reads = []

    def sample_device(self, logits, params, *, seed, step, seq_ids, histories=None, stop_tokens=()):
        self.calls.append(dict(step=step, seq_ids=list(seq_ids), seed=seed, hist=None))
        return logits.argmax(-1).to(torch.int32)

    def fetch(self, picked):
        sampler, n_calls = self, len(self.calls)

        class Pending:
            def result(self):
                sampler.reads.append((n_calls, len(sampler.calls)))     # (sample number, samples queued when read)
                return picked.tolist()
        return Pending()


@pytest.mark.parametrize("stop_tokens,max_new,max_seq_len", [((), 4, 512), ([4, 8, 23], 6, 512), ([9], 30, 14), ([2], 3, 512)])
def test_running_one_step_ahead_gives_the_same_tokens(G, stop_tokens, max_new, max_seq_len):
    gen, Params = G
    prompts = [[1], [6, 7], [20], [40, 41, 42, 43, 44]]
    params = Params.greedy_params(max_new, seed=1)
    e0, s0 = FakeEngine(max_seq_len=max_seq_len), ArgmaxSampler()
    r0 = gen.generate(e0, s0, prompts, params, stop_tokens=stop_tokens)
    e1, s1 = AheadEngine(max_seq_len=max_seq_len), AheadSampler()
    r1 = gen.generate(e1, s1, prompts, params, stop_tokens=stop_tokens)
    assert r1.tokens == r0.tokens and r1.finish_reasons == r0.finish_reasons
    assert r1.generated_tokens == r0.generated_tokens
    assert not e1.cache.slots.live and sorted(e1.closed) == sorted(e0.closed)
    # every sample but the last of a batch was read only after the next one had been queued
    assert s1.reads and all(at > n for n, at in s1.reads[:-1])
    # a sequence runs at most one step more than in the loop that reads every token at once
    for s in e0.length:
        assert e0.length[s] <= e1.length[s] <= e0.length[s] + 1
    assert max(e1.length.values()) <= max_seq_len
    # and with the switch off the same objects take the ordinary loop
    e2, s2 = AheadEngine(max_seq_len=max_seq_len), AheadSampler()
    r2 = gen.generate(e2, s2, prompts, params, stop_tokens=stop_tokens, run_ahead=False)
    assert r2.tokens == r0.tokens and not s2.reads

"""The step function's host logic, run on CPU tensors with stand-ins for the kernels (no GPU):
what it checks before launching, how it lays tokens out, how slots and pages come back."""
import pytest
import torch

import cpu_ops
import plain_model as P
from conftest import TINY, read_weights, random_tokens


@pytest.fixture(scope="module")
def setup(llogos, model_dirs):
    out = {}
    for name in TINY:
        model = llogos.weights.load_model(model_dirs[name], dtype=torch.float32, device="cpu", ops=cpu_ops)
        out[name] = (model, read_weights(llogos, model_dirs[name]))
    return out


def engine_for(llogos, model, **kw):
    kw.setdefault("max_tokens", 64 * 12)
    return llogos.engine.Engine(model, use_graphs=False, **kw)


@pytest.mark.parametrize("name", list(TINY))
def test_schedules_agree_with_plain(llogos, setup, name):
    model, w = setup[name]
    cfg = TINY[name]
    eng = engine_for(llogos, model)
    seqs = random_tokens(cfg["vocab_size"], [3, 70, 33, 100], 5)
    refs = [P.forward(w, cfg, s) for s in seqs]
    tol = 2e-4
    for s, r in zip(seqs, refs):                       # each alone and whole
        slot = eng.open()
        lg = eng.step([(slot, s)], [list(range(len(s)))])
        assert float((lg.double() - r).abs().max()) < tol
        eng.close(slot)
    for rnd in range(2):                               # unequal batch, decoded on, shorter ones end earlier
        slots = [eng.open() for _ in seqs]
        cut = [max(1, len(s) - 3 - i) for i, s in enumerate(seqs)]
        lg = eng.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)])
        for i, (s, c) in enumerate(zip(seqs, cut)):
            assert float((lg[i].double() - refs[i][c - 1]).abs().max()) < tol
        pos = list(cut)
        live = list(range(len(seqs)))
        while live:
            lg = eng.step([(slots[i], [seqs[i][pos[i]]]) for i in live])
            for j, i in enumerate(live):
                assert float((lg[j].double() - refs[i][pos[i]]).abs().max()) < tol
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.close(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]
        eng.cache.audit()
    assert eng.cache.slots.free_count == eng.cache.slots.n_slots


def test_chunked_prompt_and_mixed_step(llogos, setup):
    model, w = setup["qwen2"]
    cfg = TINY["qwen2"]
    eng = engine_for(llogos, model)
    a, b = random_tokens(cfg["vocab_size"], [150, 20], 6)
    ra, rb = P.forward(w, cfg, a), P.forward(w, cfg, b)
    sa, sb = eng.open(), eng.open()
    eng.step([(sa, a[:90])], [[]])
    lg = eng.step([(sa, a[90:]), (sb, b)], [[0, 59], [19]])           # a continues while b starts
    assert float((lg[0].double() - ra[90]).abs().max()) < 2e-4
    assert float((lg[1].double() - ra[149]).abs().max()) < 2e-4
    assert float((lg[2].double() - rb[19]).abs().max()) < 2e-4


def test_errors_come_before_any_launch(llogos, setup):
    model, _ = setup["llama"]
    eng = engine_for(llogos, model, max_tokens=64 * 3, n_slots=2)
    E = llogos.engine.StepError
    s = eng.open()
    with pytest.raises(E, match="at least one sequence"):
        eng.step([])
    with pytest.raises(E, match="no tokens"):
        eng.step([(s, [])])
    with pytest.raises(E, match="outside the vocabulary"):
        eng.step([(s, [1, 256])])
    with pytest.raises(E, match="outside the vocabulary"):
        eng.step([(s, [-1])])
    with pytest.raises(E, match="wanted position"):
        eng.step([(s, [1, 2])], [[2]])
    with pytest.raises(E, match="twice"):
        eng.step([(s, [1]), (s, [2])])
    with pytest.raises(E, match="not in use"):
        eng.step([(1, [1])])
    with pytest.raises(E, match="longest sequence|cache full"):
        eng.step([(s, [1] * (64 * 3 + 1))])
    assert eng.length(s) == 0                       # nothing happened
    eng.step([(s, [1] * 130)])
    t = eng.open()
    with pytest.raises(E, match="cache full"):
        eng.step([(t, [1] * 1)])
    eng.close(s)
    eng.step([(t, [1] * 65)])
    eng.cache.audit()


def test_context_beyond_the_models_positions_is_refused(llogos, setup, model_dirs):
    """A cache for longer sequences than ``max_position_embeddings`` allows is an error that names both numbers,
    through the engine and through the Python entry point; without an explicit length the model's limit caps it."""
    model, _ = setup["llama"]                       # max_position_embeddings 512
    with pytest.raises(ValueError, match="600.*512"):
        llogos.engine.Engine(model, max_tokens=64 * 20, max_seq_len=600, use_graphs=False)
    assert llogos.engine.Engine(model, max_tokens=64 * 20, use_graphs=False).cache.max_seq_len == 512
    api = __import__("importlib").import_module("daisi-llogos_b200.api")
    with pytest.raises(ValueError, match="max_position_embeddings"):
        api.LlogosModel(model, max_context=4096, max_batch=1, use_graphs=False)


def test_a_second_engine_leaves_the_first_ones_tables_alone(llogos, setup):
    """Two engines on one model with different longest sequences: the rotation tables only grow, so the
    first engine's steps see the same tables before and after the second engine exists."""
    model, w = setup["qwen2"]
    cfg = TINY["qwen2"]
    toks = random_tokens(cfg["vocab_size"], [200], 3)[0]
    ref = P.forward(w, cfg, toks)
    big = engine_for(llogos, model, max_tokens=64 * 8, max_seq_len=400)
    rot = next(iter(model.encodings.values())).rotation()
    small = engine_for(llogos, model, max_tokens=64 * 2, max_seq_len=100)
    assert next(iter(model.encodings.values())).rotation() is rot and model.position_limit() >= 400
    slot = big.open()
    lg = big.step([(slot, toks)])
    assert float((lg[0].double() - ref[-1]).abs().max()) < 2e-4
    with pytest.raises(llogos.engine.StepError, match="longest sequence"):
        s2 = small.open()
        small.step([(s2, toks)])


def test_padding_free_layout(llogos, setup):
    """Exactly the given tokens run: the packed layout has no padding rows."""
    model, _ = setup["llama"]
    eng = engine_for(llogos, model)
    seen = {}
    real = cpu_ops.embed_rows

    class Spy:
        def __getattr__(self, k):
            return getattr(cpu_ops, k)

        def embed_rows(self, table, ids, out):
            seen["n"] = ids.numel()
            return real(table, ids, out)

    eng.ops = Spy()
    s1, s2, s3 = eng.open(), eng.open(), eng.open()
    eng.step([(s1, [1] * 5), (s2, [2] * 9), (s3, [3] * 13)])
    assert seen["n"] == 27
    eng.step([(s1, [1]), (s3, [3])])
    assert seen["n"] == 2


@pytest.mark.parametrize("name", ["qwen3", "qwen2"])
def test_random_cuts_and_batches(llogos, setup, name):
    """Requests cut into steps at random (several tokens, one token, mixed in one step), joined in
    random batches, closed at random: every wanted logit equals the whole-sequence reference."""
    import random
    rng = random.Random(7)
    model, w = setup[name]
    cfg = TINY[name]
    eng = engine_for(llogos, model, max_tokens=64 * 10, n_slots=4)
    seqs = random_tokens(cfg["vocab_size"], [9, 70, 33, 140, 65, 128, 20, 5], 9)
    refs = [P.forward(w, cfg, s) for s in seqs]
    waiting = list(range(len(seqs)))
    live = {}                                   # request -> (slot, tokens done)
    while waiting or live:
        while waiting and eng.cache.slots.free_count and rng.random() < 0.7:
            i = waiting.pop(0)
            live[i] = [eng.open(), 0]
        if not live:
            continue
        batch = rng.sample(sorted(live), rng.randint(1, len(live)))
        entries, want, expect = [], [], []
        for i in batch:
            slot, done = live[i]
            left = len(seqs[i]) - done
            take = min(left, rng.choice([1, 1, 1, 2, 7, 40, 64, 200]))
            ws = sorted(rng.sample(range(take), rng.randint(0, min(take, 3))))
            entries.append((slot, seqs[i][done:done + take]))
            want.append(ws)
            expect += [(i, done + x) for x in ws]
            live[i][1] = done + take
        try:
            lg = eng.step(entries, want)
        except llogos.engine.StepError as e:
            assert "cache full" in str(e)           # too many long requests alive at once: end one and go on
            for i in batch:
                live[i][1] -= len(entries[batch.index(i)][1])
            victim = max(live, key=lambda i: live[i][1])
            eng.close(live.pop(victim)[0])
            waiting.append(victim)
            continue
        assert lg.shape[0] == len(expect)
        for row, (i, pos) in enumerate(expect):
            assert float((lg[row].double() - refs[i][pos]).abs().max()) < 2e-4, (i, pos)
        for i in batch:
            if live[i][1] == len(seqs[i]):
                eng.close(live.pop(i)[0])
        eng.cache.audit()
    assert eng.cache.slots.free_count == 4


def test_tokens_fed_from_the_device_side(llogos, setup):
    """step_fed takes one token per sequence out of a tensor by row: the same logits as step with the ids."""
    model, w = setup["qwen3"]
    cfg = TINY["qwen3"]
    eng = engine_for(llogos, model)
    seqs = random_tokens(cfg["vocab_size"], [20, 9, 31], 8)
    refs = [P.forward(w, cfg, s) for s in seqs]
    slots = [eng.open() for _ in seqs]
    eng.step([(sl, s[:5]) for sl, s in zip(slots, seqs)])
    source = torch.tensor([seqs[2][5], 0, seqs[0][5], seqs[1][5]], dtype=torch.int32)
    lg = eng.step_fed(slots, source, [2, 3, 0])
    for i in range(3):
        assert float((lg[i].double() - refs[i][5]).abs().max()) < 2e-4
    lg = eng.step_fed([slots[1]], torch.tensor([seqs[1][6]], dtype=torch.int32), [0])
    assert float((lg[0].double() - refs[1][6]).abs().max()) < 2e-4
    before = [eng.length(s) for s in slots]
    with pytest.raises(llogos.engine.StepError, match="source row"):
        eng.step_fed(slots, source, [0, 1, 4])
    with pytest.raises(llogos.engine.StepError, match="int32"):
        eng.step_fed(slots, source.long(), [0, 1, 2])
    with pytest.raises(llogos.engine.StepError, match="one source row"):
        eng.step_fed(slots, source, [0, 1])
    assert [eng.length(s) for s in slots] == before
    for s in slots:
        eng.close(s)
    eng.cache.audit()


def test_products_that_split_their_sums(llogos, setup, model_dirs):
    """With a tensor-core product that splits K the engine's consumers get partial sums: the branch consumers add
    them up, and the output head asks for one whole product.  A stand-in that always splits in three shows it."""
    class SplittingOps:
        def __getattr__(self, name):
            return getattr(cpu_ops, name)

        @staticmethod
        def gemm_tc_supported(x, w):
            return True

        @staticmethod
        def sm_count():
            return 4

        @staticmethod
        def gemm_tc_splits(k, wish):
            return min(wish, 3)

        @staticmethod
        def gemm_tc(x, w, out, tile_n=0, gated_features=0):
            assert gated_features == 0
            s, k = out.shape[0], x.shape[1]
            step = -(-k // s)
            for i in range(s):
                sl = slice(i * step, min(k, (i + 1) * step))
                out[i] = (x[:, sl].float() @ w[:, sl].float().t()).to(out.dtype)

    lin = __import__("importlib").import_module("daisi-llogos_b200.kernels.linear")
    wished = []
    real_plan = lin.plan_splits
    lin.plan_splits = lambda n, o, k, n_sms: wished.append((n, o, k)) or 3
    try:
        name = "llama"
        cfg = TINY[name]
        model = llogos.weights.load_model(model_dirs[name], dtype=torch.float32, device="cpu", ops=SplittingOps())
        eng = llogos.engine.Engine(model, max_tokens=256, use_graphs=False)
        toks = random_tokens(cfg["vocab_size"], [21], 5)[0]
        ref = P.forward(setup[name][1], cfg, toks)
        slot = eng.open()
        got = eng.step([(slot, toks)], [list(range(len(toks)))])
        assert float((got.double() - ref).abs().max()) < 1e-4 * float(ref.abs().max())
        assert wished and all(o != cfg["vocab_size"] for _, o, _ in wished)      # the head never asked for splits
    finally:
        lin.plan_splits = real_plan


@pytest.mark.parametrize("name", ["llama", "qwen3"])
def test_truncate_and_continue(llogos, setup, name):
    """A sequence rolled back to 25 of its 40 tokens and continued with other tokens gives the logits of
    the new sequence (the reference rolls its cache back the same way, Inference/KvCache.cs:135)."""
    model, w = setup[name]
    cfg = TINY[name]
    eng = engine_for(llogos, model)
    a, b = random_tokens(cfg["vocab_size"], [40, 12], 44)
    slot = eng.open()
    eng.step([(slot, a)])
    eng.truncate(slot, 25)
    assert eng.cache.length(slot) == 25
    new = a[:25] + b
    ref = P.forward(w, cfg, new)
    got = eng.step([(slot, b[:5])], [list(range(5))])
    assert float((got.double() - ref[25:30]).abs().max()) < 1e-4 * float(ref.abs().max())
    for i in range(5, 12):
        got = eng.step([(slot, [b[i]])])
        assert float((got[0].double() - ref[25 + i]).abs().max()) < 1e-4 * float(ref.abs().max())
    with pytest.raises(llogos.engine.StepError, match="cannot truncate"):
        eng.truncate(slot, 100)
    eng.close(slot)
    eng.cache.audit()

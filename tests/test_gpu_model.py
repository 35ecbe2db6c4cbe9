"""The engine against the plain implementation on the GPU, in float32 and bfloat16:
each request alone and whole; the last 32 tokens one by one; batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots and pages are used again;
long decoding; the first tokens of a sequence."""
import pytest
import torch

import plain_model as P
from compare import Reference, reference
from conftest import INIT, INIT_OF, TINY, read_weights, random_tokens

pytestmark = pytest.mark.gpu

# How close the logits must be is said in compare.py: float32 within 2e-5 of the request's largest |logit|;
# bfloat16 within 1e-2 of the plain model that rounds where the engine does, and within 4e-2 of the exact one.
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def plain(llogos, model_dirs):
    """References of a fixed set of requests per configuration."""
    out = {}
    for name, cfg in TINY.items():
        w = read_weights(llogos, model_dirs[name])
        seqs = random_tokens(cfg["vocab_size"], [40, 150, 33, 97, 64, 129], 11)
        out[name] = (seqs, [Reference(w, cfg, s) for s in seqs])
    return out


@pytest.fixture(scope="module")
def engines(llogos, model_dirs):
    cache = {}

    def get(name, dtype, graphs=True):
        key = (name, dtype, graphs)
        if key not in cache:
            model = llogos.weights.load_model(model_dirs[name], dtype=dtype, device="cuda:0")
            cache[key] = llogos.engine.Engine(model, max_tokens=64 * 14, use_graphs=graphs)
        return cache[key]
    return get


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(TINY))
def test_each_request_alone_and_whole(engines, plain, name, dtype):
    eng = engines(name, dtype)
    seqs, refs = plain[name]
    for s, r in zip(seqs, refs):
        slot = eng.open()
        lg = eng.step([(slot, s)], [list(range(len(s)))])
        r.check(lg, range(len(s)), dtype, ("whole", len(s)))
        eng.close(slot)
    eng.cache.audit()


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager"])
@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(TINY))
def test_last_32_tokens_one_by_one(engines, plain, name, dtype, graphs):
    eng = engines(name, dtype, graphs)
    seqs, refs = plain[name]
    for s, r in zip(seqs, refs):
        slot = eng.open()
        cut = len(s) - 32
        lg = eng.step([(slot, s[:cut])])
        r.check(lg[0], [cut - 1], dtype, ("prompt end", len(s)))
        for p in range(cut, len(s)):
            lg = eng.step([(slot, [s[p]])])
            r.check(lg[0], [p], dtype, ("decoded position", p, "of", len(s)))
        eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(TINY))
def test_unequal_batches_one_after_another(engines, plain, name, dtype):
    eng = engines(name, dtype)
    seqs, refs = plain[name]
    for order in ([0, 1, 2], [3, 4, 5], [5, 0, 3, 1], [2, 4]):
        slots = {i: eng.open() for i in order}
        cut = {i: max(1, len(seqs[i]) - 5 - 7 * k) for k, i in enumerate(order)}
        lg = eng.step([(slots[i], seqs[i][:cut[i]]) for i in order], [[0, cut[i] - 1] for i in order])
        for k, i in enumerate(order):
            for row, p in ((2 * k, 0), (2 * k + 1, cut[i] - 1)):
                refs[i].check(lg[row], [p], dtype, ("prompt", i, p))
        pos = dict(cut)
        live = list(order)
        while live:
            lg = eng.step([(slots[i], [seqs[i][pos[i]]]) for i in live])
            for k, i in enumerate(live):
                refs[i].check(lg[k], [pos[i]], dtype, ("decode", i, pos[i], "batch of", len(live)))
                pos[i] += 1
            done = [i for i in live if pos[i] == len(seqs[i])]
            for i in done:
                eng.close(slots[i])                   # a shorter request ends earlier
            live = [i for i in live if i not in done]
        eng.cache.audit()
    assert eng.cache.slots.free_count == eng.cache.slots.n_slots


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(TINY))
def test_long_decoding_from_the_first_token(llogos, model_dirs, name, dtype):
    """One token, then 299 decoded: crosses pages and the window, starts at position 0."""
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    a, b = random_tokens(cfg["vocab_size"], [300, 200], 12)
    ra, rb = reference(model_dirs[name], w, cfg, a), reference(model_dirs[name], w, cfg, b)
    model = llogos.weights.load_model(model_dirs[name], dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 9)
    sa, sb = eng.open(), eng.open()
    for p in range(300):
        entries = [(sa, [a[p]])] + ([(sb, [b[p]])] if p < 200 else [])
        lg = eng.step(entries)
        if p in (0, 1, 2, 63, 64, 65, 127, 128, 199, 299) or p % 37 == 0:
            ra.check(lg[0], [p], dtype, ("a", p))
            if p < 200:
                rb.check(lg[1], [p], dtype, ("b", p))
        if p == 199:
            eng.close(sb)


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager"])
@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["wide", "qwen2", "deep"])
def test_decoding_across_the_length_bound_of_the_recorded_steps(llogos, tmp_path, name, dtype, graphs):
    """Decode steps are planned and recorded for lengths up to a bound (1,024, then 2,048): a sequence that grows
    from 1,000 to 1,060 tokens moves at position 1,024 to the next bound's workspace, counters and recorded launches
    (a first step run directly, the following ones replayed), beside a short sequence that stays far below.  Every
    decoded position of both against the plain model.  (The kernels take the lengths themselves from the device;
    the bound only sizes their scratch and their split of the keys, so a bound that is too small must not change a
    result either: the same test passes with the bound held at 1,024.)"""
    cfg = dict(TINY[name], max_position_embeddings=2304)
    d = str(tmp_path / "model")
    llogos.weights.write_random_model(d, cfg, seed=77, **INIT_OF.get(name, INIT))
    w = read_weights(llogos, d)
    a, b = random_tokens(cfg["vocab_size"], [1060, 300], 41)
    ra, rb = Reference(w, cfg, a), Reference(w, cfg, b)
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 24, use_graphs=graphs)
    sa, sb = eng.open(), eng.open()
    lg = eng.step([(sa, a[:1000]), (sb, b[:240])])
    ra.check(lg[0], [999], dtype, "a, prompt end")
    rb.check(lg[1], [239], dtype, "b, prompt end")
    for i in range(60):
        lg = eng.step([(sa, [a[1000 + i]]), (sb, [b[240 + i]])])
        ra.check(lg[0], [1000 + i], dtype, ("a", 1000 + i))
        rb.check(lg[1], [240 + i], dtype, ("b", 240 + i))
    eng.close(sa)
    eng.close(sb)
    eng.cache.audit()


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(TINY))
def test_prompts_of_hundreds_of_tokens(llogos, model_dirs, name, dtype):
    """Steps of 256 tokens and more take the products with tokens as the tensor-core rows and the large
    attention tiles; above 512 tokens no product splits its sums.  Every position is compared, alone
    and as one batch, twice in a row: each kernel starts while its predecessor still runs, and one that
    read its input before the wait would show here."""
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    seqs = random_tokens(cfg["vocab_size"], [300, 257, 500, 70], 13)
    refs = [reference(model_dirs[name], w, cfg, s) for s in seqs]
    model = llogos.weights.load_model(model_dirs[name], dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 24)
    for rep in range(2):
        for s, r in zip(seqs, refs):
            slot = eng.open()
            lg = eng.step([(slot, s)], [list(range(len(s)))])
            r.check(lg, range(len(s)), dtype, ("alone", rep, len(s)))
            eng.close(slot)
        slots = [eng.open() for _ in seqs]
        lg = eng.step(list(zip(slots, seqs)), [list(range(len(s))) for s in seqs])
        row = 0
        for s, r in zip(seqs, refs):
            r.check(lg[row:row + len(s)], range(len(s)), dtype, ("batch", rep, len(s)))
            row += len(s)
        for slot in slots:
            eng.close(slot)
    eng.cache.audit()


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_reused_pages_do_not_leak_old_keys(llogos, model_dirs, dtype):
    """A slot and its pages are used again by a shorter request: the logits must not see the
    previous owner's keys beyond the new request's length."""
    name = "llama"
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    model = llogos.weights.load_model(model_dirs[name], dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 3, n_slots=1)
    long_, short = random_tokens(cfg["vocab_size"], [190, 70], 13)
    s = eng.open()
    eng.step([(s, long_)])
    eng.close(s)
    s = eng.open()
    r = Reference(w, cfg, short)
    lg = eng.step([(s, short[:60])])
    r.check(lg[0], [59], dtype, ("prompt end",))
    for p in range(60, 70):
        lg = eng.step([(s, [short[p]])])
        r.check(lg[0], [p], dtype, (p,))


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_a_far_key_among_hundreds(llogos, tmp_path, dtype):
    """Weights made so that one far key decides the output: the last token's query matches the
    key of position 3 only.  A kernel that drops, repeats or misplaces a key tile shows here."""
    cfg = dict(TINY["llama"], num_hidden_layers=1, max_position_embeddings=1024)
    d = str(tmp_path / "m")
    llogos.weights.write_random_model(d, cfg, seed=3, std=0.05)
    w = read_weights(llogos, d)
    # token 7 -> a key that only token 9's query likes; rotation off for the pair by using
    # the slowest frequency pair (index 7 and 15 of each head) at moderate distance
    emb = w["model.embed_tokens.weight"].float()
    emb[7] = 0
    emb[7, 0] = 8.0
    emb[9] = 0
    emb[9, 1] = 8.0
    w["model.embed_tokens.weight"] = emb.to(torch.bfloat16)
    q = torch.zeros_like(w["model.layers.0.self_attn.q_proj.weight"]).float()
    k = torch.zeros_like(w["model.layers.0.self_attn.k_proj.weight"]).float()
    for h in range(4):
        q[h * 16 + 7, 1] = 6.0          # query of token 9: element 7 of every head
    for h in range(2):
        k[h * 16 + 7, 0] = 6.0          # key of token 7: element 7 of every kv head
    w["model.layers.0.self_attn.q_proj.weight"] = q.to(torch.bfloat16)
    w["model.layers.0.self_attn.k_proj.weight"] = k.to(torch.bfloat16)
    llogos.weights.write_safetensors(d + "/model.safetensors", w)
    toks = random_tokens(cfg["vocab_size"], [700], 14)[0]
    toks = [t if t not in (7, 9) else 11 for t in toks]
    toks[3] = 7
    toks[-1] = 9
    r = Reference(w, cfg, toks)
    ref = r.exact
    other = list(toks)
    other[3] = 11
    assert float((P.forward(w, cfg, other)[-1] - ref[-1]).abs().max()) > 0.05 * float(ref[-1].abs().max())
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 12)
    s = eng.open()
    lg = eng.step([(s, toks)])
    r.check(lg[0], [len(toks) - 1], dtype, ("whole",))
    eng.close(s)
    s = eng.open()
    eng.step([(s, toks[:-1])], [[]])
    lg = eng.step([(s, [toks[-1]])])
    r.check(lg[0], [len(toks) - 1], dtype, ("decode",))


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_padded_decode_batches_change_nothing(llogos, model_dirs, dtype):
    """Decode steps run at a few fixed batch sizes (CUDA graphs); a batch of 5 or 7 is filled up with
    rows on the cache's padding slot.  The real rows must come out as without padding, and the padding
    must leave no trace in the cache's books."""
    name = "qwen3"
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    seqs = random_tokens(cfg["vocab_size"], [30, 41, 52, 63, 74, 85, 96], 17)
    refs = [reference(model_dirs[name], w, cfg, s) for s in seqs]
    model = llogos.weights.load_model(model_dirs[name], dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 16, n_slots=8)
    eng_mod = __import__("importlib").import_module("daisi-llogos_b200.engine.engine")
    assert [eng_mod.decode_bucket(b) for b in (1, 2, 3, 5, 7, 9, 65)] == [1, 2, 3, 6, 8, 12, 96]
    slots = [eng.open() for _ in seqs]
    cut = [len(s) - 12 for s in seqs]
    eng.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)], [[] for _ in seqs])
    live = list(range(7))
    for j in range(12):
        if j == 4:
            live = [0, 2, 3, 5, 6]              # 7 -> 5 rows (runs as 6)
            eng.close(slots[1])
            eng.close(slots[4])
        lg = eng.step([(slots[i], [seqs[i][cut[i] + j]]) for i in live])
        assert lg.shape[0] == len(live)
        for k, i in enumerate(live):
            refs[i].check(lg[k], [cut[i] + j], dtype, (j, i))
    for i in live:
        eng.close(slots[i])
    eng.cache.audit()
    assert eng.cache.slots.free_count == 8


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["llama", "qwen3", "deep"])
def test_truncate_and_continue(engines, llogos, model_dirs, name, dtype):
    """Rolled back from 200 tokens (a page goes back to the pool) and continued with other tokens, one prompt
    step and then token by token: the logits of the new sequence.  The window of 24 keys of the Qwen3
    configuration lives in a ring of two pages that has gone round by then: position 150 is refused, its
    keys are overwritten; position 180 still has them."""
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    a, b = random_tokens(cfg["vocab_size"], [200, 40], 45)
    eng = engines(name, dtype)
    slot = eng.open()
    eng.step([(slot, a)])
    cut = 150
    if name == "qwen3":
        with pytest.raises(llogos.engine.StepError, match="overwritten"):
            eng.truncate(slot, 150)
        assert eng.cache.length(slot) == 200
        cut = 180
    ref = reference(model_dirs[name], w, cfg, a[:cut] + b)
    eng.truncate(slot, cut)
    lg = eng.step([(slot, b[:20])], [list(range(20))])
    ref.check(lg, range(cut, cut + 20), dtype, ("prompt after truncation",))
    for i in range(20, 40):
        lg = eng.step([(slot, [b[i]])])
        ref.check(lg[0], [cut + i], dtype, ("decode after truncation", i))
    eng.close(slot)
    eng.cache.audit()

"""Every way a request can be cut into steps and joined with others, through ``Engine.step`` on the GPU,
in float32 and bfloat16, against the plain implementation of whole sequences:

* a prompt cut into portions, among them portions of 256 tokens and more that land on a length that is
  no multiple of the page size (the large attention tiles straddle old pages and the step's own keys,
  the products take the orientation for many tokens), and a portion longer than a window's ring;
* steps that mix an entry of one token with entries of hundreds (the single token then runs through the
  prompt kernels), with sequences that join and leave between steps and slots that are used again;
* tokens fed from the device (``step_fed``) against the plain model;
* a random schedule: requests cut, batched and ended at random.

The reference continues a sequence from a start position the same way when a chat session sends only the
new part of its prompt (Chat/DaisiLlogosChatSession.cs:86-93, IForwardPass.cs:40).
"""
import importlib
import random

import pytest
import torch

from compare import reference
from conftest import TINY, read_weights, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


def engine_for(llogos, model_dir, dtype, **kw):
    model = llogos.weights.load_model(model_dir, dtype=dtype, device="cuda:0")
    return llogos.engine.Engine(model, **kw)


def portions_for(cfg):
    """Portions of one request: 70 tokens, then 300 on a length of 70, one token alone, 257 on 371, the rest."""
    if cfg.get("max_position_embeddings", 1 << 30) >= 700:
        return [70, 300, 1, 257, 40]
    return [70, 300, 1, 129]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(TINY))
def test_a_prompt_cut_into_portions(llogos, model_dirs, name, dtype):
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    portions = portions_for(cfg)
    toks = random_tokens(cfg["vocab_size"], [sum(portions)], 51)[0]
    ref = reference(model_dirs[name], w, cfg, toks)
    eng = engine_for(llogos, model_dirs[name], dtype, max_tokens=64 * 12)
    for rep in range(2):                                 # the second time over pages that were used before
        slot = eng.open()
        done = 0
        for n in portions:
            lg = eng.step([(slot, toks[done:done + n])], [list(range(n))])
            ref.check(lg, range(done, done + n), dtype, (name, "portion of", n, "on", done, "run", rep))
            done += n
        eng.close(slot)
    eng.cache.audit()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(TINY))
def test_one_token_beside_hundreds(llogos, model_dirs, name, dtype):
    """Four requests over three slots.  Steps: two prompts; 300 more tokens of A beside B's last single
    token; B leaves, C joins in B's slot with 320 tokens beside one token of A; one token each; D joins with
    its whole prompt beside 28 tokens of A and 19 of C."""
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    a, b, c, d = random_tokens(cfg["vocab_size"], [400, 150, 340, 90], 52)
    ra, rb, rc, rd = (reference(model_dirs[name], w, cfg, s) for s in (a, b, c, d))
    eng = engine_for(llogos, model_dirs[name], dtype, max_tokens=64 * 17, n_slots=3)

    def run(entries):
        """entries: (slot, reference, first position, count); all positions are wanted and compared."""
        lg = eng.step([(s, r.tokens[p0:p0 + n]) for s, r, p0, n in entries], [list(range(n)) for _, _, _, n in entries])
        row = 0
        for s, r, p0, n in entries:
            r.check(lg[row:row + n], range(p0, p0 + n), dtype, (name, "slot", s, "positions", p0, p0 + n))
            row += n

    sa, sb = eng.open(), eng.open()
    run([(sa, ra, 0, 70), (sb, rb, 0, 149)])
    run([(sa, ra, 70, 300), (sb, rb, 149, 1)])
    eng.close(sb)
    sc = eng.open()
    assert sc == sb                                       # the slot and its pages are used again
    run([(sa, ra, 370, 1), (sc, rc, 0, 320)])
    run([(sa, ra, 371, 1), (sc, rc, 320, 1)])
    sd = eng.open()
    run([(sd, rd, 0, 90), (sa, ra, 372, 28), (sc, rc, 321, 19)])
    for s in (sa, sc, sd):
        eng.close(s)
    eng.cache.audit()
    assert eng.cache.slots.free_count == 3


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["llama", "qwen3", "wide"])
def test_tokens_fed_from_the_device(llogos, model_dirs, name, dtype):
    """The engine's own greedy tokens stay on the device and feed the next step; every step's logits are those
    of the plain model for the sequence that results.  The batch shrinks, and the source rows are permuted."""
    ops = importlib.import_module("daisi-llogos_b200.kernels.ops")
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    prompts = random_tokens(cfg["vocab_size"], [37, 5, 130], 53)
    eng = engine_for(llogos, model_dirs[name], dtype, max_tokens=64 * 8)
    slots = [eng.open() for _ in prompts]
    lg = eng.step(list(zip(slots, prompts)))
    seqs = [list(p) for p in prompts]
    live = [0, 1, 2]
    picked = torch.empty(8, dtype=torch.int32, device="cuda:0")
    steps = []                                            # (sequence index, position, logits row) for the check below
    for step in range(9):
        out = picked[:len(live)]
        ops.argmax(lg, out)
        host = out.cpu().tolist()
        for i, t in zip(live, host):
            seqs[i].append(int(t))
        order = list(range(len(live)))
        if step == 4:                                     # sequence 1 ends; the others are fed in reverse order
            order = [k for k in order if live[k] != 1][::-1]
            eng.close(slots[1])
        lg = eng.step_fed([slots[live[k]] for k in order], out, order)
        live = [live[k] for k in order]
        steps.append([(i, len(seqs[i]) - 1, lg[r].float().cpu()) for r, i in enumerate(live)])
    refs = [reference(model_dirs[name], w, cfg, s) for s in seqs]
    for rows in steps:
        for i, pos, got in rows:
            refs[i].check(got, [pos], dtype, (name, "sequence", i, "position", pos))
    for i in live:
        eng.close(slots[i])
    eng.cache.audit()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(TINY))
def test_random_cuts_and_batches(llogos, model_dirs, name, dtype):
    """Requests cut into steps at random (hundreds of tokens, a few, one; mixed in one step), joined in
    random batches over four slots and too few pages, ended when the cache is full and started again."""
    rng = random.Random(7 + len(name))
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    limit = min(cfg.get("max_position_embeddings", 1 << 30), 640)
    lens = [9, 70, 33, 140, 65, 128, 20, 5, min(limit, 460), 300, 257]
    seqs = random_tokens(cfg["vocab_size"], lens, 54)
    refs = [reference(model_dirs[name], w, cfg, s) for s in seqs]
    eng = engine_for(llogos, model_dirs[name], dtype, max_tokens=64 * 14, n_slots=4)
    waiting = list(range(len(seqs)))
    live = {}                                             # request -> [slot, tokens done]
    n_steps = restarts = 0
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
            take = min(left, rng.choice([1, 1, 1, 2, 7, 40, 64, 200, 256, 300]))
            ws = sorted(rng.sample(range(take), rng.randint(0, min(take, 3))))
            entries.append((slot, seqs[i][done:done + take]))
            want.append(ws)
            expect += [(i, done + x) for x in ws]
            live[i][1] = done + take
        try:
            lg = eng.step(entries, want)
        except llogos.engine.StepError as e:
            assert "cache full" in str(e)                 # too many long requests alive: end one, start it again later
            for i in batch:
                live[i][1] -= len(entries[batch.index(i)][1])
            victim = max(live, key=lambda i: live[i][1])
            eng.close(live.pop(victim)[0])
            waiting.append(victim)
            restarts += 1
            continue
        n_steps += 1
        assert lg.shape[0] == len(expect)
        for row, (i, pos) in enumerate(expect):
            refs[i].check(lg[row], [pos], dtype, (name, "request", i, "position", pos, "step", n_steps))
        for i in batch:
            if live[i][1] == len(seqs[i]):
                eng.close(live.pop(i)[0])
        eng.cache.audit()
    assert eng.cache.slots.free_count == 4 and n_steps >= 10

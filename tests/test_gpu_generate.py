"""Generation through the Python entry point and the command line, against the plain
implementation: greedy token for token, seeded sampling draw for draw."""
import os
import subprocess
import sys

import pytest
import torch

import llogos_b200 as L
import plain_model as P
from conftest import ROOT, TINY, read_weights, random_tokens

pytestmark = pytest.mark.gpu


def plain_generate(w, cfg, prompt, n, stop=(), params=None, seed=0, seq_id=0, margins=None):
    """Greedy (params None) or sampled continuation with the plain model and the plain sampler.  ``margins``
    (a list) receives, per drawn token, how far the draw's uniform number lay from the nearest boundary
    between two tokens of the cumulative distribution."""
    toks, out = list(prompt), []
    for step in range(n):
        logits = P.forward(w, cfg, toks)[-1]
        if params is None:
            t = int(max(range(len(logits)), key=lambda i: (float(logits[i]), -i)))
        else:
            probs = P.sampling_distribution(logits.float().tolist(), previous=toks[-64:], **params)
            u = P.uniform_of(seed, seq_id, step)
            t = P.draw(probs, u)
            if margins is not None:
                cdf = torch.cumsum(probs, 0) / probs.sum()
                margins.append(float((cdf - u).abs().min()))
        if t in stop:
            break
        toks.append(t)
        out.append(t)
    return out


def same_draws(got, want, margins, excuse=1e-5):
    """True when the engine drew what the plain sampler drew; a first difference is excused only where the
    plain draw fell within ``excuse`` of a boundary of the cumulative distribution (float32 logits move a
    boundary by about 1e-6), and nothing after it is compared, since the sequences differ from there."""
    for j, (a, b) in enumerate(zip(got, want)):
        if a != b:
            return margins[j] < excuse
    return len(got) == len(want)


def margin_ok(w, cfg, prompt, out, min_gap=1e-3):
    """True when every greedy choice of the plain model was clear enough for float32 to agree."""
    toks = list(prompt)
    for t in out:
        lg = P.forward(w, cfg, toks)[-1]
        top = torch.topk(lg, 2).values
        if float(top[0] - top[1]) < min_gap:
            return False
        toks.append(t)
    return True


@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_matches_plain(llogos, model_dirs, name):
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    prompts = random_tokens(cfg["vocab_size"], [5, 9, 13, 1, 30], 31)
    model = L.LlogosModel.load(model_dirs[name], dtype="float32", max_context=256, max_batch=3)
    params = L.GenerationParams.greedy_params(12, stop_tokens=())
    r = model.generate(prompts, params)
    assert r.batches == 2 and r.finish_reasons == ["length"] * 5
    for p, got in zip(prompts, r.tokens):
        want = plain_generate(w, cfg, p, 12)
        if margin_ok(w, cfg, p, want):
            assert got == want
    # a single prompt as a flat list, and stop tokens from the configuration
    stop = model.stop_token_ids
    r1 = model.generate(prompts[0], L.GenerationParams.greedy_params(40))
    want = plain_generate(w, cfg, prompts[0], 40, stop=stop)
    if margin_ok(w, cfg, prompts[0], want):
        assert r1.tokens[0] == want
        assert r1.finish_reasons[0] == ("stop" if len(want) < 40 else "length")
    assert not model.engine.cache.slots.live()


def test_seeded_sampling_matches_plain_and_ignores_batch_mates(llogos, model_dirs):
    name = "qwen3"
    cfg = TINY[name]
    w = read_weights(llogos, model_dirs[name])
    prompts = random_tokens(cfg["vocab_size"], [1, 7, 16, 31], 32)
    model = L.LlogosModel.load(model_dirs[name], dtype="float32", max_context=256, max_batch=4)
    params = L.GenerationParams(max_tokens=12, temperature=0.8, top_k=0, top_p=1.0, repetition_penalty=1.0,
                                seed=1234, stop_tokens=())
    r = model.generate(prompts, params)
    again = model.generate(prompts, params)
    assert r.tokens == again.tokens
    plain_params = dict(temperature=0.8)
    for i, p in enumerate(prompts):
        margins = []
        want = plain_generate(w, cfg, p, 12, params=plain_params, seed=1234, seq_id=i, margins=margins)
        assert same_draws(r.tokens[i], want, margins), (i, r.tokens[i], want, margins)
    other = model.generate(prompts, L.GenerationParams(max_tokens=12, temperature=0.8, top_k=0, top_p=1.0,
                                                       repetition_penalty=1.0, seed=99, stop_tokens=()))
    assert other.tokens != r.tokens
    # with the reference's default filters and penalties on
    full = L.GenerationParams(max_tokens=10, seed=5, stop_tokens=())
    rf = model.generate(prompts[:2], full)
    for i, p in enumerate(prompts[:2]):
        margins = []
        want = plain_generate(w, cfg, p, 10, params=dict(temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.1),
                              seed=5, seq_id=i, margins=margins)
        assert same_draws(rf.tokens[i], want, margins), (i, rf.tokens[i], want, margins)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_one_step_ahead_changes_no_token(llogos, model_dirs, dtype):
    """Greedy and seeded sampling without penalties run one step ahead of the tokens the host has read
    (the next step takes them from the device); with the switch off the host reads every token first.
    Stop tokens that really occur, unequal prompts, two batches."""
    name = "qwen2"
    cfg = TINY[name]
    prompts = random_tokens(cfg["vocab_size"], [5, 9, 13, 1, 30, 64, 3], 41)
    model = L.LlogosModel.load(model_dirs[name], dtype=dtype, max_context=256, max_batch=4)
    free = L.GenerationParams.greedy_params(24, stop_tokens=())
    base = model.generate(prompts, free, run_ahead=False)
    # stop at tokens that the free run produced in its middle, so that sequences end at different steps
    stop = sorted({t[len(t) // 2] for t in base.tokens[:3]})
    for params in (L.GenerationParams.greedy_params(24, stop_tokens=stop),
                   L.GenerationParams(max_tokens=17, temperature=0.9, top_k=20, top_p=0.9, repetition_penalty=1.0,
                                      seed=77, stop_tokens=stop),
                   # penalties: the recent tokens live on the device and the sampler extends them itself
                   L.GenerationParams(max_tokens=24, seed=5, stop_tokens=stop),
                   L.GenerationParams(max_tokens=24, temperature=0.0, repetition_penalty=1.4, frequency_penalty=0.3,
                                      penalty_count=5, stop_tokens=stop)):
        slow = model.generate(prompts, params, run_ahead=False)
        fast = model.generate(prompts, params)
        assert fast.tokens == slow.tokens and fast.finish_reasons == slow.finish_reasons
        if params.greedy:
            assert "stop" in slow.finish_reasons and "length" in slow.finish_reasons
        assert fast.decode_steps >= slow.decode_steps
        assert not model.engine.cache.slots.live()
        model.engine.cache.audit()


def test_bfloat16_generation_runs_and_is_deterministic(model_dirs):
    cfg = TINY["llama"]
    prompts = random_tokens(cfg["vocab_size"], [5, 9, 13], 33)
    model = L.LlogosModel.load(model_dirs["llama"], dtype="bfloat16", max_context=128, max_batch=3)
    params = L.GenerationParams.greedy_params(8, stop_tokens=())
    a, b = model.generate(prompts, params), model.generate(prompts, params)
    assert a.tokens == b.tokens and all(len(t) == 8 for t in a.tokens)
    assert a.decode_tokens_per_second > 0 and a.prefill_tokens_per_second > 0


def test_benchmark_through_the_entry_point(model_dirs):
    """``LlogosModel.benchmark``: the reference's counts and rates, and the bytes and flops the steps had by the
    model's own sizes (worked out here from the configuration)."""
    cfg = TINY["llama"]
    model = L.LlogosModel.load(model_dirs["llama"], dtype="bfloat16", max_context=128, max_batch=3)
    prompts = random_tokens(cfg["vocab_size"], [20, 33, 7], 9)
    b = model.benchmark(prompts, 10)
    assert isinstance(b, L.BenchmarkResult)
    assert b.prompt_tokens == 60 and b.generated_tokens == 30 and b.batch == 3 and b.final_lengths == [30, 43, 17]
    assert b.decode_steps == 9 and b.decode_tokens_per_second > 0 and b.prefill_tokens_per_second > 0
    h, i, v, layers = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    matrix = layers * (h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * i)
    kv_per_token = layers * 2 * nkv * hd * 2
    # step k (1..9) reads every matrix and the head once, and prompt + k keys and values per sequence
    want = (matrix + v * h) * 2 + kv_per_token * sum(n + k for n in (20, 33, 7) for k in range(1, 10)) / 9
    assert abs(b.decode_bytes_per_step - want) < 1e-6 * want
    pairs = sum(n * (n + 1) / 2 for n in (20, 33, 7))
    assert abs(b.prompt_step_flops - (2.0 * 60 * matrix + 2.0 * 3 * v * h + layers * 4 * nh * hd * pairs)) < 1e-6 * b.prompt_step_flops
    assert 0 < b.decode_fraction_of_copy_bandwidth < 1 and 0 < b.prompt_fraction_of_matrix_peak < 1
    assert not model.engine.cache.slots.live()
    # a sequence rolled back through the entry point continues as if the dropped tokens had never come
    s = model.open()
    full = model.step([(s, prompts[1])])[0]
    model.truncate(s, 20)
    again = model.step([(s, prompts[1][20:])])[0]
    assert float((full - again).abs().max()) <= 1.5e-2 * float(full.abs().max())      # another cut of the tokens: rounding only
    model.close(s)


def test_command_line(model_dirs):
    env = dict(os.environ, PYTHONPATH=ROOT)
    base = [sys.executable, "-m", "llogos_b200", "--model", model_dirs["llama"], "--dtype", "float32"]
    p = subprocess.run(base + ["--prompt-ids", "5,17,3", "-n", "6", "-t", "0", "--repeat-penalty", "1.0", "--max-context", "128"],
                       capture_output=True, text=True, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stderr
    toks = [int(x) for x in p.stdout.split()]
    assert 1 <= len(toks) <= 6 and "prefill: 3 tokens" in p.stderr and "decode:" in p.stderr
    p = subprocess.run(base + ["--bench", "-n", "5", "--max-context", "128"], capture_output=True, text=True, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stderr
    assert "Prefill:" in p.stderr and "Decode:" in p.stderr and "Load:" in p.stderr
    # a workload by numbers: three sequences with prompts of 20 to 60 tokens, decoded until each holds 100
    p = subprocess.run(base + ["--bench", "--batch", "3", "--prompt-len", "20:60", "--context", "100", "--seed", "4"],
                       capture_output=True, text=True, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stderr
    import re
    m = re.search(r"Decode:\s+(\d+) tokens", p.stderr)
    pre = re.search(r"Prefill:\s+(\d+) tokens", p.stderr)
    assert m and pre and int(m.group(1)) + int(pre.group(1)) == 300          # every sequence reached the context
    assert "longest sequence at the end 100 tokens" in p.stderr
    assert re.search(r"Decode step: .* GB to read per step, .* GB/s = .* % of", p.stderr), p.stderr
    assert re.search(r"Prompt step: .* TFLOP/s = .* % of", p.stderr), p.stderr
    p = subprocess.run(base + ["--bench", "--context", "4096"], capture_output=True, text=True, env=env, cwd=ROOT)
    assert p.returncode == 2 and "max_position_embeddings" in p.stderr
    p = subprocess.run([sys.executable, "-m", "llogos_b200", "--prompt", "hi"], capture_output=True, text=True, env=env, cwd=ROOT)
    assert p.returncode == 2 and "--model" in p.stderr


def test_command_line_prompt_file_and_ignore_eos(model_dirs, tmp_path):
    """Prompts from a file, one per line; with --ignore-eos no sequence stops before its token limit."""
    env = dict(os.environ, PYTHONPATH=ROOT)
    f = tmp_path / "prompts.txt"
    f.write_text("5, 17, 3\n9 8 7 6\n\n12\n")
    base = [sys.executable, "-m", "llogos_b200", "--model", model_dirs["qwen3"], "--dtype", "float32",
            "--prompt-file", str(f), "-n", "20", "-t", "0.9", "--top-k", "0", "--top-p", "1.0", "--seed", "3",
            "--max-context", "128"]
    p = subprocess.run(base + ["--ignore-eos", "--min-p", "0.01", "--presence-penalty", "0.1"],
                       capture_output=True, text=True, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stderr
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 3 and all(len(l.split()) == 20 for l in lines)
    stop = set(TINY["qwen3"]["eos_token_id"])
    assert not any(int(t) in stop for l in lines for t in l.split())
    assert "prefill: 8 tokens" in p.stderr

"""Trace replay as a user runs it: bin/trace_run as a child process, steps on its standard
input, logits from the files it writes, compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from compare import reference
from conftest import ROOT, TINY, read_weights, random_tokens

pytestmark = pytest.mark.gpu
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class Replay:
    def __init__(self, model_dir, dtype, out_dir, max_tokens, extra=(), env=None):
        self.out = out_dir
        self.p = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
             "--out", out_dir, "--max-tokens", str(max_tokens), *extra],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        self.n = 0

    def step(self, entries, end=()):
        rec = {"step": self.n, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w in entries], "end": list(end)}
        self.p.stdin.write(json.dumps(rec) + "\n")
        self.p.stdin.flush()
        line = self.p.stdout.readline().strip()
        assert line == f"done {self.n}", line
        path = os.path.join(self.out, f"{self.n}.f32")
        self.n += 1
        if not any(w for _, _, w in entries):
            assert not os.path.exists(path)
            return None
        return np.fromfile(path, dtype="<f4")

    def finish(self):
        self.p.stdin.close()
        assert self.p.wait(timeout=60) == 0


def check(ref, got, positions, dtype, what):
    ref.check(torch.from_numpy(got.astype(np.float32)), positions, TORCH[dtype], what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_replay_schedules(llogos, model_dirs, tmp_path, name, dtype):
    cfg = TINY[name]
    vocab = cfg["vocab_size"]
    w = read_weights(llogos, model_dirs[name])
    seqs = random_tokens(vocab, [70, 33, 129, 40], 21)
    refs = [reference(model_dirs[name], w, cfg, s) for s in seqs]
    r = Replay(model_dirs[name], dtype, str(tmp_path / "out"), max_tokens=64 * 6)
    # each request alone and whole, all places wanted
    for i, s in enumerate(seqs):
        got = r.step([(f"w{i}", s, list(range(len(s))))], end=[f"w{i}"]).reshape(len(s), vocab)
        check(refs[i], got, range(len(s)), dtype, ("whole", i))
    # the last 32 tokens one by one
    for i, s in enumerate(seqs):
        cut = len(s) - 32
        assert r.step([(f"d{i}", s[:cut], [])]) is None
        for p in range(cut, len(s)):
            got = r.step([(f"d{i}", [s[p]], [0])], end=[f"d{i}"] if p == len(s) - 1 else [])
            check(refs[i], got, [p], dtype, ("decode", i, p))
    # batches of unequal lengths, one after another; 6 pages hold seqs 0, 1 and 3, then seq 2 with 1
    for batch in ([0, 1, 3], [2, 1]):
        cut = {i: len(seqs[i]) - 4 - 3 * k for k, i in enumerate(batch)}
        got = r.step([(f"b{i}", seqs[i][:cut[i]], [cut[i] - 1]) for i in batch]).reshape(len(batch), vocab)
        for k, i in enumerate(batch):
            check(refs[i], got[k], [cut[i] - 1], dtype, ("batch prompt", i))
        pos, live = dict(cut), list(batch)
        while live:
            ending = [i for i in live if pos[i] == len(seqs[i]) - 1]
            got = r.step([(f"b{i}", [seqs[i][pos[i]]], [0]) for i in live], end=[f"b{i}" for i in ending])
            got = got.reshape(len(live), vocab)
            for k, i in enumerate(live):
                check(refs[i], got[k], [pos[i]], dtype, ("batch decode", i, pos[i]))
                pos[i] += 1
            live = [i for i in live if i not in ending]
    r.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["qwen3", "wide"])
def test_replay_of_portions_and_mixed_steps(llogos, model_dirs, tmp_path, name, dtype):
    """The replay program takes any cut of a request into steps: a prompt in portions (300 tokens on a length
    of 70, one token alone, 257 on 371), then a second request that joins with its whole prompt while the first
    goes on by one token, both windows of the configurations shorter than the portions."""
    cfg = TINY[name]
    vocab = cfg["vocab_size"]
    w = read_weights(llogos, model_dirs[name])
    a, b = random_tokens(vocab, [640, 200], 23)
    ra, rb = reference(model_dirs[name], w, cfg, a), reference(model_dirs[name], w, cfg, b)
    r = Replay(model_dirs[name], dtype, str(tmp_path / "out"), max_tokens=64 * 15)
    done = 0
    for n in (70, 300, 1, 257):
        got = r.step([("a", a[done:done + n], list(range(n)))]).reshape(n, vocab)
        check(ra, got, range(done, done + n), dtype, ("portion", n, "on", done))
        done += n
    got = r.step([("a", a[done:done + 1], [0]), ("b", b[:190], [0, 100, 189])]).reshape(4, vocab)
    check(ra, got[0], [done], dtype, ("one token beside a prompt",))
    check(rb, got[1:], [0, 100, 189], dtype, ("a prompt beside one token",))
    done += 1
    got = r.step([("b", b[190:], list(range(10))), ("a", a[done:done + 11], [10])], end=["a", "b"]).reshape(11, vocab)
    check(rb, got[:10], range(190, 200), dtype, ("second portion of b",))
    check(ra, got[10], [done + 10], dtype, ("a goes on",))
    r.finish()


def test_replay_with_a_cache_larger_than_the_models_positions(llogos, tmp_path):
    """--max-tokens sizes the cache for all live requests together; it may exceed what one request can reach
    (max_position_embeddings), and two requests then share it."""
    cfg = dict(TINY["llama"], max_position_embeddings=128)
    d = str(tmp_path / "m")
    llogos.weights.write_random_model(d, cfg, seed=5, std=0.15)
    w = read_weights(llogos, d)
    a, b = random_tokens(cfg["vocab_size"], [120, 100], 24)
    ra, rb = reference(d, w, cfg, a), reference(d, w, cfg, b)
    r = Replay(d, "float32", str(tmp_path / "out"), max_tokens=256)
    got = r.step([("a", a, [0, 119]), ("b", b, [99])], end=["a", "b"]).reshape(3, cfg["vocab_size"])
    check(ra, got[:2], [0, 119], "float32", ("a",))
    check(rb, got[2], [99], "float32", ("b",))
    r.finish()


def test_replay_rejects_nonsense(model_dirs, tmp_path):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["llama"],
                        "--dtype", "float16", "--out", str(tmp_path), "--max-tokens", "64"],
                       input="", capture_output=True, text=True)
    assert p.returncode != 0 and "float16" in p.stderr
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path),
                        "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "64"],
                       input="", capture_output=True, text=True)
    assert p.returncode != 0 and "config.json" in p.stderr


def test_replay_of_an_architecture_that_a_plugin_module_registers(llogos, tmp_path):
    """The replay program knows an architecture that a module named in LLOGOS_PLUGINS registers: a model folder whose
    config.json names it is written here (in a child process that has the plugin too), replayed whole and then
    with its last tokens one by one, and compared with the plain implementation of the dense decoder that the
    plugin's architecture is built from."""
    (tmp_path / "toy_plugin.py").write_text(
        "import importlib\n"
        "C = importlib.import_module('daisi-llogos_b200.config')\n"
        "R = importlib.import_module('daisi-llogos_b200.config.registry')\n"
        "C.register_architecture('PluginToyLM', R._dense_reader(qk_norm=True, force_bias=False), C.dense_decoder_spec)\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(tmp_path), ROOT, os.environ.get("PYTHONPATH", "")]),
               LLOGOS_PLUGINS="toy_plugin")
    cfg = dict(TINY["qwen3"], architectures=["PluginToyLM"])
    d = str(tmp_path / "model")
    code = ("import json, sys, llogos_b200 as L; "
            "L.weights.write_random_model(sys.argv[1], json.loads(sys.argv[2]), seed=5, std=0.2, norm_std=0.1)")
    subprocess.run([sys.executable, "-c", code, d, json.dumps(cfg)], check=True, env=env, cwd=str(tmp_path))
    # this process does not know the name: the plain implementation reads the folder as the dense decoder it is
    plain_cfg = dict(cfg, architectures=TINY["qwen3"]["architectures"])
    w = read_weights(llogos, d)
    vocab = cfg["vocab_size"]
    s = random_tokens(vocab, [90], 29)[0]
    ref = reference(d, w, plain_cfg, s)
    for dtype in ("float32", "bfloat16"):
        r = Replay(d, dtype, str(tmp_path / f"out_{dtype}"), max_tokens=64 * 4, env=env)
        got = r.step([("a", s, list(range(len(s))))], end=["a"]).reshape(len(s), vocab)
        check(ref, got, range(len(s)), dtype, ("plugin whole",))
        assert r.step([("b", s[:80], [])]) is None
        for p in range(80, len(s)):
            got = r.step([("b", [s[p]], [0])], end=["b"] if p == len(s) - 1 else [])
            check(ref, got, [p], dtype, ("plugin decode", p))
        r.finish()

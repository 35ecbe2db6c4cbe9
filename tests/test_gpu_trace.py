"""Trace replay as a user runs it: bin/trace_run as a child process, steps on its standard
input, logits from the files it writes, compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model as P
from conftest import ROOT, TINY, read_weights, random_tokens

pytestmark = pytest.mark.gpu
REL_TOL = {"float32": 2e-5, "bfloat16": 4e-2}


class Replay:
    def __init__(self, model_dir, dtype, out_dir, max_tokens, extra=()):
        self.out = out_dir
        self.p = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
             "--out", out_dir, "--max-tokens", str(max_tokens), *extra],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
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


def close(got, ref, dtype, scale):
    """``scale``: the largest |logit| of the request's whole reference; bfloat16 noise is absolute
    across a request's positions, so every position is judged against the same scale."""
    ref = ref.double().numpy()
    err = float(np.abs(got.astype(np.float64) - ref).max())
    return err <= REL_TOL[dtype] * scale, err


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_replay_schedules(llogos, model_dirs, tmp_path, name, dtype):
    cfg = TINY[name]
    vocab = cfg["vocab_size"]
    w = read_weights(llogos, model_dirs[name])
    seqs = random_tokens(vocab, [70, 33, 129, 40], 21)
    refs = [P.forward(w, cfg, s) for s in seqs]
    scales = [float(x.abs().max()) for x in refs]
    r = Replay(model_dirs[name], dtype, str(tmp_path / "out"), max_tokens=64 * 6)
    # each request alone and whole, all places wanted
    for i, s in enumerate(seqs):
        got = r.step([(f"w{i}", s, list(range(len(s))))], end=[f"w{i}"]).reshape(len(s), vocab)
        ok, err = close(got, refs[i], dtype, scales[i])
        assert ok, ("whole", i, err)
    # the last 32 tokens one by one
    for i, s in enumerate(seqs):
        cut = len(s) - 32
        assert r.step([(f"d{i}", s[:cut], [])]) is None
        for p in range(cut, len(s)):
            got = r.step([(f"d{i}", [s[p]], [0])], end=[f"d{i}"] if p == len(s) - 1 else [])
            ok, err = close(got, refs[i][p], dtype, scales[i])
            assert ok, ("decode", i, p, err)
    # batches of unequal lengths, one after another; 6 pages hold seqs 0, 1 and 3, then seq 2 with 1
    for batch in ([0, 1, 3], [2, 1]):
        cut = {i: len(seqs[i]) - 4 - 3 * k for k, i in enumerate(batch)}
        got = r.step([(f"b{i}", seqs[i][:cut[i]], [cut[i] - 1]) for i in batch]).reshape(len(batch), vocab)
        for k, i in enumerate(batch):
            ok, err = close(got[k], refs[i][cut[i] - 1], dtype, scales[i])
            assert ok, ("batch prompt", i, err)
        pos, live = dict(cut), list(batch)
        while live:
            ending = [i for i in live if pos[i] == len(seqs[i]) - 1]
            got = r.step([(f"b{i}", [seqs[i][pos[i]]], [0]) for i in live], end=[f"b{i}" for i in ending])
            got = got.reshape(len(live), vocab)
            for k, i in enumerate(live):
                ok, err = close(got[k], refs[i][pos[i]], dtype, scales[i])
                assert ok, ("batch decode", i, pos[i], err)
                pos[i] += 1
            live = [i for i in live if i not in ending]
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

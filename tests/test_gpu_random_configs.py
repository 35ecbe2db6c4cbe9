"""Randomly drawn configurations of the architecture against the plain implementation, in float32 and
bfloat16: head sizes in steps of 16, odd head counts and groups, widths and vocabularies that are no
power of two, windows, rotation scaling, bias and per-head norms.  Each one is run whole (prompts of
1 to about 700 tokens, so that every tile size of the prompt kernels runs), then as one batch of
unequal prompts that is decoded to its ends, shorter requests leaving earlier.  The weights' spread
follows the width (1.2 / sqrt(hidden)) so that activations stay of order one, as in trained models."""
import random

import pytest
import torch

from compare import Reference
from conftest import read_weights

pytestmark = pytest.mark.gpu

SEEDS = list(range(24))          # a plain range: no seed is left out


def draw_config(rng):
    arch = rng.choice(["LlamaForCausalLM", "Qwen2ForCausalLM", "Qwen3ForCausalLM"])
    nkv = rng.choice([1, 2, 3, 4])
    layers = rng.choice([1, 2, 3])
    cfg = {"architectures": [arch], "num_hidden_layers": layers,
           "hidden_size": rng.choice([64, 72, 88, 136, 200, 264]),
           "num_attention_heads": nkv * rng.choice([1, 2, 3, 4, 5, 8]), "num_key_value_heads": nkv,
           "head_dim": rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 128, 64]),
           "intermediate_size": rng.choice([48, 100, 176, 264, 520]),
           "vocab_size": rng.choice([130, 257, 1000, 1031]),
           "rope_theta": rng.choice([1e4, 5e5, 1e6]), "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-5]),
           "max_position_embeddings": 4096, "tie_word_embeddings": rng.random() < 0.4}
    if rng.random() < 0.4:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0]), "low_freq_factor": 1.0,
                               "high_freq_factor": 4.0,
                               "original_max_position_embeddings": rng.choice([64, 256])}
    if arch == "Qwen3ForCausalLM":
        cfg["attention_bias"] = rng.random() < 0.5
        if rng.random() < 0.6:
            cfg["sliding_window"] = rng.choice([17, 64, 100, 300])
            cfg["layer_types"] = [rng.choice(["full_attention", "sliding_attention"]) for _ in range(layers)]
    if arch == "Qwen2ForCausalLM" and rng.random() < 0.5:
        cfg.update(use_sliding_window=True, sliding_window=rng.choice([33, 128, 260]),
                   max_window_layers=rng.randrange(0, layers + 1))
    return cfg


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(llogos, tmp_path, seed):
    rng = random.Random(seed)
    check_configuration(llogos, tmp_path, draw_config(rng), rng, seed)


# widths that are no multiple of 8 (the tensor-core product refuses them: 16-byte rows for TMA) or of 4
# (no vector accesses in the norms), with an odd intermediate size and vocabulary
ODD = [
    {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 102, "num_attention_heads": 6,
     "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 99, "vocab_size": 257, "rope_theta": 1e4,
     "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "attention_bias": True},
    {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 100, "num_attention_heads": 5,
     "num_key_value_heads": 5, "head_dim": 128, "intermediate_size": 130, "vocab_size": 1031, "rope_theta": 5e5,
     "rms_norm_eps": 1e-6, "max_position_embeddings": 2048, "tie_word_embeddings": False},
]


@pytest.mark.parametrize("which", range(len(ODD)))
def test_widths_that_fit_no_vector_access(llogos, tmp_path, which):
    check_configuration(llogos, tmp_path, ODD[which], random.Random(200 + which), 200 + which)


def check_configuration(llogos, tmp_path, cfg, rng, seed):
    lens = [rng.choice([1, 5, 63, 64, 65]), rng.randrange(100, 300), rng.randrange(256, 700),
            rng.randrange(2, 90), rng.randrange(500, 640)]
    d = str(tmp_path)
    llogos.weights.write_random_model(d, cfg, seed=seed, std=1.2 / cfg["hidden_size"] ** 0.5,
                                      norm_std=0.1, bias_std=0.1)
    w = read_weights(llogos, d)
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    refs = [Reference(w, cfg, s) for s in seqs]
    for dtype in (torch.float32, torch.bfloat16):
        model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
        eng = llogos.engine.Engine(model, max_tokens=64 * 40)
        for i, s in enumerate(seqs):                                     # whole, alone
            slot = eng.open()
            lg = eng.step([(slot, s)], [list(range(len(s)))])
            refs[i].check(lg, range(len(s)), dtype, (cfg, dtype, "whole", len(s)))
            eng.close(slot)
        order = list(range(len(seqs)))                                   # one batch, cut before the ends
        rng.shuffle(order)
        slots = {i: eng.open() for i in order}
        cut = {i: max(1, len(seqs[i]) - rng.randrange(1, 40)) for i in order}
        lg = eng.step([(slots[i], seqs[i][:cut[i]]) for i in order], [[cut[i] - 1] for i in order])
        for k, i in enumerate(order):
            refs[i].check(lg[k], [cut[i] - 1], dtype, (cfg, dtype, "batch prompt", i, cut[i]))
        pos = dict(cut)
        live = []
        for i in order:
            if pos[i] < len(seqs[i]):
                live.append(i)
            else:
                eng.close(slots[i])
        while live:                                                      # decoded to their ends
            lg = eng.step([(slots[i], [seqs[i][pos[i]]]) for i in live])
            for k, i in enumerate(live):
                refs[i].check(lg[k], [pos[i]], dtype, (cfg, dtype, "decode", i, pos[i], "batch of", len(live)))
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.close(slots[i])
                live.remove(i)
        eng.cache.audit()
        assert eng.cache.slots.free_count == eng.cache.slots.n_slots

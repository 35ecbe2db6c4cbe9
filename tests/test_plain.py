"""The plain implementation against hand values and identities (no GPU).

In the spirit of the reference's op tests (tests/Daisi.Llogos.Tests/Cpu/MathOpsTests.cs: RMSNorm
known values :130-185, softmax sums to one :201, rotation keeps position 0 and norms :319-388)."""
import math

import pytest
import torch

import plain_model as P
from conftest import TINY, read_weights, random_tokens


def test_rms_norm_known_values():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    out = P.rms_norm(x, w, 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]], dtype=torch.float64))
    # eps is added to the mean, inside the root
    out = P.rms_norm(torch.tensor([[0.0, 0.0]]), w, 1e-6)
    assert torch.all(out == 0)
    out = P.rms_norm(torch.tensor([[1.0, 1.0]]), torch.ones(2), 3.0)
    assert torch.allclose(out, torch.full((1, 2), 0.5, dtype=torch.float64))


def test_rope_identities():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 3, 16, generator=g)
    inv = P.rope_inverse_frequencies(16, 10000.0, None)
    assert inv[0] == 1.0 and abs(float(inv[-1]) - 10000 ** (-14 / 16)) < 1e-15
    for pairing in ("half", "adjacent"):
        r0 = P.rope_rotate(x, [0] * 5, inv, pairing)
        assert torch.allclose(r0, x.double())
        r = P.rope_rotate(x, [0, 1, 7, 100, 5000], inv, pairing)
        assert torch.allclose(r.norm(dim=-1), x.double().norm(dim=-1))
    # relative property: <R(p) q, R(p') k> depends on p - p' only
    q, k = x[0:1, 0:1], x[1:2, 0:1]
    a = (P.rope_rotate(q, [10], inv, "half") * P.rope_rotate(k, [3], inv, "half")).sum()
    b = (P.rope_rotate(q, [107], inv, "half") * P.rope_rotate(k, [100], inv, "half")).sum()
    assert abs(float(a - b)) < 1e-9
    # the two pairings are the same rotation up to a permutation of the head's elements
    perm = torch.tensor([i // 2 + (i % 2) * 8 for i in range(16)])     # adjacent index -> half index
    ra = P.rope_rotate(x[..., perm], [1, 2, 3, 4, 5], inv, "adjacent")
    rh = P.rope_rotate(x, [1, 2, 3, 4, 5], inv, "half")
    assert torch.allclose(ra, rh[..., perm])
    # partial rotation leaves the tail alone
    inv8 = P.rope_inverse_frequencies(8, 10000.0, None)
    r = P.rope_rotate(x, [9] * 5, inv8, "half")
    assert torch.equal(r[..., 8:], x.double()[..., 8:])


def test_llama3_frequency_scaling_bands():
    sc = {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base = P.rope_inverse_frequencies(48, 50000.0, None)
    scaled = P.rope_inverse_frequencies(48, 50000.0, sc)
    wav = 2 * math.pi / base
    high, low, mid = wav < 64 / 4, wav > 64 / 1, (wav >= 16) & (wav <= 64)
    assert high.any() and low.any() and mid.any()           # all three bands occur
    assert torch.equal(scaled[high], base[high])
    assert torch.allclose(scaled[low], base[low] / 4)
    assert torch.all((scaled[mid] <= base[mid]) & (scaled[mid] >= base[mid] / 4))


def test_attention_rows_are_convex_combinations_and_causal():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(9, n, 8, generator=g) for n in (4, 2, 2))
    o = P.attention(q, k, v, 0.5)
    assert torch.allclose(o[0, 0], v[0, 0].double()) and torch.allclose(o[0, 3], v[0, 1].double())
    k2, v2 = k.clone(), v.clone()
    k2[5:] += 3
    v2[5:] -= 2
    assert torch.allclose(P.attention(q, k2, v2, 0.5)[:5], o[:5])       # the future does not matter
    assert torch.allclose(P.attention(q, k, v, 0.5, window=9), o)       # a window of the whole length
    ow = P.attention(q, k, v, 0.5, window=1)
    assert torch.allclose(ow[:, 0], v[:, 0].double())                   # W = 1: only the own key
    # one score made to stand out picks that value
    q3, k3 = q.clone() * 0, k.clone() * 0
    q3[8, 2, 0] = 50.0
    k3[3, 1, 0] = 50.0
    assert torch.allclose(P.attention(q3, k3, v, 1.0)[8, 2], v[3, 1].double(), atol=1e-9)
    assert not torch.allclose(P.attention(q3, k3, v, 1.0, window=5)[8, 2], v[3, 1].double(), atol=1e-3)


def test_swiglu_by_hand():
    x = torch.tensor([[1.0, -2.0]])
    wg = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]])
    wu = torch.tensor([[2.0, 0.0], [0.0, 1.0], [1.0, 0.0]])
    wd = torch.tensor([[1.0, 1.0, 1.0]])
    silu = lambda z: z / (1 + math.exp(-z))
    want = silu(1.0) * 2 + silu(-2.0) * -2 + silu(-1.0) * 1
    assert abs(float(P.swiglu(x, wg, wu, wd)) - want) < 1e-12


@pytest.mark.parametrize("name", list(TINY))
def test_model_is_causal_and_deterministic(llogos, model_dirs, name):
    cfg, w = TINY[name], read_weights(llogos, model_dirs[name])
    a, = random_tokens(cfg["vocab_size"], [40], 3)
    la = P.forward(w, cfg, a)
    assert la.shape == (40, cfg["vocab_size"]) and torch.isfinite(la).all()
    b = list(a)
    b[30] = (b[30] + 1) % cfg["vocab_size"]
    lb = P.forward(w, cfg, b)
    assert torch.equal(la[:30], lb[:30]) and not torch.allclose(la[30:], lb[30:])
    assert torch.equal(P.forward(w, cfg, a[:17]), la[:17]) or torch.allclose(P.forward(w, cfg, a[:17]), la[:17], atol=1e-12)


def test_window_changes_logits_only_beyond_it(llogos, model_dirs):
    cfg, w = TINY["qwen3"], read_weights(llogos, model_dirs["qwen3"])
    a, = random_tokens(cfg["vocab_size"], [60], 4)
    full = dict(cfg, layer_types=["full_attention"] * 3)
    lw, lf = P.forward(w, cfg, a), P.forward(w, full, a)
    assert torch.allclose(lw[:24], lf[:24], atol=1e-12) and not torch.allclose(lw[24:], lf[24:], atol=1e-6)


def test_sampling_pipeline_by_hand():
    logits = [2.0, 1.0, 0.0, -1.0]
    p = P.sampling_distribution(logits, temperature=1.0)
    e = torch.tensor([math.exp(x) for x in logits], dtype=torch.float64)
    assert torch.allclose(p, e / e.sum())
    assert P.sampling_distribution(logits, temperature=0.0).tolist() == [1, 0, 0, 0]
    assert P.sampling_distribution([1.0, 3.0, 3.0], temperature=0.0).tolist() == [0, 1, 0]     # first maximum
    p = P.sampling_distribution(logits, temperature=1.0, top_k=2)
    assert p[2] == 0 and p[3] == 0 and abs(float(p[0] / p[1]) - math.e) < 1e-12
    p = P.sampling_distribution(logits, temperature=0.5, top_k=2)
    assert abs(float(p[0] / p[1]) - math.e ** 2) < 1e-9
    p = P.sampling_distribution(logits, temperature=1.0, top_p=0.7)       # 0.644 <= 0.7 < 0.644 + 0.237
    assert (p > 0).tolist() == [True, True, False, False] and abs(float(p.sum()) - 1) < 1e-12
    p = P.sampling_distribution(logits, temperature=1.0, min_p=0.2)       # keep p >= 0.2 * p_max
    assert (p > 0).tolist() == [True, True, False, False]
    p = P.sampling_distribution(logits, temperature=1.0, repetition_penalty=2.0, previous=[0, 0, 3])
    q = P.sampling_distribution([0.5, 1.0, 0.0, -2.0], temperature=1.0)   # token 0 twice, token 3 once
    assert torch.allclose(p, q)
    p = P.sampling_distribution(logits, temperature=1.0, frequency_penalty=0.5, presence_penalty=0.25,
                                repetition_penalty=1.0, previous=[1, 1])
    assert torch.allclose(p, P.sampling_distribution([2.0, -0.25, 0.0, -1.0], temperature=1.0))
    p = P.sampling_distribution(logits, temperature=1.0, banned=[0])
    assert p[0] == 0 and abs(float(p.sum()) - 1) < 1e-12


def test_draw_and_uniform():
    probs = torch.tensor([0.1, 0.0, 0.6, 0.3], dtype=torch.float64)
    assert [P.draw(probs, u) for u in (0.0, 0.0999, 0.1, 0.69, 0.7, 0.9999)] == [0, 0, 2, 2, 3, 3]
    us = [P.uniform_of(7, s, t) for s in range(20) for t in range(50)]
    assert all(0 <= u < 1 for u in us) and len(set(us)) > 990 and abs(sum(us) / len(us) - 0.5) < 0.03
    assert P.uniform_of(7, 3, 4) == P.uniform_of(7, 3, 4) != P.uniform_of(8, 3, 4)

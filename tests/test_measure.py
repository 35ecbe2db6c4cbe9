"""The numbers a step is held against: bytes a decode step must read, operations of a prompt step, peaks."""
import importlib
import json

import torch

import cpu_ops
from conftest import TINY


def test_costs_follow_the_configuration(llogos):
    m = importlib.import_module("daisi-llogos_b200.measure")
    for name, cfg in TINY.items():
        model = llogos.weights.build_model(cfg, dtype=torch.bfloat16, device="cpu", ops=cpu_ops)
        c = m.model_costs(model)
        h, i, v, n = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
        q = cfg["num_attention_heads"] * cfg["head_dim"]
        kv = cfg["num_key_value_heads"] * cfg["head_dim"]
        assert c.matrix_params == n * (h * (q + 2 * kv) + q * h + 3 * h * i), name
        assert c.head_params == v * h and c.bytes_per_param == 2
        assert len(c.kv_units) == n and all(per == 2 * kv * 2 for per, _ in c.kv_units)
        assert c.attn_flops_per_pair == n * 4 * q
        # a window bounds what a layer reads of a long sequence
        windows = [w for _, w in c.kv_units]
        lengths = [1000, 10]
        want = (c.matrix_params + c.head_params) * 2 + sum(2 * kv * 2 * (min(x, w) if w else x) for w in windows for x in lengths)
        assert c.decode_step_bytes(lengths) == want
        # one token on an empty sequence: one (query, key) pair per layer and head
        assert c.prompt_step_flops([1]) == 2 * c.matrix_params + 2 * c.head_params + c.attn_flops_per_pair
        assert c.prompt_step_flops([3], [10]) == 6 * c.matrix_params + 2 * c.head_params + c.attn_flops_per_pair * (30 + 6)
    model32 = llogos.weights.build_model(TINY["llama"], dtype=torch.float32, device="cpu", ops=cpu_ops)
    assert m.model_costs(model32).bytes_per_param == 4


def test_peaks_from_a_file_or_the_fallback(tmp_path, monkeypatch):
    m = importlib.import_module("daisi-llogos_b200.measure")
    f = tmp_path / "peaks.json"
    f.write_text(json.dumps({"hbm_gbs": 6000.5, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1300.0}))
    p = m.peaks(str(f))
    assert p == {"hbm_gbs": 6000.5, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1300.0, "source": "measured"}
    monkeypatch.setenv("LLOGOS_PEAKS", str(f))
    assert m.peaks()["hbm_gbs"] == 6000.5
    bad = tmp_path / "bad.json"
    bad.write_text("{not json")
    monkeypatch.setenv("LLOGOS_PEAKS", str(bad))
    assert m.peaks(str(bad))["source"] in ("measured", "fallback")      # falls through to the next candidate
    assert m.FALLBACK_PEAKS["source"] == "fallback"

"""Safetensors input/output, the checked loader and random initialisation (no GPU)."""
import json
import os
import shutil

import pytest
import torch

import cpu_ops
from conftest import INIT, TINY_LLAMA, TINY_QWEN3, read_weights


def test_safetensors_round_trip(llogos, tmp_path):
    W = llogos.weights
    t = {"a.weight": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32),
         "c.f32": torch.randn(4, 2), "d.f16": torch.randn(2, 2).to(torch.float16)}
    path = str(tmp_path / "x.safetensors")
    W.write_safetensors(path, t, {"note": "hi"})
    f = W.SafetensorsFile(path)
    assert set(f.names()) == set(t)
    assert f.metadata["note"] == "hi"
    for n, v in t.items():
        got = f.tensor(n)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)


def test_safetensors_is_readable_by_the_safetensors_package(llogos, tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(6, 4).to(torch.bfloat16), "v": torch.randn(3)}
    path = str(tmp_path / "y.safetensors")
    llogos.weights.write_safetensors(path, t)
    back = st.load_file(path)
    assert all(torch.equal(back[n], t[n]) for n in t)
    st.save_file(t, str(tmp_path / "z.safetensors"))
    f = llogos.weights.SafetensorsFile(str(tmp_path / "z.safetensors"))
    assert all(torch.equal(f.tensor(n), t[n]) for n in t)


def test_bad_files(llogos, tmp_path):
    W = llogos.weights
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(W.SafetensorsError):
        W.SafetensorsFile(str(p))
    p = tmp_path / "hdr.safetensors"
    p.write_bytes((1000).to_bytes(8, "little") + b"{}")
    with pytest.raises(W.SafetensorsError):
        W.SafetensorsFile(str(p))
    with pytest.raises(W.SafetensorsError):
        W.ModelFiles(str(tmp_path))


def test_random_model_folder(llogos, model_dirs):
    d = model_dirs["qwen3"]
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["Qwen3ForCausalLM"]
    w = read_weights(llogos, d)
    assert "lm_head.weight" not in w                      # tied
    assert w["model.layers.1.self_attn.q_proj.bias"].shape == (6 * 32,)
    assert w["model.layers.2.self_attn.k_norm.weight"].shape == (32,)
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    norm = w["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.1 and float(norm.std()) > 0.01
    assert abs(float(w["model.layers.0.mlp.up_proj.weight"].float().std()) - INIT["std"]) < 0.02


def test_same_seed_same_weights(llogos, tmp_path):
    W = llogos.weights
    a, b, c = (str(tmp_path / n) for n in "abc")
    W.write_random_model(a, TINY_LLAMA, seed=5)
    W.write_random_model(b, TINY_LLAMA, seed=5)
    W.write_random_model(c, TINY_LLAMA, seed=6)
    wa, wb, wc = (read_weights(llogos, x) for x in (a, b, c))
    assert all(torch.equal(wa[n], wb[n]) for n in wa)
    assert not torch.equal(wa["model.norm.weight"], wc["model.norm.weight"]) or \
        not torch.equal(wa["lm_head.weight"], wc["lm_head.weight"])


def test_loader_binds_and_keeps_types(llogos, model_dirs):
    m = llogos.weights.load_model(model_dirs["llama"], dtype=torch.bfloat16, device="cpu", ops=cpu_ops)
    att = m.blocks[0].parts["mixer"]
    assert att.w_qkv.shape == ((4 + 2 * 2) * 16, 64) and att.w_qkv.dtype == torch.bfloat16
    gu = m.blocks[1].parts["ffn"].w_gate_up          # 176 gate rows, zero rows up to 256, then the up rows likewise
    assert gu.shape == (512, 64)
    w = read_weights(llogos, model_dirs["llama"])
    g, u = w["model.layers.1.mlp.gate_proj.weight"], w["model.layers.1.mlp.up_proj.weight"]
    assert g.shape[0] == 176
    assert torch.equal(gu[0:176], g) and torch.equal(gu[256:432], u)
    assert float(gu[176:256].abs().sum()) == 0 and float(gu[432:512].abs().sum()) == 0
    m32 = llogos.weights.load_model(model_dirs["llama"], dtype=torch.float32, device="cpu", ops=cpu_ops)
    assert m32.blocks[0].parts["mixer"].w_qkv.dtype == torch.float32
    assert torch.equal(m32.blocks[0].parts["mixer"].w_qkv, att.w_qkv.float())


def test_tensor_stored_in_32_bit_stays_so(llogos, model_dirs, tmp_path):
    d = str(tmp_path / "m")
    shutil.copytree(model_dirs["llama"], d)
    w = read_weights(llogos, d)
    w["model.norm.weight"] = w["model.norm.weight"].float() + 1e-4      # not representable in bfloat16
    llogos.weights.write_safetensors(os.path.join(d, "model.safetensors"), w)
    m = llogos.weights.load_model(d, dtype=torch.bfloat16, device="cpu", ops=cpu_ops)
    assert m.final_norm.weight.dtype == torch.float32
    assert torch.equal(m.final_norm.weight, w["model.norm.weight"])
    assert m.embedding.weight.dtype == torch.bfloat16


def test_shards_and_half_precision_files(llogos, model_dirs, tmp_path):
    """A model cut into two shards with an index file, some tensors stored as float16: the same model as
    from one file (float16 becomes bfloat16 where the value allows it exactly here), and an index that
    names a tensor its shard does not hold is an error."""
    import json
    d = str(tmp_path / "sharded")
    os.makedirs(d)
    shutil.copy(os.path.join(model_dirs["qwen3"], "config.json"), d)
    w = read_weights(llogos, model_dirs["qwen3"])
    names = sorted(w)
    first, second = names[: len(names) // 2], names[len(names) // 2:]
    half = {n: (w[n].to(torch.float16) if n.endswith("down_proj.weight") else w[n]) for n in names}
    llogos.weights.write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), {n: half[n] for n in first})
    llogos.weights.write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), {n: half[n] for n in second})
    weight_map = {n: "model-00001-of-00002.safetensors" for n in first}
    weight_map.update({n: "model-00002-of-00002.safetensors" for n in second})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    one = llogos.weights.load_model(model_dirs["qwen3"], dtype=torch.bfloat16, device="cpu", ops=cpu_ops)
    two = llogos.weights.load_model(d, dtype=torch.bfloat16, device="cpu", ops=cpu_ops)
    for a, b in zip(one.blocks, two.blocks):
        assert torch.equal(a.parts["mixer"].w_qkv, b.parts["mixer"].w_qkv)
        assert b.parts["ffn"].w_down.dtype == torch.bfloat16
        # bfloat16 -> float16 -> bfloat16 is exact for values whose exponent float16 can hold
        big = a.parts["ffn"].w_down.float().abs() > 1e-4
        assert torch.equal(a.parts["ffn"].w_down[big], b.parts["ffn"].w_down[big])
    weight_map[first[0]] = "model-00002-of-00002.safetensors"
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    with pytest.raises(Exception, match="is not in"):
        llogos.weights.load_model(d, dtype=torch.bfloat16, device="cpu", ops=cpu_ops)


def test_one_error_lists_everything(llogos, model_dirs, tmp_path):
    d = str(tmp_path / "m")
    shutil.copytree(model_dirs["qwen3"], d)
    w = read_weights(llogos, d)
    del w["model.layers.1.mlp.down_proj.weight"]
    del w["model.layers.2.self_attn.q_norm.weight"]
    w["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(96)             # the architecture has no such bias
    w["model.layers.7.mlp.up_proj.weight"] = torch.zeros(256, 96, dtype=torch.bfloat16)   # there is no layer 7
    w["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(96, 95, dtype=torch.bfloat16)
    llogos.weights.write_safetensors(os.path.join(d, "model.safetensors"), w)
    with pytest.raises(llogos.weights.WeightsError) as e:
        llogos.weights.load_model(d, dtype=torch.float32, device="cpu", ops=cpu_ops)
    msg = str(e.value)
    for needle in ("missing (2)", "model.layers.1.mlp.down_proj.weight", "model.layers.2.self_attn.q_norm.weight",
                   "unexpected (2)", "self_attn.o_proj.bias", "model.layers.7.mlp.up_proj.weight", "wrong shape (1)",
                   "model.layers.0.self_attn.k_proj.weight", "(96, 95)", "(96, 96)"):
        assert needle in msg, (needle, msg)


def test_harmless_extras_are_skipped_with_a_warning(llogos, model_dirs, tmp_path):
    """Checkpoints of this architecture often carry the rotation's frequency buffers, and a tied model may
    carry the output matrix a second time: both are skipped and named in ``load_warnings``.  Any other
    tensor that the model has no place for stays an error, even when nothing is missing."""
    d = str(tmp_path / "m")
    shutil.copytree(model_dirs["qwen3"], d)
    w = read_weights(llogos, d)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    w["lm_head.weight"] = torch.zeros(384, 96, dtype=torch.bfloat16)        # tied model: a second copy
    llogos.weights.write_safetensors(os.path.join(d, "model.safetensors"), w)
    m = llogos.weights.load_model(d, dtype=torch.float32, device="cpu", ops=cpu_ops)
    assert len(m.load_warnings) == 2
    assert any("rotary_emb.inv_freq" in x for x in m.load_warnings) and any("lm_head.weight" in x for x in m.load_warnings)
    assert m.head.weight is m.embedding.weight
    clean = llogos.weights.load_model(model_dirs["qwen3"], dtype=torch.float32, device="cpu", ops=cpu_ops)
    assert clean.load_warnings == []
    # an untied model has a use for lm_head.weight, so there it is no extra; a stray tensor is an error alone
    w["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(96)
    llogos.weights.write_safetensors(os.path.join(d, "model.safetensors"), w)
    with pytest.raises(llogos.weights.WeightsError, match=r"unexpected \(1\)"):
        llogos.weights.load_model(d, dtype=torch.float32, device="cpu", ops=cpu_ops)


def test_random_values_are_a_function_of_seed_name_and_index(llogos):
    """The counter-based generator: fixed values for a fixed key (so that the device kernel, which restates
    the same arithmetic, can be checked against them), moments of a normal distribution, and independence
    of how a tensor is cut into pieces."""
    ri = __import__("importlib").import_module("daisi-llogos_b200.weights.random_init")
    assert ri.splitmix64(0) == 0xE220A8397B1DCDAF
    assert ri.fnv1a64("") == 0xCBF29CE484222325 and ri.fnv1a64("a") == 0xAF63DC4C8601EC8C
    key = ri.tensor_key(7, "model.embed_tokens.weight")
    assert key != ri.tensor_key(8, "model.embed_tokens.weight") != ri.tensor_key(7, "model.norm.weight")
    v = ri.normal_values(key, 200000, 0.0, 1.0)
    assert v.dtype.name == "float32" and abs(float(v.mean())) < 0.01 and abs(float(v.std()) - 1.0) < 0.01
    assert abs(float((v ** 3).mean())) < 0.03 and abs(float((v ** 4).mean()) - 3.0) < 0.1
    part = ri.normal_values(key, 1000, 0.0, 1.0, start=150000)
    assert (part == v[150000:151000]).all()
    shifted = ri.normal_values(key, 1000, 1.0, 0.1)
    assert abs(float(shifted.mean()) - 1.0) < 0.02
    decls = {"a.weight": llogos.parts.TensorDecl((5, 8)), "a.norm": llogos.parts.TensorDecl((8,), "norm")}
    t1 = llogos.weights.random_tensors(decls, 3, std=0.5, norm_std=0.1)
    t2 = llogos.weights.random_tensors(dict(reversed(list(decls.items()))), 3, std=0.5, norm_std=0.1)
    assert torch.equal(t1["a.weight"], t2["a.weight"]) and torch.equal(t1["a.norm"], t2["a.norm"])
    assert t1["a.weight"].dtype == torch.bfloat16 and abs(float(t1["a.norm"].float().mean()) - 1.0) < 0.2


def test_missing_bias_when_config_wants_it(llogos, model_dirs, tmp_path):
    d = str(tmp_path / "m")
    shutil.copytree(model_dirs["llama"], d)
    cfg = json.load(open(os.path.join(d, "config.json")))
    cfg["attention_bias"] = True
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    with pytest.raises(llogos.weights.WeightsError, match="q_proj.bias"):
        llogos.weights.load_model(d, dtype=torch.float32, device="cpu", ops=cpu_ops)


def test_no_gpu_is_an_error_not_a_fallback(llogos, model_dirs):
    if torch.cuda.is_available():
        pytest.skip("this box has a GPU")
    with pytest.raises(Exception, match="CUDA|GPU|cuda"):
        llogos.weights.load_model(model_dirs["llama"], dtype=torch.float32, device="cuda:0")

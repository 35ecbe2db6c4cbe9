"""The stock blocks' launch chain in native code (one call per step) against the same chain driven part by part
from Python: the same kernels with the same arguments, so the logits agree bit for bit, in both precisions, for
prompt steps, mixed steps, decode steps (recorded and not) and a window that wraps."""
import importlib

import pytest
import torch

from conftest import TINY, random_tokens

pytestmark = pytest.mark.gpu


def engines(llogos, model_dir, dtype, monkeypatch, **kw):
    model = llogos.weights.load_model(model_dir, dtype=dtype, device="cuda:0")
    native = llogos.engine.Engine(model, **kw)
    monkeypatch.setenv("LLOGOS_RUNNER", "0")
    by_parts = llogos.engine.Engine(model, **kw)
    monkeypatch.delenv("LLOGOS_RUNNER")
    assert native._runner is not None and by_parts._runner is None
    return native, by_parts


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(TINY))
def test_native_chain_gives_the_parts_bits(llogos, model_dirs, monkeypatch, name, dtype, graphs):
    cfg = TINY[name]
    a, b, c, d, e = random_tokens(cfg["vocab_size"], [300, 90, 41, 300, 290], 61)
    native, by_parts = engines(llogos, model_dirs[name], dtype, monkeypatch, max_tokens=64 * 18, use_graphs=graphs)
    outs = []
    for eng in (native, by_parts):
        got = []
        sa, sb, sc = eng.open(), eng.open(), eng.open()
        got.append(eng.step([(sa, a[:70]), (sb, b[:89])], [list(range(70)), [0, 88]]))
        got.append(eng.step([(sa, a[70:290]), (sb, b[89:90]), (sc, c[:30])], [[0, 219], [0], [29]]))      # mixed, 256 tokens and more
        for j in range(6):                                                                                  # one token each
            got.append(eng.step([(sa, [a[290 + j]]), (sc, [c[30 + j]])]))
        for s in (sa, sb, sc):
            eng.close(s)
        # 590 tokens in one step: above 512 rows the q/k/v product prepares queries and keys itself where it can
        sd, se = eng.open(), eng.open()
        got.append(eng.step([(sd, d), (se, e)], [[0, 299], [289]]))
        eng.close(sd)
        eng.close(se)
        eng.cache.audit()
        outs.append([g.clone() for g in got])
    for k, (x, y) in enumerate(zip(*outs)):
        assert torch.equal(x, y), (name, dtype, "step", k, float((x - y).abs().max()))
    ops = importlib.import_module("daisi-llogos_b200.kernels.ops")
    assert ops.gemm_tc_status() == 0 and ops.attn_tc_status() == 0 and ops.attn_decode_tma_status() == 0


def test_models_with_other_parts_keep_the_python_chain(llogos, model_dirs, tmp_path):
    """The runner takes a model only when every entry of its run order is the stock block of stock parts."""
    import dataclasses
    reg = importlib.import_module("daisi-llogos_b200.config.registry")
    S = llogos.parts

    def build(cfg):
        spec = llogos.config.dense_decoder_spec(cfg)
        return dataclasses.replace(spec, schedule=(S.ScheduleEntry(0), S.ScheduleEntry(1), S.ScheduleEntry(0)))

    llogos.config.register_architecture("ToyTwiceForCausalLM", reg._dense_reader(qk_norm=False, force_bias=False), build)
    try:
        cfg = dict(TINY["llama"], architectures=["ToyTwiceForCausalLM"])
        d = str(tmp_path / "twice")
        llogos.weights.write_random_model(d, cfg, seed=1, std=0.1)
        model = llogos.weights.load_model(d, dtype=torch.bfloat16, device="cuda:0")
        eng = llogos.engine.Engine(model, max_tokens=128)
        assert eng._runner is not None and eng._runner.n_layers == 3          # a layer run twice is still stock
    finally:
        reg._ARCHITECTURES.pop("ToyTwiceForCausalLM", None)
    model = llogos.weights.load_model(model_dirs["llama"], dtype=torch.bfloat16, device="cuda:0")
    model.blocks[1].parts["norm2"].__class__ = type("OtherNorm", (model.blocks[1].parts["norm2"].__class__,), {})
    assert llogos.engine.Engine(model, max_tokens=128)._runner is None

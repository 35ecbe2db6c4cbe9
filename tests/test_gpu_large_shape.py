"""Layers of Llama-3.1-8B's sizes.

First against the plain implementation: one layer of the headline sizes (width 4096, 32 heads in 8 groups,
head size 128, 14336 gated features, llama3 rotation scaling) with a vocabulary short enough for the plain
model, in float32 and bfloat16: a prompt of 300 tokens whole, a second request in portions (80 tokens on a
length of 64) and decode steps of both.  The weights come from the counter-based generator, so the plain
model on the host holds exactly what the engine holds on the GPU.

Then two layers with the full vocabulary and a prompt of 2,048 tokens, which the plain model is too slow for:
the bfloat16 engine (tensor-core products whose blocks work through several tiles, prompt attention over
2,048 tokens, decode attention with splits) against the engine's own 32-bit path (CUDA-core kernels
throughout) on the same weights."""
import importlib

import pytest
import torch

from compare import Reference

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
    "vocab_size": 128256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 131072,
    "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
REL_TOL = 4e-2
ONE_LAYER = dict(CFG, num_hidden_layers=1, vocab_size=8003)


@pytest.fixture(scope="module")
def one_layer(llogos):
    """The weights by name on the host (for the plain model) and the requests with their references."""
    model = llogos.weights.build_model(ONE_LAYER, dtype=torch.bfloat16, device="cuda:0",
                                       ops=importlib.import_module("daisi-llogos_b200.kernels.ops"))
    on_gpu = llogos.weights.random_tensors(model.tensor_decls(), 7, std=0.02, norm_std=0.1, device="cuda:0")
    weights = {n: t.cpu() for n, t in on_gpu.items()}
    del on_gpu, model
    torch.cuda.empty_cache()
    g = torch.Generator().manual_seed(5)
    a, b = (torch.randint(0, ONE_LAYER["vocab_size"], (n,), generator=g).tolist() for n in (306, 150))
    return weights, (a, Reference(weights, ONE_LAYER, a)), (b, Reference(weights, ONE_LAYER, b))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_one_layer_of_the_headline_sizes_against_the_plain_model(llogos, one_layer, dtype):
    weights, (a, ra), (b, rb) = one_layer
    # the same seed on the device: the generator's values depend on (seed, name, index) alone
    model = llogos.weights.random_model(ONE_LAYER, seed=7, dtype=dtype, device="cuda:0", std=0.02, norm_std=0.1)
    got = model.blocks[0].parts["ffn"].w_down
    assert torch.equal(got.cpu().float(), weights["model.layers.0.mlp.down_proj.weight"].float())
    eng = llogos.engine.Engine(model, max_tokens=64 * 10)
    sa, sb = eng.open(), eng.open()
    lg = eng.step([(sa, a[:300])], [list(range(300))])
    ra.check(lg, range(300), dtype, ("300 tokens whole",))
    lg = eng.step([(sb, b[:64])], [list(range(64))])
    rb.check(lg, range(64), dtype, ("64 tokens",))
    lg = eng.step([(sb, b[64:144])], [list(range(80))])
    rb.check(lg, range(64, 144), dtype, ("80 tokens on 64",))
    for j in range(6):
        lg = eng.step([(sa, [a[300 + j]]), (sb, [b[144 + j]])])
        ra.check(lg[0], [300 + j], dtype, ("decode a", j))
        rb.check(lg[1], [144 + j], dtype, ("decode b", j))
    eng.close(sa)
    eng.close(sb)
    eng.cache.audit()
    ops = llogos.kernels.ops
    assert ops.gemm_tc_status() == 0 and ops.attn_tc_status() == 0
    del eng, model
    torch.cuda.empty_cache()


def run(llogos, dtype, seqs, want_first, decode_steps):
    """Logits of: the first request's prompt alone, some decode steps, then the other requests as one
    batch of prompts and decode steps of all four together."""
    model = llogos.weights.random_model(CFG, seed=7, dtype=dtype, device="cuda:0", std=0.02, norm_std=0.1)
    eng = llogos.engine.Engine(model, max_tokens=64 * 80)
    out = []
    cut = [len(s) - decode_steps for s in seqs]
    slots = [eng.open()]
    out.append(eng.step([(slots[0], seqs[0][:cut[0]])], [want_first]).float().cpu())
    pos = list(cut)
    for _ in range(decode_steps // 2):
        out.append(eng.step([(slots[0], [seqs[0][pos[0]]])]).float().cpu())
        pos[0] += 1
    slots += [eng.open() for _ in seqs[1:]]
    out.append(eng.step([(slots[i], seqs[i][:cut[i]]) for i in range(1, len(seqs))],
                        [[0, cut[i] // 2, cut[i] - 1] for i in range(1, len(seqs))]).float().cpu())
    for _ in range(decode_steps // 2):
        out.append(eng.step([(slots[i], [seqs[i][pos[i]]]) for i in range(len(seqs))]).float().cpu())
        for i in range(len(seqs)):
            pos[i] += 1
    for s in slots:
        eng.close(s)
    eng.cache.audit()
    del eng, model
    torch.cuda.empty_cache()
    return out


def test_bfloat16_against_the_32_bit_path_at_the_headline_layer_sizes(llogos):
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, CFG["vocab_size"], (n,), generator=g).tolist() for n in (2048 + 6, 306, 1006, 83)]
    want_first = [0, 1, 63, 64, 255, 256, 1000, 1023, 1024, 2047]
    ref = run(llogos, torch.float32, seqs, want_first, 6)
    got = run(llogos, torch.bfloat16, seqs, want_first, 6)
    scale = max(float(r.abs().max()) for r in ref)
    for k, (a, b) in enumerate(zip(got, ref)):
        assert a.shape == b.shape
        err = float((a.double() - b.double()).abs().max())
        assert err <= REL_TOL * scale, (k, err, scale)
    ops = llogos.kernels.ops
    assert ops.gemm_tc_status() == 0 and ops.attn_tc_status() == 0


def test_the_same_batch_gives_the_same_bits(llogos):
    """Nothing in a step depends on timing (sums run in a fixed order, blocks only count arrivals): a batch of
    prompts and its decode steps, run three times over reused slots and pages, give identical logits.  A kernel
    that read its input before its producer had finished would differ from run to run."""
    model = llogos.weights.random_model(CFG, seed=7, dtype=torch.bfloat16, device="cuda:0", std=0.02, norm_std=0.1)
    eng = llogos.engine.Engine(model, max_tokens=64 * 80)
    g = torch.Generator().manual_seed(4)
    lens = [2048, 300, 700, 1, 65]
    seqs = [torch.randint(0, CFG["vocab_size"], (n + 4,), generator=g).tolist() for n in lens]
    first = None
    for rep in range(3):
        slots = [eng.open() for _ in seqs]
        outs = [eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, lens)], [[0, n - 1] for n in lens]).clone()]
        for k in range(4):
            outs.append(eng.step([(s, [q[n + k]]) for s, q, n in zip(slots, seqs, lens)]).clone())
        for s in slots:
            eng.close(s)
        got = torch.cat(outs)
        if first is None:
            first = got
        else:
            assert torch.equal(got, first), rep
    del eng, model
    torch.cuda.empty_cache()

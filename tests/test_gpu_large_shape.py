"""Two layers of Llama-3.1-8B's sizes: the bfloat16 engine (tensor-core products whose blocks work
through several tiles, prompt attention over 2,048 tokens, decode attention with splits) against the
engine's own 32-bit path (CUDA-core kernels throughout) on the same weights.  The plain implementation
is too slow at these sizes; the 32-bit path is compared with it on the small configurations."""
import pytest
import torch

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

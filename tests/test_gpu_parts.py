"""Each part alone on the GPU against the plain formulas, at sizes of its own; and a toy mixer
with state of its own, defined here, that is registered, built and stepped without a change to
the library's files."""
import importlib
import math

import pytest
import torch

import plain_model as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


@pytest.fixture(scope="module")
def ops():
    return importlib.import_module("daisi-llogos_b200.kernels.ops")


def rnd(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def tol(dtype):
    return 3e-5 if dtype == torch.float32 else 2.5e-2


def check(got, ref, dtype, what=""):
    ref = ref.double()
    err = float((got.detach().cpu().double() - ref).abs().max())
    lim = tol(dtype) * max(1.0, float(ref.abs().max()))
    assert err <= lim, (what, err, lim)


def env_for(llogos, ops, dtype, encodings=None):
    return llogos.parts.BuildEnv(dtype=dtype, device=DEV, ops=ops, encodings=encodings or {})


def prompt_ctx(llogos, ops, dtype, counts, before, slots):
    """A StepContext as the engine lays it out for a step with several tokens per sequence."""
    ctx_mod = importlib.import_module("daisi-llogos_b200.engine.context")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    cu = [0]
    for c in counts:
        cu.append(cu[-1] + c)
    pos = [p for b, c in zip(before, counts) for p in range(b, b + c)]
    seq = [i for i, c in enumerate(counts) for _ in range(c)]
    decode = all(c == 1 for c in counts)
    return ctx_mod.StepContext(
        n_tokens=cu[-1], n_seqs=len(counts), decode=decode, counts=list(counts), max_count=max(counts),
        token_ids=i32([0] * cu[-1]), positions=i32(pos), seq_of_token=i32(seq), slots=i32(slots), cu_tokens=i32(cu),
        len_before=i32(before), dtype=dtype, device=DEV, ops=ops,
        workspace=ctx_mod.Workspace(DEV), max_len_after=max(b + c for b, c in zip(before, counts)),
        len_before_host=None if decode else list(before))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_rmsnorm_part(llogos, ops, dtype):
    part = llogos.parts.part_class("norm", "rmsnorm")({"size": 200, "eps": 7e-4}, "n.", env_for(llogos, ops, dtype))
    assert list(part.tensors()) == ["weight"] and part.tensors()["weight"].shape == (200,)
    w = rnd((200,), 1, dtype) + 1
    part.bind({"weight": w.to(DEV)})
    res, br = rnd((9, 200), 2), rnd((2, 9, 200), 3)
    ctx = prompt_ctx(llogos, ops, dtype, [9], [0], [0])
    r = res.to(DEV).clone()
    out = part.forward(r, llogos.parts.Branch(br.to(DEV)), ctx)
    total = res.double() + br.double().sum(0)
    check(out, P.rms_norm(total, w, 7e-4), dtype)
    check(r, total, torch.float32)


def test_rotary_part_tables(llogos, ops):
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 128}
    part = llogos.parts.part_class("position", "rotary")(
        {"head_dim": 80, "rotary_dim": 64, "theta": 5e5, "scaling": sc, "pairing": "adjacent"}, "", env_for(llogos, ops, torch.float32))
    part.prepare(3000)
    rot = part.rotation()
    inv = P.rope_inverse_frequencies(64, 5e5, sc)
    ang = torch.arange(3000, dtype=torch.float64)[:, None] * inv[None, :]
    assert rot.rotary_dim == 64 and rot.pairing == 1 and rot.cos.shape == (3000, 32)
    assert float((rot.cos.cpu().double() - torch.cos(ang)).abs().max()) < 1e-7
    assert float((rot.sin.cpu().double() - torch.sin(ang)).abs().max()) < 1e-7
    with pytest.raises(ValueError):
        llogos.parts.part_class("position", "rotary")({"head_dim": 16, "rotary_dim": 18, "theta": 1.0}, "", env_for(llogos, ops, torch.float32))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_swiglu_part(llogos, ops, dtype):
    part = llogos.parts.part_class("ffn", "swiglu")({"hidden_size": 72, "intermediate_size": 200}, "m.", env_for(llogos, ops, dtype))
    t = {"gate_proj.weight": rnd((200, 72), 4, dtype, 0.2), "up_proj.weight": rnd((200, 72), 5, dtype, 0.2),
         "down_proj.weight": rnd((72, 200), 6, dtype, 0.2)}
    assert {k: v.shape for k, v in part.tensors().items()} == {k: tuple(v.shape) for k, v in t.items()}
    part.bind({k: v.to(DEV) for k, v in t.items()})
    for n in (3, 130):                                   # the small-step and the large-step path
        x = rnd((n, 72), 7, dtype)
        ctx = prompt_ctx(llogos, ops, dtype, [n], [0], [0])
        out = part.forward(x.to(DEV), ctx)
        check(out.data.sum(0), P.swiglu(x, t["gate_proj.weight"], t["up_proj.weight"], t["down_proj.weight"]), dtype, n)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_embedding_and_head_parts(llogos, ops, dtype):
    env = env_for(llogos, ops, dtype)
    emb = llogos.parts.part_class("embedding", "token_embedding")({"vocab_size": 301, "hidden_size": 72}, "e.", env)
    head = llogos.parts.part_class("head", "linear_head")({"vocab_size": 301, "hidden_size": 72, "tied_to": None}, "h.", env)
    table, hw = rnd((301, 72), 8, dtype), rnd((301, 72), 9, dtype, 0.3)
    emb.bind({"weight": table.to(DEV)})
    head.bind({"weight": hw.to(DEV)})
    ctx = prompt_ctx(llogos, ops, dtype, [4], [0], [0])
    ctx.token_ids = torch.tensor([300, 0, 5, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ctx).cpu(), table[[300, 0, 5, 5]].float())
    x = rnd((4, 72), 10, dtype)
    lg = head.forward(x.to(DEV), ctx)
    assert lg.dtype == torch.float32
    check(lg, P.linear(x, hw), torch.float32 if dtype == torch.float32 else torch.bfloat16)
    tied = llogos.parts.part_class("head", "linear_head")({"vocab_size": 301, "hidden_size": 72, "tied_to": "e.weight"}, "h.", env)
    assert tied.tensors() == {}


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("window,qk_norm,bias", [(0, True, False), (50, False, True)])
def test_attention_part_prompt_then_decode(llogos, ops, dtype, window, qk_norm, bias):
    """The mixer alone with a cache of its own: a prompt step for two sequences, then single tokens."""
    hidden, nh, nkv, hd = 72, 6, 2, 48
    env = env_for(llogos, ops, dtype)
    rope = llogos.parts.part_class("position", "rotary")({"head_dim": hd, "rotary_dim": hd, "theta": 3e4, "scaling": None, "pairing": "half"}, "", env)
    rope.prepare(512)
    env.encodings["r"] = rope
    params = {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qkv_bias": bias,
              "qk_norm": qk_norm, "qk_norm_eps": 1e-5, "window": window, "position": "r", "softmax_scale": None}
    att = llogos.parts.part_class("mixer", "attention")(params, "a.", env)
    decls = att.tensors()
    t = {}
    for i, (name, d) in enumerate(sorted(decls.items())):
        t[name] = rnd(d.shape, 20 + i, dtype, 0.25) + (1 if d.role == "norm" else 0)
    att.bind({k: v.to(DEV) for k, v in t.items()})
    need = att.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (nkv, hd, window)
    cache = llogos.cache.SequenceCache({0: need}, max_tokens=64 * 8, max_seq_len=64 * 4, n_slots=3, dtype=dtype, device=DEV)
    xs = [rnd((n, hidden), 30 + i, dtype) for i, n in enumerate((90, 131))]

    def plain(x):
        n = x.shape[0]
        q = P.linear(x, t["q_proj.weight"]).view(n, nh, hd)
        k = P.linear(x, t["k_proj.weight"]).view(n, nkv, hd)
        v = P.linear(x, t["v_proj.weight"]).view(n, nkv, hd)
        if qk_norm:
            q, k = P.per_head_rms_norm(q, t["q_norm.weight"], 1e-5), P.per_head_rms_norm(k, t["k_norm.weight"], 1e-5)
        if bias:
            q = q + t["q_proj.bias"].double().view(nh, hd)
            k = k + t["k_proj.bias"].double().view(nkv, hd)
            v = v + t["v_proj.bias"].double().view(nkv, hd)
        inv = P.rope_inverse_frequencies(hd, 3e4, None)
        q, k = P.rope_rotate(q, range(n), inv, "half"), P.rope_rotate(k, range(n), inv, "half")
        o = P.attention(q, k, v, 1 / math.sqrt(hd), window).reshape(n, nh * hd)
        return P.linear(o, t["o_proj.weight"])

    refs = [plain(x) for x in xs]
    slots = [cache.acquire(), cache.acquire()]
    cut = [80, 120]
    growth = list(zip(slots, cut))
    for g, ups in cache.grow(growth):
        if ups:
            ops.scatter_i32(g.page_table, torch.tensor([u[0] for u in ups], dtype=torch.int32, device=DEV),
                            torch.tensor([u[1] for u in ups], dtype=torch.int32, device=DEV))
    ctx = prompt_ctx(llogos, ops, dtype, cut, [0, 0], slots)
    out = att.forward(torch.cat([x[:c] for x, c in zip(xs, cut)]).to(DEV), ctx, cache.view(0)).data.sum(0)
    cache.commit(growth)
    check(out[:80], refs[0][:80], dtype, "prompt 0")
    check(out[80:], refs[1][:120], dtype, "prompt 1")
    pos = list(cut)
    for step in range(10):
        growth = [(s, 1) for s in slots]
        for g, ups in cache.grow(growth):
            if ups:
                ops.scatter_i32(g.page_table, torch.tensor([u[0] for u in ups], dtype=torch.int32, device=DEV),
                                torch.tensor([u[1] for u in ups], dtype=torch.int32, device=DEV))
        ctx = prompt_ctx(llogos, ops, dtype, [1, 1], pos, slots)
        x = torch.stack([xs[0][pos[0]], xs[1][pos[1]]]).to(DEV)
        out = att.forward(x, ctx, cache.view(0)).data.sum(0)
        cache.commit(growth)
        check(out[0], refs[0][pos[0]], dtype, ("decode 0", pos[0]))
        check(out[1], refs[1][pos[1]], dtype, ("decode 1", pos[1]))
        pos = [p + 1 for p in pos]


# ---- a toy mixer with state of its own ---------------------------------------------------------

def _toy_parts(llogos):
    Pt = llogos.parts

    class DecayMixer(Pt.Mixer):
        """out_t = s_t, s_t = decay * s_{t-1} + W x_t: a running state per sequence, no keys."""

        def __init__(self, params, prefix, env):
            super().__init__(params, prefix, env)
            self.hidden, self.decay = int(params["hidden_size"]), float(params["decay"])

        def tensors(self):
            return {"mix.weight": Pt.TensorDecl((self.hidden, self.hidden))}

        def bind(self, tensors):
            self.w = tensors["mix.weight"].float()

        def cache_need(self):
            return Pt.StateNeed((self.hidden,), torch.float32)

        def forward(self, x, ctx, cache):
            u = x.float() @ self.w.t()
            out = torch.empty_like(u)
            slots = ctx.slots.long()
            state = cache.state[slots]
            start = 0
            for b, c in enumerate(ctx.counts):
                s = state[b]
                for j in range(c):
                    s = self.decay * s + u[start + j]
                    out[start + j] = s
                state[b] = s
                start += c
            cache.state[slots] = state
            return Pt.Branch(out.unsqueeze(0))

    return DecayMixer


def _toy_spec_builder(llogos):
    S = llogos.parts
    C = llogos.config

    def build(cfg):
        spec = C.dense_decoder_spec(cfg)
        layers = list(spec.layers)
        for i in (1, 3):                                   # layers 1 and 3 mix by state, 0 and 2 by attention
            parts = dict(layers[i].parts)
            parts["mixer"] = S.PartSpec("toy_decay", {"hidden_size": cfg.hidden_size, "decay": 0.5 + 0.1 * i},
                                        f"model.layers.{i}.toy.")
            layers[i] = S.LayerSpec("prenorm", parts)
        import dataclasses
        return dataclasses.replace(spec, layers=tuple(layers))
    return build


def _toy_plain(weights, cfg, tokens):
    """The toy model, whole sequence, in float64, from the plain parts."""
    nh, nkv, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    t = len(tokens)
    inv = P.rope_inverse_frequencies(hd, cfg["rope_theta"], None)
    h = P.embedding(weights["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = P.rms_norm(h, weights[p + "input_layernorm.weight"], eps)
        if i in (1, 3):
            u = P.linear(x, weights[p + "toy.mix.weight"])
            s = torch.zeros(cfg["hidden_size"], dtype=torch.float64)
            rows = []
            for j in range(t):
                s = (0.5 + 0.1 * i) * s + u[j]
                rows.append(s)
            h = h + torch.stack(rows)
        else:
            a = p + "self_attn."
            q = P.rope_rotate(P.linear(x, weights[a + "q_proj.weight"]).view(t, nh, hd), range(t), inv, "half")
            k = P.rope_rotate(P.linear(x, weights[a + "k_proj.weight"]).view(t, nkv, hd), range(t), inv, "half")
            v = P.linear(x, weights[a + "v_proj.weight"]).view(t, nkv, hd)
            o = P.attention(q, k, v, 1 / math.sqrt(hd)).reshape(t, nh * hd)
            h = h + P.linear(o, weights[a + "o_proj.weight"])
        x = P.rms_norm(h, weights[p + "post_attention_layernorm.weight"], eps)
        m = p + "mlp."
        h = h + P.swiglu(x, weights[m + "gate_proj.weight"], weights[m + "up_proj.weight"], weights[m + "down_proj.weight"])
    return P.linear(P.rms_norm(h, weights["model.norm.weight"], eps), weights["lm_head.weight"])


def test_toy_mixer_with_state_registers_builds_and_steps(llogos, tmp_path):
    from conftest import read_weights, random_tokens
    reg = importlib.import_module("daisi-llogos_b200.config.registry")
    llogos.parts.register_part("mixer", "toy_decay", _toy_parts(llogos))
    llogos.config.register_architecture("ToyDecayForCausalLM", reg._dense_reader(qk_norm=False, force_bias=False),
                                        _toy_spec_builder(llogos))
    try:
        cfg = {"architectures": ["ToyDecayForCausalLM"], "num_hidden_layers": 4, "hidden_size": 48,
               "num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 16, "intermediate_size": 80,
               "vocab_size": 99, "rope_theta": 777.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 256}
        d = str(tmp_path / "toy")
        llogos.weights.write_random_model(d, cfg, seed=9, std=0.2, norm_std=0.1)
        w = read_weights(llogos, d)
        assert "model.layers.1.toy.mix.weight" in w and "model.layers.1.self_attn.q_proj.weight" not in w
        model = llogos.weights.load_model(d, dtype=torch.float32, device="cuda:0")
        eng = llogos.engine.Engine(model, max_tokens=64 * 6, use_graphs=False)
        assert sorted(eng.cache.state) == [1, 3] and len(eng.cache.kv_groups) == 1
        assert eng.cache.kv_groups[0].units == [0, 2]
        seqs = random_tokens(99, [50, 21, 70], 15)
        refs = [_toy_plain(w, cfg, s) for s in seqs]
        for rnd_ in range(2):                              # twice: slots and their state are used again
            slots = [eng.open() for _ in seqs]
            cut = [len(s) - 6 for s in seqs]
            lg = eng.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)], [list(range(c)) for c in cut])
            off = 0
            for i, c in enumerate(cut):
                assert float((lg[off:off + c].cpu().double() - refs[i][:c]).abs().max()) < 1e-4
                off += c
            for j in range(6):
                lg = eng.step([(sl, [s[c + j]]) for sl, s, c in zip(slots, seqs, cut)])
                for i, c in enumerate(cut):
                    assert float((lg[i].cpu().double() - refs[i][c + j]).abs().max()) < 1e-4, (rnd_, i, j)
            for sl in slots:
                eng.close(sl)
    finally:
        llogos.parts.unregister_part("mixer", "toy_decay")
        reg._ARCHITECTURES.pop("ToyDecayForCausalLM", None)


def test_layer_run_twice_and_borrowed_cache(llogos, tmp_path):
    """The run order is data: layer 0 runs twice (own cache each time), and a last entry reads the
    cache of the first instead of keeping one."""
    from conftest import read_weights, random_tokens
    import dataclasses
    reg = importlib.import_module("daisi-llogos_b200.config.registry")
    S = llogos.parts

    def build(cfg):
        spec = llogos.config.dense_decoder_spec(cfg)
        layers = list(spec.layers)
        parts = dict(layers[2].parts)
        params = dict(parts["mixer"].params, own_kv=False)
        parts["mixer"] = S.PartSpec("attention", params, parts["mixer"].prefix)
        layers[2] = S.LayerSpec("prenorm", parts)
        sched = (S.ScheduleEntry(0), S.ScheduleEntry(1), S.ScheduleEntry(0), S.ScheduleEntry(2, cache_of=0))
        return dataclasses.replace(spec, layers=tuple(layers), schedule=sched)

    llogos.config.register_architecture("ToyLoopForCausalLM", reg._dense_reader(qk_norm=False, force_bias=False), build)
    try:
        cfg = {"architectures": ["ToyLoopForCausalLM"], "num_hidden_layers": 3, "hidden_size": 48,
               "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 80,
               "vocab_size": 99, "rope_theta": 777.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 256}
        d = str(tmp_path / "loop")
        llogos.weights.write_random_model(d, cfg, seed=10, std=0.2, norm_std=0.1)
        w = read_weights(llogos, d)
        assert "model.layers.2.self_attn.k_proj.weight" not in w

        def plain(tokens):
            t = len(tokens)
            nh, nkv, hd, eps = 3, 1, 16, 1e-5
            inv = P.rope_inverse_frequencies(hd, 777.0, None)
            h = P.embedding(w["model.embed_tokens.weight"], tokens)
            kept = {}
            for e, (layer, borrow) in enumerate([(0, None), (1, None), (0, None), (2, 0)]):
                p = f"model.layers.{layer}."
                a = p + "self_attn."
                x = P.rms_norm(h, w[p + "input_layernorm.weight"], eps)
                q = P.rope_rotate(P.linear(x, w[a + "q_proj.weight"]).view(t, nh, hd), range(t), inv, "half")
                if borrow is None:
                    k = P.rope_rotate(P.linear(x, w[a + "k_proj.weight"]).view(t, nkv, hd), range(t), inv, "half")
                    v = P.linear(x, w[a + "v_proj.weight"]).view(t, nkv, hd)
                    kept[e] = (k, v)
                else:
                    k, v = kept[borrow]
                o = P.attention(q, k, v, 0.25).reshape(t, nh * hd)
                h = h + P.linear(o, w[a + "o_proj.weight"])
                x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
                m = p + "mlp."
                h = h + P.swiglu(x, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])
            return P.linear(P.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])

        model = llogos.weights.load_model(d, dtype=torch.float32, device="cuda:0")
        eng = llogos.engine.Engine(model, max_tokens=64 * 6)
        assert sorted(u for g in eng.cache.kv_groups for u in g.units) == [0, 1, 2]
        seqs = random_tokens(99, [40, 75], 16)
        refs = [plain(s) for s in seqs]
        slots = [eng.open(), eng.open()]
        lg = eng.step([(slots[0], seqs[0][:30]), (slots[1], seqs[1][:70])], [list(range(30)), list(range(70))])
        assert float((lg[:30].cpu().double() - refs[0][:30]).abs().max()) < 1e-4
        assert float((lg[30:].cpu().double() - refs[1][:70]).abs().max()) < 1e-4
        for j in range(5):
            lg = eng.step([(slots[0], [seqs[0][30 + j]]), (slots[1], [seqs[1][70 + j]])])
            assert float((lg[0].cpu().double() - refs[0][30 + j]).abs().max()) < 1e-4
            assert float((lg[1].cpu().double() - refs[1][70 + j]).abs().max()) < 1e-4
    finally:
        reg._ARCHITECTURES.pop("ToyLoopForCausalLM", None)


def test_toy_routed_feedforward_and_learned_positions(llogos, tmp_path):
    """A feed-forward with routing (top-1 of three experts) and a position encoding that is added to the
    embeddings, both defined here and registered from outside; attention runs without rotation."""
    from conftest import read_weights, random_tokens
    import dataclasses
    reg = importlib.import_module("daisi-llogos_b200.config.registry")
    Pt = llogos.parts

    class Top1Experts(Pt.FeedForward):
        """y = expert_e(x) with e = argmax(router(x)); each expert is down(relu(up(x)))."""

        def __init__(self, params, prefix, env):
            super().__init__(params, prefix, env)
            self.h, self.i, self.e = int(params["hidden_size"]), int(params["inner"]), int(params["experts"])

        def tensors(self):
            t = {"router.weight": Pt.TensorDecl((self.e, self.h))}
            for e in range(self.e):
                t[f"experts.{e}.up.weight"] = Pt.TensorDecl((self.i, self.h))
                t[f"experts.{e}.down.weight"] = Pt.TensorDecl((self.h, self.i))
            return t

        def bind(self, tensors):
            self.router = tensors["router.weight"].float()
            self.up = torch.stack([tensors[f"experts.{e}.up.weight"].float() for e in range(self.e)])
            self.down = torch.stack([tensors[f"experts.{e}.down.weight"].float() for e in range(self.e)])

        def forward(self, x, ctx):
            xf = x.float()
            choice = (xf @ self.router.t()).argmax(-1)                     # routing in float32
            hmid = torch.relu(torch.einsum("nh,nih->ni", xf, self.up[choice]))
            return Pt.Branch(torch.einsum("ni,nhi->nh", hmid, self.down[choice]).unsqueeze(0).contiguous())

    class LearnedPositions(Pt.PositionEncoding):
        def tensors(self):
            return {"weight": Pt.TensorDecl((int(self.params["positions"]), int(self.params["hidden_size"])), "table")}

        def bind(self, tensors):
            self.table = tensors["weight"].float()

        def on_embeddings(self, residual, ctx):
            residual += self.table[ctx.positions.long()]

    def build(cfg):
        spec = llogos.config.dense_decoder_spec(cfg)
        layers = []
        for i, layer in enumerate(spec.layers):
            parts = dict(layer.parts)
            parts["mixer"] = Pt.PartSpec("attention", dict(parts["mixer"].params, position=None), parts["mixer"].prefix)
            if i == 1:
                parts["ffn"] = Pt.PartSpec("toy_top1", {"hidden_size": cfg.hidden_size, "inner": 40, "experts": 3},
                                           f"model.layers.{i}.moe.")
            layers.append(Pt.LayerSpec("prenorm", parts))
        enc = {"learned": Pt.PartSpec("toy_learned", {"positions": 128, "hidden_size": cfg.hidden_size}, "model.positions.")}
        return dataclasses.replace(spec, layers=tuple(layers), encodings=enc)

    Pt.register_part("ffn", "toy_top1", Top1Experts)
    Pt.register_part("position", "toy_learned", LearnedPositions)
    llogos.config.register_architecture("ToyRoutedForCausalLM", reg._dense_reader(qk_norm=False, force_bias=False), build)
    try:
        cfg = {"architectures": ["ToyRoutedForCausalLM"], "num_hidden_layers": 2, "hidden_size": 48,
               "num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 16, "intermediate_size": 80,
               "vocab_size": 99, "rope_theta": 777.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 128}
        d = str(tmp_path / "routed")
        llogos.weights.write_random_model(d, cfg, seed=11, std=0.25, norm_std=0.1)
        w = read_weights(llogos, d)
        assert "model.layers.1.moe.experts.2.down.weight" in w and "model.positions.weight" in w
        assert "model.layers.1.mlp.gate_proj.weight" not in w

        def plain(tokens):
            t, nh, hd, eps = len(tokens), 3, 16, 1e-5
            h = P.embedding(w["model.embed_tokens.weight"], tokens) + w["model.positions.weight"].double()[:t]
            for i in range(2):
                p = f"model.layers.{i}."
                a = p + "self_attn."
                x = P.rms_norm(h, w[p + "input_layernorm.weight"], eps)
                q = P.linear(x, w[a + "q_proj.weight"]).view(t, nh, hd)
                k = P.linear(x, w[a + "k_proj.weight"]).view(t, nh, hd)
                v = P.linear(x, w[a + "v_proj.weight"]).view(t, nh, hd)
                h = h + P.linear(P.attention(q, k, v, 0.25).reshape(t, nh * hd), w[a + "o_proj.weight"])
                x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
                if i == 1:
                    m = p + "moe."
                    # the engine routes on bfloat16 activations: route on the same rounded values
                    choice = (x.float() @ w[m + "router.weight"].float().t()).argmax(-1)
                    rows = []
                    for j in range(t):
                        e = int(choice[j])
                        mid = torch.relu(P.linear(x[j:j + 1], w[m + f"experts.{e}.up.weight"]))
                        rows.append(P.linear(mid, w[m + f"experts.{e}.down.weight"])[0])
                    h = h + torch.stack(rows)
                else:
                    m = p + "mlp."
                    h = h + P.swiglu(x, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])
            return P.linear(P.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])

        model = llogos.weights.load_model(d, dtype=torch.float32, device="cuda:0")
        eng = llogos.engine.Engine(model, max_tokens=64 * 4, use_graphs=False)
        seqs = random_tokens(99, [60, 25], 18)
        refs = [plain(s) for s in seqs]
        slots = [eng.open(), eng.open()]
        lg = eng.step([(slots[0], seqs[0][:50]), (slots[1], seqs[1][:20])], [list(range(50)), list(range(20))])
        # a token whose two best experts tie within float32 noise may be routed differently: compare rows
        # whose routing margin is clear (all of them, with these weights) and require most rows to match
        err0 = (lg[:50].cpu().double() - refs[0][:50]).abs().max(dim=1).values
        err1 = (lg[50:].cpu().double() - refs[1][:20]).abs().max(dim=1).values
        assert int((err0 < 1e-4).sum()) >= 49 and int((err1 < 1e-4).sum()) >= 19
        for j in range(5):
            lg = eng.step([(slots[0], [seqs[0][50 + j]]), (slots[1], [seqs[1][20 + j]])])
            assert float((lg[0].cpu().double() - refs[0][50 + j]).abs().max()) < 1e-4
            assert float((lg[1].cpu().double() - refs[1][20 + j]).abs().max()) < 1e-4
    finally:
        Pt.unregister_part("ffn", "toy_top1")
        Pt.unregister_part("position", "toy_learned")
        reg._ARCHITECTURES.pop("ToyRoutedForCausalLM", None)


def test_borrowed_cache_with_a_window(llogos, tmp_path):
    """An entry that reads the ring of an earlier entry: a window of 100 keys lives in a ring of three pages, and
    a second portion of 100 tokens on a length of 150 lets the positions 192..249 land on the rows of the
    positions 0..57.  The owner's writes have to wait until the reader has run, for the reader's query at
    position 150 still looks at the keys 51..57.  Then single tokens."""
    from conftest import read_weights, random_tokens
    import dataclasses
    reg = importlib.import_module("daisi-llogos_b200.config.registry")
    S = llogos.parts
    W = 100

    def build(cfg):
        spec = llogos.config.dense_decoder_spec(cfg)
        layers = list(spec.layers)
        for i in (0, 1):
            parts = dict(layers[i].parts)
            params = dict(parts["mixer"].params, window=W, own_kv=(i == 0))
            parts["mixer"] = S.PartSpec("attention", params, parts["mixer"].prefix)
            layers[i] = S.LayerSpec("prenorm", parts)
        sched = (S.ScheduleEntry(0), S.ScheduleEntry(1, cache_of=0))
        return dataclasses.replace(spec, layers=tuple(layers), schedule=sched)

    def build_mismatch(cfg):
        spec = build(cfg)
        layers = list(spec.layers)
        parts = dict(layers[1].parts)
        parts["mixer"] = S.PartSpec("attention", dict(parts["mixer"].params, window=W + 1), parts["mixer"].prefix)
        layers[1] = S.LayerSpec("prenorm", parts)
        return dataclasses.replace(spec, layers=tuple(layers))

    llogos.config.register_architecture("ToyRingForCausalLM", reg._dense_reader(qk_norm=False, force_bias=False), build)
    llogos.config.register_architecture("ToyRingMismatchForCausalLM", reg._dense_reader(qk_norm=False, force_bias=False),
                                        build_mismatch)
    try:
        cfg = {"architectures": ["ToyRingForCausalLM"], "num_hidden_layers": 2, "hidden_size": 48,
               "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 80,
               "vocab_size": 99, "rope_theta": 777.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 512}
        d = str(tmp_path / "ring")
        llogos.weights.write_random_model(d, cfg, seed=12, std=0.15, norm_std=0.1)
        w = read_weights(llogos, d)
        assert "model.layers.1.self_attn.k_proj.weight" not in w

        def plain(tokens):
            t, nh, nkv, hd, eps = len(tokens), 3, 1, 16, 1e-5
            inv = P.rope_inverse_frequencies(hd, 777.0, None)
            h = P.embedding(w["model.embed_tokens.weight"], tokens)
            kept = None
            for layer in (0, 1):
                p = f"model.layers.{layer}."
                a = p + "self_attn."
                x = P.rms_norm(h, w[p + "input_layernorm.weight"], eps)
                q = P.rope_rotate(P.linear(x, w[a + "q_proj.weight"]).view(t, nh, hd), range(t), inv, "half")
                if layer == 0:
                    k = P.rope_rotate(P.linear(x, w[a + "k_proj.weight"]).view(t, nkv, hd), range(t), inv, "half")
                    kept = (k, P.linear(x, w[a + "v_proj.weight"]).view(t, nkv, hd))
                o = P.attention(q, kept[0], kept[1], 0.25, W).reshape(t, nh * hd)
                h = h + P.linear(o, w[a + "o_proj.weight"])
                x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
                m = p + "mlp."
                h = h + P.swiglu(x, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])
            return P.linear(P.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])

        for dtype, tol_ in ((torch.float32, 1e-4), (torch.bfloat16, 4e-2)):
            model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
            eng = llogos.engine.Engine(model, max_tokens=64 * 10)
            assert eng.cache.kv_groups[0].ring_pages == 3
            seqs = random_tokens(99, [256, 180], 19)
            refs = [plain(s) for s in seqs]
            scale = [float(r.abs().max()) for r in refs]
            slots = [eng.open(), eng.open()]
            lg = eng.step([(slots[0], seqs[0][:150]), (slots[1], seqs[1][:70])], [list(range(150)), list(range(70))])
            assert float((lg[:150].cpu().double() - refs[0][:150]).abs().max()) < tol_ * scale[0]
            assert float((lg[150:].cpu().double() - refs[1][:70]).abs().max()) < tol_ * scale[1]
            lg = eng.step([(slots[0], seqs[0][150:250]), (slots[1], seqs[1][70:174])], [list(range(100)), list(range(104))])
            err = (lg[:100].cpu().double() - refs[0][150:250]).abs().max(dim=1).values
            assert float(err.max()) < tol_ * scale[0], ("second portion, worst position", 150 + int(err.argmax()), float(err.max()))
            assert float((lg[100:].cpu().double() - refs[1][70:174]).abs().max()) < tol_ * scale[1]
            for j in range(6):
                lg = eng.step([(slots[0], [seqs[0][250 + j]]), (slots[1], [seqs[1][174 + j]])])
                assert float((lg[0].cpu().double() - refs[0][250 + j]).abs().max()) < tol_ * scale[0], j
                assert float((lg[1].cpu().double() - refs[1][174 + j]).abs().max()) < tol_ * scale[1], j
        # a reader whose window is not the owner's is refused when the model is built
        with pytest.raises(ValueError, match="window"):
            llogos.weights.build_model(dict(cfg, architectures=["ToyRingMismatchForCausalLM"]), dtype=torch.float32,
                                       device="cuda:0", ops=importlib.import_module("daisi-llogos_b200.kernels.ops"))
    finally:
        reg._ARCHITECTURES.pop("ToyRingForCausalLM", None)
        reg._ARCHITECTURES.pop("ToyRingMismatchForCausalLM", None)


def test_a_block_with_roles_of_its_own(llogos, tmp_path):
    """A block defined here whose branches run side by side (one norm feeds the mixer and the feed-forward, both
    outputs are added): it names two of its roles in ``ROLES``, and the spec gives the third role's family
    itself.  Layer 0 keeps the stock arrangement, layer 1 takes the new one; nothing in the library changes."""
    from conftest import read_weights, random_tokens
    import dataclasses
    reg = importlib.import_module("daisi-llogos_b200.config.registry")
    Pt = llogos.parts

    class SideBySide(Pt.Block):
        ROLES = {"mixer": "mixer", "ffn": "ffn"}          # "ln" is not listed: its PartSpec says family="norm"

        def forward(self, residual, pending, ctx, cache):
            h = self.parts["ln"].forward(residual, pending, ctx)
            a = self.parts["mixer"].forward(h, ctx, cache)
            f = self.parts["ffn"].forward(h, ctx)
            return Pt.Branch(torch.cat([a.data, f.data], dim=0))       # partial sums, added by whoever comes next

    def build(cfg):
        spec = llogos.config.dense_decoder_spec(cfg)
        layers = list(spec.layers)
        old = layers[1].parts
        ln = dataclasses.replace(old["norm1"], family="norm")
        layers[1] = Pt.LayerSpec("toy_side_by_side", {"ln": ln, "mixer": old["mixer"], "ffn": old["ffn"]})
        return dataclasses.replace(spec, layers=tuple(layers))

    def build_without_family(cfg):
        spec = build(cfg)
        layers = list(spec.layers)
        parts = dict(layers[1].parts)
        parts["ln"] = dataclasses.replace(parts["ln"], family=None)
        layers[1] = Pt.LayerSpec("toy_side_by_side", parts)
        return dataclasses.replace(spec, layers=tuple(layers))

    Pt.register_part("block", "toy_side_by_side", SideBySide)
    llogos.config.register_architecture("ToySideForCausalLM", reg._dense_reader(qk_norm=False, force_bias=False), build)
    llogos.config.register_architecture("ToySideBadForCausalLM", reg._dense_reader(qk_norm=False, force_bias=False),
                                        build_without_family)
    try:
        cfg = {"architectures": ["ToySideForCausalLM"], "num_hidden_layers": 2, "hidden_size": 48,
               "num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 16, "intermediate_size": 80,
               "vocab_size": 99, "rope_theta": 777.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 256}
        d = str(tmp_path / "side")
        llogos.weights.write_random_model(d, cfg, seed=13, std=0.2, norm_std=0.1)
        w = read_weights(llogos, d)
        assert "model.layers.1.post_attention_layernorm.weight" not in w
        assert "model.layers.0.post_attention_layernorm.weight" in w

        def plain(tokens):
            t, nh, hd, eps = len(tokens), 3, 16, 1e-5
            inv = P.rope_inverse_frequencies(hd, 777.0, None)
            h = P.embedding(w["model.embed_tokens.weight"], tokens)
            for i in range(2):
                p = f"model.layers.{i}."
                a, m = p + "self_attn.", p + "mlp."
                x = P.rms_norm(h, w[p + "input_layernorm.weight"], eps)
                q = P.rope_rotate(P.linear(x, w[a + "q_proj.weight"]).view(t, nh, hd), range(t), inv, "half")
                k = P.rope_rotate(P.linear(x, w[a + "k_proj.weight"]).view(t, nh, hd), range(t), inv, "half")
                v = P.linear(x, w[a + "v_proj.weight"]).view(t, nh, hd)
                att = P.linear(P.attention(q, k, v, 0.25).reshape(t, nh * hd), w[a + "o_proj.weight"])
                if i == 0:
                    h = h + att
                    x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
                    h = h + P.swiglu(x, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])
                else:
                    h = h + att + P.swiglu(x, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])
            return P.linear(P.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])

        model = llogos.weights.load_model(d, dtype=torch.float32, device="cuda:0")
        eng = llogos.engine.Engine(model, max_tokens=64 * 4)
        seqs = random_tokens(99, [60, 25], 20)
        refs = [plain(s) for s in seqs]
        slots = [eng.open(), eng.open()]
        lg = eng.step([(slots[0], seqs[0][:50]), (slots[1], seqs[1][:20])], [list(range(50)), list(range(20))])
        assert float((lg[:50].cpu().double() - refs[0][:50]).abs().max()) < 1e-4
        assert float((lg[50:].cpu().double() - refs[1][:20]).abs().max()) < 1e-4
        for j in range(5):                                  # the second of these replays a recorded graph
            lg = eng.step([(slots[0], [seqs[0][50 + j]]), (slots[1], [seqs[1][20 + j]])])
            assert float((lg[0].cpu().double() - refs[0][50 + j]).abs().max()) < 1e-4
            assert float((lg[1].cpu().double() - refs[1][20 + j]).abs().max()) < 1e-4
        with pytest.raises(ValueError, match="no role 'ln'"):
            llogos.weights.build_model(dict(cfg, architectures=["ToySideBadForCausalLM"]), dtype=torch.float32,
                                       device="cuda:0", ops=importlib.import_module("daisi-llogos_b200.kernels.ops"))
    finally:
        Pt.unregister_part("block", "toy_side_by_side")
        reg._ARCHITECTURES.pop("ToySideForCausalLM", None)
        reg._ARCHITECTURES.pop("ToySideBadForCausalLM", None)


@pytest.mark.gpu
def test_toy_architecture_with_a_configuration_and_a_norm_of_its_own(llogos, tmp_path):
    """A whole architecture from outside the library: a typed configuration read from config.json keys of its own
    (none of the dense decoder's names), a norm of its own kind (mean and variance, weight and bias) in every
    place a norm stands, and a spec put together from it and the stock attention and feed-forward.  It is
    registered, written with random weights, loaded by name, stepped in both precisions against formulas
    written here, and generates through the entry point."""
    from conftest import read_weights, random_tokens
    import dataclasses
    reg = importlib.import_module("daisi-llogos_b200.config.registry")
    Pt = llogos.parts
    ConfigError = llogos.config.ConfigError

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        d_model: int
        n_layer: int
        n_head: int
        d_head: int
        d_ff: int
        vocab: int
        ln_eps: float
        n_ctx: int
        rope_base: float

        @staticmethod
        def read(d):
            missing = [k for k in ("d_model", "n_layer", "n_head", "d_head", "d_ff", "vocab", "ln_eps", "n_ctx") if k not in d]
            if missing:
                raise ConfigError(f"config.json: missing key(s) {', '.join(missing)}")
            return ToyConfig(int(d["d_model"]), int(d["n_layer"]), int(d["n_head"]), int(d["d_head"]), int(d["d_ff"]),
                             int(d["vocab"]), float(d["ln_eps"]), int(d["n_ctx"]), float(d.get("rope_base", 10000.0)))

    class MeanVarianceNorm(Pt.Norm):
        """out = (v - mean(v)) / sqrt(var(v) + eps) * weight + bias with v = residual + branch, in float32."""

        def __init__(self, params, prefix, env):
            super().__init__(params, prefix, env)
            self.size, self.eps = int(params["size"]), float(params["eps"])

        def tensors(self):
            return {"weight": Pt.TensorDecl((self.size,), "norm"), "bias": Pt.TensorDecl((self.size,), "bias")}

        def bind(self, tensors):
            self.weight, self.bias = tensors["weight"].float(), tensors["bias"].float()

        def forward(self, residual, branch, ctx, rows=None):
            if branch is not None:
                residual += branch.data.float().sum(0)
            v = residual if rows is None else residual[rows.long()]
            mean = v.mean(-1, keepdim=True)
            var = ((v - mean) ** 2).mean(-1, keepdim=True)
            return ((v - mean) / torch.sqrt(var + self.eps) * self.weight + self.bias).to(ctx.dtype)

    def build(cfg):
        norm = {"size": cfg.d_model, "eps": cfg.ln_eps}
        layers = []
        for i in range(cfg.n_layer):
            p = f"blocks.{i}."
            layers.append(Pt.LayerSpec("prenorm", {
                "norm1": Pt.PartSpec("toy_mean_variance", dict(norm), p + "ln_1."),
                "mixer": Pt.PartSpec("attention", {"hidden_size": cfg.d_model, "num_heads": cfg.n_head, "num_kv_heads": cfg.n_head,
                                                   "head_dim": cfg.d_head, "qkv_bias": False, "qk_norm": False,
                                                   "qk_norm_eps": cfg.ln_eps, "window": 0, "position": "rope",
                                                   "softmax_scale": None}, p + "attn."),
                "norm2": Pt.PartSpec("toy_mean_variance", dict(norm), p + "ln_2."),
                "ffn": Pt.PartSpec("swiglu", {"hidden_size": cfg.d_model, "intermediate_size": cfg.d_ff}, p + "ff."),
            }))
        spec = Pt.ModelSpec(
            hidden_size=cfg.d_model, vocab_size=cfg.vocab, max_positions=cfg.n_ctx,
            embedding=Pt.PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.d_model}, "wte."),
            encodings={"rope": Pt.PartSpec("rotary", {"head_dim": cfg.d_head, "rotary_dim": cfg.d_head, "theta": cfg.rope_base,
                                                      "scaling": None, "pairing": "half"})},
            layers=tuple(layers), schedule=tuple(Pt.ScheduleEntry(i) for i in range(cfg.n_layer)),
            final_norm=Pt.PartSpec("toy_mean_variance", dict(norm), "ln_f."),
            head=Pt.PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.d_model, "tied_to": "wte.weight"}, "head."))
        spec.validate()
        return spec

    Pt.register_part("norm", "toy_mean_variance", MeanVarianceNorm)
    llogos.config.register_architecture("ToyOwnConfigLM", ToyConfig.read, build)
    try:
        cfg = {"architectures": ["ToyOwnConfigLM"], "d_model": 56, "n_layer": 3, "n_head": 2, "d_head": 32, "d_ff": 72,
               "vocab": 123, "ln_eps": 2e-5, "n_ctx": 192, "rope_base": 5000.0}
        with pytest.raises(ConfigError, match="d_ff"):
            llogos.config.architecture_of(cfg).read_config({k: v for k, v in cfg.items() if k != "d_ff"})
        d = str(tmp_path / "own")
        llogos.weights.write_random_model(d, cfg, seed=17, std=0.2, norm_std=0.1, bias_std=0.1)
        w = read_weights(llogos, d)
        assert "blocks.2.ln_2.bias" in w and "ln_f.weight" in w and "wte.weight" in w and "head.weight" not in w
        assert float(w["blocks.0.ln_1.bias"].abs().max()) > 0

        def norm_plain(v, prefix):
            mean = v.mean(-1, keepdim=True)
            var = ((v - mean) ** 2).mean(-1, keepdim=True)
            return (v - mean) / torch.sqrt(var + 2e-5) * w[prefix + "weight"].double() + w[prefix + "bias"].double()

        def plain(tokens):
            t, nh, hd = len(tokens), 2, 32
            inv = P.rope_inverse_frequencies(hd, 5000.0, None)
            h = P.embedding(w["wte.weight"], tokens)
            for i in range(3):
                p = f"blocks.{i}."
                a, m = p + "attn.", p + "ff."
                x = norm_plain(h, p + "ln_1.")
                q = P.rope_rotate(P.linear(x, w[a + "q_proj.weight"]).view(t, nh, hd), range(t), inv, "half")
                k = P.rope_rotate(P.linear(x, w[a + "k_proj.weight"]).view(t, nh, hd), range(t), inv, "half")
                v = P.linear(x, w[a + "v_proj.weight"]).view(t, nh, hd)
                h = h + P.linear(P.attention(q, k, v, 1.0 / math.sqrt(hd)).reshape(t, nh * hd), w[a + "o_proj.weight"])
                x = norm_plain(h, p + "ln_2.")
                h = h + P.swiglu(x, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])
            return P.linear(norm_plain(h, "ln_f."), w["wte.weight"])

        seqs = random_tokens(123, [70, 33], 23)
        refs = [plain(s) for s in seqs]
        for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, None)):
            model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
            eng = llogos.engine.Engine(model, max_tokens=64 * 4)
            assert eng.cache.max_seq_len <= 192
            slots = [eng.open(), eng.open()]
            bound = [tol if tol else 4e-2 * float(r.abs().max()) for r in refs]
            lg = eng.step([(slots[0], seqs[0][:60]), (slots[1], seqs[1][:25])], [list(range(60)), list(range(25))])
            assert float((lg[:60].cpu().double() - refs[0][:60]).abs().max()) < bound[0]
            assert float((lg[60:].cpu().double() - refs[1][:25]).abs().max()) < bound[1]
            for j in range(6):
                lg = eng.step([(slots[0], [seqs[0][60 + j]]), (slots[1], [seqs[1][25 + j]])])
                assert float((lg[0].cpu().double() - refs[0][60 + j]).abs().max()) < bound[0]
                assert float((lg[1].cpu().double() - refs[1][25 + j]).abs().max()) < bound[1]
            eng.close(slots[0])
            eng.close(slots[1])
            eng.cache.audit()
            del eng, model
        # through the entry point: greedy tokens follow the plain model's largest logits (where the margin is clear)
        api = importlib.import_module("llogos_b200")
        lm = api.LlogosModel.load(d, dtype="float32", max_context=128)
        out = lm.generate([seqs[1][:25]], api.GenerationParams(max_tokens=5, temperature=0.0, repetition_penalty=1.0,
                                                                  stop_tokens=()))
        got = list(out.tokens[0])
        assert len(got) == 5
        full = plain(seqs[1][:25] + got)
        for j, tok in enumerate(got):
            row = full[24 + j]
            top2 = torch.topk(row, 2).values
            assert int(row.argmax()) == tok or float(top2[0] - top2[1]) < 1e-4
    finally:
        Pt.unregister_part("norm", "toy_mean_variance")
        reg._ARCHITECTURES.pop("ToyOwnConfigLM", None)

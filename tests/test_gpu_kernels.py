"""Each kernel alone against the plain float64 formulas, at sizes the models of the other tests
do not use: widths and vocabularies that are no power of two, head sizes in steps of 16, odd
numbers of heads and groups."""
import importlib
import math

import pytest
import torch

import plain_model as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


@pytest.fixture(scope="module")
def ops():
    return importlib.import_module("daisi-llogos_b200.kernels.ops")


def rnd(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.6e-2


def check(got, ref, dtype, what=""):
    ref = ref.double()
    err = float((got.detach().cpu().double() - ref).abs().max())
    lim = tol(dtype) * max(1.0, float(ref.abs().max()))
    assert err <= lim, (what, err, lim)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_embed_rows(ops, dtype):
    table = rnd((301, 200), 1, dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = torch.empty(5, 200, device=DEV)
    ops.embed_rows(table.to(DEV), ids.to(DEV), out)
    assert torch.equal(out.cpu(), P.embedding(table, ids.tolist()).float())


@pytest.mark.parametrize("wdtype", DTYPES, ids=["w32", "w16"])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("hidden", [72, 1000, 4096, 4100])
def test_add_rmsnorm(ops, dtype, wdtype, hidden):
    n, eps = 7, 3e-5
    res = rnd((n, hidden), 2)
    branch = rnd((3, n, hidden), 3)
    w = rnd((hidden,), 4, wdtype) + 1
    r_dev = res.to(DEV).clone()
    out = torch.empty(n, hidden, dtype=dtype, device=DEV)
    ops.add_rmsnorm(r_dev, branch.to(DEV), w.to(DEV), eps, out)
    total = res.double() + branch.double().sum(0)
    check(r_dev, total, torch.float32, "residual")
    check(out, P.rms_norm(total, w, eps), dtype, "normed")
    # without a branch, with a row gather
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    out2 = torch.empty(3, hidden, dtype=dtype, device=DEV)
    r2 = res.to(DEV).clone()
    ops.add_rmsnorm(r2, None, w.to(DEV), eps, out2, rows.to(DEV))
    assert torch.equal(r2.cpu(), res)
    check(out2, P.rms_norm(res[rows.long()], w, eps), dtype, "gathered")
    # gather with a branch: the gathered rows of the residual are updated
    r3 = res.to(DEV).clone()
    ops.add_rmsnorm(r3, branch.to(DEV), w.to(DEV), eps, out2, rows.to(DEV))
    check(out2, P.rms_norm(total[rows.long()], w, eps), dtype, "gathered with branch")
    # many rows (a prompt step): blocks that work through several rows, with one and with two partials
    for n, parts in ((700, 1), (1501, 2)):
        res = rnd((n, hidden), 5)
        branch = rnd((parts, n, hidden), 6)
        r_dev = res.to(DEV).clone()
        out = torch.empty(n, hidden, dtype=dtype, device=DEV)
        ops.add_rmsnorm(r_dev, branch.to(DEV), w.to(DEV), eps, out)
        total = res.double() + branch.double().sum(0)
        check(r_dev, total, torch.float32, ("residual", n))
        check(out, P.rms_norm(total, w, eps), dtype, ("normed", n))
        r_dev = res.to(DEV).clone()
        ops.add_rmsnorm(r_dev, None, w.to(DEV), eps, out)
        assert torch.equal(r_dev.cpu(), res)
        check(out, P.rms_norm(res, w, eps), dtype, ("normed without branch", n))


@pytest.mark.parametrize("xd,wd,od", [(torch.float32,) * 3, (torch.bfloat16, torch.bfloat16, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                      (torch.bfloat16, torch.float32, torch.float32)], ids=["fff", "bbf", "bbb", "bff"])
@pytest.mark.parametrize("n,o,k", [(1, 301, 72), (5, 64, 1000), (70, 130, 333), (200, 65, 16)])
def test_gemm_simt(ops, xd, wd, od, n, o, k):
    x, w = rnd((n, k), 5, xd), rnd((o, k), 6, wd, 0.1)
    out = torch.empty(n, o, dtype=od, device=DEV)
    ops.gemm_simt(x.to(DEV), w.to(DEV), out)
    check(out, P.linear(x, w), od if od == torch.bfloat16 else torch.float32)


@pytest.mark.parametrize("n,o,k", [(1, 128, 64), (3, 200, 72), (16, 129, 128), (17, 384, 1000), (33, 100, 8),
                                   (70, 130, 336), (129, 65, 16), (300, 1000, 520), (2, 301, 4104),
                                   (1100, 9000, 72), (2050, 4700, 136)])
def test_gemm_tc(ops, n, o, k):
    """The tcgen05 product at ragged sizes: rows, features and k that fill no tile."""
    x, w = rnd((n, k), 5, torch.bfloat16), rnd((o, k), 6, torch.bfloat16, 0.1)
    ref = P.linear(x, w)
    assert ops.gemm_tc_supported(x.to(DEV), w.to(DEV))
    for wish in (1, 3, 16):
        s = ops.gemm_tc_splits(k, wish)
        assert 1 <= s <= wish
        out = torch.full((s, n, o), float("nan"), device=DEV)
        ops.gemm_tc(x.to(DEV), w.to(DEV), out)
        check(out.sum(0), ref, torch.float32, ("splits", s))
    out = torch.empty(1, n, o, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x.to(DEV), w.to(DEV), out)
    check(out[0], ref, torch.bfloat16, "bfloat16 output")
    for tile in (16, 32, 64, 128, 256):
        out = torch.full((1, n, o), float("nan"), device=DEV)
        ops.gemm_tc(x.to(DEV), w.to(DEV), out, tile_n=tile)
        check(out[0], ref, torch.float32, ("tile", tile))
    assert ops.gemm_tc_status() == 0


def _gated(gate, up):
    lin = importlib.import_module("daisi-llogos_b200.kernels.linear")
    return lin.gated_layout(gate, up)


@pytest.mark.parametrize("n,feat,k", [(1, 128, 64), (5, 101, 72), (70, 300, 336), (300, 500, 520), (2100, 176, 64)])
def test_gemm_tc_gated_epilogue(ops, n, feat, k):
    """A gate/up matrix in the gated layout; the epilogue writes silu(gate) * up."""
    x = rnd((n, k), 5, torch.bfloat16)
    gate, up = rnd((feat, k), 6, torch.bfloat16, 0.2), rnd((feat, k), 7, torch.bfloat16, 0.2)
    w = _gated(gate, up)
    assert w.shape == (ops.gated_rows(feat), k)
    g, u = P.linear(x, gate), P.linear(x, up)
    ref = g / (1 + torch.exp(-g)) * u
    for dt in (torch.bfloat16, torch.float32):
        out = torch.full((1, n, feat), float("nan"), dtype=dt, device=DEV)
        ops.gemm_tc(x.to(DEV), w.to(DEV), out, gated_features=feat)
        check(out[0], ref, torch.bfloat16 if dt == torch.bfloat16 else torch.float32, dt)
    with pytest.raises(ops.KernelError, match="gated epilogue"):
        ops.gemm_tc(x.to(DEV), w[:128].contiguous().to(DEV), torch.empty(1, n, feat, device=DEV), gated_features=feat)
    assert ops.gemm_tc_status() == 0


def test_gemm_tc_refuses_what_tma_cannot_address(ops):
    x, w = rnd((4, 36), 5, torch.bfloat16).to(DEV), rnd((8, 36), 6, torch.bfloat16).to(DEV)
    assert not ops.gemm_tc_supported(x, w)                       # 72-byte rows
    assert not ops.gemm_tc_supported(x.float(), w.float())       # float32 stays off the tensor cores
    with pytest.raises(ops.KernelError, match="k % 8"):
        ops.gemm_tc(x, w, torch.empty(1, 4, 8, device=DEV))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("partials", [1, 3])
def test_silu_mul(ops, dtype, partials):
    n, inter = 5, 333
    in_dtype = torch.float32 if partials > 1 else dtype
    gu = rnd((partials, n, ops.gated_rows(inter)), 7, in_dtype, 2.0)
    out = torch.empty(n, inter, dtype=dtype, device=DEV)
    ops.silu_mul(gu.to(DEV), out)
    s = gu.double().sum(0)
    half = ops.gated_rows(inter) // 2
    g, u = s[:, :inter], s[:, half:half + inter]
    check(out, g / (1 + torch.exp(-g)) * u, dtype)


def _rope_tables(hd, rd, theta, n_pos):
    inv = P.rope_inverse_frequencies(rd, theta, None)
    ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return inv, torch.cos(ang).float(), torch.sin(ang).float()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nh,nkv,hd,rd,pairing,norm,bias", [
    (5, 1, 48, 48, "half", True, True), (6, 3, 80, 32, "adjacent", False, True),
    (4, 4, 16, 16, "half", True, False), (9, 3, 128, 128, "half", False, False), (3, 1, 64, 64, "half", True, True),
    (2, 2, 256, 256, "half", True, False), (2, 1, 128, 64, "half", False, False), (4, 2, 128, 128, "adjacent", True, False)])
def test_qk_prep(ops, dtype, nh, nkv, hd, rd, pairing, norm, bias):
    n, eps = 11, 2e-6
    width = (nh + 2 * nkv) * hd
    partials = 2 if dtype == torch.float32 else 1
    qkv = rnd((partials, n, width), 8, torch.float32 if partials > 1 else dtype)
    qw, kw = (rnd((hd,), 9, dtype) + 1, rnd((hd,), 10, dtype) + 1) if norm else (None, None)
    b = rnd((width,), 11, dtype) if bias else None
    pos = torch.tensor([0, 1, 2, 3, 500, 63, 64, 65, 7, 7, 1023], dtype=torch.int32)
    inv, cos, sin = _rope_tables(hd, rd, 12345.0, 1024)
    q = torch.empty(n, nh, hd, dtype=dtype, device=DEV)
    kn, vn = (torch.empty(n, nkv, hd, dtype=dtype, device=DEV) for _ in range(2))
    dev = lambda t: None if t is None else t.to(DEV)
    ops.qk_prep(qkv.to(DEV), n_heads=nh, n_kv_heads=nkv, head_dim=hd, q_norm_w=dev(qw), k_norm_w=dev(kw),
                norm_eps=eps, bias=dev(b), cos=cos.to(DEV), sin=sin.to(DEV), rotary_dim=rd,
                pairing=0 if pairing == "half" else 1, positions=pos.to(DEV), q_out=q, k_new=kn, v_new=vn)
    x = qkv.double().sum(0).view(n, nh + 2 * nkv, hd)
    qr, kr, vr = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]
    if norm:
        qr, kr = P.per_head_rms_norm(qr, qw, eps), P.per_head_rms_norm(kr, kw, eps)
    if bias:
        bb = b.double().view(nh + 2 * nkv, hd)
        qr, kr, vr = qr + bb[:nh], kr + bb[nh:nh + nkv], vr + bb[nh + nkv:]
    qr = P.rope_rotate(qr, pos.tolist(), inv, pairing)
    kr = P.rope_rotate(kr, pos.tolist(), inv, pairing)
    check(q, qr, dtype, "q")
    check(kn, kr, dtype, "k")
    check(vn, vr, dtype, "v")


def _paged(nkv, hd, dtype, lens, n_pages, ring_pages, seed):
    """A cache filled with random keys/values for sequences of the given lengths; pages handed out
    in a scrambled order so that a wrong page-table lookup shows."""
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(len(lens) + 2, ring_pages, dtype=torch.int32)
    slots = list(range(len(lens), 0, -1))            # slots differ from batch indices
    kp = torch.zeros(n_pages, nkv, 64, hd, dtype=dtype)
    vp = torch.zeros(n_pages, nkv, 64, hd, dtype=dtype)
    ks, vs = [], []
    for b, n in enumerate(lens):
        k = rnd((n, nkv, hd), seed + 10 + b, dtype)
        v = rnd((n, nkv, hd), seed + 20 + b, dtype)
        ks.append(k)
        vs.append(v)
        for j in range(min((n + 63) // 64, ring_pages)):
            table[slots[b], j] = order.pop()
        for p in range(max(0, n - ring_pages * 64), n):
            pg = int(table[slots[b], (p // 64) % ring_pages])
            kp[pg, :, p % 64] = k[p]
            vp[pg, :, p % 64] = v[p]
    return kp, vp, table, torch.tensor(slots, dtype=torch.int32), ks, vs


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nh,nkv,hd,window", [(5, 1, 48, 0), (6, 3, 80, 0), (12, 1, 32, 0), (4, 2, 128, 100), (8, 4, 16, 70),
                                              (34, 2, 64, 0), (3, 3, 112, 0), (2, 1, 144, 0), (4, 2, 256, 130)])
def test_attn_decode(ops, dtype, nh, nkv, hd, window):
    lens = [1, 64, 65, 300, 129]
    ring = 8 if window == 0 else (window + 63) // 64 + 1
    kp, vp, table, slots, ks, vs = _paged(nkv, hd, dtype, lens, 40, ring, 30)
    q = rnd((len(lens), nh, hd), 31, dtype)
    scale = 1 / math.sqrt(hd)
    counters = torch.zeros(len(lens) * nkv, dtype=torch.int32, device=DEV)
    for splits, balance in ((1, False), (3, False), (7, False), (7, True), (2, True), (40, True)):
        out = torch.empty(len(lens), nh * hd, dtype=dtype, device=DEV)
        scratch = torch.empty(ops.attn_decode_scratch_floats(len(lens), nh, hd, splits), device=DEV)
        lb = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
        # balance: every sequence takes as many of the splits as its length calls for (1 to 5 tiles here)
        ops.attn_decode(q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV), ring, slots.to(DEV), lb.to(DEV), out,
                        scratch, n_splits=splits, scale=scale, window=window, counters=counters, balance=balance)
        assert int(counters.abs().sum()) == 0
        for b, n in enumerate(lens):
            qq = torch.zeros(n, nh, hd, dtype=dtype)
            qq[-1] = q[b]
            ref = P.attention(qq, ks[b], vs[b], scale, window)[-1].reshape(-1)
            check(out[b], ref, dtype, (b, n, splits))
    # and as the engine calls it: the kernels' own plan for this batch (the TMA kernel where it applies)
    plan = ops.attn_decode_plan(dtype, len(lens), nh, nkv, hd, max(lens))
    out = torch.full((len(lens), nh * hd), float("nan"), dtype=dtype, device=DEV)
    scratch = torch.empty(max(1, plan.scratch_floats), device=DEV)
    counters = torch.zeros(max(1, plan.n_counters), dtype=torch.int32, device=DEV)
    ops.attn_decode(q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV), ring, slots.to(DEV), lb.to(DEV), out,
                    scratch, scale=scale, window=window, plan=plan, counters=counters)
    assert int(counters.abs().sum()) == 0
    for b, n in enumerate(lens):
        qq = torch.zeros(n, nh, hd, dtype=dtype)
        qq[-1] = q[b]
        ref = P.attention(qq, ks[b], vs[b], scale, window)[-1].reshape(-1)
        check(out[b], ref, dtype, (b, n, plan.kind))
    if plan.kind == "tma":
        assert ops.attn_decode_tma_status() == 0


def _one_query(q, k, v, scale):
    """softmax(k q * scale) v for one query of one head, in float64 (the plain formula of
    Daisi.Llogos.Cpu/CpuBackend.cs:527-571 for a single row)."""
    s = (k.double() @ q.double()) * scale
    p = torch.exp(s - s.max())
    return (p / p.sum()) @ v.double()


@pytest.mark.parametrize("seed,n_seqs,nh,nkv,hd,window,longest", [
    (1, 1, 8, 8, 128, 0, 5000), (2, 3, 32, 8, 128, 0, 3000), (3, 40, 8, 2, 64, 0, 900), (4, 200, 4, 1, 128, 0, 300),
    (5, 7, 16, 2, 64, 200, 2500), (6, 64, 6, 6, 128, 100, 400), (7, 2, 5, 5, 64, 0, 70), (8, 300, 2, 2, 64, 0, 130)])
def test_attn_decode_tma_cuts_any_batch_evenly(ops, seed, n_seqs, nh, nkv, hd, window, longest):
    """The TMA kernel cuts the list of (sequence, key/value head, tile) units into equal runs per block, wherever
    the cuts fall: batches of one to hundreds of sequences with lengths from 1 to thousands of keys (so that some
    pairs are spread over dozens of blocks and some blocks hold dozens of pairs), pages in scrambled order, a
    window, twice in a row over the same counters and scratch."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(seed)
    lens = [int(x) for x in torch.randint(1, longest + 1, (n_seqs,), generator=g)]
    lens[0] = longest
    if n_seqs > 2:
        lens[1], lens[2] = 1, 64
    ring = (longest + 63) // 64 if window == 0 else (window + 63) // 64 + 1
    pages_of = [min((n + 63) // 64, ring) for n in lens]
    n_pages = sum(pages_of) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    kp = torch.randn(n_pages, nkv, 64, hd, generator=g).to(dtype)
    vp = torch.randn(n_pages, nkv, 64, hd, generator=g).to(dtype)
    table = torch.zeros(n_seqs + 2, ring, dtype=torch.int32)
    slots = torch.randperm(n_seqs + 2, generator=g)[:n_seqs].to(torch.int32)
    for b in range(n_seqs):
        for j in range(pages_of[b]):
            table[slots[b], j] = order.pop()
    q = torch.randn(n_seqs, nh, hd, generator=g).to(dtype)
    lb = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    scale = 1 / math.sqrt(hd)
    plan = ops.attn_decode_plan(dtype, n_seqs, nh, nkv, hd, longest)
    assert plan.kind == "tma"
    counters = torch.zeros(plan.n_counters, dtype=torch.int32, device=DEV)
    scratch = torch.full((plan.scratch_floats,), float("nan"), device=DEV)
    d = lambda t: t.to(DEV)
    kpd, vpd, qd, td, sd, lbd = d(kp), d(vp), d(q), d(table), d(slots), d(lb)
    outs = []
    for rep in range(2):
        out = torch.full((n_seqs, nh * hd), float("nan"), dtype=dtype, device=DEV)
        ops.attn_decode(qd, kpd, vpd, td, ring, sd, lbd, out, scratch, scale=scale, window=window, plan=plan, counters=counters)
        outs.append(out.cpu())
        assert int(counters.abs().sum()) == 0
    assert ops.attn_decode_tma_status() == 0
    assert torch.equal(outs[0], outs[1])                                   # sums run in a fixed order
    grp = nh // nkv
    for b in [0, 1, 2, n_seqs // 2, n_seqs - 1] if n_seqs > 4 else range(n_seqs):
        n = lens[b]
        first = max(0, n - window) if window > 0 else 0
        pos = torch.arange(first, n)
        pg = table[slots[b]][(pos // 64) % ring].long()
        for h in range(nh):
            k, v = kp[pg, h // grp, pos % 64], vp[pg, h // grp, pos % 64]
            check(outs[0][b].view(nh, hd)[h], _one_query(q[b, h], k, v, scale), dtype, (seed, b, n, h))
    # every row is a number: no pair was left out
    assert bool(torch.isfinite(outs[0].float()).all())


@pytest.mark.parametrize("tc", [True, False], ids=["tcgen05", "mma"])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nh,nkv,hd,window", [(5, 1, 48, 0), (6, 3, 80, 0), (4, 2, 128, 100), (8, 4, 16, 40), (3, 1, 112, 0),
                                              (2, 2, 144, 0), (2, 1, 256, 90), (6, 2, 64, 0), (3, 3, 128, 0), (4, 1, 64, 70)])
def test_attn_prefill_and_kv_write(ops, dtype, nh, nkv, hd, window, tc, monkeypatch):
    if not tc and not (dtype == torch.bfloat16 and hd in (64, 128)):
        pytest.skip("only head sizes 64 and 128 in bfloat16 have two tensor-core kernels")
    monkeypatch.setattr(ops, "USE_TC_PROMPT_ATTENTION", tc)
    before = [0, 0, 70, 130, 64]           # tokens already in the cache
    counts = [1, 37, 16, 150, 3]           # tokens the step brings
    ring = 8 if window == 0 else (window + 63) // 64 + 1
    total = [a + c for a, c in zip(before, counts)]
    kp, vp, table, slots, ks, vs = _paged(nkv, hd, dtype, total, 40, ring, 40)
    # rebuild the cache as it was BEFORE the step: only positions < before, ring of the old length
    kp0, vp0 = torch.zeros_like(kp), torch.zeros_like(vp)
    for b, n in enumerate(before):
        for p in range(max(0, n - ring * 64), n):
            pg = int(table[slots[b], (p // 64) % ring])
            kp0[pg, :, p % 64] = ks[b][p]
            vp0[pg, :, p % 64] = vs[b][p]
    cu = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    n = int(cu[-1])
    q = rnd((n, nh, hd), 41, dtype)
    k_new = torch.cat([ks[b][before[b]:] for b in range(len(counts))])
    v_new = torch.cat([vs[b][before[b]:] for b in range(len(counts))])
    tq = ops.prefill_tile_queries(dtype, hd)
    tiles = torch.tensor([(b, q0) for b, c in enumerate(counts) for q0 in range(0, c, tq)], dtype=torch.int32)
    out = torch.empty(n, nh * hd, dtype=dtype, device=DEV)
    scale = 0.37
    d = lambda t: t.to(DEV)
    kpd, vpd = d(kp0), d(vp0)
    lb = torch.tensor(before, dtype=torch.int32)
    ops.attn_prefill(d(q), d(k_new), d(v_new), kpd, vpd, d(table), ring, d(tiles), d(cu), d(lb), d(slots), out,
                     scale=scale, window=window, tile_queries=tq)
    for b in range(len(counts)):
        qq = torch.zeros(total[b], nh, hd, dtype=dtype)
        qq[before[b]:] = q[int(cu[b]):int(cu[b + 1])]
        ref = P.attention(qq, ks[b], vs[b], scale, window)[before[b]:].reshape(counts[b], -1)
        check(out[int(cu[b]):int(cu[b + 1])], ref, dtype, ("sequence", b))
    # the write after the step leaves the cache as if all tokens had been there
    pos = torch.cat([torch.arange(a, a + c) for a, c in zip(before, counts)]).to(torch.int32)
    seq_of = torch.repeat_interleave(torch.arange(len(counts)), torch.tensor(counts)).to(torch.int32)
    ops.kv_write(d(k_new), d(v_new), kpd, vpd, d(table), ring, d(pos), d(seq_of), d(slots), d(cu), d(lb))
    for b, t in enumerate(total):
        for p in range(max(0, t - ring * 64), t):
            pg = int(table[slots[b], (p // 64) % ring])
            assert torch.equal(kpd[pg, :, p % 64].cpu(), ks[b][p]) and torch.equal(vpd[pg, :, p % 64].cpu(), vs[b][p]), (b, p)
    if dtype == torch.bfloat16 and hd in (64, 128) and tc:
        assert ops.attn_tc_status() == 0


@pytest.mark.parametrize("tc", [True, False], ids=["tcgen05", "mma"])
@pytest.mark.parametrize("shape", ["slow", "steps"])
@pytest.mark.parametrize("hd", [64, 128])
def test_attn_prefill_scores_that_rise_along_the_keys(ops, hd, shape, tc, monkeypatch):
    """Scores that grow with the key's position move every row's maximum again and again: slowly (a few
    units per tile, which the tcgen05 kernel absorbs without rescaling its accumulator) or in steps of
    twenty units (which force a rescale in the middle of a sequence).  Eleven key tiles, a prompt that
    continues 70 cached tokens."""
    monkeypatch.setattr(ops, "USE_TC_PROMPT_ATTENTION", tc)
    dtype, nh, nkv, before, count = torch.bfloat16, 4, 2, 70, 640
    total = before + count
    g = torch.Generator().manual_seed(77 + hd)
    u = torch.randn(hd, generator=g)
    u = u / u.norm()
    pos = torch.arange(total, dtype=torch.float32)
    rise = pos * (40.0 / total) if shape == "slow" else 20.0 * ((pos >= 100).float() + (pos >= 333).float() + (pos >= 600).float())
    k = (0.3 * torch.randn(total, nkv, hd, generator=g) + rise[:, None, None] * u).to(dtype)
    v = torch.randn(total, nkv, hd, generator=g).to(dtype)
    q = (0.3 * torch.randn(count, nh, hd, generator=g) + u).to(dtype)
    ring = 12
    table = torch.zeros(3, ring, dtype=torch.int32)
    table[1] = torch.tensor([11, 3, 7, 0, 9, 1, 5, 10, 2, 8, 4, 6], dtype=torch.int32)
    kp = torch.zeros(12, nkv, 64, hd, dtype=dtype)
    vp = torch.zeros_like(kp)
    for p_ in range(before):
        kp[int(table[1, p_ // 64]), :, p_ % 64] = k[p_]
        vp[int(table[1, p_ // 64]), :, p_ % 64] = v[p_]
    tq = ops.prefill_tile_queries(dtype, hd)
    tiles = torch.tensor([(0, q0) for q0 in range(0, count, tq)], dtype=torch.int32)
    cu = torch.tensor([0, count], dtype=torch.int32)
    out = torch.empty(count, nh * hd, dtype=dtype, device=DEV)
    d = lambda t: t.to(DEV)
    ops.attn_prefill(d(q), d(k[before:].contiguous()), d(v[before:].contiguous()), d(kp), d(vp), d(table), ring, d(tiles), d(cu),
                     d(torch.tensor([before], dtype=torch.int32)), d(torch.tensor([1], dtype=torch.int32)), out,
                     scale=1.0, window=0, tile_queries=tq)
    qq = torch.zeros(total, nh, hd, dtype=dtype)
    qq[before:] = q
    ref = P.attention(qq, k, v, 1.0, 0)[before:].reshape(count, -1)
    check(out, ref, dtype, shape)
    if tc:
        assert ops.attn_tc_status() == 0


@pytest.mark.parametrize("tc", [True, False], ids=["tcgen05", "mma"])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("hd,window", [(64, 70), (128, 64), (128, 129), (48, 33)])
def test_attention_window_edge(ops, dtype, hd, window, tc, monkeypatch):
    """One key per query decides the output: the oldest key that the window still holds (position p - W + 1)
    for one head, and the newest that it no longer holds (p - W) for another.  The first must come out as
    that key's value, the second must leave no trace.  Prompt kernel (fresh keys and cached keys) and
    decode kernel."""
    if not tc and not (dtype == torch.bfloat16 and hd in (64, 128)):
        pytest.skip("only head sizes 64 and 128 in bfloat16 have two tensor-core kernels")
    monkeypatch.setattr(ops, "USE_TC_PROMPT_ATTENTION", tc)
    nh, nkv, before, count = 2, 1, 150, 260
    total = before + count
    g = torch.Generator().manual_seed(5 + hd + window)
    # key j carries a code of 24 signs, the query carries the code of the key it wants: the wanted key
    # scores 24 * 1.5 * 1.5 = 54, any other key about 0 +- 11
    k = 0.05 * torch.randn(total, nkv, hd, generator=g)
    # values that differ much between neighbouring positions, the same in every element of a row
    val = ((torch.arange(total) * 37) % 101).float() / 101
    v = val[:, None, None].expand(total, nkv, hd).clone()
    code = (torch.randint(0, 2, (total, 24), generator=g).float() * 2 - 1) * 1.5
    k[:, 0, 0:24] = code
    q = torch.zeros(total, nh, hd)
    for p_ in range(total):
        inside, outside = max(0, p_ - window + 1), p_ - window
        q[p_, 0, 0:24] = code[inside]                     # head 0: the oldest key the window still holds
        if outside >= 0:
            q[p_, 1, 0:24] = code[outside]                # head 1: the newest key it no longer holds
    k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
    ref = P.attention(q, k, v, 1.0, window)                       # [total, nh, hd]
    # the construction does what it says: head 0 lands on the edge key
    p_ = total - 1
    assert abs(float(ref[p_, 0, 5]) - float(val[p_ - window + 1])) < 0.004
    # and the key just outside, had it been let in, would have shown: without the window most rows differ
    free = P.attention(q, k, v, 1.0, 0)
    assert float(((free[before:, 1, 0] - ref[before:, 1, 0]).abs() > 0.1).float().mean()) > 0.6
    ring = (window + 63) // 64 + 1
    table = torch.zeros(2, ring, dtype=torch.int32)
    table[1] = torch.randperm(ring, generator=g).to(torch.int32)
    kp = torch.zeros(ring, nkv, 64, hd, dtype=dtype)
    vp = torch.zeros_like(kp)
    for j in range(max(0, before - ring * 64), before):
        kp[int(table[1, (j // 64) % ring]), :, j % 64] = k[j]
        vp[int(table[1, (j // 64) % ring]), :, j % 64] = v[j]
    tq = ops.prefill_tile_queries(dtype, hd)
    tiles = torch.tensor([(0, q0) for q0 in range(0, count, tq)], dtype=torch.int32)
    d = lambda t: t.to(DEV)
    out = torch.empty(count, nh * hd, dtype=dtype, device=DEV)
    kpd, vpd = d(kp), d(vp)
    cu, lb, sl = torch.tensor([0, count], dtype=torch.int32), torch.tensor([before], dtype=torch.int32), torch.tensor([1], dtype=torch.int32)
    ops.attn_prefill(d(q[before:].contiguous()), d(k[before:].contiguous()), d(v[before:].contiguous()), kpd, vpd, d(table), ring,
                     d(tiles), d(cu), d(lb), d(sl), out, scale=1.0, window=window, tile_queries=tq)
    check(out, ref[before:].reshape(count, -1), dtype, "prompt")
    # decode: the last token alone against the ring as the prompt step leaves it
    pos = torch.arange(before, total, dtype=torch.int32)
    ops.kv_write(d(k[before:].contiguous()), d(v[before:].contiguous()), kpd, vpd, d(table), ring, d(pos),
                 d(torch.zeros(count, dtype=torch.int32)), d(sl), d(cu), d(lb))
    out1 = torch.empty(1, nh * hd, dtype=dtype, device=DEV)
    for splits in (1, 2):
        scratch = torch.empty(ops.attn_decode_scratch_floats(1, nh, hd, splits), device=DEV)
        ops.attn_decode(d(q[-1:].contiguous()), kpd, vpd, d(table), ring, d(sl), d(torch.tensor([total - 1], dtype=torch.int32)),
                        out1, scratch, n_splits=splits, scale=1.0, window=window,
                        counters=torch.zeros(nkv, dtype=torch.int32, device=DEV))
        check(out1[0], ref[-1].reshape(-1), dtype, ("decode", splits))
    plan = ops.attn_decode_plan(dtype, 1, nh, nkv, hd, total)
    ops.attn_decode(d(q[-1:].contiguous()), kpd, vpd, d(table), ring, d(sl), d(torch.tensor([total - 1], dtype=torch.int32)),
                    out1, torch.empty(max(1, plan.scratch_floats), device=DEV), scale=1.0, window=window, plan=plan,
                    counters=torch.zeros(max(1, plan.n_counters), dtype=torch.int32, device=DEV))
    check(out1[0], ref[-1].reshape(-1), dtype, ("decode", plan.kind))


@pytest.mark.parametrize("tc", [True, False], ids=["tcgen05", "mma"])
@pytest.mark.parametrize("hd", [64, 128, 48])
def test_attention_with_whole_number_scores_rounds_like_the_plain_model(ops, hd, tc, monkeypatch):
    """Queries and keys of -1, 0 and 1 with a softmax scale of ln 2 give scores that are whole numbers of binary
    orders, so every softmax weight is a power of two and bfloat16 holds it exactly: the only rounding left is
    that of the output.  The kernels must then give the plain model's bits, but for the few values that lie
    within float32 error of a tie (each one unit in the last place off).  A kernel that loses a hundredth of a
    row's weight, drops a tile or counts a key twice moves nearly every value of the row instead.  Prompt step
    on cached tokens, then the last token alone with its keys split over blocks in several ways."""
    if not tc and hd not in (64, 128):
        pytest.skip("only head sizes 64 and 128 have two tensor-core kernels")
    monkeypatch.setattr(ops, "USE_TC_PROMPT_ATTENTION", tc)
    dtype, nh, nkv, before, count = torch.bfloat16, 4, 2, 130, 330
    total = before + count
    g = torch.Generator().manual_seed(900 + hd)
    k = torch.randint(-1, 2, (total, nkv, hd), generator=g).to(dtype)
    q = torch.randint(-1, 2, (total, nh, hd), generator=g).to(dtype)
    v = torch.randn(total, nkv, hd, generator=g).to(dtype)
    scale = math.log(2.0)
    ref = P.round_bfloat16(P.attention(q, k, v, scale, 0, round_weights=P.round_bfloat16))      # [total, nh, hd]

    def same_bits(got, want, what):
        got, want = got.detach().cpu().double().reshape(-1), want.reshape(-1)
        off = (got != want)
        assert float(off.float().mean()) <= 0.005, (what, "values that differ", int(off.sum()), "of", off.numel())
        # what differs is one unit in the last place of a bfloat16 value (2^-7 of it, at most); a value that is
        # small because its terms cancel carries the float32 error of those terms (values are of order one)
        assert bool(((got - want).abs()[off] <= want.abs()[off] * 2.0 ** -7 + 2e-6).all()), what

    ring = 8
    table = torch.zeros(2, ring, dtype=torch.int32)
    table[1] = torch.randperm(ring, generator=g).to(torch.int32)
    kp = torch.zeros(ring, nkv, 64, hd, dtype=dtype)
    vp = torch.zeros_like(kp)
    for j in range(before):
        kp[int(table[1, j // 64]), :, j % 64] = k[j]
        vp[int(table[1, j // 64]), :, j % 64] = v[j]
    tq = ops.prefill_tile_queries(dtype, hd)
    tiles = torch.tensor([(0, q0) for q0 in range(0, count, tq)], dtype=torch.int32)
    d = lambda t: t.to(DEV)
    out = torch.empty(count, nh * hd, dtype=dtype, device=DEV)
    kpd, vpd = d(kp), d(vp)
    cu, lb, sl = torch.tensor([0, count], dtype=torch.int32), torch.tensor([before], dtype=torch.int32), torch.tensor([1], dtype=torch.int32)
    ops.attn_prefill(d(q[before:].contiguous()), d(k[before:].contiguous()), d(v[before:].contiguous()), kpd, vpd, d(table), ring,
                     d(tiles), d(cu), d(lb), d(sl), out, scale=scale, window=0, tile_queries=tq)
    same_bits(out, ref[before:], "prompt")
    ops.kv_write(d(k[before:].contiguous()), d(v[before:].contiguous()), kpd, vpd, d(table), ring,
                 d(torch.arange(before, total, dtype=torch.int32)), d(torch.zeros(count, dtype=torch.int32)), d(sl), d(cu), d(lb))
    # the last 24 tokens as a batch of 24 sequences that share the pages (each sees its own length)
    n_dec = 24
    qd = q[total - n_dec:].contiguous()
    slots = torch.ones(n_dec, dtype=torch.int32)
    lens = torch.arange(total - n_dec, total, dtype=torch.int32)             # keys before the token
    counters = torch.zeros(n_dec * nkv, dtype=torch.int32, device=DEV)
    for splits, balance in ((1, False), (3, False), (8, True)):
        out1 = torch.empty(n_dec, nh * hd, dtype=dtype, device=DEV)
        scratch = torch.empty(ops.attn_decode_scratch_floats(n_dec, nh, hd, splits), device=DEV)
        ops.attn_decode(d(qd), kpd, vpd, d(table), ring, d(slots), d(lens), out1, scratch, n_splits=splits, scale=scale,
                        window=0, counters=counters, balance=balance)
        same_bits(out1, ref[total - n_dec:], ("decode", splits, balance))
    plan = ops.attn_decode_plan(dtype, n_dec, nh, nkv, hd, total)
    out1 = torch.empty(n_dec, nh * hd, dtype=dtype, device=DEV)
    ops.attn_decode(d(qd), kpd, vpd, d(table), ring, d(slots), d(lens), out1,
                    torch.empty(max(1, plan.scratch_floats), device=DEV), scale=scale, window=0, plan=plan,
                    counters=torch.zeros(max(1, plan.n_counters), dtype=torch.int32, device=DEV))
    same_bits(out1, ref[total - n_dec:], ("decode", plan.kind))
    if tc:
        assert ops.attn_tc_status() == 0


@pytest.mark.parametrize("nh,nkv,hd,k,norm,bias,rotate,pages", [(3, 1, 128, 264, True, True, True, True), (5, 2, 64, 96, False, False, True, False),
                                                            (2, 2, 128, 512, True, False, False, True), (4, 1, 64, 200, False, True, True, True)])
def test_qkv_product_with_the_preparation_as_its_epilogue(ops, nh, nkv, hd, k, norm, bias, rotate, pages):
    """The q/k/v projection whose epilogue normalises, adds the bias, rotates and writes q, k and v (one kernel)
    against the plain formulas, and against the product followed by the preparation kernel (the same float32
    sums, so at most a value here and there rounds the other way).  Two sequences in one step of 700 tokens, the
    second continuing at position 70; widths that are no multiple of the tile."""
    dtype = torch.bfloat16
    counts, before = [430, 270], [0, 70]
    n = sum(counts)
    o = (nh + 2 * nkv) * hd
    x = rnd((n, k), 81, dtype)
    w = rnd((o, k), 82, dtype, 1.0 / math.sqrt(k))
    qw = (rnd((hd,), 83, dtype, 0.1) + 1) if norm else None
    kw_ = (rnd((hd,), 84, dtype, 0.1) + 1) if norm else None
    b = rnd((o,), 85, dtype, 0.3) if bias else None
    pos = torch.cat([torch.arange(bf, bf + c) for bf, c in zip(before, counts)]).to(torch.int32)
    seq_of = torch.repeat_interleave(torch.arange(2), torch.tensor(counts)).to(torch.int32)
    inv = P.rope_inverse_frequencies(hd, 3e4, None)
    ang = torch.arange(600, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    # plain: sums, per-head norm, bias, rotation
    y = P.linear(x, w).view(n, nh + 2 * nkv, hd)
    q, kk, v = y[:, :nh], y[:, nh:nh + nkv], y[:, nh + nkv:]
    if norm:
        q, kk = P.per_head_rms_norm(q, qw, 1e-5), P.per_head_rms_norm(kk, kw_, 1e-5)
    if bias:
        bb = b.double().view(nh + 2 * nkv, hd)
        q, kk, v = q + bb[:nh], kk + bb[nh:nh + nkv], v + bb[nh + nkv:]
    if rotate:
        q, kk = P.rope_rotate(q, pos.tolist(), inv, "half"), P.rope_rotate(kk, pos.tolist(), inv, "half")
    d = lambda t: None if t is None else t.to(DEV)
    ring, n_pages = 8, 16
    table = torch.zeros(3, ring, dtype=torch.int32)
    table[1] = torch.tensor([9, 3, 7, 0, 11, 1, 5, 10])
    table[2] = torch.tensor([2, 8, 4, 6, 12, 13, 14, 15])
    slots = torch.tensor([2, 1], dtype=torch.int32)
    common = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, q_norm_w=d(qw), k_norm_w=d(kw_), norm_eps=1e-5, bias=d(b),
                  cos=d(cos) if rotate else None, sin=d(sin) if rotate else None, rotary_dim=hd if rotate else 0, pairing=0,
                  positions=d(pos))
    outs = {}
    for way in ("fused", "two kernels"):
        q_out = torch.full((n, nh, hd), float("nan"), dtype=dtype, device=DEV)
        k_new, v_new = torch.full((n, nkv, hd), float("nan"), dtype=dtype, device=DEV), torch.full((n, nkv, hd), float("nan"), dtype=dtype, device=DEV)
        kp, vp = torch.zeros(n_pages, nkv, 64, hd, dtype=dtype, device=DEV), torch.zeros(n_pages, nkv, 64, hd, dtype=dtype, device=DEV)
        extra = dict(k_pages=kp, v_pages=vp, page_table=d(table), ring_pages=ring, seq_of_token=d(seq_of), slots=d(slots)) if pages else {}
        if way == "fused":
            assert ops.gemm_tc_qkv_supported(d(x), d(w), hd, hd if rotate else 0, 0)
            ops.gemm_tc_qkv(d(x), d(w), **common, q_out=q_out, k_new=k_new, v_new=v_new, **extra)
        else:
            sums = torch.empty(1, n, o, device=DEV)
            ops.gemm_tc(d(x), d(w), sums)
            ops.qk_prep(sums, **common, q_out=q_out, k_new=k_new, v_new=v_new, **extra)
        outs[way] = (q_out.cpu(), k_new.cpu(), v_new.cpu(), kp.cpu(), vp.cpu())
    assert ops.gemm_tc_status() == 0
    fq, fk, fv, fkp, fvp = outs["fused"]
    check(fq, q, dtype, "q")
    check(fk, kk, dtype, "k")
    check(fv, v, dtype, "v")
    for name_, a_, b_ in zip("qkv", outs["fused"][:3], outs["two kernels"][:3]):
        off = a_.float() != b_.float()
        assert float(off.float().mean()) < 0.005, (name_, int(off.sum()))
        assert bool(((a_.float() - b_.float()).abs()[off] <= b_.float().abs()[off] * 2.0 ** -7 + 1e-6).all()), name_
    if pages:
        for t in range(n):                              # every key and value lies where its position says
            s_, p_ = int(slots[seq_of[t]]), int(pos[t])
            pg = int(table[s_, (p_ // 64) % ring])
            assert torch.equal(fkp[pg, :, p_ % 64], fk[t]) and torch.equal(fvp[pg, :, p_ % 64], fv[t]), t
    else:
        assert float(fkp.abs().sum()) == 0


# ---- a norm that leaves its division to the products that consume it ------------------------------------------------

def _scale_of(ss, width, eps):
    """The factor a row scale stands for: 1 / sqrt(sum(ss) / width + eps) per row, float64."""
    return 1.0 / torch.sqrt(ss.double().sum(dim=1) / width + eps)


@pytest.mark.parametrize("hidden,n", [(70, 4), (72, 5), (1000, 3), (1024, 1), (4096, 8), (4096, 64), (4096, 300), (4100, 2), (8192, 5)])
def test_add_rmsnorm_without_the_division(ops, hidden, n):
    """With ``ss_out`` the norm writes the summed row times the weight (no division) and the row's sum of squares,
    whole or, for the few rows of a decode step, as the sums of equal slices of the row (each slice a block of its
    own); the residual is updated as always.  Rows gathered through ``rows`` as well."""
    res = rnd((n, hidden), 1)
    branch = rnd((9, n, hidden), 2, scale=0.5)
    w = (rnd((hidden,), 3, torch.bfloat16, 0.1) + 1)
    v = res.double() + branch.double().sum(0)
    parts = ops.norm_ss_parts(n, hidden)
    assert parts == (hidden // 256 if n <= 64 and hidden >= 1024 and hidden % 256 == 0 else 1)
    r = res.to(DEV)
    out = torch.empty(n, hidden, dtype=torch.bfloat16, device=DEV)
    ss = torch.full((n, parts), float("nan"), device=DEV)
    ops.add_rmsnorm(r, branch.to(DEV), w.to(DEV), 1e-5, out, ss_out=ss)
    assert float((r.cpu().double() - v).abs().max()) < 2e-5
    want = P.round_bfloat16(v * w.double())
    off = out.cpu().double() != want
    assert float(off.double().mean()) < 0.002                     # a float32 sum within an ulp of a tie
    assert bool(((out.cpu().double() - want).abs() <= want.abs() * 2.0 ** -7 + 1e-6).all())     # + what a cancelled float32 sum is off by
    sq = (v * v).view(n, parts, hidden // parts).sum(2)
    assert float(((ss.cpu().double() - sq) / sq).abs().max()) < 1e-5
    rows = torch.tensor([n - 1, 0], dtype=torch.int32)
    out2 = torch.empty(2, hidden, dtype=torch.bfloat16, device=DEV)
    ss2 = torch.empty(2, ops.norm_ss_parts(2, hidden), device=DEV)
    ops.add_rmsnorm(r, None, w.to(DEV), 1e-5, out2, rows.to(DEV), ss_out=ss2)
    assert torch.equal(out2.cpu(), out.cpu()[rows.long()])
    assert float((ss2.cpu().sum(1) / ss.cpu()[rows.long()].sum(1) - 1).abs().max()) < 1e-6     # another kernel may add in another order


@pytest.mark.parametrize("parts", [1, 5])
@pytest.mark.parametrize("n,o,k", [(1, 200, 72), (16, 384, 1000), (40, 130, 256), (100, 257, 64), (200, 300, 136), (300, 512, 264), (700, 200, 64)])
def test_products_apply_a_row_scale(ops, n, o, k, parts):
    """Every product that may follow a norm multiplies its rows by the scale the norm left: the tensor-core product in
    both orientations, with partial sums and with the gated epilogue, and the CUDA-core product."""
    x = rnd((n, k), 11, torch.bfloat16)
    w = rnd((o, k), 12, torch.bfloat16, 1.0 / math.sqrt(k))
    ss = (rnd((n, parts), 13).abs() * 50 + 1)
    scale = ops.RowScale(ss.to(DEV), 96, 1e-3)
    f = _scale_of(ss, 96, 1e-3)[:, None]
    want = P.linear(x, w) * f
    for splits in (1, ops.gemm_tc_splits(k, 3)):
        out = torch.empty(splits, n, o, device=DEV)
        ops.gemm_tc(x.to(DEV), w.to(DEV), out, row_scale=scale)
        check(out.sum(0).cpu(), want, torch.float32, f"gemm_tc splits={splits}")
    out = torch.empty(1, n, o, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x.to(DEV), w.to(DEV), out, row_scale=scale)
    check(out[0].cpu(), want, torch.bfloat16, "gemm_tc bfloat16")
    out = torch.empty(n, o, device=DEV)
    ops.gemm_simt(x.to(DEV), w.to(DEV), out, row_scale=scale)
    check(out.cpu(), want, torch.float32, "gemm_simt")
    # gated: silu(scale * gate) * (scale * up)
    feat = o // 2
    gate, up = w[:feat], w[feat:2 * feat]
    g, u = P.linear(x, gate) * f, P.linear(x, up) * f
    act = torch.empty(1, n, feat, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x.to(DEV), _gated(gate, up).to(DEV), act, gated_features=feat, row_scale=scale)
    check(act[0].cpu(), g / (1 + torch.exp(-g)) * u, torch.bfloat16, "gated")
    assert ops.gemm_tc_status() == 0
    with pytest.raises(ops.KernelError, match="rows"):
        ops.gemm_simt(x.to(DEV), w.to(DEV), out, row_scale=ops.RowScale(ss[:-1].to(DEV) if n > 1 else torch.ones(2, 1, device=DEV), 96, 1e-3))


def test_kernels_refuse_what_they_cannot_do(ops):
    q = torch.zeros(1, 2, 272, device=DEV)
    kp = torch.zeros(1, 1, 64, 272, device=DEV)
    table = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError, match="head_dim 272"):
        ops.attn_decode(q, kp, kp, table, 1, z, z, torch.zeros(1, 544, device=DEV), torch.zeros(4096, device=DEV),
                        n_splits=1, scale=1.0, window=0)
    with pytest.raises(ops.KernelError, match="not on the GPU"):
        ops.argmax(torch.zeros(1, 4), torch.zeros(1, dtype=torch.int32, device=DEV))
    with pytest.raises(ops.KernelError, match="multiple"):
        ops.attn_decode(torch.zeros(1, 3, 16, device=DEV), torch.zeros(1, 2, 64, 16, device=DEV),
                        torch.zeros(1, 2, 64, 16, device=DEV), table, 1, z, z, torch.zeros(1, 48, device=DEV),
                        torch.zeros(4096, device=DEV), n_splits=1, scale=1.0, window=0)


def test_argmax_takes_the_first_maximum(ops):
    x = rnd((6, 50001), 50)
    x[1, 4000] = x[1, 40000] = 99.0
    x[2, 50000] = 99.0
    x[3, 0] = 99.0
    x[4] = 0.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.argmax(x.to(DEV), out)
    want = [int(x[0].argmax()), 4000, 50000, 0, 0, int(x[5].argmax())]
    assert out.cpu().tolist() == want


SAMPLE_CASES = [
    dict(temperature=0.8), dict(temperature=1.3, top_k=40), dict(temperature=0.7, top_p=0.9),
    dict(temperature=1.0, min_p=0.05), dict(temperature=1.0, typical_p=0.7),
    dict(temperature=0.9, top_k=50, top_p=0.8, min_p=0.01, typical_p=0.9, repetition_penalty=1.3,
         frequency_penalty=0.2, presence_penalty=0.1),
    dict(temperature=0.0, repetition_penalty=1.5), dict(temperature=1.0, top_p=0.5, min_keep=30),
    dict(temperature=1.0, top_k=1), dict(temperature=2.0, top_k=5000), dict(temperature=0.6, banned=[3, 77]),
]


@pytest.mark.parametrize("case", range(len(SAMPLE_CASES)))
def test_sampler_distribution_and_draw(ops, case):
    c = dict(SAMPLE_CASES[case])
    banned = c.pop("banned", None)
    vocab, b = 1531, 4
    logits = rnd((b, vocab), 60, scale=3.0)
    g = torch.Generator().manual_seed(61)
    hist = torch.randint(0, vocab, (b, 16), generator=g, dtype=torch.int32)
    hist[:, 5] = hist[:, 2]
    hl = torch.tensor([16, 9, 0, 16], dtype=torch.int32)
    work = torch.empty(b * vocab, device=DEV)
    out = torch.empty(b, dtype=torch.int32, device=DEV)
    probs = torch.empty(b, vocab, device=DEV)
    seq_ids = torch.tensor([9, 2, 5, 40], dtype=torch.int32)
    ops.sample(logits.to(DEV), work, out, seed=11, step=5, history=hist.to(DEV), history_len=hl.to(DEV),
               probs_out=probs, seq_ids=seq_ids.to(DEV),
               banned=None if banned is None else torch.tensor(banned, dtype=torch.int32, device=DEV), **c)
    for i in range(b):
        ref = P.sampling_distribution(logits[i].tolist(), previous=hist[i, :hl[i]].tolist(), banned=banned or (), **c)
        got = probs[i].cpu().double()
        assert float((got - ref).abs().max()) < 2e-6, (i, c)
        assert ((got > 0) == (ref > 0)).all()
        assert int(out[i]) == P.draw(got, P.uniform_of(11, int(seq_ids[i]), 5))


@pytest.mark.parametrize("case", [dict(temperature=0.7, top_k=40, top_p=0.9, repetition_penalty=1.1),
                                  dict(temperature=1.0, top_k=64, min_p=0.02, typical_p=0.8, frequency_penalty=0.3),
                                  dict(temperature=1.4, top_k=1), dict(temperature=0.9, top_k=7, min_keep=5, top_p=0.3),
                                  dict(temperature=0.8, top_k=33, banned=[5, 9000, 20010])])
def test_sampler_by_candidates_equals_the_general_way(ops, case):
    """With top-k up to 64 the vocabulary is cut into slices whose best tokens alone reach the filters: the
    distribution and the draw are those of the general way over the whole vocabulary, also when the recent
    tokens and the banned ones lie in different slices, and when ties at a slice's k-th value overflow its
    64 candidates (that row then takes the general way)."""
    c = dict(case)
    banned = c.pop("banned", None)
    vocab, b = 20011, 5                       # three slices of 8192, the last one short
    logits = rnd((b, vocab), 70, scale=3.0)
    logits[1, 100:400] = 9.5                  # 300 equal logits at the top of a slice: more ties than candidates fit
    logits[2, 8190:8194] = 12.0               # the best tokens straddle a slice boundary
    logits[3, 19000:] = -50.0                 # a short last slice with nothing worth keeping
    g = torch.Generator().manual_seed(71)
    hist = torch.randint(0, vocab, (b, 64), generator=g, dtype=torch.int32)
    hist[:, 7] = hist[:, 3]
    hist[2, 0], hist[2, 1], hist[2, 2] = 8191, 8192, 8193
    hl = torch.tensor([64, 20, 64, 0, 33], dtype=torch.int32)
    seq_ids = torch.tensor([3, 1, 4, 1, 5], dtype=torch.int32)
    res = []
    for cand in (True, False):
        work = torch.empty(b * vocab, device=DEV)
        out = torch.empty(b, dtype=torch.int32, device=DEV)
        probs = torch.full((b, vocab), float("nan"), device=DEV)
        ops.sample(logits.to(DEV), work, out, seed=13, step=2, history=hist.to(DEV), history_len=hl.to(DEV),
                   probs_out=probs, seq_ids=seq_ids.to(DEV), candidates=cand,
                   banned=None if banned is None else torch.tensor(banned, dtype=torch.int32, device=DEV), **c)
        res.append((out.cpu(), probs.cpu()))
    assert torch.equal(res[0][0], res[1][0])
    assert ((res[0][1] > 0) == (res[1][1] > 0)).all()
    assert float((res[0][1] - res[1][1]).abs().max()) < 1e-6
    for i in (0, 2):
        ref = P.sampling_distribution(logits[i].tolist(), previous=hist[i, :hl[i]].tolist(), banned=banned or (), **c)
        assert float((res[0][1][i].double() - ref).abs().max()) < 2e-6
        assert int(res[0][0][i]) == P.draw(res[0][1][i].double(), P.uniform_of(13, int(seq_ids[i]), 2))


@pytest.mark.parametrize("case", [dict(temperature=0.7), dict(temperature=1.3, repetition_penalty=1.2, banned=[5, 9000, 20010]),
                                  dict(temperature=0.8, top_p=0.9), dict(temperature=1.0, top_p=0.5, frequency_penalty=0.4),
                                  dict(temperature=0.9, min_p=0.05), dict(temperature=1.1, min_p=0.01, top_p=0.8),
                                  dict(temperature=6.0, top_p=0.97), dict(temperature=5.0, min_p=0.001)])
def test_sampler_without_top_k_through_the_slices(ops, case):
    """Without top-k the slices' 64 largest logits and their sums stand for the row as long as they can decide the
    outcome: temperature alone draws over the whole row (the slice by the slices' masses, the token by one pass
    over that slice); top-p and min-p run on the candidates with the whole row's normaliser.  Distribution and draw
    are those of the general way; where the kept set reaches below the candidates (high temperatures here) or a
    slice has more ties than candidates fit, the row takes the general way by itself."""
    c = dict(case)
    banned = c.pop("banned", None)
    vocab, b = 20011, 6
    logits = rnd((b, vocab), 72, scale=3.0)
    logits[1, 100:400] = 9.5                  # more ties at the top of a slice than candidates fit
    logits[2, 8190:8194] = 12.0               # the best tokens straddle a slice boundary
    logits[3, 19000:] = -50.0                 # a short last slice with nothing worth keeping
    logits[4] = rnd((vocab,), 73, scale=0.2)  # nearly flat: the kept set is most of the row
    g = torch.Generator().manual_seed(74)
    hist = torch.randint(0, vocab, (b, 64), generator=g, dtype=torch.int32)
    hist[2, 0], hist[2, 1], hist[2, 2] = 8191, 8192, 8193
    hl = torch.tensor([64, 20, 64, 0, 33, 5], dtype=torch.int32)
    seq_ids = torch.tensor([3, 1, 4, 1, 5, 9], dtype=torch.int32)
    for step in (2, 3, 4):                    # three uniform numbers per row
        res = []
        for cand in (True, False):
            work = torch.empty(b * vocab, device=DEV)
            out = torch.empty(b, dtype=torch.int32, device=DEV)
            probs = torch.full((b, vocab), float("nan"), device=DEV)
            ops.sample(logits.to(DEV), work, out, seed=13, step=step, history=hist.to(DEV), history_len=hl.to(DEV),
                       probs_out=probs, seq_ids=seq_ids.to(DEV), candidates=cand,
                       banned=None if banned is None else torch.tensor(banned, dtype=torch.int32, device=DEV), **c)
            res.append((out.cpu(), probs.cpu()))
        assert ((res[0][1] > 0) == (res[1][1] > 0)).all()
        assert float((res[0][1] - res[1][1]).abs().max()) < 1e-6
        for i in range(b):
            pd = res[0][1][i].double()
            u = P.uniform_of(13, int(seq_ids[i]), step)
            cdf = torch.cumsum(pd, 0) / pd.sum()
            near = float((cdf - u).abs().min()) < 1e-5          # the drawn point within rounding of a boundary
            assert int(res[0][0][i]) == int(res[1][0][i]) or near, (i, step)
            assert int(res[0][0][i]) == P.draw(pd, u) or near, (i, step)
            assert float(pd[int(res[0][0][i])]) > 0
    for i in (0, 2, 4):
        ref = P.sampling_distribution(logits[i].tolist(), previous=hist[i, :hl[i]].tolist(), banned=banned or (),
                                      top_k=0, **c)
        assert float((res[0][1][i].double() - ref).abs().max()) < 2e-6


@pytest.mark.parametrize("top_k", [1, 3, 40, 200])
def test_top_k_keeps_exactly_k_at_ties(ops, top_k):
    """Logits on a coarse grid, so that many tie with the k-th largest: exactly k stay, the smallest tokens
    among the ties (the reference's selection keeps the first it meets, Sampler.cs:249-276), in the general
    way and through the candidates; top_k = 1 is the greedy choice."""
    vocab, b = 20011, 4
    logits = (rnd((b, vocab), 80, scale=3.0) * 2).round() / 2
    logits[1, 8000:8400] = 20.0               # 400 equal maxima across a slice boundary
    logits[2, 19990:] = 20.0
    for cand in (True, False):
        work = torch.empty(b * vocab, device=DEV)
        out = torch.empty(b, dtype=torch.int32, device=DEV)
        probs = torch.full((b, vocab), float("nan"), device=DEV)
        ops.sample(logits.to(DEV), work, out, seed=5, step=9, temperature=0.9, top_k=top_k, probs_out=probs,
                   candidates=cand)
        for i in range(b):
            ref = P.sampling_distribution(logits[i].tolist(), temperature=0.9, top_k=top_k)
            got = probs[i].cpu().double()
            assert int((got > 0).sum()) == top_k, (cand, i)
            assert ((got > 0) == (ref > 0)).all(), (cand, i)
            assert float((got - ref).abs().max()) < 2e-6
            if top_k == 1:
                assert int(out[i]) == int(logits[i].argmax())      # torch: the first maximum


def test_sampler_draws_follow_the_distribution(ops):
    vocab = 37
    logits = rnd((1, vocab), 62, scale=1.5).repeat(512, 1)
    work = torch.empty(512 * vocab, device=DEV)
    out = torch.empty(512, dtype=torch.int32, device=DEV)
    counts = torch.zeros(vocab)
    for step in range(8):
        ops.sample(logits.to(DEV), work, out, temperature=1.0, seed=123, step=step)
        counts += torch.bincount(out.cpu().long(), minlength=vocab)
    p = torch.softmax(logits[0].double(), 0)
    n = counts.sum()
    chi2 = float((((counts - n * p) ** 2) / (n * p)).sum())
    assert chi2 < 75, chi2          # 36 degrees of freedom: far in the tail beyond 75
    # same seed, same draws; another seed, other draws
    a = torch.empty(512, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), work, a, temperature=1.0, seed=123, step=7)
    assert torch.equal(a, out)
    ops.sample(logits.to(DEV), work, a, temperature=1.0, seed=124, step=7)
    assert not torch.equal(a, out)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_fill_normal_is_the_hosts_generator(ops, llogos, dtype):
    """The fill kernel and the numpy restatement of the same counter-based generator give the same bits, for
    sizes that are no multiple of anything, a mean and a spread, and keys of different tensors; so a model
    initialised on the GPU holds the weights that a model written to a file from the same seed holds."""
    ri = importlib.import_module("daisi-llogos_b200.weights.random_init")
    for n, name, mean, std in ((1, "a", 0.0, 1.0), (1000003, "model.layers.3.mlp.up_proj.weight", 0.0, 0.02),
                               (4097, "model.norm.weight", 1.0, 0.1), (65536, "b", -2.0, 3.0)):
        key = ri.tensor_key(11, name)
        got = torch.empty(n, dtype=dtype, device=DEV)
        ops.fill_normal(got, key, mean, std)
        want = torch.from_numpy(ri.normal_values(key, n, mean, std)).to(dtype)
        assert torch.equal(got.cpu(), want), (n, name)
    decls = {"x.weight": llogos.parts.TensorDecl((33, 70)), "x.norm": llogos.parts.TensorDecl((70,), "norm"),
             "x.bias": llogos.parts.TensorDecl((33,), "bias")}
    kw = dict(std=0.3, norm_std=0.1, bias_std=0.05, dtype=dtype)
    on_gpu = llogos.weights.random_tensors(decls, 5, device=DEV, **kw)
    on_cpu = llogos.weights.random_tensors(decls, 5, device="cpu", **kw)
    for k in decls:
        assert torch.equal(on_gpu[k].cpu(), on_cpu[k]), k


def test_cast_and_fill(ops):
    x = rnd((5, 1001), 71)
    half = torch.empty(5, 1001, dtype=torch.bfloat16, device=DEV)
    ops.cast(x.to(DEV), half)
    assert torch.equal(half.cpu(), x.to(torch.bfloat16))            # round to nearest even
    back = torch.empty(5, 1001, device=DEV)
    ops.cast(half, back)
    assert torch.equal(back.cpu(), x.to(torch.bfloat16).float())
    ops.fill(back, 88.0)
    assert float(back.min()) == 88.0 == float(back.max())

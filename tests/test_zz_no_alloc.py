"""llg_attn_decode_noalloc, the decode-attention entry point for callers that cannot allocate.

Some users of the kernels run where cudaMalloc is off the table (a thread that must not block on
the allocator, a plugin inside another program's memory budget, a loop that was told "no
allocation after start-up").  For them the library has one entry point whose scratch is a fixed
array inside the library itself.  This test calls it the way such a caller would: through the
exported C symbol of the shared library, with raw pointers, twice in a row, and checks that it
gives what the ordinary entry point gives.  The file's name makes pytest collect it last.
"""
import ctypes
import importlib
import math

import pytest
import torch

import plain_model as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_FLOATS = 1 << 20


def _library():
    build = importlib.import_module("daisi-llogos_b200.csrc.build")
    lib = ctypes.CDLL(build.compile_library("attention_simt"))
    fn = lib.llg_attn_decode_noalloc
    V, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [V, V, V, V, I, I, V, V, V, I, I, I, I, I, I, F, I, V]
    fn.restype = I
    lib.llg_last_error.restype = ctypes.c_char_p
    return lib, fn


def _case(seed, dtype, lens, nh, nkv, hd, n_pages=48, ring=8):
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(len(lens) + 1, ring, dtype=torch.int32)
    slots = torch.arange(len(lens), 0, -1, dtype=torch.int32)
    for b, n in enumerate(lens):
        for j in range((n + 63) // 64):
            table[slots[b], j] = order.pop()
    kp = torch.randn(n_pages, nkv, 64, hd, generator=g).to(dtype)
    vp = torch.randn(n_pages, nkv, 64, hd, generator=g).to(dtype)
    q = torch.randn(len(lens), nh, hd, generator=g).to(dtype)
    lb = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    return [t.to(DEV) for t in (q, kp, vp, table, slots, lb)]


def plain_decode(q, kp, vp, table, slots, lb, scale, window):
    """What the entry point has to give, from the plain attention of whole sequences: the keys and values of
    sequence b are gathered from its pages in position order (position p lies in page ``table[slot][(p // 64)
    % ring]`` at row ``p % 64``), the new token's query is the last row, and the last row of the plain causal
    attention (with the window, if any) is the answer."""
    q, kp, vp = q.cpu().double(), kp.cpu().double(), vp.cpu().double()
    table, slots, lb = table.cpu(), slots.cpu().tolist(), lb.cpu().tolist()
    nh, hd = q.shape[1], q.shape[2]
    ring = table.shape[1]
    out = torch.zeros(q.shape[0], nh * hd, dtype=torch.float64)
    for b, (slot, before) in enumerate(zip(slots, lb)):
        n = before + 1
        first = max(0, n - window) if window > 0 else 0          # earlier keys are outside the window anyway
        pos = list(range(first, n))
        pages = [int(table[slot, (p // 64) % ring]) for p in pos]
        k = torch.stack([kp[pg, :, p % 64] for pg, p in zip(pages, pos)])
        v = torch.stack([vp[pg, :, p % 64] for pg, p in zip(pages, pos)])
        qs = torch.zeros(len(pos), nh, hd, dtype=torch.float64)
        qs[-1] = q[b]
        out[b] = P.attention(qs, k, v, scale, window)[-1].reshape(-1)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_matches_the_ordinary_entry_point_twice_in_a_row(dtype):
    ops = importlib.import_module("daisi-llogos_b200.kernels.ops")
    lib, fn = _library()
    code = 0 if dtype == torch.float32 else 1
    tol = 2e-5 if dtype == torch.float32 else 1.6e-2
    # the second call is smaller than the first, so it finds the first call's leftovers in the array
    for seed, lens, nh, nkv, hd, splits, window in ((1, [300, 65, 1, 129], 6, 2, 80, 5, 0), (2, [70, 200], 4, 4, 32, 3, 100)):
        q, kp, vp, table, slots, lb = _case(seed, dtype, lens, nh, nkv, hd)
        scale = 1 / math.sqrt(hd)
        want = torch.empty(len(lens), nh * hd, dtype=dtype, device=DEV)
        scratch = torch.empty(ops.attn_decode_scratch_floats(len(lens), nh, hd, splits), device=DEV)
        ops.attn_decode(q, kp, vp, table, table.shape[1], slots, lb, want, scratch, n_splits=splits, scale=scale, window=window,
                        counters=torch.zeros(len(lens) * nkv, dtype=torch.int32, device=DEV))
        got = torch.full_like(want, float("nan"))
        rc = fn(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.shape[1], table.shape[1],
                slots.data_ptr(), lb.data_ptr(), got.data_ptr(), code, len(lens), nh, nkv, hd, splits, scale, window,
                torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.llg_last_error()
        torch.cuda.synchronize()
        err = float((got.double() - want.double()).abs().max())
        assert err <= tol * max(1.0, float(want.double().abs().max())), (seed, err)
        # and against the plain formula, which shares nothing with either entry point
        plain = plain_decode(q, kp, vp, table, slots, lb, scale, window)
        err = float((got.double().cpu() - plain).abs().max())
        assert err <= tol * max(1.0, float(plain.abs().max())), (seed, "plain", err)


def test_a_request_that_fills_the_array_exactly_runs():
    """8 sequences x 32 heads x 64 splits x (62 + 2) floats are the array's 1,048,576 floats to the last one;
    most sequences have fewer key tiles than splits, so many splits stay empty."""
    lib, fn = _library()
    lens, nh, nkv, hd, splits = [1500, 70, 1, 129, 640, 64, 65, 900], 32, 8, 62, 64
    assert len(lens) * nh * splits * (hd + 2) == MAX_FLOATS
    q, kp, vp, table, slots, lb = _case(4, torch.float32, lens, nh, nkv, hd, n_pages=64, ring=24)
    scale = 1 / math.sqrt(hd)
    got = torch.full((len(lens), nh * hd), float("nan"), device=DEV)
    rc = fn(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.shape[1], table.shape[1],
            slots.data_ptr(), lb.data_ptr(), got.data_ptr(), 0, len(lens), nh, nkv, hd, splits, scale, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.llg_last_error()
    torch.cuda.synchronize()
    plain = plain_decode(q, kp, vp, table, slots, lb, scale, 0)
    err = float((got.double().cpu() - plain).abs().max())
    assert err <= 2e-5 * max(1.0, float(plain.abs().max())), err
    # one split more is one float too many
    rc = fn(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.shape[1], table.shape[1],
            slots.data_ptr(), lb.data_ptr(), got.data_ptr(), 0, len(lens), nh, nkv, hd, splits + 1, scale, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "1048576" in lib.llg_last_error().decode()


def test_refuses_more_than_its_array_holds():
    lib, fn = _library()
    q, kp, vp, table, slots, lb = _case(3, torch.float32, [10], 4, 4, 32)
    out = torch.zeros(1, 128, device=DEV)
    too_many = MAX_FLOATS // (4 * 34) + 1          # splits that push 1 x 4 x splits x 34 over the limit
    rc = fn(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.shape[1], table.shape[1],
            slots.data_ptr(), lb.data_ptr(), out.data_ptr(), 0, 1, 4, 4, 32, too_many, 1.0, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.llg_last_error().decode()
    assert "1048576" in msg and "scratch" in msg
    assert float(out.abs().sum()) == 0             # nothing ran

"""Stand-ins for the CUDA kernels, for tests of the host logic where there is no GPU.

Each function has the signature and the contract of its namesake in the library's
``kernels.ops`` and is written with plain torch operations on CPU tensors.  Only tests pass
this module to the engine (as ``ops=``); the library itself never falls back to it.
"""
from __future__ import annotations

import torch

PAGE = 64


def sm_count():
    return 4


def require_gpu():
    pass


def embed_rows(table, token_ids, out_residual):
    out_residual.copy_(table[token_ids.long()].float())


def add_rmsnorm(residual, branch, weight, eps, out, rows=None):
    if branch is not None:
        if rows is None:
            residual += branch.sum(0)
        else:
            residual[rows.long()] += branch.sum(0)[rows.long()]
    x = residual if rows is None else residual[rows.long()]
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight.float()
    out.copy_(y.to(out.dtype))


def gemm_simt(x, w, out):
    out.copy_((x.float() @ w.float().t()).to(out.dtype))


def _rows_of(page_table, ring_pages, slot, pos, kvh, nkv):
    page = int(page_table[slot, (pos // PAGE) % ring_pages])
    return page, kvh, pos % PAGE


def qk_prep(qkv, *, n_heads, n_kv_heads, head_dim, q_norm_w, k_norm_w, norm_eps, bias, cos, sin, rotary_dim,
            pairing, positions, q_out, k_new=None, v_new=None, k_pages=None, v_pages=None, page_table=None,
            ring_pages=0, seq_of_token=None, slots=None):
    x = qkv.float().sum(0)
    n = x.shape[0]
    nh, nkv, hd = n_heads, n_kv_heads, head_dim
    x = x.view(n, nh + 2 * nkv, hd).clone()

    def norm(t, w):
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + norm_eps) * w.float()

    if q_norm_w is not None:
        x[:, :nh] = norm(x[:, :nh], q_norm_w)
    if k_norm_w is not None and nkv:
        x[:, nh:nh + nkv] = norm(x[:, nh:nh + nkv], k_norm_w)
    if bias is not None:
        x = x + bias.float().view(1, nh + 2 * nkv, hd)
    if cos is not None:
        half = rotary_dim // 2
        c = cos[positions.long()][:, None, :]
        s = sin[positions.long()][:, None, :]
        r = x[:, :nh + nkv]
        if pairing == 0:
            a, b = r[..., :half].clone(), r[..., half:2 * half].clone()
            r[..., :half] = a * c - b * s
            r[..., half:2 * half] = a * s + b * c
        else:
            a, b = r[..., 0:2 * half:2].clone(), r[..., 1:2 * half:2].clone()
            r[..., 0:2 * half:2] = a * c - b * s
            r[..., 1:2 * half:2] = a * s + b * c
    q_out.copy_(x[:, :nh].to(q_out.dtype))
    if nkv == 0:
        return
    k = x[:, nh:nh + nkv].to(q_out.dtype)
    v = x[:, nh + nkv:].to(q_out.dtype)
    if k_new is not None:
        k_new.copy_(k)
        v_new.copy_(v)
    if k_pages is not None:
        for t in range(n):
            slot = int(slots[int(seq_of_token[t])])
            pos = int(positions[t])
            for h in range(nkv):
                pg, hh, off = _rows_of(page_table, ring_pages, slot, pos, h, nkv)
                k_pages[pg, hh, off] = k[t, h]
                v_pages[pg, hh, off] = v[t, h]


def kv_write(k_new, v_new, k_pages, v_pages, page_table, ring_pages, positions, seq_of_token, slots,
             cu_tokens, len_before):
    n, nkv, hd = k_new.shape
    for t in range(n):
        b = int(seq_of_token[t])
        pos = int(positions[t])
        len_after = int(len_before[b]) + int(cu_tokens[b + 1] - cu_tokens[b])
        if pos < len_after - ring_pages * PAGE:
            continue
        slot = int(slots[b])
        for h in range(nkv):
            pg, hh, off = _rows_of(page_table, ring_pages, slot, pos, h, nkv)
            k_pages[pg, hh, off] = k_new[t, h]
            v_pages[pg, hh, off] = v_new[t, h]


def silu_mul(gate_up, out):
    x = gate_up.float().sum(0)
    inter = out.shape[1]
    half = x.shape[1] // 2
    g, u = x[:, :inter], x[:, half:half + inter]
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def scatter_i32(dst, idx, val):
    dst.view(-1)[idx.long()] = val


def gather_i32(dst, src, idx):
    dst.copy_(src.view(-1)[idx.long()])


def zero_rows(base, rows):
    base[rows.long()] = 0


def _attend(q, keys, vals, scale):
    s = (keys.float() @ q.float()) * scale
    p = torch.softmax(s, 0)
    return p @ vals.float()


def _gather(k_pages, v_pages, page_table, ring_pages, slot, positions, kvh):
    ks, vs = [], []
    for pos in positions:
        pg, hh, off = _rows_of(page_table, ring_pages, slot, pos, kvh, k_pages.shape[1])
        ks.append(k_pages[pg, hh, off])
        vs.append(v_pages[pg, hh, off])
    return ks, vs


def prefill_tile_queries(dtype, head_dim):
    return 16


def attn_prefill(q, k_new, v_new, k_pages, v_pages, page_table, ring_pages, tiles, cu_tokens, len_before,
                 slots, out, *, scale, window, tile_queries=16):
    n, nh, hd = q.shape
    nkv = k_new.shape[1]
    g = nh // nkv
    o = out.view(n, nh, hd)
    for b in range(slots.numel()):
        t0, t1 = int(cu_tokens[b]), int(cu_tokens[b + 1])
        lb = int(len_before[b])
        slot = int(slots[b])
        for t in range(t0, t1):
            pos = lb + (t - t0)
            lo = max(0, pos - window + 1) if window > 0 else 0
            for h in range(nh):
                kvh = h // g
                old = [p for p in range(lo, pos + 1) if p < lb]
                ks, vs = _gather(k_pages, v_pages, page_table, ring_pages, slot, old, kvh)
                for p in range(max(lo, lb), pos + 1):
                    ks.append(k_new[t0 + p - lb, kvh])
                    vs.append(v_new[t0 + p - lb, kvh])
                o[t, h] = _attend(q[t, h], torch.stack(ks), torch.stack(vs), scale).to(out.dtype)


class _Plan:
    scratch_floats, n_counters = 1, 0


def attn_decode_plan(dtype, n_seqs, n_heads, n_kv_heads, head_dim, max_len):
    return _Plan()


def attn_decode(q, k_pages, v_pages, page_table, ring_pages, slots, len_before, out, scratch, *,
                scale, window, plan=None, n_splits=0, counters=None, balance=False):
    b_n, nh, hd = q.shape
    nkv = k_pages.shape[1]
    g = nh // nkv
    o = out.view(b_n, nh, hd)
    for b in range(b_n):
        length = int(len_before[b]) + 1
        lo = max(0, length - window) if window > 0 else 0
        slot = int(slots[b])
        for h in range(nh):
            ks, vs = _gather(k_pages, v_pages, page_table, ring_pages, slot, range(lo, length), h // g)
            o[b, h] = _attend(q[b, h], torch.stack(ks), torch.stack(vs), scale).to(out.dtype)


def argmax(logits, out):
    out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))

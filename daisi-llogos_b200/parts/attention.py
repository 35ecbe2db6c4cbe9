"""Grouped-query attention with rotary positions over the paged cache.

Order of operations as in the reference (Inference/ForwardPass.cs:329-405): q, k, v
projections; optional per-head RMSNorm of q and k (:372-376); optional biases (:380-382);
rotation of q and k (:385); keys and values into the cache (:388); causal softmax attention
with ``scale = 1/sqrt(head_dim)`` applied to the dot product (:336, :399-400); output
projection (:404).  A window of W makes a query see only the last W keys, its own included
(Inference/AttentionStrategy.cs:64-71).  The reference leaves the biases out of its batched
prompt path (:783-794); here every path applies them.
"""
from __future__ import annotations

import math

import torch

from ..kernels.linear import linear
from .base import Branch, KvNeed, Mixer, TensorDecl, register_part


class Attention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, qk_norm, qk_norm_eps,
    window (0 = all keys), position (name of a position encoding or None), softmax_scale
    (None = 1/sqrt(head_dim)), own_kv (False: no k/v projections, reads another entry's cache)."""

    TAKES_ROW_SCALE = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads are not a multiple of {self.nkv} key/value heads")
        # said when the model is built, not at its first step
        limit = getattr(env.ops, "ATTN_MAX_HEAD_DIM", None)
        if limit is not None and not 0 < self.hd <= limit:
            raise ValueError(f"head_dim {self.hd}: the attention kernels take head sizes from 1 to {limit}")
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.window = int(p.get("window", 0) or 0)
        self.own_kv = bool(p.get("own_kv", True))
        scale = p.get("softmax_scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        enc = p.get("position")
        self.encoding = env.encodings[enc] if enc is not None else None
        self.w_qkv = self.w_o = self.b_qkv = self.q_norm_w = self.k_norm_w = None

    # ---- tensors -------------------------------------------------------------------------
    def tensors(self):
        q, kv = self.nh * self.hd, self.nkv * self.hd
        t = {"q_proj.weight": TensorDecl((q, self.hidden)), "o_proj.weight": TensorDecl((self.hidden, q))}
        if self.own_kv:
            t["k_proj.weight"] = TensorDecl((kv, self.hidden))
            t["v_proj.weight"] = TensorDecl((kv, self.hidden))
        if self.qkv_bias:
            t["q_proj.bias"] = TensorDecl((q,), "bias")
            if self.own_kv:
                t["k_proj.bias"] = TensorDecl((kv,), "bias")
                t["v_proj.bias"] = TensorDecl((kv,), "bias")
        if self.qk_norm:
            t["q_norm.weight"] = TensorDecl((self.hd,), "norm")
            if self.own_kv:
                t["k_norm.weight"] = TensorDecl((self.hd,), "norm")
        return t

    def bind(self, tensors):
        names = ["q_proj", "k_proj", "v_proj"] if self.own_kv else ["q_proj"]
        ws = [tensors[n + ".weight"] for n in names]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{self.prefix}: q/k/v projections are stored with different types")
        self.w_qkv = torch.cat(ws, dim=0).contiguous() if len(ws) > 1 else ws[0]
        self.w_o = tensors["o_proj.weight"]
        if self.qkv_bias:
            bs = [tensors[n + ".bias"] for n in names]
            self.b_qkv = torch.cat(bs, dim=0).contiguous() if len(bs) > 1 else bs[0]
        if self.qk_norm:
            self.q_norm_w = tensors["q_norm.weight"]
            self.k_norm_w = tensors["k_norm.weight"] if self.own_kv else None
            if self.b_qkv is not None and self.b_qkv.dtype != self.q_norm_w.dtype:
                self.b_qkv = self.b_qkv.to(self.q_norm_w.dtype)

    def cache_need(self):
        return KvNeed(self.nkv, self.hd, self.window) if self.own_kv else None

    def check_borrowed(self, need) -> None:
        if self.own_kv:
            raise ValueError("an attention part that reads another entry's cache must have own_kv = False")
        if not isinstance(need, KvNeed):
            raise ValueError("attention can only read a cache of keys and values")
        mine = (self.nkv, self.hd, self.window)
        if (need.num_kv_heads, need.head_dim, need.window) != mine:
            raise ValueError(f"the owner keeps (key/value heads, head size, window) = "
                             f"{(need.num_kv_heads, need.head_dim, need.window)}, this reader expects {mine}")

    # ---- one step ------------------------------------------------------------------------
    def forward(self, x, ctx, cache, row_scale=None) -> Branch:
        ops = ctx.ops
        n = x.shape[0]
        nkv_in = self.nkv if self.own_kv else 0
        rot = self.encoding.rotation() if self.encoding is not None else None
        # A large prompt step on the tensor cores prepares q and k in the projection's own epilogue.  Otherwise the
        # projection writes float32 (partials when the product splits K) and a second kernel prepares them; either
        # way the row scale, bias, norm and rotation see the unrounded sums, so q and k are rounded once.
        fused_qkv = getattr(ops, "gemm_tc_qkv_supported", None)
        scale_kw = {"row_scale": row_scale} if row_scale is not None else {}
        if (not ctx.decode and fused_qkv is not None
                and fused_qkv(x, self.w_qkv, self.hd, rot.rotary_dim if rot else 0, rot.pairing if rot else 0)):
            def prep(qkv_, **kw):
                ops.gemm_tc_qkv(x, self.w_qkv, **kw, **scale_kw)
            qkv = None
        else:
            def prep(qkv_, **kw):
                ops.qk_prep(qkv_, **kw, **scale_kw)
            qkv = linear(ctx, x, self.w_qkv, "attn.qkv", torch.float32)
        q = ctx.buffer("attn.q", (n, self.nh, self.hd))
        out = ctx.buffer("attn.out", (n, self.nh * self.hd))
        common = dict(n_heads=self.nh, n_kv_heads=nkv_in, head_dim=self.hd,
                      q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, norm_eps=self.qk_norm_eps,
                      bias=self.b_qkv, cos=rot.cos if rot else None, sin=rot.sin if rot else None,
                      rotary_dim=rot.rotary_dim if rot else 0, pairing=rot.pairing if rot else 0,
                      positions=ctx.positions, q_out=q)
        if ctx.decode:
            if self.own_kv:
                prep(qkv, **common, k_pages=cache.k_pages, v_pages=cache.v_pages,
                     page_table=cache.page_table, ring_pages=cache.ring_pages,
                     seq_of_token=ctx.seq_of_token, slots=ctx.slots)
            else:
                prep(qkv, **common)
            # which kernel runs and how it splits the keys is the kernels' business: the plan says what scratch it wants
            plan = ops.attn_decode_plan(q.dtype, ctx.n_seqs, self.nh, self.nkv, self.hd, ctx.max_len_after)
            scratch = ctx.buffer("attn.scratch", (max(1, plan.scratch_floats),), torch.float32)
            counters = None
            if plan.n_counters:
                counters = ctx.buffer("attn.counters", (plan.n_counters,), torch.int32, zero=True)
            ops.attn_decode(q, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages, ctx.slots,
                            ctx.len_before, out, scratch, scale=self.scale, window=self.window, plan=plan,
                            counters=counters)
        else:
            # A group that keeps every key can take the step's keys and values into its pages right away
            # (the step reads them from the packed buffer, never from the pages).  A ring must wait until
            # the attention has read the old keys that the new ones overwrite.
            write_now = self.own_kv and self.window == 0
            if self.own_kv:
                suffix = f".{cache.unit}" if cache.keep_step_kv else ""
                k_new = ctx.buffer("attn.k_new" + suffix, (n, self.nkv, self.hd))
                v_new = ctx.buffer("attn.v_new" + suffix, (n, self.nkv, self.hd))
                if write_now:
                    prep(qkv, **common, k_new=k_new, v_new=v_new, k_pages=cache.k_pages, v_pages=cache.v_pages,
                         page_table=cache.page_table, ring_pages=cache.ring_pages,
                         seq_of_token=ctx.seq_of_token, slots=ctx.slots)
                else:
                    prep(qkv, **common, k_new=k_new, v_new=v_new)
                cache.shared["k_new"], cache.shared["v_new"] = k_new, v_new
            else:
                prep(qkv, **common)
                k_new, v_new = cache.shared["k_new"], cache.shared["v_new"]
            tq = ops.prefill_tile_queries(q.dtype, self.hd)
            ops.attn_prefill(q, k_new, v_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                             ctx.query_tiles(tq), ctx.cu_tokens, ctx.len_before, ctx.slots, out,
                             scale=self.scale, window=self.window, tile_queries=tq)
            if self.own_kv and not write_now:
                def write_ring():
                    ops.kv_write(k_new, v_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                                 ctx.positions, ctx.seq_of_token, ctx.slots, ctx.cu_tokens, ctx.len_before)
                if cache.keep_step_kv:
                    # later entries of the run order read this ring in the same step: the new keys must not
                    # replace old ones before the last of them has run
                    cache.shared.setdefault("after_last_reader", []).append(write_ring)
                else:
                    write_ring()
        return Branch(linear(ctx, out, self.w_o, "attn.proj", torch.float32))


register_part("mixer", "attention", Attention)

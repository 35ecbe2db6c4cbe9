"""The stock blocks' launch chain in native code (csrc/block_runner.cu), driven from here.

When every entry of a model's run order is the stock arrangement of the stock parts (pre-norm block, RMSNorm,
attention that keeps its own keys and values, SwiGLU), a step's layers run through one call into the block runner
instead of nine Python calls per layer: Python fills one small structure per step (the packed-token layout, which
kernels the dispatch chose, scratch pointers) and hands over the layers' tensors, which were put into structures
once.  The runner launches the same kernels in the same order with the same arguments as the parts do, so both
ways give the same bits; a model with any other part, or with an entry that reads another entry's cache, runs
through the parts as before.  ``LLOGOS_RUNNER=0`` keeps every model on the parts.

The reference pays one managed-to-native call per kernel and hides it, for the token step only, behind a CUDA graph
(Daisi.Llogos.Cuda/CudaStream.cs:21-29, CudaBackend.cs:99-141).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_float, c_int, c_void_p
from typing import Dict, List, Optional

import torch

from ..csrc.build import load_library
from ..kernels import ops
from ..kernels.linear import plan_splits
from ..parts.attention import Attention
from ..parts.base import Branch
from ..parts.block import PreNormBlock
from ..parts.feedforward import SwiGLU
from ..parts.norm import RmsNorm

_API_FIELDS = ["add_rmsnorm", "gemm_tc", "gemm_simt", "qk_prep", "kv_write", "silu_mul", "attn_prefill_tc",
               "attn_prefill_mma", "attn_prefill_simt", "attn_decode_tma", "attn_decode_mma", "attn_decode_simt",
               "gemm_tc_qkv", "err_elementwise", "err_gemm_tc", "err_gemm_simt", "err_attn_tc", "err_attn_mma", "err_attn_simt",
               "err_attn_decode_tma"]


class _RunnerApi(Structure):
    _fields_ = [(n, c_void_p) for n in _API_FIELDS]


class _DenseLayer(Structure):
    _fields_ = [
        ("norm1_w", c_void_p), ("norm2_w", c_void_p), ("norm_w_dtype", c_int), ("norm1_eps", c_float), ("norm2_eps", c_float),
        ("w_qkv", c_void_p), ("b_qkv", c_void_p), ("bias_dtype", c_int),
        ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("qk_norm_w_dtype", c_int), ("qk_norm_eps", c_float),
        ("cos_table", c_void_p), ("sin_table", c_void_p), ("rotary_dim", c_int), ("pairing", c_int), ("table_positions", c_int),
        ("w_o", c_void_p), ("w_gate_up", c_void_p), ("w_down", c_void_p), ("window", c_int), ("scale", c_float),
        ("k_pages", c_void_p), ("v_pages", c_void_p), ("page_table", c_void_p),
        ("table_width", c_int), ("ring_pages", c_int), ("n_pages", c_int),
    ]


class _RunnerStep(Structure):
    _fields_ = [
        ("n_tokens", c_int), ("n_seqs", c_int), ("decode", c_int), ("dtype", c_int),
        ("hidden", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("inter", c_int),
        ("positions", c_void_p), ("seq_of_token", c_void_p), ("slots", c_void_p), ("cu_tokens", c_void_p),
        ("len_before", c_void_p), ("tiles", c_void_p), ("n_tiles", c_int), ("max_len_after", c_int),
        ("prefill_kind", c_int), ("decode_kind", c_int), ("decode_splits", c_int), ("decode_balance", c_int),
        ("tc_qkv", c_int), ("tc_o", c_int), ("tc_gate_up", c_int), ("tc_down", c_int),
        ("splits_qkv", c_int), ("splits_o", c_int), ("splits_down", c_int), ("fused_qkv", c_int),
        ("ss", c_void_p), ("ss_parts", c_int),
        ("residual", c_void_p), ("norm_out", c_void_p), ("qkv", c_void_p), ("q", c_void_p), ("k_new", c_void_p),
        ("v_new", c_void_p), ("attn_out", c_void_p), ("proj", c_void_p), ("act", c_void_p), ("ffn_out", c_void_p),
        ("gate_up", c_void_p), ("gate_up_rows", c_int), ("attn_scratch", c_void_p), ("attn_counters", c_void_p),
        ("stream", c_void_p),
    ]


_GATED_CHUNK = 16384          # rows per pass of the two-kernel gating path (as in kernels/linear.py)

# entry of the function table -> (library, function); the error text of a library goes with its first entry
_ENTRIES = {
    "add_rmsnorm": ("elementwise", "llg_add_rmsnorm"), "qk_prep": ("elementwise", "llg_qk_prep"),
    "kv_write": ("elementwise", "llg_kv_write"), "silu_mul": ("elementwise", "llg_silu_mul"),
    "gemm_tc": ("gemm_tc", "llg_gemm_tc"), "gemm_simt": ("gemm_simt", "llg_gemm_simt"),
    "gemm_tc_qkv": ("gemm_tc", "llg_gemm_tc_qkv"),
    "attn_prefill_tc": ("attention_tc", "llg_attn_prefill_tc"), "attn_prefill_mma": ("attention_mma", "llg_attn_prefill_mma"),
    "attn_prefill_simt": ("attention_simt", "llg_attn_prefill_simt"),
    "attn_decode_tma": ("attention_decode_tma", "llg_attn_decode_tma"), "attn_decode_mma": ("attention_mma", "llg_attn_decode_mma"),
    "attn_decode_simt": ("attention_simt", "llg_attn_decode_simt"),
}
_ERR_FIELD = {"elementwise": "err_elementwise", "gemm_tc": "err_gemm_tc", "gemm_simt": "err_gemm_simt",
              "attention_tc": "err_attn_tc", "attention_mma": "err_attn_mma", "attention_simt": "err_attn_simt",
              "attention_decode_tma": "err_attn_decode_tma"}
_lib = None
_api = _RunnerApi()
_bound = set()


def _library():
    """The runner's own library (once per process)."""
    global _lib
    if _lib is not None:
        return _lib
    lib = load_library("block_runner")
    api_size, layer_size, step_size = c_int(), c_int(), c_int()
    lib.llg_runner_struct_sizes(byref(api_size), byref(layer_size), byref(step_size))
    got = (api_size.value, layer_size.value, step_size.value)
    want = (ctypes.sizeof(_RunnerApi), ctypes.sizeof(_DenseLayer), ctypes.sizeof(_RunnerStep))
    if got != want:
        raise ops.KernelError(f"block runner: structure sizes {got} in the library, {want} here")
    lib.llg_runner_bind.argtypes = [POINTER(_RunnerApi)]
    lib.llg_runner_run.argtypes = [c_void_p, c_int, POINTER(_RunnerStep), c_void_p, c_int, POINTER(c_int), POINTER(c_int)]
    _lib = lib
    return lib


def _ensure(entries) -> None:
    """Binds the kernels' entry points that a step needs into the runner, loading (and, in a fresh checkout,
    compiling) only the libraries they live in."""
    missing = [e for e in entries if e not in _bound]
    if not missing:
        return
    lib = _library()
    for e in missing:
        lib_name, fn = _ENTRIES[e]
        kernels = ops._lib(lib_name)
        setattr(_api, e, ctypes.cast(getattr(kernels, fn), c_void_p).value)
        setattr(_api, _ERR_FIELD[lib_name], ctypes.cast(kernels.llg_last_error, c_void_p).value)
        _bound.add(e)
    if lib.llg_runner_bind(byref(_api)) != 0:
        raise ops.KernelError(lib.llg_last_error().decode("utf-8", "replace"))


def _code(dtype: torch.dtype) -> int:
    return ops.F32 if dtype == torch.float32 else ops.BF16


class BlockRunner:
    """The layers of one model over one cache, ready to run through the native chain."""

    def __init__(self, model, cache, layers: List[_DenseLayer], keep: list, geom: Dict[str, int]):
        self.model, self.cache = model, cache
        self.lib = _library()
        self.n_layers = len(layers)
        self.layers = layers                                  # the structures (kept alive here)
        self.table = (c_void_p * len(layers))(*[ctypes.addressof(x) for x in layers])
        self.keep = keep                                      # tensors whose addresses the structures hold
        self.g = geom
        self.step = _RunnerStep()
        self._out_parts, self._launches = c_int(), c_int()
        self._ensured = set()

    # ---- eligibility -----------------------------------------------------------------------
    @classmethod
    def build(cls, model, cache) -> Optional["BlockRunner"]:
        """A runner for ``model`` over ``cache``, or ``None`` when some entry of the run order is not the stock
        block of stock parts (then the parts run as they are)."""
        if os.environ.get("LLOGOS_RUNNER", "1") == "0" or model.device.type != "cuda" or model.env.ops is not ops:
            return None
        spec = model.spec
        if not spec.schedule or any(e.cache_of is not None for e in spec.schedule):
            return None
        layers, keep, geom, fusable = [], [], None, 1
        for e_i, e in enumerate(spec.schedule):
            block = model.blocks[e.layer]
            if type(block) is not PreNormBlock or set(block.parts) != {"norm1", "mixer", "norm2", "ffn"}:
                return None
            n1, mx, n2, ff = (block.parts[r] for r in ("norm1", "mixer", "norm2", "ffn"))
            if type(n1) is not RmsNorm or type(n2) is not RmsNorm or type(mx) is not Attention or type(ff) is not SwiGLU:
                return None
            if not mx.own_kv or n1.size != mx.hidden or n2.size != mx.hidden or ff.hidden != mx.hidden:
                return None
            g = dict(hidden=mx.hidden, nh=mx.nh, nkv=mx.nkv, hd=mx.hd, inter=ff.inter)
            if geom is None:
                geom = g
            elif g != geom:
                return None                                   # layers of different sizes: the parts handle them
            mats = [mx.w_qkv, mx.w_o, ff.w_gate_up, ff.w_down]
            if any(t is None or t.dtype != model.dtype or not t.is_contiguous() or t.data_ptr() % 16 for t in mats):
                return None
            if n1.weight.dtype != n2.weight.dtype:
                return None
            view = cache.view(e_i)
            if view is None or not hasattr(view, "k_pages"):
                return None
            rot = mx.encoding.rotation() if mx.encoding is not None else None
            L = _DenseLayer()
            L.norm1_w, L.norm2_w = n1.weight.data_ptr(), n2.weight.data_ptr()
            L.norm_w_dtype, L.norm1_eps, L.norm2_eps = _code(n1.weight.dtype), n1.eps, n2.eps
            L.w_qkv = mx.w_qkv.data_ptr()
            if mx.b_qkv is not None:
                L.b_qkv, L.bias_dtype = mx.b_qkv.data_ptr(), _code(mx.b_qkv.dtype)
            if mx.q_norm_w is not None:
                if mx.k_norm_w is None or mx.k_norm_w.dtype != mx.q_norm_w.dtype:
                    return None
                if mx.b_qkv is not None and mx.b_qkv.dtype != mx.q_norm_w.dtype:
                    return None
                L.q_norm_w, L.k_norm_w = mx.q_norm_w.data_ptr(), mx.k_norm_w.data_ptr()
                L.qk_norm_w_dtype = _code(mx.q_norm_w.dtype)
            L.qk_norm_eps = mx.qk_norm_eps
            if rot is not None:
                L.cos_table, L.sin_table = rot.cos.data_ptr(), rot.sin.data_ptr()
                L.rotary_dim, L.pairing, L.table_positions = rot.rotary_dim, rot.pairing, rot.cos.shape[0]
                keep += [rot.cos, rot.sin]
            L.w_o, L.w_gate_up, L.w_down = mx.w_o.data_ptr(), ff.w_gate_up.data_ptr(), ff.w_down.data_ptr()
            L.window, L.scale = mx.window, mx.scale
            if rot is not None and not (rot.pairing == 0 and rot.rotary_dim == mx.hd):
                fusable = 0                                 # the q/k/v product's own epilogue rotates whole heads by halves only
            L.k_pages, L.v_pages, L.page_table = view.k_pages.data_ptr(), view.v_pages.data_ptr(), view.page_table.data_ptr()
            L.table_width, L.ring_pages, L.n_pages = view.page_table.shape[1], view.ring_pages, view.k_pages.shape[0]
            keep += [view.k_pages, view.v_pages, view.page_table]
            layers.append(L)
        return cls(model, cache, layers, keep, dict(geom, fusable_rotation=fusable))

    # ---- one step ----------------------------------------------------------------------------
    def run(self, ctx, residual: torch.Tensor) -> Branch:
        """Runs every layer on the step's tokens; returns the last block's output, still to be added."""
        g, s, dtype = self.g, self.step, self.model.dtype
        n, hidden, nh, nkv, hd, inter = ctx.n_tokens, g["hidden"], g["nh"], g["nkv"], g["hd"], g["inter"]
        qkv_dim, q_dim = (nh + 2 * nkv) * hd, nh * hd
        bf16 = dtype == torch.bfloat16
        sms = ops.sm_count()

        def tc(k):                                            # the tensor-core product's rule (kernels/ops.py)
            return int(bf16 and k % 8 == 0)

        def splits(o, k):
            return ops.gemm_tc_splits(k, plan_splits(n, o, k, sms)) if tc(k) else 1

        s.n_tokens, s.n_seqs, s.decode, s.dtype = n, ctx.n_seqs, int(ctx.decode), _code(dtype)
        s.hidden, s.nh, s.nkv, s.hd, s.inter = hidden, nh, nkv, hd, inter
        s.positions, s.seq_of_token, s.slots = ctx.positions.data_ptr(), ctx.seq_of_token.data_ptr(), ctx.slots.data_ptr()
        s.cu_tokens, s.len_before = ctx.cu_tokens.data_ptr(), ctx.len_before.data_ptr()
        s.max_len_after = ctx.max_len_after
        s.tc_qkv, s.tc_o, s.tc_gate_up, s.tc_down = tc(hidden), tc(q_dim), tc(hidden), tc(inter)
        # the rule of kernels/ops.py gemm_tc_qkv_supported, on sizes
        s.fused_qkv = int(ops.USE_FUSED_QKV and not ctx.decode and bool(s.tc_qkv) and n > ops.FUSED_QKV_ABOVE and hd in (64, 128)
                          and g.get("fusable_rotation", 1) == 1)
        s.splits_qkv, s.splits_o, s.splits_down = splits(qkv_dim, hidden), splits(hidden, q_dim), splits(hidden, inter)
        # a bfloat16 step's norms leave their division to the products that consume them (parts/norm.py)
        s.ss_parts = ops.norm_ss_parts(n, hidden) if bf16 else 0
        s.ss = ctx.buffer("norm.ss", (n, s.ss_parts), torch.float32).data_ptr() if bf16 else None
        s.residual = residual.data_ptr()
        s.norm_out = ctx.buffer("norm.out", (n, hidden)).data_ptr()
        s.qkv = ctx.buffer("attn.qkv", (s.splits_qkv, n, qkv_dim), torch.float32).data_ptr()
        s.q = ctx.buffer("attn.q", (n, nh, hd)).data_ptr()
        s.attn_out = ctx.buffer("attn.out", (n, q_dim)).data_ptr()
        s.proj = ctx.buffer("attn.proj", (s.splits_o, n, hidden), torch.float32).data_ptr()
        s.act = ctx.buffer("ffn.act", (n, inter)).data_ptr()
        ffn_out = ctx.buffer("ffn.out", (s.splits_down, n, hidden), torch.float32)
        s.ffn_out = ffn_out.data_ptr()
        if not (s.tc_gate_up and bf16):
            rows = min(n, _GATED_CHUNK)
            s.gate_up = ctx.buffer("ffn.gate_up", (1, rows, ops.gated_rows(inter))).data_ptr()
            s.gate_up_rows = rows
        if ctx.decode:
            plan = ops.attn_decode_plan(dtype, ctx.n_seqs, nh, nkv, hd, ctx.max_len_after)
            s.decode_kind = {"simt": 0, "mma": 1, "tma": 2}[plan.kind]
            s.decode_splits, s.decode_balance = plan.n_splits, int(plan.balance)
            s.attn_scratch = ctx.buffer("attn.scratch", (max(1, plan.scratch_floats),), torch.float32).data_ptr()
            s.attn_counters = (ctx.buffer("attn.counters", (plan.n_counters,), torch.int32, zero=True).data_ptr()
                               if plan.n_counters else None)
            s.tiles, s.n_tiles, s.k_new, s.v_new = None, 0, None, None
        else:
            s.k_new = ctx.buffer("attn.k_new", (n, nkv, hd)).data_ptr()
            s.v_new = ctx.buffer("attn.v_new", (n, nkv, hd)).data_ptr()
            tq = ops.prefill_tile_queries(dtype, hd)
            tiles = ctx.query_tiles(tq)
            s.tiles, s.n_tiles = tiles.data_ptr(), tiles.shape[0]
            s.prefill_kind = 2 if ops._use_tc_attn(dtype, hd) else 1 if ops._use_mma(dtype, hd) else 0
        need = ["add_rmsnorm"] + (["gemm_tc_qkv"] if s.fused_qkv else ["qk_prep"])
        need.append("gemm_tc" if (s.tc_qkv or s.tc_o or s.tc_down or (s.tc_gate_up and bf16)) else "gemm_simt")
        if not (s.tc_qkv and s.tc_o and s.tc_down):
            need.append("gemm_simt")
        if not (s.tc_gate_up and bf16):
            need += ["gemm_simt", "silu_mul"]
        if ctx.decode:
            need.append(("attn_decode_simt", "attn_decode_mma", "attn_decode_tma")[s.decode_kind])
        else:
            need.append(("attn_prefill_simt", "attn_prefill_mma", "attn_prefill_tc")[s.prefill_kind])
            need.append("kv_write")
        key = tuple(need)
        if key not in self._ensured:
            _ensure(need)
            self._ensured.add(key)
        s.stream = ops._stream()
        rc = self.lib.llg_runner_run(self.table, self.n_layers, byref(s), None, 0, byref(self._out_parts), byref(self._launches))
        ops._launches += self._launches.value
        if rc != 0:
            raise ops.KernelError(self.lib.llg_last_error().decode("utf-8", "replace"))
        return Branch(ffn_out)

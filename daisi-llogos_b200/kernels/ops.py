"""Python face of the CUDA kernels: every function takes torch CUDA tensors, checks them,
and launches on the current stream.  Nothing here computes on the CPU, and nothing falls
back: a tensor that is not on the GPU, or a library that cannot be built, is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from ..csrc.build import load_library

F32, BF16 = 0, 1
PAGE = 64  # tokens per cache page; checked against the library at first use


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _ptr(t: Optional[torch.Tensor], dtype=None) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a kernel was given a tensor that is not on the GPU; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"a kernel was given a non-contiguous tensor of shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"expected {dtype}, got {t.dtype}")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """Handle of the current stream of the current device (the raw query: this runs once per launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launches() -> int:
    """Kernels launched (or recorded into a CUDA graph) by this module so far."""
    return _launches


def _check(lib, rc: int, kernels: int = 1) -> None:
    global _launches
    if rc != 0:
        raise KernelError(lib.llg_last_error().decode("utf-8", "replace"))
    _launches += kernels


# ---- libraries and prototypes ---------------------------------------------------------

class _RowScale(Structure):
    _fields_ = [("ss", c_void_p), ("parts", c_int), ("inv_width", c_float), ("eps", c_float)]


class RowScale:
    """What a norm leaves to the consumer of its output when it does not divide by the root mean square itself: the
    output holds ``x * weight`` and ``ss`` (float32 ``[rows, parts]``) the sums of squares of each row of ``x``, whole
    or as partial sums; the consumer multiplies row r of its product by ``1 / sqrt(sum(ss[r]) / width + eps)``."""

    def __init__(self, ss: torch.Tensor, width: int, eps: float):
        if ss.dim() != 2 or ss.dtype != torch.float32:
            raise KernelError("a row scale's sums are float32 [rows, parts]")
        self.ss, self.width, self.eps = ss, int(width), float(eps)

    @property
    def rows(self) -> int:
        return self.ss.shape[0]

    def slice(self, r0: int, r1: int) -> "RowScale":
        return RowScale(self.ss[r0:r1], self.width, self.eps)

    def c(self) -> "_RowScale":
        return _RowScale(_ptr(self.ss, torch.float32), self.ss.shape[1], 1.0 / self.width, self.eps)


def _scale_ref(row_scale: Optional[RowScale], rows: int):
    """ctypes argument for an optional ``const RowScale*``."""
    if row_scale is None:
        return None
    if row_scale.rows != rows:
        raise KernelError(f"a row scale for {row_scale.rows} rows was given to a product of {rows} rows")
    return byref(row_scale.c())


class _QkPrepArgs(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("qkv_dtype", c_int), ("n_partials", c_int), ("partial_stride", c_longlong),
        ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("norm_w_dtype", c_int), ("norm_eps", c_float),
        ("bias", c_void_p), ("bias_dtype", c_int),
        ("cos_table", c_void_p), ("sin_table", c_void_p), ("rotary_dim", c_int), ("pairing", c_int),
        ("table_positions", c_int), ("positions", c_void_p),
        ("q_out", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p),
        ("k_pages", c_void_p), ("v_pages", c_void_p), ("page_table", c_void_p),
        ("table_width", c_int), ("ring_pages", c_int),
        ("seq_of_token", c_void_p), ("slots", c_void_p),
        ("n_tokens", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int),
        ("row_scale", _RowScale),
    ]


class _PrefillArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p), ("k_pages", c_void_p), ("v_pages", c_void_p),
        ("page_table", c_void_p), ("table_width", c_int), ("ring_pages", c_int),
        ("tiles", c_void_p), ("cu_tokens", c_void_p), ("len_before", c_void_p), ("slots", c_void_p),
        ("out", c_void_p),
        ("n_tiles", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int),
        ("scale", c_float), ("window", c_int), ("n_tokens", c_int), ("n_pages", c_int),
    ]


class _DecodeArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k_pages", c_void_p), ("v_pages", c_void_p), ("page_table", c_void_p),
        ("table_width", c_int), ("ring_pages", c_int), ("slots", c_void_p), ("len_before", c_void_p),
        ("part_o", c_void_p), ("part_ml", c_void_p),
        ("n_seqs", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("n_splits", c_int),
        ("scale", c_float), ("window", c_int),
    ]


class _DecodeTmaArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("page_table", c_void_p), ("table_width", c_int), ("ring_pages", c_int),
        ("slots", c_void_p), ("len_before", c_void_p), ("part", c_void_p), ("counters", c_void_p), ("out", c_void_p),
        ("n_seqs", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("scale", c_float), ("window", c_int),
    ]


class _SampleArgs(Structure):
    _fields_ = [
        ("logits", c_void_p), ("work", c_void_p), ("out", c_void_p), ("probs_out", c_void_p),
        ("seq_ids", c_void_p), ("history", c_void_p), ("history_len", c_void_p), ("history_stride", c_int),
        ("n_seqs", c_int), ("vocab", c_int),
        ("temperature", c_float), ("top_k", c_int),
        ("top_p", c_float), ("min_p", c_float), ("typical_p", c_float), ("min_keep", c_int),
        ("repetition_penalty", c_float), ("frequency_penalty", c_float), ("presence_penalty", c_float),
        ("penalize_newline", c_int), ("seed", c_ulonglong), ("step", c_int),
        ("banned", c_void_p), ("n_banned", c_int),
        ("cand_val", c_void_p), ("cand_idx", c_void_p), ("cand_count", c_void_p), ("n_slices", c_int),
        ("history_rows", c_void_p), ("history_append", c_int),
        ("slice_stats", c_void_p),
    ]


_protos_done = set()


_libs = {}


def _lib(name: str):
    lib = _libs.get(name)
    if lib is not None:
        return lib
    lib = _load_lib(name)
    _libs[name] = lib
    return lib


def _load_lib(name: str):
    lib = load_library(name)
    if name in _protos_done:
        return lib
    if name == "elementwise":
        lib.llg_page_size.restype = c_int
        if lib.llg_page_size() != PAGE:
            raise KernelError(f"the kernels use pages of {lib.llg_page_size()} tokens, Python expects {PAGE}")
        lib.llg_embed_rows.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.llg_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_float,
                                        c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.llg_qk_prep.argtypes = [POINTER(_QkPrepArgs), c_int, c_void_p]
        lib.llg_kv_write.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.llg_silu_mul.argtypes = [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.llg_scatter_i32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        lib.llg_gather_i32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        lib.llg_zero_rows.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p]
    elif name == "gemm_simt":
        lib.llg_gemm_simt.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                      POINTER(_RowScale), c_void_p]
    elif name == "gemm_tc":
        lib.llg_gemm_tc_supported.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int]
        lib.llg_gemm_tc_splits.argtypes = [c_int, c_int]
        lib.llg_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                    POINTER(_RowScale), c_void_p]
        lib.llg_gemm_tc_qkv.argtypes = [c_void_p, c_void_p, c_int, c_int, POINTER(_QkPrepArgs), c_void_p]
    elif name == "attention_simt":
        lib.llg_attn_prefill_simt.argtypes = [POINTER(_PrefillArgs), c_int, c_void_p]
        lib.llg_attn_decode_simt.argtypes = [POINTER(_DecodeArgs), c_void_p, c_int, c_void_p]
        lib.llg_attn_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
        lib.llg_attn_decode_scratch_floats.restype = c_longlong
    elif name == "attention_mma":
        lib.llg_attn_mma_supported.argtypes = [c_int]
        lib.llg_attn_prefill_mma.argtypes = [POINTER(_PrefillArgs), c_void_p]
        lib.llg_attn_decode_mma.argtypes = [POINTER(_DecodeArgs), c_void_p, c_void_p, c_int, c_void_p]
    elif name == "attention_tc":
        lib.llg_attn_tc_supported.argtypes = [c_int]
        lib.llg_attn_prefill_tc.argtypes = [POINTER(_PrefillArgs), c_void_p]
        lib.llg_attn_tc_status.restype = c_int
    elif name == "attention_decode_tma":
        lib.llg_attn_decode_tma_supported.argtypes = [c_int, c_int, c_int, c_int]
        lib.llg_attn_decode_tma_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
        lib.llg_attn_decode_tma_scratch_floats.restype = c_longlong
        lib.llg_attn_decode_tma.argtypes = [POINTER(_DecodeTmaArgs), c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.llg_attn_decode_tma_status.restype = c_int
    elif name == "init":
        lib.llg_fill_normal.argtypes = [c_void_p, c_int, c_longlong, c_ulonglong, ctypes.c_double, ctypes.c_double, c_void_p]
        lib.llg_fill.argtypes = [c_void_p, c_int, c_longlong, c_float, c_void_p]
        lib.llg_cast.argtypes = [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p]
    elif name == "sampling":
        lib.llg_argmax.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.llg_sample.argtypes = [POINTER(_SampleArgs), c_void_p]
        lib.llg_sample_slices.argtypes = [c_int]
    _protos_done.add(name)
    return lib


_sm_counts = {}


def sm_count() -> int:
    """Multiprocessors of the current CUDA device (asked once per device)."""
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return n


def require_gpu() -> None:
    """Fails loudly when there is no GPU or the kernels cannot be loaded."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this library runs on the GPU only and has no CPU path")
    _lib("elementwise")


# ---- kernels ------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, token_ids: torch.Tensor, out_residual: torch.Tensor) -> None:
    """out_residual[n] = table[token_ids[n]] as float32."""
    lib = _lib("elementwise")
    vocab, hidden = table.shape
    n = token_ids.numel()
    assert out_residual.shape == (n, hidden)
    _check(lib, lib.llg_embed_rows(_ptr(table), _dt(table), _ptr(token_ids, torch.int32),
                                   _ptr(out_residual, torch.float32), n, hidden, vocab, _stream()))


def add_rmsnorm(residual: torch.Tensor, branch: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, ss_out: Optional[torch.Tensor] = None) -> None:
    """residual += sum of branch partials (if any); out[j] = RMSNorm(residual[rows[j] or j]) * weight.

    ``residual`` is float32 ``[N, H]``; ``branch`` float32 ``[S, N, H]`` or None; ``out`` ``[M, H]``.
    With ``ss_out`` (float32 ``[M, norm_ss_parts(M, H)]``) the division is left to whoever consumes ``out``: ``out[j]``
    is the row times ``weight`` and ``ss_out[j]`` holds the row's sum of squares, whole or as the sums of equal slices
    of the row in their order (see ``RowScale``).
    """
    lib = _lib("elementwise")
    n, hidden = residual.shape
    m = out.shape[0]
    assert out.shape[1] == hidden and weight.shape == (hidden,)
    if rows is not None:
        assert rows.numel() == m
    else:
        assert m == n
    if ss_out is not None:
        assert tuple(ss_out.shape) == (m, norm_ss_parts(m, hidden)), (ss_out.shape, m, hidden)
    n_part, stride = 0, 0
    if branch is not None:
        assert branch.dim() == 3 and branch.shape[1:] == (n, hidden), (branch.shape, residual.shape)
        n_part, stride = branch.shape[0], n * hidden
    _check(lib, lib.llg_add_rmsnorm(_ptr(residual, torch.float32), _ptr(branch, torch.float32), n_part, stride,
                                    _ptr(weight), _dt(weight), float(eps), _ptr(out), _dt(out),
                                    _ptr(rows, torch.int32), m, hidden, _ptr(ss_out, torch.float32), _stream()))


_ss_parts = {}


def norm_ss_parts(n_out: int, hidden: int) -> int:
    """Sums of squares per row that ``add_rmsnorm(..., ss_out=)`` writes for these sizes: one, or for the few rows
    of a decode step one per slice of the row (each slice is a block of its own there)."""
    key = (n_out <= 64, hidden)
    p = _ss_parts.get(key)
    if p is None:
        lib = _lib("elementwise")
        lib.llg_add_rmsnorm_parts.argtypes = [c_int, c_int]
        p = _ss_parts[key] = lib.llg_add_rmsnorm_parts(1 if n_out <= 64 else 65, hidden)
    return p


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_scale: Optional[RowScale] = None) -> None:
    """out[n, o] = sum_k x[n, k] w[o, k] on the CUDA cores, float32 accumulation; rows times ``row_scale`` if given."""
    lib = _lib("gemm_simt")
    n, k = x.shape
    o, k2 = w.shape
    assert k == k2 and out.shape == (n, o), (x.shape, w.shape, out.shape)
    _check(lib, lib.llg_gemm_simt(_ptr(x), _dt(x), _ptr(w), _dt(w), _ptr(out), _dt(out), n, o, k,
                                  _scale_ref(row_scale, n), _stream()))


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes this product (bfloat16 operands, k a multiple of 8)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not (x.is_cuda and w.is_cuda):
        return False
    # the library's rule (llg_gemm_tc_supported), kept here because this runs before every product
    return x.shape[0] > 0 and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


_splits_cache = {}


def gemm_tc_splits(k: int, wish: int) -> int:
    """The number of split-K partials the kernel writes when asked for ``wish``."""
    key = (k, wish)
    s = _splits_cache.get(key)
    if s is None:
        s = _splits_cache[key] = _lib("gemm_tc").llg_gemm_tc_splits(k, wish)
    return s


def gated_rows(features: int) -> int:
    """Rows of a gate/up matrix in the gated layout: the gate rows, filled up to a multiple of 128, then
    the up rows in the same way."""
    return -(-features // 128) * 256


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, tile_n: int = 0, gated_features: int = 0,
            row_scale: Optional[RowScale] = None) -> None:
    """out[s, n, o] = split-K partials of x[n, k] w[o, k] on the tensor cores (tcgen05, TMA).

    ``out`` is ``[S, N, O]`` float32 with S = ``gemm_tc_splits(k, wish)``, or ``[1, N, O]`` bfloat16.
    With ``gated_features = F`` the matrix ``w`` is in the gated layout (``gated_rows(F)`` rows) and
    ``out`` is ``[1, N, F]`` holding ``silu(gate) * up``.  ``row_scale``: what a norm left for the rows of ``x``;
    the rows of the product are multiplied by it (before the gating).
    """
    lib = _lib("gemm_tc")
    n, k = x.shape
    o, k2 = w.shape
    s = out.shape[0]
    assert k == k2 and out.shape == (s, n, gated_features if gated_features else o), (x.shape, w.shape, out.shape)
    if gemm_tc_splits(k, s) != s:
        raise KernelError(f"gemm_tc: {s} splits cannot be had for k = {k}")
    _check(lib, lib.llg_gemm_tc(_ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), _ptr(out), _dt(out), n, o, k, s,
                                tile_n, gated_features, _scale_ref(row_scale, n), _stream()))


def gemm_tc_status() -> int:
    """Error code a tensor-core product recorded when a wait ran out (0 = none); synchronises."""
    lib = _lib("gemm_tc")
    lib.llg_gemm_tc_status.restype = c_int
    return lib.llg_gemm_tc_status()


def qk_prep(qkv: torch.Tensor, *, n_heads: int, n_kv_heads: int, head_dim: int,
            q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], norm_eps: float,
            bias: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
            rotary_dim: int, pairing: int, positions: torch.Tensor, q_out: torch.Tensor,
            k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None,
            k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
            page_table: Optional[torch.Tensor] = None, ring_pages: int = 0,
            seq_of_token: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
            row_scale: Optional[RowScale] = None) -> None:
    """Per-head norm (optional), bias (optional), rotation, and the writes of q, k, v.

    ``qkv`` is ``[S, N, (nh + 2 nkv) * hd]`` (partials are summed).  Queries go to ``q_out``;
    keys and values go to ``k_new``/``v_new`` (packed, for a prompt step) and/or straight into
    the cache pages (for a one-token step).  ``row_scale``: what a norm left for the token rows; the summed
    partials are multiplied by it before anything else.
    """
    lib = _lib("elementwise")
    s, n, width = qkv.shape
    assert width == (n_heads + 2 * n_kv_heads) * head_dim
    a = _prep_args(n, n_heads, n_kv_heads, head_dim, q_norm_w, k_norm_w, norm_eps, bias, cos, sin, rotary_dim, pairing,
                   positions, q_out, k_new, v_new, k_pages, v_pages, page_table, ring_pages, seq_of_token, slots)
    a.qkv, a.qkv_dtype, a.n_partials, a.partial_stride = _ptr(qkv), _dt(qkv), s, n * width
    _set_scale(a, row_scale, n)
    _check(lib, lib.llg_qk_prep(byref(a), _dt(q_out), _stream()))


def _set_scale(a: "_QkPrepArgs", row_scale: Optional[RowScale], n: int) -> None:
    if row_scale is not None:
        if row_scale.rows != n:
            raise KernelError(f"a row scale for {row_scale.rows} rows was given to {n} token rows")
        a.row_scale = row_scale.c()


def _prep_args(n, n_heads, n_kv_heads, head_dim, q_norm_w, k_norm_w, norm_eps, bias, cos, sin, rotary_dim, pairing,
               positions, q_out, k_new, v_new, k_pages, v_pages, page_table, ring_pages, seq_of_token, slots) -> "_QkPrepArgs":
    """The argument block of the q/k/v preparation, without the q/k/v input itself."""
    a = _QkPrepArgs()
    a.q_norm_w, a.k_norm_w = _ptr(q_norm_w), _ptr(k_norm_w)
    a.norm_w_dtype = _dt(q_norm_w) if q_norm_w is not None else F32
    a.norm_eps = float(norm_eps)
    a.bias = _ptr(bias)
    a.bias_dtype = _dt(bias) if bias is not None else F32
    if cos is not None:
        assert cos.shape == sin.shape and cos.shape[1] * 2 == rotary_dim
        a.cos_table, a.sin_table = _ptr(cos, torch.float32), _ptr(sin, torch.float32)
        a.table_positions = cos.shape[0]
    a.rotary_dim, a.pairing = rotary_dim, pairing
    a.positions = _ptr(positions, torch.int32)
    a.q_out, a.k_new, a.v_new = _ptr(q_out), _ptr(k_new), _ptr(v_new)
    a.k_pages, a.v_pages = _ptr(k_pages), _ptr(v_pages)
    if page_table is not None:
        a.page_table, a.table_width = _ptr(page_table, torch.int32), page_table.shape[1]
    a.ring_pages = ring_pages
    a.seq_of_token, a.slots = _ptr(seq_of_token, torch.int32), _ptr(slots, torch.int32)
    a.n_tokens, a.nh, a.nkv, a.hd = n, n_heads, n_kv_heads, head_dim
    for t in (k_new, v_new, k_pages, v_pages):
        if t is not None and t.dtype != q_out.dtype:
            raise KernelError("qk_prep: all outputs must share one dtype")
    return a


# Rows above which a prompt step's q/k/v product prepares queries and keys in its own epilogue.  With fewer rows (three
# token tiles of 128 or fewer) the product that splits its sums over more blocks, followed by the preparation kernel, is
# faster: measured on a B200 at the 8B layer sizes, 384 rows 7.26 ms per step against 7.63 fused, 448 rows 8.49 against 8.27.
FUSED_QKV_ABOVE = 384
USE_FUSED_QKV = True        # tests switch it off to compare with the product followed by the preparation kernel


def gemm_tc_qkv_supported(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int, pairing: int) -> bool:
    """Whether ``gemm_tc_qkv`` takes this q/k/v projection: tensor-core operands, more than ``FUSED_QKV_ABOVE`` rows (with fewer the
    product splits its sums over blocks, which leaves partial sums and no place for an epilogue), head size 64 or
    128, rotation over the whole head by halves or none (``rotary_dim`` 0)."""
    return (USE_FUSED_QKV and gemm_tc_supported(x, w) and x.shape[0] > FUSED_QKV_ABOVE and head_dim in (64, 128)
            and (rotary_dim == 0 or (pairing == 0 and rotary_dim == head_dim)))


def gemm_tc_qkv(x: torch.Tensor, w: torch.Tensor, *, n_heads: int, n_kv_heads: int, head_dim: int,
                q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], norm_eps: float,
                bias: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                rotary_dim: int, pairing: int, positions: torch.Tensor, q_out: torch.Tensor,
                k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None,
                k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                page_table: Optional[torch.Tensor] = None, ring_pages: int = 0,
                seq_of_token: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                row_scale: Optional[RowScale] = None) -> None:
    """The q/k/v projection ``x w^T`` on the tensor cores with ``qk_prep`` as its epilogue (one kernel; the float32
    q/k/v array is never written).  Same arguments and results as ``gemm_tc`` followed by ``qk_prep``."""
    lib = _lib("gemm_tc")
    n, k = x.shape
    assert w.shape == ((n_heads + 2 * n_kv_heads) * head_dim, k) and q_out.dtype == torch.bfloat16
    a = _prep_args(n, n_heads, n_kv_heads, head_dim, q_norm_w, k_norm_w, norm_eps, bias, cos, sin, rotary_dim, pairing,
                   positions, q_out, k_new, v_new, k_pages, v_pages, page_table, ring_pages, seq_of_token, slots)
    _set_scale(a, row_scale, n)
    _check(lib, lib.llg_gemm_tc_qkv(_ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), n, k, byref(a), _stream()))


def kv_write(k_new, v_new, k_pages, v_pages, page_table, ring_pages, positions, seq_of_token, slots,
             cu_tokens, len_before) -> None:
    """Copies a prompt step's packed keys/values ``[N, nkv, hd]`` into the cache pages."""
    lib = _lib("elementwise")
    n, nkv, hd = k_new.shape
    assert k_pages.dtype == k_new.dtype == v_new.dtype == v_pages.dtype
    _check(lib, lib.llg_kv_write(_ptr(k_new), _ptr(v_new), _ptr(k_pages), _ptr(v_pages),
                                 _ptr(page_table, torch.int32), page_table.shape[1], ring_pages,
                                 _ptr(positions, torch.int32), _ptr(seq_of_token, torch.int32),
                                 _ptr(slots, torch.int32), _ptr(cu_tokens, torch.int32),
                                 _ptr(len_before, torch.int32), n, nkv, hd, _dt(k_new), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[n, i] = silu(g) * u; the summed partials ``[S, N, gated_rows(I)]`` hold g and u in the gated
    layout (g of feature i at i, u at ``gated_rows(I) / 2 + i``)."""
    lib = _lib("elementwise")
    s, n, two_i = gate_up.shape
    inter = out.shape[1]
    assert out.shape == (n, inter) and two_i == gated_rows(inter)
    _check(lib, lib.llg_silu_mul(_ptr(gate_up), _dt(gate_up), s, n * two_i, _ptr(out), _dt(out), n, inter, _stream()))


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor) -> None:
    """dst.flat[idx[i]] = val[i]."""
    lib = _lib("elementwise")
    assert idx.numel() == val.numel()
    _check(lib, lib.llg_scatter_i32(_ptr(dst, torch.int32), _ptr(idx, torch.int32), _ptr(val, torch.int32),
                                    idx.numel(), _stream()))


def gather_i32(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor) -> None:
    """dst[i] = src.flat[idx[i]]."""
    lib = _lib("elementwise")
    assert dst.numel() == idx.numel()
    _check(lib, lib.llg_gather_i32(_ptr(dst, torch.int32), _ptr(src, torch.int32), _ptr(idx, torch.int32),
                                   idx.numel(), _stream()))


def zero_rows(base: torch.Tensor, rows: torch.Tensor) -> None:
    """Zeroes ``base[rows[i]]`` for a 2-D (or flattened-per-row) tensor."""
    lib = _lib("elementwise")
    row_bytes = (base.numel() // base.shape[0]) * base.element_size() if base.shape[0] else 0
    _check(lib, lib.llg_zero_rows(_ptr(base), _ptr(rows, torch.int32), rows.numel(), row_bytes, _stream()))


def _use_mma(dtype: torch.dtype, head_dim: int) -> bool:
    """bfloat16 attention with a head size the tensor-core kernels take (multiples of 16 up to 128)."""
    return dtype == torch.bfloat16 and 16 <= head_dim <= 128 and head_dim % 16 == 0


ATTN_MAX_HEAD_DIM = 256          # what csrc/attention_simt.cu takes; the tensor-core kernels take less and fall back to it
USE_TC_PROMPT_ATTENTION = True     # tests switch it off to reach the mma.sync kernel at head sizes 64 and 128


def _use_tc_attn(dtype: torch.dtype, head_dim: int) -> bool:
    """bfloat16 prompt attention with a head size the tcgen05 kernel takes (64 or 128)."""
    return USE_TC_PROMPT_ATTENTION and dtype == torch.bfloat16 and head_dim in (64, 128)


def prefill_tile_queries(dtype: torch.dtype, head_dim: int) -> int:
    """Queries per block of the prompt attention kernel that ``attn_prefill`` will run."""
    if _use_tc_attn(dtype, head_dim):
        return 256
    return 64 if _use_mma(dtype, head_dim) else 16


def attn_tc_status() -> int:
    """Error code the tcgen05 prompt attention recorded when a wait ran out (0 = none); synchronises."""
    return _lib("attention_tc").llg_attn_tc_status()


def attn_prefill(q, k_new, v_new, k_pages, v_pages, page_table, ring_pages, tiles, cu_tokens, len_before,
                 slots, out, *, scale: float, window: int, tile_queries: int) -> None:
    """Causal attention for a step with several tokens per sequence.

    ``tiles`` is ``[n_tiles, 2]`` (sequence index, first query among its step tokens) cut every
    ``tile_queries`` queries, which must be ``prefill_tile_queries(q.dtype, head_dim)``.  bfloat16 runs on
    the tensor cores: head sizes 64 and 128 with tcgen05 (csrc/attention_tc.cu), other multiples of 16 up
    to 128 with mma.sync (csrc/attention_mma.cu); everything else on the CUDA cores
    (csrc/attention_simt.cu).
    """
    n, nh, hd = q.shape
    nkv = k_new.shape[1]
    assert out.shape == (n, nh * hd)
    if tile_queries != prefill_tile_queries(q.dtype, hd):
        raise KernelError(f"attn_prefill: tiles of {tile_queries} queries, the kernel works on "
                          f"{prefill_tile_queries(q.dtype, hd)}")
    if scale <= 0:
        raise KernelError("attn_prefill: the softmax scale must be positive")
    tc = _use_tc_attn(q.dtype, hd)
    mma = _use_mma(q.dtype, hd)
    lib = _lib("attention_tc" if tc else "attention_mma" if mma else "attention_simt")
    a = _PrefillArgs()
    a.q, a.k_new, a.v_new = _ptr(q), _ptr(k_new, q.dtype), _ptr(v_new, q.dtype)
    a.k_pages, a.v_pages = _ptr(k_pages, q.dtype), _ptr(v_pages, q.dtype)
    a.page_table, a.table_width, a.ring_pages = _ptr(page_table, torch.int32), page_table.shape[1], ring_pages
    a.tiles, a.cu_tokens = _ptr(tiles, torch.int32), _ptr(cu_tokens, torch.int32)
    a.len_before, a.slots = _ptr(len_before, torch.int32), _ptr(slots, torch.int32)
    a.out = _ptr(out, q.dtype)
    a.n_tiles, a.nh, a.nkv, a.hd = tiles.shape[0], nh, nkv, hd
    a.scale, a.window = float(scale), int(window)
    a.n_tokens, a.n_pages = k_new.shape[0], k_pages.shape[0]
    if tc:
        _check(lib, lib.llg_attn_prefill_tc(byref(a), _stream()))
    elif mma:
        _check(lib, lib.llg_attn_prefill_mma(byref(a), _stream()))
    else:
        _check(lib, lib.llg_attn_prefill_simt(byref(a), _dt(q), _stream()))


# tests switch it off to reach the cp.async kernel at head sizes 64 and 128; LLOGOS_DECODE_ATTENTION=mma does the same
# for a whole process (for comparing the two kernels with the same measurement program)
USE_TMA_DECODE_ATTENTION = os.environ.get("LLOGOS_DECODE_ATTENTION", "tma") != "mma"


def _use_tma_decode(dtype: torch.dtype, head_dim: int, n_heads: int, n_kv_heads: int, n_seqs: int) -> bool:
    """bfloat16 decode attention with a geometry the TMA kernel takes (csrc/attention_decode_tma.cu)."""
    return (USE_TMA_DECODE_ATTENTION and dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv_heads > 0
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 8 and n_seqs <= 1024)


class DecodePlan:
    """How ``attn_decode`` will run for one batch shape: which kernel, how the keys are split over blocks, and what
    scratch it wants.  Made by ``attn_decode_plan``; callers only read ``scratch_floats`` and ``n_counters``."""

    def __init__(self, kind: str, n_splits: int, balance: bool, max_len: int, scratch_floats: int, n_counters: int):
        self.kind, self.n_splits, self.balance, self.max_len = kind, n_splits, balance, max_len
        self.scratch_floats, self.n_counters = scratch_floats, n_counters


def _splits_for(n_seqs: int, n_kv_heads: int, max_len: int, n_sms: int, blocks_per_sm: int = 2) -> int:
    """How many blocks share one (sequence, key/value head) in the kernels that take one split count for all.

    With ``pairs = n_seqs * n_kv_heads`` and ``tiles`` 64-key tiles per sequence, ``s`` splits run in
    ``ceil(pairs * s / resident blocks)`` rounds of ``ceil(tiles / s)`` tiles each; the ``s`` with
    the least rounds x tiles wins (the smallest on ties), so that no nearly empty last round of
    blocks doubles the time."""
    pairs = max(1, n_seqs * n_kv_heads)
    tiles = max(1, -(-max_len // PAGE))
    resident = blocks_per_sm * n_sms
    best, best_cost = 1, None
    for s in range(1, min(64, tiles) + 1):
        cost = -(-pairs * s // resident) * (-(-tiles // s) + 3)     # + 3: prologue and join of a block
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def attn_decode_plan(dtype: torch.dtype, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int, max_len: int) -> DecodePlan:
    """The plan for a batch of ``n_seqs`` sequences of at most ``max_len`` keys (the new token's included).

    bfloat16 at head sizes 64 / 128: the TMA kernel, which balances the work itself from the lengths it finds on
    the device.  Other multiples of 16 up to 128: the mma.sync kernel with a split count from ``max_len`` (per
    sequence by its length for small batches).  Everything else: the CUDA-core kernel."""
    if _use_tma_decode(dtype, head_dim, n_heads, n_kv_heads, n_seqs):
        lib = _lib("attention_decode_tma")
        floats = lib.llg_attn_decode_tma_scratch_floats(n_seqs, n_heads, n_kv_heads, head_dim, max_len)
        return DecodePlan("tma", 0, False, max_len, int(floats), n_seqs * n_heads)
    n_sms = sm_count()
    splits = _splits_for(n_seqs, n_kv_heads, max_len, n_sms)
    mma = _use_mma(dtype, head_dim)
    # Sequences of unequal lengths: the kernel gives each as many splits as its length calls for, up to what
    # one long sequence among short ones could use (the blocks the GPU holds, less one per other pair).
    balance = mma and 1 < n_seqs <= 32 and n_seqs * n_kv_heads <= attn_decode_balance_pairs()
    if balance:
        tiles = max(1, -(-max_len // PAGE))
        splits = max(splits, min(64, tiles, 2 * n_sms // n_kv_heads - (n_seqs - 1)))
    return DecodePlan("mma" if mma else "simt", splits, balance, max_len,
                      attn_decode_scratch_floats(n_seqs, n_heads, head_dim, splits), n_seqs * n_kv_heads if mma else 0)


def attn_decode_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    """Floats of scratch the split kernels need for the partial results of ``n_splits`` key splits."""
    return n_seqs * n_heads * n_splits * (head_dim + 2)


def attn_decode_balance_pairs() -> int:
    """Most (sequence, key/value head) pairs for which the mma.sync decode kernel balances its splits by length: half
    the blocks of that kernel that the GPU holds at once (two per multiprocessor)."""
    return sm_count()


def attn_decode_uses_counters(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether the split kernels want ``counters`` (the tensor-core kernel joins its splits itself)."""
    return _use_mma(dtype, head_dim)


def attn_decode_tma_status() -> int:
    """Error code the TMA decode attention recorded when a wait ran out (0 = none); synchronises."""
    return _lib("attention_decode_tma").llg_attn_decode_tma_status()


def attn_decode(q, k_pages, v_pages, page_table, ring_pages, slots, len_before, out, scratch, *,
                scale: float, window: int, plan: Optional[DecodePlan] = None, n_splits: int = 0,
                counters: Optional[torch.Tensor] = None, balance: bool = False) -> None:
    """Attention of one new token per sequence over the cache; ``scratch`` holds the partial results.

    With ``plan`` (from ``attn_decode_plan`` for this batch shape) the kernel is the plan's.  Without it the
    caller names ``n_splits`` (and ``balance``) and gets the mma.sync kernel (bfloat16, head sizes in steps of 16
    up to 128) or the CUDA-core kernel.

    The tensor-core kernels need ``counters`` (``plan.n_counters``, or ``n_seqs * n_kv_heads`` without a plan):
    int32, zero when first used (the kernels leave them zero), through which the last block of a sequence joins
    the partial results.
    ``balance`` (mma.sync kernel, at most ``attn_decode_balance_pairs()`` (sequence, kv head) pairs):
    ``n_splits`` is the most splits a sequence may have; each gets as many as its length calls for."""
    b, nh, hd = q.shape
    nkv = k_pages.shape[1]
    if scale <= 0:
        raise KernelError("attn_decode: the softmax scale must be positive")
    if scratch.dtype != torch.float32:
        raise KernelError("attn_decode: the scratch must be float32")
    if plan is not None and plan.kind == "tma":
        lib = _lib("attention_decode_tma")
        if scratch.numel() < plan.scratch_floats:
            raise KernelError(f"attn_decode: scratch of {scratch.numel()} floats, {plan.scratch_floats} needed")
        if counters is None or counters.numel() < b * nh:
            raise KernelError(f"attn_decode: needs {b * nh} zeroed int32 counters")
        a = _DecodeTmaArgs()
        a.q = _ptr(q, torch.bfloat16)
        a.page_table, a.table_width, a.ring_pages = _ptr(page_table, torch.int32), page_table.shape[1], ring_pages
        a.slots, a.len_before = _ptr(slots, torch.int32), _ptr(len_before, torch.int32)
        a.part, a.counters, a.out = _ptr(scratch), _ptr(counters, torch.int32), _ptr(out, torch.bfloat16)
        a.n_seqs, a.nh, a.nkv, a.hd = b, nh, nkv, hd
        a.scale, a.window = float(scale), int(window)
        _check(lib, lib.llg_attn_decode_tma(byref(a), _ptr(k_pages, torch.bfloat16), _ptr(v_pages, torch.bfloat16),
                                            k_pages.shape[0], int(plan.max_len), _stream()))
        return
    if plan is not None:
        n_splits, balance = plan.n_splits, plan.balance
    mma = _use_mma(q.dtype, hd)
    lib = _lib("attention_mma" if mma else "attention_simt")
    need = b * nh * n_splits * (hd + 2)
    if n_splits < 1 or scratch.numel() < need:
        raise KernelError(f"attn_decode: {n_splits} splits, scratch of {scratch.numel()} floats, {need} needed")
    a = _DecodeArgs()
    a.q, a.k_pages, a.v_pages = _ptr(q), _ptr(k_pages, q.dtype), _ptr(v_pages, q.dtype)
    a.page_table, a.table_width, a.ring_pages = _ptr(page_table, torch.int32), page_table.shape[1], ring_pages
    a.slots, a.len_before = _ptr(slots, torch.int32), _ptr(len_before, torch.int32)
    base = _ptr(scratch)
    a.part_o = base
    a.part_ml = base + 4 * b * nh * n_splits * hd
    a.n_seqs, a.nh, a.nkv, a.hd, a.n_splits = b, nh, nkv, hd, n_splits
    a.scale, a.window = float(scale), int(window)
    if mma:
        if counters is None or counters.numel() < b * nkv:
            raise KernelError(f"attn_decode: needs {b * nkv} zeroed int32 counters")
        _check(lib, lib.llg_attn_decode_mma(byref(a), _ptr(out, q.dtype), _ptr(counters, torch.int32),
                                            int(bool(balance) and b * nkv <= attn_decode_balance_pairs() and b <= 32), _stream()))
    else:
        _check(lib, lib.llg_attn_decode_simt(byref(a), _ptr(out, q.dtype), _dt(q), _stream()), kernels=2)


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float) -> None:
    """out.flat[i] = mean + std * z(key, i): the counter-based normal values of csrc/init.cu, which
    weights/random_init.py restates for the host."""
    lib = _lib("init")
    _check(lib, lib.llg_fill_normal(_ptr(out), _dt(out), out.numel(), int(key) & 0xFFFFFFFFFFFFFFFF, float(mean),
                                    float(std), _stream()))


def fill(out: torch.Tensor, value: float) -> None:
    lib = _lib("init")
    _check(lib, lib.llg_fill(_ptr(out), _dt(out), out.numel(), float(value), _stream()))


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    """dst = src converted between float32 and bfloat16 (to bfloat16: round to nearest even)."""
    lib = _lib("init")
    assert src.numel() == dst.numel()
    _check(lib, lib.llg_cast(_ptr(src), _dt(src), _ptr(dst), _dt(dst), src.numel(), _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    lib = _lib("sampling")
    b, v = logits.shape
    _check(lib, lib.llg_argmax(_ptr(logits, torch.float32), b, v, _ptr(out, torch.int32), _stream()))


def sample(logits: torch.Tensor, work: torch.Tensor, out: torch.Tensor, *, temperature: float, top_k: int = 0,
           top_p: float = 1.0, min_p: float = 0.0, typical_p: float = 1.0, min_keep: int = 1,
           repetition_penalty: float = 1.0, frequency_penalty: float = 0.0, presence_penalty: float = 0.0,
           penalize_newline: bool = False, seed: int = 0, step: int = 0,
           seq_ids: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None,
           history_len: Optional[torch.Tensor] = None, banned: Optional[torch.Tensor] = None,
           probs_out: Optional[torch.Tensor] = None, candidates: bool = True,
           history_rows: Optional[torch.Tensor] = None, history_append: bool = False) -> None:
    """One token per row of ``logits`` by the sampling pipeline of csrc/sampling.cu.

    ``history`` holds recent tokens per sequence, ``history_len`` how many each has seen: a row is a ring of
    ``history.shape[1]`` entries of which the last ``min(len, width)`` count.  Row of sequence b:
    ``history_rows[b]`` (default b).  With ``history_append`` the kernel writes the token it drew into the
    ring and raises the count, so that the next step needs nothing from the host.

    ``candidates=False`` keeps the kernels on the general way over the whole vocabulary (tests compare the
    two ways)."""
    lib = _lib("sampling")
    b, v = logits.shape
    assert work.numel() >= b * v and work.dtype == torch.float32
    a = _SampleArgs()
    a.logits, a.work, a.out = _ptr(logits, torch.float32), _ptr(work), _ptr(out, torch.int32)
    a.probs_out = _ptr(probs_out, torch.float32)
    a.seq_ids = _ptr(seq_ids, torch.int32)
    if history is not None:
        a.history, a.history_len = _ptr(history, torch.int32), _ptr(history_len, torch.int32)
        a.history_stride = history.shape[1]
        a.history_rows = _ptr(history_rows, torch.int32)
        a.history_append = int(bool(history_append))
    a.n_seqs, a.vocab = b, v
    a.temperature, a.top_k = float(temperature), int(top_k)
    a.top_p, a.min_p, a.typical_p, a.min_keep = float(top_p), float(min_p), float(typical_p), int(min_keep)
    a.repetition_penalty = float(repetition_penalty)
    a.frequency_penalty, a.presence_penalty = float(frequency_penalty), float(presence_penalty)
    a.penalize_newline = int(bool(penalize_newline))
    a.seed, a.step = int(seed) & 0xFFFFFFFFFFFFFFFF, int(step)
    if banned is not None and banned.numel():
        a.banned, a.n_banned = _ptr(banned, torch.int32), banned.numel()
    if candidates:
        # scratch of the two-stage way (top-k up to the candidate cap): the kernels decide whether they take it
        slices, cap = lib.llg_sample_slices(v), lib.llg_sample_candidate_cap()
        key = (logits.device, b, slices)
        ws = _sample_scratch.get(key)
        if ws is None:
            ws = _sample_scratch[key] = (torch.empty(b * slices * cap, dtype=torch.float32, device=logits.device),
                                         torch.empty(b * slices * cap, dtype=torch.int32, device=logits.device),
                                         torch.empty(b * slices, dtype=torch.int32, device=logits.device),
                                         torch.empty(b * slices * 3, dtype=torch.float32, device=logits.device))
        a.cand_val, a.cand_idx, a.cand_count, a.n_slices = _ptr(ws[0]), _ptr(ws[1]), _ptr(ws[2]), slices
        a.slice_stats = _ptr(ws[3])
    _check(lib, lib.llg_sample(byref(a), _stream()))


_sample_scratch = {}

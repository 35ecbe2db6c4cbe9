// The launch chain of the stock decoder block in native code: given the bound tensors of a run of blocks and one
// step's packed-token layout, it issues
//     residual add + norm -> q/k/v product -> per-head norm, bias, rotation, cache write -> attention ->
//     output product -> residual add + norm -> gate/up product with gating -> down product
// for every block, with one call from Python per step instead of nine per block.  A bfloat16 step's norms leave their
// division to the products that consume them (RowScale), as the parts do.  It computes nothing itself and
// launches no kernel of its own: it calls the kernels' entry points of the other libraries through a table of
// function pointers (llg_runner_bind), in the order and with the arguments that the parts of parts/attention.py,
// parts/feedforward.py, parts/norm.py and parts/block.py use.  Blocks with other parts, or entries that read another
// entry's cache, keep the Python path.
//
// The reference drives its kernels from managed code through one launch call per kernel and replays its token step as
// a CUDA graph to hide that cost (Daisi.Llogos.Cuda/CudaStream.cs:21-29, CudaBackend.cs:99-141); prompt steps pay it
// in full (docs/inference-optimization.md:284).
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include "kernel_args.h"

#define LLG_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local char g_error[768];

enum { F32 = 0, BF16 = 1 };

}  // namespace

// Entry points of the kernel libraries (filled in by the caller with the addresses of the loaded functions; an entry
// may stay empty as long as no step needs it, so that a caller loads only the libraries its model uses).
struct RunnerApi {
  int (*add_rmsnorm)(float*, const float*, int, long long, const void*, int, float, void*, int, const int*, int, int, float*, cudaStream_t);
  int (*gemm_tc)(const void*, const void*, void*, int, int, int, int, int, int, int, const RowScale*, cudaStream_t);
  int (*gemm_simt)(const void*, int, const void*, int, void*, int, int, int, int, const RowScale*, cudaStream_t);
  int (*qk_prep)(const QkPrepArgs*, int, cudaStream_t);
  int (*kv_write)(const void*, const void*, void*, void*, const int*, int, int, const int*, const int*, const int*, const int*,
                  const int*, int, int, int, int, cudaStream_t);
  int (*silu_mul)(const void*, int, int, long long, void*, int, int, int, cudaStream_t);
  int (*attn_prefill_tc)(const PrefillArgs*, cudaStream_t);
  int (*attn_prefill_mma)(const PrefillArgs*, cudaStream_t);
  int (*attn_prefill_simt)(const PrefillArgs*, int, cudaStream_t);
  int (*attn_decode_tma)(const DecodeTmaArgs*, const void*, const void*, int, int, cudaStream_t);
  int (*attn_decode_mma)(const DecodeArgs*, void*, int*, int, cudaStream_t);
  int (*attn_decode_simt)(const DecodeArgs*, void*, int, cudaStream_t);
  int (*gemm_tc_qkv)(const void*, const void*, int, int, const QkPrepArgs*, cudaStream_t);
  // the libraries' own error texts: elementwise, gemm_tc, gemm_simt, attention (tc, mma, simt, decode tma)
  const char* (*err_elementwise)();
  const char* (*err_gemm_tc)();
  const char* (*err_gemm_simt)();
  const char* (*err_attn_tc)();
  const char* (*err_attn_mma)();
  const char* (*err_attn_simt)();
  const char* (*err_attn_decode_tma)();
};

// One block's tensors and constants (device pointers; the caller keeps the tensors alive).
struct DenseLayer {
  const void* norm1_w;
  const void* norm2_w;
  int norm_w_dtype;
  float norm1_eps, norm2_eps;
  const void* w_qkv;           // [(nh + 2 nkv) * hd][hidden]
  const void* b_qkv;           // or null
  int bias_dtype;
  const void* q_norm_w;        // [hd] or null
  const void* k_norm_w;
  int qk_norm_w_dtype;
  float qk_norm_eps;
  const float* cos_table;      // [table_positions][rotary_dim / 2] or null
  const float* sin_table;
  int rotary_dim, pairing, table_positions;
  const void* w_o;             // [hidden][nh * hd]
  const void* w_gate_up;       // gated layout: [2 * ceil(inter / 128) * 128][hidden]
  const void* w_down;          // [hidden][inter]
  int window;
  float scale;
  // this block's cache unit
  void* k_pages;
  void* v_pages;
  const int* page_table;
  int table_width, ring_pages, n_pages;
};

// One step: the packed layout, which kernels the caller chose, and scratch.
struct RunnerStep {
  int n_tokens, n_seqs, decode, dtype;      // dtype of activations, cache and matrices: F32 or BF16
  int hidden, nh, nkv, hd, inter;
  const int* positions;
  const int* seq_of_token;
  const int* slots;
  const int* cu_tokens;
  const int* len_before;
  const int* tiles;                         // prompt steps: the query tiles of the attention kernel in use
  int n_tiles;
  int max_len_after;
  int prefill_kind;                         // 0 CUDA cores, 1 mma.sync, 2 tcgen05
  int decode_kind;                          // 0 CUDA cores, 1 mma.sync, 2 TMA
  int decode_splits, decode_balance;
  int tc_qkv, tc_o, tc_gate_up, tc_down;    // 1: the tensor-core product takes this matrix
  int splits_qkv, splits_o, splits_down;    // split-K partials of the three products that feed a sum
  int fused_qkv;                            // prompt steps: the q/k/v product prepares queries and keys in its epilogue
  float* ss;                                // bfloat16: the norms' sums of squares, [n][ss_parts]
  int ss_parts;                             // sums per row that the norm kernel writes for this step's sizes
  float* residual;                          // [n][hidden]
  void* norm_out;                           // [n][hidden]
  float* qkv;                               // [splits_qkv][n][(nh + 2 nkv) * hd]
  void* q;                                  // [n][nh][hd]
  void* k_new;                              // [n][nkv][hd] (prompt steps)
  void* v_new;
  void* attn_out;                           // [n][nh * hd]
  float* proj;                              // [splits_o][n][hidden]
  void* act;                                // [n][inter]
  float* ffn_out;                           // [splits_down][n][hidden]
  void* gate_up;                            // CUDA-core path: [min(n, gate_up_rows)][gated rows]
  int gate_up_rows;
  float* attn_scratch;
  int* attn_counters;
  cudaStream_t stream;
};

namespace {

RunnerApi g_api;
bool g_bound = false;

int fail(const char* what, const char* (*err)()) {
  snprintf(g_error, sizeof(g_error), "%s: %s", what, err ? err() : "failed");
  return 1;
}

int unbound(const char* what) {
  snprintf(g_error, sizeof(g_error), "runner: the entry point of %s has not been bound", what);
  return 1;
}

#define NEED(fn) \
  do {           \
    if (!g_api.fn) return unbound(#fn); \
  } while (0)

// y[n][o] = x[n][k] w[o][k] as `splits` float32 partials (tensor cores) or one result (CUDA cores)
int product(const RunnerStep& s, const void* x, const void* w, void* out, int out_dtype, int n, int o, int k, int tc, int splits,
            int* launches) {
  if (tc) {
    NEED(gemm_tc);
    if (g_api.gemm_tc(x, w, out, out_dtype, n, o, k, splits, 0, 0, nullptr, s.stream)) return fail("gemm_tc", g_api.err_gemm_tc);
  } else {
    NEED(gemm_simt);
    if (g_api.gemm_simt(x, s.dtype, w, s.dtype, out, out_dtype, n, o, k, nullptr, s.stream)) return fail("gemm_simt", g_api.err_gemm_simt);
  }
  ++*launches;
  return 0;
}

// residual += the pending partial sums (or nothing); norm_out = the norm of it.  A bfloat16 step leaves the division
// to the consumer (*scale).
int norm_after(const RunnerStep& s, const float* pending, int pending_parts, const void* norm_w, int norm_w_dtype, float eps,
               RowScale* scale, int* launches) {
  const int n = s.n_tokens;
  const bool defer = s.dtype == BF16 && s.ss != nullptr;
  NEED(add_rmsnorm);
  if (g_api.add_rmsnorm(s.residual, pending, pending ? pending_parts : 0, (long long)n * s.hidden, norm_w, norm_w_dtype, eps, s.norm_out,
                        s.dtype, nullptr, n, s.hidden, defer ? s.ss : nullptr, s.stream))
    return fail("add_rmsnorm", g_api.err_elementwise);
  ++*launches;
  *scale = defer ? RowScale{s.ss, s.ss_parts, 1.0f / (float)s.hidden, eps} : RowScale{nullptr, 0, 0.f, 0.f};
  return 0;
}

int run_block(const DenseLayer& L, const RunnerStep& s, const float* pending, int pending_parts, int* launches) {
  const int n = s.n_tokens;
  const int qkv_dim = (s.nh + 2 * s.nkv) * s.hd;
  // residual += what is pending; x = norm1(residual)
  RowScale scale;
  if (norm_after(s, pending, pending_parts, L.norm1_w, L.norm_w_dtype, L.norm1_eps, &scale, launches)) return 1;
  // q/k/v in float32 (partials when the product splits its sums), unless the product prepares them itself
  const bool fused = s.fused_qkv && !s.decode;
  const int s_qkv = s.tc_qkv ? s.splits_qkv : 1;
  if (!fused && product(s, s.norm_out, L.w_qkv, s.qkv, F32, n, qkv_dim, s.hidden, s.tc_qkv, s_qkv, launches)) return 1;
  QkPrepArgs p;
  memset(&p, 0, sizeof(p));
  p.row_scale = scale;
  p.qkv = s.qkv;
  p.qkv_dtype = F32;
  p.n_partials = s_qkv;
  p.partial_stride = (long long)n * qkv_dim;
  p.q_norm_w = L.q_norm_w;
  p.k_norm_w = L.k_norm_w;
  p.norm_w_dtype = L.q_norm_w ? L.qk_norm_w_dtype : F32;
  p.norm_eps = L.qk_norm_eps;
  p.bias = L.b_qkv;
  p.bias_dtype = L.b_qkv ? L.bias_dtype : F32;
  p.cos_table = L.cos_table;
  p.sin_table = L.sin_table;
  p.rotary_dim = L.cos_table ? L.rotary_dim : 0;
  p.pairing = L.cos_table ? L.pairing : 0;
  p.table_positions = L.table_positions;
  p.positions = s.positions;
  p.q_out = s.q;
  p.n_tokens = n;
  p.nh = s.nh;
  p.nkv = s.nkv;
  p.hd = s.hd;
  // A group that keeps every key takes the step's keys and values into its pages right away (a prompt step reads
  // them from the packed buffer); a ring waits until the attention has read the old keys that the new ones overwrite.
  const bool write_now = s.decode || L.window == 0;
  if (!s.decode) {
    p.k_new = s.k_new;
    p.v_new = s.v_new;
  }
  if (write_now) {
    p.k_pages = L.k_pages;
    p.v_pages = L.v_pages;
    p.page_table = L.page_table;
    p.table_width = L.table_width;
    p.ring_pages = L.ring_pages;
    p.seq_of_token = s.seq_of_token;
    p.slots = s.slots;
  }
  if (fused) {
    NEED(gemm_tc_qkv);
    p.qkv = nullptr;
    if (g_api.gemm_tc_qkv(s.norm_out, L.w_qkv, n, s.hidden, &p, s.stream)) return fail("gemm_tc_qkv", g_api.err_gemm_tc);
  } else {
    NEED(qk_prep);
    if (g_api.qk_prep(&p, s.dtype, s.stream)) return fail("qk_prep", g_api.err_elementwise);
  }
  ++*launches;
  if (s.decode) {
    if (s.decode_kind == 2) {
      DecodeTmaArgs a;
      memset(&a, 0, sizeof(a));
      a.q = s.q;
      a.page_table = L.page_table;
      a.table_width = L.table_width;
      a.ring_pages = L.ring_pages;
      a.slots = s.slots;
      a.len_before = s.len_before;
      a.part = s.attn_scratch;
      a.counters = s.attn_counters;
      a.out = s.attn_out;
      a.n_seqs = s.n_seqs;
      a.nh = s.nh;
      a.nkv = s.nkv;
      a.hd = s.hd;
      a.scale = L.scale;
      a.window = L.window;
      NEED(attn_decode_tma);
      if (g_api.attn_decode_tma(&a, L.k_pages, L.v_pages, L.n_pages, s.max_len_after, s.stream))
        return fail("attn_decode_tma", g_api.err_attn_decode_tma);
      ++*launches;
    } else {
      DecodeArgs a;
      memset(&a, 0, sizeof(a));
      a.q = s.q;
      a.k_pages = L.k_pages;
      a.v_pages = L.v_pages;
      a.page_table = L.page_table;
      a.table_width = L.table_width;
      a.ring_pages = L.ring_pages;
      a.slots = s.slots;
      a.len_before = s.len_before;
      a.part_o = s.attn_scratch;
      a.part_ml = s.attn_scratch + (long long)s.n_seqs * s.nh * s.decode_splits * s.hd;
      a.n_seqs = s.n_seqs;
      a.nh = s.nh;
      a.nkv = s.nkv;
      a.hd = s.hd;
      a.n_splits = s.decode_splits;
      a.scale = L.scale;
      a.window = L.window;
      if (s.decode_kind == 1) {
        NEED(attn_decode_mma);
        if (g_api.attn_decode_mma(&a, s.attn_out, s.attn_counters, s.decode_balance, s.stream))
          return fail("attn_decode_mma", g_api.err_attn_mma);
        ++*launches;
      } else {
        NEED(attn_decode_simt);
        if (g_api.attn_decode_simt(&a, s.attn_out, s.dtype, s.stream)) return fail("attn_decode_simt", g_api.err_attn_simt);
        *launches += 2;
      }
    }
  } else {
    PrefillArgs a;
    memset(&a, 0, sizeof(a));
    a.q = s.q;
    a.k_new = s.k_new;
    a.v_new = s.v_new;
    a.k_pages = L.k_pages;
    a.v_pages = L.v_pages;
    a.page_table = L.page_table;
    a.table_width = L.table_width;
    a.ring_pages = L.ring_pages;
    a.tiles = s.tiles;
    a.cu_tokens = s.cu_tokens;
    a.len_before = s.len_before;
    a.slots = s.slots;
    a.out = s.attn_out;
    a.n_tiles = s.n_tiles;
    a.nh = s.nh;
    a.nkv = s.nkv;
    a.hd = s.hd;
    a.scale = L.scale;
    a.window = L.window;
    a.n_tokens = n;
    a.n_pages = L.n_pages;
    int rc;
    const char* (*err)();
    if (s.prefill_kind == 2) {
      NEED(attn_prefill_tc);
      rc = g_api.attn_prefill_tc(&a, s.stream);
      err = g_api.err_attn_tc;
    } else if (s.prefill_kind == 1) {
      NEED(attn_prefill_mma);
      rc = g_api.attn_prefill_mma(&a, s.stream);
      err = g_api.err_attn_mma;
    } else {
      NEED(attn_prefill_simt);
      rc = g_api.attn_prefill_simt(&a, s.dtype, s.stream);
      err = g_api.err_attn_simt;
    }
    if (rc) return fail("attn_prefill", err);
    ++*launches;
    if (!write_now) {
      NEED(kv_write);
      if (g_api.kv_write(s.k_new, s.v_new, L.k_pages, L.v_pages, L.page_table, L.table_width, L.ring_pages, s.positions,
                         s.seq_of_token, s.slots, s.cu_tokens, s.len_before, n, s.nkv, s.hd, s.dtype, s.stream))
        return fail("kv_write", g_api.err_elementwise);
      ++*launches;
    }
  }
  // output projection, then residual += it; x = norm2(residual)
  const int s_o = s.tc_o ? s.splits_o : 1;
  if (product(s, s.attn_out, L.w_o, s.proj, F32, n, s.hidden, s.nh * s.hd, s.tc_o, s_o, launches)) return 1;
  if (norm_after(s, s.proj, s_o, L.norm2_w, L.norm_w_dtype, L.norm2_eps, &scale, launches)) return 1;
  const RowScale* sc = scale.ss ? &scale : nullptr;
  // act = silu(gate) * up
  const int gated_rows = ((s.inter + 127) / 128) * 256;
  if (s.tc_gate_up && s.dtype == BF16) {
    NEED(gemm_tc);
    if (g_api.gemm_tc(s.norm_out, L.w_gate_up, s.act, BF16, n, gated_rows, s.hidden, 1, 0, s.inter, sc, s.stream))
      return fail("gemm_tc", g_api.err_gemm_tc);
    ++*launches;
  } else {
    NEED(gemm_simt);
    NEED(silu_mul);
    const size_t el = s.dtype == BF16 ? 2 : 4;
    for (int r0 = 0; r0 < n; r0 += s.gate_up_rows) {
      const int rows = n - r0 < s.gate_up_rows ? n - r0 : s.gate_up_rows;
      const char* x = (const char*)s.norm_out + (size_t)r0 * s.hidden * el;
      RowScale part = scale;
      if (part.ss) part.ss += (long long)r0 * part.parts;
      if (g_api.gemm_simt(x, s.dtype, L.w_gate_up, s.dtype, s.gate_up, s.dtype, rows, gated_rows, s.hidden, sc ? &part : nullptr, s.stream))
        return fail("gemm_simt", g_api.err_gemm_simt);
      if (g_api.silu_mul(s.gate_up, s.dtype, 1, (long long)rows * gated_rows, (char*)s.act + (size_t)r0 * s.inter * el, s.dtype, rows,
                         s.inter, s.stream))
        return fail("silu_mul", g_api.err_elementwise);
      *launches += 2;
    }
  }
  // the block's output stays to be added by whoever comes next
  const int s_down = s.tc_down ? s.splits_down : 1;
  return product(s, s.act, L.w_down, s.ffn_out, F32, n, s.hidden, s.inter, s.tc_down, s_down, launches);
}

}  // namespace

LLG_API const char* llg_last_error() { return g_error; }

LLG_API int llg_runner_bind(const RunnerApi* api) {
  if (!api) {
    snprintf(g_error, sizeof(g_error), "runner: no function table");
    return 1;
  }
  g_api = *api;
  g_bound = true;
  return 0;
}

LLG_API int llg_runner_struct_sizes(int* api, int* layer, int* step) {
  *api = (int)sizeof(RunnerApi);
  *layer = (int)sizeof(DenseLayer);
  *step = (int)sizeof(RunnerStep);
  return 0;
}

// Runs the blocks `layers[0 .. n_layers)` in order on the step's tokens.  `pending` (or null) is a branch output that
// the first block's first norm still has to add ([pending_parts][n][hidden] float32).  When it returns 0, the last
// block's output lies in step->ffn_out as `*out_parts` partial sums still to be added, and `*launches` kernels were
// launched.
LLG_API int llg_runner_run(const DenseLayer* const* layers, int n_layers, const RunnerStep* step, const float* pending,
                           int pending_parts, int* out_parts, int* launches) {
  *launches = 0;
  if (!g_bound) {
    snprintf(g_error, sizeof(g_error), "runner: llg_runner_bind has not been called");
    return 1;
  }
  if (!layers || !step || n_layers < 0 || step->n_tokens <= 0) {
    snprintf(g_error, sizeof(g_error), "runner: bad arguments");
    return 1;
  }
  const int s_down = step->tc_down ? step->splits_down : 1;
  for (int i = 0; i < n_layers; ++i) {
    if (run_block(*layers[i], *step, pending, pending_parts, launches)) return 1;
    pending = step->ffn_out;
    pending_parts = s_down;
  }
  *out_parts = n_layers > 0 ? s_down : pending_parts;
  return 0;
}

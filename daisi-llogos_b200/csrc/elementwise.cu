// Memory-bound kernels of the decoder: embedding rows, residual add + RMSNorm,
// query/key preparation (per-head norm, bias, rotation, cache write), SiLU-gating,
// cache writes and small index updates.  All statistics and the residual stream are
// float32; activations are float32 or bfloat16.
//
// Counterparts in the reference (formulas only): Daisi.Llogos.Cuda/kernels/elementwise.cu
// rms_norm :18-48, add_rms_norm_residual :703-733, rope :243-290, swiglu :942-950,
// embedding_lookup :402-457; kernels/composite_ops.cu per_head_rms_norm :106-136,
// kv_cache_write :198-224.
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }
LLG_API int llg_page_size() { return LLG_PAGE; }

// ---- embedding ----------------------------------------------------------------------

template <typename TT>
__global__ void embed_rows_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ out, int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  int id = ids[n];
  if (id < 0 || id >= vocab) id = 0;  // ids are validated on the host; never read out of range
  const TT* row = table + (long long)id * hidden;
  float* o = out + (long long)n * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(row[i]);
}

// residual[n][:] = table[ids[n]][:]   (no scaling; Inference/ForwardPass.cs:205)
LLG_API int llg_embed_rows(const void* table, int table_dtype, const int* ids, float* out,
                           int n_tokens, int hidden, int vocab, cudaStream_t stream) {
  LLG_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0, "embed_rows: bad sizes n=%d hidden=%d vocab=%d",
              n_tokens, hidden, vocab);
  if (n_tokens == 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == LLG_F32)
    llg_launch(embed_rows_kernel<float>, n_tokens, threads, 0, stream, (const float*)table, ids, out, hidden, vocab);
  else if (table_dtype == LLG_BF16)
    llg_launch(embed_rows_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, hidden, vocab);
  else
    return llg_fail("embed_rows: unknown table dtype %d", table_dtype);
  return llg_check_launch("embed_rows");
}

// four consecutive elements as float32 (the address is a multiple of 4 elements)
__device__ __forceinline__ void vec_load4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void vec_load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&t.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}
__device__ __forceinline__ void vec_store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void vec_store4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<const uint32_t*>(&lo);
  t.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = t;
}

// ---- residual add + RMSNorm ---------------------------------------------------------

// For output row j (token r = rows ? rows[j] : j):
//   v = residual[r] + sum_s branch[s][r]   (written back to residual when there is a branch)
//   out[j] = v * rsqrt(mean(v^2) + eps) * weight         (eps inside the root, weight after)
// With ss_out the division is left to the consumer of out (RowScale in kernel_args.h): out[j] = v * weight and
// ss_out[j] = sum(v^2), whole or in parts.
template <typename OT, typename WT>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const float* __restrict__ branch,
                                   int n_partials, long long partial_stride, const WT* __restrict__ weight,
                                   float eps, OT* __restrict__ out, const int* __restrict__ rows, int hidden,
                                   float* __restrict__ ss_out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int j = blockIdx.x;
  const int r = rows ? rows[j] : j;
  float* res = residual + (long long)r * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = res[i];
    if (branch) {
      const float* b = branch + (long long)r * hidden + i;
      for (int s = 0; s < n_partials; ++s) v += b[s * partial_stride];
      res[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = ss_out ? 1.0f : 1.0f / sqrtf(ss / (float)hidden + eps);
  if (ss_out && threadIdx.x == 0) ss_out[j] = ss;
  OT* o = out + (long long)j * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_f32<OT>(res[i] * inv * to_f32(weight[i]));
}

// The same for rows whose length is a multiple of 4: 16-byte accesses, the row stays in registers
// between the two passes (VPT float4 per thread), and the partials of one element are loaded together
// so that their latencies overlap (a decode step has few rows and nothing else to hide them behind).
// One block per row also for the few rows of a decode step: a row spread over a cluster of eight blocks
// (sums of squares exchanged through distributed shared memory) took 0.07 ms more per step of 32 layers.
template <typename OT, typename WT, int VPT>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ residual, const float* __restrict__ branch,
                                        int n_partials, long long partial_stride, const WT* __restrict__ weight,
                                        float eps, OT* __restrict__ out, const int* __restrict__ rows, int hidden,
                                        float* __restrict__ ss_out) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int nv = hidden >> 2;
  // the norm's weight is no result of an earlier kernel: fetch it while the predecessor still runs
  float wv[VPT][4];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nv) vec_load4(weight + 4 * i, wv[k]);
  }
  if (threadIdx.x == 0) LLG_STAMP(3, 0, 0, blockIdx.x);
  pdl_wait();
  if (threadIdx.x == 0) LLG_STAMP(3, 1, 0, blockIdx.x);
  const int j = blockIdx.x;
  const int r = rows ? rows[j] : j;
  float4* res = reinterpret_cast<float4*>(residual + (long long)r * hidden);
  float4 keep[VPT];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < nv) {
      v = res[i];
      if (branch) {
        const float4* b = reinterpret_cast<const float4*>(branch + (long long)r * hidden) + i;
        const long long ps = partial_stride >> 2;
        int s = 0;
        if (VPT == 1) {
          // few rows (one float4 a thread): nothing to hide a load behind, so the first twelve partials are all asked
          // for before the first is added (one trip to L2 instead of one per group); they are added in their order
          constexpr int AT_ONCE = 12;
          float4 pv[AT_ONCE];
#pragma unroll
          for (int q = 0; q < AT_ONCE; ++q) pv[q] = q < n_partials ? b[q * ps] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int q = 0; q < AT_ONCE; ++q)
            if (q < n_partials) { v.x += pv[q].x; v.y += pv[q].y; v.z += pv[q].z; v.w += pv[q].w; }
          s = n_partials < AT_ONCE ? n_partials : AT_ONCE;
        }
        for (; s + 4 <= n_partials; s += 4) {
          const float4 b0 = b[(s + 0) * ps], b1 = b[(s + 1) * ps], b2 = b[(s + 2) * ps], b3 = b[(s + 3) * ps];
          v.x += b0.x; v.y += b0.y; v.z += b0.z; v.w += b0.w;
          v.x += b1.x; v.y += b1.y; v.z += b1.z; v.w += b1.w;
          v.x += b2.x; v.y += b2.y; v.z += b2.z; v.w += b2.w;
          v.x += b3.x; v.y += b3.y; v.z += b3.z; v.w += b3.w;
        }
        for (; s < n_partials; ++s) {
          const float4 b0 = b[s * ps];
          v.x += b0.x; v.y += b0.y; v.z += b0.z; v.w += b0.w;
        }
        res[i] = v;
      }
    }
    keep[k] = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, red);
  const float inv = ss_out ? 1.0f : 1.0f / sqrtf(ss / (float)hidden + eps);
  if (ss_out && threadIdx.x == 0) ss_out[j] = ss;
  OT* o = out + (long long)j * hidden;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nv) {
      const float4 v = keep[k];
      const float y[4] = {v.x * inv * wv[k][0], v.y * inv * wv[k][1], v.z * inv * wv[k][2], v.w * inv * wv[k][3]};
      vec_store4(o + 4 * i, y);
    }
  }
  if (threadIdx.x == 0) LLG_STAMP(3, 3, 0, blockIdx.x);
}

// The norm of a step of few rows when the division is left to the consumer: nothing then needs a whole row, so a
// row is cut into slices of PARTS_THREADS float4 and every (slice, row) is a block of its own that adds up its
// columns' partial sums, writes the residual stream, the weighted row and its slice's sum of squares (the consumer
// adds the slices' sums in their order).  One multiprocessor fetches a row's partial sums at some 40 GB/s (4 us
// for the 147 KB of a 4096-wide row with nine partials); spread over sixteen blocks they are there in one trip.
constexpr int PARTS_THREADS = 64;

template <typename OT, typename WT>
__global__ void __launch_bounds__(PARTS_THREADS) add_rmsnorm_parts_kernel(float* __restrict__ residual, const float* __restrict__ branch,
                                                                           int n_partials, long long partial_stride,
                                                                           const WT* __restrict__ weight, OT* __restrict__ out,
                                                                           const int* __restrict__ rows, int hidden,
                                                                           float* __restrict__ ss_out) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int i = blockIdx.x * PARTS_THREADS + threadIdx.x;          // float4 of the row (the host checks divisibility)
  float wv[4];
  vec_load4(weight + 4 * i, wv);                                   // no result of an earlier kernel
  const int j = blockIdx.y;
  if (threadIdx.x == 0) LLG_STAMP(3, 0, 0, blockIdx.x + gridDim.x * blockIdx.y);
  pdl_wait();
  if (threadIdx.x == 0) LLG_STAMP(3, 1, 0, blockIdx.x + gridDim.x * blockIdx.y);
  const int r = rows ? rows[j] : j;
  float4* res = reinterpret_cast<float4*>(residual + (long long)r * hidden);
  float4 v = res[i];
  if (branch) {
    const float4* b = reinterpret_cast<const float4*>(branch + (long long)r * hidden) + i;
    const long long ps = partial_stride >> 2;
    constexpr int AT_ONCE = 12;                                    // all asked for before the first is added, added in order
    float4 pv[AT_ONCE];
#pragma unroll
    for (int q = 0; q < AT_ONCE; ++q) pv[q] = q < n_partials ? b[q * ps] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < AT_ONCE; ++q)
      if (q < n_partials) { v.x += pv[q].x; v.y += pv[q].y; v.z += pv[q].z; v.w += pv[q].w; }
    for (int q = AT_ONCE; q < n_partials; ++q) {
      const float4 b0 = b[q * ps];
      v.x += b0.x; v.y += b0.y; v.z += b0.z; v.w += b0.w;
    }
    res[i] = v;
  }
  const float y[4] = {v.x * wv[0], v.y * wv[1], v.z * wv[2], v.w * wv[3]};
  vec_store4(out + (long long)j * hidden + 4 * i, y);
  const float ss = block_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w, red);
  if (threadIdx.x == 0) ss_out[(long long)j * gridDim.x + blockIdx.x] = ss;
  if (threadIdx.x == 0) LLG_STAMP(3, 3, 0, blockIdx.x + gridDim.x * blockIdx.y);
}

// Parts that llg_add_rmsnorm writes per row into ss_out for these sizes (the consumer's RowScale.parts).
LLG_API int llg_add_rmsnorm_parts(int n_out, int hidden) {
  const bool spread = n_out <= 64 && hidden >= 1024 && hidden % (4 * PARTS_THREADS) == 0 && hidden / (4 * PARTS_THREADS) <= 64;
  return spread ? hidden / (4 * PARTS_THREADS) : 1;
}

LLG_API int llg_add_rmsnorm(float* residual, const float* branch, int n_partials, long long partial_stride,
                            const void* weight, int weight_dtype, float eps, void* out, int out_dtype,
                            const int* rows, int n_out, int hidden, float* ss_out, cudaStream_t stream) {
  LLG_REQUIRE(n_out >= 0 && hidden > 0, "add_rmsnorm: bad sizes n_out=%d hidden=%d", n_out, hidden);
  LLG_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
  LLG_REQUIRE(!branch || n_partials >= 1, "add_rmsnorm: a branch needs n_partials >= 1");
  if (n_out == 0) return 0;
  const bool vec = hidden % 4 == 0 && partial_stride % 4 == 0 && ((uintptr_t)residual % 16) == 0 &&
                   ((uintptr_t)branch % 16) == 0 && ((uintptr_t)weight % 16) == 0 && ((uintptr_t)out % 16) == 0;
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  // vector path: few rows (decode) want many threads per row, many rows want the row in registers
  int vpt = 1;
  if (vec) {
    const int nv = hidden / 4;
    if (n_out <= 256) {
      threads = nv >= 1024 ? 1024 : (nv >= 256 ? 256 : 128);
    } else {
      threads = nv >= 1024 ? 512 : 256;
    }
    vpt = (nv + threads - 1) / threads;
    if (vpt > 8) {                     // rows longer than 8 float4 per thread: more threads
      threads = 1024;
      vpt = (nv + threads - 1) / threads;
    }
  }
  const bool vec_ok = vec && vpt <= 8;
  // the division left to the consumer and few rows: every slice of a row is a block of its own
  const int parts = ss_out ? llg_add_rmsnorm_parts(n_out, hidden) : 1;
  LLG_REQUIRE(parts == 1 || vec, "add_rmsnorm: operands of a norm in parts must be 16-byte aligned");
#define LAUNCH(OT, WT)                                                                                         \
  do {                                                                                                         \
    if (parts > 1)                                                                                             \
      llg_launch(add_rmsnorm_parts_kernel<OT, WT>, dim3(parts, n_out), PARTS_THREADS, 0, stream, residual, branch, \
                 n_partials, partial_stride, (const WT*)weight, (OT*)out, rows, hidden, ss_out);               \
    else if (vec_ok && vpt <= 1)                                                                                    \
      llg_launch(add_rmsnorm_vec4_kernel<OT, WT, 1>, n_out, threads, 0, stream, residual, branch, n_partials,    \
                 partial_stride, (const WT*)weight, eps, (OT*)out, rows, hidden, ss_out);                      \
    else if (vec_ok && vpt <= 2)                                                                               \
      llg_launch(add_rmsnorm_vec4_kernel<OT, WT, 2>, n_out, threads, 0, stream, residual, branch, n_partials,    \
                 partial_stride, (const WT*)weight, eps, (OT*)out, rows, hidden, ss_out);                      \
    else if (vec_ok && vpt <= 4)                                                                               \
      llg_launch(add_rmsnorm_vec4_kernel<OT, WT, 4>, n_out, threads, 0, stream, residual, branch, n_partials,    \
                 partial_stride, (const WT*)weight, eps, (OT*)out, rows, hidden, ss_out);                      \
    else if (vec_ok)                                                                                           \
      llg_launch(add_rmsnorm_vec4_kernel<OT, WT, 8>, n_out, threads, 0, stream, residual, branch, n_partials,    \
                 partial_stride, (const WT*)weight, eps, (OT*)out, rows, hidden, ss_out);                      \
    else                                                                                                       \
      llg_launch(add_rmsnorm_kernel<OT, WT>, n_out, threads, 0, stream, residual, branch, n_partials,            \
                 partial_stride, (const WT*)weight, eps, (OT*)out, rows, hidden, ss_out);                      \
  } while (0)
  if (out_dtype == LLG_F32 && weight_dtype == LLG_F32) LAUNCH(float, float);
  else if (out_dtype == LLG_F32 && weight_dtype == LLG_BF16) LAUNCH(float, __nv_bfloat16);
  else if (out_dtype == LLG_BF16 && weight_dtype == LLG_F32) LAUNCH(__nv_bfloat16, float);
  else if (out_dtype == LLG_BF16 && weight_dtype == LLG_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return llg_fail("add_rmsnorm: unknown dtypes out=%d weight=%d", out_dtype, weight_dtype);
#undef LAUNCH
  return llg_check_launch("add_rmsnorm");
}

// ---- query/key preparation ----------------------------------------------------------

template <typename IT, typename OT, typename WT>
__global__ void qk_prep_kernel(QkPrepArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int warps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = a.nh + 2 * a.nkv;
  const long long item = (long long)blockIdx.x * warps + warp;
  if (item >= (long long)a.n_tokens * heads) return;
  const int n = (int)(item / heads);
  const int h = (int)(item % heads);
  const int hd = a.hd;
  float* x = sm + warp * hd;
  const int kind = h < a.nh ? 0 : (h < a.nh + a.nkv ? 1 : 2);  // 0 query, 1 key, 2 value
  const long long off = (long long)n * heads * hd + (long long)h * hd;
  const IT* src = (const IT*)a.qkv + off;

  const float rs = row_scale_of(a.row_scale, n);
  float ss = 0.f;
  for (int d = lane; d < hd; d += 32) {
    float v = 0.f;
    for (int s = 0; s < a.n_partials; ++s) v += to_f32(src[s * a.partial_stride + d]);
    v *= rs;
    x[d] = v;
    ss += v * v;
  }
  const WT* nw = kind == 0 ? (const WT*)a.q_norm_w : (kind == 1 ? (const WT*)a.k_norm_w : nullptr);
  if (nw) {  // per-head RMSNorm first, then bias, then rotation (Inference/ForwardPass.cs:372-385)
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hd + a.norm_eps);
    for (int d = lane; d < hd; d += 32) x[d] = x[d] * inv * to_f32(nw[d]);
  }
  if (a.bias) {
    const WT* b = (const WT*)a.bias + (long long)h * hd;
    for (int d = lane; d < hd; d += 32) x[d] += to_f32(b[d]);
  }
  __syncwarp();
  const int pos = a.positions[n];
  if (kind != 2 && a.cos_table) {
    const int half = a.rotary_dim >> 1;
    const int p = pos < a.table_positions ? pos : a.table_positions - 1;  // bounded; host checks capacity
    const float* c = a.cos_table + (long long)p * half;
    const float* s = a.sin_table + (long long)p * half;
    for (int i = lane; i < half; i += 32) {
      const int i0 = a.pairing == 0 ? i : 2 * i;
      const int i1 = a.pairing == 0 ? i + half : 2 * i + 1;
      const float x0 = x[i0], x1 = x[i1];
      const float cs = c[i], sn = s[i];
      x[i0] = x0 * cs - x1 * sn;
      x[i1] = x0 * sn + x1 * cs;
    }
    __syncwarp();
  }
  if (kind == 0) {
    OT* o = (OT*)a.q_out + ((long long)n * a.nh + h) * hd;
    for (int d = lane; d < hd; d += 32) o[d] = from_f32<OT>(x[d]);
    return;
  }
  const int kvh = kind == 1 ? h - a.nh : h - a.nh - a.nkv;
  void* packed = kind == 1 ? a.k_new : a.v_new;
  if (packed) {
    OT* o = (OT*)packed + ((long long)n * a.nkv + kvh) * hd;
    for (int d = lane; d < hd; d += 32) o[d] = from_f32<OT>(x[d]);
  }
  void* pages = kind == 1 ? a.k_pages : a.v_pages;
  if (pages) {
    const int slot = a.slots[a.seq_of_token[n]];
    const long long row = kv_row(a.page_table, a.table_width, a.ring_pages, slot, pos, kvh, a.nkv);
    OT* o = (OT*)pages + row * hd;
    for (int d = lane; d < hd; d += 32) o[d] = from_f32<OT>(x[d]);
  }
}

// The same for the common geometry (head size 64, 128 or 256; rotation by halves over the whole
// head, or none): HD / 8 lanes share a head; a lane keeps elements 4l .. 4l+3 of each half in
// registers, so a rotation pair (i, i + HD / 2) lies in one lane, every access moves four elements,
// nothing goes through shared memory, and all loads of a head are issued before the first use.
template <typename IT, typename OT, typename WT, int HD>
__global__ void __launch_bounds__(256) qk_prep_vec_kernel(QkPrepArgs a) {
  pdl_launch_dependents();
  constexpr int LPH = HD / 8, HALF = HD / 2;      // lanes per head
  const int heads = a.nh + 2 * a.nkv;
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LPH;
  const int l = threadIdx.x % LPH;
  // lanes past the last head still take part in the shuffles below
  const bool live = item < (long long)a.n_tokens * heads;
  const int n = live ? (int)(item / heads) : 0;
  const int h = live ? (int)(item % heads) : 0;
  const int kind = h < a.nh ? 0 : (h < a.nh + a.nkv ? 1 : 2);
  const int kvh = kind == 1 ? h - a.nh : h - a.nh - a.nkv;
  // Everything but the sums themselves was written before this step's first kernel started (positions, the batch's
  // slots, the page table) or never changes (weights, biases, rotation tables): it is fetched while the product ahead
  // still runs, so that after the wait only the sums are a trip to memory away.
  const WT* nw = kind == 0 ? (const WT*)a.q_norm_w : (kind == 1 ? (const WT*)a.k_norm_w : nullptr);
  float w0[4] = {1.f, 1.f, 1.f, 1.f}, w1[4] = {1.f, 1.f, 1.f, 1.f}, b0[4] = {0.f, 0.f, 0.f, 0.f}, b1[4] = {0.f, 0.f, 0.f, 0.f};
  float cs[4] = {1.f, 1.f, 1.f, 1.f}, si[4] = {0.f, 0.f, 0.f, 0.f};
  if (nw) {
    vec_load4(nw + 4 * l, w0);
    vec_load4(nw + 4 * l + HALF, w1);
  }
  if (a.bias && live) {
    const WT* bsrc = (const WT*)a.bias + (long long)h * HD + 4 * l;
    vec_load4(bsrc, b0);
    vec_load4(bsrc + HALF, b1);
  }
  const int pos = a.positions[n];
  const bool rotate = kind != 2 && a.cos_table;
  if (rotate) {
    const int p = pos < a.table_positions ? pos : a.table_positions - 1;
    vec_load4(a.cos_table + (long long)p * HALF + 4 * l, cs);
    vec_load4(a.sin_table + (long long)p * HALF + 4 * l, si);
  }
  void* pages = kind == 0 ? nullptr : (kind == 1 ? a.k_pages : a.v_pages);
  long long page_row = 0;
  if (pages && live) page_row = kv_row(a.page_table, a.table_width, a.ring_pages, a.slots[a.seq_of_token[n]], pos, kvh, a.nkv);
  if (threadIdx.x == 0) LLG_STAMP(4, 0, 0, blockIdx.x);
  pdl_wait();
  if (threadIdx.x == 0) LLG_STAMP(4, 1, 0, blockIdx.x);
  const float rs = row_scale_of(a.row_scale, n);      // the norm's sums: a kernel of this step wrote them, so after the wait
  const IT* src = (const IT*)a.qkv + (long long)n * heads * HD + (long long)h * HD + 4 * l;
  float x0[4] = {0.f, 0.f, 0.f, 0.f}, x1[4] = {0.f, 0.f, 0.f, 0.f};   // elements 4l.. of the first and second half
  // the first eight partials are all asked for before the first is added; they are added in their order
  constexpr int AT_ONCE = 8;
  float t0[AT_ONCE][4], t1[AT_ONCE][4];
#pragma unroll
  for (int s = 0; s < AT_ONCE; ++s) {
    if (s < a.n_partials) {
      vec_load4(src + s * a.partial_stride, t0[s]);
      vec_load4(src + s * a.partial_stride + HALF, t1[s]);
    }
  }
#pragma unroll
  for (int s = 0; s < AT_ONCE; ++s) {
    if (s < a.n_partials) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        x0[k] += t0[s][k];
        x1[k] += t1[s][k];
      }
    }
  }
  for (int s = AT_ONCE; s < a.n_partials; ++s) {
    float u0[4], u1[4];
    vec_load4(src + s * a.partial_stride, u0);
    vec_load4(src + s * a.partial_stride + HALF, u1);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      x0[k] += u0[k];
      x1[k] += u1[k];
    }
  }
  if (a.row_scale.ss) {                             // what the norm ahead left to its consumer
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      x0[k] *= rs;
      x1[k] *= rs;
    }
  }
  if (a.q_norm_w || a.k_norm_w) {                  // uniform over the block: the shuffles need every lane
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) ss += x0[k] * x0[k] + x1[k] * x1[k];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (nw) {
      const float inv = 1.0f / sqrtf(ss / (float)HD + a.norm_eps);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        x0[k] = x0[k] * inv * w0[k];
        x1[k] = x1[k] * inv * w1[k];
      }
    }
  }
  if (!live) return;
  if (a.bias) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      x0[k] += b0[k];
      x1[k] += b1[k];
    }
  }
  if (rotate) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float u = x0[k], v = x1[k];
      x0[k] = u * cs[k] - v * si[k];
      x1[k] = u * si[k] + v * cs[k];
    }
  }
  if (kind == 0) {
    OT* o = (OT*)a.q_out + ((long long)n * a.nh + h) * HD + 4 * l;
    vec_store4(o, x0);
    vec_store4(o + HALF, x1);
    return;
  }
  void* packed = kind == 1 ? a.k_new : a.v_new;
  if (packed) {
    OT* o = (OT*)packed + ((long long)n * a.nkv + kvh) * HD + 4 * l;
    vec_store4(o, x0);
    vec_store4(o + HALF, x1);
  }
  if (pages) {
    OT* o = (OT*)pages + page_row * HD + 4 * l;
    vec_store4(o, x0);
    vec_store4(o + HALF, x1);
  }
  if (threadIdx.x == 0) LLG_STAMP(4, 3, 0, blockIdx.x);
}

LLG_API int llg_qk_prep(const QkPrepArgs* args, int out_dtype, cudaStream_t stream) {
  const QkPrepArgs& a = *args;
  LLG_REQUIRE(a.n_tokens >= 0 && a.nh > 0 && a.nkv >= 0 && a.hd > 0, "qk_prep: bad sizes");
  LLG_REQUIRE(a.hd <= 1024, "qk_prep: head_dim %d is larger than 1024", a.hd);
  LLG_REQUIRE(!a.cos_table || (a.rotary_dim > 0 && a.rotary_dim % 2 == 0 && a.rotary_dim <= a.hd),
              "qk_prep: rotary_dim %d must be even and at most head_dim %d", a.rotary_dim, a.hd);
  LLG_REQUIRE(a.n_partials >= 1, "qk_prep: n_partials must be >= 1");
  LLG_REQUIRE(!a.k_pages || (a.page_table && a.slots && a.seq_of_token && a.ring_pages > 0),
              "qk_prep: a cache write needs page_table, slots and seq_of_token");
  if (a.n_tokens == 0) return 0;
  // the vector kernel moves four elements at a time: every pointer must be 16-byte aligned
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15u) == 0; };
  const bool lane_ok = (a.hd == 64 || a.hd == 128 || a.hd == 256) &&
                       (!a.cos_table || (a.pairing == 0 && a.rotary_dim == a.hd)) && a.partial_stride % 4 == 0 &&
                       aligned(a.qkv) && aligned(a.q_norm_w) && aligned(a.k_norm_w) && aligned(a.bias) &&
                       aligned(a.cos_table) && aligned(a.sin_table) && aligned(a.q_out) && aligned(a.k_new) &&
                       aligned(a.v_new) && aligned(a.k_pages) && aligned(a.v_pages);
  const long long items = (long long)a.n_tokens * (a.nh + 2 * a.nkv);
  // a step of few tokens spreads its heads over many small blocks: nothing but memory latency bounds it
  const bool few = lane_ok && items * (a.hd / 8) <= (long long)2 * 64 * llg_sm_count();
  const int warps = lane_ok ? (few ? 2 : 8) : 4;
  // the vector kernel gives a head to head_dim / 8 lanes, the general one to a warp
  const long long per_block = lane_ok ? (long long)warps * 32 / (a.hd / 8) : warps;
  const unsigned grid = (unsigned)((items + per_block - 1) / per_block);
  const size_t smem = lane_ok ? 0 : (size_t)warps * a.hd * sizeof(float);
  const bool w_bf16 = (a.q_norm_w || a.k_norm_w) ? a.norm_w_dtype == LLG_BF16
                                                 : (a.bias ? a.bias_dtype == LLG_BF16 : false);
  if ((a.q_norm_w || a.k_norm_w) && a.bias)
    LLG_REQUIRE(a.norm_w_dtype == a.bias_dtype, "qk_prep: norm weights and bias must share a dtype");
#define LAUNCH(IT, OT, WT)                                                        \
  do {                                                                            \
    if (lane_ok && a.hd == 64) llg_launch(qk_prep_vec_kernel<IT, OT, WT, 64>, grid, warps * 32, 0, stream, a);        \
    else if (lane_ok && a.hd == 128) llg_launch(qk_prep_vec_kernel<IT, OT, WT, 128>, grid, warps * 32, 0, stream, a);  \
    else if (lane_ok) llg_launch(qk_prep_vec_kernel<IT, OT, WT, 256>, grid, warps * 32, 0, stream, a);                 \
    else llg_launch(qk_prep_kernel<IT, OT, WT>, grid, warps * 32, smem, stream, a);         \
  } while (0)
  if (out_dtype == LLG_F32) {
    LLG_REQUIRE(a.qkv_dtype == LLG_F32, "qk_prep: float32 output needs float32 input");
    if (w_bf16) LAUNCH(float, float, __nv_bfloat16); else LAUNCH(float, float, float);
  } else if (out_dtype == LLG_BF16) {
    if (a.qkv_dtype == LLG_F32) {
      if (w_bf16) LAUNCH(float, __nv_bfloat16, __nv_bfloat16); else LAUNCH(float, __nv_bfloat16, float);
    } else {
      if (w_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
      else LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
    }
  } else {
    return llg_fail("qk_prep: unknown output dtype %d", out_dtype);
  }
#undef LAUNCH
  return llg_check_launch("qk_prep");
}

// ---- cache write after a prompt step ------------------------------------------------

// Copies this step's keys and values [n_tokens][nkv][hd] into the paged store.  A token whose
// ring position would be overwritten by a later token of the same step is skipped.
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new, T* __restrict__ k_pages,
                                T* __restrict__ v_pages, const int* __restrict__ page_table, int table_width,
                                int ring_pages, const int* __restrict__ positions,
                                const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                const int* __restrict__ cu_tokens, const int* __restrict__ len_before,
                                int n_tokens, int nkv, int hd) {
  pdl_launch_dependents();
  pdl_wait();
  const int warps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * warps + warp;
  if (item >= (long long)n_tokens * nkv) return;
  const int n = (int)(item / nkv), kvh = (int)(item % nkv);
  const int b = seq_of_token[n];
  const int pos = positions[n];
  const int len_after = len_before[b] + (cu_tokens[b + 1] - cu_tokens[b]);
  if (pos < len_after - ring_pages * LLG_PAGE) return;
  const long long row = kv_row(page_table, table_width, ring_pages, slots[b], pos, kvh, nkv);
  const T* ks = k_new + ((long long)n * nkv + kvh) * hd;
  const T* vs = v_new + ((long long)n * nkv + kvh) * hd;
  T* kd = k_pages + row * hd;
  T* vd = v_pages + row * hd;
  for (int d = lane; d < hd; d += 32) {
    kd[d] = ks[d];
    vd[d] = vs[d];
  }
}

LLG_API int llg_kv_write(const void* k_new, const void* v_new, void* k_pages, void* v_pages,
                         const int* page_table, int table_width, int ring_pages, const int* positions,
                         const int* seq_of_token, const int* slots, const int* cu_tokens,
                         const int* len_before, int n_tokens, int nkv, int hd, int dtype,
                         cudaStream_t stream) {
  LLG_REQUIRE(n_tokens >= 0 && nkv > 0 && hd > 0 && ring_pages > 0 && table_width >= ring_pages,
              "kv_write: bad sizes");
  if (n_tokens == 0) return 0;
  const int warps = 4;
  const unsigned grid = (unsigned)(((long long)n_tokens * nkv + warps - 1) / warps);
  if (dtype == LLG_F32)
    kv_write_kernel<float><<<grid, warps * 32, 0, stream>>>(
        (const float*)k_new, (const float*)v_new, (float*)k_pages, (float*)v_pages, page_table, table_width,
        ring_pages, positions, seq_of_token, slots, cu_tokens, len_before, n_tokens, nkv, hd);
  else if (dtype == LLG_BF16)
    kv_write_kernel<__nv_bfloat16><<<grid, warps * 32, 0, stream>>>(
        (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, (__nv_bfloat16*)k_pages,
        (__nv_bfloat16*)v_pages, page_table, table_width, ring_pages, positions, seq_of_token, slots,
        cu_tokens, len_before, n_tokens, nkv, hd);
  else
    return llg_fail("kv_write: unknown dtype %d", dtype);
  return llg_check_launch("kv_write");
}

// ---- SiLU gating --------------------------------------------------------------------

// The gate and up projections are stored as one matrix: the gate rows of all features, zero rows up
// to a multiple P of 128, then the up rows in the same way (the layout the tensor-core product's
// gated epilogue wants).  A product's output row therefore holds, for feature i, g at i and u at P + i:
// out[n][i] = silu(g) * u, silu(g) = g / (1 + exp(-g))  (Daisi.Llogos.Cpu/Silu.cs:9-16).
template <typename IT, typename OT>
__global__ void silu_mul_kernel(const IT* __restrict__ gu, int n_partials, long long partial_stride,
                                OT* __restrict__ out, long long total, int inter, int width) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / inter;
    const int i = (int)(idx - n * inter);
    const IT* p = gu + n * width + i;
    float g = 0.f, u = 0.f;
    for (int s = 0; s < n_partials; ++s) {
      g += to_f32(p[s * partial_stride]);
      u += to_f32(p[s * partial_stride + width / 2]);
    }
    out[idx] = from_f32<OT>(g / (1.0f + expf(-g)) * u);
  }
}

LLG_API int llg_silu_mul(const void* gu, int in_dtype, int n_partials, long long partial_stride, void* out,
                         int out_dtype, int n_tokens, int inter, cudaStream_t stream) {
  LLG_REQUIRE(n_tokens >= 0 && inter > 0 && n_partials >= 1, "silu_mul: bad sizes");
  const long long total = (long long)n_tokens * inter;
  if (total == 0) return 0;
  const int width = ((inter + 127) / 128) * 256;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > (long long)llg_sm_count() * 16) blocks = (long long)llg_sm_count() * 16;
#define LAUNCH(IT, OT)                                                                                          \
  silu_mul_kernel<IT, OT><<<(unsigned)blocks, threads, 0, stream>>>((const IT*)gu, n_partials, partial_stride, \
                                                                     (OT*)out, total, inter, width)
  if (in_dtype == LLG_F32 && out_dtype == LLG_F32) LAUNCH(float, float);
  else if (in_dtype == LLG_F32 && out_dtype == LLG_BF16) LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == LLG_BF16 && out_dtype == LLG_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return llg_fail("silu_mul: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef LAUNCH
  return llg_check_launch("silu_mul");
}

// ---- small index updates ------------------------------------------------------------

// (No early launch of dependents here: kernels further down the step read the page table before
// they wait for their predecessor, so this kernel must be complete before any of them starts.)
__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ idx,
                                   const int* __restrict__ val, int n) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[idx[i]] = val[i];
}

// dst[idx[i]] = val[i]: new page-table entries of a step, applied in one launch.
LLG_API int llg_scatter_i32(int* dst, const int* idx, const int* val, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  scatter_i32_kernel<<<(n + 255) / 256, 256, 0, stream>>>(dst, idx, val, n);
  return llg_check_launch("scatter_i32");
}

__global__ void gather_i32_kernel(int* __restrict__ dst, const int* __restrict__ src, const int* __restrict__ idx, int n) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[idx[i]];
}

// dst[i] = src[idx[i]]: the tokens that a sampler left on the device become the next step's input.
LLG_API int llg_gather_i32(int* dst, const int* src, const int* idx, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  gather_i32_kernel<<<(n + 255) / 256, 256, 0, stream>>>(dst, src, idx, n);
  return llg_check_launch("gather_i32");
}

__global__ void zero_rows_kernel(unsigned char* __restrict__ base, const int* __restrict__ rows,
                                 long long row_bytes) {
  pdl_wait();
  unsigned char* p = base + (long long)rows[blockIdx.x] * row_bytes;
  for (long long i = threadIdx.x; i < row_bytes; i += blockDim.x) p[i] = 0;
}

// Zeroes the fixed-size state of the given slots (a sequence's state starts from zero).
LLG_API int llg_zero_rows(void* base, const int* rows, int n_rows, long long row_bytes, cudaStream_t stream) {
  if (n_rows <= 0 || row_bytes <= 0) return 0;
  zero_rows_kernel<<<n_rows, 256, 0, stream>>>((unsigned char*)base, rows, row_bytes);
  return llg_check_launch("zero_rows");
}

// Attention over the paged key/value cache on the CUDA cores, in float32 arithmetic, for
// float32 and bfloat16 storage and any head size up to 256.  These kernels are the true
// 32-bit path and the reference the tensor-core kernels are checked against.
//
//   attn_prefill : a step that brings several tokens per sequence.  Keys of positions that the
//                  step itself brings are read from the step's packed buffer, older ones from the
//                  cache pages; causal, optional window of the last W keys.
//   attn_decode  : one new token per sequence; all keys from the cache; the keys of a sequence
//                  are split over several blocks whose partial results attn_decode_reduce joins.
//
// The reference computes the same quantities with an online softmax over 256-key tiles
// (Daisi.Llogos.Cpu/CpuBackend.cs:476-590; Daisi.Llogos.Cuda/kernels/composite_ops.cu:275-387
// for one token, :396-512 for several): score = (q . k) * scale with scale applied after the
// dot product, running maximum, exponentials, sum, weighted values, division by the sum.
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

constexpr int KT = 32;      // keys per tile (one per lane)
constexpr int MAXD = 8;     // head_dim / 32 rounded up, at most
constexpr int BQ = 16;      // queries per block in attn_prefill (4 per warp)

template <typename T>
__global__ void __launch_bounds__(128) attn_prefill_kernel(PrefillArgs a) {
  extern __shared__ float sm[];
  __shared__ long long src_off[KT];
  __shared__ int src_new[KT];
  const int hd = a.hd;
  float* Qs = sm;                          // [BQ][hd]
  float* Ks = Qs + BQ * hd;                // [KT][hd + 1]
  float* Vs = Ks + KT * (hd + 1);          // [KT][hd]
  float* Ps = Vs + KT * hd;                // [BQ][KT]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = a.tiles[2 * blockIdx.x], q_off = a.tiles[2 * blockIdx.x + 1];
  const int h = blockIdx.y, kvh = h / (a.nh / a.nkv);
  const int tok0 = a.cu_tokens[b];
  const int t_b = a.cu_tokens[b + 1] - tok0;
  const int nq = min(BQ, t_b - q_off);
  const int lb = a.len_before[b];
  const int slot = a.slots[b];
  const int pos0 = lb + q_off;             // position of the tile's first query
  const int k_end = pos0 + nq;
  int k_begin = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  k_begin = (k_begin / KT) * KT;
  const T* q = (const T*)a.q;

  for (int idx = tid; idx < BQ * hd; idx += 128) {
    const int qi = idx / hd, d = idx % hd;
    Qs[idx] = qi < nq ? to_f32(q[((long long)(tok0 + q_off + qi) * a.nh + h) * hd + d]) : 0.f;
  }
  float m[4], l[4], acc[4][MAXD];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int dd = 0; dd < MAXD; ++dd) acc[i][dd] = 0.f;
  }

  for (int kt = k_begin; kt < k_end; kt += KT) {
    __syncthreads();  // previous tile fully consumed (and Qs written, first time)
    if (tid < KT) {
      const int kp = kt + tid;
      if (kp < k_end) {
        if (kp >= lb) {
          src_new[tid] = 1;
          src_off[tid] = ((long long)(tok0 + kp - lb) * a.nkv + kvh) * hd;
        } else {
          src_new[tid] = 0;
          src_off[tid] = kv_row(a.page_table, a.table_width, a.ring_pages, slot, kp, kvh, a.nkv) * hd;
        }
      } else {
        src_new[tid] = -1;
        src_off[tid] = 0;
      }
    }
    __syncthreads();
    for (int idx = tid; idx < KT * hd; idx += 128) {
      const int j = idx / hd, d = idx % hd;
      float kv = 0.f, vv = 0.f;
      const int sn = src_new[j];
      if (sn == 1) {
        kv = to_f32(((const T*)a.k_new)[src_off[j] + d]);
        vv = to_f32(((const T*)a.v_new)[src_off[j] + d]);
      } else if (sn == 0) {
        kv = to_f32(((const T*)a.k_pages)[src_off[j] + d]);
        vv = to_f32(((const T*)a.v_pages)[src_off[j] + d]);
      }
      Ks[j * (hd + 1) + d] = kv;
      Vs[j * hd + d] = vv;
    }
    __syncthreads();
    const int kp = kt + lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = warp * 4 + i;
      const int qpos = pos0 + qi;
      const float* qrow = Qs + qi * hd;
      const float* krow = Ks + lane * (hd + 1);
      float s = 0.f;
      for (int d = 0; d < hd; ++d) s = fmaf(qrow[d], krow[d], s);
      const bool valid = qi < nq && kp < k_end && kp <= qpos && (a.window == 0 || kp > qpos - a.window);
      s = valid ? s * a.scale : -INFINITY;
      const float m_new = fmaxf(m[i], warp_max(s));
      float corr = 1.f, p = 0.f;
      if (m_new != -INFINITY) {
        corr = expf(m[i] - m_new);   // exp(-inf) = 0 for the first tile
        p = valid ? expf(s - m_new) : 0.f;
      }
      l[i] = l[i] * corr + warp_sum(p);
      m[i] = m_new;
      Ps[qi * KT + lane] = p;
#pragma unroll
      for (int dd = 0; dd < MAXD; ++dd) acc[i][dd] *= corr;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float* prow = Ps + (warp * 4 + i) * KT;
#pragma unroll
      for (int dd = 0; dd < MAXD; ++dd) {
        const int d = lane + 32 * dd;
        if (d < hd) {
          float o = acc[i][dd];
          for (int j = 0; j < KT; ++j) o = fmaf(prow[j], Vs[j * hd + d], o);
          acc[i][dd] = o;
        }
      }
    }
  }
  T* out = (T*)a.out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qi = warp * 4 + i;
    if (qi >= nq) continue;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
    for (int dd = 0; dd < MAXD; ++dd) {
      const int d = lane + 32 * dd;
      if (d < hd) out[((long long)(tok0 + q_off + qi) * a.nh + h) * hd + d] = from_f32<T>(acc[i][dd] * inv);
    }
  }
}

// ---- one new token per sequence -----------------------------------------------------

constexpr int GC = 8;  // query heads of one key/value head handled per pass

template <typename T>
__global__ void __launch_bounds__(128) attn_decode_kernel(DecodeArgs a) {
  extern __shared__ float sm[];
  const int hd = a.hd;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.nh / a.nkv;
  float* Qs = sm;                                   // [GC][hd]
  float* Kt = Qs + GC * hd + warp * (KT * (hd + 1) + GC * KT);   // per warp: [KT][hd + 1]
  float* Pw = Kt + KT * (hd + 1);                   // per warp: [GC][KT]
  float* merge = Qs + GC * hd;                      // reused after the key loop: [4][GC][hd + 2]

  const int len = a.len_before[b] + 1;
  const int slot = a.slots[b];
  const int lo = a.window > 0 ? max(0, len - a.window) : 0;
  const int t0 = lo / KT, t_end = (len + KT - 1) / KT;
  const int per_split = (t_end - t0 + a.n_splits - 1) / a.n_splits;
  const int my0 = t0 + split * per_split;
  const int my1 = min(t_end, my0 + per_split);
  const T* kp_base = (const T*)a.k_pages;
  const T* vp_base = (const T*)a.v_pages;

  for (int g0 = 0; g0 < G; g0 += GC) {
    const int ng = min(GC, G - g0);
    __syncthreads();
    for (int idx = tid; idx < GC * hd; idx += 128) {
      const int g = idx / hd, d = idx % hd;
      Qs[idx] = g < ng ? to_f32(((const T*)a.q)[((long long)b * a.nh + kvh * G + g0 + g) * hd + d]) : 0.f;
    }
    __syncthreads();
    float m[GC], l[GC], acc[GC][MAXD];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int dd = 0; dd < MAXD; ++dd) acc[g][dd] = 0.f;
    }
    for (int t = my0 + warp; t < my1; t += 4) {
      const int kp = t * KT + lane;
      const bool valid = kp >= lo && kp < len;
      const long long row = valid ? kv_row(a.page_table, a.table_width, a.ring_pages, slot, kp, kvh, a.nkv) : 0;
      __syncwarp();
      for (int j = 0; j < KT; ++j) {
        const long long rj = __shfl_sync(0xffffffffu, row, j);
        const bool vj = __shfl_sync(0xffffffffu, (int)valid, j);
        for (int d = lane; d < hd; d += 32) Kt[j * (hd + 1) + d] = vj ? to_f32(kp_base[rj * hd + d]) : 0.f;
      }
      __syncwarp();
      const float* krow = Kt + lane * (hd + 1);
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        if (g >= ng) break;
        const float* qrow = Qs + g * hd;
        float s = 0.f;
        for (int d = 0; d < hd; ++d) s = fmaf(qrow[d], krow[d], s);
        s = valid ? s * a.scale : -INFINITY;
        const float m_new = fmaxf(m[g], warp_max(s));
        float corr = 1.f, p = 0.f;
        if (m_new != -INFINITY) {
          corr = expf(m[g] - m_new);
          p = valid ? expf(s - m_new) : 0.f;
        }
        l[g] = l[g] * corr + warp_sum(p);
        m[g] = m_new;
        Pw[g * KT + lane] = p;
#pragma unroll
        for (int dd = 0; dd < MAXD; ++dd) acc[g][dd] *= corr;
      }
      __syncwarp();
      for (int j = 0; j < KT; ++j) {
        const bool vj = __shfl_sync(0xffffffffu, (int)valid, j);
        const long long rj = __shfl_sync(0xffffffffu, row, j);
        if (!vj) continue;
#pragma unroll
        for (int dd = 0; dd < MAXD; ++dd) {
          const int d = lane + 32 * dd;
          if (d < hd) {
            const float v = to_f32(vp_base[rj * hd + d]);
#pragma unroll
            for (int g = 0; g < GC; ++g)
              if (g < ng) acc[g][dd] = fmaf(Pw[g * KT + j], v, acc[g][dd]);
          }
        }
      }
    }
    // join the four warps
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      if (g >= ng) break;
      float* dst = merge + ((warp * GC + g) * (hd + 2));
#pragma unroll
      for (int dd = 0; dd < MAXD; ++dd) {
        const int d = lane + 32 * dd;
        if (d < hd) dst[d] = acc[g][dd];
      }
      if (lane == 0) {
        dst[hd] = m[g];
        dst[hd + 1] = l[g];
      }
    }
    __syncthreads();
    for (int g = warp; g < ng; g += 4) {
      float mw[4], M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        mw[w] = merge[(w * GC + g) * (hd + 2) + hd];
        M = fmaxf(M, mw[w]);
      }
      float L = 0.f, sc[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        sc[w] = (M == -INFINITY) ? 0.f : expf(mw[w] - M);
        L += sc[w] * merge[(w * GC + g) * (hd + 2) + hd + 1];
      }
      const int h = kvh * G + g0 + g;
      const long long pidx = ((long long)b * a.nh + h) * a.n_splits + split;
      for (int d = lane; d < hd; d += 32) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) o += sc[w] * merge[(w * GC + g) * (hd + 2) + d];
        a.part_o[pidx * hd + d] = o;
      }
      if (lane == 0) {
        a.part_ml[pidx * 2] = M;
        a.part_ml[pidx * 2 + 1] = L;
      }
    }
  }
}

template <typename T>
__global__ void attn_decode_reduce_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          T* __restrict__ out, int nh, int hd, int n_splits) {
  const int h = blockIdx.x, b = blockIdx.y;
  const long long base = ((long long)b * nh + h) * n_splits;
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms != -INFINITY) L += expf(ms - M) * part_ml[(base + s) * 2 + 1];
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) o += expf(ms - M) * part_o[(base + s) * hd + d];
    }
    out[((long long)b * nh + h) * hd + d] = from_f32<T>(o * inv);
  }
}

}  // namespace

LLG_API int llg_attn_prefill_simt(const PrefillArgs* args, int dtype, cudaStream_t stream) {
  const PrefillArgs& a = *args;
  LLG_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "attn_prefill: %d heads are no multiple of %d key/value heads",
              a.nh, a.nkv);
  LLG_REQUIRE(a.hd > 0 && a.hd <= 32 * MAXD, "attn_prefill: head_dim %d is outside [1, %d]", a.hd, 32 * MAXD);
  LLG_REQUIRE(a.window >= 0 && a.ring_pages > 0 && a.table_width >= a.ring_pages, "attn_prefill: bad cache geometry");
  LLG_REQUIRE(a.nh <= 65535, "attn_prefill: too many heads");
  if (a.n_tiles <= 0) return 0;
  const size_t smem = (size_t)(BQ * a.hd + KT * (a.hd + 1) + KT * a.hd + BQ * KT) * sizeof(float);
  dim3 grid(a.n_tiles, a.nh);
  cudaError_t e;
  if (dtype == LLG_F32) {
    e = cudaFuncSetAttribute(attn_prefill_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llg_fail("attn_prefill: shared memory %zu: %s", smem, cudaGetErrorString(e));
    attn_prefill_kernel<float><<<grid, 128, smem, stream>>>(a);
  } else if (dtype == LLG_BF16) {
    e = cudaFuncSetAttribute(attn_prefill_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llg_fail("attn_prefill: shared memory %zu: %s", smem, cudaGetErrorString(e));
    attn_prefill_kernel<__nv_bfloat16><<<grid, 128, smem, stream>>>(a);
  } else {
    return llg_fail("attn_prefill: unknown dtype %d", dtype);
  }
  return llg_check_launch("attn_prefill");
}

// Floats of scratch that attn_decode needs for its partial results.
LLG_API long long llg_attn_decode_scratch_floats(int n_seqs, int nh, int hd, int n_splits) {
  return (long long)n_seqs * nh * n_splits * (hd + 2);
}

LLG_API int llg_attn_decode_simt(const DecodeArgs* args, void* out, int dtype, cudaStream_t stream) {
  const DecodeArgs& a = *args;
  LLG_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "attn_decode: %d heads are no multiple of %d key/value heads",
              a.nh, a.nkv);
  LLG_REQUIRE(a.hd > 0 && a.hd <= 32 * MAXD, "attn_decode: head_dim %d is outside [1, %d]", a.hd, 32 * MAXD);
  LLG_REQUIRE(a.n_splits >= 1 && a.n_splits <= 65535, "attn_decode: n_splits %d", a.n_splits);
  LLG_REQUIRE(a.window >= 0 && a.ring_pages > 0 && a.table_width >= a.ring_pages, "attn_decode: bad cache geometry");
  LLG_REQUIRE(a.nkv <= 65535 && a.n_seqs <= 65535, "attn_decode: grid too large");
  if (a.n_seqs <= 0) return 0;
  const size_t per_warp = (size_t)KT * (a.hd + 1) + GC * KT;
  size_t floats = (size_t)GC * a.hd + 4 * per_warp;
  const size_t merge_floats = (size_t)GC * a.hd + 4 * GC * (a.hd + 2);
  if (merge_floats > floats) floats = merge_floats;
  const size_t smem = floats * sizeof(float);
  dim3 grid(a.n_splits, a.nkv, a.n_seqs);
  dim3 rgrid(a.nh, a.n_seqs);
  cudaError_t e;
  if (dtype == LLG_F32) {
    e = cudaFuncSetAttribute(attn_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llg_fail("attn_decode: shared memory %zu: %s", smem, cudaGetErrorString(e));
    attn_decode_kernel<float><<<grid, 128, smem, stream>>>(a);
    attn_decode_reduce_kernel<float><<<rgrid, 64, 0, stream>>>(a.part_o, a.part_ml, (float*)out, a.nh, a.hd, a.n_splits);
  } else if (dtype == LLG_BF16) {
    e = cudaFuncSetAttribute(attn_decode_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llg_fail("attn_decode: shared memory %zu: %s", smem, cudaGetErrorString(e));
    attn_decode_kernel<__nv_bfloat16><<<grid, 128, smem, stream>>>(a);
    attn_decode_reduce_kernel<__nv_bfloat16><<<rgrid, 64, 0, stream>>>(a.part_o, a.part_ml, (__nv_bfloat16*)out, a.nh, a.hd,
                                                                        a.n_splits);
  } else {
    return llg_fail("attn_decode: unknown dtype %d", dtype);
  }
  return llg_check_launch("attn_decode");
}

// ---- the entry point that allocates nothing (see attention_noalloc.h) ---------------------------

#include "attention_noalloc.h"

// Scratch for the split partials of llg_attn_decode_noalloc.  In host code this name is only a
// handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_noalloc_scratch[LLG_ATTN_NOALLOC_MAX_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES];   // device address of the array, per device, once looked up
}  // namespace

int llg_attn_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                            int table_width, int ring_pages, const int* slots, const int* len_before, void* out,
                            int dtype, int n_seqs, int n_heads, int n_kv_heads, int head_dim, int n_splits,
                            float scale, int window, cudaStream_t stream) {
  LLG_REQUIRE(n_seqs >= 0 && n_heads > 0 && head_dim > 0 && n_splits >= 1, "attn_decode_noalloc: bad sizes");
  const long long need = (long long)n_seqs * n_heads * n_splits * (head_dim + 2);
  LLG_REQUIRE(need <= (long long)LLG_ATTN_NOALLOC_MAX_FLOATS,
              "attn_decode_noalloc: %d sequences x %d heads x %d splits x (%d + 2) = %lld floats of scratch, "
              "the built-in array holds %d; use fewer splits or llg_attn_decode_simt with scratch of your own",
              n_seqs, n_heads, n_splits, head_dim, need, (int)LLG_ATTN_NOALLOC_MAX_FLOATS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return llg_fail("attn_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  LLG_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, "attn_decode_noalloc: device index %d is not supported", dev);
  if (g_noalloc_ptr[dev] == nullptr) {   // set-up, once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return llg_fail("attn_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_noalloc_ptr[dev] = p;
  }
  DecodeArgs a;
  a.q = q;
  a.k_pages = k_pages;
  a.v_pages = v_pages;
  a.page_table = page_table;
  a.table_width = table_width;
  a.ring_pages = ring_pages;
  a.slots = slots;
  a.len_before = len_before;
  a.part_o = g_noalloc_ptr[dev];
  a.part_ml = g_noalloc_ptr[dev] + (long long)n_seqs * n_heads * n_splits * head_dim;
  a.n_seqs = n_seqs;
  a.nh = n_heads;
  a.nkv = n_kv_heads;
  a.hd = head_dim;
  a.n_splits = n_splits;
  a.scale = scale;
  a.window = window;
  return llg_attn_decode_simt(&a, out, dtype, stream);
}

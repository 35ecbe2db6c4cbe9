// Attention over the paged key/value cache on the tensor cores, for bfloat16 storage and head
// sizes that are multiples of 16 up to 128.  Scores, softmax and output accumulators are float32
// (mma.sync m16n8k16 with float32 accumulation); probabilities are rounded to bfloat16 only as
// the operand of the second product.
//
//   attn_prefill_mma : 64 queries of one head per block (16 per warp); key/value tiles of 64
//                      positions are staged in shared memory with cp.async, double-buffered.  Keys
//                      of positions the step itself brings come from the step's packed buffer,
//                      older ones from cache pages (same contract as attn_prefill_simt).
//   attn_decode_mma  : one new token per sequence.  The query heads that share a key/value head
//                      fill the rows of one MMA tile, so keys and values are read once per
//                      key/value head; a block's four warps split each 64-key page, blocks split
//                      the sequence (partials in the caller's scratch, joined by attn_decode_reduce).
//
// Shared-memory rows are padded by 16 bytes, which makes every ldmatrix conflict-free for any
// head size without a swizzle.  The reference's kernels for the same step are scalar
// (Daisi.Llogos.Cuda/kernels/composite_ops.cu:275-387 one block per query head, :396-512 one
// block per query token and head) and re-read keys for every head of a group.
#include "common.cuh"

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

constexpr int TK = 64;   // keys per tile = one cache page

struct PrefillArgs {      // same layout as in attention_simt.cu
  const void* q;
  const void* k_new;
  const void* v_new;
  const void* k_pages;
  const void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* tiles;       // [n_tiles][2]: (sequence, first query), 64 queries per tile
  const int* cu_tokens;
  const int* len_before;
  const int* slots;
  void* out;
  int n_tiles, nh, nkv, hd;
  float scale;
  int window;
};

struct DecodeArgs {       // same layout as in attention_simt.cu
  const void* q;
  const void* k_pages;
  const void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* slots;
  const int* len_before;
  float* part_o;
  float* part_ml;
  int n_seqs, nh, nkv, hd, n_splits;
  float scale;
  int window;
};

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16-byte asynchronous copy; copies zeros when !valid
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// d += a (16x16, row) * b (16x8, col), bfloat16 operands, float32 accumulation
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr float LOG2E = 1.4426950408889634f;

// ---- prompt steps --------------------------------------------------------------------------------

template <int HDMAX>
__global__ void __launch_bounds__(128) attn_prefill_mma_kernel(PrefillArgs a) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int hd = a.hd;
  const int rs = hd * 2 + 16;                 // bytes per shared-memory row
  const int cpr = hd / 8;                     // 16-byte chunks per row
  const int ksteps = hd / 16;
  unsigned char* Qs = smraw;                  // [64][rs]
  unsigned char* Ks = Qs + 64 * rs;           // [2][64][rs]
  unsigned char* Vs = Ks + 2 * 64 * rs;       // [2][64][rs]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int b = a.tiles[2 * blockIdx.x], q_off = a.tiles[2 * blockIdx.x + 1];
  const int h = blockIdx.y, kvh = h / (a.nh / a.nkv);
  const int tok0 = a.cu_tokens[b];
  const int nq = min(64, a.cu_tokens[b + 1] - tok0 - q_off);
  const int lb = a.len_before[b];
  const int slot = a.slots[b];
  const int pos0 = lb + q_off;
  const int k_end = pos0 + nq;
  int k_begin = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  k_begin = (k_begin / TK) * TK;
  const int n_tiles = (k_end - k_begin + TK - 1) / TK;
  const bf16* qg = (const bf16*)a.q;
  const bf16* kn = (const bf16*)a.k_new;
  const bf16* vn = (const bf16*)a.v_new;
  const bf16* kp = (const bf16*)a.k_pages;
  const bf16* vp = (const bf16*)a.v_pages;

  auto load_kv = [&](int tile, int stage) {
    const int kt = k_begin + tile * TK;
    unsigned char* kd = Ks + stage * 64 * rs;
    unsigned char* vd = Vs + stage * 64 * rs;
    for (int c = tid; c < 64 * cpr; c += 128) {
      const int row = c / cpr, ch = c - row * cpr;
      const int pos = kt + row;
      const bool valid = pos < k_end;
      const bf16 *ks = kp, *vs = vp;
      if (valid) {
        if (pos >= lb) {
          const long long off = ((long long)(tok0 + pos - lb) * a.nkv + kvh) * hd + ch * 8;
          ks = kn + off;
          vs = vn + off;
        } else {
          const long long off = kv_row(a.page_table, a.table_width, a.ring_pages, slot, pos, kvh, a.nkv) * hd + ch * 8;
          ks = kp + off;
          vs = vp + off;
        }
      }
      cp_async16(smem_u32(kd + row * rs + ch * 16), ks, valid);
      cp_async16(smem_u32(vd + row * rs + ch * 16), vs, valid);
    }
  };

  for (int c = tid; c < 64 * cpr; c += 128) {
    const int row = c / cpr, ch = c - row * cpr;
    const bool valid = row < nq;
    const bf16* src = qg + ((long long)(tok0 + q_off + (valid ? row : 0)) * a.nh + h) * hd + ch * 8;
    cp_async16(smem_u32(Qs + row * rs + ch * 16), src, valid);
  }
  cp_async_commit();
  load_kv(0, 0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  uint32_t qf[HDMAX / 16][4];
#pragma unroll
  for (int ks = 0; ks < HDMAX / 16; ++ks) {
    if (ks < ksteps) {
      const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int col = ks * 16 + (lane >> 4) * 8;
      ldmatrix_x4(qf[ks], smem_u32(Qs + row * rs + col * 2));
    }
  }
  float o[HDMAX / 8][4];
#pragma unroll
  for (int j = 0; j < HDMAX / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const float sc = a.scale * LOG2E;
  const int qpos0 = pos0 + warp * 16 + g;      // position of this thread's first row; second is +8

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) load_kv(tile + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const unsigned char* kd = Ks + stage * 64 * rs;
    const unsigned char* vd = Vs + stage * 64 * rs;
    const int kt = k_begin + tile * TK;

    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HDMAX / 16; ++ks) {
      if (ks < ksteps) {
#pragma unroll
        for (int jp = 0; jp < 4; ++jp) {       // two 8-key tiles per ldmatrix
          uint32_t kb[4];
          const int row = jp * 16 + (lane & 7) + (lane >> 4) * 8;
          const int col = ks * 16 + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(kb, smem_u32(kd + row * rs + col * 2));
          mma_16816(s[2 * jp], qf[ks], kb[0], kb[1]);
          mma_16816(s[2 * jp + 1], qf[ks], kb[2], kb[3]);
        }
      }
    }
    // mask, running maximum, exponentials
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int key = kt + j * 8 + 2 * t + (e & 1);
        const int qp = qpos0 + r * 8;
        const bool valid = key <= qp && (a.window == 0 || key > qp - a.window);
        s[j][e] = valid ? s[j][e] : -INFINITY;
        mx[r] = fmaxf(mx[r], s[j][e]);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m[r], mx[r]);
      corr[r] = (m_new == -INFINITY) ? 1.f : exp2f((m[r] - m_new) * sc);
      m[r] = m_new;
      l[r] *= corr[r];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float p = (m[r] == -INFINITY) ? 0.f : exp2f((s[j][e] - m[r]) * sc);
        s[j][e] = p;
        l[r] += p;
      }
#pragma unroll
    for (int j = 0; j < HDMAX / 8; ++j) {
      o[j][0] *= corr[0];
      o[j][1] *= corr[0];
      o[j][2] *= corr[1];
      o[j][3] *= corr[1];
    }
    // o += p v
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int jp = 0; jp < HDMAX / 16; ++jp) {
        if (jp < ksteps) {
          uint32_t vb[4];
          const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int col = jp * 16 + (lane >> 4) * 8;
          ldmatrix_x4_trans(vb, smem_u32(vd + row * rs + col * 2));
          mma_16816(o[2 * jp], pa, vb[0], vb[1]);
          mma_16816(o[2 * jp + 1], pa, vb[2], vb[3]);
        }
      }
    }
    __syncthreads();   // the stage may be overwritten by the load issued in the next iteration
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  bf16* out = (bf16*)a.out;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + r * 8;
    if (row >= nq) continue;
    const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
    bf16* dst = out + ((long long)(tok0 + q_off + row) * a.nh + h) * hd;
#pragma unroll
    for (int j = 0; j < HDMAX / 8; ++j) {
      if (j * 8 < hd)
        *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t) = pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
  }
}

// ---- one new token per sequence ------------------------------------------------------------------

constexpr int DSTAGES = 3;

template <int HDMAX>
__global__ void __launch_bounds__(128) attn_decode_mma_kernel(DecodeArgs a) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int hd = a.hd;
  const int rs = hd * 2 + 16;
  const int cpr = hd / 8;
  const int ksteps = hd / 16;
  unsigned char* Ks = smraw;                          // [DSTAGES][64][rs]
  unsigned char* Vs = Ks + DSTAGES * 64 * rs;         // [DSTAGES][64][rs]
  float* merge = reinterpret_cast<float*>(smraw);     // after the key loop: [4 warps][16 rows][hd + 2]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.nh / a.nkv;
  const int len = a.len_before[b] + 1;
  const int slot = a.slots[b];
  const int lo = a.window > 0 ? max(0, len - a.window) : 0;
  const int t0 = lo / TK, t_end = (len + TK - 1) / TK;
  const int per_split = (t_end - t0 + a.n_splits - 1) / a.n_splits;
  const int my0 = t0 + split * per_split;
  const int my1 = min(t_end, my0 + per_split);
  const int n_my = max(0, my1 - my0);
  const bf16* kp = (const bf16*)a.k_pages;
  const bf16* vp = (const bf16*)a.v_pages;
  const bf16* qg = (const bf16*)a.q;
  const float sc = a.scale * LOG2E;

  auto load_kv = [&](int tile, int stage) {
    // positions 64 * tile .. + 63 lie in one page, contiguous for this key/value head
    const long long base = kv_row(a.page_table, a.table_width, a.ring_pages, slot, tile * TK, kvh, a.nkv) * hd;
    unsigned char* kd = Ks + stage * 64 * rs;
    unsigned char* vd = Vs + stage * 64 * rs;
    for (int c = tid; c < 64 * cpr; c += 128) {
      const int row = c / cpr, ch = c - row * cpr;
      const long long off = base + (long long)row * hd + ch * 8;
      cp_async16(smem_u32(kd + row * rs + ch * 16), kp + off, true);
      cp_async16(smem_u32(vd + row * rs + ch * 16), vp + off, true);
    }
  };

  for (int g0 = 0; g0 < G; g0 += 16) {
    const int ng = min(16, G - g0);
    __syncthreads();                                  // merge area of the previous pass is free again
    // prologue of the pipeline
#pragma unroll
    for (int s = 0; s < DSTAGES - 1; ++s) {
      if (s < n_my) load_kv(my0 + s, s);
      cp_async_commit();
    }
    // query fragments straight from global memory: rows = heads of this group
    uint32_t qf[HDMAX / 16][4];
#pragma unroll
    for (int ks = 0; ks < HDMAX / 16; ++ks) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = g + (e & 1) * 8;
        const int col = ks * 16 + 2 * t + (e >> 1) * 8;
        uint32_t v = 0;
        if (ks < ksteps && row < ng)
          v = *reinterpret_cast<const uint32_t*>(qg + ((long long)b * a.nh + kvh * G + g0 + row) * hd + col);
        qf[ks][e] = v;
      }
    }
    float o[HDMAX / 8][4];
#pragma unroll
    for (int j = 0; j < HDMAX / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int i = 0; i < n_my; ++i) {
      const int stage = i % DSTAGES;
      if (i + DSTAGES - 1 < n_my) load_kv(my0 + i + DSTAGES - 1, (i + DSTAGES - 1) % DSTAGES);
      cp_async_commit();
      cp_async_wait<DSTAGES - 1>();
      __syncthreads();
      const unsigned char* kd = Ks + stage * 64 * rs;
      const unsigned char* vd = Vs + stage * 64 * rs;
      const int kt = (my0 + i) * TK + warp * 16;     // this warp's 16 keys of the page

      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < HDMAX / 16; ++ks) {
        if (ks < ksteps) {
          uint32_t kb[4];
          const int row = warp * 16 + (lane & 7) + (lane >> 4) * 8;
          const int col = ks * 16 + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(kb, smem_u32(kd + row * rs + col * 2));
          mma_16816(s[0], qf[ks], kb[0], kb[1]);
          mma_16816(s[1], qf[ks], kb[2], kb[3]);
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kt + j * 8 + 2 * t + (e & 1);
          const bool valid = key >= lo && key < len;
          s[j][e] = valid ? s[j][e] : -INFINITY;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
        }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        corr[r] = (m_new == -INFINITY) ? 1.f : exp2f((m[r] - m_new) * sc);
        m[r] = m_new;
        l[r] *= corr[r];
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const float p = (m[r] == -INFINITY) ? 0.f : exp2f((s[j][e] - m[r]) * sc);
          s[j][e] = p;
          l[r] += p;
        }
#pragma unroll
      for (int j = 0; j < HDMAX / 8; ++j) {
        o[j][0] *= corr[0];
        o[j][1] *= corr[0];
        o[j][2] *= corr[1];
        o[j][3] *= corr[1];
      }
      uint32_t pa[4];
      pa[0] = pack_bf16(s[0][0], s[0][1]);
      pa[1] = pack_bf16(s[0][2], s[0][3]);
      pa[2] = pack_bf16(s[1][0], s[1][1]);
      pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int jp = 0; jp < HDMAX / 16; ++jp) {
        if (jp < ksteps) {
          uint32_t vb[4];
          const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int col = jp * 16 + (lane >> 4) * 8;
          ldmatrix_x4_trans(vb, smem_u32(vd + row * rs + col * 2));
          mma_16816(o[2 * jp], pa, vb[0], vb[1]);
          mma_16816(o[2 * jp + 1], pa, vb[2], vb[3]);
        }
      }
      __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();
    // each warp leaves its rows' (o, m, l); then the four are joined
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      const int row = g + r * 8;
      float* dst = merge + ((warp * 16 + row) * (hd + 2));
#pragma unroll
      for (int j = 0; j < HDMAX / 8; ++j) {
        if (j * 8 < hd) {
          dst[j * 8 + 2 * t] = o[j][2 * r];
          dst[j * 8 + 2 * t + 1] = o[j][2 * r + 1];
        }
      }
      if (t == 0) {
        dst[hd] = m[r];
        dst[hd + 1] = l[r];
      }
    }
    __syncthreads();
    for (int row = warp; row < ng; row += 4) {
      float mw[4], M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        mw[w] = merge[(w * 16 + row) * (hd + 2) + hd];
        M = fmaxf(M, mw[w]);
      }
      float L = 0.f, scw[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        scw[w] = (mw[w] == -INFINITY) ? 0.f : exp2f((mw[w] - M) * sc);
        L += scw[w] * merge[(w * 16 + row) * (hd + 2) + hd + 1];
      }
      const int head = kvh * G + g0 + row;
      const long long pidx = ((long long)b * a.nh + head) * a.n_splits + split;
      for (int d = lane; d < hd; d += 32) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) acc += scw[w] * merge[(w * 16 + row) * (hd + 2) + d];
        a.part_o[pidx * hd + d] = acc;
      }
      if (lane == 0) {
        // the running maximum is kept in units of the raw score; the reduce kernel works with
        // natural exponentials of (m * scale), so hand it the scaled value
        a.part_ml[pidx * 2] = (M == -INFINITY) ? -INFINITY : M * a.scale;
        a.part_ml[pidx * 2 + 1] = L;
      }
    }
  }
}

// joins the partials of the splits: out = sum_s exp(m_s - M) o_s / sum_s exp(m_s - M) l_s
__global__ void attn_decode_reduce_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          bf16* __restrict__ out, int nh, int hd, int n_splits) {
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
    out[((long long)b * nh + h) * hd + d] = __float2bfloat16_rn(o * inv);
  }
}

template <typename K>
int set_smem(K kernel, size_t smem, const char* what) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return llg_fail("%s: shared memory %zu: %s", what, smem, cudaGetErrorString(e));
  return 0;
}

}  // namespace

// 1 when these kernels take the head size (bfloat16 only): a multiple of 16, at most 128.
LLG_API int llg_attn_mma_supported(int hd) { return hd >= 16 && hd <= 128 && hd % 16 == 0; }

LLG_API int llg_attn_prefill_mma(const PrefillArgs* args, cudaStream_t stream) {
  const PrefillArgs& a = *args;
  LLG_REQUIRE(llg_attn_mma_supported(a.hd), "attn_prefill_mma: head_dim %d is not a multiple of 16 up to 128", a.hd);
  LLG_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "attn_prefill_mma: %d heads are no multiple of %d key/value heads",
              a.nh, a.nkv);
  LLG_REQUIRE(a.window >= 0 && a.ring_pages > 0 && a.table_width >= a.ring_pages && a.nh <= 65535,
              "attn_prefill_mma: bad cache geometry");
  if (a.n_tiles <= 0) return 0;
  const size_t smem = (size_t)5 * 64 * (a.hd * 2 + 16);
  dim3 grid(a.n_tiles, a.nh);
  if (a.hd <= 64) {
    if (set_smem(attn_prefill_mma_kernel<64>, smem, "attn_prefill_mma")) return 1;
    attn_prefill_mma_kernel<64><<<grid, 128, smem, stream>>>(a);
  } else {
    if (set_smem(attn_prefill_mma_kernel<128>, smem, "attn_prefill_mma")) return 1;
    attn_prefill_mma_kernel<128><<<grid, 128, smem, stream>>>(a);
  }
  return llg_check_launch("attn_prefill_mma");
}

LLG_API int llg_attn_decode_mma(const DecodeArgs* args, void* out, cudaStream_t stream) {
  const DecodeArgs& a = *args;
  LLG_REQUIRE(llg_attn_mma_supported(a.hd), "attn_decode_mma: head_dim %d is not a multiple of 16 up to 128", a.hd);
  LLG_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "attn_decode_mma: %d heads are no multiple of %d key/value heads",
              a.nh, a.nkv);
  LLG_REQUIRE(a.n_splits >= 1 && a.n_splits <= 65535 && a.nkv <= 65535 && a.n_seqs <= 65535, "attn_decode_mma: grid too large");
  LLG_REQUIRE(a.window >= 0 && a.ring_pages > 0 && a.table_width >= a.ring_pages, "attn_decode_mma: bad cache geometry");
  if (a.n_seqs <= 0) return 0;
  size_t smem = (size_t)2 * DSTAGES * 64 * (a.hd * 2 + 16);
  const size_t merge = (size_t)4 * 16 * (a.hd + 2) * sizeof(float);
  if (merge > smem) smem = merge;
  dim3 grid(a.n_splits, a.nkv, a.n_seqs);
  if (a.hd <= 64) {
    if (set_smem(attn_decode_mma_kernel<64>, smem, "attn_decode_mma")) return 1;
    attn_decode_mma_kernel<64><<<grid, 128, smem, stream>>>(a);
  } else {
    if (set_smem(attn_decode_mma_kernel<128>, smem, "attn_decode_mma")) return 1;
    attn_decode_mma_kernel<128><<<grid, 128, smem, stream>>>(a);
  }
  attn_decode_reduce_kernel<<<dim3(a.nh, a.n_seqs), 64, 0, stream>>>(a.part_o, a.part_ml, (bf16*)out, a.nh, a.hd, a.n_splits);
  return llg_check_launch("attn_decode_mma");
}

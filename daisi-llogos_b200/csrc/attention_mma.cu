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
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

constexpr int TK = 64;   // keys per tile = one cache page

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

// 2^x by the special-function unit alone (float32, about 2 ulp, denormal results flushed to zero);
// exp2f() adds range handling that the softmax does not need: its arguments are <= 0 or -inf.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^d for a whole number d <= 0 (or -inf), exactly.
__device__ __forceinline__ float pow2_whole(float d) {
  return d < -126.f ? 0.f : __int_as_float((127 + (int)d) << 23);
}

// The running maximum of a softmax row is kept in the exponent's own unit (score * scale * log2 e) and rounded
// up to a whole number M.  The weights are then 2^(x - M), rescaling between two maxima multiplies by an exact
// power of two, and rounding a weight to bfloat16 gives the same bits whatever M was when the weight was made:
// how the keys are cut into tiles, warps, blocks or steps does not show in the rounded weights.

// ---- prompt steps --------------------------------------------------------------------------------

// EXACT: the head size is HDMAX itself, known at compile time (all offsets become constants)
template <int HDMAX, bool EXACT>
__global__ void __launch_bounds__(128, 3) attn_prefill_mma_kernel(PrefillArgs a) {
  extern __shared__ __align__(16) unsigned char smraw[];
  pdl_launch_dependents();
  pdl_wait();
  const int hd = EXACT ? HDMAX : a.hd;
  const int rs = hd * 2 + 16;                 // bytes per shared-memory row
  const int cpr = hd / 8;                     // 16-byte chunks per row
  const int ksteps = hd / 16;
  unsigned char* Ks = smraw;                  // [2][64][rs]
  unsigned char* Vs = Ks + 2 * 64 * rs;       // [2][64][rs]
  unsigned char* Qs = Vs + 64 * rs;           // [64][rs]: the queries pass through the second value stage,
                                              // which is first needed after they are in registers
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  // the caller lists the tiles with the most keys first; blocks start head by head within a tile, tile
  // by tile, so the long blocks start first
  const int tile_id = (int)blockIdx.y;
  const int b = a.tiles[2 * tile_id], q_off = a.tiles[2 * tile_id + 1];
  const int h = blockIdx.x, kvh = h / (a.nh / a.nkv);
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

  // Thread `tid` copies 16-byte chunk `ch0` of rows `row0, row0 + rstep, ...` when 128 is a multiple of
  // the chunks per row (head sizes 16, 32, 64, 128); other head sizes take the general indexing.
  const bool regular = (128 % cpr) == 0;
  const int row0 = tid / cpr, ch0 = tid - row0 * cpr, rstep = regular ? 128 / cpr : 0;
  auto load_kv = [&](int tile, int stage) {
    const int kt = k_begin + tile * TK;           // a multiple of 64: the tile's old positions share one page
    unsigned char* kd = Ks + stage * 64 * rs;
    unsigned char* vd = Vs + stage * 64 * rs;
    const long long old_base = kt < lb ? kv_row(a.page_table, a.table_width, a.ring_pages, slot, kt, kvh, a.nkv) * hd : 0;
    const long long new_base = ((long long)(tok0 + kt - lb) * a.nkv + kvh) * hd;    // row r adds r * nkv * hd
    const long long new_step = (long long)a.nkv * hd;
    if (regular) {
      uint32_t kdst = smem_u32(kd + row0 * rs + ch0 * 16), vdst = smem_u32(vd + row0 * rs + ch0 * 16);
      for (int row = row0; row < 64; row += rstep, kdst += rstep * rs, vdst += rstep * rs) {
        const int pos = kt + row;
        const bool valid = pos < k_end;
        const bool fresh = pos >= lb;
        const long long off = (fresh ? new_base + row * new_step : old_base + (long long)row * hd) + ch0 * 8;
        cp_async16(kdst, (fresh ? kn : kp) + (valid ? off : 0), valid);
        cp_async16(vdst, (fresh ? vn : vp) + (valid ? off : 0), valid);
      }
    } else {
      for (int c = tid; c < 64 * cpr; c += 128) {
        const int row = c / cpr, ch = c - row * cpr;
        const int pos = kt + row;
        const bool valid = pos < k_end;
        const bool fresh = pos >= lb;
        const long long off = (fresh ? new_base + row * new_step : old_base + (long long)row * hd) + ch * 8;
        cp_async16(smem_u32(kd + row * rs + ch * 16), (fresh ? kn : kp) + (valid ? off : 0), valid);
        cp_async16(smem_u32(vd + row * rs + ch * 16), (fresh ? vn : vp) + (valid ? off : 0), valid);
      }
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
  __syncthreads();                             // every warp has its queries: their staging area may be overwritten
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
    // mask (only tiles that touch the diagonal or the window's edge need one), running maximum, exponentials
    float mx[2] = {-INFINITY, -INFINITY};
    const bool need_mask = (kt + TK - 1 > pos0 + warp * 16) || (a.window > 0 && kt <= pos0 + warp * 16 + 15 - a.window);
    if (need_mask) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int key = kt + j * 8 + 2 * t + (e & 1);
          const int qp = qpos0 + r * 8;
          const bool valid = key <= qp && (a.window == 0 || key > qp - a.window);
          s[j][e] = valid ? s[j][e] : -INFINITY;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m[r], ceilf(mx[r] * sc));
      corr[r] = (m_new == -INFINITY) ? 1.f : pow2_whole(m[r] - m_new);
      m[r] = m_new;
      l[r] *= corr[r];
    }
    const float ms0 = (m[0] == -INFINITY) ? 0.f : m[0], ms1 = (m[1] == -INFINITY) ? 0.f : m[1];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float p = fast_exp2(fmaf(s[j][e], sc, r ? -ms1 : -ms0));     // exp2(-inf) = 0 for masked keys
        s[j][e] = p;
        l[r] += p;
      }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
      for (int j = 0; j < HDMAX / 8; ++j) {
        o[j][0] *= corr[0];
        o[j][1] *= corr[0];
        o[j][2] *= corr[1];
        o[j][3] *= corr[1];
      }
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
//
// The products are taken transposed so that no MMA row is padding: S^T = K Q^T has the warp's 16
// keys as rows and (up to 8) query heads of the group as columns; O^T = V^T P^T has 16 head
// dimensions as rows.  P^T reaches the operand layout of the second product by movmatrix.

constexpr int DSTAGES = 3;
constexpr int GH = 8;     // query heads per pass (one MMA n-tile)

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

// `counters` ([n_seqs][nkv] ints, zero before the first launch) let the block that finishes last for a
// (sequence, key/value head) join the partials of all splits and write `out`; it leaves the counter at
// zero again.  No second kernel is needed.
//
// Work items are (sequence, key/value head, split).  Without `balance` every sequence has a.n_splits
// splits and the grid is (splits, key/value heads, sequences), one block per item.  With `balance` the
// grid is one row of at most `resident` blocks (what the GPU holds of this kernel at once), a block takes items blockIdx.x, blockIdx.x +
// gridDim.x, ..., and a sequence has as many splits as its length calls for (at most a.n_splits):
// every block works out the same number T of key tiles per item, the least with which the
// items of all sequences fit the GPU at once, and sequence b gets ceil(tiles_b / T) splits.  A batch of
// one long and seven short sequences then spreads the long one over most of the GPU; sequences of one
// length get the same count each.
constexpr int DECODE_BLOCKS_PER_SM = 2;       // blocks of this kernel that one SM holds at once

// 64-key tiles that a sequence of `len` keys reads
__device__ __forceinline__ int decode_tiles(int len, int window) {
  const int lo = window > 0 ? max(0, len - window) : 0;
  return (len + TK - 1) / TK - lo / TK;
}

template <int HDMAX, bool EXACT, bool BALANCE>
__global__ void __launch_bounds__(128) attn_decode_mma_kernel(DecodeArgs a, bf16* __restrict__ out, int* __restrict__ counters,
                                                              int resident) {
  constexpr bool balance = BALANCE;
  extern __shared__ __align__(16) unsigned char smraw[];
  __shared__ int is_last;
  pdl_launch_dependents();
  // Lengths, slots and page tables were written before this step's first kernel started.  The
  // kernel just before this one writes only the newest position (in the sequence's last page) and
  // the queries: tiles before the last page may be requested before waiting for it.
  bool waited = false;
  const int hd = EXACT ? HDMAX : a.hd;
  const int rs = hd * 2 + 16;
  const int cpr = hd / 8;
  const int ksteps = hd / 16;
  unsigned char* Ks = smraw;                          // [DSTAGES][64][rs]
  unsigned char* Vs = Ks + DSTAGES * 64 * rs;         // [DSTAGES][64][rs]
  float* merge = reinterpret_cast<float*>(smraw);     // after the key loop: [4 warps][GH heads][hd + 2]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = a.nh / a.nkv;
  // ---- the plan: key tiles per item, and how many items there are.  Lane i of every warp keeps the tile
  // count of sequence i (a balanced launch has at most 32 sequences), so no warp waits for another. ----
  int n_items = a.n_seqs * a.n_splits * a.nkv, tiles_per_item = 0;
  int my_tiles = 0;
  if (balance) {
    my_tiles = lane < a.n_seqs ? decode_tiles(a.len_before[lane] + 1, a.window) : 0;
    int hi = max(1, my_tiles);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    int lo_t = 1, n = 0;
    for (;;) {                                       // least T with nkv * sum_b min(n_splits, ceil(tiles_b / T)) <= slots
      const int mid = lo_t < hi ? (lo_t + hi) >> 1 : hi;
      n = lane < a.n_seqs ? max(1, min(a.n_splits, (my_tiles + mid - 1) / mid)) : 0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
      if (lo_t >= hi) break;
      if (n * a.nkv <= resident) hi = mid;
      else lo_t = mid + 1;
    }
    tiles_per_item = hi;
    n_items = n * a.nkv;
  }
 // (without balancing the grid is (splits, key/value heads, sequences), one block per item: the body runs once)
 for (int item = balance ? blockIdx.x : 0; item < n_items; item += balance ? gridDim.x : n_items) {
  // balanced: item -> (sequence, split, key/value head), the heads of one (sequence, split) are neighbours
  int kvh, b, split, ns = a.n_splits;
  if (balance) {
    kvh = item % a.nkv;
    split = item / a.nkv;
    const int mine = lane < a.n_seqs ? max(1, min(a.n_splits, (my_tiles + tiles_per_item - 1) / tiles_per_item)) : 0;
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    b = __ffs(__ballot_sync(0xffffffffu, incl > split)) - 1;       // first sequence whose items reach past this one
    ns = __shfl_sync(0xffffffffu, mine, b);
    split -= __shfl_sync(0xffffffffu, incl, b) - ns;
  } else {
    split = blockIdx.x;
    kvh = blockIdx.y;
    b = blockIdx.z;
  }
  const int len = a.len_before[b] + 1;
  const int slot = a.slots[b];
  const int lo = a.window > 0 ? max(0, len - a.window) : 0;
  const int t0 = lo / TK, t_end = (len + TK - 1) / TK;
  const int per_split = (t_end - t0 + ns - 1) / ns;
  const int my0 = t0 + split * per_split;
  const int my1 = min(t_end, my0 + per_split);
  const int n_my = max(0, my1 - my0);
  const bf16* kp = (const bf16*)a.k_pages;
  const bf16* vp = (const bf16*)a.v_pages;
  const bf16* qg = (const bf16*)a.q;
  const float sc = a.scale * LOG2E;

  // The page of a tile is looked up one iteration before its copies are issued, so that the
  // table read never sits between a finished tile and the next prefetch.
  auto page_base = [&](int tile) -> long long {
    // positions 64 * tile .. + 63 lie in one page, contiguous for this key/value head
    return kv_row(a.page_table, a.table_width, a.ring_pages, slot, tile * TK, kvh, a.nkv) * hd;
  };
  const bool regular = (128 % cpr) == 0;
  const int row0 = tid / cpr, ch0 = tid - row0 * cpr, rstep = regular ? 128 / cpr : 0;
  auto load_kv = [&](long long base, int stage) {
    unsigned char* kd = Ks + stage * 64 * rs;
    unsigned char* vd = Vs + stage * 64 * rs;
    if (regular) {
      uint32_t kdst = smem_u32(kd + row0 * rs + ch0 * 16), vdst = smem_u32(vd + row0 * rs + ch0 * 16);
      const bf16* ksrc = kp + base + (long long)row0 * hd + ch0 * 8;
      const bf16* vsrc = vp + base + (long long)row0 * hd + ch0 * 8;
      const int gstep = rstep * hd, sstep = rstep * rs;
      for (int row = row0; row < 64; row += rstep, kdst += sstep, vdst += sstep, ksrc += gstep, vsrc += gstep) {
        cp_async16(kdst, ksrc, true);
        cp_async16(vdst, vsrc, true);
      }
    } else {
      for (int c = tid; c < 64 * cpr; c += 128) {
        const int row = c / cpr, ch = c - row * cpr;
        const long long off = base + (long long)row * hd + ch * 8;
        cp_async16(smem_u32(kd + row * rs + ch * 16), kp + off, true);
        cp_async16(smem_u32(vd + row * rs + ch * 16), vp + off, true);
      }
    }
  };

  for (int g0 = 0; g0 < G; g0 += GH) {
    const int ng = min(GH, G - g0);
    __syncthreads();                                  // merge area of the previous pass is free again
#pragma unroll
    for (int s = 0; s < DSTAGES - 1; ++s) {
      if (s < n_my) {
        if (!waited && my0 + s >= t_end - 1) {
          pdl_wait();
          waited = true;
        }
        load_kv(page_base(my0 + s), s);
      }
      cp_async_commit();
    }
    if (!waited) {
      pdl_wait();
      waited = true;
    }
    long long next_base = (DSTAGES - 1 < n_my) ? page_base(my0 + DSTAGES - 1) : 0;
    // Q^T as the second operand: column g is head g0 + g, rows are head dimensions
    uint32_t qf[HDMAX / 16][2];
#pragma unroll
    for (int ks = 0; ks < HDMAX / 16; ++ks) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        uint32_t v = 0;
        if (ks < ksteps && g < ng)
          v = *reinterpret_cast<const uint32_t*>(qg + ((long long)b * a.nh + kvh * G + g0 + g) * hd + ks * 16 + 2 * t + e * 8);
        qf[ks][e] = v;
      }
    }
    float o[HDMAX / 16][4];      // O^T: rows = 16 head dimensions per tile, columns = heads 2t, 2t + 1
#pragma unroll
    for (int j = 0; j < HDMAX / 16; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};   // per column (head 2t, 2t + 1)

    for (int i = 0; i < n_my; ++i) {
      const int stage = i % DSTAGES;
      if (i + DSTAGES - 1 < n_my) load_kv(next_base, (i + DSTAGES - 1) % DSTAGES);
      cp_async_commit();
      if (i + DSTAGES < n_my) next_base = page_base(my0 + i + DSTAGES);
      cp_async_wait<DSTAGES - 1>();
      __syncthreads();
      const unsigned char* kd = Ks + stage * 64 * rs;
      const unsigned char* vd = Vs + stage * 64 * rs;
      const int kt = (my0 + i) * TK + warp * 16;     // this warp's 16 keys of the page

      // S^T = K Q^T, two accumulators so that the chain of dependent MMAs is half as long
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t k_addr = smem_u32(kd + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * rs + (lane >> 4) * 16);
#pragma unroll
      for (int ks = 0; ks < HDMAX / 16; ++ks) {
        if (ks < ksteps) {
          uint32_t ka[4];
          ldmatrix_x4(ka, k_addr + ks * 32);
          if (ks & 1) mma_16816(s1, ka, qf[ks][0], qf[ks][1]);
          else mma_16816(s0, ka, qf[ks][0], qf[ks][1]);
        }
      }
      float sv[4];
      const bool valid0 = (kt + g) >= lo && (kt + g) < len;
      const bool valid1 = (kt + g + 8) >= lo && (kt + g + 8) < len;
      sv[0] = valid0 ? s0[0] + s1[0] : -INFINITY;
      sv[1] = valid0 ? s0[1] + s1[1] : -INFINITY;
      sv[2] = valid1 ? s0[2] + s1[2] : -INFINITY;
      sv[3] = valid1 ? s0[3] + s1[3] : -INFINITY;
      // column maxima over the 16 keys: rows live in lanes that differ in g
      float mx[2] = {fmaxf(sv[0], sv[2]), fmaxf(sv[1], sv[3])};
      float corr[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 4));
        mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 8));
        mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 16));
        const float m_new = fmaxf(m[c], ceilf(mx[c] * sc));
        corr[c] = (m_new == -INFINITY) ? 1.f : pow2_whole(m[c] - m_new);
        m[c] = m_new;
      }
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = e & 1;
        pv[e] = (m[c] == -INFINITY) ? 0.f : fast_exp2(fmaf(sv[e], sc, -m[c]));
      }
      l[0] = l[0] * corr[0] + pv[0] + pv[2];
      l[1] = l[1] * corr[1] + pv[1] + pv[3];
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
        for (int j = 0; j < HDMAX / 16; ++j) {
          o[j][0] *= corr[0];
          o[j][1] *= corr[1];
          o[j][2] *= corr[0];
          o[j][3] *= corr[1];
        }
      }
      // P^T in the layout of the second operand: transpose the two 8x8 blocks of S^T
      const uint32_t pb0 = movmatrix_trans(pack_bf16(pv[0], pv[1]));
      const uint32_t pb1 = movmatrix_trans(pack_bf16(pv[2], pv[3]));
      // O^T += V^T P^T, 16 head dimensions per MMA
      const uint32_t v_addr = smem_u32(vd + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * rs + ((lane >> 3) & 1) * 16);
#pragma unroll
      for (int j = 0; j < HDMAX / 16; ++j) {
        if (j < ksteps) {
          uint32_t va[4];
          ldmatrix_x4_trans(va, v_addr + j * 32);
          mma_16816(o[j], va, pb0, pb1);
        }
      }
      __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();
    // each warp leaves (o, m, l) of its heads; then the four are joined
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      l[c] += __shfl_xor_sync(0xffffffffu, l[c], 4);
      l[c] += __shfl_xor_sync(0xffffffffu, l[c], 8);
      l[c] += __shfl_xor_sync(0xffffffffu, l[c], 16);
      const int head = 2 * t + c;
      float* dst = merge + ((warp * GH + head) * (hd + 2));
#pragma unroll
      for (int j = 0; j < HDMAX / 16; ++j) {
        if (j < ksteps) {
          dst[j * 16 + g] = o[j][c];
          dst[j * 16 + g + 8] = o[j][2 + c];
        }
      }
      if (g == 0) {
        dst[hd] = m[c];
        dst[hd + 1] = l[c];
      }
    }
    __syncthreads();
    for (int row = warp; row < ng; row += 4) {
      float mw[4], M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        mw[w] = merge[(w * GH + row) * (hd + 2) + hd];
        M = fmaxf(M, mw[w]);
      }
      float L = 0.f, scw[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        scw[w] = (mw[w] == -INFINITY) ? 0.f : pow2_whole(mw[w] - M);
        L += scw[w] * merge[(w * GH + row) * (hd + 2) + hd + 1];
      }
      const int head = kvh * G + g0 + row;
      const long long pidx = ((long long)b * a.nh + head) * a.n_splits + split;
      for (int d = lane; d < hd; d += 32) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) acc += scw[w] * merge[(w * GH + row) * (hd + 2) + d];
        a.part_o[pidx * hd + d] = acc;
      }
      if (lane == 0) {
        // the running maximum is a whole number of binary orders; the join works with natural exponentials
        a.part_ml[pidx * 2] = (M == -INFINITY) ? -INFINITY : M * 0.6931471805599453f;
        a.part_ml[pidx * 2 + 1] = L;
      }
    }
  }
  // ---- the last block of this (sequence, key/value head) joins the splits ---------------------------
  __threadfence();                     // this block's partials are visible to the whole device ...
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(&counters[b * a.nkv + kvh], 1);   // ... before its ticket is
    is_last = ticket == ns - 1;
    if (is_last) counters[b * a.nkv + kvh] = 0;
  }
  __syncthreads();
  if (!is_last) continue;
  __threadfence();
  // one warp per head; the splits' weights exp(m_s - M) are worked out by the lanes side by side and kept
  // in shared memory (64 at a time), then every lane sums its head dimensions over the splits with
  // independent loads
  float* wsm = reinterpret_cast<float*>(smraw) + warp * 64;
  for (int head = kvh * G + warp; head < (kvh + 1) * G; head += 4) {
    const long long base = ((long long)b * a.nh + head) * a.n_splits;
    float M = -INFINITY;
    for (int s = lane; s < ns; s += 32) M = fmaxf(M, __ldcg(&a.part_ml[(base + s) * 2]));
    M = warp_max(M);
    float L = 0.f;
    for (int s = lane; s < ns; s += 32) {
      const float ms = __ldcg(&a.part_ml[(base + s) * 2]);
      if (ms != -INFINITY) L += expf(ms - M) * __ldcg(&a.part_ml[(base + s) * 2 + 1]);
    }
    L = warp_sum(L);
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    float oacc[HDMAX / 32];
#pragma unroll
    for (int dd = 0; dd < HDMAX / 32; ++dd) oacc[dd] = 0.f;
    for (int s0 = 0; s0 < ns; s0 += 64) {
      const int nc = min(64, ns - s0);
      __syncwarp();
      for (int s = lane; s < nc; s += 32) {
        const float ms = __ldcg(&a.part_ml[(base + s0 + s) * 2]);
        wsm[s] = (ms == -INFINITY) ? 0.f : expf(ms - M);
      }
      __syncwarp();
#pragma unroll
      for (int dd = 0; dd < HDMAX / 32; ++dd) {
        const int d = lane + 32 * dd;
        if (d < hd) {
          const float* po = a.part_o + (base + s0) * hd + d;
          float o = 0.f;
          int s = 0;
          for (; s + 4 <= nc; s += 4) {
            const float p0 = __ldcg(po + (long long)(s + 0) * hd), p1 = __ldcg(po + (long long)(s + 1) * hd);
            const float p2 = __ldcg(po + (long long)(s + 2) * hd), p3 = __ldcg(po + (long long)(s + 3) * hd);
            o += wsm[s] * p0 + wsm[s + 1] * p1 + wsm[s + 2] * p2 + wsm[s + 3] * p3;
          }
          for (; s < nc; ++s) o += wsm[s] * __ldcg(po + (long long)s * hd);
          oacc[dd] += o;
        }
      }
    }
#pragma unroll
    for (int dd = 0; dd < HDMAX / 32; ++dd) {
      const int d = lane + 32 * dd;
      if (d < hd) out[((long long)b * a.nh + head) * hd + d] = __float2bfloat16_rn(oacc[dd] * inv);
    }
  }
 }   // items
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
  LLG_REQUIRE(a.window >= 0 && a.ring_pages > 0 && a.table_width >= a.ring_pages, "attn_prefill_mma: bad cache geometry");
  LLG_REQUIRE(a.n_tiles <= 65535, "attn_prefill_mma: %d query tiles in one step are more than a grid takes (65535)", a.n_tiles);
  if (a.n_tiles <= 0) return 0;
  const size_t smem = (size_t)4 * 64 * (a.hd * 2 + 16);
  dim3 grid(a.nh, a.n_tiles);
#define GO(HDM, EX)                                                                        \
  do {                                                                                     \
    if (set_smem(attn_prefill_mma_kernel<HDM, EX>, smem, "attn_prefill_mma")) return 1;      \
    llg_launch(attn_prefill_mma_kernel<HDM, EX>, grid, dim3(128), smem, stream, a);          \
  } while (0)
  if (a.hd == 64) GO(64, true);
  else if (a.hd == 128) GO(128, true);
  else if (a.hd < 64) GO(64, false);
  else GO(128, false);
#undef GO
  return llg_check_launch("attn_prefill_mma");
}

// n_splits: the most blocks that share one (sequence, key/value head), and the stride of the partials.
// balance = 1: a sequence uses as many of them as its length calls for (see the kernel); for batches whose
// (sequence, key/value head) pairs are at most half the blocks that the GPU holds.
LLG_API int llg_attn_decode_mma(const DecodeArgs* args, void* out, int* counters, int balance, cudaStream_t stream) {
  const DecodeArgs& a = *args;
  LLG_REQUIRE(llg_attn_mma_supported(a.hd), "attn_decode_mma: head_dim %d is not a multiple of 16 up to 128", a.hd);
  LLG_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "attn_decode_mma: %d heads are no multiple of %d key/value heads",
              a.nh, a.nkv);
  LLG_REQUIRE(a.n_splits >= 1 && a.n_splits <= 65535 && a.nkv <= 65535 && a.n_seqs <= 65535, "attn_decode_mma: grid too large");
  const int resident = DECODE_BLOCKS_PER_SM * llg_sm_count();
  LLG_REQUIRE(!balance || (a.n_seqs * a.nkv <= resident / 2 && a.n_seqs <= 32),
              "attn_decode_mma: balanced splits are for at most 32 sequences and %d (sequence, key/value head) pairs",
              resident / 2);
  LLG_REQUIRE(a.window >= 0 && a.ring_pages > 0 && a.table_width >= a.ring_pages, "attn_decode_mma: bad cache geometry");
  LLG_REQUIRE(counters != nullptr, "attn_decode_mma: needs n_seqs * nkv zeroed counters");
  if (a.n_seqs <= 0) return 0;
  size_t smem = (size_t)2 * DSTAGES * 64 * (a.hd * 2 + 16);
  const size_t merge = (size_t)4 * GH * (a.hd + 2) * sizeof(float);
  if (merge > smem) smem = merge;
  // balanced: as many blocks as the GPU holds, each taking the items that fall to it; otherwise one block per
  // item, which lets the hardware start the next block of an SM while its neighbour is still in its last tiles
  const long long items = (long long)a.n_splits * a.nkv * a.n_seqs;
  const dim3 grid = balance ? dim3((unsigned)(items > resident ? resident : items)) : dim3(a.n_splits, a.nkv, a.n_seqs);
#define GO(HDM, EX)                                                                                         \
  do {                                                                                                      \
    if (balance) {                                                                                          \
      if (set_smem(attn_decode_mma_kernel<HDM, EX, true>, smem, "attn_decode_mma")) return 1;                 \
      llg_launch(attn_decode_mma_kernel<HDM, EX, true>, grid, dim3(128), smem, stream, a, (bf16*)out, counters, resident);  \
    } else {                                                                                                \
      if (set_smem(attn_decode_mma_kernel<HDM, EX, false>, smem, "attn_decode_mma")) return 1;                \
      llg_launch(attn_decode_mma_kernel<HDM, EX, false>, grid, dim3(128), smem, stream, a, (bf16*)out, counters, resident); \
    }                                                                                                       \
  } while (0)
  if (a.hd == 64) GO(64, true);
  else if (a.hd == 128) GO(128, true);
  else if (a.hd < 64) GO(64, false);
  else GO(128, false);
#undef GO
  return llg_check_launch("attn_decode_mma");
}

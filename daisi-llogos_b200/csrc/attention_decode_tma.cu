// Attention of one new token per sequence over the paged cache, bfloat16, head sizes 64 and 128, groups of up
// to 8 query heads per key/value head.  The kernel streams the cache: 4 flop per byte, so the memory system
// decides its time and the arithmetic runs on mma.sync (m16n8k16, float32 accumulation) beside it.
//
//   copies     A fifth warp brings every key and value tile (one cache page of one key/value head: 64
//              positions x head size) with TMA boxes of 64 x 64 elements, 128-byte swizzled, into a ring of
//              stages; a stage is handed over by an mbarrier pair (full: the bytes have landed; empty: the four
//              working warps are done with it).  Its lanes look up the pages of 32 tiles at once and then
//              issue their tiles in turn; no thread computes the address of a single element.
//   work       The (sequence, key/value head, tile) units of the whole batch form one list, sequence by
//              sequence; the blocks cut it into equal runs, so every block streams the same number of tiles
//              whatever the lengths are.  Every block works the plan out itself from the lengths (a scan in
//              shared memory) before it waits for the kernel ahead of it.
//   products   As in the mma.sync kernel of attention_mma.cu: S^T = K Q^T has a warp's 16 keys as rows and the
//              query heads of the group as columns, O^T = V^T P^T has 16 head dimensions as rows.
//   softmax    float32; the running maximum is a whole number of binary orders (see attention_mma.cu), so the
//              rounded weights do not depend on how the list was cut.
//   joining    The four warps of a block add up their results of a pair in shared memory, one warp per head.  A run
//              that ends inside a (sequence, key/value head) pair leaves that as a partial result per head
//              (accumulators, maximum, sum) and takes a ticket at the head's counter; the warp that finds it took
//              the last ticket adds the head's partials up and writes the output.  A warp looks at its ticket only
//              when it next comes to a pair's end, so the counter's answer is never waited for.  Counters are
//              zero before and after a launch.
//
// Every wait on an mbarrier is bounded; when one runs out the thread records an error
// (llg_attn_decode_tma_status), raises a flag that ends the other waits of the block, the copying lane waits
// (bounded again) for its copies in flight, and the block returns.  The tensor maps cover this GPU's own
// page pool; no load uses cluster multicast.
//
// The reference's kernel for the same step runs one block per query head and re-reads the keys for every head of
// a group (Daisi.Llogos.Cuda/kernels/composite_ops.cu:275-387).
#include "common.cuh"
#include "kernel_args.h"

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int TK = 64;                       // keys per tile = one cache page
constexpr int WORK_WARPS = 4;                // each takes 16 keys of every tile
constexpr int THREADS = (WORK_WARPS + 1) * 32;
constexpr int MAX_SEQS = 1024;               // sequences whose tile counts fit the plan in shared memory
constexpr int STAGED_SEQS = 256;             // sequences whose length and slot are kept in shared memory beside the plan
constexpr int GH = 8;                        // query heads per key/value head, at most (one MMA n-tile)
constexpr int MERGE_HEADS = 4;               // heads whose four warp results are added up in shared memory at a time
constexpr int PART_PAD = 4;                  // a partial result is [head size] sums, the maximum, the sum of weights, and 2 unused: rows stay 16-byte aligned
constexpr int BLOCKS_PER_SM = 2;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
constexpr float LOG2E = 1.4426950408889634f;

__device__ int g_error = 0;   // 0 ok; waits that ran out: 1 tile landed, 2 stage free, 3 copies at the end; 4 shared memory not aligned

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = now_ns();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 1023) == 0) {
      if (*abort_flag) return false;
      if (now_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
  }
  return true;
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// x: first element of the box along the head dimension (0 or 64: a multiple of 8 elements, 16 bytes), y: first row
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
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
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^d for a whole number d <= 0 (or -inf), exactly
__device__ __forceinline__ float pow2_whole(float d) {
  return d < -126.f ? 0.f : __int_as_float((127 + (int)d) << 23);
}

// 64-key tiles that a sequence of `len` keys reads, and the first of them
__device__ __forceinline__ int first_tile(int len, int window) { return (window > 0 ? max(0, len - window) : 0) / TK; }
__device__ __forceinline__ int tile_count(int len, int window) { return (len + TK - 1) / TK - first_tile(len, window); }

// Where a block's run of the unit list starts: sequence, key/value head, tile within the sequence's tiles.
struct Cursor {
  int b, kvh, t, tiles;       // tiles: tile count of sequence b
};

__device__ __forceinline__ Cursor locate(const int* cum, int n_seqs, int nkv, long long u) {
  int lo = 0, hi = n_seqs - 1;                     // last b with nkv * cum[b] <= u
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((long long)nkv * cum[mid] <= u) lo = mid;
    else hi = mid - 1;
  }
  Cursor c;
  c.b = lo;
  c.tiles = cum[lo + 1] - cum[lo];
  const int r = (int)(u - (long long)nkv * cum[lo]);
  c.kvh = r / c.tiles;
  c.t = r - c.kvh * c.tiles;
  return c;
}

template <int HD, int STAGES>
__global__ void __launch_bounds__(THREADS, BLOCKS_PER_SM)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, DecodeTmaArgs a) {
  constexpr int KB = HD / 64;                  // 64-wide blocks of the head dimension
  constexpr int TILE_BYTES = KB * TK * 128;    // keys (or values) of one tile: [KB][64 positions][128 bytes]
  constexpr int KSTEPS = HD / 16;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* Ks = smem;                            // [STAGES][TILE_BYTES]
  unsigned char* Vs = smem + STAGES * TILE_BYTES;      // [STAGES][TILE_BYTES]
  __shared__ uint64_t full[STAGES], empty[STAGES];
  __shared__ uint64_t work_bar;                        // the working warps meet here: a wait with a limit, unlike a block barrier
  __shared__ int cum[MAX_SEQS + 1];                    // tiles of the sequences before b
  __shared__ int seq_len[STAGED_SEQS], seq_slot[STAGED_SEQS];      // fetched with the plan: the page look-ups start a trip to L2 earlier
  __shared__ int warp_total[THREADS / 32];
  __shared__ int abort_flag;
  __shared__ float merge[WORK_WARPS][MERGE_HEADS][HD + 2];      // the warps' results of up to four heads of a pair

  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) LLG_STAMP(2, 0, 0, blockIdx.x);
  if (tid == WORK_WARPS * 32) {                        // the copying warp's first lane: fetch the tensor maps early
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if ((smem_u32(smem) & 1023u) != 0) {                 // uniform over the block
    if (tid == 0) atomicCAS(&g_error, 0, 4);
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], WORK_WARPS);
    }
    mbar_init(&work_bar, WORK_WARPS * 32);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // ---- the plan: tiles per sequence, summed up.  Lengths, slots and page tables were written before this step's
  // first kernel started, so none of this waits for the kernel ahead. ----
  {
    const int per = (a.n_seqs + THREADS - 1) / THREADS;
    const int b0 = tid * per, b1 = min(a.n_seqs, b0 + per);
    int mine = 0;
    for (int b = b0; b < b1; ++b) {
      const int len = a.len_before[b] + 1;
      if (b < STAGED_SEQS) {
        seq_len[b] = len;
        seq_slot[b] = a.slots[b];
      }
      mine += tile_count(len, a.window);
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_total[warp] = incl;
    __syncthreads();
    int before = incl - mine;
    for (int w = 0; w < warp; ++w) before += warp_total[w];
    if (tid == 0) cum[0] = 0;
    for (int b = b0; b < b1; ++b) {
      before += tile_count(a.len_before[b] + 1, a.window);
      cum[b + 1] = before;
    }
    __syncthreads();
  }
  const int G = a.nh / a.nkv;
  const long long units = (long long)a.nkv * cum[a.n_seqs];
  const long long chunk = (units + gridDim.x - 1) / gridDim.x;
  const long long u0 = (long long)blockIdx.x * chunk, u1 = min(units, u0 + chunk);
  if (u0 >= u1) return;
  volatile int* abortp = &abort_flag;
  Cursor cur = locate(cum, a.n_seqs, a.nkv, u0);
  const int n_units = (int)(u1 - u0);

  if (warp == WORK_WARPS) {
    // ---- copies.  The lanes look up the pages of 32 tiles side by side (one trip to the page table instead of
    // 32 in a row); then each lane in turn waits for its tile's stage and issues the tile's boxes. ----
    int issued = 0;
    bool fine = true;
    for (int base = 0; base < n_units && fine; base += 32) {
      const int idx = base + lane;
      int row = 0, kvh = 0;
      bool newest = false;
      if (idx < n_units) {
        const Cursor c = locate(cum, a.n_seqs, a.nkv, u0 + idx);
        const bool staged = c.b < STAGED_SEQS;
        const int len = staged ? seq_len[c.b] : a.len_before[c.b] + 1;
        const int tile = first_tile(len, a.window) + c.t;
        newest = tile == (len - 1) / TK;                 // the kernel ahead writes the newest position only
        const int page = a.page_table[(long long)(staged ? seq_slot[c.b] : a.slots[c.b]) * a.table_width + tile % a.ring_pages];
        kvh = c.kvh;
        row = (page * a.nkv + kvh) * TK;
      }
      const int n_here = min(32, n_units - base);
      for (int k = 0; k < n_here && fine; ++k) {
        if (lane == k) {
          const int i = base + k, stage = i % STAGES;
          if (i >= STAGES && !mbar_wait(&empty[stage], ((i / STAGES) - 1) & 1, abortp)) {
            if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 2); }
            fine = false;
          } else {
            if (newest) pdl_wait();
            mbar_expect_tx(&full[stage], 2 * TILE_BYTES);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
              tma_load_2d(smem_u32(Ks + stage * TILE_BYTES + kb * (TK * 128)), &map_k, kb * 64, row, &full[stage]);
              tma_load_2d(smem_u32(Vs + stage * TILE_BYTES + kb * (TK * 128)), &map_v, kb * 64, row, &full[stage]);
            }
          }
        }
        fine = __shfl_sync(0xffffffffu, (int)fine, k) != 0;
        if (fine) ++issued;
      }
    }
    // nothing of this block may be in flight when it ends: the last copies of every stage have landed
    if (lane == 0) {
      for (int i = max(0, issued - STAGES); i < issued; ++i) {
        if (!mbar_wait(&full[i % STAGES], (i / STAGES) & 1, abortp) && !*abortp) {
          *abortp = 1;
          atomicCAS(&g_error, 0, 3);
        }
      }
    }
    return;
  }

  // ---- the working warps ------------------------------------------------------------------------------
  const int g = lane >> 2, t4 = lane & 3;
  const float sc = a.scale * LOG2E;
  const bf16* qg = (const bf16*)a.q;
  bf16* out = (bf16*)a.out;
  pdl_wait();                                           // the queries come from the kernel ahead
  if (tid == 0) LLG_STAMP(2, 1, 0, blockIdx.x);
  // a ticket this warp has taken at a head's counter and not looked at yet
  bool pending = false;
  int pend_ticket = 0, pend_parts = 0;
  const float* pend_base = nullptr;
  long long pend_row = 0;
  const long long part_stride = (long long)(a.nh / a.nkv) * (HD + PART_PAD);     // from one block's partial of a head to the next block's
  // If the pending ticket was the last of its head, this warp adds up the head's partials (their weights 2^(m - M)
  // are exact powers of two) and writes the head's output; it leaves the counter at zero.
  auto join_if_last = [&]() {
    pending = false;
    const int ticket = __shfl_sync(0xffffffffu, pend_ticket, 0);
    if (ticket != pend_parts - 1) return;
    if (lane == 0) a.counters[pend_row] = 0;
    __threadfence();
    // A lane sums four neighbouring head dimensions (one 16-byte load per partial; lanes beyond the head's size idle),
    // eight partials' loads in flight at a time.  The largest maximum is found on the way: when a batch raises it, what
    // has been summed is scaled down by the difference, an exact power of two, so the sums are those of one pass
    // against the final maximum, bit for bit, without a pass of their own to find it.
    constexpr int LANES = HD / 4;
    float M = -INFINITY, L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool live = lane < LANES;
    for (int s0 = 0; s0 < pend_parts; s0 += 8) {
      float ms[8], ls[8];
      float4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const bool there = s0 + k < pend_parts;
        const float* row = pend_base + (long long)(there ? s0 + k : 0) * part_stride;
        const float2 ml = there ? __ldcg(reinterpret_cast<const float2*>(row + HD)) : make_float2(-INFINITY, 0.f);
        ms[k] = ml.x;
        ls[k] = ml.y;
        v[k] = (there && live) ? __ldcg(reinterpret_cast<const float4*>(row) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float mb = ms[0];
#pragma unroll
      for (int k = 1; k < 8; ++k) mb = fmaxf(mb, ms[k]);
      if (mb > M) {
        const float r = (M == -INFINITY) ? 0.f : pow2_whole(M - mb);
        L *= r;
        acc.x *= r;
        acc.y *= r;
        acc.z *= r;
        acc.w *= r;
        M = mb;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float w = (ms[k] == -INFINITY) ? 0.f : pow2_whole(ms[k] - M);
        L += w * ls[k];
        acc.x += w * v[k].x;
        acc.y += w * v[k].y;
        acc.z += w * v[k].z;
        acc.w += w * v[k].w;
      }
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    if (live) {
      uint2 packed;
      packed.x = pack_bf16(acc.x * inv, acc.y * inv);
      packed.y = pack_bf16(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(out + pend_row * HD + 4 * lane) = packed;
    }
  };
  int i = 0;                                            // tiles consumed so far
  bool ok = true;
  // The working warps' own meeting point (the copying warp does not take part).  A warp whose wait for a tile ran out
  // never comes here; the others then leave after their limit, or at once when they see the block's flag.
  uint32_t work_phase = 0;
  auto work_sync = [&]() -> bool {
    mbar_arrive(&work_bar);
    const bool met = mbar_wait(&work_bar, work_phase & 1, abortp);
    ++work_phase;
    if (!met && !*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 1); }
    return met;
  };
  long long u = u0;
  while (u < u1 && ok) {
    const int b = cur.b, kvh = cur.kvh;
    const int n_seg = min(cur.tiles - cur.t, (int)(u1 - u));
    const int len = a.len_before[b] + 1;
    const int lo = a.window > 0 ? max(0, len - a.window) : 0;
    const int t_first = lo / TK;
    // Q^T as the second operand: column g is head g of the group, rows are head dimensions
    uint32_t qf[KSTEPS][2];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        uint32_t v = 0;
        if (g < G) v = *reinterpret_cast<const uint32_t*>(qg + ((long long)b * a.nh + kvh * G + g) * HD + ks * 16 + 2 * t4 + e * 8);
        qf[ks][e] = v;
      }
    }
    float o[KSTEPS][4];          // O^T: rows = 16 head dimensions per tile, columns = heads 2 t4, 2 t4 + 1
#pragma unroll
    for (int j = 0; j < KSTEPS; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};      // per column (head 2 t4, 2 t4 + 1)

    for (int j = 0; j < n_seg; ++j, ++i) {
      const int stage = i % STAGES;
      if (!mbar_wait(&full[stage], (i / STAGES) & 1, abortp)) {
        if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 1); }
        ok = false;
        break;
      }
      const uint32_t kd = smem_u32(Ks + stage * TILE_BYTES), vd = smem_u32(Vs + stage * TILE_BYTES);
      const int kt = (t_first + cur.t + j) * TK + warp * 16;      // this warp's 16 keys of the page

      // S^T = K Q^T, two accumulators so that the chain of dependent MMAs is half as long
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      const int krow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t ka[4];
        const int chunk = (lane >> 4) + 2 * ks;             // 16-byte chunk of the head's row
        ldmatrix_x4(ka, kd + (chunk >> 3) * (TK * 128) + krow * 128 + (((chunk & 7) ^ (krow & 7)) << 4));
        if (ks & 1) mma_16816(s1, ka, qf[ks][0], qf[ks][1]);
        else mma_16816(s0, ka, qf[ks][0], qf[ks][1]);
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
        for (int jj = 0; jj < KSTEPS; ++jj) {
          o[jj][0] *= corr[0];
          o[jj][1] *= corr[1];
          o[jj][2] *= corr[0];
          o[jj][3] *= corr[1];
        }
      }
      // P^T in the layout of the second operand: transpose the two 8x8 blocks of S^T
      const uint32_t pb0 = movmatrix_trans(pack_bf16(pv[0], pv[1]));
      const uint32_t pb1 = movmatrix_trans(pack_bf16(pv[2], pv[3]));
      // O^T += V^T P^T, 16 head dimensions per MMA
      const int vrow = warp * 16 + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
      for (int jj = 0; jj < KSTEPS; ++jj) {
        uint32_t va[4];
        const int chunk = ((lane >> 3) & 1) + 2 * jj;
        ldmatrix_x4_trans(va, vd + (chunk >> 3) * (TK * 128) + vrow * 128 + (((chunk & 7) ^ (vrow & 7)) << 4));
        mma_16816(o[jj], va, pb0, pb1);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
    }
    if (!ok) break;

    // ---- the block's result of the pair.  The four warps' results are added up in shared memory, four heads at a
    // time, warp w taking head h0 + w.  A pair that lies in this block alone is finished there.  Otherwise the warp
    // writes its head's partial result and takes a ticket at the head's counter; it reads the ticket only when it
    // next comes to a pair's end (or to its own end), so that nobody waits for the counter's answer, and if the
    // ticket was the last one, the warp joins that head's partials alone. ----
    const int pair = b * a.nkv + kvh;
    const long long p_first = (long long)a.nkv * cum[b] + (long long)kvh * cur.tiles;      // the pair's first unit
    const int blk_first = (int)(p_first / chunk), blk_last = (int)((p_first + cur.tiles - 1) / chunk);
    const bool whole = blk_first == blk_last;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      l[c] += __shfl_xor_sync(0xffffffffu, l[c], 4);
      l[c] += __shfl_xor_sync(0xffffffffu, l[c], 8);
      l[c] += __shfl_xor_sync(0xffffffffu, l[c], 16);
    }
    for (int h0 = 0; h0 < G; h0 += MERGE_HEADS) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int head = 2 * t4 + c - h0;
        if (head >= 0 && head < MERGE_HEADS) {
          float* dst = merge[warp][head];
#pragma unroll
          for (int jj = 0; jj < KSTEPS; ++jj) {
            dst[jj * 16 + g] = o[jj][c];
            dst[jj * 16 + g + 8] = o[jj][2 + c];
          }
          if (g == 0) {
            dst[HD] = m[c];
            dst[HD + 1] = l[c];
          }
        }
      }
      if (!work_sync()) { ok = false; break; }
      const int head = h0 + warp;                       // one warp per head
      if (head < G) {
        float mw[WORK_WARPS], M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WORK_WARPS; ++w) {
          mw[w] = merge[w][warp][HD];
          M = fmaxf(M, mw[w]);
        }
        float L = 0.f, scw[WORK_WARPS];
#pragma unroll
        for (int w = 0; w < WORK_WARPS; ++w) {
          scw[w] = (mw[w] == -INFINITY) ? 0.f : pow2_whole(mw[w] - M);
          L += scw[w] * merge[w][warp][HD + 1];
        }
        float acc[HD / 32];
#pragma unroll
        for (int dd = 0; dd < HD / 32; ++dd) {
          acc[dd] = 0.f;
#pragma unroll
          for (int w = 0; w < WORK_WARPS; ++w) acc[dd] += scw[w] * merge[w][warp][lane + 32 * dd];
        }
        const long long head_row = (long long)b * a.nh + kvh * G + head;
        if (whole) {
          const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
          for (int dd = 0; dd < HD / 32; ++dd) out[head_row * HD + lane + 32 * dd] = __float2bfloat16_rn(acc[dd] * inv);
        } else {
          if (pending) join_if_last();                  // a ticket of an earlier pair (or of this pair's head h0 - 4)
          float* mine = a.part + ((long long)(blockIdx.x + pair) * G + head) * (HD + PART_PAD);
#pragma unroll
          for (int dd = 0; dd < HD / 32; ++dd) mine[lane + 32 * dd] = acc[dd];
          if (lane == 0) {
            mine[HD] = M;
            mine[HD + 1] = L;
          }
          __threadfence();               // this warp's partial is visible to the whole device ...
          __syncwarp();
          if (lane == 0) pend_ticket = atomicAdd(&a.counters[head_row], 1);     // ... before its ticket is
          pending = true;
          pend_base = a.part + ((long long)(blk_first + pair) * G + head) * (HD + PART_PAD);
          pend_parts = blk_last - blk_first + 1;
          pend_row = head_row;
        }
      }
      if (!work_sync()) { ok = false; break; }          // the merge area is free for the next four heads
    }
    if (!ok) break;
    u += n_seg;
    cur.t += n_seg;
    if (cur.t == cur.tiles) {
      cur.t = 0;
      if (++cur.kvh == a.nkv) {
        cur.kvh = 0;
        ++cur.b;
        if (cur.b < a.n_seqs) cur.tiles = cum[cur.b + 1] - cum[cur.b];
      }
    }
  }
  if (pending && ok) join_if_last();
  if (tid == 0) LLG_STAMP(2, 3, 0, blockIdx.x);
}

// ---- host side ---------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// Boxes of 64 rows x 64 head dimensions (128 bytes, swizzled) out of the pages seen as [pages x kv heads x 64][hd].
bool page_map(const void* base, long long rows, int hd, CUtensorMap* result) {
  static std::map<std::tuple<const void*, long long, int>, CUtensorMap> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple(base, rows, hd);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *result = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  CUtensorMap m;
  cuuint32_t estr[2] = {1, 1};
  cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)TK};
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *result = m;
  return true;
}

// Blocks of a launch.  As many as the GPU holds at once (two per multiprocessor) while that leaves a block fewer than
// about a hundred tiles.  With more work per block, more and shorter blocks: the multiprocessors do not stream at the
// same rate (the time from the first block's end to the last's was a sixth of the kernel with one run per place), and
// blocks that start as places come free even that out; a block's start costs a few microseconds, so it has to be worth
// some fifty tiles.
int grid_blocks(int n_seqs, int nkv, int max_len) {
  const long long resident = (long long)BLOCKS_PER_SM * llg_sm_count();
  const long long units = (long long)n_seqs * nkv * ((max_len + TK - 1) / TK);
  long long rounds = units / (resident * 48);
  rounds = rounds < 1 ? 1 : (rounds > 4 ? 4 : rounds);
  const long long most = resident * rounds;
  return (int)(units < most ? (units < 1 ? 1 : units) : most);
}

template <int HD, int STAGES>
int launch(const DecodeTmaArgs& a, const CUtensorMap& mk, const CUtensorMap& mv, int blocks, cudaStream_t stream) {
  constexpr int smem = 2 * STAGES * (HD / 64) * TK * 128;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<HD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return llg_fail("attn_decode_tma: shared memory %d: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  cudaError_t le = llg_launch(attn_decode_tma_kernel<HD, STAGES>, dim3(blocks), dim3(THREADS), (size_t)smem, stream, mk, mv, a);
  if (le != cudaSuccess) return llg_fail("attn_decode_tma: launch: %s", cudaGetErrorString(le));
  return llg_check_launch("attn_decode_tma");
}

}  // namespace

// 1 when this kernel takes the geometry (bfloat16 only): head size 64 or 128, at most 8 query heads per key/value
// head, at most 1024 sequences.
LLG_API int llg_attn_decode_tma_supported(int hd, int nh, int nkv, int n_seqs) {
  return (hd == 64 || hd == 128) && nkv > 0 && nh % nkv == 0 && nh / nkv <= GH && n_seqs <= MAX_SEQS;
}

// Floats of scratch for the partial results of a launch over sequences of up to `max_len` keys.
LLG_API long long llg_attn_decode_tma_scratch_floats(int n_seqs, int nh, int nkv, int hd, int max_len) {
  const long long slots = (long long)grid_blocks(n_seqs, nkv, max_len) + (long long)n_seqs * nkv;
  return slots * (nh / nkv) * (hd + PART_PAD);
}

// `max_len`: an upper bound of len_before + 1 over the batch (it sizes the grid and was given to
// llg_attn_decode_tma_scratch_floats); n_pages: pages of k_pages / v_pages.
LLG_API int llg_attn_decode_tma(const DecodeTmaArgs* args, const void* k_pages, const void* v_pages, int n_pages, int max_len,
                                cudaStream_t stream) {
  const DecodeTmaArgs& a = *args;
  LLG_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "attn_decode_tma: %d heads are no multiple of %d key/value heads",
              a.nh, a.nkv);
  LLG_REQUIRE(llg_attn_decode_tma_supported(a.hd, a.nh, a.nkv, a.n_seqs),
              "attn_decode_tma: head_dim %d (64 or 128), %d heads per key/value head (at most %d) or %d sequences (at most %d) "
              "is outside what this kernel takes", a.hd, a.nh / a.nkv, GH, a.n_seqs, MAX_SEQS);
  LLG_REQUIRE(a.window >= 0 && a.ring_pages > 0 && a.table_width >= a.ring_pages, "attn_decode_tma: bad cache geometry");
  LLG_REQUIRE(a.scale > 0.f, "attn_decode_tma: the softmax scale must be positive");
  LLG_REQUIRE(a.counters != nullptr && a.part != nullptr, "attn_decode_tma: needs scratch and n_seqs * nh zeroed counters");
  LLG_REQUIRE(n_pages > 0 && max_len > 0, "attn_decode_tma: needs the number of pages and a bound on the lengths");
  LLG_REQUIRE(((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0, "attn_decode_tma: pages must be 16-byte aligned");
  LLG_REQUIRE((long long)n_pages * a.nkv * TK < 2147483647LL, "attn_decode_tma: too many page rows for a tensor map coordinate");
  if (a.n_seqs <= 0) return 0;
  CUtensorMap mk, mv;
  const long long rows = (long long)n_pages * a.nkv * TK;
  if (!page_map(k_pages, rows, a.hd, &mk) || !page_map(v_pages, rows, a.hd, &mv))
    return llg_fail("attn_decode_tma: cuTensorMapEncodeTiled failed or is not available");
  const int blocks = grid_blocks(a.n_seqs, a.nkv, max_len);
  return a.hd == 64 ? launch<64, 6>(a, mk, mv, blocks, stream) : launch<128, 3>(a, mk, mv, blocks, stream);
}

// Error code recorded when a wait ran out (0 = none); clears it.  Synchronises the device.
LLG_API int llg_attn_decode_tma_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_error, &zero, sizeof(int));
  return v;
}

// Causal attention for prompt steps on the 5th-generation tensor cores (tcgen05), bfloat16, head
// sizes 64 and 128.
//
//   per 64-key tile (one cache page):   S = Q K^T      tcgen05.mma, accumulator S[128 x 64] in TMEM
//                                       each thread reads its row of S (tcgen05.ld), masks, updates the
//                                       running maximum and sum, writes P (bfloat16) over S (tcgen05.st)
//                                       O += P V       tcgen05.mma, P from TMEM, accumulator O[128 x head] in TMEM
//
// A block owns 256 queries of one head as two tiles of 128.  Each tile has a group of four softmax
// warps: thread r of a group owns query row r of its tile, which is lane r of tensor memory, so the
// softmax of a row needs no exchange between threads.  Three more warps serve both groups: one lane
// issues every product, one warp copies the key tiles and one the value tiles (TMA boxes from the
// step's packed buffer or from a cache page; the one tile per sequence that lies partly in each row by
// row with cp.async; three stages each).
// The roles meet only at mbarriers: tiles full / free between the copying warps and the issuing lane,
// scores ready, weights ready and accumulator updated between the issuing lane and a group.  Each
// group has two score buffers in tensor memory, so that the tensor core computes the next tile's
// scores and the previous tile's O += P V while the group runs the softmax of the current one; the
// scores of tile j + 1 are issued when O += P(j-1) V(j-1) has finished with the buffer they go into.
//
// Q and K are K-major operands in shared memory with the 128-byte swizzle; V is stored as it lies in
// memory ([key][dim], dim contiguous), which makes it the MN-major second operand of the second product;
// P never leaves tensor memory (the products' operand fetch from shared memory is what bounds this
// kernel, and P would be a third of it).
// A row's accumulator is rescaled in place (tcgen05.ld / tcgen05.st) only when its maximum grows by
// more than a factor of 2^8 in the weights, warp by warp and only when some row of the warp needs it.
//
// Every mbarrier wait is bounded; on expiry the thread records an error (llg_attn_tc_status) and
// raises a flag that ends the other roles' waits; every role waits for its own copies in flight,
// and the block frees its tensor memory and returns.
#include "common.cuh"
#include "kernel_args.h"

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int BQ = 128;      // queries per tile (rows of a product, lanes of tensor memory)
constexpr int TK = 64;       // keys per tile = one cache page
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
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

// the largest of three (one instruction on sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ int g_error = 0;  // 0 ok; waits that ran out: 1 scores, 2 accumulator, 4 free stage, 5 tile copied, 6 weights, 7 copies at the end; 3 shared memory not aligned to 1024 bytes

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

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// shared memory written by threads (cp.async, st.shared) becomes visible to the tensor core's reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major operand, rows of 128 bytes with the 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand: 64 elements of the MN dimension are contiguous (one swizzled 128-byte row per k),
// 8-k groups 1024 bytes apart, the next 64 MN elements `lbo_bytes` further
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo_bytes) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// first operand from tensor memory (lane = row, one 32-bit column per two k), second from shared memory
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// true in one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` in a tile of 128-byte rows with the 128-byte swizzle
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

constexpr int GROUPS = 2;                     // query tiles of 128 rows per block, each with its own softmax warps
constexpr int KST = 3, VST = 3;               // stages of keys and of values
constexpr int WORKERS = GROUPS * BQ;          // softmax threads: thread r of group g owns query row r of tile g
constexpr int ISSUE_WARP = WORKERS / 32;      // one lane of this warp issues every product
constexpr int K_LOAD_WARP = ISSUE_WARP + 1;   // copies key tiles
constexpr int V_LOAD_WARP = ISSUE_WARP + 2;   // copies value tiles
constexpr int THREADS = (V_LOAD_WARP + 1) * 32;

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// What a block knows about its two query tiles and the key tiles they need.
struct TileInfo {
  int b, tok0, lb, slot, k_begin;
  int nq[GROUPS], pos0[GROUPS], n_tiles[GROUPS], n_max;
};

template <int HD>
__global__ void __launch_bounds__(384, 1) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k_pages,
                                                                 const __grid_constant__ CUtensorMap map_v_pages,
                                                                 const __grid_constant__ CUtensorMap map_k_new,
                                                                 const __grid_constant__ CUtensorMap map_v_new, PrefillArgs a) {
  constexpr int KB = HD / 64;                 // 64-wide blocks of the head dimension
  constexpr int Q_BYTES = KB * BQ * 128;      // [KB][128 rows][128 bytes]
  constexpr int KV_BYTES = KB * TK * 128;     // [KB][64 keys][128 bytes]
  constexpr int TMEM_COLS = 512;              // per group 256: S 2 x 64 columns, O HD columns from column 128
  constexpr uint32_t G_COLS = 256, O_COL = 128;
  constexpr int CPR = HD / 8;                 // 16-byte chunks per row of the head
  // The tiles need 1024-byte alignment (swizzle); the declaration asks for it and the kernel checks it.
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* Qs = smem;                          // [GROUPS]
  unsigned char* Ks = Qs + GROUPS * Q_BYTES;         // [KST]
  unsigned char* Vs = Ks + KST * KV_BYTES;           // [VST]
  __shared__ uint64_t k_full[KST], k_free[KST], v_full[VST], v_free[VST];
  __shared__ uint64_t s_full[GROUPS][2], p_ready[GROUPS][2], o_done[GROUPS], q_ready;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) LLG_STAMP(5, 0, 0, blockIdx.x + gridDim.x * blockIdx.y);
  if ((smem_u32(smem) & 1023u) != 0) {          // uniform over the block
    if (tid == 0) atomicCAS(&g_error, 0, 3);
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < KST; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_free[s], 1);
    }
    for (int s = 0; s < VST; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_free[s], 1);
    }
    for (int g = 0; g < GROUPS; ++g) {
      mbar_init(&s_full[g][0], 1);
      mbar_init(&s_full[g][1], 1);
      mbar_init(&p_ready[g][0], BQ);
      mbar_init(&p_ready[g][1], BQ);
      mbar_init(&o_done[g], 1);
    }
    mbar_init(&q_ready, WORKERS);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_slot;
  volatile int* abortp = &abort_flag;
  pdl_wait();
  if (tid == 0) LLG_STAMP(5, 1, 0, blockIdx.x + gridDim.x * blockIdx.y);

  // Blocks start in the order of blockIdx.x, then blockIdx.y: all heads of the list's first tile, then all
  // heads of its second ...  The caller lists the tiles with the most keys first, so that the long blocks
  // start first and the short ones fill the gaps at the end.
  TileInfo ti;
  {
    const int tile_id = (int)blockIdx.y;
    ti.b = a.tiles[2 * tile_id];
    const int q_off = a.tiles[2 * tile_id + 1];
    ti.tok0 = a.cu_tokens[ti.b];
    const int total = a.cu_tokens[ti.b + 1] - ti.tok0;
    ti.lb = a.len_before[ti.b];
    ti.slot = a.slots[ti.b];
    ti.n_max = 0;
    for (int g = 0; g < GROUPS; ++g) {
      ti.nq[g] = max(0, min(BQ, total - q_off - g * BQ));
      ti.pos0[g] = ti.lb + q_off + g * BQ;
    }
    // the first group's window starts earliest; the second masks the tiles that lie before its own
    int kb = a.window > 0 ? max(0, ti.pos0[0] - a.window + 1) : 0;
    ti.k_begin = (kb / TK) * TK;
    for (int g = 0; g < GROUPS; ++g) {
      ti.n_tiles[g] = ti.nq[g] > 0 ? (ti.pos0[g] + ti.nq[g] - ti.k_begin + TK - 1) / TK : 0;
      ti.n_max = max(ti.n_max, ti.n_tiles[g]);
    }
  }
  const int h = blockIdx.x, kvh = h / (a.nh / a.nkv);
  const int k_end = ti.pos0[0] + (ti.nq[1] > 0 ? BQ + ti.nq[1] : ti.nq[0]);   // keys past it are never copied
  const int q_tok0 = ti.tok0 + ti.pos0[0] - ti.lb;                              // first token of the first query tile

  // queries: thread r of group g copies its part of tile g; the issuing lane waits for all of them,
  // the copying warps start on the keys and values meanwhile
  if (tid < WORKERS) {
    const int g = tid / BQ, r = tid % BQ;
    const int ch = r % CPR;
    for (int row = r / CPR; row < BQ; row += BQ / CPR) {
      const bool valid = row < ti.nq[g];
      const bf16* src = (const bf16*)a.q + ((long long)(q_tok0 + g * BQ + (valid ? row : 0)) * a.nh + h) * HD + ch * 8;
      cp_async16(smem_u32(Qs + g * Q_BYTES) + (uint32_t)((ch >> 3) * (BQ * 128)) + swz(row, ch & 7), src, valid);
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_async_smem();
    mbar_arrive(&q_ready);
  }

  if (warp == K_LOAD_WARP || warp == V_LOAD_WARP) {
    // ---- copies: one warp per operand.  A tile that lies in one cache page, or in this step's packed rows,
    // is two TMA boxes (64 keys x 64 dimensions, 128-byte swizzle) that one lane requests; the one tile per
    // sequence that lies partly in each is copied row by row with cp.async by the whole warp. ------------
    const bool keys = warp == K_LOAD_WARP;
    const int stages = keys ? KST : VST;
    unsigned char* base = keys ? Ks : Vs;
    uint64_t* full = keys ? k_full : v_full;
    uint64_t* freeb = keys ? k_free : v_free;
    const CUtensorMap* map_pages = keys ? &map_k_pages : &map_v_pages;
    const CUtensorMap* map_new = keys ? &map_k_new : &map_v_new;
    const bf16* fresh_src = (const bf16*)(keys ? a.k_new : a.v_new);
    const bf16* page_src = (const bf16*)(keys ? a.k_pages : a.v_pages);
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(map_pages) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(map_new) : "memory");
    }
    const int ch = lane % CPR;
    constexpr int RSTEP = 32 / CPR;
    int requested = 0;                          // tiles whose copies have been requested
    for (int t = 0; t < ti.n_max; ++t) {
      const int st = t % stages;
      if (t >= stages && !mbar_wait(&freeb[st], (t / stages - 1) & 1, abortp)) {
        if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 4); }
        break;
      }
      requested = t + 1;
      const int kt = ti.k_begin + t * TK;
      const uint32_t dst = smem_u32(base + st * KV_BYTES);
      if (kt >= ti.lb) {
        // rows past the sequence's last token are another sequence's, or zeros past the buffer: no query sees them
        if (lane == 0) {
          mbar_expect_tx(&full[st], KV_BYTES);
#pragma unroll
          for (int blk = 0; blk < KB; ++blk)
            tma_load_3d(dst + blk * (TK * 128), map_new, blk * 64, kvh, ti.tok0 + kt - ti.lb, &full[st]);
        }
      } else if (kt + TK <= ti.lb) {
        if (lane == 0) {
          const int row0 = (int)kv_row(a.page_table, a.table_width, a.ring_pages, ti.slot, kt, kvh, a.nkv);
          mbar_expect_tx(&full[st], KV_BYTES);
#pragma unroll
          for (int blk = 0; blk < KB; ++blk) tma_load_2d(dst + blk * (TK * 128), map_pages, blk * 64, row0, &full[st]);
        }
      } else {
        const long long old_base = kv_row(a.page_table, a.table_width, a.ring_pages, ti.slot, kt, kvh, a.nkv) * HD;
        const long long new_base = ((long long)(ti.tok0 + kt - ti.lb) * a.nkv + kvh) * HD;
        for (int row = lane / CPR; row < TK; row += RSTEP) {
          const int pos = kt + row;
          const bool valid = pos < k_end, fresh = pos >= ti.lb;
          const long long off = (fresh ? new_base + (long long)row * a.nkv * HD : old_base + (long long)row * HD) + ch * 8;
          cp_async16(dst + (uint32_t)((ch >> 3) * (TK * 128)) + swz(row, ch & 7), (fresh ? fresh_src : page_src) + (valid ? off : 0),
                     valid);
        }
        cp_async_commit();
        cp_async_wait<0>();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[st]);
      }
      __syncwarp();
    }
    // Copies still write into this block's shared memory until their barrier completes: before the block
    // may end, see the last tile of every stage arrive (at once, unless a wait ran out somewhere).
    if (lane == 0) {
      for (int t = max(0, requested - stages); t < requested; ++t) {
        const unsigned long long t0 = now_ns();
        while (!mbar_try_wait(&full[t % stages], (t / stages) & 1)) {
          if (now_ns() - t0 > WAIT_LIMIT_NS) { atomicCAS(&g_error, 0, 7); break; }
        }
      }
    }
  } else if (warp == ISSUE_WARP) {
    // ---- products: one lane issues them all.  The tensor core takes them one after the other, and a
    // lane that issues is held up while its queue is full, which is why no softmax warp does this. ------
    if (elect_one()) {
      constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TK >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
      constexpr uint32_t IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
      // scores of key tile t for group g into the group's score buffer t % 2
      auto issue_scores = [&](int g, int t) {
        const uint32_t qa = smem_u32(Qs + g * Q_BYTES), ka = smem_u32(Ks + (t % KST) * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t blk = ks >> 2, kk = ks & 3;      // 64-wide block, 16-wide step inside it (32 bytes)
          umma_bf16(tmem + g * G_COLS + (uint32_t)(t & 1) * TK, desc_kmajor(qa + blk * (BQ * 128) + kk * 32),
                    desc_kmajor(ka + blk * (TK * 128) + kk * 32), IDESC_S, ks != 0);
        }
        umma_commit(&s_full[g][t & 1]);
      };
      bool ok = true;
      auto wait_or_fail = [&](uint64_t* bar, uint32_t parity, int code) {
        if (!ok) return;
        if (!mbar_wait(bar, parity, abortp)) {
          if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, code); }
          ok = false;
        }
      };
      wait_or_fail(&q_ready, 0, 5);
      if (ok && ti.n_max > 0) {
        wait_or_fail(&k_full[0], 0, 5);
        if (ok) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          for (int g = 0; g < GROUPS; ++g)
            if (0 < ti.n_tiles[g]) issue_scores(g, 0);
          umma_commit(&k_free[0]);
        }
      }
      // Step j: the scores of tile j + 1 go into the buffer whose weights P(j-1) the product of step j - 1 has
      // read by now; then, once the group has turned S(j) into P(j) (written over S(j) in tensor memory),
      // O += P(j) V(j).
      for (int j = 0; j < ti.n_max && ok; ++j) {
        wait_or_fail(&v_full[j % VST], (j / VST) & 1, 5);
        if (j + 1 < ti.n_max) wait_or_fail(&k_full[(j + 1) % KST], ((j + 1) / KST) & 1, 5);
        for (int g = 0; g < GROUPS && ok; ++g) {
          if (j >= ti.n_tiles[g]) continue;
          if (j + 1 < ti.n_tiles[g]) {
            if (j >= 1) wait_or_fail(&o_done[g], (j - 1) & 1, 6);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_scores(g, j + 1);
          }
          wait_or_fail(&p_ready[g][j & 1], (j >> 1) & 1, 6);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t pa = tmem + g * G_COLS + (uint32_t)(j & 1) * TK, va = smem_u32(Vs + (j % VST) * KV_BYTES);
#pragma unroll
          for (int kk = 0; kk < TK / 16; ++kk) {
            // 16 keys further: 8 columns of packed weights, 16 rows (2048 bytes) down V
            umma_bf16_ts(tmem + g * G_COLS + O_COL, pa + kk * 8, desc_mnmajor(va + kk * 2048, TK * 128), IDESC_O, (j | kk) != 0);
          }
          umma_commit(&o_done[g]);
        }
        if (!ok) break;
        umma_commit(&v_free[j % VST]);
        if (j + 1 < ti.n_max) umma_commit(&k_free[(j + 1) % KST]);
      }
    }
  } else if (tid < WORKERS && ti.nq[tid / BQ] > 0) {
    // ---- softmax: thread r of group g owns query row r of tile g ------------------------------------
    const int g = tid / BQ, r = tid % BQ, gw = (tid % BQ) >> 5;       // gw: warp inside the group = its lane quarter
    const uint32_t lane_base = tmem + g * G_COLS + ((uint32_t)(gw * 32) << 16);
    const int n_tiles = ti.n_tiles[g], pos0 = ti.pos0[g];
    const float sc = a.scale * LOG2E;
    // A row's weights are 2^(x - M) with x = score * scale * log2 e and M a whole number that is raised (to the
    // tile's maximum, rounded up) only when a tile exceeds it by more than 8: the weights stay below 2^8 and the
    // accumulator is rescaled rarely, by an exact power of two.  The common factor cancels in the final division,
    // and rounding a weight to bfloat16 gives the same bits whatever M was: how the keys are cut into tiles or
    // steps does not show in the rounded weights.
    const float raise_by = 8.0f;
    const int qpos = pos0 + r;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(&s_full[g][j & 1], (j >> 1) & 1, abortp)) {
        if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 1); }
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int kt = ti.k_begin + j * TK;
      float sv[TK];
      {
        uint32_t r0_[16], r1_[16], r2_[16], r3_[16];
        const uint32_t sa = lane_base + (uint32_t)(j & 1) * TK;
        tmem_ld16(sa, r0_);
        tmem_ld16(sa + 16, r1_);
        tmem_ld16(sa + 32, r2_);
        tmem_ld16(sa + 48, r3_);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          sv[c] = __uint_as_float(r0_[c]);
          sv[16 + c] = __uint_as_float(r1_[c]);
          sv[32 + c] = __uint_as_float(r2_[c]);
          sv[48 + c] = __uint_as_float(r3_[c]);
        }
      }
      const bool need_mask = (kt + TK - 1 > pos0 + gw * 32) || (a.window > 0 && kt <= pos0 + gw * 32 + 31 - a.window);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < TK; ++c) {
          const int key = kt + c;
          const bool valid = key <= qpos && (a.window == 0 || key > qpos - a.window);
          sv[c] = valid ? sv[c] : -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < TK; c += 8) {
#pragma unroll
        for (int k = 0; k < 4; ++k) mx4[k] = max3(mx4[k], sv[c + 2 * k], sv[c + 2 * k + 1]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float mxs = mx * sc;
      const bool raise = mxs > m_run + raise_by || m_run == -INFINITY;
      const float m_new = raise ? fmaxf(m_run, ceilf(mxs)) : m_run;
      const float corr = (!raise || m_new == -INFINITY) ? 1.f : pow2_whole(m_run - m_new);
      const float ms = (m_new == -INFINITY) ? 0.f : m_new;
      m_run = m_new;
      // two elements per instruction where the arithmetic allows it (fma.rn.f32x2, add.rn.f32x2); the
      // weights go straight into the tile's P buffer, which the product of two tiles ago has left
      const float2 sc2 = make_float2(sc, sc), nms2 = make_float2(-ms, -ms);
      float2 ps2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      // P(j) takes the place of S(j) in tensor memory: 64 weights of a row in 32 columns
#pragma unroll
      for (int c16 = 0; c16 < TK / 32; ++c16) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float2 x = __ffma2_rn(make_float2(sv[c16 * 32 + 2 * e], sv[c16 * 32 + 2 * e + 1]), sc2, nms2);
          const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          ps2[e & 1] = __fadd2_rn(ps2[e & 1], p);
          pk[e] = pack_bf16(p.x, p.y);
        }
        tmem_st16(lane_base + (uint32_t)(j & 1) * TK + c16 * 16, pk);
      }
      l_run = l_run * corr + ((ps2[0].x + ps2[0].y) + (ps2[1].x + ps2[1].y));

      if (j > 0) {
        // O += P(j-1) V(j-1) has finished: the accumulator may be rescaled
        if (!mbar_wait(&o_done[g], (j - 1) & 1, abortp)) {
          if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 2); }
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 16) {
            uint32_t rr[16];
            tmem_ld16(lane_base + O_COL + c0, rr);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int c = 0; c < 16; ++c) rr[c] = __float_as_uint(__uint_as_float(rr[c]) * corr);
            tmem_st16(lane_base + O_COL + c0, rr);
          }
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&p_ready[g][j & 1]);
    }
    if (ok && !mbar_wait(&o_done[g], (n_tiles - 1) & 1, abortp)) {
      if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 2); }
      ok = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && !*abortp) {
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      bf16* dst = (bf16*)a.out + ((long long)(q_tok0 + g * BQ + r) * a.nh + h) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 16) {
        uint32_t rr[16];
        tmem_ld16(lane_base + O_COL + c0, rr);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (r < ti.nq[g]) {
          uint4 v0, v1;
          v0.x = pack_bf16(__uint_as_float(rr[0]) * inv, __uint_as_float(rr[1]) * inv);
          v0.y = pack_bf16(__uint_as_float(rr[2]) * inv, __uint_as_float(rr[3]) * inv);
          v0.z = pack_bf16(__uint_as_float(rr[4]) * inv, __uint_as_float(rr[5]) * inv);
          v0.w = pack_bf16(__uint_as_float(rr[6]) * inv, __uint_as_float(rr[7]) * inv);
          v1.x = pack_bf16(__uint_as_float(rr[8]) * inv, __uint_as_float(rr[9]) * inv);
          v1.y = pack_bf16(__uint_as_float(rr[10]) * inv, __uint_as_float(rr[11]) * inv);
          v1.z = pack_bf16(__uint_as_float(rr[12]) * inv, __uint_as_float(rr[13]) * inv);
          v1.w = pack_bf16(__uint_as_float(rr[14]) * inv, __uint_as_float(rr[15]) * inv);
          *reinterpret_cast<uint4*>(dst + c0) = v0;
          *reinterpret_cast<uint4*>(dst + c0 + 8) = v1;
        }
      }
    }
  }

  // every role comes here, also after a wait that ran out: copies in flight have been waited for above
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0) LLG_STAMP(5, 3, 0, blockIdx.x + gridDim.x * blockIdx.y);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}

// ---- host side: tensor maps of the key/value sources ------------------------------------------------

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

// Boxes of 64 rows x 64 head dimensions (128 bytes, swizzled) out of [rows][hd] (cache pages: rows = pages x kv
// heads x 64 positions) or, with nkv > 0, out of [rows][nkv][hd] for one kv head (the step's packed keys or values).
bool kv_map(const void* base, long long rows, int nkv, int hd, CUtensorMap* result) {
  static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple(base, rows, nkv, hd);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *result = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  CUtensorMap m;
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r;
  if (nkv > 0) {
    cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nkv, (cuuint64_t)rows};
    cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)nkv * hd * 2};
    cuuint32_t box[3] = {64, 1, (cuuint32_t)TK};
    r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)TK};
    r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *result = m;
  return true;
}

template <int HD>
int launch(const PrefillArgs& a, cudaStream_t stream) {
  constexpr int KVB = (HD / 64) * TK * 128;
  constexpr int smem = GROUPS * (HD / 64) * BQ * 128 + (KST + VST) * KVB;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return llg_fail("attn_prefill_tc: shared memory %d: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  CUtensorMap mkp, mvp, mkn, mvn;
  const long long page_rows = (long long)a.n_pages * a.nkv * TK;
  if (!kv_map(a.k_pages, page_rows, 0, HD, &mkp) || !kv_map(a.v_pages, page_rows, 0, HD, &mvp) ||
      !kv_map(a.k_new, a.n_tokens, a.nkv, HD, &mkn) || !kv_map(a.v_new, a.n_tokens, a.nkv, HD, &mvn))
    return llg_fail("attn_prefill_tc: cuTensorMapEncodeTiled failed or is not available");
  cudaError_t le = llg_launch(attn_prefill_tc_kernel<HD>, dim3(a.nh, a.n_tiles), dim3(THREADS), (size_t)smem, stream, mkp, mvp, mkn,
                              mvn, a);
  if (le != cudaSuccess) return llg_fail("attn_prefill_tc: launch: %s", cudaGetErrorString(le));
  return llg_check_launch("attn_prefill_tc");
}

}  // namespace

// 1 when this kernel takes the head size (bfloat16 only): 64 or 128.
LLG_API int llg_attn_tc_supported(int hd) { return hd == 64 || hd == 128; }

LLG_API int llg_attn_prefill_tc(const PrefillArgs* args, cudaStream_t stream) {
  const PrefillArgs& a = *args;
  LLG_REQUIRE(llg_attn_tc_supported(a.hd), "attn_prefill_tc: head_dim %d is neither 64 nor 128", a.hd);
  LLG_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "attn_prefill_tc: %d heads are no multiple of %d key/value heads",
              a.nh, a.nkv);
  LLG_REQUIRE(a.window >= 0 && a.ring_pages > 0 && a.table_width >= a.ring_pages, "attn_prefill_tc: bad cache geometry");
  LLG_REQUIRE(a.n_tiles <= 65535, "attn_prefill_tc: %d query tiles in one step are more than a grid takes (65535)", a.n_tiles);
  LLG_REQUIRE(a.scale > 0.f, "attn_prefill_tc: the softmax scale must be positive");
  LLG_REQUIRE(a.n_tokens > 0 && a.n_pages > 0, "attn_prefill_tc: needs the sizes of the packed rows and of the pages");
  LLG_REQUIRE(((uintptr_t)a.k_new % 16) == 0 && ((uintptr_t)a.v_new % 16) == 0 && ((uintptr_t)a.k_pages % 16) == 0 &&
                  ((uintptr_t)a.v_pages % 16) == 0,
              "attn_prefill_tc: keys and values must be 16-byte aligned");
  if (a.n_tiles <= 0) return 0;
  return a.hd == 64 ? launch<64>(a, stream) : launch<128>(a, stream);
}

// Error code recorded when a wait ran out (0 = none); clears it.  Synchronises the device.
LLG_API int llg_attn_tc_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_error, &zero, sizeof(int));
  return v;
}

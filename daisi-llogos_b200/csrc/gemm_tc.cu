// Matrix product on the 5th-generation tensor cores of sm_100a:
//     out[s][n][o] = sum over the k-blocks of split s of  x[n][k] * w[o][k]      (bfloat16 in, float32 accumulate)
// for every projection of the decoder, in both regimes: a prompt step (thousands of rows of x) and
// a decode step (1..64 rows), where the kernel is a weight streamer.
//
// Mapping.  The weight matrix is the M operand of the MMA (128 output features per tile), the
// activations are the N operand (16..256 tokens per tile): a decode batch of 1..16 tokens costs one
// 16-wide tile and no extra memory traffic, because the rows past the batch are filled with zeros
// by TMA.  Both operands are K-major in memory ([rows][k]), so TMA brings [rows x 64 k] boxes with
// the 128-byte swizzle and tcgen05.mma reads them from shared memory through descriptors.  The
// accumulator (128 lanes x N columns of float32) lives in tensor memory; four warps read it back
// with tcgen05.ld and store out[n][o] so that one warp instruction writes 32 consecutive features.
//
// Roles in a block of 192 threads: a lane of warp 4 issues TMA loads into a ring of stages that runs on across the
// block's tiles, a lane of warp 5 issues the MMAs and commits each stage back to the producer, warps 0-3 run the
// epilogue.  Where the accumulator takes at most half of tensor memory there are two, so the next tile's products
// run while the last tile is read out.  Split-K (blockIdx.z) writes float32 partials that the consumer kernels sum.
//
// Every wait on an mbarrier is bounded (two seconds of %globaltimer): on expiry the block records
// an error code, stops issuing work, waits (bounded) for its own TMA copies in flight, frees its
// tensor memory and returns.  llg_gemm_tc_status() reports the code.
//
// The reference has no tensor-core kernel of its own (its prompt path calls cublasGemmEx,
// Daisi.Llogos.Cuda/CudaBackend.cs:246-260; its decode path is a scalar GEMV,
// kernels/dequant_matmul.cu:593-619).
#include "common.cuh"
#include "kernel_args.h"

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

constexpr int BM = 128;          // output features per tile (MMA M)
constexpr int BK = 64;           // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
constexpr int EPI_WARPS = 4;     // warps 0-3 read the accumulator out, each its quarter of the lanes
constexpr int PRODUCER_WARP = 4, MMA_WARP = 5;
constexpr int GEMM_THREADS = 6 * 32;

__device__ int g_error = 0;      // 0 ok; 1 producer wait, 2 consumer wait, 3 epilogue wait, 4 drain wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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

// Waits for the phase with the given parity; false when the time limit ran out or another thread
// of the block already gave up.
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

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory operand descriptor: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
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

struct GemmParams {
  void* out;        // [splits][n][o], or [n][gated_features] with the gated epilogue
  int n, o, k;
  int kb_per_split; // k-blocks of 64 per split
  int gated_features;
  int up_offset;    // gated: row of w that holds the up row of feature 0 (gate rows come first)
  int gate_rows;    // gated, weights as first operand: features per block (at most 128)
  QkPrepArgs prep;  // EPI 2 / 3: what the q/k/v preparation needs (its `qkv` field is not used)
  RowScale scale;   // of the token rows of x: the result's rows are multiplied by it (EPI 2 / 3 take prep.row_scale)
};

// an element of a weight vector stored as float32 or bfloat16
__device__ __forceinline__ float vec_elem(const void* p, int dtype, int i) {
  return dtype == LLG_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}

// MT: weight tiles of 128 rows per block (1 or 2; two tiles share every activation tile, which halves
// the shared-memory traffic per flop of a large product).  EPI 1 (MT = 2): the first tile holds gate
// rows and the second the up rows of the same features; the block writes silu(gate) * up.  A block
// takes `gate_rows` features (TMA boxes of that many rows; the accumulator lanes past them are not
// read), chosen on the host so that the blocks of a decode step are as many as the SMs.
// SWAP 0: the first operand (MMA rows, accumulator lanes) is the weight matrix, the second the activations:
// out[n][o] with o along the lanes (decode steps: the token tile can be as small as 16).
// SWAP 1: the first operand is the activations (128 tokens per tile), the second the weights (TN features):
// a thread owns a token and writes runs of consecutive features with 16-byte stores (prompt steps).
// EPI 2 (head size 128) and EPI 3 (head size 64), SWAP 1 only: the product is the q/k/v projection and its epilogue
// is the preparation of queries and keys: a thread holds whole heads of its token (the tile is a whole number of
// heads wide), so the per-head norm, the bias and the rotation need no exchange between threads; queries go out as
// bfloat16 [token][head][head size], keys and values into the step's packed buffers and the cache pages.  The sums
// are never rounded before that, and the float32 q/k/v array of the two-kernel way is neither written nor read.
// Order as in the reference: norm, bias, rotation (Inference/ForwardPass.cs:372-385).
template <int TN, int STAGES, typename OT, int MT, int EPI, int SWAP>
__global__ void __launch_bounds__(GEMM_THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                      const __grid_constant__ CUtensorMap map_x, GemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int A_TILE = BM * BK * 2;
  constexpr int A_BYTES = MT * A_TILE;
  constexpr int B_BYTES = TN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // Two accumulators where tensor memory has room for them: the products of a block's next tile run while its last
  // one is read out.  An accumulator starts at a multiple of its width rounded up to a power of two.
  constexpr int ACC_COLS = MT * TN <= 32 ? 32 : MT * TN <= 64 ? 64 : MT * TN <= 128 ? 128 : MT * TN <= 256 ? 256 : 512;
  constexpr int NACC = ACC_COLS <= 256 ? 2 : 1;
  constexpr int TMEM_COLS = NACC * ACC_COLS;
  static_assert(MT * TN <= 512, "the accumulators do not fit tensor memory");
  static_assert(TN % 16 == 0, "the second operand's tile is a multiple of 16 rows");
  static_assert(EPI != 1 || (SWAP ? TN % 32 == 0 : MT == 2), "the gated epilogue needs a gate tile and an up tile");
  static_assert(EPI < 2 || (SWAP == 1 && TN % 128 == 0), "the q/k/v epilogue works on token rows and whole heads");
  // 1024-byte alignment of the operand tiles is what the swizzle pattern of TMA and of the MMA assume
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[NACC], acc_empty[NACC];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  // tokens along the columns: their scales, worked out during the products; a copy for even and one for odd tiles of the
  // block, and an mbarrier (a bounded wait, unlike a block barrier) on which every epilogue thread arrives once it has
  // written its share: who writes tile r + 2's copy has passed tile r + 1's barrier, so everybody is done reading tile r's
  __shared__ float col_scales[2][SWAP ? 1 : TN];
  __shared__ uint64_t scale_bar;

  pdl_launch_dependents();      // the next kernel may set itself up while this one runs
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef LLG_STAMPS
  // which product this is, for the time line: k / 1024 and the first operand's rows / 512
  const int st_aux = (((p.k >> 10) & 0xff) << 8) | (((SWAP ? p.n : p.o) >> 9) & 0xff), st_blk = blockIdx.x + gridDim.x * blockIdx.z;
#endif
  if (tid == 0) LLG_STAMP(1, 0, st_aux, st_blk);
  if (tid == PRODUCER_WARP * 32) {
    // the first copies need the two descriptors: fetch them while the barriers and the tensor memory are set up
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  const int split = blockIdx.z;
  const int n_tiles_n = (p.n + TN - 1) / TN;
  constexpr bool GATED_ROWS = EPI == 1 && SWAP == 0;       // gate and up tiles fetched separately, gate_rows each
  const int total_tiles = (GATED_ROWS ? (p.gated_features + p.gate_rows - 1) / p.gate_rows
                                      : (p.o + BM * MT - 1) / (BM * MT)) * n_tiles_n;
  const int m_tiles = total_tiles / n_tiles_n;
  const uint32_t stage_tx = GATED_ROWS ? (uint32_t)(2 * p.gate_rows * BK * 2 + B_BYTES) : (uint32_t)STAGE_BYTES;
  // row of w that the weight tile `mt` of the block at first-operand offset o0 starts at
  auto w_row = [&](int o0, int mt) { return GATED_ROWS ? mt * p.up_offset + o0 : o0 + mt * BM; };
  // second operand: one box of TN rows, or (gated, tokens first) the gate half and the up half of the features
  auto load_second = [&](unsigned char* dst, int kb, int n0, uint64_t* bar) {
    if (EPI == 1 && SWAP == 1) {
      tma_load_2d(dst, &map_x, kb * BK, n0 / 2, bar);
      tma_load_2d(dst + (TN / 2) * BK * 2, &map_x, kb * BK, p.up_offset + n0 / 2, bar);
    } else {
      tma_load_2d(dst, &map_x, kb * BK, n0, bar);
    }
  };
  // first operand: MT tiles of 128 rows
  auto load_first = [&](unsigned char* dst, int kb, int o0, uint64_t* bar) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) tma_load_2d(dst + mt * A_TILE, &map_w, kb * BK, w_row(o0, mt), bar);
  };
  // A block works through tiles blockIdx.x, blockIdx.x + gridDim.x, ...: token tiles of one weight tile are neighbours
  // in that order, so blocks running side by side share the weight tile in L2.
  auto first_offset = [&](int tile) { return (SWAP ? tile % m_tiles : tile / n_tiles_n) * (GATED_ROWS ? p.gate_rows : BM * MT); };
  auto second_offset = [&](int tile) { return (SWAP ? tile / m_tiles : tile % n_tiles_n) * TN; };
  const int nkb_total = (p.k + BK - 1) / BK;
  const int kb0 = split * p.kb_per_split;
  const int nkb = min(p.kb_per_split, nkb_total - kb0);   // >= 1 by construction of the grid

  int pre = 0;                  // the producer lane: k-blocks of its first tile whose weight tiles are requested below
  if (tid == PRODUCER_WARP * 32) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < NACC; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], EPI_WARPS);
    }
    mbar_init(&scale_bar, EPI_WARPS * 32);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // The weights do not depend on the previous kernel, and requesting them needs nothing but the barriers above: the
    // first ring of weight tiles is on its way before the block's tensor memory is there and long before this kernel
    // waits for its predecessor.  The weights are the first operand of a decode step's product and the second of a
    // prompt step's.
    if ((int)blockIdx.x < total_tiles) {
      const int o0 = first_offset(blockIdx.x), n0 = second_offset(blockIdx.x);
      pre = min(nkb, STAGES);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], stage_tx);
        if (SWAP) load_second(smem + i * STAGE_BYTES + A_BYTES, kb0 + i, n0, &full_bar[i]);
        else load_first(smem + i * STAGE_BYTES, kb0 + i, o0, &full_bar[i]);
      }
    }
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;
  volatile int* abortp = &abort_flag;

  if (warp == PRODUCER_WARP) {
    // ---- producer: one lane requests every tile of every stage; the ring of stages runs on across the block's tiles,
    // so the next tile's operands arrive while this tile's accumulator is read out ----------------------------------
    if (lane == 0) {
      int it = 0;                 // k-blocks requested so far
      bool first = true;
      for (int tile = blockIdx.x; tile < total_tiles && !*abortp; tile += gridDim.x) {
        const int o0 = first_offset(tile), n0 = second_offset(tile);
        int done = 0;
        if (first) {
          // the first tile's weight tiles are on their way (above); its activation tiles follow the dependency wait
          pdl_wait();
          LLG_STAMP(1, 1, st_aux, st_blk);
          for (int i = 0; i < pre; ++i) {
            if (SWAP) load_first(smem + i * STAGE_BYTES, kb0 + i, o0, &full_bar[i]);
            else load_second(smem + i * STAGE_BYTES + A_BYTES, kb0 + i, n0, &full_bar[i]);
          }
          it = done = pre;
          first = false;
        }
        for (int i = done; i < nkb && !*abortp; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t parity = ((it / STAGES) & 1) ^ 1;     // a fresh barrier passes a wait on parity 1
          if (!mbar_wait(&empty_bar[s], parity, abortp)) {
            if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 1); }
            break;
          }
          mbar_expect_tx(&full_bar[s], stage_tx);
          unsigned char* a = smem + s * STAGE_BYTES;
          load_first(a, kb0 + i, o0, &full_bar[s]);
          load_second(a + A_BYTES, kb0 + i, n0, &full_bar[s]);
        }
      }
      if (*abortp) {
        // copies already requested still write into this block's shared memory: wait for them, bounded
        for (int i = max(0, it - STAGES); i < it; ++i) {
          const unsigned long long t0 = now_ns();
          while (!mbar_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1)) {
            if (now_ns() - t0 > WAIT_LIMIT_NS) { atomicCAS(&g_error, 1, 4); break; }
          }
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // ---- products: one lane issues every MMA.  With two accumulators in tensor memory the products of the next tile
    // run while the four other warps read the last one out. ------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      int it = 0, round = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abortp; tile += gridDim.x, ++round) {
        const int b = round % NACC;
        if (round >= NACC && !mbar_wait(&acc_empty[b], ((round / NACC) - 1) & 1, abortp)) {
          if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 3); }
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_d + (uint32_t)(b * ACC_COLS);
        bool fine = true;
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, abortp)) {
            if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 2); }
            fine = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t db = umma_desc(a_addr + A_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // 16 k = 32 bytes further along the swizzled row: +2 in the descriptor's 16-byte units
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
              umma_bf16(acc + mt * TN, umma_desc(a_addr + mt * A_TILE) + 2 * kk, db + 2 * kk, IDESC, (i | kk) != 0);
          }
          umma_commit(&empty_bar[s]);       // arrives when the MMAs above have read the stage
        }
        if (!fine) break;
        umma_commit(&acc_full[b]);          // arrives when every MMA issued so far has finished
      }
    }
  } else {
    // ---- epilogue: warps 0-3, each its quarter of the lanes: tensor memory -> registers -> out ----------------------
    pdl_wait();                 // before anything of the previous kernel is read or overwritten
    int round = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++round) {
      const int o0 = first_offset(tile), n0 = second_offset(tile);
      const int b = round % NACC;
      const float* col_scale = col_scales[round & 1];
      if (!SWAP && p.scale.ss) {
        // tokens along the columns: their scales, worked out while the products run
        for (int c = tid; c < TN; c += EPI_WARPS * 32) col_scales[round & 1][c] = n0 + c < p.n ? row_scale_of(p.scale, n0 + c) : 0.f;
        mbar_arrive(&scale_bar);
        if (!mbar_wait(&scale_bar, round & 1, abortp)) {
          if (!*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 3); }
          break;
        }
      }
      const bool have = mbar_wait(&acc_full[b], (round / NACC) & 1, abortp);
      if (!have && !*abortp) { *abortp = 1; atomicCAS(&g_error, 0, 3); }
      if (!have || *abortp) break;
      if (tid == 0 && round == 0) LLG_STAMP(1, 2, st_aux, st_blk);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      {
        const uint32_t lane_base = tmem_d + (uint32_t)(b * ACC_COLS) + ((uint32_t)(warp * 32) << 16);
        if (SWAP && EPI >= 2) {
          // lanes are tokens, columns are the features of whole heads: norm, bias, rotation, and the writes of q, k, v
          constexpr int HD = EPI == 2 ? 128 : 64, HALF = HD / 2;
          const QkPrepArgs& a = p.prep;
          const int heads = a.nh + 2 * a.nkv;
          typedef __nv_bfloat16 bf;
  #pragma unroll 1
          for (int mt = 0; mt < MT; ++mt) {
            if (o0 + mt * BM >= p.o) break;
            const int tok = o0 + mt * BM + warp * 32 + lane;
            const bool live = tok < p.o;
            const int pos = live ? a.positions[tok] : 0;
            const int slot = (live && a.k_pages) ? a.slots[a.seq_of_token[tok]] : 0;
            const float rs = live ? row_scale_of(a.row_scale, tok) : 1.0f;
  #pragma unroll 1
            for (int hb = 0; hb < TN / HD; ++hb) {
              const int head = n0 / HD + hb;
              if (head >= heads) break;                   // uniform: the tile's tail lies past the last head
              float h[HD];
  #pragma unroll
              for (int c0 = 0; c0 < HD; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(lane_base + (uint32_t)(mt * TN + hb * HD + c0), r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  #pragma unroll
                for (int c = 0; c < 16; ++c) h[c0 + c] = __uint_as_float(r[c]) * rs;
              }
              const int kind = head < a.nh ? 0 : (head < a.nh + a.nkv ? 1 : 2);      // query, key, value
              const void* nw = kind == 0 ? a.q_norm_w : (kind == 1 ? a.k_norm_w : nullptr);
              if (nw) {
                float ss = 0.f;
  #pragma unroll
                for (int d = 0; d < HD; ++d) ss += h[d] * h[d];
                const float inv = 1.0f / sqrtf(ss / (float)HD + a.norm_eps);
  #pragma unroll
                for (int d = 0; d < HD; ++d) h[d] = h[d] * inv * vec_elem(nw, a.norm_w_dtype, d);
              }
              if (a.bias) {
  #pragma unroll
                for (int d = 0; d < HD; ++d) h[d] += vec_elem(a.bias, a.bias_dtype, head * HD + d);
              }
              if (kind != 2 && a.cos_table) {
                const int pp = pos < a.table_positions ? pos : a.table_positions - 1;     // bounded; the host checks capacity
                const float4* cs = reinterpret_cast<const float4*>(a.cos_table + (long long)pp * HALF);
                const float4* sn = reinterpret_cast<const float4*>(a.sin_table + (long long)pp * HALF);
  #pragma unroll
                for (int i4 = 0; i4 < HALF / 4; ++i4) {
                  const float4 c = cs[i4], sgn = sn[i4];
                  const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sgn.x, sgn.y, sgn.z, sgn.w};
  #pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const int i = 4 * i4 + e;
                    const float u = h[i], v = h[i + HALF];
                    h[i] = u * cc[e] - v * sv[e];
                    h[i + HALF] = u * sv[e] + v * cc[e];
                  }
                }
              }
              if (live) {
                auto store_head = [&](bf* dst) {
  #pragma unroll
                  for (int q8 = 0; q8 < HD / 8; ++q8) {
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(h[8 * q8], h[8 * q8 + 1]), h1 = __floats2bfloat162_rn(h[8 * q8 + 2], h[8 * q8 + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(h[8 * q8 + 4], h[8 * q8 + 5]), h3 = __floats2bfloat162_rn(h[8 * q8 + 6], h[8 * q8 + 7]);
                    uint4 u;
                    u.x = *reinterpret_cast<uint32_t*>(&h0);
                    u.y = *reinterpret_cast<uint32_t*>(&h1);
                    u.z = *reinterpret_cast<uint32_t*>(&h2);
                    u.w = *reinterpret_cast<uint32_t*>(&h3);
                    *reinterpret_cast<uint4*>(dst + 8 * q8) = u;
                  }
                };
                if (kind == 0) {
                  store_head((bf*)a.q_out + ((long long)tok * a.nh + head) * HD);
                } else {
                  const int kvh = kind == 1 ? head - a.nh : head - a.nh - a.nkv;
                  bf* packed = (bf*)(kind == 1 ? a.k_new : a.v_new);
                  if (packed) store_head(packed + ((long long)tok * a.nkv + kvh) * HD);
                  bf* pages = (bf*)(kind == 1 ? a.k_pages : a.v_pages);
                  if (pages) store_head(pages + kv_row(a.page_table, a.table_width, a.ring_pages, slot, pos, kvh, a.nkv) * HD);
                }
              }
            }
          }
        } else if (SWAP) {
          // lanes are tokens (p.o of them), columns are features (p.n, or gate|up blocks of 128 + 128)
          constexpr int VEC = 16 / (int)sizeof(OT);      // outputs per 16-byte store
          const int width = EPI == 1 ? p.gated_features : p.n;
          const bool vec_ok = width % VEC == 0;
          OT* out = (OT*)p.out + (long long)split * p.n * p.o;
  #pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            if (o0 + mt * BM >= p.o) break;
            const int tok = o0 + mt * BM + warp * 32 + lane;
            const float rs = tok < p.o ? row_scale_of(p.scale, tok) : 1.0f;
            OT* row = out + (long long)tok * width;
            constexpr int COLS = EPI == 1 ? TN / 2 : TN;
  #pragma unroll
            for (int c0 = 0; c0 < COLS; c0 += 16) {
              const int f0 = EPI == 1 ? n0 / 2 + c0 : n0 + c0;      // first feature of this run (a gated tile: TN / 2 features)
              if (f0 >= width) break;
              float v[16];
              uint32_t r[16];
              tmem_ld16(lane_base + (uint32_t)(mt * TN + c0), r);
              if (EPI == 1) {
                uint32_t ru[16];
                tmem_ld16(lane_base + (uint32_t)(mt * TN + TN / 2 + c0), ru);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  #pragma unroll
                for (int c = 0; c < 16; ++c) {
                  const float g = __uint_as_float(r[c]) * rs;
                  v[c] = __fdividef(g, 1.0f + __expf(-g)) * (__uint_as_float(ru[c]) * rs);
                }
              } else {
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  #pragma unroll
                for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(r[c]) * rs;
              }
              if (tok < p.o) {
                if (vec_ok && f0 + 16 <= width) {
                  if (sizeof(OT) == 4) {
  #pragma unroll
                    for (int q = 0; q < 4; ++q)
                      *reinterpret_cast<float4*>((float*)row + f0 + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                  } else {
  #pragma unroll
                    for (int q = 0; q < 2; ++q) {
                      __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * q], v[8 * q + 1]), h1 = __floats2bfloat162_rn(v[8 * q + 2], v[8 * q + 3]);
                      __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * q + 4], v[8 * q + 5]), h3 = __floats2bfloat162_rn(v[8 * q + 6], v[8 * q + 7]);
                      uint4 u;
                      u.x = *reinterpret_cast<uint32_t*>(&h0);
                      u.y = *reinterpret_cast<uint32_t*>(&h1);
                      u.z = *reinterpret_cast<uint32_t*>(&h2);
                      u.w = *reinterpret_cast<uint32_t*>(&h3);
                      *reinterpret_cast<uint4*>((__nv_bfloat16*)row + f0 + 8 * q) = u;
                    }
                  }
                } else {
  #pragma unroll
                  for (int c = 0; c < 16; ++c)
                    if (f0 + c < width) row[f0 + c] = from_f32<OT>(v[c]);
                }
              }
            }
          }
        } else if (EPI == 0) {
          // Up to 64 columns of the accumulator are asked for before their arrival is waited for: one trip to tensor
          // memory per 64 tokens instead of one per 16.
          constexpr int CH = TN < 64 ? TN : 64;
          OT* out = (OT*)p.out + (long long)split * p.n * p.o;
  #pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const int o = o0 + mt * BM + warp * 32 + lane;
            if (o0 + mt * BM >= p.o) break;     // uniform: the second tile lies past the matrix
  #pragma unroll
            for (int c0 = 0; c0 < TN; c0 += CH) {
              if (n0 + c0 >= p.n) break;        // uniform over the block: the tile's tail holds no tokens
              uint32_t r[CH / 16][16];
  #pragma unroll
              for (int q = 0; q < CH / 16; ++q)
                if (n0 + c0 + 16 * q < p.n) tmem_ld16(lane_base + (uint32_t)(mt * TN + c0 + 16 * q), r[q]);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
              if (o < p.o) {
  #pragma unroll
                for (int q = 0; q < CH / 16; ++q) {
                  if (n0 + c0 + 16 * q >= p.n) break;
                  // every value is worked out before the first is stored: a store through a generic pointer may, for all
                  // the compiler knows, change the scales in shared memory, and would order every element behind the last
                  float v[16];
  #pragma unroll
                  for (int c = 0; c < 16; ++c)
                    v[c] = p.scale.ss ? __uint_as_float(r[q][c]) * col_scale[c0 + 16 * q + c] : __uint_as_float(r[q][c]);
                  OT* dst = out + (long long)(n0 + c0 + 16 * q) * p.o + o;
  #pragma unroll
                  for (int c = 0; c < 16; ++c)
                    if (n0 + c0 + 16 * q + c < p.n) dst[(long long)c * p.o] = from_f32<OT>(v[c]);
                }
              }
            }
          }
        } else {
          // accumulator 0 holds gate, accumulator 1 up, of feature o0 + lane row (the first gate_rows lanes)
          constexpr int CH = TN < 64 ? TN : 64;
          OT* out = (OT*)p.out;
          const int row = warp * 32 + lane;
          const int inter = row < p.gate_rows ? p.gated_features : 0;
          const int f = o0 + row;
  #pragma unroll
          for (int c0 = 0; c0 < TN; c0 += CH) {
            if (n0 + c0 >= p.n) break;
            uint32_t rg[CH / 16][16], ru[CH / 16][16];
  #pragma unroll
            for (int q = 0; q < CH / 16; ++q) {
              if (n0 + c0 + 16 * q < p.n) {
                tmem_ld16(lane_base + (uint32_t)(c0 + 16 * q), rg[q]);
                tmem_ld16(lane_base + (uint32_t)(TN + c0 + 16 * q), ru[q]);
              }
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (f < inter) {
  #pragma unroll
              for (int q = 0; q < CH / 16; ++q) {
                if (n0 + c0 + 16 * q >= p.n) break;
                float v[16];                  // all worked out before the first store, as above
  #pragma unroll
                for (int c = 0; c < 16; ++c) {
                  const float rs = p.scale.ss ? col_scale[c0 + 16 * q + c] : 1.0f;
                  const float g = __uint_as_float(rg[q][c]) * rs, u = __uint_as_float(ru[q][c]) * rs;
                  v[c] = __fdividef(g, 1.0f + __expf(-g)) * u;
                }
                OT* dst = out + (long long)(n0 + c0 + 16 * q) * inter + f;
  #pragma unroll
                for (int c = 0; c < 16; ++c)
                  if (n0 + c0 + 16 * q + c < p.n) dst[(long long)c * inter] = from_f32<OT>(v[c]);
              }
            }
          }
        }
      }
      // the accumulator may be overwritten only after every warp has read it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0) LLG_STAMP(1, 3, st_aux, st_blk);
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}


// ---- host side: tensor maps ------------------------------------------------------------------

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

// A [rows][k] bfloat16 matrix, row-major, read in boxes of [box_rows][64 k] with the 128-byte swizzle;
// what lies outside the matrix reads as zero.
bool tensor_map(const void* base, int rows, int k, int box_rows, CUtensorMap* result) {
  static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple(base, rows, k, box_rows);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *result = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *result = m;
  return true;
}

template <int TN, int STAGES, typename OT, int MT, int EPI, int SWAP>
int launch(const CUtensorMap* mw, const CUtensorMap* mx, const GemmParams& p, int splits, cudaStream_t stream) {
  constexpr int smem = STAGES * (MT * BM * BK * 2 + TN * BK * 2) + 1024;
  static_assert(smem <= 232448, "stage ring does not fit shared memory");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<TN, STAGES, OT, MT, EPI, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return llg_fail("gemm_tc: cannot have %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  // one block per tile for the small token tiles of a decode step; for the large ones as many blocks as
  // fit the GPU at once, each working through several tiles
  const long long m_tiles = (EPI == 1 && SWAP == 0) ? (p.gated_features + p.gate_rows - 1) / p.gate_rows : (p.o + BM * MT - 1) / (BM * MT);
  const long long tiles = m_tiles * ((p.n + TN - 1) / TN);
  long long blocks = tiles;
  if (TN >= 128) {
    const long long resident = (long long)llg_sm_count() * (smem <= 113 * 1024 ? 2 : 1);
    if (blocks > resident) blocks = resident;
  }
  if (blocks > 2147483647LL) return llg_fail("gemm_tc: too many tiles");
  dim3 grid((unsigned)blocks, 1, splits);
  cudaError_t le = llg_launch(gemm_tc_kernel<TN, STAGES, OT, MT, EPI, SWAP>, grid, dim3(GEMM_THREADS), (size_t)smem, stream, *mw, *mx, p);
  if (le != cudaSuccess) return llg_fail("gemm_tc: launch: %s", cudaGetErrorString(le));
  return llg_check_launch("gemm_tc");
}

}  // namespace

// 1 if the tensor-core kernel takes these operands: k a multiple of 8 (TMA needs 16-byte row strides)
// and 16-byte aligned base addresses.
LLG_API int llg_gemm_tc_supported(const void* x, const void* w, int n, int o, int k) {
  return n > 0 && o > 0 && k > 0 && k % 8 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0;
}

// Splits that llg_gemm_tc will really use for a wish of `splits` (every split gets at least one k-block).
LLG_API int llg_gemm_tc_splits(int k, int splits) {
  const int nkb = (k + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > nkb) splits = nkb;
  const int per = (nkb + splits - 1) / splits;
  return (nkb + per - 1) / per;
}

// out[s][n][o] for s < llg_gemm_tc_splits(k, splits); out_dtype float32, or bfloat16 when there is one split.
// gated_features > 0 (one split only): w has 2 * P rows with P = F rounded up to a multiple of 128: the gate rows of
// all features, zero rows up to P, then the up rows in the same way; out is [n][F] = silu(gate) * up.
// `scale` (may be null): what a norm left for the rows of x; the rows of the result are multiplied by it (with several
// splits every partial is).
LLG_API int llg_gemm_tc(const void* x, const void* w, void* out, int out_dtype, int n, int o, int k, int splits,
                        int tile_n, int gated_features, const RowScale* scale, cudaStream_t stream) {
  const RowScale rs = scale ? *scale : RowScale{nullptr, 0, 0.f, 0.f};
  LLG_REQUIRE(llg_gemm_tc_supported(x, w, n, o, k), "gemm_tc: needs k %% 8 == 0 and 16-byte aligned operands (n=%d o=%d k=%d)",
              n, o, k);
  splits = llg_gemm_tc_splits(k, splits);
  LLG_REQUIRE(out_dtype == LLG_F32 || (out_dtype == LLG_BF16 && splits == 1), "gemm_tc: bfloat16 output needs one split");
  const bool gated = gated_features > 0;
  LLG_REQUIRE(!gated || (splits == 1 && o == ((gated_features + BM - 1) / BM) * 2 * BM),
              "gemm_tc: the gated epilogue needs one split and ceil(features / 128) * 256 rows of w (features=%d rows=%d splits=%d)",
              gated_features, o, splits);
  const int nkb = (k + BK - 1) / BK;
  CUtensorMap map_w, map_x;
  if (n >= 256 && tile_n <= 0) {
    // ---- prompt steps: activations are the first operand (128 tokens per tile), up to 256 features per tile ----
    // in this orientation the kernel's first-operand rows (field o) are the tokens, the second's (field n) the features
    GemmParams ps{out, /*n=*/o, /*o=*/n, k, (nkb + splits - 1) / splits, gated_features, o / 2, BM, QkPrepArgs{}, rs};
    // Tile shape: blocks run in rounds of one per SM (148 on a B200); a round costs its tile's width, and a narrower tile can save a
    // round (4096 features: 16 tiles of 256 in two token rows of 8 are 128 blocks, 18 of 240 are 144).  Two token
    // tiles per block halve the weight traffic per flop (worth about 15 %) but double the tile.
    const int widths[5] = {256, gated ? 192 : 240, 224, gated ? 256 : 208, gated ? 256 : 176};
    int best_w = 256, best_mt = 1;
    double best_cost = 0;
    const long long sms = llg_sm_count();
    for (int wi = 0; wi < 5; ++wi) {
      for (int mt = 1; mt <= 2; ++mt) {
        if (mt == 1 && widths[wi] < 224) continue;      // a single token tile wants a wide second operand
        const long long tiles = (long long)((n + mt * BM - 1) / (mt * BM)) * ((o + widths[wi] - 1) / widths[wi]) * splits;
        const double cost = (double)((tiles + sms - 1) / sms) * widths[wi] * mt * (mt == 2 ? 0.85 : 1.0);
        if (best_cost == 0 || cost < best_cost * 0.999) {
          best_cost = cost;
          best_w = widths[wi];
          best_mt = mt;
        }
      }
    }
    if (gated && out_dtype == LLG_F32) best_w = 256;
    // the gated product fetches the gate half and the up half of a feature tile with a box of half the width each
    LLG_REQUIRE(tensor_map(x, n, k, BM, &map_x) && tensor_map(w, o, k, gated ? best_w / 2 : best_w, &map_w),
                "gemm_tc: cuTensorMapEncodeTiled failed or is not available");
#define GOS(W, OTT, EP)                                                                        \
  return best_mt == 2 ? launch<W, 3, OTT, 2, EP, 1>(&map_x, &map_w, ps, splits, stream)          \
                      : launch<W, 4, OTT, 1, EP, 1>(&map_x, &map_w, ps, splits, stream)
    if (gated) {
      if (out_dtype == LLG_F32) GOS(256, float, 1);      // float32 out: the widest tile only
      if (best_w == 256) GOS(256, __nv_bfloat16, 1);
      if (best_w == 224) GOS(224, __nv_bfloat16, 1);
      GOS(192, __nv_bfloat16, 1);
    }
#define GO2(W, OTT) return launch<W, 3, OTT, 2, 0, 1>(&map_x, &map_w, ps, splits, stream)
    if (out_dtype == LLG_F32) {
      if (best_w == 256) GOS(256, float, 0);
      if (best_w == 240) GOS(240, float, 0);
      if (best_w == 224) GOS(224, float, 0);
      if (best_w == 208) GO2(208, float);
      GO2(176, float);
    }
    if (best_w == 256) GOS(256, __nv_bfloat16, 0);
    if (best_w == 240) GOS(240, __nv_bfloat16, 0);
    if (best_w == 224) GOS(224, __nv_bfloat16, 0);
    if (best_w == 208) GO2(208, __nv_bfloat16);
    GO2(176, __nv_bfloat16);
#undef GO2
#undef GOS
  }
  // Features per block of a gated product: with one token tile the blocks should be as many as the SMs (or a
  // multiple), whatever the feature count; 128 per block would leave a quarter of the SMs idle at 14336 features.
  int gate_rows = BM;
  if (tile_n <= 0) tile_n = n <= 16 ? 16 : n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : 256;
  if (gated && n <= tile_n) {
    const int sms = llg_sm_count();
    const int rounds = ((gated_features + BM - 1) / BM + sms - 1) / sms;
    gate_rows = (gated_features + sms * rounds - 1) / (sms * rounds);
    if (gate_rows < 16) gate_rows = 16;
    if (gate_rows > BM) gate_rows = BM;
  }
  GemmParams p{out, n, o, k, (nkb + splits - 1) / splits, gated_features, o / 2, gate_rows, QkPrepArgs{}, rs};
  LLG_REQUIRE(splits <= 65535, "gemm_tc: grid too large");
  LLG_REQUIRE(tensor_map(w, o, k, gated ? gate_rows : BM, &map_w) && tensor_map(x, n, k, tile_n, &map_x),
              "gemm_tc: cuTensorMapEncodeTiled failed or is not available");
  const CUtensorMap *mw = &map_w, *mx = &map_x;
  // Two weight tiles per block halve the activation traffic per flop (worth about 15 %) but double the
  // tile: take them when the rounds over the SMs come out cheaper that way.
  const long long nt = (n + tile_n - 1) / tile_n;
  const long long t1 = (long long)((o + BM - 1) / BM) * nt, t2 = (long long)((o + 2 * BM - 1) / (2 * BM)) * nt;
  const long long sm_n = llg_sm_count();
  const bool wide = !gated && tile_n >= 128 && ((t2 + sm_n - 1) / sm_n) * 2 * 0.85 < (double)((t1 + sm_n - 1) / sm_n);
#define GATED(TN, ST2)                                                                               \
  if (gated)                                                                                          \
    return out_dtype == LLG_F32 ? launch<TN, ST2, float, 2, 1, 0>(mw, mx, p, splits, stream)            \
                                : launch<TN, ST2, __nv_bfloat16, 2, 1, 0>(mw, mx, p, splits, stream)
#define PLAIN(TN, ST1)                                                                               \
  return out_dtype == LLG_F32 ? launch<TN, ST1, float, 1, 0, 0>(mw, mx, p, splits, stream)              \
                              : launch<TN, ST1, __nv_bfloat16, 1, 0, 0>(mw, mx, p, splits, stream)
#define WIDE(TN, ST2)                                                                                \
  if (wide)                                                                                           \
    return out_dtype == LLG_F32 ? launch<TN, ST2, float, 2, 0, 0>(mw, mx, p, splits, stream)            \
                                : launch<TN, ST2, __nv_bfloat16, 2, 0, 0>(mw, mx, p, splits, stream)
  switch (tile_n) {
    case 16: GATED(16, 5); PLAIN(16, 5);
    case 32: GATED(32, 5); PLAIN(32, 5);
    case 64: GATED(64, 5); PLAIN(64, 4);
    case 128: GATED(128, 4); WIDE(128, 4); PLAIN(128, 6);
    case 256: GATED(256, 3); WIDE(256, 3); PLAIN(256, 4);
    default: return llg_fail("gemm_tc: tile_n %d is not one of 16, 32, 64, 128, 256", tile_n);
  }
#undef GATED
#undef PLAIN
#undef WIDE
}

// 1 when llg_gemm_tc_qkv takes this q/k/v projection: 256 tokens or more (tokens are the tensor cores' rows), head
// size 64 or 128, rotation over the whole head by halves (or none), operands as llg_gemm_tc_supported wants them.
LLG_API int llg_gemm_tc_qkv_supported(int n, int k, int hd, int has_rotation, int rotary_dim, int pairing) {
  return n >= 256 && k > 0 && k % 8 == 0 && (hd == 64 || hd == 128) && (!has_rotation || (pairing == 0 && rotary_dim == hd));
}

// The q/k/v projection of a prompt step with the preparation of queries and keys as its epilogue: what llg_gemm_tc into a
// float32 array followed by llg_qk_prep gives, in one kernel.  x [n][k] and w [(nh + 2 nkv) * hd][k] are bfloat16, all
// outputs named in `prep` are bfloat16; prep->qkv is ignored.
LLG_API int llg_gemm_tc_qkv(const void* x, const void* w, int n, int k, const QkPrepArgs* prep, cudaStream_t stream) {
  const QkPrepArgs& a = *prep;
  const int o = (a.nh + 2 * a.nkv) * a.hd;
  LLG_REQUIRE(a.nh > 0 && a.nkv >= 0 && llg_gemm_tc_supported(x, w, n, o, k), "gemm_tc_qkv: needs k %% 8 == 0 and 16-byte aligned operands");
  LLG_REQUIRE(llg_gemm_tc_qkv_supported(n, k, a.hd, a.cos_table != nullptr, a.rotary_dim, a.pairing),
              "gemm_tc_qkv: needs 256 tokens or more, head size 64 or 128 and rotation over the whole head by halves "
              "(n=%d hd=%d rotary_dim=%d pairing=%d)", n, a.hd, a.rotary_dim, a.pairing);
  LLG_REQUIRE(a.n_tokens == n && a.positions && a.q_out, "gemm_tc_qkv: the preparation's sizes do not fit the product");
  LLG_REQUIRE(!a.k_pages || (a.page_table && a.slots && a.seq_of_token && a.ring_pages > 0),
              "gemm_tc_qkv: a cache write needs page_table, slots and seq_of_token");
  if ((a.q_norm_w || a.k_norm_w) && a.bias)
    LLG_REQUIRE(a.norm_w_dtype == a.bias_dtype, "gemm_tc_qkv: norm weights and bias must share a dtype");
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15u) == 0; };
  LLG_REQUIRE(aligned(a.cos_table) && aligned(a.sin_table) && aligned(a.q_out) && aligned(a.k_new) && aligned(a.v_new) &&
                  aligned(a.k_pages) && aligned(a.v_pages),
              "gemm_tc_qkv: tables and outputs must be 16-byte aligned");
  const int nkb = (k + BK - 1) / BK;
  GemmParams ps{nullptr, /*n=*/o, /*o=*/n, k, nkb, 0, 0, BM, a, RowScale{nullptr, 0, 0.f, 0.f}};
  CUtensorMap map_w, map_x;
  LLG_REQUIRE(tensor_map(x, n, k, BM, &map_x) && tensor_map(w, o, k, 256, &map_w),
              "gemm_tc_qkv: cuTensorMapEncodeTiled failed or is not available");
  // one or two token tiles per block, by the rounds of blocks over the SMs (as in llg_gemm_tc)
  const long long sms = llg_sm_count();
  const long long t1 = (long long)((n + BM - 1) / BM) * ((o + 255) / 256), t2 = (long long)((n + 2 * BM - 1) / (2 * BM)) * ((o + 255) / 256);
  const bool two = (double)((t2 + sms - 1) / sms) * 2 * 0.85 < (double)((t1 + sms - 1) / sms);
  if (a.hd == 128)
    return two ? launch<256, 3, __nv_bfloat16, 2, 2, 1>(&map_x, &map_w, ps, 1, stream)
               : launch<256, 4, __nv_bfloat16, 1, 2, 1>(&map_x, &map_w, ps, 1, stream);
  return two ? launch<256, 3, __nv_bfloat16, 2, 3, 1>(&map_x, &map_w, ps, 1, stream)
             : launch<256, 4, __nv_bfloat16, 1, 3, 1>(&map_x, &map_w, ps, 1, stream);
}


// Error code that a block recorded when one of its waits ran out (0 = none); clears it.  Synchronises the device.
LLG_API int llg_gemm_tc_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_error, &zero, sizeof(int));
  return v;
}

// Shared helpers of the kernels: element types, error reporting, reductions.
//
// Every exported function is `extern "C"`, takes raw device pointers and the
// stream to launch on, validates its sizes on the host and returns 0 on success.
// On failure it returns non-zero and leaves a message for llg_last_error().
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#define LLG_API extern "C" __attribute__((visibility("default")))

enum { LLG_F32 = 0, LLG_BF16 = 1 };

// Tokens per page of the key/value cache.  Python reads it through llg_page_size().
#define LLG_PAGE 64

static thread_local char g_llg_error[512];

static inline int llg_fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
#include <stdarg.h>
static inline int llg_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_llg_error, sizeof(g_llg_error), fmt, ap);
  va_end(ap);
  return 1;
}

static inline int llg_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return llg_fail("%s: %s", what, cudaGetErrorString(e));
  return 0;
}

#define LLG_REQUIRE(cond, ...)            \
  do {                                    \
    if (!(cond)) return llg_fail(__VA_ARGS__); \
  } while (0)

// Number of multiprocessors of the current device (asked once per device and kept).
static inline int llg_sm_count() {
  static int count[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    count[dev] = n;
  }
  return count[dev];
}

// ---- programmatic dependent launch -----------------------------------------------------
//
// Kernels of a step run back to back on one stream, each consuming what the one before wrote.
// A kernel launched with llg_launch() may start while its predecessor is still running: it runs
// its own set-up (shared memory, barriers, tensor memory), calls pdl_wait() before it touches any
// memory that another kernel writes or reads, and calls pdl_launch_dependents() at its start so
// that its successor may do the same.  Without the launch attribute both calls do nothing.

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>

static inline bool llg_pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LLOGOS_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Launches `kernel` so that it may overlap the tail of the previous kernel on the stream (see above).
template <typename... KArgs, typename... Args>
static inline cudaError_t llg_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = llg_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- time stamps (only when compiled with -DLLG_STAMPS) ------------------------------------
//
// For looking at a step's kernels on one time line: a block's thread calls LLG_STAMP(kernel, phase, aux, block) and
// the library keeps (%globaltimer, tag) pairs in a buffer of its own that llg_stamps_read() hands out and empties.
// Phases by convention: 0 the block started, 1 its dependency wait returned, 2 its products are done, 3 it ends.
// A stamp costs about a third of a microsecond (a timer read and an atomic); without the flag the macro is empty.
#ifdef LLG_STAMPS
#define LLG_STAMP_CAP 131072
static __device__ unsigned long long g_stamps[2 * LLG_STAMP_CAP];
static __device__ unsigned int g_stamp_n;
__device__ __forceinline__ void llg_stamp(int kernel, int phase, int aux, int block) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  const unsigned i = atomicAdd(&g_stamp_n, 1u);
  if (i < (unsigned)LLG_STAMP_CAP) {
    g_stamps[2 * i] = t;
    g_stamps[2 * i + 1] = ((unsigned long long)kernel << 56) | ((unsigned long long)phase << 48) |
                          ((unsigned long long)(aux & 0xffff) << 32) | (unsigned)block;
  }
}
#define LLG_STAMP(kernel, phase, aux, block) llg_stamp(kernel, phase, aux, block)
// Copies up to `cap` (time in ns, tag) pairs to `dst` and empties the buffer; returns how many.  Synchronises the device.
LLG_API int llg_stamps_read(unsigned long long* dst, int cap) {
  unsigned n = 0, zero = 0;
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(&n, g_stamp_n, 4);
  if (n > (unsigned)LLG_STAMP_CAP) n = LLG_STAMP_CAP;
  if ((int)n > cap) n = cap;
  if (dst && n) cudaMemcpyFromSymbol(dst, g_stamps, (size_t)n * 16);
  cudaMemcpyToSymbol(g_stamp_n, &zero, 4);
  return (int)n;
}
#else
#define LLG_STAMP(kernel, phase, aux, block) ((void)0)
#endif

// ---- element access ---------------------------------------------------------------

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// ---- reductions -------------------------------------------------------------------

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  All threads get the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// Row of the paged key/value store that holds position `pos` of the sequence in `slot`,
// for key/value head `kvh`.  Pages are [n_pages][n_kv][LLG_PAGE][head_dim]; a sequence's
// logical page j lies at table[slot][j % ring_pages] (ring_pages = table width for a group
// that keeps all keys).
__device__ __forceinline__ long long kv_row(const int* __restrict__ table, int table_width,
                                            int ring_pages, int slot, int pos, int kvh, int n_kv) {
  const int lp = (pos / LLG_PAGE) % ring_pages;
  const int page = table[(long long)slot * table_width + lp];
  return ((long long)page * n_kv + kvh) * LLG_PAGE + (pos % LLG_PAGE);
}

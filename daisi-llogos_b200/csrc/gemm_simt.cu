// Matrix product on the CUDA cores: out[n][o] = sum_k x[n][k] * w[o][k], float32 accumulation
// by fused multiply-add only (no tensor cores, no reduced-precision mode).  It is the product
// of the true 32-bit path and the fallback for operand types the tensor-core kernel does not
// take.  Any n, o, k.  The reference sends float32 products to cublasSgemm / cublasSgemv
// (Daisi.Llogos.Cuda/CudaBackend.cs:506-519) and has a one-row-per-block GEMV for 16-bit
// weights (kernels/dequant_matmul.cu:593-619).
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

constexpr int BM = 64;   // rows of x (tokens) per block
constexpr int BN = 64;   // rows of w (output features) per block
constexpr int BK = 16;

template <typename AT, typename WT, typename CT>
__global__ void __launch_bounds__(256) gemm_tn_kernel(const AT* __restrict__ x, const WT* __restrict__ w,
                                                      CT* __restrict__ out, int n, int o, int k, RowScale scale) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;     // 16 x 16 threads, each a 4 x 4 sub-tile
  const int n0 = blockIdx.y * BM, o0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < k; k0 += BK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx >> 4, c = idx & 15;
      const int kk = k0 + c;
      float xv = 0.f, wv = 0.f;
      if (kk < k) {
        if (n0 + r < n) xv = to_f32(x[(long long)(n0 + r) * k + kk]);
        if (o0 + r < o) wv = to_f32(w[(long long)(o0 + r) * k + kk]);
      }
      xs[c][r] = xv;
      ws[c][r] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < BK; ++c) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[c][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[c][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = n0 + ty * 4 + i;
    if (r >= n) continue;
    const float rs = row_scale_of(scale, r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = o0 + tx * 4 + j;
      if (c < o) out[(long long)r * o + c] = from_f32<CT>(scale.ss ? acc[i][j] * rs : acc[i][j]);
    }
  }
}

}  // namespace

// With `scale` (may be null) row r of the result is multiplied by the scale that a norm left for row r of x.
LLG_API int llg_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                          int n, int o, int k, const RowScale* scale, cudaStream_t stream) {
  LLG_REQUIRE(n >= 0 && o > 0 && k > 0, "gemm_simt: bad sizes n=%d o=%d k=%d", n, o, k);
  if (n == 0) return 0;
  dim3 grid((o + BN - 1) / BN, (n + BM - 1) / BM);
  LLG_REQUIRE(grid.y <= 65535, "gemm_simt: %d rows need more than 65535 row blocks", n);
  const RowScale rs = scale ? *scale : RowScale{nullptr, 0, 0.f, 0.f};
#define LAUNCH(AT, WT, CT) \
  gemm_tn_kernel<AT, WT, CT><<<grid, 256, 0, stream>>>((const AT*)x, (const WT*)w, (CT*)out, n, o, k, rs)
  const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (key) {
    case 0: LAUNCH(float, float, float); break;
    case 1: LAUNCH(float, float, __nv_bfloat16); break;
    case 2: LAUNCH(float, __nv_bfloat16, float); break;
    case 3: LAUNCH(float, __nv_bfloat16, __nv_bfloat16); break;
    case 4: LAUNCH(__nv_bfloat16, float, float); break;
    case 5: LAUNCH(__nv_bfloat16, float, __nv_bfloat16); break;
    case 6: LAUNCH(__nv_bfloat16, __nv_bfloat16, float); break;
    case 7: LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16); break;
    default: return llg_fail("gemm_simt: unknown dtypes x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
  }
#undef LAUNCH
  return llg_check_launch("gemm_simt");
}

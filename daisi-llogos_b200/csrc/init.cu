// Filling and converting tensors on the device: counter-based normal random values, constants,
// conversions between float32 and bfloat16.
//
// The random values are a pure function of (key, element index), so that the same tensor can be made on
// the host with plain integer and double arithmetic (weights/random_init.py restates this file's
// formulas) and a model initialised on the GPU holds the weights that a model written to a file with the
// same seed holds.  The reference fills its test model from System.Random, element by element
// (tests/Daisi.Llogos.Tests/Training/TrainingForwardPassTests.cs:342-360); its device-side fill is a
// constant only (Daisi.Llogos.Cuda/kernels/elementwise.cu:1263).
//
//   h1 = splitmix64(key + 2 i), h2 = splitmix64(key + 2 i + 1)        (64-bit wrap-around)
//   u1 = ((h1 >> 11) + 1) / 2^53 in (0, 1],  u2 = (h2 >> 11) / 2^53 in [0, 1)
//   z  = sqrt(-2 ln u1) cos(2 pi u2)                                   (Box-Muller, double)
//   value = (float)(mean + std z), then rounded to the tensor's type
#include "common.cuh"

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long long n, unsigned long long key, double mean, double std) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const unsigned long long h1 = splitmix64(key + 2ull * (unsigned long long)i);
    const unsigned long long h2 = splitmix64(key + 2ull * (unsigned long long)i + 1ull);
    const double u1 = (double)((h1 >> 11) + 1ull) * (1.0 / 9007199254740992.0);
    const double u2 = (double)(h2 >> 11) * (1.0 / 9007199254740992.0);
    const double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
    // no fused multiply-add: the host restatement rounds the product and the sum separately
    out[i] = from_f32<T>(__double2float_rn(__dadd_rn(mean, __dmul_rn(std, z))));
  }
}

template <typename T>
__global__ void fill_kernel(T* __restrict__ out, long long n, float value) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const T v = from_f32<T>(value);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = v;
}

template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ src, D* __restrict__ dst, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = from_f32<D>(to_f32(src[i]));
}

inline unsigned grid_for(long long n) {
  long long blocks = (n + 255) / 256;
  const long long most = (long long)llg_sm_count() * 16;   // grid-stride loops: a few waves of blocks are enough
  if (blocks > most) blocks = most;
  return (unsigned)(blocks < 1 ? 1 : blocks);
}

}  // namespace

// out[i] = mean + std * z(key, i), rounded to float32 and then to `dtype`
LLG_API int llg_fill_normal(void* out, int dtype, long long n, unsigned long long key, double mean, double std,
                            cudaStream_t stream) {
  LLG_REQUIRE(n >= 0, "fill_normal: negative size");
  if (n == 0) return 0;
  if (dtype == LLG_F32) fill_normal_kernel<float><<<grid_for(n), 256, 0, stream>>>((float*)out, n, key, mean, std);
  else if (dtype == LLG_BF16)
    fill_normal_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>((__nv_bfloat16*)out, n, key, mean, std);
  else return llg_fail("fill_normal: unknown dtype %d", dtype);
  return llg_check_launch("fill_normal");
}

LLG_API int llg_fill(void* out, int dtype, long long n, float value, cudaStream_t stream) {
  LLG_REQUIRE(n >= 0, "fill: negative size");
  if (n == 0) return 0;
  if (dtype == LLG_F32) fill_kernel<float><<<grid_for(n), 256, 0, stream>>>((float*)out, n, value);
  else if (dtype == LLG_BF16) fill_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>((__nv_bfloat16*)out, n, value);
  else return llg_fail("fill: unknown dtype %d", dtype);
  return llg_check_launch("fill");
}

// dst[i] = (dst type) src[i]; float32 -> bfloat16 rounds to nearest even, bfloat16 -> float32 is exact
LLG_API int llg_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, cudaStream_t stream) {
  LLG_REQUIRE(n >= 0, "cast: negative size");
  if (n == 0) return 0;
  typedef __nv_bfloat16 bf;
  if (src_dtype == LLG_F32 && dst_dtype == LLG_BF16)
    cast_kernel<float, bf><<<grid_for(n), 256, 0, stream>>>((const float*)src, (bf*)dst, n);
  else if (src_dtype == LLG_BF16 && dst_dtype == LLG_F32)
    cast_kernel<bf, float><<<grid_for(n), 256, 0, stream>>>((const bf*)src, (float*)dst, n);
  else if (src_dtype == LLG_F32 && dst_dtype == LLG_F32)
    cast_kernel<float, float><<<grid_for(n), 256, 0, stream>>>((const float*)src, (float*)dst, n);
  else if (src_dtype == LLG_BF16 && dst_dtype == LLG_BF16)
    cast_kernel<bf, bf><<<grid_for(n), 256, 0, stream>>>((const bf*)src, (bf*)dst, n);
  else return llg_fail("cast: unknown dtypes %d -> %d", src_dtype, dst_dtype);
  return llg_check_launch("cast");
}

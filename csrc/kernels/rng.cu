// K12: counter-based normal fill (Philox4x32-10 + Box-Muller) and constant fill.
// Device replacement for randn / xavier / kaiming (src/init.h:11-50); the result depends only
// on (seed, offset, element index), never on the launch geometry.
#include "common.cuh"

namespace dg {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__device__ __forceinline__ void philox4x32_10(uint64_t seed, uint64_t ctr, uint32_t (&out)[4]) {
  uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

__device__ __forceinline__ float u01(uint32_t x) { return ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f); }

template <typename T>
__global__ void __launch_bounds__(256) randn_kernel(T* __restrict__ out, int64_t n, uint64_t seed, uint64_t offset,
                                                    float mean, float stdv) {
  const int64_t groups = (n + 3) / 4;
  for (int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += (int64_t)gridDim.x * blockDim.x) {
    uint32_t r[4];
    philox4x32_10(seed, offset + (uint64_t)gi, r);
    float z[4];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      float u1 = u01(r[2 * k]), u2 = u01(r[2 * k + 1]);
      float rad = sqrtf(-2.f * logf(u1));
      float s, c;
      sincospif(2.f * u2, &s, &c);
      z[2 * k] = rad * c; z[2 * k + 1] = rad * s;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      int64_t i = gi * 4 + k;
      if (i < n) stf(out, i, mean + stdv * z[k]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T* __restrict__ out, int64_t n, float value) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    stf(out, i, value);
}

}  // namespace dg

extern "C" int dg_randn(int dtype, void* out, int64_t n, uint64_t seed, uint64_t offset, float mean, float std,
                        cudaStream_t stream) {
  if (n == 0) return DG_OK;
  int blocks = dg::grid_for((n + 3) / 4, 256);
  if (dtype == DG_F32) dg::randn_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, seed, offset, mean, std);
  else if (dtype == DG_BF16)
    dg::randn_kernel<dg::bf16><<<blocks, 256, 0, stream>>>((dg::bf16*)out, n, seed, offset, mean, std);
  else return DG_ERR_BAD_ARG;
  DG_CHECK_LAUNCH();
  return DG_OK;
}

extern "C" int dg_fill(int dtype, void* out, int64_t n, float value, cudaStream_t stream) {
  if (n == 0) return DG_OK;
  int blocks = dg::grid_for(n, 256, 4);
  if (dtype == DG_F32) dg::fill_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, value);
  else if (dtype == DG_BF16) dg::fill_kernel<dg::bf16><<<blocks, 256, 0, stream>>>((dg::bf16*)out, n, value);
  else return DG_ERR_BAD_ARG;
  DG_CHECK_LAUNCH();
  return DG_OK;
}

// Exact-fp32 SIMT batched GEMM with arbitrary element strides.
// Used for fp32 tensors (the toy configs and numerics tests, where TF32/bf16 tensor-core
// rounding is not wanted) and for shapes that break the TMA alignment rules of the tcgen05
// path. 64x64 CTA tile, 16-deep k slices in shared memory, 4x4 register micro-tile per thread.
// Strides make NN/NT/TN operand layouts and stride-0 batch broadcast free of copies
// (reference semantics: src/matmul.h:86-200).
#include "common.cuh"

namespace dg {

struct SimtGemmArgs {
  int64_t M, N, K;
  int64_t a_bs, ars, acs, b_bs, brs, bcs, c_bs, crs;
  float alpha, beta;
};

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(T* __restrict__ C, const T* __restrict__ A,
                                                        const T* __restrict__ B, SimtGemmArgs g) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int64_t b = blockIdx.z;
  const T* Ab = A + b * g.a_bs;
  const T* Bb = B + b * g.b_bs;
  T* Cb = C + b * g.c_bs;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < g.K; k0 += BK) {
    // A tile: 64 x 16 elements, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int e = tid + i * 256;
      int mm, kk;
      if (g.acs == 1) { kk = e % BK; mm = e / BK; } else { mm = e % BM; kk = e / BM; }
      int64_t m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < g.M && k < g.K) ? ldf(Ab, m * g.ars + k * g.acs) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int e = tid + i * 256;
      int nn, kk;
      if (g.bcs == 1) { nn = e % BN; kk = e / BN; } else { kk = e % BK; nn = e / BK; }
      int64_t n = n0 + nn, k = k0 + kk;
      Bs[kk][nn] = (n < g.N && k < g.K) ? ldf(Bb, k * g.brs + n * g.bcs) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t m = m0 + tm + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t n = n0 + tn + j;
      if (n >= g.N) continue;
      float v = g.alpha * acc[i][j];
      if (g.beta != 0.f) v += g.beta * ldf(Cb, m * g.crs + n);
      stf(Cb, m * g.crs + n, v);
    }
  }
}

}  // namespace dg

extern "C" int dg_gemm_simt(int dtype, void* C, const void* A, const void* B, int64_t batch, int64_t M, int64_t N,
                            int64_t K, int64_t a_bs, int64_t ars, int64_t acs, int64_t b_bs, int64_t brs,
                            int64_t bcs, int64_t c_bs, int64_t crs, float alpha, float beta, cudaStream_t stream) {
  if (batch == 0 || M == 0 || N == 0) return DG_OK;
  if (batch > 65535 || (M + 63) / 64 > 65535) return DG_ERR_TOO_LARGE;
  dg::SimtGemmArgs g{M, N, K, a_bs, ars, acs, b_bs, brs, bcs, c_bs, crs, alpha, beta};
  dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64), (unsigned)batch);
  if (dtype == DG_F32)
    dg::gemm_simt_kernel<float><<<grid, 256, 0, stream>>>((float*)C, (const float*)A, (const float*)B, g);
  else if (dtype == DG_BF16)
    dg::gemm_simt_kernel<dg::bf16><<<grid, 256, 0, stream>>>((dg::bf16*)C, (const dg::bf16*)A, (const dg::bf16*)B, g);
  else
    return DG_ERR_BAD_ARG;
  DG_CHECK_LAUNCH();
  return DG_OK;
}

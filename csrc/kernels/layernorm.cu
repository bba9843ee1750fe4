// K4: LayerNorm over the last dim as one forward kernel and two backward kernels.
// Semantics follow the reference's 7-op composite (src/layernorm.h:29-39): biased variance,
// eps inside the sqrt, per-feature affine y = xhat * gamma[j] + beta[j] (the in-bounds
// reading of src/cool_ops.h:41-46). mean and rstd are saved in fp32 for the backward.
//   fwd : one warp per row, 16-byte loads, row cached in registers when d <= 32*8*VN
//   bwd : (1) dx, one warp per row; (2) dgamma/dbeta as a split column reduction through scratch
#include "common.cuh"

namespace dg {

constexpr int kLnMaxVec = 8;  // vectors cached per lane

template <typename T, bool CACHED>
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(T* __restrict__ y, float* __restrict__ mean,
                                                            float* __restrict__ rstd, const T* __restrict__ x,
                                                            const T* __restrict__ gamma, const T* __restrict__ beta,
                                                            int64_t rows, int64_t d, float eps) {
  constexpr int VN = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t nvec = d / VN;  // CACHED requires d % VN == 0
  for (int64_t row = warp; row < rows; row += nwarps) {
    const T* xr = x + row * d;
    T* yr = y + row * d;
    float mu, rs;
    if constexpr (CACHED) {
      float vals[kLnMaxVec][VN];
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < kLnMaxVec; ++k) {
        int64_t v = lane + 32 * k;
        if (v < nvec) {
          Vec16<T> t; t.load(xr + v * VN); t.unpack(vals[k]);
#pragma unroll
          for (int e = 0; e < VN; ++e) s += vals[k][e];
        }
      }
      mu = warp_sum(s) / (float)d;
      float q = 0.f;
#pragma unroll
      for (int k = 0; k < kLnMaxVec; ++k) {
        int64_t v = lane + 32 * k;
        if (v < nvec) {
#pragma unroll
          for (int e = 0; e < VN; ++e) { float t = vals[k][e] - mu; q += t * t; }
        }
      }
      rs = rsqrtf(warp_sum(q) / (float)d + eps);
#pragma unroll
      for (int k = 0; k < kLnMaxVec; ++k) {
        int64_t v = lane + 32 * k;
        if (v < nvec) {
          float gf[VN], bf[VN], of[VN];
          Vec16<T> t;
          t.load(gamma + v * VN); t.unpack(gf);
          t.load(beta + v * VN); t.unpack(bf);
#pragma unroll
          for (int e = 0; e < VN; ++e) of[e] = (vals[k][e] - mu) * rs * gf[e] + bf[e];
          t.pack(of); t.store(yr + v * VN);
        }
      }
    } else {
      float s = 0.f;
      for (int64_t j = lane; j < d; j += 32) s += ldf(xr, j);
      mu = warp_sum(s) / (float)d;
      float q = 0.f;
      for (int64_t j = lane; j < d; j += 32) { float t = ldf(xr, j) - mu; q += t * t; }
      rs = rsqrtf(warp_sum(q) / (float)d + eps);
      for (int64_t j = lane; j < d; j += 32)
        stf(yr, j, (ldf(xr, j) - mu) * rs * ldf(gamma, j) + ldf(beta, j));
    }
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
  }
}

// dx = rstd * (gh - mean(gh) - xhat * mean(gh * xhat)),  gh = g * gamma
template <typename T>
__global__ void __launch_bounds__(256) layernorm_bwd_dx_kernel(T* __restrict__ dx, const T* __restrict__ g,
                                                               const T* __restrict__ x, const T* __restrict__ gamma,
                                                               const float* __restrict__ mean,
                                                               const float* __restrict__ rstd, int64_t rows, int64_t d) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < rows; row += nwarps) {
    const T* xr = x + row * d;
    const T* gr = g + row * d;
    T* o = dx + row * d;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int64_t j = lane; j < d; j += 32) {
      float gh = ldf(gr, j) * ldf(gamma, j);
      float xh = (ldf(xr, j) - mu) * rs;
      s1 += gh; s2 += gh * xh;
    }
    s1 = warp_sum(s1) / (float)d;
    s2 = warp_sum(s2) / (float)d;
    for (int64_t j = lane; j < d; j += 32) {
      float gh = ldf(gr, j) * ldf(gamma, j);
      float xh = (ldf(xr, j) - mu) * rs;
      stf(o, j, rs * (gh - s1 - xh * s2));
    }
  }
}

// partial[s, 0, c] = sum_r g*xhat ; partial[s, 1, c] = sum_r g   over the split's rows
template <typename T>
__global__ void __launch_bounds__(256) layernorm_bwd_param_partial_kernel(float* __restrict__ partial,
                                                                          const T* __restrict__ g,
                                                                          const T* __restrict__ x,
                                                                          const float* __restrict__ mean,
                                                                          const float* __restrict__ rstd,
                                                                          int64_t rows, int64_t d,
                                                                          int64_t rows_per_split) {
  __shared__ float sg[8][33], sb[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = (int64_t)blockIdx.x * 32 + tx;
  const int64_t s = blockIdx.y;
  const int64_t r0 = s * rows_per_split;
  int64_t r1 = r0 + rows_per_split;
  if (r1 > rows) r1 = rows;
  float ag = 0.f, ab = 0.f;
  if (c < d) {
    for (int64_t r = r0 + ty; r < r1; r += 8) {
      float gv = ldf(g, r * d + c);
      float xh = (ldf(x, r * d + c) - mean[r]) * rstd[r];
      ag += gv * xh; ab += gv;
    }
  }
  sg[ty][tx] = ag; sb[ty][tx] = ab;
  __syncthreads();
  if (ty == 0 && c < d) {
    float tg = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { tg += sg[k][tx]; tb += sb[k][tx]; }
    partial[(s * 2 + 0) * d + c] = tg;
    partial[(s * 2 + 1) * d + c] = tb;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) layernorm_bwd_param_fold_kernel(T* __restrict__ dgamma, T* __restrict__ dbeta,
                                                                       const float* __restrict__ partial, int64_t d,
                                                                       int S) {
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < d; c += (int64_t)gridDim.x * blockDim.x) {
    float tg = 0.f, tb = 0.f;
    for (int s = 0; s < S; ++s) { tg += partial[(s * 2 + 0) * d + c]; tb += partial[(s * 2 + 1) * d + c]; }
    stf(dgamma, c, tg);
    stf(dbeta, c, tb);
  }
}

static inline int ln_splits(int64_t rows, int64_t d) {
  int64_t cb = (d + 31) / 32;
  int64_t want = (148 * 4 + cb - 1) / cb;
  int64_t max_s = (rows + 63) / 64;
  if (want > max_s) want = max_s;
  if (want < 1) want = 1;
  if (want > 512) want = 512;
  return (int)want;
}

template <typename T>
int launch_ln_fwd(void* y, float* mean, float* rstd, const void* x, const void* gamma, const void* beta,
                  int64_t rows, int64_t d, float eps, cudaStream_t stream) {
  constexpr int VN = Vec16<T>::N;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  bool cached = (d % VN == 0) && (d / VN <= 32 * kLnMaxVec) && al(x) && al(y) && al(gamma) && al(beta);
  int blocks = grid_for(rows, 8);
  if (cached)
    layernorm_fwd_kernel<T, true><<<blocks, 256, 0, stream>>>((T*)y, mean, rstd, (const T*)x, (const T*)gamma,
                                                              (const T*)beta, rows, d, eps);
  else
    layernorm_fwd_kernel<T, false><<<blocks, 256, 0, stream>>>((T*)y, mean, rstd, (const T*)x, (const T*)gamma,
                                                               (const T*)beta, rows, d, eps);
  DG_CHECK_LAUNCH();
  return DG_OK;
}

template <typename T>
int launch_ln_bwd(void* dx, void* dgamma, void* dbeta, const void* g, const void* x, const void* gamma,
                  const float* mean, const float* rstd, int64_t rows, int64_t d, void* scratch,
                  cudaStream_t stream) {
  int blocks = grid_for(rows, 8);
  if (dx) {
    layernorm_bwd_dx_kernel<T><<<blocks, 256, 0, stream>>>((T*)dx, (const T*)g, (const T*)x, (const T*)gamma, mean,
                                                           rstd, rows, d);
    DG_CHECK_LAUNCH();
  }
  if (dgamma && dbeta) {
    const int S = ln_splits(rows, d);
    const int64_t rps = (rows + S - 1) / S;
    dim3 grid((unsigned)((d + 31) / 32), (unsigned)S);
    layernorm_bwd_param_partial_kernel<T><<<grid, 256, 0, stream>>>((float*)scratch, (const T*)g, (const T*)x, mean,
                                                                    rstd, rows, d, rps);
    DG_CHECK_LAUNCH();
    layernorm_bwd_param_fold_kernel<T><<<grid_for(d, 256), 256, 0, stream>>>((T*)dgamma, (T*)dbeta,
                                                                             (const float*)scratch, d, S);
    DG_CHECK_LAUNCH();
  }
  return DG_OK;
}

}  // namespace dg

extern "C" int dg_layernorm_fwd(int dtype, void* y, float* mean, float* rstd, const void* x, const void* gamma,
                                const void* beta, int64_t rows, int64_t d, float eps, cudaStream_t stream) {
  if (rows == 0) return DG_OK;
  if (d <= 0) return DG_ERR_BAD_ARG;
  if (dtype == DG_F32) return dg::launch_ln_fwd<float>(y, mean, rstd, x, gamma, beta, rows, d, eps, stream);
  if (dtype == DG_BF16) return dg::launch_ln_fwd<dg::bf16>(y, mean, rstd, x, gamma, beta, rows, d, eps, stream);
  return DG_ERR_BAD_ARG;
}

extern "C" int64_t dg_layernorm_bwd_scratch_bytes(int64_t rows, int64_t d) {
  if (rows <= 0 || d <= 0) return 0;
  return (int64_t)sizeof(float) * 2 * d * dg::ln_splits(rows, d);
}

extern "C" int dg_layernorm_bwd(int dtype, void* dx, void* dgamma, void* dbeta, const void* g, const void* x,
                                const void* gamma, const float* mean, const float* rstd, int64_t rows,
                                int64_t d, void* scratch, cudaStream_t stream) {
  if (rows == 0) return DG_OK;
  if (d <= 0 || ((dgamma || dbeta) && !scratch)) return DG_ERR_BAD_ARG;
  if (dtype == DG_F32) return dg::launch_ln_bwd<float>(dx, dgamma, dbeta, g, x, gamma, mean, rstd, rows, d, scratch, stream);
  if (dtype == DG_BF16)
    return dg::launch_ln_bwd<dg::bf16>(dx, dgamma, dbeta, g, x, gamma, mean, rstd, rows, d, scratch, stream);
  return DG_ERR_BAD_ARG;
}

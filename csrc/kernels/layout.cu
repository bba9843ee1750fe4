// K10: layout kernels. A general strided copy (gather and/or scatter over up to 8
// dims) that makes any view contiguous or writes into a view (concat, slices), and a
// shared-memory tiled batched 2-D transpose. Replaces the host gather loops of the
// reference (src/engine.h:173-194, 265-275; src/concat.h:77-103).
#include "common.cuh"

namespace dg {

struct StridedDesc {
  int64_t shape[8];
  int64_t dst[8];
  int64_t src[8];
  int ndim;
  int64_t n;
};

template <typename T>
__global__ void __launch_bounds__(256) strided_copy_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                           StridedDesc d) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < d.n; i += stride) {
    int64_t rem = i, so = 0, dof = 0;
#pragma unroll 1
    for (int k = d.ndim - 1; k >= 0; --k) {
      int64_t q = rem / d.shape[k];
      int64_t idx = rem - q * d.shape[k];
      rem = q;
      so += idx * d.src[k];
      dof += idx * d.dst[k];
    }
    dst[dof] = src[so];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) transpose2d_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                          int64_t R, int64_t C) {
  __shared__ T tile[32][33];
  const int64_t b = blockIdx.z;
  const T* src = in + b * R * C;
  T* dst = out + b * R * C;
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    int64_t r = r0 + ty + j, c = c0 + tx;
    if (r < R && c < C) tile[ty + j][tx] = src[r * C + c];
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    int64_t c = c0 + ty + j, r = r0 + tx;
    if (r < R && c < C) dst[c * R + r] = tile[tx][ty + j];
  }
}

}  // namespace dg

extern "C" int dg_strided_copy(int dtype, void* dst, const int64_t* dst_strides, const void* src,
                               const int64_t* src_strides, const int64_t* shape, int ndim,
                               cudaStream_t stream) {
  if (ndim < 1 || ndim > 8) return DG_ERR_BAD_ARG;
  dg::StridedDesc d;
  d.ndim = ndim;
  d.n = 1;
  for (int i = 0; i < ndim; ++i) {
    d.shape[i] = shape[i];
    d.dst[i] = dst_strides[i];
    d.src[i] = src_strides[i];
    d.n *= shape[i];
  }
  for (int i = ndim; i < 8; ++i) { d.shape[i] = 1; d.dst[i] = 0; d.src[i] = 0; }
  if (d.n == 0) return DG_OK;
  int blocks = dg::grid_for(d.n, 256, 2);
  if (dtype == DG_F32)
    dg::strided_copy_kernel<float><<<blocks, 256, 0, stream>>>((float*)dst, (const float*)src, d);
  else if (dtype == DG_BF16)
    dg::strided_copy_kernel<dg::bf16><<<blocks, 256, 0, stream>>>((dg::bf16*)dst, (const dg::bf16*)src, d);
  else
    return DG_ERR_BAD_ARG;
  DG_CHECK_LAUNCH();
  return DG_OK;
}

extern "C" int dg_transpose2d(int dtype, void* out, const void* in, int64_t B, int64_t R, int64_t C,
                              cudaStream_t stream) {
  if (B == 0 || R == 0 || C == 0) return DG_OK;
  if (B > 65535 || (R + 31) / 32 > 65535) return DG_ERR_TOO_LARGE;
  dim3 grid((unsigned)((C + 31) / 32), (unsigned)((R + 31) / 32), (unsigned)B);
  if (dtype == DG_F32)
    dg::transpose2d_kernel<float><<<grid, 256, 0, stream>>>((float*)out, (const float*)in, R, C);
  else if (dtype == DG_BF16)
    dg::transpose2d_kernel<dg::bf16><<<grid, 256, 0, stream>>>((dg::bf16*)out, (const dg::bf16*)in, R, C);
  else
    return DG_ERR_BAD_ARG;
  DG_CHECK_LAUNCH();
  return DG_OK;
}

// K6: embedding as a row gather (with an optional fused positional-table add) and a
// scatter-add backward, replacing the reference's dense one-hot matmul
// (src/embedding.h:19-22, src/init.h:53-65). Also the float->int index conversion the
// reference API needs (indices arrive as float tensors) and one_hot itself.
#include "common.cuh"

namespace dg {

template <typename T>
__global__ void __launch_bounds__(256) embedding_fwd_kernel(T* __restrict__ out, const T* __restrict__ table,
                                                            const int64_t* __restrict__ idx,
                                                            const T* __restrict__ pos_table,
                                                            const int64_t* __restrict__ pos_idx, int64_t n, int64_t d,
                                                            int64_t vocab, bool vec) {
  constexpr int VN = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t t = warp; t < n; t += nwarps) {
    int64_t row = idx[t];
    if (row < 0 || row >= vocab) row = 0;  // bounds are validated on the host side of the API
    const T* src = table + row * d;
    const T* ps = pos_table ? pos_table + pos_idx[t] * d : nullptr;
    T* dst = out + t * d;
    if (vec) {
      for (int64_t v = lane; v < d / VN; v += 32) {
        Vec16<T> a; a.load(src + v * VN);
        if (ps) {
          Vec16<T> b; b.load(ps + v * VN);
          float af[VN], bf[VN];
          a.unpack(af); b.unpack(bf);
#pragma unroll
          for (int e = 0; e < VN; ++e) af[e] += bf[e];
          a.pack(af);
        }
        a.store(dst + v * VN);
      }
    } else {
      for (int64_t j = lane; j < d; j += 32) stf(dst, j, ldf(src, j) + (ps ? ldf(ps, j) : 0.f));
    }
  }
}

__device__ __forceinline__ void atomic_add_t(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_t(bf16* p, float v) { atomicAdd(p, __float2bfloat16_rn(v)); }

template <typename T>
__global__ void __launch_bounds__(256) embedding_bwd_kernel(T* __restrict__ dtable, const T* __restrict__ g,
                                                            const int64_t* __restrict__ idx, int64_t n, int64_t d,
                                                            int64_t vocab) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t t = warp; t < n; t += nwarps) {
    int64_t row = idx[t];
    if (row < 0 || row >= vocab) continue;
    T* dst = dtable + row * d;
    const T* src = g + t * d;
    if constexpr (sizeof(T) == 2) {
      // bf16x2 atomics when the row is 4-byte aligned and d is even
      if ((d & 1) == 0 && ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 3u) == 0) {
        for (int64_t j = lane; j < d / 2; j += 32) {
          __nv_bfloat162 v = reinterpret_cast<const __nv_bfloat162*>(src)[j];
          atomicAdd(reinterpret_cast<__nv_bfloat162*>(dst) + j, v);
        }
        continue;
      }
    }
    for (int64_t j = lane; j < d; j += 32) atomic_add_t(dst + j, ldf(src, j));
  }
}

__global__ void index_from_float_kernel(int64_t* __restrict__ out, const float* __restrict__ in, int64_t n,
                                        int64_t limit, int* __restrict__ bad) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t v = (int64_t)in[i];
    if (v < 0 || v >= limit) { if (bad) atomicExch(bad, 1); v = 0; }
    out[i] = v;
  }
}

__global__ void one_hot_kernel(float* __restrict__ out, const int64_t* __restrict__ idx, int64_t n, int64_t classes) {
  const int64_t total = n * classes;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t t = i / classes, c = i - t * classes;
    out[i] = (idx[t] == c) ? 1.f : 0.f;
  }
}

}  // namespace dg

extern "C" int dg_embedding_fwd(int dtype, void* out, const void* table, const int64_t* idx, const void* pos_table,
                                const int64_t* pos_idx, int64_t n, int64_t d, int64_t vocab, cudaStream_t stream) {
  if (n == 0 || d == 0) return DG_OK;
  if (pos_table && !pos_idx) return DG_ERR_BAD_ARG;
  int blocks = dg::grid_for(n, 8);
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (dtype == DG_F32) {
    bool vec = (d % 4 == 0) && al(out) && al(table) && (!pos_table || al(pos_table));
    dg::embedding_fwd_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, (const float*)table, idx,
                                                                (const float*)pos_table, pos_idx, n, d, vocab, vec);
  } else if (dtype == DG_BF16) {
    bool vec = (d % 8 == 0) && al(out) && al(table) && (!pos_table || al(pos_table));
    dg::embedding_fwd_kernel<dg::bf16><<<blocks, 256, 0, stream>>>((dg::bf16*)out, (const dg::bf16*)table, idx,
                                                                   (const dg::bf16*)pos_table, pos_idx, n, d, vocab, vec);
  } else {
    return DG_ERR_BAD_ARG;
  }
  DG_CHECK_LAUNCH();
  return DG_OK;
}

extern "C" int dg_embedding_bwd(int dtype, void* dtable, const void* g, const int64_t* idx, int64_t n, int64_t d,
                                int64_t vocab, cudaStream_t stream) {
  if (n == 0 || d == 0) return DG_OK;
  int blocks = dg::grid_for(n, 8);
  if (dtype == DG_F32)
    dg::embedding_bwd_kernel<float><<<blocks, 256, 0, stream>>>((float*)dtable, (const float*)g, idx, n, d, vocab);
  else if (dtype == DG_BF16)
    dg::embedding_bwd_kernel<dg::bf16><<<blocks, 256, 0, stream>>>((dg::bf16*)dtable, (const dg::bf16*)g, idx, n, d, vocab);
  else
    return DG_ERR_BAD_ARG;
  DG_CHECK_LAUNCH();
  return DG_OK;
}

extern "C" int dg_index_from_float(int64_t* out, const float* in, int64_t n, int64_t limit, int* bad,
                                   cudaStream_t stream) {
  if (n == 0) return DG_OK;
  dg::index_from_float_kernel<<<dg::grid_for(n, 256), 256, 0, stream>>>(out, in, n, limit, bad);
  DG_CHECK_LAUNCH();
  return DG_OK;
}

extern "C" int dg_one_hot(float* out, const int64_t* idx, int64_t n, int64_t classes, cudaStream_t stream) {
  if (n == 0 || classes == 0) return DG_OK;
  dg::one_hot_kernel<<<dg::grid_for(n * classes, 256, 4), 256, 0, stream>>>(out, idx, n, classes);
  DG_CHECK_LAUNCH();
  return DG_OK;
}

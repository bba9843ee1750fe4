// Small device-runtime surface exported from the kernel library so that host-only C++ code
// (the reference-API shim headers) can allocate, copy and synchronise without including or
// linking the CUDA runtime itself. Allocation is stream-ordered (cudaMallocAsync on the
// device's default memory pool), so a tensor-per-op front end does not serialise the GPU.
#include "common.cuh"

extern "C" {

int dg_rt_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

int dg_rt_malloc(void** p, size_t bytes, cudaStream_t stream) {
  if (bytes == 0) bytes = 4;
  cudaError_t e = cudaMallocAsync(p, bytes, stream);
  return (int)e;
}

int dg_rt_free(void* p, cudaStream_t stream) {
  if (!p) return 0;
  return (int)cudaFreeAsync(p, stream);
}

int dg_rt_memset(void* p, int value, size_t bytes, cudaStream_t stream) {
  return (int)cudaMemsetAsync(p, value, bytes, stream);
}

int dg_rt_h2d(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(stream);  // pageable source: finish before the caller reuses it
}

int dg_rt_d2h(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(stream);
}

int dg_rt_d2d(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  return (int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
}

int dg_rt_sync(cudaStream_t stream) { return (int)cudaStreamSynchronize(stream); }

const char* dg_rt_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

}  // extern "C"

// Host-side helper that builds TMA tensor maps (cuTensorMapEncodeTiled) without linking
// libcuda: the driver entry point is fetched through the runtime at first use, so the library
// also loads on machines that have no driver (build checks on CPU-only hosts).
#pragma once
#include <cuda.h>
#include <cuda_runtime_api.h>
#include <stdint.h>

namespace dg {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

// bf16 3-D map {inner, outer, batch} with a {box_inner, box_outer, 1} box and 128-byte swizzle.
// Strides are in elements. Returns 0 on success.
inline int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t batch,
                             uint64_t outer_stride, uint64_t batch_stride, uint32_t box_inner, uint32_t box_outer) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return -3;
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {outer_stride * 2, batch_stride * 2};
  if (batch <= 1) strides[1] = outer_stride * 2 * outer;
  if (strides[1] == 0) strides[1] = 16;
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}


// 3-D map for an output tensor of bf16 (esize 2) or fp32 (esize 4) elements, 128-byte swizzle.
inline int make_tmap_out_3d(CUtensorMap* out, int esize, const void* base, uint64_t inner, uint64_t outer,
                            uint64_t batch, uint64_t outer_stride, uint64_t batch_stride, uint32_t box_inner,
                            uint32_t box_outer) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return -3;
  cuuint64_t dims[3] = {inner, outer, batch < 1 ? 1 : batch};
  cuuint64_t strides[2] = {outer_stride * esize, batch_stride * esize};
  if (batch <= 1 || strides[1] == 0) strides[1] = outer_stride * esize * outer;
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// bf16 4-D map {d0 (contiguous), d1, d2, d3} with element strides s1, s2, s3 and a
// {box0, box1, 1, 1} box, 128-byte swizzle. Used for [B, S, H, dk] attention operands.
inline int make_tmap_bf16_4d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                             uint64_t s1, uint64_t s2, uint64_t s3, uint32_t box0, uint32_t box1) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return -3;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1 * 2, s2 * 2, s3 * 2};
  cuuint32_t box[4] = {box0, box1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}


// fp32 4-D map {d0 (contiguous), d1, d2, d3}, {32, box1, 1, 1} box (128-byte rows), 128-byte swizzle:
// the destination of the TMA reduce-add that accumulates dQ tiles.
inline int make_tmap_f32_4d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                            uint64_t s1, uint64_t s2, uint64_t s3, uint32_t box1) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return -3;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1 * 4, s2 * 4, s3 * 4};
  cuuint32_t box[4] = {32, box1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace dg

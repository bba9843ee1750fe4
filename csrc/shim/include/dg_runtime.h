// C++ front end with the reference's public API (global-namespace Tensor / Node / Edge,
// std::shared_ptr<Tensor> values, free-function ops) on top of the sm_100a kernel library.
//
// A Tensor's storage is a device buffer plus a lazily synchronised host mirror:
//   * ops read/write the device copy (kernels are enqueued on one stream, in order);
//   * data_ptr()/grad_ptr()/data_at()/grad_at()/fill()/show() use the host mirror, which is
//     downloaded on demand; data_ptr() hands out a mutable pointer, so the host copy becomes
//     authoritative and is uploaded before the next device use.
// This keeps the raw-pointer idioms of reference programs working (src/engine.h:100-135,
// src/transformer.h:98, src/mars.cpp:116,207,244) while all arithmetic runs on the GPU.
//
// Only this header tree and libdgb200.so are needed to build a program: no CUDA headers.
#pragma once
#include <algorithm>
#include <cassert>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <iostream>
#include <memory>
#include <queue>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

extern "C" {
int dg_rt_device_count(void);
int dg_rt_malloc(void** p, size_t bytes, void* stream);
int dg_rt_free(void* p, void* stream);
int dg_rt_memset(void* p, int value, size_t bytes, void* stream);
int dg_rt_h2d(void* dst, const void* src, size_t bytes, void* stream);
int dg_rt_d2h(void* dst, const void* src, size_t bytes, void* stream);
int dg_rt_d2d(void* dst, const void* src, size_t bytes, void* stream);
int dg_rt_sync(void* stream);
const char* dg_rt_error_string(int code);
int dg_elementwise(int op, int dtype, void* out, const void* x, const void* y, const void* z, const void* w,
                   int ymode, int zmode, int wmode, float s0, float s1, int64_t n, int64_t r, int64_t c, void* stream);
int dg_accumulate(int dtype, void* dst, const void* src, int64_t n, void* stream);
int dg_strided_copy(int dtype, void* dst, const int64_t* dst_strides, const void* src, const int64_t* src_strides,
                    const int64_t* shape, int ndim, void* stream);
int dg_reduce_rows(int dtype, void* out, void* mean_out, const void* x, int64_t R, int64_t C, int mode, void* stream);
int64_t dg_reduce_cols_scratch_bytes(int64_t B, int64_t R, int64_t C);
int dg_reduce_cols(int dtype, void* out, void* mean_out, const void* x, int64_t B, int64_t R, int64_t C, int mode,
                   void* scratch, void* stream);
int dg_sum_all(int dtype, void* out, const void* x, int64_t n, float scale, void* scratch, void* stream);
int dg_softmax_fwd(int dtype, void* out, const void* x, const void* mask, int mask_mode, float scale, int64_t rows,
                   int64_t r, int64_t c, void* stream);
int dg_softmax_bwd(int dtype, void* gx, const void* g, const void* out, const void* mask, int mask_mode, float scale,
                   int64_t rows, int64_t r, int64_t c, void* stream);
int dg_embedding_fwd(int dtype, void* out, const void* table, const int64_t* idx, const void* pos_table,
                     const int64_t* pos_idx, int64_t n, int64_t d, int64_t vocab, void* stream);
int dg_embedding_bwd(int dtype, void* dtable, const void* g, const int64_t* idx, int64_t n, int64_t d, int64_t vocab,
                     void* stream);
int dg_index_from_float(int64_t* out, const float* in, int64_t n, int64_t limit, int* bad, void* stream);
int dg_one_hot(float* out, const int64_t* idx, int64_t n, int64_t classes, void* stream);
int dg_adam_step(int p_dtype, void* p, float* master, int g_dtype, const void* g, float* m, float* v, int64_t n,
                 float lr, float beta1, float beta2, float eps, float wd, int step, float grad_scale, void* stream);
int dg_sgd_step(int p_dtype, void* p, float* master, int g_dtype, const void* g, int64_t n, float lr, float grad_scale,
                void* stream);
int dg_randn(int dtype, void* out, int64_t n, uint64_t seed, uint64_t offset, float mean, float std, void* stream);
int dg_fill(int dtype, void* out, int64_t n, float value, void* stream);
int dg_gemm_simt(int dtype, void* C, const void* A, const void* B, int64_t batch, int64_t M, int64_t N, int64_t K,
                 int64_t a_bs, int64_t ars, int64_t acs, int64_t b_bs, int64_t brs, int64_t bcs, int64_t c_bs,
                 int64_t crs, float alpha, float beta, void* stream);
}

namespace dgshim {

// opcode / mode constants of the kernel library (csrc/include/dgb200.h)
enum { BC_SAME = 0, BC_ROW, BC_COL, BC_SCALAR, BC_MAT, BC_ROWS, BC_COLS };
enum {
  EW_COPY = 0, EW_ADD, EW_SUB, EW_MUL, EW_DIV, EW_ADD_S, EW_MUL_S, EW_DIV_S, EW_RSUB_S, EW_RDIV_S, EW_POW_I, EW_SQRT,
  EW_LOG_EPS, EW_EXP, EW_RELU, EW_TANH, EW_GELU, EW_NEG, EW_COPY_Y, EW_MASK_FILL, EW_CAUSAL_FILL, EW_CLAMP, EW_FMA_S,
  EW_DIV_BWD_B, EW_POW_BWD, EW_SQRT_BWD, EW_LOG_BWD, EW_RDIV_BWD, EW_RELU_BWD, EW_TANH_BWD, EW_GELU_BWD, EW_MASK_BWD,
  EW_CAUSAL_BWD, EW_VAR_BWD, EW_STD_BWD, EW_XENT_PROB_BWD, EW_MSE_BWD, EW_SCALE_SHIFT
};
enum { RED_SUM = 0, RED_MEAN, RED_VAR, RED_STD };

inline void check(int rc, const char* what) {
  if (rc == 0) return;
  std::string msg = std::string(what) + " failed: ";
  msg += rc > 0 ? dg_rt_error_string(rc) : ("library error " + std::to_string(rc));
  throw std::runtime_error(msg);
}

inline void* stream() { return nullptr; }  // the legacy default stream: ordered with everything

// A device allocation that frees itself (stream-ordered).
struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  explicit DevBuf(size_t b, bool zero = false) : bytes(b) {
    check(dg_rt_malloc(&p, b, stream()), "device allocation");
    if (zero) check(dg_rt_memset(p, 0, b ? b : 4, stream()), "memset");
  }
  ~DevBuf() { if (p) dg_rt_free(p, stream()); }
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
};

}  // namespace dgshim

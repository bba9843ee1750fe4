// C ABI of the fused compute+collective kernels (part of libdgb200.so).
// All peer pointers come from symmetric allocations that every rank of the node has mapped;
// flag pads are int32 arrays in the same kind of memory. Waits inside the kernels are bounded:
// on expiry a non-zero code is written to *status and the kernel returns normally.
#pragma once
#include <stdint.h>
#include <cuda_runtime_api.h>
#include "dgb200.h"

#ifdef __cplusplus
extern "C" {
#endif

// F1 + F2(store side): reduce-scatter + optimizer + parameter all-gather for one bucket.
// Flag pad layout (int32): ready[n_buckets][world] then done[n_buckets][world].
typedef struct {
  const void* const* grad_ptrs;   // device array [world]: base of every rank's bf16 gradient buffer
  void* const* param_ptrs;        // device array [world]: base of every rank's bf16 parameter buffer
  int* const* flag_ptrs;          // device array [world]: base of every rank's flag pad
  float* master;                  // this rank's fp32 master slice of the bucket [shard_n]
  float* m;                       // Adam first moment slice (null for SGD)
  float* v;                       // Adam second moment slice (null for SGD)
  int64_t bucket_off;             // element offset of the bucket in the flat buffers
  int64_t shard_n;                // elements per rank (bucket = world * shard_n), multiple of 8
  int rank, world, bucket_id, n_buckets;
  int epoch;                      // strictly increasing per use of the flag pad
  int step;                       // Adam step (>= 1)
  float lr, beta1, beta2, eps, wd, grad_scale;
  int optimizer;                  // 0 Adam/AdamW, 1 SGD
  int* counter;                   // device int, zero-initialised, one per bucket
  int* status;                    // device (or mapped host) int for error codes; may be null
  int max_ctas;                   // cap on the grid (0: default) so backward GEMMs keep their SMs
  long long wait_cycles;          // budget of each bounded wait (0: default, about two seconds)
} dg_rs_optim_args;
int dg_rs_optim(const dg_rs_optim_args* args, cudaStream_t stream);

// Wait until flags[i] >= epoch for i < n (one tiny kernel; bounded).
int dg_flags_wait(const int* flags, int n, int epoch, int* status, long long wait_cycles, cudaStream_t stream);
// pads[r][offset] = value for every rank r (system-scope release store).
int dg_flags_signal(int* const* pads_dev, int world, int offset, int value, cudaStream_t stream);

// F3: all-gather -> GEMM.  C[M, N_local] = gather_rows(A_shard)[M, K] * B[K, N_local]
//   Every rank holds rows [rank*M/W, (rank+1)*M/W) of A. A gather role inside the same kernel
//   copies peer rows into this rank's full-A buffer chunk by chunk and raises per-chunk flags;
//   the GEMM role's TMA producer waits on the flag of the chunk it is about to load and starts
//   with the locally owned rows.
typedef struct {
  const void* const* a_shard_ptrs; // device array [world]: every rank's A shard [M/W, K] bf16 (row stride lda)
  void* a_full;                    // this rank's gathered A [M, K] bf16 (row stride lda); own rows already in place or copied too
  const void* B;                   // [K, N] (b_kmajor=0) or [N, K] (b_kmajor=1) bf16
  void* D;                         // [M, N] bf16/fp32
  const void* bias;
  int64_t M, N, K, lda, ldb, ldd;
  int b_kmajor, out_dtype, bias_dtype, epi;
  int rank, world;
  int* chunk_flags;                // device int [M / chunk_rows], local memory
  int* const* flag_ptrs;           // peer flag pads (ready handshake), int32
  int flag_offset;                 // first of `world` ints in each pad used by this call
  int epoch;
  int copy_ctas;                   // CTAs reserved for the gather role (0: default)
  int* status;
  long long wait_cycles;
} dg_ag_gemm_args;
int dg_ag_gemm(const dg_ag_gemm_args* args, cudaStream_t stream);

// F4: GEMM -> reduce-scatter.  C_local[M/W, N] = sum over ranks of (A_r[M, K_local] * B_r[K_local, N]) rows of this rank.
//   Finished fp32-accumulated tiles are written as bf16 partials straight into the owner rank's
//   staging slot for this source, followed by a per-tile flag; reducer CTAs of the same kernel
//   sum the `world` partials of each owned tile in fp32 and write the output.
typedef struct {
  const void* A;                   // [M, K_local] bf16 row-major (lda)
  const void* B;                   // [K_local, N] or [N, K_local] bf16
  void* const* staging_ptrs;       // device array [world]: every rank's staging buffer [world][M/W, N] bf16
  int* const* tile_flag_ptrs;      // device array [world]: every rank's per-(source, tile) flags
  void* D;                         // [M/W, N] bf16/fp32 output of this rank
  const void* bias;                // added once by the owner
  const void* residual;            // [M/W, N] added by the owner (may alias D)
  int64_t M, N, K, lda, ldb, ldd;
  int b_kmajor, out_dtype, bias_dtype;
  int rank, world;
  int epoch;
  int reduce_ctas;                 // CTAs reserved for the reducer role (0: default)
  int* status;
  long long wait_cycles;
} dg_gemm_rs_args;
int dg_gemm_rs(const dg_gemm_rs_args* args, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

// F3 / F4: tensor-parallel GEMMs fused with their collective, over NVLink peer memory.
//
// Both kernels are the persistent tcgen05 GEMM (gemm_sm100.cuh) with part of the grid given a
// communication role, so tensor-core tiles and NVLink traffic overlap tile by tile inside ONE
// launch; no NCCL call and no library GEMM touches peer memory.
//
//   dg_ag_gemm  (all-gather -> GEMM): copy CTAs pull the peers' row blocks of A into this GPU's
//               own memory with 16-byte peer loads and raise a flag per 128-row block; the GEMM
//               CTAs' TMA producer waits for the block's flag and then loads it LOCALLY (a
//               remote tile never feeds a TMA load directly, and nothing is multicast).
//   dg_gemm_rs  (GEMM -> reduce-scatter): the epilogue writes each finished bf16 partial tile
//               into the owning rank's staging slot with peer stores and publishes a per-tile
//               flag; reducer CTAs sum the partials of their own tiles in fp32 in rank order.
// Every wait on a peer is bounded and reports through *status.
#include <cstring>
#include "../kernels/gemm_sm100.cuh"
#include "../kernels/tma_host.h"
#include "peer.cuh"
#include "../include/dgb200_comm.h"

namespace dg {
namespace sm100 {

int get_tmap(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t batch, uint64_t ostride,
             uint64_t bstride, uint32_t box_inner, uint32_t box_outer);   // gemm_sm100.cu
int sm_count();

constexpr int kTpBN = 256;
constexpr int kTpStages = 4;

struct AgRole {
  void* const* a_full_ptrs;
  int* const* flag_ptrs;
  int* chunk_flags;
  int64_t M, K, lda;
  int rank, world, epoch, copy_ctas;
  int* status;
  long long wait_cycles;
};

// Gather role of one copy CTA. Blocks of 128 rows are taken round-robin over the copy CTAs in the
// order peer = rank+1, rank+2, ... so that data arrives in the order the GEMM consumes it.
__device__ __forceinline__ void ag_copy_role(const AgRole& r, int cta, int* s_ok) {
  const int W = r.world;
  const int64_t rows_per_rank = r.M / W;
  const int64_t blocks_per_rank = rows_per_rank / 128;
  int* my_pad = r.flag_ptrs[r.rank];
  // handshake: my rows are final (stream order put this kernel after their producer)
  if (cta == 0 && threadIdx.x == 0) {
    __threadfence_system();
    for (int q = 0; q < W; ++q) peer::st_release_sys(r.flag_ptrs[q] + r.rank, r.epoch);
  }
  if (cta == 0) {
    // locally owned blocks are ready by construction
    for (int64_t i = threadIdx.x; i < blocks_per_rank; i += blockDim.x)
      peer::st_release_sys(r.chunk_flags + r.rank * blocks_per_rank + i, r.epoch);
  }
  bool ok = true;
  const int64_t total = (int64_t)(W - 1) * blocks_per_rank;
  uint8_t* dst_base = reinterpret_cast<uint8_t*>(r.a_full_ptrs[r.rank]);
  int last_src = -1;
  for (int64_t i = cta; i < total; i += r.copy_ctas) {
    const int src = (r.rank + 1 + (int)(i / blocks_per_rank)) % W;
    const int64_t blk = (int64_t)src * blocks_per_rank + i % blocks_per_rank;
    if (src != last_src) {
      if (threadIdx.x == 0) *s_ok = peer::wait_flag(my_pad + src, r.epoch, r.wait_cycles) ? 1 : 0;
      __syncthreads();
      ok = *s_ok != 0;
      __syncthreads();
      if (!ok) break;
      last_src = src;
    }
    const uint8_t* src_base = reinterpret_cast<const uint8_t*>(r.a_full_ptrs[src]);
    const int64_t row0 = blk * 128;
    const int64_t units_per_row = r.K / 8;            // 16-byte units
    const int64_t units = 128 * units_per_row;
    for (int64_t u0 = threadIdx.x; u0 < units; u0 += (int64_t)blockDim.x * 8) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int64_t u = u0 + (int64_t)k * blockDim.x;
        if (u < units) {
          const int64_t row = row0 + u / units_per_row, col = (u % units_per_row) * 16;
          v[k] = peer::ld_peer_16(src_base + row * r.lda * 2 + col);
        }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int64_t u = u0 + (int64_t)k * blockDim.x;
        if (u < units) {
          const int64_t row = row0 + u / units_per_row, col = (u % units_per_row) * 16;
          *reinterpret_cast<uint4*>(dst_base + row * r.lda * 2 + col) = v[k];
        }
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) peer::st_release_sys(r.chunk_flags + blk, r.epoch);
  }
  if (!ok && threadIdx.x == 0 && r.status) atomicExch(r.status, 0x300 | r.rank);
}

template <bool B_K>
__global__ void __launch_bounds__(kGemmThreads, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
               const AgRole r, int* done_counter) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_ok;
  const int gemm_ctas = (int)gridDim.x - r.copy_ctas;
  if ((int)blockIdx.x < gemm_ctas) {
    gemm_cta_body<kTpBN, kTpStages, true, B_K, bf16, true, false>(&tmA, &tmB, nullptr, nullptr, p, smem_raw,
                                                                 (int)blockIdx.x, gemm_ctas);
    return;
  }
  const int cta = (int)blockIdx.x - gemm_ctas;
  ag_copy_role(r, cta, &s_ok);
  // Leave only after every peer has finished reading this rank's rows: tell each peer that this
  // rank is done reading (last copy CTA to finish), then wait for the same word from all of them.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(done_counter, 1);
    if (prev == r.copy_ctas - 1) {
      *done_counter = 0;
      for (int q = 0; q < r.world; ++q) peer::st_release_sys(r.flag_ptrs[q] + r.world + r.rank, r.epoch);
      bool ok = true;
      for (int q = 0; q < r.world && ok; ++q) ok = peer::wait_flag(r.flag_ptrs[r.rank] + r.world + q, r.epoch, r.wait_cycles);
      if (!ok && r.status) atomicExch(r.status, 0x340 | r.rank);
    }
  }
}

struct RsRole {
  const bf16* staging;
  const int* tile_flags;
  int* const* done_flag_ptrs;
  bf16* D;
  const void* bias;
  const bf16* residual;
  int64_t rows_per_rank, N, ldd;
  int bias_dtype, rank, world, epoch, reduce_ctas;
  int* status;
  long long wait_cycles;
};

// Reducer role: owned tiles (128 x kTpBN) round-robin over the reducer CTAs.
__device__ __forceinline__ void rs_reduce_role(const RsRole& r, int cta, int* s_ok) {
  const int W = r.world;
  const int64_t n_tiles = (r.N + kTpBN - 1) / kTpBN, m_tiles = r.rows_per_rank / 128;
  const int64_t tiles = m_tiles * n_tiles;
  const int64_t slot = r.rows_per_rank * r.N;        // elements per source slot
  bool ok = true;
  for (int64_t t = cta; t < tiles && ok; t += r.reduce_ctas) {
    // same tile numbering as the producers' flags: ltile = local m tile * n_tiles + n tile
    if (threadIdx.x < W) {
      // rank-rotated wait order does not matter for correctness; every source must have published
      if (!peer::wait_flag(r.tile_flags + (int64_t)threadIdx.x * tiles + t, r.epoch, r.wait_cycles)) atomicExch(s_ok, 0);
    }
    __syncthreads();
    ok = *s_ok != 0;
    if (!ok) break;
    const int64_t mt = t / n_tiles, nt = t % n_tiles;
    const int64_t row0 = mt * 128, col0 = nt * kTpBN;
    const int64_t ncols = (r.N - col0) < kTpBN ? (r.N - col0) : kTpBN;
    const int64_t units_per_row = ncols / 8;
    for (int64_t u = threadIdx.x; u < 128 * units_per_row; u += blockDim.x) {
      const int64_t row = row0 + u / units_per_row, col = col0 + (u % units_per_row) * 8;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < W; ++s) {                  // fixed rank order: deterministic
        uint4 raw = peer::ld_peer_16(r.staging + (int64_t)s * slot + row * r.N + col);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) { float2 f = __bfloat1622float2(h[k]); acc[2 * k] += f.x; acc[2 * k + 1] += f.y; }
      }
      if (r.bias) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          acc[k] += r.bias_dtype == DG_BF16 ? __bfloat162float(reinterpret_cast<const bf16*>(r.bias)[col + k])
                                            : reinterpret_cast<const float*>(r.bias)[col + k];
      }
      if (r.residual) {
        uint4 raw = *reinterpret_cast<const uint4*>(r.residual + row * r.ldd + col);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) { float2 f = __bfloat1622float2(h[k]); acc[2 * k] += f.x; acc[2 * k + 1] += f.y; }
      }
      uint4 out;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int k = 0; k < 4; ++k) oh[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
      *reinterpret_cast<uint4*>(r.D + row * r.ldd + col) = out;
    }
    __syncthreads();
  }
  if (!ok && threadIdx.x == 0 && r.status) atomicExch(r.status, 0x400 | r.rank);
}

template <bool B_K>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
               const RsRole r, const int* my_done_flags, int* done_counter) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_ok;
  const int gemm_ctas = (int)gridDim.x - r.reduce_ctas;
  // The staging slots this call writes were last read by their owners' reducers in the previous
  // call: wait until every owner has reported that call finished.
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int q = 0; q < r.world && ok; ++q) ok = peer::wait_flag(my_done_flags + q, r.epoch - 1, r.wait_cycles) ? 1 : 0;
    if (!ok && r.status) atomicExch(r.status, 0x440 | r.rank);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  if ((int)blockIdx.x < gemm_ctas) {
    gemm_cta_body<kTpBN, kTpStages, true, B_K, bf16, false, true>(&tmA, &tmB, nullptr, nullptr, p, smem_raw,
                                                                 (int)blockIdx.x, gemm_ctas);
    return;
  }
  rs_reduce_role(r, (int)blockIdx.x - gemm_ctas, &s_ok);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(done_counter, 1);
    if (prev == r.reduce_ctas - 1) {
      *done_counter = 0;
      for (int q = 0; q < r.world; ++q) peer::st_release_sys(r.done_flag_ptrs[q] + r.rank, r.epoch);
    }
  }
}

static int* tp_counter() {   // one zero-initialised device int per process for last-CTA detection
  static int* c = nullptr;
  if (!c) {
    if (cudaMalloc(&c, 2 * sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(c, 0, 2 * sizeof(int));
  }
  return c;
}

}  // namespace sm100
}  // namespace dg

extern "C" int dg_ag_gemm(const dg_ag_gemm_args* a, cudaStream_t stream) {
  using namespace dg::sm100;
  if (!a || !a->a_full_ptrs || !a->B || !a->D || !a->chunk_flags || !a->flag_ptrs) return DG_ERR_BAD_ARG;
  if (a->world < 1 || a->rank < 0 || a->rank >= a->world) return DG_ERR_BAD_ARG;
  if (a->M % (128 * a->world) || a->K % 8 || a->lda % 8 || a->ldb % 8 || a->ldd % 8) return DG_ERR_UNSUPPORTED;
  int copy_ctas = a->world > 1 ? (a->copy_ctas > 0 ? a->copy_ctas : 16) : 1;
  const int sms = sm_count();
  if (copy_ctas >= sms) return DG_ERR_BAD_ARG;
  void* a_local = a->a_local;
  if (!a_local) return DG_ERR_BAD_ARG;
  CUtensorMap tmA, tmB;
  if (get_tmap(&tmA, a_local, a->K, a->M, 1, a->lda, 0, kBK, kBM)) return DG_ERR_DRIVER;
  int rc = a->b_kmajor ? get_tmap(&tmB, a->B, a->K, a->N, 1, a->ldb, 0, kBK, kTpBN)
                       : get_tmap(&tmB, a->B, a->N, a->K, 1, a->ldb, 0, 64, kBK);
  if (rc) return DG_ERR_DRIVER;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = a->M; p.N = a->N; p.K = a->K; p.batch = 1;
  p.ldd = a->ldd; p.d_bs = a->M * a->ldd; p.D = a->D; p.bias = a->bias; p.bias_dtype = a->bias_dtype; p.epi = a->epi;
  p.alpha = 1.0f; p.status = a->status; p.a_bcast = 1; p.b_bcast = 1;
  p.a_flags = a->chunk_flags; p.a_epoch = a->epoch; p.rows_per_chunk = 128;
  p.m_tile_rotate = (int64_t)a->rank * (a->M / a->world) / 128;
  AgRole r;
  r.a_full_ptrs = a->a_full_ptrs; r.flag_ptrs = a->flag_ptrs; r.chunk_flags = a->chunk_flags;
  r.M = a->M; r.K = a->K; r.lda = a->lda; r.rank = a->rank; r.world = a->world; r.epoch = a->epoch;
  r.copy_ctas = copy_ctas; r.status = a->status;
  r.wait_cycles = a->wait_cycles > 0 ? a->wait_cycles : dg::peer::kFlagWaitCycles;
  int* counter = tp_counter();
  if (!counter) return DG_ERR_DRIVER;
  using SM = GemmSmem<kTpBN, kTpStages>;
  auto launch = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal);
    if (e != cudaSuccess) return (int)e;
    const int64_t tiles = (a->M / 128) * ((a->N + kTpBN - 1) / kTpBN);
    int gemm_ctas = (int)(tiles < sms - copy_ctas ? tiles : sms - copy_ctas);
    kern<<<gemm_ctas + copy_ctas, kGemmThreads, SM::kTotal, stream>>>(tmA, tmB, p, r, counter);
    cudaError_t le = cudaGetLastError();
    return le == cudaSuccess ? DG_OK : (int)le;
  };
  return a->b_kmajor ? launch(ag_gemm_kernel<true>) : launch(ag_gemm_kernel<false>);
}

extern "C" int dg_gemm_rs(const dg_gemm_rs_args* a, cudaStream_t stream) {
  using namespace dg::sm100;
  if (!a || !a->A || !a->B || !a->D || !a->dest_slots || !a->tile_flag_ptrs || !a->done_flag_ptrs || !a->staging ||
      !a->tile_flags || !a->done_flags)
    return DG_ERR_BAD_ARG;
  if (a->world < 1 || a->rank < 0 || a->rank >= a->world || a->epoch < 1) return DG_ERR_BAD_ARG;
  if (a->M % (128 * a->world) || a->N % 8 || a->K % 8 || a->lda % 8 || a->ldb % 8 || a->ldd % 8) return DG_ERR_UNSUPPORTED;
  const int sms = sm_count();
  int reduce_ctas = a->reduce_ctas > 0 ? a->reduce_ctas : 16;
  if (reduce_ctas >= sms) return DG_ERR_BAD_ARG;
  CUtensorMap tmA, tmB;
  if (get_tmap(&tmA, a->A, a->K, a->M, 1, a->lda, 0, kBK, kBM)) return DG_ERR_DRIVER;
  int rc = a->b_kmajor ? get_tmap(&tmB, a->B, a->K, a->N, 1, a->ldb, 0, kBK, kTpBN)
                       : get_tmap(&tmB, a->B, a->N, a->K, 1, a->ldb, 0, 64, kBK);
  if (rc) return DG_ERR_DRIVER;
  const int64_t rows_per_rank = a->M / a->world;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = a->M; p.N = a->N; p.K = a->K; p.batch = 1;
  p.ldd = a->N; p.d_bs = 0; p.D = nullptr; p.alpha = 1.0f; p.status = a->status; p.a_bcast = 1; p.b_bcast = 1;
  p.dest_base = a->dest_slots; p.rows_per_dest = rows_per_rank; p.dest_flags = a->tile_flag_ptrs;
  p.src_rank = a->rank; p.d_epoch = a->epoch;
  // start with the tiles owned by the next rank so that all links carry data from the beginning
  p.m_tile_rotate = (int64_t)((a->rank + 1) % a->world) * rows_per_rank / 128;
  RsRole r;
  r.staging = (const dg::bf16*)a->staging; r.tile_flags = a->tile_flags; r.done_flag_ptrs = a->done_flag_ptrs;
  r.D = (dg::bf16*)a->D; r.bias = a->bias; r.residual = (const dg::bf16*)a->residual;
  r.rows_per_rank = rows_per_rank; r.N = a->N; r.ldd = a->ldd; r.bias_dtype = a->bias_dtype;
  r.rank = a->rank; r.world = a->world; r.epoch = a->epoch; r.reduce_ctas = reduce_ctas; r.status = a->status;
  r.wait_cycles = a->wait_cycles > 0 ? a->wait_cycles : dg::peer::kFlagWaitCycles;
  int* counter = tp_counter();
  if (!counter) return DG_ERR_DRIVER;
  using SM = GemmSmem<kTpBN, kTpStages>;
  auto launch = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal);
    if (e != cudaSuccess) return (int)e;
    const int64_t tiles = (a->M / 128) * ((a->N + kTpBN - 1) / kTpBN);
    int gemm_ctas = (int)(tiles < sms - reduce_ctas ? tiles : sms - reduce_ctas);
    kern<<<gemm_ctas + reduce_ctas, kGemmThreads, SM::kTotal, stream>>>(tmA, tmB, p, r, a->done_flags, counter + 1);
    cudaError_t le = cudaGetLastError();
    return le == cudaSuccess ? DG_OK : (int)le;
  };
  return a->b_kmajor ? launch(gemm_rs_kernel<true>) : launch(gemm_rs_kernel<false>);
}

// K3 (forward): fused attention  O = softmax(mask(scale * Q K^T)) V  on tcgen05 tensor cores.
//
// One CTA per (128-query tile, head, batch). Q, K, V, O are addressed in place in the
// [B, S, H, dk] layout the projections produce (4-D TMA maps), so there are no head
// split/merge copies and the S x S score matrix never reaches HBM (the reference materialises
// three of them per layer: src/attention.h:84-90, src/masking.h:98, src/softmax.h:46).
//
//   warp 0      TMA producer: Q once, then a ring of K and V tiles (128 keys each)
//   warp 1      MMA issuer:   S_j = Q K_j^T  -> TMEM (double-buffered),
//                             PV_j = P_j V_j -> TMEM (double-buffered)
//   warps 2-5   softmax: thread = query row. Reads S_j from TMEM, online max / sum in base 2,
//               writes P_j (bf16) into shared memory in the 128-byte-swizzled K-major layout the
//               second MMA consumes, accumulates O in registers:  O = (O + PV_{j-1}) * alpha_j
// QK^T of tile j+1 is issued before the softmax of tile j finishes, so tensor cores and the
// exp pipeline overlap. Causal tiles above the diagonal are skipped; masked scores get
// probability exactly 0, which equals the reference's -1e9 fill after the max-subtracted exp.
#include <cstring>
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace dg {
namespace sm100 {

constexpr int kAttnThreads = 192;
constexpr int kQT = 128;   // query rows per CTA
constexpr int kKT = 128;   // keys per tile

struct AttnFwdParams {
  bf16* o;
  float* lse;
  int64_t B, H, S;
  int64_t o_row, o_bs;
  float scale_log2;   // scale * log2(e)
  int causal;
  int* status;
};

template <int DK>
struct AttnFwdSmem {
  static constexpr int kStages = 2;
  static constexpr int kTileBytes = 128 * DK * 2;       // one Q / K / V tile
  static constexpr int kPBytes = 128 * 128 * 2;
  static constexpr int kBars = 1 + 4 * kStages + 2 + 2 + 1 + 1 + 2 + 2;
  static constexpr int kTotal = kTileBytes * (1 + 2 * kStages) + kPBytes + 512;   // dk = 64: two CTAs fit one SM
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int DK>
__global__ void __launch_bounds__(kAttnThreads, DK == 64 ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using SM = AttnFwdSmem<DK>;
  constexpr int STG = SM::kStages;
  constexpr int NCH = DK / 64;                     // 64-column chunks per tile row
  constexpr uint32_t kIdescQK = make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t kIdescPV = make_idesc_bf16(128, DK, 0, 1);   // B = V is MN-major
  // dk = 64: one S buffer + two PV buffers = 256 TMEM columns, so two CTAs share an SM and hide each
  // other's softmax latency; dk = 128: two S buffers + two PV buffers = 512 columns, one CTA per SM.
  constexpr bool kDoubleS = (DK == 128);
  constexpr uint32_t kTmemCols = kDoubleS ? 512 : 256;
  constexpr uint32_t kPVCol = kDoubleS ? 256 : 128;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {   // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 0x10);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + SM::kTileBytes;
  uint8_t* sV = sK + STG * SM::kTileBytes;
  uint8_t* sP = sV + STG * SM::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + SM::kPBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + STG;
  uint64_t* v_full = k_empty + STG;
  uint64_t* v_empty = v_full + STG;
  uint64_t* s_full = v_empty + STG;     // [2]
  uint64_t* s_free = s_full + 2;        // [2]
  uint64_t* p_ready = s_free + 2;
  uint64_t* p_free = p_ready + 1;
  uint64_t* pv_full = p_free + 1;       // [2]
  uint64_t* pv_free = pv_full + 2;      // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_free + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (int)((p.S + kQT - 1) / kQT);
  const int qt = q_tiles - 1 - (int)blockIdx.x;     // heaviest (longest) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * kQT;
  const int kv_tiles_all = (int)((p.S + kKT - 1) / kKT);
  const int n_tiles = p.causal ? (qt + 1 < kv_tiles_all ? qt + 1 : kv_tiles_all) : kv_tiles_all;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STG; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&s_full[a], 1); mbar_init(&s_free[a], 4); mbar_init(&pv_full[a], 1); mbar_init(&pv_free[a], 4); }
    mbar_init(p_ready, 128);
    mbar_init(p_free, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) { tmem_alloc(tmem_holder, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(q_full, SM::kTileBytes);
#pragma unroll
      for (int c = 0; c < NCH; ++c) tma_load_4d(sQ + c * 16384, &tmQ, q_full, c * 64, q0, h, b);
      int stage = 0; uint32_t phase = 0;
      for (int j = 0; j < n_tiles && ok; ++j) {
        ok = bounded_wait(&k_empty[stage], phase ^ 1u, abort_flag);
        if (!ok) break;
        mbar_expect_tx(&k_full[stage], SM::kTileBytes);
#pragma unroll
        for (int c = 0; c < NCH; ++c) tma_load_4d(sK + stage * SM::kTileBytes + c * 16384, &tmK, &k_full[stage], c * 64, j * kKT, h, b);
        ok = bounded_wait(&v_empty[stage], phase ^ 1u, abort_flag);
        if (!ok) break;
        mbar_expect_tx(&v_full[stage], SM::kTileBytes);
#pragma unroll
        for (int c = 0; c < NCH; ++c) tma_load_4d(sV + stage * SM::kTileBytes + c * 16384, &tmV, &v_full[stage], c * 64, j * kKT, h, b);
        if (++stage == STG) { stage = 0; phase ^= 1u; }
      }
      if (!ok) { if (p.status) atomicExch(p.status, 0x11); *abort_flag = 1; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = bounded_wait(q_full, 0, abort_flag);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      int kstage = 0; uint32_t kphase = 0;
      int vstage = 0; uint32_t vphase = 0;
      auto issue_qk = [&](int j) -> bool {
        const int sb = kDoubleS ? (j & 1) : 0;
        const int use = kDoubleS ? (j >> 1) : j;
        if (!bounded_wait(&k_full[kstage], kphase, abort_flag)) return false;
        if (!bounded_wait(&s_free[sb], (use & 1) ^ 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + kstage * SM::kTileBytes);
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
          const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
          umma_f16(tmem_base + sb * 128, make_smem_desc(aQ + off, 16, 1024), make_smem_desc(aK + off, 16, 1024),
                   kIdescQK, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        umma_commit(&k_empty[kstage]);
        if (++kstage == STG) { kstage = 0; kphase ^= 1u; }
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) { ok = issue_qk(j + 1); if (!ok) break; }
        const int pb = j & 1;
        ok = bounded_wait(p_ready, j & 1, abort_flag) && bounded_wait(&v_full[vstage], vphase, abort_flag) &&
             bounded_wait(&pv_free[pb], ((j >> 1) & 1) ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + vstage * SM::kTileBytes);
#pragma unroll
        for (int t = 0; t < kKT / 16; ++t) {
          const uint64_t da = make_smem_desc(aP + (t / 4) * 16384 + (t % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(aV + t * 2048, 16384, 1024);
          umma_f16(tmem_base + kPVCol + pb * DK, da, db, kIdescPV, t > 0 ? 1u : 0u);
        }
        umma_commit(&pv_full[pb]);
        umma_commit(&v_empty[vstage]);
        umma_commit(p_free);
        if (++vstage == STG) { vstage = 0; vphase ^= 1u; }
      }
      if (!ok) { if (p.status) atomicExch(p.status, 0x12); *abort_flag = 1; }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output (warps 2..5)
    const int lg = warp & 3;
    const int row_in_tile = lg * 32 + lane;
    const int64_t row = (int64_t)q0 + row_in_tile;
    const uint32_t lane_base = (uint32_t)(lg * 32) << 16;
    float m = -INFINITY, l = 0.f;
    float acc[DK];
#pragma unroll
    for (int e = 0; e < DK; ++e) acc[e] = 0.f;
    bool ok = true;
    uint8_t* prow = sP + row_in_tile * 128;
    const int sw = row_in_tile & 7;

    auto add_pv = [&](int j, float alpha) -> bool {
      // acc = (acc + PV_j) * alpha, then release the PV buffer
      const int pb = j & 1;
      bool w = bounded_wait(&pv_full[pb], (j >> 1) & 1, abort_flag);
      w = __all_sync(0xffffffffu, w);
      if (!w) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DK / 32; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem_base + lane_base + kPVCol + pb * DK + c * 32, raw);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[c * 32 + e] = (acc[c * 32 + e] + __uint_as_float(raw[e])) * alpha;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pv_free[pb]);
      return true;
    };

    for (int j = 0; j < n_tiles; ++j) {
      const int sb = kDoubleS ? (j & 1) : 0;
      ok = bounded_wait(&s_full[sb], (kDoubleS ? (j >> 1) : j) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * kKT;
      const bool need_mask = (p.causal && j == qt) || (key0 + kKT > p.S);
      // pass 1: row maximum of this tile
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 2
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem_base + lane_base + sb * 128 + c * 32, raw);
        tc_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int64_t key = key0 + c * 32 + e;
            if (key >= p.S || (p.causal && key > row)) raw[e] = 0xff800000u;   // -inf
          }
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(raw[e]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float alpha = (m == -INFINITY) ? 0.f : ex2_approx(m - m_new);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      // P buffer must have been consumed by the previous PV MMA
      if (j > 0) {
        ok = bounded_wait(p_free, (j - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      // pass 2: probabilities -> shared memory (bf16, swizzled K-major), row sum
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem_base + lane_base + sb * 128 + c * 32, raw);
        tc_wait_ld();
        float pr[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) pr[e] = ex2_approx(fmaf(__uint_as_float(raw[e]), p.scale_log2, -m_use));
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int64_t key = key0 + c * 32 + e;
            if (key >= p.S || (p.causal && key > row)) pr[e] = 0.f;
          }
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) ls4[e & 3] += pr[e];
        uint8_t* chunk_base = prow + (c >> 1) * 16384;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 pk;
          __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(pr[q * 8 + 2 * e], pr[q * 8 + 2 * e + 1]);
          const int q16 = (c & 1) * 4 + q;
          *reinterpret_cast<uint4*>(chunk_base + ((q16 ^ sw) << 4)) = pk;
        }
      }
      // S buffer fully read: release it; publish P to the async proxy
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(p_ready);
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);
      l = l * alpha + ((ls4[0] + ls4[1]) + (ls4[2] + ls4[3]));
      if (j > 0) { ok = add_pv(j - 1, alpha); if (!ok) break; }
      m = m_new;
    }
    if (ok && n_tiles > 0) ok = add_pv(n_tiles - 1, 1.0f);
    if (ok) {
      if (row < p.S) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* orow = p.o + (int64_t)b * p.o_bs + row * p.o_row + (int64_t)h * DK;
#pragma unroll
        for (int q = 0; q < DK / 8; ++q) {
          uint4 pk;
          __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(acc[q * 8 + 2 * e] * inv, acc[q * 8 + 2 * e + 1] * inv);
          *reinterpret_cast<uint4*>(orow + q * 8) = pk;
        }
        if (p.lse) p.lse[((int64_t)b * p.H + h) * p.S + row] = (m + log2f(l)) * 0.6931471805599453f;
      }
    } else if (lane == 0) {
      if (p.status) atomicExch(p.status, 0x13);
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

template <int DK>
int launch_attn_fwd(const dg_attn_fwd_args* a, cudaStream_t stream) {
  using SM = AttnFwdSmem<DK>;
  CUtensorMap tq, tk, tv;
  if (make_tmap_bf16_4d(&tq, a->q, DK, a->S, a->H, a->B, a->q_row, DK, a->q_bs, 64, 128)) return DG_ERR_DRIVER;
  if (make_tmap_bf16_4d(&tk, a->k, DK, a->S, a->H, a->B, a->k_row, DK, a->k_bs, 64, 128)) return DG_ERR_DRIVER;
  if (make_tmap_bf16_4d(&tv, a->v, DK, a->S, a->H, a->B, a->v_row, DK, a->v_bs, 64, 128)) return DG_ERR_DRIVER;
  AttnFwdParams p;
  p.o = (bf16*)a->o; p.lse = a->lse; p.B = a->B; p.H = a->H; p.S = a->S;
  p.o_row = a->o_row; p.o_bs = a->o_bs;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.causal = a->causal; p.status = a->status;
  auto kern = attn_fwd_kernel<DK>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((unsigned)((a->S + kQT - 1) / kQT), (unsigned)a->H, (unsigned)a->B);
  kern<<<grid, kAttnThreads, SM::kTotal, stream>>>(tq, tk, tv, p);
  DG_CHECK_LAUNCH();
  return DG_OK;
}

}  // namespace sm100
}  // namespace dg

extern "C" int dg_attention_fwd_sm100(const dg_attn_fwd_args* a, cudaStream_t stream) {
  if (!a || !a->q || !a->k || !a->v || !a->o) return DG_ERR_BAD_ARG;
  if (a->B < 1 || a->H < 1 || a->S < 1 || a->B > 65535 || a->H > 65535) return DG_ERR_BAD_ARG;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al(a->q) || !al(a->k) || !al(a->v) || !al(a->o)) return DG_ERR_UNSUPPORTED;
  if (a->q_row % 8 || a->k_row % 8 || a->v_row % 8 || a->o_row % 8 || a->q_bs % 8 || a->k_bs % 8 || a->v_bs % 8 ||
      a->o_bs % 8)
    return DG_ERR_UNSUPPORTED;
  if (a->dk == 64) return dg::sm100::launch_attn_fwd<64>(a, stream);
  if (a->dk == 128) return dg::sm100::launch_attn_fwd<128>(a, stream);
  return DG_ERR_UNSUPPORTED;
}

// Warp-specialised tcgen05 GEMM main loop shared by the plain, grouped and
// collective-fused GEMM kernels.
//
//   acc[lane p, column q] = sum_k P[p0 + p, k] * Q[q0 + q, k]      (both operands K-major)
//
// P supplies the 128 TMEM lanes (UMMA M = 128), Q supplies BN TMEM columns (UMMA N = BN).
// A CTA has 6 warps: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 =
// epilogue (each owns the 32-lane TMEM quadrant `warp & 3`). Operand tiles are 64 bf16
// (128 bytes) wide, stored with the 128-byte swizzle by TMA and consumed by
// tcgen05.mma through shared-memory descriptors; accumulators live in TMEM.
//
// Which operand is the activation and which the weight is the caller's choice: for
// decode-sized problems (few tokens) the weight goes on the lanes ("swap-AB") so that a
// 128-row weight tile streams from HBM at full width while the handful of tokens ride on
// the N dimension; for prefill-sized problems the activation goes on the lanes.
#pragma once
#include "sm100.cuh"

namespace gv {
namespace gemm {

constexpr int BM = 128;        // TMEM lanes per tile
constexpr int BK = 64;         // bf16 elements per 128-byte swizzled row
constexpr int UMMA_K = 16;     // bf16 MMA depth
constexpr int NUM_THREADS = 192;

// BUDGET_KB: shared-memory budget of one CTA. 220 KB = one CTA per SM with the deepest ring
// (compute-bound tiles); 108 KB lets two CTAs share an SM, which evens out the last wave of the
// bandwidth-bound decode shapes.
template <int BN_, int BUDGET_KB = 220>
struct Cfg {
  static constexpr int BN = BN_;
  static constexpr int SMEM_BUDGET = BUDGET_KB * 1024;
  static constexpr int P_BYTES = BM * BK * 2;
  static constexpr int Q_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
  static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 10 ? 10 : STAGES_RAW;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr int RED_BYTES = BM * BN * 4;  // fp32 tile for split-K exchange
  static_assert(STAGES * STAGE_BYTES >= RED_BYTES, "reduce tile must fit in the stage ring");
  // stage ring + barriers + tmem slot + alignment slack
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

// Weight tiles of the kernel that follows in the stream: once this CTA's producer has issued its
// last load (the epilogue phase starts, HBM would go idle), it prefetches the first `stages`
// k-blocks of some of the follower's (tile, k-split) work items into L2. `tm` = tensor map of the
// follower's weight with the same [128 rows x 64 columns] box.
struct NextWeights {
  const CUtensorMap* tm;   // null: nothing to prefetch
  int tiles, splitk, kb_per, kb_total, stages;
};

struct Shared {
  uint8_t* ring;        // 1024-aligned stage ring
  uint64_t* full;       // [STAGES]
  uint64_t* empty;      // [STAGES]
  uint64_t* tmem_full;  // [1]
  uint32_t* tmem_slot;  // [1]
};

template <class C>
__device__ __forceinline__ Shared carve(uint8_t* raw) {
  Shared s;
  uintptr_t a = (reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023);
  s.ring = reinterpret_cast<uint8_t*>(a);
  uint8_t* tail = s.ring + C::STAGES * C::STAGE_BYTES;
  s.full = reinterpret_cast<uint64_t*>(tail);
  s.empty = s.full + C::STAGES;
  s.tmem_full = s.empty + C::STAGES;
  s.tmem_slot = reinterpret_cast<uint32_t*>(s.tmem_full + 1);
  return s;
}

// Runs the barrier/TMEM set-up and the producer + MMA roles for k-blocks [kb0, kb0 + nkb).
// Every thread of the CTA must call it. On return all roles have converged on nothing yet:
// epilogue warps should next call `wait_accum`. Returns the TMEM base address.
//
// `pdl_dep` handles programmatic dependent launch inside the loop: 0 = the caller has already
// waited (or the kernel is launched without the attribute); 1 = operand P is constant (weights)
// and Q is produced by the kernel in front; 2 = the reverse. With 1 or 2 the set-up and the first
// ring-full of constant-operand tiles are fetched BEFORE waiting for the predecessor, so weight
// streaming starts while the previous kernel drains; every thread has waited by the time
// run_mainloop returns. 3 = as 1 without the early trigger for the kernel behind.
template <class C>
__device__ __forceinline__ uint32_t run_mainloop(const Shared& sh, const CUtensorMap* tmP,
                                                 const CUtensorMap* tmQ, int p0, int q0, int kb0,
                                                 int nkb, unsigned int* status, int pz = -1,
                                                 int qz = -1, int pdl_mode = 0,
                                                 const NextWeights* next = nullptr) {
  constexpr int BN = C::BN;
  const int warp = threadIdx.x >> 5;
  // 3 = as 1, but the kernel behind this one is not let in early
  const int pdl_dep = pdl_mode == 3 ? 1 : pdl_mode;
  if (pdl_mode == 1 || pdl_mode == 2) pdl_trigger();
  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(tmP);
    sm100::tma_prefetch_desc(tmQ);
    for (int s = 0; s < C::STAGES; ++s) {
      sm100::mbar_init(&sh.full[s], 1);
      sm100::mbar_init(&sh.empty[s], 1);
    }
    sm100::mbar_init(sh.tmem_full, 1);
    sm100::mbar_fence_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc(sh.tmem_slot, C::TMEM_COLS);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(sh.tmem_slot);

  if (warp == 0) {
    if (sm100::elect_one()) {
      int pre = 0;
      if (pdl_dep) {
        pre = nkb < C::STAGES ? nkb : C::STAGES;
        for (int i = 0; i < pre; ++i) {  // fresh ring: every slot is free
          uint8_t* sp = sh.ring + i * C::STAGE_BYTES;
          sm100::mbar_expect_tx(&sh.full[i], C::STAGE_BYTES);
          const int kx = (kb0 + i) * BK;
          if (pdl_dep == 1) {
            if (pz >= 0) sm100::tma_load_3d(sp, tmP, &sh.full[i], kx, p0, pz);
            else sm100::tma_load_2d(sp, tmP, &sh.full[i], kx, p0);
          } else {
            if (qz >= 0) sm100::tma_load_3d(sp + C::P_BYTES, tmQ, &sh.full[i], kx, q0, qz);
            else sm100::tma_load_2d(sp + C::P_BYTES, tmQ, &sh.full[i], kx, q0);
          }
        }
        pdl_wait();
        for (int i = 0; i < pre; ++i) {
          uint8_t* sp = sh.ring + i * C::STAGE_BYTES;
          const int kx = (kb0 + i) * BK;
          if (pdl_dep == 2) {
            if (pz >= 0) sm100::tma_load_3d(sp, tmP, &sh.full[i], kx, p0, pz);
            else sm100::tma_load_2d(sp, tmP, &sh.full[i], kx, p0);
          } else {
            if (qz >= 0) sm100::tma_load_3d(sp + C::P_BYTES, tmQ, &sh.full[i], kx, q0, qz);
            else sm100::tma_load_2d(sp + C::P_BYTES, tmQ, &sh.full[i], kx, q0);
          }
        }
      }
      for (int i = pre; i < nkb; ++i) {
        const int s = i % C::STAGES;
        const uint32_t ph = (uint32_t)(i / C::STAGES) & 1u;
        if (!sm100::mbar_wait(&sh.empty[s], ph ^ 1u)) {
          atomicOr(status, GV_ST_TIMEOUT_TMA);
          break;
        }
        uint8_t* sp = sh.ring + s * C::STAGE_BYTES;
        uint8_t* sq = sp + C::P_BYTES;
        sm100::mbar_expect_tx(&sh.full[s], C::STAGE_BYTES);
        const int kx = (kb0 + i) * BK;
        if (pz >= 0) sm100::tma_load_3d(sp, tmP, &sh.full[s], kx, p0, pz);
        else sm100::tma_load_2d(sp, tmP, &sh.full[s], kx, p0);
        if (qz >= 0) sm100::tma_load_3d(sq, tmQ, &sh.full[s], kx, q0, qz);
        else sm100::tma_load_2d(sq, tmQ, &sh.full[s], kx, q0);
      }
      if (next != nullptr && next->tm != nullptr) {
        const int total = next->tiles * next->splitk;
        const int me = (int)(blockIdx.x + gridDim.x * blockIdx.z), step = (int)(gridDim.x * gridDim.z);
        for (int j = me; j < total; j += step) {
          const int tile = j % next->tiles, z = j / next->tiles;
          for (int s = 0; s < next->stages; ++s) {
            const int kb = z * next->kb_per + s;
            if (kb >= next->kb_total) break;
            sm100::tma_prefetch_l2_2d(next->tm, kb * BK, tile * BM);
          }
        }
      }
    } else if (pdl_dep) {
      pdl_wait();
    }
  } else if (warp == 1) {
    if (pdl_dep) pdl_wait();
    if (sm100::elect_one()) {
      constexpr uint32_t idesc = sm100::make_idesc(BM, BN, 1, 1);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % C::STAGES;
        const uint32_t ph = (uint32_t)(i / C::STAGES) & 1u;
        if (!sm100::mbar_wait(&sh.full[s], ph)) {
          atomicOr(status, GV_ST_TIMEOUT_MMA);
          ok = false;
          break;
        }
        sm100::tc_fence_after();
        const uint32_t pa = sm100::smem_u32(sh.ring + s * C::STAGE_BYTES);
        const uint64_t da = sm100::smem_desc_sw128(pa);
        const uint64_t db = sm100::smem_desc_sw128(pa + C::P_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // advancing 16 bf16 = 32 bytes inside the swizzle atom: +2 in 16-byte units
          sm100::mma_f16_ss(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                            (uint32_t)((i | k) != 0));
        }
        sm100::tc_commit(&sh.empty[s]);
      }
      sm100::tc_commit(sh.tmem_full);
    }
  } else if (pdl_dep) {
    pdl_wait();
  }
  return tmem_base;
}

// Epilogue warps: wait until the accumulator tile is complete.
__device__ __forceinline__ bool wait_accum(const Shared& sh, unsigned int* status) {
  bool ok = sm100::mbar_wait(sh.tmem_full, 0);
  __syncwarp();
  if (!ok && (threadIdx.x & 31) == 0) atomicOr(status, GV_ST_TIMEOUT_EPI);
  sm100::tc_fence_after();
  return ok;
}

// Must be called by every thread after the epilogue is done with TMEM.
template <class C>
__device__ __forceinline__ void finish(const Shared& sh, uint32_t tmem_base) {
  sm100::tc_fence_before();
  __syncthreads();
  if ((threadIdx.x >> 5) == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// TMEM address of (lane quadrant of this warp, column c).
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int quadrant, int col) {
  return base + ((uint32_t)(quadrant * 32) << 16) + (uint32_t)col;
}

// ---- cluster helpers (split-K exchange through distributed shared memory) ------------
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ float ld_dsmem_f32(const float* local_ptr, uint32_t cta_rank) {
  uint32_t a = sm100::smem_u32(local_ptr), r;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(cta_rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(r) : "memory");
  return v;
}

// 16-byte read of a peer CTA's shared memory. Callers issue all their loads first and consume
// them afterwards so that the (long-latency) DSMEM reads overlap.
__device__ __forceinline__ float4 ld_dsmem_v4(const float* local_ptr, uint32_t cta_rank) {
  uint32_t a = sm100::smem_u32(local_ptr), r;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(cta_rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(r));
  return v;
}

// Sum of the fp32 partial at `local_ptr` (4 consecutive lanes) over the `splitk` CTAs of the
// cluster, in cluster-rank order.
__device__ __forceinline__ float4 cluster_sum4(const float* local_ptr, int splitk) {
  float4 v[8];
#pragma unroll
  for (int s = 0; s < 8; ++s)
    if (s < splitk) v[s] = ld_dsmem_v4(local_ptr, (uint32_t)s);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int s = 0; s < 8; ++s)
    if (s < splitk) {
      acc.x += v[s].x;
      acc.y += v[s].y;
      acc.z += v[s].z;
      acc.w += v[s].w;
    }
  return acc;
}

}  // namespace gemm
}  // namespace gv

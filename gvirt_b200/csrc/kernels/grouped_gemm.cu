// Grouped (per-expert) bf16 GEMM on tcgen05:  out[r, :] = xs[r, :] . w[e]^T for the rows r of
// expert e's segment [offsets[e], offsets[e+1]).
//
// Reference: `group_matmul_<T>` (xlite/csrc/kernels/group_matmul.h:57, host
// xlite/csrc/op.cpp:879-903) — reads the per-expert row counts and a weight pointer table on the
// device and rotates the starting core per expert. Here segment offsets are also read on the
// device (no host synchronisation after routing) and the decomposition is by tile: a persistent
// grid of two CTAs per SM walks the tile list (column tiles of every segment x N / 128 lane
// tiles) that each CTA derives from a prefix sum over the segment table, so the launch does not
// depend on the routing outcome and costs nothing when few rows arrived. Orientation is weight-major: a 128-row slab of the expert's weight sits
// on the TMEM lanes (3-D TMA map over [E, N, K]) and up to BN routed tokens sit on the columns,
// so small per-expert batches still stream full-width weight tiles.
#include "gemm_core.cuh"
#include "gvirt_kernels.h"
#include <map>
#include <mutex>
#include <tuple>

namespace gv {
namespace gemm {

int cached_tmap_bf16(CUtensorMap* out, const void* base, long long rows, long long cols,
                     long long row_stride_elems, int box_rows);

constexpr int GG_MAX_SEGMENTS = 512;  // prefix table in static shared memory (2 KB)

// PERSISTENT: the grid is a fixed number of CTAs (two per SM); each walks the tile list
// t = blockIdx.x, + gridDim.x, ... derived on the device from a prefix sum over the segments'
// column-tile counts, tile t = (column tile t / tilesN, weight-row tile t % tilesN). The operand
// ring keeps running across tiles and the accumulator is double-buffered in TMEM, so the
// epilogue of one tile overlaps the K loop of the next.
//
// SWIGLU: the weight holds gate and up rows interleaved in blocks of 32 = [16 gate | 16 up] rows of
// the same 16 features, so that both halves of a feature sit in one TMEM quadrant, 16 lanes
// apart: the epilogue warp pairs them with one shuffle and writes
//     out[row, f] = silu(gate) * up        (out is [rows, N / 2])
// without the [rows, N] intermediate ever reaching memory. `clamp` > 0 bounds gate from above and
// up on both sides first (the reference's clamped SwiGLU).
template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(NUM_THREADS, 2)
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmW,
                         const __grid_constant__ CUtensorMap tmX, bf16* __restrict__ out,
                         const int* __restrict__ seg_start, const int* __restrict__ seg_end_arr, int N,
                         int K, int G, int e_mod, long long ldo, int tilesN, float clamp,
                         unsigned int* status) {
  using C = Cfg<BN, 108>;
  constexpr int TCOLS = 2 * BN < 32 ? 32 : 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_prefix[GG_MAX_SEGMENTS + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();  // the segment table is written by the kernels in front
  pdl_trigger();
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    const int rows = seg_end_arr[g] - seg_start[g];
    s_prefix[g + 1] = rows > 0 ? (rows + BN - 1) / BN : 0;
  }
  if (threadIdx.x == 0) s_prefix[0] = 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int g = 1; g <= G; ++g) {
      run += s_prefix[g];
      s_prefix[g] = run;
    }
  }
  __syncthreads();
  const long long total_tiles = (long long)s_prefix[G] * tilesN;
  struct Tile {
    int e, q0, seg_end, p0;
  };
  auto locate = [&](long long t) {
    Tile r;
    r.p0 = (int)(t % tilesN) * BM;
    const int ct = (int)(t / tilesN);
    int lo = 0, hi = G - 1;  // last g with prefix[g] <= ct
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_prefix[mid] <= ct) lo = mid;
      else hi = mid - 1;
    }
    r.e = e_mod > 0 ? lo % e_mod : lo;  // weight index of this row segment
    r.q0 = seg_start[lo] + (ct - s_prefix[lo]) * BN;
    r.seg_end = seg_end_arr[lo];
    return r;
  };
  const int nkb = (K + BK - 1) / BK;

  uintptr_t base = (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023);
  uint8_t* ring = reinterpret_cast<uint8_t*>(base);
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tfull = empty + C::STAGES;   // [2] accumulator buffer complete
  uint64_t* tempty = tfull + 2;          // [2] accumulator buffer drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  static_assert((2 * C::STAGES + 4) * 8 + 4 <= 256, "barriers must fit behind the ring");

  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(&tmW);
    sm100::tma_prefetch_desc(&tmX);
    for (int s = 0; s < C::STAGES; ++s) {
      sm100::mbar_init(&full[s], 1);
      sm100::mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      sm100::mbar_init(&tfull[b], 1);
      sm100::mbar_init(&tempty[b], 4);  // one arrival per epilogue warp
    }
    sm100::mbar_fence_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc(tmem_slot, TCOLS);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    if (sm100::elect_one()) {
      uint32_t gk = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Tile tl = locate(t);
        for (int i = 0; i < nkb; ++i, ++gk) {
          const int s = gk % C::STAGES;
          if (!sm100::mbar_wait(&empty[s], ((gk / C::STAGES) & 1u) ^ 1u)) {
            atomicOr(status, GV_ST_TIMEOUT_TMA);
            ok = false;
            break;
          }
          uint8_t* sp = ring + s * C::STAGE_BYTES;
          sm100::mbar_expect_tx(&full[s], C::STAGE_BYTES);
          sm100::tma_load_3d(sp, &tmW, &full[s], i * BK, tl.p0, tl.e);
          sm100::tma_load_2d(sp + C::P_BYTES, &tmX, &full[s], i * BK, tl.q0);
        }
      }
    }
  } else if (warp == 1) {
    if (sm100::elect_one()) {
      constexpr uint32_t idesc = sm100::make_idesc(BM, BN, 1, 1);
      uint32_t gk = 0, it = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
        const uint32_t buf = it & 1u;
        // the epilogue must have drained this accumulator buffer (used by tile it - 2)
        if (!sm100::mbar_wait(&tempty[buf], ((it >> 1) & 1u) ^ 1u)) {
          atomicOr(status, GV_ST_TIMEOUT_MMA);
          break;
        }
        for (int i = 0; i < nkb; ++i, ++gk) {
          const int s = gk % C::STAGES;
          if (!sm100::mbar_wait(&full[s], (gk / C::STAGES) & 1u)) {
            atomicOr(status, GV_ST_TIMEOUT_MMA);
            ok = false;
            break;
          }
          sm100::tc_fence_after();
          const uint32_t pa = sm100::smem_u32(ring + s * C::STAGE_BYTES);
          const uint64_t da = sm100::smem_desc_sw128(pa);
          const uint64_t db = sm100::smem_desc_sw128(pa + C::P_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            sm100::mma_f16_ss(tmem_base + buf * BN, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k),
                              idesc, (uint32_t)((i | k) != 0));
          sm100::tc_commit(&empty[s]);
        }
        if (ok) sm100::tc_commit(&tfull[buf]);
      }
    }
  } else {
    const int quad = warp & 3;
    uint32_t it = 0;
    for (long long t = blockIdx.x; t < total_tiles; t += gridDim.x, ++it) {
      const Tile tl = locate(t);
      const uint32_t buf = it & 1u;
      const int n = tl.p0 + quad * 32 + lane;
      const bool ok = sm100::mbar_wait(&tfull[buf], (it >> 1) & 1u);
      __syncwarp();
      if (!ok) {
        if (lane == 0) atomicOr(status, GV_ST_TIMEOUT_EPI);
        break;
      }
      sm100::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        uint32_t r[16];
        sm100::tmem_ld16(tmem_addr(tmem_base, quad, (int)(buf * BN) + c), r);
        sm100::tmem_ld_wait();
        if (SWIGLU) {
          const int f = (tl.p0 >> 1) + quad * 16 + (lane & 15);    // output feature of this lane pair
          const bool writer = lane < 16 && f < (N >> 1);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            // the unfused pair rounds the GEMM output to bf16 before activating: do the same
            float g = bf2f(f2bf(__uint_as_float(r[j])));
            float u = __shfl_xor_sync(0xffffffffu, g, 16);            // lanes >= 16 hold the up rows
            if (clamp > 0.f) {
              g = fminf(g, clamp);
              u = fminf(fmaxf(u, -clamp), clamp);
            }
            const int row = tl.q0 + c + j;
            if (writer && row < tl.seg_end)
              out[(long long)row * ldo + f] = f2bf(g / (1.f + __expf(-g)) * u);
          }
        } else if (n < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int row = tl.q0 + c + j;
            if (row < tl.seg_end) out[(long long)row * ldo + n] = f2bf(__uint_as_float(r[j]));
          }
        }
      }
      sm100::tc_fence_before();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&tempty[buf]);
    }
  }
  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem_base, TCOLS);
  }
}

template <int BN, bool SWIGLU>
static int launch_grouped(const CUtensorMap& tmW, const CUtensorMap& tmX, bf16* out,
                          const int* seg_start, const int* seg_end, int G, int e_mod, int rows_cap, int N,
                          int K, long long ldo, float clamp, cudaStream_t st) {
  using C = Cfg<BN, 108>;
  auto kern = grouped_gemm_bf16_kernel<BN, SWIGLU>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_last_error("grouped_gemm: smem attr", e);
      return GV_ECUDA;
    }
    configured = true;
  }
  const int tilesN = ceil_div(N, BM);
  if (G > GG_MAX_SEGMENTS) return GV_ETOOBIG;
  // persistent grid: two CTAs per SM, never more than the worst-case tile count
  long long grid = ((long long)rows_cap / BN + G) * tilesN;
  const long long slots = 2LL * num_sms();
  if (grid > slots) grid = slots;
  launch_pdl(kern, dim3((unsigned)grid), dim3(NUM_THREADS), C::SMEM_BYTES, st,
      tmW, tmX, out, seg_start, seg_end, N, K, G, e_mod, ldo, tilesN, clamp, status_word());
  return check_launch("grouped_gemm_bf16");
}

}  // namespace gemm
}  // namespace gv

using namespace gv;
using namespace gv::gemm;

static int grouped_bf16(const void* xs, const void* w, const int* seg_start, const int* seg_end,
                        long long G, long long e_mod, void* out, long long rows_cap, long long N,
                        long long K, long long E, long long avg_rows, cudaStream_t st, bool swiglu = false,
                        float clamp = 0.f) {
  // expert weights never move: encode their 3-D map once
  static std::mutex mu;
  static std::map<std::tuple<const void*, long long, long long, long long>, CUtensorMap> wmaps;
  CUtensorMap tmW, tmX;
  int rc;
  {
    std::lock_guard<std::mutex> g(mu);
    auto key = std::make_tuple(w, E, N, K);
    auto it = wmaps.find(key);
    if (it == wmaps.end()) {
      rc = sm100::make_tmap_3d(&tmW, w, 2, E, N, K, N * K * 2, K * 2, BM, BK);
      if (rc != GV_OK) return rc;
      wmaps.emplace(key, tmW);
    } else {
      tmW = it->second;
    }
  }
  const int bn = avg_rows <= 16 ? 16 : avg_rows <= 32 ? 32 : avg_rows <= 64 ? 64 : 128;
  if ((rc = cached_tmap_bf16(&tmX, xs, rows_cap, K, K, bn)) != GV_OK) return rc;
  const long long ldo = swiglu ? N / 2 : N;
#define GV_GG(BN_)                                                                                      \
  return swiglu ? launch_grouped<BN_, true>(tmW, tmX, (bf16*)out, seg_start, seg_end, (int)G, (int)e_mod, \
                                            (int)rows_cap, (int)N, (int)K, ldo, clamp, st)              \
                : launch_grouped<BN_, false>(tmW, tmX, (bf16*)out, seg_start, seg_end, (int)G, (int)e_mod, \
                                             (int)rows_cap, (int)N, (int)K, ldo, 0.f, st)
  switch (bn) {
    case 16: GV_GG(16);
    case 32: GV_GG(32);
    case 64: GV_GG(64);
    default: GV_GG(128);
  }
#undef GV_GG
}

// xs [rows_cap, K] bf16 (expert-major rows), w [E, N, K] bf16, offsets int32 [E + 1] on device,
// out [rows_cap, N] bf16. Rows outside [offsets[0], offsets[E]) are not written.
extern "C" int gv_grouped_gemm_bf16(const void* xs, const void* w, const void* offsets, void* out,
                                    long long rows_cap, long long N, long long K, long long E,
                                    void* stream) {
  if (!xs || !w || !offsets || !out || N <= 0 || K <= 0 || E <= 0) return GV_EINVAL;
  if ((K & 7) || (N & 7)) return GV_EINVAL;
  if (rows_cap == 0) return GV_OK;
  const int* off = (const int*)offsets;
  return grouped_bf16(xs, w, off, off + 1, E, 0, out, rows_cap, N, K, E, rows_cap / E, (cudaStream_t)stream);
}

// Segment form: G row segments [seg_start[g], seg_end[g]) (device arrays), segment g uses weight
// w[g % e_mod]. Used by the expert-parallel receive layout [source rank][local expert].
extern "C" int gv_grouped_gemm_bf16_seg(const void* xs, const void* w, const void* seg_start,
                                        const void* seg_end, void* out, long long rows_cap, long long N,
                                        long long K, long long E, long long G, long long avg_rows,
                                        void* stream) {
  if (!xs || !w || !seg_start || !seg_end || !out || N <= 0 || K <= 0 || E <= 0 || G <= 0) return GV_EINVAL;
  if ((K & 7) || (N & 7)) return GV_EINVAL;
  if (rows_cap == 0) return GV_OK;
  return grouped_bf16(xs, w, (const int*)seg_start, (const int*)seg_end, G, E, out, rows_cap, N, K, E,
                      avg_rows, (cudaStream_t)stream);
}

// SwiGLU forms: w [E, N = 2 I, K] with rows interleaved in blocks of [16 gate | 16 up]
// (N % 32 == 0), out [rows_cap, I] = silu(xs . gate^T) * (xs . up^T); `clamp` as in the kernel.
extern "C" int gv_grouped_gemm_bf16_swiglu(const void* xs, const void* w, const void* offsets, void* out,
                                           long long rows_cap, long long N, long long K, long long E,
                                           float clamp, void* stream) {
  if (!xs || !w || !offsets || !out || N <= 0 || K <= 0 || E <= 0) return GV_EINVAL;
  if ((K & 7) || (N & 31)) return GV_EINVAL;
  if (rows_cap == 0) return GV_OK;
  const int* off = (const int*)offsets;
  return grouped_bf16(xs, w, off, off + 1, E, 0, out, rows_cap, N, K, E, rows_cap / E, (cudaStream_t)stream,
                      true, clamp);
}

extern "C" int gv_grouped_gemm_bf16_swiglu_seg(const void* xs, const void* w, const void* seg_start,
                                               const void* seg_end, void* out, long long rows_cap,
                                               long long N, long long K, long long E, long long G,
                                               long long avg_rows, float clamp, void* stream) {
  if (!xs || !w || !seg_start || !seg_end || !out || N <= 0 || K <= 0 || E <= 0 || G <= 0) return GV_EINVAL;
  if ((K & 7) || (N & 31)) return GV_EINVAL;
  if (rows_cap == 0) return GV_OK;
  return grouped_bf16(xs, w, (const int*)seg_start, (const int*)seg_end, G, E, out, rows_cap, N, K, E,
                      avg_rows, (cudaStream_t)stream, true, clamp);
}

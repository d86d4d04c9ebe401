// Sequence-parallel tensor-parallel GEMMs fused with their collective (prefill sizes, tokens
// padded to a multiple of 128 * R):
//
//   gemm_rs : out_r[M/R, N]   = rows of rank r of  sum_s x_s[M, K_s] . w_s[N, K_s]^T
//             (row-parallel o_proj / down_proj followed by reduce-scatter)
//   ag_gemm : out[M, N_r]     = all_gather_s(x_s[M/R, K]) . w_r[N_r, K]^T (+ bias)
//             (all-gather followed by the column-parallel qkv / gate_up GEMM)
//
// The reference runs these as separate launches in its "comm optimize" layer loop —
// XliteOpReduceScatter after the matmul, XliteOpAllGather before the next one
// (xlite/csrc/model.cpp:1343-1406, 583-594, 836-850). Here both are one tcgen05 GEMM kernel each:
//
//   gemm_rs: every rank computes all 128-token x 128-feature tiles, visiting the token blocks in the
//   rotated order rank+1, rank+2, ..., rank, so tiles owned by other ranks are produced first: their
//   epilogue writes the bf16 partial straight into the owner's receive region over NVLink and raises
//   the owner's (tile, source) flag with a system-scope release. The rank's own tiles come last; their
//   epilogue waits (bounded) until the R-1 remote partials have arrived, adds them in rank order to
//   the accumulator it still holds in TMEM and writes the reduced rows. Transfers overlap the
//   remaining tiles' math.
//
//   ag_gemm: a staging launch PUSHES the local token slice into every rank's staging region
//   `[parity][source rank][rows][K]` (so each slice crosses NVLink exactly once per destination)
//   and publishes a flag; the GEMM's TMA producer then loads every token tile from this GPU's own
//   memory (plain, non-multicast TMA through tensor maps that live in global memory, one per source
//   rank and parity), own tiles first, waiting (bounded) on the source's flag before the first load
//   of its rows. Loading the tiles straight from the peers instead would re-read a remote tile once
//   per output-column tile.
//
// Generation counters live on the device (CUDA-graph replay safe); staging / receive regions are
// double-buffered by the generation's parity (see parallel/symm.py for why two suffice).
#include "gemm_core.cuh"
#include "gvirt_kernels.h"

namespace gv {
namespace gemm {

int cached_tmap_bf16(CUtensorMap* out, const void* base, long long rows, long long cols,
                     long long row_stride_elems, int box_rows);

constexpr int SP_BN = 128;
constexpr int SP_MAX_RANKS = 16;
constexpr int SP_RS_MAX_RANKS = 8;   // ranks the reduce phase of gemm_rs unrolls over

__device__ __forceinline__ void sp_epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ uint4 sp_ld_sys16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

struct SpArgs {
  void* const* peers;
  long long data_off;     // gemm_rs: recv [2][R][m_r_cap][N] bf16; ag_gemm: stage [2][R][m_r_cap][K] bf16
  long long data_stride;  // bytes per parity buffer
  long long flags_off;    // gemm_rs: per-(tile, source) flags [tiles][16]; ag_gemm: ready flags [16]
  unsigned int* state;    // local {generation, ticket}
  int rank, R, m_r_cap;
};

// ------------------------------------------------------------------ GEMM -> reduce-scatter
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
               bf16* __restrict__ out, int M, int N, int K, long long ldo, int tilesM, int tilesN,
               SpArgs a, unsigned int* status) {
  using C = Cfg<SP_BN, 220>;
  extern __shared__ uint8_t smem_raw[];
  const Shared sh = carve<C>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]) + 1u;
  const int tiles_per_rank = tilesM / a.R;
  const int tn = blockIdx.x % tilesN;
  const int tm_seq = blockIdx.x / tilesN;
  const int tm = (tm_seq + (a.rank + 1) * tiles_per_rank) % tilesM;  // other ranks' blocks first
  const int owner = tm / tiles_per_rank;
  const int row_local0 = (tm % tiles_per_rank) * BM;
  const int tile_id = (tm % tiles_per_rank) * tilesN + tn;
  const int nkb = (K + BK - 1) / BK;

  const uint32_t tmem_base = run_mainloop<C>(sh, &tmX, &tmW, tm * BM, tn * SP_BN, 0, nkb, status);

  if (warp >= 2) {
    const int quad = warp & 3;
    const int row = row_local0 + quad * 32 + lane;  // row inside the owner's slice
    const int n0 = tn * SP_BN;
    const long long par_elems = a.data_stride / 2;
    wait_accum(sh, status);
    if (owner != a.rank) {
      bf16* dst = reinterpret_cast<bf16*>(static_cast<char*>(a.peers[owner]) + a.data_off) +
                  (long long)(gen & 1u) * par_elems + ((long long)a.rank * a.m_r_cap + row) * N + n0;
#pragma unroll 1
      for (int c = 0; c < SP_BN; c += 16) {
        uint32_t r[16];
        sm100::tmem_ld16(tmem_addr(tmem_base, quad, c), r);
        sm100::tmem_ld_wait();
        if (n0 + c + 16 <= N) {
          float f[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(r[j]);
          st8(dst + c, pack8(f));
          st8(dst + c + 8, pack8(f + 8));
        }
      }
      sp_epi_bar();
      if (threadIdx.x == 64) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<unsigned int*>(static_cast<char*>(a.peers[owner]) + a.flags_off) +
                           (size_t)tile_id * SP_MAX_RANKS + a.rank,
                       gen);
      }
    } else {
      const int s = (int)threadIdx.x - 64;
      if (s < a.R && s != a.rank) {
        const unsigned int* f = reinterpret_cast<const unsigned int*>(static_cast<char*>(a.peers[a.rank]) +
                                                                      a.flags_off) +
                                (size_t)tile_id * SP_MAX_RANKS + s;
        if (!wait_ge_sys(f, gen, peer_budget(status))) atomicOr(status, GV_ST_TIMEOUT_PEER);
      }
      sp_epi_bar();
      const bf16* base = reinterpret_cast<const bf16*>(static_cast<char*>(a.peers[a.rank]) + a.data_off) +
                         (long long)(gen & 1u) * par_elems;
      bf16* orow = out + (long long)row * ldo + n0;
#pragma unroll 1
      for (int c = 0; c < SP_BN; c += 16) {
        uint32_t r[16];
        sm100::tmem_ld16(tmem_addr(tmem_base, quad, c), r);
        sm100::tmem_ld_wait();
        if (n0 + c + 16 > N) continue;
        // all remote partials of this chunk are requested before any is consumed: up to
        // 2 (R - 1) independent 16-byte loads in flight per thread instead of a chain of them
        uint4 v[SP_RS_MAX_RANKS][2];
#pragma unroll
        for (int s = 0; s < SP_RS_MAX_RANKS; ++s) {
          if (s < a.R && s != a.rank) {
            const bf16* src = base + ((long long)s * a.m_r_cap + row) * N + n0 + c;
            v[s][0] = sp_ld_sys16(src);
            v[s][1] = sp_ld_sys16(src + 8);
          }
        }
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
#pragma unroll
        for (int s = 0; s < SP_RS_MAX_RANKS; ++s) {  // rank order; this rank's own partial is the accumulator
          if (s >= a.R) continue;
          if (s == a.rank) {
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] += bf2f(f2bf(__uint_as_float(r[j])));
          } else {
            float f[16];
            unpack8(*reinterpret_cast<const bf16x8*>(&v[s][0]), f);
            unpack8(*reinterpret_cast<const bf16x8*>(&v[s][1]), f + 8);
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] += f[j];
          }
        }
        st8(orow + c, pack8(acc));
        st8(orow + c + 8, pack8(acc + 8));
      }
    }
  }
  finish<C>(sh, tmem_base);
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&a.state[1], 1u) == gridDim.x - 1) {
      a.state[1] = 0;
      __threadfence();
      a.state[0] = gen;
    }
  }
}

// ------------------------------------------------------------------ all-gather -> GEMM
// Stage: push the local slice into slot `rank` of every rank's staging region, publish flag (gen)
// to every rank. slot_elems = elements per source slot (m_r_cap * K).
__global__ void ag_stage_kernel(const bf16* __restrict__ x, long long n_elems, long long slot_elems,
                                SpArgs a) {
  __shared__ bool s_last;
  const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]) + 1u;
  const long long off = a.data_off + (long long)(gen & 1u) * a.data_stride + (long long)a.rank * slot_elems * 2;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n_elems;
       i += (long long)gridDim.x * blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + i);
    for (int p = 0; p < a.R; ++p) {
      const int peer = (a.rank + p) % a.R;
      *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(static_cast<char*>(a.peers[peer]) + off) + i) = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&a.state[1], 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    if ((int)threadIdx.x < a.R) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<unsigned int*>(static_cast<char*>(a.peers[threadIdx.x]) + a.flags_off) +
                         a.rank,
                     gen);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      a.state[1] = 0;
      __threadfence();
      a.state[0] = gen;
    }
  }
}

// maps: global array [2 * R] of tensor maps over the source slots of this rank's staging region
// (parity-major).
__global__ void __launch_bounds__(NUM_THREADS, 1)
ag_gemm_kernel(const CUtensorMap* __restrict__ maps, const __grid_constant__ CUtensorMap tmW,
               bf16* __restrict__ out, const bf16* __restrict__ bias, int M, int N, int K, long long ldo,
               int tilesM, int tilesN, SpArgs a, unsigned int* status) {
  using C = Cfg<SP_BN, 220>;
  extern __shared__ uint8_t smem_raw[];
  const Shared sh = carve<C>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]);  // staged already
  const int tiles_per_rank = tilesM / a.R;
  const int tn = blockIdx.x % tilesN;
  const int tm_seq = blockIdx.x / tilesN;
  const int tm = (tm_seq + a.rank * tiles_per_rank) % tilesM;  // own token block first
  const int owner = tm / tiles_per_rank;
  const int row_local0 = (tm % tiles_per_rank) * BM;
  const int nkb = (K + BK - 1) / BK;
  const CUtensorMap* tmX = maps + (gen & 1u) * a.R + owner;
  // the TMA producer must not touch a peer's staging buffer before that peer has published it
  if (warp == 0 && owner != a.rank) {
    if (lane == 0) {
      const unsigned int* f =
          reinterpret_cast<const unsigned int*>(static_cast<char*>(a.peers[a.rank]) + a.flags_off) + owner;
      if (!wait_ge_sys(f, gen, peer_budget(status))) atomicOr(status, GV_ST_TIMEOUT_PEER);
    }
    __syncwarp();
    // the flag was observed through the generic proxy; the tile loads go through the async proxy
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  const uint32_t tmem_base = run_mainloop<C>(sh, tmX, &tmW, row_local0, tn * SP_BN, 0, nkb, status);
  if (warp >= 2) {
    const int quad = warp & 3;
    const int row = tm * BM + quad * 32 + lane;
    const int n0 = tn * SP_BN;
    wait_accum(sh, status);
    bf16* orow = out + (long long)row * ldo + n0;
#pragma unroll 1
    for (int c = 0; c < SP_BN; c += 16) {
      uint32_t r[16];
      sm100::tmem_ld16(tmem_addr(tmem_base, quad, c), r);
      sm100::tmem_ld_wait();
      if (row < M) {
        if (n0 + c + 16 <= N) {
          float f[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            f[j] = __uint_as_float(r[j]);
            if (bias != nullptr) f[j] += bf2f(bias[n0 + c + j]);
          }
          st8(orow + c, pack8(f));
          st8(orow + c + 8, pack8(f + 8));
        } else {
          for (int j = 0; j < 16 && n0 + c + j < N; ++j) {
            float v = __uint_as_float(r[j]);
            if (bias != nullptr) v += bf2f(bias[n0 + c + j]);
            orow[c + j] = f2bf(v);
          }
        }
      }
    }
  }
  finish<C>(sh, tmem_base);
}

static bool g_rs_conf = false, g_ag_conf = false;

}  // namespace gemm
}  // namespace gv

using namespace gv;
using namespace gv::gemm;

static SpArgs sp_args(const void* peers, long long data_off, long long data_stride, long long flags_off,
                      void* state, long long rank, long long R, long long m_r_cap) {
  SpArgs a;
  a.peers = (void* const*)peers;
  a.data_off = data_off;
  a.data_stride = data_stride;
  a.flags_off = flags_off;
  a.state = (unsigned int*)state;
  a.rank = (int)rank;
  a.R = (int)R;
  a.m_r_cap = (int)m_r_cap;
  return a;
}

// x [M, K_r], w [N, K_r] (this rank's K shard), out [M / R, N]. M % (128 * R) == 0, N % 16 == 0.
// Receive region: 2 * R * m_r_cap * N bf16; flags: (m_r_cap / 128) * ceil(N / 128) * 16 words.
extern "C" int gv_gemm_rs(const void* x, const void* w, void* out, long long M, long long N, long long K,
                          long long ldx, long long ldw, long long ldo, const void* peers,
                          long long recv_off, long long recv_stride, long long cnt_off, void* state,
                          long long rank, long long R, long long m_r_cap, void* stream) {
  if (!x || !w || !out || !peers || !state) return GV_EINVAL;
  if (M <= 0 || M % (BM * R) || (N & 15) || (K & 7) || (ldx & 7) || (ldw & 7) || (ldo & 7)) return GV_EINVAL;
  if (M / R > m_r_cap || R > SP_RS_MAX_RANKS) return GV_ETOOBIG;
  if ((long long)R * m_r_cap * N * 2 > recv_stride) return GV_ETOOBIG;
  using C = Cfg<SP_BN, 220>;
  if (!g_rs_conf) {
    cudaError_t e = cudaFuncSetAttribute(gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_last_error("gemm_rs: smem attr", e);
      return GV_ECUDA;
    }
    g_rs_conf = true;
  }
  CUtensorMap tmX, tmW;
  int rc;
  if ((rc = cached_tmap_bf16(&tmX, x, M, K, ldx, BM)) != GV_OK) return rc;
  if ((rc = cached_tmap_bf16(&tmW, w, N, K, ldw, SP_BN)) != GV_OK) return rc;
  const int tilesM = (int)(M / BM), tilesN = ceil_div(N, SP_BN);
  SpArgs a = sp_args(peers, recv_off, recv_stride, cnt_off, state, rank, R, m_r_cap);
  gemm_rs_kernel<<<(unsigned)(tilesM * tilesN), NUM_THREADS, C::SMEM_BYTES, (cudaStream_t)stream>>>(
      tmX, tmW, (bf16*)out, (int)M, (int)N, (int)K, ldo, tilesM, tilesN, a, status_word());
  return check_launch("gv_gemm_rs");
}

// Encode the 2 * R tensor maps over the peers' staging buffers into `maps_dev` (device memory,
// 128 bytes each). peers_host: host array of R slab base addresses.
extern "C" int gv_ag_gemm_setup(void* maps_dev, const void* peers_host, long long stage_off,
                                long long stage_stride, long long m_r_cap, long long K, long long R,
                                long long rank, void* stream) {
  if (!maps_dev || !peers_host || R < 1 || R > SP_MAX_RANKS || (K & 7) || rank < 0 || rank >= R)
    return GV_EINVAL;
  if (R * m_r_cap * K * 2 > stage_stride) return GV_ETOOBIG;
  CUtensorMap host[2 * SP_MAX_RANKS];
  const long long* pp = (const long long*)peers_host;
  for (int par = 0; par < 2; ++par)
    for (int r = 0; r < R; ++r) {
      const char* base = reinterpret_cast<const char*>(pp[rank]) + stage_off + par * stage_stride +
                         (long long)r * m_r_cap * K * 2;
      int rc = sm100::make_tmap_2d(&host[par * R + r], base, 2, m_r_cap, K, K * 2, BM, BK);
      if (rc != GV_OK) return rc;
    }
  cudaError_t e = cudaMemcpyAsync(maps_dev, host, sizeof(CUtensorMap) * 2 * R, cudaMemcpyHostToDevice,
                                  (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) {
    set_last_error("gv_ag_gemm_setup", e);
    return GV_ECUDA;
  }
  return GV_OK;
}

// x_local [M / R, K] (any local tensor), w [N, K], out [M, N]. M % (128 * R) == 0.
extern "C" int gv_ag_gemm(const void* x_local, const void* w, const void* bias, void* out, long long M,
                          long long N, long long K, long long ldw, long long ldo, const void* maps_dev,
                          const void* peers, long long stage_off, long long stage_stride,
                          long long flags_off, void* state, long long rank, long long R,
                          long long m_r_cap, void* stream) {
  if (!x_local || !w || !out || !maps_dev || !peers || !state) return GV_EINVAL;
  if (M <= 0 || M % (BM * R) || (K & 7) || (ldw & 7) || (ldo & 7)) return GV_EINVAL;
  if (M / R > m_r_cap || R * m_r_cap * K * 2 > stage_stride) return GV_ETOOBIG;
  using C = Cfg<SP_BN, 220>;
  if (!g_ag_conf) {
    cudaError_t e = cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_last_error("ag_gemm: smem attr", e);
      return GV_ECUDA;
    }
    g_ag_conf = true;
  }
  cudaStream_t st = (cudaStream_t)stream;
  SpArgs a = sp_args(peers, stage_off, stage_stride, flags_off, state, rank, R, m_r_cap);
  const long long n_elems = (M / R) * K;
  long long g = (n_elems / 8 + 255) / 256;
  if (g > 148 * 4) g = 148 * 4;
  if (g < 1) g = 1;
  ag_stage_kernel<<<(unsigned)g, 256, 0, st>>>((const bf16*)x_local, n_elems, m_r_cap * K, a);
  CUtensorMap tmW;
  int rc;
  if ((rc = cached_tmap_bf16(&tmW, w, N, K, ldw, SP_BN)) != GV_OK) return rc;
  const int tilesM = (int)(M / BM), tilesN = ceil_div(N, SP_BN);
  ag_gemm_kernel<<<(unsigned)(tilesM * tilesN), NUM_THREADS, C::SMEM_BYTES, st>>>(
      (const CUtensorMap*)maps_dev, tmW, (bf16*)out, (const bf16*)bias, (int)M, (int)N, (int)K, ldo, tilesM,
      tilesN, a, status_word());
  return check_launch("gv_ag_gemm");
}

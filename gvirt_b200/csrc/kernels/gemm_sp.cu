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
// (xlite/csrc/model.cpp:1343-1406, 583-594, 836-850). Here both are one persistent tcgen05 GEMM
// kernel each, built like the prefill GEMM (gemm_persist.cu): one CTA per SM walks a list of
// 128-token x 256-feature tiles, the fp32 accumulator is double-buffered in TMEM so the epilogue
// of one tile (which is where the communication happens) overlaps the K loop of the next.
//
//   gemm_rs: every rank computes all tiles, visiting the token blocks in the rotated order
//   rank+1, rank+2, ..., rank, so tiles owned by other ranks are produced first. Their epilogue
//   rounds the partial to bf16, transposes it through shared memory and writes whole 128-byte row
//   segments into the owner's receive region over NVLink (a thread-per-row store pattern would put
//   16-byte packets on the links and is packet-rate bound at a fraction of the bandwidth), then
//   raises the owner's (tile, source) flag with a system-scope release. The rank's own tiles come
//   last; their epilogue waits (bounded) until the R-1 remote partials have arrived, adds them in
//   rank order to its own rounded partial and writes the reduced rows, again in row segments with
//   every remote load of a step in flight before the first is consumed.
//
//   ag_gemm: a staging launch PUSHES the local token slice into every rank's staging region
//   `[parity][source rank][rows][K]` (so each slice crosses NVLink exactly once per destination)
//   and publishes a flag; the GEMM's TMA producer then loads every token tile from this GPU's own
//   memory (plain, non-multicast TMA through tensor maps that live in global memory, one per source
//   rank and parity), own token block first, waiting (bounded) on a source's flag before the first
//   load of its rows. Loading the tiles straight from the peers instead would re-read a remote tile
//   once per output-column tile.
//
// Generation counters live on the device (CUDA-graph replay safe); staging / receive regions are
// double-buffered by the generation's parity (see parallel/symm.py for why two suffice).
#include "gemm_core.cuh"
#include "gvirt_kernels.h"

namespace gv {
namespace gemm {

int cached_tmap_bf16(CUtensorMap* out, const void* base, long long rows, long long cols,
                     long long row_stride_elems, int box_rows);

constexpr int SP_BN = 256;           // features per tile (TMEM columns of one accumulator buffer)
constexpr int SP_MAX_RANKS = 16;
constexpr int SP_RS_MAX_RANKS = 8;   // ranks the reduce phase of gemm_rs unrolls over
constexpr int SP_GROUP = 16;         // token tiles that share a sweep over the feature tiles (L2 reuse)
constexpr int SP_CHUNK = 64;         // features transposed through shared memory at a time
constexpr int SP_PITCH = SP_CHUNK * 2 + 16;            // bytes per staged row (+16: bank spread)
constexpr int SP_STAGING = 4 * 32 * SP_PITCH;          // four epilogue warps x 32 rows
using SpCfg = Cfg<SP_BN, 200>;
constexpr int SP_SMEM_BYTES = SpCfg::SMEM_BYTES + SP_STAGING;

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

struct SpTile {
  int tm, tn;
};
// tile t of the walk -> (token tile, feature tile): groups of SP_GROUP token tiles sweep the feature
// tiles together; `shift` rotates the token tiles so that a chosen rank's block comes first / last
__device__ __forceinline__ SpTile sp_locate(int t, int tilesM, int tilesN, int shift) {
  const int per_group = SP_GROUP * tilesN;
  const int g = t / per_group;
  const int first = g * SP_GROUP;
  const int gsz = (tilesM - first) < SP_GROUP ? (tilesM - first) : SP_GROUP;
  const int r = t - g * per_group;
  SpTile tl;
  tl.tm = (first + r % gsz + shift) % tilesM;
  tl.tn = r / gsz;
  return tl;
}

// MODE 1: GEMM -> reduce-scatter (x is this rank's [M, K_r]); MODE 2: all-gather -> GEMM (token tiles
// come from the staging region through `maps`).
template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sp_gemm_kernel(const __grid_constant__ CUtensorMap tmX, const CUtensorMap* __restrict__ maps,
               const __grid_constant__ CUtensorMap tmW, bf16* __restrict__ out,
               const bf16* __restrict__ bias, int M, int N, int K, long long ldo, int tilesM, int tilesN,
               SpArgs a, unsigned int* status) {
  using C = SpCfg;
  constexpr int BN = SP_BN;
  constexpr int TCOLS = 2 * BN;
  static_assert(TCOLS == 512, "the two accumulator buffers take the whole TMEM");
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // gemm_rs opens a new generation; ag_gemm runs in the one its staging launch opened
  const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]) + (MODE == 1 ? 1u : 0u);
  const int total = tilesM * tilesN;
  const int nkb = (K + BK - 1) / BK;
  const int tpr = tilesM / a.R;                       // token tiles per rank
  const int shift = (MODE == 1 ? (a.rank + 1) : a.rank) * tpr;   // RS: own block last; AG: own block first

  uintptr_t base = (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023);
  uint8_t* ring = reinterpret_cast<uint8_t*>(base);
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tfull = empty + C::STAGES;   // [2] accumulator buffer complete
  uint64_t* tempty = tfull + 2;          // [2] accumulator buffer drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  uint8_t* staging = ring + C::STAGES * C::STAGE_BYTES + 256;
  static_assert((2 * C::STAGES + 4) * 8 + 4 <= 256, "barriers must fit behind the ring");

  if (warp == 0 && sm100::elect_one()) {
    if (MODE == 1) sm100::tma_prefetch_desc(&tmX);
    sm100::tma_prefetch_desc(&tmW);
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
      uint32_t gk = 0, seen = 1u << a.rank;     // AG: sources whose staged rows are known to be complete
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const SpTile tl = sp_locate(t, tilesM, tilesN, shift);
        const CUtensorMap* tx = &tmX;
        int row0 = tl.tm * BM;
        if (MODE == 2) {
          const int owner = tl.tm / tpr;
          if (!((seen >> owner) & 1u)) {
            // the TMA loads must not touch a source's rows before that source has published them
            const unsigned int* f =
                reinterpret_cast<const unsigned int*>(static_cast<char*>(a.peers[a.rank]) + a.flags_off) + owner;
            if (!wait_ge_sys(f, gen, peer_budget(status))) atomicOr(status, GV_ST_TIMEOUT_PEER);
            // the flag was observed through the generic proxy; the tile loads go through the async proxy
            asm volatile("fence.proxy.async;" ::: "memory");
            seen |= 1u << owner;
          }
          tx = maps + (gen & 1u) * a.R + owner;
          row0 = (tl.tm % tpr) * BM;
        }
        for (int i = 0; i < nkb; ++i, ++gk) {
          const int s = gk % C::STAGES;
          if (!sm100::mbar_wait(&empty[s], ((gk / C::STAGES) & 1u) ^ 1u)) {
            atomicOr(status, GV_ST_TIMEOUT_TMA);
            ok = false;
            break;
          }
          uint8_t* sp = ring + s * C::STAGE_BYTES;
          sm100::mbar_expect_tx(&full[s], C::STAGE_BYTES);
          sm100::tma_load_2d(sp, tx, &full[s], i * BK, row0);
          sm100::tma_load_2d(sp + C::P_BYTES, &tmW, &full[s], i * BK, tl.tn * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (sm100::elect_one()) {
      constexpr uint32_t idesc = sm100::make_idesc(BM, BN, 1, 1);
      uint32_t gk = 0, it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++it) {
        const uint32_t buf = it & 1u;
        if (!sm100::mbar_wait(&tempty[buf], ((it >> 1) & 1u) ^ 1u)) {
          atomicOr(status, GV_ST_TIMEOUT_MMA);
          break;
        }
        sm100::tc_fence_after();
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
    uint8_t* stg = staging + quad * 32 * SP_PITCH;      // this warp's 32 rows of the chunk
    const int srow = lane >> 3, piece = lane & 7;       // write-out: 8 lanes cover one 128-byte row segment
    const long long par_elems = a.data_stride / 2;
    uint32_t it = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++it) {
      const SpTile tl = sp_locate(t, tilesM, tilesN, shift);
      const uint32_t buf = it & 1u;
      const bool ok = sm100::mbar_wait(&tfull[buf], (it >> 1) & 1u);
      __syncwarp();
      if (!ok) {
        if (lane == 0) atomicOr(status, GV_ST_TIMEOUT_EPI);
        break;
      }
      sm100::tc_fence_after();
      const int n0 = tl.tn * BN;
      if (MODE == 2) {
        const int p = tl.tm * BM + quad * 32 + lane;  // token row of this thread
        bf16* orow = out + (long long)p * ldo;
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          sm100::tmem_ld16(tmem_addr(tmem_base, quad, (int)(buf * BN) + c), r);
          sm100::tmem_ld_wait();
          const int q = n0 + c;
          if (p < M && q < N) {
            if (q + 16 <= N) {
              float f[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                f[j] = __uint_as_float(r[j]);
                if (bias != nullptr) f[j] += bf2f(bias[q + j]);
              }
              st8(orow + q, pack8(f));
              st8(orow + q + 8, pack8(f + 8));
            } else {
              for (int j = 0; j < 16 && q + j < N; ++j) {
                float v = __uint_as_float(r[j]);
                if (bias != nullptr) v += bf2f(bias[q + j]);
                orow[q + j] = f2bf(v);
              }
            }
          }
        }
        sm100::tc_fence_before();
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&tempty[buf]);
        continue;
      }
      // ---- MODE 1: reduce-scatter epilogue
      const int owner = tl.tm / tpr;
      const int row_local0 = (tl.tm % tpr) * BM + quad * 32;        // first row of this warp in the owner's slice
      const int tile_id = (tl.tm % tpr) * tilesN + tl.tn;
      const bool mine = owner == a.rank;
      if (mine) {
        const int s = (int)threadIdx.x - 64;
        if (s < a.R && s != a.rank) {
          const unsigned int* f = reinterpret_cast<const unsigned int*>(static_cast<char*>(a.peers[a.rank]) +
                                                                        a.flags_off) +
                                  (size_t)tile_id * SP_MAX_RANKS + s;
          if (!wait_ge_sys(f, gen, peer_budget(status))) atomicOr(status, GV_ST_TIMEOUT_PEER);
        }
        sp_epi_bar();
      }
      bf16* push = reinterpret_cast<bf16*>(static_cast<char*>(a.peers[owner]) + a.data_off) +
                   (long long)(gen & 1u) * par_elems + ((long long)a.rank * a.m_r_cap + row_local0) * N + n0;
      const bf16* recv = reinterpret_cast<const bf16*>(static_cast<char*>(a.peers[a.rank]) + a.data_off) +
                         (long long)(gen & 1u) * par_elems + (long long)row_local0 * N + n0;
      bf16* orow0 = out + (long long)row_local0 * ldo + n0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += SP_CHUNK) {
        // accumulator chunk -> bf16 -> this warp's staging rows (lane = row)
#pragma unroll
        for (int c = 0; c < SP_CHUNK; c += 16) {
          uint32_t r[16];
          sm100::tmem_ld16(tmem_addr(tmem_base, quad, (int)(buf * BN) + c0 + c), r);
          sm100::tmem_ld_wait();
          float f[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(r[j]);
          *reinterpret_cast<bf16x8*>(stg + lane * SP_PITCH + c * 2) = pack8(f);
          *reinterpret_cast<bf16x8*>(stg + lane * SP_PITCH + c * 2 + 16) = pack8(f + 8);
        }
        if (c0 + SP_CHUNK >= BN) {
          // last read of this accumulator buffer: hand it back to the MMA warp
          sm100::tc_fence_before();
          __syncwarp();
          if (lane == 0) sm100::mbar_arrive(&tempty[buf]);
        }
        __syncwarp();
        const int col = n0 + c0 + piece * 8;            // first of this lane's 8 features
        if (!mine) {
#pragma unroll
          for (int rr = 0; rr < 32; rr += 4) {
            const int row = rr + srow;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + row * SP_PITCH + piece * 16);
            if (col + 8 <= N) *reinterpret_cast<uint4*>(push + (long long)row * N + c0 + piece * 8) = v;
          }
        } else {
#pragma unroll 2
          for (int rr = 0; rr < 32; rr += 4) {
            const int row = rr + srow;
            if (col + 8 > N) continue;
            // every remote partial of this row segment is requested before any is consumed
            uint4 v[SP_RS_MAX_RANKS];
#pragma unroll
            for (int s = 0; s < SP_RS_MAX_RANKS; ++s)
              if (s < a.R && s != a.rank)
                v[s] = sp_ld_sys16(recv + ((long long)s * a.m_r_cap + row) * N + c0 + piece * 8);
            const uint4 own = *reinterpret_cast<const uint4*>(stg + row * SP_PITCH + piece * 16);
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
            for (int s = 0; s < SP_RS_MAX_RANKS; ++s) {  // rank order, so every rank rounds alike
              if (s >= a.R) continue;
              float f[8];
              unpack8(*reinterpret_cast<const bf16x8*>(s == a.rank ? &own : &v[s]), f);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] += f[j];
            }
            st8(orow0 + (long long)row * ldo + c0 + piece * 8, pack8(acc));
          }
        }
        __syncwarp();                                    // the staging rows are rewritten by the next chunk
      }
      if (!mine) {
        sp_epi_bar();                                    // all four warps' rows are on their way
        if (threadIdx.x == 64) {
          __threadfence_system();
          st_release_sys(reinterpret_cast<unsigned int*>(static_cast<char*>(a.peers[owner]) + a.flags_off) +
                             (size_t)tile_id * SP_MAX_RANKS + a.rank,
                         gen);
        }
      }
    }
  }
  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem_base, TCOLS);
  }
  if (MODE == 1 && threadIdx.x == 0) {
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

// x [M, K_r], w [N, K_r] (this rank's K shard), out [M / R, N]. M % (128 * R) == 0, N % 8 == 0.
// Receive region: 2 * R * m_r_cap * N bf16; flags: (m_r_cap / 128) * ceil(N / 256) * 16 words.
extern "C" int gv_gemm_rs(const void* x, const void* w, void* out, long long M, long long N, long long K,
                          long long ldx, long long ldw, long long ldo, const void* peers,
                          long long recv_off, long long recv_stride, long long cnt_off, void* state,
                          long long rank, long long R, long long m_r_cap, void* stream) {
  if (!x || !w || !out || !peers || !state) return GV_EINVAL;
  if (M <= 0 || M % (BM * R) || (N & 7) || (K & 7) || (ldx & 7) || (ldw & 7) || (ldo & 7)) return GV_EINVAL;
  if (M / R > m_r_cap || R > SP_RS_MAX_RANKS) return GV_ETOOBIG;
  if ((long long)R * m_r_cap * N * 2 > recv_stride) return GV_ETOOBIG;
  auto kern = sp_gemm_kernel<1>;
  if (!g_rs_conf) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SP_SMEM_BYTES);
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
  long long grid = (long long)tilesM * tilesN;
  if (grid > num_sms()) grid = num_sms();
  SpArgs a = sp_args(peers, recv_off, recv_stride, cnt_off, state, rank, R, m_r_cap);
  kern<<<(unsigned)grid, NUM_THREADS, SP_SMEM_BYTES, (cudaStream_t)stream>>>(
      tmX, (const CUtensorMap*)nullptr, tmW, (bf16*)out, (const bf16*)nullptr, (int)M, (int)N, (int)K, ldo,
      tilesM, tilesN, a, status_word());
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
  auto kern = sp_gemm_kernel<2>;
  if (!g_ag_conf) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SP_SMEM_BYTES);
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
  long long grid = (long long)tilesM * tilesN;
  if (grid > num_sms()) grid = num_sms();
  kern<<<(unsigned)grid, NUM_THREADS, SP_SMEM_BYTES, st>>>(
      tmW, (const CUtensorMap*)maps_dev, tmW, (bf16*)out, (const bf16*)bias, (int)M, (int)N, (int)K, ldo, tilesM,
      tilesN, a, status_word());
  return check_launch("gv_ag_gemm");
}

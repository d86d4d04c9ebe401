// Row-parallel GEMM fused with the tensor-parallel all-reduce (decode sizes, M <= 128):
//
//     out[M, N] = sum over ranks r of  x_r[M, K_r] . w_r[N, K_r]^T     (+ bias) (+ residual)
//
// One kernel per rank does both the tcgen05 GEMM on its K shard and the reduction over NVLink.
// The epilogue of every tile converts the fp32 accumulators to bf16, transposes them through
// shared memory and *pushes* them with plain peer stores into the receive region
// `[parity][source rank][token][feature]` of every other rank's symmetric heap. The transfer uses
// a flag-in-data protocol: every 16-byte store carries 8 bytes of payload (4 bf16) and two copies
// of the launch generation, one per 8-byte half (8-byte stores are single-copy atomic), so the
// receiver polls the data itself. No system-scope fence, no separate flag word and no second
// NVLink round trip sit between a tile's last MMA and its reduction; at these message sizes
// (<= 1 MiB per peer) latency, not bandwidth, is what the all-reduce costs. The receiver then
// sums the R partials in rank order with fp32 accumulation, taking its own from shared memory
// (rounded to bf16 exactly like the copies its peers got, so every rank computes the same bits).
// Tiles that finish early are already crossing NVSwitch while later tiles are still in their K
// loop: the transfer overlaps the math tile by tile.
//
// With `residual` the reduced rows are added to the residual stream (`out` may be `residual`
// itself), and with `ss_out` every rank also leaves the per-(tile, token) sums of squares of the
// new rows behind: the consumer GEMM (gemm_decode.cu) turns them into the RMSNorm factor in its
// epilogue, so the add + norm launch that follows o_proj / down_proj in the reference
// (xlite/csrc/model.cpp:1413-1433) disappears under tensor parallelism as well.
//
// This replaces the reference's matmul followed by a separate `XliteOpAllReduceSum` launch after
// o_proj / down_proj (xlite/csrc/model.cpp:583-594, 836-850; XCCL pull + bf16 atomic adds in
// xlite/csrc/kernels/all_reduce.cpp:237-332).
//
// Graph-replay safe: the generation is a device counter advanced by the last CTA of a launch
// (see collectives.cu); receive slots are double-buffered by generation parity and a slot whose
// flags are not the current generation is by construction stale. All CTAs of a launch are
// co-resident (grid <= 2 x SM count), so waiting on peers cannot starve local tiles. Every poll
// is bounded in time and reports through the status word. No TMA multicast; peers are only ever
// written with `st.global` and read by nobody (each rank reduces from its own memory).
#include "gemm_core.cuh"
#include "gvirt_kernels.h"

namespace gv {
namespace gemm {

int cached_tmap_bf16(CUtensorMap* out, const void* base, long long rows, long long cols,
                     long long row_stride_elems, int box_rows);

void take_next_weights(int bn, CUtensorMap* tm, NextWeights* nx);   // gemm_decode.cu

constexpr int AR_MAX_RANKS = 8;

struct ArArgs {
  void* const* peers;     // device array [R] of symmetric slab bases
  long long recv_off;     // receive region: [2 parity][R src][m_cap][N / 4] 16-byte lines
  long long flags_off;    // unused by this kernel (kept for the channel layout)
  unsigned int* state;    // local {generation, ticket}
  int rank, R, m_cap;
  int two_shot;           // 1: column c of tile t is reduced by rank (t + c) % R and broadcast
  float* ss_out;          // [tokens][ss_ld]: entry [t][tile] = sum of squares of the finished row t in tile, or null
  int ss_ld;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  bf162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// One 16-byte line = {payload lo, generation, payload hi, generation}.
__device__ __forceinline__ void st_line(uint4* p, uint32_t lo, uint32_t hi, uint32_t gen) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(lo), "r"(gen),
               "r"(hi), "r"(gen)
               : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Re-reads a line until both halves carry `gen` (bounded in time). false = gave up.
__device__ __forceinline__ bool wait_line(const uint4* p, uint32_t gen, uint4& v,
                                          unsigned long long budget_ns = GV_WAIT_NS) {
  if (v.y == gen && v.w == gen) return true;
  const unsigned long long t0 = global_ns();
  for (unsigned int i = 0; i < GV_SPIN_LIMIT; ++i) {
    v = ld_line(p);
    if (v.y == gen && v.w == gen) return true;
    if ((i & 63u) == 63u && global_ns() - t0 > budget_ns) return false;
  }
  return false;
}
__device__ __forceinline__ void add_bf2(float* acc, uint32_t packed) {
  const bf162 t = *reinterpret_cast<const bf162*>(&packed);
  acc[0] += __low2float(t);
  acc[1] += __high2float(t);
}

// Sum of squares of the four bf16 values of a finished line, summed over the 32 lanes of the
// warp (= the 128 features of the tile for one token column); lane 0 stores it. Every lane of the
// warp must call it (the launcher requires N % 128 == 0 when `ss_out` is given).
__device__ __forceinline__ void emit_sumsq(float* ss_out, int ss_ld, int tile, int c, uint32_t lo,
                                           uint32_t hi) {
  if (ss_out == nullptr) return;
  float f[4] = {0.f, 0.f, 0.f, 0.f};
  add_bf2(f, lo);
  add_bf2(f + 2, hi);
  const float ss = warp_sum(f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3]);
  if ((threadIdx.x & 31) == 0) ss_out[(long long)c * ss_ld + tile] = ss;
}

// Reduces this thread's share (entries `first`, `first + 4`, ... of the column list `cols[0..n)`)
// of one 4-feature line: NSRC remote partials polled out of this rank's receive region plus its
// own partial from `tile`, summed in rank order. RB rows are kept in flight at once so that the
// L2 round trips of the polls overlap. Returns false if a peer's line never arrived.
// bcast_peers != nullptr (two-shot): the finished line also goes to every other rank's final
// region, at byte offset bcast_off of its slab, line index c * lines_per_row + feat / 4.
template <int NSRC, int BM_>
__device__ __forceinline__ bool reduce_lines(const uint4* __restrict__ base, const bf16* tile,
                                             bf16* out, const bf16* __restrict__ bias,
                                             const bf16* residual, long long ldo,
                                             int rank, int m_cap, int lines_per_row, int feat,
                                             int line, int first, const short* cols, int n,
                                             uint32_t gen, void* const* bcast_peers,
                                             long long bcast_off, float* ss_out, int ss_ld) {
  constexpr int R = NSRC + 1;
  constexpr int RB = 16 / NSRC > 0 ? 16 / NSRC : 1;
  bool ok = true;
  float b4[4] = {0.f, 0.f, 0.f, 0.f};
  if (bias != nullptr) {
    const uint2 bv = *reinterpret_cast<const uint2*>(bias + feat);
    add_bf2(b4, bv.x);
    add_bf2(b4 + 2, bv.y);
  }
  for (int i0 = first; i0 < n; i0 += 4 * RB) {
    uint4 v[RB][NSRC];
#pragma unroll
    for (int rr = 0; rr < RB; ++rr) {
      const int i = i0 + 4 * rr;
      if (i < n) {
        const int c = cols[i];
#pragma unroll
        for (int j = 0; j < NSRC; ++j) {
          const int src = j < rank ? j : j + 1;
          v[rr][j] = ld_line(base + ((long long)src * m_cap + c) * lines_per_row + (feat >> 2));
        }
      }
    }
#pragma unroll
    for (int rr = 0; rr < RB; ++rr) {
      const int i = i0 + 4 * rr;
      if (i >= n) continue;
      const int c = cols[i];
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int src = 0; src < R; ++src) {
        if (src == rank) {
          const uint2 d = *reinterpret_cast<const uint2*>(tile + c * BM_ + line * 4);
          add_bf2(acc, d.x);
          add_bf2(acc + 2, d.y);
        } else {
          const int j = src < rank ? src : src - 1;
          // j is a compile-time constant after unrolling only when rank is; select by a chain
          uint4 w = v[rr][0];
#pragma unroll
          for (int jj = 1; jj < NSRC; ++jj)
            if (jj == j) w = v[rr][jj];
          if (!wait_line(base + ((long long)src * m_cap + c) * lines_per_row + (feat >> 2), gen, w,
                         ok ? GV_WAIT_NS : 0ull))
            ok = false;
          add_bf2(acc, w.x);
          add_bf2(acc + 2, w.z);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] += b4[k];
      if (residual != nullptr) {
        const uint2 rv = *reinterpret_cast<const uint2*>(residual + (long long)c * ldo + feat);
        add_bf2(acc, rv.x);
        add_bf2(acc + 2, rv.y);
      }
      uint2 o;
      o.x = pack2(acc[0], acc[1]);
      o.y = pack2(acc[2], acc[3]);
      *reinterpret_cast<uint2*>(out + (long long)c * ldo + feat) = o;
      emit_sumsq(ss_out, ss_ld, blockIdx.x, c, o.x, o.y);
      if (bcast_peers != nullptr) {
#pragma unroll
        for (int p = 1; p < R; ++p) {
          const int peer = (rank + p) % R;
          uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(bcast_peers[peer]) + bcast_off) +
                       (long long)c * lines_per_row + (feat >> 2);
          st_line(dst, o.x, o.y, gen);
        }
      }
    }
  }
  return ok;
}

// Two-shot, receiving side: wait for the owners' finished lines of the columns `cols[0..n)` in
// this rank's final region and copy them to `out`. Up to 16 rows in flight.
__device__ __forceinline__ bool copy_final_lines(const uint4* __restrict__ fin, bf16* out,
                                                 long long ldo, int lines_per_row, int feat, int first,
                                                 const short* cols, int n, uint32_t gen, float* ss_out,
                                                 int ss_ld) {
  bool ok = true;
  for (int i0 = first; i0 < n; i0 += 4 * 16) {
    uint4 v[16];
#pragma unroll
    for (int rr = 0; rr < 16; ++rr) {
      const int i = i0 + 4 * rr;
      if (i < n) v[rr] = ld_line(fin + (long long)cols[i] * lines_per_row + (feat >> 2));
    }
#pragma unroll
    for (int rr = 0; rr < 16; ++rr) {
      const int i = i0 + 4 * rr;
      if (i >= n) continue;
      const int c = cols[i];
      if (!wait_line(fin + (long long)c * lines_per_row + (feat >> 2), gen, v[rr], ok ? GV_WAIT_NS : 0ull)) ok = false;
      *reinterpret_cast<uint2*>(out + (long long)c * ldo + feat) = make_uint2(v[rr].x, v[rr].z);
      emit_sumsq(ss_out, ss_ld, blockIdx.x, c, v[rr].x, v[rr].z);
    }
  }
  return ok;
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 2)
gemm_allreduce_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                      const __grid_constant__ CUtensorMap tmNext, bf16* out, const bf16* __restrict__ bias,
                      const bf16* residual, int N, int M, int K, long long ldo, int splitk, ArArgs a,
                      NextWeights next, int early_trigger, unsigned int* status) {
  using C = Cfg<BN, 108>;
  extern __shared__ uint8_t smem_raw[];
  const Shared sh = carve<C>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p0 = blockIdx.x * BM;
  const int kb_total = (K + BK - 1) / BK;
  const int kb_per = (kb_total + splitk - 1) / splitk;
  const int z = blockIdx.z;
  const int kb0 = z * kb_per;
  const int nkb = max(0, min(kb_total, kb0 + kb_per) - kb0);
  const int cta = blockIdx.x + gridDim.x * blockIdx.z;

  // weights (P) are constant and are prefetched before the wait on the kernel in front
  if (next.stages > 0) next.tm = &tmNext;
  const uint32_t tmem_base = run_mainloop<C>(sh, &tmW, &tmX, p0, 0, kb0, nkb, status, -1, -1, early_trigger ? 1 : 3, &next);
  // the channel generation is bumped by the previous user of the channel: read it after the wait
  const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]) + 1u;

  const int quad = warp & 3;
  const int lrow = quad * 32 + lane;
  // shared staging (the operand ring is idle once the accumulator is complete):
  //   red  : fp32 [BN][128]  split-K exchange   (only when splitk > 1)
  //   tile : bf16 [BN][128]  transposed partial tile to push
  float* red = reinterpret_cast<float*>(sh.ring);
  bf16* tile = reinterpret_cast<bf16*>(sh.ring + (splitk > 1 ? BN * BM * 4 : 0));

  if (warp >= 2) {
    wait_accum(sh, status);
#pragma unroll 1
    for (int c = 0; c < BN; c += 16) {
      uint32_t r[16];
      sm100::tmem_ld16(tmem_addr(tmem_base, quad, c), r);
      sm100::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (splitk > 1) red[(c + j) * BM + lrow] = __uint_as_float(r[j]);
        else tile[(c + j) * BM + lrow] = f2bf(__uint_as_float(r[j]));
      }
    }
  }
  if (splitk > 1) {
    cluster_sync_all();
    if (warp >= 2) {
      const int et0 = threadIdx.x - 64;
      const int nc = (BN - z + splitk - 1) / splitk;
      for (int idx = et0; idx < nc * 32; idx += 128) {
        const int c = z + (idx >> 5) * splitk;
        const int r4 = (idx & 31) * 4;
        const float4 a4 = cluster_sum4(&red[c * BM + r4], splitk);
        uint2 pk;
        pk.x = pack2(a4.x, a4.y);
        pk.y = pack2(a4.z, a4.w);
        *reinterpret_cast<uint2*>(tile + c * BM + r4) = pk;
      }
    }
    cluster_sync_all();
  }
  // Column (token) lists of this CTA: `s_own` = columns this rank reduces, `s_oth` = columns some
  // other rank reduces (two-shot only). In two-shot mode column c of feature tile t belongs to
  // rank (t + c) % R, so every CTA of every rank reduces 1 / R of its columns and the polling
  // work is spread evenly.
  __shared__ short s_own[BN], s_oth[BN];
  __shared__ int s_nown, s_noth;
  if (warp >= 2) {
    const int et = threadIdx.x - 64;        // 0..127 among the epilogue threads
    if (et == 0) {
      const int mycols = splitk > 1 ? (BN - z + splitk - 1) / splitk : BN;
      int no = 0, nt = 0;
      for (int i = 0; i < mycols; ++i) {
        const int c = splitk > 1 ? z + i * splitk : i;
        if (c >= M) continue;
        if (!a.two_shot || (int)((blockIdx.x + (unsigned)c) % (unsigned)a.R) == a.rank) s_own[no++] = (short)c;
        else s_oth[nt++] = (short)c;
      }
      s_nown = no;
      s_noth = nt;
    }
    epi_bar();                              // `tile` and the column lists are complete
    const int line = et & 31, rsub = et >> 5;  // 32 four-feature lines per tile row, 4 rows / pass
    const int feat = p0 + line * 4;
    const bool feat_ok = feat + 4 <= N;     // N % 8 == 0 enforced by the launcher
    const int lines_per_row = N >> 2;
    const long long par_lines = (long long)a.R * a.m_cap * lines_per_row;
    const long long my_src = ((long long)(gen & 1u) * a.R + a.rank) * a.m_cap * lines_per_row;
    const int nown = s_nown, noth = s_noth;
    // final region: after the 2 x R partial regions, one per parity
    const long long fin_off =
        a.recv_off + 16ll * (2ll * par_lines + (long long)(gen & 1u) * a.m_cap * lines_per_row);
    if (feat_ok) {
      // ---- push my partial lines: one-shot = every column to every other rank; two-shot = the
      // columns I do not reduce, each to its owner only
      if (!a.two_shot) {
        for (int p = 1; p < a.R; ++p) {
          const int peer = (a.rank + p) % a.R;  // ring order spreads the first stores over the links
          uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(a.peers[peer]) + a.recv_off) + my_src;
          for (int i = rsub; i < nown; i += 4) {
            const int c = s_own[i];
            const uint2 d = *reinterpret_cast<const uint2*>(tile + c * BM + line * 4);
            st_line(dst + (long long)c * lines_per_row + (feat >> 2), d.x, d.y, gen);
          }
        }
      } else {
        for (int i = rsub; i < noth; i += 4) {
          const int c = s_oth[i];
          const int owner = (int)((blockIdx.x + (unsigned)c) % (unsigned)a.R);
          uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(a.peers[owner]) + a.recv_off) + my_src;
          const uint2 d = *reinterpret_cast<const uint2*>(tile + c * BM + line * 4);
          st_line(dst + (long long)c * lines_per_row + (feat >> 2), d.x, d.y, gen);
        }
      }
      // ---- reduce the R partials of the columns I own in rank order (and broadcast them)
      const uint4* base = reinterpret_cast<const uint4*>(static_cast<char*>(a.peers[a.rank]) + a.recv_off) +
                          (long long)(gen & 1u) * par_lines;
      bool ok = true;
      void* const* bc = a.two_shot ? a.peers : nullptr;
#define GV_AR_REDUCE(NSRC)                                                                        \
  ok = reduce_lines<NSRC, BM>(base, tile, out, bias, residual, ldo, a.rank, a.m_cap,              \
                              lines_per_row, feat, line, rsub, s_own, nown, gen, bc, fin_off,    \
                              a.ss_out, a.ss_ld)
      switch (a.R) {
        case 1: {  // single rank: own partial only
          for (int i = rsub; i < nown; i += 4) {
            const int c = s_own[i];
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint2 d = *reinterpret_cast<const uint2*>(tile + c * BM + line * 4);
            add_bf2(acc, d.x);
            add_bf2(acc + 2, d.y);
            if (bias != nullptr) {
              const uint2 bv = *reinterpret_cast<const uint2*>(bias + feat);
              add_bf2(acc, bv.x);
              add_bf2(acc + 2, bv.y);
            }
            if (residual != nullptr) {
              const uint2 rv = *reinterpret_cast<const uint2*>(residual + (long long)c * ldo + feat);
              add_bf2(acc, rv.x);
              add_bf2(acc + 2, rv.y);
            }
            uint2 o;
            o.x = pack2(acc[0], acc[1]);
            o.y = pack2(acc[2], acc[3]);
            *reinterpret_cast<uint2*>(out + (long long)c * ldo + feat) = o;
            emit_sumsq(a.ss_out, a.ss_ld, blockIdx.x, c, o.x, o.y);
          }
          break;
        }
        case 2: GV_AR_REDUCE(1); break;
        case 3: GV_AR_REDUCE(2); break;
        case 4: GV_AR_REDUCE(3); break;
        case 5: GV_AR_REDUCE(4); break;
        case 6: GV_AR_REDUCE(5); break;
        case 7: GV_AR_REDUCE(6); break;
        case 8: GV_AR_REDUCE(7); break;
        default: ok = false; break;  // the launcher rejects R > 8
      }
#undef GV_AR_REDUCE
      // ---- two-shot: collect the finished lines of the columns other ranks own
      if (a.two_shot && noth > 0) {
        const uint4* fin = reinterpret_cast<const uint4*>(static_cast<char*>(a.peers[a.rank]) + fin_off);
        if (!copy_final_lines(fin, out, ldo, lines_per_row, feat, rsub, s_oth, noth, gen, a.ss_out, a.ss_ld))
          ok = false;
      }
      if (!ok) atomicOr(status, GV_ST_TIMEOUT_PEER);
    }
  }
  finish<C>(sh, tmem_base);
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int total = gridDim.x * gridDim.z;
    if (atomicAdd(&a.state[1], 1u) == total - 1) {
      a.state[1] = 0;
      __threadfence();
      a.state[0] = gen;
    }
  }
}

// How the fused GEMM + all-reduce takes part in programmatic dependent launch (GVIRT_AR_PDL):
// bit 0 = the kernel itself may start before the kernel in front has drained, bit 1 = it lets the
// kernel behind it start early. Across GPUs the kernel's push phase is on every peer's critical
// path, so what shares the SMs and HBM with it matters more than on one GPU. Default 2: the kernel
// waits for the kernel in front to drain (measured: its early start is what costs, Llama-3-8B TP4
// 20.1 k tok/s against 16.5 k, Qwen3-30B-A3B on 4 GPUs 15.1 k against 14.9 k) and lets its follower in.
static int ar_pdl_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("GVIRT_AR_PDL");
    mode = (e != nullptr && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 2;
  }
  return mode;
}

template <int BN>
static int launch_ar(const CUtensorMap& tmW, const CUtensorMap& tmX, bf16* out, const bf16* bias,
                     const bf16* residual, int N, int M, int K, long long ldo, int splitk,
                     const ArArgs& a, cudaStream_t st, const CUtensorMap& tmNextIn, const NextWeights& next) {
  CUtensorMap tmNext = next.stages > 0 ? tmNextIn : tmW;
  using C = Cfg<BN, 108>;
  static_assert(C::STAGES * C::STAGE_BYTES >= BN * BM * 6, "staging must fit in the ring");
  auto kern = gemm_allreduce_kernel<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_last_error("gemm_allreduce: smem attr", e);
      return GV_ECUDA;
    }
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ceil_div(N, BM), 1, (unsigned)splitk);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (splitk > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = (unsigned)splitk;
    ++na;
  }
  if (pdl_enabled() && (ar_pdl_mode() & 1)) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmW, tmX, tmNext, out, bias, residual, N, M, K, ldo, splitk,
                                     a, next, (ar_pdl_mode() >> 1) & 1, status_word());
  if (e != cudaSuccess) {
    set_last_error("gemm_allreduce: launch", e);
    return GV_ECUDA;
  }
  return GV_OK;
}

}  // namespace gemm
}  // namespace gv

using namespace gv;
using namespace gv::gemm;

// x [M, K] (this rank's K shard of the activations), w [N, K] (this rank's K shard of the weight),
// out [M, N] local. Receive region must hold 2 * (R + 1) * m_cap * N / 4 sixteen-byte lines
// (= 8 * (R + 1) * m_cap * N bytes): per parity R partial regions, then (after all of them) one
// final region per parity that only the two-shot mode uses. Returns GV_EUNSUPPORTED when the shape does not fit the fused path (caller falls back).
extern "C" int gv_gemm_allreduce_ss(const void* x, const void* w, const void* bias,
                                    const void* residual, void* out, void* ss_out, long long ss_ld,
                                    long long M, long long N, long long K, long long ldx,
                                    long long ldw, long long ldo, const void* peers,
                                    long long recv_off, long long flags_off, void* state,
                                    long long rank, long long R, long long m_cap,
                                    long long max_ctas, long long two_shot, void* stream) {
  CUtensorMap tmNext;
  NextWeights next = {nullptr, 0, 0, 0, 0, 0};
  {
    const int bn0 = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    take_next_weights((M > 0 && M <= 128) ? bn0 : 0, &tmNext, &next);   // consumed even if the launch is refused
  }
  if (!x || !w || !out || !peers || !state || M <= 0 || N <= 0 || K <= 0) return GV_EINVAL;
  if (ss_out && ((N % 128) || ss_ld < N / 128)) return GV_EINVAL;
  if ((K & 7) || (ldx & 7) || (ldw & 7) || (N & 7) || (ldo & 7)) return GV_EINVAL;
  if (M > 256 || M > m_cap || R < 1 || R > AR_MAX_RANKS) return GV_EUNSUPPORTED;
  const int tiles = ceil_div(N, BM);
  if (tiles > max_ctas) return GV_EUNSUPPORTED;
  const int kb_total = ceil_div(K, BK);
  int sk = (int)(max_ctas / tiles);
  if (sk > 8) sk = 8;
  while (sk > 1 && kb_total / sk < 2) --sk;
  if (sk < 1) sk = 1;
  {
    const int per = (kb_total + sk - 1) / sk;
    sk = (kb_total + per - 1) / per;
  }
  const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  if (bn == 256) return GV_EUNSUPPORTED;  // two-CTA ring has no room for a 256-column staging tile
  CUtensorMap tmW, tmX;
  int rc;
  if ((rc = cached_tmap_bf16(&tmW, w, N, K, ldw, BM)) != GV_OK) return rc;
  if ((rc = cached_tmap_bf16(&tmX, x, M, K, ldx, bn)) != GV_OK) return rc;
  ArArgs a;
  a.peers = (void* const*)peers;
  a.recv_off = recv_off;
  a.flags_off = flags_off;
  a.state = (unsigned int*)state;
  a.rank = (int)rank;
  a.R = (int)R;
  a.m_cap = (int)m_cap;
  a.two_shot = (two_shot && R > 1) ? 1 : 0;
  a.ss_out = (float*)ss_out;
  a.ss_ld = (int)ss_ld;
  cudaStream_t st = (cudaStream_t)stream;
  switch (bn) {
    case 16: return launch_ar<16>(tmW, tmX, (bf16*)out, (const bf16*)bias, (const bf16*)residual, (int)N, (int)M, (int)K, ldo, sk, a, st, tmNext, next);
    case 32: return launch_ar<32>(tmW, tmX, (bf16*)out, (const bf16*)bias, (const bf16*)residual, (int)N, (int)M, (int)K, ldo, sk, a, st, tmNext, next);
    case 64: return launch_ar<64>(tmW, tmX, (bf16*)out, (const bf16*)bias, (const bf16*)residual, (int)N, (int)M, (int)K, ldo, sk, a, st, tmNext, next);
    default: return launch_ar<128>(tmW, tmX, (bf16*)out, (const bf16*)bias, (const bf16*)residual, (int)N, (int)M, (int)K, ldo, sk, a, st, tmNext, next);
  }
}

extern "C" int gv_gemm_allreduce(const void* x, const void* w, const void* bias,
                                 const void* residual, void* out, long long M, long long N,
                                 long long K, long long ldx, long long ldw, long long ldo,
                                 const void* peers, long long recv_off, long long flags_off,
                                 void* state, long long rank, long long R, long long m_cap,
                                 long long max_ctas, long long two_shot, void* stream) {
  return gv_gemm_allreduce_ss(x, w, bias, residual, out, nullptr, 0, M, N, K, ldx, ldw, ldo, peers,
                              recv_off, flags_off, state, rank, R, m_cap, max_ctas, two_shot, stream);
}

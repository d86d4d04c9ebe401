// bf16 GEMM on tcgen05 tensor cores:  out[M, N] = x[M, K] . w[N, K]^T (+ bias[N]).
//
// Covers the role of the reference's cube-core `matmul_<T>` (xlite/csrc/kernels/matmul.h:437,
// host side xlite/csrc/op.cpp:690-808) for the linear layers, lm_head and the router, but
// is designed around Blackwell: TMA-fed 128-byte-swizzled operand ring, one elected thread
// issuing tcgen05.mma, fp32 accumulators in TMEM, and two problem orientations:
//
//   * "token-major"  (M > 256): activations on the 128 TMEM lanes, a BN-wide weight tile on
//     the columns; grid walks tiles in groups of 16 lane tiles so a wave re-uses weights and
//     activations out of L2.
//   * "weight-major" (M <= 256, decode): the weight rows ride the 128 lanes and the few
//     tokens ride the columns, so every CTA streams a full-width weight tile from HBM. When
//     N/128 tiles cannot fill 148 SMs the K range is split across a thread-block cluster
//     and the partial tiles are summed in rank order through distributed shared memory
//     (deterministic; no global scratch, no atomics).
#include "gemm_core.cuh"
#include "gvirt_kernels.h"
#include <mutex>
#include <unordered_map>

namespace gv {
namespace gemm {

// SWAP = false: lanes index rows of `out`, columns index columns of `out` (token-major).
// SWAP = true : lanes index columns of `out` (features), columns index rows (tokens).
template <int BN, bool SWAP, int BUDGET_KB>
__global__ void __launch_bounds__(NUM_THREADS, (BUDGET_KB <= 110 ? 2 : 1))
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                 bf16* __restrict__ out, const bf16* __restrict__ bias, int rowsP, int rowsQ, int K,
                 long long ldo, int tilesP, int tilesQ, int splitk, int epi, unsigned int* status) {
  using C = Cfg<BN, BUDGET_KB>;
  extern __shared__ uint8_t smem_raw[];
  const Shared sh = carve<C>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // grouped rasterisation: 16 lane tiles share a sweep over the column tiles
  int tp, tq;
  {
    const int GROUP = 16;
    const int t = blockIdx.x;
    const int per_group = GROUP * tilesQ;
    const int g = t / per_group;
    const int first = g * GROUP;
    const int gsz = min(GROUP, tilesP - first);
    const int r = t - g * per_group;
    tp = first + r % gsz;
    tq = r / gsz;
  }
  const int p0 = tp * BM, q0 = tq * BN;
  const int kb_total = (K + BK - 1) / BK;
  const int kb_per = (kb_total + splitk - 1) / splitk;
  const int z = blockIdx.z;
  const int kb0 = z * kb_per;
  const int nkb = max(0, min(kb_total, kb0 + kb_per) - kb0);

  // the weight operand is constant: P when weights ride the lanes, Q otherwise
  const uint32_t tmem_base =
      run_mainloop<C>(sh, &tmP, &tmQ, p0, q0, kb0, nkb, status, -1, -1, SWAP ? 1 : 2);

  const int quad = warp & 3;
  const int lrow = quad * 32 + lane;  // TMEM lane handled by this thread (epilogue warps)

  if (epi == 1) {
    // ---- SwiGLU epilogue. The weight rows are stored in blocks of 128 = [64 gate | 64 up] of the
    // same 64 features, so one accumulator tile holds both halves of a feature:
    //     out[token, f] = silu(acc[gate row of f]) * acc[up row of f],   out is [tokens, N / 2].
    if (SWAP) {
      float* red = reinterpret_cast<float*>(sh.ring);  // fp32 [BN][128]; the ring is idle by now
      if (warp >= 2) {
        wait_accum(sh, status);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          sm100::tmem_ld16(tmem_addr(tmem_base, quad, c), r);
          sm100::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) red[(c + j) * BM + lrow] = __uint_as_float(r[j]);
        }
      }
      if (splitk > 1) cluster_sync_all();
      else if (warp >= 2) asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp >= 2) {
        const int et = threadIdx.x - 64;
        const int z = blockIdx.z;
        const int ncols = splitk > 1 ? (BN - z + splitk - 1) / splitk : BN;
        const int half = rowsP >> 1;  // output features
        for (int idx = et; idx < ncols * 16; idx += 128) {
          const int c = splitk > 1 ? z + (idx >> 4) * splitk : (idx >> 4);
          const int r4 = (idx & 15) * 4;
          const int q = q0 + c, f = (p0 >> 1) + r4;
          if (q >= rowsQ || f >= half) continue;
          float4 g4, u4;
          if (splitk > 1) {
            g4 = cluster_sum4(&red[c * BM + r4], splitk);
            u4 = cluster_sum4(&red[c * BM + 64 + r4], splitk);
          } else {
            g4 = *reinterpret_cast<const float4*>(&red[c * BM + r4]);
            u4 = *reinterpret_cast<const float4*>(&red[c * BM + 64 + r4]);
          }
          const float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w};
          float o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // the unfused path rounds the GEMM output to bf16 before the activation: do the same
            const float gj = bf2f(f2bf(g[j])), uj = bf2f(f2bf(u[j]));
            o[j] = gj / (1.f + __expf(-gj)) * uj;
          }
          bf16* dst = out + (long long)q * ldo + f;
          if (f + 4 <= half && ((ldo | f) & 3) == 0) {
            uint2 pk;
            pk.x = pack_bf2(o[0], o[1]);
            pk.y = pack_bf2(o[2], o[3]);
            *reinterpret_cast<uint2*>(dst) = pk;
          } else {
            for (int j = 0; j < 4 && f + j < half; ++j) dst[j] = f2bf(o[j]);
          }
        }
      }
      if (splitk > 1) cluster_sync_all();  // peers may still be reading this CTA's shared memory
    } else if (warp >= 2) {
      // token-major: lanes = tokens, every 128 accumulator columns = [64 gate | 64 up]
      wait_accum(sh, status);
      const int p = p0 + lrow;
      const int half = rowsQ >> 1;
#pragma unroll 1
      for (int blk = 0; blk < BN; blk += 128) {
#pragma unroll 1
        for (int c = 0; c < 64; c += 16) {
          uint32_t rg[16], ru[16];
          sm100::tmem_ld16(tmem_addr(tmem_base, quad, blk + c), rg);
          sm100::tmem_ld16(tmem_addr(tmem_base, quad, blk + 64 + c), ru);
          sm100::tmem_ld_wait();
          const int f = ((q0 + blk) >> 1) + c;
          if (p < rowsP && f < half) {
            float o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float gj = bf2f(f2bf(__uint_as_float(rg[j]))), uj = bf2f(f2bf(__uint_as_float(ru[j])));
              o[j] = gj / (1.f + __expf(-gj)) * uj;
            }
            bf16* dst = out + (long long)p * ldo + f;
            if (f + 16 <= half && ((ldo | f) & 7) == 0) {
              st8(dst, pack8(o));
              st8(dst + 8, pack8(o + 8));
            } else {
              for (int j = 0; j < 16 && f + j < half; ++j) dst[j] = f2bf(o[j]);
            }
          }
        }
      }
    }
  } else if (splitk == 1) {
    if (warp >= 2) {
      wait_accum(sh, status);
      const int p = p0 + lrow;
      float bias_p = 0.f;
      if (SWAP && bias != nullptr && p < rowsP) bias_p = bf2f(bias[p]);
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        uint32_t r[16];
        sm100::tmem_ld16(tmem_addr(tmem_base, quad, c), r);
        sm100::tmem_ld_wait();
        if (SWAP) {
          if (p < rowsP) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int q = q0 + c + j;
              if (q < rowsQ) out[(long long)q * ldo + p] = f2bf(__uint_as_float(r[j]) + bias_p);
            }
          }
        } else {
          if (p < rowsP) {
            bf16* orow = out + (long long)p * ldo;
            const int q = q0 + c;
            if (q + 16 <= rowsQ && ((ldo | q) & 7) == 0) {
              float f[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                f[j] = __uint_as_float(r[j]);
                if (bias != nullptr) f[j] += bf2f(bias[q + j]);
              }
              st8(orow + q, pack8(f));
              st8(orow + q + 8, pack8(f + 8));
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (q + j < rowsQ) {
                  float v = __uint_as_float(r[j]);
                  if (bias != nullptr) v += bf2f(bias[q + j]);
                  orow[q + j] = f2bf(v);
                }
              }
            }
          }
        }
      }
    }
  } else {
    // ---- split-K: exchange fp32 partial tiles through distributed shared memory ----
    float* red = reinterpret_cast<float*>(sh.ring);  // [BN][128], free once tmem_full fired
    if (warp >= 2) {
      wait_accum(sh, status);
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        uint32_t r[16];
        sm100::tmem_ld16(tmem_addr(tmem_base, quad, c), r);
        sm100::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) red[(c + j) * BM + lrow] = __uint_as_float(r[j]);
      }
    }
    cluster_sync_all();
    if (warp >= 2) {
      // this CTA finishes the columns c = z, z + splitk, ...; a thread takes 4 consecutive lanes
      const int et = threadIdx.x - 64;
      const int ncols = (BN - z + splitk - 1) / splitk;
      for (int idx = et; idx < ncols * 32; idx += 128) {
        const int c = z + (idx >> 5) * splitk;
        const int r4 = (idx & 31) * 4;
        const int q = q0 + c, p = p0 + r4;
        if (q >= rowsQ || p >= rowsP) continue;
        const float4 acc4 = cluster_sum4(&red[c * BM + r4], splitk);
        float a[4] = {acc4.x, acc4.y, acc4.z, acc4.w};
        if (SWAP) {
          bf16* dst = out + (long long)q * ldo + p;
          if (p + 4 <= rowsP && ((ldo | p) & 3) == 0) {
            if (bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 4; ++j) a[j] += bf2f(bias[p + j]);
            }
            uint2 pk;
            pk.x = pack_bf2(a[0], a[1]);
            pk.y = pack_bf2(a[2], a[3]);
            *reinterpret_cast<uint2*>(dst) = pk;
          } else {
            for (int j = 0; j < 4 && p + j < rowsP; ++j)
              dst[j] = f2bf(a[j] + (bias != nullptr ? bf2f(bias[p + j]) : 0.f));
          }
        } else {
          const float bq = bias != nullptr ? bf2f(bias[q]) : 0.f;
          for (int j = 0; j < 4 && p + j < rowsP; ++j) out[(long long)(p + j) * ldo + q] = f2bf(a[j] + bq);
        }
      }
    }
    cluster_sync_all();  // peers may still be reading this CTA's shared memory
  }
  finish<C>(sh, tmem_base);
}

// ------------------------------------------------------------------ host side
struct TmapKey {
  const void* base;
  long long rows, cols, stride;
  int box_rows;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && stride == o.stride &&
           box_rows == o.box_rows;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.stride;
    h = h * 1000003u ^ (size_t)k.box_rows;
    return h;
  }
};

// Tensor maps are pure functions of (pointer, shape, box); weights and arena tensors keep
// their addresses, so encoding is amortised across steps.
int cached_tmap_bf16(CUtensorMap* out, const void* base, long long rows, long long cols,
                     long long row_stride_elems, int box_rows) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key{base, rows, cols, row_stride_elems, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return GV_OK;
  }
  int rc = sm100::make_tmap_2d(out, base, 2, rows, cols, row_stride_elems * 2, box_rows, BK);
  if (rc != GV_OK) return rc;
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, *out);
  return GV_OK;
}

template <int BN, bool SWAP, int BUDGET_KB>
static int launch(const CUtensorMap& tmP, const CUtensorMap& tmQ, bf16* out, const bf16* bias,
                  int rowsP, int rowsQ, int K, long long ldo, int splitk, cudaStream_t st,
                  int epi = 0) {
  using C = Cfg<BN, BUDGET_KB>;
  auto kern = gemm_bf16_kernel<BN, SWAP, BUDGET_KB>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_last_error("gemm_bf16: cudaFuncSetAttribute(smem)", e);
      return GV_ECUDA;
    }
    configured = true;
  }
  const int tilesP = ceil_div(rowsP, BM), tilesQ = ceil_div(rowsQ, BN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tilesP * tilesQ), 1, (unsigned)splitk);
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
  if (pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmP, tmQ, out, bias, rowsP, rowsQ, K, ldo, tilesP,
                                     tilesQ, splitk, epi, status_word());
  if (e != cudaSuccess) {
    set_last_error("gemm_bf16: launch", e);
    return GV_ECUDA;
  }
  return GV_OK;
}

// Split factor for the weight-major path: fill ~148 SMs, keep >= 4 k-blocks per CTA,
// cluster size <= 8 (portable limit).
static int pick_splitk(int tiles, int kb_total, int num_sms) {
  // two CTAs can share an SM on the weight-major path; aiming at ~1.5 CTAs per SM measured best
  // (more splits add cluster-reduction work faster than they add bandwidth)
  const int slots = num_sms + num_sms / 2;
  if (tiles * 2 > slots) return 1;
  int s = slots / tiles;
  if (s > 8) s = 8;
  while (s > 1 && kb_total / s < 4) --s;
  if (s < 1) s = 1;
  // every split must own at least one k-block
  const int per = (kb_total + s - 1) / s;
  s = (kb_total + per - 1) / per;
  return s;
}

// Per-shape split-K overrides for the weight-major path, filled from a measured table
// (tools/gemm_sweep.py): the role of the reference's (n, k) -> swizzle table
// (xlite/csrc/swizzle.cpp:9-13, `configure_swizzle`), for the knob that matters here.
static std::mutex g_tune_mu;
static std::unordered_map<unsigned long long, int> g_splitk_override;
static inline unsigned long long tune_key(long long N, long long K, int bn) {
  return ((unsigned long long)N << 36) ^ ((unsigned long long)K << 10) ^ (unsigned long long)bn;
}
static int lookup_splitk(long long N, long long K, int bn) {
  std::lock_guard<std::mutex> g(g_tune_mu);
  auto it = g_splitk_override.find(tune_key(N, K, bn));
  return it == g_splitk_override.end() ? 0 : it->second;
}

// Cluster split-K factor of a weight-major launch over weights [N, K] with a `bn`-token tile:
// `force` if positive, else the measured table, else the heuristic; clamped so that every split
// owns at least one k-block. Shared with the fused decode GEMMs (gemm_decode.cu).
int decode_splitk(long long N, long long K, int bn, long long force) {
  const int tiles = ceil_div(N, BM);
  const int kb_total = ceil_div(K, BK);
  int sk = force > 0 ? (int)force : lookup_splitk(N, K, bn);
  if (sk <= 0) sk = pick_splitk(tiles, kb_total, num_sms());
  if (sk > 8) sk = 8;
  if (sk > kb_total) sk = kb_total;
  const int per = (kb_total + sk - 1) / sk;
  return (kb_total + per - 1) / per;
}

}  // namespace gemm
}  // namespace gv

using namespace gv;
using namespace gv::gemm;

// Pin the cluster split-K factor used for weights [N, K] when the token tile is `bn` (16, 32, 64,
// 128 or 256 = the power of two >= M); splitk 0 removes the entry.
extern "C" int gv_gemm_set_splitk(long long N, long long K, long long bn, long long splitk) {
  if (N <= 0 || K <= 0 || splitk < 0 || splitk > 8) return GV_EINVAL;
  std::lock_guard<std::mutex> g(g_tune_mu);
  if (splitk == 0) g_splitk_override.erase(tune_key(N, K, (int)bn));
  else g_splitk_override[tune_key(N, K, (int)bn)] = (int)splitk;
  return GV_OK;
}

static int gemm_bf16_any(const void* x, const void* w, const void* bias, void* out, long long M,
                         long long N, long long K, long long ldx, long long ldw, long long ldo,
                         long long force_splitk, int epi, void* stream) {
  if (!x || !w || !out || M <= 0 || N <= 0 || K <= 0) return GV_EINVAL;
  if ((K & 7) || (ldx & 7) || (ldw & 7)) return GV_EINVAL;  // 16-byte TMA pitch rule
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return GV_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  bf16* o = (bf16*)out;
  const bf16* b = (const bf16*)bias;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  CUtensorMap tmP, tmQ;
  int rc;
  if (M <= 256) {
    // weight-major: lanes = weight rows, columns = tokens
    int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    if ((rc = cached_tmap_bf16(&tmP, w, N, K, ldw, BM)) != GV_OK) return rc;
    if ((rc = cached_tmap_bf16(&tmQ, x, M, K, ldx, bn)) != GV_OK) return rc;
    const int tiles = ceil_div(N, BM);
    const int kb_total = ceil_div(K, BK);
    int sk = force_splitk > 0 ? (int)force_splitk : lookup_splitk(N, K, bn);
    if (sk <= 0) sk = pick_splitk(tiles, kb_total, num_sms);
    if (sk > 8) sk = 8;
    if (sk > kb_total) sk = kb_total;
    {
      const int per = (kb_total + sk - 1) / sk;
      sk = (kb_total + per - 1) / per;
    }
    switch (bn) {
      case 16: return launch<16, true, 108>(tmP, tmQ, o, b, (int)N, (int)M, (int)K, ldo, sk, st, epi);
      case 32: return launch<32, true, 108>(tmP, tmQ, o, b, (int)N, (int)M, (int)K, ldo, sk, st, epi);
      case 64: return launch<64, true, 108>(tmP, tmQ, o, b, (int)N, (int)M, (int)K, ldo, sk, st, epi);
      case 128: return launch<128, true, 108>(tmP, tmQ, o, b, (int)N, (int)M, (int)K, ldo, sk, st, epi);
      default: return launch<256, true, 220>(tmP, tmQ, o, b, (int)N, (int)M, (int)K, ldo, sk, st, epi);
    }
  }
  // token-major
  const int bn = (N >= 256) ? 256 : ((N > 64 || epi == 1) ? 128 : 64);
  if ((rc = cached_tmap_bf16(&tmP, x, M, K, ldx, BM)) != GV_OK) return rc;
  if ((rc = cached_tmap_bf16(&tmQ, w, N, K, ldw, bn)) != GV_OK) return rc;
  switch (bn) {
    case 64: return launch<64, false, 220>(tmP, tmQ, o, b, (int)M, (int)N, (int)K, ldo, 1, st, epi);
    case 128: return launch<128, false, 220>(tmP, tmQ, o, b, (int)M, (int)N, (int)K, ldo, 1, st, epi);
    default: return launch<256, false, 220>(tmP, tmQ, o, b, (int)M, (int)N, (int)K, ldo, 1, st, epi);
  }
}

extern "C" int gv_gemm_bf16(const void* x, const void* w, const void* bias, void* out, long long M,
                            long long N, long long K, long long ldx, long long ldw, long long ldo,
                            long long force_splitk, void* stream) {
  return gemm_bf16_any(x, w, bias, out, M, N, K, ldx, ldw, ldo, force_splitk, 0, stream);
}

// Gate/up projection with the SwiGLU in the epilogue: w [N = 2 I, K] holds the rows in blocks of
// 128 = [64 gate rows | 64 up rows] of the same 64 features (N % 128 == 0), out [M, I] =
// silu(x . gate^T) * (x . up^T). The [M, 2 I] intermediate never reaches memory.
extern "C" int gv_gemm_bf16_swiglu(const void* x, const void* w, void* out, long long M, long long N,
                                   long long K, long long ldx, long long ldw, long long ldo,
                                   long long force_splitk, void* stream) {
  if (N % 128) return GV_EINVAL;
  return gemm_bf16_any(x, w, nullptr, out, M, N, K, ldx, ldw, ldo, force_splitk, 1, stream);
}

// Decode-step GEMMs with the neighbouring layer ops folded into their epilogues (M <= 128 tokens).
//
// A decoder layer of the reference is matmul -> rope_and_cache -> attention -> matmul ->
// add+norm -> matmul -> silu_and_mul -> matmul -> add+norm, every arrow a launch
// (xlite/csrc/model.cpp:1413-1433 with the pieces at :505-594 and :807-850). At decode sizes each
// of those launches costs a few microseconds of fixed latency for well under a microsecond of
// memory traffic, so this file removes the launches instead of tuning them. One weight-major
// tcgen05 kernel (weights on the 128 TMEM lanes, tokens on the columns, cluster split-K through
// distributed shared memory exactly like gemm_bf16.cu) whose finishing phase is one of:
//
//   EPI_PLAIN   out = s_t * acc (+ bias)
//   EPI_SWIGLU  out = silu(s_t * acc_gate) * (s_t * acc_up)        ([64 gate | 64 up] row blocks)
//   EPI_RESID   x  += acc (+ bias), written in place, and the per-(tile, token) sum of squares of
//               the new x goes to `ss_out[token][tile]`
//   EPI_ROPE    one 128-row tile = one attention head: bias, per-head q/k RMSNorm, NeoX rotation,
//               q scaling; q heads to `q_out`, k / v heads straight into their paged cache slot
//
// with s_t = rsqrt(sum_tiles ss_in[t][tile] / H + eps), the RMSNorm factor of token t. RMSNorm
// never runs as a kernel of its own: the producer of the residual stream (EPI_RESID here, or the
// reduce phase of gemm_allreduce.cu under tensor parallelism) leaves the partial sums of squares
// behind, the norm weight is folded into the consumer's weight columns once at load
// (W' = W diag(g)), and (x * s_t) W'^T = s_t (x W'^T) lets the consumer apply s_t to its
// accumulator column. In the finishing phase a warp owns one token column (32 lanes x 4
// consecutive features = the 128 lanes of the tile), so the column reductions and the rotation
// partner (lane ^ 16) are warp shuffles.
#include "gemm_core.cuh"
#include "gvirt_kernels.h"

namespace gv {
namespace gemm {

int cached_tmap_bf16(CUtensorMap* out, const void* base, long long rows, long long cols,
                     long long row_stride_elems, int box_rows);
int decode_splitk(long long N, long long K, int bn, long long force);

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_RESID = 2, EPI_ROPE = 3 };

struct DecEpi {
  int mode;
  // token scale from partial sums of squares [tokens][ss_ld], entries [t][0 .. ss_tiles) (null: no scale)
  const float* ss_in;
  int ss_tiles, ss_ld;
  float inv_h, eps;
  const bf16* bias;       // [N] or null
  // EPI_RESID
  const bf16* residual;   // [M, ldo], may alias out
  float* ss_out;          // [tokens][ss_ld]: entry [t][tile], or null
  // EPI_ROPE
  const float* cos_sin;   // [max_pos, 128] = [cos | sin]
  const long long* positions;
  const int* slots;
  bf16* k_cache;
  bf16* v_cache;
  const bf16* q_norm_w;
  const bf16* k_norm_w;
  int nq, nkv, max_pos;
  long long num_slots;
  float q_scale, qk_eps;
};

__device__ __forceinline__ void unpack4f(uint2 p, float* f) {
  const bf162 a = *reinterpret_cast<const bf162*>(&p.x), b = *reinterpret_cast<const bf162*>(&p.y);
  f[0] = __low2float(a); f[1] = __high2float(a);
  f[2] = __low2float(b); f[3] = __high2float(b);
}
__device__ __forceinline__ uint2 pack4f(const float* f) {
  return make_uint2(pack_bf2(f[0], f[1]), pack_bf2(f[2], f[3]));
}
__device__ __forceinline__ float rbf(float v) { return bf2f(f2bf(v)); }

template <int BN, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 2)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const __grid_constant__ CUtensorMap tmNext, bf16* out, int N, int M, int K,
                   long long ldo, int splitk, DecEpi e, NextWeights next, unsigned int* status) {
  using C = Cfg<BN, 108>;
  extern __shared__ uint8_t smem_raw[];
  const Shared sh = carve<C>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x;
  const int p0 = tile * BM;
  const int kb_total = (K + BK - 1) / BK;
  const int kb_per = (kb_total + splitk - 1) / splitk;
  const int z = blockIdx.z;
  const int kb0 = z * kb_per;
  const int nkb = max(0, min(kb_total, kb0 + kb_per) - kb0);

  // finishing phase geometry: epilogue warp `ew` owns the columns c = z + (ew + 4 i) * splitk
  const int ew = warp - 2;
  const int ncols = (BN - z + splitk - 1) / splitk;
  const int r4 = lane * 4;
  const int p = p0 + r4;
  const bool p_ok = p + 4 <= N;                      // N % 4 == 0 is enforced by the launcher
  const int kind = tile < e.nq ? 0 : (tile < e.nq + e.nkv ? 1 : 2);   // EPI_ROPE: q, k or v head
  // Positions and cache slots are inputs of the step (copied in before its first kernel), not
  // products of the kernel in front: they may be read ahead of the dependency wait, which takes
  // the first half of the position -> cos / sin chain out of the epilogue.
  long long pos_pre[4] = {0, 0, 0, 0};
  int slot_pre[4] = {-1, -1, -1, -1};
  if (MODE == EPI_ROPE && warp >= 2) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ci = ew + 4 * i;
      const int c = z + ci * splitk;
      if (ci < ncols && c < M) {
        if (kind != 2) pos_pre[i] = e.positions[c];
        if (kind != 0) slot_pre[i] = e.slots[c];
      }
    }
  }
  if (next.stages > 0) next.tm = &tmNext;
  const uint32_t tmem_base = run_mainloop<C>(sh, &tmW, &tmX, p0, 0, kb0, nkb, status, -1, -1, 1, &next);

  const int quad = warp & 3;
  const int lrow = quad * 32 + lane;
  float* red = reinterpret_cast<float*>(sh.ring);  // fp32 [BN][128]; the ring is idle by now
  // Inputs of a column's finishing step that do not depend on the accumulator (RMSNorm partial
  // sums, residual row, cos / sin row, cache slot). For the first NPRE columns of a warp they are
  // requested while the main loop is still running, every load of every column issued before the
  // first one is consumed, so their latencies overlap each other and the MMAs.
  struct Side {
    float r[4];          // EPI_RESID: residual row; EPI_ROPE: cos
    float sn[4];         // EPI_ROPE: sin
    int slot;            // EPI_ROPE: cache slot of k / v heads
  };
  auto load_side = [&](int c, long long pos, int slot, Side& sd) {
    sd.slot = slot;
#pragma unroll
    for (int j = 0; j < 4; ++j) sd.r[j] = sd.sn[j] = 0.f;
    if (c >= M) return;
    if (MODE == EPI_RESID) {
      if (p_ok) unpack4f(*reinterpret_cast<const uint2*>(e.residual + (long long)c * ldo + p), sd.r);
    } else if (MODE == EPI_ROPE) {
      if (kind != 2) {
        if (pos < 0 || pos >= e.max_pos) {
          if (lane == 0) atomicOr(status, GV_ST_BAD_INDEX);
          pos = 0;
        }
        const int pair0 = 4 * (lane & 15);
        const float4 c4 = *reinterpret_cast<const float4*>(e.cos_sin + pos * 128 + pair0);
        const float4 s4 = *reinterpret_cast<const float4*>(e.cos_sin + pos * 128 + 64 + pair0);
        sd.r[0] = c4.x; sd.r[1] = c4.y; sd.r[2] = c4.z; sd.r[3] = c4.w;
        sd.sn[0] = s4.x; sd.sn[1] = s4.y; sd.sn[2] = s4.z; sd.sn[3] = s4.w;
      }
    }
  };
  constexpr int NPRE = 4;
  Side pre[NPRE];
  float b4[4] = {0.f, 0.f, 0.f, 0.f};
  // RMSNorm factor of the warp's i-th column, held by lane i (a warp owns at most BN / 4 <= 32
  // columns): each lane sums the partial sums of squares of one token, all lanes at once, so the
  // factors of every column cost one round of memory latency, hidden behind the main loop.
  float my_scale = 1.f;
  __shared__ float s_scale[BN];                        // EPI_SWIGLU: the factors, by column index
  if (warp >= 2) {
    if (e.bias != nullptr && p_ok) unpack4f(*reinterpret_cast<const uint2*>(e.bias + p), b4);
    if (e.ss_in != nullptr) {
      const int ci = ew + 4 * lane;
      const int c = z + ci * splitk;
      if (ci < ncols && c < M) {
        const float* row = e.ss_in + (long long)c * e.ss_ld;
        float acc = 0.f;
#pragma unroll 8
        for (int t = 0; t < e.ss_tiles; ++t) acc += row[t];
        my_scale = rsqrtf(acc * e.inv_h + e.eps);
      }
    }
    if (MODE == EPI_SWIGLU && ew + 4 * lane < BN) s_scale[ew + 4 * lane] = my_scale;
#pragma unroll
    for (int i = 0; i < NPRE; ++i) {
      const int ci = ew + 4 * i;
      load_side(ci < ncols ? z + ci * splitk : M, pos_pre[i], slot_pre[i], pre[i]);
    }
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
  else __syncthreads();
  if (MODE == EPI_SWIGLU && warp >= 2) {
    // Rows 0..63 of the tile are the gate rows of 64 features, rows 64..127 the up rows of the
    // same features: one item = 4 features of one token, all 128 threads busy.
    const int et = threadIdx.x - 64;
    const int half = N >> 1;
    for (int idx = et; idx < ncols * 16; idx += 128) {
      const int ci = idx >> 4;
      const int c = z + ci * splitk;
      const int f4 = (idx & 15) * 4;
      const int f = (p0 >> 1) + f4;
      if (c >= M || f + 4 > half) continue;
      float4 g4, u4;
      if (splitk > 1) {
        g4 = cluster_sum4(&red[c * BM + f4], splitk);
        u4 = cluster_sum4(&red[c * BM + 64 + f4], splitk);
      } else {
        g4 = *reinterpret_cast<const float4*>(&red[c * BM + f4]);
        u4 = *reinterpret_cast<const float4*>(&red[c * BM + 64 + f4]);
      }
      const float sc = s_scale[ci];
      const float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w};
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // the unfused pair rounds the GEMM output to bf16 before activating: do the same
        const float gj = rbf(g[j] * sc), uj = rbf(u[j] * sc);
        o[j] = gj / (1.f + __expf(-gj)) * uj;
      }
      *reinterpret_cast<uint2*>(out + (long long)c * ldo + f) = pack4f(o);
    }
  } else if (warp >= 2) {
    // One token column: 32 lanes x 4 consecutive features = the 128 lanes of the tile.
    auto column = [&](int c, const Side& sd, float sc) {
      float a[4];
      if (splitk > 1) {
        const float4 t = cluster_sum4(&red[c * BM + r4], splitk);
        a[0] = t.x; a[1] = t.y; a[2] = t.z; a[3] = t.w;
      } else {
        const float4 t = *reinterpret_cast<const float4*>(&red[c * BM + r4]);
        a[0] = t.x; a[1] = t.y; a[2] = t.z; a[3] = t.w;
      }
      if (MODE == EPI_PLAIN) {
        if (p_ok) {
          float o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = a[j] * sc + b4[j];
          *reinterpret_cast<uint2*>(out + (long long)c * ldo + p) = pack4f(o);
        }
      } else if (MODE == EPI_RESID) {
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        if (p_ok) {
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = rbf(a[j] + b4[j] + sd.r[j]);
          *reinterpret_cast<uint2*>(out + (long long)c * ldo + p) = pack4f(o);
        }
        if (e.ss_out != nullptr) {
          const float ss = warp_sum(o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3]);
          if (lane == 0) e.ss_out[(long long)c * e.ss_ld + tile] = ss;
        }
      } else {
        // ---- EPI_ROPE: tile = head (q heads, then k heads, then v heads), 128 features each
        const int h = tile;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = rbf(a[j] * sc + b4[j]);
        bf16* dst;
        bool live = true;
        if (kind == 0) {
          dst = out + ((long long)c * e.nq + h) * 128 + r4;
        } else {
          const int slot = sd.slot;
          live = slot >= 0;                             // negative: this token has no cache row
          if ((long long)slot >= e.num_slots) {
            if (lane == 0) atomicOr(status, GV_ST_BAD_INDEX);
            live = false;
          }
          const int kh = kind == 1 ? h - e.nq : h - e.nq - e.nkv;
          dst = (kind == 1 ? e.k_cache : e.v_cache) + ((long long)(live ? slot : 0) * e.nkv + kh) * 128 + r4;
        }
        if (kind == 2) {
          if (live) *reinterpret_cast<uint2*>(dst) = pack4f(v);
          return;
        }
        const bf16* nw = kind == 0 ? e.q_norm_w : e.k_norm_w;
        if (nw != nullptr) {
          const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
          const float ns = rsqrtf(ss / 128.f + e.qk_eps);
          float w[4];
          unpack4f(*reinterpret_cast<const uint2*>(nw + r4), w);
#pragma unroll
          for (int j = 0; j < 4; ++j) v[j] = rbf(v[j] * ns * w[j]);
        }
        const bool is_hi = lane >= 16;
        const float oscale = kind == 0 ? e.q_scale : 1.f;
        float o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
          o[j] = (is_hi ? (v[j] * sd.r[j] + other * sd.sn[j]) : (v[j] * sd.r[j] - other * sd.sn[j])) * oscale;
        }
        if (live) *reinterpret_cast<uint2*>(dst) = pack4f(o);
      }
    };
    // one copy of the column code (kernels this short are sensitive to their instruction footprint)
    Side ahead;                                        // side inputs of the column after this one
#pragma unroll 1
    for (int i = 0, ci = ew; ci < ncols; ++i, ci += 4) {
      const int c = z + ci * splitk;
      if (c >= M) break;                               // warp-uniform
      Side sd;
      if (i < NPRE) {
        sd = pre[0];
#pragma unroll
        for (int k = 1; k < NPRE; ++k)
          if (i == k) sd = pre[k];
      } else {
        sd = ahead;
      }
      if (MODE == EPI_RESID || MODE == EPI_ROPE) {
        // columns past the prefetched ones: request the next column's inputs before this one's
        // arithmetic, so only the first of them waits for memory
        const int cn = c + 4 * splitk;
        if (i + 1 >= NPRE && ci + 4 < ncols && cn < M) {
          long long pos = 0;
          int slot = -1;
          if (MODE == EPI_ROPE) {
            if (kind != 2) pos = e.positions[cn];
            if (kind != 0) slot = e.slots[cn];
          }
          load_side(cn, pos, slot, ahead);
        }
      }
      const float sc = __shfl_sync(0xffffffffu, my_scale, i);
      column(c, sd, sc);
    }
  }
  if (splitk > 1) cluster_sync_all();  // peers may still be reading this CTA's shared memory
  finish<C>(sh, tmem_base);
}

template <int BN, int MODE>
static int launch_dec(const CUtensorMap& tmW, const CUtensorMap& tmX, const CUtensorMap& tmNext,
                      const NextWeights& next, bf16* out, int N, int M, int K, long long ldo, int splitk,
                      const DecEpi& e, cudaStream_t st) {
  using C = Cfg<BN, 108>;
  auto kern = gemm_decode_kernel<BN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           C::SMEM_BYTES);
    if (err != cudaSuccess) {
      set_last_error("gemm_decode: smem attr", err);
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
  if (pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t err = cudaLaunchKernelEx(&cfg, kern, tmW, tmX, tmNext, out, N, M, K, ldo, splitk, e, next, status_word());
  if (err != cudaSuccess) {
    set_last_error("gemm_decode: launch", err);
    return GV_ECUDA;
  }
  return GV_OK;
}

// The weight of the GEMM that follows in the stream (set by gv_gemm_decode_next for the next
// launch of the calling host thread, consumed by it): its first tiles are prefetched into L2 by
// that launch's producers once their own streaming is done.
struct NextHint {
  const void* w;
  long long N, K, ldw;
};
static thread_local NextHint t_next = {nullptr, 0, 0, 0};

// Consumes the hint: fills `tm` / `nx` for a launch with a `bn`-token tile (nx->stages stays 0
// when there is no hint). Also used by the fused GEMM + all-reduce launcher.
void take_next_weights(int bn, CUtensorMap* tm, NextWeights* nx) {
  const NextHint hint = t_next;
  t_next.w = nullptr;                      // a hint serves exactly one launch attempt
  if (bn <= 0 || hint.w == nullptr || cached_tmap_bf16(tm, hint.w, hint.N, hint.K, hint.ldw, BM) != GV_OK) return;
  nx->tiles = ceil_div(hint.N, BM);
  nx->splitk = decode_splitk(hint.N, hint.K, bn, 0);
  nx->kb_total = ceil_div(hint.K, BK);
  nx->kb_per = (nx->kb_total + nx->splitk - 1) / nx->splitk;
  // about what HBM delivers during an epilogue (2.5 us x 6.5 TB/s = 16 MB), 16 KB per box
  const long long items = (long long)nx->tiles * nx->splitk;
  const long long stages = (16ll << 20) / (items * BM * BK * 2);
  nx->stages = (int)(stages < 1 ? 1 : stages > 8 ? 8 : stages);
}

static int run_decode_gemm(const void* x, const void* w, void* out, long long M, long long N, long long K,
                           long long ldx, long long ldw, long long ldo, long long force_splitk,
                           const DecEpi& e, void* stream) {
  const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  CUtensorMap tmNext;
  NextWeights next = {nullptr, 0, 0, 0, 0, 0};
  take_next_weights((w && M > 0 && M <= 128) ? bn : 0, &tmNext, &next);   // consumed even if the launch is refused
  if (!x || !w || !out || M <= 0 || N <= 0 || K <= 0) return GV_EINVAL;
  if ((K & 7) || (ldx & 7) || (ldw & 7) || (N & 3) || (ldo & 3)) return GV_EINVAL;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return GV_EINVAL;
  if (reinterpret_cast<uintptr_t>(out) & 7) return GV_EINVAL;
  if (M > 128) return GV_EUNSUPPORTED;
  if (e.ss_in != nullptr && (e.ss_tiles <= 0 || e.ss_ld < e.ss_tiles)) return GV_EINVAL;
  CUtensorMap tmW, tmX;
  int rc;
  if ((rc = cached_tmap_bf16(&tmW, w, N, K, ldw, BM)) != GV_OK) return rc;
  if ((rc = cached_tmap_bf16(&tmX, x, M, K, ldx, bn)) != GV_OK) return rc;
  const int sk = decode_splitk(N, K, bn, force_splitk);
  cudaStream_t st = (cudaStream_t)stream;
  if (next.stages == 0) tmNext = tmW;      // unused, but a valid map
#define GV_DEC_LAUNCH(BN_)                                                                              \
  switch (e.mode) {                                                                                    \
    case EPI_PLAIN: return launch_dec<BN_, EPI_PLAIN>(tmW, tmX, tmNext, next, (bf16*)out, (int)N, (int)M, (int)K, ldo, sk, e, st);   \
    case EPI_SWIGLU: return launch_dec<BN_, EPI_SWIGLU>(tmW, tmX, tmNext, next, (bf16*)out, (int)N, (int)M, (int)K, ldo, sk, e, st); \
    case EPI_RESID: return launch_dec<BN_, EPI_RESID>(tmW, tmX, tmNext, next, (bf16*)out, (int)N, (int)M, (int)K, ldo, sk, e, st);   \
    default: return launch_dec<BN_, EPI_ROPE>(tmW, tmX, tmNext, next, (bf16*)out, (int)N, (int)M, (int)K, ldo, sk, e, st);           \
  }
  switch (bn) {
    case 16: GV_DEC_LAUNCH(16)
    case 32: GV_DEC_LAUNCH(32)
    case 64: GV_DEC_LAUNCH(64)
    default: GV_DEC_LAUNCH(128)
  }
#undef GV_DEC_LAUNCH
}

}  // namespace gemm
}  // namespace gv

using namespace gv;
using namespace gv::gemm;

static void set_scale(DecEpi& e, const void* ss_in, long long ss_tiles, long long ss_ld, long long h,
                      float eps) {
  e.ss_in = (const float*)ss_in;
  e.ss_tiles = (int)ss_tiles;
  e.ss_ld = (int)ss_ld;
  e.inv_h = h > 0 ? 1.f / (float)h : 0.f;
  e.eps = eps;
}

// Names the weight [N, K] (row pitch ldw elements) of the GEMM that will follow the next
// gv_gemm_decode* launch of this host thread; that launch prefetches its first tiles into L2.
extern "C" int gv_gemm_decode_next(const void* w, long long N, long long K, long long ldw) {
  if (w && ((K & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(w) & 15))) return GV_EINVAL;
  t_next.w = w;
  t_next.N = N;
  t_next.K = K;
  t_next.ldw = ldw;
  return GV_OK;
}

// out[M, N] = s_t * (x . w^T) (+ bias), or with `swiglu` out[M, N / 2] = silu(gate) * up over
// [64 gate | 64 up] row blocks. ss_in [M][ss_ld] fp32: the first ss_tiles entries of row t are
// partial sums of squares of x[t] over `norm_h` features in total (null: s_t = 1).
extern "C" int gv_gemm_decode(const void* x, const void* w, const void* bias, void* out, long long M,
                              long long N, long long K, long long ldx, long long ldw, long long ldo,
                              const void* ss_in, long long ss_tiles, long long ss_ld,
                              long long norm_h, float eps, long long swiglu, long long force_splitk,
                              void* stream) {
  DecEpi e = {};
  e.mode = swiglu ? EPI_SWIGLU : EPI_PLAIN;
  if (swiglu && ((N % 128) || bias)) return GV_EINVAL;
  e.bias = (const bf16*)bias;
  set_scale(e, ss_in, ss_tiles, ss_ld, norm_h, eps);
  return run_decode_gemm(x, w, out, M, N, K, ldx, ldw, ldo, force_splitk, e, stream);
}

// x_out[M, N] = residual + x . w^T (+ bias) (x_out may be `residual` itself) and
// ss_out[token][tile] = sum of squares of the 128 new values of tile `tile` (N % 128 == 0,
// ss_ld >= N / 128).
extern "C" int gv_gemm_decode_residual(const void* x, const void* w, const void* bias,
                                       const void* residual, void* x_out, void* ss_out, long long M,
                                       long long N, long long K, long long ldx, long long ldw,
                                       long long ldo, long long ss_ld, long long force_splitk,
                                       void* stream) {
  if (!residual || (reinterpret_cast<uintptr_t>(residual) & 7)) return GV_EINVAL;
  if (ss_out && ((N % 128) || ss_ld < N / 128)) return GV_EINVAL;
  DecEpi e = {};
  e.mode = EPI_RESID;
  e.bias = (const bf16*)bias;
  e.residual = (const bf16*)residual;
  e.ss_out = (float*)ss_out;
  e.ss_ld = (int)ss_ld;
  return run_decode_gemm(x, w, x_out, M, N, K, ldx, ldw, ldo, force_splitk, e, stream);
}

// Fused QKV projection for 128-wide heads: w [(nq + 2 nkv) * 128, K]; q_out [M, nq * 128] gets
// the rotated, scaled queries; keys (rotated) and values go to slot `slots[t]` of the paged caches
// [num_slots, nkv, 128]. Same arithmetic as gv_gemm_bf16 followed by gv_rope_kvwrite.
extern "C" int gv_gemm_decode_rope(const void* x, const void* w, const void* bias, void* q_out,
                                   void* k_cache, void* v_cache, const void* cos_sin,
                                   const void* positions, const void* slots, const void* q_norm_w,
                                   const void* k_norm_w, long long M, long long K, long long ldx,
                                   long long ldw, long long nq, long long nkv, float q_scale,
                                   float qk_eps, long long max_pos, long long num_slots,
                                   const void* ss_in, long long ss_tiles, long long ss_ld,
                                   long long norm_h, float eps, long long force_splitk,
                                   void* stream) {
  if (!q_out || !k_cache || !v_cache || !cos_sin || !positions || !slots) return GV_EINVAL;
  if (nq <= 0 || nkv <= 0) return GV_EINVAL;
  if ((reinterpret_cast<uintptr_t>(cos_sin) & 15) ||
      ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 7))
    return GV_EINVAL;
  DecEpi e = {};
  e.mode = EPI_ROPE;
  e.bias = (const bf16*)bias;
  e.cos_sin = (const float*)cos_sin;
  e.positions = (const long long*)positions;
  e.slots = (const int*)slots;
  e.k_cache = (bf16*)k_cache;
  e.v_cache = (bf16*)v_cache;
  e.q_norm_w = (const bf16*)q_norm_w;
  e.k_norm_w = (const bf16*)k_norm_w;
  e.nq = (int)nq;
  e.nkv = (int)nkv;
  e.max_pos = (int)max_pos;
  e.num_slots = num_slots;
  e.q_scale = q_scale;
  e.qk_eps = qk_eps;
  set_scale(e, ss_in, ss_tiles, ss_ld, norm_h, eps);
  const long long N = (nq + 2 * nkv) * 128;
  return run_decode_gemm(x, w, q_out, M, N, K, ldx, ldw, nq * 128, force_splitk, e, stream);
}

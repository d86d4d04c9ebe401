// Paged causal flash attention for prefill on the 5th-generation tensor cores (head_dim 128).
//
// Same contract as `paged_prefill_kernel` (attention_prefill.cu; the reference's
// `flash_attention_<T>` prefill path, xlite/csrc/kernels/flash_attention.h:371-395,687, mask rule
// xlite/tests/kernels/attention.py:110-117): query row i of a request with `cached` tokens in the
// cache sees keys <= cached + i; K and V come from the paged cache, which already holds this
// step's tokens. What differs is the machine model:
//
//   * one CTA = 128 query tokens of one (request, q head); the rows ride the 128 TMEM lanes;
//   * Q, K and V tiles (128 x 128 bf16) arrive by TMA through tensor maps over the query matrix
//     and the paged caches: a 128-key tile is `128 / block_size` boxes addressed through the
//     block table, 128-byte swizzled, no register staging;
//   * S = Q K^T and O += P V are tcgen05.mma with fp32 accumulators in tensor memory (S double
//     buffered, then O: 128 columns). The V tile is consumed where TMA put it, as an MN-major B
//     operand, so no transposed copy of V exists anywhere;
//   * warp roles: warp 0 issues TMA, warp 1 issues every MMA, the other warps run the softmax,
//     one thread per query row (its TMEM lane): row maxima and sums need no shuffles. The MMA warp
//     issues Q K^T of tile t + 1 before it waits for P of tile t, so the tensor core works
//     while the softmax warps exponentiate;
//   * a score costs four instructions: the row maximum is taken on the raw accumulator and scaled
//     once, the softmax scale rides in the multiply-add that forms the exponent, and 2^x is the
//     special-function instruction itself (`ex2.approx`);
//   * two shapes (`Shape<BN>` below): 128-key tiles with one CTA per SM, or 64-key tiles with two
//     CTAs per SM, where one CTA's MMAs and fixed parts overlap the other's softmax. (Giving a CTA
//     two query tiles, the heaviest with the lightest, was measured too: it helps the one-CTA
//     shape by 7 % and costs the two-CTA shape 7 % at 1024 tokens, so a CTA keeps one tile);
//   * lazy rescaling: the running maximum only moves when a tile exceeds it by more than 2^8,
//     so O is read back and scaled (tcgen05.ld / tcgen05.st) for a handful of tiles only.
//
// q is pre-scaled by the RoPE kernel; `scale` is an extra factor. Every mbarrier wait is bounded
// (status word on time-out); TMEM is always released.
#include "sm100.cuh"
#include "gvirt_kernels.h"

namespace gv {

namespace gemm {
int cached_tmap_bf16(CUtensorMap* out, const void* base, long long rows, long long cols,
                     long long row_stride_elems, int box_rows);
}

namespace fa {

constexpr int HD = 128;
constexpr int BM = 128;             // query rows per CTA
constexpr int Q_BYTES = 128 * 128 * 2;      // the Q tile: 128 rows x 128 features = two 64-column chunks
constexpr int CHUNK128 = 128 * 128;         // 128 rows x 128 bytes: one chunk of Q and of P
constexpr int KV_STAGES = 2;
constexpr float RESCALE_LOG2 = 8.f; // move the running maximum only past this gap (log2 units)

struct Bars {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, pv_done;
  uint32_t tmem_slot;
};

// Two shapes of the kernel. BN = keys per tile:
//   BN = 128: one CTA per SM (Q 32 KB + 2 x (K + V) 128 KB + P 32 KB), S0 | S1 | O = 384 TMEM columns
//             (512 allocated), one or two softmax warp groups.
//   BN = 64:  two CTAs per SM (Q 32 KB + 2 x (K + V) 64 KB + P 16 KB = 112 KB each), S0 | S1 | O = 256
//             columns each. While one CTA's softmax warps exponentiate, the other CTA's MMAs run, and a
//             CTA's fixed part (set-up, first tile, epilogue) hides behind its neighbour's tiles.
template <int BN>
struct Shape {
  static constexpr int KV_BYTES = BN * 128 * 2;       // one K or V tile: BN keys x 128 features
  static constexpr int KV_CHUNK = BN * 128;           // BN key rows x 128 bytes (64 features)
  static constexpr int P_BYTES = BM * BN * 2;         // BN / 64 chunks of 128 rows x 128 bytes
  static constexpr int TMEM_COLS = BN == 128 ? 512 : 256;   // S0 [0, BN) S1 [BN, 2 BN) O [2 BN, 2 BN + 128)
  static constexpr int XCH_BYTES = BN == 128 ? 3 * 256 * 4 : 0;   // two-warp-group exchange (BN = 128 only)
  static constexpr int SMEM_BYTES = Q_BYTES + 2 * KV_STAGES * KV_BYTES + P_BYTES + 256 + XCH_BYTES
                                    + (BN == 128 ? 1024 : 0);     // BN = 64 relies on the declared alignment
};
static_assert(sizeof(Bars) <= 256, "barrier block");

template <int WG, int BN>
__global__ void __launch_bounds__(64 + 128 * WG, BN == 128 ? 1 : 2)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const int* __restrict__ block_tables,
                  const int* __restrict__ q_start, const int* __restrict__ cached_lens,
                  bf16* __restrict__ out, int nq, int nkv, int block_size, int max_blocks,
                  float scale_log2, long long num_blocks, unsigned int* status) {
  using SH = Shape<BN>;
  constexpr int KV_BYTES = SH::KV_BYTES, KV_CHUNK = SH::KV_CHUNK, TMEM_COLS = SH::TMEM_COLS;
  static_assert(WG == 1 || BN == 128, "two softmax warp groups only with 128-key tiles");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (BN != 128 && base != smem_raw) {
    // the 64-key shape has no room for alignment slack: refuse to run misaligned (never observed:
    // the dynamic window starts on a 1 KB boundary when the kernel has no static shared memory)
    if (threadIdx.x == 0) atomicOr(status, GV_ST_BAD_INDEX);
    return;
  }
  uint8_t* q_s = base;
  uint8_t* k_s = q_s + Q_BYTES;                          // [KV_STAGES]
  uint8_t* v_s = k_s + KV_STAGES * KV_BYTES;             // [KV_STAGES]
  uint8_t* p_s = v_s + KV_STAGES * KV_BYTES;
  Bars* bars = reinterpret_cast<Bars*>(p_s + SH::P_BYTES);
  float* xch_base = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int qtile = gridDim.x - 1 - blockIdx.x;          // heaviest (latest) tiles first
  const int qs0 = q_start[b], qlen = q_start[b + 1] - qs0;
  if (qtile * BM >= qlen) return;                        // uniform per CTA, before any set-up
  const int cached = cached_lens[b];
  const int kvh = h / (nq / nkv);
  const int q_lo = qtile * BM;
  const int q_hi = min(qlen, q_lo + BM);
  const int kv_end = cached + q_hi;                      // exclusive
  const int ntiles = (kv_end + BN - 1) / BN;
  const int* bt = block_tables + (long long)b * max_blocks;

  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(&tmQ);
    sm100::tma_prefetch_desc(&tmK);
    sm100::tma_prefetch_desc(&tmV);
    sm100::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      sm100::mbar_init(&bars->k_full[s], 1);
      sm100::mbar_init(&bars->k_empty[s], 1);
      sm100::mbar_init(&bars->v_full[s], 1);
      sm100::mbar_init(&bars->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      sm100::mbar_init(&bars->s_full[s], 1);
      sm100::mbar_init(&bars->s_empty[s], 128 * WG);
    }
    sm100::mbar_init(&bars->p_full, 128 * WG);
    sm100::mbar_init(&bars->pv_done, 1);
    sm100::mbar_fence_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc(&bars->tmem_slot, TMEM_COLS);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_slot);
  const uint32_t tmem_o = tmem + 2 * BN;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (sm100::elect_one()) {
      sm100::mbar_expect_tx(&bars->q_full, Q_BYTES);
      for (int c = 0; c < 2; ++c)
        sm100::tma_load_2d(q_s + c * CHUNK128, &tmQ, &bars->q_full, h * HD + c * 64, qs0 + q_lo);
      const int rows_per_box = block_size < BN ? block_size : BN;
      const int boxes = BN / rows_per_box;
      for (int t = 0; t < ntiles; ++t) {
        const int s = t % KV_STAGES;
        const uint32_t ph = (uint32_t)(t / KV_STAGES) & 1u;
        bool ok = true;
        for (int kv = 0; kv < 2 && ok; ++kv) {
          uint64_t* full = kv == 0 ? &bars->k_full[s] : &bars->v_full[s];
          uint64_t* empty = kv == 0 ? &bars->k_empty[s] : &bars->v_empty[s];
          uint8_t* dst = (kv == 0 ? k_s : v_s) + s * KV_BYTES;
          const CUtensorMap* tm = kv == 0 ? &tmK : &tmV;
          if (!sm100::mbar_wait(empty, ph ^ 1u)) {
            atomicOr(status, GV_ST_TIMEOUT_TMA);
            ok = false;
            break;
          }
          sm100::mbar_expect_tx(full, KV_BYTES);
          for (int bx = 0; bx < boxes; ++bx) {
            const int pos = t * BN + bx * rows_per_box;
            // keys past the end of the sequence are masked by the softmax; a block-table entry
            // that is out of range is replaced by block 0 and flagged
            const int bi = pos / block_size;
            int blk = bi < max_blocks ? bt[bi] : -1;
            if (blk < 0 || blk >= num_blocks) {
              if (pos < kv_end) atomicOr(status, GV_ST_BAD_INDEX);
              blk = 0;
            }
            const int row = blk * block_size + pos % block_size;
            for (int c = 0; c < 2; ++c)
              sm100::tma_load_2d(dst + c * KV_CHUNK + bx * rows_per_box * 128, tm, full,
                                 kvh * HD + c * 64, row);
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (sm100::elect_one()) {
      constexpr uint32_t idesc_qk = sm100::make_idesc(BM, BN, 1, 1);
      constexpr uint32_t idesc_pv = sm100::make_idesc(BM, HD, 1, 1) | sm100::IDESC_B_MN_MAJOR;
      bool ok = sm100::mbar_wait(&bars->q_full, 0);
      if (!ok) atomicOr(status, GV_ST_TIMEOUT_MMA);
      auto issue_qk = [&](int t) -> bool {
        const int s = t % KV_STAGES;
        const uint32_t ph = (uint32_t)(t / KV_STAGES) & 1u;
        const int sb = t & 1;
        const uint32_t sph = (uint32_t)(t >> 1) & 1u;
        if (!sm100::mbar_wait(&bars->k_full[s], ph) || !sm100::mbar_wait(&bars->s_empty[sb], sph ^ 1u)) {
          atomicOr(status, GV_ST_TIMEOUT_MMA);
          return false;
        }
        sm100::tc_fence_after();
        const uint32_t qa = sm100::smem_u32(q_s), ka = sm100::smem_u32(k_s + s * KV_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          sm100::mma_f16_ss(tmem + sb * BN,
                            sm100::smem_desc_sw128(qa + (uint32_t)(k >> 2) * CHUNK128) + (uint64_t)(2 * (k & 3)),
                            sm100::smem_desc_sw128(ka + (uint32_t)(k >> 2) * KV_CHUNK) + (uint64_t)(2 * (k & 3)), idesc_qk,
                            (uint32_t)(k != 0));
        }
        sm100::tc_commit(&bars->k_empty[s]);
        sm100::tc_commit(&bars->s_full[sb]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int t = 0; t < ntiles && ok; ++t) {
        if (t + 1 < ntiles) ok = issue_qk(t + 1);
        if (!ok) break;
        const int s = t % KV_STAGES;
        const uint32_t ph = (uint32_t)(t / KV_STAGES) & 1u;
        if (!sm100::mbar_wait(&bars->p_full, (uint32_t)t & 1u) || !sm100::mbar_wait(&bars->v_full[s], ph)) {
          atomicOr(status, GV_ST_TIMEOUT_MMA);
          ok = false;
          break;
        }
        sm100::tc_fence_after();
        const uint32_t pa = sm100::smem_u32(p_s), va = sm100::smem_u32(v_s + s * KV_BYTES);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          // A = P [128 rows x 16 keys] K-major; B = V [16 keys x 128 features] as it lies in the
          // tile: key rows of 128 bytes, the second 64 features one chunk further
          const uint64_t da = sm100::smem_desc_sw128(pa + (uint32_t)(k >> 2) * CHUNK128) + (uint64_t)(2 * (k & 3));
          const uint64_t db = sm100::smem_desc_mn_sw128(va + (uint32_t)k * 2048u, KV_CHUNK, 1024);
          sm100::mma_f16_ss(tmem_o, da, db, idesc_pv, (uint32_t)((t | k) != 0));
        }
        sm100::tc_commit(&bars->v_empty[s]);
        sm100::tc_commit(&bars->pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    // WG warp groups of 4 warps: with WG == 2 the warps w and w + 4 share the 32 query rows of
    // their TMEM quadrant and each takes one 64-key half of every score row, which doubles the
    // warps per scheduler (exponentials and conversions of one hide the latencies of the other).
    constexpr int COLS = BN / WG;                      // score columns per thread
    const int quad = warp & 3;
    const int half = WG == 2 ? (warp - 2) >> 2 : 0;    // which half of the columns
    const int r = quad * 32 + lane;                    // query row = TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int qi = q_lo + r;                           // token index inside the request
    const int limit = min(cached + qi, kv_end - 1);    // last visible key of this row
    float* xch = xch_base;                             // [2][128] row maxima / sums of the two halves
    auto pair_bar = [&]() {                            // the two warps that share this row range
      if (WG == 2) asm volatile("bar.sync %0, 64;" ::"r"(2 + quad) : "memory");
    };
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    // A wait that runs out only clears `ok`: the thread keeps walking the loop (without further
    // waits), so that every named barrier and every warp-collective TMEM access below still sees
    // all of its participants and the kernel ends.
    for (int t = 0; t < ntiles; ++t) {
      const int sb = t & 1;
      const uint32_t sph = (uint32_t)(t >> 1) & 1u;
      if (ok && !sm100::mbar_wait(&bars->s_full[sb], sph)) ok = false;
      sm100::tc_fence_after();
      float sv[COLS];
#pragma unroll
      for (int c = 0; c < COLS; c += 32)
        sm100::tmem_ld32(tmem + lane_addr + sb * BN + half * COLS + c, reinterpret_cast<uint32_t*>(sv + c));
      sm100::tmem_ld_wait();
      sm100::tc_fence_before();
      sm100::mbar_arrive(&bars->s_empty[sb]);
      const int k0 = t * BN + half * COLS;
      // sv stays unscaled: the scale (> 0) is applied to the row maximum once and to every score
      // inside the exponent's multiply-add, so a score costs max + fma + ex2 + add
      float mx = -INFINITY;
      if (t * BN + BN - 1 <= cached + q_lo && t * BN + BN <= kv_end) {
#pragma unroll
        for (int j = 0; j < COLS; ++j) mx = fmaxf(mx, sv[j]);
      } else {
#pragma unroll
        for (int j = 0; j < COLS; ++j) {
          sv[j] = (k0 + j <= limit) ? sv[j] : -INFINITY;
          mx = fmaxf(mx, sv[j]);
        }
      }
      mx *= scale_log2;
      if (WG == 2) {                                   // row maximum over both halves
        xch[(t & 1) * 256 + half * 128 + r] = mx;
        pair_bar();
        mx = fmaxf(mx, xch[(t & 1) * 256 + (half ^ 1) * 128 + r]);
      }
      // lazy rescaling: keep the old reference maximum unless this tile exceeds it by 2^8
      const bool grow = mx > m + RESCALE_LOG2;           // also true for the first finite tile
      const bool any_grow = __any_sync(0xffffffffu, grow);
      bool waited = false;
      if (any_grow) {
        const float m_new = grow ? mx : m;
        const float f = (m == -INFINITY) ? 0.f : sm100::ex2_approx(m - m_new);
        if (t > 0) {
          if (ok && !sm100::mbar_wait(&bars->pv_done, (uint32_t)(t - 1) & 1u)) ok = false;
          waited = true;
          sm100::tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < HD / WG; c += 16) {
            uint32_t o[16];
            sm100::tmem_ld16(tmem_o + lane_addr + half * (HD / WG) + c, o);
            sm100::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
            sm100::tmem_st16(tmem_o + lane_addr + half * (HD / WG) + c, o);
          }
          sm100::tmem_st_wait();
          l *= f;
        }
        m = m_new;
      }
      const float nmref = (m == -INFINITY) ? 0.f : -m;
      float rs = 0.f;
      uint32_t pk[COLS / 2];
#pragma unroll
      for (int j = 0; j < COLS; j += 2) {
        const float p0 = sm100::ex2_approx(fmaf(sv[j], scale_log2, nmref));
        const float p1 = sm100::ex2_approx(fmaf(sv[j + 1], scale_log2, nmref));
        rs += p0 + p1;
        pk[j >> 1] = pack_bf2(p0, p1);
      }
      l += rs;                                         // with WG == 2: this half's share of the row sum
      if (t > 0 && !waited && ok && !sm100::mbar_wait(&bars->pv_done, (uint32_t)(t - 1) & 1u)) ok = false;
      // P row r: 64-key chunks, 16-byte pieces XOR-swizzled by (r & 7) like a TMA tile
#pragma unroll
      for (int c = 0; c < COLS / 64; ++c) {
        uint8_t* row = p_s + (half * (COLS / 64) + c) * CHUNK128 + r * 128;
#pragma unroll
        for (int piece = 0; piece < 8; ++piece) {
          const int i = c * 32 + piece * 4;
          *reinterpret_cast<uint4*>(row + ((piece ^ (r & 7)) << 4)) = make_uint4(pk[i], pk[i + 1], pk[i + 2], pk[i + 3]);
        }
      }
      sm100::fence_proxy_async_smem();
      sm100::tc_fence_before();
      sm100::mbar_arrive(&bars->p_full);
    }
    // ---- epilogue: O / l -> bf16
    if (ok && !sm100::mbar_wait(&bars->pv_done, (uint32_t)(ntiles - 1) & 1u)) ok = false;
    if (!ok && lane == 0) atomicOr(status, GV_ST_TIMEOUT_EPI);
    sm100::tc_fence_after();
    if (WG == 2) {                                     // row sum over both halves
      xch[512 + half * 128 + r] = l;
      pair_bar();
      l += xch[512 + (half ^ 1) * 128 + r];
    }
    if (__all_sync(0xffffffffu, ok)) {
      // rows past the end of the request take part in the (warp-collective) TMEM loads too
      const bool live = qi < qlen;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* orow = out + ((long long)(qs0 + (live ? qi : 0)) * nq + h) * HD + half * (HD / WG);
#pragma unroll 1
      for (int c = 0; c < HD / WG; c += 16) {
        uint32_t o[16];
        sm100::tmem_ld16(tmem_o + lane_addr + half * (HD / WG) + c, o);
        sm100::tmem_ld_wait();
        float f[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(o[j]) * inv;
        if (live) {
          st8(orow + c, pack8(f));
          st8(orow + c + 8, pack8(f + 8));
        }
      }
    }
  }
  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace fa
}  // namespace gv

using namespace gv;

// Shape of the tcgen05 prefill attention kernel: 1 = 128-key tiles, one softmax warp group (one
// thread per query row); 2 = 128-key tiles, two warp groups (two threads per row, one 64-key half
// each); 4 = 64-key tiles, two CTAs per SM.
static long long g_prefill_tc_wg = 4;
extern "C" void gv_set_prefill_tc_warpgroups(long long wg) {
  g_prefill_tc_wg = (wg == 1 || wg == 2 || wg == 4) ? wg : 4;
}

// Same arguments as gv_paged_attention_prefill plus `total_tokens` (rows of q / out). head_dim
// must be 128 and block_size a power of two in [8, ...] that divides or is a multiple of 128;
// other shapes return GV_EUNSUPPORTED (the caller takes the mma.sync kernel).
extern "C" int gv_paged_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache,
                                             const void* block_tables, const void* q_start,
                                             const void* cached_lens, void* out,
                                             long long total_tokens, long long batch,
                                             long long max_q_len, long long nq, long long nkv,
                                             long long head_dim, long long block_size,
                                             long long max_blocks, float scale,
                                             long long num_blocks, void* stream) {
  if (!q || !k_cache || !v_cache || !block_tables || !q_start || !cached_lens || !out)
    return GV_EINVAL;
  if (batch == 0 || max_q_len == 0 || total_tokens == 0) return GV_OK;
  if (nkv <= 0 || nq % nkv != 0) return GV_EINVAL;
  if (head_dim != 128) return GV_EUNSUPPORTED;
  if (!(scale > 0.f)) return GV_EINVAL;              // the kernel scales the row maximum, not every score
  if (block_size < 8 || (block_size & (block_size - 1)) != 0) return GV_EUNSUPPORTED;
  if (batch > 65535 || nq > 65535) return GV_ETOOBIG;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) |
       reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(out)) & 15)
    return GV_EINVAL;
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  const long long kv_rows = num_blocks * block_size;
  const int bn = g_prefill_tc_wg == 4 ? 64 : 128;
  const int box = block_size < bn ? (int)block_size : bn;
  if ((rc = gemm::cached_tmap_bf16(&tmQ, q, total_tokens, nq * 128, nq * 128, 128)) != GV_OK) return rc;
  if ((rc = gemm::cached_tmap_bf16(&tmK, k_cache, kv_rows, nkv * 128, nkv * 128, box)) != GV_OK) return rc;
  if ((rc = gemm::cached_tmap_bf16(&tmV, v_cache, kv_rows, nkv * 128, nkv * 128, box)) != GV_OK) return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fa::prefill_tc_kernel<1, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         fa::Shape<128>::SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(fa::prefill_tc_kernel<2, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               fa::Shape<128>::SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(fa::prefill_tc_kernel<1, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               fa::Shape<64>::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_last_error("prefill_tc: smem attr", e);
      return GV_ECUDA;
    }
    configured = true;
  }
  dim3 grid((unsigned)((max_q_len + fa::BM - 1) / fa::BM), (unsigned)nq, (unsigned)batch);
  const float sl2 = scale * 1.4426950408889634f;
  cudaStream_t st = (cudaStream_t)stream;
#define GV_PF_ARGS tmQ, tmK, tmV, (const int*)block_tables, (const int*)q_start, (const int*)cached_lens, \
                   (bf16*)out, (int)nq, (int)nkv, (int)block_size, (int)max_blocks, sl2, num_blocks, status_word()
  if (g_prefill_tc_wg == 4)
    fa::prefill_tc_kernel<1, 64><<<grid, 64 + 128, fa::Shape<64>::SMEM_BYTES, st>>>(GV_PF_ARGS);
  else if (g_prefill_tc_wg == 2)
    fa::prefill_tc_kernel<2, 128><<<grid, 64 + 256, fa::Shape<128>::SMEM_BYTES, st>>>(GV_PF_ARGS);
  else
    fa::prefill_tc_kernel<1, 128><<<grid, 64 + 128, fa::Shape<128>::SMEM_BYTES, st>>>(GV_PF_ARGS);
#undef GV_PF_ARGS
  return check_launch("paged_prefill_tc");
}

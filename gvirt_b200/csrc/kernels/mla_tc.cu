// Absorbed multi-head latent attention for decode on the 5th-generation tensor cores.
//
// Same contract as the decode case of `mla_attention_kernel` (mla.cu; the reference's
// `mla_v2_bfloat16_t` / `flash_mla_v2_bfloat16_t`, xlite/csrc/kernels/mla_v2.h:479-540,762 and
// flash_mla_v2.h:196-222,914: all local heads packed into the M dimension of the cube GEMMs,
// S = (q_abs . Kc^T + q_pe . Kpe^T) * scale, o_abs = softmax(S) . Kc, split-KV partials merged
// afterwards): query row [q_abs (512) | q_pe (64)], cache row [kv_c (512) | k_pe (64)], so the
// score is one 576-deep dot product and the value is the first 512 columns of the key row.
//
// Mapping to sm_100a:
//   * one CTA = the 128 heads of one request x one KV split x one half of the 512 output
//     columns. The heads ride the 128 TMEM lanes. 512 fp32 output columns plus the scores do not
//     fit into the 512 TMEM columns of an SM, so two CTAs each keep 256 output columns and both
//     compute the (cheap, 576-deep) scores;
//   * the query block (128 x 576 bf16 = 147 KB) is loaded once by TMA and stays in shared
//     memory; latent tiles of 32 keys (36 KB) stream through a two-slot ring, gathered through
//     the block table with one TMA box per 64-column chunk;
//   * the latent tile is the B operand of both GEMMs where TMA put it: K-major for Q K^T
//     (9 chunks x 4 k-steps of tcgen05.mma, N = 32) and MN-major for P V (2 k-steps, N = 256):
//     the tile crosses the memory system once;
//   * softmax: one thread per head (TMEM lane), scores double-buffered in TMEM so that Q K^T of
//     tile t + 1 runs while tile t is exponentiated; P goes back through shared memory as a
//     K-major operand (64-byte rows, 64-byte swizzle); the running maximum moves lazily.
//
// Partials (nsplit > 1) use the layout of mla.cu: normalised fp32 outputs + log2-domain
// log-sum-exp per (token, head, split); `mla_tc_merge_kernel` combines them. Every wait is bounded.
#include "sm100.cuh"
#include "gvirt_kernels.h"

namespace gv {

namespace gemm {
int cached_tmap_bf16(CUtensorMap* out, const void* base, long long rows, long long cols,
                     long long row_stride_elems, int box_rows);
}

namespace mlatc {

constexpr int DC = 512, DR = 64, DQ = DC + DR;
constexpr int NCHUNK = DQ / 64;                 // 9 chunks of 64 columns
constexpr int HEADS = 128;
constexpr int BN = 32;                          // keys per tile
constexpr int Q_CHUNK = HEADS * 128;            // 16 KB
constexpr int K_CHUNK = BN * 128;               // 4 KB
constexpr int Q_BYTES = NCHUNK * Q_CHUNK;       // 147456
constexpr int K_BYTES = NCHUNK * K_CHUNK;       // 36864
constexpr int P_BYTES = HEADS * BN * 2;         // 8192
constexpr int KV_STAGES = 2;
constexpr int THREADS = 192;
constexpr int OCOLS = DC / 2;                   // output columns per CTA
constexpr int TMEM_COLS = 512;                  // S0 [0,32) S1 [32,64) O [64,320)
constexpr float RESCALE_LOG2 = 8.f;

struct Bars {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, pv_done;
  uint32_t tmem_slot;
};

constexpr int SMEM_BYTES = Q_BYTES + KV_STAGES * K_BYTES + P_BYTES + 1024 + sizeof(Bars);

__global__ void __launch_bounds__(THREADS, 1)
mla_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const int* __restrict__ block_tables, const int* __restrict__ seq_lens,
              bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_lse,
              int heads, int block_size, int max_blocks, int nsplit, float scale_log2,
              long long num_blocks, unsigned int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = base;
  uint8_t* k_s = q_s + Q_BYTES;
  uint8_t* p_s = k_s + KV_STAGES * K_BYTES;
  Bars* bars = reinterpret_cast<Bars*>(p_s + P_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = blockIdx.x, split = blockIdx.y;
  const int groups = heads / HEADS;
  const int b = blockIdx.z / groups, g = blockIdx.z % groups;
  const int kv_len = seq_lens[b];                 // keys of this request, the new token included (0: padding row)
  int chunk = (kv_len + nsplit - 1) / nsplit;
  chunk = (chunk + BN - 1) / BN * BN;
  const int start = split * chunk;
  const int end = min(kv_len, start + chunk);
  const int ntiles = end > start ? (end - start + BN - 1) / BN : 0;
  const long long head0 = (long long)b * heads + (long long)g * HEADS;
  const int* bt = block_tables + (long long)b * max_blocks;

  if (ntiles == 0) {
    // an empty split (or a padding request): neutral partial, nothing else to do
    if (nsplit > 1) {
      for (int i = threadIdx.x; i < HEADS * OCOLS; i += THREADS) {
        const int r = i / OCOLS, c = i % OCOLS;
        part_o[((head0 + r) * nsplit + split) * DC + half * OCOLS + c] = 0.f;
      }
      if (half == 0)
        for (int r = threadIdx.x; r < HEADS; r += THREADS) part_lse[(head0 + r) * nsplit + split] = -INFINITY;
    } else {
      for (int i = threadIdx.x; i < HEADS * OCOLS; i += THREADS) {
        const int r = i / OCOLS, c = i % OCOLS;
        out[(head0 + r) * DC + half * OCOLS + c] = f2bf(0.f);
      }
    }
    return;
  }

  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(&tmQ);
    sm100::tma_prefetch_desc(&tmK);
    sm100::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      sm100::mbar_init(&bars->k_full[s], 1);
      sm100::mbar_init(&bars->k_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      sm100::mbar_init(&bars->s_full[s], 1);
      sm100::mbar_init(&bars->s_empty[s], 128);
    }
    sm100::mbar_init(&bars->p_full, 128);
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
  const uint32_t tmem_o = tmem + 64;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (sm100::elect_one()) {
      sm100::mbar_expect_tx(&bars->q_full, Q_BYTES);
      for (int c = 0; c < NCHUNK; ++c)
        sm100::tma_load_2d(q_s + c * Q_CHUNK, &tmQ, &bars->q_full, c * 64, (int)head0);
      for (int t = 0; t < ntiles; ++t) {
        const int s = t % KV_STAGES;
        const uint32_t ph = (uint32_t)(t / KV_STAGES) & 1u;
        if (!sm100::mbar_wait(&bars->k_empty[s], ph ^ 1u)) {
          atomicOr(status, GV_ST_TIMEOUT_TMA);
          break;
        }
        const int pos = start + t * BN;
        const int bi = pos / block_size;
        int blk = bi < max_blocks ? bt[bi] : -1;
        if (blk < 0 || blk >= num_blocks) {
          atomicOr(status, GV_ST_BAD_INDEX);
          blk = 0;
        }
        const int row = blk * block_size + pos % block_size;
        sm100::mbar_expect_tx(&bars->k_full[s], K_BYTES);
        for (int c = 0; c < NCHUNK; ++c)
          sm100::tma_load_2d(k_s + s * K_BYTES + c * K_CHUNK, &tmK, &bars->k_full[s], c * 64, row);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (sm100::elect_one()) {
      constexpr uint32_t idesc_qk = sm100::make_idesc(HEADS, BN, 1, 1);
      constexpr uint32_t idesc_pv = sm100::make_idesc(HEADS, OCOLS, 1, 1) | sm100::IDESC_B_MN_MAJOR;
      bool ok = sm100::mbar_wait(&bars->q_full, 0);
      if (!ok) atomicOr(status, GV_ST_TIMEOUT_MMA);
      const uint32_t qa = sm100::smem_u32(q_s), pa = sm100::smem_u32(p_s);
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
        const uint32_t ka = sm100::smem_u32(k_s + s * K_BYTES);
#pragma unroll 1
        for (int c = 0; c < NCHUNK; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            sm100::mma_f16_ss(tmem + sb * 32, sm100::smem_desc_sw128(qa + c * Q_CHUNK) + (uint64_t)(2 * k),
                              sm100::smem_desc_sw128(ka + c * K_CHUNK) + (uint64_t)(2 * k), idesc_qk,
                              (uint32_t)((c | k) != 0));
        }
        sm100::tc_commit(&bars->s_full[sb]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int t = 0; t < ntiles && ok; ++t) {
        if (t + 1 < ntiles) ok = issue_qk(t + 1);
        if (!ok) break;
        const int s = t % KV_STAGES;
        if (!sm100::mbar_wait(&bars->p_full, (uint32_t)t & 1u)) {
          atomicOr(status, GV_ST_TIMEOUT_MMA);
          ok = false;
          break;
        }
        sm100::tc_fence_after();
        // V = the first 512 columns of the latent tile; this CTA's half = chunks 4 half .. 4 half + 3
        const uint32_t va = sm100::smem_u32(k_s + s * K_BYTES) + (uint32_t)(half * 4) * K_CHUNK;
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint64_t da = sm100::smem_desc_sw64(pa) + (uint64_t)(2 * k);
          const uint64_t db = sm100::smem_desc_mn_sw128(va + (uint32_t)k * 2048u, K_CHUNK, 1024);
          sm100::mma_f16_ss(tmem_o, da, db, idesc_pv, (uint32_t)((t | k) != 0));
        }
        sm100::tc_commit(&bars->k_empty[s]);      // the tile is free once P V has read it
        sm100::tc_commit(&bars->pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                    // head inside the group = TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    // A wait that runs out only clears `ok`: the thread keeps walking the loop without further
    // waits, so the warp-collective TMEM accesses below always see the whole warp.
    for (int t = 0; t < ntiles; ++t) {
      const int sb = t & 1;
      const uint32_t sph = (uint32_t)(t >> 1) & 1u;
      if (ok && !sm100::mbar_wait(&bars->s_full[sb], sph)) ok = false;
      sm100::tc_fence_after();
      float sv[BN];
      sm100::tmem_ld32(tmem + lane_addr + sb * 32, reinterpret_cast<uint32_t*>(sv));
      sm100::tmem_ld_wait();
      sm100::tc_fence_before();
      sm100::mbar_arrive(&bars->s_empty[sb]);
      const int k0 = start + t * BN;
      float mx = -INFINITY;
      // sv stays unscaled: the scale (> 0) goes onto the row maximum once and into the exponent's
      // multiply-add
#pragma unroll
      for (int j = 0; j < BN; ++j) {
        sv[j] = (k0 + j < end) ? sv[j] : -INFINITY;
        mx = fmaxf(mx, sv[j]);
      }
      mx *= scale_log2;
      const bool grow = mx > m + RESCALE_LOG2;
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
          for (int c = 0; c < OCOLS; c += 16) {
            uint32_t o[16];
            sm100::tmem_ld16(tmem_o + lane_addr + c, o);
            sm100::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
            sm100::tmem_st16(tmem_o + lane_addr + c, o);
          }
          sm100::tmem_st_wait();
          l *= f;
        }
        m = m_new;
      }
      const float nmref = (m == -INFINITY) ? 0.f : -m;
      float rs = 0.f;
      uint32_t pk[BN / 2];
#pragma unroll
      for (int j = 0; j < BN; j += 2) {
        const float p0 = sm100::ex2_approx(fmaf(sv[j], scale_log2, nmref));
        const float p1 = sm100::ex2_approx(fmaf(sv[j + 1], scale_log2, nmref));
        rs += p0 + p1;
        pk[j >> 1] = pack_bf2(p0, p1);
      }
      l += rs;
      if (t > 0 && !waited && ok && !sm100::mbar_wait(&bars->pv_done, (uint32_t)(t - 1) & 1u)) ok = false;
      // P row r: 64 bytes = 4 pieces of 16 bytes, XOR-swizzled by ((r >> 1) & 3) (64-byte swizzle)
      uint8_t* row = p_s + r * 64;
#pragma unroll
      for (int piece = 0; piece < 4; ++piece)
        *reinterpret_cast<uint4*>(row + ((piece ^ ((r >> 1) & 3)) << 4)) =
            make_uint4(pk[piece * 4], pk[piece * 4 + 1], pk[piece * 4 + 2], pk[piece * 4 + 3]);
      sm100::fence_proxy_async_smem();
      sm100::tc_fence_before();
      sm100::mbar_arrive(&bars->p_full);
    }
    if (ok && !sm100::mbar_wait(&bars->pv_done, (uint32_t)(ntiles - 1) & 1u)) ok = false;
    if (!ok && lane == 0) atomicOr(status, GV_ST_TIMEOUT_EPI);
    sm100::tc_fence_after();
    if (__all_sync(0xffffffffu, ok)) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const long long head = head0 + r;
#pragma unroll 1
      for (int c = 0; c < OCOLS; c += 16) {
        uint32_t o[16];
        sm100::tmem_ld16(tmem_o + lane_addr + c, o);
        sm100::tmem_ld_wait();
        float f[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(o[j]) * inv;
        if (nsplit == 1) {
          bf16* dst = out + head * DC + half * OCOLS + c;
          st8(dst, pack8(f));
          st8(dst + 8, pack8(f + 8));
        } else {
          float4* dst = reinterpret_cast<float4*>(part_o + (head * nsplit + split) * DC + half * OCOLS + c);
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
        }
      }
      if (nsplit > 1 && half == 0) part_lse[head * nsplit + split] = l > 0.f ? m + log2f(l) : -INFINITY;
    }
  }
  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem, TMEM_COLS);
  }
}

__global__ void mla_tc_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                    bf16* __restrict__ out, int nsplit) {
  const long long head = blockIdx.x;
  const float* lse = part_lse + head * nsplit;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, lse[s]);
  for (int d = threadIdx.x; d < DC; d += blockDim.x) {
    float W = 0.f, acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float lv = lse[s];
      if (lv == -INFINITY) continue;
      const float w = exp2f(lv - M);
      W += w;
      acc += w * part_o[(head * nsplit + s) * DC + d];
    }
    out[head * DC + d] = f2bf(W > 0.f ? acc / W : 0.f);
  }
}

}  // namespace mlatc
}  // namespace gv

using namespace gv;

// Decode-only absorbed MLA: qf [batch, heads, 576] (one token per request; seq_lens[b] keys,
// 0 for a padding row), cache
// [num_blocks * block_size, 576], out [batch, heads, 512]. heads must be a multiple of 128 and
// block_size a multiple of 32. Scratch when nsplit > 1: part_o batch*heads*nsplit*512 floats,
// part_lse batch*heads*nsplit floats. Other shapes: GV_EUNSUPPORTED (the caller takes mla.cu).
extern "C" int gv_mla_attention_tc(const void* qf, const void* cache, const void* block_tables,
                                   const void* seq_lens, void* out, void* part_o, void* part_lse,
                                   long long batch, long long heads, long long dc, long long dr,
                                   long long block_size, long long max_blocks, long long nsplit,
                                   float scale, long long num_blocks, void* stream) {
  if (!qf || !cache || !block_tables || !seq_lens || !out) return GV_EINVAL;
  if (!(scale > 0.f)) return GV_EINVAL;              // the kernel scales the row maximum, not every score
  if (batch == 0) return GV_OK;
  if (dc != mlatc::DC || dr != mlatc::DR || heads % mlatc::HEADS != 0 || block_size % mlatc::BN != 0)
    return GV_EUNSUPPORTED;
  if (nsplit < 1 || (nsplit > 1 && (!part_o || !part_lse))) return GV_EINVAL;
  if (nsplit > 65535 || batch * (heads / mlatc::HEADS) > 65535) return GV_ETOOBIG;
  if ((reinterpret_cast<uintptr_t>(qf) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(part_o)) & 15)
    return GV_EINVAL;
  CUtensorMap tmQ, tmK;
  int rc;
  if ((rc = gemm::cached_tmap_bf16(&tmQ, qf, batch * heads, mlatc::DQ, mlatc::DQ, mlatc::HEADS)) != GV_OK) return rc;
  if ((rc = gemm::cached_tmap_bf16(&tmK, cache, num_blocks * block_size, mlatc::DQ, mlatc::DQ, mlatc::BN)) != GV_OK)
    return rc;
  auto kern = mlatc::mla_tc_kernel;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, mlatc::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_last_error("mla_tc: smem attr", e);
      return GV_ECUDA;
    }
    configured = true;
  }
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(2, (unsigned)nsplit, (unsigned)(batch * (heads / mlatc::HEADS)));
  kern<<<grid, mlatc::THREADS, mlatc::SMEM_BYTES, st>>>(
      tmQ, tmK, (const int*)block_tables, (const int*)seq_lens, (bf16*)out, (float*)part_o, (float*)part_lse,
      (int)heads, (int)block_size, (int)max_blocks, (int)nsplit, scale * 1.4426950408889634f, num_blocks,
      status_word());
  rc = check_launch("mla_attention_tc");
  if (rc == GV_OK && nsplit > 1) {
    mlatc::mla_tc_merge_kernel<<<(unsigned)(batch * heads), 128, 0, st>>>((const float*)part_o,
                                                                          (const float*)part_lse, (bf16*)out,
                                                                          (int)nsplit);
    rc = check_launch("mla_tc merge");
  }
  return rc;
}

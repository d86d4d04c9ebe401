// Lightning-indexer scores of DeepSeek sparse attention on the 5th-generation tensor cores.
//
//     score[t, j] = sum_h w[t, h] * relu(q[t, h, :] . k[j, :])        (head_dim 128)
//
// The reference computes this as two chained cube GEMMs (xlite/csrc/kernels/indexer_scores.h:41-48,
// 294); `indexer_scores_kernel` in dsa.cu is the CUDA-core form (one thread per key). Here the
// keys ride the 128 TMEM lanes: for a tile of 128 cached index keys, D[key, head] = K_tile . Q_t^T
// is one tcgen05 accumulator of `Hi` columns (8 MMAs of depth 16), and the epilogue thread of a key
// applies ReLU, the per-head weights and the sum over heads to its own TMEM lane: the weighted
// head reduction never leaves the SM and the score row is written once, coalesced over keys.
// A CTA keeps its token's query block in shared memory and walks up to TILES_PER_CTA key tiles:
// index-cache tiles arrive by TMA through the block table into a two-slot ring, accumulators are
// double-buffered in TMEM, so the load of tile i + 1, the MMAs of tile i and the epilogue of tile
// i - 1 overlap. Every wait is bounded.
#include "sm100.cuh"
#include "gvirt_kernels.h"

namespace gv {

namespace gemm {
int cached_tmap_bf16(CUtensorMap* out, const void* base, long long rows, long long cols,
                     long long row_stride_elems, int box_rows);
}

namespace dsatc {

constexpr int D = 128;
constexpr int BKEYS = 128;
constexpr int CHUNK = 128 * 128;                 // 128 rows x 128 bytes
constexpr int K_BYTES = 2 * CHUNK;               // one key tile
constexpr int TILES_PER_CTA = 8;
constexpr int THREADS = 192;
constexpr int MAX_HEADS = 128;

struct Bars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_slot;
};

__global__ void __launch_bounds__(THREADS, 1)
indexer_scores_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const float* __restrict__ w, const int* __restrict__ block_tables,
                         const int* __restrict__ q_start, const int* __restrict__ cached_lens,
                         float* __restrict__ scores, int batch, int Hi, int block_size, int max_blocks,
                         long long lds, int relu, long long num_blocks, unsigned int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = base;                           // [2 chunks][Hi rows x 128 bytes] (Hi <= 128)
  uint8_t* k_s = q_s + K_BYTES;                  // [2 slots][2 chunks][128 rows x 128 bytes]
  Bars* bars = reinterpret_cast<Bars*>(k_s + 2 * K_BYTES);
  float* s_w = reinterpret_cast<float*>(bars + 1);
  __shared__ int s_req;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  if (threadIdx.x == 0) {
    int lo = 0, hi = batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (q_start[mid] <= t) lo = mid;
      else hi = mid;
    }
    s_req = lo;
  }
  for (int i = threadIdx.x; i < Hi; i += THREADS) s_w[i] = w[(long long)t * Hi + i];
  __syncthreads();
  const int b = s_req;
  const int kv_len = cached_lens[b] + (t - q_start[b]) + 1;
  const int tile0 = blockIdx.x * TILES_PER_CTA;
  const int live = min(TILES_PER_CTA, max(0, (kv_len - tile0 * BKEYS + BKEYS - 1) / BKEYS));
  // positions past the token's context read as -inf (whole tiles here, the tail of the last live
  // tile in the epilogue)
  for (long long p = (long long)(tile0 + live) * BKEYS + threadIdx.x;
       p < (long long)(tile0 + TILES_PER_CTA) * BKEYS && p < lds; p += THREADS)
    scores[(long long)t * lds + p] = -INFINITY;
  if (live == 0) return;                          // uniform per CTA
  const int* bt = block_tables + (long long)b * max_blocks;

  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(&tmQ);
    sm100::tma_prefetch_desc(&tmK);
    sm100::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      sm100::mbar_init(&bars->k_full[s], 1);
      sm100::mbar_init(&bars->k_empty[s], 1);
      sm100::mbar_init(&bars->acc_full[s], 1);
      sm100::mbar_init(&bars->acc_empty[s], 128);
    }
    sm100::mbar_fence_init();
  }
  const uint32_t tmem_cols = Hi * 2 <= 32 ? 32 : Hi * 2 <= 64 ? 64 : Hi * 2 <= 128 ? 128 : 256;
  if (warp == 1) {
    sm100::tmem_alloc(&bars->tmem_slot, tmem_cols);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_slot);

  if (warp == 0) {
    if (sm100::elect_one()) {
      sm100::mbar_expect_tx(&bars->q_full, (uint32_t)(Hi * D * 2));
      for (int c = 0; c < 2; ++c) sm100::tma_load_2d(q_s + c * CHUNK, &tmQ, &bars->q_full, c * 64, t * Hi);
      const int rows_per_box = block_size < BKEYS ? block_size : BKEYS;
      const int boxes = BKEYS / rows_per_box;
      for (int i = 0; i < live; ++i) {
        const int s = i & 1;
        const uint32_t ph = (uint32_t)(i >> 1) & 1u;
        if (!sm100::mbar_wait(&bars->k_empty[s], ph ^ 1u)) {
          atomicOr(status, GV_ST_TIMEOUT_TMA);
          break;
        }
        sm100::mbar_expect_tx(&bars->k_full[s], K_BYTES);
        for (int bx = 0; bx < boxes; ++bx) {
          const int pos = (tile0 + i) * BKEYS + bx * rows_per_box;
          const int bi = pos / block_size;
          int blk = bi < max_blocks ? bt[bi] : -1;
          if (blk < 0 || blk >= num_blocks) {
            if (pos < kv_len) atomicOr(status, GV_ST_BAD_INDEX);
            blk = 0;
          }
          const int row = blk * block_size + pos % block_size;
          for (int c = 0; c < 2; ++c)
            sm100::tma_load_2d(k_s + s * K_BYTES + c * CHUNK + bx * rows_per_box * 128, &tmK, &bars->k_full[s],
                               c * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    if (sm100::elect_one()) {
      const uint32_t idesc = sm100::make_idesc(BKEYS, Hi, 1, 1);
      bool ok = sm100::mbar_wait(&bars->q_full, 0);
      if (!ok) atomicOr(status, GV_ST_TIMEOUT_MMA);
      const uint32_t qa = sm100::smem_u32(q_s);
      for (int i = 0; i < live && ok; ++i) {
        const int s = i & 1;
        const uint32_t ph = (uint32_t)(i >> 1) & 1u;
        if (!sm100::mbar_wait(&bars->k_full[s], ph) || !sm100::mbar_wait(&bars->acc_empty[s], ph ^ 1u)) {
          atomicOr(status, GV_ST_TIMEOUT_MMA);
          break;
        }
        sm100::tc_fence_after();
        const uint32_t ka = sm100::smem_u32(k_s + s * K_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (uint32_t)(k >> 2) * CHUNK;
          sm100::mma_f16_ss(tmem + s * Hi, sm100::smem_desc_sw128(ka + off) + (uint64_t)(2 * (k & 3)),
                            sm100::smem_desc_sw128(qa + off) + (uint64_t)(2 * (k & 3)), idesc, (uint32_t)(k != 0));
        }
        sm100::tc_commit(&bars->k_empty[s]);
        sm100::tc_commit(&bars->acc_full[s]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                    // key inside the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    bool ok = true;
    for (int i = 0; i < live && ok; ++i) {
      const int s = i & 1;
      const uint32_t ph = (uint32_t)(i >> 1) & 1u;
      if (!sm100::mbar_wait(&bars->acc_full[s], ph)) {
        ok = false;
        break;
      }
      sm100::tc_fence_after();
      float total = 0.f;
#pragma unroll 1
      for (int c = 0; c < Hi; c += 16) {
        uint32_t v[16];
        sm100::tmem_ld16(tmem + lane_addr + s * Hi + c, v);
        sm100::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float d = __uint_as_float(v[j]);
          if (relu) d = fmaxf(d, 0.f);
          total += s_w[c + j] * d;
        }
      }
      sm100::tc_fence_before();
      sm100::mbar_arrive(&bars->acc_empty[s]);
      const long long pos = (long long)(tile0 + i) * BKEYS + r;
      if (pos < lds) scores[(long long)t * lds + pos] = pos < kv_len ? total : -INFINITY;
    }
    if (!ok && lane == 0) atomicOr(status, GV_ST_TIMEOUT_EPI);
  }
  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem, tmem_cols);
  }
}

}  // namespace dsatc
}  // namespace gv

using namespace gv;

// Same arguments as gv_indexer_scores. D must be 128, Hi a multiple of 16 up to 128, block_size a
// power of two >= 8; other shapes return GV_EUNSUPPORTED (the caller takes the CUDA-core kernel).
extern "C" int gv_indexer_scores_tc(const void* q, const void* w, const void* k_cache, const void* block_tables,
                                    const void* q_start, const void* cached_lens, void* scores, long long T,
                                    long long batch, long long Hi, long long D, long long block_size,
                                    long long max_blocks, long long lds, long long relu, long long num_blocks,
                                    void* stream) {
  if (!q || !w || !k_cache || !block_tables || !q_start || !cached_lens || !scores) return GV_EINVAL;
  if (T == 0) return GV_OK;
  if (D != dsatc::D || Hi < 16 || Hi > dsatc::MAX_HEADS || (Hi & 15)) return GV_EUNSUPPORTED;
  if (block_size < 8 || (block_size & (block_size - 1))) return GV_EUNSUPPORTED;
  if (T > 65535 || (lds % 128)) return GV_EUNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache)) & 15) return GV_EINVAL;
  CUtensorMap tmQ, tmK;
  int rc;
  if ((rc = gemm::cached_tmap_bf16(&tmQ, q, T * Hi, dsatc::D, dsatc::D, (int)Hi)) != GV_OK) return rc;
  const int box = block_size < 128 ? (int)block_size : 128;
  if ((rc = gemm::cached_tmap_bf16(&tmK, k_cache, num_blocks * block_size, dsatc::D, dsatc::D, box)) != GV_OK)
    return rc;
  const int smem = 3 * dsatc::K_BYTES + 1024 + (int)sizeof(dsatc::Bars) + dsatc::MAX_HEADS * 4 + 64;
  auto kern = dsatc::indexer_scores_tc_kernel;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_last_error("indexer_scores_tc: smem attr", e);
      return GV_ECUDA;
    }
    configured = true;
  }
  const long long tiles = lds / 128;
  dim3 grid((unsigned)((tiles + dsatc::TILES_PER_CTA - 1) / dsatc::TILES_PER_CTA), (unsigned)T);
  kern<<<grid, dsatc::THREADS, smem, (cudaStream_t)stream>>>(
      tmQ, tmK, (const float*)w, (const int*)block_tables, (const int*)q_start, (const int*)cached_lens,
      (float*)scores, (int)batch, (int)Hi, (int)block_size, (int)max_blocks, lds, (int)relu, num_blocks,
      status_word());
  return check_launch("gv_indexer_scores_tc");
}

// Paged GQA decode attention, split-KV with an explicit merge pass.
//
// Replaces the reference's `flash_attention_<T>` decode path (xlite/csrc/kernels/
// flash_attention.h:687, host xlite/csrc/op.cpp:968-993): tasks are (request, kv head, kv
// split); every task produces a normalised partial output plus a log-sum-exp, and a second
// kernel merges the splits. The reference serialises the merge with an unbounded
// inter-core flag chain (flash_attention.h:118-153); here the merge is a separate launch,
// so no kernel ever waits on another.
//
// A CTA has 4 warps. The q heads that share one kv head are packed into the 16-row M
// dimension of mma.sync (group size <= 16); each warp streams its own 32-token K/V tiles
// from the paged cache with cp.async (double-buffered, XOR-swizzled) and keeps an online
// softmax state; the 4 warps are merged through shared memory at the end.
// q is expected pre-scaled (the RoPE kernel multiplies by head_dim^-0.5); `scale` is an
// extra factor (1.0 for the standard models).
#include "mma_sync.cuh"
#include "gvirt_kernels.h"

namespace gv {

constexpr int DEC_WARPS = 4;
// Tile shape of the allocation-free entry point (the regular entry point picks a variant, by
// default 16 tokens x 3 stages: see g_decode_variant).
constexpr int DEC_TOK = 32;     // kv tokens per warp tile
constexpr int DEC_STAGES = 2;

// TOK kv tokens per warp tile, STAGES-deep cp.async ring per warp. Smaller tiles / rings let
// several CTAs share an SM (their start-up and merge phases then overlap another CTA's
// streaming); deeper rings keep more bytes in flight per CTA.
template <int HD, int DEC_TOK, int DEC_STAGES>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc,
                    const bf16* __restrict__ vc, const int* __restrict__ block_tables,
                    const int* __restrict__ seq_lens, bf16* __restrict__ out,
                    float* __restrict__ part_o, float* __restrict__ part_lse, int nq, int nkv,
                    int block_size, int max_blocks, int nsplit, float scale_log2,
                    long long num_blocks, unsigned int* status, int* counters) {
  constexpr int ROW_BYTES = HD * 2;
  constexpr int CH = ROW_BYTES / 16;            // 16-byte chunks per row
  constexpr int TILE_BYTES = DEC_TOK * ROW_BYTES;
  constexpr int WARP_BYTES = DEC_STAGES * 2 * TILE_BYTES;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int G = nq / nkv;
  const int len = seq_lens[b];
  int chunk = (len + nsplit - 1) / nsplit;
  chunk = ((chunk + DEC_TOK - 1) / DEC_TOK) * DEC_TOK;
  const int start = split * chunk;
  const int end = min(len, start + chunk);
  const int ntiles = end > start ? (end - start + DEC_TOK - 1) / DEC_TOK : 0;
  uint8_t* wsm = smem + warp * WARP_BYTES;
  const int* bt = block_tables + (long long)b * max_blocks;

  // ---- Q fragments (A operand), rows >= G are zero
  uint32_t qf[HD / 16][4];
  {
    const int r0 = lane >> 2, c = (lane & 3) * 2;
    const bf16* q0 = q + ((long long)b * nq + (long long)kvh * G + r0) * HD;
    const bf16* q1 = q0 + 8 * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      qf[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c) : 0u;
      qf[ks][1] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + c) : 0u;
      qf[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + c) : 0u;
      qf[ks][3] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + c) : 0u;
    }
  }

  auto load_tile = [&](int stage, int tile) {
    uint8_t* ks = wsm + stage * 2 * TILE_BYTES;
    uint8_t* vs = ks + TILE_BYTES;
    const int pos = start + tile * DEC_TOK + lane;  // this lane resolves row `lane`
    long long slot = -1;
    if (pos < end) {
      // a sequence length beyond the block-table row is bad metadata: flag it, read nothing
      const int bi = pos / block_size;
      const int blk = bi < max_blocks ? bt[bi] : -1;
      if (blk < 0 || blk >= num_blocks) atomicOr(status, GV_ST_BAD_INDEX);
      else slot = (long long)blk * block_size + pos % block_size;
    }
#pragma unroll
    for (int j = 0; j < DEC_TOK * CH / 32; ++j) {
      const int i = lane + 32 * j;
      const int r = i / CH, c = i % CH;
      const long long s = __shfl_sync(0xffffffffu, slot, r);
      const bool ok = s >= 0;
      const long long off = ((ok ? s : 0) * nkv + kvh) * HD + c * 8;
      cp_async16(ks + swz<ROW_BYTES>(r, c), kc + off, ok);
      cp_async16(vs + swz<ROW_BYTES>(r, c), vc + off, ok);
    }
  };

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (warp + s * DEC_WARPS < ntiles) load_tile(s, warp + s * DEC_WARPS);
    cp_async_commit();
  }
  int it = 0;
  for (int tile = warp; tile < ntiles; tile += DEC_WARPS, ++it) {
    const int nxt = tile + (DEC_STAGES - 1) * DEC_WARPS;
    if (nxt < ntiles) load_tile((it + DEC_STAGES - 1) % DEC_STAGES, nxt);
    cp_async_commit();
    cp_async_wait<DEC_STAGES - 1>();
    __syncwarp();
    const uint32_t kbase = smem_ptr(wsm + (it % DEC_STAGES) * 2 * TILE_BYTES);
    const uint32_t vbase = kbase + TILE_BYTES;

    float s[DEC_TOK / 8][4];
#pragma unroll
    for (int i = 0; i < DEC_TOK / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < DEC_TOK / 16; ++np) {
        uint32_t r0, r1, r2, r3;
        const int row = np * 16 + (mi >> 1) * 8 + rr;
        ldmatrix_x4(kbase + swz<ROW_BYTES>(row, 2 * ks + (mi & 1)), r0, r1, r2, r3);
        mma_bf16_16816(s[2 * np], qf[ks], r0, r1);
        mma_bf16_16816(s[2 * np + 1], qf[ks], r2, r3);
      }
    }
    // mask + online softmax (log2 domain)
    const int tile_pos = start + tile * DEC_TOK;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < DEC_TOK / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int pos = tile_pos + nt * 8 + (lane & 3) * 2 + (e & 1);
        float v = pos < end ? s[nt][e] * scale_log2 : -INFINITY;
        s[nt][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v);
        else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float c0 = m0 == -INFINITY ? 0.f : exp2f(m0 - mn0);
    const float c1 = m1 == -INFINITY ? 0.f : exp2f(m1 - mn1);
    m0 = mn0;
    m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < DEC_TOK / 8; ++nt) {
      s[nt][0] = exp2f(s[nt][0] - mn0);
      s[nt][1] = exp2f(s[nt][1] - mn0);
      s[nt][2] = exp2f(s[nt][2] - mn1);
      s[nt][3] = exp2f(s[nt][3] - mn1);
      rs0 += s[nt][0] + s[nt][1];
      rs1 += s[nt][2] + s[nt][3];
    }
    l0 = l0 * c0 + rs0;
    l1 = l1 * c1 + rs1;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      o[i][0] *= c0;
      o[i][1] *= c0;
      o[i][2] *= c1;
      o[i][3] *= c1;
    }
#pragma unroll
    for (int j = 0; j < DEC_TOK / 16; ++j) {
      uint32_t pf[4];
      pf[0] = pack_bf16x2(s[2 * j][0], s[2 * j][1]);
      pf[1] = pack_bf16x2(s[2 * j][2], s[2 * j][3]);
      pf[2] = pack_bf16x2(s[2 * j + 1][0], s[2 * j + 1][1]);
      pf[3] = pack_bf16x2(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
      for (int c = 0; c < CH; c += 2) {
        uint32_t r0, r1, r2, r3;
        const int row = j * 16 + (mi & 1) * 8 + rr;
        ldmatrix_x4_trans(vbase + swz<ROW_BYTES>(row, c + (mi >> 1)), r0, r1, r2, r3);
        mma_bf16_16816(o[c], pf, r0, r1);
        mma_bf16_16816(o[c + 1], pf, r2, r3);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  // quad-reduce the row sums
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();

  // ---- merge the 4 warps through shared memory: per warp [16 rows][HD] fp32 + m[16] + l[16]
  float* wo = reinterpret_cast<float*>(smem + warp * WARP_BYTES);
  float* wm = wo + 16 * HD;
  float* wl = wm + 16;
  {
    const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      wo[r0 * HD + i * 8 + c] = o[i][0];
      wo[r0 * HD + i * 8 + c + 1] = o[i][1];
      wo[(r0 + 8) * HD + i * 8 + c] = o[i][2];
      wo[(r0 + 8) * HD + i * 8 + c + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      wm[r0] = m0;
      wm[r0 + 8] = m1;
      wl[r0] = l0;
      wl[r0 + 8] = l1;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int row = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w)
      M = fmaxf(M, reinterpret_cast<float*>(smem + w * WARP_BYTES)[16 * HD + row]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float* base = reinterpret_cast<float*>(smem + w * WARP_BYTES);
      const float mw = base[16 * HD + row];
      if (mw == -INFINITY) continue;
      const float f = exp2f(mw - M);
      L += base[16 * HD + 16 + row] * f;
      acc += base[row * HD + d] * f;
    }
    const float val = L > 0.f ? acc / L : 0.f;
    const long long head = (long long)b * nq + (long long)kvh * G + row;
    if (nsplit == 1) {
      out[head * HD + d] = f2bf(val);
    } else {
      part_o[(head * nsplit + split) * HD + d] = val;
      if (d == 0) part_lse[head * nsplit + split] = L > 0.f ? M + log2f(L) : -INFINITY;
    }
  }
  if (nsplit == 1 || counters == nullptr) return;
  // ---- in-kernel merge: the CTA that publishes the last split of this (request, kv head) merges
  // all of them, so no second launch is needed. A ticket counter per (request, kv head) counts the
  // finished splits; it returns to zero for the next launch. Nobody waits on anybody.
  __shared__ int s_last;
  __syncthreads();                   // every thread's partials are written ...
  if (threadIdx.x == 0) {
    __threadfence();                 // ... and (fences are cumulative) visible device-wide ...
    int* cnt = counters + (long long)b * nkv + kvh;
    const int old = atomicAdd(cnt, 1);      // ... before this CTA's ticket is
    s_last = old == nsplit - 1;
    if (s_last) {
      *cnt = 0;
      __threadfence();
    }
  }
  __syncthreads();
  if (!s_last) return;
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int row = idx / HD, d = idx % HD;
    const long long head = (long long)b * nq + (long long)kvh * G + row;
    const float* lse = part_lse + head * nsplit;
    float M = -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) M = fmaxf(M, __ldcg(lse + sp));
    float W = 0.f, acc = 0.f;
    for (int sp = 0; sp < nsplit; ++sp) {
      const float l = __ldcg(lse + sp);
      if (l == -INFINITY) continue;
      const float w = exp2f(l - M);
      W += w;
      acc += w * __ldcg(part_o + (head * nsplit + sp) * HD + d);
    }
    out[head * HD + d] = f2bf(W > 0.f ? acc / W : 0.f);
  }
}

template <int HD>
__global__ void decode_merge_kernel(const float* __restrict__ part_o,
                                    const float* __restrict__ part_lse, bf16* __restrict__ out,
                                    int nsplit) {
  pdl_wait();
  pdl_trigger();
  const long long head = blockIdx.x;
  const float* lse = part_lse + head * nsplit;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, lse[s]);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float W = 0.f, acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float l = lse[s];
      if (l == -INFINITY) continue;
      const float w = exp2f(l - M);
      W += w;
      acc += w * part_o[(head * nsplit + s) * HD + d];
    }
    out[head * HD + d] = f2bf(W > 0.f ? acc / W : 0.f);
  }
}

template <int HD, int TOK = DEC_TOK, int STAGES = DEC_STAGES>
static int launch_decode(const void* q, const void* kc, const void* vc, const void* bt,
                         const void* lens, void* out, void* part_o, void* part_lse, int batch,
                         int nq, int nkv, int block_size, int max_blocks, int nsplit, float scale,
                         long long num_blocks, cudaStream_t st, int* counters = nullptr) {
  constexpr int SMEM = DEC_WARPS * STAGES * 2 * TOK * HD * 2;
  static_assert(STAGES * 2 * TOK * HD * 2 >= (16 * HD + 32) * 4, "merge area must fit");
  auto kern = paged_decode_kernel<HD, TOK, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) {
      set_last_error("paged_decode: smem attr", e);
      return GV_ECUDA;
    }
    configured = true;
  }
  dim3 grid((unsigned)nkv, (unsigned)batch, (unsigned)nsplit);
  launch_pdl(kern, grid, dim3(DEC_WARPS * 32), SMEM, st, (const bf16*)q, (const bf16*)kc,
             (const bf16*)vc, (const int*)bt, (const int*)lens, (bf16*)out, (float*)part_o,
             (float*)part_lse, nq, nkv, block_size, max_blocks, nsplit,
             scale * 1.4426950408889634f, num_blocks, status_word(), counters);
  int rc = check_launch("paged_decode");
  if (rc != GV_OK) return rc;
  if (nsplit > 1 && counters == nullptr) {
    launch_pdl(decode_merge_kernel<HD>, dim3((unsigned)(batch * nq)), dim3(HD < 128 ? HD : 128), 0,
               st, (const float*)part_o, (const float*)part_lse, (bf16*)out, nsplit);
    rc = check_launch("decode_merge");
  }
  return rc;
}

}  // namespace gv

using namespace gv;

// Scratch needed by gv_paged_attention_decode when nsplit > 1, in bytes:
//   part_o  : batch * nq * nsplit * head_dim * 4
//   part_lse: batch * nq * nsplit * 4
template <int HD>
static int dispatch_variant(long long variant, const void* q, const void* kc, const void* vc,
                            const void* bt, const void* lens, void* out, void* po, void* pl, int batch,
                            int nq, int nkv, int bs, int mb, int ns, float scale, long long nb,
                            cudaStream_t st, int* cnt = nullptr) {
  switch (variant) {
    case 1: return launch_decode<HD, 16, 2>(q, kc, vc, bt, lens, out, po, pl, batch, nq, nkv, bs, mb, ns, scale, nb, st, cnt);
    case 2: return launch_decode<HD, 16, 3>(q, kc, vc, bt, lens, out, po, pl, batch, nq, nkv, bs, mb, ns, scale, nb, st, cnt);
    case 3: return launch_decode<HD, 16, 4>(q, kc, vc, bt, lens, out, po, pl, batch, nq, nkv, bs, mb, ns, scale, nb, st, cnt);
    case 4: return launch_decode<HD, 32, 3>(q, kc, vc, bt, lens, out, po, pl, batch, nq, nkv, bs, mb, ns, scale, nb, st, cnt);
    default: return launch_decode<HD, 32, 2>(q, kc, vc, bt, lens, out, po, pl, batch, nq, nkv, bs, mb, ns, scale, nb, st, cnt);
  }
}

static long long g_decode_variant = 2;  // (16 tokens, 3 stages): two CTAs per SM, 2 tiles in flight per warp

extern "C" void gv_set_decode_variant(long long v) { g_decode_variant = v; }

static int decode_any(const void* q, const void* k_cache, const void* v_cache,
                      const void* block_tables, const void* seq_lens, void* out, void* part_o,
                      void* part_lse, void* counters, long long batch, long long nq, long long nkv,
                      long long head_dim, long long block_size, long long max_blocks,
                      long long nsplit, float scale, long long num_blocks, void* stream) {
  if (!q || !k_cache || !v_cache || !block_tables || !seq_lens || !out) return GV_EINVAL;
  if (batch == 0) return GV_OK;
  if (nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || nsplit < 1) return GV_EINVAL;
  if (nsplit > 1 && (!part_o || !part_lse)) return GV_EINVAL;
  if (batch > 65535 || nsplit > 65535) return GV_ETOOBIG;
  cudaStream_t st = (cudaStream_t)stream;
  // the per-warp merge area (16*HD + 32 floats) must fit in the warp's tile ring: true for HD >= 64
  switch (head_dim) {
    case 64:
      return dispatch_variant<64>(g_decode_variant, q, k_cache, v_cache, block_tables, seq_lens, out,
                                  part_o, part_lse, (int)batch, (int)nq, (int)nkv, (int)block_size,
                                  (int)max_blocks, (int)nsplit, scale, num_blocks, st, (int*)counters);
    case 128:
      return dispatch_variant<128>(g_decode_variant, q, k_cache, v_cache, block_tables, seq_lens, out,
                                   part_o, part_lse, (int)batch, (int)nq, (int)nkv, (int)block_size,
                                   (int)max_blocks, (int)nsplit, scale, num_blocks, st, (int*)counters);
    default:
      return GV_EUNSUPPORTED;
  }
}

extern "C" int gv_paged_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                                         const void* block_tables, const void* seq_lens, void* out,
                                         void* part_o, void* part_lse, long long batch,
                                         long long nq, long long nkv, long long head_dim,
                                         long long block_size, long long max_blocks,
                                         long long nsplit, float scale, long long num_blocks,
                                         void* stream) {
  return decode_any(q, k_cache, v_cache, block_tables, seq_lens, out, part_o, part_lse, nullptr, batch,
                    nq, nkv, head_dim, block_size, max_blocks, nsplit, scale, num_blocks, stream);
}

// Same, with the split merge done inside the kernel by whichever CTA finishes a (request, kv head)
// last: one launch instead of two. `counters`: batch * nkv int32, zero before the first call; the
// kernel leaves them zero again, so one array serves every call that is ordered on its stream.
extern "C" int gv_paged_attention_decode_merged(const void* q, const void* k_cache,
                                                const void* v_cache, const void* block_tables,
                                                const void* seq_lens, void* out, void* part_o,
                                                void* part_lse, void* counters, long long batch,
                                                long long nq, long long nkv, long long head_dim,
                                                long long block_size, long long max_blocks,
                                                long long nsplit, float scale,
                                                long long num_blocks, void* stream) {
  if (nsplit > 1 && !counters) return GV_EINVAL;
  return decode_any(q, k_cache, v_cache, block_tables, seq_lens, out, part_o, part_lse, counters, batch,
                    nq, nkv, head_dim, block_size, max_blocks, nsplit, scale, num_blocks, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (see gvirt_noalloc.h): split-KV scratch and the status word live in
// file-scope device arrays inside the library image instead of caller-provided memory.
#include "gvirt_noalloc.h"
#include <mutex>
#include <stdio.h>

namespace gv {

static __device__ __align__(256) unsigned char g_noalloc_scratch[GV_NOALLOC_SCRATCH_BYTES];
static __device__ __align__(256) unsigned int g_noalloc_status[64];

struct NoAllocDevice {
  void* scratch = nullptr;        // device address of g_noalloc_scratch on this device
  unsigned int* status = nullptr; // device address of g_noalloc_status on this device
};
static NoAllocDevice g_noalloc_dev[64];
static std::mutex g_noalloc_mu;

// In host code the array names above are only handles for the symbol; the device address has
// to be asked for, once per device, while that device is current.
static int noalloc_setup(NoAllocDevice** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_last_error("noalloc: cudaGetDevice", e);
    return GV_ECUDA;
  }
  if (dev < 0 || dev >= 64) return GV_EUNSUPPORTED;
  std::lock_guard<std::mutex> g(g_noalloc_mu);
  NoAllocDevice& d = g_noalloc_dev[dev];
  if (d.scratch == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_error("noalloc: cudaGetSymbolAddress(scratch)", e);
      return GV_ECUDA;
    }
    void* s = nullptr;
    e = cudaGetSymbolAddress(&s, g_noalloc_status);
    if (e != cudaSuccess || s == nullptr) {
      set_last_error("noalloc: cudaGetSymbolAddress(status)", e);
      return GV_ECUDA;
    }
    // opt in to the kernels' dynamic shared memory here, under the same lock, so that two host
    // threads making their first calls at once cannot interleave the set-up
    e = cudaFuncSetAttribute(paged_decode_kernel<64, DEC_TOK, DEC_STAGES>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             DEC_WARPS * DEC_STAGES * 2 * DEC_TOK * 64 * 2);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(paged_decode_kernel<128, DEC_TOK, DEC_STAGES>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               DEC_WARPS * DEC_STAGES * 2 * DEC_TOK * 128 * 2);
    if (e != cudaSuccess) {
      set_last_error("noalloc paged_decode: smem attr", e);
      return GV_ECUDA;
    }
    d.status = static_cast<unsigned int*>(s);
    d.scratch = p;
  }
  *out = &d;
  return GV_OK;
}

template <int HD>
static int launch_decode_noalloc(NoAllocDevice* d, const void* q, const void* kc,
                                 const void* vc, const void* bt, const void* lens, void* out,
                                 int batch, int nq, int nkv, int block_size, int max_blocks,
                                 int nsplit, float scale, long long num_blocks, cudaStream_t st) {
  constexpr int SMEM = DEC_WARPS * DEC_STAGES * 2 * DEC_TOK * HD * 2;
  auto kern = paged_decode_kernel<HD, DEC_TOK, DEC_STAGES>;
  // scratch layout: part_o [batch*nq*nsplit*HD] fp32, then part_lse [batch*nq*nsplit] fp32
  float* part_o = static_cast<float*>(d->scratch);
  float* part_lse = part_o + (size_t)batch * nq * nsplit * HD;
  dim3 grid((unsigned)nkv, (unsigned)batch, (unsigned)nsplit);
  kern<<<grid, DEC_WARPS * 32, SMEM, st>>>((const bf16*)q, (const bf16*)kc, (const bf16*)vc,
                                           (const int*)bt, (const int*)lens, (bf16*)out, part_o,
                                           part_lse, nq, nkv, block_size, max_blocks, nsplit,
                                           scale * 1.4426950408889634f, num_blocks, d->status,
                                           (int*)nullptr);
  int rc = check_launch("noalloc paged_decode");
  if (rc != GV_OK) return rc;
  if (nsplit > 1) {
    decode_merge_kernel<HD><<<(unsigned)(batch * nq), HD < 128 ? HD : 128, 0, st>>>(
        part_o, part_lse, (bf16*)out, nsplit);
    rc = check_launch("noalloc decode_merge");
  }
  return rc;
}

}  // namespace gv

extern "C" int gv_paged_attention_decode_noalloc(const void* q, const void* k_cache,
                                                 const void* v_cache, const void* block_tables,
                                                 const void* seq_lens, void* out, long long batch,
                                                 long long nq, long long nkv, long long head_dim,
                                                 long long block_size, long long max_blocks,
                                                 long long nsplit, float scale,
                                                 long long num_blocks, void* stream) {
  if (!q || !k_cache || !v_cache || !block_tables || !seq_lens || !out) return GV_EINVAL;
  if (batch == 0) return GV_OK;
  if (nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || nsplit < 1) return GV_EINVAL;
  if (batch > 65535 || nsplit > 65535) return GV_ETOOBIG;
  if (head_dim != 64 && head_dim != 128) return GV_EUNSUPPORTED;
  if (nsplit > 1) {
    const unsigned long long need =
        (unsigned long long)batch * nq * nsplit * (unsigned long long)(head_dim + 1) * 4ull;
    if (need > GV_NOALLOC_SCRATCH_BYTES) {
      char msg[256];
      snprintf(msg, sizeof(msg),
               "gv_paged_attention_decode_noalloc: split-KV scratch of %llu bytes exceeds the "
               "built-in %u bytes (reduce batch * nq * nsplit)",
               need, (unsigned)GV_NOALLOC_SCRATCH_BYTES);
      set_last_error(msg, cudaSuccess);
      return GV_ETOOBIG;
    }
  }
  NoAllocDevice* d = nullptr;
  int rc = noalloc_setup(&d);
  if (rc != GV_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (head_dim == 64)
    return launch_decode_noalloc<64>(d, q, k_cache, v_cache, block_tables, seq_lens, out,
                                     (int)batch, (int)nq, (int)nkv, (int)block_size,
                                     (int)max_blocks, (int)nsplit, scale, num_blocks, st);
  return launch_decode_noalloc<128>(d, q, k_cache, v_cache, block_tables, seq_lens, out,
                                    (int)batch, (int)nq, (int)nkv, (int)block_size,
                                    (int)max_blocks, (int)nsplit, scale, num_blocks, st);
}

extern "C" int gv_noalloc_status_read(unsigned int* host_out, void* stream) {
  if (!host_out) return GV_EINVAL;
  NoAllocDevice* d = nullptr;
  int rc = noalloc_setup(&d);
  if (rc != GV_OK) return rc;
  cudaError_t e = cudaMemcpyAsync(host_out, d->status, sizeof(unsigned int), cudaMemcpyDeviceToHost,
                                  (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) {
    set_last_error("gv_noalloc_status_read", e);
    return GV_ECUDA;
  }
  return GV_OK;
}

extern "C" int gv_noalloc_status_reset(void* stream) {
  NoAllocDevice* d = nullptr;
  int rc = noalloc_setup(&d);
  if (rc != GV_OK) return rc;
  cudaError_t e = cudaMemsetAsync(d->status, 0, sizeof(unsigned int), (cudaStream_t)stream);
  if (e != cudaSuccess) {
    set_last_error("gv_noalloc_status_reset", e);
    return GV_ECUDA;
  }
  return GV_OK;
}

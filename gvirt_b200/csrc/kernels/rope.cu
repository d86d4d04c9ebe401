// RoPE + query scaling + paged KV-cache write, with the QKV bias add and the per-head
// q/k RMSNorm folded in (Qwen2 bias, Qwen3 qk-norm), so the fused qkv row produced by the
// QKV GEMM is read exactly once.
//
// Reference counterparts: `rope_and_cache_<T>` (xlite/csrc/kernels/rope_and_cache.h:612,
// host xlite/csrc/op.cpp:905-943: NeoX rotation, partial rotary, q *= head_dim^-0.5, slot ->
// (block, offset) cache write, M-RoPE position rows), `qk_rms_norm_<T>`
// (xlite/csrc/kernels/qk_rms_norm.h:54), `add_bias_<T>`; the interleaved/complex flavour
// for MLA q_pe / k_pe is `rope_complex_and_cache_<T>`
// (xlite/csrc/kernels/rope_complex_and_cache.h:243).
//
// One warp per (token, head); heads of 128 fully rotated NeoX elements take a register-only
// variant with 8-byte accesses. cos/sin table is fp32 `[max_pos, rot_dim]` =
// `[cos(pos * f_i) | sin(pos * f_i)]`, i < rot_dim / 2.
#include "common.cuh"
#include <cstdint>
#include <cstdlib>
#include "gvirt_kernels.h"

namespace gv {

struct RopeArgs {
  bf16* qkv;             // [tokens, ld] fused row: q heads | k heads | v heads
  const bf16* bias;      // [(nq + 2 nkv) * hd] or null
  const bf16* q_norm_w;  // [hd] or null
  const bf16* k_norm_w;  // [hd] or null
  const float* cos_sin;  // [max_pos, rot_dim]
  const long long* positions;  // [pos_rows, tokens] int64
  const int* slot_mapping;     // [tokens] int32; negative = do not write the cache
  bf16* k_cache;         // [slots, nkv, hd]
  bf16* v_cache;
  bf16* q_out;           // [tokens, nq * hd]
  int tokens, nq, nkv, hd, rot_dim;
  long long ld;
  float q_scale, eps;
  int max_pos;
  long long num_slots;
  int mrope_mode;        // 0 = single position row, 1 = chunked sections, 2 = interleaved
  int sec0, sec1, sec2;  // M-RoPE sections in rotary pairs (temporal, height, width)
  int interleaved;       // 0 = NeoX half rotation, 1 = adjacent-pair (complex) rotation,
                         //     output written de-interleaved [re.. | im..]
};

__device__ __forceinline__ int mrope_row(const RopeArgs& a, int pair) {
  if (a.mrope_mode == 1) return pair < a.sec0 ? 0 : (pair < a.sec0 + a.sec1 ? 1 : 2);
  if (a.mrope_mode == 2) {
    // rows cycle t,h,w while both the h and w sections still have pairs left
    const int r = pair % 3;
    const int idx = pair / 3;
    if (r == 1 && idx < a.sec1) return 1;
    if (r == 2 && idx < a.sec2) return 2;
    return 0;
  }
  return 0;
}

__global__ void rope_kvwrite_kernel(RopeArgs a, unsigned int* status) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int heads = a.nq + 2 * a.nkv;
  if (gw >= (long long)a.tokens * heads) return;
  const int t = (int)(gw / heads), h = (int)(gw % heads);
  const int kind = h < a.nq ? 0 : (h < a.nq + a.nkv ? 1 : 2);  // q, k, v
  bf16* src = a.qkv + (long long)t * a.ld + (long long)h * a.hd;
  const bf16* bsrc = a.bias ? a.bias + (long long)h * a.hd : nullptr;

  // destination
  bf16* dst;
  if (kind == 0) {
    dst = a.q_out + ((long long)t * a.nq + h) * a.hd;
  } else {
    const int slot = a.slot_mapping ? a.slot_mapping[t] : -1;
    if (slot < 0) return;
    if ((long long)slot >= a.num_slots) {
      if (lane == 0) atomicOr(status, GV_ST_BAD_INDEX);
      return;
    }
    const int kh = kind == 1 ? h - a.nq : h - a.nq - a.nkv;
    dst = (kind == 1 ? a.k_cache : a.v_cache) + ((long long)slot * a.nkv + kh) * a.hd;
  }

  constexpr int MAXE = 8;  // head_dim <= 256
  float v[MAXE];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXE; ++i) {
    const int d = lane + i * 32;
    v[i] = 0.f;
    if (d < a.hd) {
      v[i] = bf2f(src[d]);
      if (bsrc) v[i] = bf2f(f2bf(v[i] + bf2f(bsrc[d])));
      ss += v[i] * v[i];
    }
  }
  if (kind == 2) {
#pragma unroll
    for (int i = 0; i < MAXE; ++i) {
      const int d = lane + i * 32;
      if (d < a.hd) dst[d] = f2bf(v[i]);
    }
    return;
  }
  const bf16* nw = kind == 0 ? a.q_norm_w : a.k_norm_w;
  if (nw) {
    ss = warp_sum(ss);
    const float sc = rsqrtf(ss / (float)a.hd + a.eps);
#pragma unroll
    for (int i = 0; i < MAXE; ++i) {
      const int d = lane + i * 32;
      if (d < a.hd) v[i] = bf2f(f2bf(v[i] * sc * bf2f(nw[d])));
    }
  }
  const float oscale = kind == 0 ? a.q_scale : 1.f;
  const int half = a.rot_dim >> 1;
  // Each lane needs its rotation partner; partners live in other lanes / registers, so stage
  // the head through shared memory (one row per warp).
  extern __shared__ float sh[];
  float* row = sh + (threadIdx.x >> 5) * 256;
#pragma unroll
  for (int i = 0; i < MAXE; ++i) {
    const int d = lane + i * 32;
    if (d < a.hd) row[d] = v[i];
  }
  __syncwarp();
  for (int d = lane; d < a.hd; d += 32) {
    float o;
    int od = d;
    if (d < a.rot_dim) {
      int pair, is_hi;
      float x1, x2;
      if (a.interleaved) {
        pair = d >> 1;
        is_hi = d & 1;
        x1 = row[pair * 2];
        x2 = row[pair * 2 + 1];
        od = is_hi ? half + pair : pair;
      } else {
        is_hi = d >= half;
        pair = is_hi ? d - half : d;
        x1 = row[pair];
        x2 = row[pair + half];
      }
      const int prow = mrope_row(a, pair);
      long long pos = a.positions[(long long)prow * a.tokens + t];
      if (pos < 0 || pos >= a.max_pos) {
        if (lane == 0) atomicOr(status, GV_ST_BAD_INDEX);
        pos = 0;
      }
      const float c = a.cos_sin[pos * a.rot_dim + pair];
      const float s = a.cos_sin[pos * a.rot_dim + half + pair];
      o = is_hi ? (x2 * c + x1 * s) : (x1 * c - x2 * s);
    } else {
      o = row[d];
    }
    dst[od] = f2bf(o * oscale);
  }
}

// Register-only variant for head_dim = rot_dim = 128 with NeoX rotation (Llama, Qwen2/3): lane l
// holds elements 4l .. 4l+3 of the head (one 8-byte access each way) and the rotation partner of
// element d, d +- 64, sits 16 lanes away, so the head never goes through shared memory. A long
// prefill chunk launches tokens x heads of these warps; the generic kernel's 2-byte accesses make
// it issue-bound there.
__device__ __forceinline__ void unpack4(const uint2 raw, float* v) {
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

__device__ __forceinline__ uint2 pack4(const float* v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 r;
  r.x = *reinterpret_cast<const unsigned int*>(&lo);
  r.y = *reinterpret_cast<const unsigned int*>(&hi);
  return r;
}

__global__ void rope_kvwrite_hd128_kernel(RopeArgs a, unsigned int* status) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int heads = a.nq + 2 * a.nkv;
  if (gw >= (long long)a.tokens * heads) return;
  const int t = (int)(gw / heads), h = (int)(gw % heads);
  const int kind = h < a.nq ? 0 : (h < a.nq + a.nkv ? 1 : 2);  // q, k, v
  const int d0 = 4 * lane;
  const bf16* src = a.qkv + (long long)t * a.ld + (long long)h * 128 + d0;
  bf16* dst;
  if (kind == 0) {
    dst = a.q_out + ((long long)t * a.nq + h) * 128 + d0;
  } else {
    const int slot = a.slot_mapping ? a.slot_mapping[t] : -1;
    if (slot < 0) return;
    if ((long long)slot >= a.num_slots) {
      if (lane == 0) atomicOr(status, GV_ST_BAD_INDEX);
      return;
    }
    const int kh = kind == 1 ? h - a.nq : h - a.nq - a.nkv;
    dst = (kind == 1 ? a.k_cache : a.v_cache) + ((long long)slot * a.nkv + kh) * 128 + d0;
  }
  float v[4];
  unpack4(*reinterpret_cast<const uint2*>(src), v);
  if (a.bias) {
    float b[4];
    unpack4(*reinterpret_cast<const uint2*>(a.bias + (long long)h * 128 + d0), b);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = bf2f(f2bf(v[j] + b[j]));
  }
  if (kind == 2) {
    *reinterpret_cast<uint2*>(dst) = pack4(v);
    return;
  }
  const bf16* nw = kind == 0 ? a.q_norm_w : a.k_norm_w;
  if (nw) {
    float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    ss = warp_sum(ss);
    const float sc = rsqrtf(ss / 128.f + a.eps);
    float w[4];
    unpack4(*reinterpret_cast<const uint2*>(nw + d0), w);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = bf2f(f2bf(v[j] * sc * w[j]));
  }
  const bool is_hi = lane >= 16;
  const int pair0 = 4 * (lane & 15);
  float c[4], s[4];
  if (a.mrope_mode == 0) {
    long long pos = a.positions[t];
    if (pos < 0 || pos >= a.max_pos) {
      if (lane == 0) atomicOr(status, GV_ST_BAD_INDEX);
      pos = 0;
    }
    const float4 c4 = *reinterpret_cast<const float4*>(a.cos_sin + pos * 128 + pair0);
    const float4 s4 = *reinterpret_cast<const float4*>(a.cos_sin + pos * 128 + 64 + pair0);
    c[0] = c4.x; c[1] = c4.y; c[2] = c4.z; c[3] = c4.w;
    s[0] = s4.x; s[1] = s4.y; s[2] = s4.z; s[3] = s4.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int prow = mrope_row(a, pair0 + j);
      long long pos = a.positions[(long long)prow * a.tokens + t];
      if (pos < 0 || pos >= a.max_pos) {
        atomicOr(status, GV_ST_BAD_INDEX);
        pos = 0;
      }
      c[j] = a.cos_sin[pos * 128 + pair0 + j];
      s[j] = a.cos_sin[pos * 128 + 64 + pair0 + j];
    }
  }
  const float oscale = kind == 0 ? a.q_scale : 1.f;
  float o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
    // low half: x1 = own, x2 = partner -> x1 c - x2 s; high half: x1 = partner, x2 = own -> x2 c + x1 s
    o[j] = (is_hi ? (v[j] * c[j] + other * s[j]) : (v[j] * c[j] - other * s[j])) * oscale;
  }
  *reinterpret_cast<uint2*>(dst) = pack4(o);
}

// Row-tiled variant of the 128-wide kernel for long chunks: one warp per token walks all of the
// token's heads, so the token's position, its cos / sin values (1 KB, four times the bytes of a
// head) and its cache slot are fetched once per token instead of once per head. Lane layout,
// rounding and rotation are those of `rope_kvwrite_hd128_kernel`. Used for chunks of 256 tokens or
// more (80 us against 97 us on 8192 tokens x 48 heads); GVIRT_ROPE_ROWS=0 turns it off.
__global__ void rope_kvwrite_hd128_rows_kernel(RopeArgs a, unsigned int* status) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= a.tokens) return;
  const int d0 = 4 * lane;
  const bool is_hi = lane >= 16;
  const int pair0 = 4 * (lane & 15);
  float c[4], s[4];
  if (a.mrope_mode == 0) {
    long long pos = a.positions[t];
    if (pos < 0 || pos >= a.max_pos) {
      if (lane == 0) atomicOr(status, GV_ST_BAD_INDEX);
      pos = 0;
    }
    const float4 c4 = *reinterpret_cast<const float4*>(a.cos_sin + pos * 128 + pair0);
    const float4 s4 = *reinterpret_cast<const float4*>(a.cos_sin + pos * 128 + 64 + pair0);
    c[0] = c4.x; c[1] = c4.y; c[2] = c4.z; c[3] = c4.w;
    s[0] = s4.x; s[1] = s4.y; s[2] = s4.z; s[3] = s4.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int prow = mrope_row(a, pair0 + j);
      long long pos = a.positions[(long long)prow * a.tokens + t];
      if (pos < 0 || pos >= a.max_pos) {
        atomicOr(status, GV_ST_BAD_INDEX);
        pos = 0;
      }
      c[j] = a.cos_sin[pos * 128 + pair0 + j];
      s[j] = a.cos_sin[pos * 128 + 64 + pair0 + j];
    }
  }
  int slot = a.slot_mapping ? a.slot_mapping[t] : -1;
  if ((long long)slot >= a.num_slots) {
    if (lane == 0) atomicOr(status, GV_ST_BAD_INDEX);
    slot = -1;
  }
  float qw[4], kw[4];
  if (a.q_norm_w) unpack4(*reinterpret_cast<const uint2*>(a.q_norm_w + d0), qw);
  if (a.k_norm_w) unpack4(*reinterpret_cast<const uint2*>(a.k_norm_w + d0), kw);
  const int heads = a.nq + 2 * a.nkv;
  const bf16* row = a.qkv + t * a.ld + d0;
#pragma unroll 4
  for (int h = 0; h < heads; ++h) {
    const int kind = h < a.nq ? 0 : (h < a.nq + a.nkv ? 1 : 2);  // q, k, v (uniform over the warp)
    if (kind != 0 && slot < 0) break;                             // no cache slot: k and v are not kept
    bf16* dst;
    if (kind == 0) {
      dst = a.q_out + (t * a.nq + h) * 128 + d0;
    } else {
      const int kh = kind == 1 ? h - a.nq : h - a.nq - a.nkv;
      dst = (kind == 1 ? a.k_cache : a.v_cache) + ((long long)slot * a.nkv + kh) * 128 + d0;
    }
    float v[4];
    unpack4(*reinterpret_cast<const uint2*>(row + (long long)h * 128), v);
    if (a.bias) {
      float b[4];
      unpack4(*reinterpret_cast<const uint2*>(a.bias + (long long)h * 128 + d0), b);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = bf2f(f2bf(v[j] + b[j]));
    }
    if (kind == 2) {
      *reinterpret_cast<uint2*>(dst) = pack4(v);
      continue;
    }
    const bool normed = kind == 0 ? a.q_norm_w != nullptr : a.k_norm_w != nullptr;
    if (normed) {
      float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
      ss = warp_sum(ss);
      const float sc = rsqrtf(ss / 128.f + a.eps);
      const float* w = kind == 0 ? qw : kw;
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = bf2f(f2bf(v[j] * sc * w[j]));
    }
    const float oscale = kind == 0 ? a.q_scale : 1.f;
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
      o[j] = (is_hi ? (v[j] * c[j] + other * s[j]) : (v[j] * c[j] - other * s[j])) * oscale;
    }
    *reinterpret_cast<uint2*>(dst) = pack4(o);
  }
}

}  // namespace gv

using namespace gv;

extern "C" int gv_rope_kvwrite(void* qkv, const void* bias, const void* q_norm_w,
                               const void* k_norm_w, const void* cos_sin, const void* positions,
                               const void* slot_mapping, void* k_cache, void* v_cache, void* q_out,
                               long long tokens, long long nq, long long nkv, long long hd,
                               long long rot_dim, long long ld, float q_scale, float eps,
                               long long max_pos, long long num_slots, long long mrope_mode,
                               long long sec0, long long sec1, long long sec2,
                               long long interleaved, void* stream) {
  if (!qkv || !cos_sin || !positions || !q_out) return GV_EINVAL;
  if (hd > 256 || hd <= 0 || rot_dim > hd || (rot_dim & 1)) return GV_EINVAL;
  if (nkv > 0 && (!k_cache || !v_cache)) return GV_EINVAL;
  if (tokens == 0) return GV_OK;
  RopeArgs a;
  a.qkv = (bf16*)qkv;
  a.bias = (const bf16*)bias;
  a.q_norm_w = (const bf16*)q_norm_w;
  a.k_norm_w = (const bf16*)k_norm_w;
  a.cos_sin = (const float*)cos_sin;
  a.positions = (const long long*)positions;
  a.slot_mapping = (const int*)slot_mapping;
  a.k_cache = (bf16*)k_cache;
  a.v_cache = (bf16*)v_cache;
  a.q_out = (bf16*)q_out;
  a.tokens = (int)tokens;
  a.nq = (int)nq;
  a.nkv = (int)nkv;
  a.hd = (int)hd;
  a.rot_dim = (int)rot_dim;
  a.ld = ld;
  a.q_scale = q_scale;
  a.eps = eps;
  a.max_pos = (int)max_pos;
  a.num_slots = num_slots;
  a.mrope_mode = (int)mrope_mode;
  a.sec0 = (int)sec0;
  a.sec1 = (int)sec1;
  a.sec2 = (int)sec2;
  a.interleaved = (int)interleaved;
  const int warps = 8;
  const long long work = tokens * (nq + 2 * nkv);
  dim3 grid((unsigned)((work + warps - 1) / warps));
  auto al = [](const void* p, uintptr_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; };
  static const bool fast_ok = [] {
    const char* e = getenv("GVIRT_DISABLE_ROPE_FAST");
    return !(e && e[0] && e[0] != '0');
  }();
  if (fast_ok && hd == 128 && rot_dim == 128 && !interleaved && (ld & 3) == 0 && al(qkv, 8) && al(q_out, 8) &&
      al(k_cache, 8) && al(v_cache, 8) && al(bias, 8) && al(q_norm_w, 8) && al(k_norm_w, 8) && al(cos_sin, 16)) {
    static const bool rows_on = [] {
      const char* e = getenv("GVIRT_ROPE_ROWS");
      return !(e && e[0] == '0');
    }();
    if (rows_on && tokens >= 256) {
      const int wpb = 4;   // one warp per token
      launch_pdl(rope_kvwrite_hd128_rows_kernel, dim3((unsigned)((tokens + wpb - 1) / wpb)), dim3(wpb * 32), 0,
                 (cudaStream_t)stream, a, status_word());
      return check_launch("gv_rope_kvwrite");
    }
    launch_pdl(rope_kvwrite_hd128_kernel, grid, dim3(warps * 32), 0, (cudaStream_t)stream, a, status_word());
    return check_launch("gv_rope_kvwrite");
  }
  launch_pdl(rope_kvwrite_kernel, grid, dim3(warps * 32), warps * 256 * sizeof(float),
             (cudaStream_t)stream, a, status_word());
  return check_launch("gv_rope_kvwrite");
}

// Expert-parallel MoE dispatch / combine over the symmetric heap (all-to-all fused with routing).
//
// Reference dataflow (xlite/csrc/model.cpp:1089-1207, A2A mode): permutation over all experts ->
// all-gather of per-expert counts -> `experts_counts_sum` -> device-to-host copy + host
// synchronisation -> host prefix sums -> HcclAlltoAllV -> `reorder_moe` (source-major ->
// expert-major) -> grouped GEMMs -> `reorder_moe` back -> HcclAlltoAllV -> unpermutation.
// Default mode instead all-gathers packed [hidden | weights | routing] over the DP group and
// reduce-scatters the result (model.cpp:889-1013).
//
// Here nothing goes through the host, there is no count exchange and no reorder pass:
//   dispatch (token rank): for every (token, k) pair the sender claims a row in the destination
//            rank's region of that expert with one remote atomic (`atomicAdd` at system scope on the
//            owner's per-expert counter), then writes the row there over NVLink — bf16, or e4m3 plus
//            per-128-column scales quantised on the fly — together with its return address
//            (source rank, pair index). Rows therefore land expert-major, ready for the grouped
//            GEMM. The last CTA publishes flag[src = me] = generation on every destination.
//   prepare  (expert rank): bounded wait for the R flags; counters -> row segments; counters reset.
//   combine  (expert rank): each down-projection row is written to `ret[pair]` on its source rank.
//   gather   (token rank): bounded wait for the R flags, then out[t] = sum_k w[t,k] * ret[t*K + k]
//            in fixed k order (row arrival order never affects the result).
// No double buffering is needed: a rank starts the next dispatch only after it has received the
// combine flags of the current one from every expert rank, i.e. after they finished reading.
// Expert regions have a fixed capacity; rows beyond it are dropped and GV_ST_OVERFLOW is raised
// (the reference sizes its buffer by XLITE_ACTIVE_TOKENS_RATIO_PER_EP and device-asserts,
// xlite/csrc/model.cpp:947-951, kernels/permutation.cpp:119).
#include "common.cuh"
#include "gvirt_kernels.h"

namespace gv {

constexpr int A2A_MAX_RANKS = 16;

struct A2AArgs {
  void* const* peers;      // device array [R] of slab bases (EP group)
  long long x_off;         // rows    [e_local][cap][row_bytes]
  long long scale_off;     // scales  [H/128][e_local*cap] fp32 (fp8 mode)
  long long meta_off;      // int32   [e_local*cap]  (src_rank << 24 | pair index)
  long long cnt_off;       // int32   [e_local] claim counters
  long long ret_off;       // bf16    [pairs_cap][H] rows returned to this rank
  long long flag_off;      // uint32  [2 kinds][16]
  unsigned int* state;     // local {generation, ticket}
  unsigned int* status;
  int rank, R, cap, H, e_local, fp8;
};

__device__ __forceinline__ char* slab(const A2AArgs& a, int r) { return static_cast<char*>(a.peers[r]); }

// One CTA per token: quantise once (fp8 mode), then claim + write one row per selected expert.
__global__ void __launch_bounds__(256)
a2a_dispatch_kernel(const bf16* __restrict__ x, const int* __restrict__ ids, int* __restrict__ row_of,
                    int T, int K, A2AArgs a) {
  extern __shared__ __align__(16) unsigned char srow[];  // fp8 mode: H bytes + H/128 floats
  __shared__ int s_slot;
  __shared__ bool s_last;
  const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]) + 1u;
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (t < T) {
    const bf16* src = x + (long long)t * a.H;
    float* sscale = reinterpret_cast<float*>(srow + a.H);
    if (a.fp8) {
      for (int g = warp; g < a.H / 128; g += nwarps) {
        const uint2 raw = *reinterpret_cast<const uint2*>(src + g * 128 + lane * 4);
        const bf162* h = reinterpret_cast<const bf162*>(&raw);
        const float2 p = __bfloat1622float2(h[0]), q = __bfloat1622float2(h[1]);
        float v[4] = {p.x, p.y, q.x, q.y};
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        amax = fmaxf(warp_max(amax), 1e-10f);
        const float scale = amax / 448.f;
        __nv_fp8_e4m3 o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = __nv_fp8_e4m3(__fdiv_rn(v[j], scale));
        *reinterpret_cast<uint32_t*>(srow + g * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(o);
        if (lane == 0) sscale[g] = scale;
      }
    }
    const long long rb = a.fp8 ? a.H : 2LL * a.H;
    for (int k = 0; k < K; ++k) {
      const int i = t * K + k;
      const int e = ids[i];
      const int d = e / a.e_local, le = e % a.e_local;
      __syncthreads();
      if (threadIdx.x == 0) {
        int slot = -1;
        if (e >= 0 && d < a.R)
          slot = atomicAdd_system(reinterpret_cast<int*>(slab(a, d) + a.cnt_off) + le, 1);
        if (slot >= a.cap) {
          atomicOr(a.status, GV_ST_OVERFLOW);
          slot = -1;
        }
        s_slot = slot;
        row_of[i] = slot >= 0 ? i : -1;
      }
      __syncthreads();
      const int slot = s_slot;
      if (slot < 0) continue;
      const long long r = (long long)le * a.cap + slot;
      char* dst = slab(a, d) + a.x_off + r * rb;
      if (a.fp8) {
        for (int c = threadIdx.x * 16; c < a.H; c += blockDim.x * 16)
          *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(srow + c);
        float* sdst = reinterpret_cast<float*>(slab(a, d) + a.scale_off) + r;
        const long long lds = (long long)a.e_local * a.cap;
        for (int g = threadIdx.x; g < a.H / 128; g += blockDim.x) sdst[g * lds] = sscale[g];
      } else {
        for (int c = threadIdx.x * 8; c < a.H; c += blockDim.x * 8)
          *reinterpret_cast<uint4*>(dst + 2LL * c) = *reinterpret_cast<const uint4*>(src + c);
      }
      if (threadIdx.x == 0)
        reinterpret_cast<int*>(slab(a, d) + a.meta_off)[r] = (a.rank << 24) | i;
    }
  }
  // ---- last CTA publishes the dispatch flags and advances the generation
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&a.state[1], 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    if ((int)threadIdx.x < a.R) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<unsigned int*>(slab(a, threadIdx.x) + a.flag_off) + a.rank, gen);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      a.state[1] = 0;
      __threadfence();
      a.state[0] = gen;
    }
  }
}

// Expert side: wait for every source rank, snapshot + reset the counters, emit the segments.
__global__ void a2a_recv_prepare_kernel(int* __restrict__ seg_start, int* __restrict__ seg_end, A2AArgs a) {
  const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]);
  const int s = threadIdx.x;
  if (s < a.R) {
    const unsigned int* f = reinterpret_cast<const unsigned int*>(slab(a, a.rank) + a.flag_off) + s;
    if (!wait_ge_sys(f, gen, peer_budget(a.status))) atomicOr(a.status, GV_ST_TIMEOUT_PEER);
  }
  __syncthreads();
  int* cnt = reinterpret_cast<int*>(slab(a, a.rank) + a.cnt_off);
  for (int e = s; e < a.e_local; e += blockDim.x) {
    int c = *reinterpret_cast<volatile int*>(cnt + e);
    if (c > a.cap) c = a.cap;
    if (c < 0) c = 0;
    seg_start[e] = e * a.cap;
    seg_end[e] = e * a.cap + c;
    cnt[e] = 0;
  }
}

// Expert side: every valid row goes back to ret[pair] on its source rank.
__global__ void a2a_combine_push_kernel(const bf16* __restrict__ ys, const int* __restrict__ seg_end,
                                        A2AArgs a) {
  __shared__ bool s_last;
  const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]);
  const long long total_rows = (long long)a.e_local * a.cap;
  const int* meta = reinterpret_cast<const int*>(slab(a, a.rank) + a.meta_off);
  // live rows only: expert e owns slots [e * cap, seg_end[e])
  for (int e = 0; e < a.e_local; ++e)
  for (long long r = (long long)e * a.cap + blockIdx.x, rend = min((long long)seg_end[e], total_rows);
       r < rend; r += gridDim.x) {
    const int m = *reinterpret_cast<const volatile int*>(meta + r);
    const int src = (m >> 24) & 0xff, pair = m & 0xffffff;
    if (src >= a.R) {
      if (threadIdx.x == 0) atomicOr(a.status, GV_ST_BAD_INDEX);
      continue;
    }
    bf16* dst = reinterpret_cast<bf16*>(slab(a, src) + a.ret_off) + (long long)pair * a.H;
    const bf16* s = ys + r * a.H;
    for (int c = threadIdx.x * 8; c < a.H; c += blockDim.x * 8)
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(s + c);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&a.state[1], 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    if ((int)threadIdx.x < a.R) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<unsigned int*>(slab(a, threadIdx.x) + a.flag_off) + A2A_MAX_RANKS + a.rank,
                     gen);
    }
    __syncthreads();
    if (threadIdx.x == 0) a.state[1] = 0;
  }
}

// Token side: wait for every expert rank's combine flag.
__global__ void a2a_combine_wait_kernel(A2AArgs a) {
  const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]);
  const int s = threadIdx.x;
  if (s < a.R) {
    const unsigned int* f =
        reinterpret_cast<const unsigned int*>(slab(a, a.rank) + a.flag_off) + A2A_MAX_RANKS + s;
    if (!wait_ge_sys(f, gen, peer_budget(a.status))) atomicOr(a.status, GV_ST_TIMEOUT_PEER);
  }
}

}  // namespace gv

using namespace gv;

// offs: host array of 6 byte offsets {x, scale, meta, cnt, ret, flag}; dims: {rank, R, cap, H, e_local, fp8}
static A2AArgs make_args(const void* peers, const long long* offs, void* state, const long long* dims) {
  A2AArgs a;
  a.peers = (void* const*)peers;
  a.x_off = offs[0];
  a.scale_off = offs[1];
  a.meta_off = offs[2];
  a.cnt_off = offs[3];
  a.ret_off = offs[4];
  a.flag_off = offs[5];
  a.state = (unsigned int*)state;
  a.status = status_word();
  a.rank = (int)dims[0];
  a.R = (int)dims[1];
  a.cap = (int)dims[2];
  a.H = (int)dims[3];
  a.e_local = (int)dims[4];
  a.fp8 = (int)dims[5];
  return a;
}

// Token side. x [T, H] bf16, ids [T, K] int32 (global expert ids), row_of int32 [T, K] (out: pair
// index or -1 when dropped).
extern "C" int gv_moe_a2a_dispatch(const void* x, const void* ids, void* row_of, long long T,
                                   long long K, const void* peers, const void* offs, void* state,
                                   const void* dims, void* stream) {
  if (!peers || !offs || !state || !dims) return GV_EINVAL;
  if (T > 0 && (!x || !ids || !row_of)) return GV_EINVAL;
  A2AArgs a = make_args(peers, (const long long*)offs, state, (const long long*)dims);
  if (a.R > A2A_MAX_RANKS || (a.H & 127) || T * K >= (1 << 24)) return GV_EINVAL;
  // at least one CTA runs so that flags are published even when this rank has no tokens
  const int grid = (int)(T > 0 ? T : 1);
  const size_t smem = a.fp8 ? (size_t)(a.H + (a.H / 128) * 4 + 16) : 16;
  a2a_dispatch_kernel<<<grid, 256, smem, (cudaStream_t)stream>>>((const bf16*)x, (const int*)ids,
                                                                 (int*)row_of, (int)T, (int)K, a);
  return check_launch("gv_moe_a2a_dispatch");
}

// Expert side: seg_start / seg_end int32 [e_local] (rows of the region [e_local * cap]).
extern "C" int gv_moe_a2a_recv_prepare(void* seg_start, void* seg_end, const void* peers,
                                       const void* offs, void* state, const void* dims, void* stream) {
  if (!seg_start || !seg_end || !peers || !offs || !state || !dims) return GV_EINVAL;
  A2AArgs a = make_args(peers, (const long long*)offs, state, (const long long*)dims);
  a2a_recv_prepare_kernel<<<1, 256, 0, (cudaStream_t)stream>>>((int*)seg_start, (int*)seg_end, a);
  return check_launch("gv_moe_a2a_recv_prepare");
}

extern "C" int gv_moe_a2a_combine_push(const void* ys, const void* seg_end, const void* peers,
                                       const void* offs, void* state, const void* dims, void* stream) {
  if (!ys || !seg_end || !peers || !offs || !state || !dims) return GV_EINVAL;
  A2AArgs a = make_args(peers, (const long long*)offs, state, (const long long*)dims);
  long long grid = (long long)a.e_local * a.cap;
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid < 1) grid = 1;
  int threads = (int)min((long long)256, ((long long)a.H / 8 + 31) / 32 * 32);
  a2a_combine_push_kernel<<<(unsigned)grid, threads, 0, (cudaStream_t)stream>>>((const bf16*)ys,
                                                                                (const int*)seg_end, a);
  return check_launch("gv_moe_a2a_combine_push");
}

extern "C" int gv_moe_a2a_combine_wait(const void* peers, const void* offs, void* state,
                                       const void* dims, void* stream) {
  if (!peers || !offs || !state || !dims) return GV_EINVAL;
  A2AArgs a = make_args(peers, (const long long*)offs, state, (const long long*)dims);
  a2a_combine_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a);
  return check_launch("gv_moe_a2a_combine_wait");
}

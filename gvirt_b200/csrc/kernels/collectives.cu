// Stand-alone collectives over the symmetric heap: all-reduce (one-shot and two-shot),
// all-gather and reduce-scatter, for bf16 and fp32 payloads.
//
// Reference: the XCCL kernels `allreduce_<T>` / `allgather_<T>` / `reduce_scatter_<T>`
// (xlite/csrc/kernels/all_reduce.cpp:366-384, all_gather.cpp:203-270, reduce_scatter.cpp:202-287):
// one-sided pulls over IPC-mapped peer pools, generation flags, bf16 atomic adds, unbounded spins.
// This design keeps the one-sided pull but
//   * works chunk by chunk: CTA c stages chunk c, raises flag (c, my rank) on every peer with a
//     system-scope release store, waits (bounded) for flag (c, p) from every peer p and then pulls
//     chunk c from all peers — no grid-wide barrier, transfers of different chunks overlap;
//   * reduces in rank order with fp32 accumulation => bitwise reproducible, no atomics;
//   * is CUDA-graph replay safe: the generation comes from a device-side counter that the last
//     CTA of a launch advances, not from a host argument; staging is double-buffered by the
//     generation's parity, which is enough because a rank cannot start launch g+2 on a channel
//     before every peer has finished reading launch g (see parallel/symm.py);
//   * every wait is bounded and reports GV_ST_TIMEOUT_PEER instead of hanging.
//
// Symmetric slab layout (same offsets on every rank): flag words `flags_off + (cta * 16 + src) * 4`
// (+ a second bank for the two-shot all-gather phase) and `stage_off + parity * stage_stride`.
#include "common.cuh"
#include "gvirt_kernels.h"

namespace gv {

constexpr int COLL_MAX_RANKS = 16;
constexpr int COLL_THREADS = 512;

// 16-byte load that is coherent at system scope (peer memory must not be served from a stale
// L1 line of this SM).
__device__ __forceinline__ uint4 ld_sys16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <typename T>
struct Vec16;
template <>
struct Vec16<bf16> {
  static constexpr int N = 8;
  __device__ static void load(const bf16* p, float* f) {
    const uint4 v = ld_sys16(p);
    unpack8(*reinterpret_cast<const bf16x8*>(&v), f);
  }
  __device__ static void store(bf16* p, const float* f) { st8(p, pack8(f)); }
};
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* f) {
    const uint4 v = ld_sys16(p);
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static void store(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

struct CollArgs {
  void* const* peers;      // device array [R]: base address of every rank's symmetric slab
  long long flags_off;     // byte offset of this channel's flag words
  long long stage_off;     // byte offset of this channel's staging area
  long long stage_stride;  // bytes per parity buffer
  unsigned int* state;     // local: {generation, finished-CTA ticket}
  unsigned int* status;
  int rank, R;
};

__device__ __forceinline__ unsigned int* flag_ptr(const CollArgs& a, int peer, int bank, int cta,
                                                  int src) {
  return reinterpret_cast<unsigned int*>(static_cast<char*>(a.peers[peer]) + a.flags_off) +
         ((size_t)bank * gridDim.x + cta) * COLL_MAX_RANKS + src;
}

// Raise flag (bank, cta, my rank) = gen on every peer, then wait for every peer's flag here.
__device__ __forceinline__ void exchange_flags(const CollArgs& a, int bank, unsigned int gen) {
  __syncthreads();
  if ((int)threadIdx.x < a.R) {
    __threadfence_system();
    st_release_sys(flag_ptr(a, threadIdx.x, bank, blockIdx.x, a.rank), gen);
    if (!wait_ge_sys(flag_ptr(a, a.rank, bank, blockIdx.x, threadIdx.x), gen, peer_budget(a.status)))
      atomicOr(a.status, GV_ST_TIMEOUT_PEER);
  }
  __syncthreads();
}

__device__ __forceinline__ void finish_launch(const CollArgs& a, unsigned int gen) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&a.state[1], 1u) == gridDim.x - 1) {
      a.state[1] = 0;
      __threadfence();
      a.state[0] = gen;  // the next launch on this stream sees the advanced generation
    }
  }
}

// mode 0: all-reduce one-shot   x[n] -> out[n]
// mode 1: all-gather            x[n] -> out[R * n]
// mode 2: reduce-scatter        x[R * n] -> out[n]   (rank r keeps slice r)
// mode 3: all-reduce two-shot   x[R * n] -> out[R * n] (reduce-scatter, then all-gather)
template <typename T>
__global__ void __launch_bounds__(COLL_THREADS)
collective_kernel(int mode, const T* __restrict__ x, T* __restrict__ out, long long n, CollArgs a) {
  constexpr int V = Vec16<T>::N;
  __shared__ unsigned int s_gen;
  if (threadIdx.x == 0) s_gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]) + 1u;
  __syncthreads();
  const unsigned int gen = s_gen;
  const long long total_in = (mode == 2 || mode == 3) ? n * a.R : n;
  char* my_slab = static_cast<char*>(a.peers[a.rank]);
  T* my_stage = reinterpret_cast<T*>(my_slab + a.stage_off + (gen & 1u) * a.stage_stride);
  // chunking is over vectors of the *per-slice* length n so that chunk c of every slice lines up
  const long long nvec = (n + V - 1) / V;
  const long long per = (nvec + gridDim.x - 1) / gridDim.x;
  const long long v0 = blockIdx.x * per, v1 = min(nvec, v0 + per);
  const int slices_in = (mode == 2 || mode == 3) ? a.R : 1;

  // 1) stage my input chunk(s)
  for (int s = 0; s < slices_in; ++s)
    for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      const long long i = s * n + v * V;
      if (v * V + V <= n) {
        *reinterpret_cast<uint4*>(my_stage + i) = *reinterpret_cast<const uint4*>(x + i);
      } else {
        for (int j = 0; j < V && v * V + j < n; ++j) my_stage[i + j] = x[i + j];
      }
    }
  exchange_flags(a, 0, gen);

  const T* peer_stage[COLL_MAX_RANKS];
#pragma unroll
  for (int p = 0; p < COLL_MAX_RANKS; ++p)
    peer_stage[p] = p < a.R ? reinterpret_cast<const T*>(static_cast<char*>(a.peers[p]) +
                                                        a.stage_off + (gen & 1u) * a.stage_stride)
                            : nullptr;

  if (mode == 0 || mode == 2 || mode == 3) {
    // 2) reduce (my slice for RS / two-shot, the whole chunk for one-shot) in rank order
    const long long base = (mode == 0) ? 0 : (long long)a.rank * n;
    T* red_dst = (mode == 3) ? my_stage + (long long)a.R * n + base  // second half of the stage
                             : out;
    for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      const long long i = v * V;
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      if (i + V <= n) {
        for (int p = 0; p < a.R; ++p) {
          float f[V];
          Vec16<T>::load(peer_stage[p] + base + i, f);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += f[j];
        }
        Vec16<T>::store(red_dst + i, acc);
      } else {
        for (int j = 0; j < V && i + j < n; ++j) {
          float s = 0.f;
          for (int p = 0; p < a.R; ++p) s += (float)peer_stage[p][base + i + j];
          red_dst[i + j] = (T)s;
        }
      }
    }
    if (mode == 3) {
      // 3) all-gather the reduced slices: chunk c of slice p was produced by peer p's CTA c
      exchange_flags(a, 1, gen);
      for (int p = 0; p < a.R; ++p) {
        const T* src = peer_stage[p] + (long long)a.R * n + (long long)p * n;
        for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
          const long long i = v * V;
          if (i + V <= n) {
            *reinterpret_cast<uint4*>(out + (long long)p * n + i) = ld_sys16(src + i);
          } else {
            for (int j = 0; j < V && i + j < n; ++j) out[(long long)p * n + i + j] = src[i + j];
          }
        }
      }
    }
  } else {
    // all-gather: pull chunk c of every peer
    for (int p = 0; p < a.R; ++p) {
      for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
        const long long i = v * V;
        if (i + V <= n) {
          *reinterpret_cast<uint4*>(out + (long long)p * n + i) = ld_sys16(peer_stage[p] + i);
        } else {
          for (int j = 0; j < V && i + j < n; ++j) out[(long long)p * n + i + j] = peer_stage[p][i + j];
        }
      }
    }
  }
  finish_launch(a, gen);
}

// ------------------------------------------------------------------------------------------
// Low-latency variants for small payloads (modes 4 = all-reduce, 5 = all-gather, 6 =
// reduce-scatter). Instead of stage + fence + flag + pull (two NVLink round trips), every rank
// PUSHES its payload straight into the peers' receive regions in 16-byte lines
// {payload lo, generation, payload hi, generation}: each 8-byte half is single-copy atomic, so a
// receiver that polls a line and finds the current generation in both halves has the payload.
// One one-way NVLink trip, no system-scope fence, no flag words. Costs 2x the bytes on the wire,
// which is irrelevant below ~1 MiB. Receive region: [parity][source rank][line], line = 8 bytes
// of the slice. Sums run in rank order with fp32 accumulation (own slice read from `x`).
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
template <typename T>
__device__ __forceinline__ void acc_line(float* acc, uint32_t lo, uint32_t hi);
template <>
__device__ __forceinline__ void acc_line<bf16>(float* acc, uint32_t lo, uint32_t hi) {
  const bf162 a = *reinterpret_cast<const bf162*>(&lo), b = *reinterpret_cast<const bf162*>(&hi);
  acc[0] += __low2float(a); acc[1] += __high2float(a);
  acc[2] += __low2float(b); acc[3] += __high2float(b);
}
template <>
__device__ __forceinline__ void acc_line<float>(float* acc, uint32_t lo, uint32_t hi) {
  acc[0] += __uint_as_float(lo);
  acc[1] += __uint_as_float(hi);
}
template <typename T>
__device__ __forceinline__ uint2 pack_line(const float* acc);
template <>
__device__ __forceinline__ uint2 pack_line<bf16>(const float* acc) {
  return make_uint2(pack_bf2(acc[0], acc[1]), pack_bf2(acc[2], acc[3]));
}
template <>
__device__ __forceinline__ uint2 pack_line<float>(const float* acc) {
  return make_uint2(__float_as_uint(acc[0]), __float_as_uint(acc[1]));
}

// L = 8-byte lines per slice. mode 4: x has L lines, out L. mode 5: x L, out R * L.
// mode 6: x R * L (slice p goes to rank p), out L. mode 7: all-reduce in two hops — warp-sized
// groups of lines are owned round-robin by the ranks; a rank sends a line only to its owner, the
// owner sums the R copies in rank order and pushes the result to everybody's final region
// (2 (R - 1) / R of a message per rank instead of R - 1 messages; used from 4 ranks on).
// Receive region per parity: [R sources + 1 final][l_cap lines].
template <typename T>
__global__ void __launch_bounds__(COLL_THREADS)
collective_ll_kernel(int mode, const uint2* __restrict__ x, uint2* __restrict__ out, long long L,
                     long long l_cap, CollArgs a) {
  __shared__ unsigned int s_gen;
  if (threadIdx.x == 0) s_gen = *reinterpret_cast<volatile unsigned int*>(&a.state[0]) + 1u;
  __syncthreads();
  const unsigned int gen = s_gen;
  const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  const long long par_off = (long long)(gen & 1u) * (a.R + 1) * l_cap;     // in lines
  if (mode == 7) {
    const uint4* base = reinterpret_cast<const uint4*>(static_cast<char*>(a.peers[a.rank]) + a.stage_off) + par_off;
    bool ok = true;
    // hop 1: lines go to their owner
    for (long long l = gtid; l < L; l += gstride) {
      const int own = (int)((l >> 5) % a.R);
      if (own == a.rank) continue;
      const uint2 mine = x[l];
      uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(a.peers[own]) + a.stage_off) + par_off +
                   (long long)a.rank * l_cap + l;
      st_line(dst, mine.x, mine.y, gen);
    }
    // owner: reduce in rank order, keep the result and broadcast it
    for (long long l = gtid; l < L; l += gstride) {
      if ((int)((l >> 5) % a.R) != a.rank) continue;
      uint4 v[COLL_MAX_RANKS];
#pragma unroll
      for (int s = 0; s < COLL_MAX_RANKS; ++s)
        if (s < a.R && s != a.rank) v[s] = ld_line(base + (long long)s * l_cap + l);
      const uint2 own = x[l];
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < COLL_MAX_RANKS; ++s) {
        if (s >= a.R) continue;
        if (s == a.rank) {
          acc_line<T>(acc, own.x, own.y);
        } else {
          if (!wait_line(base + (long long)s * l_cap + l, gen, v[s], ok ? peer_budget(a.status) : 0ull)) ok = false;
          acc_line<T>(acc, v[s].x, v[s].z);
        }
      }
      const uint2 r = pack_line<T>(acc);
      out[l] = r;
      for (int p = 1; p < a.R; ++p) {
        const int peer = (a.rank + p) % a.R;
        uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(a.peers[peer]) + a.stage_off) + par_off +
                     (long long)a.R * l_cap + l;
        st_line(dst, r.x, r.y, gen);
      }
    }
    // hop 2: collect the lines other ranks own
    for (long long l = gtid; l < L; l += gstride) {
      if ((int)((l >> 5) % a.R) == a.rank) continue;
      uint4 v = ld_line(base + (long long)a.R * l_cap + l);
      if (!wait_line(base + (long long)a.R * l_cap + l, gen, v, ok ? peer_budget(a.status) : 0ull)) ok = false;
      out[l] = make_uint2(v.x, v.z);
    }
    if (!ok) atomicOr(a.status, GV_ST_TIMEOUT_PEER);
    finish_launch(a, gen);
    return;
  }
  // ---- push
  for (long long l = gtid; l < L; l += gstride) {
    uint2 mine = mode == 6 ? make_uint2(0, 0) : x[l];
    for (int p = 1; p < a.R; ++p) {
      const int peer = (a.rank + p) % a.R;
      if (mode == 6) mine = x[(long long)peer * L + l];
      uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(a.peers[peer]) + a.stage_off) +
                   par_off + (long long)a.rank * l_cap + l;
      st_line(dst, mine.x, mine.y, gen);
    }
  }
  // ---- receive
  const uint4* base = reinterpret_cast<const uint4*>(static_cast<char*>(a.peers[a.rank]) + a.stage_off) + par_off;
  bool ok = true;
  for (long long l = gtid; l < L; l += gstride) {
    uint4 v[COLL_MAX_RANKS];
#pragma unroll
    for (int s = 0; s < COLL_MAX_RANKS; ++s)
      if (s < a.R && s != a.rank) v[s] = ld_line(base + (long long)s * l_cap + l);
    const uint2 own = mode == 6 ? x[(long long)a.rank * L + l] : x[l];
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < COLL_MAX_RANKS; ++s) {
      if (s >= a.R) continue;
      uint2 d;
      if (s == a.rank) {
        d = own;
      } else {
        if (!wait_line(base + (long long)s * l_cap + l, gen, v[s], ok ? peer_budget(a.status) : 0ull)) ok = false;
        d = make_uint2(v[s].x, v[s].z);
      }
      if (mode == 5) out[(long long)s * L + l] = d;
      else acc_line<T>(acc, d.x, d.y);
    }
    if (mode != 5) out[l] = pack_line<T>(acc);
  }
  if (!ok) atomicOr(a.status, GV_ST_TIMEOUT_PEER);
  finish_launch(a, gen);
}

}  // namespace gv

using namespace gv;

// is_f32: payload dtype (0 = bf16). n = elements per slice (see modes above); every slice start
// must be 16-byte aligned (n * sizeof(T) % 16 == 0 when R > 1 slices are involved).
// Staging need: mode 0/1: n, mode 2: R*n, mode 3: 2*R*n elements per parity buffer.
// Flag need: 2 banks * grid * 16 words. grid must be the same on every rank.
// Modes 4 / 5 / 6 are the low-latency push forms of 0 / 1 / 2 for small payloads and 7 is the
// two-hop push all-reduce: they need stage_stride >= 16 * (R + 1) * ceil(n * esz / 8) bytes per
// parity and no flag words.
extern "C" int gv_collective(long long mode, long long is_f32, const void* x, void* out,
                             long long n, const void* peers, long long flags_off,
                             long long stage_off, long long stage_stride, void* state,
                             long long rank, long long R, long long grid, void* stream) {
  if (!x || !out || !peers || !state || R < 1 || R > COLL_MAX_RANKS || rank < 0 || rank >= R)
    return GV_EINVAL;
  if (mode < 0 || mode > 7 || grid < 1 || grid > 1024) return GV_EINVAL;
  if (n == 0) return GV_OK;
  const long long esz = is_f32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) return GV_EINVAL;
  if (mode >= 4) {
    // low-latency push: n * esz must be a multiple of 8; the receive region holds
    // [R sources + 1 final][l_cap lines of 16 bytes] per parity, l_cap = stage_stride / (16 * (R + 1))
    if ((n * esz) & 7) return GV_EINVAL;
    const long long L = n * esz / 8;
    const long long l_cap = stage_stride / (16 * (R + 1));
    if (L > l_cap) return GV_ETOOBIG;
    CollArgs a;
    a.peers = (void* const*)peers;
    a.flags_off = flags_off;
    a.stage_off = stage_off;
    a.stage_stride = stage_stride;
    a.state = (unsigned int*)state;
    a.status = status_word();
    a.rank = (int)rank;
    a.R = (int)R;
    cudaStream_t st = (cudaStream_t)stream;
    if (is_f32)
      collective_ll_kernel<float><<<(unsigned)grid, COLL_THREADS, 0, st>>>(
          (int)mode, (const uint2*)x, (uint2*)out, L, l_cap, a);
    else
      collective_ll_kernel<bf16><<<(unsigned)grid, COLL_THREADS, 0, st>>>(
          (int)mode, (const uint2*)x, (uint2*)out, L, l_cap, a);
    return check_launch("gv_collective(ll)");
  }
  if (mode != 0 && ((n * esz) & 15)) return GV_EINVAL;
  const long long need = (mode == 0 || mode == 1 ? n : mode == 2 ? R * n : 2 * R * n) * esz;
  if (need > stage_stride) return GV_ETOOBIG;
  CollArgs a;
  a.peers = (void* const*)peers;
  a.flags_off = flags_off;
  a.stage_off = stage_off;
  a.stage_stride = stage_stride;
  a.state = (unsigned int*)state;
  a.status = status_word();
  a.rank = (int)rank;
  a.R = (int)R;
  cudaStream_t st = (cudaStream_t)stream;
  if (is_f32)
    collective_kernel<float><<<(unsigned)grid, COLL_THREADS, 0, st>>>((int)mode, (const float*)x,
                                                                      (float*)out, n, a);
  else
    collective_kernel<bf16><<<(unsigned)grid, COLL_THREADS, 0, st>>>((int)mode, (const bf16*)x,
                                                                     (bf16*)out, n, a);
  return check_launch("gv_collective");
}

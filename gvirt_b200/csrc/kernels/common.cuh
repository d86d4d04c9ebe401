// Shared device/host helpers for every sm_100a kernel in this library.
//
// Conventions used by all entry points (see gvirt_kernels.h):
//   * every exported launcher is `extern "C" int gv_<op>(..., void* stream)` and
//     returns 0 on success or a negative GV_E* code; nothing throws across the C ABI;
//   * integer arguments are `long long`, scalars are `float`, pointers are raw device
//     pointers; the stream is a cudaStream_t passed as void*;
//   * no launcher allocates device memory: scratch is passed in by the caller (the
//     activation arena) so addresses repeat step to step and CUDA graphs can replay.
//   * every device-side wait is bounded (GV_SPIN_LIMIT) and reports through a status
//     word instead of hanging or trapping, so a shared GPU is never wedged.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#define GV_OK 0
#define GV_EINVAL (-1)      // bad argument (shape, alignment, null pointer)
#define GV_ECUDA (-2)       // a CUDA runtime / driver call failed; see gv_last_error()
#define GV_EUNSUPPORTED (-3)
#define GV_ETOOBIG (-4)     // exceeds a compiled-in maximum

// Status word bits written by kernels whose bounded waits ran out.
#define GV_ST_TIMEOUT_TMA 1u
#define GV_ST_TIMEOUT_MMA 2u
#define GV_ST_TIMEOUT_EPI 4u
#define GV_ST_TIMEOUT_PEER 8u
#define GV_ST_OVERFLOW 16u   // MoE receive region overflow (rows dropped, counted)
#define GV_ST_BAD_INDEX 32u  // an index derived from device metadata was out of range

// Every device-side wait gives up after this much wall-clock time (nanoseconds of %globaltimer)
// and additionally after GV_SPIN_LIMIT polls, whichever comes first.
#ifndef GV_WAIT_NS
#define GV_WAIT_NS 2000000000ull
#endif
#ifndef GV_SPIN_LIMIT
#define GV_SPIN_LIMIT (1u << 26)
#endif

namespace gv {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

void set_last_error(const char* what, cudaError_t e);
int check_launch(const char* what);
// Device status word shared by all kernels of this library on the current device.
unsigned int* status_word();
// SM count of the current device (cached per device).
int num_sms();

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Programmatic dependent launch: when on (default; gv_set_pdl(0) turns it off), kernels that
// call pdl_wait() before their first dependent access are launched with the programmatic
// stream-serialisation attribute, so their prologue (barrier set-up, TMEM allocation, weight
// prefetch) overlaps the tail of the kernel in front of them.
bool pdl_enabled();

#ifdef __CUDACC__

// Blocks until every kernel this one depends on has completed and its writes are visible.
// A no-op when the kernel was launched without the programmatic attribute. Nothing produced by
// an earlier kernel may be read, and nothing at all may be written to global memory, before it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel in the stream start its pre-wait prologue once every CTA has got here.
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Launch `kern` with (grid, block, smem, stream); adds the programmatic-serialisation attribute
// when PDL is on. Only for kernels whose every thread calls pdl_wait() first.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float bf2f(bf16 x) { return __bfloat162float(x); }
__device__ __forceinline__ bf16 f2bf(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `red` must hold >= 32 floats of shared memory. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  bf162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

struct alignas(16) bf16x8 {
  bf162 v[4];
};

__device__ __forceinline__ bf16x8 ld8(const bf16* p) { return *reinterpret_cast<const bf16x8*>(p); }
__device__ __forceinline__ void st8(bf16* p, const bf16x8& x) { *reinterpret_cast<bf16x8*>(p) = x; }

__device__ __forceinline__ void unpack8(const bf16x8& x, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(x.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return r;
}

// ---- system-scope signalling over NVLink peer memory (bounded) -----------------------
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_relaxed_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Spin until *p >= want (signed-difference compare on a monotone generation counter) or the
// time budget runs out. Returns false on time-out; never traps, never loops forever.
__device__ __forceinline__ bool wait_ge_sys(const unsigned int* p, unsigned int want,
                                            unsigned long long budget_ns = GV_WAIT_NS) {
  const unsigned long long t0 = global_ns();
  for (unsigned int i = 0; i < GV_SPIN_LIMIT; ++i) {
    if ((int)(ld_acquire_sys(p) - want) >= 0) return true;
    if (i > 64) __nanosleep(64);
    if ((i & 255u) == 255u && global_ns() - t0 > budget_ns) return false;
  }
  return false;
}

// Time budget of a wait on a peer: all of GV_WAIT_NS, or 1 ms once a peer wait on this device has
// already run out (the time-out bit of the status word is up). A peer that is gone then costs one
// full wait per launch, not one per remaining line, tile or flag bank.
__device__ __forceinline__ unsigned long long peer_budget(const unsigned int* status) {
  return (*reinterpret_cast<const volatile unsigned int*>(status) & GV_ST_TIMEOUT_PEER) ? 1000000ull
                                                                                        : GV_WAIT_NS;
}

#endif  // __CUDACC__

}  // namespace gv

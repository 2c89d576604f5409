// Shared helpers of the sm_100a kernels: status plumbing, dtype access,
// bf16 rounding and order-preserving float keys.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <utility>

#include "sah_b200.h"

int sah_fail(int status, const char* fmt, ...);

#define SAH_REQUIRE(cond, ...)                                  \
  do {                                                          \
    if (!(cond)) return sah_fail(SAH_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define SAH_LAUNCH_CHECK(name)                                                     \
  do {                                                                             \
    cudaError_t e__ = cudaGetLastError();                                          \
    if (e__ != cudaSuccess)                                                        \
      return sah_fail(SAH_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e__));      \
  } while (0)

static inline int64_t sah_ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- element access -------------------------------------------------------
template <typename T>
__device__ __forceinline__ float sah_to_float(T v);
template <>
__device__ __forceinline__ float sah_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float sah_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T>
__device__ __forceinline__ T sah_from_float(float v);
template <>
__device__ __forceinline__ float sah_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 sah_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Round a float to the value grid of T (identity for float).
template <typename T>
__device__ __forceinline__ float sah_round_to(float v) {
  return sah_to_float<T>(sah_from_float<T>(v));
}

__device__ __forceinline__ float sah_bf16_bits_to_float(uint32_t b16) {
  return __uint_as_float(b16 << 16);
}
__device__ __forceinline__ uint32_t sah_float_to_bf16_bits(float v) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// Order-preserving map float -> uint32 (larger float => larger key).
__device__ __forceinline__ uint32_t sah_float_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Inverse mask weight 1 / (m + 1e-6), each op rounded to the mask dtype.
template <typename T>
__device__ __forceinline__ float sah_inv_weight(float m) {
  float s = sah_round_to<T>(__fadd_rn(m, 1e-6f));
  return sah_round_to<T>(__frcp_rn(s));  // the correctly rounded reciprocal, as 1.0f / s is
}

// Unpack 8 consecutive elements (16 B for bf16, 32 B for fp32) to floats.
__device__ __forceinline__ void sah_unpack8(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x << 16);
  f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16);
  f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16);
  f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16);
  f[7] = __uint_as_float(v.w & 0xffff0000u);
}

template <typename T>
__device__ __forceinline__ void sah_load8(const T* p, float* f);
template <>
__device__ __forceinline__ void sah_load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  sah_unpack8(v, f);
}
template <>
__device__ __forceinline__ void sah_load8<float>(const float* p, float* f) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// Exclusive scan across the CTA; `total` receives the CTA-wide sum.  `scratch`
// holds 33 values.  Ends with a barrier, so scratch may be reused right away.
template <typename V>
__device__ __forceinline__ V sah_block_excl_scan(V c, V* scratch, V* total) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  V incl = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    V n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    V s = (lane < nwarp) ? scratch[lane] : (V)0;
    V si = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      V n = __shfl_up_sync(0xffffffffu, si, o);
      if (lane >= o) si += n;
    }
    scratch[lane] = si - s;           // exclusive offset of each warp
    if (lane == 31) scratch[32] = si; // CTA total
  }
  __syncthreads();
  V res = scratch[warp] + incl - c;
  *total = scratch[32];
  __syncthreads();
  return res;
}

#define SAH_DISPATCH_DTYPE(dtype, T, ...)                              \
  do {                                                                 \
    if ((dtype) == SAH_F32) {                                          \
      using T = float;                                                 \
      __VA_ARGS__                                                      \
    } else if ((dtype) == SAH_BF16) {                                  \
      using T = __nv_bfloat16;                                         \
      __VA_ARGS__                                                      \
    } else {                                                           \
      return sah_fail(SAH_ERR_INVALID, "unknown dtype %d", (int)(dtype)); \
    }                                                                  \
  } while (0)

// ---- launch accounting and optional per-kernel event timing -------------------
// Slots name the kernels whose device time a caller may want in isolation.
enum SahProfSlot {
  SAH_PROF_ATTENTION = 0,
  SAH_PROF_HASH_TOPK = 1,
  SAH_PROF_HASH_ENCODE = 2,
  SAH_PROF_QK_SCORES = 3,
  SAH_PROF_TOPK_SELECT = 4,
  SAH_PROF_ATTN_PLAN = 5,
  SAH_PROF_ATTN_MERGE = 6,
  SAH_PROF_OTHER = 7,
  SAH_PROF_LSH_MATCH = 8,
  SAH_PROF_LSH_PROB = 9,
  SAH_PROF_PQ_SCORES = 10,
  SAH_PROF_ADAPTIVE = 11,
  SAH_PROF_TOPP = 12,
  SAH_PROF_QUEST = 13,
  SAH_PROF_SLOTS = 16
};
void sah_prof_begin(int slot, cudaStream_t st);
void sah_prof_end(int slot, cudaStream_t st);
void sah_count_launch();

#undef SAH_LAUNCH_CHECK
#define SAH_LAUNCH_CHECK(name)                                                     \
  do {                                                                             \
    sah_count_launch();                                                            \
    cudaError_t e__ = cudaGetLastError();                                          \
    if (e__ != cudaSuccess)                                                        \
      return sah_fail(SAH_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e__));      \
  } while (0)

// ---- chained launches (programmatic dependent launch) -----------------------------
// The kernels of a decode step follow one another in one stream, many of them a few
// microseconds long, so the time between the end of one grid and the first instruction of the
// next is part of the step.  A kernel that begins with sah_pdl_entry() or
// sah_pdl_entry_early() may be launched with sah_launch_chain(): with SAH_PDL=1 in the
// environment the launch carries the programmatic-stream-serialization attribute, the grid may
// be scheduled before the kernel in front of it has finished, and its threads wait, in
// hardware, until the kernels in front have completed and their writes are visible.  Nothing of
// global memory is touched before that wait, so the results are those of ordinary stream
// order; what overlaps is the launch itself.
//   sah_pdl_entry_early(): short kernels.  Also tells the hardware that the kernels behind
//     this one may be scheduled as soon as all its CTAs have started.
//   sah_pdl_entry(): long kernels (scans of all keys, attention).  Their successors are
//     scheduled when they end.
// Every kernel of a chain has to execute the wait (a grid that skipped it could complete, and
// release its own successors, before its predecessor has), which is why the attribute is only
// ever set by sah_launch_chain() and tests/test_c_abi.py checks that every kernel launched
// through it starts with one of the two.  Without the attribute the instructions do nothing.
//
// Measured on B200 (decode step as a CUDA graph, us, chained against plain): Sink+Local 23.1
// / 24.8, HashAttention 94.1 / 96.0, PQCache 95.5 / 97.6, Quest 96.7 / 95.9, oracle top-k
// 211.5 / 209.7, MagicPig at 131072 keys 164.1 / 156.8, oracle top-k + adaptive 345.5 / 346
// (with grids of up to 1024 warps chained; 362 with 4096; and 184 and 373 for the last two
// when every kernel, long ones included, released its successors at its start).  A grid that
// sits waiting beside its predecessor costs that kernel more than the hidden launch saves
// whenever the waiting grid is large or the predecessor long, and the gain where there is one
// is 2 us.  So chaining is off by default.
__device__ __forceinline__ void sah_pdl_entry() {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
}
__device__ __forceinline__ void sah_pdl_entry_early() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

// Grids of more warps than this are launched in plain stream order even with SAH_PDL=1
// (SAH_PDL_MAX_WARPS replaces the 1024); 0 = no chaining at all, the default.
int sah_pdl_max_warps();

template <typename... KArgs, typename... Args>
static inline void sah_launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
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
  const long long warps = (long long)grid.x * grid.y * grid.z * ((block.x * block.y * block.z + 31) / 32);
  cfg.numAttrs = warps <= (long long)sah_pdl_max_warps() ? 1 : 0;
  (void)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);  // the error stays for SAH_LAUNCH_CHECK
}

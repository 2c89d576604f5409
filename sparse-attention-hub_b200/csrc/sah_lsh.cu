// MagicPig: SimHash (LSH) sampling of keys (maskers/sampling/implementations/magic_pig.py).
//
//   sah_lsh_key_sums      per (batch, KV head, channel) sum of the keys in float64 (key mean, :152-183)
//   sah_lsh_key_stats     norm of every centred key and the running maximum norm (:348-353)
//   sah_lsh_key_sign      MIPS transform + random-hyperplane signatures of keys, packed per table (:332-372, :120-150)
//   sah_lsh_query         centred, normalised query, its signatures and its unit vector (:152-183, :332-403)
//   sah_lsh_match         keys that share at least one table code with the query (:455-463)
//   sah_lsh_prob          collision probability of every matched key (:374-403)
//
// Signatures are stored key-major: the L table codes of a key (uint8 for lsh_k <= 8, uint16 for
// lsh_k <= 16) sit side by side in a row padded to a multiple of 16 bytes, rows in key order,
// so that the match kernel reads one contiguous stream per (batch, KV head).  The reference
// repeats keys over the query heads of a group and uses one projection per layer, so the
// signatures of a group's heads are identical and are stored once per KV head.
//
// Reductions over the head dimension use one fixed order ("lane order"): lane t of a warp
// owns the D/32 consecutive channels starting at t*D/32 and sums them in ascending order,
// then the 32 lane sums combine by xor shuffles 16, 8, 4, 2, 1.  Every tensor operation of
// the reference is one rounding to the dtype here.
#include "sah_common.cuh"

#define LSH_MAX_PER_LANE 8  // D <= 256

// codes per signature row: L rounded up so that a row is a multiple of 16 bytes
template <typename CodeT>
__host__ __device__ __forceinline__ int lsh_row_pitch(int L) {
  const int per16 = 16 / (int)sizeof(CodeT);
  return (L + per16 - 1) / per16 * per16;
}

__device__ __forceinline__ float lsh_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---------------------------------------------------------------------------------------
// key sums
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void lsh_key_sums_kernel(const T* __restrict__ k, int64_t ks_b, int64_t ks_h,
                                    int64_t ks_s, int Hkv, int64_t s0, int64_t s1, int D,
                                    int64_t chunk, double* __restrict__ sums) {
  const int64_t bh = blockIdx.y;
  const int64_t b = bh / Hkv, h = bh % Hkv;
  const int64_t lo = s0 + (int64_t)blockIdx.x * chunk;
  const int64_t hi = lo + chunk < s1 ? lo + chunk : s1;
  const T* base = k + b * ks_b + h * ks_h;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    double acc = 0.0;
    for (int64_t s = lo; s < hi; ++s) acc += (double)sah_to_float<T>(base[s * ks_s + d]);
    atomicAdd(&sums[bh * D + d], acc);
  }
}

extern "C" int sah_lsh_key_sums(const void* keys, int dtype, int64_t ks_b, int64_t ks_h,
                                int64_t ks_s, int B, int Hkv, int64_t s0, int64_t s1, int D,
                                double* sums, void* stream) {
  SAH_REQUIRE(keys && sums, "lsh_key_sums: null pointer");
  SAH_REQUIRE(B > 0 && Hkv > 0 && D > 0 && s0 >= 0 && s1 >= s0, "lsh_key_sums: bad extents");
  if (s1 == s0) return SAH_OK;
  const int64_t chunk = 256;
  dim3 grid((unsigned)((s1 - s0 + chunk - 1) / chunk), (unsigned)(B * Hkv));
  SAH_DISPATCH_DTYPE(dtype, T, {
    lsh_key_sums_kernel<T><<<grid, 128, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const T*>(keys), ks_b, ks_h, ks_s, Hkv, s0, s1, D, chunk, sums);
  });
  SAH_LAUNCH_CHECK("lsh_key_sums");
  return SAH_OK;
}

// ---------------------------------------------------------------------------------------
// key statistics: norm of the centred key, running maximum
// ---------------------------------------------------------------------------------------
// lane `lane` loads its `per` consecutive channels of a row (one vector load when the row
// address allows it: rows of the usual 64 / 128 / 256 channels always do)
template <typename T>
__device__ __forceinline__ void lsh_load_lane(const T* row, int per, int lane, float* x) {
  const T* p = row + lane * per;
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  if (sizeof(T) == 2 && per == 4 && (a & 7) == 0) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    x[0] = __uint_as_float(v.x << 16);
    x[1] = __uint_as_float(v.x & 0xffff0000u);
    x[2] = __uint_as_float(v.y << 16);
    x[3] = __uint_as_float(v.y & 0xffff0000u);
  } else if (sizeof(T) == 2 && per == 2 && (a & 3) == 0) {
    const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
    x[0] = __uint_as_float(v << 16);
    x[1] = __uint_as_float(v & 0xffff0000u);
  } else if (sizeof(T) == 2 && per == 8 && (a & 15) == 0) {
    sah_unpack8(*reinterpret_cast<const uint4*>(p), x);
  } else if (sizeof(T) == 4 && per == 4 && (a & 15) == 0) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  } else {
#pragma unroll
    for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
      if (t < per) x[t] = sah_to_float<T>(p[t]);
  }
}

template <typename T>
__global__ void lsh_key_stats_kernel(const T* __restrict__ k, int64_t ks_b, int64_t ks_h,
                                     int64_t ks_s, int Hkv, int64_t s0, int64_t s1, int D,
                                     const T* __restrict__ mean, int64_t cap,
                                     float* __restrict__ norms, unsigned int* __restrict__ max_bits) {
  sah_pdl_entry_early();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int64_t bh = blockIdx.y;
  const int64_t b = bh / Hkv, h = bh % Hkv;
  const int per = D / 32;
  float m[LSH_MAX_PER_LANE];
  if (mean) lsh_load_lane<T>(mean + bh * D, per, lane, m);
  float local_max = 0.f;
  for (int64_t s = s0 + (int64_t)blockIdx.x * nwarp + warp; s < s1; s += (int64_t)gridDim.x * nwarp) {
    float x[LSH_MAX_PER_LANE];
    lsh_load_lane<T>(k + b * ks_b + h * ks_h + s * ks_s, per, lane, x);
    float acc = 0.f;
#pragma unroll
    for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
      if (t < per) {
        const float c = mean ? sah_round_to<T>(__fsub_rn(x[t], m[t])) : x[t];
        acc = __fadd_rn(acc, __fmul_rn(c, c));
      }
    const float nk = sah_round_to<T>(sqrtf(lsh_warp_sum(acc)));
    if (lane == 0) norms[bh * cap + s] = nk;
    local_max = fmaxf(local_max, nk);
  }
  if (lane == 0 && local_max > 0.f) atomicMax(max_bits, __float_as_uint(local_max));
}

extern "C" int sah_lsh_key_stats(const void* keys, int dtype, int64_t ks_b, int64_t ks_h,
                                 int64_t ks_s, int B, int Hkv, int64_t s0, int64_t s1, int D,
                                 const void* mean, int64_t cap, float* norms,
                                 unsigned int* max_norm_bits, int sm_count, void* stream) {
  SAH_REQUIRE(keys && norms && max_norm_bits, "lsh_key_stats: null pointer");
  SAH_REQUIRE(D % 32 == 0 && D <= 32 * LSH_MAX_PER_LANE, "lsh_key_stats: head_dim must be a multiple of 32, <= 256");
  SAH_REQUIRE(s0 >= 0 && s1 >= s0 && s1 <= cap, "lsh_key_stats: bad key range");
  if (s1 == s0) return SAH_OK;
  if (sm_count <= 0) sm_count = 148;
  int64_t gx = (s1 - s0 + 7) / 8;
  const int64_t cap_x = ((int64_t)sm_count * 16 + (int64_t)B * Hkv - 1) / ((int64_t)B * Hkv);
  if (gx > cap_x) gx = cap_x;
  dim3 grid((unsigned)gx, (unsigned)(B * Hkv));
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(lsh_key_stats_kernel<T>, grid, 256, 0, (cudaStream_t)stream,
        reinterpret_cast<const T*>(keys), ks_b, ks_h, ks_s, Hkv, s0, s1, D,
        reinterpret_cast<const T*>(mean), cap, norms, max_norm_bits);
  });
  SAH_LAUNCH_CHECK("lsh_key_stats");
  return SAH_OK;
}

// augmentation column of the MIPS transform: sqrt(M^2 - |k|^2) / M, rounded per operation
template <typename T>
__device__ __forceinline__ float lsh_augment(float nk, float M) {
  const float m2 = sah_round_to<T>(__fmul_rn(M, M));
  const float n2 = sah_round_to<T>(__fmul_rn(nk, nk));
  const float d = sah_round_to<T>(__fsub_rn(m2, n2));
  return sah_round_to<T>(__fdiv_rn(sah_round_to<T>(sqrtf(d)), M));
}

// ---------------------------------------------------------------------------------------
// key signatures
// ---------------------------------------------------------------------------------------
#define LSH_KT 64  // keys per CTA tile

template <typename T, typename CodeT>
__global__ void __launch_bounds__(256)
lsh_key_sign_kernel(const T* __restrict__ k, int64_t ks_b, int64_t ks_h, int64_t ks_s, int Hkv,
                    int64_t s0, int64_t s1, int D, const T* __restrict__ mean,
                    const float* __restrict__ norms, const unsigned int* __restrict__ max_bits,
                    const T* __restrict__ proj, int L, int K, int64_t cap,
                    CodeT* __restrict__ codes) {
  sah_pdl_entry_early();
  extern __shared__ __align__(16) unsigned char lsh_smem[];
  const int nbits = L * K;
  const int Dp = D + 1;
  float* xt = reinterpret_cast<float*>(lsh_smem);                       // [Dp][LSH_KT] transformed keys
  unsigned char* sb = lsh_smem + (size_t)Dp * LSH_KT * sizeof(float);   // [LSH_KT][nbits] sign bits
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t bh = blockIdx.y;
  const int64_t b = bh / Hkv, h = bh % Hkv;
  const int64_t t0 = s0 + (int64_t)blockIdx.x * LSH_KT;
  const int per = D / 32;
  const float M = __uint_as_float(*max_bits);

  float m[LSH_MAX_PER_LANE];
  if (mean) lsh_load_lane<T>(mean + bh * D, per, lane, m);
  for (int kk = warp; kk < LSH_KT; kk += 8) {
    const int64_t s = t0 + kk;
    float x[LSH_MAX_PER_LANE];
    if (s < s1) lsh_load_lane<T>(k + b * ks_b + h * ks_h + s * ks_s, per, lane, x);
#pragma unroll
    for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
      if (t < per) {
        float v = 0.f;
        if (s < s1) {
          const float c = mean ? sah_round_to<T>(__fsub_rn(x[t], m[t])) : x[t];
          v = sah_round_to<T>(__fdiv_rn(c, M));
        }
        xt[(lane * per + t) * LSH_KT + kk] = v;
      }
    if (lane == 0) xt[D * LSH_KT + kk] = s < s1 ? lsh_augment<T>(norms[bh * cap + s], M) : 0.f;
  }
  __syncthreads();

  // one output column per thread, 8 keys at a time; single accumulator per (key, column),
  // channels ascending (products of dtype values, added in float)
  // keys of this tile that exist (a decode step appends one key: one pass of eight, not eight)
  const int kt_used = (int)((s1 - t0 < LSH_KT ? s1 - t0 : LSH_KT) + 7) & ~7;
  if (s1 - t0 == 1) {
    // The key that a decode step appends: up to three columns per thread and the hyperplane
    // values of 8 channels x 3 columns requested before the first is used, so that a thread
    // waits for memory 17 times instead of 129 x 3 (that chain made this launch 66 us, all of
    // it load latency).  Same order of additions per column.  The body is kept small on
    // purpose: a decode step runs with cold caches, the instruction cache included, and a
    // fully unrolled 16-channel body measured slower (106 us) than the plain loop.
    constexpr int CB = 8, OC = 3;
    for (int o0 = threadIdx.x; o0 < nbits; o0 += 256 * OC) {
      const bool has1 = o0 + 256 < nbits, has2 = o0 + 512 < nbits;
      float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f;
      const T* pp = proj + o0;
#pragma unroll 1
      for (int c0 = 0; c0 + CB <= Dp; c0 += CB) {
        float p0[CB], p1[CB], p2[CB];
#pragma unroll
        for (int i = 0; i < CB; ++i) {
          const T* q = pp + (int64_t)(c0 + i) * nbits;
          p0[i] = sah_to_float<T>(q[0]);
          p1[i] = has1 ? sah_to_float<T>(q[256]) : 0.f;
          p2[i] = has2 ? sah_to_float<T>(q[512]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < CB; ++i) {
          const float a = xt[(c0 + i) * LSH_KT];
          acc0 = __fadd_rn(acc0, __fmul_rn(a, p0[i]));
          acc1 = __fadd_rn(acc1, __fmul_rn(a, p1[i]));
          acc2 = __fadd_rn(acc2, __fmul_rn(a, p2[i]));
        }
      }
      for (int c = Dp / CB * CB; c < Dp; ++c) {  // the channels left over (the augmented one)
        const T* q = pp + (int64_t)c * nbits;
        const float a = xt[c * LSH_KT];
        acc0 = __fadd_rn(acc0, __fmul_rn(a, sah_to_float<T>(q[0])));
        if (has1) acc1 = __fadd_rn(acc1, __fmul_rn(a, sah_to_float<T>(q[256])));
        if (has2) acc2 = __fadd_rn(acc2, __fmul_rn(a, sah_to_float<T>(q[512])));
      }
      sb[o0] = acc0 > 0.f ? 1 : 0;
      if (has1) sb[o0 + 256] = acc1 > 0.f ? 1 : 0;
      if (has2) sb[o0 + 512] = acc2 > 0.f ? 1 : 0;
    }
  } else {
    for (int o = threadIdx.x; o < nbits; o += 256) {
      for (int k8 = 0; k8 < kt_used; k8 += 8) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int c = 0; c < Dp; ++c) {
          const float p = sah_to_float<T>(proj[(int64_t)c * nbits + o]);
          const float4 a = *reinterpret_cast<const float4*>(xt + c * LSH_KT + k8);
          const float4 bq = *reinterpret_cast<const float4*>(xt + c * LSH_KT + k8 + 4);
          acc[0] = __fadd_rn(acc[0], __fmul_rn(a.x, p));
          acc[1] = __fadd_rn(acc[1], __fmul_rn(a.y, p));
          acc[2] = __fadd_rn(acc[2], __fmul_rn(a.z, p));
          acc[3] = __fadd_rn(acc[3], __fmul_rn(a.w, p));
          acc[4] = __fadd_rn(acc[4], __fmul_rn(bq.x, p));
          acc[5] = __fadd_rn(acc[5], __fmul_rn(bq.y, p));
          acc[6] = __fadd_rn(acc[6], __fmul_rn(bq.z, p));
          acc[7] = __fadd_rn(acc[7], __fmul_rn(bq.w, p));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) sb[(k8 + j) * nbits + o] = acc[j] > 0.f ? 1 : 0;
      }
    }
  }
  __syncthreads();
  // pack: bit j of table l is column l*K + j (magic_pig.py:120-150); the row of a key holds
  // its L codes and zero padding up to the row pitch
  const int LP = lsh_row_pitch<CodeT>(L);
  for (int i = threadIdx.x; i < LP * kt_used; i += 256) {
    const int kk = i / LP, l = i % LP;
    const int64_t s = t0 + kk;
    if (s >= s1) continue;
    unsigned int code = 0;
    if (l < L)
      for (int j = 0; j < K; ++j) code |= (unsigned int)sb[kk * nbits + l * K + j] << j;
    codes[(bh * cap + s) * LP + l] = (CodeT)code;
  }
}

extern "C" int sah_lsh_key_sign(const void* keys, int dtype, int64_t ks_b, int64_t ks_h,
                                int64_t ks_s, int B, int Hkv, int64_t s0, int64_t s1, int D,
                                const void* mean, const float* norms,
                                const unsigned int* max_norm_bits, const void* proj, int L, int K,
                                int64_t cap, void* codes, void* stream) {
  SAH_REQUIRE(keys && norms && max_norm_bits && proj && codes, "lsh_key_sign: null pointer");
  SAH_REQUIRE(D % 32 == 0 && D <= 32 * LSH_MAX_PER_LANE, "lsh_key_sign: head_dim must be a multiple of 32, <= 256");
  SAH_REQUIRE(L > 0 && K > 0, "lsh_key_sign: bad table shape");
  if (K > 16) return sah_fail(SAH_ERR_UNSUPPORTED, "lsh: lsh_k = %d > 16 bits per table is not built", K);
  SAH_REQUIRE(s0 >= 0 && s1 >= s0 && s1 <= cap, "lsh_key_sign: bad key range");
  if (s1 == s0) return SAH_OK;
  const size_t smem = (size_t)(D + 1) * LSH_KT * sizeof(float) + (size_t)LSH_KT * L * K;
  if (smem > 200 * 1024)
    return sah_fail(SAH_ERR_UNSUPPORTED, "lsh_key_sign: %d x %d signature bits exceed shared memory", L, K);
  dim3 grid((unsigned)((s1 - s0 + LSH_KT - 1) / LSH_KT), (unsigned)(B * Hkv));
  cudaStream_t st = (cudaStream_t)stream;
#define LSH_SIGN_LAUNCH(T, CodeT)                                                                  \
  do {                                                                                             \
    cudaError_t e = cudaFuncSetAttribute(lsh_key_sign_kernel<T, CodeT>,                            \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "lsh_key_sign attr: %s", cudaGetErrorString(e)); \
    sah_launch_chain(lsh_key_sign_kernel<T, CodeT>, grid, 256, smem, st, \
        reinterpret_cast<const T*>(keys), ks_b, ks_h, ks_s, Hkv, s0, s1, D,                        \
        reinterpret_cast<const T*>(mean), norms, max_norm_bits, reinterpret_cast<const T*>(proj),  \
        L, K, cap, reinterpret_cast<CodeT*>(codes));                                               \
  } while (0)
  SAH_DISPATCH_DTYPE(dtype, T, {
    if (K <= 8) LSH_SIGN_LAUNCH(T, uint8_t); else LSH_SIGN_LAUNCH(T, uint16_t);
  });
  SAH_LAUNCH_CHECK("lsh_key_sign");
  return SAH_OK;
}

#include "sah_lsh_tc.cuh"

// Workspace of sah_lsh_key_sign_tc: two status words (entries appended to the list; error word
// of the bounded waits), padding to 16 bytes, then the list of 32-column groups to redo.
extern "C" int64_t sah_lsh_key_sign_tc_ws_bytes(int B, int Hkv, int64_t n_keys) {
  if (B <= 0 || Hkv <= 0 || n_keys <= 0) return 0;
  const int64_t rows = (int64_t)B * Hkv * n_keys;
  return 16 + (rows / 4 + 4096) * (int64_t)sizeof(LtcUncertain);
}

extern "C" int sah_lsh_key_sign_tc(const void* keys, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B,
                                   int Hkv, int64_t s0, int64_t s1, int D, const void* mean,
                                   const float* norms, const unsigned int* max_norm_bits,
                                   const void* proj, int L, int K, int64_t cap, void* codes,
                                   void* workspace, int64_t workspace_bytes, int sm_count, void* stream) {
  SAH_REQUIRE(keys && norms && max_norm_bits && proj && codes && workspace, "lsh_key_sign_tc: null pointer");
  if (D != 128 || K != 8)
    return sah_fail(SAH_ERR_UNSUPPORTED, "lsh_key_sign_tc: head dim 128 and 8 bits per table (got %d, %d)", D, K);
  SAH_REQUIRE(L > 0 && s0 >= 0 && s1 >= s0 && s1 <= cap, "lsh_key_sign_tc: bad extents");
  SAH_REQUIRE((ks_s * 2) % 16 == 0 && (ks_h * 2) % 16 == 0 && (ks_b * 2) % 16 == 0 && ((uintptr_t)keys % 16) == 0 &&
                  (mean == nullptr || ((uintptr_t)mean % 16) == 0) && ((uintptr_t)codes % 16) == 0 &&
                  ((uintptr_t)workspace % 16) == 0,
              "lsh_key_sign_tc: rows must be 16-byte aligned");
  if (s1 == s0) return SAH_OK;
  const int64_t need = sah_lsh_key_sign_tc_ws_bytes(B, Hkv, s1 - s0);
  if (workspace_bytes < need)
    return sah_fail(SAH_ERR_WORKSPACE, "lsh_key_sign_tc: workspace of %lld bytes, need %lld",
                    (long long)workspace_bytes, (long long)need);
  cudaStream_t st = (cudaStream_t)stream;
  int* status = reinterpret_cast<int*>(workspace);
  LtcUncertain* list = reinterpret_cast<LtcUncertain*>(reinterpret_cast<unsigned char*>(workspace) + 16);
  const int list_cap = (int)((workspace_bytes - 16) / (int64_t)sizeof(LtcUncertain) < (1ll << 30)
                                 ? (workspace_bytes - 16) / (int64_t)sizeof(LtcUncertain)
                                 : (1ll << 30));
  cudaError_t e = cudaMemsetAsync(status, 0, 16, st);
  if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "lsh_key_sign_tc memset: %s", cudaGetErrorString(e));
  static bool allowed = false;
  if (!allowed) {
    e = cudaFuncSetAttribute(lsh_key_sign_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LtcCfg::SMEM);
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "lsh_key_sign_tc attr: %s", cudaGetErrorString(e));
    allowed = true;
  }
  if (sm_count <= 0) sm_count = 148;
  const int chunks = (L * 8 + LTC_NCHUNK - 1) / LTC_NCHUNK;
  const int64_t BH = (int64_t)B * Hkv;
  const int64_t tiles = BH * ((s1 - s0 + LTC_TILE - 1) / LTC_TILE);
  int64_t workers = sm_count / chunks;
  if (workers < 1) workers = 1;
  if (workers > tiles) workers = tiles;
  dim3 grid((unsigned)workers, (unsigned)chunks);
  lsh_key_sign_tc_kernel<<<grid, LTC_THREADS, LtcCfg::SMEM, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(keys), ks_b, ks_h, ks_s, Hkv, BH, s0, s1,
      reinterpret_cast<const __nv_bfloat16*>(mean), norms, max_norm_bits, reinterpret_cast<const __nv_bfloat16*>(proj),
      L, cap, reinterpret_cast<uint8_t*>(codes), list, list_cap, status, status + 1);
  SAH_LAUNCH_CHECK("lsh_key_sign_tc");
  lsh_sign_recheck_kernel<<<(unsigned)(sm_count * 4), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(keys), ks_b, ks_h, ks_s, Hkv, reinterpret_cast<const __nv_bfloat16*>(mean),
      norms, max_norm_bits, reinterpret_cast<const __nv_bfloat16*>(proj), L, cap, reinterpret_cast<uint8_t*>(codes),
      list, list_cap, status);
  SAH_LAUNCH_CHECK("lsh_sign_recheck");
  return SAH_OK;
}

// ---------------------------------------------------------------------------------------
// query: centre, normalise, signatures, unit vector
// ---------------------------------------------------------------------------------------
template <typename T, typename CodeT>
__global__ void __launch_bounds__(256)
lsh_query_kernel(const T* __restrict__ q, int64_t qs_b, int64_t qs_h, int64_t qs_q, int Hq, int Sq,
                 int G, int D, const T* __restrict__ mean, const T* __restrict__ proj, int L, int K,
                 CodeT* __restrict__ qcodes, float* __restrict__ qunit, T* __restrict__ qhat,
                 float* __restrict__ qmu) {
  sah_pdl_entry_early();
  extern __shared__ __align__(16) unsigned char lsh_smem[];
  float* qn = reinterpret_cast<float*>(lsh_smem);                 // [D] normalised query
  unsigned char* sb = lsh_smem + (size_t)D * sizeof(float);       // [L*K]
  const int nbits = L * K;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x;
  const int qi = (int)(row % Sq);
  const int64_t bh = row / Sq;
  const int h = (int)(bh % Hq);
  const int64_t b = bh / Hq;
  const int per = D / 32;
  if (warp == 0) {
    float x[LSH_MAX_PER_LANE], m[LSH_MAX_PER_LANE], c[LSH_MAX_PER_LANE];
    lsh_load_lane<T>(q + b * qs_b + h * qs_h + qi * qs_q, per, lane, x);
    if (mean) lsh_load_lane<T>(mean + (b * (Hq / G) + h / G) * D, per, lane, m);
    float acc = 0.f;
#pragma unroll
    for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
      if (t < per) {
        c[t] = mean ? sah_round_to<T>(__fsub_rn(x[t], m[t])) : x[t];
        acc = __fadd_rn(acc, __fmul_rn(c[t], c[t]));
      }
    // q / (|q| + 1e-8)
    const float nq = sah_round_to<T>(sqrtf(lsh_warp_sum(acc)));
    const float den = sah_round_to<T>(__fadd_rn(nq, 1e-8f));
    acc = 0.f;
#pragma unroll
    for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
      if (t < per) {
        c[t] = sah_round_to<T>(__fdiv_rn(c[t], den));
        qn[lane * per + t] = c[t];
        acc = __fadd_rn(acc, __fmul_rn(c[t], c[t]));
      }
    // unit vector of the transformed query (its extra column is zero): qn / (|qn| + 1e-8)
    const float n2 = sah_round_to<T>(sqrtf(lsh_warp_sum(acc)));
    const float den2 = sah_round_to<T>(__fadd_rn(n2, 1e-8f));
    float mu = 0.f;
#pragma unroll
    for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
      if (t < per) {
        const float u = sah_round_to<T>(__fdiv_rn(c[t], den2));
        qunit[row * D + lane * per + t] = u;
        if (qhat != nullptr) qhat[row * D + lane * per + t] = sah_from_float<T>(u);  // exact
        if (mean) mu = __fmaf_rn(u, m[t], mu);
      }
    // unit query . key mean, the query-side constant of the centred cosine
    mu = lsh_warp_sum(mu);
    if (qmu != nullptr && lane == 0) qmu[row] = mu;
  }
  __syncthreads();
  // A thread owns the columns o, o + 256, ... (four at a time); per column one accumulator and
  // channels ascending, as everywhere.  The hyperplane values of 16 channels x 4 columns are
  // requested before the first is used: this kernel sits on the critical path of every decode
  // step and would otherwise be a chain of 129 dependent (cold) loads per column.
  for (int o0 = threadIdx.x; o0 < nbits; o0 += 4 * 256) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c0 = 0; c0 < D; c0 += 16) {
      T pv[4][16];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 16; ++i)
          pv[j][i] = (o0 + j * 256 < nbits) ? proj[(int64_t)(c0 + i) * nbits + o0 + j * 256] : sah_from_float<T>(0.f);
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 16; ++i)
          acc[j] = __fadd_rn(acc[j], __fmul_rn(qn[c0 + i], sah_to_float<T>(pv[j][i])));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int o = o0 + j * 256;
      if (o < nbits) {
        const float a = __fadd_rn(acc[j], __fmul_rn(0.f, sah_to_float<T>(proj[(int64_t)D * nbits + o])));
        sb[o] = a > 0.f ? 1 : 0;
      }
    }
  }
  __syncthreads();
  for (int l = threadIdx.x; l < L; l += 256) {
    unsigned int code = 0;
    for (int j = 0; j < K; ++j) code |= (unsigned int)sb[l * K + j] << j;
    qcodes[row * L + l] = (CodeT)code;
  }
}

extern "C" int sah_lsh_query(const void* q, int dtype, int64_t qs_b, int64_t qs_h, int64_t qs_q,
                             int B, int Hq, int Sq, int G, int D, const void* mean,
                             const void* proj, int L, int K, void* qcodes, float* qunit,
                             void* qhat, float* qmu, void* stream) {
  SAH_REQUIRE(q && proj && qcodes && qunit, "lsh_query: null pointer");
  SAH_REQUIRE(D % 32 == 0 && D <= 32 * LSH_MAX_PER_LANE, "lsh_query: head_dim must be a multiple of 32, <= 256");
  SAH_REQUIRE(G > 0 && Hq % G == 0 && L > 0 && K > 0, "lsh_query: bad shape");
  if (K > 16) return sah_fail(SAH_ERR_UNSUPPORTED, "lsh: lsh_k = %d > 16 bits per table is not built", K);
  const size_t smem = (size_t)D * sizeof(float) + (size_t)L * K;
  if (smem > 48 * 1024)
    return sah_fail(SAH_ERR_UNSUPPORTED, "lsh_query: %d x %d signature bits exceed shared memory", L, K);
  const int64_t rows = (int64_t)B * Hq * Sq;
  cudaStream_t st = (cudaStream_t)stream;
  SAH_DISPATCH_DTYPE(dtype, T, {
    if (K <= 8)
      sah_launch_chain(lsh_query_kernel<T, uint8_t>, (unsigned)rows, 256, smem, st,
          reinterpret_cast<const T*>(q), qs_b, qs_h, qs_q, Hq, Sq, G, D,
          reinterpret_cast<const T*>(mean), reinterpret_cast<const T*>(proj), L, K,
          reinterpret_cast<uint8_t*>(qcodes), qunit, reinterpret_cast<T*>(qhat), qmu);
    else
      sah_launch_chain(lsh_query_kernel<T, uint16_t>, (unsigned)rows, 256, smem, st,
          reinterpret_cast<const T*>(q), qs_b, qs_h, qs_q, Hq, Sq, G, D,
          reinterpret_cast<const T*>(mean), reinterpret_cast<const T*>(proj), L, K,
          reinterpret_cast<uint16_t*>(qcodes), qunit, reinterpret_cast<T*>(qhat), qmu);
  });
  SAH_LAUNCH_CHECK("lsh_query");
  return SAH_OK;
}

// ---------------------------------------------------------------------------------------
// match: any table code equal
// ---------------------------------------------------------------------------------------
// One thread per key: it loads the key's signature row (a few 16-byte loads, all requested
// before the first compare) and tests it against the signature rows of the group's queries,
// which sit in shared memory padded with a value no key row holds in its padding.  "Some
// table code equal" is "some byte (halfword) of key XOR query is zero": with x = key ^ query,
// (x - 0x01..01) & ~x & 0x80..80 is non-zero exactly when x has a zero byte (a borrow can only
// start at a zero byte, so the test of the whole word is exact even though single positions
// above a zero byte are not), three integer instructions per word and query row.  A warp
// covers 32 consecutive keys, so a ballot of the result is the bitmap word of those keys;
// every warp does four such words and writes them side by side.
#define LSH_MATCH_WARPS 8
#define LSH_MATCH_WORDS 4
#define LSH_MAX_CHUNKS 16  // 16-byte chunks per signature row (256 byte codes, 128 halfword codes)

template <typename CodeT, int NC>
__global__ void __launch_bounds__(LSH_MATCH_WARPS * 32)
lsh_match_kernel(const CodeT* __restrict__ codes, int64_t cap, const CodeT* __restrict__ qcodes,
                 int Hq, int Sq, int G, int L, int64_t S, int64_t W,
                 const uint32_t* __restrict__ prev_bits, uint32_t* __restrict__ out_bits) {
  sah_pdl_entry();
  extern __shared__ __align__(16) unsigned char lsh_smem[];
  uint4* qs = reinterpret_cast<uint4*>(lsh_smem);  // [R][NC]
  const int R = G * Sq;
  constexpr int PER16 = 16 / (int)sizeof(CodeT);
  constexpr int LP = NC * PER16;
  const int64_t bh = blockIdx.y;           // b * Hkv + hkv
  const int Hkv = Hq / G;
  const int64_t b = bh / Hkv, hkv = bh % Hkv;
  {
    CodeT* qflat = reinterpret_cast<CodeT*>(lsh_smem);
    for (int i = threadIdx.x; i < R * LP; i += blockDim.x) {
      const int r = i / LP, l = i % LP;
      const int g = r / Sq, qi = r % Sq;
      // padding: all ones, which the zero padding of a key row never equals
      qflat[i] = l < L ? qcodes[(((b * Hq) + hkv * G + g) * Sq + qi) * L + l] : (CodeT)~(CodeT)0;
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t word0 = ((int64_t)blockIdx.x * LSH_MATCH_WARPS + warp) * LSH_MATCH_WORDS;
  if (word0 * 32 >= S) return;
  const uint4* base = reinterpret_cast<const uint4*>(codes + bh * cap * LP);
  for (int r0 = 0; r0 < R; r0 += 4) {
    uint32_t mine[4] = {0u, 0u, 0u, 0u};  // lane j keeps word j of rows r0 .. r0 + 3
#pragma unroll
    for (int j = 0; j < LSH_MATCH_WORDS; ++j) {
      const int64_t key = (word0 + j) * 32 + lane;
      unsigned int hit[4] = {0u, 0u, 0u, 0u};
      if (key < S) {
        uint4 v[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) v[c] = __ldg(base + key * NC + c);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            if (r0 + r < R) {
              const uint4 q = qs[(r0 + r) * NC + c];
              constexpr uint32_t ONES = sizeof(CodeT) == 1 ? 0x01010101u : 0x00010001u;
              constexpr uint32_t HIGH = sizeof(CodeT) == 1 ? 0x80808080u : 0x80008000u;
              const uint32_t x0 = v[c].x ^ q.x, x1 = v[c].y ^ q.y, x2 = v[c].z ^ q.z, x3 = v[c].w ^ q.w;
              const uint32_t z0 = (x0 - ONES) & ~x0 & HIGH, z1 = (x1 - ONES) & ~x1 & HIGH;
              const uint32_t z2 = (x2 - ONES) & ~x2 & HIGH, z3 = (x3 - ONES) & ~x3 & HIGH;
              hit[r] |= z0 | z1;
              hit[r] |= z2 | z3;
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const uint32_t wbits = __ballot_sync(0xffffffffu, hit[r] != 0u);
        if (lane == j) mine[r] = wbits;
      }
    }
    if (lane < LSH_MATCH_WORDS && (word0 + lane) * 32 < S) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        if (r0 + r < R) {
          const int g = (r0 + r) / Sq, qi = (r0 + r) % Sq;
          const int64_t row = ((b * Hq) + hkv * G + g) * Sq + qi;
          uint32_t bits = mine[r];  // keys past S never set a bit
          if (prev_bits != nullptr) bits |= prev_bits[row * W + word0 + lane];
          out_bits[row * W + word0 + lane] = bits;
        }
      }
    }
  }
}

// Decode shapes (at most four query rows per group, signature rows of up to 96 bytes): the
// group's query rows stay in registers (4 x NC 16-byte chunks), so that a (word, row) test is
// three integer instructions with no shared-memory operand, and a warp takes one bitmap word
// (32 consecutive keys) per round, striding over the row with all warps of the group's CTAs:
// the grid is two CTAs per SM whatever the key count, every warp gets the same number of words
// to within one.  The 32 signature rows of a round are contiguous in memory; the warp copies
// them to shared memory with 16-byte asynchronous copies, lane after lane (every copy
// instruction covers 512 contiguous bytes, where a lane loading its own row of 80 bytes makes
// each load instruction touch 20 cache lines), three rounds ahead, and every lane then reads
// its own row from there.  Lane r writes the word of row r.
// Measured at 1M keys (8.4M signature rows of 80 bytes, 671 MB): 139 us, 4.8 TB/s; the
// shared-memory form below 177 us; this form with per-lane 16-byte loads instead of the staged
// copies 164 us; with two of the four query rows read from shared memory and three CTAs per SM
// instead of two 182 us.  ~420 thread instructions per (key, group), 0.58 issue slots busy.
#define LSH_MATCH_REG_MAX_NC 6
#define LSH_MATCH_REG_STAGES 4

template <typename CodeT, int NC>
__global__ void __launch_bounds__(LSH_MATCH_WARPS * 32, 2)
lsh_match_reg_kernel(const CodeT* __restrict__ codes, int64_t cap, const CodeT* __restrict__ qcodes,
                     int Hq, int Sq, int G, int L, int64_t S, int64_t W,
                     const uint32_t* __restrict__ prev_bits, uint32_t* __restrict__ out_bits) {
  sah_pdl_entry();
  extern __shared__ __align__(16) unsigned char mr_smem[];  // [warps][stages][32 rows of NC chunks]
  __shared__ __align__(16) CodeT qflat[4 * NC * (16 / (int)sizeof(CodeT))];
  constexpr int PER16 = 16 / (int)sizeof(CodeT);
  constexpr int LP = NC * PER16;
  constexpr int NST = LSH_MATCH_REG_STAGES;
  constexpr int ROUND_BYTES = 32 * NC * 16;
  constexpr uint32_t ONES = sizeof(CodeT) == 1 ? 0x01010101u : 0x00010001u;
  constexpr uint32_t HIGH = sizeof(CodeT) == 1 ? 0x80808080u : 0x80008000u;
  const int R = G * Sq;  // <= 4
  const int64_t bh = blockIdx.y;  // b * Hkv + hkv
  const int Hkv = Hq / G;
  const int64_t b = bh / Hkv, hkv = bh % Hkv;
  for (int i = threadIdx.x; i < 4 * LP; i += blockDim.x) {
    const int r = i / LP, l = i % LP;
    CodeT c = (CodeT)~(CodeT)0;  // padding: all ones, which the zero padding of a key row never equals
    if (r < R && l < L) {
      const int g = r / Sq, qi = r % Sq;
      c = qcodes[(((b * Hq) + hkv * G + g) * Sq + qi) * L + l];
    }
    qflat[i] = c;
  }
  __syncthreads();
  uint4 q[4][NC];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < NC; ++c) q[r][c] = reinterpret_cast<const uint4*>(qflat)[r * NC + c];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t words = (S + 31) / 32;
  const uint4* base = reinterpret_cast<const uint4*>(codes + bh * cap * LP);
  const int64_t chunks_end = S * NC;  // 16-byte chunks of this (batch, KV head) that hold keys
  unsigned char* wbuf = mr_smem + (size_t)warp * NST * ROUND_BYTES;
  const uint32_t wbuf_s = (uint32_t)__cvta_generic_to_shared(wbuf);
  int64_t my_row = -1;  // lane r < R writes row r
  if (lane < R) {
    const int g = lane / Sq, qi = lane % Sq;
    my_row = ((b * Hq) + hkv * G + g) * Sq + qi;
  }
  const int64_t stride = (int64_t)gridDim.x * LSH_MATCH_WARPS;
  const int64_t w0 = (int64_t)blockIdx.x * LSH_MATCH_WARPS + warp;
  // copies of round `w` into stage `st`; one commit per call whether or not anything was copied
  auto issue = [&](int64_t w, int st) {
    if (w < words) {
      const int64_t first = w * 32 * NC;
#pragma unroll
      for (int it = 0; it < NC; ++it) {
        const int j = it * 32 + lane;
        if (first + j < chunks_end)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(wbuf_s + st * ROUND_BYTES + j * 16),
                       "l"(base + first + j)
                       : "memory");
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
#pragma unroll
  for (int s0 = 0; s0 < NST - 1; ++s0) issue(w0 + s0 * stride, s0);
  int i = 0;
  for (int64_t w = w0; w < words; w += stride, ++i) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(NST - 2) : "memory");
    __syncwarp();  // every lane's copies of this round have landed; everyone is done with round i - 1
    issue(w + (NST - 1) * stride, (i + NST - 1) % NST);
    const int64_t key = w * 32 + lane;
    uint32_t hit[4] = {0u, 0u, 0u, 0u};
    if (key < S) {
      const uint4* mine_row = reinterpret_cast<const uint4*>(wbuf + (i % NST) * ROUND_BYTES) + lane * NC;
      uint4 v[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) v[c] = mine_row[c];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint32_t x0 = v[c].x ^ q[r][c].x, x1 = v[c].y ^ q[r][c].y;
          const uint32_t x2 = v[c].z ^ q[r][c].z, x3 = v[c].w ^ q[r][c].w;
          const uint32_t z0 = (x0 - ONES) & ~x0 & HIGH, z1 = (x1 - ONES) & ~x1 & HIGH;
          const uint32_t z2 = (x2 - ONES) & ~x2 & HIGH, z3 = (x3 - ONES) & ~x3 & HIGH;
          hit[r] |= z0 | z1;
          hit[r] |= z2 | z3;
        }
      }
    }
    uint32_t mine = 0u;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint32_t wbits = __ballot_sync(0xffffffffu, hit[r] != 0u);
      if (lane == r) mine = wbits;
    }
    if (my_row >= 0) {
      if (prev_bits != nullptr) mine |= prev_bits[my_row * W + w];
      out_bits[my_row * W + w] = mine;
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

template <typename CodeT>
static int lsh_match_launch(const void* codes, int64_t cap, const void* qcodes, int Hq, int Sq, int G, int L,
                            int64_t S, int64_t W, const uint32_t* prev_bits, uint32_t* out_bits, dim3 grid,
                            size_t smem, cudaStream_t st) {
  const int nc = lsh_row_pitch<CodeT>(L) / (16 / (int)sizeof(CodeT));
  // SAH_LSH_MATCH_REG=0 in the environment keeps the shared-memory form for every shape
  static int reg_env = -1;
  if (reg_env < 0) {
    const char* e = getenv("SAH_LSH_MATCH_REG");
    reg_env = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  if (reg_env == 1 && G * Sq <= 4 && nc <= LSH_MATCH_REG_MAX_NC) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) {
      int n = 0;
      if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) sms = n;
    }
    const int64_t words = (S + 31) / 32;
    int64_t per_group = sah_ceil_div((int64_t)2 * sms, (int64_t)grid.y);
    const int64_t most = sah_ceil_div(words, LSH_MATCH_WARPS);
    if (per_group > most) per_group = most;
    if (per_group < 1) per_group = 1;
    const dim3 rgrid((unsigned)per_group, grid.y);
#define LSH_MATCH_REG_CASE(NC)                                                                      \
  case NC: {                                                                                        \
    constexpr int RSMEM = LSH_MATCH_WARPS * LSH_MATCH_REG_STAGES * 32 * NC * 16;                    \
    static bool allowed[64] = {};                                                                   \
    if (RSMEM > 48 * 1024 && dev >= 0 && dev < 64 && !allowed[dev]) {                               \
      cudaError_t e = cudaFuncSetAttribute(lsh_match_reg_kernel<CodeT, NC>,                         \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, RSMEM);     \
      if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "lsh_match attr: %s", cudaGetErrorString(e)); \
      allowed[dev] = true;                                                                          \
    }                                                                                               \
    sah_launch_chain(lsh_match_reg_kernel<CodeT, NC>, rgrid, LSH_MATCH_WARPS * 32, RSMEM, st,       \
        reinterpret_cast<const CodeT*>(codes), cap, reinterpret_cast<const CodeT*>(qcodes), Hq, Sq, \
        G, L, S, W, prev_bits, out_bits);                                                           \
  } break;
    switch (nc) {
      LSH_MATCH_REG_CASE(1) LSH_MATCH_REG_CASE(2) LSH_MATCH_REG_CASE(3) LSH_MATCH_REG_CASE(4)
      LSH_MATCH_REG_CASE(5) LSH_MATCH_REG_CASE(6)
    }
#undef LSH_MATCH_REG_CASE
    return SAH_OK;
  }
#define LSH_MATCH_CASE(NC)                                                                          \
  case NC:                                                                                          \
    sah_launch_chain(lsh_match_kernel<CodeT, NC>, grid, LSH_MATCH_WARPS * 32, smem, st, \
        reinterpret_cast<const CodeT*>(codes), cap, reinterpret_cast<const CodeT*>(qcodes), Hq, Sq, \
        G, L, S, W, prev_bits, out_bits);                                                           \
    break;
  switch (nc) {
    LSH_MATCH_CASE(1) LSH_MATCH_CASE(2) LSH_MATCH_CASE(3) LSH_MATCH_CASE(4) LSH_MATCH_CASE(5)
    LSH_MATCH_CASE(6) LSH_MATCH_CASE(7) LSH_MATCH_CASE(8) LSH_MATCH_CASE(9) LSH_MATCH_CASE(10)
    LSH_MATCH_CASE(11) LSH_MATCH_CASE(12) LSH_MATCH_CASE(13) LSH_MATCH_CASE(14) LSH_MATCH_CASE(15)
    LSH_MATCH_CASE(16)
    default:
      return sah_fail(SAH_ERR_UNSUPPORTED, "lsh_match: %d tables exceed %d bytes per signature row", L,
                      LSH_MAX_CHUNKS * 16);
  }
#undef LSH_MATCH_CASE
  return SAH_OK;
}

extern "C" int sah_lsh_match(const void* codes, int64_t cap, const void* qcodes, int B, int Hq,
                             int Sq, int G, int L, int K, int64_t S, int64_t W,
                             const uint32_t* prev_bits, uint32_t* out_bits, void* stream) {
  SAH_REQUIRE(codes && qcodes && out_bits, "lsh_match: null pointer");
  SAH_REQUIRE(G > 0 && Hq % G == 0 && L > 0 && K > 0 && S > 0 && W * 32 >= S, "lsh_match: bad shape");
  SAH_REQUIRE(cap >= S && (uintptr_t)codes % 16 == 0, "lsh_match: signature rows must be 16-byte aligned");
  if (K > 16) return sah_fail(SAH_ERR_UNSUPPORTED, "lsh: lsh_k = %d > 16 bits per table is not built", K);
  const int csz = K <= 8 ? 1 : 2;
  const int lp = csz == 1 ? lsh_row_pitch<uint8_t>(L) : lsh_row_pitch<uint16_t>(L);
  const size_t smem = (size_t)G * Sq * lp * csz;
  if (smem > 48 * 1024) return sah_fail(SAH_ERR_UNSUPPORTED, "lsh_match: too many query rows per group");
  const int64_t words = (S + 31) / 32;
  dim3 grid((unsigned)sah_ceil_div(words, LSH_MATCH_WARPS * LSH_MATCH_WORDS), (unsigned)(B * (Hq / G)));
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_LSH_MATCH, st);
  const int rc = csz == 1 ? lsh_match_launch<uint8_t>(codes, cap, qcodes, Hq, Sq, G, L, S, W, prev_bits,
                                                      out_bits, grid, smem, st)
                          : lsh_match_launch<uint16_t>(codes, cap, qcodes, Hq, Sq, G, L, S, W, prev_bits,
                                                       out_bits, grid, smem, st);
  if (rc != SAH_OK) return rc;
  SAH_LAUNCH_CHECK("lsh_match");
  sah_prof_end(SAH_PROF_LSH_MATCH, st);
  return SAH_OK;
}

// ---------------------------------------------------------------------------------------
// collision probability of matched keys
// ---------------------------------------------------------------------------------------
// 1 - (1 - (1 - acos(c) / pi)^K)^L with every operation rounded to the dtype (:374-403).
// bf16 goes through a 65536-entry table of the whole chain; fp32 evaluates acos and pow in
// double precision and rounds once, so that a CPU restatement reproduces the bits.
template <typename T>
__device__ __forceinline__ float lsh_collision_prob(float c, int K, int L, const uint16_t* table);
template <>
__device__ __forceinline__ float lsh_collision_prob<__nv_bfloat16>(float c, int, int,
                                                                   const uint16_t* table) {
  return __uint_as_float(((uint32_t)table[__float_as_uint(c) >> 16]) << 16);
}
template <>
__device__ __forceinline__ float lsh_collision_prob<float>(float c, int K, int L, const uint16_t*) {
  const float theta = (float)acos((double)c);
  const float a = __fdiv_rn(theta, 3.14159274101257324f);
  const float s = __fsub_rn(1.0f, a);
  const float st = (float)pow((double)s, (double)K);
  const float u = __fsub_rn(1.0f, st);
  const float ul = (float)pow((double)u, (double)L);
  return __fsub_rn(1.0f, ul);
}

// x / M for a fixed divisor.  bf16: the quotient of two bf16 values rounded to bf16 depends on
// the dividend only through its 7 mantissa bits (a power-of-two factor commutes with both
// roundings), so a 128-entry table of bf16((1 + m/128) / M), built with true divisions,
// replaces the division; dividends with a zero or all-ones exponent field take the division.
// fp32: the IEEE division.
template <typename T>
struct LshDivM;
template <>
struct LshDivM<__nv_bfloat16> {
  static __device__ __forceinline__ void build(float* tab, float M) {
    for (int m = threadIdx.x; m < 128; m += blockDim.x)
      tab[m] = sah_round_to<__nv_bfloat16>(__fdiv_rn(1.0f + (float)m * 0.0078125f, M));
  }
  static __device__ __forceinline__ float div(float c, float M, const float* tab) {
    const uint32_t u = __float_as_uint(c);
    const uint32_t e = (u >> 23) & 0xffu;
    if (e == 0u || e == 255u) return sah_round_to<__nv_bfloat16>(__fdiv_rn(c, M));
    const float r = __fmul_rn(__uint_as_float(u & 0xff800000u), tab[(u >> 16) & 0x7fu]);
    // the product of a power of two and a bf16 value is exact unless it leaves the normal range
    const uint32_t er = (__float_as_uint(r) >> 23) & 0xffu;
    return (er == 0u || er == 255u) ? sah_round_to<__nv_bfloat16>(__fdiv_rn(c, M)) : r;
  }
};
template <>
struct LshDivM<float> {
  static __device__ __forceinline__ void build(float*, float) {}
  static __device__ __forceinline__ float div(float c, float M, const float*) { return __fdiv_rn(c, M); }
};

// x / den for a per-key divisor.  bf16: both operands are bf16 values; with y = RN(1 / den),
// q = RN(x * y), r = x - q * den (exact in one fma), RN(q + r * y) rounded to bf16 equals the
// IEEE quotient rounded to bf16 for every pair of bf16 significands (checked exhaustively on
// the host, tests/test_magicpig.py); operands outside the normal range take the division.
template <typename T>
__device__ __forceinline__ float lsh_div_den(float x, float den, float rcp);
template <>
__device__ __forceinline__ float lsh_div_den<__nv_bfloat16>(float x, float den, float rcp) {
  const float q = __fmul_rn(x, rcp);
  const float r = __fmaf_rn(-q, den, x);
  const float q2 = __fmaf_rn(r, rcp, q);
  const uint32_t e = (__float_as_uint(q2) >> 23) & 0xffu;
  if (e < 2u || e >= 254u) return sah_round_to<__nv_bfloat16>(__fdiv_rn(x, den));
  return sah_round_to<__nv_bfloat16>(q2);
}
template <>
__device__ __forceinline__ float lsh_div_den<float>(float x, float den, float) {
  return __fdiv_rn(x, den);
}

// One CTA per (KV group, chunk of bitmap words); a warp takes a word, forms the union of the
// group's rows for it, transforms each key of the union once (centre, scale, normalise) and
// dots it with the unit query of every row that matched it.
template <typename T>
__global__ void __launch_bounds__(256)
lsh_prob_kernel(const T* __restrict__ k, int64_t ks_b, int64_t ks_h, int64_t ks_s, int Hq, int Sq,
                int G, int D, const T* __restrict__ mean, const float* __restrict__ norms,
                int64_t cap, const unsigned int* __restrict__ max_bits,
                const float* __restrict__ qunit, const uint32_t* __restrict__ bits,
                const int32_t* __restrict__ wpre, const int64_t* __restrict__ ptr, int64_t W,
                int K, int L, const uint16_t* __restrict__ table, int q_in_smem,
                T* __restrict__ data) {
  extern __shared__ __align__(16) unsigned char lsh_smem[];
  float* tab = reinterpret_cast<float*>(lsh_smem);  // [128]
  float* qs = tab + 128;                            // [R][D] when q_in_smem
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int Hkv = Hq / G;
  const int64_t kvh = blockIdx.x;  // b * Hkv + hkv
  const int64_t b = kvh / Hkv;
  const int hkv = (int)(kvh % Hkv);
  const int R = G * Sq;
  const int per = D / 32;
  const float M = __uint_as_float(*max_bits);
  const int64_t row0 = (b * Hq + (int64_t)hkv * G) * Sq;  // rows of a group are contiguous
  LshDivM<T>::build(tab, M);
  if (q_in_smem)
    for (int i = threadIdx.x; i < R * D; i += blockDim.x) qs[i] = qunit[row0 * D + i];
  __syncthreads();
  const float* qsrc = q_in_smem ? qs : qunit + row0 * D;
  float m[LSH_MAX_PER_LANE];
  if (mean) lsh_load_lane<T>(mean + kvh * D, per, lane, m);
  const T* kbase = k + b * ks_b + hkv * ks_h;
  for (int64_t w = (int64_t)blockIdx.y * nwarp + warp; w < W; w += (int64_t)gridDim.y * nwarp) {
    // union of the rows' words (lane r holds row r, r + 32, ...)
    uint32_t uni = 0u, myword = 0u;
    for (int r = lane; r < R; r += 32) {
      const uint32_t wd = bits[(row0 + r) * W + w];
      if (r < 32) myword = wd;
      uni |= wd;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) uni |= __shfl_xor_sync(0xffffffffu, uni, o);
    if (!uni) continue;
    // the next key's row is loaded while the current one is worked on
    int nbit = __ffs(uni) - 1;
    float xn[LSH_MAX_PER_LANE];
    lsh_load_lane<T>(kbase + (w * 32 + nbit) * ks_s, per, lane, xn);
    float nkn = norms[kvh * cap + w * 32 + nbit];
    while (uni) {
      const int bit = nbit;
      const float nk = nkn;
      float x[LSH_MAX_PER_LANE];
#pragma unroll
      for (int t = 0; t < LSH_MAX_PER_LANE; ++t) x[t] = xn[t];
      uni &= uni - 1;
      if (uni) {
        nbit = __ffs(uni) - 1;
        lsh_load_lane<T>(kbase + (w * 32 + nbit) * ks_s, per, lane, xn);
        nkn = norms[kvh * cap + w * 32 + nbit];
      }
      float acc = 0.f;
#pragma unroll
      for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
        if (t < per) {
          const float c = mean ? sah_round_to<T>(__fsub_rn(x[t], m[t])) : x[t];
          x[t] = LshDivM<T>::div(c, M, tab);
          acc = __fadd_rn(acc, __fmul_rn(x[t], x[t]));
        }
      const float aug = lsh_augment<T>(nk, M);
      // |transformed key|, then its unit vector
      const float n2 = __fadd_rn(lsh_warp_sum(acc), __fmul_rn(aug, aug));
      const float den = sah_round_to<T>(__fadd_rn(sah_round_to<T>(sqrtf(n2)), 1e-8f));
      const float rcp = __frcp_rn(den);
#pragma unroll
      for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
        if (t < per) x[t] = lsh_div_den<T>(x[t], den, rcp);
      for (int r = 0; r < R; ++r) {
        // warp-uniform: the first 32 rows' words sit in the lanes, the rest are re-read (L1)
        const uint32_t word = r < 32 ? __shfl_sync(0xffffffffu, myword, r) : bits[(row0 + r) * W + w];
        if (!((word >> bit) & 1u)) continue;
        const float* qu = qsrc + r * D + lane * per;
        acc = 0.f;
#pragma unroll
        for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
          if (t < per) acc = __fadd_rn(acc, __fmul_rn(qu[t], x[t]));
        float c = sah_round_to<T>(lsh_warp_sum(acc));
        c = fminf(fmaxf(c, -1.0f), 1.0f);
        if (lane == 0) {
          const int64_t pos = ptr[row0 + r] + wpre[(row0 + r) * W + w] + __popc(word & ((1u << bit) - 1u));
          data[pos] = sah_from_float<T>(lsh_collision_prob<T>(c, K, L, table));
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Cached norm of the transformed key.  |[k_c / M, sqrt(M^2 - |k_c|^2) / M]| + 1e-8 depends on
// the key, the key mean and the maximum norm M only, not on the query, so it is computed when
// keys arrive (and again for every key if M moved) instead of at every decode step.
// dens_max_bits holds the M the cached values were computed with.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
lsh_key_den_kernel(const T* __restrict__ k, int64_t ks_b, int64_t ks_h, int64_t ks_s, int Hkv,
                   int64_t s_new0, int64_t s1, int D, const T* __restrict__ mean,
                   const float* __restrict__ norms, int64_t cap,
                   const unsigned int* __restrict__ max_bits,
                   const unsigned int* __restrict__ dens_max_bits, float* __restrict__ dens) {
  sah_pdl_entry_early();
  __shared__ float tab[128];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int64_t bh = blockIdx.y;
  const int64_t b = bh / Hkv, h = bh % Hkv;
  const int per = D / 32;
  const unsigned int mb = *max_bits;
  const float M = __uint_as_float(mb);
  const int64_t begin = (mb == *dens_max_bits) ? s_new0 : 0;  // M moved: every key again
  if (begin >= s1) return;
  LshDivM<T>::build(tab, M);
  __syncthreads();
  float m[LSH_MAX_PER_LANE];
  if (mean) lsh_load_lane<T>(mean + bh * D, per, lane, m);
  for (int64_t s = begin + (int64_t)blockIdx.x * nwarp + warp; s < s1; s += (int64_t)gridDim.x * nwarp) {
    float x[LSH_MAX_PER_LANE];
    lsh_load_lane<T>(k + b * ks_b + h * ks_h + s * ks_s, per, lane, x);
    float acc = 0.f;
#pragma unroll
    for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
      if (t < per) {
        const float c = mean ? sah_round_to<T>(__fsub_rn(x[t], m[t])) : x[t];
        const float ks = LshDivM<T>::div(c, M, tab);
        acc = __fadd_rn(acc, __fmul_rn(ks, ks));
      }
    const float aug = lsh_augment<T>(norms[bh * cap + s], M);
    const float n2 = __fadd_rn(lsh_warp_sum(acc), __fmul_rn(aug, aug));
    if (lane == 0) dens[bh * cap + s] = sah_round_to<T>(__fadd_rn(sah_round_to<T>(sqrtf(n2)), 1e-8f));
  }
}

__global__ void lsh_den_commit_kernel(const unsigned int* max_bits, unsigned int* dens_max_bits) {
  sah_pdl_entry_early();
  *dens_max_bits = *max_bits;
}

extern "C" int sah_lsh_key_den(const void* keys, int dtype, int64_t ks_b, int64_t ks_h, int64_t ks_s,
                               int B, int Hkv, int64_t s_new0, int64_t s1, int D, const void* mean,
                               const float* norms, int64_t cap, const unsigned int* max_norm_bits,
                               unsigned int* dens_max_bits, float* dens, int sm_count, void* stream) {
  SAH_REQUIRE(keys && norms && max_norm_bits && dens_max_bits && dens, "lsh_key_den: null pointer");
  SAH_REQUIRE(D % 32 == 0 && D <= 32 * LSH_MAX_PER_LANE, "lsh_key_den: head_dim must be a multiple of 32, <= 256");
  SAH_REQUIRE(s_new0 >= 0 && s_new0 <= s1 && s1 <= cap, "lsh_key_den: bad key range");
  if (s1 == 0) return SAH_OK;
  if (sm_count <= 0) sm_count = 148;
  int64_t gx = (s1 + 7) / 8;
  const int64_t cap_x = ((int64_t)sm_count * 8 + (int64_t)B * Hkv - 1) / ((int64_t)B * Hkv);
  if (gx > cap_x) gx = cap_x;
  dim3 grid((unsigned)gx, (unsigned)(B * Hkv));
  cudaStream_t st = (cudaStream_t)stream;
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(lsh_key_den_kernel<T>, grid, 256, 0, st, reinterpret_cast<const T*>(keys), ks_b, ks_h, ks_s, Hkv,
                                                s_new0, s1, D, reinterpret_cast<const T*>(mean), norms,
                                                cap, max_norm_bits, dens_max_bits, dens);
  });
  SAH_LAUNCH_CHECK("lsh_key_den");
  sah_launch_chain(lsh_den_commit_kernel, 1, 1, 0, st, max_norm_bits, dens_max_bits);
  SAH_LAUNCH_CHECK("lsh_den_commit");
  return SAH_OK;
}

// bf16 with cached norms: the two divisions collapse into one table.  A centred key channel c
// (a bf16 value) times 1 / M rounded to bf16, times 1 / den rounded to bf16, equals
// 2^exponent(c) * U[den][mantissa(c)] with U = bf16(bf16((1 + m/128) / M) / den), because a
// power-of-two factor commutes with both roundings while everything stays in the normal
// range.  den is the norm of an (almost) unit vector: the 32 bf16 values from 0.9375 up
// cover it; other dens, and channels whose exponent could leave the normal range, take the
// two IEEE divisions.
#define LSH_DEN_BASE 0x3F70u
#define LSH_DEN_TABLES 32

__global__ void __launch_bounds__(256)
lsh_prob_fast_kernel(const __nv_bfloat16* __restrict__ k, int64_t ks_b, int64_t ks_h, int64_t ks_s,
                     int Hq, int Sq, int G, int D, const __nv_bfloat16* __restrict__ mean,
                     const float* __restrict__ dens, int64_t cap,
                     const unsigned int* __restrict__ max_bits, const float* __restrict__ qunit,
                     const uint32_t* __restrict__ bits, const int32_t* __restrict__ wpre,
                     const int64_t* __restrict__ ptr, int64_t W, const uint16_t* __restrict__ table,
                     int q_in_smem, __nv_bfloat16* __restrict__ data) {
  typedef __nv_bfloat16 T;
  extern __shared__ __align__(16) unsigned char lsh_smem[];
  float* U = reinterpret_cast<float*>(lsh_smem);  // [LSH_DEN_TABLES][128]
  float* qs = U + LSH_DEN_TABLES * 128;           // [R][D] when q_in_smem
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int Hkv = Hq / G;
  const int64_t kvh = blockIdx.x;
  const int64_t b = kvh / Hkv;
  const int hkv = (int)(kvh % Hkv);
  const int R = G * Sq;
  const int per = D / 32;
  const unsigned int mbits = *max_bits;
  const float M = __uint_as_float(mbits);
  const int64_t row0 = (b * Hq + (int64_t)hkv * G) * Sq;
  for (int i = threadIdx.x; i < LSH_DEN_TABLES * 128; i += blockDim.x) {
    const int di = i >> 7, m = i & 127;
    const float t = sah_round_to<T>(__fdiv_rn(1.0f + (float)m * 0.0078125f, M));
    const float d = __uint_as_float((LSH_DEN_BASE + (unsigned)di) << 16);
    U[i] = sah_round_to<T>(__fdiv_rn(t, d));
  }
  if (q_in_smem)
    for (int i = threadIdx.x; i < R * D; i += blockDim.x) qs[i] = qunit[row0 * D + i];
  __syncthreads();
  // exponent fields of c for which c / M / den surely stays normal (den is within [0.9375, 1.12])
  const int shift = 127 - (int)((mbits >> 23) & 0xffu);
  const int elo = max(1, 4 - shift), ehi = min(254, 250 - shift);
  const float* qsrc = q_in_smem ? qs : qunit + row0 * D;
  float m[LSH_MAX_PER_LANE];
  if (mean) lsh_load_lane<T>(mean + kvh * D, per, lane, m);
  const T* kbase = k + b * ks_b + hkv * ks_h;
  for (int64_t w = (int64_t)blockIdx.y * nwarp + warp; w < W; w += (int64_t)gridDim.y * nwarp) {
    uint32_t uni = 0u, myword = 0u;
    for (int r = lane; r < R; r += 32) {
      const uint32_t wd = bits[(row0 + r) * W + w];
      if (r < 32) myword = wd;
      uni |= wd;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) uni |= __shfl_xor_sync(0xffffffffu, uni, o);
    if (!uni) continue;
    int nbit = __ffs(uni) - 1;
    float xn[LSH_MAX_PER_LANE];
    lsh_load_lane<T>(kbase + (w * 32 + nbit) * ks_s, per, lane, xn);
    float dn = dens[kvh * cap + w * 32 + nbit];
    while (uni) {
      const int bit = nbit;
      const float den = dn;
      float x[LSH_MAX_PER_LANE];
#pragma unroll
      for (int t = 0; t < LSH_MAX_PER_LANE; ++t) x[t] = xn[t];
      uni &= uni - 1;
      if (uni) {
        nbit = __ffs(uni) - 1;
        lsh_load_lane<T>(kbase + (w * 32 + nbit) * ks_s, per, lane, xn);
        dn = dens[kvh * cap + w * 32 + nbit];
      }
      const unsigned int di = (__float_as_uint(den) >> 16) - LSH_DEN_BASE;
      const float* Ud = U + (di < LSH_DEN_TABLES ? di : 0u) * 128;
#pragma unroll
      for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
        if (t < per) {
          const float c = mean ? sah_round_to<T>(__fsub_rn(x[t], m[t])) : x[t];
          const uint32_t u = __float_as_uint(c);
          const int e = (int)((u >> 23) & 0xffu);
          if (di < LSH_DEN_TABLES && e >= elo && e <= ehi) {
            x[t] = __fmul_rn(__uint_as_float(u & 0xff800000u), Ud[(u >> 16) & 0x7fu]);
          } else {
            const float ks = sah_round_to<T>(__fdiv_rn(c, M));
            x[t] = sah_round_to<T>(__fdiv_rn(ks, den));
          }
        }
      for (int r = 0; r < R; ++r) {
        const uint32_t word = r < 32 ? __shfl_sync(0xffffffffu, myword, r) : bits[(row0 + r) * W + w];
        if (!((word >> bit) & 1u)) continue;
        const float* qu = qsrc + r * D + lane * per;
        float acc = 0.f;
#pragma unroll
        for (int t = 0; t < LSH_MAX_PER_LANE; ++t)
          if (t < per) acc = __fadd_rn(acc, __fmul_rn(qu[t], x[t]));
        float c = sah_round_to<T>(lsh_warp_sum(acc));
        c = fminf(fmaxf(c, -1.0f), 1.0f);
        if (lane == 0) {
          const int64_t pos = ptr[row0 + r] + wpre[(row0 + r) * W + w] + __popc(word & ((1u << bit) - 1u));
          data[pos] = __ushort_as_bfloat16(table[__float_as_uint(c) >> 16]);
        }
      }
    }
  }
}

// The decode shape of the same kernel: at most 4 rows per KV group (GQA 4, one query), head
// dim 32 * PER known at compile time, keys 8-byte aligned.  Row words, CSR bases and the unit
// queries sit in registers / shared memory for a whole bitmap word; the rows' results are
// written by lanes 0..3 side by side.
template <int PER>
__global__ void __launch_bounds__(256, 4)
lsh_prob_decode_kernel(const __nv_bfloat16* __restrict__ k, int64_t ks_b, int64_t ks_h, int64_t ks_s,
                       int Hq, int Sq, int G, const __nv_bfloat16* __restrict__ mean,
                       const float* __restrict__ dens, int64_t cap,
                       const unsigned int* __restrict__ max_bits, const float* __restrict__ qunit,
                       const uint32_t* __restrict__ bits, const int32_t* __restrict__ wpre,
                       const int64_t* __restrict__ ptr, int64_t W, const uint16_t* __restrict__ table,
                       __nv_bfloat16* __restrict__ data) {
  typedef __nv_bfloat16 T;
  constexpr int D = 32 * PER;
  __shared__ float U[LSH_DEN_TABLES * 128];
  __shared__ float qs[4 * D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int Hkv = Hq / G;
  const int64_t kvh = blockIdx.x;
  const int64_t b = kvh / Hkv;
  const int hkv = (int)(kvh % Hkv);
  const int R = G * Sq;  // <= 4
  const unsigned int mbits = *max_bits;
  const float M = __uint_as_float(mbits);
  const int64_t row0 = (b * Hq + (int64_t)hkv * G) * Sq;
  for (int i = threadIdx.x; i < LSH_DEN_TABLES * 128; i += blockDim.x) {
    const int di = i >> 7, m = i & 127;
    const float t = sah_round_to<T>(__fdiv_rn(1.0f + (float)m * 0.0078125f, M));
    const float d = __uint_as_float((LSH_DEN_BASE + (unsigned)di) << 16);
    U[i] = sah_round_to<T>(__fdiv_rn(t, d));
  }
  for (int i = threadIdx.x; i < 4 * D; i += blockDim.x) qs[i] = i < R * D ? qunit[row0 * D + i] : 0.f;
  __syncthreads();
  const int shift = 127 - (int)((mbits >> 23) & 0xffu);
  const int elo = max(1, 4 - shift), ehi = min(254, 250 - shift);
  float m[PER];
#pragma unroll
  for (int t = 0; t < PER; ++t) m[t] = mean ? __bfloat162float(mean[kvh * D + lane * PER + t]) : 0.f;
  // this lane's slice of the (up to) four unit queries
  float qu[4][PER];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int t = 0; t < PER; ++t) qu[r][t] = qs[r * D + lane * PER + t];
  const T* kbase = k + b * ks_b + hkv * ks_h;
  const float* dbase = dens + kvh * cap;
  for (int64_t w = (int64_t)blockIdx.y * nwarp + warp; w < W; w += (int64_t)gridDim.y * nwarp) {
    // lane 8r (r < R): word of row r and the CSR position of its first bit; the reduction
    // below leaves row r's cosine in lanes 8r .. 8r+7
    uint32_t myword = 0u;
    int64_t mypos = 0;
    if ((lane & 7) == 0 && (lane >> 3) < R) {
      const int r = lane >> 3;
      myword = bits[(row0 + r) * W + w];
      mypos = ptr[row0 + r] + wpre[(row0 + r) * W + w];
    }
    uint32_t uni = myword;
#pragma unroll
    for (int o = 16; o >= 8; o >>= 1) uni |= __shfl_xor_sync(0xffffffffu, uni, o);
    uni = __shfl_sync(0xffffffffu, uni, 0);
    if (!uni) continue;
    // Keys are taken four at a time: their rows are requested together, so that a warp has
    // four independent row loads in flight, then worked on one after the other.
    while (uni) {
      int kb[4];
      float xs[4][PER], dn[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kb[j] = uni ? __ffs(uni) - 1 : -1;
        uni &= uni - 1;  // 0 stays 0
        if (kb[j] >= 0) {
          lsh_load_lane<T>(kbase + (w * 32 + kb[j]) * ks_s, PER, lane, xs[j]);
          dn[j] = dbase[w * 32 + kb[j]];
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (kb[j] < 0) break;
        const int bit = kb[j];
        const float den = dn[j];
        float x[PER];
        const unsigned int di = (__float_as_uint(den) >> 16) - LSH_DEN_BASE;
        const float* Ud = U + (di < LSH_DEN_TABLES ? di : 0u) * 128;
        float cc[PER];
        bool slow = di >= LSH_DEN_TABLES;
#pragma unroll
        for (int t = 0; t < PER; ++t) {
          cc[t] = mean ? sah_round_to<T>(__fsub_rn(xs[j][t], m[t])) : xs[j][t];
          const uint32_t u = __float_as_uint(cc[t]);
          const unsigned int e = (u >> 23) & 0xffu;
          slow |= (e - (unsigned)elo) > (unsigned)(ehi - elo);
          x[t] = __fmul_rn(__uint_as_float(u & 0xff800000u), Ud[(u >> 16) & 0x7fu]);
        }
        if (__any_sync(0xffffffffu, slow)) {  // rare: zero channels, denormals, an unusual norm
          if (slow) {
#pragma unroll
            for (int t = 0; t < PER; ++t) {
              const unsigned int e = (__float_as_uint(cc[t]) >> 23) & 0xffu;
              if (di >= LSH_DEN_TABLES || (e - (unsigned)elo) > (unsigned)(ehi - elo))
                x[t] = sah_round_to<T>(__fdiv_rn(sah_round_to<T>(__fdiv_rn(cc[t], M)), den));
            }
          }
        }
        // Four dot products at once.  Each row's 32 lane partials combine in the fixed tree
        // (xor 16, 8, 4, 2, 1); the first two levels also sort the rows onto lane groups, so
        // six shuffles serve all four rows and every sum is associated exactly as in a
        // per-row tree.
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int t = 0; t < PER; ++t) {
          a0 = __fadd_rn(a0, __fmul_rn(qu[0][t], x[t]));
          a1 = __fadd_rn(a1, __fmul_rn(qu[1][t], x[t]));
          a2 = __fadd_rn(a2, __fmul_rn(qu[2][t], x[t]));
          a3 = __fadd_rn(a3, __fmul_rn(qu[3][t], x[t]));
        }
        const bool hi16 = (lane & 16) != 0, hi8 = (lane & 8) != 0;
        const float r0 = __shfl_xor_sync(0xffffffffu, hi16 ? a0 : a2, 16);
        const float r1 = __shfl_xor_sync(0xffffffffu, hi16 ? a1 : a3, 16);
        const float k0 = __fadd_rn(hi16 ? a2 : a0, r0);  // rows 0 / 2
        const float k1 = __fadd_rn(hi16 ? a3 : a1, r1);  // rows 1 / 3
        const float r2 = __shfl_xor_sync(0xffffffffu, hi8 ? k0 : k1, 8);
        float cosv = __fadd_rn(hi8 ? k1 : k0, r2);       // row 2 * bit4 + bit3
        cosv = __fadd_rn(cosv, __shfl_xor_sync(0xffffffffu, cosv, 4));
        cosv = __fadd_rn(cosv, __shfl_xor_sync(0xffffffffu, cosv, 2));
        cosv = __fadd_rn(cosv, __shfl_xor_sync(0xffffffffu, cosv, 1));
        if ((myword >> bit) & 1u) {  // only lanes 8r hold a word
          float c = sah_round_to<T>(cosv);
          c = fminf(fmaxf(c, -1.0f), 1.0f);
          data[mypos + __popc(myword & ((1u << bit) - 1u))] =
              __ushort_as_bfloat16(table[__float_as_uint(c) >> 16]);
        }
      }
    }
  }
}

extern "C" int sah_lsh_prob(const void* keys, int dtype, int64_t ks_b, int64_t ks_h, int64_t ks_s,
                            int B, int Hq, int Sq, int G, int D, const void* mean,
                            const float* norms, const float* dens, int64_t cap,
                            const unsigned int* max_norm_bits, const float* qunit,
                            const uint32_t* bits, const int32_t* wpre, const int64_t* ptr, int64_t W,
                            int K, int L, const uint16_t* table, void* data, int sm_count,
                            void* stream) {
  SAH_REQUIRE(keys && norms && max_norm_bits && qunit && bits && wpre && ptr && data,
              "lsh_prob: null pointer");
  SAH_REQUIRE(D % 32 == 0 && D <= 32 * LSH_MAX_PER_LANE, "lsh_prob: head_dim must be a multiple of 32, <= 256");
  SAH_REQUIRE(G > 0 && Hq % G == 0, "lsh_prob: bad head grouping");
  SAH_REQUIRE(dtype != SAH_BF16 || table != nullptr, "lsh_prob: bf16 needs the probability table");
  const int64_t groups = (int64_t)B * (Hq / G);
  const int R = G * Sq;
  if (sm_count <= 0) sm_count = 148;
  int64_t gy = (W + 7) / 8;
  const int64_t cap_y = ((int64_t)sm_count * 8 + groups - 1) / groups;
  if (gy > cap_y) gy = cap_y;
  if (gy < 1) gy = 1;
  if (gy > 65535) gy = 65535;
  const int q_in_smem = (size_t)R * D * sizeof(float) <= 24 * 1024;
  dim3 grid((unsigned)groups, (unsigned)gy);
  sah_prof_begin(SAH_PROF_LSH_PROB, (cudaStream_t)stream);
  if (dtype == SAH_BF16 && dens != nullptr) {
    // cached key norms (sah_lsh_key_den): one table lookup per channel
    if (R <= 4 && (D == 64 || D == 128 || D == 256)) {
#define LSH_DECODE_LAUNCH(PER)                                                                       \
  lsh_prob_decode_kernel<PER><<<grid, 256, 0, (cudaStream_t)stream>>>(                               \
      reinterpret_cast<const __nv_bfloat16*>(keys), ks_b, ks_h, ks_s, Hq, Sq, G,                     \
      reinterpret_cast<const __nv_bfloat16*>(mean), dens, cap, max_norm_bits, qunit, bits, wpre, ptr, \
      W, table, reinterpret_cast<__nv_bfloat16*>(data))
      if (D == 64) LSH_DECODE_LAUNCH(2);
      else if (D == 128) LSH_DECODE_LAUNCH(4);
      else LSH_DECODE_LAUNCH(8);
      SAH_LAUNCH_CHECK("lsh_prob");
      sah_prof_end(SAH_PROF_LSH_PROB, (cudaStream_t)stream);
      return SAH_OK;
    }
    size_t fsmem = (size_t)LSH_DEN_TABLES * 128 * sizeof(float);
    if (q_in_smem) fsmem += (size_t)R * D * sizeof(float);
    lsh_prob_fast_kernel<<<grid, 256, fsmem, (cudaStream_t)stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(keys), ks_b, ks_h, ks_s, Hq, Sq, G, D,
        reinterpret_cast<const __nv_bfloat16*>(mean), dens, cap, max_norm_bits, qunit, bits, wpre, ptr,
        W, table, q_in_smem, reinterpret_cast<__nv_bfloat16*>(data));
    SAH_LAUNCH_CHECK("lsh_prob");
    sah_prof_end(SAH_PROF_LSH_PROB, (cudaStream_t)stream);
    return SAH_OK;
  }
  size_t smem = 128 * sizeof(float);
  if (q_in_smem) smem += (size_t)R * D * sizeof(float);
  SAH_DISPATCH_DTYPE(dtype, T, {
    lsh_prob_kernel<T><<<grid, 256, smem, (cudaStream_t)stream>>>(
        reinterpret_cast<const T*>(keys), ks_b, ks_h, ks_s, Hq, Sq, G, D,
        reinterpret_cast<const T*>(mean), norms, cap, max_norm_bits, qunit, bits, wpre, ptr, W, K, L,
        table, q_in_smem, reinterpret_cast<T*>(data));
  });
  SAH_LAUNCH_CHECK("lsh_prob");
  sah_prof_end(SAH_PROF_LSH_PROB, (cudaStream_t)stream);
  return SAH_OK;
}

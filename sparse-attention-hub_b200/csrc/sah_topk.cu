// Dense score streams and the generic exact top-k:
//   sah_qk_scores    q . k over every key, GQA heads sharing each streamed K row
//                    (maskers/fixed/implementations/oracle_top_k.py:70-73)
//   sah_topk_select  radix select over a [rows][S] score tensor
//                    (maskers/fixed/base.py:74-85)
#include "sah_common.cuh"
#include "sah_select.cuh"

// ---------------------------------------------------------------------------
// q . k scores.  One thread owns one key and walks its row in 8-element
// chunks; the rows of the key's GQA group (up to 4 at a time) share the chunk.
// Accumulation order per (row, key): eight interleaved fp32 partial sums
// p_i = sum_t x[8t+i] * y[8t+i] (t ascending), then
// ((p0+p1)+(p2+p3)) + ((p4+p5)+(p6+p7)).  Products of two bf16 values are
// exact in fp32, so fma and mul+add agree there; fp32 inputs use an explicit
// mul then add so that a CPU restatement without fma gets the same bits.
// ---------------------------------------------------------------------------
#define QK_THREADS 128
#define QK_MAXR 16

template <typename T>
__device__ __forceinline__ float qk_mac(float a, float b, float c);
template <>
__device__ __forceinline__ float qk_mac<__nv_bfloat16>(float a, float b, float c) {
  return fmaf(a, b, c);
}
template <>
__device__ __forceinline__ float qk_mac<float>(float a, float b, float c) {
  return __fadd_rn(c, __fmul_rn(a, b));
}

template <typename T>
__global__ void __launch_bounds__(QK_THREADS)
qk_scores_kernel(const T* __restrict__ q, const T* __restrict__ k, int64_t qs_b, int64_t qs_h,
                 int64_t qs_q, int64_t ks_b, int64_t ks_h, int64_t ks_s, int Hq, int Hkv, int Sq,
                 int64_t S, int D, const T* __restrict__ bias, int64_t bias_s_b,
                 int64_t bias_s_h, int64_t bias_s_q, T* __restrict__ scores) {
  extern __shared__ __align__(16) float q_sm[];  // [R][D]
  const int G = Hq / Hkv;
  const int R = G * Sq;  // rows sharing this KV head
  const int kvh = blockIdx.y, b = blockIdx.z;
  // Stage the group's queries as fp32: row r = g * Sq + qi.
  for (int idx = threadIdx.x; idx < R * D; idx += QK_THREADS) {
    int r = idx / D, d = idx - r * D;
    int g = r / Sq, qi = r - g * Sq;
    q_sm[idx] = sah_to_float<T>(q[b * qs_b + (int64_t)(kvh * G + g) * qs_h + qi * qs_q + d]);
  }
  __syncthreads();
  const int64_t j = (int64_t)blockIdx.x * QK_THREADS + threadIdx.x;
  if (j >= S) return;
  const T* kr = k + b * ks_b + kvh * ks_h + j * ks_s;
  const int chunks = D / 8;
  for (int r0 = 0; r0 < R; r0 += 4) {
    float acc[4][8];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[r][i] = 0.f;
    for (int t = 0; t < chunks; ++t) {
      float kf[8];
      sah_load8<T>(kr + t * 8, kf);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        if (r0 + r < R) {
          const float4 qa = *reinterpret_cast<const float4*>(q_sm + (r0 + r) * D + t * 8);
          const float4 qb = *reinterpret_cast<const float4*>(q_sm + (r0 + r) * D + t * 8 + 4);
          acc[r][0] = qk_mac<T>(qa.x, kf[0], acc[r][0]);
          acc[r][1] = qk_mac<T>(qa.y, kf[1], acc[r][1]);
          acc[r][2] = qk_mac<T>(qa.z, kf[2], acc[r][2]);
          acc[r][3] = qk_mac<T>(qa.w, kf[3], acc[r][3]);
          acc[r][4] = qk_mac<T>(qb.x, kf[4], acc[r][4]);
          acc[r][5] = qk_mac<T>(qb.y, kf[5], acc[r][5]);
          acc[r][6] = qk_mac<T>(qb.z, kf[6], acc[r][6]);
          acc[r][7] = qk_mac<T>(qb.w, kf[7], acc[r][7]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (r0 + r < R) {
        float s = __fadd_rn(__fadd_rn(__fadd_rn(acc[r][0], acc[r][1]), __fadd_rn(acc[r][2], acc[r][3])),
                            __fadd_rn(__fadd_rn(acc[r][4], acc[r][5]), __fadd_rn(acc[r][6], acc[r][7])));
        s = sah_round_to<T>(s);
        const int rr = r0 + r, g = rr / Sq, qi = rr - g * Sq, h = kvh * G + g;
        if (bias != nullptr) {
          float bv = sah_to_float<T>(bias[b * bias_s_b + h * bias_s_h + qi * bias_s_q + j]);
          s = sah_round_to<T>(__fadd_rn(s, bv));
        }
        const int64_t row = ((int64_t)b * Hq + h) * Sq + qi;
        scores[row * S + j] = sah_from_float<T>(s);
      }
    }
  }
}

extern "C" int sah_qk_scores(const void* q, const void* k, int dtype, int64_t qs_b, int64_t qs_h,
                             int64_t qs_q, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B,
                             int Hq, int Hkv, int Sq, int64_t S, int D, const void* bias,
                             int64_t bias_s_b, int64_t bias_s_h, int64_t bias_s_q, void* scores,
                             void* stream) {
  SAH_REQUIRE(q && k && scores, "qk_scores: null pointer");
  SAH_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Sq > 0 && S > 0,
              "qk_scores: bad extents");
  SAH_REQUIRE(D % 8 == 0 && D > 0, "qk_scores: head dim must be a multiple of 8");
  SAH_REQUIRE(ks_s % 8 == 0 && ks_h % 8 == 0 && ks_b % 8 == 0 && (uintptr_t)k % 32 == 0,
              "qk_scores: K rows must be 32-byte aligned");
  const int R = (Hq / Hkv) * Sq;
  const size_t smem = (size_t)R * D * sizeof(float);
  if (smem > 200 * 1024)
    return sah_fail(SAH_ERR_UNSUPPORTED, "qk_scores: %d query rows per KV head do not fit", R);
  dim3 grid((unsigned)sah_ceil_div(S, QK_THREADS), (unsigned)Hkv, (unsigned)B);
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_QK_SCORES, (cudaStream_t)stream);
  SAH_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(qk_scores_kernel<T>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "qk_scores attr: %s", cudaGetErrorString(e));
    }
    qk_scores_kernel<T><<<grid, QK_THREADS, smem, st>>>(
        (const T*)q, (const T*)k, qs_b, qs_h, qs_q, ks_b, ks_h, ks_s, Hq, Hkv, Sq, S, D,
        (const T*)bias, bias_s_b, bias_s_h, bias_s_q, (T*)scores);
  });
  SAH_LAUNCH_CHECK("qk_scores");
  sah_prof_end(SAH_PROF_QK_SCORES, (cudaStream_t)stream);
  return SAH_OK;
}

// ---------------------------------------------------------------------------
// Generic top-k over a score tensor.
// ---------------------------------------------------------------------------
template <typename T, int KEYBITS>
struct ScoreKey {
  const T* s;
  __device__ __forceinline__ unsigned int operator()(int64_t j) const {
    unsigned int key = sah_float_key(sah_to_float<T>(s[j]) + 0.0f);  // -0 ranks with +0
    return KEYBITS == 16 ? (key >> 16) : key;
  }
};

template <typename T, int KEYBITS>
__global__ void __launch_bounds__(SAH_SELECT_THREADS)
topk_select_kernel(const T* __restrict__ scores, int64_t S, int64_t W, int64_t col_begin,
                   int64_t col_end, const uint32_t* __restrict__ prev_bits, int64_t k,
                   uint32_t* __restrict__ out_bits) {
  __shared__ SahSelectSmem sm;
  const int64_t row = blockIdx.x;
  ScoreKey<T, KEYBITS> kf{scores + row * S};
  sah_select_row<KEYBITS>(kf, prev_bits + row * W, out_bits + row * W, S, W, col_begin, col_end,
                          k, sm);
}

extern "C" int sah_topk_select(const void* scores, int dtype, int64_t rows, int64_t S, int64_t W,
                               int64_t col_begin, int64_t col_end, const uint32_t* prev_bits,
                               int64_t k, uint32_t* out_bits, void* stream) {
  SAH_REQUIRE(scores && prev_bits && out_bits, "topk_select: null pointer");
  SAH_REQUIRE(rows >= 0 && S > 0 && W * 32 >= S, "topk_select: bad extents");
  if (rows == 0) return SAH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_TOPK_SELECT, (cudaStream_t)stream);
  if (dtype == SAH_BF16) {
    topk_select_kernel<__nv_bfloat16, 16><<<(unsigned)rows, SAH_SELECT_THREADS, 0, st>>>(
        (const __nv_bfloat16*)scores, S, W, col_begin, col_end, prev_bits, k, out_bits);
  } else if (dtype == SAH_F32) {
    topk_select_kernel<float, 32><<<(unsigned)rows, SAH_SELECT_THREADS, 0, st>>>(
        (const float*)scores, S, W, col_begin, col_end, prev_bits, k, out_bits);
  } else {
    return sah_fail(SAH_ERR_INVALID, "topk_select: unknown dtype %d", dtype);
  }
  SAH_LAUNCH_CHECK("topk_select");
  sah_prof_end(SAH_PROF_TOPK_SELECT, (cudaStream_t)stream);
  return SAH_OK;
}

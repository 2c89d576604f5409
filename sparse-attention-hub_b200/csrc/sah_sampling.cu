// Sampling maskers (maskers/sampling/implementations/adaptive_sampling.py,
// utils/mask_attention_utils.py:105-184):
//   sah_adaptive_budget   per-row sample budget of the adaptive (epsilon, delta) masker
//   sah_sample_scatter    budgeted uniform draws scattered into a bitmap
//
// Random draws are a pure function of (seed, draw index): Philox4x32-10 with the
// counter (index, 0, 0, 0) and key (seed_lo, seed_hi); the first output word u gives the
// column  start + floor(u * n / 2^32).  A caller that wants the very same sample from
// another implementation regenerates or hands in the same draws.
#include "sah_common.cuh"

__host__ __device__ __forceinline__ uint32_t sah_mulhi32(uint32_t a, uint32_t b) {
  return (uint32_t)(((uint64_t)a * (uint64_t)b) >> 32);
}

__host__ __device__ __forceinline__ uint32_t sah_philox_u32(uint64_t seed, uint64_t index) {
  uint32_t c0 = (uint32_t)index, c1 = (uint32_t)(index >> 32), c2 = 0u, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = sah_mulhi32(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = sah_mulhi32(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

__device__ __forceinline__ int64_t sah_draw_column(uint64_t seed, uint64_t index, int64_t start,
                                                   int64_t n) {
  return start + (int64_t)sah_mulhi32(sah_philox_u32(seed, index), (uint32_t)n);
}

// Sum over the CTA in a fixed order: each thread already holds the sequential sum of its
// strided elements; lanes combine by xor shuffles (16, 8, 4, 2, 1), then the 32 warp sums
// combine the same way.  Every thread returns the same value.  blockDim.x must be 1024.
__device__ __forceinline__ float sah_block_sum_fixed(float v, float* scratch32) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch32[threadIdx.x >> 5] = v;
  __syncthreads();
  float w = scratch32[threadIdx.x & 31];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) w = __fadd_rn(w, __shfl_xor_sync(0xffffffffu, w, o));
  return w;
}

__device__ __forceinline__ float sah_block_max(float v, float* scratch32) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch32[threadIdx.x >> 5] = v;
  __syncthreads();
  float w = scratch32[threadIdx.x & 31];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, o));
  return w;
}

template <typename T>
__device__ __forceinline__ float ad_exp(float x, const uint16_t* table);
template <>
__device__ __forceinline__ float ad_exp<__nv_bfloat16>(float x, const uint16_t* table) {
  return __uint_as_float(((uint32_t)table[__float_as_uint(x) >> 16]) << 16);
}
template <>
// fp32: the double-precision exponential rounded once, so that a CPU restatement using the
// same recipe reproduces the value (expf differs between libraries in the last place)
__device__ __forceinline__ float ad_exp<float>(float x, const uint16_t*) { return (float)exp((double)x); }

struct AdaptiveArgs {
  const void* scores;      // [rows][S] unscaled q.k in dtype
  float scaling;
  const void* bias;
  int64_t bias_s_b, bias_s_h, bias_s_q;
  const uint32_t* prev_bits;  // null: previous mask empty or full (plain sum over all keys)
  const void* prev_data;
  const int32_t* wpre;
  const int64_t* ptr;
  int Hq, Sq;
  int64_t S, W, start, end, nb;
  uint64_t seed;
  const int64_t* base_draws;  // optional [rows][nb] columns; null: Philox(seed, row * nb + i)
  const uint16_t* exp_table;
  float delta_ppf, epsilon;
  int64_t* budget;
  void* prob;
  float* stats;  // optional [rows][4]: static denominator, std, estimated denominator, budget^2
};

// One CTA (1024 threads) per mask row.  Every tensor operation of the reference is one
// rounding to the dtype here; reductions use the fixed order above.
template <typename T>
__global__ void __launch_bounds__(1024)
adaptive_budget_kernel(AdaptiveArgs a) {
  sah_pdl_entry();
  extern __shared__ uint32_t ad_base_bits[];  // W words: distinct base-sample columns
  __shared__ float scratch[32];
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.x;
  const int qi = (int)(row % a.Sq);
  const int64_t bh = row / a.Sq;
  const int h = (int)(bh % a.Hq);
  const int64_t b = bh / a.Hq;
  const T* s = reinterpret_cast<const T*>(a.scores) + row * a.S;
  const T* bias = a.bias ? reinterpret_cast<const T*>(a.bias) + b * a.bias_s_b + h * a.bias_s_h +
                               qi * a.bias_s_q
                         : nullptr;
  const int64_t n = a.end - a.start;

  auto logit = [&](int64_t j) {
    float t = sah_round_to<T>(__fmul_rn(sah_to_float<T>(s[j]), a.scaling));
    if (bias) t = sah_round_to<T>(__fadd_rn(t, sah_to_float<T>(bias[j])));
    return t;
  };
  for (int64_t w = tid; w < a.W; w += 1024) ad_base_bits[w] = 0u;

  // 1. row maximum over all keys
  float mx = -INFINITY;
  for (int64_t j = tid; j < a.S; j += 1024) mx = fmaxf(mx, logit(j));
  mx = sah_block_max(mx, scratch);
  auto expw = [&](int64_t j) { return ad_exp<T>(sah_round_to<T>(__fsub_rn(logit(j), mx)), a.exp_table); };

  // 2. static denominator: exp weights of the previous mask under its inverse weights
  float part = 0.f;
  const float unit_w = sah_inv_weight<T>(1.f);
  const uint32_t* pb = a.prev_bits ? a.prev_bits + row * a.W : nullptr;
  for (int64_t j = tid; j < a.S; j += 1024) {
    float term = 0.f;
    if (pb == nullptr) {
      term = expw(j);
    } else {
      const uint32_t word = pb[j >> 5];
      const int bit = (int)(j & 31);
      if ((word >> bit) & 1u) {
        float w = unit_w;  // unit weights still pass through 1 / (1 + 1e-6)
        if (a.prev_data != nullptr) {
          const int64_t pos = a.ptr[row] + a.wpre[row * a.W + (j >> 5)] + __popc(word & ((1u << bit) - 1u));
          w = sah_inv_weight<T>(sah_to_float<T>(reinterpret_cast<const T*>(a.prev_data)[pos]));
        }
        term = sah_round_to<T>(__fmul_rn(expw(j), w));
      }
    }
    part = __fadd_rn(part, term);
  }
  const float static_den = sah_round_to<T>(sah_block_sum_fixed(part, scratch));

  // 3. base sample: unbiased standard deviation of the sampled exp weights
  auto base_col = [&](int64_t i) {
    return a.base_draws ? a.base_draws[row * a.nb + i]
                        : sah_draw_column(a.seed, (uint64_t)(row * a.nb + i), a.start, n);
  };
  part = 0.f;
  for (int64_t i = tid; i < a.nb; i += 1024) {
    const int64_t c = base_col(i);
    atomicOr(&ad_base_bits[c >> 5], 1u << (c & 31));
    part = __fadd_rn(part, expw(c));
  }
  const float mean = __fdiv_rn(sah_block_sum_fixed(part, scratch), (float)a.nb);
  part = 0.f;
  for (int64_t i = tid; i < a.nb; i += 1024) {
    const float d = __fsub_rn(expw(base_col(i)), mean);
    part = __fadd_rn(part, __fmul_rn(d, d));
  }
  const float var = __fdiv_rn(sah_block_sum_fixed(part, scratch), (float)(a.nb - 1));
  float sd = sah_round_to<T>(sqrtf(var));
  sd = fmaxf(sd, sah_round_to<T>(1e-8f));

  // 4. denominator estimate from the distinct base positions, weight 1 / (nb / n)
  const float p_base = sah_round_to<T>((float)((double)a.nb / (double)n));
  const float w_base = sah_inv_weight<T>(p_base);
  __syncthreads();
  part = 0.f;
  for (int64_t j = tid; j < a.S; j += 1024) {
    if ((ad_base_bits[j >> 5] >> (j & 31)) & 1u)
      part = __fadd_rn(part, sah_round_to<T>(__fmul_rn(expw(j), w_base)));
  }
  const float sampled_den = sah_round_to<T>(sah_block_sum_fixed(part, scratch));
  const float est_den = sah_round_to<T>(__fadd_rn(static_den, sampled_den));

  // 5. budget (adaptive_sampling.py:282-302, :394-397)
  if (tid == 0) {
    const float err = fmaxf(sah_round_to<T>(__fmul_rn(a.epsilon, est_den)), sah_round_to<T>(1e-8f));
    float num = sah_round_to<T>(__fmul_rn(a.delta_ppf, sd));
    num = sah_round_to<T>(__fmul_rn(num, (float)n));
    const float ratio = sah_round_to<T>(__fdiv_rn(num, err));
    float b2 = sah_round_to<T>(__fmul_rn(ratio, ratio));
    float clamped = fminf(fmaxf(b2, 1.0f), sah_round_to<T>((float)n));
    if (!(b2 == b2)) clamped = b2;  // NaN propagates as in the reference
    long long bud = (long long)clamped;  // truncation, as .long()
    if (bud < a.nb) bud = a.nb;
    if (bud > n) bud = n;
    a.budget[row] = bud;
    reinterpret_cast<T*>(a.prob)[row] = sah_from_float<T>(__fdiv_rn((float)bud, (float)n));
    if (a.stats) {
      a.stats[row * 4 + 0] = static_den;
      a.stats[row * 4 + 1] = sd;
      a.stats[row * 4 + 2] = est_den;
      a.stats[row * 4 + 3] = b2;
    }
  }
}

extern "C" int sah_adaptive_budget(const void* scores, int dtype, float scaling, const void* bias,
                                   int64_t bias_s_b, int64_t bias_s_h, int64_t bias_s_q,
                                   const uint32_t* prev_bits, const void* prev_data,
                                   const int32_t* wpre, const int64_t* ptr, int B, int Hq, int Sq,
                                   int64_t S, int64_t W, int64_t start, int64_t end, int64_t nb,
                                   uint64_t seed, const int64_t* base_draws,
                                   const uint16_t* exp_table, float delta_ppf, float epsilon,
                                   int64_t* budget, void* prob, float* stats, void* stream) {
  SAH_REQUIRE(scores && budget && prob, "adaptive_budget: null pointer");
  SAH_REQUIRE(B > 0 && Hq > 0 && Sq > 0 && S > 0 && W * 32 >= S, "adaptive_budget: bad extents");
  SAH_REQUIRE(0 <= start && start < end && end <= S && end - start >= 2 && nb >= 2,
              "adaptive_budget: bad sampling range");
  SAH_REQUIRE(end - start < (1ll << 32), "adaptive_budget: range too long");
  SAH_REQUIRE(prev_data == nullptr || (prev_bits && wpre && ptr), "adaptive_budget: data needs bits, wpre, ptr");
  SAH_REQUIRE(dtype != SAH_BF16 || exp_table != nullptr, "adaptive_budget: bf16 needs the exp table");
  AdaptiveArgs a;
  a.scores = scores; a.scaling = scaling; a.bias = bias;
  a.bias_s_b = bias_s_b; a.bias_s_h = bias_s_h; a.bias_s_q = bias_s_q;
  a.prev_bits = prev_bits; a.prev_data = prev_data; a.wpre = wpre; a.ptr = ptr;
  a.Hq = Hq; a.Sq = Sq; a.S = S; a.W = W; a.start = start; a.end = end; a.nb = nb;
  a.seed = seed; a.base_draws = base_draws; a.exp_table = exp_table;
  a.delta_ppf = delta_ppf; a.epsilon = epsilon; a.budget = budget; a.prob = prob; a.stats = stats;
  const size_t smem = (size_t)W * sizeof(uint32_t);
  if (smem > 200 * 1024)
    return sah_fail(SAH_ERR_UNSUPPORTED, "adaptive_budget: %lld keys per row exceed the base-sample bitmap",
                    (long long)S);
  const int64_t rows = (int64_t)B * Hq * Sq;
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_ADAPTIVE, st);
  SAH_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(adaptive_budget_kernel<T>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "adaptive_budget attr: %s", cudaGetErrorString(e));
    }
    sah_launch_chain(adaptive_budget_kernel<T>, (unsigned)rows, 1024, smem, st, a);
  });
  SAH_LAUNCH_CHECK("adaptive_budget");
  sah_prof_end(SAH_PROF_ADAPTIVE, st);
  return SAH_OK;
}

// sample j (0 <= j < sptr[rows]) belongs to the row r with sptr[r] <= j < sptr[r+1] and is
// the column pool[j], or start + floor(philox(seed, j) * n / 2^32) without a pool
// (create_sampling_mask_with_per_head_budget, utils/mask_attention_utils.py:145-173).
__global__ void sample_scatter_kernel(const int64_t* __restrict__ sptr, int64_t rows,
                                      const int64_t* __restrict__ pool, uint64_t seed,
                                      int64_t start, int64_t n, int64_t S, int64_t W,
                                      uint32_t* __restrict__ bits) {
  sah_pdl_entry_early();
  const int64_t total = sptr[rows];
  for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < total;
       j += (int64_t)gridDim.x * blockDim.x) {
    int64_t lo = 0, hi = rows;  // invariant: sptr[lo] <= j < sptr[hi]
    while (hi - lo > 1) {
      const int64_t mid = (lo + hi) >> 1;
      if (sptr[mid] <= j) lo = mid; else hi = mid;
    }
    const int64_t c = pool ? pool[j] : sah_draw_column(seed, (uint64_t)j, start, n);
    if (c >= 0 && c < S) atomicOr(bits + lo * W + (c >> 5), 1u << (c & 31));
  }
}

extern "C" int sah_sample_scatter(const int64_t* sptr, int64_t rows, const int64_t* pool,
                                  uint64_t seed, int64_t start, int64_t n, int64_t S, int64_t W,
                                  int sm_count, uint32_t* bits, void* stream) {
  SAH_REQUIRE(sptr && bits, "sample_scatter: null pointer");
  SAH_REQUIRE(rows >= 0 && n > 0 && n < (1ll << 32) && W * 32 >= S, "sample_scatter: bad extents");
  if (rows == 0) return SAH_OK;
  if (sm_count <= 0) sm_count = 148;
  sah_launch_chain(sample_scatter_kernel, (unsigned)(sm_count * 8), 256, 0, (cudaStream_t)stream, sptr, rows,
      pool, seed, start, n, S, W, bits);
  SAH_LAUNCH_CHECK("sample_scatter");
  return SAH_OK;
}

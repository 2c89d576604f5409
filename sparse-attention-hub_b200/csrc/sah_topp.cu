// Oracle top-p: the keys whose softmax weight reaches the row's threshold, the threshold being
// the sorted weight at which the cumulative mass passes top_p
// (research_attention/maskers/fixed/implementations/oracle_top_p.py:85-169).
//
// The reference sorts the exp weights of a row (bf16 values), takes a running sum in sorted
// order -- torch's CPU cumsum: one float32 accumulator, every prefix rounded to bf16 --
// normalises by the last prefix and searches for top_p.  The threshold is a value of the
// sorted list, so only sums at the ends of runs of equal values matter, and a bf16 weight in
// (0, 1] is one of 16256 bit patterns: a histogram over bit patterns replaces the sort, and
// one thread replays the accumulator over the non-empty bins from the largest value down.
// Inside a run the accumulator moves by a constant amount while it stays in one binade (two
// steps in after entering it, which also settles round-to-even ties), so the replay jumps to
// the end of the binade instead of adding one by one; once an add no longer changes the
// accumulator nothing smaller will, and the replay stops.
#include "sah_common.cuh"

#define TP_THREADS 1024
#define TP_BINS 16257            // bf16 bit patterns 0 .. 0x3F80 (0.0 .. 1.0)
#define TP_WORDS ((TP_BINS + 31) / 32)

struct ToppArgs {
  const void* scores;      // [rows][S] unscaled q.k in bf16
  float scaling;
  const void* bias;
  int64_t bias_s_b, bias_s_h, bias_s_q;
  const uint32_t* prev_bits;
  int Hq, Sq;
  int64_t S, W;
  float top_p;
  int or_prev;
  const uint16_t* exp_table;
  uint32_t* out_bits;
};

__device__ __forceinline__ float tp_block_max(float v, float* scratch32) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch32[threadIdx.x >> 5] = v;
  __syncthreads();
  float w = scratch32[threadIdx.x & 31];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, o));
  __syncthreads();
  return w;
}

// Adds `count` copies of v (> 0) to acc one after the other in float32; returns false when an
// add left acc unchanged (then no smaller value changes it either).
__device__ __forceinline__ bool tp_add_run(float& acc, float v, unsigned int count) {
  int same = 0;   // consecutive single steps that stayed in the binade they started in
  while (count > 0u) {
    const float next = __fadd_rn(acc, v);
    if (next == acc) return false;
    const bool stay = (__float_as_uint(next) >> 23) == (__float_as_uint(acc) >> 23);
    const float step = __fsub_rn(next, acc);   // exact when both lie in one binade
    acc = next;
    --count;
    same = stay ? same + 1 : 0;
    if (same >= 2 && count > 0u) {
      // acc is a multiple of the binade's spacing, `step` too; every further add moves acc by
      // `step` until it reaches the next power of two
      const float hi = __uint_as_float(((__float_as_uint(acc) >> 23) + 1u) << 23);
      double n = floor(((double)hi - (double)acc) / (double)step);
      if (n > (double)count) n = (double)count;
      acc = (float)((double)acc + n * (double)step);
      count -= (unsigned int)n;
      same = 0;
    }
  }
  return true;
}

__global__ void __launch_bounds__(TP_THREADS)
topp_select_kernel(ToppArgs a) {
  sah_pdl_entry();
  extern __shared__ unsigned int tp_hist[];   // [TP_BINS] counts, then the run-end sums
  __shared__ unsigned int nz[TP_WORDS];       // non-empty bins
  __shared__ float scratch[32];
  __shared__ float total_sm;
  __shared__ int stop_sm;                     // bins below it were not replayed: sum = total
  __shared__ int pick_sm, low_sm;
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.x;
  const int qi = (int)(row % a.Sq);
  const int64_t bh = row / a.Sq;
  const int h = (int)(bh % a.Hq);
  const int64_t b = bh / a.Hq;
  typedef __nv_bfloat16 T;
  const T* s = reinterpret_cast<const T*>(a.scores) + row * a.S;
  const T* bias = a.bias ? reinterpret_cast<const T*>(a.bias) + b * a.bias_s_b + h * a.bias_s_h +
                               qi * a.bias_s_q
                         : nullptr;
  const uint32_t* pb = a.prev_bits + row * a.W;
  const float lowest = __uint_as_float(0xFF7F0000u);   // the most negative finite bf16

  // scaled logit, previously active positions pushed to the lowest value (:96-104)
  auto logit = [&](int64_t j) {
    if ((pb[j >> 5] >> (j & 31)) & 1u) return lowest;
    float t = sah_round_to<T>(__fmul_rn(sah_to_float<T>(s[j]), a.scaling));
    if (bias) t = sah_round_to<T>(__fadd_rn(t, sah_to_float<T>(bias[j])));
    return t;
  };
  for (int i = tid; i < TP_BINS; i += TP_THREADS) tp_hist[i] = 0u;
  for (int i = tid; i < TP_WORDS; i += TP_THREADS) nz[i] = 0u;
  if (tid == 0) { pick_sm = -1; low_sm = TP_BINS; stop_sm = 0; }

  float mx = -INFINITY;
  for (int64_t j = tid; j < a.S; j += TP_THREADS) mx = fmaxf(mx, logit(j));
  mx = tp_block_max(mx, scratch);
  auto weight_bits = [&](int64_t j) {   // bf16 bits of exp(logit - max), 0 .. 0x3F80
    const float d = sah_round_to<T>(__fsub_rn(logit(j), mx));
    unsigned int e = a.exp_table[__float_as_uint(d) >> 16];
    return e > 0x3F80u ? 0x3F80u : e;   // not reached for finite logits
  };

  // histogram over bit patterns
  for (int64_t j = tid; j < a.S; j += TP_THREADS) atomicAdd(&tp_hist[weight_bits(j)], 1u);
  __syncthreads();
  for (int i = tid; i < TP_BINS; i += TP_THREADS)
    if (i > 0 && tp_hist[i] != 0u) atomicOr(&nz[i >> 5], 1u << (i & 31));
  __syncthreads();

  // replay of the accumulator, largest value first
  if (tid == 0) {
    float acc = 0.f;
    bool alive = true;
    int stop = 0;
    for (int wi = TP_WORDS - 1; wi >= 0 && alive; --wi) {
      unsigned int m = nz[wi];
      while (m) {
        const int bit = 31 - __clz(m);
        m &= ~(1u << bit);
        const int bin = wi * 32 + bit;
        alive = tp_add_run(acc, __uint_as_float((unsigned int)bin << 16), tp_hist[bin]);
        tp_hist[bin] = __float_as_uint(acc);
        if (!alive) { stop = bin; break; }
      }
    }
    total_sm = sah_round_to<T>(acc);
    stop_sm = stop;
  }
  __syncthreads();

  // first run (largest value) whose normalised prefix exceeds top_p (:118-131)
  const float total = total_sm;
  const float p = sah_round_to<T>(a.top_p);
  const int stop = stop_sm;
  int best = -1, low = TP_BINS;
  for (int i = tid; i < TP_BINS; i += TP_THREADS) {
    if (i == 0 || !((nz[i >> 5] >> (i & 31)) & 1u)) continue;
    low = min(low, i);
    const float sum = (i < stop) ? total : sah_round_to<T>(__uint_as_float(tp_hist[i]));
    const float ratio = sah_round_to<T>(__fdiv_rn(sum, total));
    if (ratio > p) best = max(best, i);
  }
  atomicMax(&pick_sm, best);
  atomicMin(&low_sm, low);
  __syncthreads();
  // nothing exceeds top_p: the search position is clamped to the last sorted element (:127-130)
  unsigned int thr;
  if (pick_sm >= 0) thr = (unsigned int)pick_sm;
  else thr = (tp_hist[0] != 0u || low_sm >= TP_BINS) ? 0u : (unsigned int)low_sm;

  // emit: weight >= threshold (:158-160)
  uint32_t* out = a.out_bits + row * a.W;
  for (int64_t w = tid; w < a.W; w += TP_THREADS) {
    uint32_t bits = 0u;
    const int64_t c0 = w * 32;
    for (int i = 0; i < 32; ++i) {
      const int64_t j = c0 + i;
      if (j < a.S && weight_bits(j) >= thr) bits |= 1u << i;
    }
    out[w] = a.or_prev ? (bits | pb[w]) : bits;
  }
}

extern "C" int sah_topp_select(const void* scores, int dtype, float scaling, const void* bias,
                               int64_t bias_s_b, int64_t bias_s_h, int64_t bias_s_q, int B, int Hq,
                               int Sq, int64_t S, int64_t W, const uint32_t* prev_bits, float top_p,
                               const uint16_t* exp_table, int or_prev, uint32_t* out_bits,
                               void* stream) {
  SAH_REQUIRE(scores && prev_bits && exp_table && out_bits, "topp_select: null pointer");
  SAH_REQUIRE(B > 0 && Hq > 0 && Sq > 0 && S > 0 && W * 32 >= S, "topp_select: bad extents");
  SAH_REQUIRE(top_p >= 0.f && top_p <= 1.f, "topp_select: top_p must be in [0, 1]");
  if (dtype != SAH_BF16)
    return sah_fail(SAH_ERR_UNSUPPORTED,
                    "topp_select: bfloat16 only (a float32 row is accumulated in float64 by the "
                    "reference over values that do not fall into a small set)");
  ToppArgs a;
  a.scores = scores; a.scaling = scaling; a.bias = bias;
  a.bias_s_b = bias_s_b; a.bias_s_h = bias_s_h; a.bias_s_q = bias_s_q;
  a.prev_bits = prev_bits; a.Hq = Hq; a.Sq = Sq; a.S = S; a.W = W; a.top_p = top_p;
  a.or_prev = or_prev; a.exp_table = exp_table; a.out_bits = out_bits;
  const int64_t rows = (int64_t)B * Hq * Sq;
  SAH_REQUIRE(rows <= 2147483647, "topp_select: too many rows");
  const int smem = TP_BINS * (int)sizeof(unsigned int);
  cudaError_t e = cudaFuncSetAttribute(topp_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "topp_select attr: %s", cudaGetErrorString(e));
  sah_prof_begin(SAH_PROF_TOPP, (cudaStream_t)stream);
  sah_launch_chain(topp_select_kernel, (unsigned)rows, TP_THREADS, smem, (cudaStream_t)stream, a);
  SAH_LAUNCH_CHECK("topp_select");
  sah_prof_end(SAH_PROF_TOPP, (cudaStream_t)stream);
  return SAH_OK;
}

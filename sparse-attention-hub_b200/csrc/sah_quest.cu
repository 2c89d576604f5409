// Quest page top-k (research_attention/maskers/fixed/implementations/quest_top_k.py:108-196,
// utils/quest_utils.py): per-page minimum and maximum of every key channel, an upper bound of
// q.k per page from them, top pages, pages expanded to keys.
//
// The page bounds are kept per KV head (the reference repeats the keys over the query heads of
// a group first, which repeats the bounds), as [B][Hkv][D/8][page capacity][8]: the scoring
// kernel has one thread per page, and with eight channels of consecutive pages next to each
// other its 16-byte loads are coalesced.  The bound is a sum over the head dimension of
// dtype-rounded products; it is taken in the order of the reference's CPU row reduction so that
// page scores, and with them the chosen pages, are the reference's bit for bit: float32
// accumulation in vectors of 8 lanes (a bfloat16 load brings 16 elements and adds its two
// halves), four interleaved vector accumulators added in order, then the lanes in order.
#include "sah_common.cuh"

// ---- page bounds ---------------------------------------------------------------------------
template <typename T>
__global__ void quest_minmax_kernel(const T* __restrict__ k, int64_t ks_b, int64_t ks_h, int64_t ks_s,
                                    int Hkv, int64_t S, int D, int page_size, int64_t page_begin,
                                    int64_t P_cap, T* __restrict__ pmin, T* __restrict__ pmax) {
  const int64_t page = page_begin + blockIdx.x;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int64_t s0 = page * page_size;
  const int64_t s1 = s0 + page_size < S ? s0 + page_size : S;
  const T* base = k + b * ks_b + h * ks_h;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float lo = INFINITY, hi = -INFINITY;
#pragma unroll 4
    for (int64_t s = s0; s < s1; ++s) {
      const float x = sah_to_float<T>(base[s * ks_s + d]);
      lo = fminf(lo, x);
      hi = fmaxf(hi, x);
    }
    const int64_t o = ((((b * Hkv + h) * (D / 8) + d / 8) * P_cap + page) << 3) + (d & 7);
    pmin[o] = sah_from_float<T>(lo);
    pmax[o] = sah_from_float<T>(hi);
  }
}

extern "C" int sah_quest_page_minmax(const void* k, int dtype, int64_t ks_b, int64_t ks_h, int64_t ks_s,
                                     int B, int Hkv, int64_t S, int D, int page_size,
                                     int64_t page_begin, int64_t P_cap, void* pmin, void* pmax,
                                     void* stream) {
  SAH_REQUIRE(k && pmin && pmax, "quest_page_minmax: null pointer");
  SAH_REQUIRE(B > 0 && Hkv > 0 && S > 0 && D > 0 && D % 8 == 0 && page_size > 0,
              "quest_page_minmax: bad extents (the head dimension must be a multiple of 8)");
  const int64_t P = sah_ceil_div(S, page_size);
  SAH_REQUIRE(page_begin >= 0 && page_begin <= P && P <= P_cap, "quest_page_minmax: bad page range");
  SAH_REQUIRE(Hkv <= 65535 && B <= 65535, "quest_page_minmax: too many heads or batches");
  if (page_begin == P) return SAH_OK;
  dim3 grid((unsigned)(P - page_begin), (unsigned)Hkv, (unsigned)B);
  const int threads = D >= 256 ? 256 : ((D + 31) / 32) * 32;
  SAH_DISPATCH_DTYPE(dtype, T, {
    quest_minmax_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const T*)k, ks_b, ks_h, ks_s, Hkv, S, D, page_size, page_begin, P_cap, (T*)pmin, (T*)pmax);
  });
  SAH_LAUNCH_CHECK("quest_page_minmax");
  return SAH_OK;
}

// ---- page scores ---------------------------------------------------------------------------
#define QS_THREADS 128
#define QS_MAXD 512

template <typename T>
struct QuestVec {  // elements one vector load of the reference's reduction brings
  static constexpr int N = sizeof(T) == 2 ? 16 : 8;
};

template <typename T>
__global__ void __launch_bounds__(QS_THREADS)
quest_scores_kernel(const T* __restrict__ q, int64_t qs_b, int64_t qs_h, int64_t qs_q,
                    const T* __restrict__ pmin, const T* __restrict__ pmax, int64_t P_cap, int Hq,
                    int Hkv, int Sq, int64_t S, int D, int page_size, const T* __restrict__ bias,
                    int64_t bias_s_b, int64_t bias_s_q, T* __restrict__ scores) {
  sah_pdl_entry();
  __shared__ float q_sm[QS_MAXD];
  const int64_t row = blockIdx.y;
  const int qi = (int)(row % Sq);
  const int64_t bh = row / Sq;
  const int h = (int)(bh % Hq);
  const int64_t b = bh / Hq;
  const int kvh = h / (Hq / Hkv);
  const T* qr = q + b * qs_b + h * qs_h + qi * qs_q;
  for (int d = threadIdx.x; d < D; d += QS_THREADS) q_sm[d] = sah_to_float<T>(qr[d]);
  __syncthreads();
  const int64_t P = (S + page_size - 1) / page_size;
  const int64_t page = (int64_t)blockIdx.x * QS_THREADS + threadIdx.x;
  if (page >= P) return;
  // chunk c (channels 8c .. 8c+7) of this page: base + (c * P_cap + page) * 8
  const T* lo = pmin + (b * Hkv + kvh) * (int64_t)D * P_cap + page * 8;
  const T* hi = pmax + (b * Hkv + kvh) * (int64_t)D * P_cap + page * 8;
  const int64_t cstride = P_cap * 8;

  constexpr int VEC = QuestVec<T>::N;
  const int nv = D / VEC;
  const int full = nv / 4;
  float acc[4][8];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
#pragma unroll
    for (int l = 0; l < 8; ++l) acc[kk][l] = 0.f;

  // the 8 lane values one vector load contributes: max(q*lo, q*hi), products rounded to T
  auto load_vec = [&](int v, float* out) {
    float a[8], c[8];
#pragma unroll
    for (int half = 0; half < VEC / 8; ++half) {
      const int j0 = v * VEC + half * 8;
      sah_load8<T>(lo + (j0 >> 3) * cstride, a);
      sah_load8<T>(hi + (j0 >> 3) * cstride, c);
#pragma unroll
      for (int l = 0; l < 8; ++l) {
        const float qv = q_sm[j0 + l];
        const float m = fmaxf(sah_round_to<T>(__fmul_rn(qv, a[l])), sah_round_to<T>(__fmul_rn(qv, c[l])));
        out[l] = half == 0 ? m : __fadd_rn(out[l], m);   // a bf16 load adds its two halves
      }
    }
  };
  for (int i = 0; i < full; ++i) {
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      float val[8];
      load_vec(i * 4 + kk, val);
#pragma unroll
      for (int l = 0; l < 8; ++l) acc[kk][l] = __fadd_rn(acc[kk][l], val[l]);
    }
  }
  for (int v = full * 4; v < nv; ++v) {
    float val[8];
    load_vec(v, val);
#pragma unroll
    for (int l = 0; l < 8; ++l) acc[0][l] = __fadd_rn(acc[0][l], val[l]);
  }
#pragma unroll
  for (int kk = 1; kk < 4; ++kk)
#pragma unroll
    for (int l = 0; l < 8; ++l) acc[0][l] = __fadd_rn(acc[0][l], acc[kk][l]);
  float fin = 0.f;
  for (int j = nv * VEC; j < D; ++j) {   // elements past the last whole vector come first
    const float qv = q_sm[j];
    const int64_t o = (j >> 3) * cstride + (j & 7);
    const float m = fmaxf(sah_round_to<T>(__fmul_rn(qv, sah_to_float<T>(lo[o]))),
                          sah_round_to<T>(__fmul_rn(qv, sah_to_float<T>(hi[o]))));
    fin = __fadd_rn(fin, m);
  }
#pragma unroll
  for (int l = 0; l < 8; ++l) fin = __fadd_rn(fin, acc[0][l]);
  float sc = sah_round_to<T>(fin);

  if (bias != nullptr) {   // a page none of whose keys is allowed scores the lowest value
    const T* br = bias + b * bias_s_b + qi * bias_s_q;
    const int64_t s0 = page * page_size;
    const int64_t s1 = s0 + page_size < S ? s0 + page_size : S;
    bool any = false;
    for (int64_t s = s0; s < s1 && !any; ++s) any = sah_to_float<T>(br[s]) >= 0.f;
    if (!any) sc = sizeof(T) == 2 ? __uint_as_float(0xFF7F0000u) : -3.402823466e38f;
  }
  scores[row * P + page] = sah_from_float<T>(sc);
}

extern "C" int sah_quest_scores(const void* q, int dtype, int64_t qs_b, int64_t qs_h, int64_t qs_q,
                                const void* pmin, const void* pmax, int64_t P_cap, int B, int Hq,
                                int Hkv, int Sq, int64_t S, int D, int page_size, const void* bias,
                                int64_t bias_s_b, int64_t bias_s_h, int64_t bias_s_q, void* scores,
                                void* stream) {
  SAH_REQUIRE(q && pmin && pmax && scores, "quest_scores: null pointer");
  SAH_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Sq > 0 && S > 0 && page_size > 0,
              "quest_scores: bad extents");
  if (D % 8 != 0 || D > QS_MAXD)
    return sah_fail(SAH_ERR_UNSUPPORTED, "quest_scores: head dimension %d (multiples of 8 up to %d)", D,
                    QS_MAXD);
  if (bias != nullptr && bias_s_h != 0)
    return sah_fail(SAH_ERR_UNSUPPORTED, "quest_scores: the attention mask must be shared by the heads");
  const int64_t P = sah_ceil_div(S, page_size);
  SAH_REQUIRE(P <= P_cap, "quest_scores: page capacity below the page count");
  SAH_REQUIRE(((uintptr_t)pmin & 15) == 0 && ((uintptr_t)pmax & 15) == 0, "quest_scores: bounds must be 16-byte aligned");
  const int64_t rows = (int64_t)B * Hq * Sq;
  SAH_REQUIRE(rows <= 65535, "quest_scores: more than 65535 mask rows");
  dim3 grid((unsigned)sah_ceil_div(P, QS_THREADS), (unsigned)rows);
  sah_prof_begin(SAH_PROF_QUEST, (cudaStream_t)stream);
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(quest_scores_kernel<T>, grid, QS_THREADS, 0, (cudaStream_t)stream, (const T*)q, qs_b,
        qs_h, qs_q, (const T*)pmin, (const T*)pmax, P_cap, Hq, Hkv, Sq, S, D, page_size,
        (const T*)bias, bias_s_b, bias_s_q, (T*)scores);
  });
  SAH_LAUNCH_CHECK("quest_scores");
  sah_prof_end(SAH_PROF_QUEST, (cudaStream_t)stream);
  return SAH_OK;
}

// ---- chosen pages -> key bitmap --------------------------------------------------------------
template <typename T>
__global__ void quest_expand_kernel(const uint32_t* __restrict__ page_bits, int64_t Wp,
                                    const uint32_t* __restrict__ prev_bits, const T* __restrict__ bias,
                                    int64_t bias_s_b, int64_t bias_s_q, int Hq, int Sq, int64_t S,
                                    int64_t W, int page_size, uint32_t* __restrict__ out_bits) {
  sah_pdl_entry_early();
  const int64_t row = blockIdx.y;
  const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= W) return;
  const uint32_t* pg = page_bits + row * Wp;
  uint32_t bits = 0u;
  const int64_t c0 = w * 32;
  if (page_size % 32 == 0) {   // the word lies inside one page
    const int64_t page = c0 / page_size;
    if (c0 < S && ((pg[page >> 5] >> (page & 31)) & 1u)) bits = 0xffffffffu;
  } else {
#pragma unroll 4
    for (int i = 0; i < 32; ++i) {
      const int64_t page = (c0 + i) / page_size;
      if (c0 + i < S && ((pg[page >> 5] >> (page & 31)) & 1u)) bits |= 1u << i;
    }
  }
  if (c0 + 32 > S) bits &= (c0 >= S) ? 0u : ((1u << (S - c0)) - 1u);
  if (prev_bits != nullptr) bits |= prev_bits[row * W + w];
  if (bias != nullptr && bits) {   // keys the attention mask forbids leave the mask (:188-191)
    const int qi = (int)(row % Sq);
    const int64_t b = row / Sq / Hq;
    const T* br = bias + b * bias_s_b + qi * bias_s_q;
    uint32_t allowed = 0u;
    for (int i = 0; i < 32; ++i)
      if (c0 + i < S && sah_to_float<T>(br[c0 + i]) >= 0.f) allowed |= 1u << i;
    bits &= allowed;
  }
  out_bits[row * W + w] = bits;
}

extern "C" int sah_quest_expand(const uint32_t* page_bits, int64_t Wp, const uint32_t* prev_bits,
                                const void* bias, int dtype, int64_t bias_s_b, int64_t bias_s_h,
                                int64_t bias_s_q, int B, int Hq, int Sq, int64_t S, int64_t W,
                                int page_size, uint32_t* out_bits, void* stream) {
  SAH_REQUIRE(page_bits && out_bits, "quest_expand: null pointer");
  SAH_REQUIRE(B > 0 && Hq > 0 && Sq > 0 && S > 0 && W * 32 >= S && page_size > 0, "quest_expand: bad extents");
  SAH_REQUIRE(Wp * 32 >= sah_ceil_div(S, page_size), "quest_expand: page bitmap too short");
  if (bias != nullptr && bias_s_h != 0)
    return sah_fail(SAH_ERR_UNSUPPORTED, "quest_expand: the attention mask must be shared by the heads");
  const int64_t rows = (int64_t)B * Hq * Sq;
  SAH_REQUIRE(rows <= 65535, "quest_expand: more than 65535 mask rows");
  dim3 grid((unsigned)sah_ceil_div(W, 256), (unsigned)rows);
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(quest_expand_kernel<T>, grid, 256, 0, (cudaStream_t)stream, page_bits, Wp, prev_bits,
        (const T*)bias, bias_s_b, bias_s_q, Hq, Sq, S, W, page_size, out_bits);
  });
  SAH_LAUNCH_CHECK("quest_expand");
  return SAH_OK;
}

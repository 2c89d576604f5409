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
#define QK_STAGES 1
#define QK_TILES_PER_CTA 1

// Two of those at once: sm_100 issues a pair of fp32 operations per instruction
// (fma.rn.f32x2), each lane rounding exactly as the scalar fma; used for bf16 inputs, whose
// products are exact in fp32.
template <typename T>
__device__ __forceinline__ void qk_mac2(float& c0, float& c1, float a0, float a1, float b0, float b1);
template <>
__device__ __forceinline__ void qk_mac2<__nv_bfloat16>(float& c0, float& c1, float a0, float a1,
                                                       float b0, float b1) {
  unsigned long long a, b, c;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(b0), "f"(b1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(c) : "f"(c0), "f"(c1));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(a), "l"(b));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(c0), "=f"(c1) : "l"(c));
}
template <>
__device__ __forceinline__ void qk_mac2<float>(float& c0, float& c1, float a0, float a1, float b0,
                                               float b1) {
  // fp32 inputs: a rounded product, then a rounded sum (no fma), one lane at a time
  c0 = __fadd_rn(c0, __fmul_rn(a0, b0));
  c1 = __fadd_rn(c1, __fmul_rn(a1, b1));
}

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

// DT: head dim known at compile time (0: use the runtime value); FULL4: the number of rows
// per KV head is a multiple of 4, so no row needs a bounds test.  Both only remove
// instructions; the arithmetic is the same.
template <typename T, int DT, bool FULL4>
__global__ void __launch_bounds__(QK_THREADS, 5)
qk_scores_kernel(const T* __restrict__ q, const T* __restrict__ k, int64_t qs_b, int64_t qs_h,
                 int64_t qs_q, int64_t ks_b, int64_t ks_h, int64_t ks_s, int Hq, int Hkv, int Sq,
                 int64_t S, int D_rt, const T* __restrict__ bias, int64_t bias_s_b,
                 int64_t bias_s_h, int64_t bias_s_q, T* __restrict__ scores) {
  sah_pdl_entry();
  extern __shared__ __align__(16) float q_sm[];  // [R][D] queries, then the K tile
  const int D = DT ? DT : D_rt;
  const int G = Hq / Hkv;
  const int R = G * Sq;  // rows sharing this KV head
  const int kvh = blockIdx.y, b = blockIdx.z;
  // The CTA's QK_THREADS keys are copied to shared memory with coalesced 16-byte cp.async
  // (a thread walking its own row in global memory would touch a new 128-byte line per
  // load); rows are padded by 16 bytes so that the per-thread row reads do not collide.
  const int row_bytes = D * (int)sizeof(T);
  const int row_stride = row_bytes + 16;
  const int stage_bytes = QK_THREADS * row_stride;
  unsigned char* k_sm = reinterpret_cast<unsigned char*>(q_sm + R * D);  // QK_STAGES tiles
  const int64_t n_tiles = (S + QK_THREADS - 1) / QK_THREADS;
  const int64_t t_first = (int64_t)blockIdx.x * QK_TILES_PER_CTA;
  const int64_t t_last = t_first + QK_TILES_PER_CTA < n_tiles ? t_first + QK_TILES_PER_CTA : n_tiles;
  const int cpr = row_bytes / 16;
  const unsigned char* kbase = reinterpret_cast<const unsigned char*>(k + b * ks_b + kvh * ks_h);
  const int64_t src_stride = ks_s * (int64_t)sizeof(T);
  const uint32_t sm0 = (uint32_t)__cvta_generic_to_shared(k_sm);
  auto issue = [&](int64_t tile, int stage) {
    const int64_t j0 = tile * QK_THREADS;
    const int nkeys = (int)(S - j0 < QK_THREADS ? S - j0 : QK_THREADS);
    const unsigned char* src = kbase + j0 * src_stride;
    const uint32_t dst0 = sm0 + stage * stage_bytes;
    for (int c = threadIdx.x; c < nkeys * cpr; c += QK_THREADS) {
      const int row = c / cpr, col = c - row * cpr;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst0 + row * row_stride + col * 16),
                   "l"(src + row * src_stride + col * 16));
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  if (t_first < t_last) issue(t_first, 0);
  // Stage the group's queries as fp32: row r = g * Sq + qi.
  for (int idx = threadIdx.x; idx < R * D; idx += QK_THREADS) {
    int r = idx / D, d = idx - r * D;
    int g = r / Sq, qi = r - g * Sq;
    q_sm[idx] = sah_to_float<T>(q[b * qs_b + (int64_t)(kvh * G + g) * qs_h + qi * qs_q + d]);
  }
  const int chunks = D / 8;
  for (int64_t tile = t_first; tile < t_last; ++tile) {
    const int stage = (int)((tile - t_first) & 1);
    if (tile + 1 < t_last) {
      issue(tile + 1, stage ^ 1);  // the other stage was released by the barrier below
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const int64_t j = tile * QK_THREADS + threadIdx.x;
    if (j < S) {
      const T* kr = reinterpret_cast<const T*>(k_sm + stage * stage_bytes + threadIdx.x * row_stride);
      for (int r0 = 0; r0 < R; r0 += 4) {
        float acc[4][8];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[r][i] = 0.f;
#pragma unroll(DT ? 4 : 1)
        for (int t = 0; t < chunks; ++t) {
          float kf[8];
          sah_load8<T>(kr + t * 8, kf);
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            if (FULL4 || r0 + r < R) {
              const float4 qa = *reinterpret_cast<const float4*>(q_sm + (r0 + r) * D + t * 8);
              const float4 qb = *reinterpret_cast<const float4*>(q_sm + (r0 + r) * D + t * 8 + 4);
              qk_mac2<T>(acc[r][0], acc[r][1], qa.x, qa.y, kf[0], kf[1]);
              qk_mac2<T>(acc[r][2], acc[r][3], qa.z, qa.w, kf[2], kf[3]);
              qk_mac2<T>(acc[r][4], acc[r][5], qb.x, qb.y, kf[4], kf[5]);
              qk_mac2<T>(acc[r][6], acc[r][7], qb.z, qb.w, kf[6], kf[7]);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          if (FULL4 || r0 + r < R) {
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
    __syncthreads();  // the tile may be overwritten by the copy issued two iterations on
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
  const size_t elt = dtype == SAH_BF16 ? 2 : 4;
  const size_t smem = (size_t)R * D * sizeof(float) + (size_t)QK_STAGES * QK_THREADS * (D * elt + 16);
  if (smem > 200 * 1024)
    return sah_fail(SAH_ERR_UNSUPPORTED, "qk_scores: %d query rows per KV head do not fit", R);
  dim3 grid((unsigned)sah_ceil_div(sah_ceil_div(S, QK_THREADS), QK_TILES_PER_CTA), (unsigned)Hkv, (unsigned)B);
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_QK_SCORES, (cudaStream_t)stream);
#define QK_LAUNCH(T, DT, F4)                                                                        \
  do {                                                                                              \
    if (smem > 48 * 1024) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(qk_scores_kernel<T, DT, F4>,                             \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "qk_scores attr: %s", cudaGetErrorString(e)); \
    }                                                                                               \
    sah_launch_chain(qk_scores_kernel<T, DT, F4>, grid, QK_THREADS, smem, st, \
        (const T*)q, (const T*)k, qs_b, qs_h, qs_q, ks_b, ks_h, ks_s, Hq, Hkv, Sq, S, D,            \
        (const T*)bias, bias_s_b, bias_s_h, bias_s_q, (T*)scores);                                  \
  } while (0)
  const bool full4 = (R % 4) == 0;
  SAH_DISPATCH_DTYPE(dtype, T, {
    if (D == 128 && full4) QK_LAUNCH(T, 128, true);
    else if (D == 64 && full4) QK_LAUNCH(T, 64, true);
    else QK_LAUNCH(T, 0, false);
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
  sah_pdl_entry();
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
    sah_launch_chain(topk_select_kernel<__nv_bfloat16, 16>, (unsigned)rows, SAH_SELECT_THREADS, 0, st,
        (const __nv_bfloat16*)scores, S, W, col_begin, col_end, prev_bits, k, out_bits);
  } else if (dtype == SAH_F32) {
    sah_launch_chain(topk_select_kernel<float, 32>, (unsigned)rows, SAH_SELECT_THREADS, 0, st,
        (const float*)scores, S, W, col_begin, col_end, prev_bits, k, out_bits);
  } else {
    return sah_fail(SAH_ERR_INVALID, "topk_select: unknown dtype %d", dtype);
  }
  SAH_LAUNCH_CHECK("topk_select");
  sah_prof_end(SAH_PROF_TOPK_SELECT, (cudaStream_t)stream);
  return SAH_OK;
}

// ---------------------------------------------------------------------------
// The same exact top-k with every row spread over many CTAs (long rows, few rows).
//
// A row is cut into chunks of SEL_CHUNK_WORDS bitmap words; a CTA histograms one chunk of
// one row for the current 8-bit digit (most significant first), the chunk histograms add up
// in global memory, one CTA per row picks the digit where the descending count reaches k,
// and so on for KEYBITS / 8 digits.  The last digit's per-chunk histograms also tell how
// many keys equal to the threshold each chunk holds, which orders the ties by column
// across chunks.  The emit pass writes prev | {key > T} | first `need` keys == T.
// State lives in a caller-provided workspace; nothing is read back by the host.
// ---------------------------------------------------------------------------
#define SEL_CHUNK_WORDS 256
#define SEL_THREADS 256

struct SelState {
  unsigned int prefix, pmask;
  long long need;
  int mode;  // 0: threshold found / being refined, 1: every candidate, 2: none
  int pad;
};

struct SelWorkspace {
  SelState* state;          // [rows]
  unsigned int* hist;       // [rows][256]
  unsigned int* chunk_hist; // [rows][chunks][256]
  long long* chunk_before;  // [rows][chunks]
};

static size_t sel_ws_bytes(int64_t rows, int64_t chunks) {
  return (size_t)rows * sizeof(SelState) + (size_t)rows * 256 * 4 + (size_t)rows * chunks * 256 * 4 +
         (size_t)rows * chunks * 8;
}

static SelWorkspace sel_ws_carve(void* ws, int64_t rows, int64_t chunks) {
  SelWorkspace o;
  unsigned char* p = reinterpret_cast<unsigned char*>(ws);
  o.chunk_before = reinterpret_cast<long long*>(p);
  p += (size_t)rows * chunks * 8;
  o.state = reinterpret_cast<SelState*>(p);
  p += (size_t)rows * sizeof(SelState);
  o.hist = reinterpret_cast<unsigned int*>(p);
  p += (size_t)rows * 256 * 4;
  o.chunk_hist = reinterpret_cast<unsigned int*>(p);
  return o;
}

__global__ void sel_init_kernel(SelState* state, unsigned int* hist, int64_t rows, long long k) {
  sah_pdl_entry_early();
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < rows * 256) hist[t] = 0u;
  if (t < rows) {
    SelState s;
    s.prefix = 0u; s.pmask = 0u; s.need = k; s.mode = k <= 0 ? 2 : 0; s.pad = 0;
    state[t] = s;
  }
}

// keys of the 32 columns of bitmap word w of a row, as order-preserving integers
template <typename T, int KEYBITS>
__device__ __forceinline__ void sel_load_keys(const T* __restrict__ srow, int64_t w, int64_t S,
                                              bool vec, unsigned int* keys) {
  const int64_t c0 = w * 32;
  if (vec && c0 + 32 <= S) {
    float f[32];
    if (sizeof(T) == 2) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        sah_unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(srow) + c0 + i * 8), f + i * 8);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(srow) + c0 + i * 4);
        f[i * 4] = v.x; f[i * 4 + 1] = v.y; f[i * 4 + 2] = v.z; f[i * 4 + 3] = v.w;
      }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const unsigned int key = sah_float_key(f[i] + 0.0f);
      keys[i] = KEYBITS == 16 ? (key >> 16) : key;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      unsigned int key = 0u;
      if (c0 + i < S) key = sah_float_key(sah_to_float<T>(srow[c0 + i]) + 0.0f);
      keys[i] = KEYBITS == 16 ? (key >> 16) : key;
    }
  }
}

// candidate columns of word w: inside [col_begin, col_end) and [0, S), not in prev
__device__ __forceinline__ uint32_t sel_valid(uint32_t pw, int64_t w, int64_t col_begin, int64_t col_end) {
  const int64_t c0 = w * 32;
  uint32_t m = ~pw;
  if (col_begin > c0) m &= (col_begin >= c0 + 32) ? 0u : ~((1u << (col_begin - c0)) - 1u);
  if (col_end < c0 + 32) m &= (col_end <= c0) ? 0u : ((1u << (col_end - c0)) - 1u);
  return m;
}

template <typename T, int KEYBITS>
__global__ void __launch_bounds__(SEL_THREADS)
sel_hist_kernel(const T* __restrict__ scores, int64_t S, int64_t W, int64_t col_begin, int64_t col_end,
                const uint32_t* __restrict__ prev_bits, const SelState* __restrict__ state,
                unsigned int* __restrict__ hist, unsigned int* __restrict__ chunk_hist, int64_t chunks,
                int shift, int vec) {
  sah_pdl_entry();
  __shared__ unsigned int hs[SEL_THREADS / 32][256];
  const int tid = threadIdx.x, warp = tid >> 5;
  const int64_t row = blockIdx.y, chunk = blockIdx.x;
  const SelState st = state[row];
  if (st.mode != 0) return;  // the whole CTA leaves together
  for (int i = tid; i < (SEL_THREADS / 32) * 256; i += SEL_THREADS) (&hs[0][0])[i] = 0u;
  __syncthreads();
  const int64_t w = chunk * SEL_CHUNK_WORDS + tid;
  if (w < W) {
    const uint32_t valid = sel_valid(prev_bits[row * W + w], w, col_begin, col_end);
    if (valid) {
      unsigned int keys[32];
      sel_load_keys<T, KEYBITS>(scores + row * S, w, S, vec != 0, keys);
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (((valid >> i) & 1u) && (keys[i] & st.pmask) == st.prefix)
          atomicAdd(&hs[warp][(keys[i] >> shift) & 255u], 1u);
    }
  }
  __syncthreads();
  unsigned int sum = 0u;
#pragma unroll
  for (int i = 0; i < SEL_THREADS / 32; ++i) sum += hs[i][tid];
  if (sum) atomicAdd(&hist[row * 256 + tid], sum);
  if (chunk_hist != nullptr) chunk_hist[(row * chunks + chunk) * 256 + tid] = sum;
}

__global__ void __launch_bounds__(256)
sel_pick_kernel(SelState* __restrict__ state, unsigned int* __restrict__ hist, int shift, int first,
                const unsigned int* __restrict__ chunk_hist, long long* __restrict__ chunk_before,
                int64_t chunks, long long* __restrict__ eq_total_out) {
  sah_pdl_entry_early();
  __shared__ long long scan[33];
  __shared__ int bin_sm;
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.x;
  SelState st = state[row];
  // thread t looks at bin 255 - t: the exclusive scan in thread order is the count above the bin
  const int bin = 255 - tid;
  const long long cnt = hist[row * 256 + bin];
  hist[row * 256 + bin] = 0u;  // ready for the next digit
  if (eq_total_out != nullptr && tid == 0) eq_total_out[row] = 0;
  if (st.mode != 0) return;
  long long total;
  const long long above = sah_block_excl_scan<long long>(cnt, scan, &total);
  if (tid == 0) bin_sm = -1;
  __syncthreads();
  if (total < st.need || (first && total <= st.need)) {
    if (tid == 0) { st.mode = 1; state[row] = st; }
    return;
  }
  if (above < st.need && above + cnt >= st.need) {
    st.prefix |= (unsigned int)bin << shift;
    st.pmask |= 255u << shift;
    st.need -= above;
    state[row] = st;
    bin_sm = bin;
  }
  if (chunk_hist == nullptr) return;
  __syncthreads();
  // ties: keys equal to the threshold in the chunks before each chunk
  const int tb = bin_sm;
  long long base = 0;
  for (int64_t c0 = 0; c0 < chunks; c0 += 256) {
    const int64_t c = c0 + tid;
    const long long e = c < chunks ? (long long)chunk_hist[(row * chunks + c) * 256 + tb] : 0;
    long long tot;
    const long long ex = sah_block_excl_scan<long long>(e, scan, &tot);
    if (c < chunks) chunk_before[row * chunks + c] = base + ex;
    base += tot;
  }
  // keys equal to the threshold in this rank's range (ties are served to lower ranks first)
  if (eq_total_out != nullptr && tid == 0) eq_total_out[row] = base;
}

template <typename T, int KEYBITS>
__global__ void __launch_bounds__(SEL_THREADS)
sel_emit_kernel(const T* __restrict__ scores, int64_t S, int64_t W, int64_t col_begin, int64_t col_end,
                const uint32_t* __restrict__ prev_bits, const SelState* __restrict__ state,
                const long long* __restrict__ chunk_before, int64_t chunks, int vec,
                const long long* __restrict__ tie_offset, uint32_t* __restrict__ out_bits) {
  sah_pdl_entry();
  __shared__ long long scan[33];
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.y, chunk = blockIdx.x;
  const SelState st = state[row];
  const int64_t w = chunk * SEL_CHUNK_WORDS + tid;
  uint32_t pw = 0u, gt = 0u, eq = 0u;
  if (w < W) {
    pw = prev_bits[row * W + w];
    const uint32_t valid = sel_valid(pw, w, col_begin, col_end);
    if (st.mode == 1) {
      gt = valid;
    } else if (st.mode == 0 && valid) {
      unsigned int keys[32];
      sel_load_keys<T, KEYBITS>(scores + row * S, w, S, vec != 0, keys);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        gt |= (keys[i] > st.prefix ? 1u : 0u) << i;
        eq |= (keys[i] == st.prefix ? 1u : 0u) << i;
      }
      gt &= valid;
      eq &= valid;
    }
  }
  long long total;
  const long long before = sah_block_excl_scan<long long>((long long)__popc(eq), scan, &total);
  if (w < W) {
    const long long lower = tie_offset != nullptr ? tie_offset[row] : 0;  // ties taken by lower ranks
    const long long quota = st.need - (lower + chunk_before[row * chunks + chunk] + before);
    const int take = st.mode != 0 ? 0 : (quota > 32 ? 32 : (quota < 0 ? 0 : (int)quota));
    out_bits[row * W + w] = pw | gt | sah_lowest_bits(eq, take);
  }
}

// ---------------------------------------------------------------------------
// One-rank form of the same selection without state kernels: every CTA derives the threshold
// found so far from the chunk histograms of the digits already counted (a few hundred loads),
// so a selection is one launch per digit plus the emit -- 3 launches for bfloat16 keys instead
// of 6.  A row is cut into at most SELF_MAX_CHUNKS chunks (a multiple of 256 words each); the
// chunk histograms are plain stores, nothing has to be zeroed between calls.
// ---------------------------------------------------------------------------
#define SELF_MAX_CHUNKS 32

struct SelFusedGeom {
  int64_t chunk_words;
  int chunks;
};
static SelFusedGeom sel_fused_geom(int64_t W) {
  SelFusedGeom g;
  int64_t cw = (W + SELF_MAX_CHUNKS - 1) / SELF_MAX_CHUNKS;
  cw = (cw + SEL_THREADS - 1) / SEL_THREADS * SEL_THREADS;
  if (cw < SEL_THREADS) cw = SEL_THREADS;
  g.chunk_words = cw;
  g.chunks = (int)((W + cw - 1) / cw);
  return g;
}
static size_t sel_fused_ws_bytes(int64_t rows, int64_t W) {
  return (size_t)4 * rows * sel_fused_geom(W).chunks * 256 * sizeof(unsigned int);
}

// The selection state after the first `ndig` digits, replayed from their chunk histograms
// ch[digit][row][chunk][256].  Called by all SEL_THREADS threads; the result is uniform.
template <int KEYBITS>
__device__ SelState sel_replay(const unsigned int* __restrict__ ch, int64_t rows, int64_t row, int chunks,
                               int ndig, long long k, long long* scan, SelState* st_sm) {
  const int tid = threadIdx.x;
  if (tid == 0) {
    SelState s0;
    s0.prefix = 0u; s0.pmask = 0u; s0.need = k; s0.mode = k <= 0 ? 2 : 0; s0.pad = 0;
    *st_sm = s0;
  }
  __syncthreads();
  for (int d = 0; d < ndig; ++d) {
    SelState st = *st_sm;
    __syncthreads();  // everyone holds the state before anyone replaces it
    if (st.mode != 0) break;
    const int shift = KEYBITS - 8 * (d + 1);
    const int bin = 255 - tid;  // the exclusive scan in thread order counts the keys above the bin
    const unsigned int* hp = ch + (((int64_t)d * rows + row) * chunks) * 256 + bin;
    long long cnt = 0;
    for (int c = 0; c < chunks; ++c) cnt += hp[(int64_t)c * 256];
    long long total;
    const long long above = sah_block_excl_scan<long long>(cnt, scan, &total);
    if (total < st.need || (d == 0 && total <= st.need)) {
      if (tid == 0) st_sm->mode = 1;  // every candidate is selected
    } else if (above < st.need && above + cnt >= st.need) {
      st.prefix |= (unsigned int)bin << shift;
      st.pmask |= 255u << shift;
      st.need -= above;
      *st_sm = st;
    }
    __syncthreads();
  }
  const SelState out = *st_sm;
  __syncthreads();
  return out;
}

template <typename T, int KEYBITS>
__global__ void __launch_bounds__(SEL_THREADS)
sel_fused_hist_kernel(const T* __restrict__ scores, int64_t S, int64_t W, int64_t col_begin, int64_t col_end,
                      const uint32_t* __restrict__ prev_bits, long long k, unsigned int* __restrict__ ch,
                      int64_t rows, int chunks, int64_t chunk_words, int digit, int vec) {
  sah_pdl_entry_early();
  __shared__ unsigned int hs[SEL_THREADS / 32][256];
  __shared__ long long scan[33];
  __shared__ SelState st_sm;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int64_t row = blockIdx.y, chunk = blockIdx.x;
  const SelState st = sel_replay<KEYBITS>(ch, rows, row, chunks, digit, k, scan, &st_sm);
  unsigned int* outp = ch + (((int64_t)digit * rows + row) * chunks + chunk) * 256;
  if (st.mode != 0) {  // the whole CTA: nothing left to refine
    outp[tid] = 0u;
    return;
  }
  for (int i = tid; i < (SEL_THREADS / 32) * 256; i += SEL_THREADS) (&hs[0][0])[i] = 0u;
  __syncthreads();
  const int shift = KEYBITS - 8 * (digit + 1);
  const int64_t w_end = (chunk + 1) * chunk_words < W ? (chunk + 1) * chunk_words : W;
  for (int64_t w = chunk * chunk_words + tid; w < w_end; w += SEL_THREADS) {
    const uint32_t valid = sel_valid(prev_bits[row * W + w], w, col_begin, col_end);
    if (valid) {
      unsigned int keys[32];
      sel_load_keys<T, KEYBITS>(scores + row * S, w, S, vec != 0, keys);
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (((valid >> i) & 1u) && (keys[i] & st.pmask) == st.prefix)
          atomicAdd(&hs[warp][(keys[i] >> shift) & 255u], 1u);
    }
  }
  __syncthreads();
  unsigned int sum = 0u;
#pragma unroll
  for (int i = 0; i < SEL_THREADS / 32; ++i) sum += hs[i][tid];
  outp[tid] = sum;
}

template <typename T, int KEYBITS>
__global__ void __launch_bounds__(SEL_THREADS)
sel_fused_emit_kernel(const T* __restrict__ scores, int64_t S, int64_t W, int64_t col_begin, int64_t col_end,
                      const uint32_t* __restrict__ prev_bits, long long k, const unsigned int* __restrict__ ch,
                      int64_t rows, int chunks, int64_t chunk_words, int vec, uint32_t* __restrict__ out_bits) {
  sah_pdl_entry_early();
  __shared__ long long scan[33];
  __shared__ SelState st_sm;
  __shared__ long long before_sm;
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.y, chunk = blockIdx.x;
  constexpr int NDIG = KEYBITS / 8;
  const SelState st = sel_replay<KEYBITS>(ch, rows, row, chunks, NDIG, k, scan, &st_sm);
  // ties: keys equal to the threshold in the chunks before this one are served first
  if (tid < 32) {
    long long e = 0;
    if (st.mode == 0 && tid < chunk)
      e = ch[(((int64_t)(NDIG - 1) * rows + row) * chunks + tid) * 256 + (st.prefix & 255u)];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(0xffffffffu, e, o);
    if (tid == 0) before_sm = e;
  }
  __syncthreads();
  long long running = before_sm;
  const int64_t w0 = chunk * chunk_words;
  const int64_t w_end = w0 + chunk_words < W ? w0 + chunk_words : W;
  for (int64_t wb = w0; wb < w_end; wb += SEL_THREADS) {
    const int64_t w = wb + tid;
    uint32_t pw = 0u, gt = 0u, eq = 0u;
    if (w < w_end) {
      pw = prev_bits[row * W + w];
      const uint32_t valid = sel_valid(pw, w, col_begin, col_end);
      if (st.mode == 1) {
        gt = valid;
      } else if (st.mode == 0 && valid) {
        unsigned int keys[32];
        sel_load_keys<T, KEYBITS>(scores + row * S, w, S, vec != 0, keys);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          gt |= (keys[i] > st.prefix ? 1u : 0u) << i;
          eq |= (keys[i] == st.prefix ? 1u : 0u) << i;
        }
        gt &= valid;
        eq &= valid;
      }
    }
    long long total;
    const long long before = sah_block_excl_scan<long long>((long long)__popc(eq), scan, &total);
    if (w < w_end) {
      const long long quota = st.need - (running + before);
      const int take = st.mode != 0 ? 0 : (quota > 32 ? 32 : (quota < 0 ? 0 : (int)quota));
      out_bits[row * W + w] = pw | gt | sah_lowest_bits(eq, take);
    }
    running += total;
  }
}

extern "C" int64_t sah_topk_select_ws_bytes(int64_t rows, int64_t W) {
  if (rows <= 0 || W <= 0) return 0;
  const size_t stepwise = sel_ws_bytes(rows, (W + SEL_CHUNK_WORDS - 1) / SEL_CHUNK_WORDS);
  const size_t fused = sel_fused_ws_bytes(rows, W);
  return (int64_t)(stepwise > fused ? stepwise : fused);
}

// ---- the selection step by step (a multi-rank caller reduces the digit histogram between
// sah_topk_sel_hist and sah_topk_sel_pick, and gathers the ranks' tie counts before the emit)
extern "C" int64_t sah_topk_sel_hist_offset(int64_t rows, int64_t W) {
  const int64_t chunks = (W + SEL_CHUNK_WORDS - 1) / SEL_CHUNK_WORDS;
  return rows * chunks * 8 + rows * (int64_t)sizeof(SelState);
}

extern "C" int sah_topk_sel_begin(int64_t rows, int64_t W, int64_t k, void* workspace,
                                  int64_t workspace_bytes, void* stream) {
  SAH_REQUIRE(workspace != nullptr && ((uintptr_t)workspace % 16) == 0, "topk_sel_begin: bad workspace");
  SAH_REQUIRE(rows > 0 && rows <= 65535 && W > 0, "topk_sel_begin: bad extents");
  if (workspace_bytes < sah_topk_select_ws_bytes(rows, W))
    return sah_fail(SAH_ERR_WORKSPACE, "topk_sel_begin: workspace of %lld bytes, need %lld",
                    (long long)workspace_bytes, (long long)sah_topk_select_ws_bytes(rows, W));
  const int64_t chunks = (W + SEL_CHUNK_WORDS - 1) / SEL_CHUNK_WORDS;
  SelWorkspace o = sel_ws_carve(workspace, rows, chunks);
  cudaStream_t st = (cudaStream_t)stream;
  sah_launch_chain(sel_init_kernel, (unsigned)sah_ceil_div(rows * 256, 256), 256, 0, st, o.state, o.hist, rows, k);
  SAH_LAUNCH_CHECK("topk_select init");
  cudaMemsetAsync(o.chunk_before, 0, (size_t)rows * chunks * 8, st);
  return SAH_OK;
}

template <typename T, int KEYBITS>
static int sel_hist_step(const T* scores, int64_t rows, int64_t S, int64_t W, int64_t col_begin,
                         int64_t col_end, const uint32_t* prev_bits, void* ws, int shift, cudaStream_t st) {
  const int64_t chunks = (W + SEL_CHUNK_WORDS - 1) / SEL_CHUNK_WORDS;
  SelWorkspace o = sel_ws_carve(ws, rows, chunks);
  const int vec = ((S * (int64_t)sizeof(T)) % 16 == 0 && ((uintptr_t)scores % 16) == 0) ? 1 : 0;
  dim3 grid((unsigned)chunks, (unsigned)rows);
  sah_launch_chain(sel_hist_kernel<T, KEYBITS>, grid, SEL_THREADS, 0, st, scores, S, W, col_begin, col_end,
      prev_bits, o.state,
                                                            o.hist, shift == 0 ? o.chunk_hist : nullptr, chunks,
                                                            shift, vec);
  SAH_LAUNCH_CHECK("topk_select hist");
  return SAH_OK;
}

extern "C" int sah_topk_sel_hist(const void* scores, int dtype, int64_t rows, int64_t S, int64_t W,
                                 int64_t col_begin, int64_t col_end, const uint32_t* prev_bits,
                                 void* workspace, int shift, void* stream) {
  SAH_REQUIRE(scores && prev_bits && workspace, "topk_sel_hist: null pointer");
  SAH_REQUIRE(shift >= 0 && shift % 8 == 0, "topk_sel_hist: shift must be a multiple of 8");
  if (col_begin < 0) col_begin = 0;
  if (col_end > S) col_end = S;
  if (dtype == SAH_BF16) {
    SAH_REQUIRE(shift <= 8, "topk_sel_hist: bf16 keys have 16 bits");
    return sel_hist_step<__nv_bfloat16, 16>((const __nv_bfloat16*)scores, rows, S, W, col_begin, col_end,
                                            prev_bits, workspace, shift, (cudaStream_t)stream);
  }
  if (dtype == SAH_F32) {
    SAH_REQUIRE(shift <= 24, "topk_sel_hist: fp32 keys have 32 bits");
    return sel_hist_step<float, 32>((const float*)scores, rows, S, W, col_begin, col_end, prev_bits, workspace,
                                    shift, (cudaStream_t)stream);
  }
  return sah_fail(SAH_ERR_INVALID, "topk_sel_hist: unknown dtype %d", dtype);
}

extern "C" int sah_topk_sel_pick(int64_t rows, int64_t W, void* workspace, int shift, int first,
                                 int64_t* eq_total, void* stream) {
  SAH_REQUIRE(workspace != nullptr && rows > 0, "topk_sel_pick: bad arguments");
  const int64_t chunks = (W + SEL_CHUNK_WORDS - 1) / SEL_CHUNK_WORDS;
  SelWorkspace o = sel_ws_carve(workspace, rows, chunks);
  sah_launch_chain(sel_pick_kernel, (unsigned)rows, 256, 0, (cudaStream_t)stream, o.state, o.hist, shift,
      first, shift == 0 ? o.chunk_hist : nullptr, o.chunk_before, chunks,
      reinterpret_cast<long long*>(eq_total));
  SAH_LAUNCH_CHECK("topk_select pick");
  return SAH_OK;
}

template <typename T, int KEYBITS>
static int sel_emit_step(const T* scores, int64_t rows, int64_t S, int64_t W, int64_t col_begin,
                         int64_t col_end, const uint32_t* prev_bits, void* ws, const int64_t* tie_offset,
                         uint32_t* out_bits, cudaStream_t st) {
  const int64_t chunks = (W + SEL_CHUNK_WORDS - 1) / SEL_CHUNK_WORDS;
  SelWorkspace o = sel_ws_carve(ws, rows, chunks);
  const int vec = ((S * (int64_t)sizeof(T)) % 16 == 0 && ((uintptr_t)scores % 16) == 0) ? 1 : 0;
  dim3 grid((unsigned)chunks, (unsigned)rows);
  sah_launch_chain(sel_emit_kernel<T, KEYBITS>, grid, SEL_THREADS, 0, st, scores, S, W, col_begin, col_end,
      prev_bits, o.state,
                                                            o.chunk_before, chunks, vec,
                                                            reinterpret_cast<const long long*>(tie_offset),
                                                            out_bits);
  SAH_LAUNCH_CHECK("topk_select emit");
  return SAH_OK;
}

extern "C" int sah_topk_sel_emit(const void* scores, int dtype, int64_t rows, int64_t S, int64_t W,
                                 int64_t col_begin, int64_t col_end, const uint32_t* prev_bits,
                                 void* workspace, const int64_t* tie_offset, uint32_t* out_bits,
                                 void* stream) {
  SAH_REQUIRE(scores && prev_bits && workspace && out_bits, "topk_sel_emit: null pointer");
  if (col_begin < 0) col_begin = 0;
  if (col_end > S) col_end = S;
  if (dtype == SAH_BF16)
    return sel_emit_step<__nv_bfloat16, 16>((const __nv_bfloat16*)scores, rows, S, W, col_begin, col_end,
                                            prev_bits, workspace, tie_offset, out_bits, (cudaStream_t)stream);
  if (dtype == SAH_F32)
    return sel_emit_step<float, 32>((const float*)scores, rows, S, W, col_begin, col_end, prev_bits, workspace,
                                    tie_offset, out_bits, (cudaStream_t)stream);
  return sah_fail(SAH_ERR_INVALID, "topk_sel_emit: unknown dtype %d", dtype);
}

template <typename T, int KEYBITS>
static int sel_run(const T* scores, int64_t rows, int64_t S, int64_t W, int64_t col_begin, int64_t col_end,
                   const uint32_t* prev_bits, int64_t k, uint32_t* out_bits, void* ws, cudaStream_t st) {
  const SelFusedGeom g = sel_fused_geom(W);
  unsigned int* ch = reinterpret_cast<unsigned int*>(ws);
  const int vec = ((S * (int64_t)sizeof(T)) % 16 == 0 && ((uintptr_t)scores % 16) == 0) ? 1 : 0;
  dim3 grid((unsigned)g.chunks, (unsigned)rows);
  if (k > 0) {
    for (int digit = 0; digit < KEYBITS / 8; ++digit) {
      sah_launch_chain(sel_fused_hist_kernel<T, KEYBITS>, grid, SEL_THREADS, 0, st, scores, S, W, col_begin,
          col_end, prev_bits, (long long)k, ch, rows, g.chunks, g.chunk_words, digit, vec);
      SAH_LAUNCH_CHECK("topk_select digit histogram");
    }
  }
  sah_launch_chain(sel_fused_emit_kernel<T, KEYBITS>, grid, SEL_THREADS, 0, st, scores, S, W, col_begin,
      col_end, prev_bits, (long long)k, ch, rows, g.chunks, g.chunk_words, vec, out_bits);
  SAH_LAUNCH_CHECK("topk_select emit");
  return SAH_OK;
}

extern "C" int sah_topk_select_ws(const void* scores, int dtype, int64_t rows, int64_t S, int64_t W,
                                  int64_t col_begin, int64_t col_end, const uint32_t* prev_bits,
                                  int64_t k, uint32_t* out_bits, void* workspace,
                                  int64_t workspace_bytes, void* stream) {
  SAH_REQUIRE(scores && prev_bits && out_bits && workspace, "topk_select_ws: null pointer");
  SAH_REQUIRE(rows >= 0 && S > 0 && W * 32 >= S, "topk_select_ws: bad extents");
  SAH_REQUIRE(rows <= 65535, "topk_select_ws: more than 65535 rows (use sah_topk_select)");
  if (rows == 0) return SAH_OK;
  if (workspace_bytes < sah_topk_select_ws_bytes(rows, W))
    return sah_fail(SAH_ERR_WORKSPACE, "topk_select_ws: workspace of %lld bytes, need %lld",
                    (long long)workspace_bytes, (long long)sah_topk_select_ws_bytes(rows, W));
  SAH_REQUIRE(((uintptr_t)workspace % 16) == 0, "topk_select_ws: workspace must be 16-byte aligned");
  if (col_begin < 0) col_begin = 0;
  if (col_end > S) col_end = S;
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_TOPK_SELECT, st);
  int rc;
  if (dtype == SAH_BF16)
    rc = sel_run<__nv_bfloat16, 16>((const __nv_bfloat16*)scores, rows, S, W, col_begin, col_end, prev_bits, k,
                                    out_bits, workspace, st);
  else if (dtype == SAH_F32)
    rc = sel_run<float, 32>((const float*)scores, rows, S, W, col_begin, col_end, prev_bits, k, out_bits,
                            workspace, st);
  else
    return sah_fail(SAH_ERR_INVALID, "topk_select_ws: unknown dtype %d", dtype);
  if (rc != SAH_OK) return rc;
  sah_prof_end(SAH_PROF_TOPK_SELECT, st);
  return SAH_OK;
}

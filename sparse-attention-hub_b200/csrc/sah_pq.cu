// PQCache kernels (maskers/fixed/implementations/pq_top_k.py and utils/pq_utils.py):
//   sah_pq_assign         nearest centroid of every key sub-vector (k-means assignment
//                         step, pq_utils.py:246-255 + :353; new-key quantisation,
//                         pq_top_k.py:388-404)
//   sah_pq_accumulate     per-cluster sums and counts of one Lloyd iteration
//   sah_pq_update         new centres, empty-cluster reseeding and centre shift
//                         (pq_utils.py:360-423)
//   sah_pq_scores         query-centroid lookup tables and the code stream
//                         (pq_top_k.py:406-490)
//
// A "group" is one (batch, KV head, sub-vector): groups = B * Hkv * n_sub,
// group id = (b * Hkv + kvh) * n_sub + sub.  Codes are bytes laid out
// [B][Hkv][capacity][n_sub], i.e. the n_sub codes of one key are contiguous, so the
// scoring stream reads one 16-byte word per key for n_sub = 16.
#include "sah_common.cuh"

#define PQ_MAX_SUBD 16
#define PQ_TILE 256

// Squared distance in the fixed order the CPU restatement follows: dimensions
// ascending, (x - c) * (x - c) rounded, then added.
__device__ __forceinline__ float pq_dist(const float* x, const float* c, int sub_d) {
  float d = 0.f;
  for (int j = 0; j < sub_d; ++j) {
    const float t = __fsub_rn(x[j], c[j]);
    d = __fadd_rn(d, __fmul_rn(t, t));
  }
  return d;
}

// The same distance with every operation rounded to the key dtype: what the
// reference's quantisation of appended keys computes, since there both the keys and
// the stored centroids are dtype tensors (pq_top_k.py:388-404).
template <typename T>
__device__ __forceinline__ float pq_dist_dtype(const float* x, const float* c, int sub_d) {
  float d = 0.f;
  for (int j = 0; j < sub_d; ++j) {
    const float t = sah_round_to<T>(__fsub_rn(x[j], c[j]));
    d = __fadd_rn(d, sah_round_to<T>(__fmul_rn(t, t)));
  }
  return sah_round_to<T>(d);
}

template <typename T, bool DTYPE_MATH>
__global__ void __launch_bounds__(PQ_TILE)
pq_assign_kernel(const T* __restrict__ x, int64_t xs_b, int64_t xs_h, int64_t xs_s, int Hkv,
                 int64_t key_begin, int64_t key_end, int64_t init_offset, int n_sub, int sub_d,
                 int n_cent, const float* __restrict__ centroids, uint8_t* __restrict__ codes,
                 int64_t cap) {
  extern __shared__ float pq_cent_sm[];  // [n_cent][sub_d]
  const int sub = blockIdx.y;
  const int64_t bk = blockIdx.z;
  const int kvh = (int)(bk % Hkv);
  const int64_t b = bk / Hkv;
  const int64_t grp = bk * n_sub + sub;
  for (int i = threadIdx.x; i < n_cent * sub_d; i += PQ_TILE)
    pq_cent_sm[i] = centroids[grp * n_cent * sub_d + i];
  __syncthreads();
  const int64_t j = key_begin + (int64_t)blockIdx.x * PQ_TILE + threadIdx.x;
  if (j >= key_end) return;
  const T* xr = x + b * xs_b + kvh * xs_h + j * xs_s + sub * sub_d;
  float xv[PQ_MAX_SUBD];
  for (int d = 0; d < sub_d; ++d) xv[d] = sah_to_float<T>(xr[d]);
  float best = INFINITY;
  int arg = 0;
  for (int c = 0; c < n_cent; ++c) {
    const float dist = DTYPE_MATH ? pq_dist_dtype<T>(xv, pq_cent_sm + c * sub_d, sub_d)
                                  : pq_dist(xv, pq_cent_sm + c * sub_d, sub_d);
    if (dist < best) { best = dist; arg = c; }  // first minimum wins, as argmin does
  }
  codes[(bk * cap + (j - init_offset)) * n_sub + sub] = (uint8_t)arg;
}

extern "C" int sah_pq_assign(const void* x, int dtype, int64_t xs_b, int64_t xs_h, int64_t xs_s,
                             int B, int Hkv, int64_t key_begin, int64_t key_end,
                             int64_t init_offset, int n_sub, int sub_d, int n_cent,
                             const float* centroids, uint8_t* codes, int64_t cap, int dtype_math,
                             void* stream) {
  SAH_REQUIRE(x && centroids && codes, "pq_assign: null pointer");
  SAH_REQUIRE(B > 0 && Hkv > 0 && n_sub > 0 && sub_d > 0 && n_cent > 0, "pq_assign: bad extents");
  SAH_REQUIRE(init_offset <= key_begin && key_begin <= key_end && key_end - init_offset <= cap,
              "pq_assign: bad key range");
  if (sub_d > PQ_MAX_SUBD || n_cent > 256)
    return sah_fail(SAH_ERR_UNSUPPORTED, "pq_assign: sub-vector dim %d (<= %d) / %d centroids (<= 256)",
                    sub_d, PQ_MAX_SUBD, n_cent);
  if (key_begin == key_end) return SAH_OK;
  dim3 grid((unsigned)sah_ceil_div(key_end - key_begin, PQ_TILE), (unsigned)n_sub,
            (unsigned)((int64_t)B * Hkv));
  const size_t smem = (size_t)n_cent * sub_d * sizeof(float);
  SAH_DISPATCH_DTYPE(dtype, T, {
    if (dtype_math)
      pq_assign_kernel<T, true><<<grid, PQ_TILE, smem, (cudaStream_t)stream>>>(
          (const T*)x, xs_b, xs_h, xs_s, Hkv, key_begin, key_end, init_offset, n_sub, sub_d, n_cent,
          centroids, codes, cap);
    else
      pq_assign_kernel<T, false><<<grid, PQ_TILE, smem, (cudaStream_t)stream>>>(
          (const T*)x, xs_b, xs_h, xs_s, Hkv, key_begin, key_end, init_offset, n_sub, sub_d, n_cent,
          centroids, codes, cap);
  });
  SAH_LAUNCH_CHECK("pq_assign");
  return SAH_OK;
}

#include "sah_pq_tc.cuh"

// The assignment step on the tensor cores; same codes as sah_pq_assign(dtype_math = 0).
extern "C" int sah_pq_assign_tc(const void* x, int64_t xs_b, int64_t xs_h, int64_t xs_s, int B, int Hkv,
                                int64_t key_begin, int64_t key_end, int64_t init_offset, int n_sub,
                                int sub_d, int n_cent, const float* centroids, uint8_t* codes, int64_t cap,
                                int* errflag, int sm_count, void* stream) {
  SAH_REQUIRE(x && centroids && codes && errflag, "pq_assign_tc: null pointer");
  SAH_REQUIRE(B > 0 && Hkv > 0 && n_sub > 0, "pq_assign_tc: bad extents");
  SAH_REQUIRE(init_offset <= key_begin && key_begin <= key_end && key_end - init_offset <= cap,
              "pq_assign_tc: bad key range");
  if (sub_d != 8 || n_cent < 16 || n_cent > 256 || n_cent % 16 != 0)
    return sah_fail(SAH_ERR_UNSUPPORTED, "pq_assign_tc: sub-vectors of 8 channels and 16..256 centroids in "
                    "multiples of 16 (got %d, %d)", sub_d, n_cent);
  SAH_REQUIRE((xs_s * 2) % 16 == 0 && (xs_h * 2) % 16 == 0 && (xs_b * 2) % 16 == 0 && ((uintptr_t)x % 16) == 0,
              "pq_assign_tc: key rows must be 16-byte aligned");
  if (key_begin == key_end) return SAH_OK;
  static bool allowed = false;
  if (!allowed) {
    cudaError_t e = cudaFuncSetAttribute(pq_assign_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PtcCfg::SMEM);
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "pq_assign_tc attr: %s", cudaGetErrorString(e));
    allowed = true;
  }
  if (sm_count <= 0) sm_count = 148;
  const int64_t groups = (int64_t)B * Hkv * n_sub;
  const int64_t n_tiles = sah_ceil_div(key_end - key_begin, (int64_t)PTC_TILE);
  int64_t slices = sah_ceil_div((int64_t)4 * sm_count, groups);  // about two waves of two CTAs per SM
  if (slices > n_tiles) slices = n_tiles;
  if (slices < 1) slices = 1;
  SAH_REQUIRE(groups <= 65535, "pq_assign_tc: too many groups per launch");
  dim3 grid((unsigned)slices, (unsigned)groups);
  pq_assign_tc_kernel<<<grid, PTC_THREADS, PtcCfg::SMEM, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), xs_b, xs_h, xs_s, Hkv, key_begin, key_end, init_offset, n_sub,
      n_cent, centroids, codes, cap, errflag);
  SAH_LAUNCH_CHECK("pq_assign_tc");
  return SAH_OK;
}

// Cluster sums in fp64 (so that the summation order does not reach the fp32
// result) and counts; shared-memory accumulation per CTA, then global atomics.
template <typename T>
__global__ void __launch_bounds__(PQ_TILE)
pq_accumulate_kernel(const T* __restrict__ x, int64_t xs_b, int64_t xs_h, int64_t xs_s, int Hkv,
                     int64_t n_keys, int64_t init_offset, int n_sub, int sub_d, int n_cent,
                     const uint8_t* __restrict__ codes, int64_t cap, double* __restrict__ sums,
                     int* __restrict__ counts) {
  extern __shared__ double pq_sum_sm[];  // [n_cent][sub_d] then int [n_cent]
  int* cnt_sm = reinterpret_cast<int*>(pq_sum_sm + n_cent * sub_d);
  const int sub = blockIdx.y;
  const int64_t bk = blockIdx.z;
  const int kvh = (int)(bk % Hkv);
  const int64_t b = bk / Hkv;
  const int64_t grp = bk * n_sub + sub;
  for (int i = threadIdx.x; i < n_cent * sub_d; i += PQ_TILE) pq_sum_sm[i] = 0.0;
  for (int i = threadIdx.x; i < n_cent; i += PQ_TILE) cnt_sm[i] = 0;
  __syncthreads();
  // each CTA walks a strip of keys so that the global atomics stay few
  const int64_t strip = (n_keys + gridDim.x - 1) / gridDim.x;
  const int64_t j0 = (int64_t)blockIdx.x * strip;
  const int64_t j1 = j0 + strip < n_keys ? j0 + strip : n_keys;
  for (int64_t j = j0 + threadIdx.x; j < j1; j += PQ_TILE) {
    const int c = codes[(bk * cap + j) * n_sub + sub];
    const T* xr = x + b * xs_b + kvh * xs_h + (j + init_offset) * xs_s + sub * sub_d;
    for (int d = 0; d < sub_d; ++d) atomicAdd(&pq_sum_sm[c * sub_d + d], (double)sah_to_float<T>(xr[d]));
    atomicAdd(&cnt_sm[c], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_cent * sub_d; i += PQ_TILE)
    if (pq_sum_sm[i] != 0.0) atomicAdd(&sums[grp * n_cent * sub_d + i], pq_sum_sm[i]);
  for (int i = threadIdx.x; i < n_cent; i += PQ_TILE)
    if (cnt_sm[i]) atomicAdd(&counts[grp * n_cent + i], cnt_sm[i]);
}

extern "C" int sah_pq_accumulate(const void* x, int dtype, int64_t xs_b, int64_t xs_h, int64_t xs_s,
                                 int B, int Hkv, int64_t n_keys, int64_t init_offset, int n_sub,
                                 int sub_d, int n_cent, const uint8_t* codes, int64_t cap,
                                 double* sums, int* counts, void* stream) {
  SAH_REQUIRE(x && codes && sums && counts, "pq_accumulate: null pointer");
  SAH_REQUIRE(B > 0 && Hkv > 0 && n_sub > 0 && sub_d > 0 && n_cent > 0 && n_keys >= 0,
              "pq_accumulate: bad extents");
  if (n_keys == 0) return SAH_OK;
  int strips = (int)sah_ceil_div(n_keys, 4096);
  if (strips > 64) strips = 64;
  dim3 grid((unsigned)strips, (unsigned)n_sub, (unsigned)((int64_t)B * Hkv));
  const size_t smem = (size_t)n_cent * sub_d * sizeof(double) + (size_t)n_cent * sizeof(int);
  SAH_DISPATCH_DTYPE(dtype, T, {
    pq_accumulate_kernel<T><<<grid, PQ_TILE, smem, (cudaStream_t)stream>>>(
        (const T*)x, xs_b, xs_h, xs_s, Hkv, n_keys, init_offset, n_sub, sub_d, n_cent, codes, cap,
        sums, counts);
  });
  SAH_LAUNCH_CHECK("pq_accumulate");
  return SAH_OK;
}

// new centre = fp32(sum) / fp32(count); an empty cluster takes the key sub-vector at
// reseed[group][cluster] (pq_utils.py:384-396); shift2[group] = (sum over clusters of
// the centre's Euclidean move)^2, the quantity compared with the tolerance (:399-423).
template <typename T>
__global__ void pq_update_kernel(const T* __restrict__ x, int64_t xs_b, int64_t xs_h, int64_t xs_s,
                                 int Hkv, int64_t init_offset, int n_sub, int sub_d, int n_cent,
                                 const double* __restrict__ sums, const int* __restrict__ counts,
                                 const int64_t* __restrict__ reseed, float* __restrict__ centroids,
                                 float* __restrict__ shift2) {
  __shared__ float scratch[33];
  const int64_t grp = blockIdx.x;
  const int sub = (int)(grp % n_sub);
  const int64_t bk = grp / n_sub;
  const int kvh = (int)(bk % Hkv);
  const int64_t b = bk / Hkv;
  float move = 0.f;
  const int c = threadIdx.x;
  if (c < n_cent) {
    const int cnt = counts[grp * n_cent + c];
    float d2 = 0.f;
    for (int d = 0; d < sub_d; ++d) {
      float nv;
      if (cnt > 0) {
        nv = __fdiv_rn((float)sums[(grp * n_cent + c) * sub_d + d], (float)cnt);
      } else {
        const int64_t j = reseed[grp * n_cent + c];
        nv = sah_to_float<T>(x[b * xs_b + kvh * xs_h + (j + init_offset) * xs_s + sub * sub_d + d]);
      }
      float* cp = centroids + (grp * n_cent + c) * sub_d + d;
      const float t = __fsub_rn(nv, *cp);
      d2 = __fadd_rn(d2, __fmul_rn(t, t));
      *cp = nv;
    }
    move = sqrtf(d2);
  }
  float total;
  sah_block_excl_scan<float>(move, scratch, &total);
  if (threadIdx.x == 0) shift2[grp] = total * total;
}

extern "C" int sah_pq_update(const void* x, int dtype, int64_t xs_b, int64_t xs_h, int64_t xs_s,
                             int B, int Hkv, int64_t init_offset, int n_sub, int sub_d, int n_cent,
                             const double* sums, const int* counts, const int64_t* reseed,
                             float* centroids, float* shift2, void* stream) {
  SAH_REQUIRE(x && sums && counts && reseed && centroids && shift2, "pq_update: null pointer");
  SAH_REQUIRE(n_cent > 0 && n_cent <= 256, "pq_update: 1..256 centroids");
  const int64_t groups = (int64_t)B * Hkv * n_sub;
  SAH_DISPATCH_DTYPE(dtype, T, {
    pq_update_kernel<T><<<(unsigned)groups, 256, 0, (cudaStream_t)stream>>>(
        (const T*)x, xs_b, xs_h, xs_s, Hkv, init_offset, n_sub, sub_d, n_cent, sums, counts, reseed,
        centroids, shift2);
  });
  SAH_LAUNCH_CHECK("pq_update");
  return SAH_OK;
}

// ---------------------------------------------------------------------------
// Scores.  Per CTA: the lookup tables of up to PQ_ROWS mask rows of one KV group
// (lut[r][sub][c] = q_sub . centroid, fma over ascending dims, rounded to the
// dtype), then one thread per key sums its n_sub table entries in ascending
// sub-vector order in fp32 and rounds once (the reference sums a dtype tensor
// with an fp32 accumulator, pq_top_k.py:481-488).
// ---------------------------------------------------------------------------
#define PQ_ROWS 4

// One CTA: builds the table of one (KV group, block of 4 rows) in shared memory --
// lut[sub][c][rr] = q_sub(row rblk*4 + rr) . centroid(sub, c), fma over ascending dims, rounded
// to the dtype; rows past R hold 0 -- then scores a contiguous range of the group's keys: a
// key's n_sub codes index one entry each (the four rows of a centroid side by side: four
// bfloat16 in 8 bytes, or four floats in 16).  The key range per CTA is sized so that the grid
// is about two CTAs per SM: the table is built a few hundred times per call.
// The query rows are staged in shared memory as floats; a centroid is read with 16-byte loads
// when its sub-vector allows it (VEC: sub_d * sizeof(T) is a multiple of 16).
template <typename T>
struct PqEntry;
template <>
struct PqEntry<float> {
  typedef float4 type;
  static __device__ __forceinline__ float4 pack(const float* v) { return make_float4(v[0], v[1], v[2], v[3]); }
  static __device__ __forceinline__ void add(float* s, const float4& e) {
    s[0] = __fadd_rn(s[0], e.x); s[1] = __fadd_rn(s[1], e.y);
    s[2] = __fadd_rn(s[2], e.z); s[3] = __fadd_rn(s[3], e.w);
  }
};
template <>
struct PqEntry<__nv_bfloat16> {
  typedef uint2 type;  // the table values are bfloat16 numbers: two per word
  static __device__ __forceinline__ uint2 pack(const float* v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
  }
  static __device__ __forceinline__ void add(float* s, const uint2& e) {
    s[0] = __fadd_rn(s[0], __uint_as_float(e.x << 16)); s[1] = __fadd_rn(s[1], __uint_as_float(e.x & 0xffff0000u));
    s[2] = __fadd_rn(s[2], __uint_as_float(e.y << 16)); s[3] = __fadd_rn(s[3], __uint_as_float(e.y & 0xffff0000u));
  }
};

template <typename T, bool VEC>
__global__ void __launch_bounds__(PQ_TILE)
pq_scores_kernel(const T* __restrict__ q, int64_t qs_b, int64_t qs_h, int64_t qs_q,
                 const T* __restrict__ centroids, const uint8_t* __restrict__ codes, int64_t cap, int Hq,
                 int Hkv, int Sq, int64_t n_keys, int64_t init_offset, int64_t S, int n_sub, int sub_d,
                 int n_cent, int64_t keys_per_cta, T* __restrict__ scores) {
  sah_pdl_entry();
  typedef typename PqEntry<T>::type Entry;
  extern __shared__ __align__(16) unsigned char pq_sm_raw[];
  const int G = Hq / Hkv;
  const int R = G * Sq;
  const int64_t bk = blockIdx.z;
  const int kvh = (int)(bk % Hkv);
  const int64_t b = bk / Hkv;
  const int rblk = blockIdx.y;
  const int entries = n_sub * n_cent;
  const int Dh = n_sub * sub_d;
  Entry* lut = reinterpret_cast<Entry*>(pq_sm_raw);                  // [n_sub][n_cent]
  float* q_sm = reinterpret_cast<float*>(lut + entries);             // [PQ_ROWS][Dh]
  for (int idx = threadIdx.x; idx < PQ_ROWS * Dh; idx += PQ_TILE) {
    const int rr = idx / Dh, d = idx - rr * Dh;
    const int r = rblk * PQ_ROWS + rr;
    float v = 0.f;
    if (r < R) {
      const int g = r / Sq, qi = r - g * Sq;
      v = sah_to_float<T>(q[b * qs_b + (int64_t)(kvh * G + g) * qs_h + qi * qs_q + d]);
    }
    q_sm[idx] = v;
  }
  __syncthreads();
  constexpr int PER16 = 16 / (int)sizeof(T);  // elements per 16-byte load
  for (int idx = threadIdx.x; idx < entries; idx += PQ_TILE) {
    const int sub = idx / n_cent;
    const T* cp = centroids + (bk * n_sub * (int64_t)n_cent + idx) * sub_d;
    float acc[PQ_ROWS] = {0.f, 0.f, 0.f, 0.f};
    if constexpr (VEC) {
      for (int d0 = 0; d0 < sub_d; d0 += PER16) {
        const uint4 raw = *reinterpret_cast<const uint4*>(cp + d0);
        const T* cv = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < PER16; ++e) {
          const float c = sah_to_float<T>(cv[e]);
#pragma unroll
          for (int rr = 0; rr < PQ_ROWS; ++rr) acc[rr] = fmaf(q_sm[rr * Dh + sub * sub_d + d0 + e], c, acc[rr]);
        }
      }
    } else {
      for (int d = 0; d < sub_d; ++d) {
        const float c = sah_to_float<T>(cp[d]);
#pragma unroll
        for (int rr = 0; rr < PQ_ROWS; ++rr) acc[rr] = fmaf(q_sm[rr * Dh + sub * sub_d + d], c, acc[rr]);
      }
    }
    float out[PQ_ROWS];
#pragma unroll
    for (int rr = 0; rr < PQ_ROWS; ++rr) out[rr] = (rblk * PQ_ROWS + rr < R) ? sah_round_to<T>(acc[rr]) : 0.f;
    lut[idx] = PqEntry<T>::pack(out);
  }
  __syncthreads();
  const bool vec = (n_sub == 16) && ((reinterpret_cast<uintptr_t>(codes) & 15) == 0);
  int64_t rowoff[PQ_ROWS];
#pragma unroll
  for (int rr = 0; rr < PQ_ROWS; ++rr) {
    const int r = rblk * PQ_ROWS + rr;
    const int g = r / Sq, qi = r - g * Sq;
    rowoff[rr] = r < R ? ((b * Hq + kvh * G + g) * Sq + qi) * S + init_offset : -1;
  }
  const int64_t j0 = (int64_t)blockIdx.x * keys_per_cta;
  const int64_t j1 = j0 + keys_per_cta < n_keys ? j0 + keys_per_cta : n_keys;
  for (int64_t j = j0 + threadIdx.x; j < j1; j += PQ_TILE) {
    const uint8_t* cj = codes + (bk * cap + j) * n_sub;
    float s[PQ_ROWS] = {0.f, 0.f, 0.f, 0.f};
    if (vec) {
      const uint4 cv = *reinterpret_cast<const uint4*>(cj);
      const uint32_t w[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
      for (int sub = 0; sub < 16; ++sub) {
        const uint32_t c = (w[sub >> 2] >> ((sub & 3) * 8)) & 255u;
        PqEntry<T>::add(s, lut[sub * n_cent + c]);
      }
    } else {
      for (int sub = 0; sub < n_sub; ++sub) PqEntry<T>::add(s, lut[sub * n_cent + cj[sub]]);
    }
#pragma unroll
    for (int rr = 0; rr < PQ_ROWS; ++rr)
      if (rowoff[rr] >= 0) scores[rowoff[rr] + j] = sah_from_float<T>(s[rr]);
  }
}

extern "C" int64_t sah_pq_scores_ws_bytes(int B, int Hq, int Hkv, int Sq, int n_sub, int n_cent) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || n_sub <= 0 || n_cent <= 0) return 0;
  const int64_t R = (int64_t)(Hq / Hkv) * Sq;
  const int64_t rblocks = (R + PQ_ROWS - 1) / PQ_ROWS;
  return (int64_t)B * Hkv * rblocks * n_sub * n_cent * PQ_ROWS * (int64_t)sizeof(float);
}

extern "C" int sah_pq_scores(const void* q, int dtype, int64_t qs_b, int64_t qs_h, int64_t qs_q,
                             const void* centroids, const uint8_t* codes, int64_t cap, int B, int Hq,
                             int Hkv, int Sq, int64_t n_keys, int64_t init_offset, int64_t S,
                             int n_sub, int sub_d, int n_cent, void* scores, void* workspace,
                             int64_t workspace_bytes, void* stream) {
  SAH_REQUIRE(q && centroids && codes && scores, "pq_scores: null pointer");
  SAH_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Sq > 0, "pq_scores: bad heads");
  SAH_REQUIRE(n_keys >= 0 && init_offset >= 0 && init_offset + n_keys <= S && n_keys <= cap,
              "pq_scores: bad key range");
  SAH_REQUIRE(n_cent <= 256, "pq_scores: codes are bytes, at most 256 centroids");
  (void)workspace_bytes;
  if (n_keys == 0) return SAH_OK;
  const int R = (Hq / Hkv) * Sq;
  const int rblocks = (R + PQ_ROWS - 1) / PQ_ROWS;
  const size_t esz = (dtype == SAH_BF16) ? 8 : 16;  // one table entry: the four rows of a centroid
  const size_t smem = esz * n_sub * n_cent + (size_t)PQ_ROWS * n_sub * sub_d * sizeof(float);
  if (smem > 200 * 1024)
    return sah_fail(SAH_ERR_UNSUPPORTED, "pq_scores: %d x %d lookup table does not fit", n_sub, n_cent);
  SAH_REQUIRE(rblocks <= 65535 && (int64_t)B * Hkv <= 65535, "pq_scores: too many rows per launch");
  cudaStream_t st = (cudaStream_t)stream;
  (void)workspace;  // the tables live in shared memory; the argument is kept for callers that pass one
  sah_prof_begin(SAH_PROF_PQ_SCORES, st);
  // about two CTAs per SM, each with a contiguous key range that is a multiple of the CTA width
  const int64_t groups = (int64_t)B * Hkv * rblocks;
  int64_t per_group = (2 * 148 + groups - 1) / groups;
  if (per_group < 1) per_group = 1;
  int64_t keys_per_cta = sah_ceil_div(sah_ceil_div(n_keys, per_group), PQ_TILE) * PQ_TILE;
  if (keys_per_cta < 2048) keys_per_cta = 2048;
  dim3 grid((unsigned)sah_ceil_div(n_keys, keys_per_cta), (unsigned)rblocks, (unsigned)((int64_t)B * Hkv));
  const int64_t tsz = (dtype == SAH_BF16) ? 2 : 4;
  const bool vecc = (sub_d * tsz) % 16 == 0 && (reinterpret_cast<uintptr_t>(centroids) & 15) == 0;
  static int smem_allowed[4] = {0, 0, 0, 0};  // largest dynamic shared memory granted per instantiation
#define PQ_SCORES_LAUNCH(T, VEC, SLOT)                                                                    \
  do {                                                                                                    \
    if ((int)smem > 48 * 1024 && (int)smem > smem_allowed[SLOT]) {                                        \
      cudaError_t e = cudaFuncSetAttribute(pq_scores_kernel<T, VEC>,                                      \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "pq_scores attr: %s", cudaGetErrorString(e));   \
      smem_allowed[SLOT] = (int)smem;                                                                     \
    }                                                                                                     \
    sah_launch_chain(pq_scores_kernel<T, VEC>, grid, PQ_TILE, smem, st, (const T*)q, qs_b, qs_h, qs_q, (const T*)centroids, \
                                                          codes, cap, Hq, Hkv, Sq, n_keys, init_offset, S, \
                                                          n_sub, sub_d, n_cent, keys_per_cta, (T*)scores); \
  } while (0)
  if (dtype == SAH_BF16) {
    if (vecc) PQ_SCORES_LAUNCH(__nv_bfloat16, true, 0);
    else PQ_SCORES_LAUNCH(__nv_bfloat16, false, 1);
  } else if (dtype == SAH_F32) {
    if (vecc) PQ_SCORES_LAUNCH(float, true, 2);
    else PQ_SCORES_LAUNCH(float, false, 3);
  } else {
    return sah_fail(SAH_ERR_INVALID, "pq_scores: unknown dtype %d", dtype);
  }
#undef PQ_SCORES_LAUNCH
  SAH_LAUNCH_CHECK("pq_scores");
  sah_prof_end(SAH_PROF_PQ_SCORES, st);
  return SAH_OK;
}

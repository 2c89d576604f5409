// Mask container kernels: the active set of a Mask lives on the device as a
// bitmap (uint32 [rows][W]); these kernels edit it, scan it into the CSR
// companion arrays (ptr / wpre) and convert between the bitmap form and the
// reference's dense and indices/ptr/data forms (utils/mask.py).
#include <stdarg.h>
#include <string.h>

#include "sah_common.cuh"

// ---- status plumbing --------------------------------------------------------
static thread_local char g_sah_err[512] = "";

int sah_fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_sah_err, sizeof(g_sah_err), fmt, ap);
  va_end(ap);
  return status;
}

extern "C" const char* sah_last_error(void) { return g_sah_err; }
extern "C" const char* sah_version(void) { return "sah_b200 0.1 (sm_100a)"; }

// ---- launch accounting / per-kernel timing ---------------------------------------
#include <atomic>
#include <mutex>
#include <vector>

static std::atomic<long long> g_launches{0};
static std::atomic<int> g_prof_on{0};
static std::mutex g_prof_mu;
struct ProfPair { cudaEvent_t a, b; };
static std::vector<ProfPair> g_prof_events[SAH_PROF_SLOTS];
static thread_local cudaEvent_t g_prof_open[SAH_PROF_SLOTS];

void sah_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// Chained launches are off unless SAH_PDL=1 is in the environment (read once);
// SAH_PDL_MAX_WARPS then replaces the grid size up to which a launch may be chained.
int sah_pdl_max_warps() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SAH_PDL");
    const char* m = getenv("SAH_PDL_MAX_WARPS");
    v = (e != nullptr && e[0] == '1') ? (m != nullptr && atoi(m) > 0 ? atoi(m) : 1024) : 0;
  }
  return v;
}

void sah_prof_begin(int slot, cudaStream_t st) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, st);
  g_prof_open[slot] = e;
}

void sah_prof_end(int slot, cudaStream_t st) {
  if (!g_prof_on.load(std::memory_order_relaxed) || g_prof_open[slot] == nullptr) return;
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, st);
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_prof_events[slot].push_back({g_prof_open[slot], e});
  g_prof_open[slot] = nullptr;
}

extern "C" long long sah_launch_count(void) { return g_launches.load(); }

extern "C" int sah_profile_enable(int on) {
  g_prof_on.store(on ? 1 : 0);
  return SAH_OK;
}

extern "C" int sah_profile_read(int slot, float* total_ms, int* launches) {
  SAH_REQUIRE(slot >= 0 && slot < SAH_PROF_SLOTS && total_ms && launches, "profile_read: bad argument");
  std::lock_guard<std::mutex> lk(g_prof_mu);
  float sum = 0.f;
  int n = 0;
  for (auto& pr : g_prof_events[slot]) {
    cudaEventSynchronize(pr.b);
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, pr.a, pr.b) == cudaSuccess) { sum += ms; ++n; }
    cudaEventDestroy(pr.a);
    cudaEventDestroy(pr.b);
  }
  g_prof_events[slot].clear();
  *total_ms = sum;
  *launches = n;
  return SAH_OK;
}

// ---- band fill --------------------------------------------------------------
__global__ void mask_fill_band_kernel(uint32_t* __restrict__ bits, int64_t rows, int Sq,
                                      int64_t S, int64_t W, int64_t w_begin, int64_t w_count,
                                      int64_t lo_base, int64_t lo_qstep, int64_t hi_base,
                                      int64_t hi_qstep, int value) {
  sah_pdl_entry_early();
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * w_count) return;
  int64_t row = t / w_count;
  int64_t w = w_begin + (t - row * w_count);
  int64_t q = row % Sq;
  int64_t lo = lo_base + q * lo_qstep;
  int64_t hi = hi_base + q * hi_qstep;
  if (lo < 0) lo = 0;
  if (hi > S) hi = S;
  int64_t c0 = w * 32, c1 = c0 + 32;
  if (hi <= c0 || lo >= c1 || lo >= hi) return;
  int64_t a = lo > c0 ? lo - c0 : 0;        // first bit in word
  int64_t b = hi < c1 ? hi - c0 : 32;       // one past last bit
  uint32_t m = (b >= 32 ? 0xffffffffu : ((1u << b) - 1u)) & ~((1u << a) - 1u);
  uint32_t* p = bits + row * W + w;
  if (value) *p |= m; else *p &= ~m;
}

extern "C" int sah_mask_fill_band(uint32_t* bits, int64_t rows, int Sq, int64_t S, int64_t W,
                                  int64_t lo_base, int64_t lo_qstep, int64_t hi_base,
                                  int64_t hi_qstep, int value, void* stream) {
  SAH_REQUIRE(bits != nullptr, "fill_band: bits is null");
  SAH_REQUIRE(rows >= 0 && Sq > 0 && S > 0 && W * 32 >= S, "fill_band: bad extents");
  if (rows == 0) return SAH_OK;
  // Column hull over all query positions bounds the words any row touches.
  int64_t lo0 = lo_base, lo1 = lo_base + (Sq - 1) * lo_qstep;
  int64_t hi0 = hi_base, hi1 = hi_base + (Sq - 1) * hi_qstep;
  int64_t lo = lo0 < lo1 ? lo0 : lo1, hi = hi0 > hi1 ? hi0 : hi1;
  if (lo < 0) lo = 0;
  if (hi > S) hi = S;
  if (hi <= lo) return SAH_OK;
  int64_t w_begin = lo / 32, w_end = (hi + 31) / 32;
  int64_t w_count = w_end - w_begin;
  int64_t total = rows * w_count;
  int threads = 256;
  int64_t blocks = sah_ceil_div(total, threads);
  sah_launch_chain(mask_fill_band_kernel, (unsigned)blocks, threads, 0, (cudaStream_t)stream, bits, rows, Sq,
      S, W, w_begin, w_count, lo_base, lo_qstep, hi_base, hi_qstep, value);
  SAH_LAUNCH_CHECK("mask_fill_band");
  return SAH_OK;
}

// ---- several band fills in one pass ------------------------------------------
// A stack of fixed-pattern maskers (sink, local window, ...) is a short list of band edits on a
// bitmap that starts empty: one launch writes every word once, applying the bands in order.
#define SAH_MAX_BANDS 6
struct MaskBands {
  int n;
  int64_t lo_base[SAH_MAX_BANDS], lo_qstep[SAH_MAX_BANDS], hi_base[SAH_MAX_BANDS], hi_qstep[SAH_MAX_BANDS];
  int value[SAH_MAX_BANDS];
};

__global__ void mask_fill_bands_kernel(uint32_t* __restrict__ bits, int64_t rows, int Sq, int64_t S,
                                       int64_t W, MaskBands bands, int init_zero) {
  sah_pdl_entry_early();
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * W) return;
  const int64_t row = t / W;
  const int64_t w = t - row * W;
  const int64_t q = row % Sq;
  const int64_t c0 = w * 32, c1 = c0 + 32;
  uint32_t v = init_zero ? 0u : bits[t];
#pragma unroll
  for (int i = 0; i < SAH_MAX_BANDS; ++i) {
    if (i >= bands.n) break;
    int64_t lo = bands.lo_base[i] + q * bands.lo_qstep[i];
    int64_t hi = bands.hi_base[i] + q * bands.hi_qstep[i];
    if (lo < 0) lo = 0;
    if (hi > S) hi = S;
    if (hi <= c0 || lo >= c1 || lo >= hi) continue;
    const int64_t a = lo > c0 ? lo - c0 : 0;        // first bit in word
    const int64_t b = hi < c1 ? hi - c0 : 32;       // one past last bit
    const uint32_t m = (b >= 32 ? 0xffffffffu : ((1u << b) - 1u)) & ~((1u << a) - 1u);
    if (bands.value[i]) v |= m; else v &= ~m;
  }
  bits[t] = v;
}

extern "C" int sah_mask_fill_bands(uint32_t* bits, int64_t rows, int Sq, int64_t S, int64_t W,
                                   int n_bands, const int64_t* bands, int init_zero, void* stream) {
  SAH_REQUIRE(bits != nullptr, "fill_bands: bits is null");
  SAH_REQUIRE(rows >= 0 && Sq > 0 && S > 0 && W * 32 >= S, "fill_bands: bad extents");
  SAH_REQUIRE(n_bands >= 0 && n_bands <= SAH_MAX_BANDS && (n_bands == 0 || bands != nullptr),
              "fill_bands: 0..%d bands", SAH_MAX_BANDS);
  if (rows == 0 || (n_bands == 0 && !init_zero)) return SAH_OK;
  MaskBands mb;
  mb.n = n_bands;
  for (int i = 0; i < SAH_MAX_BANDS; ++i) {
    const bool on = i < n_bands;
    mb.lo_base[i] = on ? bands[5 * i + 0] : 0;
    mb.lo_qstep[i] = on ? bands[5 * i + 1] : 0;
    mb.hi_base[i] = on ? bands[5 * i + 2] : 0;
    mb.hi_qstep[i] = on ? bands[5 * i + 3] : 0;
    mb.value[i] = on ? (int)bands[5 * i + 4] : 0;
  }
  const int64_t total = rows * W;
  sah_launch_chain(mask_fill_bands_kernel, (unsigned)sah_ceil_div(total, 256), 256, 0, (cudaStream_t)stream,
      bits, rows, Sq, S, W, mb, init_zero);
  SAH_LAUNCH_CHECK("mask_fill_bands");
  return SAH_OK;
}

// ---- row scan: wpre (per word exclusive popcount) and ptr --------------------
// One CTA per row; the running base carries across blockDim-word chunks.
__global__ void mask_rowscan_kernel(const uint32_t* __restrict__ bits, int64_t W,
                                    int32_t* __restrict__ wpre, int64_t* __restrict__ rowcnt) {
  sah_pdl_entry_early();
  __shared__ int scratch[33];
  int64_t row = blockIdx.x;
  const uint32_t* b = bits + row * W;
  int base = 0;
  for (int64_t w0 = 0; w0 < W; w0 += blockDim.x) {
    int64_t w = w0 + threadIdx.x;
    int c = (w < W) ? __popc(b[w]) : 0;
    int total;
    int ex = sah_block_excl_scan<int>(c, scratch, &total);
    if (w < W && wpre != nullptr) wpre[row * W + w] = base + ex;
    base += total;
  }
  if (threadIdx.x == 0) rowcnt[row] = base;
}

// Exclusive scan of rowcnt[rows] into ptr[rows+1] (single CTA, looped).
__global__ void mask_ptrscan_kernel(const int64_t* rowcnt, int64_t rows, int64_t* ptr) {
  sah_pdl_entry_early();
  __shared__ long long scratch[33];
  long long base = 0;
  for (int64_t r0 = 0; r0 < rows; r0 += blockDim.x) {
    int64_t r = r0 + threadIdx.x;
    long long c = (r < rows) ? rowcnt[r] : 0;
    long long total;
    long long ex = sah_block_excl_scan<long long>(c, scratch, &total);
    if (r < rows) ptr[r] = base + ex;
    base += total;
  }
  __syncthreads();
  if (threadIdx.x == 0) ptr[rows] = base;
}

extern "C" int sah_mask_rowscan(const uint32_t* bits, int64_t rows, int64_t W, int32_t* wpre,
                                int64_t* ptr, void* stream) {
  SAH_REQUIRE(bits != nullptr && ptr != nullptr, "rowscan: null pointer");
  SAH_REQUIRE(rows >= 0 && W > 0, "rowscan: bad extents");
  cudaStream_t st = (cudaStream_t)stream;
  if (rows > 0) {
    // Row counts are staged in ptr[1 .. rows]; the scan kernel reads them
    // from there before overwriting (it walks forward, one chunk at a time,
    // and every chunk is read completely before any of it is written).
    sah_launch_chain(mask_rowscan_kernel, (unsigned)rows, 1024, 0, st, bits, W, wpre, ptr + 1);
    SAH_LAUNCH_CHECK("mask_rowscan");
  }
  // In-place: chunk r0 reads ptr[1 + r] for r in the chunk, then writes ptr[r]
  // for the same r; ptr[1 + last r of chunk] is read by the next chunk, so the
  // write of ptr[r] (r <= last) never clobbers an unread count.
  sah_launch_chain(mask_ptrscan_kernel, 1, 1024, 0, st, ptr + 1, rows, ptr);
  SAH_LAUNCH_CHECK("mask_ptrscan");
  return SAH_OK;
}

// ---- bits -> flat indices ----------------------------------------------------
__global__ void mask_bits_to_indices_kernel(const uint32_t* __restrict__ bits,
                                            const int32_t* __restrict__ wpre,
                                            const int64_t* __restrict__ ptr, int64_t rows,
                                            int64_t S, int64_t W, int64_t* __restrict__ idx) {
  sah_pdl_entry_early();
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * W) return;
  int64_t row = t / W, w = t - row * W;
  uint32_t m = bits[t];
  if (!m) return;
  int64_t o = ptr[row] + wpre[t];
  int64_t base = row * S + w * 32;
  while (m) {
    int b = __ffs(m) - 1;
    idx[o++] = base + b;
    m &= m - 1;
  }
}

extern "C" int sah_mask_bits_to_indices(const uint32_t* bits, const int32_t* wpre,
                                        const int64_t* ptr, int64_t rows, int64_t S, int64_t W,
                                        int64_t* indices, void* stream) {
  SAH_REQUIRE(bits && wpre && ptr, "bits_to_indices: null pointer");
  if (rows == 0) return SAH_OK;
  SAH_REQUIRE(indices != nullptr, "bits_to_indices: indices is null");
  int64_t total = rows * W;
  sah_launch_chain(mask_bits_to_indices_kernel, (unsigned)sah_ceil_div(total, 256), 256, 0,
                                (cudaStream_t)stream, bits, wpre, ptr, rows, S, W, indices);
  SAH_LAUNCH_CHECK("mask_bits_to_indices");
  return SAH_OK;
}

// ---- bits (+data) -> dense ----------------------------------------------------
template <typename T>
__global__ void mask_bits_to_dense_kernel(const uint32_t* __restrict__ bits,
                                          const T* __restrict__ data,
                                          const int32_t* __restrict__ wpre,
                                          const int64_t* __restrict__ ptr, int64_t rows,
                                          int64_t S, int64_t W, T* __restrict__ dense) {
  sah_pdl_entry_early();
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * S) return;
  int64_t row = t / S, j = t - row * S;
  int64_t wi = row * W + (j >> 5);
  uint32_t m = bits[wi];
  int b = (int)(j & 31);
  float v = 0.f;
  if ((m >> b) & 1u) {
    if (data == nullptr) {
      v = 1.f;
    } else {
      int64_t pos = ptr[row] + wpre[wi] + __popc(m & ((1u << b) - 1u));
      v = sah_to_float<T>(data[pos]);
    }
  }
  dense[t] = sah_from_float<T>(v);
}

extern "C" int sah_mask_bits_to_dense(const uint32_t* bits, const void* data,
                                      const int32_t* wpre, const int64_t* ptr, int dtype,
                                      int64_t rows, int64_t S, int64_t W, void* dense,
                                      void* stream) {
  SAH_REQUIRE(bits && dense, "bits_to_dense: null pointer");
  SAH_REQUIRE(data == nullptr || (wpre && ptr), "bits_to_dense: data needs wpre and ptr");
  if (rows == 0) return SAH_OK;
  int64_t total = rows * S;
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_bits_to_dense_kernel<T>, (unsigned)sah_ceil_div(total, 256), 256, 0,
                                   (cudaStream_t)stream, bits, (const T*)data, wpre, ptr,
                                                           rows, S, W, (T*)dense);
  });
  SAH_LAUNCH_CHECK("mask_bits_to_dense");
  return SAH_OK;
}

// ---- dense -> bits -------------------------------------------------------------
template <typename T>
__global__ void mask_dense_to_bits_kernel(const T* __restrict__ dense, int64_t rows, int64_t S,
                                          int64_t W, uint32_t* __restrict__ bits) {
  sah_pdl_entry_early();
  int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;  // one warp per word
  int lane = threadIdx.x & 31;
  if (gw >= rows * W) return;
  int64_t row = gw / W, w = gw - row * W;
  int64_t j = w * 32 + lane;
  bool on = false;
  if (j < S) on = sah_to_float<T>(dense[row * S + j]) != 0.f;
  uint32_t m = __ballot_sync(0xffffffffu, on);
  if (lane == 0) bits[gw] = m;
}

extern "C" int sah_mask_dense_to_bits(const void* dense, int dtype, int64_t rows, int64_t S,
                                      int64_t W, uint32_t* bits, void* stream) {
  SAH_REQUIRE(dense && bits, "dense_to_bits: null pointer");
  SAH_REQUIRE(W * 32 >= S, "dense_to_bits: W too small");
  if (rows == 0) return SAH_OK;
  int64_t threads_total = rows * W * 32;
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_dense_to_bits_kernel<T>, (unsigned)sah_ceil_div(threads_total, 256), 256, 0,
                                   (cudaStream_t)stream, (const T*)dense, rows, S, W, bits);
  });
  SAH_LAUNCH_CHECK("mask_dense_to_bits");
  return SAH_OK;
}

// ---- dense -> data (CSR order) ---------------------------------------------------
template <typename T>
__global__ void mask_dense_gather_data_kernel(const T* __restrict__ dense,
                                              const uint32_t* __restrict__ bits,
                                              const int32_t* __restrict__ wpre,
                                              const int64_t* __restrict__ ptr, int64_t rows,
                                              int64_t S, int64_t W, T* __restrict__ data) {
  sah_pdl_entry_early();
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * S) return;
  int64_t row = t / S, j = t - row * S;
  int64_t wi = row * W + (j >> 5);
  uint32_t m = bits[wi];
  int b = (int)(j & 31);
  if ((m >> b) & 1u) {
    int64_t pos = ptr[row] + wpre[wi] + __popc(m & ((1u << b) - 1u));
    data[pos] = dense[t];
  }
}

extern "C" int sah_mask_dense_gather_data(const void* dense, int dtype, const uint32_t* bits,
                                          const int32_t* wpre, const int64_t* ptr,
                                          int64_t rows, int64_t S, int64_t W, void* data,
                                          void* stream) {
  SAH_REQUIRE(dense && bits && wpre && ptr, "dense_gather_data: null pointer");
  if (rows == 0) return SAH_OK;
  int64_t total = rows * S;
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_dense_gather_data_kernel<T>, (unsigned)sah_ceil_div(total, 256), 256, 0,
                                       (cudaStream_t)stream, (const T*)dense, bits, wpre,
                                                               ptr, rows, S, W, (T*)data);
  });
  SAH_LAUNCH_CHECK("mask_dense_gather_data");
  return SAH_OK;
}

// ---- bitmap OR ---------------------------------------------------------------------
__global__ void mask_or_kernel(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b,
                               int64_t words, uint32_t* __restrict__ out) {
  sah_pdl_entry_early();
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < words) out[t] = a[t] | b[t];
}

extern "C" int sah_mask_or(const uint32_t* a, const uint32_t* b, int64_t words, uint32_t* out,
                           void* stream) {
  SAH_REQUIRE(a && b && out, "mask_or: null pointer");
  if (words == 0) return SAH_OK;
  sah_launch_chain(mask_or_kernel, (unsigned)sah_ceil_div(words, 256), 256, 0, (cudaStream_t)stream, a, b, words, out);
  SAH_LAUNCH_CHECK("mask_or");
  return SAH_OK;
}

// ---- weights of a sampled merge --------------------------------------------------------
// data of out_bits = prev | samp where prev has unit weights: entries of prev
// keep 1, new entries take the per-row weight (or the per-key dense weight).
template <typename T>
__global__ void mask_sample_data_kernel(const uint32_t* __restrict__ prev,
                                        const uint32_t* __restrict__ outb,
                                        const int32_t* __restrict__ wpre,
                                        const int64_t* __restrict__ ptr,
                                        const T* __restrict__ row_weight,
                                        const T* __restrict__ dense_weight, int64_t rows,
                                        int64_t S, int64_t W, T* __restrict__ data) {
  sah_pdl_entry_early();
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * W) return;
  int64_t row = t / W, w = t - row * W;
  uint32_t m = outb[t];
  if (!m) return;
  uint32_t p = prev ? prev[t] : 0u;
  int64_t o = ptr[row] + wpre[t];
  while (m) {
    int b = __ffs(m) - 1;
    T v;
    if ((p >> b) & 1u) {
      v = sah_from_float<T>(1.f);
    } else if (dense_weight) {
      v = dense_weight[row * S + w * 32 + b];
    } else {
      v = row_weight[row];
    }
    data[o++] = v;
    m &= m - 1;
  }
}

extern "C" int sah_mask_sample_data(const uint32_t* prev_bits, const uint32_t* out_bits,
                                    const int32_t* wpre, const int64_t* ptr,
                                    const void* row_weight, const void* dense_weight,
                                    int dtype, int64_t rows, int64_t S, int64_t W, void* data,
                                    void* stream) {
  SAH_REQUIRE(out_bits && wpre && ptr, "sample_data: null pointer");
  SAH_REQUIRE(row_weight || dense_weight, "sample_data: no weight source");
  if (rows == 0) return SAH_OK;
  SAH_REQUIRE(data != nullptr, "sample_data: data is null");
  int64_t total = rows * W;
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_sample_data_kernel<T>, (unsigned)sah_ceil_div(total, 256), 256, 0,
                                 (cudaStream_t)stream, prev_bits, out_bits, wpre, ptr,
                                                         (const T*)row_weight,
                                                         (const T*)dense_weight, rows, S, W,
                                                         (T*)data);
  });
  SAH_LAUNCH_CHECK("mask_sample_data");
  return SAH_OK;
}

// ---- weight 1 for the entries of a sub-set ------------------------------------------------------
// data[entry] = 1 for every entry of `bits` whose column is also set in `unit_bits`: the
// clamp(prev + p, 0, 1) of a dense merge when `prev` has unit weights and p <= 1.
template <typename T>
__global__ void mask_unit_data_kernel(const uint32_t* __restrict__ bits,
                                      const uint32_t* __restrict__ unit_bits,
                                      const int32_t* __restrict__ wpre,
                                      const int64_t* __restrict__ ptr, int64_t rows, int64_t W,
                                      T* __restrict__ data) {
  sah_pdl_entry_early();
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * W) return;
  const uint32_t m = bits[t];
  uint32_t u = unit_bits[t] & m;
  if (!u) return;
  const int64_t row = t / W;
  const int64_t o = ptr[row] + wpre[t];
  while (u) {
    const int b = __ffs(u) - 1;
    u &= u - 1;
    data[o + __popc(m & ((1u << b) - 1u))] = sah_from_float<T>(1.f);
  }
}

extern "C" int sah_mask_unit_data(const uint32_t* bits, const uint32_t* unit_bits,
                                  const int32_t* wpre, const int64_t* ptr, int dtype, int64_t rows,
                                  int64_t W, void* data, void* stream) {
  SAH_REQUIRE(bits && unit_bits && wpre && ptr, "unit_data: null pointer");
  if (rows == 0) return SAH_OK;
  SAH_REQUIRE(data != nullptr, "unit_data: data is null");
  const int64_t total = rows * W;
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_unit_data_kernel<T>, (unsigned)sah_ceil_div(total, 256), 256, 0,
        (cudaStream_t)stream, bits, unit_bits, wpre, ptr, rows, W, (T*)data);
  });
  SAH_LAUNCH_CHECK("mask_unit_data");
  return SAH_OK;
}

// ---- row-wise column lists -> dense, last duplicate wins -----------------------------------------
// Mask.create_from_row_wise_idx in dense mode (utils/mask.py:335-395) scatters data[row][j] to
// dense[row][idx[row][j]]; on the CPU the last duplicate of a column wins.  Here every (row, j)
// claims its column with an atomic maximum of (j + 1, value bits), so the winner is the same
// whatever order the threads run in; a second pass turns the claims into the dense tensor.
template <typename T>
__device__ __forceinline__ unsigned int mask_value_bits(T v);
template <>
__device__ __forceinline__ unsigned int mask_value_bits<float>(float v) { return __float_as_uint(v); }
template <>
__device__ __forceinline__ unsigned int mask_value_bits<__nv_bfloat16>(__nv_bfloat16 v) {
  return (unsigned int)__bfloat16_as_ushort(v);
}
template <typename T>
__device__ __forceinline__ T mask_value_from_bits(unsigned int b);
template <>
__device__ __forceinline__ float mask_value_from_bits<float>(unsigned int b) { return __uint_as_float(b); }
template <>
__device__ __forceinline__ __nv_bfloat16 mask_value_from_bits<__nv_bfloat16>(unsigned int b) {
  return __ushort_as_bfloat16((unsigned short)b);
}

template <typename T>
__global__ void mask_rowwise_claim_kernel(const int64_t* __restrict__ idx, const T* __restrict__ vals,
                                          int64_t rows, int64_t k, int64_t S,
                                          unsigned long long* __restrict__ claims) {
  sah_pdl_entry_early();
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * k) return;
  const int64_t row = t / k, j = t - row * k;
  const int64_t col = idx[t];
  if (col < 0 || col >= S) return;
  atomicMax(&claims[row * S + col],
            ((unsigned long long)(j + 1) << 32) | (unsigned long long)mask_value_bits<T>(vals[t]));
}

template <typename T>
__global__ void mask_rowwise_settle_kernel(const unsigned long long* __restrict__ claims, int64_t n,
                                           T* __restrict__ dense) {
  sah_pdl_entry_early();
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) return;
  const unsigned long long c = claims[t];
  dense[t] = c ? mask_value_from_bits<T>((unsigned int)(c & 0xffffffffull)) : sah_from_float<T>(0.f);
}

extern "C" int sah_mask_rowwise_scatter(const int64_t* idx, const void* vals, int dtype, int64_t rows,
                                        int64_t k, int64_t S, void* claims, void* dense, void* stream) {
  SAH_REQUIRE(idx && vals && claims && dense, "rowwise_scatter: null pointer");
  SAH_REQUIRE(rows >= 0 && k > 0 && S > 0 && k < (1ll << 31), "rowwise_scatter: bad extents");
  if (rows == 0) return SAH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(claims, 0, (size_t)(rows * S) * sizeof(unsigned long long), st);
  if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "rowwise_scatter: memset: %s", cudaGetErrorString(e));
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_rowwise_claim_kernel<T>, (unsigned)sah_ceil_div(rows * k, 256), 256, 0, st, idx,
        (const T*)vals, rows, k, S, (unsigned long long*)claims);
    SAH_LAUNCH_CHECK("mask_rowwise_claim");
    sah_launch_chain(mask_rowwise_settle_kernel<T>, (unsigned)sah_ceil_div(rows * S, 256), 256, 0, st,
        (const unsigned long long*)claims, rows * S, (T*)dense);
  });
  SAH_LAUNCH_CHECK("mask_rowwise_settle");
  return SAH_OK;
}

// ---- index-form merge: sum of duplicates, clamp -------------------------------------------------
// Mask.merge_mask_sparse (utils/mask.py:893-1062) concatenates the two index lists, sorts them,
// sums the values of equal indices and clamps to [0, 1].  The sums are taken here in a float32
// array over all positions (atomic adds: exact for the one or two terms a position normally
// gets, order-independent up to float32 rounding beyond that), then clamped and rounded once.
template <typename T>
__global__ void mask_flat_add_kernel(const int64_t* __restrict__ flat, const T* __restrict__ vals,
                                     int64_t n, int64_t total, float* __restrict__ acc) {
  sah_pdl_entry_early();
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) return;
  const int64_t i = flat[t];
  if (i < 0 || i >= total) return;
  atomicAdd(&acc[i], vals ? sah_to_float<T>(vals[t]) : 1.f);
}

template <typename T>
__global__ void mask_clamp_kernel(const float* __restrict__ acc, int64_t total, T* __restrict__ dense) {
  sah_pdl_entry_early();
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const float v = sah_round_to<T>(acc[t]);  // the sum lives in the mask dtype
  dense[t] = sah_from_float<T>(fminf(fmaxf(v, 0.f), 1.f));
}

extern "C" int sah_mask_flat_add(const int64_t* flat_idx, const void* vals, int dtype, int64_t n,
                                 int64_t total, float* acc, void* stream) {
  SAH_REQUIRE(acc != nullptr && n >= 0 && total > 0, "flat_add: bad argument");
  if (n == 0) return SAH_OK;
  SAH_REQUIRE(flat_idx != nullptr, "flat_add: indices are null");
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_flat_add_kernel<T>, (unsigned)sah_ceil_div(n, 256), 256, 0, (cudaStream_t)stream,
        flat_idx, (const T*)vals, n, total, acc);
  });
  SAH_LAUNCH_CHECK("mask_flat_add");
  return SAH_OK;
}

extern "C" int sah_mask_clamp_to_dense(const float* acc, int dtype, int64_t total, void* dense,
                                       void* stream) {
  SAH_REQUIRE(acc && dense && total > 0, "clamp_to_dense: bad argument");
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_clamp_kernel<T>, (unsigned)sah_ceil_div(total, 256), 256, 0, (cudaStream_t)stream,
        acc, total, (T*)dense);
  });
  SAH_LAUNCH_CHECK("mask_clamp");
  return SAH_OK;
}

// ---- ragged sample list -> bitmap ----------------------------------------------------------
__global__ void mask_scatter_samples_kernel(const int64_t* __restrict__ cols,
                                            const int64_t* __restrict__ sptr, int64_t rows,
                                            int64_t n_max, int64_t S, int64_t W,
                                            uint32_t* __restrict__ bits) {
  sah_pdl_entry_early();
  int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n_max || j >= sptr[rows]) return;
  // row = last r with sptr[r] <= j
  int64_t lo = 0, hi = rows;  // invariant: sptr[lo] <= j < sptr[hi]
  while (hi - lo > 1) {
    int64_t mid = (lo + hi) >> 1;
    if (sptr[mid] <= j) lo = mid; else hi = mid;
  }
  int64_t c = cols[j];
  if (c < 0 || c >= S) return;
  atomicOr(bits + lo * W + (c >> 5), 1u << (c & 31));
}

extern "C" int sah_mask_scatter_samples(const int64_t* cols, const int64_t* sptr, int64_t rows,
                                        int64_t n_max, int64_t S, int64_t W, uint32_t* bits,
                                        void* stream) {
  SAH_REQUIRE(cols && sptr && bits, "scatter_samples: null pointer");
  if (rows == 0 || n_max == 0) return SAH_OK;
  sah_launch_chain(mask_scatter_samples_kernel, (unsigned)sah_ceil_div(n_max, 256), 256, 0,
                                (cudaStream_t)stream, cols, sptr, rows, n_max, S, W, bits);
  SAH_LAUNCH_CHECK("mask_scatter_samples");
  return SAH_OK;
}

// ---- merge of two weighted bitmap masks -------------------------------------------------------
// Mask.merge_mask_dense (utils/mask.py:875-877): clamp(a + b, 0, 1) in the mask dtype, an
// entry being active when the result is non-zero.  A mask without a data array has unit
// weights.  Two passes: the bitmap of the result, then (after a row scan of that bitmap) its
// weights in CSR order.
struct MergeSide {
  const uint32_t* bits;
  const void* data;      // null: unit weights
  const int32_t* wpre;   // needed with data
  const int64_t* ptr;    // needed with data
};

template <typename T>
__device__ __forceinline__ float merge_side_weight(const MergeSide& s, int64_t row, int64_t t,
                                                   uint32_t word, int bit) {
  if (!((word >> bit) & 1u)) return 0.f;
  if (s.data == nullptr) return 1.f;
  const int64_t pos = s.ptr[row] + s.wpre[t] + __popc(word & ((1u << bit) - 1u));
  return sah_to_float<T>(reinterpret_cast<const T*>(s.data)[pos]);
}

template <typename T>
__device__ __forceinline__ float merge_weight(float a, float b) {
  const float s = sah_round_to<T>(__fadd_rn(a, b));
  return fminf(fmaxf(s, 0.f), 1.f);
}

template <typename T>
__global__ void mask_merge_bits_kernel(MergeSide a, MergeSide b, int64_t rows, int64_t W,
                                       uint32_t* __restrict__ out) {
  sah_pdl_entry_early();
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * W) return;
  const uint32_t wa = a.bits[t], wb = b.bits[t];
  uint32_t m = wa | wb, keep = m;
  if (a.data != nullptr || b.data != nullptr) {
    const int64_t row = t / W;
    while (m) {
      const int bit = __ffs(m) - 1;
      m &= m - 1;
      const float w = merge_weight<T>(merge_side_weight<T>(a, row, t, wa, bit),
                                      merge_side_weight<T>(b, row, t, wb, bit));
      if (!(w != 0.f)) keep &= ~(1u << bit);
    }
  }
  out[t] = keep;
}

template <typename T>
__global__ void mask_merge_data_kernel(MergeSide a, MergeSide b, int64_t rows, int64_t W,
                                       const uint32_t* __restrict__ outb,
                                       const int32_t* __restrict__ out_wpre,
                                       const int64_t* __restrict__ out_ptr, T* __restrict__ data) {
  sah_pdl_entry_early();
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * W) return;
  uint32_t m = outb[t];
  if (!m) return;
  const int64_t row = t / W;
  const uint32_t wa = a.bits[t], wb = b.bits[t];
  int64_t o = out_ptr[row] + out_wpre[t];
  while (m) {
    const int bit = __ffs(m) - 1;
    m &= m - 1;
    data[o++] = sah_from_float<T>(merge_weight<T>(merge_side_weight<T>(a, row, t, wa, bit),
                                                  merge_side_weight<T>(b, row, t, wb, bit)));
  }
}

static int merge_check(const uint32_t* bits, const void* data, const int32_t* wpre, const int64_t* ptr) {
  return bits != nullptr && (data == nullptr || (wpre != nullptr && ptr != nullptr));
}

extern "C" int sah_mask_merge_bits(const uint32_t* a_bits, const void* a_data, const int32_t* a_wpre,
                                   const int64_t* a_ptr, const uint32_t* b_bits, const void* b_data,
                                   const int32_t* b_wpre, const int64_t* b_ptr, int dtype,
                                   int64_t rows, int64_t W, uint32_t* out_bits, void* stream) {
  SAH_REQUIRE(merge_check(a_bits, a_data, a_wpre, a_ptr) && merge_check(b_bits, b_data, b_wpre, b_ptr) && out_bits,
              "mask_merge_bits: null pointer (data needs wpre and ptr)");
  if (rows == 0 || W == 0) return SAH_OK;
  MergeSide a{a_bits, a_data, a_wpre, a_ptr}, b{b_bits, b_data, b_wpre, b_ptr};
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_merge_bits_kernel<T>, (unsigned)sah_ceil_div(rows * W, 256), 256, 0,
        (cudaStream_t)stream, a, b, rows, W, out_bits);
  });
  SAH_LAUNCH_CHECK("mask_merge_bits");
  return SAH_OK;
}

extern "C" int sah_mask_merge_data(const uint32_t* a_bits, const void* a_data, const int32_t* a_wpre,
                                   const int64_t* a_ptr, const uint32_t* b_bits, const void* b_data,
                                   const int32_t* b_wpre, const int64_t* b_ptr, int dtype,
                                   int64_t rows, int64_t W, const uint32_t* out_bits,
                                   const int32_t* out_wpre, const int64_t* out_ptr, void* out_data,
                                   void* stream) {
  SAH_REQUIRE(merge_check(a_bits, a_data, a_wpre, a_ptr) && merge_check(b_bits, b_data, b_wpre, b_ptr),
              "mask_merge_data: null pointer (data needs wpre and ptr)");
  SAH_REQUIRE(out_bits && out_wpre && out_ptr && out_data, "mask_merge_data: null output");
  if (rows == 0 || W == 0) return SAH_OK;
  MergeSide a{a_bits, a_data, a_wpre, a_ptr}, b{b_bits, b_data, b_wpre, b_ptr};
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(mask_merge_data_kernel<T>, (unsigned)sah_ceil_div(rows * W, 256), 256, 0,
        (cudaStream_t)stream, a, b, rows, W, out_bits, out_wpre, out_ptr, reinterpret_cast<T*>(out_data));
  });
  SAH_LAUNCH_CHECK("mask_merge_data");
  return SAH_OK;
}

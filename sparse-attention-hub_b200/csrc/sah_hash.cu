// HashAttention kernels (maskers/fixed/implementations/hashattention_top_k.py):
//   sah_hash_encode  per-head MLP -> sign bits -> one uint32 per vector
//   sah_hash_topk    Hamming-score top-k with lowest-column tie-break
#include "sah_common.cuh"
#include "sah_select.cuh"

// ---------------------------------------------------------------------------
// Encode.  One CTA hashes a tile of TK vectors of one (batch, output head).
// Activations live in shared memory as fp32 [channel][vector]; one layer is a
// register-tiled product where each thread owns KT vectors x 4 outputs and
// walks the input channels in ascending order with a single fp32 accumulator
// per output, which fixes the summation order the CPU restatement follows.
// ---------------------------------------------------------------------------
#define HE_TK 64        // vectors per CTA
#define HE_THREADS 256
#define HE_MAXD 128     // widest layer

struct HashEncodeArgs {
  const void* x;
  int64_t xs_b, xs_h, xs_n;
  int H_in, H_out;
  int64_t n_begin, n_end, n_total;
  int n_layers;
  int dims[5];
  const void* weights[4];
  const void* bias[4];
  int act;
  const uint16_t* act_table;
  uint32_t* codes;
};

template <typename T>
__device__ __forceinline__ float he_activate(float v, int act, const uint16_t* table);

template <>
__device__ __forceinline__ float he_activate<__nv_bfloat16>(float v, int act,
                                                            const uint16_t* table) {
  // v is a bf16 value; the table maps bf16 bit patterns to bf16 bit patterns.
  uint32_t b = __float_as_uint(v) >> 16;
  return __uint_as_float(((uint32_t)table[b]) << 16);
}

template <>
__device__ __forceinline__ float he_activate<float>(float v, int act, const uint16_t*) {
  switch (act) {
    case SAH_ACT_RELU: return fmaxf(v, 0.f);
    case SAH_ACT_SILU: return v / (1.f + expf(-v));
    case SAH_ACT_GELU: return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f));
    default: return tanhf(v);
  }
}

#include "sah_hash_tc.cuh"

template <typename T, int KT>
__device__ __forceinline__ void he_layer(const float* __restrict__ a_in, float* __restrict__ a_out,
                                         const float* __restrict__ w_sm,
                                         const T* __restrict__ bias_h, int din, int dout,
                                         bool last, int act, const uint16_t* act_table,
                                         unsigned int* codes_sm) {
  const int nkg = HE_TK / KT;  // vector groups
  const int tk = threadIdx.x % nkg, to = threadIdx.x / nkg;
  float acc[KT][4];
#pragma unroll
  for (int i = 0; i < KT; ++i)
#pragma unroll
    for (int o = 0; o < 4; ++o) acc[i][o] = 0.f;

  for (int d = 0; d < din; ++d) {
    float a[KT];
    const float* ap = a_in + d * HE_TK + tk * KT;
#pragma unroll
    for (int i = 0; i < KT; ++i) a[i] = ap[i];
    const float4 w = *reinterpret_cast<const float4*>(w_sm + d * dout + to * 4);
#pragma unroll
    for (int i = 0; i < KT; ++i) {
      acc[i][0] = fmaf(a[i], w.x, acc[i][0]);
      acc[i][1] = fmaf(a[i], w.y, acc[i][1]);
      acc[i][2] = fmaf(a[i], w.z, acc[i][2]);
      acc[i][3] = fmaf(a[i], w.w, acc[i][3]);
    }
  }

  float b[4];
#pragma unroll
  for (int o = 0; o < 4; ++o) b[o] = sah_to_float<T>(bias_h[to * 4 + o]);

#pragma unroll
  for (int i = 0; i < KT; ++i) {
    unsigned int nib = 0u;
#pragma unroll
    for (int o = 0; o < 4; ++o) {
      float v = sah_round_to<T>(acc[i][o]);        // einsum output in dtype
      v = sah_round_to<T>(__fadd_rn(v, b[o]));     // + bias, rounded
      if (!last) {
        v = he_activate<T>(v, act, act_table);
        a_out[(to * 4 + o) * HE_TK + tk * KT + i] = v;
      } else {
        nib |= (v > 0.f ? 1u : 0u) << o;
      }
    }
    if (last && nib) atomicOr(&codes_sm[tk * KT + i], nib << (to * 4));
  }
}

template <typename T>
__global__ void __launch_bounds__(HE_THREADS)
hash_encode_kernel(HashEncodeArgs p) {
  extern __shared__ __align__(16) unsigned char he_smem[];
  float* act0 = reinterpret_cast<float*>(he_smem);
  float* act1 = act0 + HE_MAXD * HE_TK;
  float* w_sm = act1 + HE_MAXD * HE_TK;
  __shared__ unsigned int codes_sm[HE_TK];

  const int64_t tile = blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int h_in = h / (p.H_out / p.H_in);
  const int64_t n0 = p.n_begin + tile * HE_TK;
  const int D = p.dims[0];
  const T* xb = reinterpret_cast<const T*>(p.x) + b * p.xs_b + h_in * p.xs_h;

  // Stage the input tile transposed: act0[d][i].
  const int chunks = D / 8;
  for (int idx = threadIdx.x; idx < HE_TK * chunks; idx += HE_THREADS) {
    int i = idx % HE_TK, c = idx / HE_TK;
    int64_t n = n0 + i;
    float f[8];
    if (n < p.n_end) {
      sah_load8<T>(xb + n * p.xs_n + c * 8, f);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) act0[(c * 8 + e) * HE_TK + i] = f[e];
  }
  if (threadIdx.x < HE_TK) codes_sm[threadIdx.x] = 0u;

  float* a_in = act0;
  float* a_out = act1;
  for (int l = 0; l < p.n_layers; ++l) {
    const int din = p.dims[l], dout = p.dims[l + 1];
    __syncthreads();  // previous layer done with w_sm / a_out complete
    const T* wl = reinterpret_cast<const T*>(p.weights[l]) + (int64_t)h * din * dout;
    for (int idx = threadIdx.x; idx < din * dout; idx += HE_THREADS)
      w_sm[idx] = sah_to_float<T>(wl[idx]);
    __syncthreads();
    const T* bl = reinterpret_cast<const T*>(p.bias[l]) + (int64_t)h * dout;
    const bool last = (l == p.n_layers - 1);
    switch (dout) {
      case 128: he_layer<T, 8>(a_in, a_out, w_sm, bl, din, dout, last, p.act, p.act_table, codes_sm); break;
      case 64:  he_layer<T, 4>(a_in, a_out, w_sm, bl, din, dout, last, p.act, p.act_table, codes_sm); break;
      case 32:  he_layer<T, 2>(a_in, a_out, w_sm, bl, din, dout, last, p.act, p.act_table, codes_sm); break;
      default:  he_layer<T, 1>(a_in, a_out, w_sm, bl, din, dout, last, p.act, p.act_table, codes_sm); break;
    }
    float* t = a_in; a_in = a_out; a_out = t;
  }
  __syncthreads();
  if (threadIdx.x < HE_TK) {
    int64_t n = n0 + threadIdx.x;
    if (n < p.n_end)
      p.codes[((int64_t)b * p.H_out + h) * p.n_total + n] = codes_sm[threadIdx.x];
  }
}

// Few vectors per head (a decode step hashes one query and at most a few new
// keys): one CTA per vector, thread e owns output e of the current layer and
// walks the input channels in the same ascending order as the tiled kernel, so
// both produce identical bits.  Weight reads are coalesced across outputs.
#define HE_SMALL_MAX 16

__device__ __forceinline__ void he_cp_async16(void* smem_dst, const void* gmem_src) {
  unsigned int d = (unsigned int)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src));
}

template <typename T>
__global__ void __launch_bounds__(HE_MAXD)
hash_encode_small_kernel(HashEncodeArgs p) {
  sah_pdl_entry_early();
  extern __shared__ __align__(16) unsigned char hes_smem[];  // every layer's weights of head h
  __shared__ float xa[HE_MAXD];
  __shared__ float xb[HE_MAXD];
  const int64_t n = p.n_begin + blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int h_in = h / (p.H_out / p.H_in);
  const int e = threadIdx.x;
  const T* xr = reinterpret_cast<const T*>(p.x) + b * p.xs_b + h_in * p.xs_h + n * p.xs_n;
  if (e < p.dims[0]) xa[e] = sah_to_float<T>(xr[e]);
  float* a_in = xa;
  float* a_out = xb;
  unsigned int code = 0u;
  // Every layer's matrix is requested up front, one cp.async group per layer, each into its
  // own region: the step is latency bound, so later layers load while earlier ones compute.
  const int layer_bytes = HE_MAXD * HE_MAXD * (int)sizeof(T);
  for (int l = 0; l < p.n_layers; ++l) {
    const int din = p.dims[l], dout = p.dims[l + 1];
    const unsigned char* src = reinterpret_cast<const unsigned char*>(
        reinterpret_cast<const T*>(p.weights[l]) + (int64_t)h * din * dout);
    const int n16 = din * dout * (int)sizeof(T) / 16;
    for (int i = threadIdx.x; i < n16; i += HE_MAXD)
      he_cp_async16(hes_smem + l * layer_bytes + i * 16, src + i * 16);
    asm volatile("cp.async.commit_group;\n" ::);
  }
  // The step is a chain of dependent latencies; whatever does not depend on the activations is
  // asked for now: every layer's bias, and (bf16) the activation table pulled towards L2, one
  // 128-byte line per thread and a different eighth of the table per head.
  float bias_r[4];
#pragma unroll
  for (int l = 0; l < 4; ++l)
    bias_r[l] = (l < p.n_layers && e < p.dims[l + 1])
                    ? sah_to_float<T>(reinterpret_cast<const T*>(p.bias[l])[(int64_t)h * p.dims[l + 1] + e])
                    : 0.f;
  if (sizeof(T) == 2 && p.act_table != nullptr && p.n_layers > 1) {
    const unsigned char* line = reinterpret_cast<const unsigned char*>(p.act_table) +
                                ((size_t)((h & 7) * HE_MAXD + e) << 7);
    asm volatile("prefetch.global.L2 [%0];\n" ::"l"(line));
  }
#pragma unroll
  for (int l = 0; l < 4; ++l) {
    if (l >= p.n_layers) break;
    const int din = p.dims[l], dout = p.dims[l + 1];
    const bool last = (l == p.n_layers - 1);
    const T* w_l = reinterpret_cast<const T*>(hes_smem + l * layer_bytes);
    // groups complete in order: layer l is there once at most n_layers - 1 - l are pending
    switch (p.n_layers - 1 - l) {
      case 0: asm volatile("cp.async.wait_group 0;\n" ::); break;
      case 1: asm volatile("cp.async.wait_group 1;\n" ::); break;
      case 2: asm volatile("cp.async.wait_group 2;\n" ::); break;
      default: asm volatile("cp.async.wait_group 3;\n" ::); break;
    }
    __syncthreads();  // everybody's copies of layer l have landed, and a_in is written
    float v = 0.f;
    if (e < dout) {
      float acc = 0.f;
#pragma unroll 8
      for (int d = 0; d < din; ++d) acc = fmaf(a_in[d], sah_to_float<T>(w_l[d * dout + e]), acc);
      v = sah_round_to<T>(acc);
      v = sah_round_to<T>(__fadd_rn(v, bias_r[l]));
      if (!last) a_out[e] = he_activate<T>(v, p.act, p.act_table);
    }
    if (last && threadIdx.x < 32) code = __ballot_sync(0xffffffffu, e < dout && v > 0.f);
    float* t = a_in; a_in = a_out; a_out = t;
  }
  if (threadIdx.x == 0) p.codes[((int64_t)b * p.H_out + h) * p.n_total + n] = code;
}

extern "C" int sah_hash_encode(const void* x, int dtype, int64_t xs_b, int64_t xs_h,
                               int64_t xs_n, int B, int H_in, int H_out, int64_t n_begin,
                               int64_t n_end, int64_t n_total, int n_layers, const int* dims,
                               const void* const* weights, const void* const* bias, int act,
                               const uint16_t* act_table, uint32_t* codes, void* stream) {
  SAH_REQUIRE(x && dims && weights && bias && codes, "hash_encode: null pointer");
  SAH_REQUIRE(B > 0 && H_in > 0 && H_out > 0 && H_out % H_in == 0, "hash_encode: bad heads");
  SAH_REQUIRE(0 <= n_begin && n_begin <= n_end && n_end <= n_total, "hash_encode: bad range");
  if (n_layers < 1 || n_layers > 4)
    return sah_fail(SAH_ERR_UNSUPPORTED, "hash_encode: %d layers (1..4 supported)", n_layers);
  for (int l = 0; l <= n_layers; ++l) {
    int d = dims[l];
    bool ok = (l == 0) ? (d % 8 == 0 && d >= 8 && d <= HE_MAXD)
                       : (d == 16 || d == 32 || d == 64 || d == 128);
    if (!ok)
      return sah_fail(SAH_ERR_UNSUPPORTED,
                      "hash_encode: layer width %d at position %d (input: multiple of 8 up to "
                      "128; outputs: 16, 32, 64 or 128)", d, l);
  }
  if (dims[n_layers] > 32)
    return sah_fail(SAH_ERR_UNSUPPORTED, "hash_encode: %d signature bits (<= 32 supported)",
                    dims[n_layers]);
  SAH_REQUIRE(act >= SAH_ACT_RELU && act <= SAH_ACT_TANH, "hash_encode: bad activation");
  SAH_REQUIRE(dtype != SAH_BF16 || n_layers == 1 || act_table != nullptr,
              "hash_encode: bf16 needs the activation table");
  SAH_REQUIRE(xs_n % 8 == 0 && xs_h % 8 == 0 && xs_b % 8 == 0 &&
                  ((uintptr_t)x % 16 == 0),
              "hash_encode: x rows must be 16-byte aligned");
  if (n_begin == n_end) return SAH_OK;

  HashEncodeArgs p;
  p.x = x; p.xs_b = xs_b; p.xs_h = xs_h; p.xs_n = xs_n;
  p.H_in = H_in; p.H_out = H_out;
  p.n_begin = n_begin; p.n_end = n_end; p.n_total = n_total;
  p.n_layers = n_layers;
  for (int l = 0; l < 5; ++l) p.dims[l] = (l <= n_layers) ? dims[l] : 0;
  for (int l = 0; l < 4; ++l) {
    p.weights[l] = (l < n_layers) ? weights[l] : nullptr;
    p.bias[l] = (l < n_layers) ? bias[l] : nullptr;
    if (l < n_layers) SAH_REQUIRE(p.weights[l] && p.bias[l], "hash_encode: null layer %d", l);
  }
  p.act = act; p.act_table = act_table; p.codes = codes;

  cudaStream_t st = (cudaStream_t)stream;
  const size_t small_bytes = (size_t)n_layers * HE_MAXD * HE_MAXD * (dtype == SAH_BF16 ? 2 : 4);
  if (n_end - n_begin <= HE_SMALL_MAX && small_bytes <= 200 * 1024) {
    // decode-time shapes (queries, appended keys): one CTA per vector
    sah_prof_begin(SAH_PROF_HASH_ENCODE, st);
    dim3 sgrid((unsigned)(n_end - n_begin), (unsigned)H_out, (unsigned)B);
    SAH_DISPATCH_DTYPE(dtype, T, {
      const int wbytes = n_layers * HE_MAXD * HE_MAXD * (int)sizeof(T);
      if (wbytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(hash_encode_small_kernel<T>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, wbytes);
        if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "hash_encode attr: %s", cudaGetErrorString(e));
      }
      for (int l = 0; l < n_layers; ++l)
        SAH_REQUIRE(((uintptr_t)weights[l] % 16) == 0, "hash_encode: weights must be 16-byte aligned");
      sah_launch_chain(hash_encode_small_kernel<T>, sgrid, HE_MAXD, wbytes, st, p);
    });
    SAH_LAUNCH_CHECK("hash_encode_small");
    sah_prof_end(SAH_PROF_HASH_ENCODE, st);
    return SAH_OK;
  }
  // SAH_HASH_TC=1 in the environment sends bfloat16 index builds through the tensor-core kernel
  // (same bits, see sah_hash_tc.cuh).  It is not the default: each layer rounds its products to
  // bfloat16, about 31 % of the accumulators lie within the error band of a rounding midpoint, so
  // nearly every warp repeats nearly every output in the fixed order and the build takes 2.6x to
  // 4.6x as long as hash_encode_kernel (134 ms against 52 ms for 8 x 32768 keys x 32 heads).
  const char* tc_e = getenv("SAH_HASH_TC");
  const int tc_env = (tc_e != nullptr && tc_e[0] == '1') ? 1 : 0;
  bool tc = tc_env == 1 && dtype == SAH_BF16 && n_layers <= HTC_MAX_LAYERS && n_end - n_begin >= 1024 &&
            (n_layers == 1 || act_table != nullptr);
  for (int l = 0; l <= n_layers && tc; ++l) tc = dims[l] % 16 == 0 && dims[l] >= 16 && dims[l] <= 128;
  for (int l = 0; l < n_layers && tc; ++l) tc = ((uintptr_t)weights[l] % 2) == 0;
  if (tc) {
    HashTcArgs a;
    a.x = reinterpret_cast<const __nv_bfloat16*>(x);
    a.xs_b = xs_b; a.xs_h = xs_h; a.xs_n = xs_n;
    a.H_in = H_in; a.H_out = H_out;
    a.n_begin = n_begin; a.n_end = n_end; a.n_total = n_total;
    a.n_layers = n_layers;
    int off = 2 * HTC_TILE * 128;  // the A tile
    for (int l = 0; l <= HTC_MAX_LAYERS; ++l) a.dims[l] = l <= n_layers ? dims[l] : 0;
    for (int l = 0; l < HTC_MAX_LAYERS; ++l) {
      a.weights[l] = l < n_layers ? reinterpret_cast<const __nv_bfloat16*>(weights[l]) : nullptr;
      a.bias[l] = l < n_layers ? reinterpret_cast<const __nv_bfloat16*>(bias[l]) : nullptr;
      a.b_off[l] = off;
      if (l < n_layers) off += ((dims[l] + 63) / 64) * dims[l + 1] * 128;
      off = (off + 1023) & ~1023;
    }
    a.wn_off = off;   off += HTC_MAX_LAYERS * 128 * 4;
    a.bias_off = off; off += HTC_MAX_LAYERS * 128 * 4;
    a.misc_off = off; off += 64;
    a.act_table = act_table;
    a.codes = codes;
    const int tc_smem = 1024 + off;
    static int tc_allowed = 0;
    if (tc_smem > tc_allowed) {
      cudaError_t e = cudaFuncSetAttribute(hash_encode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem);
      if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "hash_encode_tc attr: %s", cudaGetErrorString(e));
      tc_allowed = tc_smem;
    }
    // about two CTAs per SM in all, each with a contiguous slice of the key tiles
    const int64_t n_tiles = sah_ceil_div(n_end - n_begin, (int64_t)HTC_TILE);
    int64_t slices = sah_ceil_div((int64_t)2 * 148, (int64_t)H_out * B);
    if (slices > n_tiles) slices = n_tiles;
    if (slices < 1) slices = 1;
    dim3 tgrid((unsigned)slices, (unsigned)H_out, (unsigned)B);
    sah_prof_begin(SAH_PROF_HASH_ENCODE, st);
    hash_encode_tc_kernel<<<tgrid, HTC_THREADS, tc_smem, st>>>(a);
    SAH_LAUNCH_CHECK("hash_encode_tc");
    sah_prof_end(SAH_PROF_HASH_ENCODE, st);
    return SAH_OK;
  }
  const size_t smem = (size_t)(2 * HE_MAXD * HE_TK + HE_MAXD * HE_MAXD) * sizeof(float);
  dim3 grid((unsigned)sah_ceil_div(n_end - n_begin, HE_TK), (unsigned)H_out, (unsigned)B);
  sah_prof_begin(SAH_PROF_HASH_ENCODE, (cudaStream_t)stream);
  SAH_DISPATCH_DTYPE(dtype, T, {
    cudaError_t e = cudaFuncSetAttribute(hash_encode_kernel<T>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "hash_encode attr: %s", cudaGetErrorString(e));
    hash_encode_kernel<T><<<grid, HE_THREADS, smem, st>>>(p);
  });
  SAH_LAUNCH_CHECK("hash_encode");
  sah_prof_end(SAH_PROF_HASH_ENCODE, (cudaStream_t)stream);
  return SAH_OK;
}

// ---------------------------------------------------------------------------
// Top-k over Hamming scores.
// ---------------------------------------------------------------------------
struct HashKeyPlain {
  const uint32_t* kc;
  uint32_t qc;
  int nbits;
  __device__ __forceinline__ unsigned int operator()(int64_t j) const {
    return (unsigned int)(nbits - __popc(kc[j] ^ qc));  // matching bits: monotone in the score
  }
};

template <typename T, int KEYBITS>
struct HashKeyBiased {
  const uint32_t* kc;
  uint32_t qc;
  int nbits;
  const T* bias;
  __device__ __forceinline__ unsigned int operator()(int64_t j) const {
    float s = (float)(nbits - 2 * __popc(kc[j] ^ qc));
    float f = sah_round_to<T>(__fadd_rn(s, sah_to_float<T>(bias[j]))) + 0.0f;
    unsigned int key = sah_float_key(f);
    return KEYBITS == 16 ? (key >> 16) : key;
  }
};

template <typename T, int KEYBITS, bool BIASED>
__global__ void __launch_bounds__(SAH_SELECT_THREADS)
hash_topk_kernel(const uint32_t* __restrict__ kcodes, int64_t kc_stride,
                 const uint32_t* __restrict__ qcodes, int nbits, const T* __restrict__ bias, int64_t bias_s_b, int64_t bias_s_h,
                 int64_t bias_s_q, int Hq, int Sq, int64_t S, int64_t W,
                 const uint32_t* __restrict__ prev_bits, int64_t k,
                 uint32_t* __restrict__ out_bits) {
  sah_pdl_entry();
  __shared__ SahSelectSmem sm;
  const int64_t row = blockIdx.x;
  const int q = (int)(row % Sq);
  const int64_t bh = row / Sq;
  const int h = (int)(bh % Hq);
  const int64_t b = bh / Hq;
  const uint32_t* kc = kcodes + bh * kc_stride;
  const uint32_t qc = qcodes[row];
  if (BIASED) {
    HashKeyBiased<T, KEYBITS> kf{kc, qc, nbits, bias + b * bias_s_b + h * bias_s_h + q * bias_s_q};
    sah_select_row<KEYBITS>(kf, prev_bits + row * W, out_bits + row * W, S, W, 0, S, k, sm);
  } else {
    HashKeyPlain kf{kc, qc, nbits};
    sah_select_row<8>(kf, prev_bits + row * W, out_bits + row * W, S, W, 0, S, k, sm);
  }
}

// Counting select for the unbiased case: a score takes at most nbits + 1
// values, so the k-th best score and the number of ties to take at it follow
// from one histogram.  Each thread owns one bitmap word, i.e. 32 consecutive
// keys (128 contiguous bytes of codes, read with 16-byte loads, all of them in
// flight before the first use).  Pass 1 histograms the inactive keys (per-warp
// shared-memory bins); pass 2 re-reads the codes (cache resident) and emits
// the word: keys above the threshold, plus ties in column order through one
// ordered block scan.
#define HT_BINS 40  // >= nbits + 1, padded

__device__ __forceinline__ void ht_load_codes(const uint32_t* __restrict__ kc, int64_t w, int64_t S,
                                              bool aligned, uint32_t* codes) {
  const int64_t c0 = w * 32;
  if (aligned && c0 + 32 <= S) {
    const uint4* p = reinterpret_cast<const uint4*>(kc + c0);
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = p[i];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      codes[4 * i + 0] = v[i].x; codes[4 * i + 1] = v[i].y;
      codes[4 * i + 2] = v[i].z; codes[4 * i + 3] = v[i].w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) codes[i] = (c0 + i < S) ? kc[c0 + i] : 0u;
  }
}

__global__ void __launch_bounds__(1024)
hash_topk_fast_kernel(const uint32_t* __restrict__ kcodes, int64_t kc_stride,
                      const uint32_t* __restrict__ qcodes, int nbits, int Sq, int64_t S, int64_t W,
                      const uint32_t* __restrict__ prev_bits, int64_t k,
                      uint32_t* __restrict__ out_bits) {
  sah_pdl_entry();
  __shared__ unsigned int hist[32][HT_BINS];
  __shared__ long long scan[33];
  __shared__ int thr_sm;
  __shared__ long long need_sm;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row = blockIdx.x;
  const uint32_t* kc = kcodes + (row / Sq) * kc_stride;  // codes are shared by a head's queries
  const uint32_t qc = qcodes[row];
  const uint32_t* prev_row = prev_bits + row * W;
  uint32_t* out_row = out_bits + row * W;
  const bool aligned = ((reinterpret_cast<uintptr_t>(kc) & 15) == 0);

  // Scores below `floor_sm` are left out of the histogram; a floor above zero is
  // only a shortcut (retried at zero when fewer than k keys clear it).
  __shared__ int floor_sm;
  __shared__ int retry_sm;
  if (tid == 0) floor_sm = 0;

  for (int attempt = 0; attempt < 2; ++attempt) {
  for (int i = tid; i < 32 * HT_BINS; i += 1024) (&hist[0][0])[i] = 0u;
  __syncthreads();
  const int floor_bin = floor_sm;

  // ---- pass 1: histogram of matching-bit counts >= floor over inactive keys ----
  for (int64_t w = tid; w < W; w += 1024) {
    uint32_t codes[32];
    ht_load_codes(kc, w, S, aligned, codes);
    const uint32_t pw = prev_row[w];
    const int64_t c0 = w * 32;
    uint32_t valid = ~pw;
    if (c0 + 32 > S) valid &= (c0 >= S) ? 0u : ((1u << (S - c0)) - 1u);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int sc = nbits - __popc(codes[i] ^ qc);
      if (sc >= floor_bin && ((valid >> i) & 1u)) atomicAdd(&hist[warp][sc], 1u);
    }
  }
  __syncthreads();
  if (warp == 0) {
    // lane b owns bin b (b = 0..31); bin 32 (all bits match) is handled aside
    unsigned int mine = 0u, top = 0u;
    for (int w2 = 0; w2 < 32; ++w2) {
      mine += hist[w2][lane];
      top += hist[w2][32];
    }
    unsigned int incl = mine;  // suffix sum over lanes: keys with bin >= lane (bins <= 31)
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned int n = __shfl_down_sync(0xffffffffu, incl, o);
      if (lane + o < 32) incl += n;
    }
    const long long ge = (long long)incl + top;   // keys scoring >= this lane's bin
    const long long total = __shfl_sync(0xffffffffu, (long long)incl, 0) + top;
    int thr;
    long long need;
    int retry = 0;
    if (k <= 0) {
      thr = 64; need = 0;                 // nothing qualifies
    } else if (total < k && floor_bin > 0) {
      thr = 64; need = 0; retry = 1;      // the floor was too high for this row
    } else if (total <= k && floor_bin == 0) {
      thr = -1; need = 0;                 // every candidate qualifies
    } else if ((long long)top >= k) {
      thr = 32; need = k;
    } else {
      const unsigned int ok = __ballot_sync(0xffffffffu, ge >= k);
      thr = 31 - __clz(ok);               // highest bin whose ">=" count reaches k
      const long long ge_thr = __shfl_sync(0xffffffffu, ge, thr);
      const long long mine_thr = __shfl_sync(0xffffffffu, (long long)mine, thr);
      need = k - (ge_thr - mine_thr);     // ties to take at the threshold
    }
    if (lane == 0) {
      thr_sm = thr;
      need_sm = need;
      retry_sm = retry;
      if (retry) floor_sm = 0;
    }
  }
  __syncthreads();
  if (!retry_sm) break;
  }  // attempt
  const int thr = thr_sm;
  const long long need = need_sm;

  // ---- pass 2: emit ----
  long long base = 0;
  for (int64_t w0 = 0; w0 < W; w0 += 1024) {
    const int64_t w = w0 + tid;
    uint32_t gt = 0u, eq = 0u, pw = 0u;
    if (w < W) {
      uint32_t codes[32];
      ht_load_codes(kc, w, S, aligned, codes);
      pw = prev_row[w];
      const int64_t c0 = w * 32;
      uint32_t valid = ~pw;
      if (c0 + 32 > S) valid &= (c0 >= S) ? 0u : ((1u << (S - c0)) - 1u);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int sc = nbits - __popc(codes[i] ^ qc);
        gt |= (sc > thr ? 1u : 0u) << i;
        eq |= (sc == thr ? 1u : 0u) << i;
      }
      gt &= valid;
      eq &= valid;
    }
    long long total_eq;
    const long long before = sah_block_excl_scan<long long>((long long)__popc(eq), scan, &total_eq);
    if (w < W) {
      const long long quota = need - (base + before);
      const int take = quota > 32 ? 32 : (quota < 0 ? 0 : (int)quota);
      out_row[w] = pw | gt | sah_lowest_bits(eq, take);
    }
    base += total_eq;
  }
}

// ---------------------------------------------------------------------------------------
// Warp tiles.  A warp takes 32 consecutive bitmap words (1024 keys, 4 KB of codes) with eight
// coalesced 16-byte loads per lane: lane L, slot j holds keys 128 j + 4 L .. + 3 of the tile,
// which are bits 4 (L % 8) .. + 3 of the tile's word 4 j + L / 8 ("load order").  Bitmap words
// are owned one per lane (lane W owns word W of the tile, "owner order"); eight shuffles move a
// set of per-key flags from load order to owner order.
// ---------------------------------------------------------------------------------------
// Per-lane private counters: cnt[distance][lane] bytes of one warp (33 rows).  No two lanes
// share a counter, so the histogram needs no atomics; a lane may count 255 keys between flushes.
#define HT_CNT_BYTES (33 * 32)

__device__ __forceinline__ void ht_count1(unsigned char* cnt_lane, unsigned int dist, unsigned int inc) {
  unsigned char* c = cnt_lane + dist * 32;
  *c = (unsigned char)(*c + inc);
}

// Hamming distances of a tile's keys to the query code, four per register (d4[8]); the score
// of a key is nbits - distance.  With COUNT the keys whose flag in `vflags` (load order, bit
// 4 j + i) is set are counted into the lane's private counters on the way.
template <bool COUNT>
__device__ __forceinline__ void ht_tile_dist(const uint32_t* __restrict__ kc, int64_t c0, int64_t S,
                                             bool aligned, uint32_t qc, int lane, uint32_t* d4,
                                             unsigned char* cnt_lane = nullptr, uint32_t vflags = 0u,
                                             bool all_valid = false) {
  uint4 v[8];
  if (aligned && c0 + 1024 <= S) {
    const uint4* p = reinterpret_cast<const uint4*>(kc + c0) + lane;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = p[j * 32];
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t c = c0 + 128 * j + 4 * lane;
      v[j].x = (c + 0 < S) ? kc[c + 0] : 0u;
      v[j].y = (c + 1 < S) ? kc[c + 1] : 0u;
      v[j].z = (c + 2 < S) ? kc[c + 2] : 0u;
      v[j].w = (c + 3 < S) ? kc[c + 3] : 0u;
    }
  }
  if (COUNT && all_valid) {   // warp-uniform: no key of the tile is masked out
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned int a = __popc(v[j].x ^ qc), b = __popc(v[j].y ^ qc);
      const unsigned int c = __popc(v[j].z ^ qc), d = __popc(v[j].w ^ qc);
      ht_count1(cnt_lane, a, 1u);
      ht_count1(cnt_lane, b, 1u);
      ht_count1(cnt_lane, c, 1u);
      ht_count1(cnt_lane, d, 1u);
      d4[j] = a | (b << 8) | (c << 16) | (d << 24);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned int a = __popc(v[j].x ^ qc), b = __popc(v[j].y ^ qc);
      const unsigned int c = __popc(v[j].z ^ qc), d = __popc(v[j].w ^ qc);
      if (COUNT) {
        ht_count1(cnt_lane, a, (vflags >> (4 * j + 0)) & 1u);
        ht_count1(cnt_lane, b, (vflags >> (4 * j + 1)) & 1u);
        ht_count1(cnt_lane, c, (vflags >> (4 * j + 2)) & 1u);
        ht_count1(cnt_lane, d, (vflags >> (4 * j + 3)) & 1u);
      }
      d4[j] = a | (b << 8) | (c << 16) | (d << 24);
    }
  }
}

// Loads and counts a tile: `valid` is the owner-order candidate word of this lane.
__device__ __forceinline__ void ht_tile_dist_count(const uint32_t* __restrict__ kc, int64_t c0, int64_t S,
                                                   bool aligned, uint32_t qc, int lane, uint32_t valid,
                                                   unsigned char* cnt_lane, uint32_t* d4);

// Owner-order word -> load order: bit 4 j + i is the flag of this lane's key i of slot j.
__device__ __forceinline__ uint32_t ht_tile_scatter(uint32_t owner_word, int lane) {
  uint32_t out = 0u;
  const int sh = 4 * (lane & 7);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t wv = __shfl_sync(0xffffffffu, owner_word, 4 * j + (lane >> 3));
    out |= ((wv >> sh) & 0xFu) << (4 * j);
  }
  return out;
}

// Load-order flags (bit 4 j + i) -> the owner-order word of this lane.
__device__ __forceinline__ uint32_t ht_tile_gather(uint32_t flags, int lane) {
  uint32_t out = 0u;
  const int src0 = 8 * (lane & 3), sh = 4 * (lane >> 2);
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const uint32_t v = __shfl_sync(0xffffffffu, flags, src0 + p);
    out |= ((v >> sh) & 0xFu) << (4 * p);
  }
  return out;
}

// bit 7 of every byte -> 4 bits
__device__ __forceinline__ unsigned int ht_flags4(unsigned int w) {
  return (((w >> 7) & 0x01010101u) * 0x01020408u) >> 24;
}

// "above" and "equal" flags (load order) of a tile's packed distances against a score threshold
// thr in -1..64: score > thr is distance < nbits - thr.  Distances are 0..32, so plain 32-bit
// adds act on the four bytes at once: byte + (128 - t) stays below bit 7 exactly when
// distance < t, and (byte ^ t) + 127 stays below it exactly when distance == t; no byte carries
// into its neighbour.
__device__ __forceinline__ void ht_tile_compare(const uint32_t* d4, int nbits, int thr, uint32_t* gt,
                                                uint32_t* eq) {
  int t = nbits - thr;                    // -32 .. 33
  if (t < 0) t = 0;                       // nothing is closer than 0
  const unsigned int add_lt = (unsigned int)(128 - t) * 0x01010101u;
  const unsigned int t_eq = ((thr >= 0 && thr <= nbits) ? (unsigned int)(nbits - thr) : 127u) * 0x01010101u;
  uint32_t g = 0u, e = 0u;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    g |= ht_flags4(~(d4[j] + add_lt)) << (4 * j);
    e |= ht_flags4(~((d4[j] ^ t_eq) + 0x7f7f7f7fu)) << (4 * j);
  }
  *gt = g;
  *eq = e;
}

__device__ __forceinline__ void ht_tile_dist_count(const uint32_t* __restrict__ kc, int64_t c0, int64_t S,
                                                   bool aligned, uint32_t qc, int lane, uint32_t valid,
                                                   unsigned char* cnt_lane, uint32_t* d4) {
  const bool all_valid = __all_sync(0xffffffffu, valid == 0xffffffffu);
  const uint32_t vflags = all_valid ? 0xffffffffu : ht_tile_scatter(valid, lane);
  ht_tile_dist<true>(kc, c0, S, aligned, qc, lane, d4, cnt_lane, vflags, all_valid);
}

// Adds a warp's private counters into hist[33] (shared, u32, indexed by score = nbits -
// distance) and clears them.
__device__ __forceinline__ void ht_cnt_flush(unsigned char* cnt_warp, unsigned int* hist, int nbits, int lane) {
  __syncwarp();
  uint32_t* row = reinterpret_cast<uint32_t*>(cnt_warp + lane * 32);   // distance = lane
  unsigned int s = 0u;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int ii = (i + (lane >> 2)) & 7;  // 32 lanes on 32 banks
    s += __vsadu4(row[ii], 0u);
    row[ii] = 0u;
  }
  if (s && lane <= nbits) atomicAdd(&hist[nbits - lane], s);
  if (lane < 8) {
    uint32_t* top = reinterpret_cast<uint32_t*>(cnt_warp + 32 * 32);     // distance 32
    const unsigned int t = __vsadu4(top[lane], 0u);
    top[lane] = 0u;
    if (t && nbits == 32) atomicAdd(&hist[0], t);
  }
  __syncwarp();
}

// Threshold and ties from a histogram hist[33] held in shared memory; called by one full warp.
__device__ __forceinline__ void ht_pick(const unsigned int* hist, long long k, int lane, int* thr_out,
                                        long long* need_out) {
  const unsigned int mine = hist[lane], top = hist[32];
  unsigned int incl = mine;  // suffix sum over lanes: keys with bin >= lane (bins <= 31)
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    unsigned int n = __shfl_down_sync(0xffffffffu, incl, o);
    if (lane + o < 32) incl += n;
  }
  const long long ge = (long long)incl + top;
  const long long total = __shfl_sync(0xffffffffu, (long long)incl, 0) + top;
  int thr;
  long long need;
  if (k <= 0) {
    thr = 64; need = 0;                 // nothing qualifies
  } else if (total <= k) {
    thr = -1; need = 0;                 // every candidate qualifies
  } else if ((long long)top >= k) {
    thr = 32; need = k;
  } else {
    const unsigned int ok = __ballot_sync(0xffffffffu, ge >= k);
    thr = 31 - __clz(ok);               // highest bin whose ">=" count reaches k
    const long long ge_thr = __shfl_sync(0xffffffffu, ge, thr);
    const long long mine_thr = __shfl_sync(0xffffffffu, (long long)mine, thr);
    need = k - (ge_thr - mine_thr);     // ties to take at the threshold
  }
  *thr_out = thr;
  *need_out = need;
}

// The counting select with 512 threads per row and the scores kept in registers between the
// two passes (rows of up to 512 * WPT words): warp v takes tiles v, v + 16, ...; pass 2 neither
// reloads the codes nor recounts bits, byte-wise SIMD compares give the "above" and "equal"
// flags.  Two CTAs fit on an SM, so 256 rows make one balanced wave on 148 SMs.
#define HT2_THREADS 512

template <int WPT>
__global__ void __launch_bounds__(HT2_THREADS, 2)
hash_topk_reg_kernel(const uint32_t* __restrict__ kcodes, int64_t kc_stride,
                     const uint32_t* __restrict__ qcodes, int nbits, int Sq, int64_t S, int64_t W,
                     const uint32_t* __restrict__ prev_bits, int64_t k,
                     uint32_t* __restrict__ out_bits) {
  sah_pdl_entry();
  __shared__ __align__(16) unsigned char cnt[HT2_THREADS / 32][HT_CNT_BYTES];
  __shared__ unsigned int hist[HT_BINS];
  __shared__ int scan[33];
  __shared__ int thr_sm;
  __shared__ long long need_sm;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row = blockIdx.x;
  const uint32_t* kc = kcodes + (row / Sq) * kc_stride;
  const uint32_t qc = qcodes[row];
  const uint32_t* prev_row = prev_bits + row * W;
  uint32_t* out_row = out_bits + row * W;
  const bool aligned = ((reinterpret_cast<uintptr_t>(kc) & 15) == 0);
  for (int i = tid; i < (HT2_THREADS / 32) * HT_CNT_BYTES / 4; i += HT2_THREADS)
    reinterpret_cast<uint32_t*>(&cnt[0][0])[i] = 0u;
  if (tid < HT_BINS) hist[tid] = 0u;
  __syncthreads();

  uint32_t s4[WPT][8];   // packed distances of the tiles this warp owns
  uint32_t validm[WPT], prevw[WPT];
#pragma unroll
  for (int j = 0; j < WPT; ++j) {
    const int64_t w = tid + (int64_t)j * HT2_THREADS;   // the word this lane owns
    const int64_t c0 = (w - lane) * 32;                 // first key of the warp's tile
    uint32_t pw = 0u, valid = 0u;
    if (w < W) {
      pw = prev_row[w];
      valid = ~pw;
      if (w * 32 + 32 > S) valid &= (w * 32 >= S) ? 0u : ((1u << (S - w * 32)) - 1u);
    }
    prevw[j] = pw;
    validm[j] = valid;
    if (c0 < S) {  // warp-uniform
      ht_tile_dist_count(kc, c0, S, aligned, qc, lane, valid, &cnt[warp][lane], s4[j]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) s4[j][i] = 0u;
    }
  }
  ht_cnt_flush(cnt[warp], hist, nbits, lane);
  __syncthreads();
  if (warp == 0) {
    int thr;
    long long need;
    ht_pick(hist, k, lane, &thr, &need);
    if (lane == 0) {
      thr_sm = thr;
      need_sm = need;
    }
  }
  __syncthreads();
  const int thr = thr_sm;
  const int need = (int)need_sm;   // at most 65536 keys in a row here

  int base = 0;
#pragma unroll
  for (int j = 0; j < WPT; ++j) {
    const int64_t w = tid + (int64_t)j * HT2_THREADS;
    uint32_t gl, el;
    ht_tile_compare(s4[j], nbits, thr, &gl, &el);
    const uint32_t gt = ht_tile_gather(gl, lane) & validm[j];
    const uint32_t eq = ht_tile_gather(el, lane) & validm[j];
    int total_eq;
    const int before = sah_block_excl_scan<int>(__popc(eq), scan, &total_eq);
    if (w < W) {
      const int quota = need - (base + before);
      const int take = quota > 32 ? 32 : (quota < 0 ? 0 : quota);
      out_row[w] = prevw[j] | gt | sah_lowest_bits(eq, take);
    }
    base += total_eq;
  }
}

extern "C" int sah_hash_topk(const uint32_t* kcodes, int64_t kc_stride, const uint32_t* qcodes,
                             int nbits,
                             const void* bias, int dtype, int64_t bias_s_b, int64_t bias_s_h,
                             int64_t bias_s_q, int B, int Hq, int Sq, int64_t S, int64_t W,
                             const uint32_t* prev_bits, int64_t k, uint32_t* out_bits,
                             void* stream) {
  SAH_REQUIRE(kcodes && qcodes && prev_bits && out_bits, "hash_topk: null pointer");
  SAH_REQUIRE(nbits > 0 && nbits <= 32, "hash_topk: nbits must be 1..32");
  SAH_REQUIRE(kc_stride >= S, "hash_topk: kc_stride shorter than S");
  SAH_REQUIRE(B > 0 && Hq > 0 && Sq > 0 && S > 0 && W * 32 >= S, "hash_topk: bad extents");
  const int64_t rows = (int64_t)B * Hq * Sq;
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_HASH_TOPK, (cudaStream_t)stream);
  if (bias == nullptr) {
    const int64_t wpt = sah_ceil_div(W, HT2_THREADS);
    if (wpt <= 1)
      sah_launch_chain(hash_topk_reg_kernel<1>, (unsigned)rows, HT2_THREADS, 0, st, kcodes, kc_stride, qcodes, nbits, Sq,
                                                                     S, W, prev_bits, k, out_bits);
    else if (wpt <= 2)
      sah_launch_chain(hash_topk_reg_kernel<2>, (unsigned)rows, HT2_THREADS, 0, st, kcodes, kc_stride, qcodes, nbits, Sq,
                                                                     S, W, prev_bits, k, out_bits);
    else if (wpt <= 4)
      sah_launch_chain(hash_topk_reg_kernel<4>, (unsigned)rows, HT2_THREADS, 0, st, kcodes, kc_stride, qcodes, nbits, Sq,
                                                                     S, W, prev_bits, k, out_bits);
    else
      sah_launch_chain(hash_topk_fast_kernel, (unsigned)rows, 1024, 0, st, kcodes, kc_stride, qcodes, nbits, Sq, S,
                                                            W, prev_bits, k, out_bits);
  } else if (dtype == SAH_BF16) {
    sah_launch_chain(hash_topk_kernel<__nv_bfloat16, 16, true>, (unsigned)rows, SAH_SELECT_THREADS, 0, st,
        kcodes, kc_stride, qcodes, nbits, (const __nv_bfloat16*)bias, bias_s_b, bias_s_h, bias_s_q, Hq, Sq,
        S, W, prev_bits, k, out_bits);
  } else if (dtype == SAH_F32) {
    sah_launch_chain(hash_topk_kernel<float, 32, true>, (unsigned)rows, SAH_SELECT_THREADS, 0, st, kcodes,
        kc_stride, qcodes, nbits, (const float*)bias, bias_s_b, bias_s_h, bias_s_q, Hq, Sq, S, W,
        prev_bits, k, out_bits);
  } else {
    return sah_fail(SAH_ERR_INVALID, "hash_topk: unknown dtype %d", dtype);
  }
  SAH_LAUNCH_CHECK("hash_topk");
  sah_prof_end(SAH_PROF_HASH_TOPK, (cudaStream_t)stream);
  return SAH_OK;
}

// ---------------------------------------------------------------------------------------
// Hamming top-k in pieces: a row's keys are cut into `parts` contiguous column ranges -- the
// `chunks` chunks of each of `world` ranks, rank-major, so part index order is column order.
// Every part is histogrammed by its own CTA (sah_hash_hist), all parts' histograms are put
// side by side (across ranks by the caller's all-gather), every part derives the same
// threshold and its own share of the ties at the threshold -- ties go to the lowest column,
// that is to the lower parts first (sah_hash_shard_plan) -- and emits its range
// (sah_hash_emit).  The union over parts is exactly the selection of hash_topk_fast_kernel.
// With world = 1 this is the single-device path for few, long rows (sah_hash_topk_ws).
// ---------------------------------------------------------------------------------------
#define HP_THREADS 256

// words per chunk: whole warp tiles (32 words), so that chunk borders are tile borders
static inline int64_t hash_chunk_words(int64_t W, int chunks) {
  return sah_ceil_div(sah_ceil_div(W, (int64_t)chunks), (int64_t)32) * 32;
}

// Packed distances of a tile in the scratch that carries them from the histogram pass to the emit
// pass: 64 uint4 per tile, [half][lane], lane L holding slots 4 half .. 4 half + 3.
__device__ __forceinline__ void ht_scores_store(uint4* __restrict__ tile, int lane, const uint32_t* s4) {
  tile[lane] = make_uint4(s4[0], s4[1], s4[2], s4[3]);
  tile[32 + lane] = make_uint4(s4[4], s4[5], s4[6], s4[7]);
}
__device__ __forceinline__ void ht_scores_load(const uint4* __restrict__ tile, int lane, uint32_t* s4) {
  const uint4 a = tile[lane], b = tile[32 + lane];
  s4[0] = a.x; s4[1] = a.y; s4[2] = a.z; s4[3] = a.w;
  s4[4] = b.x; s4[5] = b.y; s4[6] = b.z; s4[7] = b.w;
}

__global__ void __launch_bounds__(HP_THREADS, 4)
hash_hist_kernel(const uint32_t* __restrict__ kcodes, int64_t kc_stride,
                 const uint32_t* __restrict__ qcodes, int nbits, int Sq, int64_t S, int64_t W,
                 int64_t chunk_words, const uint32_t* __restrict__ prev_bits, int64_t rows,
                 int32_t* __restrict__ hist_out, uint4* __restrict__ scores_out) {
  sah_pdl_entry();
  __shared__ __align__(16) unsigned char cnt[HP_THREADS / 32][HT_CNT_BYTES];
  __shared__ unsigned int hist[HT_BINS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row = blockIdx.x, chunk = blockIdx.y;
  const uint32_t* kc = kcodes + (row / Sq) * kc_stride;
  const uint32_t qc = qcodes[row];
  const uint32_t* prev_row = prev_bits + row * W;
  const bool aligned = ((reinterpret_cast<uintptr_t>(kc) & 15) == 0);
  const int64_t row_tiles = (W + 31) >> 5;
  for (int i = tid; i < (HP_THREADS / 32) * HT_CNT_BYTES / 4; i += HP_THREADS)
    reinterpret_cast<uint32_t*>(&cnt[0][0])[i] = 0u;
  if (tid < HT_BINS) hist[tid] = 0u;
  __syncthreads();
  const int64_t w_lo = chunk * chunk_words;   // chunk_words is a multiple of 32: whole tiles
  const int64_t w_hi = w_lo + chunk_words < W ? w_lo + chunk_words : W;
  int pending = 0;
  for (int64_t t0 = w_lo + 32 * warp; t0 < w_hi; t0 += HP_THREADS) {
    if (t0 * 32 >= S) break;
    const int64_t w = t0 + lane;
    uint32_t valid = 0u;
    if (w < w_hi) {
      valid = ~prev_row[w];
      if (w * 32 + 32 > S) valid &= (w * 32 >= S) ? 0u : ((1u << (S - w * 32)) - 1u);
    }
    uint32_t s4[8];
    ht_tile_dist_count(kc, t0 * 32, S, aligned, qc, lane, valid, &cnt[warp][lane], s4);
    if (scores_out != nullptr) ht_scores_store(scores_out + (row * row_tiles + (t0 >> 5)) * 64, lane, s4);
    if (++pending == 7) {  // a lane's byte counters hold 255
      ht_cnt_flush(cnt[warp], hist, nbits, lane);
      pending = 0;
    }
  }
  ht_cnt_flush(cnt[warp], hist, nbits, lane);
  __syncthreads();
  if (tid < 33) hist_out[(chunk * rows + row) * 33 + tid] = (int32_t)hist[tid];
}

extern "C" int sah_hash_hist(const uint32_t* kcodes, int64_t kc_stride, const uint32_t* qcodes,
                             int nbits, int B, int Hq, int Sq, int64_t S, int64_t W, int chunks,
                             const uint32_t* prev_bits, int32_t* hist, void* scores, void* stream) {
  SAH_REQUIRE(kcodes && qcodes && prev_bits && hist, "hash_hist: null pointer");
  SAH_REQUIRE(((uintptr_t)scores & 15) == 0, "hash_hist: scores must be 16-byte aligned");
  SAH_REQUIRE(nbits > 0 && nbits <= 32, "hash_hist: nbits must be 1..32");
  SAH_REQUIRE(kc_stride >= S && B > 0 && Hq > 0 && Sq > 0 && S > 0 && W * 32 >= S, "hash_hist: bad extents");
  SAH_REQUIRE(chunks >= 1 && chunks <= 65535, "hash_hist: 1..65535 chunks");
  const int64_t rows = (int64_t)B * Hq * Sq;
  const int64_t chunk_words = hash_chunk_words(W, chunks);
  dim3 grid((unsigned)rows, (unsigned)chunks);
  sah_launch_chain(hash_hist_kernel, grid, HP_THREADS, 0, (cudaStream_t)stream, kcodes, kc_stride, qcodes, nbits, Sq, S, W,
                                                                chunk_words, prev_bits, rows, hist,
                                                                reinterpret_cast<uint4*>(scores));
  SAH_LAUNCH_CHECK("hash_hist");
  return SAH_OK;
}

// Threshold and tie share of part `me` from the per-bin sums over all parts; one full warp,
// lane L holding bin 31 - L (here / before_me / mine) and every lane the sums of bin 32.  A
// prefix scan over the lanes walks the bins from the top.
__device__ __forceinline__ void hash_plan_scan(long long here, long long before_me, long long mine,
                                               long long here32, long long before32, long long mine32,
                                               long long k, int lane, int* thr_out, long long* need_out) {
  long long incl = here;   // candidates scoring >= this lane's bin, bin 32 aside
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const long long n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  incl += here32;
  int thr = -1;
  long long need = 0;
  if (k <= 0) {
    thr = 64;
  } else if (here32 >= k) {  // the k-th best score is the top bin
    thr = 32;
    const long long left = k - before32;
    need = left <= 0 ? 0 : (left < mine32 ? left : mine32);
  } else {
    const unsigned int ok = __ballot_sync(0xffffffffu, incl >= k);
    if (ok) {
      const int src = __ffs(ok) - 1;            // first lane (highest bin) reaching k
      const long long ties = k - (incl - here); // ties to take over all parts
      const long long left = ties - before_me;  // what lower parts leave for this one
      const long long nd = left <= 0 ? 0 : (left < mine ? left : mine);
      thr = 31 - src;
      need = __shfl_sync(0xffffffffu, nd, src);
    }
  }
  *thr_out = thr;
  *need_out = need;
}

// One warp per (row, chunk of this rank): lane L sums bin 31 - L over all parts, bin 32 is
// summed by all lanes together.
__device__ __forceinline__ void hash_plan_warp(const int32_t* __restrict__ hist_all, int parts, int me,
                                               int64_t rows, int64_t row, long long k, int lane,
                                               int* thr_out, long long* need_out) {
  const int bin = 31 - lane;
  long long here = 0, before_me = 0, mine = 0;
  for (int g = 0; g < parts; ++g) {
    const long long c = hist_all[((int64_t)g * rows + row) * 33 + bin];
    here += c;
    if (g < me) before_me += c;
    if (g == me) mine = c;
  }
  long long here32 = 0, before32 = 0, mine32 = 0;
  for (int g = lane; g < parts; g += 32) {
    const long long c = hist_all[((int64_t)g * rows + row) * 33 + 32];
    here32 += c;
    if (g < me) before32 += c;
    if (g == me) mine32 = c;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    here32 += __shfl_xor_sync(0xffffffffu, here32, o);
    before32 += __shfl_xor_sync(0xffffffffu, before32, o);
    mine32 += __shfl_xor_sync(0xffffffffu, mine32, o);
  }
  hash_plan_scan(here, before_me, mine, here32, before32, mine32, k, lane, thr_out, need_out);
}

// The same by a whole CTA: every thread fetches a few of the parts * 33 counters (all loads in
// flight together), shared-memory sums, then warp 0 scans.  pl: [3][33] (all, before me, mine).
__device__ __forceinline__ void hash_plan_cta(const int32_t* __restrict__ hist_all, int parts, int me,
                                              int64_t rows, int64_t row, long long k,
                                              unsigned long long (*pl)[33], int* thr_sm, long long* need_sm) {
  const int tid = threadIdx.x, lane = tid & 31;
  for (int i = tid; i < 3 * 33; i += blockDim.x) (&pl[0][0])[i] = 0ull;
  __syncthreads();
  for (int idx = tid; idx < parts * 33; idx += blockDim.x) {
    const int g = idx / 33, bin = idx - g * 33;
    const unsigned long long c = (unsigned long long)hist_all[((int64_t)g * rows + row) * 33 + bin];
    if (c) {
      atomicAdd(&pl[0][bin], c);
      if (g < me) atomicAdd(&pl[1][bin], c);
      if (g == me) pl[2][bin] = c;
    }
  }
  __syncthreads();
  if (tid < 32) {
    int thr;
    long long need;
    hash_plan_scan((long long)pl[0][31 - lane], (long long)pl[1][31 - lane], (long long)pl[2][31 - lane],
                   (long long)pl[0][32], (long long)pl[1][32], (long long)pl[2][32], k, lane, &thr, &need);
    if (lane == 0) {
      *thr_sm = thr;
      *need_sm = need;
    }
  }
  __syncthreads();
}

// hist_all [world][chunks][rows][33].  thr: scores above it are taken whole (-1: every
// candidate, 64: none); need: ties at thr this part takes.  Outputs are [chunks][rows].
__global__ void hash_shard_plan_kernel(const int32_t* __restrict__ hist_all, int world, int rank,
                                       int chunks, int64_t rows, int64_t k,
                                       int32_t* __restrict__ thr_out, int64_t* __restrict__ need_out) {
  sah_pdl_entry_early();
  const int lane = threadIdx.x & 31;
  const int64_t t = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= rows * chunks) return;   // warp-uniform
  const int64_t row = t % rows;
  const int chunk = (int)(t / rows);
  int thr;
  long long need;
  hash_plan_warp(hist_all, world * chunks, rank * chunks + chunk, rows, row, k, lane, &thr, &need);
  if (lane == 0) {
    thr_out[t] = thr;
    need_out[t] = need;
  }
}

extern "C" int sah_hash_shard_plan(const int32_t* hist_all, int world, int rank, int chunks,
                                   int64_t rows, int64_t k, int32_t* thr, int64_t* need,
                                   void* stream) {
  SAH_REQUIRE(hist_all && thr && need, "hash_shard_plan: null pointer");
  SAH_REQUIRE(world > 0 && rank >= 0 && rank < world && rows > 0 && chunks >= 1,
              "hash_shard_plan: bad extents");
  sah_launch_chain(hash_shard_plan_kernel, (unsigned)sah_ceil_div(rows * chunks, 4), 128, 0,
      (cudaStream_t)stream, hist_all, world, rank, chunks, rows, k, thr, need);
  SAH_LAUNCH_CHECK("hash_shard_plan");
  return SAH_OK;
}

// thr_in/need_in: the plan of sah_hash_shard_plan; when they are null the CTA derives its own
// entry from hist_all (the single-device path, one launch less).  scores_in: the packed scores
// left by the histogram pass, or null to recompute them from the codes.  A warp takes HE_TILES
// consecutive tiles at a time, so the ordered count of ties needs one CTA barrier per
// 8 * HE_TILES tiles.
#define HE_TILES 4

__global__ void __launch_bounds__(HP_THREADS, 4)
hash_emit_kernel(const uint32_t* __restrict__ kcodes, int64_t kc_stride,
                 const uint32_t* __restrict__ qcodes, int nbits, int Sq, int64_t S, int64_t W,
                 int64_t chunk_words, const uint32_t* __restrict__ prev_bits, int64_t rows,
                 const int32_t* __restrict__ thr_in, const int64_t* __restrict__ need_in,
                 const int32_t* __restrict__ hist_all, int chunks, int64_t k,
                 const uint4* __restrict__ scores_in, uint32_t* __restrict__ out_bits) {
  sah_pdl_entry();
  __shared__ int wsum[2][HP_THREADS / 32];
  __shared__ unsigned long long pl[3][33];
  __shared__ int thr_sm;
  __shared__ long long need_sm;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row = blockIdx.x, chunk = blockIdx.y;
  const uint32_t* kc = kcodes + (row / Sq) * kc_stride;
  const uint32_t qc = qcodes[row];
  const uint32_t* prev_row = prev_bits + row * W;
  uint32_t* out_row = out_bits + row * W;
  const bool aligned = ((reinterpret_cast<uintptr_t>(kc) & 15) == 0);
  const int64_t row_tiles = (W + 31) >> 5;
  if (thr_in != nullptr) {
    if (tid == 0) {
      thr_sm = thr_in[chunk * rows + row];
      need_sm = need_in[chunk * rows + row];
    }
    __syncthreads();
  } else {
    hash_plan_cta(hist_all, chunks, (int)chunk, rows, row, k, pl, &thr_sm, &need_sm);
  }
  const int thr = thr_sm;
  const long long need = need_sm;
  const int64_t w_lo = chunk * chunk_words;
  const int64_t w_hi = w_lo + chunk_words < W ? w_lo + chunk_words : W;
  long long base = 0;
  int it = 0;
  for (int64_t sb = w_lo; sb < w_hi; sb += HP_THREADS * HE_TILES, ++it) {
    uint32_t gt[HE_TILES], eq[HE_TILES], pw[HE_TILES];
    int excl[HE_TILES];
    int run = 0;   // ties in this warp's earlier tiles of the block
#pragma unroll
    for (int t = 0; t < HE_TILES; ++t) {
      const int64_t t0 = sb + (int64_t)(warp * HE_TILES + t) * 32;   // first word of the tile
      const int64_t w = t0 + lane;
      gt[t] = 0u; eq[t] = 0u; pw[t] = 0u;
      if (t0 < w_hi) {   // warp-uniform
        uint32_t valid = 0u;
        if (w < w_hi) {
          pw[t] = prev_row[w];
          valid = ~pw[t];
          if (w * 32 + 32 > S) valid &= (w * 32 >= S) ? 0u : ((1u << (S - w * 32)) - 1u);
        }
        if (t0 * 32 < S) {
          uint32_t s4[8], gl, el;
          if (scores_in != nullptr) ht_scores_load(scores_in + (row * row_tiles + (t0 >> 5)) * 64, lane, s4);
          else ht_tile_dist<false>(kc, t0 * 32, S, aligned, qc, lane, s4);
          ht_tile_compare(s4, nbits, thr, &gl, &el);
          gt[t] = ht_tile_gather(gl, lane) & valid;
          eq[t] = ht_tile_gather(el, lane) & valid;
        }
      }
      const int c = __popc(eq[t]);
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      excl[t] = run + incl - c;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) wsum[it & 1][warp] = run;
    __syncthreads();
    int before_warps = 0, total = 0;
#pragma unroll
    for (int v = 0; v < HP_THREADS / 32; ++v) {
      const int x = wsum[it & 1][v];
      total += x;
      if (v < warp) before_warps += x;
    }
#pragma unroll
    for (int t = 0; t < HE_TILES; ++t) {
      const int64_t w = sb + (int64_t)(warp * HE_TILES + t) * 32 + lane;
      if (w < w_hi) {
        const long long quota = need - (base + before_warps + excl[t]);
        const int take = quota > 32 ? 32 : (quota < 0 ? 0 : (int)quota);
        out_row[w] = pw[t] | gt[t] | sah_lowest_bits(eq[t], take);
      }
    }
    base += total;
  }
}

extern "C" int sah_hash_emit(const uint32_t* kcodes, int64_t kc_stride, const uint32_t* qcodes,
                             int nbits, int B, int Hq, int Sq, int64_t S, int64_t W, int chunks,
                             const uint32_t* prev_bits, const int32_t* thr, const int64_t* need,
                             const void* scores, uint32_t* out_bits, void* stream) {
  SAH_REQUIRE(kcodes && qcodes && prev_bits && thr && need && out_bits, "hash_emit: null pointer");
  SAH_REQUIRE(((uintptr_t)scores & 15) == 0, "hash_emit: scores must be 16-byte aligned");
  SAH_REQUIRE(nbits > 0 && nbits <= 32, "hash_emit: nbits must be 1..32");
  SAH_REQUIRE(kc_stride >= S && B > 0 && Hq > 0 && Sq > 0 && S > 0 && W * 32 >= S, "hash_emit: bad extents");
  SAH_REQUIRE(chunks >= 1 && chunks <= 65535, "hash_emit: 1..65535 chunks");
  const int64_t rows = (int64_t)B * Hq * Sq;
  const int64_t chunk_words = hash_chunk_words(W, chunks);
  dim3 grid((unsigned)rows, (unsigned)chunks);
  sah_launch_chain(hash_emit_kernel, grid, HP_THREADS, 0, (cudaStream_t)stream, kcodes, kc_stride, qcodes, nbits, Sq, S, W,
                                                                chunk_words, prev_bits, rows, thr, need,
                                                                nullptr, chunks, 0,
                                                                reinterpret_cast<const uint4*>(scores), out_bits);
  SAH_LAUNCH_CHECK("hash_emit");
  return SAH_OK;
}

// The single-device use of the three kernels above: rows cut into chunks so that the grid
// fills the GPU whatever the row count.
static int hash_ws_chunks(int64_t rows, int64_t W, int sm_count) {
  if (sm_count <= 0) sm_count = 148;
  int64_t chunks = sah_ceil_div((int64_t)sm_count * 8, rows);
  const int64_t max_chunks = sah_ceil_div(W, HP_THREADS);  // at least one word per thread
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  if (chunks > 1024) chunks = 1024;
  return (int)chunks;
}

extern "C" int64_t sah_hash_scores_bytes(int64_t rows, int64_t W) {
  if (rows <= 0 || W <= 0) return 0;
  return rows * ((W + 31) / 32) * 1024;   // one byte per key, whole 1024-key tiles
}

static int64_t hash_ws_hist_bytes(int64_t rows, int64_t chunks) {
  return (rows * chunks * 33 * 4 + 15) / 16 * 16;
}

extern "C" int64_t sah_hash_topk_ws_bytes(int64_t rows, int64_t W, int sm_count) {
  if (rows <= 0 || W <= 0) return 0;
  const int64_t chunks = hash_ws_chunks(rows, W, sm_count);
  return hash_ws_hist_bytes(rows, chunks) + sah_hash_scores_bytes(rows, W);
}

extern "C" int sah_hash_topk_ws(const uint32_t* kcodes, int64_t kc_stride, const uint32_t* qcodes,
                                int nbits, int B, int Hq, int Sq, int64_t S, int64_t W,
                                const uint32_t* prev_bits, int64_t k, uint32_t* out_bits,
                                void* workspace, int64_t workspace_bytes, int sm_count, void* stream) {
  SAH_REQUIRE(workspace != nullptr && ((uintptr_t)workspace & 15) == 0,
              "hash_topk_ws: workspace must be a 16-byte aligned device pointer");
  SAH_REQUIRE(kcodes && qcodes && prev_bits && out_bits, "hash_topk_ws: null pointer");
  const int64_t rows = (int64_t)B * Hq * Sq;
  SAH_REQUIRE(rows > 0 && rows <= 2147483647, "hash_topk_ws: bad row count");
  if (workspace_bytes < sah_hash_topk_ws_bytes(rows, W, sm_count))
    return sah_fail(SAH_ERR_WORKSPACE, "hash_topk_ws: workspace of %lld bytes, need %lld",
                    (long long)workspace_bytes, (long long)sah_hash_topk_ws_bytes(rows, W, sm_count));
  const int chunks = hash_ws_chunks(rows, W, sm_count);
  unsigned char* p = reinterpret_cast<unsigned char*>(workspace);
  int32_t* hist = reinterpret_cast<int32_t*>(p);
  void* scores = p + hash_ws_hist_bytes(rows, chunks);
  sah_prof_begin(SAH_PROF_HASH_TOPK, (cudaStream_t)stream);
  int rc = sah_hash_hist(kcodes, kc_stride, qcodes, nbits, B, Hq, Sq, S, W, chunks, prev_bits, hist, scores,
                         stream);
  if (rc != SAH_OK) return rc;
  {
    // every emit CTA derives its threshold and tie share from the chunk histograms itself
    dim3 grid((unsigned)rows, (unsigned)chunks);
    sah_launch_chain(hash_emit_kernel, grid, HP_THREADS, 0, (cudaStream_t)stream, kcodes, kc_stride, qcodes,
        nbits, Sq, S, W, hash_chunk_words(W, chunks), prev_bits, rows, nullptr,
        nullptr, hist, chunks, k, reinterpret_cast<const uint4*>(scores), out_bits);
    SAH_LAUNCH_CHECK("hash_topk_ws emit");
  }
  sah_prof_end(SAH_PROF_HASH_TOPK, (cudaStream_t)stream);
  return SAH_OK;
}

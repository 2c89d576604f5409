// HashAttention key signatures on the fifth-generation tensor cores (bfloat16; layer widths
// multiples of 16 up to 128; at most three layers): the per-head MLP of
// hashattention_top_k.py:203-253 with every layer's product as tcgen05.mma and every output
// whose rounding the tensor core's summation order could change redone in the fixed order of
// hash_encode_kernel.
//
// One CTA of 128 threads serves one (batch, output head) and a slice of the keys, 128 keys per
// tile, one thread per key.  Per CTA, once: each layer's weight matrix, transposed to
// [outputs][inputs], in the 128-byte swizzled K-major layout of the shared-memory matrix
// descriptors; the Euclidean norm of every weight column; the biases.  Per tile and layer:
//   D[128 keys][dout] = A[128 keys][din] . W   (din / 16 tcgen05.mma, accumulator in tensor memory)
//   thread-per-key epilogue: v = bf16(bf16(acc) + bias), activation through the bfloat16 table
//   (or the sign, for the last layer), written back as the next layer's A row.
// The fixed-order kernel rounds acc to bfloat16, so the only way the summation order can show is
// an acc within E of a bfloat16 rounding midpoint, E = 2^-15 |a| |w_column| >= the sum of both
// orders' error bounds (128 * 2^-24 * sum|a_d w_d| each, sum|a_d w_d| <= |a||w|).  Those outputs
// are recomputed by the key's thread from the A row and the weight column in shared memory,
// channels ascending, one fused multiply-add per channel, exactly as hash_encode_kernel does.
// The bits are therefore the same whichever kernel built them.
// If the (bounded) wait for a product runs out, the tile's outputs are all computed that way.
//
// Measured: not a gain.  With |acc| ~ |a||w| / sqrt(128) the band E is about a third of the
// bfloat16 spacing at acc, so 31 % of the outputs (all three layers, Gaussian keys with outlier
// channels) are redone and a warp of 32 keys redoes practically every output; the kernel is
// 2.6x to 4.6x slower than hash_encode_kernel.  sah_hash_encode therefore takes it only on
// request (SAH_HASH_TC=1); it stays as the checked record of why the hash index is built in
// the fixed order on the CUDA cores.
#pragma once
#include "sah_tcgen05.cuh"

#define HTC_TILE 128
#define HTC_THREADS 128
#define HTC_MAX_LAYERS 3

struct HashTcArgs {
  const __nv_bfloat16* x;
  int64_t xs_b, xs_h, xs_n;
  int H_in, H_out;
  int64_t n_begin, n_end, n_total;
  int n_layers;
  int dims[HTC_MAX_LAYERS + 1];
  const __nv_bfloat16* weights[HTC_MAX_LAYERS];
  const __nv_bfloat16* bias[HTC_MAX_LAYERS];
  const uint16_t* act_table;
  uint32_t* codes;
  int b_off[HTC_MAX_LAYERS];   // byte offsets of the layers' B tiles behind the A tile
  int wn_off, bias_off, misc_off;  // float arrays [layer][128], then barrier + words
};

__device__ __forceinline__ void htc_tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// 16-byte chunk c (8 channels) of row r of a K-major tile whose 64-channel atoms are
// `atom_bytes` apart: atom c / 8, slot (c % 8) ^ (r % 8)
__device__ __forceinline__ int htc_chunk_off(int r, int c, int atom_bytes) {
  return (c >> 3) * atom_bytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}

// acc of output o of this thread's key in the fixed order: channels ascending, one fma each
__device__ __forceinline__ float htc_exact(const unsigned char* a_tile, int row, const unsigned char* b_tile,
                                           int o, int din, int dout) {
  float acc = 0.f;
  for (int c = 0; c < din / 8; ++c) {
    float a8[8], w8[8];
    sah_unpack8(*reinterpret_cast<const uint4*>(a_tile + htc_chunk_off(row, c, HTC_TILE * 128)), a8);
    sah_unpack8(*reinterpret_cast<const uint4*>(b_tile + htc_chunk_off(o, c, dout * 128)), w8);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc = fmaf(a8[e], w8[e], acc);
  }
  return acc;
}

__global__ void __launch_bounds__(HTC_THREADS)
hash_encode_tc_kernel(HashTcArgs p) {
  extern __shared__ __align__(1024) unsigned char htc_raw[];
  const uint32_t raw_s = (uint32_t)__cvta_generic_to_shared(htc_raw);
  unsigned char* sm = htc_raw + (((raw_s + 1023u) & ~1023u) - raw_s);
  const uint32_t sm_s = (uint32_t)__cvta_generic_to_shared(sm);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.y, b = blockIdx.z;
  const int h_in = h / (p.H_out / p.H_in);
  unsigned char* a_tile = sm;  // two atoms of [128 keys][128 B]
  float* wn_sm = reinterpret_cast<float*>(sm + p.wn_off);      // [layer][128] column norms
  float* bias_sm = reinterpret_cast<float*>(sm + p.bias_off);  // [layer][128]
  const uint32_t bar = sm_s + p.misc_off;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + p.misc_off + 8);
  volatile int* abort_sm = reinterpret_cast<volatile int*>(sm + p.misc_off + 12);
  int* err_sm = reinterpret_cast<int*>(sm + p.misc_off + 16);  // stands in for a global error word

  if (tid == 0) {
    atm_mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    *abort_sm = 0;
    *err_sm = 0;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::
                     "r"((uint32_t)__cvta_generic_to_shared(tmem_slot)),
                 "r"(128));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
  }
  // ---- the head's weights: B_l[o][d] = W_l[d][o], column norms, biases ----
  for (int l = 0; l < p.n_layers; ++l) {
    const int din = p.dims[l], dout = p.dims[l + 1];
    const __nv_bfloat16* wl = p.weights[l] + (int64_t)h * din * dout;
    unsigned char* bt = sm + p.b_off[l];
    for (int i = tid; i < dout * (din / 8); i += HTC_THREADS) {
      const int o = i % dout, c = i / dout;
      __align__(16) __nv_bfloat16 v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = wl[(int64_t)(c * 8 + e) * dout + o];
      *reinterpret_cast<uint4*>(bt + htc_chunk_off(o, c, dout * 128)) = *reinterpret_cast<const uint4*>(v);
    }
    for (int o = tid; o < dout; o += HTC_THREADS) {
      float ss = 0.f;
      for (int d = 0; d < din; ++d) {
        const float w = __bfloat162float(wl[(int64_t)d * dout + o]);
        ss = fmaf(w, w, ss);
      }
      wn_sm[l * 128 + o] = sqrtf(ss);
      bias_sm[l * 128 + o] = __bfloat162float(p.bias[l][(int64_t)h * dout + o]);
    }
  }
  // the unused part of the A rows (inputs narrower than 64 channels per atom) stays zero
  for (int i = tid; i < 2 * HTC_TILE * 8; i += HTC_THREADS)
    *reinterpret_cast<uint4*>(a_tile + i * 16) = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  aum_fence_before();
  __syncthreads();
  aum_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;

  const int64_t n_tiles = (p.n_end - p.n_begin + HTC_TILE - 1) / HTC_TILE;
  const int64_t per = (n_tiles + gridDim.x - 1) / gridDim.x;
  const int64_t t0 = (int64_t)blockIdx.x * per;
  const int64_t t1 = t0 + per < n_tiles ? t0 + per : n_tiles;
  const __nv_bfloat16* xb = p.x + b * p.xs_b + h_in * p.xs_h;
  uint32_t phase = 0;
  bool mma_ok = true;  // uniform over the CTA
  for (int64_t t = t0; t < t1; ++t) {
    const int64_t n0 = p.n_begin + t * HTC_TILE;
    // ---- stage the keys of the tile: coalesced 16-byte chunks into the swizzled rows ----
    {
      const int d0 = p.dims[0], chunks = d0 / 8;
      for (int i = tid; i < HTC_TILE * chunks; i += HTC_THREADS) {
        const int r = i / chunks, c = i - r * chunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (n0 + r < p.n_end) v = *reinterpret_cast<const uint4*>(xb + (n0 + r) * p.xs_n + c * 8);
        *reinterpret_cast<uint4*>(a_tile + htc_chunk_off(r, c, HTC_TILE * 128)) = v;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    aum_fence_before();
    __syncthreads();
    // |a|^2 of this thread's key
    float an2 = 0.f;
    for (int c = 0; c < p.dims[0] / 8; ++c) {
      float a8[8];
      sah_unpack8(*reinterpret_cast<const uint4*>(a_tile + htc_chunk_off(tid, c, HTC_TILE * 128)), a8);
#pragma unroll
      for (int e = 0; e < 8; ++e) an2 = fmaf(a8[e], a8[e], an2);
    }
    uint32_t code = 0u;
    for (int l = 0; l < p.n_layers; ++l) {
      const int din = p.dims[l], dout = p.dims[l + 1];
      const bool last = (l == p.n_layers - 1);
      const unsigned char* bt = sm + p.b_off[l];
      if (tid == 0 && mma_ok) {
        aum_fence_after();
        const uint32_t idesc = aum_idesc(false, false, (uint32_t)dout);
        for (int ks = 0; ks < din / 16; ++ks) {
          const uint64_t ad = aum_desc(sm_s + (ks >> 2) * (HTC_TILE * 128) + (ks & 3) * 32, 0, 1024, 2);
          const uint64_t bd = aum_desc(sm_s + p.b_off[l] + (ks >> 2) * (dout * 128) + (ks & 3) * 32, 0, 1024, 2);
          aum_mma(tmem, ad, bd, idesc, ks > 0 ? 1u : 0u);
        }
        aum_commit(bar);
      }
      if (mma_ok) {
        const bool okw = aum_wait_warp(bar, phase, abort_sm, err_sm);
        phase ^= 1u;
        mma_ok = __syncthreads_and(okw ? 1 : 0) != 0;
      }
      if (mma_ok) aum_fence_after();
      const float an = sqrtf(an2) * 3.0517578125e-05f * 1.001f;  // 2^-15 |a|
      uint32_t outp[64];  // this key's outputs of the layer, two bfloat16 per word
      float next2 = 0.f;
#pragma unroll
      for (int g32 = 0; g32 < 4; ++g32) {
        if (g32 * 32 >= dout) {  // narrower layer: the remaining words of the row are zero
#pragma unroll
          for (int i = 0; i < 16; ++i) outp[g32 * 16 + i] = 0u;
          continue;
        }
        uint32_t accb[32];
        if (mma_ok) htc_tmem_ld32(tmem + lane_base + g32 * 32, accb);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int o = g32 * 32 + i;
          float v = 0.f;
          if (o < dout) {
            float acc;
            bool redo = !mma_ok;
            if (!redo) {
              acc = __uint_as_float(accb[i]);
              const uint32_t bits = accb[i];
              const float ulp = __uint_as_float(bits & 0x7F800000u) * 1.1920928955078125e-07f;  // 2^-23 * 2^e
              const float dist = fabsf((float)(int)(bits & 0xFFFFu) - 32768.f) * ulp;  // to the rounding midpoint
              redo = !(dist > an * wn_sm[l * 128 + o]);
            }
            if (redo) acc = htc_exact(a_tile, tid, bt, o, din, dout);
            v = sah_round_to<__nv_bfloat16>(acc);
            v = sah_round_to<__nv_bfloat16>(__fadd_rn(v, bias_sm[l * 128 + o]));
            if (!last) {
              v = he_activate<__nv_bfloat16>(v, 0, p.act_table);
              next2 = fmaf(v, v, next2);
            } else {
              code |= (v > 0.f ? 1u : 0u) << o;
            }
          }
          // pack (constant indices after unrolling)
          if ((i & 1) == 0) outp[g32 * 16 + (i >> 1)] = __float_as_uint(v) >> 16;
          else outp[g32 * 16 + (i >> 1)] |= __float_as_uint(v) & 0xFFFF0000u;
        }
      }
      aum_fence_before();
      __syncthreads();  // every thread has read its inputs and the accumulator
      if (!last) {
#pragma unroll
        for (int c = 0; c < 16; ++c)
          if (c < dout / 8)
            *reinterpret_cast<uint4*>(a_tile + htc_chunk_off(tid, c, HTC_TILE * 128)) =
                make_uint4(outp[c * 4], outp[c * 4 + 1], outp[c * 4 + 2], outp[c * 4 + 3]);
        an2 = next2;
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        aum_fence_before();
        __syncthreads();
      }
    }
    if (n0 + tid < p.n_end)
      p.codes[((int64_t)b * p.H_out + h) * p.n_total + n0 + tid] = code;
  }
  aum_fence_before();
  __syncthreads();
  if (warp == 0) {
    aum_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(128));
  }
}

// SimHash key signatures on the fifth-generation tensor cores (bfloat16, head dim 128, 8 bits
// per table): the projection of the transformed keys onto the L * 8 hyperplanes
// (magic_pig.py:120-150, :332-372) as a tcgen05 GEMM, with every sign that the tensor core's
// summation order could have changed redone in the fixed order of lsh_key_sign_kernel.
//
//   A  = transformed keys, 128 per tile, [128][144] bf16 (129 channels, zero padded), built by
//        the producer warps from K, the key mean, the key norms and the maximum norm exactly as
//        the fixed-order kernel builds them (every operation rounded to bfloat16), stored
//        K-major in the 128-byte swizzled layout;
//   B  = a chunk of 256 hyperplanes, [256][144] bf16, K-major, same layout, resident in shared
//        memory for the life of the CTA (gridDim.y chunks cover the L * 8 columns);
//   D  = A . B^T, [128 keys][256 columns] fp32 in tensor memory, two accumulators so that the
//        epilogue of a tile overlaps the products of the next.
//
// The products are exact in float32 (bf16 x bf16); only the order of the 129 additions differs
// from the fixed-order kernel.  Both sums are within 129 * 2^-24 * sum|x_c p_c| of the exact
// value (the tensor core at least as close), and sum|x_c p_c| <= |x| |p| with |x| <= 1.01 for a
// transformed key, so a projection whose magnitude exceeds tau = 2^-15 * |p| has the same sign in
// both.  The epilogue (one thread per key) packs the sign bits of 32 columns at a time into
// the key's signature row and appends the groups that hold a projection within tau to a list;
// lsh_sign_recheck_kernel recomputes exactly those in the fixed order and corrects the bits.
// A list that overflows sets a flag, and the caller redoes the range with the fixed-order kernel.
//
// Every mbarrier wait is bounded (sah_tcgen05.cuh); a wait that runs out sets the error word,
// all roles leave their loops, tensor memory is freed.
#pragma once
#include "sah_tcgen05.cuh"

#define LTC_TILE 128
#define LTC_NCHUNK 256   // hyperplanes per CTA
#define LTC_KSTEPS 9     // 144 = 9 x 16 channels (129 used)
#define LTC_THREADS 288  // 4 epilogue warps, 4 producer warps, 1 issuing warp
#define LTC_TAU_SCALE 3.0517578125e-05f  // 2^-15

struct LtcCfg {
  static constexpr int A_ATOM = LTC_TILE * 128;    // [128 rows][128 B]: 64 channels
  static constexpr int A_TILE = 3 * A_ATOM;        // channels 0-63, 64-127, 128-191 (128-143 read)
  static constexpr int B_ATOM = LTC_NCHUNK * 128;  // [256 rows][128 B]
  static constexpr int B_OFF = 0;
  static constexpr int A_OFF = 3 * B_ATOM;         // two A tiles
  static constexpr int TAU_OFF = A_OFF + 2 * A_TILE;          // [256] floats
  static constexpr int BAR_OFF = TAU_OFF + LTC_NCHUNK * 4;    // a_full[2] a_empty[2] d_full[2] d_free[2]
  static constexpr int MISC_OFF = BAR_OFF + 64;               // tmem slot, abort word
  static constexpr int SMEM = 1024 + MISC_OFF + 16;
};

struct LtcUncertain {
  long long key;      // row of the signature array (bh * cap + s)
  int col0;           // first of the 32 columns of the group
  unsigned int mask;  // columns of the group whose projection was within tau
};

__device__ __forceinline__ void ltc_tmem_ld32(uint32_t taddr, uint32_t* r) {
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

// Grid: (workers, column chunks).  Worker w of a chunk takes the tiles w, w + workers, ... of the
// flattened (batch x KV head, key tile) space.
__global__ void __launch_bounds__(LTC_THREADS, 1)
lsh_key_sign_tc_kernel(const __nv_bfloat16* __restrict__ k, int64_t ks_b, int64_t ks_h, int64_t ks_s, int Hkv,
                       int64_t BH, int64_t s0, int64_t s1, const __nv_bfloat16* __restrict__ mean,
                       const float* __restrict__ norms, const unsigned int* __restrict__ max_bits,
                       const __nv_bfloat16* __restrict__ proj, int L, int64_t cap, uint8_t* __restrict__ codes,
                       LtcUncertain* __restrict__ list, int list_cap, int* __restrict__ list_count,
                       int* __restrict__ errflag) {
  constexpr int D = 128;
  using C = LtcCfg;
  extern __shared__ __align__(1024) unsigned char ltc_raw[];
  const uint32_t raw_s = (uint32_t)__cvta_generic_to_shared(ltc_raw);
  unsigned char* sm = ltc_raw + (((raw_s + 1023u) & ~1023u) - raw_s);
  const uint32_t sm_s = (uint32_t)__cvta_generic_to_shared(sm);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nbits = L * 8;
  const int LP = lsh_row_pitch<uint8_t>(L);
  const int col_base = blockIdx.y * LTC_NCHUNK;
  int ncols = nbits - col_base;               // real columns of this chunk
  if (ncols > LTC_NCHUNK) ncols = LTC_NCHUNK;
  const uint32_t n_mma = (uint32_t)((ncols + 15) / 16 * 16);
  const int64_t tiles_per_bh = (s1 - s0 + LTC_TILE - 1) / LTC_TILE;
  const int64_t total_tiles = BH * tiles_per_bh;
  const int64_t first = blockIdx.x, stride = gridDim.x;
  const int my_tiles = first < total_tiles ? (int)((total_tiles - first + stride - 1) / stride) : 0;

  const uint32_t bar0 = sm_s + C::BAR_OFF;
  const uint32_t a_full = bar0, a_empty = bar0 + 16, d_full = bar0 + 32, d_free = bar0 + 48;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + C::MISC_OFF);
  volatile int* abort_sm = reinterpret_cast<volatile int*>(sm + C::MISC_OFF + 4);
  float* tau_sm = reinterpret_cast<float*>(sm + C::TAU_OFF);

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      atm_mbar_init(a_full + i * 8, 4);   // one arrival per producer warp
      atm_mbar_init(a_empty + i * 8, 1);  // tcgen05.commit
      atm_mbar_init(d_full + i * 8, 1);   // tcgen05.commit
      atm_mbar_init(d_free + i * 8, 4);   // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    *abort_sm = 0;
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::
                     "r"((uint32_t)__cvta_generic_to_shared(tmem_slot)),
                 "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
  }
  // ---- B chunk: row n = hyperplane col_base + n, 144 channels (zero beyond 128 and beyond the
  //      real columns); 16-byte chunk c of row n sits in atom c / 8 at slot (c % 8) ^ (n % 8) ----
  for (int i = tid; i < LTC_NCHUNK * 24; i += LTC_THREADS) {
    const int n = i / 24, c = i - n * 24;  // 24 chunks of 8 channels = 192 channels
    __align__(16) __nv_bfloat16 v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int ch = c * 8 + e;
      v[e] = (n < ncols && ch <= D) ? proj[(int64_t)ch * nbits + col_base + n] : __float2bfloat16(0.f);
    }
    *reinterpret_cast<uint4*>(sm + C::B_OFF + (c >> 3) * C::B_ATOM + n * 128 + (((c & 7) ^ (n & 7)) << 4)) =
        *reinterpret_cast<const uint4*>(v);
  }
  // tau of every column: 2^-15 * 1.01 * |p|
  for (int n = tid; n < LTC_NCHUNK; n += LTC_THREADS) {
    float ss = 0.f;
    if (n < ncols)
      for (int ch = 0; ch <= D; ++ch) {
        const float p = __bfloat162float(proj[(int64_t)ch * nbits + col_base + n]);
        ss = fmaf(p, p, ss);
      }
    tau_sm[n] = LTC_TAU_SCALE * 1.01f * sqrtf(ss) * 1.0001f;
  }
  // the padding channels of the third atom of both A tiles stay zero for the whole kernel
  for (int i = tid; i < 2 * LTC_TILE * 8; i += LTC_THREADS) {
    const int buf = i / (LTC_TILE * 8), r = (i / 8) % LTC_TILE, c = i % 8;
    *reinterpret_cast<uint4*>(sm + C::A_OFF + buf * C::A_TILE + 2 * C::A_ATOM + r * 128 + (c << 4)) =
        make_uint4(0u, 0u, 0u, 0u);
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  aum_fence_before();
  __syncthreads();
  aum_fence_after();
  const uint32_t tmem = *tmem_slot;
  const float M = __uint_as_float(*max_bits);

  if (warp >= 4 && warp < 8) {
    // =========================== producers: transformed keys ===========================
    // 16 lanes cover one key row (8 channels each), two rows per pass, 32 rows per warp.
    const int pw = warp - 4;
    const int my_chunk = lane & 15, my_sub = lane >> 4;
    int64_t bh_cur = -1;
    float m8[8];
    for (int t = 0; t < my_tiles; ++t) {
      const int buf = t & 1;
      const int64_t flat = first + (int64_t)t * stride;
      const int64_t bh = flat / tiles_per_bh;
      const int64_t key0 = s0 + (flat - bh * tiles_per_bh) * LTC_TILE;
      if (bh != bh_cur) {
        bh_cur = bh;
        if (mean != nullptr) sah_unpack8(*reinterpret_cast<const uint4*>(mean + bh * D + my_chunk * 8), m8);
      }
      if (t >= 2 && !aum_wait_warp(a_empty + buf * 8, (uint32_t)(((t >> 1) - 1) & 1), abort_sm, errflag)) break;
      const __nv_bfloat16* kb = k + (bh / Hkv) * ks_b + (bh % Hkv) * ks_h;
      unsigned char* at = sm + C::A_OFF + buf * C::A_TILE;
#pragma unroll 4
      for (int it = 0; it < 16; ++it) {
        const int r = pw * 32 + it * 2 + my_sub;
        const int64_t s = key0 + r;
        float x[8];
        __align__(16) __nv_bfloat16 v[8];
        if (s < s1) {
          sah_unpack8(*reinterpret_cast<const uint4*>(kb + s * ks_s + my_chunk * 8), x);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float c = mean != nullptr ? sah_round_to<__nv_bfloat16>(__fsub_rn(x[e], m8[e])) : x[e];
            v[e] = __float2bfloat16_rn(__fdiv_rn(c, M));
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __float2bfloat16(0.f);
        }
        *reinterpret_cast<uint4*>(at + (my_chunk >> 3) * C::A_ATOM + r * 128 + (((my_chunk & 7) ^ (r & 7)) << 4)) =
            *reinterpret_cast<const uint4*>(v);
        if (my_chunk == 0) {  // channel 128: the augmentation column (chunk 0 of the third atom)
          const float aug = s < s1 ? lsh_augment<__nv_bfloat16>(norms[bh * cap + s], M) : 0.f;
          *reinterpret_cast<__nv_bfloat16*>(at + 2 * C::A_ATOM + r * 128 + ((r & 7) << 4)) = __float2bfloat16_rn(aug);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) aum_arrive(a_full + buf * 8);
    }
  } else if (warp == 8) {
    // =========================== tensor-core issuer ===========================
    if (lane == 0) {
      const uint32_t idesc = aum_idesc(false, false, n_mma);
      for (int t = 0; t < my_tiles; ++t) {
        const int buf = t & 1;
        if (!aum_wait(a_full + buf * 8, (uint32_t)((t >> 1) & 1), abort_sm, errflag)) break;
        if (t >= 2 && !aum_wait(d_free + buf * 8, (uint32_t)(((t >> 1) - 1) & 1), abort_sm, errflag)) break;
        aum_fence_after();
        const uint32_t a_s = sm_s + C::A_OFF + buf * C::A_TILE, b_s = sm_s + C::B_OFF;
#pragma unroll
        for (int ks = 0; ks < LTC_KSTEPS; ++ks) {
          const uint64_t ad = aum_desc(a_s + (ks >> 2) * C::A_ATOM + (ks & 3) * 32, 0, 1024, 2);
          const uint64_t bd = aum_desc(b_s + (ks >> 2) * C::B_ATOM + (ks & 3) * 32, 0, 1024, 2);
          aum_mma(tmem + buf * LTC_NCHUNK, ad, bd, idesc, ks > 0 ? 1u : 0u);
        }
        aum_commit(d_full + buf * 8);
        aum_commit(a_empty + buf * 8);
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue: one thread per key ===========================
    const int keyl = tid;  // 0..127
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    const int groups = (ncols + 31) / 32;
    for (int t = 0; t < my_tiles; ++t) {
      const int buf = t & 1;
      const int64_t flat = first + (int64_t)t * stride;
      const int64_t bh = flat / tiles_per_bh;
      const int64_t s = s0 + (flat - bh * tiles_per_bh) * LTC_TILE + keyl;
      if (!aum_wait_warp(d_full + buf * 8, (uint32_t)((t >> 1) & 1), abort_sm, errflag)) break;
      aum_fence_after();
      const int64_t row = bh * cap + s;
      for (int gq = 0; gq < groups; ++gq) {
        uint32_t acc[32];
        ltc_tmem_ld32(tmem + lane_base + buf * LTC_NCHUNK + gq * 32, acc);
        uint32_t bits = 0u, unsure = 0u;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float vv = __uint_as_float(acc[i]);
          bits |= (vv > 0.f ? 1u : 0u) << i;
          unsure |= (fabsf(vv) <= tau_sm[gq * 32 + i] ? 1u : 0u) << i;
        }
        const int c0 = col_base + gq * 32;
        const int valid = nbits - c0;  // real columns in this group
        if (valid < 32) {
          const uint32_t vm = valid <= 0 ? 0u : ((1u << valid) - 1u);
          bits &= vm;
          unsure &= vm;
        }
        if (s < s1) {
          // bit j of table l is column 8 l + j: the 32 columns of the group are 4 code bytes in order
          const int byte0 = c0 >> 3;
          if (byte0 + 4 <= LP) {
            *reinterpret_cast<uint32_t*>(codes + row * LP + byte0) = bits;
          } else {
            for (int bq = 0; bq < 4 && byte0 + bq < LP; ++bq) codes[row * LP + byte0 + bq] = (uint8_t)(bits >> (8 * bq));
          }
          if (unsure) {
            const int slot = atomicAdd(list_count, 1);
            if (slot < list_cap) {
              LtcUncertain u;
              u.key = row; u.col0 = c0; u.mask = unsure;
              list[slot] = u;
            }
          }
        }
      }
      // the row's padding bytes beyond the last table (the last chunk owns them)
      if (blockIdx.y == gridDim.y - 1 && s < s1)
        for (int bq = (col_base >> 3) + groups * 4; bq < LP; bq += 4)
          *reinterpret_cast<uint32_t*>(codes + row * LP + bq) = 0u;
      aum_fence_before();
      __syncwarp();
      if (lane == 0) aum_arrive(d_free + buf * 8);
    }
  }
  aum_fence_before();
  __syncthreads();
  if (warp == 8) {
    aum_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512));
  }
}

// One warp per list entry; lane j redoes the j-th flagged column of the group in the fixed
// order of lsh_key_sign_kernel (single float32 accumulator, channels ascending) and sets or
// clears the bit.  The bits of one signature word may be corrected by several lanes: atomics.
__global__ void __launch_bounds__(256)
lsh_sign_recheck_kernel(const __nv_bfloat16* __restrict__ k, int64_t ks_b, int64_t ks_h, int64_t ks_s, int Hkv,
                        const __nv_bfloat16* __restrict__ mean, const float* __restrict__ norms,
                        const unsigned int* __restrict__ max_bits, const __nv_bfloat16* __restrict__ proj, int L,
                        int64_t cap, uint8_t* __restrict__ codes, const LtcUncertain* __restrict__ list,
                        int list_cap, const int* __restrict__ list_count) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  int n = *list_count;
  if (n > list_cap) n = list_cap;
  const int nbits = L * 8;
  const int LP = lsh_row_pitch<uint8_t>(L);
  const float M = __uint_as_float(*max_bits);
  for (int64_t e = wid; e < n; e += nwarps) {
    const LtcUncertain u = list[e];
    const int64_t bh = u.key / cap, s = u.key - bh * cap;
    // lane j takes the j-th set bit of the mask
    unsigned int mk = u.mask;
    int mybit = -1;
    for (int j = 0; j <= lane && mk; ++j) {
      const int bpos = __ffs(mk) - 1;
      mk &= mk - 1;
      if (j == lane) mybit = bpos;
    }
    if (mybit < 0) continue;
    const int col = u.col0 + mybit;
    const __nv_bfloat16* kr = k + (bh / Hkv) * ks_b + (bh % Hkv) * ks_h + s * ks_s;
    float acc = 0.f;
    for (int c = 0; c < D; ++c) {
      const float x = __bfloat162float(kr[c]);
      const float cx = mean != nullptr ? sah_round_to<__nv_bfloat16>(__fsub_rn(x, __bfloat162float(mean[bh * D + c]))) : x;
      const float v = sah_round_to<__nv_bfloat16>(__fdiv_rn(cx, M));
      acc = __fadd_rn(acc, __fmul_rn(v, __bfloat162float(proj[(int64_t)c * nbits + col])));
    }
    const float aug = lsh_augment<__nv_bfloat16>(norms[u.key], M);
    acc = __fadd_rn(acc, __fmul_rn(aug, __bfloat162float(proj[(int64_t)D * nbits + col])));
    // the code byte of column col is byte col / 8 of the row; its 32-bit word is aligned (rows
    // are multiples of 16 bytes)
    const int64_t byte = u.key * LP + (col >> 3);
    unsigned int* word = reinterpret_cast<unsigned int*>(codes + (byte & ~3ll));
    const unsigned int bit = 1u << (((int)(byte & 3) << 3) + (col & 7));
    if (acc > 0.f) atomicOr(word, bit);
    else atomicAnd(word, ~bit);
  }
}

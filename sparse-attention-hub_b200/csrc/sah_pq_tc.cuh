// k-means assignment of PQCache on the fifth-generation tensor cores (bfloat16 keys, sub-vectors
// of 8 channels, 16..256 centroids): the distance contraction of kmeans_batched
// (utils/pq_utils.py:220-257) as a tcgen05 product, with the argmin decided by the fixed-order
// distance of pq_assign_kernel among the centroids that the product cannot tell apart.
//
//   Per (batch, KV head, sub-vector) group and tile of 128 keys:
//     A = [128 keys][16]: the key's 8 channels twice;  B = [n_cent][16]: each float32 centroid
//     split into two bfloat16 numbers, high parts in columns 0-7, low parts in 8-15, so that one
//     tcgen05.mma (K = 16) gives x . c_hi + x . c_lo = x . c up to 2^-17 |x||c|.
//     score_c = |c|^2 - 2 x . c  (= distance - |x|^2), one thread per key reads its 256 scores
//     from tensor memory twice: first the minimum, then every centroid within 2 E of it is
//     measured with the fixed-order float32 distance (dimensions ascending, (x - c)^2 rounded,
//     then added) and the first minimum of those wins, as torch.argmin does.
//   E = 2^-12 (|x|^2 + max_c |c|^2) bounds |score_c - (fixed-order distance - |x|^2)| with a wide
//   margin (the split loses 2^-17 |x||c|, the float32 sums ~2^-21 of the magnitudes), so the
//   fixed-order argmin is always among the candidates: the codes equal pq_assign_kernel's bit
//   for bit, and with them every later centre.
//
// One CTA of 128 threads per (group, slice of the keys); a CTA holds 256 columns of tensor
// memory, so two CTAs share an SM and overlap each other's phases.  The only mbarrier wait
// (tcgen05.commit) is bounded; when it runs out the error word is set and the CTA stops.
#pragma once
#include "sah_tcgen05.cuh"

#define PTC_TILE 128
#define PTC_THREADS 128

struct PtcCfg {
  static constexpr int A_OFF = 0;                       // [128 rows][128 B], first 32 B of a row used
  static constexpr int B_OFF = PTC_TILE * 128;          // [256 rows][128 B]
  static constexpr int CENT_OFF = B_OFF + 256 * 128;    // float32 [256][8]
  static constexpr int CN_OFF = CENT_OFF + 256 * 8 * 4; // float32 [256] |c|^2
  static constexpr int MISC_OFF = CN_OFF + 256 * 4;     // mbarrier, tmem slot, abort word, scratch
  // padded so that two CTAs, not three, share an SM: each holds half of the tensor memory
  static constexpr int SMEM = 100 * 1024;
  static_assert(1024 + MISC_OFF + 64 <= SMEM, "layout exceeds the request");
};

__device__ __forceinline__ void ptc_tmem_ld32(uint32_t taddr, uint32_t* r) {
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

__global__ void __launch_bounds__(PTC_THREADS, 2)
pq_assign_tc_kernel(const __nv_bfloat16* __restrict__ x, int64_t xs_b, int64_t xs_h, int64_t xs_s, int Hkv,
                    int64_t key_begin, int64_t key_end, int64_t init_offset, int n_sub, int n_cent,
                    const float* __restrict__ centroids, uint8_t* __restrict__ codes, int64_t cap,
                    int* __restrict__ errflag) {
  constexpr int SD = 8;
  using C = PtcCfg;
  extern __shared__ __align__(1024) unsigned char ptc_raw[];
  const uint32_t raw_s = (uint32_t)__cvta_generic_to_shared(ptc_raw);
  unsigned char* sm = ptc_raw + (((raw_s + 1023u) & ~1023u) - raw_s);
  const uint32_t sm_s = (uint32_t)__cvta_generic_to_shared(sm);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t grp = blockIdx.y;
  const int sub = (int)(grp % n_sub);
  const int64_t bk = grp / n_sub;
  const int kvh = (int)(bk % Hkv);
  const int64_t b = bk / Hkv;
  float* cent_sm = reinterpret_cast<float*>(sm + C::CENT_OFF);
  float* cn_sm = reinterpret_cast<float*>(sm + C::CN_OFF);
  const uint32_t bar = sm_s + C::MISC_OFF;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + C::MISC_OFF + 8);
  volatile int* abort_sm = reinterpret_cast<volatile int*>(sm + C::MISC_OFF + 12);
  float* red_sm = reinterpret_cast<float*>(sm + C::MISC_OFF + 16);  // [4]

  if (tid == 0) {
    atm_mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    *abort_sm = 0;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::
                     "r"((uint32_t)__cvta_generic_to_shared(tmem_slot)),
                 "r"(256));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
  }
  // ---- the group's centroids: float32 copy, |c|^2 in the fixed order, and the B tile
  //      (row c: high parts in chunk 0, low parts in chunk 1; chunk j of row c at slot j ^ (c % 8)) ----
  float cmax = 0.f;
  for (int c = tid; c < 256; c += PTC_THREADS) {
    __align__(16) __nv_bfloat16 hi[8], lo[8];
    float n2 = 0.f;
#pragma unroll
    for (int d = 0; d < SD; ++d) {
      const float v = c < n_cent ? centroids[(grp * n_cent + c) * SD + d] : 0.f;
      cent_sm[c * SD + d] = v;
      n2 = __fadd_rn(n2, __fmul_rn(v, v));
      hi[d] = __float2bfloat16_rn(v);
      lo[d] = __float2bfloat16_rn(__fsub_rn(v, __bfloat162float(hi[d])));
    }
    cn_sm[c] = n2;
    cmax = fmaxf(cmax, n2);
    unsigned char* row = sm + C::B_OFF + c * 128;
    *reinterpret_cast<uint4*>(row + ((0 ^ (c & 7)) << 4)) = *reinterpret_cast<const uint4*>(hi);
    *reinterpret_cast<uint4*>(row + ((1 ^ (c & 7)) << 4)) = *reinterpret_cast<const uint4*>(lo);
  }
#pragma unroll
  for (int of = 16; of > 0; of >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, of));
  if (lane == 0) red_sm[warp] = cmax;
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  aum_fence_before();
  __syncthreads();
  aum_fence_after();
  cmax = fmaxf(fmaxf(red_sm[0], red_sm[1]), fmaxf(red_sm[2], red_sm[3]));
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
  const uint32_t idesc = aum_idesc(false, false, (uint32_t)n_cent);
  const int groups32 = n_cent / 32 + ((n_cent % 32) ? 1 : 0);

  // this CTA's slice of the key range, in whole tiles
  const int64_t n_tiles = (key_end - key_begin + PTC_TILE - 1) / PTC_TILE;
  const int64_t per = (n_tiles + gridDim.x - 1) / gridDim.x;
  const int64_t t0 = (int64_t)blockIdx.x * per;
  const int64_t t1 = t0 + per < n_tiles ? t0 + per : n_tiles;
  const __nv_bfloat16* xb = x + b * xs_b + kvh * xs_h + sub * SD;
  uint32_t phase = 0;
  bool ok = true;
  for (int64_t t = t0; t < t1 && ok; ++t) {
    const int64_t j = key_begin + t * PTC_TILE + tid;
    float xv[SD];
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (j < key_end) raw = *reinterpret_cast<const uint4*>(xb + j * xs_s);
    sah_unpack8(raw, xv);
    {
      unsigned char* row = sm + C::A_OFF + tid * 128;
      *reinterpret_cast<uint4*>(row + ((0 ^ (tid & 7)) << 4)) = raw;
      *reinterpret_cast<uint4*>(row + ((1 ^ (tid & 7)) << 4)) = raw;
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    aum_fence_before();
    __syncthreads();
    if (tid == 0) {
      aum_fence_after();
      const uint64_t ad = aum_desc(sm_s + C::A_OFF, 0, 1024, 2);
      const uint64_t bd = aum_desc(sm_s + C::B_OFF, 0, 1024, 2);
      aum_mma(tmem, ad, bd, idesc, 0u);
      aum_commit(bar);
    }
    ok = aum_wait_warp(bar, phase, abort_sm, errflag);
    phase ^= 1u;
    if (ok) {
      aum_fence_after();
      float x2 = 0.f;
#pragma unroll
      for (int d = 0; d < SD; ++d) x2 = fmaf(xv[d], xv[d], x2);
      const float twoE = 2.f * 0.000244140625f * (x2 + cmax);  // 2 * 2^-12 * (|x|^2 + max |c|^2)
      float smin = INFINITY;
      for (int gq = 0; gq < groups32; ++gq) {
        uint32_t acc[32];
        ptc_tmem_ld32(tmem + lane_base + gq * 32, acc);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int c = gq * 32 + i;
          if (c < n_cent) smin = fminf(smin, fmaf(-2.f, __uint_as_float(acc[i]), cn_sm[c]));
        }
      }
      float best = INFINITY;
      int arg = 0;
      for (int gq = 0; gq < groups32; ++gq) {
        uint32_t acc[32];
        ptc_tmem_ld32(tmem + lane_base + gq * 32, acc);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int c = gq * 32 + i;
          if (c < n_cent && fmaf(-2.f, __uint_as_float(acc[i]), cn_sm[c]) <= smin + twoE) {
            const float dist = pq_dist(xv, cent_sm + c * SD, SD);
            if (dist < best) { best = dist; arg = c; }  // ascending c: the first minimum wins
          }
        }
      }
      if (j < key_end) codes[(bk * cap + (j - init_offset)) * n_sub + sub] = (uint8_t)arg;
    }
    aum_fence_before();
    // every thread is done with the accumulator and the A tile; all warps agree on going on
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
  }
  aum_fence_before();
  __syncthreads();
  if (warp == 0) {
    aum_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(256));
  }
}

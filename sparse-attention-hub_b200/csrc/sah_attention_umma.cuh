// bf16 gather attention on the fifth-generation tensor cores (tcgen05), head dim 128.
//
// Long union lists are bound by the K/V row gather; the mma.sync kernel spends ~48 warp
// instructions per key on fragment loads, address arithmetic and the softmax in the mma
// fragment layout, and its warps stall on each other's issue slots.  Here the keys are the
// M dimension of the tensor-core tile, so one thread owns one key:
//
//   tile = 128 union entries.  A producer warp gathers their K rows and V rows with tensor-map
//   gathers (cp.async.bulk.tensor.2d ... tile::gather4, four indexed rows per instruction, no
//   multicast qualifier) into a three-stage ring in the 128-byte swizzled layout.
//     S^T[128 keys x 16]  = Ktile[128 x 128] . Qtile[16 x 128]^T    8 tcgen05.mma (K = 16 each),
//                           accumulator in tensor memory, double buffered
//     thread-per-key softmax: each of 128 threads reads its key's row of S^T from tensor memory
//                           (mask rows in columns), applies scaling, bias, weights and the
//                           running maximum, and writes the key's row of P (bf16) to shared memory
//     O^T[128 dims x 16] += Vtile^T[128 dims x 128 keys] . P[128 keys x 16]   8 tcgen05.mma,
//                           accumulator in tensor memory for the whole list
//   One elected thread issues all tcgen05.mma; completion is tracked with tcgen05.commit on
//   mbarriers.  The running maximum is lazy: the accumulator is rescaled (tensor memory load,
//   multiply, store) only when a row's maximum grew by more than AUM_RESCALE_T, so that P stays
//   below e^AUM_RESCALE_T; the final normalisation uses the same maximum, so the result is the
//   softmax whatever the history of rescales.
//
// With LSHW the columns 4..7 of the Q tile hold the centred unit queries and the MagicPig weight
// of a (row, key) pair is evaluated by the key's thread exactly as in the mma.sync kernel.
//
// Every wait on an mbarrier is bounded (about a second) and watches a CTA-wide abort word; a
// wait that runs out sets the abort word and the caller's error word, every role leaves its
// loop, the producer gives its copies in flight a bounded chance to land, tensor memory is
// freed, and the CTA still takes its ticket so that no other CTA waits for it.
#pragma once

#define AUM_TILE 128
#define AUM_STAGES 3
#define AUM_THREADS 192
#define AUM_TMEM_COLS 64
#define AUM_RESCALE_T 8.0f
#define AUM_MIN_TILES 2        // tiles a CTA should have before a further CTA joins the group
#define AUM_ONE_WAVE_TILES 16  // below this many tiles per CTA, one wave of CTAs instead of two

struct AumCfg {
  static constexpr int KV_TILE = AUM_TILE * 256;  // one K (or V) tile: two halves of [128 rows][128 B]
  static constexpr int HALF_BYTES = AUM_TILE * 128;
  static constexpr int K_RING = 0;
  static constexpr int V_RING = AUM_STAGES * KV_TILE;
  static constexpr int Q_OFF = 2 * AUM_STAGES * KV_TILE;  // two halves of [16 rows][128 B]
  static constexpr int P_OFF = Q_OFF + 4096;              // two buffers of [128 keys][32 B]
  static constexpr int BAR_OFF = P_OFF + 2 * 4096;
  // barriers: full_k[3] full_v[3] empty_k[3] empty_v[3] s_full[2] s_free[2] p_full[2] p_free[2] max[2]
  static constexpr int N_BARS = 4 * AUM_STAGES + 10;
  static constexpr int MISC_OFF = BAR_OFF + ((N_BARS * 8 + 15) & ~15);
  // misc: tmem slot, abort word, last flag, pad; then wmax [2][4][16], lred [4][16], qmu [16],
  // bias offsets [16] (int64)
  static constexpr int WMAX_OFF = MISC_OFF + 16;
  static constexpr int LRED_OFF = WMAX_OFF + 2 * 4 * 16 * 4;
  static constexpr int QMU_OFF = LRED_OFF + 4 * 16 * 4;
  static constexpr int BOFF_OFF = QMU_OFF + 16 * 4;
  static constexpr int END = BOFF_OFF + 16 * 8;
  static constexpr int SMEM = 1024 + END;
};

__device__ __forceinline__ int aum_active_splits(int total_tiles, int nsplit) {
  int active = nsplit;
  if (nsplit >= 2 && total_tiles < nsplit * AUM_ONE_WAVE_TILES) active = (nsplit + 1) / 2;
  const int by_length = (total_tiles + AUM_MIN_TILES - 1) / AUM_MIN_TILES;
  if (by_length < active) active = by_length;
  return active < 1 ? 1 : active;
}

// Shared-memory matrix descriptor of tcgen05.mma: start address, leading-dimension and stride
// byte offsets (all in units of 16 bytes), the descriptor version of this architecture, and
// the swizzle mode (0 none, 2 128-byte).
__device__ __forceinline__ uint64_t aum_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout & 7u) << 61;
  return d;
}
// Instruction descriptor, kind::f16: fp32 accumulator, bf16 operands, M = 128, N = 16;
// bit 15 / 16: A / B are MN-major (0 = K-major).
__device__ __forceinline__ uint32_t aum_idesc(bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((16u >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void aum_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when all tcgen05.mma issued so far by this thread are complete.
__device__ __forceinline__ void aum_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void aum_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void aum_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void aum_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}
// 8 or 16 consecutive columns of this thread's lane of tensor memory
__device__ __forceinline__ void aum_tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void aum_tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void aum_tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::
          "r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// P tile (B operand of O^T += V^T . P): [128 keys][16 mask rows] bf16, MN-major (the 16 rows of
// a key are contiguous: 32 bytes), 32-byte swizzle: 16-byte chunk j of key k sits at slot
// j ^ ((k >> 2) & 1); 8 keys form a 256-byte atom, a k-step of 16 keys is 512 bytes.
#define AUM_P_MN_MAJOR 1
__device__ __forceinline__ uint64_t aum_p_desc(uint32_t p_s, int ks) {
  return aum_desc(p_s + ks * 512, 0, 256, 6);
}
__device__ __forceinline__ void aum_store_p(unsigned char* base, int key, const uint32_t* pk) {
  const int sw = (key >> 2) & 1;
  *reinterpret_cast<uint4*>(base + key * 32 + (sw << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  *reinterpret_cast<uint4*>(base + key * 32 + ((sw ^ 1) << 4)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
}

// Bounded wait that also gives up when another role of the CTA has given up.  The phase test
// carries no suspend-time hint: most waits of this kernel are entered before the phase
// completes and are satisfied a few hundred cycles later, and a hinted test was seen to keep
// the thread asleep for a good part of the hint.  The bound is wall time (about a second),
// looked at every 256 tests.
__device__ __forceinline__ bool aum_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0u;
}
__device__ __forceinline__ uint64_t aum_now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool aum_wait(uint32_t bar, uint32_t parity, volatile int* abort_sm,
                                         int* __restrict__ errflag) {
  if (aum_try(bar, parity)) return true;
  const uint64_t t0 = aum_now_ns();
  for (int round = 0; round < (1 << 24); ++round) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (aum_try(bar, parity)) return true;
    if (*abort_sm) return false;
    if (aum_now_ns() - t0 > 1000000000ull) break;
  }
  *abort_sm = 1;
  atomicExch(errflag, 1);
  return false;
}

// The same for a whole warp: every lane waits, and the warp continues only if all lanes saw the
// phase complete, so that no lane leaves a loop that the others stay in.
__device__ __forceinline__ bool aum_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_sm,
                                              int* __restrict__ errflag) {
  const bool ok = aum_wait(bar, parity, abort_sm, errflag);
  return __all_sync(0xffffffffu, ok);
}

// float -> int whose signed order is the float order (no NaNs here), for redux.sync
__device__ __forceinline__ int aum_ordered(float f) {
  const int i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float aum_unordered(int i) {
  return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff);
}

#ifdef AUM_PROF
// Development aid (not compiled into the library): cycles that the roles of CTA (0, 0) spend
// in each wait, accumulated in a device array.
__device__ long long aum_prof[32];
#define AUM_T0() const long long prof_t0_ = clock64()
#define AUM_T1(slot) do { if (blockIdx.x == 0 && blockIdx.y == 0) atomicAdd((unsigned long long*)&aum_prof[slot], (unsigned long long)(clock64() - prof_t0_)); } while (0)
#else
#define AUM_T0() do {} while (0)
#define AUM_T1(slot) do {} while (0)
#endif

// RMAX: mask rows a thread handles (4 or 16); LSHW needs RMAX == 4.
template <bool LSHW, int RMAX>
__global__ void __launch_bounds__(AUM_THREADS, 1)
masked_attention_umma_kernel(AttnArgs a, const __grid_constant__ AtmMaps maps, int* __restrict__ tickets,
                             int* __restrict__ errflag, const float* __restrict__ sinks,
                             __nv_bfloat16* __restrict__ out, float* __restrict__ part_out) {
  static_assert(!LSHW || RMAX == 4, "in-place MagicPig weights: at most 4 mask rows");
  constexpr int D = 128;
  constexpr int NST = AUM_STAGES;
  using C = AumCfg;
  extern __shared__ __align__(1024) unsigned char aum_raw[];
  const uint32_t raw_s = (uint32_t)__cvta_generic_to_shared(aum_raw);
  unsigned char* sm = aum_raw + (((raw_s + 1023u) & ~1023u) - raw_s);
  const uint32_t sm_s = (uint32_t)__cvta_generic_to_shared(sm);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  const int split = blockIdx.x;
  const int64_t g = blockIdx.y;
  const int qb = (int)(g % a.nqb);
  const int64_t bk = g / a.nqb;
  const int kvh = (int)(bk % a.Hkv);
  const int64_t b = bk / a.Hkv;
  const int32_t* gcols = a.ucols + g * a.S;
  const uint16_t* gmemb = a.umemb + g * a.S;
  const float* guw = (!LSHW && a.uw) ? a.uw + g * a.S * a.R : nullptr;
  const float* ginv = LSHW ? a.uw + g * a.S : nullptr;

  const int U = a.ucount[g];
  const int total_tiles = (U + AUM_TILE - 1) / AUM_TILE;
  const int active = aum_active_splits(total_tiles, (int)gridDim.x);
  if (split >= active) return;  // before any barrier or tensor memory exists
  const int my_tiles = (total_tiles > split) ? (total_tiles - split + active - 1) / active : 0;

  // barrier addresses
  const uint32_t bar0 = sm_s + C::BAR_OFF;
  const uint32_t full_k = bar0, full_v = bar0 + NST * 8, empty_k = bar0 + 2 * NST * 8,
                 empty_v = bar0 + 3 * NST * 8, s_full = bar0 + 4 * NST * 8, s_free = s_full + 16,
                 p_full = s_full + 32, p_free = s_full + 48, max_bar = s_full + 64;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + C::MISC_OFF);
  volatile int* abort_sm = reinterpret_cast<volatile int*>(sm + C::MISC_OFF + 4);
  int* is_last_sm = reinterpret_cast<int*>(sm + C::MISC_OFF + 8);
  float* wmax_sm = reinterpret_cast<float*>(sm + C::WMAX_OFF);
  float* lred_sm = reinterpret_cast<float*>(sm + C::LRED_OFF);
  float* qmu_sm = reinterpret_cast<float*>(sm + C::QMU_OFF);
  int64_t* boff_sm = reinterpret_cast<int64_t*>(sm + C::BOFF_OFF);

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 4 * NST; ++i) atm_mbar_init(bar0 + i * 8, 1);
    atm_mbar_init(s_full, 1);        atm_mbar_init(s_full + 8, 1);
    atm_mbar_init(s_free, 128);      atm_mbar_init(s_free + 8, 128);
    atm_mbar_init(p_full, 128);      atm_mbar_init(p_full + 8, 128);
    atm_mbar_init(p_free, 1);        atm_mbar_init(p_free + 8, 1);
    atm_mbar_init(max_bar, 4);       atm_mbar_init(max_bar + 8, 4);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    *abort_sm = 0;
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::
                     "r"((uint32_t)__cvta_generic_to_shared(tmem_slot)),
                 "r"(AUM_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
  }
  // ---- Q tile: rows = mask rows (LSHW: rows 4..7 = centred unit queries), zero padded to 16;
  //      two halves of [16 rows][128 B], 16-byte chunk c of a row at slot (c % 8) ^ (row % 8) ----
  for (int idx = tid; idx < 16 * 16; idx += AUM_THREADS) {
    const int r = idx >> 4, c = idx & 15;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    const int rq = (LSHW && r >= 4) ? r - 4 : r;
    if (rq < a.R && (LSHW ? r < 8 : true)) {
      const int gi = rq / a.q_block, qo = rq - gi * a.q_block;
      const int qi = qb * a.q_block + qo;
      if (qi < a.Sq) {
        const int h = kvh * a.G + gi;
        if (LSHW && r >= 4)
          val = *reinterpret_cast<const uint4*>(a.qhat + ((b * a.Hq + h) * a.Sq + qi) * D + c * 8);
        else
          val = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.q) + b * a.qs_b +
                                                (int64_t)h * a.qs_h + qi * a.qs_q + c * 8);
      }
    }
    *reinterpret_cast<uint4*>(sm + C::Q_OFF + (c >> 3) * 2048 + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = val;
  }
  if (tid < 16) {
    const int r = tid;
    float mu = 0.f;
    int64_t bo = -1;
    if (r < a.R) {
      const int gi = r / a.q_block, qo = r - gi * a.q_block;
      const int qi = qb * a.q_block + qo;
      if (qi < a.Sq) {
        const int h = kvh * a.G + gi;
        if (LSHW) mu = a.qmu[(b * a.Hq + h) * a.Sq + qi];
        if (a.bias != nullptr) bo = b * a.bias_s_b + (int64_t)h * a.bias_s_h + (int64_t)qi * a.bias_s_q;
      }
    }
    qmu_sm[r] = mu;
    boff_sm[r] = bo;
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic writes -> tensor-core reads
  aum_fence_before();
  __syncthreads();
  aum_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_o = tmem + 32;  // columns 0..15 and 16..31: the two S buffers

  if (warp == 4) {
    // =========================== producer ===========================
    const int krow0 = (int)(b * a.k_rows_b + kvh * a.k_rows_h);
    const int vrow0 = (int)(b * a.v_rows_b + kvh * a.v_rows_h);
    int issued = 0;
    // the rows of a tile are read one tile ahead, so that the list read does not sit between
    // two issues
    auto load_rows = [&](int t, int* yk, int* yv) {
      const int u0 = (split + t * active) * AUM_TILE + 4 * lane;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = (t < my_tiles && u0 + i < U) ? gcols[u0 + i] : -1;
        yk[i] = col >= 0 ? krow0 + col : a.k_rows_total;  // outside the tensor: reads as zeros
        yv[i] = col >= 0 ? vrow0 + col : a.v_rows_total;
      }
    };
    int nk[4], nv[4];
    load_rows(0, nk, nv);
    for (int t = 0; t < my_tiles; ++t) {
      const int st = t % NST;
      int yk[4], yv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { yk[i] = nk[i]; yv[i] = nv[i]; }
      load_rows(t + 1, nk, nv);
      {
        AUM_T0();
        const bool okk = !(t >= NST) || aum_wait_warp(empty_k + st * 8, (uint32_t)(((t / NST) - 1) & 1), abort_sm, errflag);
        if (lane == 0) AUM_T1(0);
        if (!okk) break;
      }
      if (lane == 0) atm_mbar_expect_tx(full_k + st * 8, (uint32_t)C::KV_TILE);
      __syncwarp();
      const uint32_t kd = sm_s + C::K_RING + st * C::KV_TILE + lane * 512;
      atm_tma_gather4(kd, &maps.k, 0, yk[0], yk[1], yk[2], yk[3], full_k + st * 8);
      atm_tma_gather4(kd + C::HALF_BYTES, &maps.k, 64, yk[0], yk[1], yk[2], yk[3], full_k + st * 8);
      {
        AUM_T0();
        const bool okv = !(t >= NST) || aum_wait_warp(empty_v + st * 8, (uint32_t)(((t / NST) - 1) & 1), abort_sm, errflag);
        if (lane == 0) AUM_T1(1);
        if (!okv) {
          issued = t + 1;  // the K half of this tile is in flight
          break;
        }
      }
      if (lane == 0) atm_mbar_expect_tx(full_v + st * 8, (uint32_t)C::KV_TILE);
      __syncwarp();
      const uint32_t vd = sm_s + C::V_RING + st * C::KV_TILE + lane * 512;
      atm_tma_gather4(vd, &maps.v, 0, yv[0], yv[1], yv[2], yv[3], full_v + st * 8);
      atm_tma_gather4(vd + C::HALF_BYTES, &maps.v, 64, yv[0], yv[1], yv[2], yv[3], full_v + st * 8);
      issued = t + 1;
    }
    if (*abort_sm) {
      // copies of the last NST tiles may still be in flight: bounded wait for each
      for (int t = issued > NST ? issued - NST : 0; t < issued; ++t) {
        const uint32_t par = (uint32_t)((t / NST) & 1);
        for (int i = 0; i < 4096 && !atm_mbar_try(full_k + (t % NST) * 8, par, 2000u); ++i) {}
        for (int i = 0; i < 4096 && !atm_mbar_try(full_v + (t % NST) * 8, par, 2000u); ++i) {}
      }
    }
  } else if (warp == 5) {
    // =========================== tensor-core issuer ===========================
    if (lane == 0) {
      const uint32_t idesc_qk = aum_idesc(false, false);
      const uint32_t idesc_pv = aum_idesc(true, AUM_P_MN_MAJOR != 0);
      const uint32_t q_s = sm_s + C::Q_OFF;
      bool ok = true;
      auto pv = [&](int t) {
        const int st = t % NST, bb = t & 1;
        {
          AUM_T0();
          const bool o1 = aum_wait(full_v + st * 8, (uint32_t)((t / NST) & 1), abort_sm, errflag);
          AUM_T1(4);
          if (!o1) return false;
        }
        {
          AUM_T0();
          const bool o2 = aum_wait(p_full + bb * 8, (uint32_t)((t >> 1) & 1), abort_sm, errflag);
          AUM_T1(5);
          if (!o2) return false;
        }
        aum_fence_after();
        const uint32_t v_s = sm_s + C::V_RING + st * C::KV_TILE;
        const uint32_t p_s = sm_s + C::P_OFF + bb * 4096;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // A = V^T, MN-major: 64 dims contiguous per 128-byte row, 8 keys per 1 KB atom,
          // the second 64 dims one half further
          const uint64_t ad = aum_desc(v_s + ks * 2048, C::HALF_BYTES, 1024, 2);
          const uint64_t bd = aum_p_desc(p_s, ks);
          aum_mma(tmem_o, ad, bd, idesc_pv, (t > 0 || ks > 0) ? 1u : 0u);
        }
        aum_commit(empty_v + st * 8);
        aum_commit(p_free + bb * 8);
        return true;
      };
      for (int t = 0; t < my_tiles && ok; ++t) {
        const int st = t % NST, bb = t & 1;
        {
          AUM_T0();
          ok = aum_wait(full_k + st * 8, (uint32_t)((t / NST) & 1), abort_sm, errflag);
          AUM_T1(6);
        }
        {
          AUM_T0();
          if (ok && t >= 2) ok = aum_wait(s_free + bb * 8, (uint32_t)(((t >> 1) - 1) & 1), abort_sm, errflag);
          AUM_T1(7);
        }
        if (!ok) break;
        aum_fence_after();
        const uint32_t k_s = sm_s + C::K_RING + st * C::KV_TILE;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // both K-major, 128-byte swizzle: 8-row groups 1 KB apart, 32 bytes per k-step
          const uint64_t ad = aum_desc(k_s + (ks >> 2) * C::HALF_BYTES + (ks & 3) * 32, 0, 1024, 2);
          const uint64_t bd = aum_desc(q_s + (ks >> 2) * 2048 + (ks & 3) * 32, 0, 1024, 2);
          aum_mma(tmem + bb * 16, ad, bd, idesc_qk, ks > 0 ? 1u : 0u);
        }
        aum_commit(s_full + bb * 8);
        aum_commit(empty_k + st * 8);
        if (t >= 1) ok = pv(t - 1);
      }
      if (ok && my_tiles > 0) pv(my_tiles - 1);
    }
    __syncwarp();
  } else {
    // =========================== softmax: one thread per key ===========================
    const int key = tid;  // 0..127 = lane of tensor memory
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    float m_used[RMAX], l_thr[RMAX];
#pragma unroll
    for (int r = 0; r < RMAX; ++r) { m_used[r] = -INFINITY; l_thr[r] = 0.f; }
    struct Meta { int col; unsigned int memb; float inv; };
    auto load_meta = [&](int t) {
      Meta m;
      m.col = -1; m.memb = 0u; m.inv = 0.f;
      if (t < my_tiles) {
        const int u = (split + t * active) * AUM_TILE + key;
        if (u < U) {
          m.col = gcols[u];
          m.memb = gmemb[u];
          if constexpr (LSHW) m.inv = ginv[u];
        }
      }
      return m;
    };
    Meta nxt = load_meta(0);
    bool ok = true;
    for (int t = 0; t < my_tiles; ++t) {
      const int bb = t & 1, j = t >> 1;
      const Meta cur = nxt;
      nxt = load_meta(t + 1);
      const int u = (split + t * active) * AUM_TILE + key;
      {
        AUM_T0();
        ok = aum_wait_warp(s_full + bb * 8, (uint32_t)(j & 1), abort_sm, errflag);
        if (tid == 0) AUM_T1(8);
      }
      if (!ok) break;
#ifdef AUM_PROF
      const long long prof_tile_t0 = clock64();
#endif
      aum_fence_after();
      uint32_t sr[RMAX == 4 ? 8 : 16];
      if constexpr (RMAX == 4) aum_tmem_ld8(tmem + lane_base + bb * 16, sr);
      else aum_tmem_ld16(tmem + lane_base + bb * 16, sr);
      aum_fence_before();
      aum_arrive(s_free + bb * 8);

      float sv[RMAX], wv[RMAX];
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        sv[r] = -INFINITY;
        wv[r] = 0.f;
        if (r < a.R && cur.col >= 0 && ((cur.memb >> r) & 1u)) {
          float x = __uint_as_float(sr[r]) * a.scaling;
          const int64_t bo = boff_sm[r];
          if (bo >= 0) x += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.bias)[bo + cur.col]);
          float w;
          if constexpr (LSHW) {
            w = ((cur.memb >> (8 + r)) & 1u)
                    ? 1.f
                    : atm_lsh_weight(__uint_as_float(sr[4 + r]), qmu_sm[r], cur.inv, a.ptable);
            if (a.w_dump != nullptr) a.w_dump[((int64_t)g * a.S + u) * a.R + r] = w;
          } else {
            w = guw ? guw[(int64_t)u * a.R + r] : 1.f;
          }
          if (!(LSHW && w == 0.f)) {  // probability zero: not part of the mask
            sv[r] = x;
            wv[r] = w;
          }
        }
      }
      // tile maximum per row: warp reduction, then the four warps exchange through shared memory
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        const int mx = __reduce_max_sync(0xffffffffu, aum_ordered(sv[r]));
        if (lane == 0) wmax_sm[(bb * 4 + warp) * 16 + r] = aum_unordered(mx);
      }
      __syncwarp();
      if (lane == 0) aum_arrive(max_bar + bb * 8);
      {
        AUM_T0();
        ok = aum_wait_warp(max_bar + bb * 8, (uint32_t)(j & 1), abort_sm, errflag);
        if (tid == 0) AUM_T1(9);
      }
      if (!ok) break;
      float alpha[RMAX];
      bool rescale = false;
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        const float* wm = wmax_sm + bb * 64 + r;
        const float tm = fmaxf(fmaxf(wm[0], wm[16]), fmaxf(wm[32], wm[48]));
        alpha[r] = 1.f;
        if (tm > m_used[r] + AUM_RESCALE_T) {  // also the first finite maximum (-inf + T = -inf)
          alpha[r] = (m_used[r] == -INFINITY) ? 0.f : __expf(m_used[r] - tm);
          rescale |= (alpha[r] != 0.f);  // an accumulator column scaled by 0 was 0 already
          m_used[r] = tm;
        }
      }
      uint32_t pk[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) pk[i] = 0u;
#pragma unroll
      for (int r = 0; r < RMAX; r += 2) {
        float p0 = 0.f, p1 = 0.f;
        if (sv[r] != -INFINITY) p0 = __expf(sv[r] - m_used[r]) * wv[r];
        if (sv[r + 1] != -INFINITY) p1 = __expf(sv[r + 1] - m_used[r + 1]) * wv[r + 1];
        l_thr[r] = l_thr[r] * alpha[r] + p0;
        l_thr[r + 1] = l_thr[r + 1] * alpha[r + 1] + p1;
        pk[r >> 1] = atm_pack_bf16(p0, p1);
      }
      // the P buffer is free once the product that read it two tiles ago has completed
      {
        AUM_T0();
        if (j >= 1) ok = aum_wait_warp(p_free + bb * 8, (uint32_t)((j - 1) & 1), abort_sm, errflag);
        if (tid == 0) AUM_T1(10);
      }
      if (!ok) break;
      if (rescale && t > 0) {
        // the accumulator is quiet once the product of the previous tile has completed
        if (!(ok = aum_wait_warp(p_free + ((t - 1) & 1) * 8, (uint32_t)(((t - 1) >> 1) & 1), abort_sm, errflag))) break;
        aum_fence_after();
        uint32_t orow[16];
        aum_tmem_ld16(tmem_o + lane_base, orow);
#pragma unroll
        for (int r = 0; r < RMAX; ++r) orow[r] = __float_as_uint(__uint_as_float(orow[r]) * alpha[r]);
        aum_tmem_st16(tmem_o + lane_base, orow);
      }
      aum_store_p(sm + C::P_OFF + bb * 4096, key, pk);
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      aum_fence_before();
      aum_arrive(p_full + bb * 8);
#ifdef AUM_PROF
      if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
        atomicAdd((unsigned long long*)&aum_prof[11], (unsigned long long)(clock64() - prof_tile_t0));
        atomicAdd((unsigned long long*)&aum_prof[12], 1ull);
        if (rescale && t > 0) atomicAdd((unsigned long long*)&aum_prof[13], 1ull);
      }
#endif
    }
    // ---- the CTA's partial: O^T column r of this thread's lane = O[r][dim] ----
    float* pout = a.partial + ((int64_t)g * a.nsplit + split) * a.R * (D + 2);
    uint32_t orow[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) orow[i] = 0u;
    if (ok && my_tiles > 0) {
      const int last = my_tiles - 1;
      ok = aum_wait_warp(p_free + (last & 1) * 8, (uint32_t)((last >> 1) & 1), abort_sm, errflag);
      if (ok) {
        aum_fence_after();
        aum_tmem_ld16(tmem_o + lane_base, orow);
      }
    }
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      if (r < a.R) pout[r * (D + 2) + key] = ok ? __uint_as_float(orow[r]) : 0.f;
      float l = l_thr[r];
#pragma unroll
      for (int of = 16; of > 0; of >>= 1) l += __shfl_xor_sync(0xffffffffu, l, of);
      if (lane == 0) lred_sm[warp * 16 + r] = l;
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");  // after the loops: every softmax thread gets here
    if (key < a.R && key < RMAX) {
      const int r = key;
      float mr = -INFINITY;
#pragma unroll
      for (int q = 0; q < RMAX; ++q)
        if (q == r) mr = m_used[q];
      const float L = lred_sm[r] + lred_sm[16 + r] + lred_sm[32 + r] + lred_sm[48 + r];
      pout[r * (D + 2) + D] = ok ? mr : -INFINITY;
      pout[r * (D + 2) + D + 1] = ok ? L : 0.f;
    }
  }
  aum_fence_before();
  __syncthreads();
  if (warp == 5) {
    aum_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(AUM_TMEM_COLS));
  }
  atm_finish_group<D, AUM_THREADS>(a, g, active, sm, is_last_sm, tickets, sinks, out, part_out);
}

// Which problems take the tcgen05 kernel when the environment does not say.
static bool aum_default(bool lsh, int64_t S) {
  (void)lsh;
  (void)S;
  return false;
}

// The kernel choice: a process-wide setting (sah_attn_select_kernel), else SAH_ATTN_UMMA in the
// environment (1 selects the tcgen05 kernel wherever it applies, 0 never), else aum_default.
static int aum_setting = -1;
static int aum_requested() {
  if (aum_setting >= 0) return aum_setting;
  static int v = -2;
  if (v == -2) {
    const char* e = getenv("SAH_ATTN_UMMA");
    v = (e == nullptr) ? -1 : (e[0] == '1' ? 1 : 0);
  }
  return v;
}

static int aum_sm_count() {
  static int sms[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

// Launches the tcgen05 kernel when it applies (head dim 128, K and V viewable as 2-D row tensors,
// at most 4 mask rows with in-place weights, 16 otherwise).  Returns SAH_OK and sets *launched.
static int launch_attention_umma(AttnArgs a, int B, int groups, int* tickets, int* errflag,
                                 const float* sinks, void* out, float* part_out, bool lsh, cudaStream_t st,
                                 bool* launched) {
  static bool allowed[3][64] = {};
  *launched = false;
  if (lsh && a.R > 4) return SAH_OK;
  AtmMaps maps;
  memset(&maps, 0, sizeof(maps));
  if (!(atm_make_map(&maps.k, a.k, a.ks_b, a.ks_h, a.ks_s, B, a.Hkv, a.S, 128, &a.k_rows_b, &a.k_rows_h,
                     &a.k_rows_total) &&
        atm_make_map(&maps.v, a.v, a.vs_b, a.vs_h, a.vs_s, B, a.Hkv, a.S, 128, &a.v_rows_b, &a.v_rows_h,
                     &a.v_rows_total)))
    return SAH_OK;
  // one CTA per SM; two waves of CTAs over the groups (the kernel halves that for shorter lists)
  int64_t nsplit = (2 * (int64_t)aum_sm_count()) / groups;
  if (nsplit > a.nsplit) nsplit = a.nsplit;
  if (nsplit < 1) nsplit = 1;
  if ((size_t)16 * nsplit * 4 + 128 > (size_t)AumCfg::V_RING)
    return sah_fail(SAH_ERR_UNSUPPORTED, "attention: %d splits do not fit the merge scratch", (int)nsplit);
  dim3 grid((unsigned)nsplit, (unsigned)groups);
  cudaError_t e = cudaSuccess;
#define AUM_LAUNCH(LSHW, RMAX, SLOT)                                                                  \
  do {                                                                                                \
    e = atm_allow_smem(masked_attention_umma_kernel<LSHW, RMAX>, AumCfg::SMEM, allowed[SLOT]);        \
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "attention attr: %s", cudaGetErrorString(e)); \
    masked_attention_umma_kernel<LSHW, RMAX><<<grid, AUM_THREADS, AumCfg::SMEM, st>>>(                \
        a, maps, tickets, errflag, sinks, (__nv_bfloat16*)out, part_out);                             \
  } while (0)
  if (lsh) AUM_LAUNCH(true, 4, 0);
  else if (a.R <= 4) AUM_LAUNCH(false, 4, 1);
  else AUM_LAUNCH(false, 16, 2);
#undef AUM_LAUNCH
  *launched = true;
  return SAH_OK;
}

// bf16 gather attention on the fifth-generation tensor cores (tcgen05), head dim 128.
//
// Long union lists are bound by the K/V row gather; the mma.sync kernel spends ~48 warp
// instructions per key on fragment loads, address arithmetic and the softmax in the mma
// fragment layout.  Here the keys are the M dimension of the tensor-core tile, so one thread
// owns one key:
//
//   tile = 128 union entries.  Four producer warps gather their K rows and V rows with 16-byte
//   asynchronous copies (16 lanes cover one 256-byte row, so every 32-byte sector that is
//   fetched is used) into a three-stage ring (separate rings for K and V, with K slots freed as
//   soon as S^T has completed, measured slower), in the 128-byte swizzled layout that the tensor
//   core's shared-memory descriptors expect: two halves of [128 rows][128 B] per tile, 16-byte
//   chunk c of row i at chunk slot c ^ (i % 8).  (Tensor-map gathers, tile::gather4, were
//   measured first: one gather4 -- four 128-byte rows -- every ~64 cycles per SM, 2.2 TB/s over
//   the device, below what the copies reach.)
//     S^T[128 keys x 16]  = Ktile[128 x 128] . Qtile[16 x 128]^T    8 tcgen05.mma (K = 16 each),
//                           accumulator in tensor memory
//     thread-per-key softmax: each of 128 threads reads its key's row of S^T from tensor memory
//                           (mask rows in columns), applies scaling, bias, weights and the
//                           running maximum, and writes the key's row of P (bf16) to shared memory
//     O^T[128 dims x 16] += Vtile^T[128 dims x 128 keys] . P[128 keys x 16]   8 tcgen05.mma,
//                           accumulator in tensor memory for the whole list
//   Two softmax groups of four warps take the even and the odd tiles of the CTA, each with its
//   own S, P and O buffers and its own running maximum and denominator, so that the softmax of
//   one tile overlaps the next tile's; the groups are merged in shared memory at the end.
//   One elected thread issues all tcgen05.mma; completion is tracked with tcgen05.commit on
//   mbarriers.  The running maximum is lazy: the accumulator is rescaled (tensor memory load,
//   multiply, store) only when a row's maximum grew by more than AUM_RESCALE_T, so that P stays
//   below e^AUM_RESCALE_T; the final normalisation uses the same maximum, so the result is the
//   softmax whatever the history of rescales.
//
// With LSHW the columns 4..7 of the Q tile hold the centred unit queries and the MagicPig weight
// of a (row, key) pair is evaluated by the key's thread exactly as in the mma.sync kernel.
//
// Every wait on an mbarrier is bounded (about a second of wall time) and watches a CTA-wide
// abort word; a wait that runs out sets the abort word and the caller's error word, every role
// leaves its loop, the producers wait for their copies in flight, tensor memory is freed, and
// the CTA still takes its ticket so that no other CTA waits for it.
#pragma once
#include "sah_tcgen05.cuh"

#define AUM_TILE 128
#define AUM_STAGES 3
#define AUM_SOFT_WARPS 8     // two groups of four
#define AUM_PROD_WARPS 4
#define AUM_THREADS ((AUM_SOFT_WARPS + AUM_PROD_WARPS + 1) * 32)
#define AUM_TMEM_COLS 64
#define AUM_RESCALE_T 8.0f
#define AUM_MIN_TILES 2        // tiles a CTA should have before a further CTA joins the group
#define AUM_ONE_WAVE_TILES 128  // below this many tiles per CTA, one wave of CTAs instead of two

struct AumCfg {
  static constexpr int KV_TILE = AUM_TILE * 256;  // one K (or V) tile: two halves of [128 rows][128 B]
  static constexpr int HALF_BYTES = AUM_TILE * 128;
  static constexpr int K_RING = 0;
  static constexpr int V_RING = AUM_STAGES * KV_TILE;
  static constexpr int Q_OFF = 2 * AUM_STAGES * KV_TILE;  // two halves of [16 rows][128 B]
  static constexpr int P_OFF = Q_OFF + 4096;              // two buffers of [128 keys][32 B]
  static constexpr int BAR_OFF = P_OFF + 2 * 4096;
  // barriers: full[3] empty[3] s_full[2] s_free[2] p_full[2] p_free[2] max[2]
  static constexpr int N_BARS = 2 * AUM_STAGES + 10;
  static constexpr int MISC_OFF = BAR_OFF + ((N_BARS * 8 + 15) & ~15);
  // misc: tmem slot, abort word, last flag, pad; then wmax [2][4][16], lred [2][4][16], group
  // maxima [2][16], qmu [16], bias offsets [16] (int64)
  static constexpr int WMAX_OFF = MISC_OFF + 16;
  static constexpr int LRED_OFF = WMAX_OFF + 2 * 4 * 16 * 4;
  static constexpr int GMAX_OFF = LRED_OFF + 2 * 4 * 16 * 4;
  static constexpr int QMU_OFF = GMAX_OFF + 2 * 16 * 4;
  static constexpr int BOFF_OFF = QMU_OFF + 16 * 4;
  static constexpr int END = BOFF_OFF + 16 * 8;
  static constexpr int SMEM = 1024 + END;
};

__device__ __forceinline__ int aum_active_splits(int total_tiles, int nsplit, int one_wave_tiles) {
  int active = nsplit;
  // the grid holds two CTAs per SM; half of it, rounded down, is at most one per SM
  if (nsplit >= 2 && total_tiles < nsplit * one_wave_tiles) active = nsplit / 2;
  const int by_length = (total_tiles + AUM_MIN_TILES - 1) / AUM_MIN_TILES;
  if (by_length < active) active = by_length;
  return active < 1 ? 1 : active;
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
masked_attention_umma_kernel(AttnArgs a, int* __restrict__ tickets, int* __restrict__ errflag,
                             const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out,
                             float* __restrict__ part_out) {
  sah_pdl_entry();
  static_assert(!LSHW || RMAX == 4, "in-place MagicPig weights: at most 4 mask rows");
  constexpr int D = 128;
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
  const int active = aum_active_splits(total_tiles, (int)gridDim.x, a.one_wave_tiles);
  if (split >= active) return;  // before any barrier or tensor memory exists
  const int my_tiles = (total_tiles > split) ? (total_tiles - split + active - 1) / active : 0;

  // barrier addresses
  const uint32_t bar0 = sm_s + C::BAR_OFF;
  constexpr int NST = AUM_STAGES;
  const uint32_t full = bar0, empty = bar0 + NST * 8, s_full = bar0 + 2 * NST * 8, s_free = s_full + 16,
                 p_full = s_full + 32, p_free = s_full + 48, max_bar = s_full + 64;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + C::MISC_OFF);
  volatile int* abort_sm = reinterpret_cast<volatile int*>(sm + C::MISC_OFF + 4);
  int* is_last_sm = reinterpret_cast<int*>(sm + C::MISC_OFF + 8);
  float* wmax_sm = reinterpret_cast<float*>(sm + C::WMAX_OFF);
  float* lred_sm = reinterpret_cast<float*>(sm + C::LRED_OFF);
  float* gmax_sm = reinterpret_cast<float*>(sm + C::GMAX_OFF);
  float* qmu_sm = reinterpret_cast<float*>(sm + C::QMU_OFF);
  int64_t* boff_sm = reinterpret_cast<int64_t*>(sm + C::BOFF_OFF);
  constexpr int MMA_WARP = AUM_SOFT_WARPS + AUM_PROD_WARPS;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < NST; ++i) {
      atm_mbar_init(full + i * 8, AUM_PROD_WARPS);  // one arrival per producer warp
      atm_mbar_init(empty + i * 8, 1);              // tcgen05.commit after the tile's second product
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      atm_mbar_init(s_full + i * 8, 1);
      atm_mbar_init(s_free + i * 8, 4);  // one arrival per warp of the softmax group
      atm_mbar_init(p_full + i * 8, 4);
      atm_mbar_init(p_free + i * 8, 1);
      atm_mbar_init(max_bar + i * 8, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    *abort_sm = 0;
  }
  if (warp == MMA_WARP) {
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
  // tensor memory columns: S of group 0, S of group 1, O of group 0, O of group 1 (16 each)

  if (warp >= AUM_SOFT_WARPS && warp < MMA_WARP) {
    // =========================== producers ===========================
    // Warp pw copies rows 32 * pw .. 32 * pw + 31 of every tile: 16 lanes cover one 256-byte
    // row, two rows per instruction.
    const int pw = warp - AUM_SOFT_WARPS;
    const int my_chunk = lane & 15, my_sub = lane >> 4;
    const unsigned char* k_bytes = reinterpret_cast<const unsigned char*>(
                                       reinterpret_cast<const __nv_bfloat16*>(a.k) + b * a.ks_b + kvh * a.ks_h) +
                                   my_chunk * 16;
    const unsigned char* v_bytes = reinterpret_cast<const unsigned char*>(
                                       reinterpret_cast<const __nv_bfloat16*>(a.v) + b * a.vs_b + kvh * a.vs_h) +
                                   my_chunk * 16;
    const int64_t ks_bytes = a.ks_s * 2, vs_bytes = a.vs_s * 2;
    // destination of (row 2 * it + my_sub, chunk my_chunk) inside a K (or V) tile
    const uint32_t half_off = (uint32_t)(my_chunk >> 3) * C::HALF_BYTES;
    auto load_col = [&](int t) {
      int col = -1;
      if (t < my_tiles) {
        const int u = (split + t * active) * AUM_TILE + pw * 32 + lane;
        if (u < U) col = gcols[u];
      }
      return col;
    };
    int col_next = load_col(0);
    auto issue = [&](int t) {
      const int st = t % NST;
      const int col = col_next;
      col_next = load_col(t + 1);
      const uint32_t kt = C::K_RING + st * C::KV_TILE + half_off;
#pragma unroll
      for (int it = 0; it < 16; ++it) {
        const int rw = it * 2 + my_sub;  // row within the warp's 32
        const int rc = __shfl_sync(0xffffffffu, col, rw);
        const uint32_t off = kt + (uint32_t)(pw * 32 + rw) * 128 + ((uint32_t)((my_chunk & 7) ^ (rw & 7)) << 4);
        if (rc >= 0) {
          atm_cp_async16(sm_s + off, k_bytes + rc * ks_bytes);
          atm_cp_async16(sm_s + off + (C::V_RING - C::K_RING), v_bytes + rc * vs_bytes);
        } else {  // past the end of the list: zeros, not stale bits, go into the tensor core
          *reinterpret_cast<uint4*>(sm + off) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(sm + off + (C::V_RING - C::K_RING)) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    };
    // issue() takes the tiles in order (it carries the prefetched columns along)
#pragma unroll
    for (int s0 = 0; s0 < NST - 1; ++s0) {
      if (s0 < my_tiles) issue(s0);
      asm volatile("cp.async.commit_group;\n" ::);
    }
    for (int t = 0; t < my_tiles; ++t) {
      // tile t has landed (this thread's share): make it visible to the tensor core, signal
      asm volatile("cp.async.wait_group %0;\n" ::"n"(NST - 2));
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) aum_arrive(full + (t % NST) * 8);
      // refill the stage that tile t - 1 used once its second product has completed
      const int nx = t + NST - 1;
      if (nx < my_tiles) {
        bool okp = true;
        if (nx >= NST) {
          AUM_T0();
          okp = aum_wait_warp(empty + (nx % NST) * 8, (uint32_t)(((nx / NST) - 1) & 1), abort_sm, errflag);
          if (lane == 0 && pw == 0) AUM_T1(0);
        }
        if (!okp) break;
        issue(nx);
      }
      asm volatile("cp.async.commit_group;\n" ::);
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
  } else if (warp == MMA_WARP) {
    // =========================== tensor-core issuer ===========================
    if (lane == 0) {
      const uint32_t idesc_qk = aum_idesc(false, false);
      const uint32_t idesc_pv = aum_idesc(true, AUM_P_MN_MAJOR != 0);
      const uint32_t q_s = sm_s + C::Q_OFF;
      bool ok = true;
      auto pv = [&](int t) {
        const int st = t % NST, gg = t & 1, j = t >> 1;
        {
          AUM_T0();
          const bool o2 = aum_wait(p_full + gg * 8, (uint32_t)(j & 1), abort_sm, errflag);
          AUM_T1(5);
          if (!o2) return false;
        }
        aum_fence_after();
        const uint32_t v_s = sm_s + C::V_RING + st * C::KV_TILE;
        const uint32_t p_s = sm_s + C::P_OFF + gg * 4096;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // A = V^T, MN-major: 64 dims contiguous per 128-byte row, 8 keys per 1 KB atom,
          // the second 64 dims one half further
          const uint64_t ad = aum_desc(v_s + ks * 2048, C::HALF_BYTES, 1024, 2);
          const uint64_t bd = aum_p_desc(p_s, ks);
          aum_mma(tmem + 32 + gg * 16, ad, bd, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        }
        aum_commit(empty + st * 8);
        aum_commit(p_free + gg * 8);
        return true;
      };
      for (int t = 0; t < my_tiles && ok; ++t) {
        const int st = t % NST, gg = t & 1, j = t >> 1;
        {
          AUM_T0();
          ok = aum_wait(full + st * 8, (uint32_t)((t / NST) & 1), abort_sm, errflag);
          AUM_T1(6);
        }
        {
          AUM_T0();
          if (ok && j >= 1) ok = aum_wait(s_free + gg * 8, (uint32_t)((j - 1) & 1), abort_sm, errflag);
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
          aum_mma(tmem + gg * 16, ad, bd, idesc_qk, ks > 0 ? 1u : 0u);
        }
        aum_commit(s_full + gg * 8);
        if (t >= 1) ok = pv(t - 1);
      }
      if (ok && my_tiles > 0) pv(my_tiles - 1);
    }
    __syncwarp();
  } else {
    // =========================== softmax: one thread per key, two groups ===========================
    const int gg = warp >> 2;            // group: tiles gg, gg + 2, ...
    const int wg = warp & 3;             // warp within the group = quarter of tensor memory lanes
    const int key = (wg << 5) | lane;    // 0..127 = lane of tensor memory = key of the tile
    const uint32_t lane_base = ((uint32_t)(wg * 32)) << 16;
    const uint32_t tmem_s = tmem + gg * 16, tmem_o = tmem + 32 + gg * 16;
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
    Meta nxt = load_meta(gg);
    bool ok = true;
    int j = 0;
    for (int t = gg; t < my_tiles; t += 2, ++j) {
      const Meta cur = nxt;
      nxt = load_meta(t + 2);
      const int u = (split + t * active) * AUM_TILE + key;
      {
        AUM_T0();
        ok = aum_wait_warp(s_full + gg * 8, (uint32_t)(j & 1), abort_sm, errflag);
        if (tid == 0) AUM_T1(8);
      }
      if (!ok) break;
#ifdef AUM_PROF
      const long long prof_tile_t0 = clock64();
#endif
      aum_fence_after();
      uint32_t sr[RMAX == 4 ? 8 : 16];
      if constexpr (RMAX == 4) aum_tmem_ld8(tmem_s + lane_base, sr);
      else aum_tmem_ld16(tmem_s + lane_base, sr);
      aum_fence_before();
      __syncwarp();
      if (lane == 0) aum_arrive(s_free + gg * 8);
#ifdef AUM_PROF
      if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) atomicAdd((unsigned long long*)&aum_prof[14], (unsigned long long)(clock64() - prof_tile_t0));
#endif

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
      // tile maximum per row: warp reduction, then the group's four warps exchange through
      // shared memory
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        const int mx = __reduce_max_sync(0xffffffffu, aum_ordered(sv[r]));
        if (lane == 0) wmax_sm[(gg * 4 + wg) * 16 + r] = aum_unordered(mx);
      }
      __syncwarp();
      if (lane == 0) aum_arrive(max_bar + gg * 8);
#ifdef AUM_PROF
      if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) atomicAdd((unsigned long long*)&aum_prof[15], (unsigned long long)(clock64() - prof_tile_t0));
#endif
      // Probabilities with the maxima in use so far, before the other warps' maxima are known:
      // in the common case no row's maximum grows by more than the threshold and these stand, so
      // the exchange is off the critical path; otherwise they are redone below.
      float pr[RMAX];
      auto probabilities = [&]() {
#pragma unroll
        for (int r = 0; r < RMAX; ++r)
          pr[r] = (sv[r] != -INFINITY) ? __expf(sv[r] - m_used[r]) * wv[r] : 0.f;
      };
      probabilities();
      {
        AUM_T0();
        ok = aum_wait_warp(max_bar + gg * 8, (uint32_t)(j & 1), abort_sm, errflag);
        if (tid == 0) AUM_T1(9);
      }
      if (!ok) break;
      float alpha[RMAX];
      bool rescale = false, moved = false;
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        const float* wm = wmax_sm + gg * 64 + r;
        const float tm = fmaxf(fmaxf(wm[0], wm[16]), fmaxf(wm[32], wm[48]));
        alpha[r] = 1.f;
        if (tm > m_used[r] + AUM_RESCALE_T) {  // also the first finite maximum (-inf + T = -inf)
          alpha[r] = (m_used[r] == -INFINITY) ? 0.f : __expf(m_used[r] - tm);
          rescale |= (alpha[r] != 0.f);  // an accumulator column scaled by 0 was 0 already
          m_used[r] = tm;
          moved = true;
        }
      }
      if (moved) probabilities();  // uniform over the group: every thread sees the same maxima
      uint32_t pk[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) pk[i] = 0u;
#pragma unroll
      for (int r = 0; r < RMAX; r += 2) {
        l_thr[r] = l_thr[r] * alpha[r] + pr[r];
        l_thr[r + 1] = l_thr[r + 1] * alpha[r + 1] + pr[r + 1];
        pk[r >> 1] = atm_pack_bf16(pr[r], pr[r + 1]);
      }
      // the group's P buffer is free, and its accumulator quiet, once the product of the group's
      // previous tile has completed
      {
        AUM_T0();
        if (j >= 1) ok = aum_wait_warp(p_free + gg * 8, (uint32_t)((j - 1) & 1), abort_sm, errflag);
        if (tid == 0) AUM_T1(10);
      }
      if (!ok) break;
      if (rescale && j >= 1) {
        aum_fence_after();
        uint32_t orow[16];
        aum_tmem_ld16(tmem_o + lane_base, orow);
#pragma unroll
        for (int r = 0; r < RMAX; ++r) orow[r] = __float_as_uint(__uint_as_float(orow[r]) * alpha[r]);
        aum_tmem_st16(tmem_o + lane_base, orow);
      }
      aum_store_p(sm + C::P_OFF + gg * 4096, key, pk);
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      aum_fence_before();
      __syncwarp();
      if (lane == 0) aum_arrive(p_full + gg * 8);
#ifdef AUM_PROF
      if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
        atomicAdd((unsigned long long*)&aum_prof[11], (unsigned long long)(clock64() - prof_tile_t0));
        atomicAdd((unsigned long long*)&aum_prof[12], 1ull);
        if (rescale && j >= 1) atomicAdd((unsigned long long*)&aum_prof[13], 1ull);
      }
#endif
    }
    // ---- this group's share: O^T column r of this thread's lane = O[r][dim] ----
    uint32_t orow[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) orow[i] = 0u;
    if (ok && j > 0) {  // j = tiles this group took
      ok = aum_wait_warp(p_free + gg * 8, (uint32_t)((j - 1) & 1), abort_sm, errflag);
      if (ok) {
        aum_fence_after();
        aum_tmem_ld16(tmem_o + lane_base, orow);
      }
    }
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      float l = l_thr[r];
#pragma unroll
      for (int of = 16; of > 0; of >>= 1) l += __shfl_xor_sync(0xffffffffu, l, of);
      if (lane == 0) lred_sm[(gg * 4 + wg) * 16 + r] = l;
      if (key == 0) gmax_sm[gg * 16 + r] = ok ? m_used[r] : -INFINITY;
    }
    asm volatile("bar.sync 1, 256;\n" ::: "memory");  // after the loops: every softmax thread gets here
    // ---- merge the two groups: group 1 leaves its scaled accumulator in shared memory (the
    //      ring is idle now), group 0 adds its own and writes the CTA's partial ----
    float* obuf = reinterpret_cast<float*>(sm + C::K_RING);  // [RMAX][128]
    float scale_me[RMAX], m_cta[RMAX];
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      const float m0 = gmax_sm[r], m1 = gmax_sm[16 + r];
      const float mm = fmaxf(m0, m1);
      const float mine = gg ? m1 : m0;
      m_cta[r] = mm;
      scale_me[r] = (mine == -INFINITY) ? 0.f : __expf(mine - mm);
    }
    if (gg == 1) {
#pragma unroll
      for (int r = 0; r < RMAX; ++r) obuf[r * 128 + key] = __uint_as_float(orow[r]) * scale_me[r];
    }
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    if (gg == 0) {
      float* pout = a.partial + ((int64_t)g * a.nsplit + split) * a.R * (D + 2);
#pragma unroll
      for (int r = 0; r < RMAX; ++r)
        if (r < a.R) pout[r * (D + 2) + key] = __uint_as_float(orow[r]) * scale_me[r] + obuf[r * 128 + key];
      if (key < a.R && key < RMAX) {
        const int r = key;
        float mm = -INFINITY, L = 0.f;
#pragma unroll
        for (int q = 0; q < RMAX; ++q)
          if (q == r) {
            const float m0 = gmax_sm[q], m1 = gmax_sm[16 + q];
            mm = m_cta[q];
            const float s0 = (m0 == -INFINITY) ? 0.f : __expf(m0 - mm);
            const float s1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - mm);
            L = (lred_sm[q] + lred_sm[16 + q] + lred_sm[32 + q] + lred_sm[48 + q]) * s0 +
                (lred_sm[64 + q] + lred_sm[80 + q] + lred_sm[96 + q] + lred_sm[112 + q]) * s1;
          }
        pout[r * (D + 2) + D] = mm;
        pout[r * (D + 2) + D + 1] = L;
      }
    }
  }
  aum_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    aum_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(AUM_TMEM_COLS));
  }
  atm_finish_group<D, AUM_THREADS, __nv_bfloat16>(a, g, active, sm, is_last_sm, tickets, sinks, out, part_out);
}

// Which problems take the tcgen05 kernel when neither the caller nor the environment says.
// Measured on B200 (attention kernel, tcgen05 against mma.sync).  MagicPig weights in place,
// 8 KV groups: 1M keys (~770 000 rows per group, two waves of CTAs) 639 us; with one wave of
// CTAs (AUM_ONE_WAVE_TILES) 512K keys 332 against 366 us; 256K keys 177 against 189 us; 128K
// keys 99 against 108 us; 64K keys 63 against 73 us (two waves from 512K down: 337, 185 and
// 111 us -- a CTA's prologue, pipeline fill and merge are paid once per SM instead of twice).  64 KV groups with lists of a few
// thousand rows (HashAttention and Quest at B = 8, S = 32768): 63 against 69 us and 56 against
// 61 us.  In between -- 8 to 32 groups with lists of 10^4..10^5 rows -- the mma.sync kernel,
// with two CTAs per SM and lower fixed costs, was ahead by 5-40 % (measured with two waves).
#define AUM_DEFAULT_MIN_KEYS (64 * 1024)
static bool aum_default(bool lsh, int64_t S, int groups) {
  return (lsh && S >= AUM_DEFAULT_MIN_KEYS) || (groups >= 64 && S <= 65536);
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

// Launches the tcgen05 kernel when it applies (head dim 128, at most 4 mask rows with in-place
// weights, 16 otherwise).  Returns SAH_OK and sets *launched.
static int launch_attention_umma(AttnArgs a, int B, int groups, int* tickets, int* errflag,
                                 const float* sinks, void* out, float* part_out, bool lsh, cudaStream_t st,
                                 bool* launched) {
  static bool allowed[3][64] = {};
  *launched = false;
  if (lsh && a.R > 4) return SAH_OK;
  (void)B;
  // one CTA per SM; two waves of CTAs over the groups (the kernel halves that for shorter lists)
  int64_t nsplit = (2 * (int64_t)aum_sm_count()) / groups;
  if (nsplit > a.nsplit) nsplit = a.nsplit;
  if (nsplit < 1) nsplit = 1;
  if ((size_t)16 * nsplit * 4 + 128 > (size_t)AumCfg::Q_OFF)
    return sah_fail(SAH_ERR_UNSUPPORTED, "attention: %d splits do not fit the merge scratch", (int)nsplit);
  dim3 grid((unsigned)nsplit, (unsigned)groups);
  static int one_wave = -1;  // SAH_AUM_ONE_WAVE in the environment replaces AUM_ONE_WAVE_TILES
  if (one_wave < 0) {
    const char* ow = getenv("SAH_AUM_ONE_WAVE");
    one_wave = (ow != nullptr && atoi(ow) >= 0) ? atoi(ow) : AUM_ONE_WAVE_TILES;
  }
  a.one_wave_tiles = one_wave;
  cudaError_t e = cudaSuccess;
#define AUM_LAUNCH(LSHW, RMAX, SLOT)                                                                  \
  do {                                                                                                \
    e = atm_allow_smem(masked_attention_umma_kernel<LSHW, RMAX>, AumCfg::SMEM, allowed[SLOT]);        \
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "attention attr: %s", cudaGetErrorString(e)); \
    sah_launch_chain(masked_attention_umma_kernel<LSHW, RMAX>, grid, AUM_THREADS, AumCfg::SMEM, st, \
        a, tickets, errflag, sinks, (__nv_bfloat16*)out, part_out);                             \
  } while (0)
  if (lsh) AUM_LAUNCH(true, 4, 0);
  else if (a.R <= 4) AUM_LAUNCH(false, 4, 1);
  else AUM_LAUNCH(false, 16, 2);
#undef AUM_LAUNCH
  *launched = true;
  return SAH_OK;
}

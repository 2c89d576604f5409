// bf16 gather attention on the tensor cores.
//
// Every warp runs its own pipeline with no CTA-wide barrier in the main loop:
// it takes 16-key tiles of the group's union list (tiles are dealt round-robin
// to the warps of the CTAs that share the group) and gathers the 16 K rows and
// 16 V rows with 16-byte asynchronous copies into a private ring in shared
// memory.  Rows are padded by 16 bytes so that the 8 rows of an ldmatrix tile
// fall into different banks.  Per tile:
//     S[rows x 16 keys] = Q . K^T          mma.m16n8k16, Q fragments in registers
//     P = exp(S * scaling + bias - m) * w  online softmax in the C fragment
//     O[rows x D]      += P . V            mma.m16n8k16, V fragments via ldmatrix.trans
// "rows" are the mask rows of one KV group (query heads x query block, zero
// padded to 16, or to 8 when HALF), so each gathered K/V row is read once for
// all of them.  At the end the warps of a CTA merge their (m, l, O) in shared
// memory, the CTA writes its partial, and the last CTA of a group (atomic
// ticket) merges the group's partials and writes the output.
//
// LSHW (MagicPig weights evaluated in place; HALF tiles with at most 4 mask rows):
// rows 4..7 of the Q tile, otherwise zero padding, hold the group's centred unit
// queries, so the same mma that gives q.k also gives qhat.k.  The cosine between
// the transformed key and query is (qhat.k - qhat.mean) / (M * |transformed key|)
// (magic_pig.py:332-403), the collision probability comes from the cosine's bf16
// table, and the weight is 1 / (p + 1e-6) in bf16 -- or exactly 1 for columns
// that the unit-weight part of the mask (sink, window) selected.  No per-entry
// weight array is read or written.
#pragma once

//
// TMA (optional copy stage, HALF tiles): instead of 16-byte copies issued by every lane, four
// lanes of the warp issue tensor-map gathers (cp.async.bulk.tensor.2d ... tile::gather4: four
// indexed rows of a 2-D view of K or V per instruction, 64 columns wide) that land in the ring
// in the 128-byte swizzled layout; completion is counted on one mbarrier per stage.  No
// multicast qualifier: every CTA fetches its own rows, and the tensor maps cover this GPU's
// own K/V allocation only.  Every wait on an mbarrier is bounded; a wait that runs out sets
// the error word, the warp stops consuming tiles, and the kernel still goes through its
// merge and ticket protocol so that no other CTA is left waiting.
#include <cuda.h>
#include "sah_tcgen05.cuh"

#ifndef ATM_WARPS
#define ATM_WARPS 4
#endif
#ifndef ATM_STAGES
#define ATM_STAGES 3
#endif
#define ATM_THREADS (ATM_WARPS * 32)
#define ATM_TILE 16
#define ATM_MIN_TILES 8        // tiles a warp should have before a further CTA joins the group
#define ATM_ONE_WAVE_TILES 48  // below this many tiles per warp, one wave of CTAs instead of two
#define ATM_FINE_SPLITS 16     // ... when the grid has at least this many CTAs per group

struct AtmMaps {
  CUtensorMap k, v;
};

// Four rows y0..y3 of the 2-D tensor, columns [x, x + box width), to shared memory.
__device__ __forceinline__ void atm_tma_gather4(uint32_t dst, const CUtensorMap* map, int x, int y0,
                                                int y1, int y2, int y3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];\n" ::"r"(dst),
      "l"(map), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void atm_ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                uint32_t& r3, uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(saddr));
}
__device__ __forceinline__ void atm_ldmatrix_x2(uint32_t& r0, uint32_t& r1, uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r0), "=r"(r1)
               : "r"(saddr));
}
__device__ __forceinline__ void atm_ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                      uint32_t& r3, uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(saddr));
}
// D(16x8) += A(16x16) . B(16x8), all four accumulator registers live.
__device__ __forceinline__ void atm_mma_full(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Same product when rows 8..15 of A are zero: only the two registers of rows 0..7
// are carried; the other half reads constant zeros and its result is dropped.
__device__ __forceinline__ void atm_mma_half(float& c0, float& c1, uint32_t a0, uint32_t a2,
                                             uint32_t b0, uint32_t b1) {
  float j0, j1;
  const uint32_t z = 0u;
  const float zf = 0.f;
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%10,%11};\n"
      : "+f"(c0), "+f"(c1), "=f"(j0), "=f"(j1)
      : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1), "f"(zf), "f"(zf));
}
__device__ __forceinline__ uint32_t atm_pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}


// CTAs that share one group's union list.  The grid holds nsplit per group: two waves of the
// device for long lists (the second wave evens out groups of different length).  When the
// groups are few (nsplit >= ATM_FINE_SPLITS) and a list would give a warp fewer than
// ATM_ONE_WAVE_TILES tiles in that arrangement, half of the CTAs work on it: one wave, half as
// many pipeline fills and partials.  A short list is shared by as few CTAs as give every warp
// a run of ATM_MIN_TILES tiles; the others leave at once (they hold no ticket).
__device__ __forceinline__ int atm_active_splits(int total_tiles, int nsplit) {
  int active = nsplit;
  if (nsplit >= ATM_FINE_SPLITS && total_tiles < nsplit * ATM_WARPS * ATM_ONE_WAVE_TILES) active = nsplit / 2;
  const int by_length = (total_tiles + ATM_WARPS * ATM_MIN_TILES - 1) / (ATM_WARPS * ATM_MIN_TILES);
  if (by_length < active) active = by_length;
  return active < 1 ? 1 : active;
}

template <int D, bool TMA = false, int NST = ATM_STAGES>
struct AtmCfg {
  static constexpr int ROWB = D * 2;                        // bytes of one bf16 row
  // cp.async ring: whole rows padded by 16 bytes.  TMA ring: per K (or V) tile D/64 blocks of
  // [16 rows][128 bytes], each 2 KB and 1 KB aligned, 16-byte chunks swizzled by the row.
  static constexpr int RSTR = ROWB + 16;                    // padded row stride (cp.async ring, Q tile)
  static constexpr int HALVES = D / 64;
  static constexpr int KSTEPS = D / 16;                     // k-steps of Q.K^T
  static constexpr int NT = D / 8;                          // n-tiles of the output
  static constexpr int TILE_BYTES = TMA ? HALVES * ATM_TILE * 128 : ATM_TILE * RSTR;  // one K (or V) tile
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;        // K tile + V tile
  static constexpr int WARP_BYTES = NST * STAGE_BYTES;
  static constexpr int Q_BYTES = 16 * RSTR;                 // staged in the first ring before the pipeline starts
  static constexpr int RS = D + 8;                          // fp32 row stride of the reduction scratch
  static constexpr int RED_BYTES = 16 * RS * 4 + 16 * 2 * 4;
  static constexpr int META_BYTES = ATM_WARPS * NST * 16 * 16;  // (col, memb, 1/(M den), -)
  static constexpr int BAR_BYTES = ATM_WARPS * NST * 8;
  static constexpr int SMEM = (TMA ? 1024 : 0) + ATM_WARPS * WARP_BYTES + META_BYTES + BAR_BYTES;
};

// MagicPig weight of one (row, key) pair from the centred cosine (see the header comment): the
// table maps the cosine's bfloat16 bits to the bits of 1 / (p + 1e-6), rounded as the reference
// rounds it, and to 0 where the probability is 0 in bfloat16: the reference's dense mask holds
// a zero there, which means "not selected" (utils/mask.py:19-21).
__device__ __forceinline__ float atm_lsh_weight(float dot_hat, float qmu, float inv_md,
                                                const uint16_t* __restrict__ wtable) {
  float c = __fmul_rn(__fsub_rn(dot_hat, qmu), inv_md);
  c = __bfloat162float(__float2bfloat16_rn(c));
  c = fminf(fmaxf(c, -1.0f), 1.0f);
  return __uint_as_float(((uint32_t)__ldg(wtable + (__float_as_uint(c) >> 16))) << 16);
}

// The CTA has written its partial (running maximum, denominator and unnormalised output per
// mask row).  It takes a ticket; the last CTA of the group to arrive merges the `active`
// partials of the group, applies the sink logits and writes the output rows (and, when
// `part_out` is given, the group's merged partial for a merge across sequence shards).
// Called by all NT threads of the CTA; `scratch` is shared memory the CTA no longer needs
// (16 * active + 32 floats).
__device__ __forceinline__ void atm_store2(__nv_bfloat16* p, float x, float y) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y);
}
__device__ __forceinline__ void atm_store2(float* p, float x, float y) {
  *reinterpret_cast<float2*>(p) = make_float2(x, y);
}

template <int D, int NT, typename OutT>
__device__ __forceinline__ void atm_finish_group(const AttnArgs& a, int64_t g, int active,
                                                 unsigned char* scratch, int* is_last_sm,
                                                 int* __restrict__ tickets, const float* __restrict__ sinks,
                                                 OutT* __restrict__ out,
                                                 float* __restrict__ part_out) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qb = (int)(g % a.nqb);
  const int64_t bk = g / a.nqb;
  const int kvh = (int)(bk % a.Hkv);
  const int64_t b = bk / a.Hkv;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&tickets[g], 1);
    const int last = (old == active - 1);
    if (last) tickets[g] = 0;  // ready for the next call
    *is_last_sm = last;
  }
  __syncthreads();
  if (!*is_last_sm) return;
  __threadfence();
  const float* p0 = a.partial + (int64_t)g * a.nsplit * a.R * (D + 2);
  const int64_t pstride = (int64_t)a.R * (D + 2);
  // phase 1: one warp per row finds the row maximum, the per-split rescale
  // factors and the denominator
  float* sc_sm = reinterpret_cast<float*>(scratch);  // [R][active]
  float* ml_sm = sc_sm + 16 * active;                // [R][2]
  for (int r = warp; r < a.R; r += NT / 32) {
    const float* pr = p0 + (int64_t)r * (D + 2);
    float mloc = -INFINITY;
    for (int s2 = lane; s2 < active; s2 += 32) mloc = fmaxf(mloc, __ldcg(pr + s2 * pstride + D));
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, of));
    float lsum = 0.f;
    for (int s2 = lane; s2 < active; s2 += 32) {
      const float ms = __ldcg(pr + s2 * pstride + D);
      const float sc = (ms == -INFINITY) ? 0.f : __expf(ms - mloc);
      sc_sm[r * active + s2] = sc;
      lsum += __ldcg(pr + s2 * pstride + D + 1) * sc;
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, of);
    if (lane == 0) {
      ml_sm[r * 2] = mloc;
      ml_sm[r * 2 + 1] = lsum;
    }
  }
  __syncthreads();
  // phase 2: every thread owns (row, pair of dims) items and sums them over the splits with
  // 8-byte loads, eight in flight
  for (int idx = tid; idx < a.R * (D / 2); idx += NT) {
    const int r = idx / (D / 2), d = (idx - r * (D / 2)) * 2;
    const int gi = r / a.q_block, qo = r - gi * a.q_block;
    const int qi = qb * a.q_block + qo;
    if (qi >= a.Sq) continue;
    const int h = kvh * a.G + gi;
    const float* pr = p0 + (int64_t)r * (D + 2) + d;
    const float* sc = sc_sm + r * active;
    float2 accv = make_float2(0.f, 0.f);
#pragma unroll 8
    for (int s2 = 0; s2 < active; ++s2) {
      const float2 x = __ldcg(reinterpret_cast<const float2*>(pr + s2 * pstride));
      accv.x = fmaf(x.x, sc[s2], accv.x);
      accv.y = fmaf(x.y, sc[s2], accv.y);
    }
    const float M = ml_sm[r * 2], L = ml_sm[r * 2 + 1];
    float Mx = M, sink_term = 0.f;
    if (sinks != nullptr) {
      const float sk = sinks[h];
      Mx = fmaxf(M, sk);
      sink_term = __expf(sk - Mx);
    }
    const float resc = (M == -INFINITY) ? 0.f : __expf(M - Mx);
    const float den = L * resc + sink_term;
    const int64_t row = (b * a.Hq + h) * a.Sq + qi;
    if (part_out != nullptr) *reinterpret_cast<float2*>(part_out + row * (D + 2) + d) = accv;
    atm_store2(out + ((b * a.Sq + qi) * a.Hq + h) * D + d, accv.x * resc / den, accv.y * resc / den);
    if (part_out != nullptr && d == 0) {
      part_out[row * (D + 2) + D] = M;
      part_out[row * (D + 2) + D + 1] = L;
    }
  }
}

// NST: stages of the per-warp ring.  Three stages fit two CTAs (8 warps) per SM; two stages,
// with the register count capped accordingly, fit three CTAs (12 warps): fewer tiles in flight
// per warp, more warps to overlap one warp's arithmetic with the others' copies.
template <int D, bool HALF, bool LSHW, bool TMA, int NST>
__global__ void __launch_bounds__(ATM_THREADS, NST == 2 ? 3 : 2)
masked_attention_mma_kernel(AttnArgs a, const __grid_constant__ AtmMaps maps, int* __restrict__ tickets,
                            int* __restrict__ errflag, const float* __restrict__ sinks,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ part_out) {
  sah_pdl_entry();
  static_assert(!LSHW || HALF, "in-place MagicPig weights use the spare rows of the half tile");
  using C = AtmCfg<D, TMA, NST>;
  static_assert(C::Q_BYTES <= C::WARP_BYTES, "the Q tile is staged in the first ring");
  constexpr int NR = HALF ? 1 : 2;  // row halves a thread owns in the C fragment
  extern __shared__ __align__(128) unsigned char atm_smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the swizzled blocks of the TMA ring must start on 1 KB boundaries of the shared window
  unsigned char* atm_smem = atm_smem_raw;
  if constexpr (TMA) {
    const uint32_t raw_s = (uint32_t)__cvta_generic_to_shared(atm_smem_raw);
    atm_smem = atm_smem_raw + (((raw_s + 1023u) & ~1023u) - raw_s);
  }
  unsigned char* ring = atm_smem + warp * C::WARP_BYTES;
  unsigned char* q_sm = atm_smem;  // the first ring, before any copy is issued
  unsigned char* meta_base = atm_smem + ATM_WARPS * C::WARP_BYTES;
  int4* meta_sm = reinterpret_cast<int4*>(meta_base) + warp * NST * 16;
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
  const uint32_t bar_s = (uint32_t)__cvta_generic_to_shared(meta_base + C::META_BYTES) + warp * NST * 8;
  __shared__ int is_last_sm;
  if constexpr (TMA) {
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < NST; ++s) atm_mbar_init(bar_s + s * 8, 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
  }

  const int split = blockIdx.x;
  const int64_t g = blockIdx.y;
  const int qb = (int)(g % a.nqb);
  const int64_t bk = g / a.nqb;
  const int kvh = (int)(bk % a.Hkv);
  const int64_t b = bk / a.Hkv;
  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(a.k) + b * a.ks_b + kvh * a.ks_h;
  const __nv_bfloat16* vbase = reinterpret_cast<const __nv_bfloat16*>(a.v) + b * a.vs_b + kvh * a.vs_h;
  const int32_t* gcols = a.ucols + g * a.S;
  const uint16_t* gmemb = a.umemb + g * a.S;
  const float* guw = (!LSHW && a.uw) ? a.uw + g * a.S * a.R : nullptr;
  const float* ginv = LSHW ? a.uw + g * a.S : nullptr;  // 1 / (M * |transformed key|) per entry

  // ---- this warp's tiles ----
  const int U = a.ucount[g];
  const int total_tiles = (U + ATM_TILE - 1) / ATM_TILE;
  const int active = atm_active_splits(total_tiles, a.nsplit);
  if (split >= active) return;
  const int lanes_total = active * ATM_WARPS;     // warps sharing the group
  const int my_first = split * ATM_WARPS + warp;  // tile t of this warp = my_first + t * lanes_total
  const int my_tiles =
      (total_tiles > my_first) ? (total_tiles - my_first + lanes_total - 1) / lanes_total : 0;

  // Column, membership (and key constant) of the tiles to issue are fetched two tiles early,
  // so that their latency hides behind the tiles being computed and the first tiles of a
  // warp do not wait for one list read after the other.
  struct Meta { int col; unsigned int memb; float inv; };
  auto load_meta = [&](int t) {
    Meta m;
    m.col = -1; m.memb = 0u; m.inv = 0.f;
    if (t < my_tiles) {
      const int u = (my_first + t * lanes_total) * ATM_TILE + lane;
      if (lane < ATM_TILE && u < U) {
        m.col = gcols[u];
        m.memb = gmemb[u];
        if constexpr (LSHW) m.inv = ginv[u];
      }
    }
    return m;
  };
  Meta pre0 = load_meta(0), pre1 = load_meta(1);

  // ---- stage Q (zero padded to 16 rows; LSHW: rows 4..7 = centred unit queries) ----
  for (int idx = tid; idx < 16 * (C::ROWB / 16); idx += ATM_THREADS) {
    const int r = idx / (C::ROWB / 16), c = idx - r * (C::ROWB / 16);
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    const int rq = (LSHW && r >= 4) ? r - 4 : r;
    if (rq < a.R && (LSHW || r < a.R) && r < (LSHW ? 8 : 16)) {
      const int gi = rq / a.q_block, qo = rq - gi * a.q_block;
      const int qi = qb * a.q_block + qo;
      if (qi < a.Sq) {
        const int h = kvh * a.G + gi;
        if (LSHW && r >= 4)
          val = *reinterpret_cast<const uint4*>(a.qhat + ((b * a.Hq + h) * a.Sq + qi) * D + c * 8);
        else
          val = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.q) +
                                                b * a.qs_b + (int64_t)h * a.qs_h + qi * a.qs_q + c * 8);
      }
    }
    *reinterpret_cast<uint4*>(q_sm + r * C::RSTR + c * 16) = val;
  }
  __syncthreads();

  // Q fragments.  Full: [ks][0..3] = (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi),
  // (rows 8-15, k hi).  HALF: [ks][0..1] = (rows 0-7, k lo), (rows 0-7, k hi).
  uint32_t qf[C::KSTEPS][HALF ? 2 : 4];
  {
    const uint32_t q_s = (uint32_t)__cvta_generic_to_shared(q_sm);
    const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
    for (int ks = 0; ks < C::KSTEPS; ++ks) {
      if constexpr (HALF) {
        const int c = 2 * ks + (mi & 1);  // lanes 0-7: k lo, lanes 8-15: k hi
        atm_ldmatrix_x2(qf[ks][0], qf[ks][1], q_s + rr * C::RSTR + c * 16);
      } else {
        const int row = (mi & 1) * 8 + rr;
        const int c = 2 * ks + (mi >> 1);
        atm_ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][HALF ? 0 : 2], qf[ks][HALF ? 1 : 3],
                        q_s + row * C::RSTR + c * 16);
      }
    }
  }

  __syncthreads();  // every warp holds its Q fragments: the first ring is free for the pipeline

  // rows this thread owns in the C fragment, and their bias rows
  const int r0 = lane >> 2, r1 = r0 + 8;
  const __nv_bfloat16* bias_row[2] = {nullptr, nullptr};
  if (a.bias != nullptr) {
    const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(a.bias) + b * a.bias_s_b;
#pragma unroll
    for (int rs = 0; rs < NR; ++rs) {
      const int r = rs ? r1 : r0;
      const int gi = r / a.q_block, qo = r - gi * a.q_block;
      const int qi = qb * a.q_block + qo;
      if (r < a.R && qi < a.Sq) bias_row[rs] = bb + (kvh * a.G + gi) * a.bias_s_h + qi * a.bias_s_q;
    }
  }
  float qmu0 = 0.f;  // qhat . mean of this thread's row
  if constexpr (LSHW) {
    if (r0 < a.R) {
      const int gi = r0 / a.q_block, qo = r0 - gi * a.q_block;
      const int qi = qb * a.q_block + qo;
      if (qi < a.Sq) qmu0 = a.qmu[(b * a.Hq + kvh * a.G + gi) * a.Sq + qi];
    }
  }

  float o[C::NT][2 * NR];
#pragma unroll
  for (int nt = 0; nt < C::NT; ++nt)
#pragma unroll
    for (int e = 0; e < 2 * NR; ++e) o[nt][e] = 0.f;
  float m_run[NR], l_run[NR];
#pragma unroll
  for (int rs = 0; rs < NR; ++rs) { m_run[rs] = -INFINITY; l_run[rs] = 0.f; }

  // 16-byte asynchronous copies: CPR lanes cover one row, so a warp instruction
  // moves 32 / CPR whole rows; destination offsets are compile-time constants
  // plus a per-lane base.
  constexpr int CPR = C::ROWB / 16;        // chunks per row
  constexpr int RPS = 32 / CPR;            // rows per warp instruction
  const int my_chunk = lane % CPR, my_sub = lane / CPR;
  const uint32_t my_dst = my_sub * C::RSTR + my_chunk * 16;
  const unsigned char* k_bytes = reinterpret_cast<const unsigned char*>(kbase) + my_chunk * 16;
  const unsigned char* v_bytes = reinterpret_cast<const unsigned char*>(vbase) + my_chunk * 16;
  const int64_t ks_bytes = a.ks_s * 2, vs_bytes = a.vs_s * 2;

  // row of (batch b, KV head kvh, key 0) in the 2-D views of K and V that the tensor maps describe
  const int krow0 = TMA ? (int)(b * a.k_rows_b + kvh * a.k_rows_h) : 0;
  const int vrow0 = TMA ? (int)(b * a.v_rows_b + kvh * a.v_rows_h) : 0;

  auto issue = [&](int t) {
    const int st = t % NST;
    const Meta cur = pre0;
    pre0 = pre1;
    pre1 = load_meta(t + 2);
    if (lane < ATM_TILE)
      meta_sm[st * 16 + lane] = make_int4(cur.col, (int)cur.memb, __float_as_int(cur.inv), 0);
    if constexpr (TMA) {
      const uint32_t bar = bar_s + st * 8;
      if (lane == 0) atm_mbar_expect_tx(bar, (uint32_t)C::STAGE_BYTES);
      // lanes 0..3 fetch rows 4 * lane .. 4 * lane + 3; a row past the list reads as zeros
      // (its coordinate lies outside the tensor), and still counts its bytes
      int y[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) y[i] = __shfl_sync(0xffffffffu, cur.col, (4 * lane + i) & 15);
      __syncwarp();
      if (lane < 4) {
        const uint32_t dst = ring_s + st * C::STAGE_BYTES + lane * 4 * 128;
        int yk[4], yv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          yk[i] = y[i] >= 0 ? krow0 + y[i] : a.k_rows_total;
          yv[i] = y[i] >= 0 ? vrow0 + y[i] : a.v_rows_total;
        }
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h) {
          atm_tma_gather4(dst + h * 2048, &maps.k, h * 64, yk[0], yk[1], yk[2], yk[3], bar);
          atm_tma_gather4(dst + C::TILE_BYTES + h * 2048, &maps.v, h * 64, yv[0], yv[1], yv[2], yv[3], bar);
        }
      }
    } else {
      const uint32_t dst0 = ring_s + st * C::STAGE_BYTES + my_dst;
#pragma unroll
      for (int it = 0; it < ATM_TILE / RPS; ++it) {
        const int rc = __shfl_sync(0xffffffffu, cur.col, it * RPS + my_sub);
        const uint32_t dst = dst0 + it * RPS * C::RSTR;
        if (rc >= 0) {
          atm_cp_async16(dst, k_bytes + rc * ks_bytes);
          atm_cp_async16(dst + C::TILE_BYTES, v_bytes + rc * vs_bytes);
        } else {
          // unused rows must not feed NaNs into the tensor cores
          unsigned char* p = ring + st * C::STAGE_BYTES + my_dst + it * RPS * C::RSTR;
          *reinterpret_cast<uint4*>(p) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(p + C::TILE_BYTES) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
  };

#pragma unroll
  for (int s = 0; s < NST - 1; ++s) {
    if (s < my_tiles) issue(s);
    if constexpr (!TMA) asm volatile("cp.async.commit_group;\n" ::);
  }

  bool alive = true;
  int t = 0;
  for (; t < my_tiles; ++t) {
    if (t + NST - 1 < my_tiles) issue(t + NST - 1);
    const int st = t % NST;
    if constexpr (TMA) {
      if (!atm_mbar_wait(bar_s + st * 8, (uint32_t)((t / NST) & 1))) {
        alive = false;
        break;
      }
    } else {
      asm volatile("cp.async.commit_group;\n" ::);
      asm volatile("cp.async.wait_group %0;\n" ::"n"(NST - 1));
      __syncwarp();
    }
    const uint32_t kst = ring_s + st * C::STAGE_BYTES;
    const uint32_t vst = kst + C::TILE_BYTES;
    const int u0 = (my_first + t * lanes_total) * ATM_TILE;

    // ---- S = Q . K^T ----
    // even and odd k-steps accumulate separately: four chains of dependent mma instead of two
    float s[2][2 * NR], s_odd[2][2 * NR];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2 * NR; ++e) s[nt][e] = s_odd[nt][e] = 0.f;
    {
      const int mi = lane >> 3, rr = lane & 7;
      const uint32_t kaddr = TMA ? kst + ((mi >> 1) * 8 + rr) * 128
                                 : kst + ((mi >> 1) * 8 + rr) * C::RSTR + (mi & 1) * 16;
#pragma unroll
      for (int ks = 0; ks < C::KSTEPS; ++ks) {
        uint32_t b0, b1, b2, b3;
        // TMA ring: 16-byte chunk c of a row sits in block c / 8 at chunk slot (c % 8) ^ (row % 8)
        const int kc = 2 * ks + (mi & 1);
        atm_ldmatrix_x4(b0, b1, b2, b3,
                        TMA ? kaddr + (kc >> 3) * 2048 + (((kc & 7) ^ rr) << 4) : kaddr + ks * 32);
        float(*acc)[2 * NR] = (ks & 1) ? s_odd : s;
        if constexpr (HALF) {
          atm_mma_half(acc[0][0], acc[0][1], qf[ks][0], qf[ks][1], b0, b1);
          atm_mma_half(acc[1][0], acc[1][1], qf[ks][0], qf[ks][1], b2, b3);
        } else {
          atm_mma_full(acc[0], qf[ks], b0, b1);
          atm_mma_full(acc[1], qf[ks], b2, b3);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2 * NR; ++e) s[nt][e] += s_odd[nt][e];
    // LSHW: the products with the centred unit queries sit four rows further down,
    // i.e. in the lane 16 higher
    float hat[2][2];
    if constexpr (LSHW) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) hat[nt][e] = __shfl_down_sync(0xffffffffu, s[nt][e], 16);
    }

    // ---- online softmax in the C fragment ----
    // element (nt, e): row half rs = e >> 1, key j = nt * 8 + 2 * (lane & 3) + (e & 1)
    float wts[2][2 * NR];
    float tmax[NR];
#pragma unroll
    for (int rs = 0; rs < NR; ++rs) tmax[rs] = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2 * NR; ++e) {
        const int j = nt * 8 + 2 * (lane & 3) + (e & 1);
        const int rs = e >> 1;
        const int r = rs ? r1 : r0;
        const int4 cm = meta_sm[st * 16 + j];
        float sv = -INFINITY, wv = 0.f;
        if (cm.x >= 0 && ((cm.y >> r) & 1) && (!LSHW || r < 4)) {
          sv = s[nt][e] * a.scaling;
          if (bias_row[rs] != nullptr) sv += __bfloat162float(bias_row[rs][cm.x]);
          if constexpr (LSHW) {
            wv = ((cm.y >> (8 + r)) & 1)
                     ? 1.f
                     : atm_lsh_weight(hat[nt][e & 1], qmu0, __int_as_float(cm.z), a.ptable);
            if (a.w_dump != nullptr) a.w_dump[((int64_t)g * a.S + u0 + j) * a.R + r] = wv;
            if (wv == 0.f) sv = -INFINITY;  // probability zero: not part of the mask
          } else {
            wv = guw ? guw[(int64_t)(u0 + j) * a.R + r] : 1.f;
          }
        }
        s[nt][e] = sv;
        wts[nt][e] = wv;
        tmax[rs] = fmaxf(tmax[rs], sv);
      }
    }
    float alpha[NR];
#pragma unroll
    for (int rs = 0; rs < NR; ++rs) {
      tmax[rs] = fmaxf(tmax[rs], __shfl_xor_sync(0xffffffffu, tmax[rs], 1));
      tmax[rs] = fmaxf(tmax[rs], __shfl_xor_sync(0xffffffffu, tmax[rs], 2));
      const float m_new = fmaxf(m_run[rs], tmax[rs]);
      alpha[rs] = (m_new == m_run[rs]) ? 1.f : __expf(m_run[rs] - m_new);
      m_run[rs] = m_new;
    }
    float psum[NR];
#pragma unroll
    for (int rs = 0; rs < NR; ++rs) psum[rs] = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2 * NR; ++e) {
        const int rs = e >> 1;
        float pv = 0.f;
        if (s[nt][e] != -INFINITY) pv = __expf(s[nt][e] - m_run[rs]) * wts[nt][e];
        s[nt][e] = pv;  // s now holds P
        psum[rs] += pv;
      }
    }
    bool rescale = false;
#pragma unroll
    for (int rs = 0; rs < NR; ++rs) {
      psum[rs] += __shfl_xor_sync(0xffffffffu, psum[rs], 1);
      psum[rs] += __shfl_xor_sync(0xffffffffu, psum[rs], 2);
      l_run[rs] = l_run[rs] * alpha[rs] + psum[rs];
      rescale |= (alpha[rs] != 1.f);
    }
    if (__any_sync(0xffffffffu, rescale)) {  // the running maximum moved for some row
#pragma unroll
      for (int nt = 0; nt < C::NT; ++nt)
#pragma unroll
        for (int e = 0; e < 2 * NR; ++e) o[nt][e] *= alpha[e >> 1];
    }

    // ---- O += P . V ----
    uint32_t pa[4];
    pa[0] = atm_pack_bf16(s[0][0], s[0][1]);
    pa[2] = atm_pack_bf16(s[1][0], s[1][1]);
    pa[1] = HALF ? 0u : atm_pack_bf16(s[0][2 * NR - 2], s[0][2 * NR - 1]);
    pa[3] = HALF ? 0u : atm_pack_bf16(s[1][2 * NR - 2], s[1][2 * NR - 1]);
    {
      const int mi = lane >> 3, rr = lane & 7;
      const uint32_t vaddr = TMA ? vst + ((mi & 1) * 8 + rr) * 128
                                 : vst + ((mi & 1) * 8 + rr) * C::RSTR + (mi >> 1) * 16;
#pragma unroll
      for (int np = 0; np < C::NT / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        const int vc = 2 * np + (mi >> 1);
        atm_ldmatrix_x4_trans(b0, b1, b2, b3,
                              TMA ? vaddr + (vc >> 3) * 2048 + (((vc & 7) ^ rr) << 4) : vaddr + np * 32);
        if constexpr (HALF) {
          atm_mma_half(o[2 * np][0], o[2 * np][1], pa[0], pa[2], b0, b1);
          atm_mma_half(o[2 * np + 1][0], o[2 * np + 1][1], pa[0], pa[2], b2, b3);
        } else {
          atm_mma_full(o[2 * np], pa, b0, b1);
          atm_mma_full(o[2 * np + 1], pa, b2, b3);
        }
      }
    }
    __syncwarp();  // all lanes done with this stage before it is refilled
  }
  if constexpr (TMA) {
    if (!alive) {
      if (lane == 0) atomicExch(errflag, 1);
      // give the copies still in flight a bounded chance to land before the ring is reused
      for (int tt = t; tt < my_tiles && tt < t + NST; ++tt)
        atm_mbar_wait(bar_s + (tt % NST) * 8, (uint32_t)((tt / NST) & 1));
    }
  } else {
    asm volatile("cp.async.wait_group 0;\n" ::);
  }
  __syncthreads();

  // ---- merge the warps of this CTA (ring reused as fp32 scratch) ----
  // (LSHW: rows 4..7 of the tile carried no softmax state: their maximum is -inf and they
  // are beyond a.R, so nothing below reads them)
  constexpr int RS = C::RS;
  float* red_o = reinterpret_cast<float*>(ring);  // [16][RS]
  float* red_ml = red_o + 16 * RS;                // [16][2]
#pragma unroll
  for (int nt = 0; nt < C::NT; ++nt) {
    const int d = nt * 8 + 2 * (lane & 3);
    *reinterpret_cast<float2*>(red_o + r0 * RS + d) = make_float2(o[nt][0], o[nt][1]);
    if constexpr (!HALF)
      *reinterpret_cast<float2*>(red_o + r1 * RS + d) =
          make_float2(o[nt][2 * NR - 2], o[nt][2 * NR - 1]);
  }
  if ((lane & 3) == 0) {
    red_ml[r0 * 2] = m_run[0];
    red_ml[r0 * 2 + 1] = l_run[0];
    if constexpr (!HALF) {
      red_ml[r1 * 2] = m_run[NR - 1];
      red_ml[r1 * 2 + 1] = l_run[NR - 1];
    }
  }
  __syncthreads();
  float* pout = a.partial + ((int64_t)g * a.nsplit + split) * a.R * (D + 2);
  for (int idx = tid; idx < a.R * D; idx += ATM_THREADS) {
    const int r = idx / D, d = idx - r * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATM_WARPS; ++w)
      M = fmaxf(M, reinterpret_cast<const float*>(atm_smem + w * C::WARP_BYTES)[16 * RS + r * 2]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < ATM_WARPS; ++w) {
      const float* wo = reinterpret_cast<const float*>(atm_smem + w * C::WARP_BYTES);
      const float mw = wo[16 * RS + r * 2];
      if (mw != -INFINITY) {
        const float sc = __expf(mw - M);
        acc += wo[r * RS + d] * sc;
        L += wo[16 * RS + r * 2 + 1] * sc;
      }
    }
    pout[r * (D + 2) + d] = acc;
    if (d == 0) {
      pout[r * (D + 2) + D] = M;
      pout[r * (D + 2) + D + 1] = L;
    }
  }

  atm_finish_group<D, ATM_THREADS, __nv_bfloat16>(a, g, active, atm_smem, &is_last_sm, tickets, sinks, out, part_out);
}

// Row-gather probe: the copy half of the attention kernel alone.  Same grid, same dealing of
// 16-key tiles to warps, same 16-byte asynchronous copies into the same per-warp ring, no
// arithmetic: the time of this kernel on a union list is what the K/V row gather of that list
// costs on this device, i.e. the ceiling the attention kernel can approach.
template <int D>
__global__ void __launch_bounds__(ATM_THREADS, 2)
attention_gather_probe_kernel(AttnArgs a, unsigned int* __restrict__ sink) {
  using C = AtmCfg<D>;
  extern __shared__ __align__(128) unsigned char atm_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned char* ring = atm_smem + warp * C::WARP_BYTES;
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
  const int split = blockIdx.x;
  const int64_t g = blockIdx.y;
  const int64_t bk = g / a.nqb;
  const int kvh = (int)(bk % a.Hkv);
  const int64_t b = bk / a.Hkv;
  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(a.k) + b * a.ks_b + kvh * a.ks_h;
  const __nv_bfloat16* vbase = reinterpret_cast<const __nv_bfloat16*>(a.v) + b * a.vs_b + kvh * a.vs_h;
  const int32_t* gcols = a.ucols + g * a.S;
  const int U = a.ucount[g];
  const int total_tiles = (U + ATM_TILE - 1) / ATM_TILE;
  const int active = atm_active_splits(total_tiles, a.nsplit);
  if (split >= active) return;
  const int lanes_total = active * ATM_WARPS;
  const int my_first = split * ATM_WARPS + warp;
  const int my_tiles =
      (total_tiles > my_first) ? (total_tiles - my_first + lanes_total - 1) / lanes_total : 0;
  auto load_col = [&](int t) {
    int col = -1;
    if (t < my_tiles) {
      const int u = (my_first + t * lanes_total) * ATM_TILE + lane;
      if (lane < ATM_TILE && u < U) col = gcols[u];
    }
    return col;
  };
  int pre0 = load_col(0), pre1 = load_col(1);
  constexpr int CPR = C::ROWB / 16;
  constexpr int RPS = 32 / CPR;
  const int my_chunk = lane % CPR, my_sub = lane / CPR;
  const uint32_t my_dst = my_sub * C::RSTR + my_chunk * 16;
  const unsigned char* k_bytes = reinterpret_cast<const unsigned char*>(kbase) + my_chunk * 16;
  const unsigned char* v_bytes = reinterpret_cast<const unsigned char*>(vbase) + my_chunk * 16;
  const int64_t ks_bytes = a.ks_s * 2, vs_bytes = a.vs_s * 2;
  auto issue = [&](int t) {
    const int st = t % ATM_STAGES;
    const int col = pre0;
    pre0 = pre1;
    pre1 = load_col(t + 2);
    const uint32_t dst0 = ring_s + st * C::STAGE_BYTES + my_dst;
#pragma unroll
    for (int it = 0; it < ATM_TILE / RPS; ++it) {
      const int rc = __shfl_sync(0xffffffffu, col, it * RPS + my_sub);
      const uint32_t dst = dst0 + it * RPS * C::RSTR;
      if (rc >= 0) {
        atm_cp_async16(dst, k_bytes + rc * ks_bytes);
        atm_cp_async16(dst + C::TILE_BYTES, v_bytes + rc * vs_bytes);
      }
    }
  };
#pragma unroll
  for (int s = 0; s < ATM_STAGES - 1; ++s) {
    if (s < my_tiles) issue(s);
    asm volatile("cp.async.commit_group;\n" ::);
  }
  unsigned int acc = 0u;
  for (int t = 0; t < my_tiles; ++t) {
    if (t + ATM_STAGES - 1 < my_tiles) issue(t + ATM_STAGES - 1);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group %0;\n" ::"n"(ATM_STAGES - 1));
    __syncwarp();
    acc += *reinterpret_cast<const unsigned int*>(ring + (t % ATM_STAGES) * C::STAGE_BYTES + lane * 16);
    __syncwarp();
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  if (acc == 0x9e3779b9u) *sink = acc;  // keeps the reads alive; practically never true
}

// The kernels ask for more dynamic shared memory than the default limit; the attribute is
// set once per device and instantiation.
template <typename Kernel>
static cudaError_t atm_allow_smem(Kernel kernel, int smem, bool* done_by_device) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && done_by_device[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess && dev >= 0 && dev < 64) done_by_device[dev] = true;
  return e;
}

// ---- tensor maps of K and V for the TMA copy stage --------------------------------------
typedef CUresult (*AtmEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

// The driver's encoder, looked up through the runtime (the library does not link libcuda).
static AtmEncodeTiled atm_encoder() {
  static AtmEncodeTiled fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AtmEncodeTiled>(p);
  }
  return fn;
}

// 2-D view [rows][D] of a [B][Hkv][S][D] tensor whose batch and head strides are whole rows:
// row = b * rows_b + h * rows_h + s.  Box: 64 columns x 1 row (gather4 takes four such rows),
// 128-byte swizzle, zero fill outside the tensor.  False when the layout is not such a view.
static bool atm_make_map(CUtensorMap* map, const void* base, int64_t s_b, int64_t s_h, int64_t s_s, int B,
                         int Hkv, int64_t S, int D, int64_t* rows_b, int64_t* rows_h, int* rows_total) {
  AtmEncodeTiled enc = atm_encoder();
  if (enc == nullptr || s_s <= 0 || s_b % s_s != 0 || s_h % s_s != 0 || s_b < 0 || s_h < 0) return false;
  *rows_b = s_b / s_s;
  *rows_h = s_h / s_s;
  const int64_t total = (int64_t)(B - 1) * *rows_b + (int64_t)(Hkv - 1) * *rows_h + S;
  if (total <= 0 || total >= (1ll << 31) - 8) return false;
  *rows_total = (int)total;
  const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)total};
  const cuuint64_t strides[1] = {(cuuint64_t)s_s * 2};
  const cuuint32_t box[2] = {64, 1};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// SAH_ATTN_TMA=1 in the environment selects the tensor-map gather for the copy stage of the
// bfloat16 kernel (half tiles); the default is the 16-byte cp.async ring.
static bool atm_tma_requested() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SAH_ATTN_TMA");
    v = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

// SAH_ATTN_STAGES=2 in the environment selects the two-stage ring (three CTAs per SM) for the
// half-tile kernels; the default is three stages (two CTAs per SM).
static int atm_stages_requested() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SAH_ATTN_STAGES");
    v = (e != nullptr && e[0] == '2') ? 2 : 3;
  }
  return v;
}

template <int D>
static int launch_attention_mma(AttnArgs a, int B, int groups, int* tickets, int* errflag,
                                const float* sinks, void* out, float* part_out, bool lsh,
                                cudaStream_t st) {
  static bool allowed[9][64] = {};
  // shared memory that the last CTA of a group needs to merge the splits (atm_finish_group)
  const size_t merge_bytes = (size_t)16 * a.nsplit * 4 + 128;
  static_assert(AtmCfg<D, false, 2>::RED_BYTES <= AtmCfg<D, false, 2>::WARP_BYTES &&
                AtmCfg<D, true, 2>::RED_BYTES <= AtmCfg<D, true, 2>::WARP_BYTES,
                "reduction scratch must fit the ring");
  if (lsh && a.R > 4)
    return sah_fail(SAH_ERR_UNSUPPORTED, "attention: in-place MagicPig weights need <= 4 mask rows "
                    "per KV group, got %d", a.R);
  dim3 grid((unsigned)a.nsplit, (unsigned)groups);
  AtmMaps maps;
  memset(&maps, 0, sizeof(maps));
  bool tma = false;
  if (atm_tma_requested() && a.R <= 8) {
    tma = atm_make_map(&maps.k, a.k, a.ks_b, a.ks_h, a.ks_s, B, a.Hkv, a.S, D, &a.k_rows_b, &a.k_rows_h,
                       &a.k_rows_total) &&
          atm_make_map(&maps.v, a.v, a.vs_b, a.vs_h, a.vs_s, B, a.Hkv, a.S, D, &a.v_rows_b, &a.v_rows_h,
                       &a.v_rows_total);
  }
  const bool two = atm_stages_requested() == 2;
  cudaError_t e = cudaSuccess;
#define ATM_LAUNCH(HALF, LSHW, TMA, NST, SLOT)                                                      \
  do {                                                                                              \
    const int smem = AtmCfg<D, TMA, NST>::SMEM;                                                     \
    if (merge_bytes > (size_t)ATM_WARPS * AtmCfg<D, TMA, NST>::WARP_BYTES)                          \
      return sah_fail(SAH_ERR_UNSUPPORTED, "attention: %d splits do not fit the merge scratch", a.nsplit); \
    e = atm_allow_smem(masked_attention_mma_kernel<D, HALF, LSHW, TMA, NST>, smem, allowed[SLOT]);  \
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "attention attr: %s", cudaGetErrorString(e)); \
    sah_launch_chain(masked_attention_mma_kernel<D, HALF, LSHW, TMA, NST>, grid, ATM_THREADS, smem, st, \
        a, maps, tickets, errflag, sinks, (__nv_bfloat16*)out, part_out);                           \
  } while (0)
  if (lsh) {
    if (tma && two) ATM_LAUNCH(true, true, true, 2, 5);
    else if (tma) ATM_LAUNCH(true, true, true, 3, 3);
    else if (two) ATM_LAUNCH(true, true, false, 2, 6);
    else ATM_LAUNCH(true, true, false, 3, 2);
  } else if (a.R <= 8) {
    if (tma && two) ATM_LAUNCH(true, false, true, 2, 7);
    else if (tma) ATM_LAUNCH(true, false, true, 3, 4);
    else if (two) ATM_LAUNCH(true, false, false, 2, 8);
    else ATM_LAUNCH(true, false, false, 3, 0);
  } else {
    ATM_LAUNCH(false, false, false, 3, 1);
  }
#undef ATM_LAUNCH
  return SAH_OK;
}

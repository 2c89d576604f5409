// Masked attention over a bitmap Mask (utils/mask_attention_utils.py:406-491):
//   sah_attn_query_sizes   work-list geometry for one call
//   sah_attn_plan          per KV group: ascending union of the selected columns,
//                          which rows selected each, inverse weights
//   sah_masked_attention   gather of the selected K/V rows through a cp.async
//                          pipeline, weighted online softmax in fp32, every row
//                          fetched once per group and shared by its query heads
//   sah_attn_merge_parts   associative merge of sequence-sharded partials
#include <mutex>
#include <stdlib.h>
#include <string.h>

#include "sah_common.cuh"

#define AT_THREADS 128
#define AT_STAGES 3
#define AT_MAXR 16
#define PLAN_CHUNK_WORDS 32  // one warp scans 32 bitmap words = 1024 columns

// Chunk counters per group: a function of the key count alone, so that the plan, the
// attention kernel and the size query agree on where the counters, the merge tickets and
// the error word sit, whatever row stride W the caller's bitmap has.
static inline int64_t plan_chunks(int64_t S) {
  return (((S + 31) / 32 + 3) / 4 * 4 + PLAN_CHUNK_WORDS - 1) / PLAN_CHUNK_WORDS;
}

// ---------------------------------------------------------------------------
// geometry
// ---------------------------------------------------------------------------
extern "C" int sah_attn_query_sizes(int B, int Hq, int Hkv, int Sq, int64_t S, int D,
                                    int has_data, int sm_count, sah_attn_sizes* out) {
  SAH_REQUIRE(out != nullptr, "attn_query_sizes: out is null");
  SAH_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Sq > 0 && S > 0 && D > 0,
              "attn_query_sizes: bad extents");
  const int G = Hq / Hkv;
  if (G > AT_MAXR)
    return sah_fail(SAH_ERR_UNSUPPORTED, "attention: %d query heads per KV head (<= %d)", G,
                    AT_MAXR);
  // One register quad (4 mask rows) per group whenever the GQA ratio allows it.
  int q_block = (G <= 4) ? (4 / G) : 1;
  if (q_block > Sq) q_block = Sq;
  const int nqb = (Sq + q_block - 1) / q_block;
  const int64_t groups = (int64_t)B * Hkv * nqb;
  SAH_REQUIRE(groups < (1ll << 30), "attn_query_sizes: too many groups");
  if (sm_count <= 0) sm_count = 148;
  // Two resident CTAs per SM; the split count is rounded down so that the grid
  // fills whole waves of 2 * sm_count CTAs instead of spilling into a short tail.
  const int64_t slots = (int64_t)sm_count * 2;
  int64_t waves = (groups + slots - 1) / slots;
  if (waves < 2) waves = 2;
  int64_t nsplit = (waves * slots) / groups;
  int64_t max_split = (S + 255) / 256;  // at least 256 columns of range per CTA
  if (nsplit > max_split) nsplit = max_split;
  if (nsplit > 256) nsplit = 256;
  if (nsplit < 1) nsplit = 1;
  const int R = G * q_block;
  const int64_t nchunks = plan_chunks(S);
  out->groups = (int32_t)groups;
  out->q_block = q_block;
  out->rows_per_group = R;
  out->nsplit = (int32_t)nsplit;
  out->ucols_bytes = groups * S * (int64_t)sizeof(int32_t);
  out->umemb_bytes = groups * S * (int64_t)sizeof(uint16_t);
  // has_data: 0 unit weights, 1 per-entry weights (uw [groups][S][R]), 2 MagicPig weights
  // evaluated inside the attention kernel (one key constant per union entry, [groups][S])
  out->uw_bytes = has_data == 1 ? groups * S * R * (int64_t)sizeof(float)
                                : (has_data == 2 ? groups * S * (int64_t)sizeof(float) : 0);
  // [groups] union counts, [groups][nchunks] chunk counts, [groups] merge tickets
  // and one error word (non-zero after a bounded device-side wait ran out)
  out->ucount_bytes = (2 * groups + groups * nchunks + 4) * (int64_t)sizeof(int32_t);
  out->partial_bytes = groups * nsplit * R * (int64_t)(D + 2) * (int64_t)sizeof(float);
  return SAH_OK;
}

// ---------------------------------------------------------------------------
// plan
// ---------------------------------------------------------------------------
struct PlanGeom {
  int Hq, Hkv, Sq, G, q_block, nqb, R;
  int64_t S, W, nchunks, groups;
  int64_t Wv;          // words that hold columns < S (<= W)
  uint32_t tail_mask;  // valid bits of word Wv - 1
};

// word w of a row with the bits of columns >= S dropped
__device__ __forceinline__ uint32_t plan_word(const PlanGeom& p, uint32_t v, int64_t w) {
  return w == p.Wv - 1 ? (v & p.tail_mask) : v;
}

// mask row of member r of group g, or -1 when the member's query is past Sq
__device__ __forceinline__ int64_t plan_member_row(const PlanGeom& p, int64_t g, int r) {
  int qb = (int)(g % p.nqb);
  int64_t bk = g / p.nqb;
  int kvh = (int)(bk % p.Hkv);
  int64_t b = bk / p.Hkv;
  int gi = r / p.q_block, qo = r - gi * p.q_block;
  int qi = qb * p.q_block + qo;
  if (qi >= p.Sq) return -1;
  int h = kvh * p.G + gi;
  return (b * p.Hq + h) * p.Sq + qi;
}

__global__ void attn_plan_count_kernel(const uint32_t* __restrict__ bits,
                                       const uint32_t* __restrict__ ubits, PlanGeom p,
                                       int32_t* __restrict__ chunkcnt) {
  sah_pdl_entry_early();
  const int lane = threadIdx.x & 31;
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t g = wid / p.nchunks, c = wid - g * p.nchunks;
  if (g >= p.groups) return;  // surplus warps of the last block
  const int64_t w = c * PLAN_CHUNK_WORDS + lane;
  uint32_t u = 0u;
  if (w < p.Wv) {
    for (int r = 0; r < p.R; ++r) {
      int64_t row = plan_member_row(p, g, r);
      if (row >= 0) {
        u |= bits[row * p.W + w];
        if (ubits != nullptr) u |= ubits[row * p.W + w];  // a second set joined with the first
      }
    }
    u = plan_word(p, u, w);
  }
  int cnt = __popc(u);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0) chunkcnt[g * p.nchunks + c] = cnt;
}

// Short rows (W <= 1024 words, i.e. up to 32768 keys): PLAN_FUSED_THREADS bitmap words per CTA,
// one per thread, up to four CTAs per group.  A CTA first counts the union bits of the words in
// front of its own (a few loads per thread from a bitmap that is cache resident), then a single
// ordered block scan places every word's entries; no second kernel and no chunk counters.
#define PLAN_FUSED_THREADS 256

template <typename T, int RMAX>
__global__ void __launch_bounds__(PLAN_FUSED_THREADS)
attn_plan_fused_kernel(const uint32_t* __restrict__ bits, const T* __restrict__ data,
                       const int32_t* __restrict__ wpre, const int64_t* __restrict__ ptr,
                       PlanGeom p, int32_t* __restrict__ ucols, uint16_t* __restrict__ umemb,
                       float* __restrict__ uw, int32_t* __restrict__ ucount) {
  sah_pdl_entry_early();
  __shared__ int scan[33];
  __shared__ int64_t rows_sm[RMAX];
  const int64_t g = blockIdx.x;
  const int64_t w0 = (int64_t)blockIdx.y * PLAN_FUSED_THREADS;   // first word of this CTA
  const int64_t w = w0 + threadIdx.x;
  if (threadIdx.x < RMAX) rows_sm[threadIdx.x] = (threadIdx.x < p.R) ? plan_member_row(p, g, threadIdx.x) : -1;
  __syncthreads();
  uint32_t words[RMAX];
  int64_t rows[RMAX];
  int64_t dbase[RMAX];  // CSR position of the first entry of this row's word
  uint32_t u = 0u;
  int ahead = 0;        // union bits in this thread's share of the words before w0
#pragma unroll
  for (int r = 0; r < RMAX; ++r) rows[r] = rows_sm[r];
  for (int64_t wa = threadIdx.x; wa < w0; wa += PLAN_FUSED_THREADS) {
    uint32_t ua = 0u;
#pragma unroll
    for (int r = 0; r < RMAX; ++r)
      if (rows[r] >= 0) ua |= bits[rows[r] * p.W + wa];
    ahead += __popc(ua);
  }
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    words[r] = 0u;
    dbase[r] = 0;
    if (w < p.Wv && rows[r] >= 0) {
      // wpre counts every set bit of the caller's words; bits past S are dropped after
      // the CSR offsets were taken from the unmasked prefix (they can only sit last)
      words[r] = plan_word(p, bits[rows[r] * p.W + w], w);
      if (uw != nullptr && words[r]) dbase[r] = ptr[rows[r]] + wpre[rows[r] * p.W + w];
    }
    u |= words[r];
  }
  int base = 0;
  if (w0 > 0) {
    int dummy = sah_block_excl_scan<int>(ahead, scan, &base);
    (void)dummy;
  }
  int total;
  const int before = sah_block_excl_scan<int>(__popc(u), scan, &total);
  int64_t pos = (int64_t)g * p.S + base + before;
  uint32_t m = u;
  while (m) {
    const int b = __ffs(m) - 1;
    m &= m - 1;
    unsigned int memb = 0u;
#pragma unroll
    for (int r = 0; r < RMAX; ++r) memb |= ((words[r] >> b) & 1u) << r;
    ucols[pos] = (int32_t)(w * 32 + b);
    umemb[pos] = (uint16_t)memb;
    if (uw != nullptr) {
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        if (r < p.R) {
          float wv = 0.f;
          if ((memb >> r) & 1u) {
            const int64_t dp = dbase[r] + __popc(words[r] & ((1u << b) - 1u));
            wv = sah_inv_weight<T>(sah_to_float<T>(data[dp]));
          }
          uw[pos * p.R + r] = wv;
        }
      }
    }
    ++pos;
  }
  if (threadIdx.x == 0 && blockIdx.y == gridDim.y - 1) ucount[g] = base + total;
}

// Long rows: one warp per (group, chunk of 32 bitmap words).  Lane j owns word j of the chunk
// (its rows' words, CSR offsets and the count of columns in the words before it go to shared
// memory); then the warp walks the 32 words and lane i takes column i of each, so that the
// entries of a word are written side by side: every store of the list is coalesced.
// LSH: union list for a MagicPig mask whose weights the attention kernel evaluates itself
// (at most 4 mask rows per group).  `bits` are the LSH matches, `ubits` (may be NULL) the
// unit-weight part of the mask; the active set is their union.  Per union entry: the column,
// membership in the low byte and "weight is 1" flags in the high byte of umemb, and in `uw`
// ([groups][S]) the key's constant of the cosine, 1 / (M * |transformed key|).
#define PLAN_EMIT_WARPS 4

template <typename T, int RMAX, bool LSH>
__global__ void __launch_bounds__(PLAN_EMIT_WARPS * 32)
attn_plan_emit_kernel(const uint32_t* __restrict__ bits, const uint32_t* __restrict__ ubits,
                      const T* __restrict__ data, const int32_t* __restrict__ wpre,
                      const int64_t* __restrict__ ptr, const float* __restrict__ dens, int64_t dens_cap,
                      const unsigned int* __restrict__ max_bits, PlanGeom p,
                      const int32_t* __restrict__ chunkcnt, int32_t* __restrict__ ucols,
                      uint16_t* __restrict__ umemb, float* __restrict__ uw,
                      int32_t* __restrict__ ucount) {
  sah_pdl_entry();
  __shared__ uint32_t words_sm[PLAN_EMIT_WARPS][RMAX][32];
  __shared__ uint32_t units_sm[PLAN_EMIT_WARPS][LSH ? RMAX : 1][32];
  __shared__ int64_t dbase_sm[PLAN_EMIT_WARPS][RMAX][32];
  __shared__ uint32_t union_sm[PLAN_EMIT_WARPS][32];
  __shared__ int before_sm[PLAN_EMIT_WARPS][32];
  const int lane = threadIdx.x & 31, wl = threadIdx.x >> 5;
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t g = wid / p.nchunks, c = wid - g * p.nchunks;
  if (g >= p.groups) return;  // surplus warps of the last block (whole warps)
  // columns selected in earlier chunks of this group
  int base = 0;
  for (int64_t cc = lane; cc < c; cc += 32) base += chunkcnt[g * p.nchunks + cc];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) base += __shfl_xor_sync(0xffffffffu, base, o);

  const int64_t w = c * PLAN_CHUNK_WORDS + lane;
  const bool weighted = !LSH && uw != nullptr;
  uint32_t u = 0u;
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    uint32_t wd = 0u, un = 0u;
    int64_t db = 0;
    if (r < p.R && w < p.Wv) {
      const int64_t row = plan_member_row(p, g, r);
      if (row >= 0) {
        wd = plan_word(p, bits[row * p.W + w], w);
        if (LSH && ubits != nullptr) {
          un = plan_word(p, ubits[row * p.W + w], w);
          wd |= un;
        }
        if (weighted && wd) db = ptr[row] + wpre[row * p.W + w];
      }
    }
    words_sm[wl][r][lane] = wd;
    if (LSH) units_sm[wl][r][lane] = un;
    if (weighted) dbase_sm[wl][r][lane] = db;
    u |= wd;
  }
  const int cnt = __popc(u);
  int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  union_sm[wl][lane] = u;
  before_sm[wl][lane] = incl - cnt;
  __syncwarp();

  const int64_t list0 = (int64_t)g * p.S + base;
  const uint32_t lt = (1u << lane) - 1u;
  // LSH: the key constants of this lane's column in each of the 32 words, requested together
  // (one round trip to memory instead of one per word)
  float M = 0.f;
  float dcol[LSH ? 32 : 1];
  if constexpr (LSH) {
    M = __uint_as_float(*max_bits);
    const float* gd = dens + (g / p.nqb) * dens_cap;  // (batch, KV head) of the group
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int64_t col = (c * PLAN_CHUNK_WORDS + j) * 32 + lane;
      dcol[j] = col < p.S ? __ldg(gd + col) : 1.f;
    }
  }
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const uint32_t uj = union_sm[wl][j];
    if (uj == 0u) continue;  // the same for every lane
    if (!((uj >> lane) & 1u)) continue;
    const int64_t pos = list0 + before_sm[wl][j] + __popc(uj & lt);
    const int64_t col = (c * PLAN_CHUNK_WORDS + j) * 32 + lane;
    unsigned int memb = 0u;
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      memb |= ((words_sm[wl][r][j] >> lane) & 1u) << r;
      if (LSH) memb |= ((units_sm[wl][r][j] >> lane) & 1u) << (8 + r);
    }
    ucols[pos] = (int32_t)col;
    umemb[pos] = (uint16_t)memb;
    if constexpr (LSH) {
      uw[pos] = __frcp_rn(__fmul_rn(M, dcol[j]));
    } else if (weighted) {
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        if (r < p.R) {
          float wv = 0.f;
          if ((memb >> r) & 1u) {
            const int64_t dp = dbase_sm[wl][r][j] + __popc(words_sm[wl][r][j] & lt);
            wv = sah_inv_weight<T>(sah_to_float<T>(data[dp]));
          }
          uw[pos * p.R + r] = wv;
        }
      }
    }
  }
  if (c == p.nchunks - 1) {
    int total = __shfl_sync(0xffffffffu, incl, 31);
    if (lane == 0) ucount[g] = base + total;
  }
}

// Geometry shared by the plan entry points.  The chunk counters are laid out by the key
// count (plan_chunks), not by the caller's row stride W, which may be padded further than
// the library's own bitmaps are; words past the last key are never read and the bits of the
// last word past S are ignored.
static int plan_geometry(int B, int Hq, int Hkv, int Sq, int64_t S, int64_t W,
                         const sah_attn_sizes* sizes, PlanGeom* out) {
  PlanGeom p;
  p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.G = Hq / Hkv;
  p.q_block = sizes->q_block;
  p.nqb = (Sq + p.q_block - 1) / p.q_block;
  p.R = sizes->rows_per_group;
  p.S = S; p.W = W;
  p.Wv = (S + 31) / 32;
  p.tail_mask = (S % 32) ? ((1u << (S % 32)) - 1u) : 0xffffffffu;
  p.nchunks = plan_chunks(S);
  p.groups = sizes->groups;
  SAH_REQUIRE(p.groups == (int64_t)B * Hkv * p.nqb && p.R == p.G * p.q_block && p.R <= AT_MAXR,
              "attn_plan: sizes do not match the extents");
  SAH_REQUIRE(sizes->ucount_bytes >= (2 * p.groups + p.groups * p.nchunks + 4) * (int64_t)sizeof(int32_t),
              "attn_plan: sizes were not made by sah_attn_query_sizes for this key count");
  *out = p;
  return SAH_OK;
}

extern "C" int sah_attn_plan(const uint32_t* bits, const void* data, const int32_t* wpre,
                             const int64_t* ptr, int dtype, int B, int Hq, int Hkv, int Sq,
                             int64_t S, int64_t W, const sah_attn_sizes* sizes, int32_t* ucols,
                             uint16_t* umemb, float* uw, int32_t* ucount, void* stream) {
  SAH_REQUIRE(bits && sizes && ucols && umemb && ucount, "attn_plan: null pointer");
  SAH_REQUIRE(data == nullptr || (wpre && ptr && uw), "attn_plan: data needs wpre, ptr and uw");
  SAH_REQUIRE(W * 32 >= S, "attn_plan: W too small");
  PlanGeom p;
  int rc0 = plan_geometry(B, Hq, Hkv, Sq, S, W, sizes, &p);
  if (rc0 != SAH_OK) return rc0;
  const int64_t groups = p.groups;
  int32_t* chunkcnt = ucount + groups;
  const int64_t warps = groups * p.nchunks;
  const int threads = 256;
  const int64_t blocks = sah_ceil_div(warps * 32, threads);
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_ATTN_PLAN, (cudaStream_t)stream);
  if (p.Wv <= 1024) {
    const dim3 fgrid((unsigned)groups, (unsigned)sah_ceil_div(p.Wv, PLAN_FUSED_THREADS));
    SAH_DISPATCH_DTYPE(dtype, T, {
      if (p.R <= 4)
        sah_launch_chain(attn_plan_fused_kernel<T, 4>, fgrid, PLAN_FUSED_THREADS, 0, st, bits, (const T*)data,
            wpre, ptr, p, ucols, umemb, data ? uw : nullptr, ucount);
      else
        sah_launch_chain(attn_plan_fused_kernel<T, AT_MAXR>, fgrid, PLAN_FUSED_THREADS, 0, st, bits,
            (const T*)data, wpre, ptr, p, ucols, umemb, data ? uw : nullptr, ucount);
    });
    SAH_LAUNCH_CHECK("attn_plan_fused");
    sah_prof_end(SAH_PROF_ATTN_PLAN, (cudaStream_t)stream);
    return SAH_OK;
  }
  sah_launch_chain(attn_plan_count_kernel, (unsigned)blocks, threads, 0, st, bits, nullptr, p, chunkcnt);
  SAH_LAUNCH_CHECK("attn_plan_count");
  const int64_t eblocks = sah_ceil_div(warps, PLAN_EMIT_WARPS);
  SAH_DISPATCH_DTYPE(dtype, T, {
    if (p.R <= 4)
      sah_launch_chain(attn_plan_emit_kernel<T, 4, false>, (unsigned)eblocks, PLAN_EMIT_WARPS * 32, 0, st,
          bits, nullptr, (const T*)data, wpre, ptr, nullptr, 0, nullptr, p, chunkcnt, ucols, umemb,
          data ? uw : nullptr, ucount);
    else
      sah_launch_chain(attn_plan_emit_kernel<T, AT_MAXR, false>, (unsigned)eblocks, PLAN_EMIT_WARPS * 32, 0,
          st, bits, nullptr, (const T*)data, wpre, ptr, nullptr, 0, nullptr, p, chunkcnt, ucols, umemb,
          data ? uw : nullptr, ucount);
  });
  SAH_LAUNCH_CHECK("attn_plan_emit");
  sah_prof_end(SAH_PROF_ATTN_PLAN, (cudaStream_t)stream);
  return SAH_OK;
}

extern "C" int sah_attn_plan_lsh(const uint32_t* bits, const uint32_t* unit_bits, const float* dens,
                                 int64_t dens_cap, const unsigned int* max_norm_bits, int B, int Hq,
                                 int Hkv, int Sq, int64_t S, int64_t W, const sah_attn_sizes* sizes,
                                 int32_t* ucols, uint16_t* umemb, float* uinv, int32_t* ucount,
                                 void* stream) {
  SAH_REQUIRE(bits && dens && max_norm_bits && sizes && ucols && umemb && uinv && ucount,
              "attn_plan_lsh: null pointer");
  SAH_REQUIRE(W * 32 >= S && dens_cap >= S, "attn_plan_lsh: W or the key-constant stride too small");
  PlanGeom p;
  int rc0 = plan_geometry(B, Hq, Hkv, Sq, S, W, sizes, &p);
  if (rc0 != SAH_OK) return rc0;
  if (p.R > 4)
    return sah_fail(SAH_ERR_UNSUPPORTED, "attn_plan_lsh: %d mask rows per KV group (<= 4)", p.R);
  SAH_REQUIRE(sizes->uw_bytes >= p.groups * S * (int64_t)sizeof(float),
              "attn_plan_lsh: sizes were not queried for in-kernel MagicPig weights");
  int32_t* chunkcnt = ucount + p.groups;
  const int64_t warps = p.groups * p.nchunks;
  const int threads = 256;
  const int64_t blocks = sah_ceil_div(warps * 32, threads);
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_ATTN_PLAN, st);
  sah_launch_chain(attn_plan_count_kernel, (unsigned)blocks, threads, 0, st, bits, unit_bits, p, chunkcnt);
  SAH_LAUNCH_CHECK("attn_plan_count");
  sah_launch_chain(attn_plan_emit_kernel<float, 4, true>, (unsigned)sah_ceil_div(warps, PLAN_EMIT_WARPS),
                   PLAN_EMIT_WARPS * 32, 0, st, bits, unit_bits, nullptr, nullptr, nullptr, dens, dens_cap,
                   max_norm_bits, p, chunkcnt, ucols, umemb, uinv, ucount);
  SAH_LAUNCH_CHECK("attn_plan_emit_lsh");
  sah_prof_end(SAH_PROF_ATTN_PLAN, st);
  return SAH_OK;
}

// ---------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------
__device__ __forceinline__ void at_cp_async16(void* smem_dst, const void* gmem_src) {
  unsigned int d = (unsigned int)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void at_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void at_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

struct AttnArgs {
  const void *q, *k, *v;
  int64_t qs_b, qs_h, qs_q, ks_b, ks_h, ks_s, vs_b, vs_h, vs_s;
  int Hq, Hkv, Sq, G, q_block, nqb, R, nsplit;
  int64_t S;
  float scaling;
  const void* bias;
  int64_t bias_s_b, bias_s_h, bias_s_q;
  const int32_t* ucols;
  const uint16_t* umemb;
  const float* uw;
  const int32_t* ucount;
  float* partial;
  // MagicPig weights evaluated inside the bf16 kernel (uw then holds one constant per entry)
  const __nv_bfloat16* qhat;  // [rows][D] centred unit queries
  const float* qmu;           // [rows] qhat . key mean
  const uint16_t* ptable;     // [65536] bf16 bits of the cosine -> bits of the weight 1 / (p + 1e-6)
  float* w_dump;              // optional [groups][S][R]: the weights used (tests)
  // TMA copy stage: K and V as 2-D [rows][D] tensors, row = b * rows_b + h * rows_h + key
  int64_t k_rows_b, k_rows_h, v_rows_b, v_rows_h;
  int k_rows_total, v_rows_total;
  int one_wave_tiles;  // tcgen05 kernel: tiles per CTA below which only half of the grid works
};

// Shared-memory rows are stored in 16-byte chunks; chunk c of tile row i sits
// at chunk slot (c ^ (i & 7)), which spreads the rows of a quarter warp over
// all banks for both the row-wise (QK) and the column-wise (PV) reads.
template <typename T, int D>
struct AttnCfg {
  static constexpr int ROWB = D * (int)sizeof(T);        // bytes per K or V row
  static constexpr int CPR = ROWB / 16;                  // 16-byte chunks per row
  static constexpr int EPC = 16 / (int)sizeof(T);        // elements per chunk
  static constexpr int TILE = (sizeof(T) == 2) ? 64 : 32;  // keys per pipeline stage
  static constexpr int PARTS = AT_THREADS / TILE;        // threads sharing one key in QK
  static constexpr int CPP = CPR / PARTS;                // chunks per part
  static constexpr int KPL = TILE / 32;                  // keys per lane in the softmax phase
  static constexpr int DPL = D / 32;                     // output dims per lane in PV
  static constexpr int STAGE_BYTES = 2 * TILE * ROWB;    // K tile + V tile
};

static const char* g_last_attn_kernel = "none";

#include "sah_attention_tc.cuh"
#include "sah_attention_umma.cuh"

template <typename T, int D, int NQUAD>
__global__ void __launch_bounds__(AT_THREADS)
masked_attention_kernel(AttnArgs a, int* __restrict__ tickets, const float* __restrict__ sinks,
                        T* __restrict__ out, float* __restrict__ part_out) {
  sah_pdl_entry();
  __shared__ int is_last_sm;
  using C = AttnCfg<T, D>;
  constexpr int RP = NQUAD * 4;  // padded row count
  extern __shared__ __align__(128) unsigned char at_smem[];
  unsigned char* stage_base = at_smem;
  float* q_sm = reinterpret_cast<float*>(at_smem + AT_STAGES * C::STAGE_BYTES);  // [RP][D]
  float* s_part = q_sm + RP * D;                       // [PARTS][TILE][RP]
  float* p_sm = s_part + C::PARTS * C::TILE * RP;      // [TILE][RP]
  float* m_sm = p_sm + C::TILE * RP;                   // [RP]
  float* l_sm = m_sm + RP;                             // [RP]
  float* alpha_sm = l_sm + RP;                         // [RP]
  int* cols_sm = reinterpret_cast<int*>(alpha_sm + RP);  // [STAGES][TILE]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x;
  const int64_t g = blockIdx.y;
  const int qb = (int)(g % a.nqb);
  const int64_t bk = g / a.nqb;
  const int kvh = (int)(bk % a.Hkv);
  const int64_t b = bk / a.Hkv;

  const T* kbase = reinterpret_cast<const T*>(a.k) + b * a.ks_b + kvh * a.ks_h;
  const T* vbase = reinterpret_cast<const T*>(a.v) + b * a.vs_b + kvh * a.vs_h;
  const int32_t* gcols = a.ucols + g * a.S;
  const uint16_t* gmemb = a.umemb + g * a.S;
  const float* guw = a.uw ? a.uw + g * a.S * a.R : nullptr;

  // this CTA's slice of the group's union list
  const int U = a.ucount[g];
  int per = (U + a.nsplit - 1) / a.nsplit;
  per = ((per + C::TILE - 1) / C::TILE) * C::TILE;
  int start = split * per;
  if (start > U) start = U;
  int end = start + per;
  if (end > U) end = U;
  const int ntiles = (end - start + C::TILE - 1) / C::TILE;

  // stage queries (fp32), reset softmax state
  for (int idx = tid; idx < RP * D; idx += AT_THREADS) {
    int r = idx / D, d = idx - r * D;
    float val = 0.f;
    if (r < a.R) {
      int gi = r / a.q_block, qo = r - gi * a.q_block;
      int qi = qb * a.q_block + qo;
      if (qi < a.Sq) {
        int h = kvh * a.G + gi;
        val = sah_to_float<T>(
            reinterpret_cast<const T*>(a.q)[b * a.qs_b + (int64_t)h * a.qs_h + qi * a.qs_q + d]);
      }
    }
    q_sm[idx] = val;
  }
  if (tid < RP) {
    m_sm[tid] = -INFINITY;
    l_sm[tid] = 0.f;
    alpha_sm[tid] = 1.f;
  }

  float acc[NQUAD][4][C::DPL];
#pragma unroll
  for (int qd = 0; qd < NQUAD; ++qd)
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int e = 0; e < C::DPL; ++e) acc[qd][r][e] = 0.f;

  auto issue = [&](int t) {
    const int st = t % AT_STAGES;
    unsigned char* kst = stage_base + st * C::STAGE_BYTES;
    unsigned char* vst = kst + C::TILE * C::ROWB;
    const int t0 = start + t * C::TILE;
    for (int idx = tid; idx < C::TILE * C::CPR; idx += AT_THREADS) {
      const int i = idx / C::CPR, c = idx - i * C::CPR;
      const int u = t0 + i;
      if (u < end) {
        const int64_t col = gcols[u];
        const int slot = (c ^ (i & 7)) * 16;
        at_cp_async16(kst + i * C::ROWB + slot,
                      reinterpret_cast<const unsigned char*>(kbase + col * a.ks_s) + c * 16);
        at_cp_async16(vst + i * C::ROWB + slot,
                      reinterpret_cast<const unsigned char*>(vbase + col * a.vs_s) + c * 16);
      }
    }
    if (tid < C::TILE) cols_sm[st * C::TILE + tid] = (t0 + tid < end) ? gcols[t0 + tid] : -1;
  };

#pragma unroll
  for (int s = 0; s < AT_STAGES - 1; ++s) {
    if (s < ntiles) issue(s);
    at_cp_async_commit();
  }

  for (int t = 0; t < ntiles; ++t) {
    if (t + AT_STAGES - 1 < ntiles) issue(t + AT_STAGES - 1);
    at_cp_async_commit();
    at_cp_async_wait<AT_STAGES - 1>();
    __syncthreads();

    const int st = t % AT_STAGES;
    const unsigned char* kst = stage_base + st * C::STAGE_BYTES;
    const unsigned char* vst = kst + C::TILE * C::ROWB;
    const int t0 = start + t * C::TILE;
    const int nvalid = (end - t0 < C::TILE) ? (end - t0) : C::TILE;

    // ---- phase A: partial dot products, thread = (key, part of D) ----
    {
      const int i = tid % C::TILE, part = tid / C::TILE;
      float sp[RP];
#pragma unroll
      for (int r = 0; r < RP; ++r) sp[r] = 0.f;
      if (i < nvalid) {
#pragma unroll
        for (int cc = 0; cc < C::CPP; ++cc) {
          const int c = part * C::CPP + cc;
          float kf[C::EPC];
          const unsigned char* src = kst + i * C::ROWB + ((c ^ (i & 7)) * 16);
          if (sizeof(T) == 2) {
            uint4 raw = *reinterpret_cast<const uint4*>(src);
            float tmp[8];
            sah_unpack8(raw, tmp);
#pragma unroll
            for (int e = 0; e < C::EPC; ++e) kf[e] = tmp[e];
          } else {
            float4 raw = *reinterpret_cast<const float4*>(src);
            kf[0] = raw.x; kf[1] = raw.y; kf[2] = raw.z; kf[3] = raw.w;
          }
#pragma unroll
          for (int r = 0; r < RP; ++r) {
            const float* qp = q_sm + r * D + c * C::EPC;
#pragma unroll
            for (int e = 0; e < C::EPC; e += 4) {
              const float4 qv = *reinterpret_cast<const float4*>(qp + e);
              sp[r] = fmaf(qv.x, kf[e + 0], sp[r]);
              sp[r] = fmaf(qv.y, kf[e + 1], sp[r]);
              sp[r] = fmaf(qv.z, kf[e + 2], sp[r]);
              sp[r] = fmaf(qv.w, kf[e + 3], sp[r]);
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RP; ++r) s_part[(part * C::TILE + i) * RP + r] = sp[r];
    }
    __syncthreads();

    // ---- phase B: logits, running max, weights; warp w owns rows w, w+4, ... ----
    for (int r = warp; r < RP; r += AT_THREADS / 32) {
      float sv[C::KPL], wv[C::KPL];
      float tmax = -INFINITY;
      const bool row_ok = r < a.R;
      int h = 0, qi = 0;
      if (row_ok) {
        int gi = r / a.q_block, qo = r - gi * a.q_block;
        qi = qb * a.q_block + qo;
        h = kvh * a.G + gi;
      }
#pragma unroll
      for (int kk = 0; kk < C::KPL; ++kk) {
        const int i = lane + kk * 32;
        sv[kk] = -INFINITY;
        wv[kk] = 0.f;
        if (row_ok && i < nvalid) {
          const int u = t0 + i;
          const unsigned int memb = gmemb[u];
          if ((memb >> r) & 1u) {
            float s = 0.f;
#pragma unroll
            for (int pp = 0; pp < C::PARTS; ++pp) s += s_part[(pp * C::TILE + i) * RP + r];
            s *= a.scaling;
            if (a.bias != nullptr) {
              const int64_t col = cols_sm[st * C::TILE + i];
              s += sah_to_float<T>(reinterpret_cast<const T*>(
                  a.bias)[b * a.bias_s_b + h * a.bias_s_h + qi * a.bias_s_q + col]);
            }
            sv[kk] = s;
            wv[kk] = guw ? guw[(int64_t)u * a.R + r] : 1.f;
            tmax = fmaxf(tmax, s);
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
      const float m_old = m_sm[r];
      const float m_new = fmaxf(m_old, tmax);
      float psum = 0.f;
#pragma unroll
      for (int kk = 0; kk < C::KPL; ++kk) {
        const int i = lane + kk * 32;
        float pv = 0.f;
        if (sv[kk] != -INFINITY) pv = expf(sv[kk] - m_new) * wv[kk];
        p_sm[i * RP + r] = pv;
        psum += pv;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
      if (lane == 0) {
        const float alpha = (m_new == -INFINITY) ? 1.f : expf(m_old - m_new);
        alpha_sm[r] = alpha;
        l_sm[r] = l_sm[r] * alpha + psum;
        m_sm[r] = m_new;
      }
    }
    __syncthreads();

    // ---- phase C: acc = acc * alpha + p . V; thread = (dims of lane, keys of warp) ----
    {
#pragma unroll
      for (int qd = 0; qd < NQUAD; ++qd)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float al = alpha_sm[qd * 4 + r];
#pragma unroll
          for (int e = 0; e < C::DPL; ++e) acc[qd][r][e] *= al;
        }
      const int d0 = lane * C::DPL;                 // first output dim of this lane
      const int c = (d0 * (int)sizeof(T)) / 16;     // chunk holding it
      const int off = (d0 * (int)sizeof(T)) % 16;   // byte offset inside the chunk
      for (int i = warp; i < nvalid; i += AT_THREADS / 32) {
        const unsigned char* src = vst + i * C::ROWB + ((c ^ (i & 7)) * 16) + off;
        float vf[C::DPL];
        if (sizeof(T) == 2) {
          if (C::DPL == 4) {
            uint2 raw = *reinterpret_cast<const uint2*>(src);
            vf[0] = __uint_as_float(raw.x << 16);
            vf[1] = __uint_as_float(raw.x & 0xffff0000u);
            vf[2] = __uint_as_float(raw.y << 16);
            vf[3] = __uint_as_float(raw.y & 0xffff0000u);
          } else {
            unsigned int raw = *reinterpret_cast<const unsigned int*>(src);
            vf[0] = __uint_as_float(raw << 16);
            vf[1] = __uint_as_float(raw & 0xffff0000u);
          }
        } else {
          if (C::DPL == 4) {
            float4 raw = *reinterpret_cast<const float4*>(src);
            vf[0] = raw.x; vf[1] = raw.y; vf[2] = raw.z; vf[3] = raw.w;
          } else {
            float2 raw = *reinterpret_cast<const float2*>(src);
            vf[0] = raw.x; vf[1] = raw.y;
          }
        }
#pragma unroll
        for (int qd = 0; qd < NQUAD; ++qd) {
          const float4 pv = *reinterpret_cast<const float4*>(p_sm + i * RP + qd * 4);
#pragma unroll
          for (int e = 0; e < C::DPL; ++e) {
            acc[qd][0][e] = fmaf(pv.x, vf[e], acc[qd][0][e]);
            acc[qd][1][e] = fmaf(pv.y, vf[e], acc[qd][1][e]);
            acc[qd][2][e] = fmaf(pv.z, vf[e], acc[qd][2][e]);
            acc[qd][3][e] = fmaf(pv.w, vf[e], acc[qd][3][e]);
          }
        }
      }
    }
    __syncthreads();
  }
  at_cp_async_wait<0>();
  __syncthreads();

  // ---- combine the four warps' accumulators and write the partial ----
  float* red = reinterpret_cast<float*>(stage_base);  // [4][RP][D]
#pragma unroll
  for (int qd = 0; qd < NQUAD; ++qd)
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int e = 0; e < C::DPL; ++e)
        red[(warp * RP + qd * 4 + r) * D + lane * C::DPL + e] = acc[qd][r][e];
  __syncthreads();
  float* pout = a.partial + ((int64_t)g * a.nsplit + split) * a.R * (D + 2);
  for (int idx = tid; idx < a.R * D; idx += AT_THREADS) {
    const int r = idx / D, d = idx - r * D;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < AT_THREADS / 32; ++w) s += red[(w * RP + r) * D + d];
    pout[r * (D + 2) + d] = s;
  }
  if (tid < a.R) {
    pout[tid * (D + 2) + D] = m_sm[tid];
    pout[tid * (D + 2) + D + 1] = l_sm[tid];
  }
  // the last CTA of the group to get here merges the splits and writes the output rows (every
  // CTA of the grid writes a partial, an empty one included)
  __syncthreads();  // the reduction buffer is read no more: it becomes the merge scratch
  atm_finish_group<D, AT_THREADS, T>(a, g, a.nsplit, stage_base, &is_last_sm, tickets, sinks, out, part_out);
}

template <typename T, int D>
static int launch_attention(const AttnArgs& a, int groups, int* tickets, const float* sinks, void* out,
                            float* part_out, cudaStream_t st) {
  using C = AttnCfg<T, D>;
  const int nquad = (a.R + 3) / 4;
  const int RP = nquad * 4;
  size_t smem = (size_t)AT_STAGES * C::STAGE_BYTES +
                sizeof(float) * ((size_t)RP * D + (size_t)C::PARTS * C::TILE * RP +
                                 (size_t)C::TILE * RP + 3 * RP) +
                sizeof(int) * AT_STAGES * C::TILE;
  size_t red = sizeof(float) * 4 * RP * D;
  if (red > (size_t)AT_STAGES * C::STAGE_BYTES ||
      sizeof(float) * (16 * (size_t)a.nsplit + 32) > (size_t)AT_STAGES * C::STAGE_BYTES)
    return sah_fail(SAH_ERR_UNSUPPORTED, "attention: reduction buffer does not fit");
  dim3 grid((unsigned)a.nsplit, (unsigned)groups);
#define SAH_AT_LAUNCH(NQ)                                                                        \
  {                                                                                              \
    cudaError_t e = cudaFuncSetAttribute(masked_attention_kernel<T, D, NQ>,                      \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "attention attr: %s", cudaGetErrorString(e)); \
    sah_launch_chain(masked_attention_kernel<T, D, NQ>, grid, AT_THREADS, smem, st, a, tickets, sinks, \
        (T*)out, part_out); \
  }
  switch (nquad) {
    case 1: SAH_AT_LAUNCH(1) break;
    case 2: SAH_AT_LAUNCH(2) break;
    case 3: SAH_AT_LAUNCH(3) break;
    default: SAH_AT_LAUNCH(4) break;
  }
#undef SAH_AT_LAUNCH
  return SAH_OK;
}

struct AttnLsh {
  const void* qhat;
  const float* qmu;
  const uint16_t* ptable;
  float* w_dump;
};

static int masked_attention_impl(const void* q, const void* k, const void* v, int dtype,
                                 int64_t qs_b, int64_t qs_h, int64_t qs_q, int64_t ks_b,
                                 int64_t ks_h, int64_t ks_s, int64_t vs_b, int64_t vs_h,
                                 int64_t vs_s, int B, int Hq, int Hkv, int Sq, int64_t S, int D,
                                 float scaling, const void* bias, int64_t bias_s_b,
                                 int64_t bias_s_h, int64_t bias_s_q, const float* sinks,
                                 const sah_attn_sizes* sizes, const int32_t* ucols,
                                 const uint16_t* umemb, const float* uw, const int32_t* ucount,
                                 float* partial, void* out, float* part_out,
                                 const AttnLsh* lsh, void* stream) {
  SAH_REQUIRE(q && k && v && sizes && ucols && umemb && ucount && partial && out,
              "masked_attention: null pointer");
  SAH_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Sq > 0 && S > 0,
              "masked_attention: bad extents");
  if (D != 64 && D != 128)
    return sah_fail(SAH_ERR_UNSUPPORTED, "masked_attention: head dim %d (64 or 128 supported)", D);
  const int64_t esz = (dtype == SAH_BF16) ? 2 : 4;
  SAH_REQUIRE((ks_s * esz) % 16 == 0 && (ks_h * esz) % 16 == 0 && (ks_b * esz) % 16 == 0 &&
                  (vs_s * esz) % 16 == 0 && (vs_h * esz) % 16 == 0 && (vs_b * esz) % 16 == 0 &&
                  (uintptr_t)k % 16 == 0 && (uintptr_t)v % 16 == 0,
              "masked_attention: K and V rows must be 16-byte aligned");
  AttnArgs a;
  a.q = q; a.k = k; a.v = v;
  a.qs_b = qs_b; a.qs_h = qs_h; a.qs_q = qs_q;
  a.ks_b = ks_b; a.ks_h = ks_h; a.ks_s = ks_s;
  a.vs_b = vs_b; a.vs_h = vs_h; a.vs_s = vs_s;
  a.Hq = Hq; a.Hkv = Hkv; a.Sq = Sq; a.G = Hq / Hkv;
  a.q_block = sizes->q_block;
  a.nqb = (Sq + a.q_block - 1) / a.q_block;
  a.R = sizes->rows_per_group;
  a.nsplit = sizes->nsplit;
  a.S = S; a.scaling = scaling;
  a.bias = bias; a.bias_s_b = bias_s_b; a.bias_s_h = bias_s_h; a.bias_s_q = bias_s_q;
  a.ucols = ucols; a.umemb = umemb; a.uw = uw; a.ucount = ucount; a.partial = partial;
  a.qhat = lsh ? reinterpret_cast<const __nv_bfloat16*>(lsh->qhat) : nullptr;
  a.qmu = lsh ? lsh->qmu : nullptr;
  a.ptable = lsh ? lsh->ptable : nullptr;
  a.w_dump = lsh ? lsh->w_dump : nullptr;
  a.k_rows_b = a.k_rows_h = a.v_rows_b = a.v_rows_h = 0;
  a.k_rows_total = a.v_rows_total = 0;
  a.one_wave_tiles = 0;
  const int groups = sizes->groups;
  SAH_REQUIRE((int64_t)groups == (int64_t)B * Hkv * a.nqb && a.R == a.G * a.q_block &&
                  a.R <= AT_MAXR && a.nsplit >= 1,
              "masked_attention: sizes do not match the extents");
  cudaStream_t st = (cudaStream_t)stream;
  sah_prof_begin(SAH_PROF_ATTENTION, (cudaStream_t)stream);
  int rc = SAH_OK;
  if (dtype == SAH_BF16) {
    // tensor-core path; the split merge is fused into the kernel (ticket per group)
    int* tickets = const_cast<int*>(ucount) + groups + (int64_t)groups * plan_chunks(S);
    int* errflag = tickets + groups;  // set when a bounded wait inside the kernel ran out
    // long lists: keys as the M dimension of tcgen05 tiles; otherwise the mma.sync kernel
    const int umma = aum_requested();
    if (D == 128 && (umma == 1 || (umma < 0 && aum_default(lsh != nullptr, S, groups)))) {
      bool launched = false;
      rc = launch_attention_umma(a, B, groups, tickets, errflag, sinks, out, part_out, lsh != nullptr, st,
                                 &launched);
      if (rc != SAH_OK) return rc;
      if (launched) {
        g_last_attn_kernel = "masked_attention_umma_kernel";
        SAH_LAUNCH_CHECK("masked_attention_umma");
        sah_prof_end(SAH_PROF_ATTENTION, (cudaStream_t)stream);
        return SAH_OK;
      }
    }
    rc = (D == 128)
             ? launch_attention_mma<128>(a, B, groups, tickets, errflag, sinks, out, part_out, lsh != nullptr, st)
             : launch_attention_mma<64>(a, B, groups, tickets, errflag, sinks, out, part_out, lsh != nullptr, st);
    if (rc != SAH_OK) return rc;
    g_last_attn_kernel = "masked_attention_mma_kernel";
    SAH_LAUNCH_CHECK("masked_attention_mma");
    sah_prof_end(SAH_PROF_ATTENTION, (cudaStream_t)stream);
    return SAH_OK;
  }
  if (dtype != SAH_F32) return sah_fail(SAH_ERR_INVALID, "masked_attention: unknown dtype %d", dtype);
  if (lsh != nullptr)
    return sah_fail(SAH_ERR_UNSUPPORTED, "masked_attention_lsh: bfloat16 only");
  // the split merge is fused into the kernel here too (ticket per group, as in bfloat16)
  int* tickets32 = const_cast<int*>(ucount) + groups + (int64_t)groups * plan_chunks(S);
  rc = (D == 128) ? launch_attention<float, 128>(a, groups, tickets32, sinks, out, part_out, st)
                  : launch_attention<float, 64>(a, groups, tickets32, sinks, out, part_out, st);
  if (rc != SAH_OK) return rc;
  g_last_attn_kernel = "masked_attention_kernel";
  SAH_LAUNCH_CHECK("masked_attention");
  sah_prof_end(SAH_PROF_ATTENTION, (cudaStream_t)stream);
  return SAH_OK;
}

#ifdef AUM_PROF
extern "C" int sah_debug_umma_prof(long long* host_out, int reset) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(host_out, aum_prof, sizeof(long long) * 32);
  if (reset) {
    long long z[32] = {};
    cudaMemcpyToSymbol(aum_prof, z, sizeof(z));
  }
  return 0;
}
#endif

extern "C" const char* sah_attn_last_kernel(void) { return g_last_attn_kernel; }

// Self-test of the bounded wait that every mbarrier wait of the tcgen05 kernels goes through:
// one CTA waits, for at most `limit_us`, on a barrier that nothing will ever arrive at.  The
// wait runs out, the error word is set, the kernel returns normally and the context stays
// usable -- the behaviour the kernels rely on when a producer or a peer does not show up.
__global__ void wait_selftest_kernel(unsigned long long limit_ns, int* __restrict__ errflag,
                                     unsigned long long* __restrict__ waited_ns) {
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ int abort_word;
  const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&bar_storage);
  if (threadIdx.x == 0) {
    atm_mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    abort_word = 0;
  }
  __syncthreads();
  const unsigned long long t0 = aum_now_ns();
  const bool ok = aum_wait_warp(bar, 0u, &abort_word, errflag, 0u, limit_ns);
  if (threadIdx.x == 0) *waited_ns = ok ? 0ull : aum_now_ns() - t0;
}

extern "C" int sah_wait_selftest(int limit_us, int* errflag, unsigned long long* waited_ns, void* stream) {
  SAH_REQUIRE(errflag && waited_ns, "wait_selftest: null pointer");
  SAH_REQUIRE(limit_us > 0 && limit_us <= 100000, "wait_selftest: limit of 1 us .. 100 ms");
  wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>((unsigned long long)limit_us * 1000ull, errflag, waited_ns);
  SAH_LAUNCH_CHECK("wait_selftest");
  return SAH_OK;
}

extern "C" int sah_attn_select_kernel(int which) {
  if (which < -1 || which > 1) return -2;
  const int prev = aum_setting;
  aum_setting = which;
  return prev;
}

extern "C" int sah_masked_attention(const void* q, const void* k, const void* v, int dtype,
                                    int64_t qs_b, int64_t qs_h, int64_t qs_q, int64_t ks_b,
                                    int64_t ks_h, int64_t ks_s, int64_t vs_b, int64_t vs_h,
                                    int64_t vs_s, int B, int Hq, int Hkv, int Sq, int64_t S, int D,
                                    float scaling, const void* bias, int64_t bias_s_b,
                                    int64_t bias_s_h, int64_t bias_s_q, const float* sinks,
                                    const sah_attn_sizes* sizes, const int32_t* ucols,
                                    const uint16_t* umemb, const float* uw, const int32_t* ucount,
                                    float* partial, void* out, float* part_out,
                                    void* stream) {
  return masked_attention_impl(q, k, v, dtype, qs_b, qs_h, qs_q, ks_b, ks_h, ks_s, vs_b, vs_h, vs_s,
                               B, Hq, Hkv, Sq, S, D, scaling, bias, bias_s_b, bias_s_h, bias_s_q,
                               sinks, sizes, ucols, umemb, uw, ucount, partial, out, part_out,
                               nullptr, stream);
}

extern "C" int sah_masked_attention_lsh(const void* q, const void* k, const void* v, int64_t qs_b,
                                        int64_t qs_h, int64_t qs_q, int64_t ks_b, int64_t ks_h,
                                        int64_t ks_s, int64_t vs_b, int64_t vs_h, int64_t vs_s,
                                        int B, int Hq, int Hkv, int Sq, int64_t S, int D,
                                        float scaling, const void* bias, int64_t bias_s_b,
                                        int64_t bias_s_h, int64_t bias_s_q, const float* sinks,
                                        const sah_attn_sizes* sizes, const int32_t* ucols,
                                        const uint16_t* umemb, const float* uinv,
                                        const int32_t* ucount, float* partial, const void* qhat,
                                        const float* qmu, const uint16_t* weight_table, void* out,
                                        float* part_out, float* w_dump,
                                        void* stream) {
  SAH_REQUIRE(uinv && qhat && qmu && weight_table, "masked_attention_lsh: null pointer");
  SAH_REQUIRE((uintptr_t)qhat % 16 == 0, "masked_attention_lsh: qhat must be 16-byte aligned");
  AttnLsh lsh = {qhat, qmu, weight_table, w_dump};
  return masked_attention_impl(q, k, v, SAH_BF16, qs_b, qs_h, qs_q, ks_b, ks_h, ks_s, vs_b, vs_h,
                               vs_s, B, Hq, Hkv, Sq, S, D, scaling, bias, bias_s_b, bias_s_h,
                               bias_s_q, sinks, sizes, ucols, umemb, uinv, ucount, partial, out,
                               part_out, &lsh, stream);
}

extern "C" int sah_attn_gather_probe(const void* k, const void* v, int64_t ks_b, int64_t ks_h,
                                     int64_t ks_s, int64_t vs_b, int64_t vs_h, int64_t vs_s, int B,
                                     int Hkv, int Sq, int64_t S, int D, const sah_attn_sizes* sizes,
                                     const int32_t* ucols, const int32_t* ucount,
                                     unsigned int* sink, void* stream) {
  SAH_REQUIRE(k && v && sizes && ucols && ucount && sink, "attn_gather_probe: null pointer");
  if (D != 64 && D != 128)
    return sah_fail(SAH_ERR_UNSUPPORTED, "attn_gather_probe: head dim %d (64 or 128 supported)", D);
  SAH_REQUIRE((ks_s * 2) % 16 == 0 && (vs_s * 2) % 16 == 0 && (uintptr_t)k % 16 == 0 &&
                  (uintptr_t)v % 16 == 0, "attn_gather_probe: K and V rows must be 16-byte aligned");
  AttnArgs a = {};
  a.k = k; a.v = v;
  a.ks_b = ks_b; a.ks_h = ks_h; a.ks_s = ks_s;
  a.vs_b = vs_b; a.vs_h = vs_h; a.vs_s = vs_s;
  a.Hkv = Hkv; a.Sq = Sq;
  a.q_block = sizes->q_block;
  a.nqb = (Sq + a.q_block - 1) / a.q_block;
  a.nsplit = sizes->nsplit;
  a.S = S;
  a.ucols = ucols; a.ucount = ucount;
  SAH_REQUIRE((int64_t)sizes->groups == (int64_t)B * Hkv * a.nqb,
              "attn_gather_probe: sizes do not match the extents");
  dim3 grid((unsigned)a.nsplit, (unsigned)sizes->groups);
  cudaStream_t st = (cudaStream_t)stream;
  static bool allowed[2][64] = {};
  cudaError_t e;
  sah_prof_begin(SAH_PROF_OTHER, st);
  if (D == 128) {
    e = atm_allow_smem(attention_gather_probe_kernel<128>, AtmCfg<128>::SMEM, allowed[0]);
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "gather probe attr: %s", cudaGetErrorString(e));
    attention_gather_probe_kernel<128><<<grid, ATM_THREADS, AtmCfg<128>::SMEM, st>>>(a, sink);
  } else {
    e = atm_allow_smem(attention_gather_probe_kernel<64>, AtmCfg<64>::SMEM, allowed[1]);
    if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "gather probe attr: %s", cudaGetErrorString(e));
    attention_gather_probe_kernel<64><<<grid, ATM_THREADS, AtmCfg<64>::SMEM, st>>>(a, sink);
  }
  SAH_LAUNCH_CHECK("attn_gather_probe");
  sah_prof_end(SAH_PROF_OTHER, st);
  return SAH_OK;
}

// Merge partial results computed on different sequence shards: parts [n_parts][rows][D+2]
// holds, per row, the unnormalised accumulator, the running maximum and the denominator.
template <typename T>
__global__ void attn_merge_parts_kernel(const float* __restrict__ parts, int n_parts, int64_t rows,
                                        int Hq, int Sq, int D, const float* __restrict__ sinks,
                                        T* __restrict__ out) {
  sah_pdl_entry_early();
  const int64_t row = blockIdx.x;
  const int qi = (int)(row % Sq);
  const int64_t bh = row / Sq;
  const int h = (int)(bh % Hq);
  const int64_t b = bh / Hq;
  const int64_t ld = D + 2, pstride = rows * ld;
  const float* pr = parts + row * ld;
  float M = -INFINITY;
  for (int p = 0; p < n_parts; ++p) M = fmaxf(M, pr[p * pstride + D]);
  float L = 0.f;
  for (int p = 0; p < n_parts; ++p) {
    const float mp = pr[p * pstride + D];
    if (mp != -INFINITY) L += pr[p * pstride + D + 1] * expf(mp - M);
  }
  float Mx = M, sink_term = 0.f;
  if (sinks != nullptr) {
    const float sk = sinks[h];
    Mx = fmaxf(M, sk);
    sink_term = expf(sk - Mx);
  }
  const float resc = (M == -INFINITY) ? 0.f : expf(M - Mx);
  const float den = L * resc + sink_term;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int p = 0; p < n_parts; ++p) {
      const float mp = pr[p * pstride + D];
      if (mp != -INFINITY) a += pr[p * pstride + d] * expf(mp - M);
    }
    out[((b * Sq + qi) * Hq + h) * D + d] = sah_from_float<T>(a * resc / den);
  }
}

extern "C" int sah_attn_merge_parts(const float* parts, int n_parts, int B, int Hq, int Sq, int D,
                                    const float* sinks, int dtype, void* out, void* stream) {
  SAH_REQUIRE(parts && out, "attn_merge_parts: null pointer");
  SAH_REQUIRE(n_parts > 0 && B > 0 && Hq > 0 && Sq > 0 && D > 0, "attn_merge_parts: bad extents");
  const int64_t rows = (int64_t)B * Hq * Sq;
  int threads = D < 32 ? 32 : (D > 256 ? 256 : D);
  SAH_DISPATCH_DTYPE(dtype, T, {
    sah_launch_chain(attn_merge_parts_kernel<T>, (unsigned)rows, threads, 0, (cudaStream_t)stream, parts,
        n_parts, rows, Hq, Sq, D, sinks, (T*)out);
  });
  SAH_LAUNCH_CHECK("attn_merge_parts");
  return SAH_OK;
}

// ---------------------------------------------------------------------------
// Exchange + merge of sequence-shard partials over peer memory (NVLink): one kernel per rank
// per step instead of an all-gather and a merge kernel.
//
// Every rank owns a receive buffer [2 parities][world][rows][D+2] floats and a flag array
// [world][rows] ints in memory that its peers have mapped.  One CTA per row:
//   1. stores its rank's partial of the row into every rank's receive buffer (its own too),
//      slot [step parity][my rank][row], with plain stores to the peer addresses,
//   2. fences at system scope and stores the step number into every rank's flag [my rank][row],
//   3. waits until the flags [src][row] of its own array have reached the step number -- a
//      bounded wait (about a second): when it runs out the error word is set and the row is
//      merged from what is there, so that the kernel always returns,
//   4. merges the world's partials of the row exactly as attn_merge_parts_kernel does.
// The step number of a row lives in device memory (`steps[row]`, advanced by the row's CTA),
// so a CUDA graph can replay the launch.  Two parities make the buffer safe: a rank can be at
// most one step ahead of a peer (step e + 1 cannot end before the peer has started it, i.e.
// finished step e), and a slot of parity e & 1 is next written at step e + 2.
// The kernels of different ranks wait on one another: they must run on different GPUs.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int sah_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void sah_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long sah_globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}

#define SAH_XCHG_MAX_WORLD 16

struct XchgPeers {
  float* buf[SAH_XCHG_MAX_WORLD];
  int* flag[SAH_XCHG_MAX_WORLD];
};

template <typename T>
__global__ void __launch_bounds__(256)
attn_exchange_merge_kernel(const float* __restrict__ part, XchgPeers peers, int rank, int world, int64_t rows,
                           int Hq, int Sq, int D, const float* __restrict__ sinks, int* __restrict__ steps,
                           int* __restrict__ errflag, T* __restrict__ out) {
  __shared__ float scale_sm[SAH_XCHG_MAX_WORLD];
  __shared__ float ml_sm[2];
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x;
  const int64_t ld = D + 2;
  const int step = steps[row] + 1;
  const int par = step & 1;
  // 1. this rank's partial of the row to every rank
  const float* src = part + row * ld;
  for (int i = tid; i < world * (int)ld; i += blockDim.x) {
    const int p = i / (int)ld, e = i - p * (int)ld;
    peers.buf[p][(((int64_t)par * world + rank) * rows + row) * ld + e] = src[e];
  }
  // 2. publish
  __threadfence_system();
  __syncthreads();
  if (tid < world) sah_st_release_sys(peers.flag[tid] + (int64_t)rank * rows + row, step);
  // 3. wait for every rank's partial of this row
  if (tid < world) {
    const int* f = peers.flag[rank] + (int64_t)tid * rows + row;
    const unsigned long long t0 = sah_globaltimer_ns();
    bool ok = false;
    for (long long spin = 0; spin < (1ll << 40); ++spin) {
      if (sah_ld_acquire_sys(f) - step >= 0) { ok = true; break; }
      if ((spin & 1023) == 1023 && sah_globaltimer_ns() - t0 > 1000000000ull) break;
    }
    if (!ok) atomicExch(errflag, 2);
  }
  __syncthreads();
  // 4. merge (reads bypass L1: the lines were written by other GPUs)
  const float* mine = peers.buf[rank] + ((int64_t)par * world * rows + row) * ld;
  const int64_t pstride = rows * ld;
  if (tid == 0) {
    float M = -INFINITY;
    for (int p = 0; p < world; ++p) M = fmaxf(M, __ldcv(mine + p * pstride + D));
    float L = 0.f;
    for (int p = 0; p < world; ++p) {
      const float mp = __ldcv(mine + p * pstride + D);
      const float sc = (mp == -INFINITY) ? 0.f : expf(mp - M);
      scale_sm[p] = sc;
      L += __ldcv(mine + p * pstride + D + 1) * sc;
    }
    ml_sm[0] = M;
    ml_sm[1] = L;
    steps[row] = step;
  }
  __syncthreads();
  const int qi = (int)(row % Sq);
  const int64_t bh = row / Sq;
  const int h = (int)(bh % Hq);
  const int64_t b = bh / Hq;
  const float M = ml_sm[0], L = ml_sm[1];
  float Mx = M, sink_term = 0.f;
  if (sinks != nullptr) {
    const float sk = sinks[h];
    Mx = fmaxf(M, sk);
    sink_term = expf(sk - Mx);
  }
  const float resc = (M == -INFINITY) ? 0.f : expf(M - Mx);
  const float den = L * resc + sink_term;
  for (int d = tid; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int p = 0; p < world; ++p) {
      const float sc = scale_sm[p];
      if (sc != 0.f) acc += __ldcv(mine + p * pstride + d) * sc;
    }
    out[((b * Sq + qi) * Hq + h) * D + d] = sah_from_float<T>(acc * resc / den);
  }
}

extern "C" int64_t sah_attn_exchange_bytes(int world, int B, int Hq, int Sq, int D) {
  if (world <= 0 || B <= 0 || Hq <= 0 || Sq <= 0 || D <= 0) return 0;
  return 2ll * world * B * Hq * Sq * (D + 2) * (int64_t)sizeof(float);
}

extern "C" int sah_attn_exchange_merge(const float* part, const void* const* peer_bufs,
                                       const void* const* peer_flags, int rank, int world, int B, int Hq,
                                       int Sq, int D, const float* sinks, int dtype, int* steps,
                                       int* errflag, void* out, void* stream) {
  SAH_REQUIRE(part && peer_bufs && peer_flags && steps && errflag && out, "attn_exchange_merge: null pointer");
  SAH_REQUIRE(world > 0 && world <= SAH_XCHG_MAX_WORLD && rank >= 0 && rank < world,
              "attn_exchange_merge: bad rank / world (at most 16 ranks)");
  SAH_REQUIRE(B > 0 && Hq > 0 && Sq > 0 && D > 0, "attn_exchange_merge: bad extents");
  XchgPeers peers;
  for (int p = 0; p < SAH_XCHG_MAX_WORLD; ++p) {
    peers.buf[p] = p < world ? reinterpret_cast<float*>(const_cast<void*>(peer_bufs[p])) : nullptr;
    peers.flag[p] = p < world ? reinterpret_cast<int*>(const_cast<void*>(peer_flags[p])) : nullptr;
    if (p < world) SAH_REQUIRE(peers.buf[p] && peers.flag[p], "attn_exchange_merge: null peer pointer");
  }
  const int64_t rows = (int64_t)B * Hq * Sq;
  int threads = D + 2 < 64 ? 64 : (D + 2 > 256 ? 256 : ((D + 2 + 31) / 32) * 32);
  SAH_DISPATCH_DTYPE(dtype, T, {
    attn_exchange_merge_kernel<T><<<(unsigned)rows, threads, 0, (cudaStream_t)stream>>>(
        part, peers, rank, world, rows, Hq, Sq, D, sinks, steps, errflag, (T*)out);
  });
  SAH_LAUNCH_CHECK("attn_exchange_merge");
  return SAH_OK;
}

// ---------------------------------------------------------------------------
// Masked attention with library-owned scratch (no allocation by anybody).
//
// Some hosts of this library cannot hand it scratch memory: an embedding whose
// device memory is carved up once at start-up by another runtime, or a caller
// that runs under a "no allocation after initialisation" rule (allocating from
// the CUDA driver mid-run stalls every stream of the process), has nowhere to
// get the work lists and partial buffers that plan + gather attention need.
// This entry point keeps them in one statically sized device array that is
// part of the library image, so nothing is allocated at any time -- at the
// price of a fixed upper bound on the problem size and of one copy of the
// array per GPU that loads the library.
// ---------------------------------------------------------------------------
#define SAH_STATIC_MAX_ENTRIES (1ll << 20)   // groups * S union-list slots
#define SAH_STATIC_MAX_COUNTERS (1ll << 16)  // int32 counters (counts, chunk counts, tickets)
#define SAH_STATIC_MAX_PARTIAL (1ll << 21)   // fp32 words of split partials

#define SAH_STATIC_OFF_UCOLS 0ll
#define SAH_STATIC_OFF_UMEMB (SAH_STATIC_OFF_UCOLS + SAH_STATIC_MAX_ENTRIES * 4)
#define SAH_STATIC_OFF_COUNT (SAH_STATIC_OFF_UMEMB + SAH_STATIC_MAX_ENTRIES * 2)
#define SAH_STATIC_OFF_PARTIAL (SAH_STATIC_OFF_COUNT + SAH_STATIC_MAX_COUNTERS * 4)
#define SAH_STATIC_BYTES (SAH_STATIC_OFF_PARTIAL + SAH_STATIC_MAX_PARTIAL * 4)

// 14.25 MiB of device memory on every GPU that loads this library, until exit.
static __device__ __align__(256) unsigned char g_sah_static_scratch[SAH_STATIC_BYTES];

#define SAH_STATIC_MAX_DEVICES 64
static std::mutex g_static_mu;
static unsigned char* g_static_ptr[SAH_STATIC_MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device.  In host code the
// array's name is only a handle, not an address a kernel could use; the address
// is asked for once per device, with that device current, and remembered.
static int sah_static_scratch_ptr(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "static scratch: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= SAH_STATIC_MAX_DEVICES)
    return sah_fail(SAH_ERR_UNSUPPORTED, "static scratch: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_sah_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return sah_fail(SAH_ERR_CUDA, "static scratch: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_static_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_static_ptr[dev];
  return SAH_OK;
}

extern "C" int sah_masked_attention_static(
    const uint32_t* bits, const void* q, const void* k, const void* v, int dtype, int64_t qs_b,
    int64_t qs_h, int64_t qs_q, int64_t ks_b, int64_t ks_h, int64_t ks_s, int64_t vs_b,
    int64_t vs_h, int64_t vs_s, int B, int Hq, int Hkv, int Sq, int64_t S, int64_t W, int D,
    float scaling, const void* bias, int64_t bias_s_b, int64_t bias_s_h, int64_t bias_s_q,
    const float* sinks, int sm_count, void* out, void* stream) {
  SAH_REQUIRE(bits && q && k && v && out, "masked_attention_static: null pointer");
  sah_attn_sizes sizes;
  int rc = sah_attn_query_sizes(B, Hq, Hkv, Sq, S, D, /*has_data=*/0, sm_count, &sizes);
  if (rc != SAH_OK) return rc;
  const long long entries = (long long)sizes.groups * S;
  const long long counters = sizes.ucount_bytes / 4;
  const long long partial_words = sizes.partial_bytes / 4;
  if (entries > SAH_STATIC_MAX_ENTRIES || counters > SAH_STATIC_MAX_COUNTERS ||
      partial_words > SAH_STATIC_MAX_PARTIAL)
    return sah_fail(SAH_ERR_WORKSPACE,
                    "masked_attention_static: problem needs %lld list slots, %lld counters and %lld "
                    "partial words; the built-in scratch holds %lld, %lld and %lld "
                    "(use sah_attn_plan + sah_masked_attention with caller memory instead)",
                    entries, counters, partial_words, (long long)SAH_STATIC_MAX_ENTRIES,
                    (long long)SAH_STATIC_MAX_COUNTERS, (long long)SAH_STATIC_MAX_PARTIAL);
  unsigned char* base = nullptr;
  rc = sah_static_scratch_ptr(&base);
  if (rc != SAH_OK) return rc;
  int32_t* ucols = reinterpret_cast<int32_t*>(base + SAH_STATIC_OFF_UCOLS);
  uint16_t* umemb = reinterpret_cast<uint16_t*>(base + SAH_STATIC_OFF_UMEMB);
  int32_t* ucount = reinterpret_cast<int32_t*>(base + SAH_STATIC_OFF_COUNT);
  float* partial = reinterpret_cast<float*>(base + SAH_STATIC_OFF_PARTIAL);
  // The array keeps whatever the previous call left; the counters (union counts,
  // merge tickets, error word) are the part that has to start from zero.
  cudaError_t e = cudaMemsetAsync(ucount, 0, (size_t)sizes.ucount_bytes, (cudaStream_t)stream);
  if (e != cudaSuccess)
    return sah_fail(SAH_ERR_CUDA, "masked_attention_static: memset: %s", cudaGetErrorString(e));
  rc = sah_attn_plan(bits, nullptr, nullptr, nullptr, dtype, B, Hq, Hkv, Sq, S, W, &sizes, ucols,
                     umemb, nullptr, ucount, stream);
  if (rc != SAH_OK) return rc;
  return sah_masked_attention(q, k, v, dtype, qs_b, qs_h, qs_q, ks_b, ks_h, ks_s, vs_b, vs_h, vs_s,
                              B, Hq, Hkv, Sq, S, D, scaling, bias, bias_s_b, bias_s_h, bias_s_q,
                              sinks, &sizes, ucols, umemb, nullptr, ucount, partial, out, nullptr,
                              stream);
}

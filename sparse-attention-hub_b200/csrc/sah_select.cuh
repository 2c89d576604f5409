// Exact per-row top-k by radix select over order-preserving integer keys, with
// ties going to the lowest column.  One CTA (SAH_SELECT_THREADS threads) owns
// one mask row.  Only columns inside [col_begin, col_end) whose `prev` bit is
// clear compete; the row written is prev | winners.
//
// Passes over the row's keys: KEYBITS / 8 histogram passes (most significant
// digit first) fix the k-th largest key T and how many keys equal to T are
// still needed; one counting pass and one emit pass then resolve ties in
// column order: each warp owns a contiguous run of bitmap words, counts its
// keys equal to T, a 32-entry scan orders the warps, and the warp emits its
// words front to back taking "equal" keys while the quota lasts.
#pragma once

#include "sah_common.cuh"

#define SAH_SELECT_THREADS 1024

struct SahSelectSmem {
  unsigned int hist[256];
  long long scan[33];
  unsigned int prefix;       // key bits fixed so far
  unsigned int prefix_mask;  // which bits are fixed
  long long need;            // keys still to take among the current candidates
  int take_all;              // fewer candidates than k: take every candidate
};

// Adds 1 to hist[digit] for every lane with digit < 256, one atomic per
// distinct digit in the warp.
__device__ __forceinline__ void sah_hist_add(unsigned int* hist, unsigned int digit) {
  unsigned int peers = __match_any_sync(0xffffffffu, digit);
  int lane = threadIdx.x & 31;
  if (digit < 256u && lane == (__ffs(peers) - 1)) atomicAdd(&hist[digit], (unsigned)__popc(peers));
}

// Keep the lowest n set bits of m.
__device__ __forceinline__ uint32_t sah_lowest_bits(uint32_t m, int n) {
  int c = __popc(m);
  if (n >= c) return m;
  if (n <= 0) return 0u;
  unsigned pos = __fns(m, 0, n + 1);  // position of the (n+1)-th set bit
  return m & ((1u << pos) - 1u);
}

template <int KEYBITS, typename KeyFn>
__device__ void sah_select_row(const KeyFn& keyf, const uint32_t* __restrict__ prev_row,
                               uint32_t* __restrict__ out_row, int64_t S, int64_t W,
                               int64_t col_begin, int64_t col_end, int64_t k,
                               SahSelectSmem& sm) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int NT = SAH_SELECT_THREADS;
  if (col_begin < 0) col_begin = 0;
  if (col_end > S) col_end = S;

  if (tid == 0) {
    sm.prefix = 0u;
    sm.prefix_mask = 0u;
    sm.need = k;
    sm.take_all = (k <= 0) ? 2 : 0;  // 2: take nothing
  }
  __syncthreads();

  // ---- histogram passes ----
  if (k > 0) {
    for (int shift = KEYBITS - 8; shift >= 0; shift -= 8) {
      if (tid < 256) sm.hist[tid] = 0u;
      __syncthreads();
      const unsigned int pfx = sm.prefix, pmask = sm.prefix_mask;
      const int stop = sm.take_all;
      if (!stop) {
        // The loop bound is warp-uniform so that every lane reaches the
        // warp-wide match inside sah_hist_add.
        int64_t j0 = col_begin - (col_begin & 31);
        for (int64_t base = j0 + (tid & ~31); base < col_end; base += NT) {
          const int64_t j = base + lane;
          unsigned int digit = 256u;
          if (j >= col_begin && j < col_end) {
            uint32_t pw = prev_row[j >> 5];
            if (!((pw >> (j & 31)) & 1u)) {
              unsigned int key = keyf(j);
              if ((key & pmask) == pfx) digit = (key >> shift) & 255u;
            }
          }
          sah_hist_add(sm.hist, digit);
        }
      }
      __syncthreads();
      if (warp == 0 && !stop) {
        // lane l owns bins [8l, 8l+8); find the bin where the descending
        // cumulative count reaches `need`.
        unsigned int loc[8];
        unsigned int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { loc[i] = sm.hist[lane * 8 + i]; s += loc[i]; }
        // suffix sum over lanes: above = sum of lanes > lane
        unsigned int incl = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          unsigned int n = __shfl_down_sync(0xffffffffu, incl, o);
          if (lane + o < 32) incl += n;
        }
        unsigned int above = incl - s;
        unsigned int total = __shfl_sync(0xffffffffu, incl, 0);
        long long need = sm.need;
        if ((long long)total < need || (shift == KEYBITS - 8 && (long long)total <= need)) {
          if (lane == 0) sm.take_all = 1;
        } else {
          bool mine = ((long long)above < need) && ((long long)above + s >= need);
          if (mine) {
            long long cum = above;
            int d = 7;
            for (; d >= 0; --d) {
              if (cum + loc[d] >= need) break;
              cum += loc[d];
            }
            sm.prefix = pfx | ((unsigned int)(lane * 8 + d) << shift);
            sm.prefix_mask = pmask | (255u << shift);
            sm.need = need - cum;
          }
        }
      }
      __syncthreads();
    }
  }

  // ---- tie resolution in column order ----
  const unsigned int T = sm.prefix;
  const int mode = sm.take_all;          // 0: threshold, 1: all candidates, 2: none
  const long long need = sm.need;        // keys equal to T to take
  const int64_t words_per_warp = (W + 31) / 32;
  const int64_t w_lo = (int64_t)warp * words_per_warp;
  int64_t w_hi = w_lo + words_per_warp;
  if (w_hi > W) w_hi = W;

  long long eq_here = 0;
  if (mode == 0) {
    for (int64_t w = w_lo; w < w_hi; ++w) {
      int64_t j = w * 32 + lane;
      bool eq = false;
      if (j >= col_begin && j < col_end) {
        uint32_t pw = prev_row[w];
        if (!((pw >> lane) & 1u)) eq = (keyf(j) == T);
      }
      eq_here += __popc(__ballot_sync(0xffffffffu, eq));
    }
  }
  long long total_eq;
  long long before = sah_block_excl_scan<long long>(lane == 0 ? eq_here : 0, sm.scan, &total_eq);
  before = __shfl_sync(0xffffffffu, before, 0);

  long long quota = need - before;  // equal keys this warp may still take
  for (int64_t w = w_lo; w < w_hi; ++w) {
    int64_t j = w * 32 + lane;
    uint32_t pw = prev_row[w];
    bool gt = false, eq = false;
    if (mode != 2 && j >= col_begin && j < col_end && !((pw >> lane) & 1u)) {
      if (mode == 1) {
        gt = true;
      } else {
        unsigned int key = keyf(j);
        gt = key > T;
        eq = key == T;
      }
    }
    uint32_t gm = __ballot_sync(0xffffffffu, gt);
    uint32_t em = __ballot_sync(0xffffffffu, eq);
    int take = quota > 32 ? 32 : (quota < 0 ? 0 : (int)quota);
    uint32_t sel = gm | sah_lowest_bits(em, take);
    quota -= __popc(em);
    if (lane == 0) out_row[w] = pw | sel;
  }
}

/*
 * sah_b200.h -- C ABI of the B200 (sm_100a) sparse-decode attention library.
 *
 * Every entry point is `extern "C"`, takes plain device pointers, extents and
 * element strides, launches its kernels on the CUDA stream passed as the last
 * argument (a `cudaStream_t` carried as `void*`), never synchronises the host
 * and never allocates.  The return value is an `sah_status`; on a non-zero
 * status nothing has been launched and `sah_last_error()` describes why.
 *
 * Shared conventions
 *   rows        one mask row per (batch b, query head h, query position q):
 *               row = (b * Hq + h) * Sq + q.
 *   bits        the active set of a mask: uint32 [rows][W], bit (j & 31) of
 *               word (j >> 5) is key column j.  W >= ceil(S / 32); bits at
 *               columns >= S are zero.
 *   ptr/wpre    CSR companion of `bits`: ptr int64 [rows + 1] is the exclusive
 *               scan of the per-row popcounts; wpre int32 [rows][W] is the
 *               exclusive popcount scan of the words inside one row.  The
 *               k-th set bit of a row (ascending column order) owns
 *               data[ptr[row] + k].
 *   data        per active entry weight in the mask dtype (the reference's
 *               Mask.data); NULL means every active entry has weight 1.
 *   dtype       SAH_F32 or SAH_BF16: element type of Q/K/V, of the additive
 *               attention bias and of mask weights.
 *   strides     counted in elements; the head dimension is always contiguous.
 *   GQA         query head h reads KV head h / (Hq / Hkv).
 *
 * Reference citations name files of skylight-org/sparse-attention-hub by
 * their path inside that project.
 */
#ifndef SAH_B200_H
#define SAH_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  SAH_OK = 0,
  SAH_ERR_INVALID = 1,     /* bad argument (null pointer, extent, alignment) */
  SAH_ERR_UNSUPPORTED = 2, /* legal in the reference, not built here        */
  SAH_ERR_CUDA = 3,        /* the CUDA runtime refused a launch             */
  SAH_ERR_WORKSPACE = 4    /* caller-provided workspace too small           */
} sah_status;

typedef enum { SAH_F32 = 0, SAH_BF16 = 1 } sah_dtype;

typedef enum {
  SAH_ACT_RELU = 0,
  SAH_ACT_SILU = 1,
  SAH_ACT_GELU = 2,
  SAH_ACT_TANH = 3
} sah_activation;

/* Library identity and the message of the last non-zero status returned on
 * the calling thread. */
const char* sah_version(void);
const char* sah_last_error(void);

/* Number of kernels this library has launched in the process so far. */
long long sah_launch_count(void);

/* Optional per-kernel device timing, off by default.  While enabled, the
 * kernels named by a slot are bracketed by CUDA events on the launching
 * stream (0 gather attention, 1 hash top-k, 2 hash encode, 3 q.k scores,
 * 4 generic top-k, 5 attention plan, 6 split merge).  sah_profile_read waits
 * for the recorded events of one slot, returns their summed duration and
 * count, and forgets them.  This mirrors what the reference's timing harness
 * does around whole calls with torch.cuda.synchronize
 * (profile/profile_research_attention.py:294-330), at kernel granularity. */
int sah_profile_enable(int on);
int sah_profile_read(int slot, float* total_ms, int* launches);

/* ------------------------------------------------------------------------ *
 * Mask container kernels
 * ------------------------------------------------------------------------ */

/* Set (value = 1) or clear (value = 0) a per-row column band: row (b,h,q)
 * touches columns [lo_base + q * lo_qstep, hi_base + q * hi_qstep) clipped
 * to [0, S).
 *   SinkMasker  : lo = 0, hi = sink, steps 0, value 1
 *                 (maskers/fixed/implementations/basic_fixed.py:354-363).
 *   LocalMasker : band lo = S-Sq-W+1+q, hi = S-Sq+1+q, value 1, followed by a
 *                 clear of [S-Sq+1+q, S) (basic_fixed.py:48-67).
 * Valid only for masks whose weights are all 1 (data == NULL). */
int sah_mask_fill_band(uint32_t* bits, int64_t rows, int Sq, int64_t S, int64_t W,
                       int64_t lo_base, int64_t lo_qstep, int64_t hi_base,
                       int64_t hi_qstep, int value, void* stream);

/* Several band edits in one pass over the bitmap: bands is a HOST array of n_bands (<= 6)
 * quintuples (lo_base, lo_qstep, hi_base, hi_qstep, value), applied in order with the
 * meaning of sah_mask_fill_band; with init_zero != 0 the bitmap's previous contents are
 * ignored (it starts empty), so a fresh mask needs no separate clear. */
int sah_mask_fill_bands(uint32_t* bits, int64_t rows, int Sq, int64_t S, int64_t W, int n_bands,
                        const int64_t* bands, int init_zero, void* stream);

/* ptr[rows+1] and (optionally, may be NULL) wpre[rows][W] from bits.
 * Replaces the nonzero/count_nonzero/cumsum chain of Mask.get_index_mask
 * (utils/mask.py:553-573). */
int sah_mask_rowscan(const uint32_t* bits, int64_t rows, int64_t W, int32_t* wpre,
                     int64_t* ptr, void* stream);

/* Flat int64 indices (row * S + column, ascending) of every set bit, laid out
 * by ptr/wpre: the `indices` array of utils/mask.py:233-270. */
int sah_mask_bits_to_indices(const uint32_t* bits, const int32_t* wpre,
                             const int64_t* ptr, int64_t rows, int64_t S, int64_t W,
                             int64_t* indices, void* stream);

/* Dense [rows][S] weights in `dtype` from bits (+ data): Mask.get_dense_mask
 * (utils/mask.py:577-611). */
int sah_mask_bits_to_dense(const uint32_t* bits, const void* data, const int32_t* wpre,
                           const int64_t* ptr, int dtype, int64_t rows, int64_t S,
                           int64_t W, void* dense, void* stream);

/* bits from a dense [rows][S] weight tensor (non-zero = active):
 * Mask.create_mask_from_dense_mask (utils/mask.py:272-299). */
int sah_mask_dense_to_bits(const void* dense, int dtype, int64_t rows, int64_t S,
                           int64_t W, uint32_t* bits, void* stream);

/* data[ptr[row] + k] = dense[row][column of k-th set bit]. */
int sah_mask_dense_gather_data(const void* dense, int dtype, const uint32_t* bits,
                               const int32_t* wpre, const int64_t* ptr, int64_t rows,
                               int64_t S, int64_t W, void* data, void* stream);

/* Sampled-set merge, the `clamp(previous + sampled, 0, 1)` of
 * Mask.merge_mask_dense (utils/mask.py:875-877) when the previous mask has
 * unit weights: out_bits = prev | samp;  an entry already in prev keeps
 * weight 1, an entry only in samp gets row_weight[row] (weights in `dtype`,
 * rounded as the reference rounds them).  Writes out_bits, then the caller
 * runs sah_mask_rowscan on out_bits and sah_mask_sample_data to fill data. */
int sah_mask_or(const uint32_t* a, const uint32_t* b, int64_t words, uint32_t* out,
                void* stream);
int sah_mask_sample_data(const uint32_t* prev_bits, const uint32_t* out_bits,
                         const int32_t* wpre, const int64_t* ptr, const void* row_weight,
                         const void* dense_weight, int dtype, int64_t rows, int64_t S,
                         int64_t W, void* data, void* stream);

/* data[entry] = 1 for every entry of `bits` whose column is also set in unit_bits
 * (other entries keep their value): the clamp(previous + p, 0, 1) of
 * Mask.merge_mask_dense (utils/mask.py:875-877) for a unit-weight previous mask and
 * probabilities p <= 1 that were written for every entry of the joined set. */
int sah_mask_unit_data(const uint32_t* bits, const uint32_t* unit_bits, const int32_t* wpre,
                       const int64_t* ptr, int dtype, int64_t rows, int64_t W, void* data,
                       void* stream);

/* Mask.create_from_row_wise_idx, dense mode (utils/mask.py:335-395): dense[row][idx[row][j]] =
 * vals[row][j] for idx int64 [rows][k], vals [rows][k] in `dtype`; every other position 0; of
 * several j with the same column the last one wins, as the sequential scatter of the CPU
 * reference does.  claims: device scratch of rows * S * 8 bytes (zeroed by the call). */
int sah_mask_rowwise_scatter(const int64_t* idx, const void* vals, int dtype, int64_t rows, int64_t k,
                             int64_t S, void* claims, void* dense, void* stream);

/* Mask.merge_mask_sparse (utils/mask.py:893-1062) in two steps: sah_mask_flat_add adds the
 * values of an index list (flat int64 indices row * S + col, values in `dtype`, NULL = ones)
 * into acc, float32 [total] zeroed by the caller -- once per operand -- and
 * sah_mask_clamp_to_dense rounds every sum to `dtype` and clamps it to [0, 1]. */
int sah_mask_flat_add(const int64_t* flat_idx, const void* vals, int dtype, int64_t n, int64_t total,
                      float* acc, void* stream);
int sah_mask_clamp_to_dense(const float* acc, int dtype, int64_t total, void* dense, void* stream);

/* Scatter a ragged list of sampled columns into a bitmap.  sample j belongs
 * to the row r with sptr[r] <= j < sptr[r+1] (sptr int64 [rows+1], device);
 * cols int64 [n].  Duplicates collapse, as the dense conversion of the
 * reference does (utils/mask.py:604-608).  `bits` must be zeroed by the
 * caller (or hold a mask to OR into). */
int sah_mask_scatter_samples(const int64_t* cols, const int64_t* sptr, int64_t rows,
                             int64_t n_max, int64_t S, int64_t W, uint32_t* bits,
                             void* stream);

/* ------------------------------------------------------------------------ *
 * HashAttention top-k  (maskers/fixed/implementations/hashattention_top_k.py)
 * ------------------------------------------------------------------------ */

/* Sign-bit signatures of an MLP, packed one uint32 per vector
 * (_get_signatures :203-238, _apply_single_layer :240-253).
 *   x       [B][H_in][n][D] with strides (xs_b, xs_h, xs_n), vectors
 *           n_begin .. n_end-1 are encoded
 *   codes   uint32 [B][H_out][n_total]; head h_out uses weight set h_out and
 *           reads input head h_out / (H_out / H_in) (keys are hashed per
 *           query head, :354-359)
 *   layers  n_layers <= 4; weights[l] is [H_out][dims[l]][dims[l+1]],
 *           bias[l] is [H_out][dims[l+1]], both contiguous in `dtype`;
 *           dims[0] = D, dims[n_layers] = bits <= 32
 *   act     activation between layers; for SAH_BF16 `act_table` is a device
 *           table uint16[65536] mapping the bf16 bit pattern of x to the bf16
 *           bit pattern of act(x) (every bf16 rounding of the reference chain
 *           is reproduced: product sums are accumulated in fp32 in ascending
 *           input-channel order and rounded to bf16 after the sum, after the
 *           bias add and after the activation).
 * bit e of a code is 1 when output e is > 0 (the reference's sign() == +1). */
int sah_hash_encode(const void* x, int dtype, int64_t xs_b, int64_t xs_h, int64_t xs_n,
                    int B, int H_in, int H_out, int64_t n_begin, int64_t n_end,
                    int64_t n_total, int n_layers, const int* dims,
                    const void* const* weights, const void* const* bias, int act,
                    const uint16_t* act_table, uint32_t* codes, void* stream);

/* Top-k over Hamming scores with lowest-index tie-break
 * (_compute_hashattention_score :343-371 followed by
 * TopKMasker._get_topk_indices_from_inactive_positions,
 * maskers/fixed/base.py:74-85).  score(j) = nbits - 2 * popcount(q ^ k_j)
 * (+ bias[b][.][q][j], added and rounded in `dtype`, when bias != NULL).
 * Only columns whose prev bit is clear compete; out_bits = prev | winners.
 * kcodes uint32 [B][Hq][kc_stride] (first S of each row used), qcodes uint32
 * [B][Hq][Sq].  out_bits may alias prev_bits. */
int sah_hash_topk(const uint32_t* kcodes, int64_t kc_stride, const uint32_t* qcodes, int nbits,
                  const void* bias, int dtype, int64_t bias_s_b, int64_t bias_s_h,
                  int64_t bias_s_q, int B, int Hq, int Sq, int64_t S, int64_t W,
                  const uint32_t* prev_bits, int64_t k, uint32_t* out_bits, void* stream);

/* ------------------------------------------------------------------------ *
 * Oracle top-k  (maskers/fixed/implementations/oracle_top_k.py:48-125)
 * ------------------------------------------------------------------------ */

/* scores[row][j] = q_row . k_j in `dtype` (unscaled, :70), plus the additive
 * bias.  The dot product is accumulated in fp32 in a fixed order (eight
 * interleaved partial sums over ascending 8-element chunks, then a fixed
 * pairwise tree) and rounded once to `dtype`; the bias add is rounded again,
 * as the reference's tensor ops do.  scores is [rows][S] in `dtype`. */
int sah_qk_scores(const void* q, const void* k, int dtype, int64_t qs_b, int64_t qs_h,
                  int64_t qs_q, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B, int Hq,
                  int Hkv, int Sq, int64_t S, int D, const void* bias, int64_t bias_s_b,
                  int64_t bias_s_h, int64_t bias_s_q, void* scores, void* stream);

/* Generic top-k of a [rows][S] score tensor in `dtype` over the columns whose
 * prev bit is clear, in the column window [col_begin, col_end), ties to the
 * lowest column; out_bits = prev | winners (maskers/fixed/base.py:74-85).
 * out_bits may alias prev_bits. */
int sah_topk_select(const void* scores, int dtype, int64_t rows, int64_t S, int64_t W,
                    int64_t col_begin, int64_t col_end, const uint32_t* prev_bits,
                    int64_t k, uint32_t* out_bits, void* stream);

/* The same selection with every row spread over many CTAs (sah_topk_select gives
 * a row to one CTA, which leaves most SMs idle when there are few, long rows).
 * Needs a 16-byte aligned device workspace of sah_topk_select_ws_bytes(rows, W)
 * bytes (SAH_ERR_WORKSPACE when smaller); rows <= 65535.  out_bits may alias
 * prev_bits.  Same result as sah_topk_select, bit for bit. */
int64_t sah_topk_select_ws_bytes(int64_t rows, int64_t W);
/* The same selection step by step, for rows whose keys are spread over ranks
 * (contiguous column ranges in rank order; every rank works on its own columns with
 * its own workspace of sah_topk_select_ws_bytes bytes):
 *   sah_topk_sel_begin(k)            reset the state (k counts keys of the whole row);
 *   for shift = keybits-8, ..., 0    (keybits 16 for bf16, 32 for fp32):
 *     sah_topk_sel_hist(shift)       digit histogram of this rank's candidates into the
 *                                    uint32 [rows][256] array that starts
 *                                    sah_topk_sel_hist_offset(rows, W) bytes into the
 *                                    workspace; the caller sums it over the ranks in place;
 *     sah_topk_sel_pick(shift, first = (shift == keybits-8), eq_total)
 *                                    fix the digit; at shift 0, eq_total[row] (int64, may
 *                                    be NULL) = this rank's keys equal to the threshold;
 *   sah_topk_sel_emit(tie_offset)    tie_offset[row] (int64, may be NULL) = such keys on
 *                                    lower ranks; out_bits = prev | above | first ties.
 * With one rank and NULL eq_total / tie_offset this is sah_topk_select_ws. */
int64_t sah_topk_sel_hist_offset(int64_t rows, int64_t W);
int sah_topk_sel_begin(int64_t rows, int64_t W, int64_t k, void* workspace,
                       int64_t workspace_bytes, void* stream);
int sah_topk_sel_hist(const void* scores, int dtype, int64_t rows, int64_t S, int64_t W,
                      int64_t col_begin, int64_t col_end, const uint32_t* prev_bits,
                      void* workspace, int shift, void* stream);
int sah_topk_sel_pick(int64_t rows, int64_t W, void* workspace, int shift, int first,
                      int64_t* eq_total, void* stream);
int sah_topk_sel_emit(const void* scores, int dtype, int64_t rows, int64_t S, int64_t W,
                      int64_t col_begin, int64_t col_end, const uint32_t* prev_bits,
                      void* workspace, const int64_t* tie_offset, uint32_t* out_bits,
                      void* stream);
int sah_topk_select_ws(const void* scores, int dtype, int64_t rows, int64_t S, int64_t W,
                       int64_t col_begin, int64_t col_end, const uint32_t* prev_bits,
                       int64_t k, uint32_t* out_bits, void* workspace,
                       int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------ *
 * Adaptive sampling  (maskers/sampling/implementations/adaptive_sampling.py)
 * ------------------------------------------------------------------------ */

/* Per-row sample budget and sampling probability of the (epsilon, delta) masker
 * (add_mask :304-407): exp weights of the scaled scores in `dtype`
 * (_compute_exp_attention_scores :183-197), static denominator over the previous
 * mask under its inverse weights (apply_inv_mask_sum), base sample of `nb` draws
 * in [start, end) -> unbiased standard deviation and denominator estimate
 * (_get_std_estimate_using_base_sample :237-280), budget
 * clamp((ppf * std * n / max(eps * den, 1e-8))^2, 1, n) truncated, then clamped to
 * [nb, n] (_compute_adaptive_budget :282-302, :394), probability budget / n.
 * Every tensor operation of the reference is one rounding to `dtype`; sums run in
 * a fixed order (1024 strided partial sums, then xor trees over lanes and warps).
 *   scores      [rows][S] unscaled q.k in `dtype` (sah_qk_scores without bias)
 *   prev_bits   NULL when the previous mask is empty or full (plain sum)
 *   base_draws  optional int64 [rows][nb] columns; NULL: Philox4x32-10 of
 *               (seed, row * nb + i) mapped to start + floor(u * n / 2^32)
 *   exp_table   uint16[65536] bf16 exp table (SAH_BF16 only)
 *   budget      int64 [rows];  prob `dtype` [rows];  stats optional float [rows][4]
 *               (static denominator, std, estimated denominator, squared ratio) */
int sah_adaptive_budget(const void* scores, int dtype, float scaling, const void* bias,
                        int64_t bias_s_b, int64_t bias_s_h, int64_t bias_s_q,
                        const uint32_t* prev_bits, const void* prev_data, const int32_t* wpre,
                        const int64_t* ptr, int B, int Hq, int Sq, int64_t S, int64_t W,
                        int64_t start, int64_t end, int64_t nb, uint64_t seed,
                        const int64_t* base_draws, const uint16_t* exp_table, float delta_ppf,
                        float epsilon, int64_t* budget, void* prob, float* stats, void* stream);

/* Budgeted draws into a bitmap (create_sampling_mask_with_per_head_budget,
 * utils/mask_attention_utils.py:105-184): sample j < sptr[rows] belongs to the row
 * r with sptr[r] <= j < sptr[r+1] and is column pool[j], or, with pool == NULL,
 * start + floor(philox(seed, j) * n / 2^32).  `bits` must be zeroed by the caller. */
int sah_sample_scatter(const int64_t* sptr, int64_t rows, const int64_t* pool, uint64_t seed,
                       int64_t start, int64_t n, int64_t S, int64_t W, int sm_count,
                       uint32_t* bits, void* stream);

/* ------------------------------------------------------------------------ *
 * Oracle top-p  (maskers/fixed/implementations/oracle_top_p.py:85-169)
 * ------------------------------------------------------------------------ */

/* out_bits = {j : w_j >= t_row} (| prev_bits when or_prev != 0), where
 * w = exp(scaling * scores + bias - rowmax) with the previously active positions at
 * the lowest finite value (_compute_exp_attention_scores :85-106, every tensor
 * operation one rounding to bf16) and t_row is the sorted weight at which the
 * normalised cumulative sum first exceeds top_p, the search position clamped to the
 * last element (_compute_top_p_thresholds :108-136).  The cumulative sum is the
 * reference's on a CPU: one float32 accumulator over the weights in descending
 * order, prefixes rounded to bf16.  dtype must be SAH_BF16 (SAH_ERR_UNSUPPORTED
 * otherwise).
 *   scores     [rows][S] unscaled q.k (sah_qk_scores without bias)
 *   exp_table  uint16[65536]: bf16 bits of x -> bf16 bits of exp(x) */
int sah_topp_select(const void* scores, int dtype, float scaling, const void* bias,
                    int64_t bias_s_b, int64_t bias_s_h, int64_t bias_s_q, int B, int Hq, int Sq,
                    int64_t S, int64_t W, const uint32_t* prev_bits, float top_p,
                    const uint16_t* exp_table, int or_prev, uint32_t* out_bits, void* stream);

/* ------------------------------------------------------------------------ *
 * Quest page top-k  (maskers/fixed/implementations/quest_top_k.py:108-196,
 * utils/quest_utils.py)
 * ------------------------------------------------------------------------ */

/* Per-page bounds (compute_page_min_max, quest_utils.py:10-50): pmin/pmax
 * [B][Hkv][D/8][P_cap][8] in `dtype` (channel d of page p at chunk d/8, slot d%8; D a multiple
 * of 8), page p covering keys [p*page_size, min(S, (p+1)*page_size));
 * pages page_begin .. ceil(S/page_size)-1 are (re)computed, so appended keys cost only the
 * pages they touch.  Bounds are kept per KV head: the reference's repeat over the query
 * heads of a group repeats them. */
int sah_quest_page_minmax(const void* k, int dtype, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B,
                          int Hkv, int64_t S, int D, int page_size, int64_t page_begin,
                          int64_t P_cap, void* pmin, void* pmax, void* stream);
/* scores[row][p] = sum_j max(q_j * pmin_j, q_j * pmax_j) in `dtype` (quest_page_scores :53-67),
 * every product rounded to `dtype`, the sum in the order of the reference's CPU row reduction
 * (8-lane float32 vectors, four interleaved accumulators, lanes last).  With a bias (additive
 * attention mask shared by the heads, bias_s_h == 0) a page without any key of bias >= 0
 * scores the lowest finite value (pages_valid :115-137, quest_top_k.py:156-170).
 * scores is [rows][ceil(S/page_size)].  D: multiple of 8, at most 512. */
int sah_quest_scores(const void* q, int dtype, int64_t qs_b, int64_t qs_h, int64_t qs_q,
                     const void* pmin, const void* pmax, int64_t P_cap, int B, int Hq, int Hkv,
                     int Sq, int64_t S, int D, int page_size, const void* bias, int64_t bias_s_b,
                     int64_t bias_s_h, int64_t bias_s_q, void* scores, void* stream);
/* out_bits = (prev_bits | keys of the pages set in page_bits) & {bias >= 0}
 * (pages_to_token_mask :70-93, maximum with the previous mask and the gate by the attention
 * mask, quest_top_k.py:178-191).  page_bits uint32 [rows][Wp]; prev_bits and bias may be NULL. */
int sah_quest_expand(const uint32_t* page_bits, int64_t Wp, const uint32_t* prev_bits,
                     const void* bias, int dtype, int64_t bias_s_b, int64_t bias_s_h,
                     int64_t bias_s_q, int B, int Hq, int Sq, int64_t S, int64_t W, int page_size,
                     uint32_t* out_bits, void* stream);

/* sah_hash_topk in pieces (no additive bias): the keys of a row are cut into
 * world * chunks contiguous column ranges ("parts") -- `chunks` per rank, ranks in
 * column order -- each worked on by its own CTA.
 *   sah_hash_hist        hist[chunk][row][33]: candidates (not in prev_bits) per score
 *                        0..32 in each of this rank's chunks (chunk c covers bitmap
 *                        words [c*cw, (c+1)*cw), cw = ceil(W/chunks) rounded up to 32);
 *   (a multi-rank caller gathers all ranks' histograms: hist_all [world][chunks][rows][33])
 *   sah_hash_shard_plan  thr[chunk][row]: scores above it are taken whole (-1 every
 *                        candidate, 64 none); need[chunk][row]: ties at thr the part
 *                        takes, lower parts (lower columns) being served first;
 *   sah_hash_emit        out_bits = prev | {score > thr} | first need ties, per chunk.
 * The union over parts equals the selection of sah_hash_topk on the whole row.
 * `scores` (optional, NULL to do without): 16-byte aligned device scratch of
 * sah_hash_scores_bytes(rows, W) bytes in which sah_hash_hist leaves one byte per key (its
 * score) and from which sah_hash_emit, given the same pointer and chunk count, reads them
 * instead of re-reading the four-byte codes.
 * sah_hash_topk_ws runs histogram and emit on one device (world = 1; every emit CTA plans
 * for itself) with a chunk count that fills the GPU for any row count; workspace: 16-byte
 * aligned device memory of sah_hash_topk_ws_bytes(rows, W, sm_count) bytes
 * (SAH_ERR_WORKSPACE when smaller). */
int64_t sah_hash_scores_bytes(int64_t rows, int64_t W);
int sah_hash_hist(const uint32_t* kcodes, int64_t kc_stride, const uint32_t* qcodes, int nbits,
                  int B, int Hq, int Sq, int64_t S, int64_t W, int chunks,
                  const uint32_t* prev_bits, int32_t* hist, void* scores, void* stream);
int sah_hash_shard_plan(const int32_t* hist_all, int world, int rank, int chunks, int64_t rows,
                        int64_t k, int32_t* thr, int64_t* need, void* stream);
int sah_hash_emit(const uint32_t* kcodes, int64_t kc_stride, const uint32_t* qcodes, int nbits,
                  int B, int Hq, int Sq, int64_t S, int64_t W, int chunks,
                  const uint32_t* prev_bits, const int32_t* thr, const int64_t* need,
                  const void* scores, uint32_t* out_bits, void* stream);
int64_t sah_hash_topk_ws_bytes(int64_t rows, int64_t W, int sm_count);
int sah_hash_topk_ws(const uint32_t* kcodes, int64_t kc_stride, const uint32_t* qcodes, int nbits,
                     int B, int Hq, int Sq, int64_t S, int64_t W, const uint32_t* prev_bits,
                     int64_t k, uint32_t* out_bits, void* workspace, int64_t workspace_bytes,
                     int sm_count, void* stream);

/* ------------------------------------------------------------------------ *
 * Merge of two weighted bitmap masks  (Mask.merge_mask_dense, utils/mask.py:809-891)
 * ------------------------------------------------------------------------ */

/* out = clamp(a + b, 0, 1) in the mask dtype; an entry is active when the sum is
 * non-zero.  Each side is bits [rows][W] with an optional CSR weight array (data
 * NULL = unit weights; with data, wpre and ptr of sah_mask_rowscan are needed).
 * Pass 1 writes the result's bitmap; the caller runs sah_mask_rowscan on it; pass 2
 * writes the result's weights in CSR order. */
int sah_mask_merge_bits(const uint32_t* a_bits, const void* a_data, const int32_t* a_wpre,
                        const int64_t* a_ptr, const uint32_t* b_bits, const void* b_data,
                        const int32_t* b_wpre, const int64_t* b_ptr, int dtype, int64_t rows,
                        int64_t W, uint32_t* out_bits, void* stream);
int sah_mask_merge_data(const uint32_t* a_bits, const void* a_data, const int32_t* a_wpre,
                        const int64_t* a_ptr, const uint32_t* b_bits, const void* b_data,
                        const int32_t* b_wpre, const int64_t* b_ptr, int dtype, int64_t rows,
                        int64_t W, const uint32_t* out_bits, const int32_t* out_wpre,
                        const int64_t* out_ptr, void* out_data, void* stream);

/* ------------------------------------------------------------------------ *
 * MagicPig: SimHash sampling  (maskers/sampling/implementations/magic_pig.py)
 * ------------------------------------------------------------------------ */

/* Signatures are stored once per KV head (the reference hashes keys repeated over
 * the query heads of a group with one projection per layer, magic_pig.py:564-565,
 * :476-491), key-major: codes[(b*Hkv + h)*cap + s][LP] holds the L table codes of
 * key s (bit j of a code = sign bit of projection column l*K + j, :120-150) followed
 * by zero padding up to the row pitch LP = L rounded up to a whole number of 16-byte
 * chunks; codes are uint8 for lsh_k <= 8 and uint16 for lsh_k <= 16 (larger lsh_k:
 * SAH_ERR_UNSUPPORTED).  head_dim must be a multiple of 32, at most 256. */

/* sums[(b*Hkv + h)*D + d] += sum over keys [s0, s1) in float64 (the key mean of
 * _center_KQ, :152-183, is sums / S rounded to the dtype; the caller zeroes sums). */
int sah_lsh_key_sums(const void* keys, int dtype, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B,
                     int Hkv, int64_t s0, int64_t s1, int D, double* sums, void* stream);

/* norms[(b*Hkv + h)*cap + s] = |k_s - mean| rounded to the dtype, for s in [s0, s1);
 * *max_norm_bits = max(*max_norm_bits, bits of the largest such norm): the global
 * maximum key norm of _transform_for_mips (:348-353).  mean [B*Hkv][D] in the key
 * dtype, or NULL when center=False. */
int sah_lsh_key_stats(const void* keys, int dtype, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B,
                      int Hkv, int64_t s0, int64_t s1, int D, const void* mean, int64_t cap,
                      float* norms, unsigned int* max_norm_bits, int sm_count, void* stream);

/* Signatures of keys [s0, s1): centre, scale by the maximum norm, append
 * sqrt(M^2 - |k|^2) / M (:332-372), project with proj [D+1][L*K] (key dtype), take
 * sign bits (bit = projection > 0), pack per table. */
int sah_lsh_key_sign(const void* keys, int dtype, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B,
                     int Hkv, int64_t s0, int64_t s1, int D, const void* mean, const float* norms,
                     const unsigned int* max_norm_bits, const void* proj, int L, int K,
                     int64_t cap, void* codes, void* stream);

/* The same signatures for bfloat16 keys of head dim 128 with 8 bits per table, with the
 * projections computed on the tensor cores (tcgen05) and every sign that the summation order
 * could have changed redone in the fixed order of sah_lsh_key_sign, so the codes are bit for
 * bit the same (magic_pig.py:120-150, :332-372).  `workspace` (16-byte aligned,
 * sah_lsh_key_sign_tc_ws_bytes) starts with two status words that the caller may read after the
 * stream has finished: [0] the number of 32-column groups that were redone -- a value above
 * (workspace_bytes - 16) / 16 means the list overflowed and the range must be redone with
 * sah_lsh_key_sign; [1] non-zero when a bounded wait inside the kernel ran out (the range must
 * be redone as well). */
int64_t sah_lsh_key_sign_tc_ws_bytes(int B, int Hkv, int64_t n_keys);
int sah_lsh_key_sign_tc(const void* keys, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B, int Hkv,
                        int64_t s0, int64_t s1, int D, const void* mean, const float* norms,
                        const unsigned int* max_norm_bits, const void* proj, int L, int K,
                        int64_t cap, void* codes, void* workspace, int64_t workspace_bytes,
                        int sm_count, void* stream);

/* Per mask row (b, h, q): centred query normalised to unit length, its L codes
 * (qcodes [rows][L], same code type as the key codes, no padding) and the unit vector of the
 * transformed query (qunit float [rows][D]; the appended column is zero).
 * Optional (NULL to skip): qhat [rows][D], the same unit vector in `dtype` (its values
 * are representable, so nothing is lost), and qmu float [rows] = qunit . mean; both
 * feed sah_masked_attention_lsh. */
int sah_lsh_query(const void* q, int dtype, int64_t qs_b, int64_t qs_h, int64_t qs_q, int B, int Hq,
                  int Sq, int G, int D, const void* mean, const void* proj, int L, int K,
                  void* qcodes, float* qunit, void* qhat, float* qmu, void* stream);

/* out_bits[row][w]: keys whose code equals the query's in at least one table
 * (_compute_matches_int64, :455-463), joined with prev_bits[row][w] when prev_bits is
 * not NULL (the active set of the dense merge with the previous mask, :593).  Every
 * word that holds keys (w < ceil(S / 32)) of every row is written; padding words of the
 * row stride W are left as they are. */
int sah_lsh_match(const void* codes, int64_t cap, const void* qcodes, int B, int Hq, int Sq, int G,
                  int L, int K, int64_t S, int64_t W, const uint32_t* prev_bits, uint32_t* out_bits,
                  void* stream);

/* data[ptr[row] + i] = collision probability 1 - (1 - (1 - theta/pi)^K)^L of the
 * i-th set bit of the row (:374-403), theta the angle between the transformed
 * key and query, every operation rounded to the dtype.  bf16 needs `table`,
 * uint16 [65536]: bits of the clamped cosine -> bits of the probability.
 * `dens` (optional, bf16 only): the cached norms of sah_lsh_key_den, which
 * shorten the per-key work; they must be current for the keys and *max_norm_bits. */
int sah_lsh_key_den(const void* keys, int dtype, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B,
                    int Hkv, int64_t s_new0, int64_t s1, int D, const void* mean,
                    const float* norms, int64_t cap, const unsigned int* max_norm_bits,
                    unsigned int* dens_max_bits, float* dens, int sm_count, void* stream);
/* ^ dens[(b*Hkv + h)*cap + s] = |transformed key s| + 1e-8 (rounded per operation) for
 * s in [s_new0, s1), or for every s in [0, s1) when *max_norm_bits differs from
 * *dens_max_bits (the maximum the cached values were made with); then
 * *dens_max_bits = *max_norm_bits.  Call after sah_lsh_key_stats whenever keys arrived. */
int sah_lsh_prob(const void* keys, int dtype, int64_t ks_b, int64_t ks_h, int64_t ks_s, int B,
                 int Hq, int Sq, int G, int D, const void* mean, const float* norms,
                 const float* dens, int64_t cap,
                 const unsigned int* max_norm_bits, const float* qunit, const uint32_t* bits,
                 const int32_t* wpre, const int64_t* ptr, int64_t W, int K, int L,
                 const uint16_t* table, void* data, int sm_count, void* stream);

/* ------------------------------------------------------------------------ *
 * PQCache  (maskers/fixed/implementations/pq_top_k.py, utils/pq_utils.py)
 * ------------------------------------------------------------------------ */

/* A "group" is one (batch, KV head, sub-vector): group = (b*Hkv + kvh)*n_sub + sub.
 * centroids (k-means state) are float32 [groups][n_cent][sub_d]; codes are bytes
 * [B][Hkv][cap][n_sub] (code of key j sits at row j - init_offset). */

/* Nearest centroid of the sub-vectors of keys [key_begin, key_end): the assignment
 * step of kmeans_batched (pq_utils.py:246-255, :353) and the quantisation of
 * appended keys (pq_top_k.py:388-404).  Distance = sum over ascending dims of
 * (x - c)^2 in fp32; the first minimum wins.  With dtype_math != 0 every
 * operation is rounded to `dtype`, which is how the reference quantises appended
 * keys against its stored dtype centroids. */
int sah_pq_assign(const void* x, int dtype, int64_t xs_b, int64_t xs_h, int64_t xs_s, int B,
                  int Hkv, int64_t key_begin, int64_t key_end, int64_t init_offset, int n_sub,
                  int sub_d, int n_cent, const float* centroids, uint8_t* codes, int64_t cap,
                  int dtype_math, void* stream);

/* The assignment step of kmeans_batched (utils/pq_utils.py:220-257, :346-358) for bfloat16 keys,
 * sub-vectors of 8 channels and 16..256 centroids (a multiple of 16), with the distance
 * contraction on the tensor cores (tcgen05) and the argmin decided by the fixed-order float32
 * distance among the centroids the product cannot tell apart: the codes equal those of
 * sah_pq_assign(dtype_math = 0) bit for bit.  *errflag (device) is set when the bounded wait
 * inside the kernel ran out; the caller then redoes the range with sah_pq_assign. */
int sah_pq_assign_tc(const void* x, int64_t xs_b, int64_t xs_h, int64_t xs_s, int B, int Hkv,
                     int64_t key_begin, int64_t key_end, int64_t init_offset, int n_sub, int sub_d,
                     int n_cent, const float* centroids, uint8_t* codes, int64_t cap, int* errflag,
                     int sm_count, void* stream);

/* Per-cluster sums (float64 [groups][n_cent][sub_d]) and counts (int32
 * [groups][n_cent]) of the current assignment; both must be zeroed by the caller
 * (pq_utils.py:360-381 computes the same through one-hot masks). */
int sah_pq_accumulate(const void* x, int dtype, int64_t xs_b, int64_t xs_h, int64_t xs_s, int B,
                      int Hkv, int64_t n_keys, int64_t init_offset, int n_sub, int sub_d,
                      int n_cent, const uint8_t* codes, int64_t cap, double* sums, int* counts,
                      void* stream);

/* New centres = fp32(sum) / fp32(count); an empty cluster takes the key at
 * reseed[group][cluster] (int64 key index inside the clustered region, drawn by
 * the caller: pq_utils.py:384-396); shift2[group] = (sum of centre moves)^2, the
 * value kmeans_batched compares with its tolerance (:399-423). */
int sah_pq_update(const void* x, int dtype, int64_t xs_b, int64_t xs_h, int64_t xs_s, int B,
                  int Hkv, int64_t init_offset, int n_sub, int sub_d, int n_cent,
                  const double* sums, const int* counts, const int64_t* reseed, float* centroids,
                  float* shift2, void* stream);

/* scores[row][init_offset + j] = sum over sub-vectors of lut[sub][code(j, sub)],
 * lut[sub][c] = q_sub . centroid (rounded to `dtype`), the sum taken in fp32 in
 * ascending sub-vector order and rounded once (_compute_pq_scores,
 * pq_top_k.py:406-490).  centroids here are in `dtype`:
 * [B][Hkv][n_sub][n_cent][sub_d].  Columns outside the clustered region are not
 * written.  scores is [rows][S] in `dtype`.  Every CTA builds the tables of its rows
 * in shared memory and scores a contiguous key range; `workspace` is not used any more
 * (NULL is accepted; sah_pq_scores_ws_bytes stays for callers that size one). */
int64_t sah_pq_scores_ws_bytes(int B, int Hq, int Hkv, int Sq, int n_sub, int n_cent);
int sah_pq_scores(const void* q, int dtype, int64_t qs_b, int64_t qs_h, int64_t qs_q,
                  const void* centroids, const uint8_t* codes, int64_t cap, int B, int Hq, int Hkv,
                  int Sq, int64_t n_keys, int64_t init_offset, int64_t S, int n_sub, int sub_d,
                  int n_cent, void* scores, void* workspace, int64_t workspace_bytes,
                  void* stream);

/* ------------------------------------------------------------------------ *
 * Masked attention  (utils/mask_attention_utils.py:187-240, :406-491)
 * ------------------------------------------------------------------------ */

/* Work-list sizes for one call of sah_attn_plan / sah_masked_attention.
 * group = (b, kv head, block of q positions); a group owns
 * rows_per_group = (Hq/Hkv) * q_block mask rows (<= 16). */
typedef struct {
  int32_t groups;          /* B * Hkv * ceil(Sq / q_block)                  */
  int32_t q_block;         /* query positions per group                     */
  int32_t rows_per_group;  /* (Hq / Hkv) * q_block                          */
  int32_t nsplit;          /* CTAs cooperating on one group                 */
  int64_t ucols_bytes;     /* int32  [groups][S]                            */
  int64_t umemb_bytes;     /* uint16 [groups][S]                            */
  int64_t uw_bytes;        /* float  [groups][S][rows_per_group] (has_data 1)
                              or float [groups][S] (has_data 2)             */
  int64_t ucount_bytes;    /* int32  [groups] + chunk counters              */
  int64_t partial_bytes;   /* float  [groups][nsplit][rows_per_group][D+2]  */
} sah_attn_sizes;

/* has_data: 0 unit-weight mask, 1 mask with per-entry weights, 2 MagicPig mask whose
 * weights the attention kernel evaluates (sah_attn_plan_lsh / sah_masked_attention_lsh).
 * The counter block (ucount_bytes) ends with one merge ticket per group, which must be
 * zero when an attention call starts (the kernel leaves them zero) and one error word. */
int sah_attn_query_sizes(int B, int Hq, int Hkv, int Sq, int64_t S, int D, int has_data,
                         int sm_count, sah_attn_sizes* out);

/* Union list of one group: the ascending columns selected by any of its
 * rows (ucols), which rows selected each (umemb, bit i = i-th row of the
 * group), and -- when data != NULL -- the inverse weights
 * 1 / (data + 1e-6) evaluated in `dtype` exactly as Mask.apply_inv_mask_dense
 * does (utils/mask.py:718-740), zero for non-members (uw). */
int sah_attn_plan(const uint32_t* bits, const void* data, const int32_t* wpre,
                  const int64_t* ptr, int dtype, int B, int Hq, int Hkv, int Sq, int64_t S,
                  int64_t W, const sah_attn_sizes* sizes, int32_t* ucols, uint16_t* umemb,
                  float* uw, int32_t* ucount, void* stream);

/* The same for a MagicPig mask whose weights sah_masked_attention_lsh evaluates itself
 * (sizes queried with has_data = 2; at most 4 mask rows per KV group).  `bits` are the
 * LSH matches (sah_lsh_match), `unit_bits` (may be NULL) what the previous maskers
 * selected with weight 1 -- magic_pig.py:593 clamps those to 1; the active set is the
 * union of the two.  umemb carries membership in its low byte and "weight is 1" flags in its high
 * byte; uinv [groups][S] holds 1 / (M * dens[col]) per union entry, dens and
 * max_norm_bits being those of sah_lsh_key_den (dens_cap = their row stride). */
int sah_attn_plan_lsh(const uint32_t* bits, const uint32_t* unit_bits, const float* dens,
                      int64_t dens_cap, const unsigned int* max_norm_bits, int B, int Hq, int Hkv,
                      int Sq, int64_t S, int64_t W, const sah_attn_sizes* sizes, int32_t* ucols,
                      uint16_t* umemb, float* uinv, int32_t* ucount, void* stream);

/* out[b][q][h][:] = sum_j e_j w_j v_j / (sum_j e_j w_j [+ exp(sink_h)]),
 * e_j = exp(scaling * q.k_j + bias_j), over the planned union list; fp32
 * math, online softmax, every KV row fetched once per group and shared by
 * the group's query heads.  out is [B][Sq][Hq][D] contiguous in `dtype`
 * (utils/mask_attention_utils.py:479-481).  sinks: optional float [Hq]
 * (apply_sink_bias :357-402).  part_out: optional float [rows][D+2] = the
 * unnormalised accumulator, the running max and the denominator of each row,
 * for cross-device merging (one buffer, so that a sequence-sharded caller
 * gathers it with one collective). */
int sah_masked_attention(const void* q, const void* k, const void* v, int dtype,
                         int64_t qs_b, int64_t qs_h, int64_t qs_q, int64_t ks_b,
                         int64_t ks_h, int64_t ks_s, int64_t vs_b, int64_t vs_h,
                         int64_t vs_s, int B, int Hq, int Hkv, int Sq, int64_t S, int D,
                         float scaling, const void* bias, int64_t bias_s_b,
                         int64_t bias_s_h, int64_t bias_s_q, const float* sinks,
                         const sah_attn_sizes* sizes, const int32_t* ucols,
                         const uint16_t* umemb, const float* uw, const int32_t* ucount,
                         float* partial, void* out, float* part_out, void* stream);

/* sah_masked_attention (bfloat16) over a union list made by sah_attn_plan_lsh, with the
 * MagicPig sampling weights computed where the key row already is: the weight of a
 * sampled key is 1 / (p + 1e-6) (Mask.apply_inv_mask_dense, utils/mask.py:718-740) with
 * p = 1 - (1 - (1 - acos(c)/pi)^K)^L (the chain of magic_pig.py:389-403); the weight is read
 * from weight_table (uint16 [65536]: bf16 bits of the clamped cosine -> bf16 bits of
 * bf16(1 / bf16(p + 1e-6)), 0 where p is 0: such an entry is not part of the mask) and
 * c = (qhat . k - qmu) / (M * |transformed key|) evaluated in float32 and rounded once
 * to bfloat16.  The reference rounds every step of that cosine to bfloat16
 * (:332-372), so a weight can differ from the reference's by the effect of one bfloat16
 * step of the cosine; the selected index set does not depend on the weights.
 * qhat [rows][D] bfloat16 (16-byte aligned) and qmu [rows] come from sah_lsh_query.
 * w_dump (optional): float [groups][S][rows_per_group], receives the weight used for
 * every (union entry, member row) pair. */
int sah_masked_attention_lsh(const void* q, const void* k, const void* v, int64_t qs_b,
                             int64_t qs_h, int64_t qs_q, int64_t ks_b, int64_t ks_h, int64_t ks_s,
                             int64_t vs_b, int64_t vs_h, int64_t vs_s, int B, int Hq, int Hkv,
                             int Sq, int64_t S, int D, float scaling, const void* bias,
                             int64_t bias_s_b, int64_t bias_s_h, int64_t bias_s_q,
                             const float* sinks, const sah_attn_sizes* sizes, const int32_t* ucols,
                             const uint16_t* umemb, const float* uinv, const int32_t* ucount,
                             float* partial, const void* qhat, const float* qmu,
                             const uint16_t* weight_table, void* out, float* part_out, float* w_dump,
                             void* stream);

/* Measurement aid (no counterpart in the reference): the K/V row gather of a planned
 * union list on its own -- the grid, tiling and copy pipeline of the bfloat16
 * sah_masked_attention without its arithmetic.  Timing it gives the bandwidth that
 * this access pattern can reach on the device, the ceiling for the attention kernel
 * on the same list.  `sink` is one device word that is (practically) never written. */
int sah_attn_gather_probe(const void* k, const void* v, int64_t ks_b, int64_t ks_h, int64_t ks_s,
                          int64_t vs_b, int64_t vs_h, int64_t vs_s, int B, int Hkv, int Sq,
                          int64_t S, int D, const sah_attn_sizes* sizes, const int32_t* ucols,
                          const int32_t* ucount, unsigned int* sink, void* stream);

/* Which bfloat16 attention kernel the library launches (no counterpart in the reference):
 *   SAH_ATTN_KERNEL_AUTO (-1)  the library decides per call (the start-up value; the environment
 *                              variable SAH_ATTN_UMMA=0/1 overrides the decision),
 *   SAH_ATTN_KERNEL_MMA  (0)   per-warp mma.sync pipeline over 16-key tiles,
 *   SAH_ATTN_KERNEL_UMMA (1)   tcgen05 pipeline over 128-key tiles (head dim 128 only; other
 *                              problems still take the mma.sync kernel).
 * Process-wide; returns the previous setting, or -2 for an unknown `which`. */
#define SAH_ATTN_KERNEL_AUTO (-1)
#define SAH_ATTN_KERNEL_MMA 0
#define SAH_ATTN_KERNEL_UMMA 1
int sah_attn_select_kernel(int which);
/* Name of the attention kernel that the most recent sah_masked_attention* call launched. */
const char* sah_attn_last_kernel(void);
/* Self-test of the bounded device-side wait used by the tcgen05 kernels (no counterpart in the
 * reference): one CTA waits on an mbarrier that nothing arrives at, for at most limit_us
 * (1 .. 100000).  After the stream has finished, *errflag (device int, zeroed by the caller) is
 * non-zero and *waited_ns (device) holds how long the wait lasted; the kernel has returned
 * normally and the context is usable.  Nothing faults, traps or hangs. */
int sah_wait_selftest(int limit_us, int* errflag, unsigned long long* waited_ns, void* stream);

/* Merge n_parts partial results (parts [n_parts][rows][D+2], the part_out of
 * sah_masked_attention on every shard) into out [B][Sq][Hq][D]: the
 * associative combine of sequence-sharded softmax partials. */
int sah_attn_merge_parts(const float* parts, int n_parts, int B, int Hq, int Sq, int D,
                         const float* sinks, int dtype, void* out, void* stream);

/* Exchange + merge of the sequence shards' partials over peer memory, one launch per rank per
 * step (replaces an all-gather of part_out followed by sah_attn_merge_parts; the reference has
 * no sequence sharding, its softmax over the whole row is utils/mask_attention_utils.py:269-340).
 * Every rank owns a receive buffer of sah_attn_exchange_bytes() bytes and a flag array of
 * world * rows ints, both zeroed once and mapped by every peer; peer_bufs[p] / peer_flags[p]
 * (host arrays of `world` device pointers) are rank p's buffer and flags as addressed from
 * this process.  `steps` ([rows] ints, zeroed once, private to the rank) carries the step
 * number, so the launch can be replayed by a CUDA graph; all ranks must make the same
 * sequence of calls.  The kernel stores this rank's partial into every rank's buffer, signals,
 * waits (bounded: about a second, then *errflag = 2 and the kernel still returns) for the
 * other ranks' partials and writes out [B][Sq][Hq][D].  The kernels of different ranks wait
 * on one another: one rank per GPU. */
int64_t sah_attn_exchange_bytes(int world, int B, int Hq, int Sq, int D);
int sah_attn_exchange_merge(const float* part, const void* const* peer_bufs,
                            const void* const* peer_flags, int rank, int world, int B, int Hq, int Sq,
                            int D, const float* sinks, int dtype, int* steps, int* errflag, void* out,
                            void* stream);

/* Masked attention that brings its own scratch: plan + gather attention for a
 * unit-weight bitmap mask, with the union lists, counters and split partials
 * held in a device array that is part of the library image.
 *
 * This entry point has no counterpart in the reference.  It exists for callers
 * that have no way to hand the library scratch memory: a host whose device
 * memory was partitioned once at start-up by another runtime, or one that must
 * not allocate from the CUDA driver after initialisation because an allocation
 * stalls every stream of the process.  Such a caller still passes the inputs
 * (bits, Q, K, V, optional bias and sinks) and the output buffer; it passes no
 * workspace and nothing is allocated, by this call or by anything it calls.
 *
 * Limits: B * Hkv * ceil(Sq / q_block) * S <= 2^20 union-list slots (for
 * example 8 KV groups of 131072 keys, or 32 groups of 32768 keys), at most
 * 2^16 counters and 2^21 fp32 words of split partials; larger problems are
 * rejected with SAH_ERR_WORKSPACE and a message that states the three sizes.
 * The array is 14.25 MiB and stays resident on every GPU that loads the
 * library until the process exits.
 *
 * The first call on a device looks up the array's device address (once per
 * device, with that device current); make that first call outside any stream
 * capture.  All calls on a device share the one array, which keeps the
 * contents of the previous call: each call re-zeroes the counters it needs on
 * `stream` before use, but two calls whose kernels overlap on the GPU (two
 * streams, two host threads) race on it and must be serialised by the caller.
 * The mask must have unit weights (the data == NULL case of sah_attn_plan). */
int sah_masked_attention_static(const uint32_t* bits, const void* q, const void* k, const void* v,
                                int dtype, int64_t qs_b, int64_t qs_h, int64_t qs_q,
                                int64_t ks_b, int64_t ks_h, int64_t ks_s, int64_t vs_b,
                                int64_t vs_h, int64_t vs_s, int B, int Hq, int Hkv, int Sq,
                                int64_t S, int64_t W, int D, float scaling, const void* bias,
                                int64_t bias_s_b, int64_t bias_s_h, int64_t bias_s_q,
                                const float* sinks, int sm_count, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SAH_B200_H */

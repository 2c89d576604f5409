// bf16 gather attention on the tensor cores.
//
// Every warp runs its own pipeline with no CTA-wide barrier in the main loop:
// it takes 16-key tiles of the group's union list (tiles are dealt round-robin
// to the warps of the CTAs that share the group), gathers the 16 K rows and 16
// V rows with cp.async into a private 3-stage ring in shared memory (rows
// stored in 16-byte chunks, chunk c of row i at slot c ^ (i & 7)), and per
// tile computes
//     S[16 rows x 16 keys] = Q . K^T        mma.m16n8k16, Q fragments in registers
//     P = exp(S * scaling + bias - m) * w   online softmax in the C fragment
//     O[16 rows x D]      += P . V          mma.m16n8k16, V fragments via ldmatrix.trans
// The 16 "rows" are the mask rows of one KV group (query heads x query block,
// zero padded), so each gathered K/V row is read once for all of them.
// At the end the warps of a CTA merge their (m, l, O) in shared memory, the CTA
// writes its partial, and the last CTA of a group (atomic ticket) merges the
// group's partials and writes the output.
#pragma once

#define ATM_WARPS 4
#define ATM_THREADS (ATM_WARPS * 32)
#define ATM_STAGES 3
#define ATM_TILE 16

__device__ __forceinline__ void atm_ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                uint32_t& r3, const void* smem_ptr) {
  unsigned int a = (unsigned int)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}
__device__ __forceinline__ void atm_ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                      uint32_t& r3, const void* smem_ptr) {
  unsigned int a = (unsigned int)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}
__device__ __forceinline__ void atm_mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t atm_pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
struct AtmCfg {
  static constexpr int ROWB = D * 2;                       // bytes per bf16 row
  static constexpr int CPR = ROWB / 16;                    // 16-byte chunks per row
  static constexpr int KSTEPS = D / 16;                    // k-steps of Q.K^T
  static constexpr int NT = D / 8;                         // n-tiles of the output
  static constexpr int STAGE_BYTES = 2 * ATM_TILE * ROWB;  // K tile + V tile
  static constexpr int WARP_BYTES = ATM_STAGES * STAGE_BYTES;
  static constexpr int Q_BYTES = 16 * ROWB;
  // after the main loop the ring is reused as the per-warp reduction buffer
  static constexpr int RED_BYTES = 16 * (D + 8) * 4 + 16 * 2 * 4;  // O fp32 (padded rows) + (m, l)
  static constexpr int SMEM = ATM_WARPS * WARP_BYTES + Q_BYTES + ATM_WARPS * ATM_STAGES * 16 * 8;
};

template <int D>
__global__ void __launch_bounds__(ATM_THREADS, 2)
masked_attention_mma_kernel(AttnArgs a, int* __restrict__ tickets, const float* __restrict__ sinks,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ acc_out,
                            float* __restrict__ lse_out) {
  using C = AtmCfg<D>;
  extern __shared__ __align__(128) unsigned char atm_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* ring = atm_smem + warp * C::WARP_BYTES;
  unsigned char* q_sm = atm_smem + ATM_WARPS * C::WARP_BYTES;
  int2* meta_sm = reinterpret_cast<int2*>(q_sm + C::Q_BYTES) + warp * ATM_STAGES * 16;  // (col, memb)
  __shared__ int is_last_sm;

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
  const float* guw = a.uw ? a.uw + g * a.S * a.R : nullptr;

  // ---- stage Q (zero padded to 16 rows), swizzled like the K rows ----
  for (int idx = tid; idx < 16 * C::CPR; idx += ATM_THREADS) {
    const int r = idx / C::CPR, c = idx - r * C::CPR;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < a.R) {
      const int gi = r / a.q_block, qo = r - gi * a.q_block;
      const int qi = qb * a.q_block + qo;
      if (qi < a.Sq) {
        const int h = kvh * a.G + gi;
        val = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.q) +
                                              b * a.qs_b + (int64_t)h * a.qs_h + qi * a.qs_q + c * 8);
      }
    }
    *reinterpret_cast<uint4*>(q_sm + r * C::ROWB + ((c ^ (r & 7)) * 16)) = val;
  }
  __syncthreads();
  uint32_t qf[C::KSTEPS][4];
  {
    const int mi = lane >> 3, rr = lane & 7;
    const int row = (mi & 1) * 8 + rr;
#pragma unroll
    for (int ks = 0; ks < C::KSTEPS; ++ks) {
      const int c = 2 * ks + (mi >> 1);
      atm_ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                      q_sm + row * C::ROWB + ((c ^ (row & 7)) * 16));
    }
  }

  // ---- this warp's tiles ----
  const int U = a.ucount[g];
  const int total_tiles = (U + ATM_TILE - 1) / ATM_TILE;
  const int lanes_total = a.nsplit * ATM_WARPS;        // warps sharing the group
  const int my_first = split * ATM_WARPS + warp;       // tile t of this warp = my_first + t * lanes_total
  const int my_tiles = (total_tiles > my_first) ? (total_tiles - my_first + lanes_total - 1) / lanes_total : 0;

  // rows this thread owns in the C fragment, and their bias / weight addressing
  const int r0 = lane >> 2, r1 = r0 + 8;
  int h0 = 0, qi0 = 0, h1 = 0, qi1 = 0;
  {
    int gi = r0 / a.q_block, qo = r0 - gi * a.q_block;
    h0 = kvh * a.G + gi; qi0 = qb * a.q_block + qo;
    gi = r1 / a.q_block; qo = r1 - gi * a.q_block;
    h1 = kvh * a.G + gi; qi1 = qb * a.q_block + qo;
  }
  const __nv_bfloat16* bias0 = nullptr;
  const __nv_bfloat16* bias1 = nullptr;
  if (a.bias != nullptr) {
    const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(a.bias) + b * a.bias_s_b;
    if (r0 < a.R && qi0 < a.Sq) bias0 = bb + h0 * a.bias_s_h + qi0 * a.bias_s_q;
    if (r1 < a.R && qi1 < a.Sq) bias1 = bb + h1 * a.bias_s_h + qi1 * a.bias_s_q;
  }

  float o[C::NT][4];
#pragma unroll
  for (int nt = 0; nt < C::NT; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  auto issue = [&](int t) {
    const int st = t % ATM_STAGES;
    unsigned char* kst = ring + st * C::STAGE_BYTES;
    unsigned char* vst = kst + ATM_TILE * C::ROWB;
    const int u0 = (my_first + t * lanes_total) * ATM_TILE;
    int col = -1;
    unsigned int memb = 0u;
    if (lane < ATM_TILE && u0 + lane < U) {
      col = gcols[u0 + lane];
      memb = gmemb[u0 + lane];
    }
    if (lane < ATM_TILE) meta_sm[st * 16 + lane] = make_int2(col, (int)memb);
    // lane handles chunk (lane % CPR') of rows; 32 lanes cover 32 (row, chunk) pairs per step
#pragma unroll
    for (int it = 0; it < (ATM_TILE * C::CPR) / 32; ++it) {
      const int idx = it * 32 + lane;
      const int i = idx / C::CPR, c = idx - i * C::CPR;
      const int rc = __shfl_sync(0xffffffffu, col, i);
      const int slot = (c ^ (i & 7)) * 16;
      if (rc >= 0) {
        at_cp_async16(kst + i * C::ROWB + slot,
                      reinterpret_cast<const unsigned char*>(kbase + (int64_t)rc * a.ks_s) + c * 16);
        at_cp_async16(vst + i * C::ROWB + slot,
                      reinterpret_cast<const unsigned char*>(vbase + (int64_t)rc * a.vs_s) + c * 16);
      } else {
        // unused slots must not feed NaNs into the tensor cores
        *reinterpret_cast<uint4*>(kst + i * C::ROWB + slot) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(vst + i * C::ROWB + slot) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };

#pragma unroll
  for (int s = 0; s < ATM_STAGES - 1; ++s) {
    if (s < my_tiles) issue(s);
    at_cp_async_commit();
  }

  for (int t = 0; t < my_tiles; ++t) {
    if (t + ATM_STAGES - 1 < my_tiles) issue(t + ATM_STAGES - 1);
    at_cp_async_commit();
    at_cp_async_wait<ATM_STAGES - 1>();
    __syncwarp();

    const int st = t % ATM_STAGES;
    const unsigned char* kst = ring + st * C::STAGE_BYTES;
    const unsigned char* vst = kst + ATM_TILE * C::ROWB;
    const int u0 = (my_first + t * lanes_total) * ATM_TILE;

    // ---- S = Q . K^T ----
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
    {
      const int mi = lane >> 3, rr = lane & 7;
      const int i = (mi >> 1) * 8 + rr;
#pragma unroll
      for (int ks = 0; ks < C::KSTEPS; ++ks) {
        const int c = 2 * ks + (mi & 1);
        uint32_t b0, b1, b2, b3;
        atm_ldmatrix_x4(b0, b1, b2, b3, kst + i * C::ROWB + ((c ^ (i & 7)) * 16));
        atm_mma_bf16(s[0], qf[ks], b0, b1);
        atm_mma_bf16(s[1], qf[ks], b2, b3);
      }
    }

    // ---- online softmax in the C fragment ----
    // element (nt, e): row = (e < 2 ? r0 : r1), key j = nt * 8 + 2 * (lane & 3) + (e & 1)
    float p[2][4];
    float tmax[2] = {-INFINITY, -INFINITY};
    float wts[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = nt * 8 + 2 * (lane & 3) + (e & 1);
        const int rsel = e >> 1;
        const int r = rsel ? r1 : r0;
        const int2 cm = meta_sm[st * 16 + j];
        float sv = -INFINITY, wv = 0.f;
        if (cm.x >= 0 && ((cm.y >> r) & 1)) {
          sv = s[nt][e] * a.scaling;
          const __nv_bfloat16* bp = rsel ? bias1 : bias0;
          if (bp != nullptr) sv += __bfloat162float(bp[cm.x]);
          wv = guw ? guw[(int64_t)(u0 + j) * a.R + r] : 1.f;
        }
        s[nt][e] = sv;
        wts[nt][e] = wv;
        tmax[rsel] = fmaxf(tmax[rsel], sv);
      }
    }
    float alpha[2];
#pragma unroll
    for (int rs = 0; rs < 2; ++rs) {
      tmax[rs] = fmaxf(tmax[rs], __shfl_xor_sync(0xffffffffu, tmax[rs], 1));
      tmax[rs] = fmaxf(tmax[rs], __shfl_xor_sync(0xffffffffu, tmax[rs], 2));
      const float m_new = fmaxf(m_run[rs], tmax[rs]);
      alpha[rs] = (m_new == -INFINITY) ? 1.f : __expf(m_run[rs] - m_new);
      m_run[rs] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int rsel = e >> 1;
        float pv = 0.f;
        if (s[nt][e] != -INFINITY) pv = __expf(s[nt][e] - m_run[rsel]) * wts[nt][e];
        p[nt][e] = pv;
        psum[rsel] += pv;
      }
    }
#pragma unroll
    for (int rs = 0; rs < 2; ++rs) {
      psum[rs] += __shfl_xor_sync(0xffffffffu, psum[rs], 1);
      psum[rs] += __shfl_xor_sync(0xffffffffu, psum[rs], 2);
      l_run[rs] = l_run[rs] * alpha[rs] + psum[rs];
    }
#pragma unroll
    for (int nt = 0; nt < C::NT; ++nt) {
      o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0];
      o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
    }

    // ---- O += P . V ----
    uint32_t pa[4];
    pa[0] = atm_pack_bf16(p[0][0], p[0][1]);
    pa[1] = atm_pack_bf16(p[0][2], p[0][3]);
    pa[2] = atm_pack_bf16(p[1][0], p[1][1]);
    pa[3] = atm_pack_bf16(p[1][2], p[1][3]);
    {
      const int mi = lane >> 3, rr = lane & 7;
      const int i = (mi & 1) * 8 + rr;
#pragma unroll
      for (int np = 0; np < C::NT / 2; ++np) {
        const int c = 2 * np + (mi >> 1);
        uint32_t b0, b1, b2, b3;
        atm_ldmatrix_x4_trans(b0, b1, b2, b3, vst + i * C::ROWB + ((c ^ (i & 7)) * 16));
        atm_mma_bf16(o[2 * np], pa, b0, b1);
        atm_mma_bf16(o[2 * np + 1], pa, b2, b3);
      }
    }
    __syncwarp();  // all lanes done with this stage before it is refilled
  }
  at_cp_async_wait<0>();
  __syncthreads();

  // ---- merge the warps of this CTA (ring reused as fp32 scratch) ----
  constexpr int RS = D + 8;                                     // padded row stride
  float* red_o = reinterpret_cast<float*>(ring);               // [16][RS]
  float* red_ml = red_o + 16 * RS;                              // [16][2]
#pragma unroll
  for (int nt = 0; nt < C::NT; ++nt) {
    const int d = nt * 8 + 2 * (lane & 3);
    *reinterpret_cast<float2*>(red_o + r0 * RS + d) = make_float2(o[nt][0], o[nt][1]);
    *reinterpret_cast<float2*>(red_o + r1 * RS + d) = make_float2(o[nt][2], o[nt][3]);
  }
  if ((lane & 3) == 0) {
    red_ml[r0 * 2] = m_run[0]; red_ml[r0 * 2 + 1] = l_run[0];
    red_ml[r1 * 2] = m_run[1]; red_ml[r1 * 2 + 1] = l_run[1];
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

  // ---- last CTA of the group merges the group's partials ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&tickets[g], 1);
    const int last = (old == a.nsplit - 1);
    if (last) tickets[g] = 0;  // ready for the next call
    is_last_sm = last;
  }
  __syncthreads();
  if (!is_last_sm) return;
  __threadfence();
  const float* p0 = a.partial + (int64_t)g * a.nsplit * a.R * (D + 2);
  const int64_t pstride = (int64_t)a.R * (D + 2);
  // phase 1: one warp per row finds the row maximum, the per-split rescale
  // factors and the denominator (ring memory reused as scratch)
  float* sc_sm = reinterpret_cast<float*>(atm_smem);   // [R][nsplit]
  float* ml_sm = sc_sm + 16 * a.nsplit;                 // [R][2]
  for (int r = warp; r < a.R; r += ATM_WARPS) {
    const float* pr = p0 + (int64_t)r * (D + 2);
    float mloc = -INFINITY;
    for (int s2 = lane; s2 < a.nsplit; s2 += 32) mloc = fmaxf(mloc, __ldcg(pr + s2 * pstride + D));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
    float lsum = 0.f;
    for (int s2 = lane; s2 < a.nsplit; s2 += 32) {
      const float ms = __ldcg(pr + s2 * pstride + D);
      const float sc = (ms == -INFINITY) ? 0.f : __expf(ms - mloc);
      sc_sm[r * a.nsplit + s2] = sc;
      lsum += __ldcg(pr + s2 * pstride + D + 1) * sc;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
    if (lane == 0) { ml_sm[r * 2] = mloc; ml_sm[r * 2 + 1] = lsum; }
  }
  __syncthreads();
  // phase 2: every (row, dim) sums its column over the splits; the loads are independent
  for (int idx = tid; idx < a.R * D; idx += ATM_THREADS) {
    const int r = idx / D, d = idx - r * D;
    const int gi = r / a.q_block, qo = r - gi * a.q_block;
    const int qi = qb * a.q_block + qo;
    if (qi >= a.Sq) continue;
    const int h = kvh * a.G + gi;
    const float* pr = p0 + (int64_t)r * (D + 2) + d;
    const float* sc = sc_sm + r * a.nsplit;
    float accv = 0.f;
#pragma unroll 8
    for (int s2 = 0; s2 < a.nsplit; ++s2) accv = fmaf(__ldcg(pr + s2 * pstride), sc[s2], accv);
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
    if (acc_out != nullptr) acc_out[row * D + d] = accv;
    out[((b * a.Sq + qi) * a.Hq + h) * D + d] = __float2bfloat16_rn(accv * resc / den);
    if (lse_out != nullptr && d == 0) {
      lse_out[row * 2 + 0] = M;
      lse_out[row * 2 + 1] = L;
    }
  }
}

template <int D>
static int launch_attention_mma(const AttnArgs& a, int groups, int* tickets, const float* sinks,
                                void* out, float* acc_out, float* lse_out, cudaStream_t st) {
  using C = AtmCfg<D>;
  static_assert(C::RED_BYTES <= C::WARP_BYTES, "reduction scratch must fit the ring");
  const int smem = C::SMEM;
  cudaError_t e = cudaFuncSetAttribute(masked_attention_mma_kernel<D>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return sah_fail(SAH_ERR_CUDA, "attention attr: %s", cudaGetErrorString(e));
  dim3 grid((unsigned)a.nsplit, (unsigned)groups);
  masked_attention_mma_kernel<D><<<grid, ATM_THREADS, smem, st>>>(
      a, tickets, sinks, (__nv_bfloat16*)out, acc_out, lse_out);
  return SAH_OK;
}

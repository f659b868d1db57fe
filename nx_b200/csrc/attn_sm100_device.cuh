// Fused attention for sm_100a:  O = softmax(f(Q K^T)) V  without writing the scores to memory.
//
// The planner recognises  dot(q,k) -> elementwise f (scale, mask ...) -> softmax over the key
// axis -> dot(p,v)  in a defn graph and generates this kernel with `f` compiled in as
// AttnXform::apply.  One CTA owns TWO blocks of 128 query rows of one (batch, head) pair and walks
// the key blocks of 128 once for both, so that the tensor pipe works on one block's products while
// the other block's softmax runs, and every K / V block is fetched once per 256 query rows:
//   warp 0      TMA producer: both Q tiles once, then K_j into a two-stage ring and V_j into a
//               single buffer (V_j is needed late in step j and released at its end)
//   warp 1      MMA issuer, per key block j and query tile t, back to back:  S_t(j+1) = Q_t K_{j+1}^T
//               into the tile's score accumulator as soon as the softmax has read S_t(j), then
//               PV_t(j) = P_t V_j into the tile's output accumulator (P from shared memory, V with its
//               head-dim index contiguous, i.e. an MN-major B operand)
//   warps 2..5  softmax of tile 0, warps 6..9 of tile 1: one thread per query row (a row is one
//               TMEM lane, so maxima and sums need no exchange between threads).  The row's 128
//               scores are read from tensor memory twice, 32 at a time with the next 32 in flight:
//               once for the maximum, once for the probabilities (no spills, rolled loops, a small
//               instruction footprint).  Running maximum m and running sum l; the output row O
//               accumulates in TMEM across key blocks and is read back and rescaled only when the
//               maximum moves by more than a threshold (rare after the first blocks).
// Three forms of the score transform are compiled in: the full one; with a proven causal mask
// X = select(row >= col, Y, -inf), Y alone for key blocks entirely below the diagonal; and when
// Y = c * scores with a positive constant c, a form that takes maxima of the raw scores (3-input max)
// and folds c into the exponent's multiply-add, two scores per instruction (f32x2).
// Tensor memory: S_0, S_1, O_0, O_1, 128 columns each.  Keys beyond a causal diagonal are skipped
// block-wise when the planner proved the mask is causal (the two tiles then differ by one key
// block; the tile of the later rows is tile 0).  Every mbarrier wait is bounded; on expiry the CTA
// raises an abort flag, all roles leave their loops, tensor memory is released and the host reports
// NXB_ERR_TIMEOUT.
//
// Compiled only through NVRTC, after device_lib.cuh and gemm_sm100_device.cuh (whose PTX
// wrappers it reuses).
#pragma once

namespace nxb_attn {
using namespace nxb_gemm;

struct AttnParams {
  void* out;           // [bh][sq][128] by default; strides below in elements
  long long out_bh_hi, out_bh_lo, out_row;   // address = (bh / heads) * hi + (bh % heads) * lo + row * out_row + d
  int* status;
  int heads, batch_heads, sq, sk;   // heads: the size of the axis before the rows, 1 when there is a single leading axis
  int causal;          // 1: keys j > query i contribute nothing (proved by the planner)
  void* ep[14];        // buffers read by the generated score transform
};

constexpr int BQ = 128, BKV = 128;          // head dim 128
constexpr int TILE = 128 * 128 * 2;                 // one 128 x 128 bf16 tile = two 16 KB halves
// shared memory: Q x 2, K x 2 stages, V x 2 stages, 1 KB of alignment slack, barriers (the host's attn_smem_bytes())

// 32 consecutive columns of one TMEM lane per thread, without waiting for them ...
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// ... and the wait.  The registers are passed through it so that no use of them is scheduled before it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
        "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
        "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
        "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
      :: "memory");
}

// 16 consecutive columns of one TMEM lane per thread, written without waiting for the write
__device__ __forceinline__ void tmem_st16_issue(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (row = lane, two 16-bit
// elements of consecutive k per 32-bit column)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One score after the generated transform.  MODE 0: the variant of the transform without its causal
// mask (the caller knows the mask holds), 1: the transform, 2: the transform, and keys >= sk give -inf.
template <class Xform, int MODE>
__device__ __forceinline__ float score_of(uint32_t raw, long long bh, long long qi, long long kj, const AttnParams& p) {
  if (MODE == 0) return Xform::plain(__uint_as_float(raw), bh, qi, kj, p.ep);
  float x = Xform::apply(__uint_as_float(raw), bh, qi, kj, p.ep);
  if (MODE == 2) x = (kj < p.sk) ? x : -NXB_INF;
  return x;
}

// Maximum of the 128 transformed scores of this thread's row.  On entry the load of columns 0..31
// into `xa` is in flight; on exit the same load has been started again (for row_probs).  While one
// block of 32 is worked on the next one is on its way.  The loops over blocks stay rolled (two blocks
// per trip, for the two buffers): unrolled, the softmax of one key block is about 18 KB of straight-line
// code per warp, and the warps then wait for instruction fetch more than for anything else.
template <class Xform, int MODE>
__device__ __forceinline__ void max32(float (&mxs)[4], const uint32_t (&x)[32], int bh, long long qi, long long kj, const AttnParams& p) {
  if constexpr (MODE == 3) {
    // raw scores (the transform is a multiplication by a positive constant, applied to the maximum later)
#if NXB_NVRTC_VERSION >= 1209
    // three-input max: PTX ISA 8.8
#pragma unroll
    for (int e = 0; e < 32; e += 2)
      asm("max.NaN.f32 %0, %0, %1, %2;" : "+f"(mxs[(e >> 1) & 3]) : "f"(__uint_as_float(x[e])), "f"(__uint_as_float(x[e + 1])));
#else
#pragma unroll
    for (int e = 0; e < 32; ++e) mxs[e & 3] = nx_max(mxs[e & 3], __uint_as_float(x[e]));
#endif
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) mxs[e & 3] = nx_max(mxs[e & 3], score_of<Xform, MODE>(x[e], bh, qi, kj + e, p));
  }
}
template <class Xform, int MODE>
__device__ __forceinline__ float row_max(uint32_t tS, uint32_t (&xa)[32], uint32_t (&xc)[32], int bh, long long qi, long long kj0, const AttnParams& p) {
  float mxs[4] = {-NXB_INF, -NXB_INF, -NXB_INF, -NXB_INF};
#pragma unroll 1
  for (int cc = 0; cc < 2; ++cc) {
    tmem_ld_wait(xa);
    tmem_ld32_issue(tS + (uint32_t)(cc * 64 + 32), xc);
    max32<Xform, MODE>(mxs, xa, bh, qi, kj0 + cc * 64, p);
    tmem_ld_wait(xc);
    tmem_ld32_issue(tS + (uint32_t)((cc * 64 + 64) & 127), xa);
    max32<Xform, MODE>(mxs, xc, bh, qi, kj0 + cc * 64 + 32, p);
  }
  const float mx = nx_max(nx_max(mxs[0], mxs[1]), nx_max(mxs[2], mxs[3]));
  return MODE == 3 ? mx * Xform::scale() : mx;
}

// Probabilities ex2(x * log2(e) + off) of 32 scores, in bf16 pairs into 16 columns of the row's lane of
// tensor memory at `tP` (the A operand of P V), and their sums.
template <class Xform, int MODE>
__device__ __forceinline__ void probs32(float (&ls)[4], const uint32_t (&x)[32], int bh, long long qi, long long kj, const AttnParams& p,
                                        float off, uint32_t tP) {
  uint32_t pk16[16];
  constexpr float LOG2E = 1.4426950408889634f;
  if constexpr (MODE == 3) {
    // ex2(s * (scale * log2 e) + off), two scores per multiply-add and per addition (f32x2)
    const float c2 = Xform::scale() * LOG2E;
    unsigned long long cc, oo;
    asm("mov.b64 %0, {%1, %1};" : "=l"(cc) : "f"(c2));
    asm("mov.b64 %0, {%1, %1};" : "=l"(oo) : "f"(off));
    unsigned long long acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) asm("mov.b64 %0, {%1, %2};" : "=l"(acc[u]) : "f"(ls[u]), "f"(0.f));
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t (&pk)[4] = reinterpret_cast<uint32_t (&)[4]>(pk16[g * 4]);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = g * 8 + u * 2;
        unsigned long long xx, yy;
        asm("mov.b64 %0, {%1, %2};" : "=l"(xx) : "r"(x[e]), "r"(x[e + 1]));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(yy) : "l"(xx), "l"(cc), "l"(oo));
        float y0, y1;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(y0), "=f"(y1) : "l"(yy));
        const float e0 = nx_exp2(y0), e1 = nx_exp2(y1);
        unsigned long long ee;
        asm("mov.b64 %0, {%1, %2};" : "=l"(ee) : "f"(e0), "f"(e1));
        asm("add.rn.f32x2 %0, %0, %1;" : "+l"(acc[u]) : "l"(ee));
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk[u]) : "f"(e1), "f"(e0));
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float a0, a1;
      asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(acc[u]));
      ls[u] = a0 + a1;
    }
  } else {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t (&pk)[4] = reinterpret_cast<uint32_t (&)[4]>(pk16[g * 4]);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = g * 8 + u * 2;
        const float e0 = nx_exp2(fmaf(score_of<Xform, MODE>(x[e], bh, qi, kj + e, p), LOG2E, off));
        const float e1 = nx_exp2(fmaf(score_of<Xform, MODE>(x[e + 1], bh, qi, kj + e + 1, p), LOG2E, off));
        ls[u] += e0 + e1;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk[u]) : "f"(e1), "f"(e0));
      }
    }
  }
  tmem_st16_issue(tP, pk16);
}
// The whole row.  On entry the load of columns 0..31 into `xa` is in flight.  P overwrites the first 64
// columns of the scores it was computed from: the 16 columns of block c lie below the columns of block
// c + 1, the only ones still to be read when they are written.
template <class Xform, int MODE>
__device__ __forceinline__ float row_probs(uint32_t tS, uint32_t (&xa)[32], uint32_t (&xc)[32], int bh, long long qi, long long kj0, const AttnParams& p,
                                           float off) {
  float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
  for (int cc = 0; cc < 2; ++cc) {
    tmem_ld_wait(xa);
    tmem_ld32_issue(tS + (uint32_t)(cc * 64 + 32), xc);
    probs32<Xform, MODE>(ls, xa, bh, qi, kj0 + cc * 64, p, off, tS + (uint32_t)(cc * 32));
    tmem_ld_wait(xc);
    if (cc == 0) tmem_ld32_issue(tS + 64u, xa);
    probs32<Xform, MODE>(ls, xc, bh, qi, kj0 + cc * 64 + 32, p, off, tS + (uint32_t)(cc * 32 + 16));
  }
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  return (ls[0] + ls[1]) + (ls[2] + ls[3]);
}

template <class Xform>
__device__ __forceinline__ void attn_body(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, const AttnParams& p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = base + 2 * TILE, sV = sK + 2 * TILE;
  const uint32_t bars = sV + 2 * TILE;
  // barriers (8 bytes each): q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], then per tile s_full, p_full, pv_full
  const uint32_t q_full = bars, k_full0 = bars + 8, k_empty0 = bars + 24, v_full0 = bars + 40, v_empty0 = bars + 56;
  const uint32_t s_full0 = bars + 72, p_full0 = bars + 88, pv_full0 = bars + 104, tmem_slot = bars + 120;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + (tmem_slot - base));
  volatile int* abort_flag = (volatile int*)(gen_base + (tmem_slot - base) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // pairs of query blocks, heavy (late) pairs first: with a causal mask block i needs i+1 key blocks.
  // Tile 0 is the later block of the pair, tile 1 the one before it (absent for the last pair of an odd count).
  const int nqb = (p.sq + BQ - 1) / BQ;                 // (nqb + 1) / 2 pairs per (batch, head): the grid's second factor
  // The grid runs in block order: the heaviest pair of every (batch, head) first, the lightest last, so
  // that the last wave is made of short CTAs (measured at {8,32,2048,128}: 0.38 ms against 0.40 with the
  // pairs of one (batch, head) next to each other, although keys and values are then fetched once per pair).
  const int pi = (int)(blockIdx.x / (unsigned)p.batch_heads);
  const int bh = (int)(blockIdx.x % (unsigned)p.batch_heads);
  const int qb0 = nqb - 1 - 2 * pi;
  const int ntiles = qb0 >= 1 ? 2 : 1;
  const int nkv_all = (p.sk + BKV - 1) / BKV;
  int nkv[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0t = (qb0 - t) * BQ;
    nkv[t] = nkv_all;
    if (p.causal) { const int lim = (q0t + BQ - 1) / BKV + 1; if (lim < nkv[t]) nkv[t] = lim; }
    if (t >= ntiles) nkv[t] = 0;
  }
  const int nkv_max = nkv[0] > nkv[1] ? nkv[0] : nkv[1];

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1);
      mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full0 + 8 * t, 1);
      mbar_init(p_full0 + 8 * t, 4);
      mbar_init(pv_full0 + 8 * t, 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, (uint32_t)(ntiles * TILE));
      for (int t = 0; t < ntiles; ++t) {
        tma_load_3d(sQ + t * TILE, &map_q, q_full, 0, (qb0 - t) * BQ, bh);
        tma_load_3d(sQ + t * TILE + TILE / 2, &map_q, q_full, 64, (qb0 - t) * BQ, bh);
      }
      auto load_k = [&](int j) {
        const int s = j & 1;
        if (!mbar_wait(k_empty0 + 8 * s, (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag)) return false;
        mbar_expect_tx(k_full0 + 8 * s, TILE);
        tma_load_3d(sK + s * TILE, &map_k, k_full0 + 8 * s, 0, j * BKV, bh);
        tma_load_3d(sK + s * TILE + TILE / 2, &map_k, k_full0 + 8 * s, 64, j * BKV, bh);
        return true;
      };
      auto load_v = [&](int j) {
        const int s = j & 1;
        if (!mbar_wait(v_empty0 + 8 * s, (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag)) return false;
        mbar_expect_tx(v_full0 + 8 * s, TILE);
        // V_j: rows are keys, 64 head-dim elements per 128-byte row, one box per head-dim half.  The map
        // of V is four-dimensional (head dim, key, head, batch): V may be stored {batch, key, head, dim},
        // as a projection leaves it, without a transposed copy.
        tma_load_4d(sV + s * TILE, &map_v, v_full0 + 8 * s, 0, j * BKV, bh % p.heads, bh / p.heads);
        tma_load_4d(sV + s * TILE + TILE / 2, &map_v, v_full0 + 8 * s, 64, j * BKV, bh % p.heads, bh / p.heads);
        return true;
      };
      // both rings run one block ahead of the products: K_{j+1} and V_{j+1} are requested during step j
      bool ok = nkv_max > 0 && load_k(0) && load_v(0);
      for (int j = 1; j < nkv_max && ok; ++j) ok = load_k(j) && load_v(j);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // S = Q K^T: both K-major.  PV = P V: A K-major, B with N (head dim) contiguous.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_pv = idesc_s | (1u << 16);
      auto issue_s = [&](int t, int j) {
        const uint32_t k = sK + (j & 1) * TILE, q = sQ + t * TILE;
        const uint32_t d = tmem_base + (uint32_t)(t * 128);
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {
          const uint32_t half = (k8 >> 2) * (TILE / 2), off = (k8 & 3) * 2;      // 32 bytes per step inside a 64-wide half
          tc_mma(d, make_desc(q + half) + off, make_desc(k + half) + off, idesc_s, k8 > 0 ? 1u : 0u, false);
        }
        tc_commit(s_full0 + 8 * t);
      };
      bool ok = nkv_max > 0 && mbar_wait(q_full, 0, abort_flag) && mbar_wait(k_full0, 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < ntiles; ++t) issue_s(t, 0);
        tc_commit(k_empty0);
      }
      // Per key block and tile, back to back as soon as the tile's softmax has written P_t(j) over the
      // scores it came from:  PV_t(j) = P_t V_j  with P read from tensor memory, then  S_t(j+1)  into the
      // same columns (the tensor pipe executes in issue order, so the product that reads P is done with
      // it before the next scores land there).  The two tiles run half a step apart: one tile's products
      // execute under the other's softmax.
      auto issue_pv = [&](int t, int j) {
        const uint32_t v = sV + (j & 1) * TILE;
        const uint32_t d = tmem_base + 256u + (uint32_t)(t * 128), a = tmem_base + (uint32_t)(t * 128);
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {
          // A = P: 16 keys = 8 columns per step.  B = V: 8-key groups are 1024 bytes apart inside a
          // head-dim half (16 KB), the two halves 16 KB apart (leading offset).
          const uint64_t bdesc = ((uint64_t)(((v + k8 * 2048) & 0x3FFFF) >> 4)) | ((uint64_t)(16384 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
                                 ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
          tc_mma_ts(d, a + (uint32_t)(k8 * 8), bdesc, idesc_pv, (j > 0 || k8 > 0) ? 1u : 0u);
        }
      };
      for (int j = 0; j < nkv_max && ok; ++j) {
        const bool more = j + 1 < nkv_max;
        bool k_ready = false, v_ready = false;
        for (int t = 0; t < ntiles && ok; ++t) {
          if (j >= nkv[t]) continue;
          if (!v_ready) {
            if (!mbar_wait(v_full0 + 8 * (j & 1), (uint32_t)((j >> 1) & 1), abort_flag)) { ok = false; break; }
            v_ready = true;
          }
          if (!mbar_wait(p_full0 + 8 * t, (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, j);
          if (j + 1 < nkv[t]) {
            if (!k_ready) {
              if (!mbar_wait(k_full0 + 8 * ((j + 1) & 1), (uint32_t)(((j + 1) >> 1) & 1), abort_flag)) { ok = false; break; }
              k_ready = true;
            }
            issue_s(t, j + 1);              // its commit covers PV_t(j) too
          } else {
            tc_commit(pv_full0 + 8 * t);    // the tile's last product
          }
        }
        if (!ok) break;
        if (more) {
          // the producer loads K_{j+1} whenever there is a block j+1, also when only one tile still uses it
          if (!k_ready && !mbar_wait(k_full0 + 8 * ((j + 1) & 1), (uint32_t)(((j + 1) >> 1) & 1), abort_flag)) { ok = false; break; }
          tc_commit(k_empty0 + 8 * ((j + 1) & 1));
        }
        tc_commit(v_empty0 + 8 * (j & 1));
      }
    }
  } else {
    // softmax: warps 2..5 own tile 0, warps 6..9 tile 1; one thread per query row (= TMEM lane)
    const int q = warp & 3;
    const int t = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    const long long qi = (long long)(qb0 - t) * BQ + row;
    const long long b_idx = bh / p.heads, h_idx = bh % p.heads;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t tS = tmem_base + (uint32_t)(t * 128) + lane_addr, tO = tmem_base + 256u + (uint32_t)(t * 128) + lane_addr;
    const uint32_t s_full = s_full0 + 8 * t, p_full = p_full0 + 8 * t, pv_full = pv_full0 + 8 * t;
    const int my_nkv = nkv[t];
    // The output row stays in its TMEM accumulator: PV products accumulate there, and it is only
    // read back and rescaled when the running maximum moves by more than RESCALE_STEP (until then
    // the old maximum keeps being used, so probabilities may reach e^RESCALE_STEP = 256, far inside
    // bf16's range; the final division by the sum makes the result independent of that choice).
    constexpr float LOG2E = 1.4426950408889634f, RESCALE_STEP = 5.545177444f;
    float m = -NXB_INF, l = 0.f;
    bool ok = true;
    const long long q_first = (long long)(qb0 - t) * BQ;
    for (int j = 0; j < my_nkv && ok; ++j) {
      // one lane polls on behalf of its warp; the tensor-memory loads below need the whole warp
      if (!mbar_wait_warp_tight(s_full, (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      const long long kj0 = (long long)j * BKV;
      // how the scores of this block are read: 0 = the mask is known to hold for every element (a block
      // entirely below a proven causal diagonal) and all keys exist, 1 = the full transform, all keys
      // exist, 2 = the full transform and columns beyond the last key contribute nothing, 3 = as 0 when the
      // unmasked transform is a multiplication by a positive constant (folded into the exponent's multiply-add)
      const bool unmasked = Xform::kPlainAlways || (Xform::kHasPlain && p.causal && kj0 + BKV - 1 <= q_first);
      const int mode = (kj0 + BKV > p.sk) ? 2 : !unmasked ? 1 : Xform::kScaleOnly ? 3 : Xform::kHasPlain ? 0 : 1;
      // A row's 128 scores are read from tensor memory twice, 32 at a time: once for the maximum, once
      // for the probabilities.  Holding all 128 (plus the packed probabilities) in registers does not
      // fit beside three warps per scheduler, and spilled scores cost more than the second read.
      uint32_t xa[32], xc[32];
      float mx;
      tmem_ld32_issue(tS, xa);
      if (mode == 3) mx = row_max<Xform, 3>(tS, xa, xc, bh, qi, kj0, p);
      else if (mode == 0) mx = row_max<Xform, 0>(tS, xa, xc, bh, qi, kj0, p);
      else if (mode == 1) mx = row_max<Xform, 1>(tS, xa, xc, bh, qi, kj0, p);
      else mx = row_max<Xform, 2>(tS, xa, xc, bh, qi, kj0, p);
      // (the last step of row_max started the load of columns 0..31 again, into xa)
      const float m_seen = nx_max(m, mx);
      const bool move = m_seen > m + RESCALE_STEP || m == -NXB_INF;
      const float m_use = move ? m_seen : m;
      if (j > 0) {
        // S_t(j) was issued after PV_t(j-1) and its completion (s_full) covers it: O may be touched
        if (__any_sync(0xffffffffu, move && m != -NXB_INF)) {
          const float alpha = (move && m != -NXB_INF) ? nx_exp2(m * LOG2E - m_use * LOG2E) : 1.f;
          tmem_ld_wait(xa);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t ov[32];
            tmem_ld32(tO + (uint32_t)(c * 32), ov);
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
            tmem_st32(tO + (uint32_t)(c * 32), ov);
          }
          l *= alpha;
        }
      }
      m = m_use;
      // probabilities of the 128 keys (one FMA and one ex2 each), their sum, and P in bf16 over the
      // first 64 columns of the scores: the A operand of PV.  A fully masked row has m = -inf: every x
      // is -inf too, and with a zero offset ex2(-inf) = 0 without a NaN.
      const float off = (m == -NXB_INF) ? 0.f : -m * LOG2E;
      float ls;
      if (mode == 3) ls = row_probs<Xform, 3>(tS, xa, xc, bh, qi, kj0, p, off);
      else if (mode == 0) ls = row_probs<Xform, 0>(tS, xa, xc, bh, qi, kj0, p, off);
      else if (mode == 1) ls = row_probs<Xform, 1>(tS, xa, xc, bh, qi, kj0, p, off);
      else ls = row_probs<Xform, 2>(tS, xa, xc, bh, qi, kj0, p, off);
      l += ls;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && my_nkv > 0) {
      // the tile's last product commits pv_full (once)
      if (mbar_wait_warp_tight(pv_full, 0u, abort_flag)) {
        tc_fence_after();
        const float inv = 1.f / l;
        unsigned short* out = (unsigned short*)p.out + b_idx * p.out_bh_hi + h_idx * p.out_bh_lo + qi * p.out_row;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tmem_ld32(tO + (uint32_t)(c * 32), ov);
          if (qi < p.sq) {
#pragma unroll
            for (int d = 0; d < 32; d += 8) {
              uint4 w;
              uint32_t* ww = &w.x;
#pragma unroll
              for (int e = 0; e < 4; ++e)
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(ww[e]) : "f"(__uint_as_float(ov[d + 2 * e + 1]) * inv), "f"(__uint_as_float(ov[d + 2 * e]) * inv));
              *reinterpret_cast<uint4*>(out + c * 32 + d) = w;
            }
          }
        }
      }
    }
    tc_fence_before();
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) *(volatile int*)p.status = 1;
    const long long t0 = now_cycles();
    while (now_cycles() - t0 < 400000ll) { }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

}  // namespace nxb_attn

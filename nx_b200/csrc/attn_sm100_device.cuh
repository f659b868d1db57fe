// Fused attention for sm_100a:  O = softmax(f(Q K^T)) V  without writing the scores to memory.
//
// The planner recognises  dot(q,k) -> elementwise f (scale, mask ...) -> softmax over the key
// axis -> dot(p,v)  in a defn graph and generates this kernel with `f` compiled in as
// AttnXform::apply.  One CTA owns 128 query rows of one (batch, head) pair and walks the key
// blocks of 128:
//   warp 0      TMA producer: Q once, then K_j / V_j into a two-stage ring
//   warp 1      MMA issuer:   S_j = Q K_j^T into one of two TMEM accumulators (so the next
//               block's scores are computed while this block's softmax runs), then
//               PV_j = P_j V_j into a third accumulator (P from shared memory, V with its
//               head-dim index contiguous, i.e. an MN-major B operand)
//   warps 2..9  softmax, two threads per query row (a row lives in one TMEM lane; each thread
//               owns 64 key columns and 64 head dims, the halves exchange maxima through shared
//               memory): running maximum m and running sum l; the output row O accumulates in
//               TMEM across key blocks and is read back and rescaled only when the maximum
//               moves by more than a threshold (rare after the first blocks)
// Keys beyond a causal diagonal are skipped block-wise when the planner proved the mask is
// causal.  Every mbarrier wait is bounded; on expiry the CTA raises an abort flag, all roles
// leave their loops, tensor memory is released and the host reports NXB_ERR_TIMEOUT.
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
  int heads, batch_heads, sq, sk;
  int causal;          // 1: keys j > query i contribute nothing (proved by the planner)
  void* ep[14];        // buffers read by the generated score transform
};

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE = 128 * 128 * 2;                 // one 128 x 128 bf16 tile = two 16 KB halves
constexpr int ATTN_SMEM = TILE /*Q*/ + 2 * 2 * TILE /*K,V x 2 stages*/ + TILE /*P*/ + 1024 + 256 + 3072 /*exchange*/;

template <class Xform>
__device__ __forceinline__ void attn_body(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, const AttnParams& p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sKV = base + TILE, sP = sKV + 4 * TILE;
  const uint32_t bars = sP + TILE;
  // barriers: q_full, kv_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, pv_full
  const uint32_t q_full = bars, kv_full0 = bars + 8, kv_empty0 = bars + 24, s_full0 = bars + 40, s_empty0 = bars + 56,
                 p_full = bars + 72, pv_full = bars + 80, xchg_bar = bars + 88, tmem_slot = bars + 96;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + (tmem_slot - base));
  volatile int* abort_flag = (volatile int*)(gen_base + (tmem_slot - base) + 8);
  // exchange areas of the softmax half-rows: maxima [parity][half][row], sums [half][row]
  volatile float* xmax = (volatile float*)(gen_base + (bars - base) + 256);
  volatile float* xsum = xmax + 2 * 2 * 128;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query blocks first: with a causal mask block i needs i+1 key blocks
  const int nqb = (p.sq + BQ - 1) / BQ;
  const int qb = nqb - 1 - (int)(blockIdx.x % nqb);
  const int bh = (int)(blockIdx.x / nqb);
  const int q0 = qb * BQ;
  int nkv = (p.sk + BKV - 1) / BKV;
  if (p.causal) { int lim = (q0 + BQ - 1) / BKV + 1; if (lim < nkv) nkv = lim; }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); mbar_init(s_full0 + 8 * s, 1); mbar_init(s_empty0 + 8 * s, 8); }
    mbar_init(p_full, 8);
    mbar_init(pv_full, 1);
    mbar_init(xchg_bar, 8);
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
  const uint32_t tS0 = tmem_base, tPV = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE);
      tma_load_3d(sQ, &map_q, q_full, 0, q0, bh);
      tma_load_3d(sQ + TILE / 2, &map_q, q_full, 64, q0, bh);
      uint32_t ph = 0;
      for (int j = 0; j < nkv; ++j) {
        const int s = j & 1;
        if (!mbar_wait(kv_empty0 + 8 * s, ph ^ 1, abort_flag)) break;
        mbar_expect_tx(kv_full0 + 8 * s, 2 * TILE);
        const uint32_t k = sKV + s * 2 * TILE, v = k + TILE;
        tma_load_3d(k, &map_k, kv_full0 + 8 * s, 0, j * BKV, bh);
        tma_load_3d(k + TILE / 2, &map_k, kv_full0 + 8 * s, 64, j * BKV, bh);
        // V_j: rows are keys, 64 head-dim elements per 128-byte row, one box per head-dim half
        tma_load_3d(v, &map_v, kv_full0 + 8 * s, 0, j * BKV, bh);
        tma_load_3d(v + TILE / 2, &map_v, kv_full0 + 8 * s, 64, j * BKV, bh);
        if (s == 1) ph ^= 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // S = Q K^T: both K-major.  PV = P V: A K-major, B with N (head dim) contiguous.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_pv = idesc_s | (1u << 16);
      auto issue_s = [&](int j) {
        const uint32_t k = sKV + (j & 1) * 2 * TILE;
        const uint32_t d = tS0 + (uint32_t)((j & 1) * 128);
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {
          const uint32_t half = (k8 >> 2) * (TILE / 2), off = (k8 & 3) * 2;      // 32 bytes per step inside a 64-wide half
          tc_mma(d, make_desc(sQ + half) + off, make_desc(k + half) + off, idesc_s, k8 > 0 ? 1u : 0u, false);
        }
        tc_commit(s_full0 + 8 * (j & 1));
      };
      bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(kv_full0, 0, abort_flag);
      if (ok) { tc_fence_after(); issue_s(0); }
      uint32_t kvph[2] = {0, 0}, seph[2] = {0, 0};
      kvph[0] = 1;             // stage 0 was consumed once above
      for (int j = 0; j < nkv && ok; ++j) {
        if (j + 1 < nkv) {
          const int s = (j + 1) & 1;
          if (!mbar_wait(kv_full0 + 8 * s, kvph[s], abort_flag)) { ok = false; break; }
          kvph[s] ^= 1;
          if (j + 1 >= 2) {     // the S buffer was used by block j-1: wait until the softmax has read it
            if (!mbar_wait(s_empty0 + 8 * s, seph[s], abort_flag)) { ok = false; break; }
            seph[s] ^= 1;
          }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(p_full, (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v = sKV + (j & 1) * 2 * TILE + TILE;
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {
          // A = P: two 64-key halves, 32 bytes per step.  B = V: 8-key groups are 1024 bytes apart
          // inside a head-dim half (16 KB), the two halves 16 KB apart (leading offset).
          const uint64_t adesc = make_desc(sP + (k8 >> 2) * (TILE / 2)) + (uint64_t)((k8 & 3) * 2);
          const uint64_t bdesc = ((uint64_t)(((v + k8 * 2048) & 0x3FFFF) >> 4)) | ((uint64_t)(16384 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
                                 ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
          tc_mma(tPV, adesc, bdesc, idesc_pv, (j > 0 || k8 > 0) ? 1u : 0u, false);
        }
        tc_commit(pv_full);
        tc_commit(kv_empty0 + 8 * (j & 1));
      }
    }
  } else {
    // softmax: 8 warps, two threads per query row.  Warps 2..5 take key columns / head dims 0..63
    // of their TMEM lane quarter, warps 6..9 take 64..127; the two halves of a row exchange their
    // maxima (and, at the end, their sums) through shared memory.
    const int q = warp & 3;
    const int hf = (warp - 2) >> 2;
    const int row = q * 32 + lane;                 // query row inside the block == TMEM lane
    const long long qi = (long long)q0 + row;
    const long long b_idx = bh / p.heads, h_idx = bh % p.heads;
    const uint32_t lane_addr = ((uint32_t)(q * 32) << 16) + (uint32_t)(hf * 64);
    // The output row stays in its TMEM accumulator: PV products accumulate there, and it is only
    // read back and rescaled when the running maximum moves by more than RESCALE_STEP (until then
    // the old maximum keeps being used, so probabilities may reach e^RESCALE_STEP = 256, far inside
    // bf16's range; the final division by the sum makes the result independent of that choice).
    constexpr float LOG2E = 1.4426950408889634f, RESCALE_STEP = 5.545177444f;
    float m = -NXB_INF, l = 0.f;
    uint32_t sfph[2] = {0, 0};
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      const int s = j & 1;
      // one lane polls on behalf of its warp; the tensor-memory loads below need the whole warp
      if (!mbar_wait_warp_tight(s_full0 + 8 * s, sfph[s], abort_flag)) { ok = false; break; }
      sfph[s] ^= 1;
      tc_fence_after();
      const uint32_t tS = tS0 + (uint32_t)(s * 128) + lane_addr;
      uint32_t sv[64];
      tmem_ld32x2(tS, sv);
      float x[64];
      float mx = -NXB_INF;
      const long long kj0 = (long long)j * BKV + hf * 64;
      if (kj0 + 64 <= p.sk) {
#pragma unroll
        for (int t = 0; t < 64; ++t) {
          x[t] = Xform::apply(__uint_as_float(sv[t]), (long long)bh, qi, kj0 + t, p.ep);
          mx = nx_max(mx, x[t]);
        }
      } else {
        // the last key block: columns beyond the keys contribute nothing
#pragma unroll
        for (int t = 0; t < 64; ++t) {
          const float xv = Xform::apply(__uint_as_float(sv[t]), (long long)bh, qi, kj0 + t, p.ep);
          x[t] = (kj0 + t < p.sk) ? xv : -NXB_INF;
          mx = nx_max(mx, x[t]);
        }
      }
      // exchange the half-row maxima (double buffered by block parity: one bounded wait per block)
      xmax[(s * 2 + hf) * 128 + row] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(xchg_bar);
      if (!mbar_wait_warp_tight(xchg_bar, (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
      const float m_seen = nx_max(m, nx_max(mx, xmax[(s * 2 + (hf ^ 1)) * 128 + row]));
      // both threads of a row take the same decision: they see the same three numbers
      const bool move = m_seen > m + RESCALE_STEP || m == -NXB_INF;
      const float m_use = move ? m_seen : m;
      if (j > 0) {
        // PV of the previous block is complete: P's buffer is free, and O may be touched
        if (!mbar_wait_warp_tight(pv_full, (uint32_t)((j - 1) & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, move && m != -NXB_INF)) {
          const float alpha = (move && m != -NXB_INF) ? nx_exp2(m * LOG2E - m_use * LOG2E) : 1.f;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t ov[32];
            tmem_ld32(tPV + lane_addr + (uint32_t)(c * 32), ov);
#pragma unroll
            for (int t = 0; t < 32; ++t) ov[t] = __float_as_uint(__uint_as_float(ov[t]) * alpha);
            tmem_st32(tPV + lane_addr + (uint32_t)(c * 32), ov);
          }
          l *= alpha;
        }
      }
      m = m_use;
      // probabilities of my 64 keys (one FMA and one ex2 each), their sum, and P in bf16: exactly
      // one 64-key half of the A operand.  A fully masked row has m = -inf: every x is -inf too,
      // and with a zero offset ex2(-inf) = 0 without a NaN.
      const float off = (m == -NXB_INF) ? 0.f : -m * LOG2E;
      const uint32_t rowbase = sP + (uint32_t)hf * (TILE / 2) + (uint32_t)row * 128u;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        uint32_t pk[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float e0 = nx_exp2(fmaf(x[g * 8 + u * 2], LOG2E, off));
          const float e1 = nx_exp2(fmaf(x[g * 8 + u * 2 + 1], LOG2E, off));
          l += e0 + e1;
          asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk[u]) : "f"(e1), "f"(e0));
        }
        const uint32_t dst = rowbase + (((uint32_t)g ^ (uint32_t)(row & 7)) * 16u);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(s_empty0 + 8 * s); mbar_arrive(p_full); }
    }
    if (ok && nkv > 0) {
      if (mbar_wait_warp_tight(pv_full, (uint32_t)((nkv - 1) & 1), abort_flag)) {
        tc_fence_after();
        // total of the two half-row sums
        xsum[hf * 128 + row] = l;
        __syncwarp();
        if (lane == 0) mbar_arrive(xchg_bar);
        if (mbar_wait_warp_tight(xchg_bar, (uint32_t)(nkv & 1), abort_flag)) {
          const float inv = 1.f / (l + xsum[(hf ^ 1) * 128 + row]);
          unsigned short* out = (unsigned short*)p.out + b_idx * p.out_bh_hi + h_idx * p.out_bh_lo + qi * p.out_row + hf * 64;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t ov[32];
            tmem_ld32(tPV + lane_addr + (uint32_t)(c * 32), ov);
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

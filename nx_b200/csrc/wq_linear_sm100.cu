// Weight-only quantised linear for small batches on sm_100a:
//
//   y[m][n] = S[n] * sum_k x[m][k] * W[n][k]       x bf16 {M,K}, W s8 {N,K}, S f32 {N}, M <= 512
//
// With few rows of x the layer is a stream over W (N*K bytes), so W must cross HBM exactly once
// and never exist as 16-bit values in memory.  The product is computed transposed: a CTA owns a
// band of output channels n (the M side of the tensor-core tile, one TMEM lane each) and up to
// 256 rows of x (the N side), so every weight is converted once.  The band is ceil(N / SMs)
// channels wide (at most 128): every SM gets one, because what bounds the kernel is the work per
// SM on the stream (bytes to pull, weights to convert), not the tensor pipe, which runs its
// 128-lane instruction just as fast on a band that fills 75 lanes.
//   warp 0      TMA producer: per 64-wide k block the raw s8 tile of W (band rows x 64 bytes,
//               64-byte swizzle) and the bf16 tile of x (128-byte swizzle; rows beyond M arrive
//               as zeros) into a deep ring (up to 16 stages: the stream is latency bound, a CTA
//               needs ~100 KB in flight to draw its share of the memory bandwidth)
//   12 warps    converters (every warp outside scheduler partition 0): s8 -> bf16 (exact), written
//               as 128-byte-swizzled K-major A tiles into a second ring.  Three groups of four warps
//               take the ring stages round-robin; a stage holds up to four k blocks, because what a
//               hand-over between the roles costs (barrier polls, proxy fence: ~800 cycles per pass,
//               ~230 cycles per copy instruction, ~100 per MMA instruction) does not depend on how
//               much data it covers.  Afterwards the same warps are the epilogue (tcgen05.ld, scale
//               per lane, store)
//   warps 4,8,12 MMA issuers (scheduler partition 0, like the producer): one thread each (three
//               for narrow batches, else one), k blocks round-robin, own accumulators; tcgen05.mma
//               M=128, N=padded batch, K=16, f32 accumulators in TMEM summed by the epilogue
// (The weights cannot be handed over as f16, which would convert in half the instructions: an
// instruction descriptor with A in f16 and B in bf16 is rejected as an illegal instruction.)
// Every mbarrier wait is bounded; a stalled wait raises the abort flag, all roles leave their
// loops, tensor memory is released and the host reports NXB_ERR_TIMEOUT.
#include <cuda.h>

#include "gemm.h"
#include "gemm_sm100_device.cuh"

namespace nxb {
namespace {

using namespace nxb_gemm;

struct WqParams {
  void* out;
  const float* scale;
  int* status;
  int m, n, k;
  int mb;        // rows of x per CTA: a multiple of 16, at most 256
  int ch;        // output channels per CTA (rows of the W tile): a multiple of 8, at most 128
  int g;         // k blocks of 64 per ring stage (one hand-over between the roles per stage): 1, 2 or 4
  int raw_bytes; // bytes of the raw W part of a stage: g slabs of ch x 64, rounded up to 1024
  int conv_slab; // bytes of one converted tile: ch rows of 128 bytes, rounded up to 1024
  int blocked;   // the tensor maps count k blocks in their third coordinate (else: k offset in the first, g == 1)
  int out_dt;
  int stages;    // depth of the {raw W, x} ring
  int conv_stages;   // depth of the converted-tile ring
  int tmem_cols;
  int issuers;   // threads issuing MMAs (1 or 2, alternate k blocks)
  int nacc;      // accumulators used round-robin by consecutive MMAs (summed in the epilogue)
};

constexpr int WQ_RAW = 128 * 64;      // s8 tile of W, 64 bytes per row
constexpr int WQ_WB = 128 * 128;      // the same tile as bf16, 128 bytes per row
constexpr int WQ_MAX_STAGES = 16;
constexpr int WQ_MAX_CONV_STAGES = 8;  // converted tiles between the converters and the MMA issuer
constexpr int WQ_SMEM_LIMIT = 232448 - 1024 - 512;

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// four signed bytes (k0..k3 of one channel) -> bf16 pairs (k0,k1), (k2,k3), exact.  With
// v = lo - 128*b7, both 128 + lo and -(128 + 128*b7) are bf16 bit patterns made by one logic operation
// each (0x4300 | low bits, 0xC300 | bit 7), and their bf16x2 sum is exact.  Six integer
// instructions and two bf16x2 fused multiply-adds per word; the integer pipe runs at half rate, which
// is what the instruction count is chosen for.
__device__ __forceinline__ void s8x4_to_bf16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t l0 = __byte_perm(w, 0u, 0x4140), l1 = __byte_perm(w, 0u, 0x4342);      // (k0, k1) and (k2, k3) in 16-bit lanes
  const uint32_t p0 = (l0 & 0x007F007Fu) | 0x43004300u, c0 = (l0 & 0x00800080u) | 0xC300C300u;
  const uint32_t p1 = (l1 & 0x007F007Fu) | 0x43004300u, c1 = (l1 & 0x00800080u) | 0xC300C300u;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(lo) : "r"(p0), "r"(0x3F803F80u), "r"(c0));
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(hi) : "r"(p1), "r"(0x3F803F80u), "r"(c1));
}

constexpr int WQ_THREADS = 512;
constexpr int WQ_MMA_WARP = 4;      // same scheduler partition as the producer (warp 0): none of the busy converter warps run there

__global__ void __launch_bounds__(WQ_THREADS, 1)
wq_linear_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, WqParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // a ring stage holds g k blocks: [g slabs of raw W, ch x 64 bytes each][g slabs of x, mb x 128 bytes each];
  // a stage of the converted ring holds g tiles of ch rows x 128 bytes.  The converted ring comes first:
  // the MMA reads 128 rows of every tile, and what it reads beyond the band (the next tile, or the start
  // of the other ring) only reaches accumulator lanes that are never stored.
  const uint32_t x_bytes = (uint32_t)p.mb * 128u, raw_slab = (uint32_t)p.ch * 64u;
  const uint32_t stage_bytes = (uint32_t)p.raw_bytes + (uint32_t)p.g * x_bytes;
  const uint32_t conv_slab = (uint32_t)p.conv_slab, conv_bytes = (uint32_t)p.g * conv_slab;
  const uint32_t wb0 = base;
  const uint32_t ring0 = base + (uint32_t)p.conv_stages * conv_bytes;
  const uint32_t bars = ring0 + (uint32_t)p.stages * stage_bytes;
  const uint32_t full0 = bars, empty0 = bars + 128, conv0 = bars + 256, wbe0 = bars + 320, acc_full = bars + 384, tmem_slot = bars + 392;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + (tmem_slot - base));
  volatile int* abort_flag = (volatile int*)(gen_base + (tmem_slot - base) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (int)blockIdx.x * p.ch, m0 = (int)blockIdx.y * p.mb;
  const int kblocks = (p.k + 63) / 64;
  const int nst = (kblocks + p.g - 1) / p.g;       // ring stages to go through; k blocks beyond the last arrive as zeros

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int c = 0; c < p.conv_stages; ++c) { mbar_init(conv0 + 8 * c, 4); mbar_init(wbe0 + 8 * c, 1); }
    mbar_init(acc_full, p.issuers);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == WQ_MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(p.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // MMA issue by one thread each of up to three warps (4, 8, 12) that take the k blocks round-robin.
  // With a narrow N an MMA is a few cycles of tensor work, so the rate at which a single thread can
  // issue them (and commit the stages back) paces the kernel; more issuers, each with its own
  // accumulators, raise it.
  auto issue_mmas = [&](int which) {
    // bf16 x bf16 -> f32, both operands K-major, M = 128 channels, N = padded batch
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.mb >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const int step = p.issuers;
    const int my_acc = p.nacc / p.issuers;
    const uint32_t acc0 = tmem_base + (uint32_t)(which * my_acc * p.mb), acc_end = acc0 + (uint32_t)(my_acc * p.mb);
    uint32_t acc = acc0;
    int fresh = my_acc;                       // accumulators not written yet
    int s = which % p.stages, c = which % p.conv_stages;
    uint32_t cph = (uint32_t)((which / p.conv_stages) & 1);
    bool ok = true;
    for (int st = which; st < nst; st += step) {
      // the converters arrive on conv only after the stage's TMA data (x included) has landed
      if (!mbar_wait(conv0 + 8 * c, cph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      for (int gi = 0; gi < p.g; ++gi) {
        const uint64_t adesc = make_desc(wb0 + (uint32_t)c * conv_bytes + (uint32_t)gi * conv_slab);
        const uint64_t bdesc = make_desc(ring0 + (uint32_t)s * stage_bytes + (uint32_t)p.raw_bytes + (uint32_t)gi * x_bytes);
        // consecutive MMAs go to different accumulators: accumulating into the columns the
        // previous one is still writing would serialise them on the pipeline's latency
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          tc_mma(acc, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc, fresh > 0 ? 0u : 1u, false);
          if (fresh > 0) --fresh;
          acc += (uint32_t)p.mb;
          if (acc == acc_end) acc = acc0;
        }
      }
      tc_commit(empty0 + 8 * s);
      tc_commit(wbe0 + 8 * c);
      s += step;
      while (s >= p.stages) s -= p.stages;
      c += step;
      while (c >= p.conv_stages) { c -= p.conv_stages; cph ^= 1; }
    }
    if (ok) tc_commit(acc_full);
  };

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int st = 0; st < nst; ++st) {
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag)) break;
        const uint32_t sb = ring0 + (uint32_t)s * stage_bytes;
        // one copy each for W and x: the third coordinate of both maps counts k blocks
        mbar_expect_tx(full0 + 8 * s, (uint32_t)p.g * (raw_slab + x_bytes));
        tma_load_3d(sb, &map_w, full0 + 8 * s, p.blocked ? 0 : st * 64, n0, p.blocked ? st * p.g : 0);
        tma_load_3d(sb + (uint32_t)p.raw_bytes, &map_x, full0 + 8 * s, p.blocked ? 0 : st * 64, m0, p.blocked ? st * p.g : 0);
        if (++s == p.stages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == WQ_MMA_WARP) {
    if (lane == 0) issue_mmas(0);
  } else {
    // warps 8 and 12 are the second and third issuer when the launch asks for them
    if ((warp & 3) == 0 && (warp >> 2) - 1 < p.issuers && lane == 0) issue_mmas((warp >> 2) - 1);
    __syncwarp();
    // The converter warps are the twelve outside scheduler partition 0 (where the producer and
    // the MMA issuers live: a single thread issuing MMAs loses most of its issue slots to busy
    // warps on the same scheduler).  Three groups of four warps take the ring stages round-robin:
    // one pass of a group (wait, load, convert, store, proxy fence, arrive) is some 800 cycles of
    // latency whatever the amount of data, so three passes are in flight at a time and each covers
    // g k blocks.  Within a group, thread t takes the 16-byte pieces t, t + 128, ... of the stage:
    // piece (k block, row, quarter) = 16 weights of one channel, written as 32 bytes of bf16.
    const bool converter = (warp & 3) != 0;
    const int ci = (warp >> 2) * 3 + (warp & 3) - 1;      // 0..11
    const int grp = ci >> 2;
    const int ct = (ci & 3) * 32 + lane;                  // 0..127 inside the group
    int s = grp % p.stages, cs = grp % p.conv_stages;
    uint32_t ph = (uint32_t)((grp / p.stages) & 1), cph = (uint32_t)((grp / p.conv_stages) & 1);
    bool ok = true;
    const int tasks = p.g * p.ch * 4;               // 16-byte pieces of raw W per stage
    for (int st = grp; converter && st < nst && ok; st += 3) {
      // one lane per warp polls the barriers
      int okw = 1;
      if (lane == 0) okw = mbar_wait_relaxed(full0 + 8 * s, ph, abort_flag) && mbar_wait_relaxed(wbe0 + 8 * cs, cph ^ 1, abort_flag);
      okw = __shfl_sync(0xffffffffu, okw, 0);
      __syncwarp();
      if (!okw) { ok = false; break; }
      const uint32_t sb = ring0 + (uint32_t)s * stage_bytes;
      const uint32_t wb = wb0 + (uint32_t)cs * conv_bytes;
#pragma unroll 2
      for (int t = ct; t < tasks; t += 128) {
        const int gi = t / (p.ch * 4), rc = t - gi * (p.ch * 4);
        const int r = rc >> 2, c = rc & 3;
        uint32_t w[4], o[8];
        const uint32_t src = sb + (uint32_t)gi * raw_slab + (uint32_t)r * 64u + (uint32_t)((c ^ ((r >> 1) & 3)) * 16);
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(src));
        s8x4_to_bf16x4(w[0], o[0], o[1]);
        s8x4_to_bf16x4(w[1], o[2], o[3]);
        s8x4_to_bf16x4(w[2], o[4], o[5]);
        s8x4_to_bf16x4(w[3], o[6], o[7]);
        const uint32_t row = wb + (uint32_t)gi * conv_slab + (uint32_t)r * 128u;
        const uint32_t d0 = row + (uint32_t)(((2 * c) ^ (r & 7)) * 16), d1 = row + (uint32_t)(((2 * c + 1) ^ (r & 7)) * 16);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d0), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d1), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(conv0 + 8 * cs);
      s += 3;
      while (s >= p.stages) { s -= p.stages; ph ^= 1; }
      cs += 3;
      while (cs >= p.conv_stages) { cs -= p.conv_stages; cph ^= 1; }
    }
    // epilogue: lane = output channel, columns = rows of x
    int acc_ok = 1;
    if (lane == 0) acc_ok = ok && mbar_wait_relaxed(acc_full, 0, abort_flag);
    acc_ok = __shfl_sync(0xffffffffu, acc_ok, 0);
    __syncwarp();
    if (acc_ok) {
      tc_fence_after();
      const int q = warp & 3;
      const long long n = (long long)n0 + q * 32 + lane;
      const bool mine = q * 32 + lane < p.ch && n < p.n;            // lanes beyond the band hold stale rows of the tile
      const float sc = mine ? p.scale[n] : 0.f;
      // TMEM quarter 0 is served by the two idle warps of partition 0 (8 and 12), the others by four warps each
      const int nshare = q == 0 ? 2 : 4, share = q == 0 ? (warp >> 2) - 2 : (warp >> 2);
      for (int c16 = share; c16 < p.mb / 16; c16 += nshare) {
        if (m0 + c16 * 16 >= p.m) break;                 // warp-uniform
        uint32_t v[16];
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c16 * 16), v);
        for (int a = 1; a < p.nacc; ++a) {
          uint32_t u[16];
          tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * p.mb + c16 * 16), u);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
        }
        if (mine) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const long long m = (long long)m0 + c16 * 16 + j;
            if (m >= p.m) break;
            const float y = __uint_as_float(v[j]) * sc;
            if (p.out_dt == NXB_F32) ((float*)p.out)[m * p.n + n] = y;
            else ((unsigned short*)p.out)[m * p.n + n] = f32_to_bf16_bits(y);
          }
        }
      }
      tc_fence_before();
    }
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
  if (warp == WQ_MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
  }
}

// ---- M <= 16: a pure stream over W ---------------------------------------------------------------
// With at most 16 rows of x the layer is one pass over W (N*K bytes) and nothing else matters: every
// SM has to keep its share of the memory system busy from the first to the last microsecond.  The
// kernel is a free-running pipeline with no CTA-wide synchronisation inside its loop:
//   * warp 16, one thread: the producer.  A CTA takes groups of 8 output channels round-robin over
//     the grid; the 8 rows of a group (k bytes each, contiguous) arrive by eight bulk copies into a
//     ring of SW_DEPTH stages (five groups, 160 KiB, in flight per SM).  Rows are laid 64 bytes
//     further apart than their length so that the 16-byte reads below do not collide on banks.  A
//     stage is refilled as soon as the 16 compute warps have taken their bytes of it into registers.
//   * warps 0..15: compute.  Warp w owns the 64-wide k chunks {i*16 + w}, i < 4; the x fragments of
//     its chunks are loaded once and stay in registers for every group.  Per group a lane reads four
//     16-byte pieces of W (row lane/4, 16 consecutive k each), hands the stage back, turns the bytes
//     into bf16 pairs and feeds mma.sync m16n8k16 (rows = the padded batch, columns = the 8 channels).
//     Which k lands in which slot of the MMA's contraction index does not matter as long as x uses
//     the same order, so the bytes are taken as they come: even bytes of a word form one pair, odd
//     bytes the other (x is permuted accordingly, once).  s8 -> bf16 without converts: with
//     v = lo - 128*b7, both 128 + lo and 128 + 128*b7 are bf16 bit patterns made by one logic
//     operation each (0x4300 | bits), and their bf16x2 difference is exact: 7 instructions per word.
//     The warp's partial tile goes to its slot of one of two exchange buffers; the warp moves on.
//   * warp 17: the epilogue.  Sums the 16 partial tiles of a group in warp order (so the result does
//     not depend on timing), applies the channel scale, stores, and hands the buffer back.
// Every wait is on an mbarrier and bounded; a stalled wait raises the abort flag, all roles leave
// their loops and the host reports NXB_ERR_TIMEOUT.
// tcgen05 would not help: at 16 rows the tensor work is a fraction of a percent of the pipe's capacity.
constexpr int SW_WARPS = 16, SW_IT = 4, SW_MAX_K = SW_WARPS * SW_IT * 64;
constexpr int SW_ROWS = 8;                                    // channels per group (one MMA tile)
constexpr int SW_DEPTH = 6;                                   // ring stages
constexpr int SW_ROW_BYTES = SW_MAX_K + 64;                   // row pitch in the ring
constexpr int SW_STAGE_BYTES = SW_ROWS * SW_ROW_BYTES;
constexpr int SW_RED_BYTES = SW_WARPS * 32 * 16;              // one exchange buffer: a float4 per lane per warp
constexpr int SW_THREADS = (SW_WARPS + 2) * 32;
constexpr int SW_SMEM = SW_DEPTH * SW_STAGE_BYTES + 2 * SW_RED_BYTES;

struct SwParams {
  const signed char* w;
  const unsigned short* x;
  const float* scale;
  void* out;
  int* status;
  int m, n, k, groups, out_dt;
  long long ldw, ldx;
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  // not volatile: a pure function of its operands, so the compiler may interleave the chains
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// bytes 0 and 2 of w -> `even` (a bf16 pair), bytes 1 and 3 -> `odd`; exact.  The difference is taken
// by the fused multiply-add (x * 1 + (-c)), which is a native bf16x2 instruction
__device__ __forceinline__ void s8x4_to_bf16_pairs(uint32_t w, uint32_t& even, uint32_t& odd) {
  const uint32_t w1 = w >> 8;
  const uint32_t pe = (w & 0x007F007Fu) | 0x43004300u, ce = (w & 0x00800080u) | 0xC300C300u;
  const uint32_t po = (w1 & 0x007F007Fu) | 0x43004300u, co = (w1 & 0x00800080u) | 0xC300C300u;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(even) : "r"(pe), "r"(0x3F803F80u), "r"(ce));
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(odd) : "r"(po), "r"(0x3F803F80u), "r"(co));
}

// x values k+0..k+3 as loaded (pairs (0,1), (2,3)) -> pairs (0,2), (1,3), the order the weights use
__device__ __forceinline__ void pair_even_odd(uint32_t& p01, uint32_t& p23) {
  const uint32_t e = __byte_perm(p01, p23, 0x5410), o = __byte_perm(p01, p23, 0x7632);
  p01 = e; p23 = o;
}

template <bool HI>      // HI: rows 8..15 of the batch exist
__global__ void __launch_bounds__(SW_THREADS, 1) wq_stream_kernel(SwParams p) {
  __shared__ __align__(8) unsigned long long bar_mem[2 * SW_DEPTH + 4];
  __shared__ int abort_word;
  extern __shared__ __align__(128) unsigned char sw_smem[];
  volatile int* abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = smem_u32(sw_smem), red = ring + SW_DEPTH * SW_STAGE_BYTES;
  const uint32_t full0 = smem_u32(bar_mem), empty0 = full0 + 8 * SW_DEPTH, rfull0 = empty0 + 8 * SW_DEPTH, rfree0 = rfull0 + 16;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int s = 0; s < SW_DEPTH; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, SW_WARPS); }
    for (int b = 0; b < 2; ++b) { mbar_init(rfull0 + 8 * b, SW_WARPS); mbar_init(rfree0 + 8 * b, 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int first = (int)blockIdx.x, stride = (int)gridDim.x;
  const int rounds = first < p.groups ? (p.groups - first + stride - 1) / stride : 0;

  if (warp == SW_WARPS) {
    // ---- producer ----
    if (lane == 0) {
      for (int r = 0; r < rounds; ++r) {
        const int s = r % SW_DEPTH;
        if (!mbar_wait(empty0 + 8 * s, (uint32_t)(((r / SW_DEPTH) & 1) ^ 1), abort_flag)) break;
        const int grp = first + r * stride;
        const int rows = min(SW_ROWS, p.n - grp * SW_ROWS);
        mbar_expect_tx(full0 + 8 * s, (uint32_t)(rows * p.k));
        for (int j = 0; j < rows; ++j) {
          const signed char* src = p.w + ((long long)grp * SW_ROWS + j) * p.ldw;
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(ring + (uint32_t)(s * SW_STAGE_BYTES + j * SW_ROW_BYTES)), "l"(src), "r"((uint32_t)p.k), "r"(full0 + 8 * s)
                       : "memory");
        }
      }
    }
  } else if (warp == SW_WARPS + 1) {
    // ---- epilogue: lane (g, q) owns rows g, g + 8 of x and channels 2q, 2q + 1 of the group ----
    const int g = lane >> 2, q = lane & 3;
    for (int r = 0; r < rounds; ++r) {
      const int b = r & 1;
      const long long n = ((long long)first + (long long)r * stride) * SW_ROWS + 2 * q;
      const float sc0 = n < p.n ? p.scale[n] : 0.f, sc1 = n + 1 < p.n ? p.scale[n + 1] : 0.f;
      if (!mbar_wait_warp(rfull0 + 8 * b, (uint32_t)((r >> 1) & 1), abort_flag)) break;
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      const float4* src = reinterpret_cast<const float4*>(sw_smem + SW_DEPTH * SW_STAGE_BYTES + b * SW_RED_BYTES) + lane;
#pragma unroll
      for (int w = 0; w < SW_WARPS; ++w) {
        const float4 v = src[w * 32];
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(rfree0 + 8 * b);
      const float y[4] = {sum.x * sc0, sum.y * sc1, sum.z * sc0, sum.w * sc1};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int m = g + (e >> 1) * 8;
        const long long nn = n + (e & 1);
        if (m < p.m && nn < p.n) {
          if (p.out_dt == NXB_F32) reinterpret_cast<float*>(p.out)[(long long)m * p.n + nn] = y[e];
          else reinterpret_cast<unsigned short*>(p.out)[(long long)m * p.n + nn] = f32_to_bf16_bits(y[e]);
        }
      }
    }
  } else {
    // ---- compute ----
    const int g = lane >> 2, q = lane & 3;
    // x fragments: 16 consecutive k of row g (and g + 8) per chunk, paired like the weights
    uint32_t xa[SW_IT][8], xb[HI ? SW_IT : 1][8];
#pragma unroll
    for (int it = 0; it < SW_IT; ++it) {
      const int kb = (it * SW_WARPS + warp) * 64 + q * 16;
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      if (kb < p.k && g < p.m) {
        const uint4* src = reinterpret_cast<const uint4*>(p.x + (long long)g * p.ldx + kb);
        lo = src[0]; hi = src[1];
      }
      xa[it][0] = lo.x; xa[it][1] = lo.y; xa[it][2] = lo.z; xa[it][3] = lo.w;
      xa[it][4] = hi.x; xa[it][5] = hi.y; xa[it][6] = hi.z; xa[it][7] = hi.w;
#pragma unroll
      for (int j = 0; j < 4; ++j) pair_even_odd(xa[it][2 * j], xa[it][2 * j + 1]);
      if (HI) {
        lo = make_uint4(0, 0, 0, 0); hi = lo;
        if (kb < p.k && g + 8 < p.m) {
          const uint4* src = reinterpret_cast<const uint4*>(p.x + (long long)(g + 8) * p.ldx + kb);
          lo = src[0]; hi = src[1];
        }
        xb[it][0] = lo.x; xb[it][1] = lo.y; xb[it][2] = lo.z; xb[it][3] = lo.w;
        xb[it][4] = hi.x; xb[it][5] = hi.y; xb[it][6] = hi.z; xb[it][7] = hi.w;
#pragma unroll
        for (int j = 0; j < 4; ++j) pair_even_odd(xb[it][2 * j], xb[it][2 * j + 1]);
      }
    }
    const unsigned char* my_piece = sw_smem + g * SW_ROW_BYTES + warp * 64 + q * 16;
    float4* my_red = reinterpret_cast<float4*>(sw_smem + SW_DEPTH * SW_STAGE_BYTES) + warp * 32 + lane;
    for (int r = 0; r < rounds; ++r) {
      const int s = r % SW_DEPTH, b = r & 1;
      if (!mbar_wait_warp_tight(full0 + 8 * s, (uint32_t)((r / SW_DEPTH) & 1), abort_flag)) break;
      // this warp's bytes of the stage: 16 per chunk; rows beyond n hold stale bytes, their columns are never stored
      uint4 words[SW_IT];
#pragma unroll
      for (int it = 0; it < SW_IT; ++it)
        words[it] = (it * SW_WARPS + warp) * 64 < p.k ? *reinterpret_cast<const uint4*>(my_piece + s * SW_STAGE_BYTES + it * SW_WARPS * 64)
                                                     : make_uint4(0, 0, 0, 0);
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);          // the values are in registers: the stage may be refilled
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int it = 0; it < SW_IT; ++it) {
        const uint32_t wj[4] = {words[it].x, words[it].y, words[it].z, words[it].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t b0, b1;
          s8x4_to_bf16_pairs(wj[j], b0, b1);
          mma_bf16_16816(acc[it & 1], xa[it][2 * j], HI ? xb[HI ? it : 0][2 * j] : 0u, xa[it][2 * j + 1], HI ? xb[HI ? it : 0][2 * j + 1] : 0u, b0, b1);
        }
      }
      // the exchange buffer of two rounds ago has been summed
      if (!mbar_wait_warp_tight(rfree0 + 8 * b, (uint32_t)(((r >> 1) & 1) ^ 1), abort_flag)) break;
      my_red[b * (SW_RED_BYTES / 16)] = make_float4(acc[0][0] + acc[1][0], acc[0][1] + acc[1][1], acc[0][2] + acc[1][2], acc[0][3] + acc[1][3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(rfull0 + 8 * b);
    }
  }
  __syncthreads();
  if (*abort_flag) {
    // a copy never arrived: report it, give the copies still in flight time to land before the
    // shared memory is handed to another CTA
    if (threadIdx.x == 0) *(volatile int*)p.status = 1;
    const long long t0 = now_cycles();
    while (now_cycles() - t0 < 400000ll) { }
  }
}

bool wq_stream_usable(const GemmArgs& g) {
  return g.m <= 16 && g.k % 64 == 0 && g.k <= SW_MAX_K && !getenv("NXB200_NO_WQ_STREAM");
}

void launch_wq_stream(const GemmArgs& g, int* status_word, int sm_count, cudaStream_t stream) {
  SwParams p{};
  p.w = (const signed char*)g.b;
  p.x = (const unsigned short*)g.a;
  p.scale = (const float*)g.scale;
  p.out = g.c;
  p.m = (int)g.m; p.n = (int)g.n; p.k = (int)g.k;
  p.groups = (int)((g.n + SW_ROWS - 1) / SW_ROWS);
  p.out_dt = (int)g.dc;
  p.ldw = g.ldb; p.ldx = g.lda;
  p.status = status_word;
  const unsigned grid = (unsigned)std::min<int64_t>(p.groups, sm_count);
  if (g.m > 8) {
    NXB_CUDA(cudaFuncSetAttribute(wq_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SW_SMEM));
    wq_stream_kernel<true><<<grid, SW_THREADS, SW_SMEM, stream>>>(p);
  } else {
    NXB_CUDA(cudaFuncSetAttribute(wq_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SW_SMEM));
    wq_stream_kernel<false><<<grid, SW_THREADS, SW_SMEM, stream>>>(p);
  }
  NXB_CUDA(cudaGetLastError());
}

// Tensor map over a row-major [rows][k] matrix in units of 64 k: coordinates (k within the block, row,
// k block).  `blocked`: the third dimension walks the k blocks of a row (stride 64 elements), so a box
// of `g` blocks arrives as g consecutive tiles of [box_rows][64 k]; needs k % 64 == 0.  Otherwise the
// map is the plain two-dimensional view (third dimension of extent 1) and the first coordinate is the k
// offset itself, with out-of-range k filled with zeros.
CUtensorMap wq_map(const void* ptr, CUtensorMapDataType type, size_t es, int64_t k, int64_t rows, int64_t ld, int box_rows, int g, bool blocked,
                   CUtensorMapSwizzle sw) {
  const DriverApi& drv = driver();
  if (!drv.cuTensorMapEncodeTiled) fail(NXB_ERR_RUNTIME, "cuTensorMapEncodeTiled is unavailable");
  CUtensorMap m;
  cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, 1};
  cuuint64_t strides[2] = {(cuuint64_t)(ld * es), (cuuint64_t)(ld * es) * (cuuint64_t)rows};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  if (blocked) {
    dims[0] = 64; dims[2] = (cuuint64_t)(k / 64);
    strides[1] = (cuuint64_t)(64 * es);
    box[2] = (cuuint32_t)g;
  }
  cuuint32_t estr[3] = {1, 1, 1};
  check_cu(drv.cuTensorMapEncodeTiled(&m, type, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
           "cuTensorMapEncodeTiled");
  return m;
}

}  // namespace

bool wq_linear_supported(const GemmArgs& g) {
  return g.da == NXB_BF16 && g.db == NXB_S8 && g.scale && !g.ta && !g.tb && g.batch == 1 && g.m >= 1 && g.m <= WQ_LINEAR_MAX_ROWS &&
         g.k % 16 == 0 && (g.lda * 2) % 16 == 0 && g.ldb % 16 == 0 && (g.dc == NXB_F32 || g.dc == NXB_BF16) &&
         ((uintptr_t)g.a % 16) == 0 && ((uintptr_t)g.b % 16) == 0;
}

void launch_wq_linear(const GemmArgs& g, int* status_word, int sm_count, cudaStream_t stream) {
  if (wq_stream_usable(g)) { launch_wq_stream(g, status_word, sm_count, stream); return; }
  WqParams p{};
  p.out = g.c;
  p.scale = (const float*)g.scale;
  p.status = status_word;
  p.m = (int)g.m; p.n = (int)g.n; p.k = (int)g.k;
  p.mb = (int)std::min<int64_t>(256, (g.m + 15) / 16 * 16);
  p.out_dt = (int)g.dc;
  // one band of channels per SM (a multiple of 8 channels, at most 128)
  p.ch = (int)std::min<int64_t>(128, ((g.n + sm_count - 1) / sm_count + 7) / 8 * 8);
  if (const char* e = getenv("NXB200_WQ_BAND")) { const int v = atoi(e); if (v >= 8 && v <= 128 && v % 8 == 0) p.ch = v; }
  const int kblocks = (p.k + 63) / 64;
  // Several k blocks per ring stage cut the hand-overs between the roles (and the copies to issue) per
  // byte of W; the x part of a stage grows with the batch, which bounds it.  A k that ends inside a
  // block needs the zero fill of the two-dimensional view, i.e. one block per stage.
  p.g = p.mb <= 32 ? 4 : p.mb <= 128 ? 2 : 1;
  if (p.k % 64 != 0) p.g = 1;
  if (const char* e = getenv("NXB200_WQ_KBLOCKS")) { const int v = atoi(e); if ((v == 1 || v == 2 || v == 4) && p.k % 64 == 0) p.g = v; }
  p.raw_bytes = (p.g * p.ch * 64 + 1023) / 1024 * 1024;
  const int stage = p.raw_bytes + p.g * p.mb * 128;
  p.conv_slab = (p.ch * 128 + 1023) / 1024 * 1024;
  const int conv_stage = p.g * p.conv_slab;
  const char* cs_env = getenv("NXB200_WQ_CONV_STAGES");
  p.conv_stages = cs_env ? std::max(2, std::min(WQ_MAX_CONV_STAGES, atoi(cs_env))) : (p.g > 1 ? 3 : (p.mb <= 64 ? 8 : 4));
  p.stages = std::max(3, std::min(WQ_MAX_STAGES, (WQ_SMEM_LIMIT - p.conv_stages * conv_stage) / stage));
  const int nst = (kblocks + p.g - 1) / p.g;
  // narrow batches are bound by the rate at which MMAs can be issued: up to three issuing threads
  const char* iss_env = getenv("NXB200_WQ_ISSUERS");
  p.issuers = iss_env ? std::max(1, std::min(3, atoi(iss_env))) : (p.mb <= 64 ? 3 : 1);
  p.issuers = std::min(p.issuers, std::max(1, nst));
  p.issuers = std::min(p.issuers, 512 / p.mb);          // one accumulator each must fit the 512 TMEM columns
  const int per_issuer = std::max(1, std::min(std::min(8, 512 / p.mb) / p.issuers, 4));
  p.nacc = per_issuer * p.issuers;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.nacc * p.mb) p.tmem_cols *= 2;
  // W and x as [k block][row][64 k]: the third coordinate counts k blocks, so one copy brings g of them.
  // (With a k that is not a multiple of 64 the blocked view would run into the next row: then g is 1 and
  // the plain two-dimensional view zero-fills the ragged end.)
  p.blocked = (p.g > 1) ? 1 : 0;
  CUtensorMap mw = wq_map(g.b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.k, g.n, g.ldb, p.ch, p.g, p.blocked != 0, CU_TENSOR_MAP_SWIZZLE_64B);
  CUtensorMap mx = wq_map(g.a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g.k, g.m, g.lda, p.mb, p.g, p.blocked != 0, CU_TENSOR_MAP_SWIZZLE_128B);
  const int smem = p.stages * stage + p.conv_stages * conv_stage + 1024 + 512;
  if (smem > 232448) fail(NXB_ERR_RUNTIME, "internal: quantised linear stage sizes exceed shared memory");
  NXB_CUDA(cudaFuncSetAttribute(wq_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((unsigned)((g.n + p.ch - 1) / p.ch), (unsigned)((g.m + p.mb - 1) / p.mb));
  wq_linear_kernel<<<grid, WQ_THREADS, smem, stream>>>(mw, mx, p);
  NXB_CUDA(cudaGetLastError());
}

}  // namespace nxb

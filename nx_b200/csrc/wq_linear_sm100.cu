// Weight-only quantised linear for small batches on sm_100a:
//
//   y[m][n] = S[n] * sum_k x[m][k] * W[n][k]       x bf16 {M,K}, W s8 {N,K}, S f32 {N}, M <= 512
//
// With few rows of x the layer is a stream over W (N*K bytes), so W must cross HBM exactly once
// and never exist as 16-bit values in memory.  The product is computed transposed: a CTA owns
// 128 output channels n (the M side of the tensor-core tile, one TMEM lane each) and up to 256
// rows of x (the N side), so every weight is converted once.
//   warp 0      TMA producer: per 64-wide k block the raw s8 tile of W (128 rows x 64 bytes,
//               64-byte swizzle) and the bf16 tile of x (128-byte swizzle; rows beyond M arrive
//               as zeros) into a deep ring (up to 16 stages: the stream is latency bound, a CTA
//               needs ~100 KB in flight to draw its share of the memory bandwidth)
//   12 warps    converters (every warp outside scheduler partition 0): s8 -> bf16 (exact), written as the 128-byte-swizzled K-major A tile
//               into a second ring.  Three groups of four warps take the k blocks round-robin,
//               so each group has three k-block periods for its wait -> convert -> fence ->
//               arrive sequence: the latency of that sequence, not its instruction count, is
//               what paces a pipeline whose MMAs are a few cycles each.  Afterwards the same
//               warps are the epilogue (tcgen05.ld, scale per lane, store)
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

// four signed bytes -> four bf16 (exact).  Each byte, biased by 128, becomes the low mantissa
// byte of 2^23; subtracting 2^23 + 128 leaves the integer as an f32.
__device__ __forceinline__ void s8x4_to_bf16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t x = w ^ 0x80808080u;
  const float f0 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540)) - 8388736.f;
  const float f1 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7541)) - 8388736.f;
  const float f2 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7542)) - 8388736.f;
  const float f3 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7543)) - 8388736.f;
  // exact in bf16: the upper halves of the f32 words are the result (a byte permute, not a
  // quarter-rate convert)
  lo = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
  hi = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
}

constexpr int WQ_THREADS = 512;
constexpr int WQ_MMA_WARP = 4;      // same scheduler partition as the producer (warp 0): none of the busy converter warps run there

__global__ void __launch_bounds__(WQ_THREADS, 1)
wq_linear_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, WqParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t x_bytes = (uint32_t)p.mb * 128u;
  const uint32_t stage_bytes = WQ_RAW + x_bytes;
  const uint32_t wb0 = base + (uint32_t)p.stages * stage_bytes;
  const uint32_t bars = wb0 + (uint32_t)p.conv_stages * WQ_WB;
  const uint32_t full0 = bars, empty0 = bars + 128, conv0 = bars + 256, wbe0 = bars + 320, acc_full = bars + 384, tmem_slot = bars + 392;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + (tmem_slot - base));
  volatile int* abort_flag = (volatile int*)(gen_base + (tmem_slot - base) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (int)blockIdx.x * 128, m0 = (int)blockIdx.y * p.mb;
  const int kblocks = (p.k + 63) / 64;

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
    for (int kb = which; kb < kblocks; kb += step) {
      // the converters arrive on conv only after the stage's TMA data (x included) has landed
      if (!mbar_wait(conv0 + 8 * c, cph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint64_t adesc = make_desc(wb0 + (uint32_t)c * WQ_WB), bdesc = make_desc(base + (uint32_t)s * stage_bytes + WQ_RAW);
      // consecutive MMAs go to different accumulators: accumulating into the columns the
      // previous one is still writing would serialise them on the pipeline's latency
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        tc_mma(acc, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc, fresh > 0 ? 0u : 1u, false);
        if (fresh > 0) --fresh;
        acc += (uint32_t)p.mb;
        if (acc == acc_end) acc = acc0;
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
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag)) break;
        const uint32_t st = base + (uint32_t)s * stage_bytes;
        mbar_expect_tx(full0 + 8 * s, WQ_RAW + x_bytes);
        tma_load_3d(st, &map_w, full0 + 8 * s, kb * 64, n0, 0);
        tma_load_3d(st + WQ_RAW, &map_x, full0 + 8 * s, kb * 64, m0, 0);
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
    // the MMA issuer live: a single thread issuing MMAs loses most of its issue slots to busy
    // warps on the same scheduler).  Three groups of four warps take the k blocks round-robin,
    // one thread per row of W, so a group has three k-block periods for its wait -> convert ->
    // fence -> arrive sequence.
    const bool converter = (warp & 3) != 0;
    const int ci = (warp >> 2) * 3 + (warp & 3) - 1;
    const int grp = ci >> 2;
    const int r = (ci & 3) * 32 + lane;
    int s = grp % p.stages, cs = grp % p.conv_stages;
    uint32_t ph = (uint32_t)((grp / p.stages) & 1), cph = (uint32_t)((grp / p.conv_stages) & 1);
    bool ok = true;
    for (int kb = grp; converter && kb < kblocks && ok; kb += 3) {
      // one lane per warp polls the barriers
      int okw = 1;
      if (lane == 0) okw = mbar_wait_relaxed(full0 + 8 * s, ph, abort_flag) && mbar_wait_relaxed(wbe0 + 8 * cs, cph ^ 1, abort_flag);
      okw = __shfl_sync(0xffffffffu, okw, 0);
      __syncwarp();
      if (!okw) { ok = false; break; }
      const uint32_t st = base + (uint32_t)s * stage_bytes;
      const uint32_t row = wb0 + (uint32_t)cs * WQ_WB + (uint32_t)r * 128u;
      uint32_t w[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {                     // 16-byte chunks of the 64-byte s8 row
        const uint32_t src = st + (uint32_t)r * 64u + (uint32_t)((c ^ ((r >> 1) & 3)) * 16);
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[4 * c]), "=r"(w[4 * c + 1]), "=r"(w[4 * c + 2]), "=r"(w[4 * c + 3]) : "r"(src));
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[8];
        s8x4_to_bf16x4(w[4 * c], o[0], o[1]);
        s8x4_to_bf16x4(w[4 * c + 1], o[2], o[3]);
        s8x4_to_bf16x4(w[4 * c + 2], o[4], o[5]);
        s8x4_to_bf16x4(w[4 * c + 3], o[6], o[7]);
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
      const float sc = n < p.n ? p.scale[n] : 0.f;
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
        if (n < p.n) {
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
// With at most 16 rows of x the tcgen05 pipeline above is paced by its per-k-block hand-offs
// (TMA -> converter warps -> shared memory -> MMA issuer) and only N/128 CTAs have work.  Here every
// SM streams its share of W and converts it in registers on its way to the tensor cores:
//   * a CTA of 16 warps owns groups of 16 output channels (all 148 SMs take groups round-robin);
//     the 16 rows of a group (k bytes each, contiguous) arrive by sixteen bulk copies issued by one
//     thread into a ring of 3 stages, two groups (128 KiB) ahead.  Rows are laid 64 bytes further
//     apart than their length so that the 16-byte reads below do not collide on banks.  Every
//     round ends in a CTA-wide hand-over (partial sums through shared memory), whose latency all
//     warps pay in lockstep: with 8 channels per round the kernel took 20.5 us, with 16 it takes 16.5
//   * warp w owns the 64-wide k chunks {i*16 + w}, i < 4; the x fragments of its chunks are loaded
//     once and stay in registers (64 of them) for every group
//   * per group a lane reads four 16-byte pieces of W (row lane/4, 16 consecutive k each), turns
//     them into bf16 pairs and feeds mma.sync m16n8k16 (rows = the padded batch, columns = 8
//     channels; two such tiles per group).  Which k lands in which slot of the MMA's contraction
//     index does not matter as long as x uses the same order, so the bytes are taken as they come: even bytes of a word form one
//     pair, odd bytes the other (x is permuted accordingly, once).  s8 -> bf16 without converts: with
//     v = lo - 128*b7, both 128 + lo and 128 + 128*b7 are bf16 bit patterns made by one logic
//     operation each (0x4300 | bits), and their bf16x2 difference is exact: 7 instructions per word
//   * the 16 partial tiles are summed through shared memory in a fixed order (deterministic)
// tcgen05 would not help: at 16 rows the tensor work is a fraction of a percent of the pipe's
// capacity.  Measured, the kernel is bound by neither HBM (2.7 TB/s of W stream) nor a pipe (ALU 40 %)
// but by the per-round latency chain above.
constexpr int GV_WARPS = 16, GV_IT = 4, GV_MAX_K = GV_WARPS * GV_IT * 64;
constexpr int GV_TILES = 2;                                   // 8-channel MMA tiles per group
constexpr int GV_ROWS = 8 * GV_TILES;                         // channels per group
constexpr int GV_DEPTH = 3;                                   // ring stages: 2 groups (128 KiB) in flight
constexpr int GV_ROW_BYTES = GV_MAX_K + 64;                   // row pitch in the ring
constexpr int GV_STAGE_BYTES = GV_ROWS * GV_ROW_BYTES;

struct GvParams {
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
__global__ void __launch_bounds__(GV_WARPS * 32, 1) wq_stream_kernel(GvParams p) {
  __shared__ float red[GV_WARPS][32][4 * GV_TILES];
  __shared__ __align__(8) unsigned long long full_bar[GV_DEPTH];
  __shared__ int abort_word;
  extern __shared__ __align__(128) unsigned char gv_ring[];
  volatile int* abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const uint32_t ring = smem_u32(gv_ring), bars = smem_u32(full_bar);
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int s = 0; s < GV_DEPTH; ++s) mbar_init(bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // the eight rows of a group: one bulk copy each, completion counted on the stage's barrier
  auto issue = [&](int grp, int stage) {
    if (grp >= p.groups) return;
    const int rows = min(GV_ROWS, p.n - grp * GV_ROWS);
    mbar_expect_tx(bars + 8 * stage, (uint32_t)(rows * p.k));
    for (int r = 0; r < rows; ++r) {
      const signed char* src = p.w + ((long long)grp * GV_ROWS + r) * p.ldw;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(ring + (uint32_t)(stage * GV_STAGE_BYTES + r * GV_ROW_BYTES)), "l"(src), "r"((uint32_t)p.k), "r"(bars + 8 * stage)
                   : "memory");
    }
  };
  int grp = (int)blockIdx.x;
  if (threadIdx.x == 0)
    for (int d = 0; d < GV_DEPTH - 1; ++d) issue(grp + d * (int)gridDim.x, d);
  // x fragments: 16 consecutive k of row g (and g + 8) per chunk, paired like the weights
  uint32_t xa[GV_IT][8], xb[HI ? GV_IT : 1][8];
#pragma unroll
  for (int it = 0; it < GV_IT; ++it) {
    const int kb = (it * GV_WARPS + warp) * 64 + q * 16;
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
  const uint32_t my_piece = ring + (uint32_t)(g * GV_ROW_BYTES + warp * 64 + q * 16);
  for (int round = 0; grp < p.groups; grp += (int)gridDim.x, ++round) {
    const int stage = round % GV_DEPTH;
    // the stage read in the previous round is free (every warp passed that round's barrier)
    if (threadIdx.x == 0) issue(grp + (GV_DEPTH - 1) * (int)gridDim.x, (round + GV_DEPTH - 1) % GV_DEPTH);
    // this thread's share of the epilogue: output (row m, channel nn) of the group, partial sums of
    // eight warps; the scale is fetched now so that its latency hides behind the products
    const int o = threadIdx.x >> 1, part = threadIdx.x & 1;
    const int m = o / GV_ROWS, nn = o % GV_ROWS;
    const long long n = (long long)grp * GV_ROWS + nn;
    const float sc = n < p.n ? p.scale[n] : 0.f;
    const bool ok = mbar_wait_warp_tight(bars + 8 * stage, (uint32_t)((round / GV_DEPTH) & 1), abort_flag);
    float acc[GV_TILES][2][4];                // two dependency chains per tile (even / odd chunks)
#pragma unroll
    for (int t = 0; t < GV_TILES; ++t)
#pragma unroll
      for (int h = 0; h < 2; ++h) acc[t][h][0] = acc[t][h][1] = acc[t][h][2] = acc[t][h][3] = 0.f;
    const unsigned char* my_stage = gv_ring + (my_piece - ring) + stage * GV_STAGE_BYTES;
#pragma unroll
    for (int it = 0; it < GV_IT; ++it) {
      // warp-uniform: the whole 64-wide chunk lies inside k or outside; rows beyond n hold stale
      // bytes, their columns are never stored
      if (ok && (it * GV_WARPS + warp) * 64 < p.k) {
        uint4 words[GV_TILES];
#pragma unroll
        for (int t = 0; t < GV_TILES; ++t)     // ordinary loads: ordered after the wait above, free to move among the MMAs
          words[t] = *reinterpret_cast<const uint4*>(my_stage + t * 8 * GV_ROW_BYTES + it * GV_WARPS * 64);
#pragma unroll
        for (int t = 0; t < GV_TILES; ++t) {
          const uint32_t wj[4] = {words[t].x, words[t].y, words[t].z, words[t].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t b0, b1;
            s8x4_to_bf16_pairs(wj[j], b0, b1);
            mma_bf16_16816(acc[t][it & 1], xa[it][2 * j], HI ? xb[HI ? it : 0][2 * j] : 0u, xa[it][2 * j + 1], HI ? xb[HI ? it : 0][2 * j + 1] : 0u, b0, b1);
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < GV_TILES; ++t)
      *reinterpret_cast<float4*>(&red[warp][lane][4 * t]) =
          make_float4(acc[t][0][0] + acc[t][1][0], acc[t][0][1] + acc[t][1][1], acc[t][0][2] + acc[t][1][2], acc[t][0][3] + acc[t][1][3]);
    __syncthreads();
    {
      // per tile, acc[0..1]: row g, channels 2q, 2q+1; acc[2..3]: row g + 8.  All 512 threads take
      // part: two lanes per output, each sums eight warps' partials in a fixed order
      const int n8 = nn & 7, t = nn >> 3;
      const int src_lane = (m & 7) * 4 + (n8 >> 1), c = 4 * t + (m >> 3) * 2 + (n8 & 1);
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < GV_WARPS / 2; ++w) sum += red[part * (GV_WARPS / 2) + w][src_lane][c];
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      if (part == 0 && m < p.m && n < p.n && !*abort_flag) {
        const float y = sum * sc;
        if (p.out_dt == NXB_F32) reinterpret_cast<float*>(p.out)[(long long)m * p.n + n] = y;
        else reinterpret_cast<unsigned short*>(p.out)[(long long)m * p.n + n] = f32_to_bf16_bits(y);
      }
    }
    __syncthreads();                         // the partial sums are rewritten in the next round
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
  return g.m <= 16 && g.k % 64 == 0 && g.k <= GV_MAX_K && !getenv("NXB200_NO_WQ_STREAM");
}

void launch_wq_stream(const GemmArgs& g, int* status_word, int sm_count, cudaStream_t stream) {
  GvParams p{};
  p.w = (const signed char*)g.b;
  p.x = (const unsigned short*)g.a;
  p.scale = (const float*)g.scale;
  p.out = g.c;
  p.m = (int)g.m; p.n = (int)g.n; p.k = (int)g.k;
  p.groups = (int)((g.n + GV_ROWS - 1) / GV_ROWS);
  p.out_dt = (int)g.dc;
  p.ldw = g.ldb; p.ldx = g.lda;
  p.status = status_word;
  const unsigned grid = (unsigned)std::min<int64_t>(p.groups, sm_count);
  const int smem = GV_DEPTH * GV_STAGE_BYTES;
  if (g.m > 8) {
    NXB_CUDA(cudaFuncSetAttribute(wq_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    wq_stream_kernel<true><<<grid, GV_WARPS * 32, smem, stream>>>(p);
  } else {
    NXB_CUDA(cudaFuncSetAttribute(wq_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    wq_stream_kernel<false><<<grid, GV_WARPS * 32, smem, stream>>>(p);
  }
  NXB_CUDA(cudaGetLastError());
}

CUtensorMap wq_map(const void* ptr, CUtensorMapDataType type, size_t es, int64_t k, int64_t rows, int64_t ld, int box_rows, CUtensorMapSwizzle sw) {
  const DriverApi& drv = driver();
  if (!drv.cuTensorMapEncodeTiled) fail(NXB_ERR_RUNTIME, "cuTensorMapEncodeTiled is unavailable");
  CUtensorMap m;
  cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, 1};
  cuuint64_t strides[2] = {(cuuint64_t)(ld * es), (cuuint64_t)(ld * es) * (cuuint64_t)rows};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
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
  const int stage = WQ_RAW + p.mb * 128;
  const char* cs_env = getenv("NXB200_WQ_CONV_STAGES");
  p.conv_stages = cs_env ? std::max(2, std::min(WQ_MAX_CONV_STAGES, atoi(cs_env))) : (p.mb <= 64 ? 8 : 4);
  p.stages = std::min(WQ_MAX_STAGES, (WQ_SMEM_LIMIT - p.conv_stages * WQ_WB) / stage);
  const int kblocks = (p.k + 63) / 64;
  // narrow batches are bound by the rate at which MMAs can be issued: up to three issuing threads
  const char* iss_env = getenv("NXB200_WQ_ISSUERS");
  p.issuers = iss_env ? std::max(1, std::min(3, atoi(iss_env))) : (p.mb <= 64 ? 3 : 1);
  p.issuers = std::min(p.issuers, std::max(1, kblocks));
  p.issuers = std::min(p.issuers, 512 / p.mb);          // one accumulator each must fit the 512 TMEM columns
  const int per_issuer = std::max(1, std::min(std::min(8, 512 / p.mb) / p.issuers, 4));
  p.nacc = per_issuer * p.issuers;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.nacc * p.mb) p.tmem_cols *= 2;
  CUtensorMap mw = wq_map(g.b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.k, g.n, g.ldb, 128, CU_TENSOR_MAP_SWIZZLE_64B);
  CUtensorMap mx = wq_map(g.a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g.k, g.m, g.lda, p.mb, CU_TENSOR_MAP_SWIZZLE_128B);
  const int smem = p.stages * stage + p.conv_stages * WQ_WB + 1024 + 512;
  NXB_CUDA(cudaFuncSetAttribute(wq_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((unsigned)((g.n + 127) / 128), (unsigned)((g.m + p.mb - 1) / p.mb));
  wq_linear_kernel<<<grid, WQ_THREADS, smem, stream>>>(mw, mx, p);
  NXB_CUDA(cudaGetLastError());
}

}  // namespace nxb

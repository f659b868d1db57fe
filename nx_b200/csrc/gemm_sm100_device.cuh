// Device side of the tensor-core matrix product (tcgen05 + TMA + TMEM) for sm_100a.
// Shared by the ahead-of-time build (gemm_sm100.cu) and by kernels the planner generates
// at run time with a fused, graph-specific epilogue (compiled with NVRTC), hence no host
// headers here: under NVRTC the tensor-map type is declared as the opaque 128-byte
// object it is.
#pragma once
#ifdef __CUDACC_RTC__
struct alignas(64) CUtensorMap_st { unsigned long long opaque[16]; };
typedef CUtensorMap_st CUtensorMap;
enum { NXB_U8 = 0, NXB_U16 = 1, NXB_U32 = 2, NXB_U64 = 3, NXB_S8 = 4, NXB_S16 = 5, NXB_S32 = 6, NXB_S64 = 7,
       NXB_F16 = 8, NXB_BF16 = 9, NXB_F32 = 10, NXB_F64 = 11 };
#endif

namespace nxb_gemm {

constexpr int BM = 128;
constexpr int ROW_BYTES = 128;                        // one swizzle row: 64 bf16 or 128 s8
constexpr int A_STAGE = BM * ROW_BYTES;
// The tile width BN is 256 for large products; narrow outputs (few rows, e.g. a linear layer
// applied to 1..128 tokens) use 128 or 64 so that enough tiles exist to occupy every SM, with a
// deeper ring since the product is then bound by streaming the weights.
__host__ __device__ constexpr int stages_for(int bn) { return bn == 256 ? 4 : bn == 128 ? 6 : 8; }
constexpr int STORE_STAGE = 4 * 2 * 4096;   // per epilogue warp: two 32x32 staging tiles of up to 4 bytes per element
__host__ __device__ constexpr int smem_bytes_for(int bn) {
  return stages_for(bn) * (A_STAGE + bn * ROW_BYTES) + STORE_STAGE + 1024 /*alignment*/ + 256 /*barriers*/;
}
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;   // about two seconds of SM clock

enum Kind { KIND_BF16 = 0, KIND_F16 = 1, KIND_S8 = 2 };

struct TcParams {
  void* c;
  const void* bias;
  const float* scale;
  int* status;
  int m, n, k, batch;
  int mtiles, ntiles;
  int out_dt;        // nxb200_dtype of C
  int epilogue;
  int a_mn, b_mn;    // operand stored with its free index contiguous ([k][m] / [k][n]) instead of k: 1 = one copy per
                     // 64 rows of the tile (3-D map), 2 = one copy per tile (4-D map {64 rows, k, row group, batch})
  int tma_store;     // results leave through shared memory and a TMA store (rows of C 16-byte aligned); 2: the plain 16-bit
                     // epilogue stores all staging tiles of a warp at once (map_c is the four-dimensional grouped view)
  int panel_m;       // row tiles per panel of the tile walk (>= 1)
  void* ep[14];      // buffers of a generated epilogue, in its argument order
};

// Product fused with a sum over ranks (tensor parallelism), over peer memory.  Every rank owns the
// row tiles mt with mt % world == rank.  Buffers are per rank and mapped into every process
// (`[rank]` is the local one): `partial` holds this rank's product tiles, `result` the reduced
// tiles it owns; `ready` / `reduced` hold one word per (tile, 32-row quarter) carrying the epoch
// (launch number) of the last complete write.  All waits are reads: nothing is pushed to a peer.
struct CommArgs {
  int rank, world;
  uint32_t epoch;
  int pad;
  const unsigned short* partial[8];
  unsigned short* result[8];
  uint32_t* ready[8];
  uint32_t* reduced[8];
  unsigned short* out;       // this rank's copy of the reduced matrix [m][n] (bf16 or f16 bits)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// SM cycle counter: cheap to read (the global nanosecond timer costs a long round trip, which a
// wait that misses its first poll would pay on the critical path)
__device__ __forceinline__ long long now_cycles() { return clock64(); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises *abort) when the limit passes or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = now_cycles();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (now_cycles() - t0 > WAIT_LIMIT_CYCLES) {
      *abort_flag = 1;
      return false;
    }
  }
}
// Bounded wait that sleeps between polls: for roles with slack (an epilogue waiting out a whole
// main loop), so that their polling does not take issue slots and barrier-unit bandwidth from
// the single threads that feed the tensor cores on the same scheduler.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = now_cycles();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      __nanosleep(40);
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag) return false;
    if (now_cycles() - t0 > WAIT_LIMIT_CYCLES) {
      *abort_flag = 1;
      return false;
    }
  }
}
// The same wait done by lane 0 on behalf of its warp (all 32 lanes must call).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_relaxed(bar, parity, abort_flag);
  ok = __shfl_sync(0xffffffffu, ok, 0);
  __syncwarp();
  return ok != 0;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Bounded wait until a flag (possibly in a peer's memory) has reached `epoch`.
__device__ __forceinline__ bool flag_wait(const uint32_t* f, uint32_t epoch, volatile int* abort_flag,
                                          long long limit_cycles = 15 * WAIT_LIMIT_CYCLES) {
  const long long t0 = now_cycles();
  for (;;) {
    for (int i = 0; i < 16; ++i) {
      if ((int)(ld_acquire_sys(f) - epoch) >= 0) return true;
      __nanosleep(200);
    }
    if (*abort_flag) return false;
    // ranks may reach the kernel seconds apart (host-side skew): by default about half a minute
    if (now_cycles() - t0 > limit_cycles) {
      *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate, bool s8) {
  if (s8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The same load without the wait: the registers hold the data only after tmem_ld_wait().  Lets the
// next chunk's load run while the current chunk is converted and stored.
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
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// ex2.approx: the hardware exponential (2 ulp); ex2(-inf) = 0
__device__ __forceinline__ float nx_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// Latency-critical wait done by lane 0 on behalf of its warp (all 32 lanes must call).
__device__ __forceinline__ bool mbar_wait_warp_tight(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag);
  ok = __shfl_sync(0xffffffffu, ok, 0);
  __syncwarp();
  return ok != 0;
}
// 64 consecutive columns of one TMEM lane per thread: both loads are in flight before the wait
__device__ __forceinline__ void tmem_ld32x2(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
        "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
        "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
        "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored in 128-byte swizzled rows:
// 8-row groups are 1024 bytes apart (stride offset), the leading offset is unused (1),
// version 1, layout type 2 = SWIZZLE_128B.
// The same for a tile whose rows run along the free index (M or N): a row holds 64 consecutive
// m/n elements of one k, 8 rows of consecutive k form a 1024-byte group (stride offset), and the
// next 64 m/n elements start 8192 bytes further (leading offset: one 64-row TMA box).
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(8192 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}

__device__ __forceinline__ unsigned short f32_to_bf16_bits(float f) {
  unsigned short h;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f));
  return h;
}
// (lo, hi) -> one register holding both 16-bit values, lo in the low half
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t f32x2_to_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// Volatile forms: kept inside the branch that selected the type (a pure asm on both sides of a
// type test is computed twice and selected).
__device__ __forceinline__ uint32_t bits2_to_bf16x2(uint32_t lo, uint32_t hi) {
  uint32_t r;
  asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
  return r;
}
__device__ __forceinline__ uint32_t bits2_to_f16x2(uint32_t lo, uint32_t hi) {
  uint32_t r;
  asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
  return r;
}
__device__ __forceinline__ unsigned short f32_to_f16_bits(float f) {
  unsigned short h;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f));
  return h;
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"((unsigned long long)map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"((unsigned long long)map), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Default epilogue: convert the 32 accumulator values of one row segment to the output type
// and store them (128-bit stores when the segment is complete and rows are 16-byte aligned).
struct EpiStore {
  static constexpr bool kStaged = true;     // may leave through the shared-memory staged TMA store
  static constexpr bool kTransform = false; // a generated epilogue sets this and rewrites the 32 values in place before a staged store
  static __device__ __forceinline__ void transform(const TcParams&, float (&)[32], long long, long long, long long) {}
  static __device__ __forceinline__ void store(const TcParams& p, float (&f)[32], const uint32_t (&v)[32], long long b, long long m, long long n0) {
    const long long rowoff = (b * p.m + m) * p.n;
    // vector stores need 16-byte aligned rows: the row length and the base of C both count
    const bool base_ok = ((unsigned long long)p.c & 15ull) == 0;
    const bool vec_ok = (p.n % 8) == 0 && base_ok;
    const bool full = n0 + 32 <= p.n;
    if (p.out_dt == NXB_BF16 || p.out_dt == NXB_F16) {
      unsigned short* out = (unsigned short*)p.c + rowoff + n0;
      if (full && vec_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 pk;
          unsigned short h[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) h[e] = p.out_dt == NXB_BF16 ? f32_to_bf16_bits(f[j + e]) : f32_to_f16_bits(f[j + e]);
          pk.x = h[0] | ((uint32_t)h[1] << 16); pk.y = h[2] | ((uint32_t)h[3] << 16);
          pk.z = h[4] | ((uint32_t)h[5] << 16); pk.w = h[6] | ((uint32_t)h[7] << 16);
          *reinterpret_cast<uint4*>(out + j) = pk;
        }
      } else {
        for (int j = 0; j < 32 && n0 + j < p.n; ++j) out[j] = p.out_dt == NXB_BF16 ? f32_to_bf16_bits(f[j]) : f32_to_f16_bits(f[j]);
      }
    } else if (p.out_dt == NXB_F32) {
      float* out = (float*)p.c + rowoff + n0;
      if (full && (p.n % 4) == 0 && base_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
      } else {
        for (int j = 0; j < 32 && n0 + j < p.n; ++j) out[j] = f[j];
      }
    } else if (p.out_dt == NXB_S32 || p.out_dt == NXB_U32) {
      int* out = (int*)p.c + rowoff + n0;
      if (full && (p.n % 4) == 0 && base_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) *reinterpret_cast<int4*>(out + j) = make_int4((int)v[j], (int)v[j + 1], (int)v[j + 2], (int)v[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (n0 + j < p.n) out[j] = (int)v[j];
      }
    } else {   // 8-bit integer result: the 32-bit sum written modulo 2^8
      unsigned char* out = (unsigned char*)p.c + rowoff + n0;
      if (full && (p.n % 16) == 0 && base_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 16) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            w[e] = (v[j + 4 * e] & 0xFFu) | ((v[j + 4 * e + 1] & 0xFFu) << 8) | ((v[j + 4 * e + 2] & 0xFFu) << 16) | (v[j + 4 * e + 3] << 24);
          *reinterpret_cast<uint4*>(out + j) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (n0 + j < p.n) out[j] = (unsigned char)v[j];
      }
    }
  }
};

// Tile t of this CTA's walk.  Plain products: consecutive CTAs share a column panel of B and walk
// down M.  Fused with the sum over ranks: the tiles owned by the next rank come first and this
// rank's own tiles last, so every owner finds its peers' contributions early.
template <bool COMM>
__device__ __forceinline__ void tile_coords(long long t, const TcParams& p, const CommArgs* cm, int& b, int& mt, int& nt) {
  if (!COMM) {
    const long long tiles_per_batch = (long long)p.mtiles * p.ntiles;
    b = (int)(t / tiles_per_batch);
    const int r = (int)(t % tiles_per_batch);
    // Panels of `panel_m` row tiles, walked column by column: the 148 tiles in flight then cover about
    // 16 x 9 tiles, so one wave touches a few tens of MB of the operands (they stay in L2 from wave to
    // wave) instead of every row of A.
    const int per_panel = p.panel_m * p.ntiles;
    const int panel = r / per_panel, j = r % per_panel;
    const int rows = min(p.panel_m, p.mtiles - panel * p.panel_m);
    nt = j / rows;
    if (panel & 1) nt = p.ntiles - 1 - nt;     // odd panels walk back: the columns of B just used are still in L2
    mt = panel * p.panel_m + j % rows;
  } else {
    const int mpo = p.mtiles / cm->world;
    const long long per_owner = (long long)mpo * p.ntiles;
    const int k = (int)(t / per_owner), j = (int)(t % per_owner);
    const int owner = (cm->rank + 1 + k) % cm->world;
    b = 0;
    nt = j / mpo;
    mt = (j % mpo) * cm->world + owner;
  }
}

// The role of warps 6..9 of the fused kernel: reduce the tiles this rank owns (reading every
// rank's partial tile), then fetch the tiles the other ranks reduced.  `cw` = 32-row quarter.
template <int BN>
__device__ __forceinline__ void comm_role(const TcParams& p, const CommArgs& cm, volatile int* abort_flag) {
  const int cw = (threadIdx.x >> 5) - 6, lane = threadIdx.x & 31;
  const int mpo = p.mtiles / cm.world;
  const int per_owner = mpo * p.ntiles;
  constexpr int VPR = BN / 8;                 // 16-byte vectors per tile row
  bool ok = true;
  // ---- reduce the tiles this rank owns ----
  for (int j = blockIdx.x; j < per_owner && ok; j += gridDim.x) {
    const int nt = j / mpo, mt = (j % mpo) * cm.world + cm.rank;
    const long long fi = ((long long)nt * p.mtiles + mt) * 4 + cw;
    int got = 1;
    if (lane < cm.world) got = flag_wait(cm.ready[lane] + fi, cm.epoch, abort_flag);
    if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
    __syncwarp();
    // A warp pass covers 32 vectors of 16 bytes; eight passes are loaded together per rank so that
    // enough requests are in flight to cover the NVLink round trip.
    constexpr int RB = 8;
    for (int pb = 0; pb < VPR; pb += RB) {
      long long off[RB];
      float acc[RB][8];
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        const int idx = (pb + u) * 32 + lane;
        const long long gm = (long long)mt * BM + cw * 32 + idx / VPR, gn = (long long)nt * BN + (idx % VPR) * 8;
        off[u] = (gm < p.m && gn < p.n) ? gm * p.n + gn : -1;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      }
      // two ranks' tiles are requested together: 16 loads in flight per lane
      for (int r = 0; r < cm.world; r += 2) {
        uint4 v[2][RB];
        const bool two = r + 1 < cm.world;
#pragma unroll
        for (int u = 0; u < RB; ++u) {
          v[0][u] = off[u] >= 0 ? ld_sys_v4(cm.partial[r] + off[u]) : make_uint4(0, 0, 0, 0);
          v[1][u] = (two && off[u] >= 0) ? ld_sys_v4(cm.partial[r + 1] + off[u]) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int u = 0; u < RB; ++u) {
            const uint32_t w[4] = {v[h][u].x, v[h][u].y, v[h][u].z, v[h][u].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (p.out_dt == NXB_BF16) {
                acc[u][2 * e] += __uint_as_float(w[e] << 16);
                acc[u][2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
              } else {
                float lo, hi;
                asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}" : "=f"(lo), "=f"(hi) : "r"(w[e]));
                acc[u][2 * e] += lo;
                acc[u][2 * e + 1] += hi;
              }
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        if (off[u] < 0) continue;
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const unsigned short l = p.out_dt == NXB_BF16 ? f32_to_bf16_bits(acc[u][2 * e]) : f32_to_f16_bits(acc[u][2 * e]);
          const unsigned short h = p.out_dt == NXB_BF16 ? f32_to_bf16_bits(acc[u][2 * e + 1]) : f32_to_f16_bits(acc[u][2 * e + 1]);
          ow[e] = (uint32_t)l | ((uint32_t)h << 16);
        }
        *reinterpret_cast<uint4*>(cm.result[cm.rank] + off[u]) = o;
        *reinterpret_cast<uint4*>(cm.out + off[u]) = o;
      }
    }
    __syncwarp();
    if (lane == 0) {
      __threadfence_system();
      st_release_sys(cm.reduced[cm.rank] + fi, cm.epoch);
    }
  }
  // ---- fetch the tiles the other ranks own ----
  for (int k = 1; k < cm.world && ok; ++k) {
    const int owner = (cm.rank + k) % cm.world;
    for (int j = blockIdx.x; j < per_owner && ok; j += gridDim.x) {
      const int nt = j / mpo, mt = (j % mpo) * cm.world + owner;
      const long long fi = ((long long)nt * p.mtiles + mt) * 4 + cw;
      int got = 1;
      if (lane == 0) got = flag_wait(cm.reduced[owner] + fi, cm.epoch, abort_flag);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      __syncwarp();
      constexpr int CB = VPR < 16 ? VPR : 16;
      for (int pb = 0; pb < VPR; pb += CB) {
        long long off[CB];
        uint4 v[CB];
#pragma unroll
        for (int u = 0; u < CB; ++u) {
          const int idx = (pb + u) * 32 + lane;
          const long long gm = (long long)mt * BM + cw * 32 + idx / VPR, gn = (long long)nt * BN + (idx % VPR) * 8;
          off[u] = (gm < p.m && gn < p.n) ? gm * p.n + gn : -1;
          if (off[u] >= 0) v[u] = ld_sys_v4(cm.result[owner] + off[u]);
        }
#pragma unroll
        for (int u = 0; u < CB; ++u)
          if (off[u] >= 0) *reinterpret_cast<uint4*>(cm.out + off[u]) = v[u];
      }
    }
  }
}

template <int KIND, int BN, class Epi, bool COMM = false>
__device__ __forceinline__ void tc_gemm_body(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c, const TcParams& p,
                                             const CommArgs* cm = nullptr) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int STAGES = stages_for(BN);
  constexpr int B_STAGE = BN * ROW_BYTES;
  constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;      // two accumulators; a power of two >= 32
  constexpr int BK = (KIND == KIND_S8) ? 128 : 64;          // elements per 128-byte row
  constexpr int UMMA_K_BYTES = 32;                          // one MMA consumes 32 bytes of K per row

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = base, sB = base + STAGES * A_STAGE;
  const uint32_t sStore = sB + STAGES * B_STAGE;          // 1024-byte aligned: stage sizes are multiples of 8 KB
  const uint32_t bars = sStore + STORE_STAGE;
  const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, tfull0 = bars + 16 * STAGES, tempty0 = tfull0 + 16;
  const uint32_t tmem_slot = tempty0 + 16;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + (tmem_slot - base));
  volatile int* abort_flag = (volatile int*)(gen_base + (tmem_slot - base) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A block of ten warps (without the exchange role) has two groups of four epilogue warps; each group
  // takes half of the tile's columns.  Products with a short k loop are bound by the epilogue.
  const int epi_groups = (!COMM && blockDim.x >= 320) ? 2 : 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4 * epi_groups); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  const int kblocks = (p.k + BK - 1) / BK;
  const long long tiles_per_batch = (long long)p.mtiles * p.ntiles;
  const long long ntiles_total = tiles_per_batch * p.batch;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < ntiles_total && ok; t += gridDim.x) {
        int b, mt, nt;
        tile_coords<COMM>(t, p, cm, b, mt, nt);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full0 + 8 * s, A_STAGE + B_STAGE);
          if (!p.a_mn) {
            tma_load_3d(sA + s * A_STAGE, &map_a, full0 + 8 * s, kb * BK, mt * BM, b);
          } else if (p.a_mn == 2) {
            // [k][m] operand: groups of 64 m x 64 k, 8 KB each, all groups of the tile in one copy
            tma_load_4d(sA + s * A_STAGE, &map_a, full0 + 8 * s, 0, kb * BK, mt * (BM / 64), b);
          } else {
            for (int j = 0; j < BM / 64; ++j) tma_load_3d(sA + s * A_STAGE + j * 8192, &map_a, full0 + 8 * s, mt * BM + j * 64, kb * BK, b);
          }
          if (!p.b_mn) {
            tma_load_3d(sB + s * B_STAGE, &map_b, full0 + 8 * s, kb * BK, nt * BN, b);
          } else if (p.b_mn == 2) {
            tma_load_4d(sB + s * B_STAGE, &map_b, full0 + 8 * s, 0, kb * BK, nt * (BN / 64), b);
          } else {
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(sB + s * B_STAGE + j * 8192, &map_b, full0 + 8 * s, nt * BN + j * 64, kb * BK, b);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: f32 (or s32) accumulate, both operands K-major, N=256, M=128
      uint32_t idesc;
      if (KIND == KIND_S8) idesc = (2u << 4) | (1u << 7) | (1u << 10);
      else if (KIND == KIND_BF16) idesc = (1u << 4) | (1u << 7) | (1u << 10);
      else idesc = (1u << 4);
      idesc |= ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      idesc |= (p.a_mn ? (1u << 15) : 0u) | (p.b_mn ? (1u << 16) : 0u);
      // descriptor advance per MMA: 32 bytes along a K-major row, or two 8-row groups (2048 bytes)
      const uint64_t astep = p.a_mn ? (2048 >> 4) : (UMMA_K_BYTES >> 4), bstep = p.b_mn ? (2048 >> 4) : (UMMA_K_BYTES >> 4);
      int s = 0, a = 0;
      uint32_t ph = 0, aph = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < ntiles_total && ok; t += gridDim.x) {
        if (!mbar_wait(tempty0 + 8 * a, aph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = p.a_mn ? make_desc_mn(sA + s * A_STAGE) : make_desc(sA + s * A_STAGE);
          const uint64_t bdesc = p.b_mn ? make_desc_mn(sB + s * B_STAGE) : make_desc(sB + s * B_STAGE);
#pragma unroll
          for (int k4 = 0; k4 < ROW_BYTES / UMMA_K_BYTES; ++k4)
            tc_mma(d_tmem, adesc + (uint64_t)k4 * astep, bdesc + (uint64_t)k4 * bstep, idesc,
                   (kb > 0 || k4 > 0) ? 1u : 0u, KIND == KIND_S8);
          tc_commit(empty0 + 8 * s);        // the stage is free once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) tc_commit(tfull0 + 8 * a);  // accumulator complete
        if (++a == 2) { a = 0; aph ^= 1; }
      }
    }
  } else if (COMM && warp >= 6) {
    comm_role<BN>(p, *cm, abort_flag);
  } else {
    // epilogue warps 2..5 (and 6..9 as a second group); a warp may only read the TMEM lanes of its
    // quarter (warp id mod 4)
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;
    const int c_per = (BN / 32) / epi_groups, c0 = grp * c_per, c1 = c0 + c_per;
    const uint32_t stage_bytes = 8192u / (uint32_t)epi_groups;     // staging memory of one warp
    // Plain 16-bit results without a scale take a short path: packed converts straight from the
    // accumulator registers, store offsets of this lane computed once.
    const bool lean = KIND != KIND_S8 && Epi::kStaged && !Epi::kTransform && p.tma_store != 0 && !p.scale && (p.out_dt == NXB_BF16 || p.out_dt == NXB_F16);
    const uint32_t lean_slots = stage_bytes / 2048u;                // 4 or 2
    const uint32_t lean_base = sStore + (uint32_t)(warp - 2) * stage_bytes + (uint32_t)lane * 64u;
    const uint32_t lean_sw = (uint32_t)((lane >> 1) & 3);
    uint32_t store_iter = 0;
    int a = 0;
    uint32_t aph = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < ntiles_total && ok; t += gridDim.x) {
      int b, mt, nt;
      tile_coords<COMM>(t, p, cm, b, mt, nt);
      // warp-uniform outcome: the tensor-memory loads below need the whole warp
      if (!mbar_wait_warp(tfull0 + 8 * a, aph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const long long m = (long long)mt * BM + q * 32 + lane;
      const bool staged = Epi::kStaged && p.tma_store != 0;
      const uint32_t tacc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN);
      auto chunk = [&](int c, uint32_t (&v)[32]) {
        const long long n0 = (long long)nt * BN + c * 32;
        if (lean) {
          if ((long long)mt * BM + q * 32 >= p.m || n0 >= p.n) return;        // warp-uniform
          uint32_t h[16];
          if (p.out_dt == NXB_BF16) {
#pragma unroll
            for (int e = 0; e < 16; ++e) h[e] = bits2_to_bf16x2(v[2 * e], v[2 * e + 1]);
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) h[e] = bits2_to_f16x2(v[2 * e], v[2 * e + 1]);
          }
          if (p.tma_store == 2) {
            // all staging tiles of this warp are one group: written side by side, handed over in ONE store
            // through the four-dimensional map {32 columns, m, group of 32 columns, batch}
            const uint32_t slot = (uint32_t)(c - c0) & (lean_slots - 1);
            const uint32_t gbuf = lean_base + slot * 2048u;
            if (slot == 0) {
              if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous group has been read
              __syncwarp();
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(gbuf + (((uint32_t)j ^ lean_sw) << 4)), "r"(h[4 * j]), "r"(h[4 * j + 1]),
                           "r"(h[4 * j + 2]), "r"(h[4 * j + 3]) : "memory");
            if (slot == lean_slots - 1 || n0 + 32 >= p.n) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0)
                tma_store_4d(&map_c, sStore + (uint32_t)(warp - 2) * stage_bytes, 0, mt * BM + q * 32, (int)(n0 / 32) - (int)slot, b);
            }
            return;
          }
          const uint32_t buf = lean_base + (store_iter & (lean_slots - 1)) * 2048u;    // this lane's 64-byte row
          if (lane == 0) {   // the tile about to be overwritten must have been read by the TMA unit
            if (lean_slots == 4) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j)      // 64-byte swizzle: 16-byte chunk j of row r sits at chunk j ^ ((r >> 1) & 3)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(buf + (((uint32_t)j ^ lean_sw) << 4)), "r"(h[4 * j]), "r"(h[4 * j + 1]),
                         "r"(h[4 * j + 2]), "r"(h[4 * j + 3]) : "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) tma_store_3d(&map_c, buf, (int)n0, mt * BM + q * 32, b);
          ++store_iter;
          return;
        }
        if (staged) {
          // 32 rows x 32 columns of this warp go to a swizzled staging tile; one lane hands the
          // tile to the TMA unit, which writes full lines and clips at the matrix edges.
          if ((long long)mt * BM + q * 32 >= p.m || n0 >= p.n) return;        // warp-uniform
          // each warp owns 8 KB of staging (4 KB with two groups): tiles of 2 KB for 2-byte results, of 4 KB otherwise
          const bool two_byte = p.out_dt == NXB_BF16 || p.out_dt == NXB_F16;
          const uint32_t slots = stage_bytes / (two_byte ? 2048u : 4096u);      // 4, 2 or 1
          const uint32_t buf = sStore + (uint32_t)(warp - 2) * stage_bytes + (store_iter & (slots - 1)) * (two_byte ? 2048u : 4096u);
          if (lane == 0) {   // the tile about to be overwritten must have been read by the TMA unit
            if (slots == 4) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
            else if (slots == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          __syncwarp();
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = (KIND == KIND_S8) ? (float)(int)v[j] : __uint_as_float(v[j]);
          if (p.scale) {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (n0 + j < p.n) f[j] *= p.scale[n0 + j];
          }
          if (Epi::kTransform && m < p.m) Epi::transform(p, f, (long long)b, m, n0);
          if (p.out_dt == NXB_BF16 || p.out_dt == NXB_F16) {
            // rows of 64 bytes, 64-byte swizzle: 16-byte chunk j of row r sits at chunk j ^ ((r >> 1) & 3)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t h[4];                 // one packed convert per pair
#pragma unroll
              for (int e = 0; e < 4; ++e)
                h[e] = p.out_dt == NXB_BF16 ? f32x2_to_bf16x2(f[j * 8 + 2 * e], f[j * 8 + 2 * e + 1]) : f32x2_to_f16x2(f[j * 8 + 2 * e], f[j * 8 + 2 * e + 1]);
              const uint32_t dst = buf + (uint32_t)lane * 64u + (uint32_t)((j ^ ((lane >> 1) & 3)) * 16);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
            }
          } else {
            // 4-byte results: rows of 128 bytes, 128-byte swizzle: chunk j of row r sits at chunk j ^ (r & 7)
            const bool as_int = p.out_dt == NXB_S32 || p.out_dt == NXB_U32;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) w[e] = as_int ? v[j * 4 + e] : __float_as_uint(f[j * 4 + e]);
              const uint32_t dst = buf + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) * 16);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) tma_store_3d(&map_c, buf, (int)n0, mt * BM + q * 32, b);
          ++store_iter;
          return;
        }
        if (m < p.m && n0 < p.n) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = (KIND == KIND_S8) ? (float)(int)v[j] : __uint_as_float(v[j]);
          if (p.scale) {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (n0 + j < p.n) f[j] *= p.scale[n0 + j];
          }
          Epi::store(p, f, v, (long long)b, m, n0);
        }
      };
      // two register sets: the load of the next 32 columns is in flight while these are handled
      uint32_t va[32], vb[32];
      tmem_ld32_issue(tacc + (uint32_t)(c0 * 32), va);
#pragma unroll 1
      for (int c = c0; c < c1; c += 2) {
        tmem_ld_wait();
        if (c + 1 < c1) tmem_ld32_issue(tacc + (uint32_t)((c + 1) * 32), vb);
        chunk(c, va);
        if (c + 1 < c1) {
          tmem_ld_wait();
          if (c + 2 < c1) tmem_ld32_issue(tacc + (uint32_t)((c + 2) * 32), va);
          chunk(c + 1, vb);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * a);
      if (COMM && lane == 0) {
        // this warp's 32 rows of the tile are in memory: publish them to every rank
        __threadfence_system();
        st_release_sys(cm->ready[cm->rank] + ((long long)nt * p.mtiles + mt) * 4 + q, cm->epoch);
      }
      if (++a == 2) { a = 0; aph ^= 1; }
    }
    // the staging tiles must stay valid until the TMA unit has read them
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // teardown: everyone meets, copies in flight are given time to land if a wait gave up
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}


}  // namespace nxb_gemm

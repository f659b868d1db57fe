// Tensor-core matrix product for sm_100a: tcgen05.mma with the accumulator in
// tensor memory, operands staged in shared memory by TMA.
//
//   C[b][m][n] = sum_k A[b][m][k] * B[b][n][k]        (both operands K-major)
//
// One persistent CTA per SM walks output tiles of 128 x 256.  Warp roles:
//   warp 0      TMA producer: fills a 4-stage ring of {A 128x64, B 256x64} tiles
//               (128-byte swizzle; out-of-range rows/columns arrive as zeros)
//   warp 1      MMA issuer: one elected lane issues 4 tcgen05.mma (K=16 each, or
//               K=32 for 8-bit operands) per stage into one of two 256-column TMEM
//               accumulators, then commits the stage back to the producer
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (32 lanes per warp),
//               convert, and store; runs while the next tile's MMAs fill the other
//               accumulator
// Every mbarrier wait is bounded: after about two seconds a waiter raises the
// abort flag, all roles leave their loops, tensor memory is released, and the
// host reports NXB_ERR_TIMEOUT.
#include <cuda.h>

#include "gemm.h"

namespace nxb {
namespace {

constexpr int BM = 128;
constexpr int ROW_BYTES = 128;                        // one swizzle row: 64 bf16 or 128 s8
constexpr int A_STAGE = BM * ROW_BYTES;
// The tile width BN is 256 for large products; narrow outputs (few rows, e.g. a linear layer
// applied to 1..128 tokens) use 128 or 64 so that enough tiles exist to occupy every SM, with a
// deeper ring since the product is then bound by streaming the weights.
__host__ __device__ constexpr int stages_for(int bn) { return bn == 256 ? 4 : bn == 128 ? 6 : 8; }
__host__ __device__ constexpr int smem_bytes_for(int bn) { return stages_for(bn) * (A_STAGE + bn * ROW_BYTES) + 1024 /*alignment*/ + 256 /*barriers*/; }
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

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
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
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
  const unsigned long long t0 = now_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (now_ns() - t0 > WAIT_LIMIT_NS) {
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

// Shared-memory matrix descriptor of a K-major tile stored in 128-byte swizzled rows:
// 8-row groups are 1024 bytes apart (stride offset), the leading offset is unused (1),
// version 1, layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}

__device__ __forceinline__ unsigned short f32_to_bf16_bits(float f) {
  unsigned short h;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f));
  return h;
}
__device__ __forceinline__ unsigned short f32_to_f16_bits(float f) {
  unsigned short h;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f));
  return h;
}

template <int KIND, int BN>
__global__ void __launch_bounds__(192, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int STAGES = stages_for(BN);
  constexpr int B_STAGE = BN * ROW_BYTES;
  constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;      // two accumulators; a power of two >= 32
  constexpr int BK = (KIND == KIND_S8) ? 128 : 64;          // elements per 128-byte row
  constexpr int UMMA_K_BYTES = 32;                          // one MMA consumes 32 bytes of K per row

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = base, sB = base + STAGES * A_STAGE;
  const uint32_t bars = sB + STAGES * B_STAGE;
  const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, tfull0 = bars + 16 * STAGES, tempty0 = tfull0 + 16;
  const uint32_t tmem_slot = tempty0 + 16;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + (tmem_slot - base));
  volatile int* abort_flag = (volatile int*)(gen_base + (tmem_slot - base) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
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
        const int b = (int)(t / tiles_per_batch);
        const int r = (int)(t % tiles_per_batch);
        // consecutive CTAs share the same 256-wide column panel of B and walk down M
        const int nt = r / p.mtiles, mt = r % p.mtiles;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full0 + 8 * s, A_STAGE + B_STAGE);
          tma_load_3d(sA + s * A_STAGE, &map_a, full0 + 8 * s, kb * BK, mt * BM, b);
          tma_load_3d(sB + s * B_STAGE, &map_b, full0 + 8 * s, kb * BK, nt * BN, b);
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
          const uint64_t adesc = make_desc(sA + s * A_STAGE), bdesc = make_desc(sB + s * B_STAGE);
#pragma unroll
          for (int k4 = 0; k4 < ROW_BYTES / UMMA_K_BYTES; ++k4)
            tc_mma(d_tmem, adesc + (uint64_t)(k4 * (UMMA_K_BYTES >> 4)), bdesc + (uint64_t)(k4 * (UMMA_K_BYTES >> 4)), idesc,
                   (kb > 0 || k4 > 0) ? 1u : 0u, KIND == KIND_S8);
          tc_commit(empty0 + 8 * s);        // the stage is free once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) tc_commit(tfull0 + 8 * a);  // accumulator complete
        if (++a == 2) { a = 0; aph ^= 1; }
      }
    }
  } else {
    // epilogue warps 2..5; a warp may only read the TMEM lanes of its quarter (warp id mod 4)
    const int q = warp & 3;
    int a = 0;
    uint32_t aph = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < ntiles_total && ok; t += gridDim.x) {
      const int b = (int)(t / tiles_per_batch);
      const int r = (int)(t % tiles_per_batch);
      const int nt = r / p.mtiles, mt = r % p.mtiles;
      if (!mbar_wait(tfull0 + 8 * a, aph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const long long m = (long long)mt * BM + q * 32 + lane;
      const long long rowoff = ((long long)b * p.m + m) * p.n;
      const bool vec_ok = (p.n % 8) == 0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN + c * 32), v);
        const long long n0 = (long long)nt * BN + c * 32;
        if (m < p.m && n0 < p.n) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = (KIND == KIND_S8) ? (float)(int)v[j] : __uint_as_float(v[j]);
          if (p.scale) {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (n0 + j < p.n) f[j] *= p.scale[n0 + j];
          }
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
            if (full && (p.n % 4) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            } else {
              for (int j = 0; j < 32 && n0 + j < p.n; ++j) out[j] = f[j];
            }
          } else if (p.out_dt == NXB_S32 || p.out_dt == NXB_U32) {
            int* out = (int*)p.c + rowoff + n0;
            for (int j = 0; j < 32 && n0 + j < p.n; ++j) out[j] = (int)v[j];
          } else {   // 8-bit integer result: the 32-bit sum written modulo 2^8
            unsigned char* out = (unsigned char*)p.c + rowoff + n0;
            for (int j = 0; j < 32 && n0 + j < p.n; ++j) out[j] = (unsigned char)v[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * a);
      if (++a == 2) { a = 0; aph ^= 1; }
    }
  }

  // teardown: everyone meets, copies in flight are given time to land if a wait gave up
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) *(volatile int*)p.status = 1;
    const unsigned long long t0 = now_ns();
    while (now_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

CUtensorMapDataType tm_type(DType t) {
  switch (t) {
    case NXB_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case NXB_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

// K-major operand [batch][rows][k] as a 3-D tensor map with 128-byte swizzled boxes of `box_rows` rows.
CUtensorMap make_map(const void* ptr, DType dt, int64_t k, int64_t rows, int64_t batch, int64_t ld, int64_t bs, int box_rows) {
  const DriverApi& drv = driver();
  if (!drv.cuTensorMapEncodeTiled) fail(NXB_ERR_RUNTIME, "cuTensorMapEncodeTiled is unavailable");
  CUtensorMap m;
  const size_t es = dtype_size(dt);
  cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)(ld * es), (cuuint64_t)(std::max<int64_t>(bs, 1) * es)};
  if (batch == 1) strides[1] = (cuuint64_t)(ld * es) * (cuuint64_t)rows;
  cuuint32_t box[3] = {(cuuint32_t)(ROW_BYTES / es), (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  check_cu(drv.cuTensorMapEncodeTiled(&m, tm_type(dt), 3, const_cast<void*>(ptr), dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
           "cuTensorMapEncodeTiled");
  return m;
}

// out[b][c][r] = in[b][r][c] for 1- and 2-byte elements (operands whose reduction index is
// not contiguous are brought to K-major form before the tensor-core product).
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T* __restrict__ in, T* __restrict__ out, long long rows, long long cols) {
  __shared__ T tile[64][64 + 2];
  const long long b = blockIdx.z;
  in += b * rows * cols;
  out += b * rows * cols;
  const long long r0 = (long long)blockIdx.y * 64, c0 = (long long)blockIdx.x * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int i = ty; i < 64; i += 4) {
    long long r = r0 + i, c = c0 + tx;
    if (r < rows && c < cols) tile[i][tx] = in[r * cols + c];
  }
  __syncthreads();
  for (int i = ty; i < 64; i += 4) {
    long long c = c0 + i, r = r0 + tx;
    if (r < rows && c < cols) out[c * rows + r] = tile[tx][i];
  }
}

}  // namespace

void launch_transpose(const void* in, void* out, int64_t batch, int64_t rows, int64_t cols, size_t elem_size, cudaStream_t stream) {
  if (batch == 0 || rows == 0 || cols == 0) return;
  dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64), (unsigned)batch);
  if (elem_size == 2) transpose_kernel<unsigned short><<<grid, 256, 0, stream>>>((const unsigned short*)in, (unsigned short*)out, rows, cols);
  else if (elem_size == 1) transpose_kernel<unsigned char><<<grid, 256, 0, stream>>>((const unsigned char*)in, (unsigned char*)out, rows, cols);
  else fail(NXB_ERR_RUNTIME, "internal: transpose of this element size");
  NXB_CUDA(cudaGetLastError());
}

// Types and sizes the tensor-core kernel takes.  Operands that are not K-major are
// transposed into scratch first by the caller, so `ta`/`tb` do not matter here.
bool tc_gemm_supported(const GemmArgs& g) {
  if (g.da != g.db) return false;
  const bool f16 = g.da == NXB_BF16 || g.da == NXB_F16;
  const bool i8 = g.da == NXB_S8;
  if (!f16 && !i8) return false;
  if (f16 && !(g.dc == g.da || g.dc == NXB_F32)) return false;
  if (i8 && !(g.dc == NXB_S32 || g.dc == NXB_S8 || g.dc == NXB_F32)) return false;
  const size_t es = dtype_size(g.da);
  // TMA: 16-byte aligned base, strides multiple of 16 bytes (after any transpose both
  // operands have leading dimension k)
  if ((g.k * es) % 16 || ((g.m * g.k) * es) % 16 || ((g.n * g.k) * es) % 16) return false;
  if (((uintptr_t)g.a) % 16 || ((uintptr_t)g.b) % 16) return false;
  if (g.batch > 65535) return false;
  if (g.m < 1 || g.n < 1 || g.k < 1 || g.batch < 1) return false;
  if (g.k >= (int64_t(1) << 31) || g.m >= (int64_t(1) << 31) || g.n >= (int64_t(1) << 31)) return false;
  return true;
}

void launch_tc_gemm(const GemmArgs& g, int* status_word, int sm_count, cudaStream_t stream) {
  CUtensorMap ma = make_map(g.a, g.da, g.k, g.m, g.batch, g.lda, g.bsa, BM);
  // tile width: the widest one that still yields at least one tile per SM
  const long long mt = (g.m + BM - 1) / BM;
  int bn = 256;
  if (mt * ((g.n + 255) / 256) * g.batch < sm_count) bn = 128;
  if (bn == 128 && mt * ((g.n + 127) / 128) * g.batch < sm_count) bn = 64;
  CUtensorMap mb = make_map(g.b, g.db, g.k, g.n, g.batch, g.ldb, g.bsb, bn);
  TcParams p{};
  p.c = g.c;
  p.bias = g.bias;
  p.scale = (const float*)g.scale;
  p.status = status_word;
  p.m = (int)g.m; p.n = (int)g.n; p.k = (int)g.k; p.batch = (int)g.batch;
  p.mtiles = (int)((g.m + BM - 1) / BM);
  p.ntiles = (int)((g.n + bn - 1) / bn);
  p.out_dt = g.dc;
  p.epilogue = g.epilogue;
  long long tiles = (long long)p.mtiles * p.ntiles * p.batch;
  unsigned grid = (unsigned)std::min<long long>(tiles, sm_count);
  auto launch = [&](auto kern, int smem) {
    NXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, 192, smem, stream>>>(ma, mb, p);
    NXB_CUDA(cudaGetLastError());
  };
#define NXB_LAUNCH_KIND(K)                                                      \
  do {                                                                          \
    if (bn == 256) launch(tc_gemm_kernel<K, 256>, smem_bytes_for(256));         \
    else if (bn == 128) launch(tc_gemm_kernel<K, 128>, smem_bytes_for(128));    \
    else launch(tc_gemm_kernel<K, 64>, smem_bytes_for(64));                     \
  } while (0)
  if (g.da == NXB_BF16) NXB_LAUNCH_KIND(KIND_BF16);
  else if (g.da == NXB_F16) NXB_LAUNCH_KIND(KIND_F16);
  else NXB_LAUNCH_KIND(KIND_S8);
#undef NXB_LAUNCH_KIND
}

}  // namespace nxb

// ---------------------------------------------------------------------------------------
// Matrix product that allocates nothing.
//
// Some callers cannot let this library call cudaMalloc: an application that has
// already given (nearly) all device memory to another allocator — e.g. an XLA
// client started with `preallocate: true`, which takes its memory fraction up
// front — would see the allocation fail, and a serving loop with a latency
// budget cannot afford the device-wide synchronisation a cudaMalloc implies.
// For them the scratch the product needs (the K-major copy of B) lives in a
// fixed array inside the library image: every GPU that loads the library
// reserves NOALLOC_SCRATCH_BYTES for as long as the process lives.
constexpr size_t NOALLOC_SCRATCH_BYTES = size_t(32) << 20;   // 32 MiB: B of up to 16 Mi bf16 elements
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
static __device__ int g_noalloc_status;

namespace {
struct NoAllocDevice {
  void* scratch = nullptr;   // device address of g_noalloc_scratch on this device
  int* status = nullptr;     // device address of g_noalloc_status on this device
  int sm_count = 0;
};
std::mutex g_noalloc_mu;
std::map<int, NoAllocDevice> g_noalloc_devices;
}  // namespace

extern "C" int nxb200_dot_bf16_static_scratch(int device, const void* a, const void* b, void* c, int64_t m, int64_t n,
                                              int64_t k, void* stream_handle) {
  using namespace nxb;
  try {
    cudaStream_t stream = (cudaStream_t)stream_handle;
    if (!a || !b || !c) fail(NXB_ERR_INVALID_ARGUMENT, "a, b and c must be device pointers");
    if (m < 1 || n < 1 || k < 1) fail(NXB_ERR_INVALID_ARGUMENT, "m, n and k must be positive");
    if (k % 8 != 0 || n % 8 != 0)
      fail(NXB_ERR_INVALID_ARGUMENT, "k and n must be multiples of 8 (rows of both operands must start on 16-byte boundaries)");
    const size_t need = (size_t)n * (size_t)k * 2;
    if (need > NOALLOC_SCRATCH_BYTES)
      fail(NXB_ERR_INVALID_ARGUMENT, "operand b has " + std::to_string(need) + " bytes; the built-in scratch holds at most " +
                                         std::to_string(NOALLOC_SCRATCH_BYTES) + " (k*n <= " + std::to_string(NOALLOC_SCRATCH_BYTES / 2) + " elements)");
    NXB_CUDA(cudaSetDevice(device));
    NoAllocDevice dev;
    {
      // One-time set-up per device, with that device current: in host code the array's
      // name is only a handle, the address a kernel can use comes from the runtime.
      std::lock_guard<std::mutex> g(g_noalloc_mu);
      auto it = g_noalloc_devices.find(device);
      if (it == g_noalloc_devices.end()) {
        NoAllocDevice d;
        NXB_CUDA(cudaGetSymbolAddress(&d.scratch, g_noalloc_scratch));
        NXB_CUDA(cudaGetSymbolAddress((void**)&d.status, g_noalloc_status));
        NXB_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device));
        it = g_noalloc_devices.emplace(device, d).first;
      }
      dev = it->second;
    }
    // the status word must start at zero; the scratch is fully rewritten before it is read
    NXB_CUDA(cudaMemsetAsync(dev.status, 0, sizeof(int), stream));
    launch_transpose(b, dev.scratch, 1, k, n, 2, stream);          // B {k,n} -> {n,k}
    GemmArgs g{};
    g.a = a; g.b = dev.scratch; g.c = c;
    g.batch = 1; g.m = m; g.n = n; g.k = k;
    g.lda = k; g.ldb = k; g.bsa = m * k; g.bsb = n * k;
    g.ta = g.tb = false;
    g.da = g.db = g.dc = NXB_BF16;
    if (!tc_gemm_supported(g)) fail(NXB_ERR_INVALID_ARGUMENT, "operands must be 16-byte aligned");
    launch_tc_gemm(g, dev.status, dev.sm_count, stream);
    int status = 0;
    NXB_CUDA(cudaMemcpyAsync(&status, dev.status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    NXB_CUDA(cudaStreamSynchronize(stream));
    if (status) fail(NXB_ERR_TIMEOUT, "the product gave up waiting on an internal barrier; c is invalid");
    return NXB_OK;
  } catch (const Error& e) {
    set_last_error(e.msg);
    return e.status;
  } catch (const std::exception& e) {
    set_last_error(e.what());
    return NXB_ERR_RUNTIME;
  }
}

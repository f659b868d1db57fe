// CUDA-core matrix product for every Nx type combination.
//
// This is the exact path: integer products accumulate in wrapping integer
// arithmetic of the output width (the reference writes integers modulo 2^bits,
// nx/lib/nx/shared.ex:190-194), f32 accumulates in f32 with FMA, f64 in f64,
// and 16-bit floats accumulate in f32 and round once on store.  The tensor-core
// kernels take over the large bf16 / int8 shapes; this one covers small and
// mixed-type products (e.g. the MLP of the smallest configuration).
#include "gemm.h"

namespace nxb {
namespace {

__device__ __forceinline__ float bf16_bits_to_f32(unsigned short h) { return __uint_as_float(((unsigned)h) << 16); }
__device__ __forceinline__ float f16_bits_to_f32(unsigned short h) {
  float f;
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
  return f;
}

template <typename Acc>
__device__ __forceinline__ Acc load_as(const void* p, int dt, long long i) {
  switch (dt) {
    case NXB_U8: return (Acc)((const unsigned char*)p)[i];
    case NXB_U16: return (Acc)((const unsigned short*)p)[i];
    case NXB_U32: return (Acc)((const unsigned int*)p)[i];
    case NXB_U64: return (Acc)((const unsigned long long*)p)[i];
    case NXB_S8: return (Acc)((const signed char*)p)[i];
    case NXB_S16: return (Acc)((const short*)p)[i];
    case NXB_S32: return (Acc)((const int*)p)[i];
    case NXB_S64: return (Acc)((const long long*)p)[i];
    case NXB_F16: return (Acc)f16_bits_to_f32(((const unsigned short*)p)[i]);
    case NXB_BF16: return (Acc)bf16_bits_to_f32(((const unsigned short*)p)[i]);
    case NXB_F32: return (Acc)((const float*)p)[i];
    default: return (Acc)((const double*)p)[i];
  }
}

template <typename Acc>
__device__ __forceinline__ void store_as(void* p, int dt, long long i, Acc v) {
  switch (dt) {
    case NXB_U8: case NXB_S8: ((unsigned char*)p)[i] = (unsigned char)(unsigned long long)v; break;
    case NXB_U16: case NXB_S16: ((unsigned short*)p)[i] = (unsigned short)(unsigned long long)v; break;
    case NXB_U32: case NXB_S32: ((unsigned int*)p)[i] = (unsigned int)(unsigned long long)v; break;
    case NXB_U64: case NXB_S64: ((unsigned long long*)p)[i] = (unsigned long long)v; break;
    case NXB_F16: { unsigned short h; float f = (float)v; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); ((unsigned short*)p)[i] = h; break; }
    case NXB_BF16: { unsigned short h; float f = (float)v; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f)); ((unsigned short*)p)[i] = h; break; }
    case NXB_F32: ((float*)p)[i] = (float)v; break;
    default: ((double*)p)[i] = (double)v; break;
  }
}

// When a float operand is narrower than the output type of a mixed product it is first
// converted to the output type (rounded), as the reference's lowering converts operands.
template <typename Acc>
__device__ __forceinline__ Acc round_to(Acc v, int dt) {
  if (dt == NXB_BF16) { unsigned short h; float f = (float)v; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f)); return (Acc)bf16_bits_to_f32(h); }
  if (dt == NXB_F16) { unsigned short h; float f = (float)v; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return (Acc)f16_bits_to_f32(h); }
  if (dt == NXB_F32) return (Acc)(float)v;
  return v;
}

constexpr int TM = 64, TN = 64, TK = 16;

template <typename Acc>
__global__ void __launch_bounds__(256) simt_gemm_kernel(GemmArgs g) {
  __shared__ Acc As[TK][TM + 1];
  __shared__ Acc Bs[TK][TN + 1];
  const long long b = blockIdx.z;
  const long long m0 = (long long)blockIdx.y * TM, n0 = (long long)blockIdx.x * TN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  // element (m,k) of A and (k,n) of B through strides
  const long long sam = g.ta ? 1 : g.lda, sak = g.ta ? g.lda : 1;
  const long long sbn = g.tb ? 1 : g.ldb, sbk = g.tb ? g.ldb : 1;
  const char* abase = (const char*)g.a;
  const char* bbase = (const char*)g.b;
  const long long aoff = b * g.bsa, boff = b * g.bsb;
  Acc acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = (Acc)0;
  const bool cvt_a = g.da != g.dc && g.dc >= NXB_F16, cvt_b = g.db != g.dc && g.dc >= NXB_F16;
  for (long long k0 = 0; k0 < g.k; k0 += TK) {
    for (int e = threadIdx.x; e < TM * TK; e += 256) {
      // consecutive threads walk the contiguous index of the operand
      int kk = g.ta ? e / TM : e % TK, mm = g.ta ? e % TM : e / TK;
      long long m = m0 + mm, k = k0 + kk;
      Acc v = (Acc)0;
      if (m < g.m && k < g.k) { v = load_as<Acc>(abase, g.da, aoff + m * sam + k * sak); if (cvt_a) v = round_to(v, g.dc); }
      As[kk][mm] = v;
    }
    for (int e = threadIdx.x; e < TN * TK; e += 256) {
      int kk = g.tb ? e / TN : e % TK, nn = g.tb ? e % TN : e / TK;
      long long n = n0 + nn, k = k0 + kk;
      Acc v = (Acc)0;
      if (n < g.n && k < g.k) { v = load_as<Acc>(bbase, g.db, boff + n * sbn + k * sbk); if (cvt_b) v = round_to(v, g.dc); }
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      Acc av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      long long m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < g.m && n < g.n) store_as<Acc>(g.c, g.dc, (b * g.m + m) * g.n + n, acc[i][j]);
    }
}

// f32 x f32 -> f32: typed loads, the next k chunk fetched into registers while the current one
// is multiplied, one barrier per chunk (two shared-memory buffers).  TM x TN outputs per CTA of
// 256 threads, RM x RN per thread; the small tile spreads small products (the MLP configuration)
// over more SMs.
template <int TM, int TN, int RM, int RN, int TK>
__global__ void __launch_bounds__(256) sgemm_kernel(GemmArgs g) {
  constexpr int LA = TM * TK / 256, LB = TN * TK / 256;      // elements each thread stages per chunk
  static_assert((TM / RM) * (TN / RN) == 256, "256 threads per tile");
  __shared__ float As[2][TK][TM + 4];
  __shared__ float Bs[2][TK][TN + 4];
  const long long b = blockIdx.z;
  const long long m0 = (long long)blockIdx.y * TM, n0 = (long long)blockIdx.x * TN;
  const int tx = threadIdx.x % (TN / RN), ty = threadIdx.x / (TN / RN);
  const long long sam = g.ta ? 1 : g.lda, sak = g.ta ? g.lda : 1;
  const long long sbn = g.tb ? 1 : g.ldb, sbk = g.tb ? g.ldb : 1;
  const float* A = (const float*)g.a + b * g.bsa;
  const float* B = (const float*)g.b + b * g.bsb;
  float ra[LA], rb[LB];
  auto fetch = [&](long long k0) {
#pragma unroll
    for (int i = 0; i < LA; ++i) {
      const int e = threadIdx.x + i * 256;
      // consecutive threads walk the contiguous index of the operand
      const int kk = g.ta ? e / TM : e % TK, mm = g.ta ? e % TM : e / TK;
      const long long m = m0 + mm, k = k0 + kk;
      ra[i] = (m < g.m && k < g.k) ? A[m * sam + k * sak] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < LB; ++i) {
      const int e = threadIdx.x + i * 256;
      const int kk = g.tb ? e / TN : e % TK, nn = g.tb ? e % TN : e / TK;
      const long long n = n0 + nn, k = k0 + kk;
      rb[i] = (n < g.n && k < g.k) ? B[n * sbn + k * sbk] : 0.f;
    }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int i = 0; i < LA; ++i) {
      const int e = threadIdx.x + i * 256;
      const int kk = g.ta ? e / TM : e % TK, mm = g.ta ? e % TM : e / TK;
      As[buf][kk][mm] = ra[i];
    }
#pragma unroll
    for (int i = 0; i < LB; ++i) {
      const int e = threadIdx.x + i * 256;
      const int kk = g.tb ? e / TN : e % TK, nn = g.tb ? e % TN : e / TK;
      Bs[buf][kk][nn] = rb[i];
    }
  };
  float acc[RM][RN];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < RN; ++j) acc[i][j] = 0.f;
  fetch(0);
  stage(0);
  __syncthreads();
  int buf = 0;
  for (long long k0 = 0; k0 < g.k; k0 += TK) {
    const bool more = k0 + TK < g.k;
    if (more) fetch(k0 + TK);
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float av[RM], bv[RN];
#pragma unroll
      for (int i = 0; i < RM; ++i) av[i] = As[buf][kk][ty * RM + i];
#pragma unroll
      for (int j = 0; j < RN; ++j) bv[j] = Bs[buf][kk][tx * RN + j];
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < RN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (more) stage(buf ^ 1);        // the other buffer was last read before the previous barrier
    __syncthreads();
    buf ^= 1;
  }
  float* C = (float*)g.c + b * g.m * g.n;
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < RN; ++j) {
      const long long m = m0 + ty * RM + i, n = n0 + tx * RN + j;
      if (m < g.m && n < g.n) C[m * g.n + n] = acc[i][j];
    }
}

}  // namespace

void launch_simt_gemm(const GemmArgs& g, cudaStream_t stream) {
  if (g.batch == 0 || g.m == 0 || g.n == 0) return;
  if (g.batch > 65535) fail(NXB_ERR_UNSUPPORTED, "dot with more than 65535 batch entries on the CUDA-core path");
  if (g.da == NXB_F32 && g.db == NXB_F32 && g.dc == NXB_F32 && !g.bias && !g.scale) {
    // small tiles until the grid fills the machine a few times over
    const long long big = ((g.m + 63) / 64) * ((g.n + 63) / 64) * g.batch;
    if (big >= 296) {
      dim3 grid((unsigned)((g.n + 63) / 64), (unsigned)((g.m + 63) / 64), (unsigned)g.batch);
      sgemm_kernel<64, 64, 4, 4, 16><<<grid, 256, 0, stream>>>(g);
    } else {
      dim3 grid((unsigned)((g.n + 31) / 32), (unsigned)((g.m + 15) / 16), (unsigned)g.batch);
      sgemm_kernel<16, 32, 1, 2, 32><<<grid, 256, 0, stream>>>(g);
    }
    NXB_CUDA(cudaGetLastError());
    return;
  }
  dim3 grid((unsigned)((g.n + TN - 1) / TN), (unsigned)((g.m + TM - 1) / TM), (unsigned)g.batch);
  switch (g.dc) {
    case NXB_F64: simt_gemm_kernel<double><<<grid, 256, 0, stream>>>(g); break;
    case NXB_F16: case NXB_BF16: case NXB_F32: simt_gemm_kernel<float><<<grid, 256, 0, stream>>>(g); break;
    case NXB_U64: case NXB_S64: simt_gemm_kernel<unsigned long long><<<grid, 256, 0, stream>>>(g); break;
    default: simt_gemm_kernel<unsigned int><<<grid, 256, 0, stream>>>(g); break;
  }
  NXB_CUDA(cudaGetLastError());
}

}  // namespace nxb

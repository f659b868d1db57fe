// Nx.sort / Nx.argsort along the last axis (nx/lib/nx.ex:15600-15700, 15949-15990): one CTA per row,
// bitonic network over (key, position) pairs in shared memory.
//
// Every element type is mapped to an unsigned key whose integer order is the order Nx defines:
// signed integers by flipping the sign bit, floats by the usual sign-magnitude trick with -0.0
// folded onto +0.0 and every NaN mapped to the largest key ("NaN always sorts higher than any other
// value", nx.ex:15676-15689).  Ties are broken by position, which makes the result the stable one
// (the same permutation a stable sort returns) although a bitonic network itself is not stable.
// Descending order sorts the complemented keys, still breaking ties by ascending position.
#include "gemm.h"

namespace nxb {
namespace {

constexpr int SORT_MAX_LEN = 16384;

__device__ __forceinline__ unsigned f32_key(unsigned u) {
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;      // NaN
  if (u == 0x80000000u) u = 0;                                  // -0.0 == +0.0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long f64_key(unsigned long long u) {
  if ((u & 0x7fffffffffffffffull) > 0x7ff0000000000000ull) return ~0ull;
  if (u == 0x8000000000000000ull) u = 0;
  return (u & 0x8000000000000000ull) ? ~u : (u | 0x8000000000000000ull);
}
__device__ __forceinline__ unsigned half_key(unsigned short h, bool bf) {
  // widen to f32 bits (exactly) and reuse the f32 mapping
  unsigned u;
  if (bf) u = (unsigned)h << 16;
  else { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); u = __float_as_uint(f); }
  return f32_key(u);
}

template <typename K>
__device__ __forceinline__ K load_key(const void* p, int dt, long long i) {
  switch (dt) {
    case NXB_U8: return (K)((const unsigned char*)p)[i];
    case NXB_U16: return (K)((const unsigned short*)p)[i];
    case NXB_U32: return (K)((const unsigned int*)p)[i];
    case NXB_U64: return (K)((const unsigned long long*)p)[i];
    case NXB_S8: return (K)(unsigned)(((const signed char*)p)[i] + 128);
    case NXB_S16: return (K)(unsigned)(((const short*)p)[i] + 32768);
    case NXB_S32: return (K)(((const unsigned int*)p)[i] ^ 0x80000000u);
    case NXB_S64: return (K)(((const unsigned long long*)p)[i] ^ 0x8000000000000000ull);
    case NXB_F16: return (K)half_key(((const unsigned short*)p)[i], false);
    case NXB_BF16: return (K)half_key(((const unsigned short*)p)[i], true);
    case NXB_F32: return (K)f32_key(((const unsigned int*)p)[i]);
    default: return (K)f64_key(((const unsigned long long*)p)[i]);
  }
}

__device__ __forceinline__ void copy_elem(void* dst, long long di, const void* src, long long si, int size) {
  switch (size) {
    case 1: ((unsigned char*)dst)[di] = ((const unsigned char*)src)[si]; break;
    case 2: ((unsigned short*)dst)[di] = ((const unsigned short*)src)[si]; break;
    case 4: ((unsigned int*)dst)[di] = ((const unsigned int*)src)[si]; break;
    default: ((unsigned long long*)dst)[di] = ((const unsigned long long*)src)[si]; break;
  }
}

__device__ __forceinline__ void store_index(void* dst, long long di, int idx, int out_dt) {
  switch (out_dt) {
    case NXB_U8: case NXB_S8: ((unsigned char*)dst)[di] = (unsigned char)idx; break;
    case NXB_U16: case NXB_S16: ((unsigned short*)dst)[di] = (unsigned short)idx; break;
    case NXB_U32: case NXB_S32: ((unsigned int*)dst)[di] = (unsigned int)idx; break;
    case NXB_U64: case NXB_S64: ((unsigned long long*)dst)[di] = (unsigned long long)idx; break;
    case NXB_F32: ((float*)dst)[di] = (float)idx; break;
    default: ((double*)dst)[di] = (double)idx; break;
  }
}

template <typename K>
__global__ void __launch_bounds__(1024) sort_rows_kernel(const void* in, void* out, long long rows, int len, int pow2, int dt, int elem_size,
                                                         int out_dt, int descending, int want_indices) {
  extern __shared__ unsigned char smem[];
  K* keys = reinterpret_cast<K*>(smem);
  int* pos = reinterpret_cast<int*>(smem + (size_t)pow2 * sizeof(K));
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = row * len;
    for (int i = threadIdx.x; i < pow2; i += blockDim.x) {
      K k = ~(K)0;                       // padding sorts behind everything, NaN included (larger position)
      if (i < len) {
        k = load_key<K>(in, dt, base + i);
        if (descending) k = ~k;
      }
      keys[i] = k;
      pos[i] = i < len ? i : 0x7fffffff;
    }
    __syncthreads();
    for (int k = 2; k <= pow2; k <<= 1) {
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int i = threadIdx.x; i < pow2; i += blockDim.x) {
          const int l = i ^ j;
          if (l > i) {
            const K a = keys[i], b = keys[l];
            const int pa = pos[i], pb = pos[l];
            const bool a_after_b = a > b || (a == b && pa > pb);
            const bool up = (i & k) == 0;
            if (a_after_b == up) { keys[i] = b; keys[l] = a; pos[i] = pb; pos[l] = pa; }
          }
        }
        __syncthreads();
      }
    }
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
      if (want_indices) store_index(out, base + i, pos[i], out_dt);
      else copy_elem(out, base + i, in, base + pos[i], elem_size);
    }
    __syncthreads();
  }
}

}  // namespace

bool sort_rows_supported(int64_t len) { return len >= 1 && len <= SORT_MAX_LEN; }

void launch_sort_rows(const void* in, void* out, int64_t rows, int64_t len, DType dt, DType out_dt, bool descending, bool want_indices,
                      int sm_count, cudaStream_t stream) {
  if (rows == 0 || len == 0) return;
  if (!sort_rows_supported(len)) fail(NXB_ERR_UNSUPPORTED, "sort along an axis longer than 16384 elements is not implemented");
  int pow2 = 1;
  while (pow2 < len) pow2 <<= 1;
  const bool wide = dtype_size(dt) == 8;
  const size_t smem = (size_t)pow2 * ((wide ? 8 : 4) + 4);
  const int block = (int)std::min<int64_t>(1024, std::max<int64_t>(32, pow2 / 2));
  const unsigned grid = (unsigned)std::min<int64_t>(rows, (int64_t)sm_count * 8);
  if (wide) {
    NXB_CUDA(cudaFuncSetAttribute(sort_rows_kernel<unsigned long long>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    sort_rows_kernel<unsigned long long><<<grid, block, smem, stream>>>(in, out, rows, (int)len, pow2, (int)dt, (int)dtype_size(dt), (int)out_dt,
                                                                         descending ? 1 : 0, want_indices ? 1 : 0);
  } else {
    NXB_CUDA(cudaFuncSetAttribute(sort_rows_kernel<unsigned int>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    sort_rows_kernel<unsigned int><<<grid, block, smem, stream>>>(in, out, rows, (int)len, pow2, (int)dt, (int)dtype_size(dt), (int)out_dt,
                                                                  descending ? 1 : 0, want_indices ? 1 : 0);
  }
  NXB_CUDA(cudaGetLastError());
}

}  // namespace nxb

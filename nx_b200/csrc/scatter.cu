// Scatter for Nx.indexed_add / Nx.indexed_put (nx/lib/nx.ex:8277,8466; XLA lowers both to
// stablehlo.scatter, exla/lib/exla/defn.ex:1829-1848).
//
// The result starts as a copy of the target (made by the executor); this kernel then applies the
// updates: one thread per element of `updates`.  Row b of `indices` {n, depth} names a position
// along the indexed axes, the matching slice of `updates` lands there, starting at 0 along the
// other axes.  A row with a coordinate outside the target is dropped (scatter semantics).
// indexed_add uses atomic adds, so repeated positions accumulate whatever the thread order
// (integers exactly; floating-point sums up to rounding order); indexed_put stores, and with
// repeated positions one of the written values stays, as the reference documents.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "gemm.h"

namespace nxb {
namespace {

struct ScatterParams {
  void* out;
  const void* indices;
  const void* updates;
  long long total, slice_elems;
  int depth, rank_u, index_bytes, dt, add;
  long long tdim[NXB_MAX_RANK];         // extent of the k-th indexed axis
  long long tstride_idx[NXB_MAX_RANK];  // its stride in the target, elements
  long long udim[NXB_MAX_RANK];         // extents of the update slice (the other axes, in order)
  long long tstride_u[NXB_MAX_RANK];    // strides of those axes in the target
};

// add into an 8- or 16-bit integer through a compare-and-swap on the aligned word that holds it
template <int BYTES>
__device__ __forceinline__ void add_small_int(void* base, long long off, unsigned v) {
  unsigned char* addr = (unsigned char*)base + off * BYTES;
  unsigned* word = (unsigned*)((uintptr_t)addr & ~(uintptr_t)3);
  const unsigned shift = (unsigned)((uintptr_t)addr & 3) * 8u;
  const unsigned mask = (BYTES == 1 ? 0xFFu : 0xFFFFu) << shift;
  unsigned old = *word, seen;
  do {
    seen = old;
    const unsigned sum = (((seen & mask) >> shift) + v) << shift;
    old = atomicCAS(word, seen, (seen & ~mask) | (sum & mask));
  } while (old != seen);
}

__global__ void __launch_bounds__(256) scatter_kernel(ScatterParams p) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < p.total; e += (long long)gridDim.x * blockDim.x) {
    const long long b = e / p.slice_elems;
    long long rem = e - b * p.slice_elems, off = 0;
    for (int j = p.rank_u - 1; j >= 0; --j) {
      const long long c = rem % p.udim[j];
      rem /= p.udim[j];
      off += c * p.tstride_u[j];
    }
    bool inside = true;
    for (int k = 0; k < p.depth; ++k) {
      const long long i = p.index_bytes == 8 ? ((const long long*)p.indices)[b * p.depth + k] : (long long)((const int*)p.indices)[b * p.depth + k];
      inside = inside && i >= 0 && i < p.tdim[k];
      off += i * p.tstride_idx[k];
    }
    if (!inside) continue;
    switch (p.dt) {
      case NXB_F32: { const float v = ((const float*)p.updates)[e]; if (p.add) atomicAdd((float*)p.out + off, v); else ((float*)p.out)[off] = v; break; }
      case NXB_F64: { const double v = ((const double*)p.updates)[e]; if (p.add) atomicAdd((double*)p.out + off, v); else ((double*)p.out)[off] = v; break; }
      case NXB_BF16: { const __nv_bfloat16 v = ((const __nv_bfloat16*)p.updates)[e]; if (p.add) atomicAdd((__nv_bfloat16*)p.out + off, v); else ((__nv_bfloat16*)p.out)[off] = v; break; }
      case NXB_F16: { const __half v = ((const __half*)p.updates)[e]; if (p.add) atomicAdd((__half*)p.out + off, v); else ((__half*)p.out)[off] = v; break; }
      case NXB_S32: case NXB_U32: { const unsigned v = ((const unsigned*)p.updates)[e]; if (p.add) atomicAdd((unsigned*)p.out + off, v); else ((unsigned*)p.out)[off] = v; break; }
      case NXB_S64: case NXB_U64: {
        const unsigned long long v = ((const unsigned long long*)p.updates)[e];
        if (p.add) atomicAdd((unsigned long long*)p.out + off, v); else ((unsigned long long*)p.out)[off] = v;
        break;
      }
      case NXB_S16: case NXB_U16: { const unsigned short v = ((const unsigned short*)p.updates)[e]; if (p.add) add_small_int<2>(p.out, off, v); else ((unsigned short*)p.out)[off] = v; break; }
      default: { const unsigned char v = ((const unsigned char*)p.updates)[e]; if (p.add) add_small_int<1>(p.out, off, v); else ((unsigned char*)p.out)[off] = v; break; }
    }
  }
}

}  // namespace

void launch_scatter(const ScatterSpec& ss, const void* target, const void* indices, const void* updates, void* out, int sm_count, cudaStream_t stream) {
  const size_t bytes = (size_t)shape_numel(ss.target_shape) * dtype_size(ss.dt);
  if (bytes && out != target) NXB_CUDA(cudaMemcpyAsync(out, target, bytes, cudaMemcpyDeviceToDevice, stream));
  ScatterParams p{};
  p.out = out; p.indices = indices; p.updates = updates;
  p.depth = (int)ss.axes.size();
  p.index_bytes = (int)dtype_size(ss.index_dt);
  p.dt = (int)ss.dt;
  p.add = ss.add ? 1 : 0;
  std::vector<long long> stride(ss.target_shape.size(), 1);
  for (int a = (int)ss.target_shape.size() - 2; a >= 0; --a) stride[a] = stride[a + 1] * ss.target_shape[a + 1];
  for (size_t k = 0; k < ss.axes.size(); ++k) { p.tdim[k] = ss.target_shape[ss.axes[k]]; p.tstride_idx[k] = stride[ss.axes[k]]; }
  int j = 0;
  p.slice_elems = 1;
  for (size_t a = 0; a < ss.target_shape.size(); ++a) {
    if (std::find(ss.axes.begin(), ss.axes.end(), (int)a) != ss.axes.end()) continue;
    p.udim[j] = ss.update_shape[1 + j];
    p.tstride_u[j] = stride[a];
    p.slice_elems *= p.udim[j];
    ++j;
  }
  p.rank_u = j;
  p.total = ss.update_shape.empty() ? 0 : ss.update_shape[0] * p.slice_elems;
  if (p.total == 0) return;
  const unsigned grid = (unsigned)std::min<long long>((p.total + 255) / 256, (long long)sm_count * 8);
  scatter_kernel<<<grid, 256, 0, stream>>>(p);
  NXB_CUDA(cudaGetLastError());
}

}  // namespace nxb

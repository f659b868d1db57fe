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
#include "gemm_sm100_device.cuh"

namespace nxb {
namespace {

using namespace nxb_gemm;

// Launched with 192 threads (four epilogue warps) or, when the k loop is short and the epilogue bounds
// the tile time, with 320 (eight epilogue warps in two groups).
template <int KIND, int BN>
__global__ void __launch_bounds__(320, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, TcParams p) {
  tc_gemm_body<KIND, BN, EpiStore>(map_a, map_b, map_c, p);
}

template <int KIND, int BN>
__global__ void __launch_bounds__(320, 1)
tc_gemm_allreduce_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_c, TcParams p, const __grid_constant__ CommArgs cm) {
  tc_gemm_body<KIND, BN, EpiStore, true>(map_a, map_b, map_c, p, &cm);
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

// Operand stored [batch][k][rows] (the free index contiguous).  The tile's rows arrive as groups of 64
// (one 128-byte swizzled line per k), 8 KB per group and k block.  When the row count is a multiple of
// 64 the map is four-dimensional {64 rows, k, group of 64 rows, batch} and ONE copy fetches all the
// groups of a tile (*mode = 2); otherwise one copy per group over a three-dimensional map (*mode = 1).
// (Four copies per k block for a 256-wide tile kept the single producer thread busier than the tensor
// pipe: 8192^3 with B stored [k][n] ran at 1273 TFLOP/s against 1414 with B stored [n][k].)
CUtensorMap make_map_mn(const void* ptr, DType dt, int64_t k, int64_t rows, int64_t batch, int64_t ld, int64_t bs, int box_rows, int* mode) {
  const DriverApi& drv = driver();
  if (!drv.cuTensorMapEncodeTiled) fail(NXB_ERR_RUNTIME, "cuTensorMapEncodeTiled is unavailable");
  CUtensorMap m;
  const size_t es = dtype_size(dt);
  const cuuint64_t batch_stride = batch == 1 ? (cuuint64_t)(ld * es) * (cuuint64_t)k : (cuuint64_t)(std::max<int64_t>(bs, 1) * es);
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (es == 2 && rows % 64 == 0 && box_rows % 64 == 0 && !getenv("NXB200_NO_GROUPED_TMA")) {
    cuuint64_t dims[4] = {64, (cuuint64_t)k, (cuuint64_t)(rows / 64), (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)(ld * es), (cuuint64_t)(64 * es), batch_stride};
    cuuint32_t box[4] = {64, 64, (cuuint32_t)(box_rows / 64), 1};
    CUresult r = drv.cuTensorMapEncodeTiled(&m, tm_type(dt), 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) { *mode = 2; return m; }
  }
  cuuint64_t dims[3] = {(cuuint64_t)rows, (cuuint64_t)k, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)(ld * es), batch_stride};
  cuuint32_t box[3] = {64, 64, 1};
  check_cu(drv.cuTensorMapEncodeTiled(&m, tm_type(dt), 3, const_cast<void*>(ptr), dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
           "cuTensorMapEncodeTiled");
  *mode = 1;
  return m;
}

// Result C [batch][m][n] for the staged store: boxes of 32 x 32 elements, swizzled like the
// staging tiles (64-byte rows for 2-byte elements, 128-byte rows for 4-byte ones).  When C cannot
// be described (rows not 16-byte aligned) a map over a dummy is returned and *ok is false.
CUtensorMap make_map_c(void* ptr, DType dt, int64_t m, int64_t n, int64_t batch, bool* ok) {
  const DriverApi& drv = driver();
  CUtensorMap t;
  memset(&t, 0, sizeof t);
  const size_t es = dtype_size(dt);
  *ok = ptr && (es == 2 || es == 4) && (n * es) % 16 == 0 && ((uintptr_t)ptr) % 16 == 0 && dt != NXB_U16 && dt != NXB_S16;
  if (!*ok) return t;
  CUtensorMapDataType ty = dt == NXB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : dt == NXB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                           : dt == NXB_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_INT32;
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)(n * es), (cuuint64_t)(m * n * es)};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  check_cu(drv.cuTensorMapEncodeTiled(&t, ty, 3, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      es == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
           "cuTensorMapEncodeTiled (result)");
  return t;
}

// The same result for the plain 16-bit epilogue, which hands `groups` neighbouring 32 x 32 staging tiles
// of a warp to the TMA unit in ONE store: a four-dimensional view {32 columns, m, group of 32 columns,
// batch}.  (One store per 32 x 32 tile kept an epilogue warp ~200 cycles per tile in the store's issue;
// with a short k loop the epilogue, not the tensor pipe, sets the tile time.)  Needs n % 32 == 0.
CUtensorMap make_map_c_grouped(void* ptr, DType dt, int64_t m, int64_t n, int64_t batch, int groups, bool* ok) {
  const DriverApi& drv = driver();
  CUtensorMap t;
  memset(&t, 0, sizeof t);
  const size_t es = dtype_size(dt);
  *ok = ptr && es == 2 && n % 32 == 0 && ((uintptr_t)ptr) % 16 == 0 && (dt == NXB_BF16 || dt == NXB_F16) && groups > 1 && !getenv("NXB200_NO_GROUPED_TMA");
  if (!*ok) return t;
  cuuint64_t dims[4] = {32, (cuuint64_t)m, (cuuint64_t)(n / 32), (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)(n * es), (cuuint64_t)(32 * es), (cuuint64_t)(m * n * es)};
  cuuint32_t box[4] = {32, 32, (cuuint32_t)groups, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = drv.cuTensorMapEncodeTiled(&t, dt == NXB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, ptr, dims, strides,
                                          box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  *ok = r == CUDA_SUCCESS;
  return t;
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
  // TMA: 16-byte aligned base, strides multiple of 16 bytes.  16-bit operands may have either
  // index contiguous; 8-bit operands are transposed to K-major by the caller first.
  if ((g.ta || g.tb) && !f16) return false;
  if (((g.ta ? g.m : g.k) * es) % 16 || ((g.tb ? g.n : g.k) * es) % 16) return false;
  if (((g.m * g.k) * es) % 16 || ((g.n * g.k) * es) % 16) return false;
  if (((uintptr_t)g.a) % 16 || ((uintptr_t)g.b) % 16) return false;
  if (g.batch > 65535) return false;
  if (g.m < 1 || g.n < 1 || g.k < 1 || g.batch < 1) return false;
  if (g.k >= (int64_t(1) << 31) || g.m >= (int64_t(1) << 31) || g.n >= (int64_t(1) << 31)) return false;
  return true;
}

int tc_pick_bn(int64_t m, int64_t n, int64_t batch, int sm_count) {
  // the widest tile that still yields at least one tile per SM
  const long long mt = (m + BM - 1) / BM;
  int bn = 256;
  if (mt * ((n + 255) / 256) * batch < sm_count) bn = 128;
  if (bn == 128 && mt * ((n + 127) / 128) * batch < sm_count) bn = 64;
  return bn;
}

int tc_smem_bytes(int bn) { return smem_bytes_for(bn); }
int tc_block_threads(int64_t k) { return k <= 1024 ? 320 : 192; }

static TcParams make_params(const GemmArgs& g, int bn, int* status_word, int a_mode, int b_mode) {
  TcParams p{};
  p.a_mn = g.ta ? a_mode : 0;
  p.b_mn = g.tb ? b_mode : 0;
  p.c = g.c;
  p.bias = g.bias;
  p.scale = (const float*)g.scale;
  p.status = status_word;
  p.m = (int)g.m; p.n = (int)g.n; p.k = (int)g.k; p.batch = (int)g.batch;
  p.mtiles = (int)((g.m + BM - 1) / BM);
  p.ntiles = (int)((g.n + bn - 1) / bn);
  p.out_dt = g.dc;
  p.epilogue = g.epilogue;
  // The wave of sm_count tiles in flight covers panel_m x (sm_count / panel_m) tiles; its operand footprint
  // panel_m * BM + (sm_count / panel_m) * bn rows is smallest near sqrt(sm_count * bn / BM).
  p.panel_m = bn == 256 ? 16 : bn == 128 ? 12 : 8;
  if (const char* e = getenv("NXB200_PANEL_M")) { const int v = atoi(e); if (v >= 1) p.panel_m = v; }
  return p;
}

void tc_prepare_launch(const GemmArgs& g, int bn, void* const* ep, int n_ep, int* status_word, int sm_count, TcLaunch* out,
                       int staged_arg, DType staged_dt) {
  static_assert(sizeof(CUtensorMap) == 128 && sizeof(TcParams) <= sizeof(out->params), "launch block too small");
  int a_mode = 0, b_mode = 0;
  CUtensorMap ma = g.ta ? make_map_mn(g.a, g.da, g.k, g.m, g.batch, g.lda, g.bsa, BM, &a_mode) : make_map(g.a, g.da, g.k, g.m, g.batch, g.lda, g.bsa, BM);
  CUtensorMap mb = g.tb ? make_map_mn(g.b, g.db, g.k, g.n, g.batch, g.ldb, g.bsb, bn, &b_mode) : make_map(g.b, g.db, g.k, g.n, g.batch, g.ldb, g.bsb, bn);
  TcParams p = make_params(g, bn, status_word, a_mode, b_mode);
  if (n_ep > (int)(sizeof(p.ep) / sizeof(p.ep[0]))) fail(NXB_ERR_UNSUPPORTED, "fused epilogue reads too many buffers");
  for (int i = 0; i < n_ep; ++i) p.ep[i] = ep[i];
  bool c_ok = false;
  CUtensorMap mc;
  if (staged_arg >= 0 && staged_arg < n_ep) {
    // the epilogue hands its result back; the kernel converts to `staged_dt` and stores the tile
    mc = make_map_c(ep[staged_arg], staged_dt, g.m, g.n, g.batch, &c_ok);
    p.out_dt = staged_dt;
    p.tma_store = c_ok ? 1 : 0;
  } else {
    mc = make_map_c(nullptr, g.dc, g.m, g.n, g.batch, &c_ok);    // the generated epilogue stores by itself
    p.tma_store = 0;
  }
  memcpy(out->map_a, &ma, 128);
  memcpy(out->map_b, &mb, 128);
  memcpy(out->map_c, &mc, 128);
  memcpy(out->params, &p, sizeof p);
  long long tiles = (long long)p.mtiles * p.ntiles * p.batch;
  out->grid = (unsigned)std::min<long long>(tiles, sm_count);
  out->smem = smem_bytes_for(bn);
}

void launch_tc_gemm(const GemmArgs& g, int* status_word, int sm_count, cudaStream_t stream) {
  const int bn = tc_pick_bn(g.m, g.n, g.batch, sm_count);
  int a_mode = 0, b_mode = 0;
  CUtensorMap ma = g.ta ? make_map_mn(g.a, g.da, g.k, g.m, g.batch, g.lda, g.bsa, BM, &a_mode) : make_map(g.a, g.da, g.k, g.m, g.batch, g.lda, g.bsa, BM);
  CUtensorMap mb = g.tb ? make_map_mn(g.b, g.db, g.k, g.n, g.batch, g.ldb, g.bsb, bn, &b_mode) : make_map(g.b, g.db, g.k, g.n, g.batch, g.ldb, g.bsb, bn);
  TcParams p = make_params(g, bn, status_word, a_mode, b_mode);
  bool c_ok = false;
  CUtensorMap mc = make_map_c(g.c, g.dc, g.m, g.n, g.batch, &c_ok);
  p.tma_store = c_ok ? 1 : 0;
  if (c_ok && !g.scale && (g.da == NXB_BF16 || g.da == NXB_F16) && (g.dc == NXB_BF16 || g.dc == NXB_F16)) {
    // the plain 16-bit epilogue: all staging tiles of a warp leave in one store when they divide its columns
    const int epi_groups = tc_block_threads(g.k) >= 320 ? 2 : 1;
    const int slots = (8192 / epi_groups) / 2048, c_per = (bn / 32) / epi_groups;
    bool g_ok = false;
    if (slots > 1 && c_per % slots == 0) {
      CUtensorMap mg = make_map_c_grouped(g.c, g.dc, g.m, g.n, g.batch, slots, &g_ok);
      if (g_ok) { mc = mg; p.tma_store = 2; }
    }
  }
  long long tiles = (long long)p.mtiles * p.ntiles * p.batch;
  unsigned grid = (unsigned)std::min<long long>(tiles, sm_count);
  auto launch = [&](auto kern, int smem) {
    NXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, tc_block_threads(g.k), smem, stream>>>(ma, mb, mc, p);
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

bool launch_tc_gemm_allreduce(const GemmArgs& g, void* out, int* status_word, int sm_count, cudaStream_t stream) {
  // NXB200_FUSED_ALLREDUCE = never | always | auto (default).  The fused kernel hides the exchange
  // behind the product; NCCL (with in-switch reduction on NVSwitch) moves the bytes faster.  Measured
  // on two B200: fused wins once the product is longer than the exchange, i.e. for a contracted
  // extent per rank of a few thousand; below that, and for wider groups whose exchange dwarfs the
  // product, NCCL after the product is faster.
  const char* mode = getenv("NXB200_FUSED_ALLREDUCE");
  if (getenv("NXB200_NO_FUSED_ALLREDUCE") || (mode && !strcmp(mode, "never"))) return false;
  const bool always = mode && !strcmp(mode, "always");
  if (!always && g.k * comm_world() < 8192LL * (comm_world() - 1)) return false;
  if (!tc_gemm_supported(g) || g.batch != 1 || g.scale || g.bias || g.dc != g.da || (g.da != NXB_BF16 && g.da != NXB_F16) || g.n % 8 != 0) return false;
  const int bn = tc_pick_bn(g.m, g.n, g.batch, sm_count);
  int a_mode = 0, b_mode = 0;
  CUtensorMap ma = g.ta ? make_map_mn(g.a, g.da, g.k, g.m, g.batch, g.lda, g.bsa, BM, &a_mode) : make_map(g.a, g.da, g.k, g.m, g.batch, g.lda, g.bsa, BM);
  CUtensorMap mb = g.tb ? make_map_mn(g.b, g.db, g.k, g.n, g.batch, g.ldb, g.bsb, bn, &b_mode) : make_map(g.b, g.db, g.k, g.n, g.batch, g.ldb, g.bsb, bn);
  TcParams p = make_params(g, bn, status_word, a_mode, b_mode);
  PeerView pv;
  // (comm_peer_view also checks that every rank owns the same number of row tiles)
  if (!comm_peer_view(g.m, g.n, p.mtiles, p.ntiles, &pv)) return false;
  CommArgs cm{};
  cm.rank = pv.rank; cm.world = pv.world; cm.epoch = pv.epoch;
  for (int r = 0; r < pv.world; ++r) {
    char* b = (char*)pv.base[r];
    cm.partial[r] = (const unsigned short*)(b + pv.partial_off);
    cm.result[r] = (unsigned short*)(b + pv.result_off);
    cm.ready[r] = (uint32_t*)(b + pv.ready_off);
    cm.reduced[r] = (uint32_t*)(b + pv.reduced_off);
  }
  cm.out = (unsigned short*)out;
  p.c = (void*)cm.partial[pv.rank];
  p.tma_store = 0;
  CUtensorMap mc;
  memset(&mc, 0, sizeof mc);
  long long tiles = (long long)p.mtiles * p.ntiles;
  unsigned grid = (unsigned)std::min<long long>(tiles, sm_count);
  auto launch = [&](auto kern, int smem) {
    NXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, 320, smem, stream>>>(ma, mb, mc, p, cm);
    NXB_CUDA(cudaGetLastError());
  };
#define NXB_LAUNCH_AR(K)                                                                 \
  do {                                                                                   \
    if (bn == 256) launch(tc_gemm_allreduce_kernel<K, 256>, smem_bytes_for(256));        \
    else if (bn == 128) launch(tc_gemm_allreduce_kernel<K, 128>, smem_bytes_for(128));   \
    else launch(tc_gemm_allreduce_kernel<K, 64>, smem_bytes_for(64));                    \
  } while (0)
  if (g.da == NXB_BF16) NXB_LAUNCH_AR(KIND_BF16);
  else NXB_LAUNCH_AR(KIND_F16);
#undef NXB_LAUNCH_AR
  return true;
}

const char* attention_device_source() {
  static const char* src =
#include "attn_device_embed.inc"
      ;
  return src;
}

// host mirror of nxb_attn::AttnParams (attn_sm100_device.cuh); the layouts must match
struct AttnParamsHost {
  void* out;
  long long out_bh_hi, out_bh_lo, out_row;
  int* status;
  int heads, batch_heads, sq, sk;
  int causal;
  void* ep[14];
};

int attn_smem_bytes() { return 128 * 128 * 2 * 6 + 1024 + 256; }      // Q x 2, K x 2, V x 2 (attn_sm100_device.cuh)

// V as (head dim, key, head, batch) with the strides of either layout: boxes of 64 dims x 128 keys
static CUtensorMap make_map_v4(const void* ptr, int64_t sk, int64_t heads, int64_t batch, bool bshd) {
  const DriverApi& drv = driver();
  if (!drv.cuTensorMapEncodeTiled) fail(NXB_ERR_RUNTIME, "cuTensorMapEncodeTiled is unavailable");
  CUtensorMap m;
  const cuuint64_t row = 128 * 2;
  cuuint64_t dims[4] = {128, (cuuint64_t)sk, (cuuint64_t)heads, (cuuint64_t)batch};
  // {batch, head, key, dim}: key rows are adjacent; {batch, key, head, dim}: the heads of one key are adjacent
  cuuint64_t strides[3] = {bshd ? row * (cuuint64_t)heads : row, bshd ? row : row * (cuuint64_t)sk, row * (cuuint64_t)sk * (cuuint64_t)heads};
  cuuint32_t box[4] = {64, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  check_cu(drv.cuTensorMapEncodeTiled(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
           "cuTensorMapEncodeTiled (values)");
  return m;
}

void attn_prepare_launch(const void* q, const void* k, const void* v, void* out, int64_t batch_heads, int64_t sq, int64_t sk, int causal,
                         void* const* ep, int n_ep, int* status_word, TcLaunch* outl, int64_t heads, bool v_bshd, bool out_bshd) {
  static_assert(sizeof(AttnParamsHost) <= sizeof(outl->params), "launch block too small");
  if (heads < 1 || batch_heads % heads != 0) fail(NXB_ERR_RUNTIME, "internal: attention head count does not divide batch * heads");
  const int64_t batch = batch_heads / heads;
  CUtensorMap mq = make_map(q, NXB_BF16, 128, sq, batch_heads, 128, sq * 128, 128);
  CUtensorMap mk = make_map(k, NXB_BF16, 128, sk, batch_heads, 128, sk * 128, 128);
  CUtensorMap mv = make_map_v4(v, sk, heads, batch, v_bshd);
  AttnParamsHost p{};
  p.out = out;
  p.heads = (int)heads;
  // address of output row (b, h, i) in elements: b * hi + h * lo + i * out_row
  if (out_bshd) { p.out_bh_hi = sq * heads * 128; p.out_bh_lo = 128; p.out_row = heads * 128; }
  else { p.out_bh_hi = heads * sq * 128; p.out_bh_lo = sq * 128; p.out_row = 128; }
  p.status = status_word;
  p.batch_heads = (int)batch_heads;
  p.sq = (int)sq;
  p.sk = (int)sk;
  p.causal = causal;
  if (n_ep > 14) fail(NXB_ERR_UNSUPPORTED, "attention score transform reads too many buffers");
  for (int i = 0; i < n_ep; ++i) p.ep[i] = ep[i];
  memcpy(outl->map_a, &mq, 128);
  memcpy(outl->map_b, &mk, 128);
  memcpy(outl->map_c, &mv, 128);
  memcpy(outl->params, &p, sizeof p);
  outl->grid = (unsigned)(batch_heads * (((sq + 127) / 128 + 1) / 2));      // two blocks of 128 query rows per CTA
  outl->smem = attn_smem_bytes();
}

// One thread waits, with the bounded wait the fused kernels use on their peers' flags, for a flag
// that nothing sets; when the limit passes the wait returns false and the kernel reports it the way
// every kernel does: through the device's status word.
__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t epoch, long long limit_cycles, int* status) {
  __shared__ int abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  if (threadIdx.x == 0 && !nxb_gemm::flag_wait(flag, epoch, &abort_word, limit_cycles)) *(volatile int*)status = 1;
}

void launch_wait_probe(const uint32_t* flag, long long limit_cycles, int* status_word, cudaStream_t stream) {
  wait_probe_kernel<<<1, 32, 0, stream>>>(flag, 1u, limit_cycles, status_word);
  NXB_CUDA(cudaGetLastError());
}

const char* gemm_device_source() {
  static const char* src =
#include "gemm_device_embed.inc"
      ;
  return src;
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
    // every check comes before the first enqueue: a rejected call leaves the shared scratch untouched
    if (((uintptr_t)a) % 16 || ((uintptr_t)b) % 16 || ((uintptr_t)c) % 16)
      fail(NXB_ERR_INVALID_ARGUMENT, "a, b and c must be 16-byte aligned device pointers");
    if (m >= (int64_t(1) << 31) || n >= (int64_t(1) << 31) || k >= (int64_t(1) << 31))
      fail(NXB_ERR_INVALID_ARGUMENT, "m, n and k must be below 2^31");
    // the caller's current device is put back on every way out
    struct DeviceGuard {
      int prev = -1;
      ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
    } guard;
    {
      int cur = -1;
      NXB_CUDA(cudaGetDevice(&cur));
      NXB_CUDA(cudaSetDevice(device));
      if (cur != device) guard.prev = cur;
    }
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
    GemmArgs g{};
    g.a = a; g.b = dev.scratch; g.c = c;
    g.batch = 1; g.m = m; g.n = n; g.k = k;
    g.lda = k; g.ldb = k; g.bsa = m * k; g.bsb = n * k;
    g.ta = g.tb = false;
    g.da = g.db = g.dc = NXB_BF16;
    if (!tc_gemm_supported(g)) fail(NXB_ERR_INVALID_ARGUMENT, "operands must be 16-byte aligned");
    // the status word must start at zero; the scratch is fully rewritten before it is read
    NXB_CUDA(cudaMemsetAsync(dev.status, 0, sizeof(int), stream));
    launch_transpose(b, dev.scratch, 1, k, n, 2, stream);          // B {k,n} -> {n,k}
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

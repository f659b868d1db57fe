// Matrix-product launchers shared by the planner and the executor.
#pragma once
#include "program.h"

namespace nxb {

// C[b][m][n] = sum_k A[b][m][k] * B[b][k][n], C row-major [batch][m][n].
// An operand with trans == false has the reduction index k contiguous
// (A stored [m][k], B stored [n][k]); with trans == true the other index is
// contiguous (A stored [k][m], B stored [k][n]).  `ld` is the stride of the
// non-contiguous index, `batch_stride` the distance between matrices.
struct GemmArgs {
  const void* a; const void* b; void* c;
  const void* bias;     // optional, per output column n, in the output type
  const void* scale;    // optional, f32 per output column n
  int64_t batch, m, n, k;
  int64_t lda, ldb, bsa, bsb;
  bool ta, tb;
  DType da, db, dc;
  int epilogue;
};

enum GemmEpilogue { EPI_NONE = 0 };

// Generic CUDA-core product for every type combination (exact for integers).
void launch_simt_gemm(const GemmArgs& g, cudaStream_t stream);

// Tensor-core product (tcgen05 + TMA).  Needs both operands K-major (ta == tb == false).
bool tc_gemm_supported(const GemmArgs& g);
void launch_tc_gemm(const GemmArgs& g, int* status_word, int sm_count, cudaStream_t stream);
// Everything a generated tensor-core kernel needs at launch: the two tensor maps and the
// parameter block, laid out as the device code expects.
struct TcLaunch {
  alignas(64) unsigned char map_a[128];
  alignas(64) unsigned char map_b[128];
  alignas(64) unsigned char map_c[128];
  alignas(16) unsigned char params[256];
  unsigned grid = 1;
  int smem = 0;
};
int tc_pick_bn(int64_t m, int64_t n, int64_t batch, int sm_count);
int tc_smem_bytes(int bn);
// Threads per block of the tensor-core product: 192, or 320 (eight epilogue warps) when the contracted
// extent is short enough that writing the tile out takes longer than computing it.
int tc_block_threads(int64_t k);
// `staged_arg` >= 0: ep[staged_arg] is the one result (of type `staged_dt`) that the kernel stores itself through
// shared memory and TMA; the tensor map of the result is then built over that buffer.
void tc_prepare_launch(const GemmArgs& g, int bn, void* const* ep, int n_ep, int* status_word, int sm_count, TcLaunch* out,
                       int staged_arg = -1, DType staged_dt = NXB_F32);
const char* gemm_device_source();
const char* attention_device_source();
int attn_smem_bytes();
// Launch block of a generated attention kernel: tensor maps of q, k ([batch*heads][S][128] bf16) and v,
// and its parameter block.  `heads` splits batch_heads into (batch, head); `v_bshd`: v is stored
// {batch, key, head, 128} (a projection's own layout) instead of {batch, head, key, 128}; `out_bshd`: the
// result is written as {batch, row, head, 128}, which is what the projection after it reads.
void attn_prepare_launch(const void* q, const void* k, const void* v, void* out, int64_t batch_heads, int64_t sq, int64_t sk, int causal,
                         void* const* ep, int n_ep, int* status_word, TcLaunch* outl, int64_t heads = 1, bool v_bshd = false,
                         bool out_bshd = false);
// Peer memory of the tensor-parallel group (comm.cpp): one region per rank, mapped into every
// process, holding [partial product][reduced tiles][ready flags][reduced flags].
struct PeerView {
  int rank = 0, world = 1;
  uint32_t epoch = 0;              // launch number, the same on every rank
  void* base[8] = {};              // region of each rank ([rank] is the local one)
  size_t partial_off = 0, result_off = 0, ready_off = 0, reduced_off = 0;
  size_t elems = 0, flag_words = 0;
};
// Fills `v` and advances the epoch when peer memory is set up, a matrix of m x n 16-bit elements
// with mtiles x ntiles output tiles fits and the ranks can share the row tiles evenly; false
// otherwise (the caller uses NCCL instead).
int comm_world();
bool comm_peer_view(int64_t m, int64_t n, int64_t mtiles, int64_t ntiles, PeerView* v);
// Product of a row-parallel linear fused with the sum over ranks (one kernel over peer memory).
// Returns false, launching nothing, when the shape or the communicator does not allow it.
bool launch_tc_gemm_allreduce(const GemmArgs& g, void* out, int* status_word, int sm_count, cudaStream_t stream);
// Weight-only quantised linear with the s8 -> bf16 conversion inside the kernel (x bf16 {m,k},
// W s8 {n,k}, f32 scale per n): for batches of at most WQ_LINEAR_MAX_ROWS rows, where the layer
// is a single stream over W.
constexpr int64_t WQ_LINEAR_MAX_ROWS = 512;
bool wq_linear_supported(const GemmArgs& g);
void launch_wq_linear(const GemmArgs& g, int* status_word, int sm_count, cudaStream_t stream);
// Sort / argsort of `rows` rows of `len` elements each (the last axis), see sort_rows.cu.
bool sort_rows_supported(int64_t len);
void launch_sort_rows(const void* in, void* out, int64_t rows, int64_t len, DType dt, DType out_dt, bool descending, bool want_indices,
                      int sm_count, cudaStream_t stream);
// indexed_add / indexed_put (scatter.cu): copies the target into `out` (unless they are the same memory)
// and applies the updates.
void launch_scatter(const ScatterSpec& ss, const void* target, const void* indices, const void* updates, void* out, int sm_count,
                    cudaStream_t stream);
// Self-test of the bounded wait: see nxb200_selftest_bounded_wait.
void launch_wait_probe(const uint32_t* flag, long long limit_cycles, int* status_word, cudaStream_t stream);
void launch_transpose(const void* in, void* out, int64_t batch, int64_t rows, int64_t cols, size_t elem_size, cudaStream_t stream);

}  // namespace nxb

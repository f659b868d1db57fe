/*
 * nxb200 — C ABI of the B200 runtime behind an Nx backend and defn compiler.
 *
 * This is the native boundary an Erlang NIF shim (or any FFI: ctypes, cgo …)
 * binds.  It replaces, for one device type, what the reference reaches through
 * EXLA.NIF (exla/lib/exla/nif.ex:23-106, exla/c_src/exla/exla.cc).  Every entry
 * point:
 *   - is extern "C", takes plain pointers/sizes, and never throws;
 *   - returns 0 on success or a negative nxb200_status; the text of the last
 *     failure on the calling thread is read with nxb200_last_error();
 *   - may be called from any host thread (the reference calls its NIFs from
 *     arbitrary dirty-scheduler threads).  Work for one device is serialised
 *     on that device's stream, which matches the reference's one-run-at-a-time
 *     lock per {client, device} (exla/lib/exla/defn.ex:165-168).
 *
 * Tensors are dense, row-major, native-endian, with no strides in the API
 * (nx/lib/nx.ex:2070-2077).
 */
#ifndef NXB200_H
#define NXB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types: the {kind, bits} pairs of nx/lib/nx/type.ex:27-48 that the
 * hot path uses (EXLA's typespec codec: exla/c_src/exla/exla_nif_util.h:82-153). */
typedef enum {
  NXB_U8 = 0, NXB_U16 = 1, NXB_U32 = 2, NXB_U64 = 3,
  NXB_S8 = 4, NXB_S16 = 5, NXB_S32 = 6, NXB_S64 = 7,
  NXB_F16 = 8, NXB_BF16 = 9, NXB_F32 = 10, NXB_F64 = 11
} nxb200_dtype;

typedef enum {
  NXB_OK = 0,
  NXB_ERR_INVALID_ARGUMENT = -1,   /* -> ArgumentError                           */
  NXB_ERR_RUNTIME = -2,            /* -> RuntimeError (CUDA / NVRTC / NCCL text) */
  NXB_ERR_ALREADY_DEALLOCATED = -3,/* -> {:error, :already_deallocated}          */
  NXB_ERR_OUT_OF_MEMORY = -4,
  NXB_ERR_UNSUPPORTED = -5,        /* op outside the implemented subset          */
  NXB_ERR_NO_DEVICE = -6,
  NXB_ERR_TIMEOUT = -7             /* a bounded device-side wait gave up         */
} nxb200_status;

#define NXB_MAX_RANK 8

typedef struct nxb200_buffer nxb200_buffer;     /* device tensor (NIF resource) */
typedef struct nxb200_program nxb200_program;   /* compiled defn (NIF resource) */

/* Copies the calling thread's last error text (NUL terminated) into dst.
 * Replaces the status->exception text path of exla/c_src/exla/exla.cc:280-292. */
size_t nxb200_last_error(char *dst, size_t cap);

/* ---- client / devices -------------------------------------------------------
 * exla.cc:534-540 (get_gpu_client) and :576-580 (get_device_count).  Safe to
 * call on a machine without a GPU: the count is then 0 and init still
 * succeeds, so programs can be built (compiled) but not run. */
int nxb200_init(void);
int nxb200_device_count(int *count);

/* ---- buffers ----------------------------------------------------------------
 * binary_to_device_mem (exla.cc:439-445; exla_client.cc:118-151): copies
 * `nbytes` of host data into a new device tensor.  The call returns once the
 * host memory may be reused. */
int nxb200_buffer_from_host(int device, nxb200_dtype dtype, const int64_t *dims, int rank,
                            const void *src, size_t nbytes, nxb200_buffer **out);
/* The same without waiting: the call returns as soon as the upload is queued.  A thread of the library
 * copies the source through pinned staging buffers (the caller's memory need not be pinned: an Erlang
 * binary is not) and calls `on_done(ctx)`, from that thread, once the last byte of `src` has been read;
 * until then `src` must stay alive and unchanged.  This is the reference's zero-copy upload with its
 * completion callback (exla/c_src/exla/exla_client.cc:118-151: the binary is held in a private
 * environment until the transfer is done).  The tensor may be used at once: its first use waits until
 * the copies are queued and orders the device's work after them.  `on_done` may be NULL. */
typedef void (*nxb200_upload_done)(void *ctx);
int nxb200_buffer_from_host_async(int device, nxb200_dtype dtype, const int64_t *dims, int rank,
                                  const void *src, size_t nbytes, nxb200_upload_done on_done,
                                  void *ctx, nxb200_buffer **out);
/* Uninitialised device tensor (used for outputs and by benchmarks). */
int nxb200_buffer_alloc(int device, nxb200_dtype dtype, const int64_t *dims, int rank,
                        nxb200_buffer **out);
/* read_device_mem (exla.cc:447-453; exla_client.cc:58-72): waits for pending
 * work on the buffer's device, then copies the first `nbytes` bytes to dst. */
int nxb200_buffer_to_host(nxb200_buffer *buf, void *dst, size_t nbytes);
/* Asynchronous variants for callers that own pinned memory and want to overlap
 * transfers with compute; complete at the next nxb200_device_synchronize. */
int nxb200_buffer_write_async(nxb200_buffer *buf, const void *pinned_src, size_t nbytes);
int nxb200_buffer_read_async(nxb200_buffer *buf, void *pinned_dst, size_t nbytes);
/* copy_buffer_to_device (exla.cc:513-524; exla_client.cc:97-108). */
int nxb200_buffer_copy_to_device(nxb200_buffer *buf, int device, nxb200_buffer **out);
/* get_buffer_typespec (exla.cc:455-460). dims must hold NXB_MAX_RANK entries. */
int nxb200_buffer_info(nxb200_buffer *buf, nxb200_dtype *dtype, int64_t *dims, int *rank,
                       int *device);
/* Raw device address, for interop and benchmarks (get_buffer_device_pointer,
 * exla.cc:325-389, :local mode only). */
int nxb200_buffer_device_pointer(nxb200_buffer *buf, void **ptr);
/* Nx.from_pointer / Nx.to_pointer (exla/lib/exla/backend.ex:86-181; create_buffer_from_device_pointer
 * and get_buffer_device_pointer, exla.cc:325-437).  from_pointer wraps device memory the caller owns
 * (never freed by the library).  ipc_export gives the CUDA IPC handle of a tensor this library
 * allocated; from_ipc, in ANOTHER process, maps it (unmapped again by deallocate / release). */
#define NXB_IPC_HANDLE_BYTES 64
int nxb200_buffer_from_pointer(int device, nxb200_dtype dtype, const int64_t *dims, int rank,
                               void *device_ptr, nxb200_buffer **out);
int nxb200_buffer_ipc_export(nxb200_buffer *buf, uint8_t handle[NXB_IPC_HANDLE_BYTES]);
int nxb200_buffer_from_ipc(int device, nxb200_dtype dtype, const int64_t *dims, int rank,
                           const uint8_t handle[NXB_IPC_HANDLE_BYTES], nxb200_buffer **out);
/* deallocate_device_mem (exla.cc:462-475): frees the device memory now; a
 * second call returns NXB_ERR_ALREADY_DEALLOCATED; any later use of the
 * handle fails with NXB_ERR_RUNTIME.  The handle itself stays valid until
 * nxb200_buffer_release. */
int nxb200_buffer_deallocate(nxb200_buffer *buf);
/* is_device_buffer_deleted (exla.cc:477-482). */
int nxb200_buffer_is_deallocated(nxb200_buffer *buf, int *flag);
/* Resource destructor (exla_client.cc:22-26): drops the handle. */
int nxb200_buffer_release(nxb200_buffer *buf);

/* ---- programs ---------------------------------------------------------------
 * One call replaces the thirteen MLIR-builder NIFs plus mlir_compile
 * (exla.cc:64-323): `bytes` is a serialised Nx.Defn.Expr graph.
 *
 *   "NXB1"  u32 n_nodes
 *   node := u8 oplen, op[oplen] (the Expr op atom as text, nx/lib/nx/defn/expr.ex:17-51)
 *           u8 dtype, u8 rank, i64 dims[rank]            (the node's result)
 *           u16 nargs,  u32 arg[nargs]                   (indices of earlier nodes)
 *           u16 nints,  i64 ints[nints]                  (op attributes, below)
 *           u16 nflts,  f64 flts[nflts]
 *           u64 bloblen, blob[bloblen]                   (literal data of a :tensor node)
 *   u32 n_outputs, u32 output[n_outputs]
 *   optional: u32 n_donated, (u32 parameter, u32 output)[n_donated]   buffer donation
 *             (Nx.donatable, exla/lib/exla/defn.ex:598-645): nxb200_program_run hands the
 *             argument's memory to that result (or releases it) and the argument handle
 *             becomes deallocated; nxb200_program_run_into consumes nothing
 *
 * Attributes: parameter [index]; constant ints=[v] (integer types) or
 * flts=[v]; iota [axis|-1]; sum/product/reduce_max/reduce_min/all/any
 * [keep_axes, n, axes…]; argmax/argmin [tie_break_high, axis|-1, keep_axis];
 * dot [nc1,c1…, nb1,b1…, nc2,c2…, nb2,b2…]; squeeze [n, axes…]; broadcast
 * [n, axes…]; transpose [perm…]; slice [starts…, lengths…, strides…] (with
 * dynamic starts the node has 1 + rank arguments: the tensor, then one scalar
 * integer start per axis, and the starts attribute is ignored); gather [axes…]
 * (arguments: tensor, indices); indexed_add / indexed_put [axes…] (arguments: tensor and
 * updates already of the result's type, indices s32 or s64 {n, axes}); put_slice none (arguments: tensor, slice, one
 * scalar integer start per axis); pad [lows…, highs…, interiors…] (arguments:
 * tensor, scalar pad value); reverse [axes…]; window_sum/max/min/product
 * [window…, strides…, low padding…, high padding…, dilations…]; sort
 * [descending] and argsort [descending, stable], both along the last axis;
 * concatenate [axis]; everything else none.
 *
 * Building needs no GPU (kernels are generated and compiled for sm_100a on
 * the host); the first run on a device loads them. */
int nxb200_program_build(const uint8_t *bytes, size_t nbytes, nxb200_program **out);
int nxb200_program_io(nxb200_program *prog, int *n_params, int *n_outputs);
/* Result typespec of output i (what executable.ex:150-161 reads back). */
int nxb200_program_output_info(nxb200_program *prog, int i, nxb200_dtype *dtype,
                               int64_t *dims, int *rank);
/* run_io (exla.cc:626-634; exla_client.cc:258-398).  `args[i]` binds parameter
 * i; all must live on `device`.  New output buffers are returned in outs[].
 * The call enqueues the work and returns; reading an output (or
 * nxb200_device_synchronize) waits for it. */
int nxb200_program_run(nxb200_program *prog, int device, nxb200_buffer *const *args, int n_args,
                       nxb200_buffer **outs, int n_outs);
/* Same, writing into caller-provided output buffers (steady-state loops that
 * must not allocate; shapes and types must match program_output_info). */
int nxb200_program_run_into(nxb200_program *prog, int device, nxb200_buffer *const *args,
                            int n_args, nxb200_buffer *const *outs, int n_outs);
int nxb200_program_release(nxb200_program *prog);
/* Human-readable plan: one line per launched kernel with its name, grid and
 * the graph nodes fused into it.  Returns the number of bytes needed. */
size_t nxb200_program_describe(nxb200_program *prog, char *dst, size_t cap);
/* Generated CUDA source of the i-th fused kernel (diagnostics; 0 when i is out
 * of range).  Returns the number of bytes needed. */
size_t nxb200_program_kernel_source(nxb200_program *prog, int i, char *dst, size_t cap);
/* Where the build time went, in seconds: planning (parse, fusion, code generation) and
 * compilation of the generated sources (NVRTC).  The reference reports the same split in its
 * [:exla, :compilation] telemetry event (eval_time / compile_time / total_time,
 * exla/lib/exla/defn.ex:515-523). */
int nxb200_program_build_times(nxb200_program *prog, double *plan_seconds, double *codegen_seconds);
/* Number of kernels one run launches. */
int nxb200_program_launch_count(nxb200_program *prog, int *count);

/* Matrix product that allocates nothing: c {m,n} = a {m,k} . b {k,n}, bf16 operands
 * and result, f32 accumulation, all three given as raw device pointers on `device`.
 * No counterpart in the reference, whose runtime always allocates through its client.
 * It exists for callers that must not trigger a cudaMalloc inside this library: a
 * process that has handed the device's memory to another allocator up front (an XLA
 * client with preallocation, say) and would see the allocation fail, or a serving
 * loop that cannot take the device-wide stall an allocation causes.  The scratch the
 * product needs (a copy of b with k contiguous) is a fixed 32 MiB array inside the
 * library, so k*n may be at most 16,777,216 elements; larger operands, k or n not a
 * multiple of 8, or pointers that are not 16-byte aligned are rejected with
 * NXB_ERR_INVALID_ARGUMENT.  Every GPU that loads the library holds those 32 MiB
 * until the process exits.
 *
 * The first call on a device looks up the array's device address; that first call
 * should come before any stream capture.  Every call enqueues on `stream` (a
 * cudaStream_t, or NULL for the default stream), reads a status word back and waits
 * for `stream` to drain before it returns, so the result is complete on return.
 * All arguments are checked before anything is enqueued: a rejected call leaves the
 * scratch and the stream untouched.  The caller's current device is restored.
 * All calls share the one array: calls that overlap on the same GPU (different
 * streams or threads) race on it. */
int nxb200_dot_bf16_static_scratch(int device, const void *a, const void *b, void *c,
                                   int64_t m, int64_t n, int64_t k, void *stream);

/* ---- device control ---------------------------------------------------------*/
int nxb200_device_synchronize(int device);
/* Device-side timing of everything enqueued between the two calls on the
 * device's stream (CUDA events).  end returns elapsed milliseconds. */
int nxb200_timer_begin(int device);
int nxb200_timer_end(int device, float *ms);
/* Self-test of the failure path every kernel shares: one thread waits, with the same bounded
 * wait the fused kernels use on flags their peers set, for a flag that nothing sets.  After
 * `limit_us` microseconds the wait gives up, the kernel returns normally and reports through the
 * device's status word; the call then answers NXB_ERR_TIMEOUT (anything else means the failure path
 * is broken).  The device stays usable.  No counterpart in the reference. */
int nxb200_selftest_bounded_wait(int device, uint32_t limit_us);
/* The device's compute stream as a cudaStream_t, for callers that interleave
 * their own work (e.g. an L2 flush in a benchmark). */
int nxb200_device_stream(int device, void **stream);

/* get_allocated_memory / get_peak_memory / reset_peak_memory /
 * get_per_device_memory (exla.cc:655-686; exla_client.cc:597-630). */
int nxb200_memory_stats(int device, uint64_t *allocated, uint64_t *peak, uint64_t *reserved);
int nxb200_memory_reset_peak(int device);

/* ---- sharded execution (Nx.Mesh, exla/lib/exla/defn.ex:40-72) -------------------
 * One process per GPU.  Rank 0 creates an id, the host distributes its
 * NXB_COMM_ID_BYTES bytes to the other ranks by its own means, then every rank
 * calls comm_init.  all_reduce sums `buf` in place across ranks on the
 * device's stream (the collective a row-parallel linear needs). */
#define NXB_COMM_ID_BYTES 128
int nxb200_comm_id(uint8_t id[NXB_COMM_ID_BYTES]);
int nxb200_comm_init(int device, int rank, int world, const uint8_t id[NXB_COMM_ID_BYTES]);
int nxb200_comm_all_reduce_sum(nxb200_buffer *buf);
/* Peer memory for the product fused with the sum over ranks (XLA would emit the all-reduce
 * as its own NCCL call after the dot, exla/lib/exla/defn.ex:40-72; here one kernel does both
 * when this is set up).  peer_alloc reserves this rank's region for matrices of up to `elems`
 * 16-bit elements and returns a blob (CUDA IPC handle + device UUID); the host gathers the
 * blobs of all ranks in rank order and passes them to peer_open, which sets *enabled to 0 and
 * keeps the group on NCCL when two ranks share a GPU or a region cannot be mapped. */
#define NXB_COMM_PEER_BLOB_BYTES 80
int nxb200_comm_peer_alloc(int device, uint64_t elems, uint8_t blob[NXB_COMM_PEER_BLOB_BYTES]);
int nxb200_comm_peer_open(const uint8_t *blobs, int *enabled);
/* Number of products this process has run fused with their all-reduce (diagnostics). */
int nxb200_comm_fused_launches(uint64_t *count);
int nxb200_comm_destroy(void);

#ifdef __cplusplus
}
#endif
#endif /* NXB200_H */

// Shared declarations of the nxb200 runtime: status/error plumbing, element
// types, the plan a program compiles to, and the per-device runtime objects.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/nxb200.h"

struct nxb200_buffer;

namespace nxb {

struct Error : std::exception {
  int status;
  std::string msg;
  Error(int s, std::string m) : status(s), msg(std::move(m)) {}
  const char* what() const noexcept override { return msg.c_str(); }
};

void set_last_error(const std::string& msg);

[[noreturn]] inline void fail(int status, const std::string& msg) { throw Error(status, msg); }

#define NXB_CUDA(expr)                                                                         \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      ::nxb::fail(_e == cudaErrorMemoryAllocation ? NXB_ERR_OUT_OF_MEMORY : NXB_ERR_RUNTIME,   \
                  std::string(#expr) + ": " + cudaGetErrorString(_e));                         \
  } while (0)

// ---- element types ---------------------------------------------------------------
typedef nxb200_dtype DType;

inline size_t dtype_size(DType t) {
  switch (t) {
    case NXB_U8: case NXB_S8: return 1;
    case NXB_U16: case NXB_S16: case NXB_F16: case NXB_BF16: return 2;
    case NXB_U32: case NXB_S32: case NXB_F32: return 4;
    default: return 8;
  }
}
inline bool dtype_is_float(DType t) { return t >= NXB_F16; }
inline bool dtype_is_signed(DType t) { return t >= NXB_S8; }
inline bool dtype_is_int(DType t) { return t < NXB_F16; }
const char* dtype_name(DType t);
DType dtype_merge(DType a, DType b);   // nx/lib/nx/type.ex:463-473

inline int64_t shape_numel(const std::vector<int64_t>& s) {
  int64_t n = 1;
  for (auto d : s) n *= d;
  return n;
}
std::string shape_str(const std::vector<int64_t>& s);

// ---- driver entry points (resolved through the runtime; no link-time libcuda) ----
struct DriverApi {
  CUresult (*cuModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*cuModuleUnload)(CUmodule) = nullptr;
  CUresult (*cuModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*cuLaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                             unsigned, CUstream, void**, void**) = nullptr;
  CUresult (*cuFuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*cuGetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                     const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                     const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
  CUresult (*cuMemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr) = nullptr;
};
const DriverApi& driver();
void check_cu(CUresult r, const char* what);

// ---- device runtime -------------------------------------------------------------------
// Caching allocator: freed blocks are kept per size class and reused on the same
// stream, so steady-state runs make no cudaMalloc/cudaFree calls.  Counters mirror
// exla/c_src/exla/exla_client.cc:597-630.
class Allocator {
 public:
  void* alloc(size_t nbytes);
  void free(void* p);
  void release_cached();
  // `allocated` / `peak` count the bytes callers asked for (what the reference's counters report,
  // exla/test/exla/memory_tracking_test.exs); `reserved` counts what was taken from the device
  uint64_t allocated = 0, peak = 0, reserved = 0;

 private:
  static size_t round_size(size_t n);
  std::multimap<size_t, void*> cache_;
  std::map<void*, std::pair<size_t, size_t>> live_;   // block -> (size class, bytes asked for)
};

struct Device {
  int id = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  // Asynchronous transfers run on streams of their own, so that an upload can overlap a
  // download (the link is full duplex) and both can overlap kernels.  Ordering against the
  // compute stream is by events; `pending_reads` are device addresses a download may still read.
  cudaStream_t h2d = nullptr, d2h = nullptr;
  cudaEvent_t ev_compute = nullptr, ev_h2d = nullptr, ev_d2h = nullptr;
  std::vector<const void*> pending_reads;
  Allocator alloc;
  std::mutex mu;             // serialises enqueue + allocator state for this device
  int sm_count = 148;
  // Word in mapped host memory that a kernel sets when one of its bounded waits gives up.
  volatile int* status_host = nullptr;
  int* status_dev = nullptr;
};
void check_device_status(Device& d);   // throws NXB_ERR_TIMEOUT if a kernel reported a stalled wait

int device_count();
Device& device(int id);       // makes the device current on the calling thread

// Asynchronous upload from pageable host memory through a pinned staging ring (uploader.cpp).
typedef void (*UploadDone)(void* ctx);
void upload_enqueue(Device& d, nxb200_buffer* b, const void* src, size_t nbytes, UploadDone on_done, void* ctx);
void upload_join(nxb200_buffer* b);     // no-op unless an upload is pending; afterwards the compute stream is ordered after it

}  // namespace nxb

// Handle types behind the opaque pointers of the C ABI.
struct nxb200_buffer {
  uint32_t magic = 0x4e584242;          // "NXBB"
  int device = 0;
  nxb::DType dtype = NXB_F32;
  std::vector<int64_t> dims;
  void* ptr = nullptr;
  size_t nbytes = 0;
  std::atomic<bool> deallocated{false};
  // Memory the library does not own: a pointer the caller lent (from_pointer), or another
  // process's allocation mapped through CUDA IPC (`ipc_base` is then what has to be unmapped).
  bool borrowed = false;
  void* ipc_base = nullptr;
  // An upload in progress (nxb200_buffer_from_host_async): the copies are enqueued by the device's
  // uploader thread; `ready` is recorded after the last one.  The first use of the buffer waits (on the
  // host) until they are enqueued and makes the compute stream wait for `ready`.
  struct Upload;
  std::shared_ptr<Upload> upload;
};

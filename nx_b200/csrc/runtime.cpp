// Device runtime: device table, streams, caching allocator, driver entry points.
// The counterpart of ExlaClient / ExlaBuffer in exla/c_src/exla/exla_client.cc.
#include "common.h"

#include <deque>
#include <sstream>

namespace nxb {

static thread_local std::string g_last_error;
void set_last_error(const std::string& msg) { g_last_error = msg; }
const std::string& last_error() { return g_last_error; }

const char* dtype_name(DType t) {
  static const char* n[] = {"u8", "u16", "u32", "u64", "s8", "s16", "s32", "s64", "f16", "bf16", "f32", "f64"};
  return n[(int)t];
}

DType dtype_merge(DType a, DType b) {
  if (a == b) return a;
  auto kind = [](DType t) { return t < NXB_S8 ? 0 : t < NXB_F16 ? 1 : t == NXB_BF16 ? 2 : 3; };
  auto bits = [](DType t) { return (int)dtype_size(t) * 8; };
  int ka = kind(a), kb = kind(b);
  auto make = [](int k, int bits) -> DType {
    int idx = bits == 8 ? 0 : bits == 16 ? 1 : bits == 32 ? 2 : 3;
    if (k == 0) return (DType)(NXB_U8 + idx);
    if (k == 1) return (DType)(NXB_S8 + idx);
    if (k == 2) return NXB_BF16;
    return bits == 16 ? NXB_F16 : bits == 32 ? NXB_F32 : NXB_F64;
  };
  if (ka == kb) return make(ka, std::max(bits(a), bits(b)));
  DType lo = ka < kb ? a : b, hi = ka < kb ? b : a;
  if (kind(lo) == 0 && kind(hi) == 1) return make(1, std::max(std::min(bits(lo) * 2, 64), bits(hi)));
  return hi;
}

std::string shape_str(const std::vector<int64_t>& s) {
  std::ostringstream o;
  o << "{";
  for (size_t i = 0; i < s.size(); ++i) o << (i ? "," : "") << s[i];
  o << "}";
  return o.str();
}

// ---- driver API ------------------------------------------------------------------------
static DriverApi g_driver;
static std::once_flag g_driver_once;

const DriverApi& driver() {
  std::call_once(g_driver_once, [] {
    auto get = [](const char* name, void** fn) {
      cudaDriverEntryPointQueryResult q;
      cudaError_t e = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q);
      if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !*fn) {
        (void)cudaGetLastError();
        *fn = nullptr;
      }
    };
    get("cuModuleLoadData", (void**)&g_driver.cuModuleLoadData);
    get("cuModuleUnload", (void**)&g_driver.cuModuleUnload);
    get("cuModuleGetFunction", (void**)&g_driver.cuModuleGetFunction);
    get("cuLaunchKernel", (void**)&g_driver.cuLaunchKernel);
    get("cuFuncSetAttribute", (void**)&g_driver.cuFuncSetAttribute);
    get("cuGetErrorString", (void**)&g_driver.cuGetErrorString);
    get("cuTensorMapEncodeTiled", (void**)&g_driver.cuTensorMapEncodeTiled);
    get("cuMemGetAddressRange", (void**)&g_driver.cuMemGetAddressRange);
  });
  return g_driver;
}

void check_cu(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* s = nullptr;
  if (g_driver.cuGetErrorString) g_driver.cuGetErrorString(r, &s);
  fail(NXB_ERR_RUNTIME, std::string(what) + ": " + (s ? s : "CUDA driver error ") + " (" + std::to_string((int)r) + ")");
}

// ---- allocator ----------------------------------------------------------------------------
size_t Allocator::round_size(size_t n) {
  if (n == 0) n = 1;
  if (n < (1u << 20)) return (n + 511) & ~size_t(511);
  return (n + (2u << 20) - 1) & ~size_t((2u << 20) - 1);
}

void* Allocator::alloc(size_t nbytes) {
  size_t sz = round_size(nbytes);
  void* p = nullptr;
  auto it = cache_.find(sz);
  if (it != cache_.end()) {
    p = it->second;
    cache_.erase(it);
  } else {
    cudaError_t e = cudaMalloc(&p, sz);
    if (e == cudaErrorMemoryAllocation) {
      (void)cudaGetLastError();
      release_cached();
      e = cudaMalloc(&p, sz);
    }
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      fail(e == cudaErrorMemoryAllocation ? NXB_ERR_OUT_OF_MEMORY : NXB_ERR_RUNTIME,
           "device allocation of " + std::to_string(sz) + " bytes failed: " + cudaGetErrorString(e));
    }
    reserved += sz;
  }
  live_[p] = {sz, nbytes};
  allocated += nbytes;
  if (allocated > peak) peak = allocated;
  return p;
}

void Allocator::free(void* p) {
  auto it = live_.find(p);
  if (it == live_.end()) return;
  allocated -= it->second.second;
  cache_.emplace(it->second.first, p);
  live_.erase(it);
}

void Allocator::release_cached() {
  for (auto& kv : cache_) {
    cudaFree(kv.second);
    reserved -= kv.first;
  }
  cache_.clear();
}

// ---- devices ----------------------------------------------------------------------------------
static std::deque<Device> g_devices;
static std::once_flag g_dev_once;
static int g_device_count = 0;

static void init_devices() {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  g_device_count = n;
  g_devices.resize(n);
  for (int i = 0; i < n; ++i) g_devices[i].id = i;
}

int device_count() {
  std::call_once(g_dev_once, init_devices);
  return g_device_count;
}

Device& device(int id) {
  int n = device_count();
  if (n == 0) fail(NXB_ERR_NO_DEVICE, "no CUDA device is visible to this process");
  if (id < 0 || id >= n) fail(NXB_ERR_INVALID_ARGUMENT, "device " + std::to_string(id) + " out of range (have " + std::to_string(n) + ")");
  Device& d = g_devices[id];
  NXB_CUDA(cudaSetDevice(id));
  if (!d.stream) {
    std::lock_guard<std::mutex> g(d.mu);
    if (!d.stream) {
      cudaStream_t s;
      NXB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
      NXB_CUDA(cudaEventCreate(&d.ev0));
      NXB_CUDA(cudaEventCreate(&d.ev1));
      NXB_CUDA(cudaStreamCreateWithFlags(&d.h2d, cudaStreamNonBlocking));
      NXB_CUDA(cudaStreamCreateWithFlags(&d.d2h, cudaStreamNonBlocking));
      NXB_CUDA(cudaEventCreateWithFlags(&d.ev_compute, cudaEventDisableTiming));
      NXB_CUDA(cudaEventCreateWithFlags(&d.ev_h2d, cudaEventDisableTiming));
      NXB_CUDA(cudaEventCreateWithFlags(&d.ev_d2h, cudaEventDisableTiming));
      int sms = 148;
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, id);
      d.sm_count = sms;
      int* host = nullptr;
      NXB_CUDA(cudaHostAlloc((void**)&host, 64, cudaHostAllocMapped));
      *host = 0;
      NXB_CUDA(cudaHostGetDevicePointer((void**)&d.status_dev, host, 0));
      d.status_host = host;
      d.stream = s;
    }
  }
  return d;
}

void check_device_status(Device& d) {
  if (d.status_host && *d.status_host) {
    *d.status_host = 0;
    fail(NXB_ERR_TIMEOUT, "a kernel gave up waiting on an internal barrier (results of the last run are invalid)");
  }
}

}  // namespace nxb

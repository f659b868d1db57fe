// Collectives for sharded programs: NCCL over NVLink, one process per GPU.
// The library is opened at first use so that single-GPU processes (and machines
// without NCCL) never load it.
#include <dlfcn.h>

#include "common.h"

namespace nxb {
namespace {

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclInt8 = 0, ncclUint8 = 1, ncclInt32 = 2, ncclUint32 = 3, ncclInt64 = 4, ncclUint64 = 5, ncclFloat16 = 6,
       ncclFloat32 = 7, ncclFloat64 = 8, ncclBfloat16 = 9 };
enum { ncclSum = 0 };

struct Nccl {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

Nccl& nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    // prefer a copy already in the process (e.g. the one torch loaded)
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      n.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (n.lib) break;
    }
    if (!n.lib) return;
    n.GetUniqueId = (decltype(n.GetUniqueId))dlsym(n.lib, "ncclGetUniqueId");
    n.CommInitRank = (decltype(n.CommInitRank))dlsym(n.lib, "ncclCommInitRank");
    n.CommDestroy = (decltype(n.CommDestroy))dlsym(n.lib, "ncclCommDestroy");
    n.AllReduce = (decltype(n.AllReduce))dlsym(n.lib, "ncclAllReduce");
    n.GetErrorString = (decltype(n.GetErrorString))dlsym(n.lib, "ncclGetErrorString");
  });
  if (!n.lib || !n.AllReduce) fail(NXB_ERR_RUNTIME, "NCCL (libnccl.so.2) could not be loaded");
  return n;
}

void check_nccl(ncclResult_t r, const char* what) {
  if (r == 0) return;
  fail(NXB_ERR_RUNTIME, std::string(what) + ": " + nccl().GetErrorString(r));
}

ncclComm_t g_comm = nullptr;
int g_comm_device = -1, g_world = 1, g_rank = 0;

}  // namespace

int comm_world() { return g_world; }
int comm_rank() { return g_rank; }

void comm_id(uint8_t* id) {
  ncclUniqueId u;
  check_nccl(nccl().GetUniqueId(&u), "ncclGetUniqueId");
  static_assert(sizeof(u) == NXB_COMM_ID_BYTES, "id size");
  memcpy(id, &u, sizeof u);
}

void comm_init(int dev, int rank, int world, const uint8_t* id) {
  if (g_comm) fail(NXB_ERR_INVALID_ARGUMENT, "communicator already initialised in this process");
  Device& d = device(dev);
  (void)d;
  ncclUniqueId u;
  memcpy(&u, id, sizeof u);
  check_nccl(nccl().CommInitRank(&g_comm, world, u, rank), "ncclCommInitRank");
  g_comm_device = dev;
  g_world = world;
  g_rank = rank;
}

void comm_all_reduce(const void* in, void* out, size_t count, DType dt, Device& d);
void comm_all_reduce_sum_ptr(void* p, size_t count, DType dt, Device& d) { comm_all_reduce(p, p, count, dt, d); }

void comm_all_reduce(const void* in, void* out, size_t count, DType dt, Device& d) {
  if (!g_comm) fail(NXB_ERR_INVALID_ARGUMENT, "no communicator: call nxb200_comm_init first");
  int t;
  switch (dt) {
    case NXB_S8: t = ncclInt8; break;
    case NXB_U8: t = ncclUint8; break;
    case NXB_S32: t = ncclInt32; break;
    case NXB_U32: t = ncclUint32; break;
    case NXB_S64: t = ncclInt64; break;
    case NXB_U64: t = ncclUint64; break;
    case NXB_F16: t = ncclFloat16; break;
    case NXB_BF16: t = ncclBfloat16; break;
    case NXB_F32: t = ncclFloat32; break;
    case NXB_F64: t = ncclFloat64; break;
    default: fail(NXB_ERR_UNSUPPORTED, "all-reduce of 16-bit integers");
  }
  check_nccl(nccl().AllReduce(in, out, count, t, ncclSum, g_comm, d.stream), "ncclAllReduce");
}

void comm_destroy() {
  if (g_comm) {
    nccl().CommDestroy(g_comm);
    g_comm = nullptr;
    g_world = 1;
    g_rank = 0;
  }
}

}  // namespace nxb

using namespace nxb;

extern "C" {

static int guarded_comm(void (*f)(void*), void* ctx) {
  try {
    f(ctx);
    return NXB_OK;
  } catch (const Error& e) {
    set_last_error(e.msg);
    return e.status;
  } catch (const std::exception& e) {
    set_last_error(e.what());
    return NXB_ERR_RUNTIME;
  }
}

int nxb200_comm_id(uint8_t id[NXB_COMM_ID_BYTES]) {
  return guarded_comm([](void* p) { comm_id((uint8_t*)p); }, id);
}

int nxb200_comm_init(int dev, int rank, int world, const uint8_t id[NXB_COMM_ID_BYTES]) {
  struct A { int d, r, w; const uint8_t* id; } a{dev, rank, world, id};
  return guarded_comm([](void* p) { A* a = (A*)p; comm_init(a->d, a->r, a->w, a->id); }, &a);
}

int nxb200_comm_all_reduce_sum(nxb200_buffer* buf) {
  return guarded_comm([](void* p) {
    nxb200_buffer* b = (nxb200_buffer*)p;
    if (!b || b->magic != 0x4e584242 || b->deallocated.load()) fail(NXB_ERR_INVALID_ARGUMENT, "not a live buffer handle");
    Device& d = device(b->device);
    comm_all_reduce_sum_ptr(b->ptr, (size_t)shape_numel(b->dims), b->dtype, d);
  }, buf);
}

int nxb200_comm_destroy(void) {
  return guarded_comm([](void*) { comm_destroy(); }, nullptr);
}

}  // extern "C"

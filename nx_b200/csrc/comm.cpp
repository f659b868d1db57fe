// Collectives for sharded programs: NCCL over NVLink, one process per GPU.
// The library is opened at first use so that single-GPU processes (and machines
// without NCCL) never load it.
#include <dlfcn.h>

#include "gemm.h"

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

// Peer memory of the group: see PeerView (gemm.h).
struct PeerState {
  bool enabled = false;
  void* local = nullptr;
  void* peers[8] = {};
  size_t bytes = 0;
  PeerView view;
} g_peer;

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

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

// Allocates this rank's region for matrices of up to `elems` 16-bit elements and writes the
// blob the other ranks need: the 64-byte IPC handle followed by the device's 16-byte UUID.
void comm_peer_alloc(int dev, size_t elems, uint8_t* blob) {
  if (!g_comm) fail(NXB_ERR_INVALID_ARGUMENT, "no communicator: call nxb200_comm_init first");
  if (g_world > 8) fail(NXB_ERR_UNSUPPORTED, "peer memory for more than 8 ranks");
  if (g_peer.local) fail(NXB_ERR_INVALID_ARGUMENT, "peer memory already allocated in this process");
  Device& d = device(dev);
  (void)d;
  PeerView& v = g_peer.view;
  v = PeerView();
  v.rank = g_rank;
  v.world = g_world;
  v.elems = elems;
  v.flag_words = 4 * (elems / (128 * 64) + 64);     // 4 words per output tile of at least 128 x 64
  v.partial_off = 0;
  v.result_off = align256(elems * 2);
  v.ready_off = v.result_off + align256(elems * 2);
  v.reduced_off = v.ready_off + align256(v.flag_words * 4);
  g_peer.bytes = v.reduced_off + align256(v.flag_words * 4);
  NXB_CUDA(cudaMalloc(&g_peer.local, g_peer.bytes));
  NXB_CUDA(cudaMemset(g_peer.local, 0, g_peer.bytes));
  NXB_CUDA(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  NXB_CUDA(cudaIpcGetMemHandle(&h, g_peer.local));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(blob, &h, 64);
  cudaDeviceProp prop;
  NXB_CUDA(cudaGetDeviceProperties(&prop, dev));
  memcpy(blob + 64, &prop.uuid, 16);
}

// Maps the other ranks' regions.  `blobs` holds world x NXB_COMM_PEER_BLOB_BYTES bytes in rank
// order.  Returns false (and leaves the group on NCCL) when two ranks share a GPU - kernels that
// wait on one another must never share one - or a region cannot be mapped.
bool comm_peer_open(const uint8_t* blobs) {
  if (!g_peer.local) fail(NXB_ERR_INVALID_ARGUMENT, "peer memory was not allocated");
  for (int a = 0; a < g_world; ++a)
    for (int b = a + 1; b < g_world; ++b)
      if (memcmp(blobs + a * 80 + 64, blobs + b * 80 + 64, 16) == 0) return false;
  for (int r = 0; r < g_world; ++r) {
    if (r == g_rank) { g_peer.peers[r] = g_peer.local; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, blobs + r * 80, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      for (int q = 0; q < r; ++q)
        if (q != g_rank && g_peer.peers[q]) { cudaIpcCloseMemHandle(g_peer.peers[q]); g_peer.peers[q] = nullptr; }
      return false;
    }
    g_peer.peers[r] = p;
  }
  for (int r = 0; r < g_world; ++r) g_peer.view.base[r] = g_peer.peers[r];
  g_peer.enabled = true;
  return true;
}

bool comm_peer_view(int64_t m, int64_t n, int64_t mtiles, int64_t ntiles, PeerView* v) {
  if (!g_peer.enabled) return false;
  if ((size_t)(m * n) > g_peer.view.elems || (size_t)(mtiles * ntiles * 4) > g_peer.view.flag_words) return false;
  if (mtiles % g_world != 0) return false;
  g_peer.view.epoch += 1;
  *v = g_peer.view;
  return true;
}

void comm_destroy() {
  if (g_peer.local) {
    cudaDeviceSynchronize();
    for (int r = 0; r < g_world; ++r)
      if (r != g_rank && g_peer.peers[r]) cudaIpcCloseMemHandle(g_peer.peers[r]);
    cudaFree(g_peer.local);
    g_peer = PeerState();
  }
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

int nxb200_comm_peer_alloc(int dev, uint64_t elems, uint8_t blob[NXB_COMM_PEER_BLOB_BYTES]) {
  struct A { int d; uint64_t e; uint8_t* b; } a{dev, elems, blob};
  return guarded_comm([](void* p) { A* a = (A*)p; comm_peer_alloc(a->d, (size_t)a->e, a->b); }, &a);
}

int nxb200_comm_peer_open(const uint8_t* blobs, int* enabled) {
  struct A { const uint8_t* b; int* e; } a{blobs, enabled};
  return guarded_comm([](void* p) { A* a = (A*)p; *a->e = comm_peer_open(a->b) ? 1 : 0; }, &a);
}

int nxb200_comm_fused_launches(uint64_t* count) {
  return guarded_comm([](void* p) { *(uint64_t*)p = g_peer.enabled ? g_peer.view.epoch : 0; }, count);
}

int nxb200_comm_destroy(void) {
  return guarded_comm([](void*) { comm_destroy(); }, nullptr);
}

}  // extern "C"

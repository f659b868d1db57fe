// Asynchronous host -> device upload from memory the caller cannot pin (an Erlang binary, a numpy
// array): the counterpart of the reference's zero-copy host view with an on-done callback
// (exla/c_src/exla/exla_client.cc:118-151: the binary is kept alive in a private environment
// until the transfer completes, then released).
//
// One uploader thread per device owns a ring of pinned staging buffers.  For each job it copies a
// chunk of the source into a free slot, enqueues the slot's DMA on the device's upload stream and
// moves on, so the host copy of chunk i+1 overlaps the DMA of chunk i.  As soon as the last byte of
// the source has been copied into staging the caller's callback fires: the source may be released
// then, the DMA no longer needs it.  After the last DMA is enqueued the job's `ready` event is
// recorded; the first use of the buffer orders the compute stream after it.
#include <condition_variable>
#include <deque>
#include <thread>

#include "common.h"

struct nxb200_buffer::Upload {
  std::mutex mu;
  std::condition_variable cv;
  bool enqueued = false, joined = false;
  cudaEvent_t after = nullptr;     // compute-stream work queued before the upload (the memory may be recycled)
  cudaEvent_t ready = nullptr;     // recorded on the upload stream after the last chunk
  cudaError_t error = cudaSuccess;
  int device = 0;
};

namespace nxb {
namespace {

constexpr size_t SLOT_BYTES = size_t(4) << 20;
constexpr int SLOTS = 4;

struct Job {
  std::shared_ptr<nxb200_buffer::Upload> up;
  void* dst;
  const unsigned char* src;
  size_t nbytes;
  UploadDone on_done;
  void* ctx;
};

struct Uploader {
  std::mutex mu;
  std::condition_variable cv;
  std::deque<Job> jobs;
  bool started = false;
  unsigned char* slot[SLOTS] = {};
  cudaEvent_t slot_free[SLOTS] = {};
  int next = 0;
};

// The uploaders live until the process ends and are never destroyed: their threads are detached and
// wait on the condition variables inside, and destroying a condition variable that has a waiter blocks
// (a process that had uploaded anything would hang at exit in the static destructors).
Uploader& uploader(int dev) {
  static std::mutex* mu = new std::mutex;
  static std::map<int, Uploader*>* all = new std::map<int, Uploader*>;
  std::lock_guard<std::mutex> g(*mu);
  Uploader*& u = (*all)[dev];
  if (!u) u = new Uploader;
  return *u;
}

void run(Uploader* u, int dev, cudaStream_t h2d) {
  cudaSetDevice(dev);
  for (;;) {
    Job job;
    {
      std::unique_lock<std::mutex> lk(u->mu);
      u->cv.wait(lk, [&] { return !u->jobs.empty(); });
      job = std::move(u->jobs.front());
      u->jobs.pop_front();
    }
    cudaError_t err = cudaSuccess;
    if (!u->slot[0]) {
      for (int i = 0; i < SLOTS && err == cudaSuccess; ++i) {
        err = cudaHostAlloc((void**)&u->slot[i], SLOT_BYTES, cudaHostAllocDefault);
        if (err == cudaSuccess) err = cudaEventCreateWithFlags(&u->slot_free[i], cudaEventDisableTiming);
      }
    }
    if (err == cudaSuccess) err = cudaStreamWaitEvent(h2d, job.up->after, 0);
    for (size_t off = 0; off < job.nbytes && err == cudaSuccess; off += SLOT_BYTES) {
      const size_t n = std::min(SLOT_BYTES, job.nbytes - off);
      const int s = u->next;
      u->next = (u->next + 1) % SLOTS;
      err = cudaEventSynchronize(u->slot_free[s]);          // the slot's previous DMA has read it (a fresh event is complete)
      if (err != cudaSuccess) break;
      memcpy(u->slot[s], job.src + off, n);
      err = cudaMemcpyAsync((char*)job.dst + off, u->slot[s], n, cudaMemcpyHostToDevice, h2d);
      if (err == cudaSuccess) err = cudaEventRecord(u->slot_free[s], h2d);
    }
    // every byte of the source has been copied out of the caller's memory (or the upload failed)
    if (job.on_done) job.on_done(job.ctx);
    if (err == cudaSuccess) err = cudaEventRecord(job.up->ready, h2d);
    {
      std::lock_guard<std::mutex> g(job.up->mu);
      job.up->error = err;
      job.up->enqueued = true;
    }
    job.up->cv.notify_all();
  }
}

}  // namespace

void upload_enqueue(Device& d, nxb200_buffer* b, const void* src, size_t nbytes, UploadDone on_done, void* ctx) {
  auto up = std::make_shared<nxb200_buffer::Upload>();
  up->device = d.id;
  NXB_CUDA(cudaEventCreateWithFlags(&up->after, cudaEventDisableTiming));
  NXB_CUDA(cudaEventCreateWithFlags(&up->ready, cudaEventDisableTiming));
  {
    std::lock_guard<std::mutex> g(d.mu);
    NXB_CUDA(cudaEventRecord(up->after, d.stream));
  }
  b->upload = up;
  Uploader& u = uploader(d.id);
  {
    std::lock_guard<std::mutex> g(u.mu);
    if (!u.started) {
      u.started = true;
      std::thread(run, &u, d.id, d.h2d).detach();
    }
    u.jobs.push_back(Job{up, b->ptr, (const unsigned char*)src, nbytes, on_done, ctx});
  }
  u.cv.notify_one();
}

void upload_join(nxb200_buffer* b) {
  std::shared_ptr<nxb200_buffer::Upload> up = b->upload;
  if (!up) return;
  cudaError_t err;
  {
    std::unique_lock<std::mutex> lk(up->mu);
    up->cv.wait(lk, [&] { return up->enqueued; });
    err = up->error;
    if (up->joined) return;
    up->joined = true;
  }
  Device& d = device(up->device);
  if (err == cudaSuccess) {
    std::lock_guard<std::mutex> g(d.mu);
    err = cudaStreamWaitEvent(d.stream, up->ready, 0);
    // the events are destroyed once the waits that use them are enqueued (CUDA keeps what it needs)
    cudaEventDestroy(up->after);
    cudaEventDestroy(up->ready);
  }
  b->upload.reset();
  if (err != cudaSuccess) fail(NXB_ERR_RUNTIME, std::string("asynchronous upload failed: ") + cudaGetErrorString(err));
}

}  // namespace nxb

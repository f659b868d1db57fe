// extern "C" surface of libnxb200.so (declared in include/nxb200.h).
#include <algorithm>

#include "gemm.h"
#include "program.h"

namespace nxb {
const std::string& last_error();
void canonicalize_dots(Graph& g);
void comm_all_reduce(const void* in, void* out, size_t count, DType dt, Device& d);
}  // namespace nxb

using namespace nxb;

namespace {

template <typename F> int guarded(F&& f) {
  try {
    f();
    return NXB_OK;
  } catch (const Error& e) {
    set_last_error(e.msg);
    return e.status;
  } catch (const std::bad_alloc&) {
    set_last_error("host allocation failed");
    return NXB_ERR_OUT_OF_MEMORY;
  } catch (const std::exception& e) {
    set_last_error(e.what());
    return NXB_ERR_RUNTIME;
  }
}

nxb200_buffer* check_buffer(nxb200_buffer* b, bool need_live = true) {
  if (!b || b->magic != 0x4e584242) fail(NXB_ERR_INVALID_ARGUMENT, "not a buffer handle");
  if (need_live && b->deallocated.load()) fail(NXB_ERR_RUNTIME, "buffer has been deallocated (use after free)");
  if (b->upload) upload_join(b);       // an asynchronous upload: from here on the compute stream is ordered after it
  return b;
}

nxb200_program* check_program(nxb200_program* p) {
  if (!p || p->magic != 0x4e584250) fail(NXB_ERR_INVALID_ARGUMENT, "not a program handle");
  return p;
}

nxb200_buffer* make_buffer(Device& d, DType dt, const int64_t* dims, int rank) {
  if (rank < 0 || rank > NXB_MAX_RANK) fail(NXB_ERR_INVALID_ARGUMENT, "rank out of range");
  if ((int)dt < 0 || dt > NXB_F64) fail(NXB_ERR_INVALID_ARGUMENT, "unknown element type");
  auto b = std::make_unique<nxb200_buffer>();
  b->device = d.id;
  b->dtype = dt;
  for (int i = 0; i < rank; ++i) {
    if (dims[i] < 0) fail(NXB_ERR_INVALID_ARGUMENT, "negative dimension");
    b->dims.push_back(dims[i]);
  }
  b->nbytes = (size_t)shape_numel(b->dims) * dtype_size(dt);
  {
    std::lock_guard<std::mutex> g(d.mu);
    b->ptr = d.alloc.alloc(b->nbytes);
  }
  return b.release();
}

// Compute work queued from here on starts after the downloads in flight (caller holds d.mu).
void order_after_downloads(Device& d) {
  if (d.pending_reads.empty()) return;
  NXB_CUDA(cudaStreamWaitEvent(d.stream, d.ev_d2h, 0));
  d.pending_reads.clear();
}

void ensure_loaded(nxb200_program* p, Device& d) {
  auto it = p->loaded.find(d.id);
  if (it != p->loaded.end()) return;
  const DriverApi& drv = driver();
  if (!drv.cuModuleLoadData || !drv.cuLaunchKernel) fail(NXB_ERR_RUNTIME, "CUDA driver entry points are unavailable");
  nxb200_program::Loaded L;
  for (auto& ks : p->plan->kernels) {
    CUmodule m;
    check_cu(drv.cuModuleLoadData(&m, ks.cubin.data()), ("loading kernel " + ks.name).c_str());
    CUfunction f;
    check_cu(drv.cuModuleGetFunction(&f, m, ks.name.c_str()), ("resolving kernel " + ks.name).c_str());
    if (ks.smem > 48 * 1024)
      check_cu(drv.cuFuncSetAttribute(f, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)ks.smem), ("configuring " + ks.name).c_str());
    L.modules.push_back(m);
    L.functions.push_back(f);
  }
  for (size_t s = 0; s < p->plan->slots.size(); ++s) {
    const Slot& sl = p->plan->slots[s];
    if (sl.kind != Slot::LITERAL) continue;
    void* ptr = d.alloc.alloc(sl.nbytes);
    const std::string& blob = p->plan->g.nodes[sl.node].blob;
    NXB_CUDA(cudaMemcpyAsync(ptr, blob.data(), blob.size(), cudaMemcpyHostToDevice, d.stream));
    L.literals[(int)s] = ptr;
  }
  NXB_CUDA(cudaStreamSynchronize(d.stream));
  p->loaded.emplace(d.id, std::move(L));
}

void run_program(nxb200_program* p, int device, nxb200_buffer* const* args, int n_args, nxb200_buffer** outs, int n_outs,
                 bool outs_provided) {
  Plan& plan = *p->plan;
  if (n_args != (int)plan.param_slots.size())
    fail(NXB_ERR_INVALID_ARGUMENT, "program takes " + std::to_string(plan.param_slots.size()) + " arguments, got " + std::to_string(n_args));
  if (n_outs != (int)plan.output_slots.size())
    fail(NXB_ERR_INVALID_ARGUMENT, "program has " + std::to_string(plan.output_slots.size()) + " outputs, got room for " + std::to_string(n_outs));
  Device& d = nxb::device(device);
  std::vector<void*> ptr(plan.slots.size(), nullptr);
  for (int i = 0; i < n_args; ++i) {
    int s = plan.param_slots[i];
    nxb200_buffer* b = check_buffer(args[i]);
    if (b->device != device) fail(NXB_ERR_INVALID_ARGUMENT, "argument " + std::to_string(i) + " lives on device " + std::to_string(b->device) + ", program runs on " + std::to_string(device));
    if (s < 0) continue;
    const Slot& sl = plan.slots[s];
    if (b->dtype != sl.dt || b->dims != sl.shape)
      fail(NXB_ERR_INVALID_ARGUMENT, "argument " + std::to_string(i) + " is " + dtype_name(b->dtype) + shape_str(b->dims) + ", program was built for " +
                                         dtype_name(sl.dt) + shape_str(sl.shape));
    ptr[s] = b->ptr;
  }
  std::lock_guard<std::mutex> pg(p->mu);
  std::lock_guard<std::mutex> dg(d.mu);
  ensure_loaded(p, d);
  order_after_downloads(d);
  auto& L = p->loaded[device];
  for (auto& kv : L.literals) ptr[kv.first] = kv.second;
  std::vector<nxb200_buffer*> made;
  try {
    for (int i = 0; i < n_outs; ++i) {
      const Slot& sl = plan.slots[plan.output_slots[i]];
      if (outs_provided) {
        nxb200_buffer* b = check_buffer(outs[i]);
        if (b->device != device || b->dtype != sl.dt || b->dims != sl.shape)
          fail(NXB_ERR_INVALID_ARGUMENT, "output buffer " + std::to_string(i) + " does not match " + dtype_name(sl.dt) + shape_str(sl.shape));
        ptr[plan.output_slots[i]] = b->ptr;
      } else {
        auto b = std::make_unique<nxb200_buffer>();
        b->device = device;
        b->dtype = sl.dt;
        b->dims = sl.shape;
        b->nbytes = sl.nbytes;
        // a result that takes over a donated argument's buffer is written straight into it
        void* taken = nullptr;
        for (auto& al : plan.aliases)
          if (al.output == i && al.in_place && !args[al.param]->deallocated.load() && !args[al.param]->borrowed) taken = args[al.param]->ptr;
        // The plan proved "one reader, same position" per parameter slot, not per address: a buffer that
        // is also passed as another argument, or was already taken for an earlier result, keeps its memory
        // and this result gets its own.
        if (taken) {
          int uses = 0;
          for (int a2 = 0; a2 < n_args; ++a2) if (args[a2]->ptr == taken) ++uses;
          for (auto* mb : made) if (mb->ptr == taken) ++uses;
          if (uses > 1) taken = nullptr;
        }
        b->ptr = taken ? taken : d.alloc.alloc(sl.nbytes);
        ptr[plan.output_slots[i]] = b->ptr;
        made.push_back(b.release());
      }
    }
    // a window update whose result does not share the argument's memory starts from a copy of it
    for (auto& al : plan.aliases) {
      if (!al.window) continue;
      void* dst = ptr[plan.output_slots[al.output]];
      if (dst != args[al.param]->ptr)
        NXB_CUDA(cudaMemcpyAsync(dst, args[al.param]->ptr, plan.slots[plan.output_slots[al.output]].nbytes, cudaMemcpyDeviceToDevice, d.stream));
    }
    const DriverApi& drv = driver();
    // Runs the plan's steps on the device's stream.  With `held` the temporaries are kept (their
    // addresses are baked into a graph being captured) and anything that needs scratch memory of
    // its own makes the program unfit for replay.
    struct NotReplayable {};
    auto run_steps = [&](std::vector<void*>* held) {
    bool skip_step = false;      // the previous product already did this step's all-reduce
    for (size_t st = 0; st < plan.steps.size(); ++st) {
      for (size_t s = 0; s < plan.slots.size(); ++s)
        if (plan.slots[s].kind == Slot::TEMP && plan.slots[s].first_step == (int)st && !ptr[s]) ptr[s] = d.alloc.alloc(plan.slots[s].nbytes);
      const Step& step = plan.steps[st];
      if (skip_step) {
        skip_step = false;
      } else if (step.kind == Step::KERNEL) {
        const KernelSpec& ks = plan.kernels[step.index];
        std::vector<void*> argv(ks.arg_slots.size());
        std::vector<void*> argp(ks.arg_slots.size());
        for (size_t a = 0; a < ks.arg_slots.size(); ++a) {
          void* base = ptr[ks.arg_slots[a]];
          if (!base) fail(NXB_ERR_RUNTIME, "internal: kernel " + ks.name + " reads a buffer that was never produced");
          argv[a] = (char*)base + ks.arg_offsets[a];
          argp[a] = &argv[a];
        }
        check_cu(drv.cuLaunchKernel(L.functions[step.index], ks.grid, 1, 1, ks.block, 1, 1, ks.smem, (CUstream)d.stream, argp.data(), nullptr),
                 ("launching " + ks.name).c_str());
      } else if (step.kind == Step::ATTENTION) {
        const AttentionSpec& as = plan.attentions[step.index];
        const KernelSpec& ks = plan.kernels[as.jit_kernel];
        std::vector<void*> ep(ks.arg_slots.size());
        for (size_t a = 0; a < ks.arg_slots.size(); ++a) ep[a] = ptr[ks.arg_slots[a]];
        TcLaunch tl;
        attn_prepare_launch(ptr[as.q_slot], ptr[as.k_slot], ptr[as.v_slot], ptr[as.out_slot], as.batch_heads, as.sq, as.sk, as.causal, ep.data(),
                            (int)ep.size(), d.status_dev, &tl, as.heads, as.v_bshd, as.out_bshd);
        void* params[4] = {tl.map_a, tl.map_b, tl.map_c, tl.params};
        check_cu(drv.cuLaunchKernel(L.functions[as.jit_kernel], tl.grid, 1, 1, 320, 1, 1, (unsigned)tl.smem, (CUstream)d.stream, params, nullptr),
                 ("launching " + ks.name).c_str());
      } else if (step.kind == Step::SORT) {
        const SortSpec& ss = plan.sorts[step.index];
        launch_sort_rows(ptr[ss.in_slot], ptr[ss.out_slot], ss.rows, ss.len, ss.dt, ss.out_dt, ss.descending, ss.indices, d.sm_count, d.stream);
      } else if (step.kind == Step::SCATTER) {
        const ScatterSpec& sc = plan.scatters[step.index];
        launch_scatter(sc, ptr[sc.target_slot], ptr[sc.indices_slot], ptr[sc.updates_slot], ptr[sc.out_slot], d.sm_count, d.stream);
      } else if (step.kind == Step::ALLREDUCE) {
        if (held) throw NotReplayable();
        const CollectiveSpec& cs = plan.collectives[step.index];
        comm_all_reduce(ptr[cs.in_slot], ptr[cs.out_slot], (size_t)cs.count, cs.dt, d);
      } else {
        const GemmSpec& gs = plan.gemms[step.index];
        GemmArgs ga{};
        ga.a = ptr[gs.a.slot];
        ga.b = ptr[gs.b.slot];
        ga.c = gs.jit_kernel >= 0 ? nullptr : ptr[gs.out_slot];
        ga.batch = gs.batch; ga.m = gs.m; ga.n = gs.n; ga.k = gs.k;
        ga.lda = gs.a.ld; ga.ldb = gs.b.ld; ga.bsa = gs.a.batch_stride; ga.bsb = gs.b.batch_stride;
        ga.ta = gs.a.trans; ga.tb = gs.b.trans;
        ga.da = gs.a.dt; ga.db = gs.b.dt; ga.dc = gs.out_dt;
        ga.epilogue = gs.epilogue;
        if (gs.scale_slot >= 0) ga.scale = ptr[gs.scale_slot];
        // 16-bit operands are consumed with either index contiguous when their rows are 16-byte
        // aligned; everything else is first copied into K-major form
        const size_t es = dtype_size(ga.da);
        const bool mn_a = ga.ta && es == 2 && (ga.m * es) % 16 == 0;
        const bool mn_b = ga.tb && es == 2 && (ga.n * es) % 16 == 0;
        GemmArgs fin = ga;
        if (ga.ta && !mn_a) { fin.ta = false; fin.lda = ga.k; fin.bsa = ga.m * ga.k; }
        if (ga.tb && !mn_b) { fin.tb = false; fin.ldb = ga.k; fin.bsb = ga.n * ga.k; }
        if (ga.scale && ga.db == NXB_S8 && ga.da == NXB_BF16) {
          // s8 weights converted inside the product kernel (few rows of x)
          if (!wq_linear_supported(ga)) fail(NXB_ERR_RUNTIME, "internal: quantised linear outside the in-kernel conversion path");
          launch_wq_linear(ga, d.status_dev, d.sm_count, d.stream);
          goto step_done;
        }
        const bool on_tensor_cores = tc_gemm_supported(fin);
        if ((ga.scale || gs.jit_kernel >= 0) && !on_tensor_cores) fail(NXB_ERR_RUNTIME, "internal: fused product outside the tensor-core path");
        if (on_tensor_cores) {
          void* ta = nullptr;
          void* tb = nullptr;
          if (held && ((ga.ta && !mn_a) || (ga.tb && !mn_b))) throw NotReplayable();
          if (ga.ta && !mn_a) {
            ta = d.alloc.alloc((size_t)(ga.batch * ga.m * ga.k) * es);
            launch_transpose(ga.a, ta, ga.batch, ga.k, ga.m, es, d.stream);
            fin.a = ta;
          }
          if (ga.tb && !mn_b) {
            tb = d.alloc.alloc((size_t)(ga.batch * ga.n * ga.k) * es);
            launch_transpose(ga.b, tb, ga.batch, ga.k, ga.n, es, d.stream);
            fin.b = tb;
          }
          ga = fin;
          if (gs.jit_kernel >= 0) {
            const KernelSpec& ks = plan.kernels[gs.jit_kernel];
            std::vector<void*> ep(ks.arg_slots.size());
            for (size_t a = 0; a < ks.arg_slots.size(); ++a) {
              ep[a] = ptr[ks.arg_slots[a]];
              if (!ep[a]) fail(NXB_ERR_RUNTIME, "internal: epilogue of " + ks.name + " reads a buffer that was never produced");
            }
            TcLaunch tl;
            tc_prepare_launch(ga, gs.bn, ep.data(), (int)ep.size(), d.status_dev, d.sm_count, &tl, gs.staged_arg, gs.staged_dt);
            void* params[4] = {tl.map_a, tl.map_b, tl.map_c, tl.params};
            check_cu(drv.cuLaunchKernel(L.functions[gs.jit_kernel], tl.grid, 1, 1, ks.block, 1, 1, (unsigned)tl.smem, (CUstream)d.stream, params, nullptr),
                     ("launching " + ks.name).c_str());
          } else {
            // a row-parallel product whose only reader is the sum over ranks: one kernel does
            // both over peer memory when the group has it (otherwise NCCL follows as its own step)
            bool fused = false;
            if (st + 1 < plan.steps.size() && plan.steps[st + 1].kind == Step::ALLREDUCE) {
              const CollectiveSpec& cs = plan.collectives[plan.steps[st + 1].index];
              const Slot& prod = plan.slots[gs.out_slot];
              if (cs.in_slot == gs.out_slot && prod.kind == Slot::TEMP && prod.last_step == (int)st + 1 && cs.dt == ga.dc) {
                if (!ptr[cs.out_slot]) ptr[cs.out_slot] = d.alloc.alloc(plan.slots[cs.out_slot].nbytes);
                fused = launch_tc_gemm_allreduce(ga, ptr[cs.out_slot], d.status_dev, d.sm_count, d.stream);
              }
            }
            if (fused) skip_step = true;
            else launch_tc_gemm(ga, d.status_dev, d.sm_count, d.stream);
          }
          if (ta) d.alloc.free(ta);
          if (tb) d.alloc.free(tb);
        } else {
          launch_simt_gemm(ga, d.stream);
        }
      }
    step_done:
      for (size_t s = 0; s < plan.slots.size(); ++s)
        if (plan.slots[s].kind == Slot::TEMP && plan.slots[s].last_step == (int)st && ptr[s]) {
          if (held) held->push_back(ptr[s]);
          else d.alloc.free(ptr[s]);
          ptr[s] = nullptr;
        }
    }
    };

    // ---- replay of small programs as CUDA graphs ----
    static const bool graphs_off = getenv("NXB200_NO_GRAPHS") != nullptr;
    size_t temp_bytes = 0;
    for (auto& sl : plan.slots) if (sl.kind == Slot::TEMP) temp_bytes += sl.nbytes;
    const bool small = plan.steps.size() <= 64 && temp_bytes <= (64u << 20) && plan.collectives.empty();
    bool done = false;
    if (!graphs_off && small && L.graphable) {
      std::vector<void*> key;
      for (int i = 0; i < n_args; ++i) key.push_back(args[i]->ptr);
      for (int i = 0; i < n_outs; ++i) key.push_back(ptr[plan.output_slots[i]]);
      ++L.tick;
      for (auto& r : L.replays)
        if (r.key == key) {
          NXB_CUDA(cudaGraphLaunch(r.exec, d.stream));
          r.last_use = L.tick;
          done = true;
          break;
        }
      if (!done) {
        auto it = std::find(L.seen.begin(), L.seen.end(), key);
        if (it == L.seen.end()) {
          if (L.seen.size() >= 16) L.seen.erase(L.seen.begin());
          L.seen.push_back(key);
        } else {
          L.seen.erase(it);
          nxb200_program::Loaded::Replay r;
          r.key = key;
          cudaGraph_t graph = nullptr;
          bool captured = false;
          if (cudaStreamBeginCapture(d.stream, cudaStreamCaptureModeRelaxed) == cudaSuccess) {
            try {
              run_steps(&r.held);
              captured = cudaStreamEndCapture(d.stream, &graph) == cudaSuccess && graph != nullptr;
            } catch (const NotReplayable&) {
              cudaStreamEndCapture(d.stream, &graph);
            } catch (...) {
              // whatever failed under capture is retried below as plain launches, which report it properly
              cudaStreamEndCapture(d.stream, &graph);
            }
          }
          if (captured && cudaGraphInstantiate(&r.exec, graph, 0) == cudaSuccess) {
            cudaGraphDestroy(graph);
            NXB_CUDA(cudaGraphLaunch(r.exec, d.stream));
            r.last_use = L.tick;
            if (L.replays.size() >= 8) {      // evict the least recently used (its work is ordered before ours on the stream)
              auto lru = std::min_element(L.replays.begin(), L.replays.end(), [](auto& x, auto& y) { return x.last_use < y.last_use; });
              cudaGraphExecDestroy(lru->exec);
              for (void* h : lru->held) d.alloc.free(h);
              L.replays.erase(lru);
            }
            L.replays.push_back(std::move(r));
            done = true;
          } else {
            // not fit for replay (scratch memory, a collective, or the capture failed): plain launches from now on
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            for (void* h : r.held) d.alloc.free(h);
            for (size_t s2 = 0; s2 < plan.slots.size(); ++s2)
              if (plan.slots[s2].kind == Slot::TEMP && ptr[s2]) { d.alloc.free(ptr[s2]); ptr[s2] = nullptr; }
            L.graphable = false;
          }
        }
      }
    }
    if (!done) run_steps(nullptr);
  } catch (...) {
    for (auto* b : made) {
      bool taken = false;
      for (int i = 0; i < n_args; ++i) if (args[i]->ptr == b->ptr) taken = true;
      if (!taken) d.alloc.free(b->ptr);
      delete b;
    }
    for (size_t s = 0; s < plan.slots.size(); ++s)
      if (plan.slots[s].kind == Slot::TEMP && ptr[s]) d.alloc.free(ptr[s]);
    throw;
  }
  if (!outs_provided) {
    for (int i = 0; i < n_outs; ++i) outs[i] = made[i];
    // donated arguments are consumed: their memory now belongs to a result, or goes back to the
    // pool (the stream orders any reuse after this program's kernels)
    for (auto& al : plan.aliases) {
      nxb200_buffer* a = args[al.param];
      if (a->deallocated.exchange(true)) continue;
      if (!(al.in_place && made[al.output]->ptr == a->ptr)) d.alloc.free(a->ptr);
      a->ptr = nullptr;
    }
  }
}

}  // namespace

extern "C" {

size_t nxb200_last_error(char* dst, size_t cap) {
  const std::string& e = last_error();
  if (dst && cap) {
    size_t n = std::min(cap - 1, e.size());
    memcpy(dst, e.data(), n);
    dst[n] = 0;
  }
  return e.size();
}

int nxb200_init(void) {
  return guarded([] { (void)device_count(); });
}

int nxb200_device_count(int* count) {
  return guarded([&] {
    if (!count) fail(NXB_ERR_INVALID_ARGUMENT, "count is NULL");
    *count = device_count();
  });
}

int nxb200_buffer_alloc(int dev, nxb200_dtype dtype, const int64_t* dims, int rank, nxb200_buffer** out) {
  return guarded([&] {
    if (!out) fail(NXB_ERR_INVALID_ARGUMENT, "out is NULL");
    Device& d = nxb::device(dev);
    *out = make_buffer(d, dtype, dims, rank);
  });
}

int nxb200_buffer_from_host(int dev, nxb200_dtype dtype, const int64_t* dims, int rank, const void* src, size_t nbytes,
                            nxb200_buffer** out) {
  return guarded([&] {
    if (!out) fail(NXB_ERR_INVALID_ARGUMENT, "out is NULL");
    Device& d = nxb::device(dev);
    nxb200_buffer* b = make_buffer(d, dtype, dims, rank);
    if (nbytes != b->nbytes) {
      size_t want = b->nbytes;
      { std::lock_guard<std::mutex> g(d.mu); d.alloc.free(b->ptr); }
      delete b;
      fail(NXB_ERR_INVALID_ARGUMENT, "binary has " + std::to_string(nbytes) + " bytes, tensor needs " + std::to_string(want));
    }
    if (nbytes) {
      cudaError_t e = cudaMemcpyAsync(b->ptr, src, nbytes, cudaMemcpyHostToDevice, d.stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(d.stream);
      if (e != cudaSuccess) {
        { std::lock_guard<std::mutex> g(d.mu); d.alloc.free(b->ptr); }
        delete b;
        fail(NXB_ERR_RUNTIME, std::string("host to device copy failed: ") + cudaGetErrorString(e));
      }
    }
    *out = b;
  });
}

int nxb200_buffer_from_host_async(int dev, nxb200_dtype dtype, const int64_t* dims, int rank, const void* src, size_t nbytes,
                                  nxb200_upload_done on_done, void* ctx, nxb200_buffer** out) {
  return guarded([&] {
    if (!out) fail(NXB_ERR_INVALID_ARGUMENT, "out is NULL");
    Device& d = nxb::device(dev);
    nxb200_buffer* b = make_buffer(d, dtype, dims, rank);
    if (nbytes != b->nbytes || (nbytes && !src)) {
      size_t want = b->nbytes;
      { std::lock_guard<std::mutex> g(d.mu); d.alloc.free(b->ptr); }
      delete b;
      fail(NXB_ERR_INVALID_ARGUMENT, "binary has " + std::to_string(nbytes) + " bytes, tensor needs " + std::to_string(want));
    }
    try {
      upload_enqueue(d, b, src, nbytes, on_done, ctx);
    } catch (...) {
      { std::lock_guard<std::mutex> g(d.mu); d.alloc.free(b->ptr); }
      delete b;
      throw;
    }
    *out = b;
  });
}

int nxb200_buffer_to_host(nxb200_buffer* buf, void* dst, size_t nbytes) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf);
    if (nbytes > b->nbytes) fail(NXB_ERR_INVALID_ARGUMENT, "asked for more bytes than the tensor holds");
    Device& d = nxb::device(b->device);
    if (nbytes) NXB_CUDA(cudaMemcpyAsync(dst, b->ptr, nbytes, cudaMemcpyDeviceToHost, d.stream));
    NXB_CUDA(cudaStreamSynchronize(d.stream));
    check_device_status(d);
  });
}

int nxb200_buffer_write_async(nxb200_buffer* buf, const void* src, size_t nbytes) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf);
    if (nbytes > b->nbytes) fail(NXB_ERR_INVALID_ARGUMENT, "more bytes than the tensor holds");
    Device& d = nxb::device(b->device);
    std::lock_guard<std::mutex> g(d.mu);
    // after the kernels already queued (they may still read the buffer), before the ones to come;
    // concurrent with downloads in flight unless one of them reads this very buffer
    NXB_CUDA(cudaEventRecord(d.ev_compute, d.stream));
    NXB_CUDA(cudaStreamWaitEvent(d.h2d, d.ev_compute, 0));
    if (std::find(d.pending_reads.begin(), d.pending_reads.end(), (const void*)b->ptr) != d.pending_reads.end())
      NXB_CUDA(cudaStreamWaitEvent(d.h2d, d.ev_d2h, 0));
    NXB_CUDA(cudaMemcpyAsync(b->ptr, src, nbytes, cudaMemcpyHostToDevice, d.h2d));
    NXB_CUDA(cudaEventRecord(d.ev_h2d, d.h2d));
    NXB_CUDA(cudaStreamWaitEvent(d.stream, d.ev_h2d, 0));
  });
}

int nxb200_buffer_read_async(nxb200_buffer* buf, void* dst, size_t nbytes) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf);
    if (nbytes > b->nbytes) fail(NXB_ERR_INVALID_ARGUMENT, "more bytes than the tensor holds");
    Device& d = nxb::device(b->device);
    std::lock_guard<std::mutex> g(d.mu);
    // after the kernels already queued (they produce the data); the next program waits for it
    // (order_after_downloads), so the buffer is not overwritten while it is being read
    NXB_CUDA(cudaEventRecord(d.ev_compute, d.stream));
    NXB_CUDA(cudaStreamWaitEvent(d.d2h, d.ev_compute, 0));
    NXB_CUDA(cudaMemcpyAsync(dst, b->ptr, nbytes, cudaMemcpyDeviceToHost, d.d2h));
    NXB_CUDA(cudaEventRecord(d.ev_d2h, d.d2h));
    d.pending_reads.push_back(b->ptr);
  });
}

int nxb200_buffer_copy_to_device(nxb200_buffer* buf, int dev, nxb200_buffer** out) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf);
    if (!out) fail(NXB_ERR_INVALID_ARGUMENT, "out is NULL");
    Device& src = nxb::device(b->device);
    NXB_CUDA(cudaStreamSynchronize(src.stream));
    Device& d = nxb::device(dev);
    nxb200_buffer* nb = make_buffer(d, b->dtype, b->dims.data(), (int)b->dims.size());
    cudaError_t e = cudaSuccess;
    if (b->nbytes) {
      e = cudaMemcpyPeerAsync(nb->ptr, dev, b->ptr, b->device, b->nbytes, d.stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(d.stream);
    }
    if (e != cudaSuccess) {
      { std::lock_guard<std::mutex> g(d.mu); d.alloc.free(nb->ptr); }
      delete nb;
      fail(NXB_ERR_RUNTIME, std::string("device to device copy failed: ") + cudaGetErrorString(e));
    }
    *out = nb;
  });
}

int nxb200_buffer_info(nxb200_buffer* buf, nxb200_dtype* dtype, int64_t* dims, int* rank, int* dev) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf, false);
    if (dtype) *dtype = b->dtype;
    if (rank) *rank = (int)b->dims.size();
    if (dims) for (size_t i = 0; i < b->dims.size(); ++i) dims[i] = b->dims[i];
    if (dev) *dev = b->device;
  });
}

int nxb200_buffer_device_pointer(nxb200_buffer* buf, void** ptr) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf);
    if (!ptr) fail(NXB_ERR_INVALID_ARGUMENT, "ptr is NULL");
    *ptr = b->ptr;
  });
}

/* create_buffer_from_device_pointer, :local mode (exla/lib/exla/backend.ex:137-181, exla.cc:391-437) */
int nxb200_buffer_from_pointer(int dev, nxb200_dtype dtype, const int64_t* dims, int rank, void* device_ptr, nxb200_buffer** out) {
  return guarded([&] {
    if (!out || !device_ptr) fail(NXB_ERR_INVALID_ARGUMENT, "out or the device pointer is NULL");
    if (rank < 0 || rank > NXB_MAX_RANK) fail(NXB_ERR_INVALID_ARGUMENT, "rank out of range");
    if ((int)dtype < 0 || dtype > NXB_F64) fail(NXB_ERR_INVALID_ARGUMENT, "unknown element type");
    nxb::device(dev);
    cudaPointerAttributes at{};
    if (cudaPointerGetAttributes(&at, device_ptr) != cudaSuccess || at.type != cudaMemoryTypeDevice || at.device != dev) {
      (void)cudaGetLastError();
      fail(NXB_ERR_INVALID_ARGUMENT, "the address is not device memory of device " + std::to_string(dev));
    }
    auto b = std::make_unique<nxb200_buffer>();
    b->device = dev;
    b->dtype = (DType)dtype;
    for (int i = 0; i < rank; ++i) {
      if (dims[i] < 0) fail(NXB_ERR_INVALID_ARGUMENT, "negative dimension");
      b->dims.push_back(dims[i]);
    }
    b->nbytes = (size_t)shape_numel(b->dims) * dtype_size(b->dtype);
    // Generated kernels and tensor maps take vector accesses from element offsets alone: the base has
    // to sit on a 16-byte boundary, and the tensor has to lie inside the allocation it points into.
    if (((uintptr_t)device_ptr) % 16 != 0)
      fail(NXB_ERR_INVALID_ARGUMENT, "the device address must be 16-byte aligned");
    if (driver().cuMemGetAddressRange) {
      CUdeviceptr base = 0;
      size_t size = 0;
      if (driver().cuMemGetAddressRange(&base, &size, (CUdeviceptr)(uintptr_t)device_ptr) == CUDA_SUCCESS) {
        const size_t before = (size_t)((CUdeviceptr)(uintptr_t)device_ptr - base);
        if (before > size || b->nbytes > size - before)
          fail(NXB_ERR_INVALID_ARGUMENT, "the tensor needs " + std::to_string(b->nbytes) + " bytes, the allocation holds " +
                                             std::to_string(size - std::min(before, size)) + " from that address");
      }
    }
    b->ptr = device_ptr;
    b->borrowed = true;
    *out = b.release();
  });
}

/* get_buffer_device_pointer, :cuda_ipc mode (exla.cc:325-389; exla_cuda.cc) */
int nxb200_buffer_ipc_export(nxb200_buffer* buf, uint8_t handle[NXB_IPC_HANDLE_BYTES]) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf);
    if (!handle) fail(NXB_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (b->borrowed) fail(NXB_ERR_INVALID_ARGUMENT, "only memory this library allocated can be exported");
    Device& d = nxb::device(b->device);
    NXB_CUDA(cudaStreamSynchronize(d.stream));          // the importer sees finished data
    cudaIpcMemHandle_t h;
    NXB_CUDA(cudaIpcGetMemHandle(&h, b->ptr));
    static_assert(sizeof h == NXB_IPC_HANDLE_BYTES, "IPC handle size");
    memcpy(handle, &h, sizeof h);
  });
}

/* create_buffer_from_device_pointer, :cuda_ipc mode: maps another process's allocation */
int nxb200_buffer_from_ipc(int dev, nxb200_dtype dtype, const int64_t* dims, int rank, const uint8_t handle[NXB_IPC_HANDLE_BYTES], nxb200_buffer** out) {
  return guarded([&] {
    if (!out || !handle) fail(NXB_ERR_INVALID_ARGUMENT, "out or handle is NULL");
    if (rank < 0 || rank > NXB_MAX_RANK) fail(NXB_ERR_INVALID_ARGUMENT, "rank out of range");
    if ((int)dtype < 0 || dtype > NXB_F64) fail(NXB_ERR_INVALID_ARGUMENT, "unknown element type");
    nxb::device(dev);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      fail(NXB_ERR_RUNTIME, std::string("the IPC handle could not be opened: ") + cudaGetErrorString(e));
    }
    auto b = std::make_unique<nxb200_buffer>();
    b->device = dev;
    b->dtype = (DType)dtype;
    for (int i = 0; i < rank; ++i) b->dims.push_back(dims[i]);
    b->nbytes = (size_t)shape_numel(b->dims) * dtype_size(b->dtype);
    b->ptr = p;
    b->borrowed = true;
    b->ipc_base = p;
    *out = b.release();
  });
}

int nxb200_buffer_deallocate(nxb200_buffer* buf) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf, false);
    bool was = b->deallocated.exchange(true);
    if (was) fail(NXB_ERR_ALREADY_DEALLOCATED, "buffer was already deallocated");
    if (b->upload) upload_join(b);
    Device& d = nxb::device(b->device);
    std::lock_guard<std::mutex> g(d.mu);
    order_after_downloads(d);      // whoever gets this memory next writes it on the compute stream
    if (b->ipc_base) {
      cudaStreamSynchronize(d.stream);
      cudaIpcCloseMemHandle(b->ipc_base);
      b->ipc_base = nullptr;
    }
    d.alloc.free(b->ptr);          // (a no-op for memory the allocator does not know)
    b->ptr = nullptr;
  });
}

int nxb200_buffer_is_deallocated(nxb200_buffer* buf, int* flag) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf, false);
    if (flag) *flag = b->deallocated.load() ? 1 : 0;
  });
}

int nxb200_buffer_release(nxb200_buffer* buf) {
  return guarded([&] {
    nxb200_buffer* b = check_buffer(buf, false);
    if (b->upload) upload_join(b);
    if (!b->deallocated.exchange(true) && b->ptr) {
      Device& d = nxb::device(b->device);
      std::lock_guard<std::mutex> g(d.mu);
      order_after_downloads(d);    // as in deallocate: the next owner of this memory writes it on the compute stream
      if (b->ipc_base) {
        cudaStreamSynchronize(d.stream);
        cudaIpcCloseMemHandle(b->ipc_base);
      }
      d.alloc.free(b->ptr);
    }
    b->magic = 0;
    delete b;
  });
}

int nxb200_program_build(const uint8_t* bytes, size_t nbytes, nxb200_program** out) {
  return guarded([&] {
    if (!bytes || !out) fail(NXB_ERR_INVALID_ARGUMENT, "NULL argument");
    auto p = std::make_unique<nxb200_program>();
    p->plan = build_plan(bytes, nbytes);
    *out = p.release();
  });
}

int nxb200_program_io(nxb200_program* prog, int* n_params, int* n_outputs) {
  return guarded([&] {
    nxb200_program* p = check_program(prog);
    if (n_params) *n_params = (int)p->plan->param_slots.size();
    if (n_outputs) *n_outputs = (int)p->plan->output_slots.size();
  });
}

int nxb200_program_output_info(nxb200_program* prog, int i, nxb200_dtype* dtype, int64_t* dims, int* rank) {
  return guarded([&] {
    nxb200_program* p = check_program(prog);
    if (i < 0 || i >= (int)p->plan->output_slots.size()) fail(NXB_ERR_INVALID_ARGUMENT, "output index out of range");
    const Slot& sl = p->plan->slots[p->plan->output_slots[i]];
    if (dtype) *dtype = sl.dt;
    if (rank) *rank = (int)sl.shape.size();
    if (dims) for (size_t k = 0; k < sl.shape.size(); ++k) dims[k] = sl.shape[k];
  });
}

int nxb200_program_run(nxb200_program* prog, int dev, nxb200_buffer* const* args, int n_args, nxb200_buffer** outs, int n_outs) {
  return guarded([&] { run_program(check_program(prog), dev, args, n_args, outs, n_outs, false); });
}

int nxb200_program_run_into(nxb200_program* prog, int dev, nxb200_buffer* const* args, int n_args, nxb200_buffer* const* outs,
                            int n_outs) {
  return guarded([&] { run_program(check_program(prog), dev, args, n_args, const_cast<nxb200_buffer**>(outs), n_outs, true); });
}

int nxb200_program_release(nxb200_program* prog) {
  return guarded([&] {
    nxb200_program* p = check_program(prog);
    for (auto& kv : p->loaded) {
      if (cudaSetDevice(kv.first) != cudaSuccess) { (void)cudaGetLastError(); continue; }
      Device& d = nxb::device(kv.first);
      cudaStreamSynchronize(d.stream);
      std::lock_guard<std::mutex> g(d.mu);
      // the captured graphs refer to kernels of the modules: they go first
      for (auto& r : kv.second.replays) {
        cudaGraphExecDestroy(r.exec);
        for (void* h : r.held) d.alloc.free(h);
      }
      for (auto m : kv.second.modules) driver().cuModuleUnload(m);
      for (auto& l : kv.second.literals) d.alloc.free(l.second);
    }
    p->magic = 0;
    delete p;
  });
}

size_t nxb200_program_describe(nxb200_program* prog, char* dst, size_t cap) {
  if (!prog || prog->magic != 0x4e584250) return 0;
  std::string s = prog->plan->describe();
  if (dst && cap) {
    size_t n = std::min(cap - 1, s.size());
    memcpy(dst, s.data(), n);
    dst[n] = 0;
  }
  return s.size();
}

size_t nxb200_program_kernel_source(nxb200_program* prog, int i, char* dst, size_t cap) {
  if (!prog || prog->magic != 0x4e584250 || i < 0 || i >= (int)prog->plan->kernels.size()) return 0;
  const std::string& s = prog->plan->kernels[i].source;
  if (dst && cap) {
    size_t n = std::min(cap - 1, s.size());
    memcpy(dst, s.data(), n);
    dst[n] = 0;
  }
  return s.size();
}

int nxb200_program_build_times(nxb200_program* prog, double* plan_seconds, double* codegen_seconds) {
  return guarded([&] {
    nxb200_program* p = check_program(prog);
    if (plan_seconds) *plan_seconds = p->plan->plan_seconds;
    if (codegen_seconds) *codegen_seconds = p->plan->codegen_seconds;
  });
}

int nxb200_program_launch_count(nxb200_program* prog, int* count) {
  return guarded([&] {
    nxb200_program* p = check_program(prog);
    if (count) *count = (int)p->plan->steps.size();
  });
}

int nxb200_device_synchronize(int dev) {
  return guarded([&] {
    Device& d = nxb::device(dev);
    NXB_CUDA(cudaStreamSynchronize(d.stream));
    NXB_CUDA(cudaStreamSynchronize(d.h2d));
    NXB_CUDA(cudaStreamSynchronize(d.d2h));
    {
      std::lock_guard<std::mutex> g(d.mu);
      d.pending_reads.clear();
    }
    check_device_status(d);
  });
}

int nxb200_timer_begin(int dev) {
  return guarded([&] {
    Device& d = nxb::device(dev);
    NXB_CUDA(cudaEventRecord(d.ev0, d.stream));
  });
}

int nxb200_timer_end(int dev, float* ms) {
  return guarded([&] {
    Device& d = nxb::device(dev);
    NXB_CUDA(cudaEventRecord(d.ev1, d.stream));
    NXB_CUDA(cudaEventSynchronize(d.ev1));
    float t = 0;
    NXB_CUDA(cudaEventElapsedTime(&t, d.ev0, d.ev1));
    if (ms) *ms = t;
  });
}

int nxb200_selftest_bounded_wait(int dev, uint32_t limit_us) {
  return guarded([&] {
    Device& d = nxb::device(dev);
    if (limit_us == 0 || limit_us > 2000000) fail(NXB_ERR_INVALID_ARGUMENT, "limit must be between 1 microsecond and 2 seconds");
    uint32_t* flag = nullptr;
    {
      std::lock_guard<std::mutex> g(d.mu);
      flag = (uint32_t*)d.alloc.alloc(sizeof(uint32_t));
    }
    cudaError_t e = cudaMemsetAsync(flag, 0, sizeof(uint32_t), d.stream);
    int khz = 1965000;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
    if (e == cudaSuccess) {
      try {
        launch_wait_probe(flag, (long long)limit_us * (long long)khz / 1000, d.status_dev, d.stream);
      } catch (...) {
        std::lock_guard<std::mutex> g(d.mu);
        d.alloc.free(flag);
        throw;
      }
      e = cudaStreamSynchronize(d.stream);
    }
    {
      std::lock_guard<std::mutex> g(d.mu);
      d.alloc.free(flag);
    }
    NXB_CUDA(e);
    check_device_status(d);      // the wait gave up: NXB_ERR_TIMEOUT
  });
}

int nxb200_device_stream(int dev, void** stream) {
  return guarded([&] {
    Device& d = nxb::device(dev);
    if (stream) *stream = (void*)d.stream;
  });
}

int nxb200_memory_stats(int dev, uint64_t* allocated, uint64_t* peak, uint64_t* reserved) {
  return guarded([&] {
    Device& d = nxb::device(dev);
    std::lock_guard<std::mutex> g(d.mu);
    if (allocated) *allocated = d.alloc.allocated;
    if (peak) *peak = d.alloc.peak;
    if (reserved) *reserved = d.alloc.reserved;
  });
}

int nxb200_memory_reset_peak(int dev) {
  return guarded([&] {
    Device& d = nxb::device(dev);
    std::lock_guard<std::mutex> g(d.mu);
    d.alloc.peak = d.alloc.allocated;
  });
}

}  // extern "C"

// The compiled form of a defn: graph, buffer slots, generated kernels, steps.
#pragma once

#include "common.h"

namespace nxb {

struct Node {
  std::string op;
  DType dt = NXB_F32;
  std::vector<int64_t> shape;
  std::vector<int> args;
  std::vector<int64_t> ints;
  std::vector<double> flts;
  std::string blob;
  // planner state
  int alias = -1;        // node whose buffer this node shares (metadata, contiguous reshape)
  int slot = -1;         // buffer slot when the value lives in global memory
  bool live = false;
  // A piece of a concatenate result: written into the parent's buffer at this element
  // offset with these strides instead of densely into a buffer of its own.
  int piece_of = -1;
  int64_t out_offset = 0;
  std::vector<int64_t> out_strides;
  // a piece written at a position given by scalar tensors (put_slice into a donated buffer):
  // window_axes[i] is the axis whose start is args[1 + i], clamped into [0, window_limit[i] - 1]
  std::vector<int> window_axes;
  std::vector<int64_t> window_limit;
  // dot only: node holding a per-output-column f32 factor applied to the product (-1: none)
  int scale_arg = -1;
};

struct Graph {
  std::vector<Node> nodes;
  std::vector<int> outputs;
  int n_params = 0;
  std::vector<std::pair<int, int>> aliases;   // donated (parameter index, output index) pairs
};

Graph parse_graph(const uint8_t* bytes, size_t nbytes);

struct Slot {
  enum Kind { PARAM, OUTPUT, TEMP, LITERAL } kind = TEMP;
  int index = 0;          // parameter index / output index / literal node
  DType dt = NXB_F32;
  std::vector<int64_t> shape;
  size_t nbytes = 0;
  int node = -1;
  int first_step = -1, last_step = -1;
};

struct KernelSpec {
  std::string name, source, desc, cubin;
  unsigned grid = 1, block = 1, smem = 0;
  std::vector<int> arg_slots;     // one pointer argument per entry
  std::vector<size_t> arg_offsets;  // byte offset added to the slot's base pointer
  std::vector<int> written_slots;   // slots this kernel stores to
  std::string prologue;             // preprocessor definitions placed before the device library (per-kernel switches)
  std::vector<int> inplace_ok;      // read slots whose every load is at the loading thread's own position
                                    // (s >= 0), and written slots stored there (encoded -1 - s)
  bool tensor_core = false;       // a generated matrix-product kernel (needs the GEMM device source)
  bool attention = false;         // ... and the attention device source
};

// Operand of a matrix product as a strided batch of row-major matrices.
struct GemmOperand {
  int slot = -1;
  int64_t batch_stride = 0;   // elements
  int64_t ld = 0;             // leading dimension, elements
  bool trans = false;         // false: the reduction index is contiguous
  DType dt = NXB_F32;
};

struct GemmSpec {
  int64_t batch = 1, m = 0, n = 0, k = 0;
  GemmOperand a, b;           // a: [m,k] (trans: [k,m]);  b: [k,n] stored as [n,k] when !trans... see gemm.h
  int out_slot = -1;
  DType out_dt = NXB_F32;
  std::string desc;
  // fused epilogue (see gemm.h)
  int epilogue = 0;
  int bias_slot = -1;
  int scale_slot = -1;
  // >= 0: index of a generated kernel (plan.kernels) whose epilogue computes and stores the
  // consumers of this product; the product itself is then never written to memory
  int jit_kernel = -1;
  int bn = 256;
  // >= 0: the generated epilogue hands its one result back in registers and the kernel stores the tile
  // itself; index (among the kernel's buffer arguments) and type of that result
  int staged_arg = -1;
  DType staged_dt = NXB_F32;
};

struct AttentionSpec {
  int q_slot = -1, k_slot = -1, v_slot = -1, out_slot = -1;
  int64_t batch_heads = 1, sq = 0, sk = 0;
  int causal = 0;
  int64_t heads = 1;                      // size of the axis before the rows (1: one leading axis)
  bool v_bshd = false, out_bshd = false;  // v read / result written as {batch, row, head, 128}
  int jit_kernel = -1;
  std::string desc;
};

struct CollectiveSpec {
  int in_slot = -1, out_slot = -1;
  int64_t count = 0;
  DType dt = NXB_F32;
  std::string desc;
};

struct SortSpec {
  int in_slot = -1, out_slot = -1;
  int64_t rows = 0, len = 0;
  DType dt = NXB_F32, out_dt = NXB_F32;
  bool descending = false, indices = false;
  std::string desc;
};

// indexed_add / indexed_put: the result is a copy of the target with the updates applied (scatter.cu)
struct ScatterSpec {
  int target_slot = -1, indices_slot = -1, updates_slot = -1, out_slot = -1;
  DType dt = NXB_F32, index_dt = NXB_S32;
  bool add = true;
  std::vector<int64_t> target_shape, update_shape;
  std::vector<int> axes;
  std::string desc;
};

struct Step {
  enum Kind { KERNEL, GEMM, ALLREDUCE, ATTENTION, SORT, SCATTER } kind = KERNEL;
  int index = 0;
};

struct Plan {
  Graph g;
  std::vector<Slot> slots;
  std::vector<Step> steps;
  std::vector<KernelSpec> kernels;
  std::vector<GemmSpec> gemms;
  std::vector<CollectiveSpec> collectives;
  std::vector<AttentionSpec> attentions;
  std::vector<SortSpec> sorts;
  std::vector<ScatterSpec> scatters;
  std::vector<int> param_slots;   // by parameter index (-1 when unused)
  std::vector<int> output_slots;  // by output index
  // Buffer donation (Nx.donatable, exla/lib/exla/defn.ex:598-645): the result takes over the
  // argument's buffer.  `in_place`: the result is written straight into the argument's memory
  // (its only reader is the kernel that writes the result, at each thread's own positions);
  // otherwise the result gets memory of its own and the argument's is released after the run.
  // `window`: the program writes only a window of the result (put_slice); the rest of it is the
  // argument's data, so a result that does not share the argument's memory is first copied from it.
  struct Alias { int param, output; bool in_place; bool window = false; };
  std::vector<Alias> aliases;
  // seconds spent building: parsing + planning + code generation, and NVRTC (source -> cubin)
  double plan_seconds = 0, codegen_seconds = 0;
  std::string describe() const;
};

std::unique_ptr<Plan> build_plan(const uint8_t* bytes, size_t nbytes);

// NVRTC: compile CUDA source to an sm_100a cubin (needs no GPU).
std::string compile_to_cubin(const std::string& source, const std::string& name, bool tensor_core = false, bool attention = false,
                             const std::string& prologue = std::string());
const char* device_lib_source();

}  // namespace nxb

struct nxb200_program {
  uint32_t magic = 0x4e584250;    // "NXBP"
  std::unique_ptr<nxb::Plan> plan;
  std::mutex mu;
  // per device: loaded modules/functions and uploaded literals
  struct Loaded {
    std::vector<CUmodule> modules;
    std::vector<CUfunction> functions;
    std::map<int, void*> literals;   // slot -> device pointer
    // Replay of small programs as CUDA graphs: a program whose argument and result
    // addresses were seen before is captured once (its temporaries stay reserved for
    // the graph) and afterwards costs one graph launch instead of one launch per step.
    struct Replay {
      std::vector<void*> key;          // argument pointers, then result pointers
      cudaGraphExec_t exec = nullptr;
      std::vector<void*> held;         // temporaries the captured kernels write
      uint64_t last_use = 0;
    };
    std::vector<Replay> replays;
    std::vector<std::vector<void*>> seen;   // keys met once (capture on the second meeting)
    bool graphable = true;
    uint64_t tick = 0;
  };
  std::map<int, Loaded> loaded;
};

// Deserialiser for the program wire format (layout in include/nxb200.h) and
// NVRTC front door.
#include "program.h"

#include <nvrtc.h>

namespace nxb {

namespace {
struct Reader {
  const uint8_t* p;
  size_t n, pos = 0;
  void need(size_t k) {
    if (pos + k > n) fail(NXB_ERR_INVALID_ARGUMENT, "program bytes are truncated");
  }
  template <typename T> T get() {
    need(sizeof(T));
    T v;
    memcpy(&v, p + pos, sizeof(T));
    pos += sizeof(T);
    return v;
  }
  std::string bytes(size_t k) {
    need(k);
    std::string s((const char*)p + pos, k);
    pos += k;
    return s;
  }
};
}  // namespace

Graph parse_graph(const uint8_t* bytes, size_t nbytes) {
  Reader r{bytes, nbytes};
  if (nbytes < 8 || memcmp(bytes, "NXB1", 4) != 0) fail(NXB_ERR_INVALID_ARGUMENT, "not an NXB1 program");
  r.pos = 4;
  Graph g;
  uint32_t n = r.get<uint32_t>();
  if (n > (1u << 24)) fail(NXB_ERR_INVALID_ARGUMENT, "program has too many nodes");
  g.nodes.resize(n);
  for (uint32_t i = 0; i < n; ++i) {
    Node& nd = g.nodes[i];
    uint8_t l = r.get<uint8_t>();
    nd.op = r.bytes(l);
    uint8_t dt = r.get<uint8_t>();
    if (dt > NXB_F64) fail(NXB_ERR_INVALID_ARGUMENT, "node " + std::to_string(i) + ": unknown element type code");
    nd.dt = (DType)dt;
    uint8_t rank = r.get<uint8_t>();
    if (rank > NXB_MAX_RANK) fail(NXB_ERR_INVALID_ARGUMENT, "node " + std::to_string(i) + ": rank above " + std::to_string(NXB_MAX_RANK));
    for (int k = 0; k < rank; ++k) {
      int64_t d = r.get<int64_t>();
      if (d < 0) fail(NXB_ERR_INVALID_ARGUMENT, "negative dimension");
      nd.shape.push_back(d);
    }
    uint16_t na = r.get<uint16_t>();
    for (int k = 0; k < na; ++k) {
      uint32_t a = r.get<uint32_t>();
      if (a >= i) fail(NXB_ERR_INVALID_ARGUMENT, "node " + std::to_string(i) + " refers to a later node");
      nd.args.push_back((int)a);
    }
    uint16_t ni = r.get<uint16_t>();
    for (int k = 0; k < ni; ++k) nd.ints.push_back(r.get<int64_t>());
    uint16_t nf = r.get<uint16_t>();
    for (int k = 0; k < nf; ++k) nd.flts.push_back(r.get<double>());
    uint64_t nb = r.get<uint64_t>();
    nd.blob = r.bytes((size_t)nb);
    if (nd.op == "parameter") {
      if (nd.ints.size() != 1 || nd.ints[0] < 0) fail(NXB_ERR_INVALID_ARGUMENT, "parameter node without an index");
      g.n_params = std::max(g.n_params, (int)nd.ints[0] + 1);
    }
    if (nd.op == "tensor" && nd.blob.size() != (size_t)shape_numel(nd.shape) * dtype_size(nd.dt))
      fail(NXB_ERR_INVALID_ARGUMENT, "tensor literal has the wrong number of bytes");
  }
  uint32_t no = r.get<uint32_t>();
  for (uint32_t i = 0; i < no; ++i) {
    uint32_t o = r.get<uint32_t>();
    if (o >= n) fail(NXB_ERR_INVALID_ARGUMENT, "output index out of range");
    g.outputs.push_back((int)o);
  }
  // optional: buffer donation, (parameter index, output index) pairs
  if (r.pos < nbytes) {
    uint32_t na = r.get<uint32_t>();
    for (uint32_t i = 0; i < na; ++i) {
      uint32_t p = r.get<uint32_t>(), o = r.get<uint32_t>();
      if ((int)p >= g.n_params || o >= no) fail(NXB_ERR_INVALID_ARGUMENT, "donation pair out of range");
      g.aliases.push_back({(int)p, (int)o});
    }
  }
  return g;
}

const char* device_lib_source() {
  static const char* src =
#include "device_lib_embed.inc"
      ;
  return src;
}

const char* gemm_device_source();
const char* attention_device_source();

std::string compile_to_cubin(const std::string& source, const std::string& name, bool tensor_core, bool attention, const std::string& prologue) {
  nvrtcProgram prog;
  std::string full = prologue + std::string(device_lib_source()) + "\n" + (tensor_core ? std::string(gemm_device_source()) + "\n" : std::string()) +
                     (attention ? std::string(attention_device_source()) + "\n" : std::string()) + source;
  if (nvrtcCreateProgram(&prog, full.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr) != NVRTC_SUCCESS)
    fail(NXB_ERR_RUNTIME, "nvrtcCreateProgram failed");
  const char* opts[] = {"-arch=sm_100a", "-std=c++17", "-lineinfo", "--use_fast_math=false", "-default-device"};
  // NXB200_PTXAS_INFO=1: registers, spills and shared memory of every generated kernel on stderr
  static const bool ptxas_info = getenv("NXB200_PTXAS_INFO") != nullptr;
  // NXB200_KERNEL_DEFINE=NAME[=VALUE]: one preprocessor definition for every generated kernel (diagnostics)
  static const char* extra_define = getenv("NXB200_KERNEL_DEFINE");
  static const std::string define_opt = std::string("-D") + (extra_define ? extra_define : "NXB_NO_EXTRA_DEFINE");
  // The process may have loaded another NVRTC than the one this library was built beside (a Python package
  // imported earlier can bring its own); kernels test NXB_NVRTC_VERSION before using newer PTX instructions.
  static const std::string version_opt = [] {
    int major = 0, minor = 0;
    nvrtcVersion(&major, &minor);
    return "-DNXB_NVRTC_VERSION=" + std::to_string(major * 100 + minor);
  }();
  const char* use[] = {opts[0], opts[1], opts[2], define_opt.c_str(), version_opt.c_str(), "--ptxas-options=-v"};
  nvrtcResult r = nvrtcCompileProgram(prog, ptxas_info ? 6 : 5, use);
  if (ptxas_info && r == NVRTC_SUCCESS) {
    size_t n = 0;
    nvrtcGetProgramLogSize(prog, &n);
    std::string log(n, '\0');
    nvrtcGetProgramLog(prog, &log[0]);
    fprintf(stderr, "[nxb200] %s:\n%s\n", name.c_str(), log.c_str());
  }
  if (r != NVRTC_SUCCESS) {
    size_t n = 0;
    nvrtcGetProgramLogSize(prog, &n);
    std::string log(n, '\0');
    nvrtcGetProgramLog(prog, &log[0]);
    nvrtcDestroyProgram(&prog);
    fail(NXB_ERR_RUNTIME, "kernel " + name + " failed to compile:\n" + log + "\n--- source ---\n" + source);
  }
  size_t n = 0;
  if (nvrtcGetCUBINSize(prog, &n) != NVRTC_SUCCESS || n == 0) {
    nvrtcDestroyProgram(&prog);
    fail(NXB_ERR_RUNTIME, "nvrtc produced no cubin for " + name);
  }
  std::string cubin(n, '\0');
  nvrtcGetCUBIN(prog, &cubin[0]);
  nvrtcDestroyProgram(&prog);
  return cubin;
}

}  // namespace nxb

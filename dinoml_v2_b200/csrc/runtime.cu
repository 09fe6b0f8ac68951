// Artifact / session runtime: the `dino_*` C ABI over an interpreted launch plan.
//
// The reference generates one module.so per model from src/dinoml/templates/gpu_module.cu.j2 (module
// and session structs, constant loading, per-run validation, the launch sequence, a CUDA-graph
// benchmark loop).  This runtime provides the same entry points from one prebuilt library: the
// artifact directory carries `module_plan.txt`, a line-based description of tensors, constants and
// gemm nodes written by the Python compiler, and a session walks it - one fused launch per
// quantized linear on the session stream, no dequantization scratch.
//
// Plan grammar (whitespace-separated tokens, one record per line):
//   dinoml_b200_module_plan 1
//   tensor <name> input|output|temp <DinoDtype> <ndim> <dim>...          dim = N  or  ?min:max
//   constant <name> dense <DinoDtype> <offset> <nbytes> <ndim> <dim>...
//   constant <name> gguf <qtype_value> <offset> <nbytes> <rows> <n_per_row> <residency>
//   node gemm_rcr <a> <b> <bias|-> <out> <variant>                       also gemm_rcr_bias; dual_gemm_rcr_silu / _fast_gelu with
//                                                                         <b> = the two weights' rows interleaved in groups of 8
//   dispatch <node_index> <m> <n> <k> <variant>                          shape-guarded selection
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/dinoml_b200_runtime.h"
#include "gguf_common.cuh"

namespace b200gguf {
int set_error_message(int rc, const std::string& message);
const char* last_error();
int dual_gemm_rcr(const void* a, const void* b01, void* c, int qtype, int dtype, int m, int n, int k, int activation, int variant,
                  cudaStream_t s);
int gemm_rcr(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
             int variant, cudaStream_t s);
}  // namespace b200gguf

using b200gguf::set_error_message;

namespace {

int fail(const std::string& message) { return set_error_message(1, message); }
int cuda_fail(const char* what, cudaError_t err) { return fail(std::string(what) + ": " + cudaGetErrorString(err)); }

size_t dtype_size(int dtype) {
  switch (dtype) {
    case DINO_DTYPE_FLOAT16: case DINO_DTYPE_BFLOAT16: return 2;
    case DINO_DTYPE_FLOAT32: case DINO_DTYPE_INT32: return 4;
    case DINO_DTYPE_INT64: return 8;
    case DINO_DTYPE_BOOL: case DINO_DTYPE_FLOAT8_E4M3: case DINO_DTYPE_FLOAT8_E5M2: return 1;
    default: return 0;
  }
}

struct DimSpec { int64_t min = 0, max = 0; bool dynamic() const { return min != max; } };

struct TensorSpec {
  std::string name;
  int role = 0;  // 0 input, 1 output, 2 temp
  int dtype = 0;
  std::vector<DimSpec> dims;
  size_t max_bytes() const {
    size_t n = dtype_size(dtype);
    for (const DimSpec& d : dims) n *= size_t(d.max);
    return n;
  }
};

struct ConstantSpec {
  std::string name;
  bool encoded = false;
  int dtype = 0;        // dense
  int qtype = 0;        // encoded
  size_t offset = 0, nbytes = 0;
  std::vector<int64_t> shape;   // dense: logical shape; encoded: {rows, n_per_row}
  std::string residency;
  void* device = nullptr;
  bool loaded = false;
};

struct NodeSpec {
  int a = -1, out = -1;       // tensor indices
  int b = -1, bias = -1;      // constant indices
  int variant = 0;
  int activation = 0;         // 0: gemm_rcr[_bias]; 1 / 2: dual_gemm_rcr_silu / _fast_gelu on a row-interleaved weight
};
struct DispatchSpec { int node, m, n, k, variant; };

}  // namespace

struct DinoModule {
  std::string artifact_dir, metadata_json;
  std::vector<TensorSpec> tensors;
  std::vector<int> inputs, outputs;
  std::vector<ConstantSpec> constants;
  std::vector<NodeSpec> nodes;
  std::vector<DispatchSpec> dispatch;
};

struct DinoSession {
  DinoModule* module = nullptr;
  cudaStream_t owned_stream = nullptr, stream = nullptr;
  bool external_stream = false;
  std::vector<void*> temps;                         // per tensor index (temp role only)
  std::vector<std::vector<int64_t>> shapes;         // per tensor index, as of the last run
  std::vector<bool> output_shape_valid;
};

namespace {

int find_tensor(const DinoModule& m, const std::string& name) {
  for (size_t i = 0; i < m.tensors.size(); ++i) if (m.tensors[i].name == name) return int(i);
  return -1;
}
int find_constant(const DinoModule& m, const std::string& name) {
  for (size_t i = 0; i < m.constants.size(); ++i) if (m.constants[i].name == name) return int(i);
  return -1;
}

bool parse_dim(const std::string& tok, DimSpec* out) {
  if (tok.empty()) return false;
  if (tok[0] == '?') {
    long long lo = 0, hi = 0;
    if (std::sscanf(tok.c_str(), "?%lld:%lld", &lo, &hi) != 2 || lo < 0 || hi < lo) return false;
    out->min = lo; out->max = hi;
    return true;
  }
  char* end = nullptr;
  const long long v = std::strtoll(tok.c_str(), &end, 10);
  if (*end != '\0' || v < 0) return false;
  out->min = out->max = v;
  return true;
}

int parse_plan(DinoModule* mod, const std::string& path) {
  std::ifstream in(path);
  if (!in) return fail("cannot open " + path);
  std::string line;
  bool header = false;
  int lineno = 0;
  while (std::getline(in, line)) {
    ++lineno;
    std::istringstream ls(line);
    std::string kind;
    if (!(ls >> kind) || kind[0] == '#') continue;
    const std::string where = path + ":" + std::to_string(lineno) + ": ";
    if (kind == "dinoml_b200_module_plan") {
      int version = 0;
      if (!(ls >> version) || version != 1) return fail(where + "unsupported plan version");
      header = true;
    } else if (kind == "tensor") {
      TensorSpec t;
      std::string role;
      size_t ndim = 0;
      if (!(ls >> t.name >> role >> t.dtype >> ndim)) return fail(where + "malformed tensor record");
      t.role = role == "input" ? 0 : role == "output" ? 1 : role == "temp" ? 2 : -1;
      if (t.role < 0 || dtype_size(t.dtype) == 0 || ndim == 0 || ndim > 8) return fail(where + "bad tensor role/dtype/rank");
      for (size_t i = 0; i < ndim; ++i) {
        std::string tok;
        DimSpec d;
        if (!(ls >> tok) || !parse_dim(tok, &d)) return fail(where + "bad tensor dimension");
        t.dims.push_back(d);
      }
      if (t.role == 0) mod->inputs.push_back(int(mod->tensors.size()));
      if (t.role == 1) mod->outputs.push_back(int(mod->tensors.size()));
      mod->tensors.push_back(t);
    } else if (kind == "constant") {
      ConstantSpec c;
      std::string storage;
      if (!(ls >> c.name >> storage)) return fail(where + "malformed constant record");
      if (storage == "dense") {
        size_t ndim = 0;
        if (!(ls >> c.dtype >> c.offset >> c.nbytes >> ndim) || dtype_size(c.dtype) == 0) return fail(where + "bad dense constant");
        size_t numel = 1;
        for (size_t i = 0; i < ndim; ++i) {
          long long d = 0;
          if (!(ls >> d) || d < 0) return fail(where + "bad constant dimension");
          c.shape.push_back(d);
          numel *= size_t(d);
        }
        if (numel * dtype_size(c.dtype) != c.nbytes) return fail(where + "dense constant byte size does not match its shape");
      } else if (storage == "gguf") {
        long long rows = 0, npr = 0;
        c.encoded = true;
        if (!(ls >> c.qtype >> c.offset >> c.nbytes >> rows >> npr >> c.residency)) return fail(where + "bad gguf constant");
        const int bs = b200gguf::qtype_block_size(c.qtype);
        if (bs == 0) return fail(where + "unsupported GGUF qtype " + std::to_string(c.qtype));
        if (rows <= 0 || npr <= 0 || npr % bs) return fail(where + "n_per_row is not a multiple of the block size");
        if (size_t(rows) * size_t(npr / bs) * size_t(b200gguf::qtype_block_bytes(c.qtype)) != c.nbytes)
          return fail(where + "encoded_nbytes does not match rows x n_per_row");
        c.shape = {rows, npr};
      } else {
        return fail(where + "unknown constant storage " + storage);
      }
      mod->constants.push_back(c);
    } else if (kind == "node") {
      std::string op, a, b, bias, out;
      NodeSpec n;
      if (!(ls >> op >> a >> b >> bias >> out >> n.variant)) return fail(where + "malformed node record");
      if (op == "dual_gemm_rcr_silu") n.activation = 1;
      else if (op == "dual_gemm_rcr_fast_gelu") n.activation = 2;
      else if (op != "gemm_rcr" && op != "gemm_rcr_bias") return fail(where + "unsupported op " + op);
      if (n.activation != 0 && bias != "-") return fail(where + "dual_gemm_rcr takes no bias");
      n.a = find_tensor(*mod, a);
      n.out = find_tensor(*mod, out);
      n.b = find_constant(*mod, b);
      n.bias = bias == "-" ? -1 : find_constant(*mod, bias);
      if (n.a < 0 || n.out < 0 || n.b < 0 || (bias != "-" && n.bias < 0)) return fail(where + "node references an unknown tensor");
      if (!mod->constants[n.b].encoded) return fail(where + "gemm weight must be a GGUF-encoded constant");
      if (n.bias >= 0 && mod->constants[n.bias].encoded) return fail(where + "bias must be a dense constant");
      if (n.variant < 0 || (n.variant & 0xff) > 4 || n.variant > 0xffff) return fail(where + "bad variant");   // family | config << 8
      mod->nodes.push_back(n);
    } else if (kind == "dispatch") {
      DispatchSpec d;
      if (!(ls >> d.node >> d.m >> d.n >> d.k >> d.variant) || d.node < 0 || size_t(d.node) >= mod->nodes.size() ||
          (d.variant & 0xff) < 1 || (d.variant & 0xff) > 4 || d.variant > 0xffff)
        return fail(where + "malformed dispatch record");
      mod->dispatch.push_back(d);
    } else {
      return fail(where + "unknown record " + kind);
    }
  }
  if (!header) return fail(path + ": missing plan header");
  if (mod->nodes.empty()) return fail(path + ": plan has no nodes");
  return 0;
}

int read_file(const std::string& path, std::string* out) {
  std::ifstream in(path, std::ios::binary);
  if (!in) return fail("cannot open " + path);
  std::ostringstream ss;
  ss << in.rdbuf();
  *out = ss.str();
  return 0;
}

int load_module(const char* artifact_dir, bool eager, DinoModule** out) {
  if (artifact_dir == nullptr || out == nullptr) return fail("dino_module_load received null pointer");
  *out = nullptr;
  DinoModule* mod = new DinoModule();
  mod->artifact_dir = artifact_dir;
  if (int rc = parse_plan(mod, mod->artifact_dir + "/module_plan.txt")) { delete mod; return rc; }
  if (int rc = read_file(mod->artifact_dir + "/metadata.json", &mod->metadata_json)) { delete mod; return rc; }
  if (eager) {
    if (int rc = dino_module_load_constants(mod, (mod->artifact_dir + "/constants.bin").c_str())) {
      dino_module_free(mod);
      return rc;
    }
  }
  *out = mod;
  return 0;
}

int ensure_constant_buffer(ConstantSpec& c) {
  if (c.device != nullptr || c.nbytes == 0) return 0;
  const cudaError_t err = cudaMalloc(&c.device, c.nbytes);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMalloc (constant)", err);
}

int check_tensor(const TensorSpec& spec, const DinoTensor& t, const char* what, std::vector<int64_t>* shape) {
  const std::string who = std::string(what) + " '" + spec.name + "'";
  if (t.data == nullptr) return fail(who + " has a null data pointer");
  if (t.shape == nullptr) return fail(who + " has a null shape pointer");
  if (t.dtype != spec.dtype) return fail(who + " has dtype " + std::to_string(t.dtype) + ", expected " + std::to_string(spec.dtype));
  if (t.device_type != DINO_DEVICE_CUDA) return fail(who + " must live on a CUDA device");
  if (t.ndim != spec.dims.size()) return fail(who + " has rank " + std::to_string(t.ndim) + ", expected " + std::to_string(spec.dims.size()));
  shape->assign(t.shape, t.shape + t.ndim);
  size_t numel = 1;
  for (size_t i = 0; i < t.ndim; ++i) {
    if (t.shape[i] < spec.dims[i].min || t.shape[i] > spec.dims[i].max)
      return fail(who + " dimension " + std::to_string(i) + " = " + std::to_string(t.shape[i]) + " outside [" +
                  std::to_string(spec.dims[i].min) + ", " + std::to_string(spec.dims[i].max) + "]");
    numel *= size_t(t.shape[i]);
  }
  if (t.strides != nullptr) {  // contiguous row-major only, as runtime/include/dinoml/module_support.h:163-177
    int64_t expect = 1;
    for (size_t i = t.ndim; i-- > 0;) {
      if (t.shape[i] != 1 && t.strides[i] != expect) return fail(who + " must be contiguous");
      expect *= t.shape[i];
    }
  }
  const size_t esz = dtype_size(spec.dtype);
  if (t.byte_offset % esz) return fail(who + " byte_offset is not a multiple of the element size");
  if (t.nbytes != 0 && t.nbytes < numel * esz) return fail(who + " nbytes is smaller than its shape requires");
  return 0;
}

void* tensor_ptr(const DinoTensor& t) { return static_cast<uint8_t*>(t.data) + t.byte_offset; }

// One pass over the plan.  `launch == false` only validates and computes shapes.
int run_plan(DinoSession* s, const DinoTensor* inputs, size_t num_inputs, DinoTensor* outputs, size_t num_outputs,
             bool validate) {
  DinoModule& mod = *s->module;
  if (validate) {
    if (num_inputs != mod.inputs.size()) return fail("dino_session_run expected " + std::to_string(mod.inputs.size()) + " inputs");
    if (num_outputs != mod.outputs.size()) return fail("dino_session_run expected " + std::to_string(mod.outputs.size()) + " outputs");
    if ((num_inputs && inputs == nullptr) || (num_outputs && outputs == nullptr)) return fail("dino_session_run received null tensor arrays");
    for (size_t i = 0; i < num_inputs; ++i)
      if (int rc = check_tensor(mod.tensors[mod.inputs[i]], inputs[i], "input", &s->shapes[mod.inputs[i]])) return rc;
    for (const ConstantSpec& c : mod.constants)
      if (!c.loaded) return fail("constant '" + c.name + "' is not loaded" + (c.encoded ? " (call dino_module_set_encoded_constant)" : ""));
  }
  std::vector<void*> ptr(mod.tensors.size(), nullptr);
  for (size_t i = 0; i < num_inputs; ++i) ptr[mod.inputs[i]] = tensor_ptr(inputs[i]);
  for (size_t i = 0; i < num_outputs; ++i) ptr[mod.outputs[i]] = outputs[i].data ? tensor_ptr(outputs[i]) : nullptr;
  for (size_t i = 0; i < mod.tensors.size(); ++i) if (mod.tensors[i].role == 2) ptr[i] = s->temps[i];

  for (size_t ni = 0; ni < mod.nodes.size(); ++ni) {
    const NodeSpec& node = mod.nodes[ni];
    const ConstantSpec& w = mod.constants[node.b];
    const std::vector<int64_t>& ashape = s->shapes[node.a];
    if (ashape.empty()) return fail("node " + std::to_string(ni) + " consumes a tensor that has no shape yet");
    const int64_t k = ashape.back();
    int64_t m = 1;
    for (size_t i = 0; i + 1 < ashape.size(); ++i) m *= ashape[i];
    if (node.activation != 0 && w.shape[0] % 16 != 0) return fail("dual_gemm_rcr weight must hold 2N rows with N % 8 == 0");
    const int64_t n = node.activation != 0 ? w.shape[0] / 2 : w.shape[0];
    if (k != w.shape[1]) return fail("gemm_rcr K dimension " + std::to_string(k) + " does not match n_per_row " + std::to_string(w.shape[1]));
    if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return fail("gemm_rcr dimension exceeds int range");
    std::vector<int64_t> oshape(ashape.begin(), ashape.end() - 1);
    oshape.push_back(n);
    const TensorSpec& ospec = mod.tensors[node.out];
    if (validate) {
      if (ospec.dtype != mod.tensors[node.a].dtype) return fail("gemm_rcr operands must share one dtype");
      if (ospec.role == 1) {
        size_t oi = 0;
        while (mod.outputs[oi] != node.out) ++oi;
        std::vector<int64_t> given;
        if (int rc = check_tensor(ospec, outputs[oi], "output", &given)) return rc;
        if (given != oshape) return fail("output '" + ospec.name + "' shape does not match the gemm_rcr result shape");
        s->output_shape_valid[oi] = true;
      }
      s->shapes[node.out] = oshape;
    }
    if (m == 0) continue;
    int variant = node.variant;
    for (const DispatchSpec& d : mod.dispatch)
      if (d.node == int(ni) && d.m == m && d.n == n && d.k == k) { variant = d.variant; break; }
    const void* bias = node.bias >= 0 ? mod.constants[node.bias].device : nullptr;
    if (node.bias >= 0 && mod.constants[node.bias].shape.back() != n) return fail("bias length does not match N");
    const int rc = node.activation != 0
                       ? b200gguf::dual_gemm_rcr(ptr[node.a], w.device, ptr[node.out], w.qtype, ospec.dtype, int(m), int(n), int(k),
                                                 node.activation, variant, s->stream)
                       : b200gguf::gemm_rcr(ptr[node.a], w.device, bias, ptr[node.out], w.qtype, ospec.dtype, int(m), int(n), int(k),
                                            variant, s->stream);
    if (rc != 0) {
      static const char* const kText[] = {"ok", "null pointer", "non-positive dimension", "k not a multiple of the block",
                                          "CUDA launch failed", "unsupported qtype", "unsupported dtype", "alignment",
                                          "shape outside variant range", "device wait gave up"};
      return fail("gemm_rcr node " + std::to_string(ni) + " failed: " + (rc < 10 ? kText[rc] : "error"));
    }
  }
  return 0;
}

}  // namespace

extern "C" {

int dino_runtime_fail(const char* message) { return fail(message ? message : "unknown error"); }
int dino_abi_version(void) { return DINO_RUNTIME_ABI_VERSION; }

int dino_device_malloc(void** out, size_t nbytes) {
  if (out == nullptr) return fail("dino_device_malloc received null pointer");
  const cudaError_t err = cudaMalloc(out, nbytes);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMalloc", err);
}
int dino_device_free(void* ptr) {
  const cudaError_t err = cudaFree(ptr);
  return err == cudaSuccess ? 0 : cuda_fail("cudaFree", err);
}
int dino_copy_host_to_device(void* dst, const void* src, size_t nbytes) {
  const cudaError_t err = cudaMemcpy(dst, src, nbytes, cudaMemcpyHostToDevice);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMemcpy H2D", err);
}
int dino_copy_device_to_host(void* dst, const void* src, size_t nbytes) {
  const cudaError_t err = cudaMemcpy(dst, src, nbytes, cudaMemcpyDeviceToHost);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMemcpy D2H", err);
}
int dino_copy_device_to_device(void* dst, const void* src, size_t nbytes) {
  const cudaError_t err = cudaMemcpy(dst, src, nbytes, cudaMemcpyDeviceToDevice);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMemcpy D2D", err);
}

int dino_module_load(const char* artifact_dir, DinoModule** out) { return load_module(artifact_dir, true, out); }
int dino_module_load_deferred(const char* artifact_dir, DinoModule** out) { return load_module(artifact_dir, false, out); }

int dino_module_load_constants(DinoModule* module, const char* constants_path) {
  if (module == nullptr || constants_path == nullptr) return fail("dino_module_load_constants received null pointer");
  std::ifstream in(constants_path, std::ios::binary);
  if (!in) return fail(std::string("cannot open ") + constants_path);
  std::vector<char> staging;
  for (ConstantSpec& c : module->constants) {
    if (c.encoded && c.residency == "manual_runtime_load") continue;   // uploaded by dino_module_set_encoded_constant
    staging.resize(c.nbytes);
    in.seekg(std::streamoff(c.offset));
    if (!in.read(staging.data(), std::streamsize(c.nbytes))) return fail("constants file is too short for '" + c.name + "'");
    if (int rc = ensure_constant_buffer(c)) return rc;
    const cudaError_t err = cudaMemcpy(c.device, staging.data(), c.nbytes, cudaMemcpyHostToDevice);
    if (err != cudaSuccess) return cuda_fail("cudaMemcpy (constant)", err);
    c.loaded = true;
  }
  return 0;
}

int dino_module_unload_constants(DinoModule* module) {
  if (module == nullptr) return fail("dino_module_unload_constants received null pointer");
  cudaDeviceSynchronize();
  for (ConstantSpec& c : module->constants) {
    if (c.device != nullptr) cudaFree(c.device);
    c.device = nullptr;
    c.loaded = false;
  }
  return 0;
}

int dino_module_set_constant(DinoModule* module, const char* name, const DinoTensor* tensor) {
  if (module == nullptr || name == nullptr || tensor == nullptr) return fail("dino_module_set_constant received null pointer");
  const int idx = find_constant(*module, name);
  if (idx < 0) return fail(std::string("unknown constant '") + name + "'");
  ConstantSpec& c = module->constants[idx];
  if (c.encoded) return fail(std::string("constant '") + name + "' is GGUF-encoded; use dino_module_set_encoded_constant");
  if (tensor->data == nullptr || tensor->shape == nullptr) return fail("dino_module_set_constant tensor has null data or shape");
  if (tensor->dtype != c.dtype || tensor->ndim != c.shape.size()) return fail(std::string("constant '") + name + "' dtype/rank mismatch");
  for (size_t i = 0; i < tensor->ndim; ++i)
    if (tensor->shape[i] != c.shape[i]) return fail(std::string("constant '") + name + "' shape mismatch");
  if (tensor->device_type != DINO_DEVICE_CUDA) return fail("dino_module_set_constant expects a CUDA tensor");
  if (int rc = ensure_constant_buffer(c)) return rc;
  const cudaError_t err = cudaMemcpy(c.device, tensor_ptr(*tensor), c.nbytes, cudaMemcpyDeviceToDevice);
  if (err != cudaSuccess) return cuda_fail("cudaMemcpy (set_constant)", err);
  c.loaded = true;
  return 0;
}

int dino_module_set_encoded_constant(DinoModule* module, const char* name, const void* device_bytes, size_t nbytes) {
  if (module == nullptr || name == nullptr || device_bytes == nullptr) return fail("dino_module_set_encoded_constant received null pointer");
  const int idx = find_constant(*module, name);
  if (idx < 0) return fail(std::string("unknown constant '") + name + "'");
  ConstantSpec& c = module->constants[idx];
  if (!c.encoded) return fail(std::string("constant '") + name + "' is not GGUF-encoded");
  if (nbytes != c.nbytes)
    return fail(std::string("constant '") + name + "' expects exactly " + std::to_string(c.nbytes) + " encoded bytes, got " + std::to_string(nbytes));
  if (int rc = ensure_constant_buffer(c)) return rc;
  const cudaError_t err = cudaMemcpy(c.device, device_bytes, nbytes, cudaMemcpyDeviceToDevice);
  if (err != cudaSuccess) return cuda_fail("cudaMemcpy (set_encoded_constant)", err);
  c.loaded = true;
  return 0;
}

int dino_module_free(DinoModule* module) {
  if (module == nullptr) return 0;
  for (ConstantSpec& c : module->constants) if (c.device != nullptr) cudaFree(c.device);
  delete module;
  return 0;
}

const char* dino_module_get_metadata_json(DinoModule* module) { return module ? module->metadata_json.c_str() : ""; }

int dino_session_create(DinoModule* module, DinoSession** out) {
  if (module == nullptr || out == nullptr) return fail("dino_session_create received null pointer");
  *out = nullptr;
  DinoSession* s = new DinoSession();
  s->module = module;
  cudaError_t err = cudaStreamCreateWithFlags(&s->owned_stream, cudaStreamNonBlocking);
  if (err != cudaSuccess) { delete s; return cuda_fail("cudaStreamCreateWithFlags", err); }
  s->stream = s->owned_stream;
  s->temps.assign(module->tensors.size(), nullptr);
  s->shapes.assign(module->tensors.size(), {});
  s->output_shape_valid.assign(module->outputs.size(), false);
  for (size_t i = 0; i < module->tensors.size(); ++i) {
    if (module->tensors[i].role != 2) continue;
    err = cudaMalloc(&s->temps[i], module->tensors[i].max_bytes());
    if (err != cudaSuccess) { dino_session_destroy(s); return cuda_fail("cudaMalloc (session temporary)", err); }
  }
  *out = s;
  return 0;
}

int dino_session_destroy(DinoSession* session) {
  if (session == nullptr) return 0;
  if (session->owned_stream != nullptr) {
    cudaStreamSynchronize(session->owned_stream);
    cudaStreamDestroy(session->owned_stream);
  }
  for (void* p : session->temps) if (p != nullptr) cudaFree(p);
  delete session;
  return 0;
}

int dino_session_set_stream(DinoSession* session, void* stream) {
  if (session == nullptr) return fail("dino_session_set_stream received null pointer");
  session->external_stream = stream != nullptr;
  session->stream = stream != nullptr ? static_cast<cudaStream_t>(stream) : session->owned_stream;
  return 0;
}

int dino_session_get_output_shape(DinoSession* session, size_t output_index, int64_t* out_shape, size_t* inout_ndim) {
  if (session == nullptr || inout_ndim == nullptr) return fail("dino_session_get_output_shape received null pointer");
  if (output_index >= session->module->outputs.size()) return fail("output index out of range");
  if (!session->output_shape_valid[output_index]) return fail("output shape is not available before the first run");
  const std::vector<int64_t>& shape = session->shapes[session->module->outputs[output_index]];
  if (out_shape == nullptr || *inout_ndim < shape.size()) { *inout_ndim = shape.size(); return out_shape == nullptr ? 0 : fail("output shape buffer too small"); }
  std::memcpy(out_shape, shape.data(), shape.size() * sizeof(int64_t));
  *inout_ndim = shape.size();
  return 0;
}

int dino_session_run(DinoSession* session, const DinoTensor* inputs, size_t num_inputs, DinoTensor* outputs, size_t num_outputs) {
  if (session == nullptr) return fail("dino_session_run received null session");
  if (int rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, true)) return rc;
  if (!session->external_stream) {
    const cudaError_t err = cudaStreamSynchronize(session->stream);
    if (err != cudaSuccess) return cuda_fail("dino_session_run synchronize", err);
  }
  return 0;
}

int dino_session_benchmark(DinoSession* session, const DinoTensor* inputs, size_t num_inputs, DinoTensor* outputs,
                           size_t num_outputs, size_t warmup_runs, size_t measured_runs, double* out_elapsed_ms,
                           size_t out_elapsed_count) {
  if (session == nullptr) return fail("dino_session_benchmark received null session");
  if (measured_runs == 0 || out_elapsed_ms == nullptr || out_elapsed_count < measured_runs)
    return fail("dino_session_benchmark needs measured_runs > 0 and an output array of at least that length");
  if (int rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, true)) return rc;   // validates + first warm run
  for (size_t i = 1; i < warmup_runs; ++i)
    if (int rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, false)) return rc;
  cudaError_t err = cudaStreamSynchronize(session->stream);
  if (err != cudaSuccess) return cuda_fail("dino_session_benchmark warm-up", err);

  // Graph replay on the owned stream (skipped on an external stream, as the reference does); set
  // DINOML_REQUIRE_BENCHMARK_GRAPH to turn a capture failure into an error instead of direct launches.
  cudaGraphExec_t exec = nullptr;
  if (!session->external_stream) {
    cudaGraph_t graph = nullptr;
    bool ok = cudaStreamBeginCapture(session->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    if (ok) {
      const int rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, false);
      ok = cudaStreamEndCapture(session->stream, &graph) == cudaSuccess && rc == 0 && graph != nullptr;
    }
    if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
    if (graph != nullptr) cudaGraphDestroy(graph);
    if (!ok) {
      exec = nullptr;
      cudaGetLastError();
      if (std::getenv("DINOML_REQUIRE_BENCHMARK_GRAPH") != nullptr) return fail("dino_session_benchmark could not capture a CUDA graph");
    }
  }
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return fail("cudaEventCreate failed");
  int rc = 0;
  for (size_t i = 0; i < measured_runs && rc == 0; ++i) {
    cudaEventRecord(e0, session->stream);
    if (exec != nullptr) {
      if (cudaGraphLaunch(exec, session->stream) != cudaSuccess) rc = fail("cudaGraphLaunch failed");
    } else {
      rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, false);
    }
    cudaEventRecord(e1, session->stream);
    if (rc == 0 && cudaEventSynchronize(e1) != cudaSuccess) rc = fail("cudaEventSynchronize failed");
    float ms = 0.f;
    if (rc == 0 && cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) rc = fail("cudaEventElapsedTime failed");
    out_elapsed_ms[i] = double(ms);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (exec != nullptr) cudaGraphExecDestroy(exec);
  return rc;
}

}  // extern "C"
